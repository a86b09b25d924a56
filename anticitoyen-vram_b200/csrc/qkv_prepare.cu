// From a stacked projection [q | k | v] to queries ready for the attention kernels and keys and values in their pages,
// for attention layers whose steps between the two span more than a head: one block a token, everything in float,
// one rounding at the end.  Each step is optional:
//
//   whole-projection norm   q <- q / sqrt(mean over all NH*D elements of q^2 + eps) * wq, the same for k with wk
//                           (one root mean square for all heads together, a weight for every element)
//   rotation                the first R elements of every q and k head, element i paired with i + R/2, by the table
//                           cos_sin[position] = [cos of R/2 angles | sin of them] (any factor already in the table)
//   query temperature       q <- q * (1 + coef * ln(floor((position + 1) / every) + 1))
//   value norm              every value head <- v / sqrt(mean(v^2) + eps)
//   value sharing           mode 1: the values (after their norm) are left in `shared` (float [T, NKV*DV]) for later
//                           layers of the step; mode 2: v <- (1 - lambda) v + lambda shared[t]
//   append                  k and v of the token into its request's page at its position
//
// q is rewritten in place in the projection's type; k and v go to the pages only (page < 0: nowhere).
#include "common.cuh"

template <typename T>
__global__ void qkv_prepare_kernel(T* __restrict__ qkv, int ld, int NH, int NKV, int D, int DV,
                                   const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                   const float* __restrict__ cos_sin, int R, int table_rows,
                                   float temp_coef, int temp_every, int value_norm, float value_eps,
                                   float* __restrict__ shared_v, int share_mode, float lambda,
                                   const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                   const int* __restrict__ block_table, int bt_stride, const int* __restrict__ bt_rows,
                                   T* __restrict__ k_pages, T* __restrict__ v_pages, int page_size, int num_pages) {
    extern __shared__ float sm[];
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int QS = NH * D, KS = NKV * D, VS = NKV * DV;
    float* q = sm;
    float* k = q + QS;
    float* v = k + KS;
    T* row = qkv + (size_t)t * ld;
    for (int i = threadIdx.x; i < QS + KS + VS; i += blockDim.x) sm[i] = to_f32(row[i]);
    __syncthreads();
    const int p = positions[t];
    if (wq) {
        float sq = 0.f, sk = 0.f;
        for (int i = threadIdx.x; i < QS; i += blockDim.x) sq = fmaf(q[i], q[i], sq);
        for (int i = threadIdx.x; i < KS; i += blockDim.x) sk = fmaf(k[i], k[i], sk);
        sq = block_sum(sq, red);
        sk = block_sum(sk, red);
        const float rq = 1.f / sqrtf(sq / (float)QS + eps), rk = 1.f / sqrtf(sk / (float)KS + eps);
        for (int i = threadIdx.x; i < QS; i += blockDim.x) q[i] = q[i] * rq * wq[i];
        for (int i = threadIdx.x; i < KS; i += blockDim.x) k[i] = k[i] * rk * wk[i];
        __syncthreads();
    }
    if (cos_sin && R > 0) {
        const int half = R >> 1;
        const float* cs = cos_sin + (size_t)min(p, table_rows - 1) * R;
        for (int i = threadIdx.x; i < (NH + NKV) * half; i += blockDim.x) {
            const int head = i / half, e = i - head * half;
            float* x = (head < NH ? q + head * D : k + (head - NH) * D);
            const float c = cs[e], s = cs[half + e];
            const float a = x[e], b = x[e + half];
            x[e] = a * c - b * s;
            x[e + half] = b * c + a * s;
        }
        __syncthreads();
    }
    float temp = 1.f;
    if (temp_coef != 0.f && temp_every > 0) temp = 1.f + temp_coef * logf((float)((p + 1) / temp_every + 1));
    for (int i = threadIdx.x; i < QS; i += blockDim.x) row[i] = from_f32<T>(q[i] * temp);
    if (value_norm) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
        for (int g = warp; g < NKV; g += nwarp) {
            float ss = 0.f;
            for (int e = lane; e < DV; e += 32) ss = fmaf(v[g * DV + e], v[g * DV + e], ss);
            ss = warp_sum(ss);
            const float rs = 1.f / sqrtf(ss / (float)DV + value_eps);
            for (int e = lane; e < DV; e += 32) v[g * DV + e] *= rs;
        }
        __syncthreads();
    }
    if (share_mode == 1) {
        for (int i = threadIdx.x; i < VS; i += blockDim.x) shared_v[(size_t)t * VS + i] = v[i];
    } else if (share_mode == 2) {
        for (int i = threadIdx.x; i < VS; i += blockDim.x)
            v[i] = (1.f - lambda) * v[i] + lambda * shared_v[(size_t)t * VS + i];     // (each thread its own elements)
    }
    if (!k_pages) return;
    const int seq = seq_of_token[t];
    const int pg = block_table[(size_t)(bt_rows ? bt_rows[seq] : seq) * bt_stride + p / page_size];
    if (pg < 0 || pg >= num_pages) return;
    const int in_page = p % page_size;
    for (int i = threadIdx.x; i < KS; i += blockDim.x) {
        const int g = i / D, e = i - g * D;
        k_pages[(((size_t)pg * NKV + g) * page_size + in_page) * D + e] = from_f32<T>(k[i]);
    }
    for (int i = threadIdx.x; i < VS; i += blockDim.x) {
        const int g = i / DV, e = i - g * DV;
        v_pages[(((size_t)pg * NKV + g) * page_size + in_page) * DV + e] = from_f32<T>(v[i]);
    }
}

ACV_API int acv_qkv_prepare(void* qkv, int ld, int T_tokens, int NH, int NKV, int D, int DV, const float* wq, const float* wk,
                            float eps, const float* cos_sin, int R, int table_rows, float temp_coef, int temp_every,
                            int value_norm, float value_eps, float* shared_v, int share_mode, float lambda,
                            const int* positions, const int* seq_of_token, const int* block_table, int bt_stride,
                            const int* bt_rows, void* k_pages, void* v_pages, int page_size, int num_pages, int dtype,
                            cudaStream_t stream) {
    if (T_tokens <= 0) return 0;
    if (NH <= 0 || NKV <= 0 || D <= 0 || DV <= 0 || (R & 1) || R > D || (share_mode && !shared_v) || (!wq != !wk))
        return ACV_ERR_SIZE;
    const size_t smem = (size_t)((NH + NKV) * D + NKV * DV) * sizeof(float);
    if (smem > 200 * 1024) return ACV_ERR_SIZE;
    const int threads = smem >= 16 * 1024 ? 256 : 128;
#define QP_LAUNCH(TT)                                                                                                  \
    {                                                                                                                  \
        if (smem > 48 * 1024) {                                                                                        \
            static AcvSmemConfig cfg;                                                                                  \
            if (int e = acv_ensure_smem(cfg, qkv_prepare_kernel<TT>, (int)smem)) return e;                             \
        }                                                                                                              \
        acv_launch(PDL_ROPE, qkv_prepare_kernel<TT>, T_tokens, threads, smem, stream, (TT*)qkv, ld, NH, NKV, D, DV, wq, wk,  \
                   eps, cos_sin, R, table_rows, temp_coef, temp_every, value_norm, value_eps, shared_v, share_mode, lambda, \
                   positions, seq_of_token, block_table, bt_stride, bt_rows, (TT*)k_pages, (TT*)v_pages, page_size, num_pages); \
    }
    if (dtype == ACV_F32) QP_LAUNCH(float)
    else if (dtype == ACV_BF16) QP_LAUNCH(bf16)
    else return ACV_ERR_DTYPE;
#undef QP_LAUNCH
    return acv_launch_status();
}
