// Attention whose keys and values are made from one kept latent per token.
//
// Per token the layer keeps one row [c | r]: c = the normed latent (KR elements), r = a rotated key part (R elements)
// that all heads share.  Head h's key is [W_uk,h c | r] and its value W_uv,h c.  The products with W_uk and W_uv move
// to the query's side, where they cost one product per query instead of one per (query, key):
//
//   <q_h, W_uk,h c> = <W_uk,h^T q_h, c>             the query the kept rows are scored with: [W_uk,h^T q_h | q_rot,h]
//   sum_j p_j W_uv,h c_j = W_uv,h (sum_j p_j c_j)   the weighted sum is taken over the latents, then projected
//
// so the attention itself is one key/value head of KR + R elements whose values are the first KR elements of the same
// rows (the generic paged kernel with v_pages == k_pages), read by every query head.
//
// acv_latent_prepare, one block a token:
//   kv row [KR + R] of the down projection: c = kv[:KR] / sqrt(mean(kv[:KR]^2) + eps) * w (32-bit), r = rot(kv[KR:]);
//     [c | r] goes into the token's row of its page (a page index < 0 writes nothing);
//   q rows [H][D + R]: rot(q_h[D:]) goes to q_out[h][KR:], beside the place where the caller's per-head product leaves
//     W_uk,h^T q_h[:D].
// rot turns the interleaved pairs (2i, 2i+1), 2i < rot, by the angle of pair i at the token's position (cos and sin
// from a float table [positions][rot]: rot/2 cosines, then rot/2 sines); elements from rot on pass unchanged.
#include "common.cuh"

__device__ __forceinline__ float rot_interleaved(const float* x, int e, int rot, const float* cs) {
    if (e >= rot) return x[e];
    const int i = e >> 1;
    const float c = cs[i], s = cs[(rot >> 1) + i];
    return (e & 1) ? fmaf(x[e], c, x[e - 1] * s) : fmaf(x[e], c, -x[e + 1] * s);
}

template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ q_out, int qo_stride,
                                      const T* __restrict__ kv, int kv_stride, const float* __restrict__ w, float eps,
                                      const float* __restrict__ cos_sin, int rot, int table_rows,
                                      const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                      const int* __restrict__ block_table, int bt_stride, const int* __restrict__ bt_rows,
                                      T* __restrict__ pages, int page_size, int num_pages, int H, int D, int R, int KR) {
    extern __shared__ float sm[];           // [KR + R] the kv row, then [H * R] the heads' rotated parts
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x, nthr = blockDim.x;
    int pos = positions[t];
    if (pos >= table_rows) pos = table_rows - 1;
    const float* cs = cos_sin + (size_t)pos * rot;
    float* row = sm;
    float* qr = sm + KR + R;
    const T* kvr = kv + (size_t)t * kv_stride;
    float ss = 0.f;
    for (int e = tid; e < KR + R; e += nthr) {
        const float v = to_f32(kvr[e]);
        row[e] = v;
        if (e < KR) ss = fmaf(v, v, ss);
    }
    for (int i = tid; i < H * R; i += nthr) {
        const int h = i / R, e = i - h * R;
        qr[i] = to_f32(q[(size_t)t * q_stride + (size_t)h * (D + R) + D + e]);
    }
    ss = block_sum(ss, red);                // (meets the block: row and qr are whole)
    const float inv = 1.f / sqrtf(ss / (float)KR + eps);
    for (int i = tid; i < H * R; i += nthr) {
        const int h = i / R, e = i - h * R;
        q_out[(size_t)t * qo_stride + (size_t)h * (KR + R) + KR + e] = from_f32<T>(rot_interleaved(qr + h * R, e, rot, cs));
    }
    if (!pages) return;
    const int seq = seq_of_token[t];
    const int pg = block_table[(size_t)(bt_rows ? bt_rows[seq] : seq) * bt_stride + positions[t] / page_size];
    if (pg < 0 || pg >= num_pages) return;
    T* dst = pages + ((size_t)pg * page_size + (positions[t] % page_size)) * (KR + R);
    for (int e = tid; e < KR; e += nthr) dst[e] = from_f32<T>(row[e] * inv * w[e]);
    for (int e = tid; e < R; e += nthr) dst[KR + e] = from_f32<T>(rot_interleaved(row + KR, e, rot, cs));
}

// q: rows of H*(D+R) at q_stride; q_out: rows of H*(KR+R) at qo_stride; kv: rows of KR+R at kv_stride; w float [KR];
// cos_sin float [table_rows][rot]; pages [num_pages][1][page_size][KR+R] (null: nothing is kept, queries only).
ACV_API int acv_latent_prepare(const void* q, int q_stride, void* q_out, int qo_stride, const void* kv, int kv_stride,
                               const float* w, float eps, const float* cos_sin, int rot, int table_rows,
                               const int* positions, const int* seq_of_token, const int* block_table, int bt_stride,
                               const int* bt_rows, void* pages, int page_size, int num_pages, int T_tokens, int H, int D,
                               int R, int KR, int dtype, cudaStream_t stream) {
    if (T_tokens <= 0) return 0;
    if (H <= 0 || D < 0 || R <= 0 || KR <= 0 || rot < 0 || rot > R || (rot & 1) || (rot && (!cos_sin || table_rows <= 0)))
        return ACV_ERR_SIZE;
    const size_t smem = (size_t)(KR + R + H * R) * sizeof(float);
    if (smem > 200 * 1024) return ACV_ERR_SIZE;
    const int threads = 256;
#define LP_LAUNCH(T)                                                                                                    \
    do {                                                                                                                \
        if (smem > 48 * 1024) {                                                                                         \
            static AcvSmemConfig cfg;                                                                                   \
            const int e = acv_ensure_smem(cfg, latent_prepare_kernel<T>, (int)smem);                                    \
            if (e) return e;                                                                                            \
        }                                                                                                               \
        acv_launch(PDL_ROPE, latent_prepare_kernel<T>, T_tokens, threads, smem, stream, (const T*)q, q_stride, (T*)q_out, \
                   qo_stride, (const T*)kv, kv_stride, w, eps, cos_sin, rot, table_rows, positions, seq_of_token,       \
                   block_table, bt_stride, bt_rows, (T*)pages, page_size, num_pages, H, D, R, KR);                      \
    } while (0)
    if (dtype == ACV_F32) LP_LAUNCH(float);
    else if (dtype == ACV_BF16) LP_LAUNCH(bf16);
    else return ACV_ERR_DTYPE;
#undef LP_LAUNCH
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- RMS norm of rows at any stride
// out[r][:] = x[r][:] / sqrt(mean(x[r]^2) + eps) * w, 32-bit, rounded once; x and out are column ranges of wider
// matrices (a latent inside a stacked projection's output).  One block a row.
template <typename T>
__global__ void rmsnorm_rows_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ w, float eps,
                                    T* __restrict__ out, int ldo, int H) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const T* xr = x + (size_t)blockIdx.x * ldx;
    T* o = out + (size_t)blockIdx.x * ldo;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = to_f32(xr[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<T>(to_f32(xr[i]) * inv * (w ? w[i] : 1.f));
}

ACV_API int acv_rmsnorm_rows(const void* x, int ldx, const float* w, float eps, void* out, int ldo, int n_rows, int H,
                             int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0) return ACV_ERR_SIZE;
    const int threads = H >= 2048 ? 256 : 128;
    if (dtype == ACV_F32)
        acv_launch(PDL_NORM, rmsnorm_rows_kernel<float>, n_rows, threads, 0, stream, (const float*)x, ldx, w, eps, (float*)out, ldo, H);
    else if (dtype == ACV_BF16)
        acv_launch(PDL_NORM, rmsnorm_rows_kernel<bf16>, n_rows, threads, 0, stream, (const bf16*)x, ldx, w, eps, (bf16*)out, ldo, H);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}
