// Paged causal attention whose scores are mixed across the heads before the softmax.
//
// For the query at position i and the key at position j <= i (and j > i - window where window > 0), per head g:
//
//   s_g = <q_g, k_kv(g)> * scale * temp[g]                     temp null: 1
//   s_g = cap * tanh(s_g / cap)                                 cap <= 0: none
//   s_g += rel[bucket(i - j)][g]                                rel null: none
//   m_h = sum_g talk[h][g] * s_g                                talk null: m = s
//   p_h = softmax_j(m_h),   o_h = sum_j p_h[j] v_kv(h)[j]
//
// bucket(n) comes from a table of the first `n_dist` distances (made by the caller, in double precision); every larger
// distance reads the last row of rel.  q-head h reads kv-head h / (NH/NKV).  Scores, the mix, the softmax and the
// weighted sums are 32-bit; q, pages and out are float or bfloat16.
//
// A head's softmax needs every head's score of the same (query, key) pair, so a block owns all heads of its queries:
//
// acv_attention_mixed (any sizes; the 32-bit path): one block a query token, one warp a head (two heads a warp from 33
// heads on, up to 64).  For a tile of 32 keys
// warp g leaves its 32 scores in shared memory, the block meets, warp h mixes its row of `talk` over them and goes on
// as a flash-attention warp of its own head (running maximum and sum, values of its kv-head).
#include "common.cuh"

template <typename T, int NR, int HPW>
__global__ void attn_mixed_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                                  const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                  const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                  const int* __restrict__ block_table, int bt_stride, const int* __restrict__ bt_rows,
                                  int NH, int NKV, int D, int DV, int page_size, int num_pages, float scale, int window,
                                  const float* __restrict__ temp, float cap, const float* __restrict__ rel,
                                  const int* __restrict__ bucket_of, int n_dist, int last_row,
                                  const float* __restrict__ talk) {
    extern __shared__ float sm_all[];
    float* qs = sm_all;                     // [NH][D], scaled
    float* sc = qs + (size_t)NH * D;        // [NH][32] scores of the tile, before the mix
    float* tk = sc + (size_t)NH * 32;       // [NH][NH]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    // a warp's heads: warp, warp + nw, ... (HPW of them; more than 32 heads share the block's 32 warps)
    const int t = blockIdx.x;
    const int group = NH / NKV;
    const int p = positions[t];
    const int seq = seq_of_token[t];
    const int* bt = block_table + (size_t)(bt_rows ? bt_rows[seq] : seq) * bt_stride;
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int h = warp + i * nw;
        if (h >= NH) break;
        const T* qrow = q + (size_t)t * q_stride + (size_t)h * D;
        const float qscale = scale * (temp ? temp[h] : 1.f);
        for (int e = lane; e < D; e += 32) qs[h * D + e] = to_f32(qrow[e]) * qscale;
        for (int g = lane; g < NH; g += 32) tk[h * NH + g] = talk ? talk[h * NH + g] : (g == h ? 1.f : 0.f);
    }
    __syncthreads();
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;

    float acc[HPW][NR];
    float m[HPW], l[HPW];
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[i][r] = 0.f;
    }
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    for (int j0 = lo; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        bool valid = j <= p;
        long long page_row = 0;             // the key's row in kv-head 0 of its page
        if (valid) {
            const int pg = bt[j / page_size];
            valid = pg >= 0 && pg < num_pages;
            page_row = (long long)pg * NKV * page_size + (j % page_size);
        }
#pragma unroll
        for (int i = 0; i < HPW; ++i) {
            const int h = warp + i * nw;
            if (h >= NH) break;
            float s = 0.f;
            if (valid) {
                const T* kr = k_pages + (page_row + (long long)(h / group) * page_size) * D;
                const float* qh = qs + h * D;
                float dot = 0.f;
                for (int e = 0; e < D; ++e) dot = fmaf(qh[e], to_f32(kr[e]), dot);
                if (cap > 0.f) dot = cap * tanhf(dot * inv_cap);
                if (rel) {
                    const int dist = p - j;
                    dot += rel[(size_t)(dist < n_dist ? bucket_of[dist] : last_row) * NH + h];
                }
                s = dot;
            }
            sc[h * 32 + lane] = s;
        }
        __syncthreads();
        float mixed[HPW];
#pragma unroll
        for (int i = 0; i < HPW; ++i) {
            const int h = warp + i * nw;
            mixed[i] = 0.f;
            if (h >= NH) break;
            for (int g = 0; g < NH; ++g) mixed[i] = fmaf(tk[h * NH + g], sc[g * 32 + lane], mixed[i]);
        }
        __syncthreads();                    // the next tile's scores overwrite sc
        const int n_in_tile = min(32, p - j0 + 1);
#pragma unroll
        for (int i = 0; i < HPW; ++i) {
            const int h = warp + i * nw;
            if (h >= NH) break;
            const float s = valid ? mixed[i] : -INFINITY;
            const float tmax = warp_max(s);
            if (tmax == -INFINITY) continue;    // uniform in the warp
            const float m_new = fmaxf(m[i], tmax);
            const float alpha = expf(m[i] - m_new);
            const float pl = valid ? expf(s - m_new) : 0.f;
            l[i] = l[i] * alpha + warp_sum(pl);
            m[i] = m_new;
#pragma unroll
            for (int r = 0; r < NR; ++r) acc[i][r] *= alpha;
            const long long head_rows = (long long)(h / group) * page_size;
            for (int kk = 0; kk < n_in_tile; ++kk) {
                const float pk = __shfl_sync(0xffffffffu, pl, kk);
                const long long ro = __shfl_sync(0xffffffffu, page_row, kk);
                if (pk == 0.f) continue;
                const T* vr = v_pages + (ro + head_rows) * DV;
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const int e = lane + 32 * r;
                    if (e < DV) acc[i][r] = fmaf(pk, to_f32(vr[e]), acc[i][r]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int h = warp + i * nw;
        if (h >= NH) break;
        T* orow = out + (size_t)t * out_stride + (size_t)h * DV;
        const float inv_l = l[i] > 0.f ? 1.f / l[i] : 0.f;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const int e = lane + 32 * r;
            if (e < DV) orow[e] = from_f32<T>(acc[i][r] * inv_l);
        }
    }
}

template <typename T>
static int launch_mixed(const void* q, int q_stride, void* out, int out_stride, const void* k_pages, const void* v_pages,
                        const int* positions, const int* seq_of_token, const int* block_table, int bt_stride,
                        const int* bt_rows, int T_tokens, int NH, int NKV, int D, int DV, int page_size, int num_pages,
                        float scale, int window, const float* temp, float cap, const float* rel, const int* bucket_of,
                        int n_dist, int last_row, const float* talk, cudaStream_t stream) {
    const size_t smem = ((size_t)NH * D + (size_t)NH * 32 + (size_t)NH * NH) * sizeof(float);
    if (smem > 200 * 1024) return ACV_ERR_SIZE;
    const int nr = (DV + 31) / 32;
    const int hpw = (NH + 31) / 32, nw = (NH + hpw - 1) / hpw;      // heads of a warp; warps of a block
    if (hpw > 2) return ACV_ERR_SIZE;
#define AM_LAUNCH(N, W)                                                                                                \
    {                                                                                                                  \
        if (smem > 48 * 1024) {                                                                                        \
            static AcvSmemConfig cfg;                                                                                  \
            const int e = acv_ensure_smem(cfg, attn_mixed_kernel<T, N, W>, (int)smem);                                 \
            if (e) return e;                                                                                           \
        }                                                                                                              \
        acv_launch(PDL_ATTN, attn_mixed_kernel<T, N, W>, T_tokens, nw * 32, smem, stream, (const T*)q, q_stride,       \
                   (T*)out, out_stride, (const T*)k_pages, (const T*)v_pages, positions, seq_of_token, block_table,    \
                   bt_stride, bt_rows, NH, NKV, D, DV, page_size, num_pages, scale, window, temp, cap, rel, bucket_of, \
                   n_dist, last_row, talk);                                                                            \
    }
#define AM_CASE(N)                                                                                                     \
    case N:                                                                                                            \
        if (hpw == 1) AM_LAUNCH(N, 1) else AM_LAUNCH(N, 2)                                                             \
        break;
    switch (nr) {
        AM_CASE(1) AM_CASE(2) AM_CASE(3) AM_CASE(4) AM_CASE(5) AM_CASE(6) AM_CASE(7) AM_CASE(8)
        default: return ACV_ERR_SIZE;
    }
#undef AM_LAUNCH
#undef AM_CASE
    return acv_launch_status();
}

// q: rows of NH*D at q_stride; out: rows of NH*DV; pages [NP][NKV][page][D] and [..][DV]; temp float [NH]; rel float
// [rows][NH]; bucket_of int [n_dist]; talk float [NH][NH].
ACV_API int acv_attention_mixed(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                const void* v_pages, const int* positions, const int* seq_of_token,
                                const int* block_table, int bt_stride, const int* bt_rows, int T_tokens, int NH, int NKV,
                                int D, int DV, int page_size, int num_pages, float scale, int window, const float* temp,
                                float cap, const float* rel, const int* bucket_of, int n_dist, int last_row,
                                const float* talk, int dtype, cudaStream_t stream) {
    if (T_tokens <= 0) return 0;
    if (D <= 0 || DV <= 0 || DV > 256 || NKV <= 0 || NH % NKV || NH > 64) return ACV_ERR_SIZE;
    if (rel && (!bucket_of || n_dist < 0 || last_row < 0)) return ACV_ERR_SIZE;
    if (dtype == ACV_F32)
        return launch_mixed<float>(q, q_stride, out, out_stride, k_pages, v_pages, positions, seq_of_token, block_table,
                                   bt_stride, bt_rows, T_tokens, NH, NKV, D, DV, page_size, num_pages, scale, window, temp,
                                   cap, rel, bucket_of, n_dist, last_row, talk, stream);
    if (dtype == ACV_BF16)
        return launch_mixed<bf16>(q, q_stride, out, out_stride, k_pages, v_pages, positions, seq_of_token, block_table,
                                  bt_stride, bt_rows, T_tokens, NH, NKV, D, DV, page_size, num_pages, scale, window, temp,
                                  cap, rel, bucket_of, n_dist, last_row, talk, stream);
    return ACV_ERR_DTYPE;
}
