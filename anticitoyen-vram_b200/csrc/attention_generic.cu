// Paged causal attention, generic form: any number of query tokens per request,
// any head size up to 1024 (value rows may have another size than key rows, DV != D, up to 512; with v_pages == k_pages
// and v_row = D the values are the first DV elements of the key rows themselves: one kept row per token serves as key
// and as value, as a latent that every head reads does), float or bfloat16 pages.  One warp per
// (query token, query head).  It is the 32-bit path of the engine and the
// fallback of the bfloat16 path for head sizes the tensor-core kernels do not take.
//
// Query-head h reads kv-head h / (NH/NKV) (acvram/engine/layers.py:1012-1017).
// The keys of the step's own tokens are already in the pages, so the query at
// absolute position p sees the keys j <= p, and with a window w > 0 only
// j > p - w (mask aligned to absolute positions, acvram/engine/layers.py:1020-1041); with keep_first = f > 0 the
// first f keys of the request stay visible to every later query, whatever the window (they keep their own
// positions: nothing is shifted).
// s = scale * q.k - slope_h * (p - j) (slopes: one per query head, or none); with sinks (one number per query head) the
// softmax's denominator also holds exp(sink_h), which has no key and no value.  Softmax over the visible keys with a running maximum and sum in
// 32-bit (acvram/kernels/acvram_kernels.cu:993-1146 has the same recurrence).
#include "common.cuh"

#define AG_WARPS 4

template <typename T, int NR>
__global__ void attn_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                                    const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ bt_rows, int NH, int NKV, int D, int DV,
                                    int page_size, int num_pages, float scale, int window, int keep_first, int v_row,
                                    const float* __restrict__ sinks, const float* __restrict__ slopes) {
    extern __shared__ float sm_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * AG_WARPS + warp;
    const int t = blockIdx.x;
    if (h >= NH) return;
    float* qs = sm_all + warp * D;
    const int kvh = h / (NH / NKV);
    const int p = positions[t];
    const int seq = seq_of_token[t];
    const int* bt = block_table + (size_t)(bt_rows ? bt_rows[seq] : seq) * bt_stride;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * D;
    for (int e = lane; e < D; e += 32) qs[e] = to_f32(qrow[e]) * scale;
    __syncwarp();

    float acc[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = 0.f;
    float m = -INFINITY, l = 0.f;
    const float slope = slopes ? slopes[h] : 0.f;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    // two runs of keys: the kept first ones that the window has passed, [0, min(keep_first, lo)), then [lo, p]
    const int kept = window > 0 ? min(max(keep_first, 0), lo) : 0;

    for (int run = kept > 0 ? 0 : 1; run < 2; ++run) {
    const int j_begin = run == 0 ? 0 : lo, j_last = run == 0 ? kept - 1 : p;
    for (int j0 = j_begin; j0 <= j_last; j0 += 32) {
        const int j = j0 + lane;
        bool valid = j <= j_last;
        long long row = 0;
        if (valid) {
            const int pg = bt[j / page_size];
            valid = pg >= 0 && pg < num_pages;
            row = ((long long)pg * NKV + kvh) * page_size + (j % page_size);
        }
        float s = -INFINITY;
        if (valid) {
            const T* kr = k_pages + row * D;
            float dot = 0.f;
            if ((D & 7) == 0 && sizeof(T) == 2) {       // rows of 16-byte pieces: eight elements a load
                const uint4* kv = reinterpret_cast<const uint4*>(kr);
                for (int e = 0; e < D; e += 8) {
                    const uint4 u = kv[e >> 3];
                    const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        dot = fmaf(qs[e + 2 * i], __uint_as_float(w4[i] << 16), dot);
                        dot = fmaf(qs[e + 2 * i + 1], __uint_as_float(w4[i] & 0xffff0000u), dot);
                    }
                }
            } else {
                for (int e = 0; e < D; ++e) dot = fmaf(qs[e], to_f32(kr[e]), dot);
            }
            s = dot - slope * (float)(p - j);
        }
        const float tmax = warp_max(s);
        if (tmax == -INFINITY) continue;  // uniform: no readable key in this tile
        const float m_new = fmaxf(m, tmax);
        const float alpha = expf(m - m_new);
        const float pl = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(pl);
        m = m_new;
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] *= alpha;
        const int n_in_tile = min(32, j_last - j0 + 1);
        for (int kk = 0; kk < n_in_tile; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, pl, kk);
            const long long ro = __shfl_sync(0xffffffffu, row, kk);
            if (pk == 0.f) continue;
            const T* vr = v_pages + ro * v_row;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const int e = lane + 32 * r;
                if (e < DV) acc[r] = fmaf(pk, to_f32(vr[e]), acc[r]);
            }
        }
    }
    }
    if (sinks) {        // a score without key or value: it takes its share of the weights and adds nothing
        const float sink = sinks[h];
        const float m_new = fmaxf(m, sink);
        const float alpha = expf(m - m_new);
        l = l * alpha + expf(sink - m_new);
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] *= alpha;
    }
    T* orow = out + (size_t)t * out_stride + (size_t)h * DV;
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int e = lane + 32 * r;
        if (e < DV) orow[e] = from_f32<T>(acc[r] * inv_l);
    }
}

template <typename T>
static int launch_generic(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                          const void* v_pages, const int* positions, const int* seq_of_token, const int* block_table,
                          int bt_stride, const int* bt_rows, int T_tokens, int NH, int NKV, int D, int DV, int page_size, int num_pages,
                          float scale, int window, int keep_first, int v_row, const float* sinks, const float* slopes, cudaStream_t stream) {
    dim3 grid(T_tokens, (NH + AG_WARPS - 1) / AG_WARPS);
    const size_t smem = (size_t)AG_WARPS * D * sizeof(float);
    const int nr = (DV + 31) / 32;
#define AG_CASE(N)                                                                                                   \
    case N:                                                                                                          \
        attn_generic_kernel<T, N><<<grid, AG_WARPS * 32, smem, stream>>>(                                            \
            (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_pages, (const T*)v_pages, positions,             \
            seq_of_token, block_table, bt_stride, bt_rows, NH, NKV, D, DV, page_size, num_pages, scale, window, keep_first, v_row, sinks, slopes);                \
        break;
    switch (nr) {
        AG_CASE(1) AG_CASE(2) AG_CASE(3) AG_CASE(4) AG_CASE(5) AG_CASE(6) AG_CASE(7) AG_CASE(8)
        AG_CASE(9) AG_CASE(10) AG_CASE(11) AG_CASE(12) AG_CASE(13) AG_CASE(14) AG_CASE(15) AG_CASE(16)
        default: return ACV_ERR_SIZE;
    }
#undef AG_CASE
    return acv_launch_status();
}

ACV_API int acv_attention_generic(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                  const void* v_pages, const int* positions, const int* seq_of_token,
                                  const int* block_table, int bt_stride, const int* bt_rows, int T_tokens, int NH, int NKV, int D,
                                  int page_size, int num_pages, float scale, int window, int dtype,
                                  int value_dim, int keep_first, const float* sinks, const float* slopes, cudaStream_t stream) {
    if (T_tokens <= 0) return 0;
    const int DV = value_dim > 0 ? value_dim : D;
    if (D <= 0 || D > 1024 || DV > 512 || NKV <= 0 || NH % NKV) return ACV_ERR_SIZE;
    // values inside the key rows: the same pages, rows of D elements
    const int v_row = v_pages == k_pages ? D : DV;
    if (v_row < DV) return ACV_ERR_SIZE;
    if (dtype == ACV_F32)
        return launch_generic<float>(q, q_stride, out, out_stride, k_pages, v_pages, positions, seq_of_token,
                                     block_table, bt_stride, bt_rows, T_tokens, NH, NKV, D, DV, page_size, num_pages, scale, window,
                                     keep_first, v_row, sinks, slopes, stream);
    if (dtype == ACV_BF16)
        return launch_generic<bf16>(q, q_stride, out, out_stride, k_pages, v_pages, positions, seq_of_token,
                                    block_table, bt_stride, bt_rows, T_tokens, NH, NKV, D, DV, page_size, num_pages, scale, window,
                                    keep_first, v_row, sinks, slopes, stream);
    return ACV_ERR_DTYPE;
}
