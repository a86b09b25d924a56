// An RMS norm taken in groups, and a short causal convolution on a mixer's input, over a float32 residual stream.
//
//   acv_add_group_rmsnorm       x += c * delta (float, written back unless rows are given);
//                               out = x_g / sqrt(mean(x_g^2) + eps) * w for each of the G equal consecutive parts x_g of
//                               the row (G = 1: the plain RMS norm), computed in float, rounded once to out's type
//   acv_input_conv              out[t] = h[t] + sum_j taps[:, j] * h[t - K + 1 + j] along each request's tokens; the K-1
//                               rows before a step's first token come from the request's state slot (float, zero when
//                               the request begins), which is replaced by the step's last K-1 rows
//   acv_add_group_rmsnorm_conv  both for steps in which every request brings one token: one launch, the normed row
//                               never leaves the block
//
// The convolution's tokens that reach back into the state (the first K-1 of a request's portion) are all computed by
// the block of the portion's first token, which then replaces the state: a channel's state is read and written by one
// thread only, whatever else runs in the step.
#include "common.cuh"

#define GN_MAX_GROUPS 4096      // the groups' sums wait in shared memory behind the row

// four neighbouring elements at once (16 bytes of float, 8 of bfloat16)
__device__ __forceinline__ float4 gn_ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 gn_ld4(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                       __uint_as_float(u.y & 0xffff0000u));
}
__device__ __forceinline__ void gn_st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void gn_st4(bf16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&lo);
    u.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}

// sums of squares of the G parts of a row held in shared memory, left in red[0..G) for every thread
__device__ __forceinline__ void group_sums(const float* row, int H, int G, float* red) {
    const int per = H / G;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    // a warp takes whole groups in turn: the order of a group's sum depends on the launch shape only
    for (int g = warp; g < G; g += nwarp) {
        float ss = 0.f;
        for (int i = lane; i < per; i += 32) {
            const float v = row[g * per + i];
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) red[g] = ss;
    }
    __syncthreads();
}

// VEC: the row's length and a group's are multiples of four and every pointer is aligned: four elements a thread and pass
template <typename TD, typename TO, bool VEC>
__global__ void add_group_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, float delta_scale,
                                         const float* __restrict__ w, TO* __restrict__ out, const int* __restrict__ rows,
                                         int H, int G, float eps) {
    extern __shared__ __align__(16) float row[];
    float* red = row + H;                   // [G]
    pdl_launch_dependents();
    pdl_wait();
    const int r_out = blockIdx.x;
    const int r_in = rows ? rows[r_out] : r_out;
    float* xr = x + (size_t)r_in * H;
    const TD* dr = delta ? delta + (size_t)r_in * H : nullptr;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float4 v = gn_ld4(xr + i);
            if (dr) {
                const float4 d = gn_ld4(dr + i);
                v = make_float4(fmaf(delta_scale, d.x, v.x), fmaf(delta_scale, d.y, v.y), fmaf(delta_scale, d.z, v.z),
                                fmaf(delta_scale, d.w, v.w));
                if (!rows) gn_st4(xr + i, v);
            }
            gn_st4(row + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = xr[i];
            if (dr) {
                v = fmaf(delta_scale, to_f32(dr[i]), v);
                if (!rows) xr[i] = v;
            }
            row[i] = v;
        }
    }
    __syncthreads();
    group_sums(row, H, G, red);
    const int per = H / G;
    TO* o = out + (size_t)r_out * H;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float rs = 1.f / sqrtf(red[i / per] / (float)per + eps);
            const float4 v = gn_ld4(row + i), ww = gn_ld4(w + i);
            gn_st4(o + i, make_float4(v.x * rs * ww.x, v.y * rs * ww.y, v.z * rs * ww.z, v.w * rs * ww.w));
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float rs = 1.f / sqrtf(red[i / per] / (float)per + eps);
            o[i] = from_f32<TO>(row[i] * rs * w[i]);
        }
    }
}

template <typename TD, typename TO>
static int launch_group_norm(float* x, const void* delta, float delta_scale, const float* w, void* out, const int* rows,
                             int n_rows, int H, int G, float eps, cudaStream_t stream) {
    const size_t smem = (size_t)(H + G) * sizeof(float);
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    const bool vec = H % 4 == 0 && (H / G) % 4 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)delta & 15) && !((uintptr_t)w & 15) &&
                     !((uintptr_t)out & 15);
    if (smem > 48 * 1024) {
        static AcvSmemConfig cfg, cfg_v;
        if (int e = vec ? acv_ensure_smem(cfg_v, add_group_rmsnorm_kernel<TD, TO, true>, (int)smem)
                        : acv_ensure_smem(cfg, add_group_rmsnorm_kernel<TD, TO, false>, (int)smem)) return e;
    }
    if (vec)
        acv_launch(PDL_NORM, add_group_rmsnorm_kernel<TD, TO, true>, n_rows, threads, smem, stream, x, (const TD*)delta,
                   delta_scale, w, (TO*)out, rows, H, G, eps);
    else
        acv_launch(PDL_NORM, add_group_rmsnorm_kernel<TD, TO, false>, n_rows, threads, smem, stream, x, (const TD*)delta,
                   delta_scale, w, (TO*)out, rows, H, G, eps);
    return acv_launch_status();
}

// delta_dtype: the type of delta (ignored without one); out_dtype: the type of out
ACV_API int acv_add_group_rmsnorm(float* x, const void* delta, float delta_scale, const float* w, void* out, const int* rows,
                                  int n_rows, int H, int groups, float eps, int delta_dtype, int out_dtype,
                                  cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (groups < 1 || groups > GN_MAX_GROUPS || H % groups || (size_t)(H + groups) * 4 > 200 * 1024) return ACV_ERR_SIZE;
    if (!delta) delta_dtype = out_dtype;
#define GN_CASE(D, TD, O, TO)                                                                                        \
    if (delta_dtype == D && out_dtype == O)                                                                           \
        return launch_group_norm<TD, TO>(x, delta, delta_scale, w, out, rows, n_rows, H, groups, eps, stream);
    GN_CASE(ACV_F32, float, ACV_F32, float)
    GN_CASE(ACV_BF16, bf16, ACV_BF16, bf16)
    GN_CASE(ACV_BF16, bf16, ACV_F32, float)
    GN_CASE(ACV_F32, float, ACV_BF16, bf16)
#undef GN_CASE
    return ACV_ERR_DTYPE;
}

// ----------------------------------------------------------------------------- the convolution
// h float [T, C]; taps float [C, K] (tap K-1 meets the token itself); state float [slots, K-1, C], oldest row first.
// grid (tokens, channel tiles).
template <typename TO>
__global__ void input_conv_kernel(const float* __restrict__ h, const float* __restrict__ taps, float* __restrict__ state,
                                  const int* __restrict__ slots, const int* __restrict__ cu_q,
                                  const int* __restrict__ seq_of_token, TO* __restrict__ out, int C, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int seq = seq_of_token[t];
    const int first = cu_q[seq], len = cu_q[seq + 1] - first;
    const int off = t - first;
    const float* wc = taps + (size_t)c * K;
    if (off >= K - 1) {
        float acc = h[(size_t)t * C + c];
        for (int j = 0; j < K; ++j) acc = fmaf(wc[j], h[(size_t)(t - K + 1 + j) * C + c], acc);
        out[(size_t)t * C + c] = from_f32<TO>(acc);
        return;
    }
    if (off != 0) return;
    float* st = state + (size_t)slots[seq] * (K - 1) * C;
    const int n_here = len < K - 1 ? len : K - 1;
    for (int n = 0; n < n_here; ++n) {
        float acc = h[(size_t)(first + n) * C + c];
        for (int j = 0; j < K; ++j) {
            const int src = n - K + 1 + j;          // a row of the portion, or (negative) of the state
            const float v = src >= 0 ? h[(size_t)(first + src) * C + c] : st[(size_t)(K - 1 + src) * C + c];
            acc = fmaf(wc[j], v, acc);
        }
        out[(size_t)(first + n) * C + c] = from_f32<TO>(acc);
    }
    for (int i = 0; i < K - 1; ++i) {       // ascending: what is read lies behind what has been written
        const int src = len - (K - 1) + i;
        st[(size_t)i * C + c] = src >= 0 ? h[(size_t)(first + src) * C + c] : st[(size_t)(len + i) * C + c];
    }
}

// The same with four neighbouring channels to a thread (16-byte loads of h and of the state): C a multiple of four, taps
// transposed ([K][C]) so that a lag's four taps are one vector.  TO is float (float4 stores) or bf16 (8-byte stores).
__device__ __forceinline__ float4 ic_fma(float4 w, float4 v, float4 acc) {
    return make_float4(fmaf(w.x, v.x, acc.x), fmaf(w.y, v.y, acc.y), fmaf(w.z, v.z, acc.z), fmaf(w.w, v.w, acc.w));
}
__device__ __forceinline__ void ic_store(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void ic_store(bf16* dst, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&lo);
    u.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = u;
}

template <typename TO>
__global__ void input_conv4_kernel(const float* __restrict__ h, const float* __restrict__ taps_t, float* __restrict__ state,
                                   const int* __restrict__ slots, const int* __restrict__ cu_q,
                                   const int* __restrict__ seq_of_token, TO* __restrict__ out, int C, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= C) return;
    const int seq = seq_of_token[t];
    const int first = cu_q[seq], len = cu_q[seq + 1] - first;
    const int off = t - first;
    auto tap = [&](int j) { return *reinterpret_cast<const float4*>(taps_t + (size_t)j * C + c); };
    auto in = [&](int row) { return *reinterpret_cast<const float4*>(h + (size_t)row * C + c); };
    if (off >= K - 1) {
        float4 acc = in(t);
        for (int j = 0; j < K; ++j) acc = ic_fma(tap(j), in(t - K + 1 + j), acc);
        ic_store(out + (size_t)t * C + c, acc);
        return;
    }
    if (off != 0) return;
    float* st = state + (size_t)slots[seq] * (K - 1) * C;
    const int n_here = len < K - 1 ? len : K - 1;
    for (int n = 0; n < n_here; ++n) {
        float4 acc = in(first + n);
        for (int j = 0; j < K; ++j) {
            const int src = n - K + 1 + j;
            const float4 v = src >= 0 ? in(first + src) : *reinterpret_cast<const float4*>(st + (size_t)(K - 1 + src) * C + c);
            acc = ic_fma(tap(j), v, acc);
        }
        ic_store(out + (size_t)(first + n) * C + c, acc);
    }
    for (int i = 0; i < K - 1; ++i) {       // ascending: what is read lies behind what has been written
        const int src = len - (K - 1) + i;
        const float4 v = src >= 0 ? in(first + src) : *reinterpret_cast<const float4*>(st + (size_t)(len + i) * C + c);
        *reinterpret_cast<float4*>(st + (size_t)i * C + c) = v;
    }
}

// taps_t (may be null): the taps transposed, [K][C]; with it, C a multiple of four and aligned pointers, a thread takes
// four neighbouring channels
ACV_API int acv_input_conv(const float* h, const float* taps, float* state, const int* slots, const int* cu_q,
                           const int* seq_of_token, void* out, int T, int C, int K, int out_dtype, const float* taps_t,
                           cudaStream_t stream) {
    if (T <= 0) return 0;
    if (C <= 0 || K < 1) return ACV_ERR_SIZE;
    if (taps_t && C % 4 == 0 && !((uintptr_t)h & 15) && !((uintptr_t)taps_t & 15) && !((uintptr_t)state & 15) && !((uintptr_t)out & 15)) {
        dim3 grid4(T, (C / 4 + 127) / 128);
        if (out_dtype == ACV_F32)
            acv_launch(PDL_MISC, input_conv4_kernel<float>, grid4, 128, 0, stream, h, taps_t, state, slots, cu_q, seq_of_token, (float*)out, C, K);
        else if (out_dtype == ACV_BF16)
            acv_launch(PDL_MISC, input_conv4_kernel<bf16>, grid4, 128, 0, stream, h, taps_t, state, slots, cu_q, seq_of_token, (bf16*)out, C, K);
        else
            return ACV_ERR_DTYPE;
        return acv_launch_status();
    }
    dim3 grid(T, (C + 127) / 128);
    if (out_dtype == ACV_F32)
        acv_launch(PDL_MISC, input_conv_kernel<float>, grid, 128, 0, stream, h, taps, state, slots, cu_q, seq_of_token, (float*)out, C, K);
    else if (out_dtype == ACV_BF16)
        acv_launch(PDL_MISC, input_conv_kernel<bf16>, grid, 128, 0, stream, h, taps, state, slots, cu_q, seq_of_token, (bf16*)out, C, K);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- both, one token a request
// Row r is request r's one token: sum, grouped norm, convolution over the state's rows and the normed row, the state
// shifted by one row.  One block a row.
template <typename TD, typename TO>
__global__ void add_group_rmsnorm_conv_kernel(float* __restrict__ x, const TD* __restrict__ delta, float delta_scale,
                                              const float* __restrict__ w, const float* __restrict__ taps,
                                              float* __restrict__ state, const int* __restrict__ slots, TO* __restrict__ out,
                                              int H, int G, float eps, int K) {
    extern __shared__ float row[];
    float* red = row + H;                   // [G]
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * H;
    const TD* dr = delta ? delta + (size_t)r * H : nullptr;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (dr) {
            v = fmaf(delta_scale, to_f32(dr[i]), v);
            xr[i] = v;
        }
        row[i] = v;
    }
    __syncthreads();
    group_sums(row, H, G, red);
    const int per = H / G;
    float* st = state + (size_t)slots[r] * (K - 1) * H;
    TO* o = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float rs = 1.f / sqrtf(red[i / per] / (float)per + eps);
        const float hv = row[i] * rs * w[i];
        const float* wc = taps + (size_t)i * K;
        float acc = fmaf(wc[K - 1], hv, hv);
        for (int j = 0; j < K - 1; ++j) {
            const float v = st[(size_t)j * H + i];
            acc = fmaf(wc[j], v, acc);
            if (j > 0) st[(size_t)(j - 1) * H + i] = v;
        }
        if (K > 1) st[(size_t)(K - 2) * H + i] = hv;
        o[i] = from_f32<TO>(acc);
    }
}

template <typename TD, typename TO>
static int launch_group_norm_conv(float* x, const void* delta, float delta_scale, const float* w, const float* taps,
                                  float* state, const int* slots, void* out, int n_rows, int H, int G, float eps, int K,
                                  cudaStream_t stream) {
    const size_t smem = (size_t)(H + G) * sizeof(float);
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    if (smem > 48 * 1024) {
        static AcvSmemConfig cfg;
        if (int e = acv_ensure_smem(cfg, add_group_rmsnorm_conv_kernel<TD, TO>, (int)smem)) return e;
    }
    acv_launch(PDL_NORM, add_group_rmsnorm_conv_kernel<TD, TO>, n_rows, threads, smem, stream, x, (const TD*)delta, delta_scale,
               w, taps, state, slots, (TO*)out, H, G, eps, K);
    return acv_launch_status();
}

ACV_API int acv_add_group_rmsnorm_conv(float* x, const void* delta, float delta_scale, const float* w, const float* taps,
                                       float* state, const int* slots, void* out, int n_rows, int H, int groups, float eps,
                                       int K, int delta_dtype, int out_dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (groups < 1 || groups > GN_MAX_GROUPS || H % groups || (size_t)(H + groups) * 4 > 200 * 1024 || K < 1) return ACV_ERR_SIZE;
    if (!delta) delta_dtype = out_dtype;
#define GN_CASE(D, TD, O, TO)                                                                                        \
    if (delta_dtype == D && out_dtype == O)                                                                           \
        return launch_group_norm_conv<TD, TO>(x, delta, delta_scale, w, taps, state, slots, out, n_rows, H, groups, eps, K, stream);
    GN_CASE(ACV_F32, float, ACV_F32, float)
    GN_CASE(ACV_BF16, bf16, ACV_BF16, bf16)
#undef GN_CASE
    return ACV_ERR_DTYPE;
}
