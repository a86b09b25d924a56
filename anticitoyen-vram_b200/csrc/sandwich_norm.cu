// Norms on both sides of a part, over a float residual stream, and two small helpers of such layers.
//
//   x += delta / sqrt(mean(delta^2) + eps_b) * w_b          (the norm behind a part, as its output joins the stream)
//   out = x / sqrt(mean(x^2) + eps) * w                     (the norm in front of the next part; optional)
//
// Both in one launch, one block a row: the part's output is read once, the stream read and written once, and the row
// never leaves shared memory between the two norms.  Sums, both statistics and the stream are 32-bit in every run
// precision; `out` is rounded once to the parts' element type.  delta may be float or of the parts' type.
//
// acv_cast_rows_f32: a float matrix into a column range of a wider matrix of the parts' type (the stream beside another
// vector as the input of one product).  acv_activation: elementwise activations with parameters.
#include "common.cuh"

template <typename T, typename TD>
__global__ void add_normed_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, const float* __restrict__ wb,
                                          float eps_b, const float* __restrict__ w, float eps, T* __restrict__ out, int H) {
    extern __shared__ float row[];          // [H] delta, then the new stream row
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * H;
    const TD* dr = delta + (size_t)r * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = to_f32(dr[i]);
        row[i] = d;
        ss = fmaf(d, d, ss);
    }
    ss = block_sum(ss, red);
    const float rb = 1.f / sqrtf(ss / (float)H + eps_b);
    float s2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = xr[i] + row[i] * rb * wb[i];
        xr[i] = v;
        row[i] = v;
        s2 = fmaf(v, v, s2);
    }
    if (!out) return;
    s2 = block_sum(s2, red);
    const float rs = 1.f / sqrtf(s2 / (float)H + eps);
    T* o = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<T>(row[i] * rs * w[i]);
}

// x: float [rows][H], updated in place; delta: [rows][H] float (delta_dtype 0) or bfloat16 (1); out: [rows][H] of
// `dtype`, or null when no norm follows (w is then not read).
ACV_API int acv_add_normed_rmsnorm(float* x, const void* delta, int delta_dtype, const float* wb, float eps_b, const float* w,
                                   float eps, void* out, int n_rows, int H, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return ACV_ERR_SIZE;
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
#define ANR_LAUNCH(T, TD)                                                                                               \
    do {                                                                                                                \
        if (smem > 48 * 1024) {                                                                                         \
            static AcvSmemConfig cfg;                                                                                   \
            const int e = acv_ensure_smem(cfg, add_normed_rmsnorm_kernel<T, TD>, (int)smem);                            \
            if (e) return e;                                                                                            \
        }                                                                                                               \
        acv_launch(PDL_NORM, add_normed_rmsnorm_kernel<T, TD>, n_rows, threads, smem, stream, x, (const TD*)delta, wb,  \
                   eps_b, w, eps, (T*)out, H);                                                                          \
    } while (0)
    if (dtype == ACV_F32 && delta_dtype == ACV_F32) ANR_LAUNCH(float, float);
    else if (dtype == ACV_BF16 && delta_dtype == ACV_F32) ANR_LAUNCH(bf16, float);
    else if (dtype == ACV_BF16 && delta_dtype == ACV_BF16) ANR_LAUNCH(bf16, bf16);
    else return ACV_ERR_DTYPE;
#undef ANR_LAUNCH
    return acv_launch_status();
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, int ld_x, T* __restrict__ out, int ld_out, int rows, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t n = (size_t)rows * H;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / H, c = i - r * H;
        out[r * ld_out + c] = from_f32<T>(x[r * ld_x + c]);
    }
}

ACV_API int acv_cast_rows_f32(const float* x, int ld_x, void* out, int ld_out, int rows, int H, int dtype, cudaStream_t stream) {
    if (rows <= 0 || H <= 0) return 0;
    const size_t n = (size_t)rows * H;
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    if (dtype == ACV_F32) acv_launch(PDL_MISC, cast_rows_kernel<float>, blocks, 256, 0, stream, x, ld_x, (float*)out, ld_out, rows, H);
    else if (dtype == ACV_BF16) acv_launch(PDL_MISC, cast_rows_kernel<bf16>, blocks, 256, 0, stream, x, ld_x, (bf16*)out, ld_out, rows, H);
    else return ACV_ERR_DTYPE;
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- activations with parameters
// kind 0: z > 0: p0 z^2 + z/2;  z <= 0: p1 (exp(z) - 1 - z) + z/2     (p0 = softplus(p), p1 = 1/2 + softplus(q) of the
//         layer's two learned numbers, folded by the caller)
// kind 1: gelu_tanh: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
// kind 2: silu
// kind 3: gelu (exact): 0.5 z (1 + erf(z / sqrt 2))
__device__ __forceinline__ float activation_f32(float z, int kind, float p0, float p1) {
    if (kind == 0) return z > 0.f ? fmaf(p0 * z, z, 0.5f * z) : fmaf(p1, expm1f(z) - z, 0.5f * z);
    if (kind == 1) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    if (kind == 3) return 0.5f * z * (1.f + erff(z * 0.7071067811865476f));
    return z / (1.f + expf(-z));
}

template <typename T>
__global__ void activation_kernel(const T* __restrict__ in, T* __restrict__ out, size_t n, int kind, float p0, float p1) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(activation_f32(to_f32(in[i]), kind, p0, p1));
}

// eight bfloat16 values a thread and pass
__global__ void activation_bf16x8_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, size_t n8, int kind, float p0, float p1) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 u = in[i];
        uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float a = activation_f32(__uint_as_float(w4[k] << 16), kind, p0, p1);
            const float b = activation_f32(__uint_as_float(w4[k] & 0xffff0000u), kind, p0, p1);
            const __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
            w4[k] = *reinterpret_cast<const uint32_t*>(&r);
        }
        out[i] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    }
}

ACV_API int acv_activation(const void* in, void* out, long long n, int kind, float p0, float p1, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (kind < 0 || kind > 3) return ACV_ERR_SIZE;
    if (dtype == ACV_BF16 && (n & 7) == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const size_t n8 = (size_t)n / 8;
        const int blocks = (int)((n8 + 255) / 256 < 148 * 8 ? (n8 + 255) / 256 : 148 * 8);
        acv_launch(PDL_ACT, activation_bf16x8_kernel, blocks, 256, 0, stream, (const uint4*)in, (uint4*)out, n8, kind, p0, p1);
        return acv_launch_status();
    }
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    if (dtype == ACV_F32) acv_launch(PDL_ACT, activation_kernel<float>, blocks, 256, 0, stream, (const float*)in, (float*)out, (size_t)n, kind, p0, p1);
    else if (dtype == ACV_BF16) acv_launch(PDL_ACT, activation_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)in, (bf16*)out, (size_t)n, kind, p0, p1);
    else return ACV_ERR_DTYPE;
    return acv_launch_status();
}
