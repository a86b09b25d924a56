// Mixture of experts: routing, grouping of the tokens by expert, the experts' products, the sum.
//
//   z = W_r h (32-bit);  score = sigmoid(z) (or softmax(z));  the `top` largest scores choose the experts
//   (ties go to the lower index); the chosen scores, as they are or divided by their sum, are the weights.
//   An expert is a gated unit:  a = W_gate x, b = W_up x, y = act(a, b), out = W_down y.
//   The weight w multiplies the expert's input (x = w h) or its output, as the model says.  With the
//   weight on the input the products are linear in it, a = w (W_gate h), so the kernels multiply the
//   accumulators by w, in 32-bit, instead of making scaled copies of h.
//
// The step is four launches whatever the routing turns out to be, so that it can be captured in a graph:
//   acv_moe_route    one warp per token: router logits, scores, choice; also the shared expert's gate
//   acv_moe_group    one block: rows (token, choice) counted per expert, each expert's rows padded to
//                    whole tiles of MOE_TILE rows; a tile belongs to one expert
//   acv_moe_gemm_*   tiles x column blocks: rows gathered by the grouping, the expert's weights by tile
//   acv_moe_combine  per token: the chosen experts' outputs in the order of the choice, plus the
//                    shared expert's output times its gate, summed in 32-bit
#include "common.cuh"
#include "mma_tiles.cuh"

#define MOE_TILE 64          // rows of a tile of the grouped products (ops.MOE_TILE)

// gated activation of an expert (ops.GLU_*)
#define GLU_SWISH_CLAMPED 0  // g = min(a, limit), u = clamp(b, -limit, limit): g * sigmoid(alpha g) * (u + 1)
// acv_glu also takes 1, 2, 3: act(a) * b with act the plain activation of that number (gelu_tanh, silu, gelu)

template <typename T> __device__ __forceinline__ float sigmoid_f32(float x);
template <> __device__ __forceinline__ float sigmoid_f32<float>(float x) { return 1.f / (1.f + expf(-x)); }
template <> __device__ __forceinline__ float sigmoid_f32<bf16>(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

template <typename T>
__device__ __forceinline__ float glu_act(float a, float b, float limit, float alpha) {
    const float g = fminf(a, limit);
    const float u = fminf(fmaxf(b, -limit), limit);
    return g * sigmoid_f32<T>(alpha * g) * (u + 1.f);
}

// activation of an expert that has no gate: y = act(W_up x), out = W_down y  (ops.ACTIVATIONS)
__device__ __forceinline__ float plain_act(float z, int kind) {
    if (kind == 1) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    if (kind == 2) return z / (1.f + expf(-z));
    if (kind == 3) return 0.5f * z * (1.f + erff(z * 0.7071067811865476f));
    return z;
}

// ----------------------------------------------------------------------------- routing
#define MR_WARPS 4
// scores in shared memory, E floats per warp.  ids/weights: [T, top].  gate_w (optional, [H]): the shared
// expert's gate, sigmoid(<gate_w, h>), one number per token.
// With z (float [T, ldz]) the logits come from a matrix product made before: columns 0..E-1 the router's, column E
// the shared expert's gate (when gate is asked for); h and the weights are then not read.
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ h, int h_stride, const float* __restrict__ w_router,
                                 const float* __restrict__ gate_w, const float* __restrict__ z, int ldz, int T_tokens, int H,
                                 int E, int top, int softmax, int renorm, int* __restrict__ ids, float* __restrict__ weights,
                                 float* __restrict__ gate, int n_groups, int keep_groups, float renorm_eps) {
    extern __shared__ float sm_all[];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * MR_WARPS + warp;
    if (t >= T_tokens) return;
    float* sc = sm_all + warp * (E + n_groups);
    if (z) {
        for (int e = lane; e < E; e += 32) sc[e] = z[(size_t)t * ldz + e];
        if (gate && lane == 0) gate[t] = 1.f / (1.f + expf(-z[(size_t)t * ldz + E]));
    } else {
        const T* row = h + (size_t)t * h_stride;
        for (int e = 0; e < E; ++e) {
            const float* wr = w_router + (size_t)e * H;
            float d = 0.f;
            for (int k = lane; k < H; k += 32) d = fmaf(to_f32(row[k]), wr[k], d);
            d = warp_sum(d);
            if (lane == 0) sc[e] = d;
        }
        if (gate_w) {
            float d = 0.f;
            for (int k = lane; k < H; k += 32) d = fmaf(to_f32(row[k]), gate_w[k], d);
            d = warp_sum(d);
            if (lane == 0) gate[t] = 1.f / (1.f + expf(-d));
        }
    }
    __syncwarp();
    if (softmax) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, sc[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float x = expf(sc[e] - mx);
            sc[e] = x;
            sum += x;
        }
        sum = warp_sum(sum);
        __syncwarp();
        for (int e = lane; e < E; e += 32) sc[e] /= sum;
    } else {
        for (int e = lane; e < E; e += 32) sc[e] = 1.f / (1.f + expf(-sc[e]));
    }
    __syncwarp();
    if (n_groups > 1 && keep_groups < n_groups) {
        // The experts stand in n_groups equal groups of neighbours; a group is worth its best score, and only the
        // keep_groups best groups (ties: the lower index) can be chosen from.  gw: the groups' worths, behind the scores;
        // a kept group's worth is replaced by a mark.
        const int per = E / n_groups;
        float* gw = sc + E;
        for (int g = lane; g < n_groups; g += 32) {
            float worth = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) worth = fmaxf(worth, sc[e]);
            gw[g] = worth;
        }
        __syncwarp();
        const float KEPT = INFINITY;
        for (int j = 0; j < keep_groups; ++j) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32) {
                const float x = gw[g];
                if (x != KEPT && (arg == 0x7fffffff || x > best)) { best = x; arg = g; }    // ascending g: the first of equals stays
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (oa != 0x7fffffff && (arg == 0x7fffffff || ob > best || (ob == best && oa < arg))) { best = ob; arg = oa; }
            }
            if (lane == 0 && arg != 0x7fffffff) gw[arg] = KEPT;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gw[e / per] != KEPT) sc[e] = -INFINITY;
        __syncwarp();
    }
    float total = 0.f;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float x = sc[e];
            if (x > best) { best = x; arg = e; }       // ascending e: the first of equal scores stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg == 0x7fffffff) arg = 0;     // top > E, or scores that are not numbers: never an index outside
        if (lane == 0) {
            ids[(size_t)t * top + j] = arg;
            weights[(size_t)t * top + j] = best;
            sc[arg] = -INFINITY;
        }
        total += best;
        __syncwarp();
    }
    if (renorm && lane == 0)
        for (int j = 0; j < top; ++j) weights[(size_t)t * top + j] /= total + renorm_eps;
}

ACV_API int acv_moe_route(const void* h, int h_stride, const float* w_router, const float* gate_w, const float* z, int ldz,
                          int T_tokens, int H, int E, int top, int softmax, int renorm, int* ids, float* weights, float* gate,
                          int dtype, int n_groups, int keep_groups, float renorm_eps, cudaStream_t stream) {
    if (T_tokens <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || E > 4096) return ACV_ERR_SIZE;
    if (n_groups < 1) n_groups = 1;
    if (E % n_groups || keep_groups < 1 || (n_groups > 1 && top > keep_groups * (E / n_groups))) return ACV_ERR_SIZE;
    const size_t smem = (size_t)MR_WARPS * (E + n_groups) * sizeof(float);
    const int grid = (T_tokens + MR_WARPS - 1) / MR_WARPS;
    if (dtype == ACV_F32)
        acv_launch(PDL_MISC, moe_route_kernel<float>, grid, MR_WARPS * 32, smem, stream, (const float*)h, h_stride, w_router,
                   gate_w, z, ldz, T_tokens, H, E, top, softmax, renorm, ids, weights, gate, n_groups, keep_groups, renorm_eps);
    else if (dtype == ACV_BF16)
        acv_launch(PDL_MISC, moe_route_kernel<bf16>, grid, MR_WARPS * 32, smem, stream, (const bf16*)h, h_stride, w_router,
                   gate_w, z, ldz, T_tokens, H, E, top, softmax, renorm, ids, weights, gate, n_groups, keep_groups, renorm_eps);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- grouping by expert
// N = T * top rows (row r = token r / top, choice r % top).  Expert e's rows take the positions
// [start[e], start[e] + count[e]) of the grouped list, start[e] a multiple of MOE_TILE; the positions up
// to the next multiple hold -1.  tile_expert[i] names the expert of tile i (-1: no such tile).
// The order of an expert's rows among themselves is whatever the atomics make it; a row's result does
// not depend on its place.
#define GR_BATCH 8
__global__ void moe_group_kernel(const int* __restrict__ ids, int N, int E, int max_tiles, int tile_rows,
                                 int* __restrict__ grouped, int* __restrict__ place, int* __restrict__ tile_expert,
                                 int* __restrict__ tiles_used) {
    extern __shared__ int sm_int[];
    int* count = sm_int;          // [E]
    int* start = sm_int + E;      // [E + 1]
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_expert[i] = -1;
    __syncthreads();
    // rows in batches of GR_BATCH per thread: the batch's loads are issued together, so that the loop waits for memory
    // once a batch and not once a row (the block is alone on the device and nothing hides its latencies)
    for (int r0 = threadIdx.x; r0 < N; r0 += blockDim.x * GR_BATCH) {
        int e[GR_BATCH];
#pragma unroll
        for (int b = 0; b < GR_BATCH; ++b) {
            const int r = r0 + b * blockDim.x;
            e[b] = r < N ? ids[r] : -1;
        }
#pragma unroll
        for (int b = 0; b < GR_BATCH; ++b)
            if (e[b] >= 0 && e[b] < E) atomicAdd(&count[e[b]], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = at;
            at += (count[e] + tile_rows - 1) / tile_rows * tile_rows;
        }
        start[E] = at;
        if (tiles_used) *tiles_used = at / tile_rows;
    }
    __syncthreads();
    // the places behind an expert's rows, up to the end of its last tile, hold no row (tiles that belong to no expert
    // are never read)
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        for (int i = start[e] / tile_rows; i < start[e + 1] / tile_rows; ++i)
            if (i < max_tiles) tile_expert[i] = e;
        for (int i = start[e] + count[e]; i < start[e + 1]; ++i)
            if (i < max_tiles * tile_rows) grouped[i] = -1;
        count[e] = 0;       // now the cursor inside the expert's rows
    }
    __syncthreads();
    for (int r0 = threadIdx.x; r0 < N; r0 += blockDim.x * GR_BATCH) {
        int e[GR_BATCH];
#pragma unroll
        for (int b = 0; b < GR_BATCH; ++b) {
            const int r = r0 + b * blockDim.x;
            e[b] = r < N ? ids[r] : -2;
        }
#pragma unroll
        for (int b = 0; b < GR_BATCH; ++b) {
            const int r = r0 + b * blockDim.x;
            if (e[b] == -2) continue;
            if (e[b] < 0 || e[b] >= E) { place[r] = -1; continue; }
            const int at = start[e[b]] + atomicAdd(&count[e[b]], 1);
            place[r] = at;
            grouped[at] = r;
        }
    }
}

// tile_rows: rows of a tile (MOE_TILE for the kernels of this file, 128 for the tcgen05 product); tiles_used
// (may be null): one int that gets the number of tiles that hold rows.
ACV_API int acv_moe_group(const int* ids, int N, int E, int max_tiles, int tile_rows, int* grouped, int* place,
                          int* tile_expert, int* tiles_used, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (E <= 0 || E > 4096 || tile_rows <= 0 || max_tiles < (N + tile_rows - 1) / tile_rows + E) return ACV_ERR_SIZE;
    acv_launch(PDL_MISC, moe_group_kernel, 1, 1024, (size_t)(2 * E + 1) * sizeof(int), stream, ids, N, E, max_tiles, tile_rows,
               grouped, place, tile_expert, tiles_used);
    return acv_launch_status();
}

// The tokens' rows in grouped order, for products that want their A operand contiguous: out[r] = h[grouped[r] / top]
// (zeros where the grouped list holds no row), scale_out[r] = weights[grouped[r]] (1 there).  16-byte copies.
__global__ void moe_gather_kernel(const bf16* __restrict__ h, int ldh, const int* __restrict__ grouped, const float* __restrict__ weights,
                                  int top, int H, bf16* __restrict__ out, float* __restrict__ scale_out, const int* __restrict__ tiles_used,
                                  int tile_rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    if (tiles_used && r >= *tiles_used * tile_rows) return;
    const int s = grouped[r];
    if (scale_out && threadIdx.x == 0) scale_out[r] = s >= 0 && weights ? weights[s] : 1.f;
    const uint4* src = s >= 0 ? reinterpret_cast<const uint4*>(h + (size_t)(s / top) * ldh) : nullptr;
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src ? src[i] : make_uint4(0, 0, 0, 0);
}

ACV_API int acv_moe_gather(const void* h, int ldh, const int* grouped, const float* weights, int top, int H, void* out,
                           float* scale_out, const int* tiles_used, int tile_rows, int rows, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if ((H % 8) || (ldh % 8) || ((uintptr_t)h & 15) || ((uintptr_t)out & 15)) return ACV_ERR_ALIGN;
    acv_launch(PDL_MISC, moe_gather_kernel, rows, 128, 0, stream, (const bf16*)h, ldh, grouped, weights, top, H, (bf16*)out,
               scale_out, tiles_used, tile_rows);
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- grouped products on the CUDA cores
// Tile i (MOE_TILE rows of the grouped list) x 64 output columns; 256 threads, each a 4 x 4 micro-tile.
// GLU: the expert's matrix is [2 * N, K], gate rows then up rows (or, with `pairs`, (gate, up) row by row, the layout of
//      the tcgen05 product); row r of A is token grouped[r] / top; the
//      accumulators are multiplied by the row's weight (when given) and go through the activation; output T.
// else: A's row r is row r of the grouped list itself (the activations of the product before); output float,
//      multiplied by the row's weight when given (the weight on the expert's output).
// Sums run over k in ascending order inside fixed slabs of 16: a row's result does not depend on the others.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_gemm_simt_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, long long w_expert_stride, int ldw,
                     void* __restrict__ C, int ldc, const int* __restrict__ grouped, const int* __restrict__ tile_expert,
                     const float* __restrict__ row_weight, int top, int N, int K, float limit, float alpha, int pairs) {
    constexpr bool GLU = MODE == 1, GATHER = MODE != 0;
    __shared__ float As[16][MOE_TILE + 4];
    __shared__ float Ws[16][64 + 4];
    __shared__ float Us[GLU ? 16 : 1][64 + 4];
    __shared__ int src[MOE_TILE];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.y;
    const int expert = tile_expert[tile];
    if (expert < 0) return;
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * 64;
    if (tid < MOE_TILE) src[tid] = grouped[tile * MOE_TILE + tid];
    __syncthreads();
    const T* We = W + (size_t)expert * w_expert_stride;
    const int tx = tid & 15, ty = tid >> 4;
    float acc[4][4], acu[GLU ? 4 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.f;
            if constexpr (GLU) acu[i][j] = 0.f;
        }
    for (int k0 = 0; k0 < K; k0 += 16) {
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int gk = k0 + kk, gn = n0 + r;
            const int s = src[r];
            const long long arow = GATHER ? (s >= 0 ? s / top : -1) : (s >= 0 ? tile * MOE_TILE + r : -1);
            As[kk][r] = (arow >= 0 && gk < K) ? to_f32(A[(size_t)arow * lda + gk]) : 0.f;
            Ws[kk][r] = (gn < N && gk < K) ? to_f32(We[(size_t)(GLU && pairs ? 2 * gn : gn) * ldw + gk]) : 0.f;
            if constexpr (GLU) Us[kk][r] = (gn < N && gk < K) ? to_f32(We[(size_t)(pairs ? 2 * gn + 1 : N + gn) * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
            float a[4], b[4], u[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                b[j] = Ws[kk][tx * 4 + j];
                if constexpr (GLU) u[j] = Us[kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if constexpr (GLU) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        const int s = src[r];
        if (s < 0) continue;
        const float w = row_weight ? row_weight[s] : 1.f;
        const size_t crow = (size_t)(tile * MOE_TILE + r) * ldc;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            if constexpr (GLU)
                ((T*)C)[crow + gn] = from_f32<T>(glu_act<T>(acc[i][j] * w, acu[i][j] * w, limit, alpha));
            else if constexpr (MODE == 2)
                ((T*)C)[crow + gn] = from_f32<T>(plain_act(acc[i][j] * w, pairs));
            else
                ((float*)C)[crow + gn] = acc[i][j] * w;
        }
    }
}

// which: 0 = gate/up with the gated activation (C of A's type), 1 = down (C float), 2 = up alone with a plain activation
// (C of A's type; the activation's kind travels in `pairs`)
ACV_API int acv_moe_gemm_simt(const void* A, int lda, const void* W, long long w_expert_stride, int ldw, void* C, int ldc,
                              const int* grouped, const int* tile_expert, const float* row_weight, int top, int max_tiles,
                              int N, int K, int which, float limit, float alpha, int pairs, int dtype, cudaStream_t stream) {
    if (max_tiles <= 0 || N <= 0) return 0;
    if (K <= 0 || top <= 0 || max_tiles > 65535) return ACV_ERR_SIZE;
    dim3 grid((N + 63) / 64, max_tiles);
#define MG_LAUNCH(TT, G)                                                                                              \
    acv_launch(PDL_GEMM, moe_gemm_simt_kernel<TT, G>, grid, 256, 0, stream, (const TT*)A, lda, (const TT*)W,          \
               w_expert_stride, ldw, C, ldc, grouped, tile_expert, row_weight, top, N, K, limit, alpha, pairs)
    if (dtype == ACV_F32) {
        if (which == 0) MG_LAUNCH(float, 1); else if (which == 2) MG_LAUNCH(float, 2); else MG_LAUNCH(float, 0);
    } else if (dtype == ACV_BF16) {
        if (which == 0) MG_LAUNCH(bf16, 1); else if (which == 2) MG_LAUNCH(bf16, 2); else MG_LAUNCH(bf16, 0);
    } else {
        return ACV_ERR_DTYPE;
    }
#undef MG_LAUNCH
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- grouped products on the tensor cores
// bfloat16, mma.sync m16n8k16 with float accumulators.  A CTA of four warps owns a tile of MOE_TILE grouped rows x 64
// output columns (with GLU: 64 gate and the 64 up columns of the same numbers); a warp owns 16 rows.  Operands come in
// slabs of 64 k through three stages of 16-byte asynchronous copies into swizzled tiles: the rows of A gathered by the
// grouping (rows without a token are zero-filled), the expert's weight rows by the tile's expert.  Same epilogues as
// the CUDA-core form: the row's weight times the accumulators, then the activation (GLU), or float output (down).
// Rows of 16-byte alignment are needed: K, lda, ldw and the experts' stride multiples of 8.
#define MM_BN 64
#define MM_BK 64
#define MM_THREADS 128
#define MM_STAGES 3

template <int MODE>
__global__ void __launch_bounds__(MM_THREADS)
moe_gemm_mma_kernel(const bf16* __restrict__ A, int lda, const bf16* __restrict__ W, long long w_expert_stride, int ldw,
                    void* __restrict__ C, int ldc, const int* __restrict__ grouped, const int* __restrict__ tile_expert,
                    const float* __restrict__ row_weight, int top, int N, int K, float limit, float alpha, int pairs) {
    extern __shared__ __align__(128) unsigned char mm_smem[];
    constexpr bool GLU = MODE == 1, GATHER = MODE != 0;
    constexpr int A_BYTES = MOE_TILE * MM_BK * 2;
    constexpr int W_BYTES = MM_BN * MM_BK * 2;
    constexpr int STAGE = A_BYTES + (GLU ? 2 : 1) * W_BYTES;
    __shared__ int src[MOE_TILE];
    pdl_launch_dependents();
    pdl_wait();
    const int tile = blockIdx.y;
    const int expert = tile_expert[tile];
    if (expert < 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * MM_BN;
    // an expert's rows stand at the front of its tiles: a tile of a decode step holds a few rows and then nothing, and
    // a warp whose 16 rows are all empty only helps to load (measured at 64 tokens over 64 experts: the tensor pipe was
    // busy 43 % of the time on rows that hold nothing, and the weights came at 0.45 of the memory's rate)
    const int mine = tid < MOE_TILE ? grouped[tile * MOE_TILE + tid] : -1;
    if (tid < MOE_TILE) src[tid] = mine;
    const int n_valid = __syncthreads_count(mine >= 0);
    const bool warp_has_rows = warp * 16 < n_valid;
    const bf16* We = W + (size_t)expert * w_expert_stride;

    auto load = [&](int kb, int stage) {
        unsigned char* base = mm_smem + stage * STAGE;
        const int k0 = kb * MM_BK;
#pragma unroll
        for (int it = 0; it < MOE_TILE * 8 / MM_THREADS; ++it) {
            const int id = tid + it * MM_THREADS;
            const int r = id >> 3, c = id & 7;
            const int s = src[r];
            const long long arow = GATHER ? (s >= 0 ? s / top : -1) : (s >= 0 ? (long long)tile * MOE_TILE + r : -1);
            const bool ok = arow >= 0 && k0 + c * 8 < K;
            cp_async16(smem_u32(base + tile_off<MM_BK>(r, c)), ok ? (const void*)(A + arow * lda + k0 + c * 8) : (const void*)A, ok);
        }
#pragma unroll
        for (int it = 0; it < MM_BN * 8 / MM_THREADS; ++it) {
            const int id = tid + it * MM_THREADS;
            const int r = id >> 3, c = id & 7;
            const int n = n0 + r;
            const bool ok = n < N && k0 + c * 8 < K;
            cp_async16(smem_u32(base + A_BYTES + tile_off<MM_BK>(r, c)),
                       ok ? (const void*)(We + (size_t)(GLU && pairs ? 2 * n : n) * ldw + k0 + c * 8) : (const void*)We, ok);
            if constexpr (GLU)
                cp_async16(smem_u32(base + A_BYTES + W_BYTES + tile_off<MM_BK>(r, c)),
                           ok ? (const void*)(We + (size_t)(pairs ? 2 * n + 1 : N + n) * ldw + k0 + c * 8) : (const void*)We, ok);
        }
    };

    float acc[MM_BN / 8][4], acu[GLU ? MM_BN / 8 : 1][4];
#pragma unroll
    for (int i = 0; i < MM_BN / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            acc[i][e] = 0.f;
            if constexpr (GLU) acu[i][e] = 0.f;
        }
    const int nkb = (K + MM_BK - 1) / MM_BK;
    const int mi = lane >> 3, lr = lane & 7;
    // three stages: while slab kb is multiplied, kb + 1 is landing and kb + 2 is asked for.  One barrier a slab: behind
    // it slab kb has landed for every thread, and every warp is done with slab kb - 1, whose stage the next copies take.
    load(0, 0);
    cp_async_commit();
    if (nkb > 1) load(1, 1);
    cp_async_commit();
    for (int kb = 0; kb < nkb; ++kb) {
        const int stage = kb % MM_STAGES;
        cp_async_wait<1>();
        __syncthreads();
        if (kb + 2 < nkb) load(kb + 2, (kb + 2) % MM_STAGES);
        cp_async_commit();
        const uint32_t ab = smem_u32(mm_smem + stage * STAGE), wb = ab + A_BYTES;
        if (warp_has_rows)
#pragma unroll
        for (int kd = 0; kd < MM_BK / 16; ++kd) {
            uint32_t af[4];
            ldmatrix_x4(af, ab + tile_off<MM_BK>(warp * 16 + (mi & 1) * 8 + lr, kd * 2 + (mi >> 1)));
#pragma unroll
            for (int np = 0; np < MM_BN / 16; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, wb + tile_off<MM_BK>(np * 16 + (mi >> 1) * 8 + lr, kd * 2 + (mi & 1)));
                mma_bf16(acc[2 * np], af, b[0], b[1]);
                mma_bf16(acc[2 * np + 1], af, b[2], b[3]);
                if constexpr (GLU) {
                    ldmatrix_x4(b, wb + W_BYTES + tile_off<MM_BK>(np * 16 + (mi >> 1) * 8 + lr, kd * 2 + (mi & 1)));
                    mma_bf16(acu[2 * np], af, b[0], b[1]);
                    mma_bf16(acu[2 * np + 1], af, b[2], b[3]);
                }
            }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + (lane >> 2) + half * 8;
        const int s = src[r];
        if (s < 0) continue;
        const float w = row_weight ? row_weight[s] : 1.f;
        const size_t crow = (size_t)(tile * MOE_TILE + r) * ldc;
#pragma unroll
        for (int nt = 0; nt < MM_BN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int col = n0 + nt * 8 + (lane & 3) * 2 + e;
                if (col >= N) continue;
                const float v = acc[nt][half * 2 + e] * w;
                if constexpr (GLU)
                    ((bf16*)C)[crow + col] = __float2bfloat16_rn(glu_act<bf16>(v, acu[nt][half * 2 + e] * w, limit, alpha));
                else if constexpr (MODE == 2)
                    ((bf16*)C)[crow + col] = __float2bfloat16_rn(plain_act(v, pairs));
                else
                    ((float*)C)[crow + col] = v;
            }
        }
    }
}

// which: 0 = gate/up with the gated activation (C bfloat16), 1 = down (C float), 2 = up alone with a plain activation
// (C bfloat16; the activation's kind travels in `pairs`)
ACV_API int acv_moe_gemm_mma(const void* A, int lda, const void* W, long long w_expert_stride, int ldw, void* C, int ldc,
                             const int* grouped, const int* tile_expert, const float* row_weight, int top, int max_tiles,
                             int N, int K, int which, float limit, float alpha, int pairs, cudaStream_t stream) {
    if (max_tiles <= 0 || N <= 0) return 0;
    if (K <= 0 || top <= 0 || max_tiles > 65535) return ACV_ERR_SIZE;
    if ((K % 8) || (lda % 8) || (ldw % 8) || (w_expert_stride % 8) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return ACV_ERR_ALIGN;
    dim3 grid((N + MM_BN - 1) / MM_BN, max_tiles);
    if (which == 0) {
        const int smem = MM_STAGES * (MOE_TILE * MM_BK * 2 + 2 * MM_BN * MM_BK * 2);
        static AcvSmemConfig cfg;
        if (int rc = acv_ensure_smem(cfg, moe_gemm_mma_kernel<1>, smem)) return rc;
        acv_launch(PDL_GEMM, moe_gemm_mma_kernel<1>, grid, MM_THREADS, smem, stream, (const bf16*)A, lda, (const bf16*)W,
                   w_expert_stride, ldw, C, ldc, grouped, tile_expert, row_weight, top, N, K, limit, alpha, pairs);
    } else {
        const int smem = MM_STAGES * (MOE_TILE * MM_BK * 2 + MM_BN * MM_BK * 2);
        static AcvSmemConfig cfg;
        if (which == 2) {
            static AcvSmemConfig cfg2;
            if (int rc = acv_ensure_smem(cfg2, moe_gemm_mma_kernel<2>, smem)) return rc;
            acv_launch(PDL_GEMM, moe_gemm_mma_kernel<2>, grid, MM_THREADS, smem, stream, (const bf16*)A, lda, (const bf16*)W,
                       w_expert_stride, ldw, C, ldc, grouped, tile_expert, row_weight, top, N, K, limit, alpha, pairs);
            return acv_launch_status();
        }
        if (int rc = acv_ensure_smem(cfg, moe_gemm_mma_kernel<0>, smem)) return rc;
        acv_launch(PDL_GEMM, moe_gemm_mma_kernel<0>, grid, MM_THREADS, smem, stream, (const bf16*)A, lda, (const bf16*)W,
                   w_expert_stride, ldw, C, ldc, grouped, tile_expert, row_weight, top, N, K, limit, alpha, pairs);
    }
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- the sum
// out[t] = sum over the token's choices, in their order, of D[place[t * top + j]]  (+ gate[t] * S[t]),
// summed in 32-bit, rounded once to T.
template <typename T, typename TD>
__global__ void moe_combine_kernel(const TD* __restrict__ D, int ldd, const int* __restrict__ place, int top,
                                   const T* __restrict__ S, int lds, const float* __restrict__ gate, T* __restrict__ out,
                                   int ldo, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float sum = 0.f;
        for (int j = 0; j < top; ++j) {
            const int at = place[(size_t)t * top + j];
            if (at >= 0) sum += to_f32(D[(size_t)at * ldd + c]);
        }
        if (S) sum += (gate ? gate[t] : 1.f) * to_f32(S[(size_t)t * lds + c]);
        out[(size_t)t * ldo + c] = from_f32<T>(sum);
    }
}

// All bfloat16 with rows of 16-byte alignment: a thread sums eight neighbouring columns, 16 bytes from every row.
__global__ void moe_combine_vec_kernel(const bf16* __restrict__ D, int ldd, const int* __restrict__ place, int top,
                                       const bf16* __restrict__ S, int lds, const float* __restrict__ gate, bf16* __restrict__ out,
                                       int ldo, int H) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const float g = S ? (gate ? gate[t] : 1.f) : 0.f;
    for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
        float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < top; ++j) {
            const int at = place[(size_t)t * top + j];
            if (at < 0) continue;
            const uint4 raw = *reinterpret_cast<const uint4*>(D + (size_t)at * ldd + c);
            const bf16* v = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
            for (int e = 0; e < 8; ++e) sum[e] += __bfloat162float(v[e]);
        }
        if (S) {
            const uint4 raw = *reinterpret_cast<const uint4*>(S + (size_t)t * lds + c);
            const bf16* v = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
            for (int e = 0; e < 8; ++e) sum[e] += g * __bfloat162float(v[e]);
        }
        bf16 o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = __float2bfloat16_rn(sum[e]);
        *reinterpret_cast<uint4*>(out + (size_t)t * ldo + c) = *reinterpret_cast<const uint4*>(o);
    }
}

// d_dtype: the type of D (float, or bfloat16 beside a bfloat16 output)
ACV_API int acv_moe_combine(const void* D, int ldd, int d_dtype, const int* place, int top, const void* S, int lds,
                            const float* gate, void* out, int ldo, int T_tokens, int H, int dtype, cudaStream_t stream) {
    if (T_tokens <= 0 || H <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == ACV_F32 && d_dtype == ACV_F32)
        acv_launch(PDL_MISC, moe_combine_kernel<float, float>, T_tokens, threads, 0, stream, (const float*)D, ldd, place, top,
                   (const float*)S, lds, gate, (float*)out, ldo, H);
    else if (dtype == ACV_BF16 && d_dtype == ACV_F32)
        acv_launch(PDL_MISC, moe_combine_kernel<bf16, float>, T_tokens, threads, 0, stream, (const float*)D, ldd, place, top,
                   (const bf16*)S, lds, gate, (bf16*)out, ldo, H);
    else if (dtype == ACV_BF16 && d_dtype == ACV_BF16 && H % 8 == 0 && ldd % 8 == 0 && ldo % 8 == 0 && (!S || lds % 8 == 0) &&
             !((uintptr_t)D & 15) && !((uintptr_t)out & 15) && !((uintptr_t)S & 15))
        acv_launch(PDL_MISC, moe_combine_vec_kernel, T_tokens, H >= 2048 ? 256 : 128, 0, stream, (const bf16*)D, ldd, place, top,
                   (const bf16*)S, lds, gate, (bf16*)out, ldo, H);
    else if (dtype == ACV_BF16 && d_dtype == ACV_BF16)
        acv_launch(PDL_MISC, moe_combine_kernel<bf16, bf16>, T_tokens, threads, 0, stream, (const bf16*)D, ldd, place, top,
                   (const bf16*)S, lds, gate, (bf16*)out, ldo, H);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- gated activation of a stacked product
// gu [T, 2I]: gate columns, then up columns, or with `pairs` (gate, up) column by column (one expert applied to every
// token, e.g. a shared expert).
template <typename T>
__global__ void glu_kernel(const T* __restrict__ gu, int ldg, T* __restrict__ out, int ldo, int I, size_t total, float limit,
                           float alpha, int pairs, int kind) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I;
        const int i = (int)(idx - t * I);
        const float a = to_f32(gu[t * ldg + (pairs ? 2 * i : i)]), b = to_f32(gu[t * ldg + (pairs ? 2 * i + 1 : I + i)]);
        out[t * ldo + i] = from_f32<T>(kind == GLU_SWISH_CLAMPED ? glu_act<T>(a, b, limit, alpha) : plain_act(a, kind) * b);
    }
}

ACV_API int acv_glu(const void* gu, int ldg, void* out, int ldo, int T_tokens, int I, int kind, float limit, float alpha,
                    int pairs, int dtype, cudaStream_t stream) {
    const size_t total = (size_t)T_tokens * I;
    if (total == 0) return 0;
    if (kind < 0 || kind > 3) return ACV_ERR_SIZE;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dtype == ACV_F32)
        acv_launch(PDL_ACT, glu_kernel<float>, blocks, 256, 0, stream, (const float*)gu, ldg, (float*)out, ldo, I, total, limit, alpha, pairs, kind);
    else if (dtype == ACV_BF16)
        acv_launch(PDL_ACT, glu_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)gu, ldg, (bf16*)out, ldo, I, total, limit, alpha, pairs, kind);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}
