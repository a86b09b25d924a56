// Products side by side, one for each head over strided views, on the tensor cores:
//
//   C[m, b, :] = A[m, b, :] W[b]^T        A [M][batches][K], W [batches][N][K], C [M][batches][N], bfloat16, float sums
//
// (a head's own matrix on that head's slice of every token's row: W_uk,h^T on the queries and W_uv,h on the weighted
// sums of the latent attention).  The tcgen05 product of the framework takes one weight for all rows; here every batch
// has its own small one (64 to 512 on a side), so a CTA computes a 64 x 64 tile of one batch with mma.sync m16n8k16,
// four warps of 16 rows each, K in steps of 64 through two cp.async buffers (rows padded by 16 bytes against bank
// conflicts).  acv_gemm_simt_batched takes what this kernel refuses (float32, K or strides that are no 16-byte pieces).
#include "mma_tiles.cuh"

#define GB_BM 64
#define GB_BN 64
#define GB_BK 64
#define GB_PITCH (GB_BK * 2 + 16)

__global__ void __launch_bounds__(128)
gemm_mma_batched_kernel(const bf16* __restrict__ A, int lda, long long a_batch, const bf16* __restrict__ W, int ldw,
                        long long w_batch, bf16* __restrict__ C, int ldc, long long c_batch, int M, int N, int K) {
    __shared__ __align__(128) unsigned char a_s[2][GB_BM * GB_PITCH];
    __shared__ __align__(128) unsigned char w_s[2][GB_BN * GB_PITCH];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * GB_BN, m0 = blockIdx.y * GB_BM, b = blockIdx.z;
    A += (size_t)b * a_batch;
    W += (size_t)b * w_batch;
    C += (size_t)b * c_batch;
    const int nk = (K + GB_BK - 1) / GB_BK;

    auto load = [&](int kt) {
        const int k0 = kt * GB_BK, buf = kt & 1;
        for (int id = tid; id < GB_BM * (GB_BK / 8); id += 128) {
            const int r = id >> 3, c = id & 7;
            const int gk = k0 + c * 8;
            const bool ok_a = m0 + r < M && gk < K, ok_w = n0 + r < N && gk < K;
            cp_async16(smem_u32(a_s[buf] + r * GB_PITCH + c * 16), ok_a ? (const void*)(A + (size_t)(m0 + r) * lda + gk) : (const void*)A, ok_a);
            cp_async16(smem_u32(w_s[buf] + r * GB_PITCH + c * 16), ok_w ? (const void*)(W + (size_t)(n0 + r) * ldw + gk) : (const void*)W, ok_w);
        }
    };
    float acc[GB_BN / 8][4];
#pragma unroll
    for (int i = 0; i < GB_BN / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
    const int mi = lane >> 3, lr = lane & 7;
    load(0);
    cp_async_commit();
    for (int kt = 0; kt < nk; ++kt) {
        if (kt + 1 < nk) load(kt + 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t ab = smem_u32(a_s[kt & 1] + warp * 16 * GB_PITCH), wb = smem_u32(w_s[kt & 1]);
#pragma unroll
        for (int kk = 0; kk < GB_BK / 16; ++kk) {
            uint32_t af[4];
            ldmatrix_x4(af, ab + ((mi & 1) * 8 + lr) * GB_PITCH + (kk * 2 + (mi >> 1)) * 16);
#pragma unroll
            for (int np = 0; np < GB_BN / 16; ++np) {
                uint32_t bf[4];
                ldmatrix_x4(bf, wb + (np * 16 + (mi >> 1) * 8 + lr) * GB_PITCH + (kk * 2 + (mi & 1)) * 16);
                mma_bf16(acc[2 * np], af, bf[0], bf[1]);
                mma_bf16(acc[2 * np + 1], af, bf[2], bf[3]);
            }
        }
        __syncthreads();
    }
    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int gm = m0 + warp * 16 + r_lo + hh * 8;
        if (gm >= M) continue;
#pragma unroll
        for (int i = 0; i < GB_BN / 8; ++i) {
            const int gn = n0 + i * 8 + c_lo;
            if (gn < N)     // N is even: the pair is inside
                *reinterpret_cast<__nv_bfloat162*>(C + (size_t)gm * ldc + gn) = __floats2bfloat162_rn(acc[i][2 * hh], acc[i][2 * hh + 1]);
        }
    }
}

// 1 if acv_gemm_mma_batched runs these views (strides in elements; bfloat16 in and out)
ACV_API int acv_gemm_mma_batched_takes(const void* A, int lda, long long a_batch, const void* W, int ldw, long long w_batch,
                                       const void* C, int ldc, long long c_batch, int N, int K) {
    return K > 0 && K % 8 == 0 && lda % 8 == 0 && a_batch % 8 == 0 && ldw % 8 == 0 && w_batch % 8 == 0 &&
           ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0 && N % 2 == 0 && ldc % 2 == 0 && c_batch % 2 == 0 &&
           ((uintptr_t)C & 3) == 0;
}

ACV_API int acv_gemm_mma_batched(const void* A, int lda, long long a_batch, const void* W, int ldw, long long w_batch,
                                 void* C, int ldc, long long c_batch, int M, int N, int K, int batches, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batches <= 0) return 0;
    if (!acv_gemm_mma_batched_takes(A, lda, a_batch, W, ldw, w_batch, C, ldc, c_batch, N, K)) return ACV_ERR_ALIGN;
    dim3 grid((N + GB_BN - 1) / GB_BN, (M + GB_BM - 1) / GB_BM, batches);
    if (grid.y > 65535 || batches > 65535) return ACV_ERR_SIZE;
    acv_launch(PDL_GEMM, gemm_mma_batched_kernel, grid, dim3(128), 0, stream, (const bf16*)A, lda, a_batch, (const bf16*)W, ldw,
               w_batch, (bf16*)C, ldc, c_batch, M, N, K);
    return acv_launch_status();
}
