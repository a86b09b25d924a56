// A linear recurrence whose decay depends on the token and on the key channel, with a bonus for the current token
// (time mixing in the manner of RWKV), and the small kernels in front of it.
//
//   acv_token_shift_multi   x_s[t] = h[t] + (h[t-1] - h[t]) * mu_s for each of S vectors mu_s; h[t-1] of a request's first
//                           token of the step is the row kept in its state slot (zeros when the request begins), which
//                           the step's last row replaces
//   acv_wkv_decay           w[t][c] = exp(-exp(w0[c] + sum_j W2[c][j] tanh(a[t][j]))), all in float
//   acv_wkv                 per (request, head), S: [D, DV] float in a state slot:
//                               o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t
//                               S_t = diag(w_t) S_{t-1} + k_t v_t^T
//
// acv_wkv: grid (items, heads, tiles of DVT value columns).  The block's threads are G groups of DVT: thread (g, c)
// keeps rows g*R .. g*R+R-1 of column c of S in registers and walks its tokens in chunks of TC (r, k, w, v staged in
// shared memory, the partial sums of a chunk reduced over the groups afterwards).
//
// The recurrence is linear in S, so a long portion is cut into segments of seg_len tokens that run side by side (the
// step's list of (request, segment) items): a first launch leaves the state that each segment reaches from zero (the
// first one from the request's state) and the product of its decays per key channel; a small launch folds them,
// S_in(z+1) = diag(P(z)) S_in(z) + S_seg(z); a last launch walks every segment again from what lies in front of it and
// writes the outputs.  Steps of short portions and single tokens run the last launch alone.
#include "mma_tiles.cuh"
#include <type_traits>

// ----------------------------------------------------------------------------- token shift with several mixes
// h: [T, C] of type T; mu: float [S, C]; out: [S, T, C] of type T; state: float [slots, C].  grid (tokens, channel tiles).
// Only the block of a portion's first token reads the state, and it writes the portion's last row there.
template <typename T>
__global__ void token_shift_multi_kernel(const T* __restrict__ h, const float* __restrict__ mu, float* __restrict__ state,
                                         const int* __restrict__ slots, const int* __restrict__ cu_q,
                                         const int* __restrict__ seq_of_token, T* __restrict__ out, int T_tokens, int C, int S) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int seq = seq_of_token[t];
    const int first = cu_q[seq], last = cu_q[seq + 1] - 1;
    const float cur = to_f32(h[(size_t)t * C + c]);
    float prev;
    if (t == first) {
        float* st = state + (size_t)slots[seq] * C;
        prev = st[c];
        st[c] = to_f32(h[(size_t)last * C + c]);
    } else {
        prev = to_f32(h[(size_t)(t - 1) * C + c]);
    }
    const float d = prev - cur;
    for (int s = 0; s < S; ++s)
        out[((size_t)s * T_tokens + t) * C + c] = from_f32<T>(fmaf(d, mu[(size_t)s * C + c], cur));
}

ACV_API int acv_token_shift_multi(const void* h, const float* mu, float* state, const int* slots, const int* cu_q,
                                  const int* seq_of_token, void* out, int T_tokens, int C, int S, int dtype,
                                  cudaStream_t stream) {
    if (T_tokens <= 0) return 0;
    if (C <= 0 || S <= 0) return ACV_ERR_SIZE;
    dim3 grid(T_tokens, (C + 127) / 128);
    if (dtype == ACV_F32)
        acv_launch(PDL_MISC, token_shift_multi_kernel<float>, grid, 128, 0, stream, (const float*)h, mu, state, slots, cu_q,
                   seq_of_token, (float*)out, T_tokens, C, S);
    else if (dtype == ACV_BF16)
        acv_launch(PDL_MISC, token_shift_multi_kernel<bf16>, grid, 128, 0, stream, (const bf16*)h, mu, state, slots, cu_q,
                   seq_of_token, (bf16*)out, T_tokens, C, S);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- the decay
// a: float [T, L] (the first product's output); w2t: float [L, C] (the second matrix transposed); w0: float [C];
// w: float [T, C].  One block for WD_TOK tokens: tanh of their L inputs once, in shared memory; a thread owns channels
// and walks the L rows of the matrix once for all of the block's tokens.
#define WD_TOK 8
__global__ void wkv_decay_kernel(const float* __restrict__ a, int lda, const float* __restrict__ w2t,
                                 const float* __restrict__ w0, float* __restrict__ w, int T_tokens, int C, int L) {
    extern __shared__ float th[];           // [L][WD_TOK]
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * WD_TOK;
    const int n = min(WD_TOK, T_tokens - t0);
    for (int i = threadIdx.x; i < L * WD_TOK; i += blockDim.x) {
        const int j = i / WD_TOK, tt = i - j * WD_TOK;
        th[i] = tt < n ? tanhf(a[(size_t)(t0 + tt) * lda + j]) : 0.f;
    }
    __syncthreads();
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float z[WD_TOK];
        const float z0 = w0[c];
#pragma unroll
        for (int tt = 0; tt < WD_TOK; ++tt) z[tt] = z0;
        for (int j = 0; j < L; ++j) {
            const float m = w2t[(size_t)j * C + c];
#pragma unroll
            for (int tt = 0; tt < WD_TOK; ++tt) z[tt] = fmaf(m, th[j * WD_TOK + tt], z[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < WD_TOK; ++tt)
            if (tt < n) w[(size_t)(t0 + tt) * C + c] = expf(-expf(z[tt]));
    }
}

ACV_API int acv_wkv_decay(const float* a, int lda, const float* w2t, const float* w0, float* w, int T_tokens, int C, int L,
                          cudaStream_t stream) {
    if (T_tokens <= 0) return 0;
    if (C <= 0 || L <= 0 || L > 1024) return ACV_ERR_SIZE;
    const int blocks_t = (T_tokens + WD_TOK - 1) / WD_TOK;
    // a thread owns one channel (a block 128 of them): enough blocks for every SM whatever the number of tokens
    const int blocks_c = min((C + 127) / 128, 65535);
    acv_launch(PDL_MISC, wkv_decay_kernel, dim3(blocks_t, blocks_c), 128, (size_t)L * WD_TOK * sizeof(float), stream, a, lda,
               w2t, w0, w, T_tokens, C, L);
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- the recurrence
struct WkvSegments {
    const int* seq;         // the request of each item (null: item i is request i, whole)
    const int* idx;         // its segment's number
    int len;                // tokens of a segment
    float* state;           // [items][H][D][DV]: what the first launch leaves
    float* decay;           // [items][H][D]: the product of a segment's decays
};

constexpr int wkv_max_threads(int R) { return R <= 8 ? 1024 : 512; }

template <typename T, int R, bool SUMMARY>
__global__ void __launch_bounds__(wkv_max_threads(R))
wkv_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v, int ld, const float* __restrict__ w,
           const float* __restrict__ u, float* __restrict__ state, const int* __restrict__ slots,
           const int* __restrict__ cu_q, WkvSegments sg, float* __restrict__ o, int ldo, int H, int D, int DV, int G, int TC,
           int DVT, int prefetch) {
    extern __shared__ __align__(16) float sm[];
    const bool whole_rows = D % R == 0;     // (R is a multiple of four, so D is one as well, and rows of k, r, w are 16-byte pieces)
    // two sets of staged tokens (with `prefetch`: float inputs in 16-byte pieces, the next chunk copied asynchronously
    // while this one is computed; otherwise the first set alone is used), then the chunk's partial sums
    const size_t set = (size_t)TC * (3 * D + DVT);
    float* red = sm + 2 * set;              // [TC][G][DVT]
    pdl_launch_dependents();
    pdl_wait();
    const int item = blockIdx.x, h = blockIdx.y;
    const int seq = sg.seq ? sg.seq[item] : item, z = sg.idx ? sg.idx[item] : 0;
    const int q0 = cu_q[seq], q1 = cu_q[seq + 1];
    const int t0 = q0 + z * sg.len, t1 = min(q1, t0 + sg.len);
    if (t1 <= t0) return;
    const bool last = t1 == q1;
    if (SUMMARY && last) return;
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int cl = tid % DVT, g = tid / DVT, c0 = blockIdx.z * DVT;
    const int c = c0 + cl;                  // this thread's column of S
    const bool owner = g < G && c < DV;
    const size_t HS = (size_t)D * DV;
    float* st = state + ((size_t)slots[seq] * H + h) * HS;
    // The request's state as this step found it: read from its slot by the first launch (and by a request's only
    // segment), which also leaves it in the unused entry of the request's last segment for the last launch, whose
    // last segment replaces the slot while its first one may not have begun.
    const int last_item = item - z + (q1 - q0 + sg.len - 1) / sg.len - 1;
    float* keep = sg.state ? sg.state + ((size_t)last_item * H + h) * HS : nullptr;
    float S[R], U[R], P[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int d = g * R + i;
        float s0 = 0.f;
        if (owner && d < D) {
            const size_t at = (size_t)d * DV + c;
            if (z == 0) {
                s0 = (SUMMARY || last) ? st[at] : keep[at];
                if (SUMMARY) keep[at] = s0;
            } else if (!SUMMARY) {
                s0 = sg.state[((size_t)(item - 1) * H + h) * HS + at];      // after the fold: what lies in front of this segment
            }
        }
        S[i] = s0;
        U[i] = (g < G && d < D) ? u[(size_t)h * D + d] : 0.f;
        P[i] = 1.f;
    }
    // a chunk's tokens as 16-byte pieces, asynchronously: rows of r, k, w (D floats) and of v (DVT floats)
    auto prefetch_chunk = [&](int tb, int n, float* base) {
        if constexpr (std::is_same<T, float>::value) {
            const int d4 = D >> 2, v4 = DVT >> 2;
            float* rs_ = base; float* ks_ = rs_ + (size_t)TC * D; float* ws_ = ks_ + (size_t)TC * D; float* vs_ = ws_ + (size_t)TC * D;
            for (int i = tid; i < n * d4; i += nthr) {
                const int tt = i / d4, e = (i - tt * d4) << 2;
                const size_t at = (size_t)(tb + tt) * ld + (size_t)h * D + e;
                if (!SUMMARY) cp_async16(smem_u32(rs_ + tt * D + e), r + at, true);
                cp_async16(smem_u32(ks_ + tt * D + e), k + at, true);
                cp_async16(smem_u32(ws_ + tt * D + e), w + (size_t)(tb + tt) * H * D + (size_t)h * D + e, true);
            }
            for (int i = tid; i < n * v4; i += nthr) {
                const int tt = i / v4, e = (i - tt * v4) << 2;
                const bool in = c0 + e < DV;
                cp_async16(smem_u32(vs_ + tt * DVT + e), in ? (const void*)(v + (size_t)(tb + tt) * ld + (size_t)h * DV + c0 + e) : (const void*)v, in);
            }
        }
    };
    if (prefetch) {
        prefetch_chunk(t0, min(TC, t1 - t0), sm);
        cp_async_commit();
    }
    int turn = 0;
    for (int tb = t0; tb < t1; tb += TC, turn ^= 1) {
        const int n = min(TC, t1 - tb);
        float* rs = sm + (prefetch ? turn * set : 0);   // [TC][D]
        float* ks = rs + (size_t)TC * D;                 // [TC][D]
        float* ws = ks + (size_t)TC * D;                 // [TC][D]
        float* vs = ws + (size_t)TC * D;                 // [TC][DVT]
        if (prefetch) {
            // the other set was read in the turn before this one, whose last barrier every thread has passed
            if (tb + TC < t1) prefetch_chunk(tb + TC, min(TC, t1 - tb - TC), sm + (turn ^ 1) * set);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
        for (int i = tid; i < n * D; i += nthr) {
            const int tt = i / D, e = i - tt * D;
            const size_t at = (size_t)(tb + tt) * ld + (size_t)h * D + e;
            if (!SUMMARY) rs[i] = to_f32(r[at]);
            ks[i] = to_f32(k[at]);
            ws[i] = w[(size_t)(tb + tt) * H * D + (size_t)h * D + e];
        }
        for (int i = tid; i < n * DVT; i += nthr) {
            const int tt = i / DVT, e = i - tt * DVT;
            vs[i] = c0 + e < DV ? to_f32(v[(size_t)(tb + tt) * ld + (size_t)h * DV + c0 + e]) : 0.f;
        }
        }
        __syncthreads();
        if (owner) {
            for (int tt = 0; tt < n; ++tt) {
                const float vv = vs[tt * DVT + cl];
                const float* kr = ks + tt * D + g * R;
                const float* rr = rs + tt * D + g * R;
                const float* wr = ws + tt * D + g * R;
                float part = 0.f;
                if (whole_rows) {       // every group's rows lie inside the head: 16-byte loads of k, r and w
#pragma unroll
                    for (int i4 = 0; i4 < R / 4; ++i4) {
                        const float4 k4 = reinterpret_cast<const float4*>(kr)[i4], w4 = reinterpret_cast<const float4*>(wr)[i4];
                        float4 r4 = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (!SUMMARY) r4 = reinterpret_cast<const float4*>(rr)[i4];
                        const float kx[4] = {k4.x, k4.y, k4.z, k4.w}, wx[4] = {w4.x, w4.y, w4.z, w4.w}, rx[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int i = i4 * 4 + e;
                            const float kv = kx[e] * vv;
                            if (!SUMMARY) part = fmaf(fmaf(U[i], kv, S[i]), rx[e], part);
                            S[i] = fmaf(wx[e], S[i], kv);
                            if (SUMMARY) P[i] *= wx[e];
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < R; ++i) {
                        if (g * R + i < D) {
                            const float kv = kr[i] * vv;
                            if (!SUMMARY) part = fmaf(fmaf(U[i], kv, S[i]), rr[i], part);
                            S[i] = fmaf(wr[i], S[i], kv);
                            if (SUMMARY) P[i] *= wr[i];
                        }
                    }
                }
                if (!SUMMARY) red[((size_t)tt * G + g) * DVT + cl] = part;
            }
        }
        __syncthreads();
        if (!SUMMARY) {
            for (int i = tid; i < n * DVT; i += nthr) {
                const int tt = i / DVT, e = i - tt * DVT;
                if (c0 + e >= DV) continue;
                float sum = 0.f;
                for (int gg = 0; gg < G; ++gg) sum += red[((size_t)tt * G + gg) * DVT + e];
                o[(size_t)(tb + tt) * ldo + (size_t)h * DV + c0 + e] = sum;
            }
        }
        // the next chunk's staging writes rs, ks, ws, vs only; its first barrier stands between this read of red and
        // the next write of it
    }
    if (owner && (SUMMARY || last)) {
        float* dst = SUMMARY ? sg.state + ((size_t)item * H + h) * HS : st;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int d = g * R + i;
            if (d < D) dst[(size_t)d * DV + c] = S[i];
        }
    }
    if (SUMMARY && owner && c == 0) {
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int d = g * R + i;
            if (d < D) sg.decay[((size_t)item * H + h) * D + d] = P[i];
        }
    }
}

// Between the two launches: S_in(z + 1) = diag(P(z)) S_in(z) + entry(z), in place over a request's entries.  grid
// (items, heads, tiles of 256 elements); the blocks of a request's first segment walk the request's entries.
__global__ void wkv_fold_kernel(WkvSegments sg, const int* __restrict__ cu_q, int H, int D, int DV) {
    pdl_launch_dependents();
    pdl_wait();
    const int item = blockIdx.x, h = blockIdx.y;
    if (sg.idx[item] != 0) return;
    const int seq = sg.seq[item];
    const int nseg = (cu_q[seq + 1] - cu_q[seq] + sg.len - 1) / sg.len;
    if (nseg < 3) return;           // the entry of a first segment already is what lies in front of the second
    const int HS = D * DV;
    float* e = sg.state + ((size_t)item * H + h) * HS;
    const float* p = sg.decay + ((size_t)item * H + h) * D;
    const size_t step = (size_t)H * HS, pstep = (size_t)H * D;
    const int i = blockIdx.z * blockDim.x + threadIdx.x;
    if (i >= HS) return;
    const int d = i / DV;
    float s = e[i];
    for (int z0 = 1; z0 < nseg - 1; ++z0) {
        s = fmaf(p[z0 * pstep + d], s, e[z0 * step + i]);
        e[z0 * step + i] = s;
    }
}

template <typename T, int R>
static int launch_wkv(const void* r, const void* k, const void* v, int ld, const float* w, const float* u, float* state,
                      const int* slots, const int* cu_q, WkvSegments sg, int summaries, float* o, int ldo, int n_items, int H,
                      int D, int DV, int DVT, cudaStream_t stream) {
    const int G = (D + R - 1) / R;
    const int threads = ((G * DVT + 31) / 32) * 32;
    const size_t per_token = (size_t)(2 * (3 * D + DVT) + G * DVT) * sizeof(float);
    const dim3 grid(n_items, H, (DV + DVT - 1) / DVT);
    // float inputs whose rows are 16-byte pieces are copied asynchronously, a chunk ahead
    const int prefetch = std::is_same<T, float>::value && D % 4 == 0 && DV % 4 == 0 && DVT % 4 == 0 && ld % 4 == 0 &&
                         !((uintptr_t)r & 15) && !((uintptr_t)k & 15) && !((uintptr_t)v & 15) && !((uintptr_t)w & 15);
    int TC = (int)((48 * 1024) / per_token);
    TC = TC > 32 ? 32 : TC;
    if (TC < 1) TC = 1;
    const size_t smem = per_token * TC;
    if (smem > 200 * 1024) return ACV_ERR_SIZE;
    if (smem > 48 * 1024) {
        static AcvSmemConfig cfg, cfg_s;
        int e = acv_ensure_smem(cfg, wkv_kernel<T, R, false>, (int)smem);
        if (!e && summaries) e = acv_ensure_smem(cfg_s, wkv_kernel<T, R, true>, (int)smem);
        if (e) return e;
    }
    if (summaries) {
        acv_launch(PDL_ATTN, wkv_kernel<T, R, true>, grid, threads, smem, stream, (const T*)r, (const T*)k, (const T*)v, ld, w, u,
                   state, slots, cu_q, sg, o, ldo, H, D, DV, G, TC, DVT, prefetch);
        acv_launch(PDL_ATTN, wkv_fold_kernel, dim3(n_items, H, (D * DV + 255) / 256), 256, 0, stream, sg, cu_q, H, D, DV);
    }
    acv_launch(PDL_ATTN, wkv_kernel<T, R, false>, grid, threads, smem, stream, (const T*)r, (const T*)k, (const T*)v, ld, w, u,
               state, slots, cu_q, sg, o, ldo, H, D, DV, G, TC, DVT, prefetch);
    return acv_launch_status();
}

template <typename T>
static int wkv_by_rows(int R, const void* r, const void* k, const void* v, int ld, const float* w, const float* u, float* state,
                       const int* slots, const int* cu_q, WkvSegments sg, int summaries, float* o, int ldo, int n_items,
                       int H, int D, int DV, int DVT, cudaStream_t stream) {
#define WKV_CASE(N)                                                                                                  \
    case N:                                                                                                          \
        return launch_wkv<T, N>(r, k, v, ld, w, u, state, slots, cu_q, sg, summaries, o, ldo, n_items, H, D, DV, DVT, stream);
    switch (R) {
        WKV_CASE(4) WKV_CASE(8) WKV_CASE(16) WKV_CASE(32)
    }
#undef WKV_CASE
    return ACV_ERR_SIZE;
}

// r, k: rows of H*D at stride ld; v: rows of H*DV at stride ld (all of one type); w: float [T, H*D] dense; u: float [H*D];
// o: float rows of H*DV at stride ldo; state: float [slots][H][D][DV].
// seg_seq, seg_idx: the step's n_items items (null: one item for each request, its whole portion); seg_state: float
// [n_items][H][D][DV] and seg_decay: float [n_items][H][D], scratch of the first launch, which runs when `summaries` is set.
ACV_API int acv_wkv(const void* r, const void* k, const void* v, int ld, const float* w, const float* u, float* state,
                    const int* slots, const int* cu_q, const int* seg_seq, const int* seg_idx, int seg_len, float* seg_state,
                    float* seg_decay, int summaries, float* o, int ldo, int n_items, int H, int D, int DV, int dtype,
                    cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (H <= 0 || D <= 0 || DV <= 0) return ACV_ERR_SIZE;
    if (seg_len <= 0 || (summaries && (!seg_seq || !seg_idx || !seg_state || !seg_decay))) return ACV_ERR_SIZE;
    WkvSegments sg;
    sg.seq = seg_seq; sg.idx = seg_idx; sg.len = seg_len; sg.state = seg_state; sg.decay = seg_decay;
    // value columns of a block: all of them up to 128; rows of the state a thread keeps: the fewest with which the
    // block has 512 threads at most (three arrays of R registers a thread)
    int DVT = DV <= 128 ? DV : 128;
    while (DVT > 32 && ((D + 31) / 32) * DVT > 512) DVT = (DVT / 2 + 3) & ~3;      // (a very long key: fewer columns a block)
    int R = 4;
    while (R < 32 && ((D + R - 1) / R) * DVT > 512) R *= 2;     // (measured at 64 x 64: blocks of 512 threads 238 us for 2048 tokens, of 256 and 128 threads 288 and 290)
    if (((D + R - 1) / R) * DVT > wkv_max_threads(R)) return ACV_ERR_SIZE;
    if (dtype == ACV_F32)
        return wkv_by_rows<float>(R, r, k, v, ld, w, u, state, slots, cu_q, sg, summaries, o, ldo, n_items, H, D, DV, DVT, stream);
    if (dtype == ACV_BF16)
        return wkv_by_rows<bf16>(R, r, k, v, ld, w, u, state, slots, cu_q, sg, summaries, o, ldo, n_items, H, D, DV, DVT, stream);
    return ACV_ERR_DTYPE;
}
