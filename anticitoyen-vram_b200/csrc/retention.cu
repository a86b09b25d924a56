// Retention: linear attention with a fixed decay per head, no softmax and no denominator.
//
//   S_t = decay_h * S_{t-1} + k_t v_t^T          S: [D, DV] per (request, head), float, kept in a state slot
//   o_t = S_t^T q_t
//
// q and k are rotated by position (rotate-half over the first `rot` elements, cos and sin from a table) and k is
// multiplied by k_scale, all in float, as they are staged (with `act` set, q, k and v first pass through silu); scores, state and sums are 32-bit.  A second kernel
// brings each head's o to unit RMS (no weight), multiplies by silu(gate) and a constant, and rounds once.
//
// acv_retention: grid (items, heads, tiles of DVT value columns: the columns of S do not know of one another, and a
// head too wide for one block's threads is cut).  The block's threads are G groups of DVT: thread (g, c) keeps rows
// g*R .. g*R+R-1 of column c of S in registers (R as large as the registers allow, up to 64: a thread that holds a
// whole column needs no other thread for its sums, and a block of DV threads leaves room for several blocks on an SM), walks its tokens in chunks of TC (q, k, v staged in shared memory,
// the partial sums of the chunk reduced over the groups afterwards), and writes S back.
//
// The recurrence is linear in S, so a long portion is cut into segments of seg_len tokens that run side by side (the
// step's list of (request, segment) items): a first launch leaves the state that each segment reaches from zero (the
// first one from the request's state), without outputs; a second one folds what lies before its segment,
// S_in(z) = decay^seg_len S_in(z-1) + S_seg(z-1) (a small launch of its own between the two), and walks the segment again with outputs.  Steps of short portions and
// single tokens run the second launch alone.
#include "common.cuh"
#include <stdlib.h>

#define RET_WANT_THREADS 512

// the most threads of a block by the rows a thread keeps: the registers of the whole block have to fit an SM's file
constexpr int ret_max_threads(int R) { return R <= 16 ? 1024 : (R <= 32 ? 512 : 256); }

struct RetSegments {
    const int* seq;         // the request of each item (null: item i is request i, whole)
    const int* idx;         // its segment's number
    int len;                // tokens of a segment
    float* state;           // [items][H][D][DV]: what the first launch leaves
};

template <typename T, int R, bool SUMMARY>
__global__ void __launch_bounds__(ret_max_threads(R)) retention_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int ld,
                                 const float* __restrict__ cos_sin, int rot, int table_rows,
                                 const int* __restrict__ positions, const float* __restrict__ decay, float k_scale,
                                 float* __restrict__ state, const int* __restrict__ slots,
                                 const int* __restrict__ cu_q, RetSegments sg, float* __restrict__ o, int ldo, int H, int D, int DV,
                                 int G, int TC, int DVT, int act) {
    extern __shared__ float sm[];
    float* qs = sm;                         // [TC][D]
    float* ks = qs + (size_t)TC * D;        // [TC][D]
    float* vs = ks + (size_t)TC * D;        // [TC][DVT]
    float* red = vs + (size_t)TC * DVT;     // [TC][G][DVT]
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
    const float dec = decay[h];
    const size_t HS = (size_t)D * DV;
    float* st = state + ((size_t)slots[seq] * H + h) * HS;
    // The request's state as this step found it: read from its slot by the first launch (and by a request's only
    // segment), which also leaves it in the unused entry of the request's last segment for the second launch, whose
    // last segment replaces the slot while its first one may not have begun.
    const int last_item = item - z + (q1 - q0 + sg.len - 1) / sg.len - 1;
    float* keep = sg.state ? sg.state + ((size_t)last_item * H + h) * HS : nullptr;
    float S[R];
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
                // what lies in front of this segment: the entry of the segment before, after acv_retention's fold
                s0 = sg.state[((size_t)(item - 1) * H + h) * HS + at];
            }
        }
        S[i] = s0;
    }
    const int half = rot >> 1;
    for (int tb = t0; tb < t1; tb += TC) {
        const int n = min(TC, t1 - tb);
        for (int i = tid; i < n * D; i += nthr) {
            const int tt = i / D, e = i - tt * D;
            const size_t at = (size_t)(tb + tt) * ld + (size_t)h * D + e;
            float qv = to_f32(q[at]), kv = to_f32(k[at]);
            if (act) {          // silu of the projections, in float, before anything else
                qv = qv / (1.f + expf(-qv));
                kv = kv / (1.f + expf(-kv));
            }
            qs[i] = qv;
            ks[i] = kv * k_scale;
        }
        for (int i = tid; i < n * DVT; i += nthr) {
            const int tt = i / DVT, e = i - tt * DVT;
            float vv = c0 + e < DV ? to_f32(v[(size_t)(tb + tt) * ld + (size_t)h * DV + c0 + e]) : 0.f;
            if (act) vv = vv / (1.f + expf(-vv));
            vs[i] = vv;
        }
        __syncthreads();
        if (cos_sin) {
            for (int i = tid; i < n * half; i += nthr) {        // a pair (e, e + half) is turned by one thread
                const int tt = i / half, e = i - tt * half;
                const int pos = positions[tb + tt];
                if (pos < 0 || pos >= table_rows) continue;
                const float* cs = cos_sin + (size_t)pos * rot;
                const float co = cs[e], si = cs[half + e];
                float* a = qs + tt * D;
                const float q0 = a[e], q1 = a[e + half];
                a[e] = q0 * co - q1 * si;
                a[e + half] = q1 * co + q0 * si;
                a = ks + tt * D;
                const float k0 = a[e], k1 = a[e + half];
                a[e] = k0 * co - k1 * si;
                a[e + half] = k1 * co + k0 * si;
            }
            __syncthreads();
        }
        if (owner) {
            for (int tt = 0; tt < n; ++tt) {
                const float vv = vs[tt * DVT + cl];
                const float* kr = ks + tt * D + g * R;
                const float* qr = qs + tt * D + g * R;
                float part = 0.f;
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    if (g * R + i < D) {
                        S[i] = fmaf(dec, S[i], kr[i] * vv);
                        if (!SUMMARY) part = fmaf(S[i], qr[i], part);
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
        // the next chunk's staging writes qs, ks, vs only; its first barrier stands between this read of red and the
        // next write of it
    }
    if (owner && (SUMMARY || last)) {
        float* dst = SUMMARY ? sg.state + ((size_t)item * H + h) * HS : st;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int d = g * R + i;
            if (d < D) dst[(size_t)d * DV + c] = S[i];
        }
    }
}

// Between the two launches: the entries of a request's segments, each the state its segment reaches from zero (the
// first one from the request's state), become the states in front of the segments that follow,
// S_in(z + 1) = decay^seg_len S_in(z) + entry(z), in place.  grid (items, heads, tiles of 256 elements); the blocks of a
// request's first segment walk the request's entries, a thread one element, eight entries' loads at a time.
__global__ void retention_fold_kernel(RetSegments sg, const int* __restrict__ cu_q, const float* __restrict__ decay, int H, int HS) {
    pdl_launch_dependents();
    pdl_wait();
    const int item = blockIdx.x, h = blockIdx.y;
    if (sg.idx[item] != 0) return;
    const int seq = sg.seq[item];
    const int nseg = (cu_q[seq + 1] - cu_q[seq] + sg.len - 1) / sg.len;
    if (nseg < 3) return;           // the entry of a first segment already is what lies in front of the second
    const float dec_len = exp2f((float)sg.len * log2f(decay[h]));
    float* e = sg.state + ((size_t)item * H + h) * HS;
    const size_t step = (size_t)H * HS;
    const int i = blockIdx.z * blockDim.x + threadIdx.x;
    if (i >= HS) return;
    float s = e[i];
    for (int z0 = 1; z0 < nseg - 1; z0 += 8) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = z0 + k < nseg - 1 ? e[(z0 + k) * step + i] : 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (z0 + k < nseg - 1) {
                s = fmaf(dec_len, s, v[k]);
                e[(z0 + k) * step + i] = s;
            }
        }
    }
}

template <typename T, int R>
static int launch_retention(const void* q, const void* k, const void* v, int ld, const float* cos_sin, int rot,
                            int table_rows, const int* positions, const float* decay, float k_scale, float* state,
                            const int* slots, const int* cu_q, RetSegments sg, int summaries, float* o, int ldo, int num_seqs, int H, int D, int DV,
                            int DVT, int act, cudaStream_t stream) {
    const int G = (D + R - 1) / R;
    const int threads = ((G * DVT + 31) / 32) * 32;
    const size_t per_token = (size_t)(2 * D + DVT + G * DVT) * sizeof(float);
    const dim3 grid(num_seqs, H, (DV + DVT - 1) / DVT);
    int TC = (int)((48 * 1024) / per_token);
    TC = TC > 32 ? 32 : TC;
    if (TC < 1) TC = 1;
    const size_t smem = per_token * TC;
    if (smem > 200 * 1024) return ACV_ERR_SIZE;
    if (smem > 48 * 1024) {
        static AcvSmemConfig cfg, cfg_s;
        int e = acv_ensure_smem(cfg, retention_kernel<T, R, false>, (int)smem);
        if (!e && summaries) e = acv_ensure_smem(cfg_s, retention_kernel<T, R, true>, (int)smem);
        if (e) return e;
    }
    if (summaries) {
        acv_launch(PDL_ATTN, retention_kernel<T, R, true>, grid, threads, smem, stream, (const T*)q, (const T*)k,
                   (const T*)v, ld, cos_sin, rot, table_rows, positions, decay, k_scale, state, slots, cu_q, sg, o, ldo, H, D, DV, G, TC, DVT, act);
        acv_launch(PDL_ATTN, retention_fold_kernel, dim3(num_seqs, H, (D * DV + 255) / 256), 256, 0, stream, sg, cu_q, decay, H, D * DV);
    }
    acv_launch(PDL_ATTN, retention_kernel<T, R, false>, grid, threads, smem, stream, (const T*)q, (const T*)k,
               (const T*)v, ld, cos_sin, rot, table_rows, positions, decay, k_scale, state, slots, cu_q, sg, o, ldo, H, D, DV, G, TC, DVT, act);
    return acv_launch_status();
}

template <typename T>
static int retention_by_rows(int R, const void* q, const void* k, const void* v, int ld, const float* cos_sin, int rot,
                             int table_rows, const int* positions, const float* decay, float k_scale, float* state,
                             const int* slots, const int* cu_q, RetSegments sg, int summaries, float* o, int ldo, int num_seqs, int H, int D, int DV,
                             int DVT, int act, cudaStream_t stream) {
#define RET_CASE(N)                                                                                                  \
    case N:                                                                                                          \
        return launch_retention<T, N>(q, k, v, ld, cos_sin, rot, table_rows, positions, decay, k_scale, state, slots, \
                                      cu_q, sg, summaries, o, ldo, num_seqs, H, D, DV, DVT, act, stream);
    switch (R) {
        RET_CASE(4) RET_CASE(8) RET_CASE(16) RET_CASE(32) RET_CASE(64)
    }
#undef RET_CASE
    return ACV_ERR_SIZE;
}

// q, k: rows of H*D at stride ld; v: rows of H*DV at stride ld; o: float rows of H*DV at stride ldo;
// state: [slots][H][D][DV] float; decay: [H] float; cos_sin: [table_rows][rot] float or null.
// seg_seq, seg_idx: the step's n_items items (null: one item for each request, its whole portion); seg_state: float
// [n_items][H][D][DV] scratch of the first launch, which runs when `summaries` is set.
ACV_API int acv_retention(const void* q, const void* k, const void* v, int ld, const float* cos_sin, int rot,
                          int table_rows, const int* positions, const float* decay, float k_scale, float* state,
                          const int* slots, const int* cu_q, const int* seg_seq, const int* seg_idx, int seg_len,
                          float* seg_state, int summaries, float* o, int ldo, int n_items, int H, int D, int DV,
                          int dtype, int act, cudaStream_t stream) {
    const int num_seqs = n_items;
    if (num_seqs <= 0) return 0;
    if (H <= 0 || D <= 0 || DV <= 0 || (cos_sin && (rot <= 0 || rot > D || (rot & 1)))) return ACV_ERR_SIZE;
    if (seg_len <= 0 || (summaries && (!seg_seq || !seg_idx || !seg_state))) return ACV_ERR_SIZE;
    RetSegments sg;
    sg.seq = seg_seq; sg.idx = seg_idx; sg.len = seg_len; sg.state = seg_state;
    // rows of the state that a thread keeps: the fewest that let the block fit `want` threads (measured on a B200 at
    // 64 x 128 per head: blocks of 1024, 512 and 128 threads, see the design notes); ACVRAM_RETENTION_ROWS forces a choice
    static const int forced = getenv("ACVRAM_RETENTION_ROWS") ? atoi(getenv("ACVRAM_RETENTION_ROWS")) : 0;
    auto rows_for = [&](int dvt, int want) {        // the fewest rows with which G groups of dvt threads fit `want`, 0: none
        for (int r = 4; r <= 64; r *= 2) {
            const int most = ret_max_threads(r) < want ? ret_max_threads(r) : want;
            if (((D + r - 1) / r) * dvt <= most) return r;
        }
        return 0;
    };
    // a head whose columns do not fit one block is cut into tiles of columns (each a block of its own)
    int DVT = DV, R = 0;
    while (true) {
        R = rows_for(DVT, RET_WANT_THREADS);
        if (!R) R = rows_for(DVT, 1024);
        if (R || DVT <= 32) break;
        DVT = DVT > 128 ? 128 : DVT / 2;
    }
    if (forced == 4 || forced == 8 || forced == 16 || forced == 32 || forced == 64)
        if (((D + forced - 1) / forced) * DVT <= ret_max_threads(forced)) R = forced;
    if (!R) return ACV_ERR_SIZE;          // (key rows of more than 512 elements are not built)
    if (dtype == ACV_F32)
        return retention_by_rows<float>(R, q, k, v, ld, cos_sin, rot, table_rows, positions, decay, k_scale, state, slots,
                                        cu_q, sg, summaries, o, ldo, num_seqs, H, D, DV, DVT, act, stream);
    if (dtype == ACV_BF16)
        return retention_by_rows<bf16>(R, q, k, v, ld, cos_sin, rot, table_rows, positions, decay, k_scale, state, slots,
                                       cu_q, sg, summaries, o, ldo, num_seqs, H, D, DV, DVT, act, stream);
    return ACV_ERR_DTYPE;
}

// ----------------------------------------------------------------------------- unit RMS, weight, gate, constant
// out[t][u*group + e] = o / sqrt(mean_e(o^2) + eps) * w[u*group + e] * gate_fn(gate) * out_scale over groups of `group`
// elements (a head's DV: each head by itself; all H*DV: the heads side by side normed together); w null: no weight;
// gate_fn silu (0) or sigmoid (1).  One warp per (token, group).
template <typename T>
__global__ void retention_gate_kernel(const float* __restrict__ o, int ldo, const T* __restrict__ gate, int ldg,
                                      T* __restrict__ out, int ld_out, int groups, int group, const float* __restrict__ w,
                                      int gate_kind, float eps, float out_scale, int T_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (blockDim.x >> 5) + warp;
    if (unit >= T_tokens * groups) return;
    const int t = unit / groups, u = unit - t * groups;
    const float* orow = o + (size_t)t * ldo + (size_t)u * group;
    float ss = 0.f;
    for (int e = lane; e < group; e += 32) ss = fmaf(orow[e], orow[e], ss);
    ss = warp_sum(ss);
    const float inv = out_scale / sqrtf(ss / (float)group + eps);
    const T* grow = gate + (size_t)t * ldg + (size_t)u * group;
    const float* wr = w ? w + (size_t)u * group : nullptr;
    T* dst = out + (size_t)t * ld_out + (size_t)u * group;
    for (int e = lane; e < group; e += 32) {
        const float z = to_f32(grow[e]);
        const float sg = 1.f / (1.f + expf(-z));
        float v = orow[e] * inv;
        if (wr) v *= wr[e];
        dst[e] = from_f32<T>(v * (gate_kind == 1 ? sg : z * sg));
    }
}

ACV_API int acv_retention_gate(const float* o, int ldo, const void* gate, int ldg, void* out, int ld_out, int T_tokens,
                               int H, int DV, float eps, float out_scale, int dtype, const float* weight, int joint,
                               int gate_kind, cudaStream_t stream) {
    if (T_tokens <= 0) return 0;
    const int warps = 8;
    const int groups = joint ? 1 : H, group = joint ? H * DV : DV;
    const int grid = (T_tokens * groups + warps - 1) / warps;
    if (dtype == ACV_F32)
        acv_launch(PDL_MISC, retention_gate_kernel<float>, grid, warps * 32, 0, stream, o, ldo, (const float*)gate, ldg,
                   (float*)out, ld_out, groups, group, weight, gate_kind, eps, out_scale, T_tokens);
    else if (dtype == ACV_BF16)
        acv_launch(PDL_MISC, retention_gate_kernel<bf16>, grid, warps * 32, 0, stream, o, ldo, (const bf16*)gate, ldg,
                   (bf16*)out, ld_out, groups, group, weight, gate_kind, eps, out_scale, T_tokens);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}
