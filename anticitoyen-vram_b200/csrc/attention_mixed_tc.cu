// Head-mixing attention (see attention_mixed.cu for the score steps) on the tensor cores, bfloat16 pages and queries.
//
// The softmax of head h at (query i, key j) needs every head's score of that pair, so the unit of work is a tile of 16
// query tokens of one request with ALL heads: one warp a head, 16 x BN scores a warp and key tile on mma.sync m16n8k16
// (float accumulation).  Each warp leaves its scores, after temp, soft cap and distance bias (all float), in shared
// memory; after a barrier warp h mixes its row of `talk` over them straight into the accumulator layout of the tile,
// masks, runs the online softmax and multiplies the weights (rounded to bfloat16 as the other tensor-core attention
// kernels do) with its kv-head's values.
//
// More than 16 heads: the tile is shared by a thread-block cluster of 2 or 4 CTAs, each with NH / cluster heads (and
// the key/value heads those read); the mix reads the other CTAs' scores through distributed shared memory and the two
// barriers around the scores become cluster barriers.
//
// Keys and values arrive by cp.async, one buffer each: the next key tile is fetched while the mix, softmax and value
// product of this one run (its buffer is free once the scores are written), the next value tile while the next
// scores are computed.  Rows are padded by 16 bytes instead of swizzled, so head sizes need only be multiples of 8
// (zero-filled to the next multiple of 16 in shared memory).
//
// Work: `n_tiles` tiles of 128 query tokens from the step's work list, each cut into 8 sub-tiles of 16, then `n_dec`
// requests with one token each (a sub-tile with one row).
#include "mma_tiles.cuh"

#define MT_ROWS 16
#define MT_SUB 8            // sub-tiles in a work-list tile of 128 tokens
#define MT_MAX_WARPS 16
#define MT_LOG2E 1.4426950408889634f

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}
__device__ __forceinline__ float2 ld_cluster_f2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
    return v;
}

// tanh(x) = 1 - 2 / (e^(2x) + 1) on the hardware's 2^x and reciprocal: absolute error about 2e-7 (the subtraction loses
// nothing that matters where |x| is small: the result is then scaled by the cap, and the error stays absolute)
__device__ __forceinline__ float fast_tanh(float x) {
    const float e = fast_exp2(x * (2.f * MT_LOG2E));
    return 1.f - __fdividef(2.f, e + 1.f);
}

struct MixedArgs {
    const bf16* q; int q_stride; bf16* out; int out_stride;
    const bf16* k_pages; const bf16* v_pages;
    const int* tile_seq; const int* tile_q0; int n_tiles;
    const int* dec_tokens; const int* dec_seqs; int n_dec;
    const int* cu_q; const int* kv_len;
    const int* block_table; int bt_stride; const int* bt_rows;
    int NH, NKV, D, DV, page_size, num_pages;
    float scale; int window;
    const float* temp; float cap; const float* rel; const int* bucket_of; int n_dist, last_row, rel_rows;
    const float* talk;
    int cl;                 // CTAs in a cluster (1, 2 or 4)
    int n_split;            // CTAs (or clusters) that share the keys of a one-token request (1: none)
    float* part_acc;        // n_split > 1: [n_dec][n_split][NH][DV] unnormalised sums
    float* part_ml;         //              [n_dec][n_split][NH][2] running maximum (in powers of two) and sum
};

template <int BN, int NDV>
__global__ void __launch_bounds__(MT_MAX_WARPS * 32)
attn_mixed_tc_kernel(const MixedArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int NH = a.NH, NKV = a.NKV, D = a.D, DV = a.DV;
    const int cl = a.cl;
    const int HPC = NH / cl;                    // heads of this CTA = its warps
    const int DP = (D + 15) & ~15, DVP = (DV + 15) & ~15;
    const int QP = DP * 2 + 16, VP = DVP * 2 + 16;          // row pitches in bytes
    const int SP = BN + 8;                                   // floats in a row of scores
    const int rank = cl > 1 ? (int)cluster_rank() : 0;
    const int h_first = rank * HPC;
    const int group = NH / NKV;
    const int kv_first = h_first / group;
    const int n_kv = (h_first + HPC - 1) / group - kv_first + 1;    // the same in every CTA: the launcher sees to it
    const int n_kv_max = n_kv;

    unsigned char* q_s = smem;                                              // [HPC][16][QP]
    unsigned char* k_s = q_s + (size_t)HPC * MT_ROWS * QP;                  // [n_kv][BN][QP]
    unsigned char* v_s = k_s + (size_t)n_kv_max * BN * QP;                  // [n_kv][BN][VP]
    float* s_s = reinterpret_cast<float*>(v_s + (size_t)n_kv_max * BN * VP);    // [HPC][16][SP]
    float* tk_s = s_s + (size_t)HPC * MT_ROWS * SP;                         // [HPC][NH]: rows of talk of this CTA's heads
    float* rel_s = tk_s + (size_t)HPC * NH;                                 // [rel_rows][NH]
    float* bias_s = rel_s + (size_t)a.rel_rows * NH;                        // [HPC][BN + 16]: this tile's bias by distance
    constexpr int NDD = BN + 16;
    int* keyrow_s = reinterpret_cast<int*>(bias_s + (size_t)HPC * NDD);     // [2][BN]: a key's row in kv-head 0 of its page, -1: none

    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nthr = blockDim.x;
    const int unit = blockIdx.x / cl;
    int seq, tok0, rows, pos0;
    int split = 0, part = -1;                   // part >= 0: this CTA leaves a partial result at that index
    if (unit < a.n_tiles * MT_SUB) {
        const int tile = unit / MT_SUB;
        seq = a.tile_seq[tile];
        const int q0 = a.tile_q0[tile] + (unit % MT_SUB) * MT_ROWS;
        const int q_len = a.cu_q[seq + 1] - a.cu_q[seq];
        if (q0 >= q_len) return;                 // the same for every CTA of the cluster
        tok0 = a.cu_q[seq] + q0;
        rows = min(MT_ROWS, q_len - q0);
        pos0 = a.kv_len[seq] - q_len + q0;
    } else {
        const int u = unit - a.n_tiles * MT_SUB;
        const int i = u / a.n_split;
        split = u % a.n_split;
        if (a.n_split > 1) part = u;
        seq = a.dec_seqs[i];
        tok0 = a.dec_tokens[i];
        rows = 1;
        pos0 = a.kv_len[seq] - 1;
    }
    const int h = h_first + warp;
    const int kv_local = h / group - kv_first;
    if (pos0 < 0) {                              // a padded slot of a captured batch: nothing is kept for it
        if (part >= 0) {
            if (lane == 0) {
                a.part_ml[((size_t)part * NH + h) * 2] = -INFINITY;
                a.part_ml[((size_t)part * NH + h) * 2 + 1] = 0.f;
            }
            return;
        }
        for (int e = lane; e < DV; e += 32) a.out[(size_t)tok0 * a.out_stride + (size_t)h * DV + e] = from_f32<bf16>(0.f);
        return;
    }
    const int* bt = a.block_table + (size_t)(a.bt_rows ? a.bt_rows[seq] : seq) * a.bt_stride;
    const int window = a.window;
    const int hi = pos0 + rows - 1;
    const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int j_first = lo & ~(BN - 1);
    const int n_all = (hi - j_first) / BN + 1;
    // the tiles of this CTA: all of them, or its share of a one-token request's
    const int per_split = (n_all + a.n_split - 1) / a.n_split;
    const int t_first = part >= 0 ? split * per_split : 0;
    const int n_t = part >= 0 ? min(n_all, t_first + per_split) : n_all;
    const int CH = DP / 8, CHV = DVP / 8;

    // queries of all local heads, the talk rows, the bias table
    for (int id = tid; id < HPC * MT_ROWS * CH; id += nthr) {
        const int c = id % CH, r = (id / CH) % MT_ROWS, w = id / (CH * MT_ROWS);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows && c * 8 < D)
            v = *reinterpret_cast<const uint4*>(a.q + (size_t)(tok0 + r) * a.q_stride + (size_t)(h_first + w) * D + c * 8);
        *reinterpret_cast<uint4*>(q_s + ((size_t)w * MT_ROWS + r) * QP + c * 16) = v;
    }
    for (int id = tid; id < HPC * NH; id += nthr) {
        const int w = id / NH, g = id % NH;
        tk_s[id] = a.talk ? a.talk[(size_t)(h_first + w) * NH + g] : (g == h_first + w ? 1.f : 0.f);
    }
    if (a.rel)
        for (int id = tid; id < a.rel_rows * NH; id += nthr) rel_s[id] = a.rel[id];

    // a chunk's place: id = (kvl * BN + r) * CH + c, one division by CH (BN is a power of two); the place of a tile's
    // keys in their pages is looked up once per tile, a tile ahead, not once per copied chunk
    const int page_shift = (a.page_size & (a.page_size - 1)) == 0 ? __ffs(a.page_size) - 1 : -1;
    auto find_rows = [&](int t) {
        for (int r = tid; r < BN; r += nthr) {
            const int j = j_first + t * BN + r;
            int row = -1;
            if (j <= hi && j >= lo) {
                const int pi = page_shift >= 0 ? j >> page_shift : j / a.page_size;
                const int pg = bt[pi];
                if (pg >= 0 && pg < a.num_pages) row = pg * NKV * a.page_size + (j - pi * a.page_size);
            }
            keyrow_s[(t & 1) * BN + r] = row;
        }
    };
    auto load_keys = [&](int t) {
        const int* rows_of = keyrow_s + (t & 1) * BN;
        for_row_chunks(tid, nthr, n_kv * BN, CH, [&](int rr, int c) {
            const int r = rr & (BN - 1), kvl = rr / BN;
            const int row = rows_of[r];
            const bool ok = row >= 0 && c * 8 < D;
            const size_t off = ok ? ((size_t)row + (size_t)(kv_first + kvl) * a.page_size) * D + c * 8 : 0;
            cp_async16(smem_u32(k_s + (size_t)rr * QP + c * 16), a.k_pages + off, ok);
        });
    };
    auto load_values = [&](int t) {
        const int* rows_of = keyrow_s + (t & 1) * BN;
        for_row_chunks(tid, nthr, n_kv * BN, CHV, [&](int rr, int c) {
            const int r = rr & (BN - 1), kvl = rr / BN;
            const int row = rows_of[r];
            const bool ok = row >= 0 && c * 8 < DV;
            const size_t off = ok ? ((size_t)row + (size_t)(kv_first + kvl) * a.page_size) * DV + c * 8 : 0;
            cp_async16(smem_u32(v_s + (size_t)rr * VP + c * 16), a.v_pages + off, ok);
        });
    };
    find_rows(t_first);
    __syncthreads();
    load_keys(t_first);
    cp_async_commit();
    load_values(t_first);
    cp_async_commit();

    const int mi = lane >> 3, lr = lane & 7;
    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;
    const int p_row[2] = {pos0 + r_lo, pos0 + r_lo + 8};
    const int lo_row[2] = {window > 0 ? max(0, p_row[0] - window + 1) : 0, window > 0 ? max(0, p_row[1] - window + 1) : 0};
    const float qk_scale = a.scale * (a.temp ? a.temp[h] : 1.f);
    const float cap = a.cap, inv_cap = a.cap > 0.f ? 1.f / a.cap : 0.f;
    const uint32_t qb = smem_u32(q_s + (size_t)warp * MT_ROWS * QP);
    const uint32_t kb = smem_u32(k_s + (size_t)kv_local * BN * QP);
    const uint32_t vb = smem_u32(v_s + (size_t)kv_local * BN * VP);
    float* s_own = s_s + (size_t)warp * MT_ROWS * SP;
    const uint32_t s_base = smem_u32(s_s);

    float acc[2 * NDV][4];
#pragma unroll
    for (int i = 0; i < 2 * NDV; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    if (a.rel) __syncthreads();                 // the bias table is in shared memory
    for (int t = t_first; t < n_t; ++t) {
        const int j0 = j_first + t * BN;
        if (a.rel) {
            // the distances of this tile's (query, key) pairs span BN + 15 values from dmin on (row r, key c of the tile:
            // dmin + r + BN - 1 - c): each head's bias for every one of them, looked up once
            const int dmin = pos0 - (j0 + BN - 1);
            for (int id = tid; id < HPC * NDD; id += nthr) {
                const int w = id / NDD, dist = dmin + (id - w * NDD);
                bias_s[id] = dist >= 0 ? rel_s[(dist < a.n_dist ? a.bucket_of[dist] : a.last_row) * NH + h_first + w] : 0.f;
            }
        }
        if (t + 1 < n_t) find_rows(t + 1);
        cp_async_wait<1>();                     // this tile's keys (its values may still be on their way)
        __syncthreads();
        float s[BN / 8][4];
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
        for (int kd = 0; kd < DP / 16; ++kd) {
            uint32_t qf[4];
            ldmatrix_x4(qf, qb + ((mi & 1) * 8 + lr) * QP + (kd * 2 + (mi >> 1)) * 16);
#pragma unroll
            for (int np = 0; np < BN / 16; ++np) {
                uint32_t b[4];
                ldmatrix_x4(b, kb + (np * 16 + (mi >> 1) * 8 + lr) * QP + (kd * 2 + (mi & 1)) * 16);
                mma_bf16(s[2 * np], qf, b[0], b[1]);
                mma_bf16(s[2 * np + 1], qf, b[2], b[3]);
            }
        }
        // this head's steps on its own scores, then into shared memory for every head's mix
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float x = s[nt][e] * qk_scale;
                if (cap > 0.f) x = cap * fast_tanh(x * inv_cap);
                if (a.rel) x += bias_s[warp * NDD + (r_lo + (e >> 1) * 8 + BN - 1) - (nt * 8 + c_lo + (e & 1))];
                s[nt][e] = x;
            }
            *reinterpret_cast<float2*>(s_own + r_lo * SP + nt * 8 + c_lo) = make_float2(s[nt][0], s[nt][1]);
            *reinterpret_cast<float2*>(s_own + (r_lo + 8) * SP + nt * 8 + c_lo) = make_float2(s[nt][2], s[nt][3]);
        }
        if (cl > 1) cluster_barrier(); else __syncthreads();       // every head's scores are there; the key buffer is free
        if (t + 1 < n_t) load_keys(t + 1);
        cp_async_commit();
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
        const float* tk = tk_s + (size_t)warp * NH;
        if (cl == 1) {
            for (int g = 0; g < NH; ++g) {
                const float w = tk[g];
                const float* sg = s_s + (size_t)g * MT_ROWS * SP + r_lo * SP + c_lo;
#pragma unroll
                for (int nt = 0; nt < BN / 8; ++nt) {
                    const float2 u = *reinterpret_cast<const float2*>(sg + nt * 8);
                    const float2 v = *reinterpret_cast<const float2*>(sg + 8 * SP + nt * 8);
                    s[nt][0] = fmaf(w, u.x, s[nt][0]); s[nt][1] = fmaf(w, u.y, s[nt][1]);
                    s[nt][2] = fmaf(w, v.x, s[nt][2]); s[nt][3] = fmaf(w, v.y, s[nt][3]);
                }
            }
        } else {
            for (int g = 0; g < NH; ++g) {
                const float w = tk[g];
                const uint32_t sg = map_to_rank(s_base + (uint32_t)((((g % HPC) * MT_ROWS + r_lo) * SP + c_lo) * 4), (uint32_t)(g / HPC));
#pragma unroll
                for (int nt = 0; nt < BN / 8; ++nt) {
                    const float2 u = ld_cluster_f2(sg + nt * 32);
                    const float2 v = ld_cluster_f2(sg + (8 * SP + nt * 8) * 4);
                    s[nt][0] = fmaf(w, u.x, s[nt][0]); s[nt][1] = fmaf(w, u.y, s[nt][1]);
                    s[nt][2] = fmaf(w, v.x, s[nt][2]); s[nt][3] = fmaf(w, v.y, s[nt][3]);
                }
            }
        }
        // mask, online softmax (in powers of two)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + nt * 8 + c_lo + (e & 1);
                const bool seen = j <= p_row[e >> 1] && j >= lo_row[e >> 1];
                s[nt][e] = seen ? s[nt][e] * MT_LOG2E : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
            }
        float alpha[2], m_use[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
            const float m_new = fmaxf(m_run[hh], mx[hh]);
            m_use[hh] = m_new == -INFINITY ? 0.f : m_new;
            alpha[hh] = fast_exp2(m_run[hh] - m_use[hh]);
            m_run[hh] = m_new;
            l_run[hh] *= alpha[hh];
        }
        if (alpha[0] != 1.f || alpha[1] != 1.f) {
#pragma unroll
            for (int i = 0; i < 2 * NDV; ++i) {
                acc[i][0] *= alpha[0]; acc[i][1] *= alpha[0];
                acc[i][2] *= alpha[1]; acc[i][3] *= alpha[1];
            }
        }
        cp_async_wait<1>();                     // this tile's values (the next keys may still be on their way)
        if (cl > 1) cluster_barrier(); else __syncthreads();       // and nobody reads this tile's scores any more
#pragma unroll
        for (int kp = 0; kp < BN / 16; ++kp) {
            uint32_t pa[4];
            float pv[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    pv[nt][e] = fast_exp2(s[2 * kp + nt][e] - m_use[e >> 1]);
                    l_run[e >> 1] += pv[nt][e];
                }
            pa[0] = pack_bf16(pv[0][0], pv[0][1]);
            pa[1] = pack_bf16(pv[0][2], pv[0][3]);
            pa[2] = pack_bf16(pv[1][0], pv[1][1]);
            pa[3] = pack_bf16(pv[1][2], pv[1][3]);
#pragma unroll
            for (int nd = 0; nd < NDV; ++nd) {
                if (nd * 16 < DVP) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vb + (kp * 16 + (mi & 1) * 8 + lr) * VP + (nd * 2 + (mi >> 1)) * 16);
                    mma_bf16(acc[2 * nd], pa, b[0], b[1]);
                    mma_bf16(acc[2 * nd + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();                        // the value buffer is free
        if (t + 1 < n_t) load_values(t + 1);
        cp_async_commit();
    }
    cp_async_wait<0>();

#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
    }
    if (part >= 0) {
        // row 0 alone is a query: its unnormalised sums, running maximum and sum, for the merge
        if (r_lo == 0) {
            float* pa = a.part_acc + ((size_t)part * NH + h) * DV + c_lo;
#pragma unroll
            for (int i = 0; i < 2 * NDV; ++i)
                if (i * 8 + c_lo < DV) *reinterpret_cast<float2*>(pa + i * 8) = make_float2(acc[i][0], acc[i][1]);
            if (lane == 0) {
                a.part_ml[((size_t)part * NH + h) * 2] = m_run[0];
                a.part_ml[((size_t)part * NH + h) * 2 + 1] = l_run[0];
            }
        }
        if (cl > 1) cluster_barrier();
        return;
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = r_lo + hh * 8;
        if (r >= rows) continue;
        const float inv = l_run[hh] > 0.f ? 1.f / l_run[hh] : 0.f;
        bf16* o = a.out + (size_t)(tok0 + r) * a.out_stride + (size_t)h * DV + c_lo;
#pragma unroll
        for (int i = 0; i < 2 * NDV; ++i)
            if (i * 8 + c_lo < DV)
                *reinterpret_cast<__nv_bfloat162*>(o + i * 8) = __floats2bfloat162_rn(acc[i][2 * hh] * inv, acc[i][2 * hh + 1] * inv);
    }
    if (cl > 1) cluster_barrier();              // a CTA's scores may be read by the others until their last mix is done
}

// out[token][h] = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M) over the splits of a one-token request: a block a
// (request, head), a thread a value column
__global__ void attn_mixed_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                        const int* __restrict__ dec_tokens, bf16* __restrict__ out, int out_stride,
                                        int n_split, int NH, int DV) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x / NH, h = blockIdx.x % NH;
    float M = -INFINITY;
    for (int s = 0; s < n_split; ++s) M = fmaxf(M, part_ml[(((size_t)i * n_split + s) * NH + h) * 2]);
    for (int e = threadIdx.x; e < DV; e += blockDim.x) {
        float sum = 0.f, L = 0.f;
        if (M != -INFINITY)
            for (int s = 0; s < n_split; ++s) {
                const size_t at = ((size_t)i * n_split + s) * NH + h;
                const float m = part_ml[at * 2];
                if (m == -INFINITY) continue;
                const float w = fast_exp2(m - M);
                L = fmaf(part_ml[at * 2 + 1], w, L);
                sum = fmaf(part_acc[at * DV + e], w, sum);
            }
        out[(size_t)dec_tokens[i] * out_stride + (size_t)h * DV + e] = from_f32<bf16>(L > 0.f ? sum / L : 0.f);
    }
}

static int mixed_tc_cluster(int NH) {
    for (int cl = 1; cl <= 4; cl *= 2)
        if (NH % cl == 0 && NH / cl <= MT_MAX_WARPS) return cl;
    return 0;
}

static size_t mixed_tc_smem(const MixedArgs& a, int BN) {
    const int HPC = a.NH / a.cl, group = a.NH / a.NKV;
    const int n_kv = HPC >= group ? HPC / group : 1;
    const size_t QP = ((a.D + 15) & ~15) * 2 + 16, VP = ((a.DV + 15) & ~15) * 2 + 16;
    return (size_t)HPC * MT_ROWS * QP + (size_t)n_kv * BN * (QP + VP) + (size_t)HPC * MT_ROWS * (BN + 8) * 4 +
           (size_t)HPC * a.NH * 4 + (size_t)a.rel_rows * a.NH * 4 + (size_t)HPC * (BN + 16) * 4 + (size_t)2 * BN * 4;
}

template <int BN, int NDV>
static int launch_mixed_tc(const MixedArgs& a, size_t smem, cudaStream_t stream) {
    static AcvSmemConfig cfg;
    if (int rc = acv_ensure_smem(cfg, attn_mixed_tc_kernel<BN, NDV>, (int)smem)) return rc;
    const int units = a.n_tiles * MT_SUB + a.n_dec * a.n_split;
    acv_launch_cluster(PDL_ATTN, dim3(a.cl), attn_mixed_tc_kernel<BN, NDV>, dim3(units * a.cl), dim3(a.NH / a.cl * 32), smem,
                       stream, a);
    if (a.n_split > 1 && a.n_dec > 0)
        acv_launch(PDL_ATTN, attn_mixed_merge_kernel, dim3(a.n_dec * a.NH), dim3(a.DV < 32 ? 32 : (a.DV + 31) / 32 * 32), 0,
                   stream, (const float*)a.part_acc, (const float*)a.part_ml, a.dec_tokens, a.out, a.out_stride, a.n_split,
                   a.NH, a.DV);
    return acv_launch_status();
}

#define MT_SMEM_LIMIT (200 * 1024)

#include "attention_mixed_dec.cuh"

// 1 if one-token requests of these sizes run with a warp a key/value head (attention_mixed_dec.cuh)
ACV_API int acv_attention_mixed_dec_takes(int NH, int NKV, int D, int DV, int rel_rows) {
    if (NH <= 0 || NKV <= 0 || NH % NKV || D <= 0 || DV <= 0 || D % 8 || DV % 8 || DV > 128 || D > 512) return 0;
    MixedArgs a = {};
    a.NH = NH; a.NKV = NKV; a.D = D; a.DV = DV; a.rel_rows = rel_rows;
    return mixed_dec_tile(a) > 0;
}

// 1 if acv_attention_mixed_tc runs these sizes, 0 if they belong to acv_attention_mixed
ACV_API int acv_attention_mixed_tc_takes(int NH, int NKV, int D, int DV, int rel_rows) {
    if (NH <= 0 || NKV <= 0 || NH % NKV || D <= 0 || DV <= 0 || D % 8 || DV % 8 || DV > 128 || D > 512) return 0;
    MixedArgs a = {};
    a.NH = NH; a.NKV = NKV; a.D = D; a.DV = DV; a.rel_rows = rel_rows;
    a.cl = mixed_tc_cluster(NH);
    if (!a.cl) return 0;
    const int HPC = NH / a.cl, group = NH / NKV;
    if (HPC % group && group % HPC) return 0;       // a CTA's heads read whole key/value heads, every CTA as many
    return mixed_tc_smem(a, 16) <= MT_SMEM_LIMIT;
}

// Portions (tiles of 128 query tokens: tile_seq, tile_q0) and one-token requests (dec_tokens, dec_seqs) of a step in
// one launch.  q rows of NH*D bfloat16 at q_stride, out rows of NH*DV; pages [NP][NKV][page][D] and [..][DV]; temp
// float [NH]; rel float [rel_rows][NH]; bucket_of int [n_dist]; talk float [NH][NH]; each of the four may be null.
// n_split > 1: that many CTAs (or clusters) share the keys of every one-token request and leave partial results in
// part_acc (float [n_dec][n_split][NH][DV]) and part_ml ([..][NH][2]), which a second launch merges into out.
ACV_API int acv_attention_mixed_tc(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                   const void* v_pages, const int* tile_seq, const int* tile_q0, int n_tiles,
                                   const int* dec_tokens, const int* dec_seqs, int n_dec, const int* cu_q,
                                   const int* kv_len, const int* block_table, int bt_stride, const int* bt_rows, int NH,
                                   int NKV, int D, int DV, int page_size, int num_pages, float scale, int window,
                                   const float* temp, float cap, const float* rel, int rel_rows, const int* bucket_of,
                                   int n_dist, int last_row, const float* talk, int n_split, float* part_acc,
                                   float* part_ml, cudaStream_t stream) {
    if (n_tiles <= 0 && n_dec <= 0) return 0;
    if (n_split < 1 || (n_split > 1 && (!part_acc || !part_ml))) return ACV_ERR_SIZE;
    if (!acv_attention_mixed_tc_takes(NH, NKV, D, DV, rel ? rel_rows : 0)) return ACV_ERR_SIZE;
    if (rel && (!bucket_of || n_dist < 0 || last_row < 0 || last_row >= rel_rows)) return ACV_ERR_SIZE;
    if (((uintptr_t)q & 15) || ((size_t)q_stride * 2) % 16 || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) ||
        ((uintptr_t)out & 3) || (out_stride & 1))
        return ACV_ERR_ALIGN;
    MixedArgs a = {(const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_pages, (const bf16*)v_pages,
                   tile_seq, tile_q0, n_tiles < 0 ? 0 : n_tiles, dec_tokens, dec_seqs, n_dec < 0 ? 0 : n_dec, cu_q, kv_len,
                   block_table, bt_stride, bt_rows, NH, NKV, D, DV, page_size, num_pages, scale, window,
                   temp, cap, rel, bucket_of, n_dist, last_row, rel ? rel_rows : 0, talk, mixed_tc_cluster(NH), n_split,
                   part_acc, part_ml};
    const int ndv = (DV + 15) / 16;
    // one-token requests: a warp a key/value head where the sizes allow, in a launch of their own
    const int dec_bn = a.n_dec > 0 ? mixed_dec_tile(a) : 0;
    if (dec_bn) {
        const size_t dsmem = mixed_dec_smem(a, dec_bn);
        int rc = ACV_ERR_SIZE;
#define MD_CASE(B, N) if (rc == ACV_ERR_SIZE && dec_bn == B && ndv <= N) rc = launch_mixed_dec<B, N>(a, dsmem, stream);
        MD_CASE(64, 2) MD_CASE(64, 4)
        MD_CASE(32, 2) MD_CASE(32, 4) MD_CASE(32, 8)
        MD_CASE(16, 2) MD_CASE(16, 4) MD_CASE(16, 8)
#undef MD_CASE
        if (rc) return rc;
        if (a.n_split > 1) {
            acv_launch(PDL_ATTN, attn_mixed_merge_kernel, dim3(a.n_dec * NH), dim3(DV < 32 ? 32 : (DV + 31) / 32 * 32), 0, stream,
                       (const float*)part_acc, (const float*)part_ml, dec_tokens, (bf16*)out, out_stride, a.n_split, NH, DV);
            if (int e = acv_launch_status()) return e;
        }
        if (a.n_tiles == 0) return 0;
        a.n_dec = 0;
        a.n_split = 1;
    }
    // the widest key tile that fits; 64 keys only with few accumulators (registers)
    int BN = 16;
    if (mixed_tc_smem(a, 32) <= MT_SMEM_LIMIT) BN = 32;
    if (ndv <= 4 && mixed_tc_smem(a, 64) <= MT_SMEM_LIMIT) BN = 64;
    const size_t smem = mixed_tc_smem(a, BN);
#define MT_CASE(B, N) if (BN == B && ndv <= N) return launch_mixed_tc<B, N>(a, smem, stream);
    MT_CASE(64, 2) MT_CASE(64, 4)
    MT_CASE(32, 2) MT_CASE(32, 4) MT_CASE(32, 8)
    MT_CASE(16, 2) MT_CASE(16, 4) MT_CASE(16, 8)
#undef MT_CASE
    return ACV_ERR_SIZE;
}
