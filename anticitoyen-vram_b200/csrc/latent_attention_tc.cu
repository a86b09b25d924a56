// Attention over kept latent rows (see latent_attention.cu) on the tensor cores, bfloat16 pages and queries.
//
// Every query head reads the same rows [c | r] of ROW elements, and the values are the first KR elements of the same
// rows, so a key tile is fetched once and serves as keys and as values, for all heads.  The unit of work is a few
// query tokens of one request with a block of heads: rows (token t, head h) -> R = t * HPC + h, in groups of 16 (the
// M of mma.sync m16n8k16).  A row group is served by S warps: for a tile of BN keys each computes the scores of BN/S
// keys (over all ROW elements), the S warps exchange their row maxima through shared memory and leave their softmax
// weights there as bfloat16; then each multiplies all BN weights with its own slice of NDV*16 value columns.  So no
// score is computed twice, and the accumulators of a row (KR floats) are spread over S warps.
//
//   barrier A   tile t has arrived (cp.async), and everyone is done with tile t-1: fetch tile t+1 into the other buffer
//   scores      q . k over ROW, * scale * log2(e), masked (causal, window)
//   barrier B   row maxima of the S warps are there (S > 1)
//   weights     p = 2^(s - m); running maximum and sum; accumulators rescaled; p into shared memory
//   barrier C   all weights of the tile are there
//   values      acc += p . c[:, slice]
//
// One token with 16 heads is one row group (the decode step's shape); a portion takes as many tokens as 16 warps and
// the shared memory hold.  Rows are padded by 16 bytes instead of swizzled, so ROW and KR need only be multiples of 8.
#include "mma_tiles.cuh"

#define LT_LOG2E 1.4426950408889634f
#define LT_TILE_TOKENS 128      // query tokens in a tile of the step's work list

struct LatentArgs {
    const bf16* q; int q_stride; bf16* out; int out_stride;
    const bf16* pages;
    const int* tile_seq; const int* tile_q0; int n_tiles;
    const int* dec_tokens; const int* dec_seqs; int n_dec;
    const int* cu_q; const int* kv_len;
    const int* block_table; int bt_stride; const int* bt_rows;
    int NH, ROW, KR, page_size, num_pages;
    float scale; int window;
    int TOK;                // query tokens of a unit (divides 16)
    int HPC, HB;            // heads of a CTA, head blocks (HPC * HB == NH)
    int RG;                 // row groups of a CTA = ceil(TOK * HPC / 16)
    int n_split;            // CTAs that share the rows of a one-token request (1: none)
    float* part_acc;        // n_split > 1: [n_dec][n_split][NH][KR] unnormalised sums
    float* part_ml;         //              [n_dec][n_split][NH][2] running maximum (in powers of two) and sum
};

template <int BN, int S, int NDV>
__global__ void __launch_bounds__(512)
attn_latent_tc_kernel(const LatentArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int KPW = BN / S;             // keys whose scores a warp computes
    constexpr int NT = KPW / 8;
    static_assert(KPW >= 8 && KPW % 8 == 0, "a warp scores whole n8 tiles");
    const int ROW = a.ROW, KR = a.KR, HPC = a.HPC, RG = a.RG;
    const int DP = (ROW + 15) & ~15, KRP = (KR + 15) & ~15;
    const int QP = DP * 2 + 16;             // bytes of a padded row
    constexpr int PP = (BN + 8) * 2;        // bytes of a row of weights

    unsigned char* q_s = smem;                                      // [RG * 16][QP]
    unsigned char* k_s = q_s + (size_t)RG * 16 * QP;                // [2][BN][QP]
    unsigned char* p_s = k_s + (size_t)2 * BN * QP;                 // [RG][16][PP]
    float* mx_s = reinterpret_cast<float*>(p_s + (size_t)RG * 16 * PP);     // [RG][S][16]
    float* l_s = mx_s + (size_t)RG * S * 16;                        // [RG][S][16]

    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nthr = blockDim.x;
    const int rg = warp / S, sl = warp % S;
    const int hb = blockIdx.x % a.HB, unit = blockIdx.x / a.HB;
    const int per_tile = LT_TILE_TOKENS / a.TOK;
    int seq, tok0, ntok, pos0;
    int split = 0, part = -1;                    // part >= 0: this CTA leaves a partial result at that index
    if (unit < a.n_tiles * per_tile) {
        const int tile = unit / per_tile;
        seq = a.tile_seq[tile];
        const int q0 = a.tile_q0[tile] + (unit % per_tile) * a.TOK;
        const int q_len = a.cu_q[seq + 1] - a.cu_q[seq];
        if (q0 >= q_len) return;
        tok0 = a.cu_q[seq] + q0;
        ntok = min(a.TOK, q_len - q0);
        pos0 = a.kv_len[seq] - q_len + q0;
    } else {
        const int u = unit - a.n_tiles * per_tile;
        const int i = u / a.n_split;
        split = u % a.n_split;
        if (a.n_split > 1) part = u;
        seq = a.dec_seqs[i];
        tok0 = a.dec_tokens[i];
        ntok = 1;
        pos0 = a.kv_len[seq] - 1;
    }
    const int h_first = hb * HPC;
    const int n_rows = ntok * HPC;
    if (pos0 < 0) {                              // a padded slot of a captured batch: nothing is kept for it
        if (part >= 0) {
            for (int e = tid; e < HPC; e += nthr) {
                a.part_ml[((size_t)part * a.NH + h_first + e) * 2] = -INFINITY;
                a.part_ml[((size_t)part * a.NH + h_first + e) * 2 + 1] = 0.f;
            }
            return;
        }
        for (int e = tid; e < HPC * KR; e += nthr)
            a.out[(size_t)tok0 * a.out_stride + (size_t)h_first * KR + e] = from_f32<bf16>(0.f);
        return;
    }
    const int* bt = a.block_table + (size_t)(a.bt_rows ? a.bt_rows[seq] : seq) * a.bt_stride;
    const int window = a.window;
    const int hi = pos0 + ntok - 1;
    const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int j_first = lo & ~(BN - 1);
    const int n_all = (hi - j_first) / BN + 1;
    // the tiles of this CTA: all of them, or its share of a one-token request's
    const int per_split = (n_all + a.n_split - 1) / a.n_split;
    const int t_first = part >= 0 ? split * per_split : 0;
    const int n_t = part >= 0 ? min(n_all, t_first + per_split) : n_all;
    const int CH = DP / 8;

    for (int id = tid; id < RG * 16 * CH; id += nthr) {
        const int c = id % CH, R = id / CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (R < n_rows && c * 8 < ROW)
            v = *reinterpret_cast<const uint4*>(a.q + (size_t)(tok0 + R / HPC) * a.q_stride +
                                                (size_t)(h_first + R % HPC) * ROW + c * 8);
        *reinterpret_cast<uint4*>(q_s + (size_t)R * QP + c * 16) = v;
    }
    auto load_keys = [&](int t) {
        const int j0 = j_first + t * BN;
        unsigned char* dst = k_s + (size_t)(t & 1) * BN * QP;
        for (int id = tid; id < BN * CH; id += nthr) {
            const int c = id % CH, r = id / CH;
            const int j = j0 + r;
            bool ok = j <= hi && j >= lo && c * 8 < ROW;
            size_t off = 0;
            if (ok) {
                const int pg = bt[j / a.page_size];
                ok = pg >= 0 && pg < a.num_pages;
                off = ((size_t)pg * a.page_size + (j % a.page_size)) * ROW + c * 8;
            }
            cp_async16(smem_u32(dst + (size_t)r * QP + c * 16), ok ? (const void*)(a.pages + off) : (const void*)a.pages, ok);
        }
    };
    load_keys(t_first);
    cp_async_commit();

    const int mi = lane >> 3, lr = lane & 7;
    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;
    // positions of this thread's two rows (rows past the unit's last one see nothing that is stored)
    const int p_row[2] = {pos0 + (rg * 16 + r_lo) / HPC, pos0 + (rg * 16 + r_lo + 8) / HPC};
    const int lo_row[2] = {window > 0 ? max(0, p_row[0] - window + 1) : 0, window > 0 ? max(0, p_row[1] - window + 1) : 0};
    const float sc_log2 = a.scale * LT_LOG2E;
    const uint32_t qb = smem_u32(q_s + (size_t)rg * 16 * QP);
    const uint32_t pb = smem_u32(p_s + (size_t)rg * 16 * PP);
    unsigned char* p_own = p_s + (size_t)rg * 16 * PP;
    float* mx_own = mx_s + (size_t)rg * S * 16;

    float acc[2 * NDV][4];
#pragma unroll
    for (int i = 0; i < 2 * NDV; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    for (int t = t_first; t < n_t; ++t) {
        const int j0 = j_first + t * BN;
        cp_async_wait<0>();
        __syncthreads();                                            // A
        if (t + 1 < n_t) load_keys(t + 1);
        cp_async_commit();
        const uint32_t kb = smem_u32(k_s + (size_t)(t & 1) * BN * QP);
        const int key0 = sl * KPW;
        float s[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
        for (int kd = 0; kd < DP / 16; ++kd) {
            uint32_t qf[4];
            ldmatrix_x4(qf, qb + ((mi & 1) * 8 + lr) * QP + (kd * 2 + (mi >> 1)) * 16);
            if constexpr (NT == 1) {
                uint32_t b[4];              // one n8 tile: both halves of the load read the same eight keys
                ldmatrix_x4(b, kb + (key0 + lr) * QP + (kd * 2 + (mi & 1)) * 16);
                mma_bf16(s[0], qf, b[0], b[1]);
            } else {
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, kb + (key0 + np * 16 + (mi >> 1) * 8 + lr) * QP + (kd * 2 + (mi & 1)) * 16);
                    mma_bf16(s[2 * np], qf, b[0], b[1]);
                    mma_bf16(s[2 * np + 1], qf, b[2], b[3]);
                }
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + key0 + nt * 8 + c_lo + (e & 1);
                const bool seen = j <= p_row[e >> 1] && j >= lo_row[e >> 1];
                s[nt][e] = seen ? s[nt][e] * sc_log2 : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
            }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
            mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
        }
        if constexpr (S > 1) {
            if ((lane & 3) == 0) {
                mx_own[sl * 16 + r_lo] = mx[0];
                mx_own[sl * 16 + r_lo + 8] = mx[1];
            }
            __syncthreads();                                        // B
#pragma unroll
            for (int w = 0; w < S; ++w) {
                mx[0] = fmaxf(mx[0], mx_own[w * 16 + r_lo]);
                mx[1] = fmaxf(mx[1], mx_own[w * 16 + r_lo + 8]);
            }
        }
        float alpha[2], m_use[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
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
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float pv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                pv[e] = fast_exp2(s[nt][e] - m_use[e >> 1]);
                l_run[e >> 1] += pv[e];
            }
            const int col = key0 + nt * 8 + c_lo;
            *reinterpret_cast<uint32_t*>(p_own + (size_t)r_lo * PP + col * 2) = pack_bf16(pv[0], pv[1]);
            *reinterpret_cast<uint32_t*>(p_own + (size_t)(r_lo + 8) * PP + col * 2) = pack_bf16(pv[2], pv[3]);
        }
        if constexpr (S > 1) __syncthreads(); else __syncwarp();    // C
#pragma unroll
        for (int kp = 0; kp < BN / 16; ++kp) {
            uint32_t pa[4];
            ldmatrix_x4(pa, pb + ((mi & 1) * 8 + lr) * PP + (kp * 2 + (mi >> 1)) * 16);
#pragma unroll
            for (int nd = 0; nd < NDV; ++nd) {
                const int c16 = sl * NDV + nd;          // which 16 value columns
                if (c16 * 16 < KRP) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, kb + (kp * 16 + (mi & 1) * 8 + lr) * QP + (c16 * 2 + (mi >> 1)) * 16);
                    mma_bf16(acc[2 * nd], pa, b[0], b[1]);
                    mma_bf16(acc[2 * nd + 1], pa, b[2], b[3]);
                }
            }
        }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
    }
    if constexpr (S > 1) {
        float* l_own = l_s + (size_t)rg * S * 16;
        if ((lane & 3) == 0) {
            l_own[sl * 16 + r_lo] = l_run[0];
            l_own[sl * 16 + r_lo + 8] = l_run[1];
        }
        __syncthreads();
        l_run[0] = l_run[1] = 0.f;
#pragma unroll
        for (int w = 0; w < S; ++w) {
            l_run[0] += l_own[w * 16 + r_lo];
            l_run[1] += l_own[w * 16 + r_lo + 8];
        }
    }
    if (part >= 0) {
        // one token: row R is head h_first + R; unnormalised sums, running maximum and sum, for the merge
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int R = rg * 16 + r_lo + hh * 8;
            if (R >= n_rows) continue;
            const size_t at = (size_t)part * a.NH + h_first + R;
            float* pa = a.part_acc + at * KR + sl * NDV * 16 + c_lo;
#pragma unroll
            for (int i = 0; i < 2 * NDV; ++i)
                if (sl * NDV * 16 + i * 8 + c_lo < KR)
                    *reinterpret_cast<float2*>(pa + i * 8) = make_float2(acc[i][2 * hh], acc[i][2 * hh + 1]);
            if (sl == 0 && (lane & 3) == 0) {
                a.part_ml[at * 2] = m_run[hh];
                a.part_ml[at * 2 + 1] = l_run[hh];
            }
        }
        return;
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int R = rg * 16 + r_lo + hh * 8;
        if (R >= n_rows) continue;
        const float inv = l_run[hh] > 0.f ? 1.f / l_run[hh] : 0.f;
        bf16* o = a.out + (size_t)(tok0 + R / HPC) * a.out_stride + (size_t)(h_first + R % HPC) * KR + sl * NDV * 16 + c_lo;
#pragma unroll
        for (int i = 0; i < 2 * NDV; ++i)
            if (sl * NDV * 16 + i * 8 + c_lo < KR)
                *reinterpret_cast<__nv_bfloat162*>(o + i * 8) = __floats2bfloat162_rn(acc[i][2 * hh] * inv, acc[i][2 * hh + 1] * inv);
    }
}

// out[token][h] = sum_s acc_s 2^(m_s - M) / sum_s l_s 2^(m_s - M) over the CTAs that shared a one-token request's rows:
// a block a (request, head), a thread a few columns
__global__ void attn_latent_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                         const int* __restrict__ dec_tokens, bf16* __restrict__ out, int out_stride,
                                         int n_split, int NH, int KR) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x / NH, h = blockIdx.x % NH;
    float M = -INFINITY;
    for (int s = 0; s < n_split; ++s) M = fmaxf(M, part_ml[(((size_t)i * n_split + s) * NH + h) * 2]);
    for (int e = threadIdx.x; e < KR; e += blockDim.x) {
        float sum = 0.f, L = 0.f;
        if (M != -INFINITY)
            for (int s = 0; s < n_split; ++s) {
                const size_t at = ((size_t)i * n_split + s) * NH + h;
                const float m = part_ml[at * 2];
                if (m == -INFINITY) continue;
                const float w = fast_exp2(m - M);
                L = fmaf(part_ml[at * 2 + 1], w, L);
                sum = fmaf(part_acc[at * KR + e], w, sum);
            }
        out[(size_t)dec_tokens[i] * out_stride + (size_t)h * KR + e] = from_f32<bf16>(L > 0.f ? sum / L : 0.f);
    }
}

struct LatentShape {
    int S, NDV, TOK, HPC, HB, RG, BN;
    size_t smem;
};

#define LT_SMEM_LIMIT (200 * 1024)

static size_t latent_tc_smem(int ROW, int RG, int S, int BN) {
    const size_t QP = ((ROW + 15) & ~15) * 2 + 16, PP = (BN + 8) * 2;
    return (size_t)RG * 16 * QP + (size_t)2 * BN * QP + (size_t)RG * 16 * PP + (size_t)2 * RG * S * 16 * 4;
}

// how a launch is cut for these sizes (portions: as many tokens a unit as fit; one-token requests alone: one); 0 if not at all
static int latent_tc_shape(int NH, int ROW, int KR, bool portions, LatentShape& sh) {
    if (NH <= 0 || ROW <= 0 || KR <= 0 || KR > ROW || ROW % 8 || KR % 8 || KR > 512) return 0;
    sh.NDV = KR <= 64 ? 4 : 8;
    sh.S = KR <= 128 ? 1 : (KR <= 256 ? 2 : 4);
    const int max_rg = 16 / sh.S;
    sh.HPC = 0;
    for (int hpc = NH < 16 * max_rg ? NH : 16 * max_rg; hpc >= 1; --hpc)
        if (NH % hpc == 0) { sh.HPC = hpc; break; }
    sh.HB = NH / sh.HPC;
    for (int tok = portions ? 16 : 1; tok >= 1; tok /= 2) {
        const int rg = (tok * sh.HPC + 15) / 16;
        if (rg > max_rg) continue;
        for (int bn = 64; bn >= 32; bn /= 2) {
            if (bn / sh.S < 8) continue;
            const size_t smem = latent_tc_smem(ROW, rg, sh.S, bn);
            if (smem <= LT_SMEM_LIMIT) {
                sh.TOK = tok; sh.RG = rg; sh.BN = bn; sh.smem = smem;
                return 1;
            }
        }
    }
    return 0;
}

template <int BN, int S, int NDV>
static int launch_latent_tc(const LatentArgs& a, const LatentShape& sh, cudaStream_t stream) {
    static AcvSmemConfig cfg;
    if (int rc = acv_ensure_smem(cfg, attn_latent_tc_kernel<BN, S, NDV>, (int)sh.smem)) return rc;
    const int units = a.n_tiles * (LT_TILE_TOKENS / a.TOK) + a.n_dec * a.n_split;
    acv_launch(PDL_ATTN, attn_latent_tc_kernel<BN, S, NDV>, dim3(units * a.HB), dim3(a.RG * S * 32), sh.smem, stream, a);
    if (a.n_split > 1 && a.n_dec > 0)
        acv_launch(PDL_ATTN, attn_latent_merge_kernel, dim3(a.n_dec * a.NH), dim3(128), 0, stream, (const float*)a.part_acc,
                   (const float*)a.part_ml, a.dec_tokens, a.out, a.out_stride, a.n_split, a.NH, a.KR);
    return acv_launch_status();
}

// 1 if acv_attention_latent_tc runs these sizes (a step with portions needs the larger shape: asked for both)
ACV_API int acv_attention_latent_tc_takes(int NH, int ROW, int KR) {
    LatentShape sh;
    return latent_tc_shape(NH, ROW, KR, true, sh) && latent_tc_shape(NH, ROW, KR, false, sh);
}

// Portions (tiles of 128 query tokens: tile_seq, tile_q0) and one-token requests (dec_tokens, dec_seqs) of a step in one
// launch.  q rows of NH*ROW bfloat16 at q_stride (the queries that meet the kept rows), out rows of NH*KR (the weighted
// sums of latents); pages [NP][1][page][ROW].  n_split > 1: that many CTAs share the rows of every one-token request and
// leave partial results in part_acc (float [n_dec][n_split][NH][KR]) and part_ml ([..][NH][2]); a second launch merges.
ACV_API int acv_attention_latent_tc(const void* q, int q_stride, void* out, int out_stride, const void* pages,
                                    const int* tile_seq, const int* tile_q0, int n_tiles, const int* dec_tokens,
                                    const int* dec_seqs, int n_dec, const int* cu_q, const int* kv_len,
                                    const int* block_table, int bt_stride, const int* bt_rows, int NH, int ROW, int KR,
                                    int page_size, int num_pages, float scale, int window, int n_split, float* part_acc,
                                    float* part_ml, cudaStream_t stream) {
    if (n_split < 1 || (n_split > 1 && (!part_acc || !part_ml))) return ACV_ERR_SIZE;
    if (n_tiles < 0) n_tiles = 0;
    if (n_dec < 0) n_dec = 0;
    if (n_tiles == 0 && n_dec == 0) return 0;
    LatentShape sh;
    if (!latent_tc_shape(NH, ROW, KR, n_tiles > 0, sh)) return ACV_ERR_SIZE;
    if (((uintptr_t)q & 15) || ((size_t)q_stride * 2) % 16 || ((uintptr_t)pages & 15) || ((uintptr_t)out & 3) || (out_stride & 1))
        return ACV_ERR_ALIGN;
    LatentArgs a = {(const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)pages, tile_seq, tile_q0, n_tiles,
                    dec_tokens, dec_seqs, n_dec, cu_q, kv_len, block_table, bt_stride, bt_rows, NH, ROW, KR, page_size,
                    num_pages, scale, window, sh.TOK, sh.HPC, sh.HB, sh.RG, n_split, part_acc, part_ml};
#define LT_CASE(B, SS, N) if (sh.BN == B && sh.S == SS && sh.NDV == N) return launch_latent_tc<B, SS, N>(a, sh, stream);
    LT_CASE(64, 1, 4) LT_CASE(64, 1, 8) LT_CASE(64, 2, 8) LT_CASE(64, 4, 8)
    LT_CASE(32, 1, 4) LT_CASE(32, 1, 8) LT_CASE(32, 2, 8) LT_CASE(32, 4, 8)
#undef LT_CASE
    return ACV_ERR_SIZE;
}
