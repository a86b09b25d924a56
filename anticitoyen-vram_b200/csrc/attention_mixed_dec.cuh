// Head-mixing attention for requests that bring ONE token (included by attention_mixed_tc.cu).
//
// With one query token a tile of 16 tokens has one useful row.  Here the 16 rows of a warp's tile are the query heads
// that share one key/value head (group = NH / NKV <= 16 of them), so a warp is a key/value head: its scores, softmax
// and value product serve `group` heads at once, a CTA of NKV warps holds all heads of the request (no cluster), and
// the mix reads one row of scores per head.  Where group <= 8 the upper half of the tile is skipped.  The keys of a
// request may be shared among several CTAs (a.n_split), as in the tile kernel.  A CTA has at least eight warps: those
// beyond NKV only copy.  The place of a tile's keys in their pages is looked up once per tile (by BN threads, a tile
// ahead) instead of once per copied 16-byte chunk.  Keys and values have two buffers each: the copies of tile t+1 start
// when tile t's have arrived and run during all of tile t's work, behind two block barriers a tile.
template <int BN, int NDV>
__global__ void __launch_bounds__(MT_MAX_WARPS * 32)
attn_mixed_dec_kernel(const MixedArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int NH = a.NH, NKV = a.NKV, D = a.D, DV = a.DV;
    const int group = NH / NKV;
    const int DP = (D + 15) & ~15, DVP = (DV + 15) & ~15;
    const int QP = DP * 2 + 16, VP = DVP * 2 + 16;
    constexpr int SP = BN + 8;

    unsigned char* q_s = smem;                                              // [NKV][16][QP]: row r of warp w is head w*group + r
    unsigned char* k_s = q_s + (size_t)NKV * MT_ROWS * QP;                  // [2][NKV][BN][QP]
    unsigned char* v_s = k_s + (size_t)2 * NKV * BN * QP;                   // [2][NKV][BN][VP]
    float* s_s = reinterpret_cast<float*>(v_s + (size_t)2 * NKV * BN * VP); // [NH][SP]: one row of scores a head
    float* tk_s = s_s + (size_t)NH * SP;                                    // [NH][NH] transposed: tk_s[g][h] = talk[h][g]
    float* rel_s = tk_s + (size_t)NH * NH;                                  // [rel_rows][NH]
    float* bias_s = rel_s + (size_t)a.rel_rows * NH;                        // [NH][BN]: this tile's bias of every key
    int* keyrow_s = reinterpret_cast<int*>(bias_s + (size_t)NH * BN);       // [2][BN]: a key's row in kv-head 0 of its page, -1: none

    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nthr = blockDim.x;
    const int i = blockIdx.x / a.n_split, split = blockIdx.x % a.n_split;
    const int part = a.n_split > 1 ? (int)blockIdx.x : -1;
    const int seq = a.dec_seqs[i], tok0 = a.dec_tokens[i];
    const int pos0 = a.kv_len[seq] - 1;
    if (pos0 < 0) {                              // a padded slot of a captured batch: nothing is kept for it
        if (part >= 0) {
            for (int h = tid; h < NH; h += nthr) {
                a.part_ml[((size_t)part * NH + h) * 2] = -INFINITY;
                a.part_ml[((size_t)part * NH + h) * 2 + 1] = 0.f;
            }
        } else {
            for (int e = tid; e < NH * DV; e += nthr) a.out[(size_t)tok0 * a.out_stride + e] = from_f32<bf16>(0.f);
        }
        return;
    }
    const int* bt = a.block_table + (size_t)(a.bt_rows ? a.bt_rows[seq] : seq) * a.bt_stride;
    const int window = a.window;
    const int hi = pos0;
    const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int j_first = lo & ~(BN - 1);
    const int n_all = (hi - j_first) / BN + 1;
    const int per_split = (n_all + a.n_split - 1) / a.n_split;
    const int t_first = part >= 0 ? split * per_split : 0;
    const int n_t = part >= 0 ? min(n_all, t_first + per_split) : n_all;
    const int CH = DP / 8, CHV = DVP / 8;

    for (int id = tid; id < NKV * MT_ROWS * CH; id += nthr) {
        const int rr = id / CH, c = id - rr * CH, r = rr & (MT_ROWS - 1), w = rr / MT_ROWS;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < group && c * 8 < D)
            v = *reinterpret_cast<const uint4*>(a.q + (size_t)tok0 * a.q_stride + (size_t)(w * group + r) * D + c * 8);
        *reinterpret_cast<uint4*>(q_s + (size_t)rr * QP + c * 16) = v;
    }
    for (int id = tid; id < NH * NH; id += nthr) {
        const int g = id / NH, h = id - g * NH;
        tk_s[id] = a.talk ? a.talk[(size_t)h * NH + g] : (g == h ? 1.f : 0.f);
    }
    if (a.rel)
        for (int id = tid; id < a.rel_rows * NH; id += nthr) rel_s[id] = a.rel[id];

    const int page_shift = (a.page_size & (a.page_size - 1)) == 0 ? __ffs(a.page_size) - 1 : -1;
    auto find_rows = [&](int t) {
        if (tid < BN) {
            const int j = j_first + t * BN + tid;
            int row = -1;
            if (j <= hi && j >= lo) {
                const int pi = page_shift >= 0 ? j >> page_shift : j / a.page_size;
                const int pg = bt[pi];
                if (pg >= 0 && pg < a.num_pages) row = pg * NKV * a.page_size + (j - pi * a.page_size);
            }
            keyrow_s[(t & 1) * BN + tid] = row;
        }
    };
    auto load_keys = [&](int t) {
        const int* rows = keyrow_s + (t & 1) * BN;
        unsigned char* dst = k_s + (size_t)(t & 1) * NKV * BN * QP;
        for (int id = tid; id < NKV * BN * CH; id += nthr) {
            const int rr = id / CH, c = id - rr * CH, r = rr & (BN - 1), kvh = rr / BN;
            const int row = rows[r];
            const bool ok = row >= 0 && c * 8 < D;
            const size_t off = ok ? ((size_t)row + (size_t)kvh * a.page_size) * D + c * 8 : 0;
            cp_async16(smem_u32(dst + (size_t)rr * QP + c * 16), a.k_pages + off, ok);
        }
    };
    auto load_values = [&](int t) {
        const int* rows = keyrow_s + (t & 1) * BN;
        unsigned char* dst = v_s + (size_t)(t & 1) * NKV * BN * VP;
        for (int id = tid; id < NKV * BN * CHV; id += nthr) {
            const int rr = id / CHV, c = id - rr * CHV, r = rr & (BN - 1), kvh = rr / BN;
            const int row = rows[r];
            const bool ok = row >= 0 && c * 8 < DV;
            const size_t off = ok ? ((size_t)row + (size_t)kvh * a.page_size) * DV + c * 8 : 0;
            cp_async16(smem_u32(dst + (size_t)rr * VP + c * 16), a.v_pages + off, ok);
        }
    };
    find_rows(t_first);
    __syncthreads();
    load_keys(t_first);
    load_values(t_first);
    cp_async_commit();

    const int mi = lane >> 3, lr = lane & 7;
    const int r_lo = lane >> 2, c_lo = (lane & 3) * 2;
    const bool worker = warp < NKV;             // the other warps only copy
    const int wk = worker ? warp : 0;
    const bool top = group > 8;                 // rows 8..15 of the tile hold heads
    const bool row_on[2] = {worker && r_lo < group, worker && r_lo + 8 < group};
    // this thread's two heads (a row without a head computes on head 0's numbers and is never stored)
    const int h_row[2] = {row_on[0] ? wk * group + r_lo : 0, row_on[1] ? wk * group + r_lo + 8 : 0};
    const float qk_scale[2] = {a.scale * (a.temp ? a.temp[h_row[0]] : 1.f), a.scale * (a.temp ? a.temp[h_row[1]] : 1.f)};
    const float cap = a.cap, inv_cap = a.cap > 0.f ? 1.f / a.cap : 0.f;
    const uint32_t qb = smem_u32(q_s + (size_t)wk * MT_ROWS * QP);

    float acc[2 * NDV][4];
#pragma unroll
    for (int n = 0; n < 2 * NDV; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    if (a.rel) __syncthreads();                 // the bias table is in shared memory
    for (int t = t_first; t < n_t; ++t) {
        const int j0 = j_first + t * BN;
        if (a.rel) {
            for (int id = tid; id < NH * BN; id += nthr) {
                const int h = id / BN, dist = pos0 - (j0 + (id & (BN - 1)));
                bias_s[id] = dist >= 0 ? rel_s[(dist < a.n_dist ? a.bucket_of[dist] : a.last_row) * NH + h] : 0.f;
            }
        }
        if (t + 1 < n_t) find_rows(t + 1);
        cp_async_wait<0>();                     // this tile's keys and values
        __syncthreads();                        // ... and everyone is done with the tile before: its buffers are free
        if (t + 1 < n_t) {
            load_keys(t + 1);
            load_values(t + 1);
        }
        cp_async_commit();
        const uint32_t kb = smem_u32(k_s + ((size_t)(t & 1) * NKV + wk) * BN * QP);
        const uint32_t vb = smem_u32(v_s + ((size_t)(t & 1) * NKV + wk) * BN * VP);
        float s[BN / 8][4];
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
        for (int kd = 0; worker && kd < DP / 16; ++kd) {
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
        // each head's steps on its own scores, then one row a head into shared memory for the mix
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            if (hh == 1 && !top) break;
            if (!row_on[hh]) continue;
#pragma unroll
            for (int nt = 0; nt < BN / 8; ++nt) {
                float x[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    x[e] = s[nt][2 * hh + e] * qk_scale[hh];
                    if (cap > 0.f) x[e] = cap * fast_tanh(x[e] * inv_cap);
                    if (a.rel) x[e] += bias_s[h_row[hh] * BN + nt * 8 + c_lo + e];
                }
                *reinterpret_cast<float2*>(s_s + (size_t)h_row[hh] * SP + nt * 8 + c_lo) = make_float2(x[0], x[1]);
            }
        }
        __syncthreads();                        // every head's scores are there
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
        for (int g = 0; worker && g < NH; ++g) {
            const float w0 = tk_s[g * NH + h_row[0]];
            const float* sg = s_s + (size_t)g * SP + c_lo;
            if (top) {
                const float w1 = tk_s[g * NH + h_row[1]];
#pragma unroll
                for (int nt = 0; nt < BN / 8; ++nt) {
                    const float2 u = *reinterpret_cast<const float2*>(sg + nt * 8);
                    s[nt][0] = fmaf(w0, u.x, s[nt][0]); s[nt][1] = fmaf(w0, u.y, s[nt][1]);
                    s[nt][2] = fmaf(w1, u.x, s[nt][2]); s[nt][3] = fmaf(w1, u.y, s[nt][3]);
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < BN / 8; ++nt) {
                    const float2 u = *reinterpret_cast<const float2*>(sg + nt * 8);
                    s[nt][0] = fmaf(w0, u.x, s[nt][0]); s[nt][1] = fmaf(w0, u.y, s[nt][1]);
                }
            }
        }
        // mask (every row is the same query position), online softmax in powers of two
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + nt * 8 + c_lo + (e & 1);
                const bool seen = j <= hi && j >= lo && (e < 2 || top);
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
            for (int n = 0; n < 2 * NDV; ++n) {
                acc[n][0] *= alpha[0]; acc[n][1] *= alpha[0];
                acc[n][2] *= alpha[1]; acc[n][3] *= alpha[1];
            }
        }
        if (worker)
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
    }
    cp_async_wait<0>();

#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        if (!row_on[hh]) continue;
        const int h = h_row[hh];
        if (part >= 0) {
            float* pa = a.part_acc + ((size_t)part * NH + h) * DV + c_lo;
#pragma unroll
            for (int n = 0; n < 2 * NDV; ++n)
                if (n * 8 + c_lo < DV) *reinterpret_cast<float2*>(pa + n * 8) = make_float2(acc[n][2 * hh], acc[n][2 * hh + 1]);
            if ((lane & 3) == 0) {
                a.part_ml[((size_t)part * NH + h) * 2] = m_run[hh];
                a.part_ml[((size_t)part * NH + h) * 2 + 1] = l_run[hh];
            }
        } else {
            const float inv = l_run[hh] > 0.f ? 1.f / l_run[hh] : 0.f;
            bf16* o = a.out + (size_t)tok0 * a.out_stride + (size_t)h * DV + c_lo;
#pragma unroll
            for (int n = 0; n < 2 * NDV; ++n)
                if (n * 8 + c_lo < DV)
                    *reinterpret_cast<__nv_bfloat162*>(o + n * 8) = __floats2bfloat162_rn(acc[n][2 * hh] * inv, acc[n][2 * hh + 1] * inv);
        }
    }
}

static size_t mixed_dec_smem(const MixedArgs& a, int BN) {
    const size_t QP = ((a.D + 15) & ~15) * 2 + 16, VP = ((a.DV + 15) & ~15) * 2 + 16;
    return (size_t)a.NKV * MT_ROWS * QP + (size_t)2 * a.NKV * BN * (QP + VP) + (size_t)a.NH * (BN + 8) * 4 + (size_t)a.NH * a.NH * 4 +
           (size_t)a.rel_rows * a.NH * 4 + (size_t)a.NH * BN * 4 + (size_t)2 * BN * 4;
}

// the widest key tile with which one-token requests take this kernel; 0: they stay with the tile kernel
static int mixed_dec_tile(const MixedArgs& a) {
    if (a.NKV > MT_MAX_WARPS || a.NH / a.NKV > MT_ROWS) return 0;
    const int ndv = (a.DV + 15) / 16;
    if (ndv <= 4 && mixed_dec_smem(a, 64) <= MT_SMEM_LIMIT) return 64;
    if (mixed_dec_smem(a, 32) <= MT_SMEM_LIMIT) return 32;
    return mixed_dec_smem(a, 16) <= MT_SMEM_LIMIT ? 16 : 0;
}

template <int BN, int NDV>
static int launch_mixed_dec(const MixedArgs& a, size_t smem, cudaStream_t stream) {
    static AcvSmemConfig cfg;
    if (int rc = acv_ensure_smem(cfg, attn_mixed_dec_kernel<BN, NDV>, (int)smem)) return rc;
    acv_launch(PDL_ATTN, attn_mixed_dec_kernel<BN, NDV>, dim3(a.n_dec * a.n_split), dim3((a.NKV < 8 ? 8 : a.NKV) * 32), smem, stream, a);
    return acv_launch_status();
}
