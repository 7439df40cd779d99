// Attention for steps whose tiles have at most 16 rows (single tokens: the q-heads of one kv-head), one
// block per run.  Included by attention_tcgen05.cu, whose arithmetic it repeats row by row and bit for
// bit: the same scores (a chain of head_dim / 16 multiply-accumulate steps from zero), the same running
// maximum moved in the same blocks, the same 2^(s - m) with the same four-chain sum, p rounded to
// bfloat16, the same chain of P . V steps through a run's key blocks with the same rescaling between
// them, and the same fold of the runs (the code of it is shared).  What differs is the schedule.  The
// tcgen05 kernel walks a run's key blocks one after another, each through tensor memory and four
// hand-overs between warps: for 16 rows that is all latency.  Here a run's blocks are worked on side by
// side with mma.sync fragments (whose chains give the same bits as tcgen05's):
//   A  scores of all blocks, four warps taking the blocks in turn, to shared memory
//   B  a thread per (row, block): masked maximum; a thread per row: the scan that moves the maximum;
//      a thread per (row, block): p, its sum, P as bfloat16 into shared memory
//   C  O = sum over blocks of P . V, each warp a quarter of head_dim, rescaled between blocks
//   D  the run's (m, l, O) to scratch and the count, or straight to the output if the tile has one run
// Keys and values arrive by TMA into rings of their own, requested as early as there is room.
// The reference's single-token path: src/detllm/ops/fused_attn.py:47-115.
#pragma once

#define AF_THREADS 160
#define AF_MAX_RUN_BLOCKS 8
#define AF_MAX_ROWS 16
#define AF_MAX_STAGES 8
#define AF_S_STRIDE 65                     // floats between a (row, block)'s scores and the next one's: no two threads on one bank
#define AF_P_ROW_BYTES (AF_MAX_RUN_BLOCKS * AP_BN * 2)

__device__ __forceinline__ void af_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void af_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void af_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// Shared memory of a block, from the first 1024-byte border on: the rings, the barriers, P (a zero row
// behind the tile's rows), the scores, the per-(row, block) and per-row numbers.
struct AttnFewLayout {
    int block_bytes, stages, rows;
    __host__ __device__ int k_off() const { return 0; }
    __host__ __device__ int v_off() const { return stages * block_bytes; }
    __host__ __device__ int bar_off() const { return 2 * stages * block_bytes; }
    __host__ __device__ int p_off() const { return bar_off() + 512; }
    __host__ __device__ int s_off() const { return p_off() + (rows + 1) * AF_P_ROW_BYTES; }
    __host__ __device__ int stat_off() const { return s_off() + rows * AF_MAX_RUN_BLOCKS * AF_S_STRIDE * 4; }
    __host__ __device__ int need() const { return stat_off() + rows * (4 * AF_MAX_RUN_BLOCKS + 2) * 4; }
    __host__ __device__ int total() const { return need() + 1024; }
};

template <int HD>
__global__ void __launch_bounds__(AF_THREADS)
attention_few_rows_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                          AttnTcArgs a, const T* __restrict__ q, int stages) {
    constexpr int HT = HD / 64;
    constexpr int BLOCK_BYTES = HT * AP_BN * 128;
    constexpr int NT = HD / 32;                                  // 8-wide pieces of head_dim per warp in C
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    AttnFewLayout lay;
    lay.block_bytes = BLOCK_BYTES; lay.stages = stages; lay.rows = a.rows_cap;
    const uint32_t bars = base + lay.bar_off();
    auto k_full = [&](int i) { return bars + 8u * i; };
    auto k_empty = [&](int i) { return bars + 64 + 8u * i; };
    auto v_full = [&](int i) { return bars + 128 + 8u * i; };
    auto v_empty = [&](int i) { return bars + 192 + 8u * i; };
    volatile int* abort_flag = (volatile int*)(gbase + lay.bar_off() + 256);
    volatile int* last_flag = abort_flag + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    if (threadIdx.x == 0) attn_stamp(0);

    // (what is read here was written before the step began, not by the kernel before this one)
    const int tile = blockIdx.y;
    const int hg = blockIdx.x / a.max_runs, run = blockIdx.x % a.max_runs;
    const int gs = a.gp_shift, gp = 1 << gs;
    const int seq = a.tile_seq[tile], tstart = a.tile_start[tile];
    const int head0 = hg << gs;
    const int g = head0 / (a.n_q / a.n_kv);
    const int tok0 = a.cu_q[seq] + tstart;
    const int q_len = a.cu_q[seq + 1] - a.cu_q[seq];
    const int toks_valid = min(a.rows_cap >> gs, q_len - tstart);
    const int rows_valid = toks_valid << gs;
    const int p_first = a.q_start[seq] + tstart;
    const int p_last = p_first + toks_valid - 1;
    const int kv_len = a.kv_len[seq];
    const int nb_tile = p_last / AP_BN + 1;
    const int R = a.run_blocks;
    const int n_runs = (nb_tile + R - 1) / R;
    if (run >= n_runs) return;
    const int b_first = run * R;
    const int nb = min(R, nb_tile - b_first);
    const int n_hg = a.n_q >> gs;

    if (threadIdx.x == 0) {
        for (int i = 0; i < stages; ++i) {
            mbar_init(k_full(i), 1); mbar_init(k_empty(i), 1);
            mbar_init(v_full(i), 1); mbar_init(v_empty(i), 4);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    // the zero row of P (rows of the fragment beyond the tile's read it)
    if (threadIdx.x < AF_P_ROW_BYTES / 16)
        reinterpret_cast<uint4*>(gbase + lay.p_off() + a.rows_cap * AF_P_ROW_BYTES)[threadIdx.x] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    pdl_wait();
    if (threadIdx.x == 0) attn_stamp(1);

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer
        // Keys first (the scores wait for them), values into what room there is; then the rest of the keys
        // as their buffers come free, and only then the rest of the values, whose buffers come free last.
        const int* pages = a.table + (size_t)a.slots[seq] * a.table_stride + b_first;
        const int my_page = lane < nb ? pages[lane] : 0;         // (nb <= 8)
        if (lane == 0) attn_stamp(2);
        bool ok = true;
        for (int pass = 0; pass < 4 && ok; ++pass) {
            const bool keys = (pass & 1) == 0;
            const int from = pass < 2 ? 0 : stages, to = pass < 2 ? min(nb, stages) : nb;
            for (int b = from; b < to && ok; ++b) {
                const int page = __shfl_sync(0xffffffffu, my_page, b);
                const int row = (page * a.n_kv + g) * IDM_PAGE;
                const int st = b % stages, use = b / stages;
                if (lane == 0) {
                    const uint32_t full = keys ? k_full(st) : v_full(st);
                    if (use > 0) ok = mbar_wait(keys ? k_empty(st) : v_empty(st), (use - 1) & 1, abort_flag, &g_attn_tc_error);
                    if (ok) {
                        mbar_expect_tx(full, BLOCK_BYTES);
                        const uint32_t dst = base + (keys ? lay.k_off() : lay.v_off()) + st * BLOCK_BYTES;
                        for (int h = 0; h < HT; ++h)
                            tma_load_2d(dst + h * AP_BN * 128, keys ? &map_k : &map_v, h * 64, row, full);
                    }
                }
                ok = __shfl_sync(0xffffffffu, (int)ok, 0);
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- the four working warps
    const int tid = threadIdx.x;                                 // 0 .. 127
    const int gid = lane >> 2, tig = lane & 3;                   // the fragment's row (and row + 8) and column pair
    float* s_sm = reinterpret_cast<float*>(gbase + lay.s_off());
    float* st_sm = reinterpret_cast<float*>(gbase + lay.stat_off());
    const int rows = a.rows_cap;
    float* mblk_sm = st_sm;                                      // [rows][8] the block's maximum (scaled)
    float* alpha_sm = st_sm + rows * AF_MAX_RUN_BLOCKS;          // [rows][8] what the context is scaled by before the block
    float* negm_sm = alpha_sm + rows * AF_MAX_RUN_BLOCKS;        // [rows][8] minus the reference maximum in the block
    float* rsum_sm = negm_sm + rows * AF_MAX_RUN_BLOCKS;         // [rows][8] the block's sum of p
    float* mfin_sm = rsum_sm + rows * AF_MAX_RUN_BLOCKS;         // [rows] the run's m
    float* lfin_sm = mfin_sm + rows;                             // [rows] the run's l
    const uint32_t p_base = base + lay.p_off();
    bool ok = true;

    // ---- A: scores
    {
        uint32_t qa[HD / 16][4];
        const int r_lo = gid, r_hi = gid + 8;
        const T* q_lo = q + ((size_t)(tok0 + (r_lo >> gs)) * a.n_q + head0 + (r_lo & (gp - 1))) * HD;
        const T* q_hi = q + ((size_t)(tok0 + (r_hi >> gs)) * a.n_q + head0 + (r_hi & (gp - 1))) * HD;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            const int d = kk * 16 + tig * 2;
            qa[kk][0] = r_lo < rows_valid ? *reinterpret_cast<const uint32_t*>(q_lo + d) : 0u;
            qa[kk][1] = r_hi < rows_valid ? *reinterpret_cast<const uint32_t*>(q_hi + d) : 0u;
            qa[kk][2] = r_lo < rows_valid ? *reinterpret_cast<const uint32_t*>(q_lo + d + 8) : 0u;
            qa[kk][3] = r_hi < rows_valid ? *reinterpret_cast<const uint32_t*>(q_hi + d + 8) : 0u;
        }
        // ldmatrix x4: lanes 0-7 keys n0.. chunk c, 8-15 the same keys chunk c + 1, 16-23 keys n0 + 8.. chunk c, 24-31 chunk c + 1
        const int key_in_pair = (lane & 7) + ((lane >> 4) << 3), chunk_sel = (lane >> 3) & 1;
        // (a buffer of the ring always goes to the same warp: a warp that skipped one of a barrier's phases
        // could take an earlier phase of the same parity for the one it waits for)
        for (int bl = 0; bl < nb && ok; ++bl) {
            const int st = bl % stages;
            if ((st & 3) != warp) continue;
            ok = mbar_wait(k_full(st), (bl / stages) & 1, abort_flag, &g_attn_tc_error);
            if (!ok) break;
            const uint32_t kb = base + lay.k_off() + st * BLOCK_BYTES;
            float acc[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                const int chunk = (kk & 3) * 2 + chunk_sel;
#pragma unroll
                for (int np = 0; np < 4; ++np) {                 // two 8-key pieces at a time
                    const int key = np * 16 + key_in_pair;
                    uint32_t bfr[4];
                    af_ldmatrix_x4(bfr, kb + (kk >> 2) * (AP_BN * 128) + key * 128 + ((chunk ^ (key & 7)) << 4));
                    af_mma(acc[2 * np], qa[kk], bfr[0], bfr[1]);
                    af_mma(acc[2 * np + 1], qa[kk], bfr[2], bfr[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(k_empty(st));
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const int col = nt * 8 + tig * 2;
                if (r_lo < rows_valid) {
                    float* d = s_sm + (r_lo * AF_MAX_RUN_BLOCKS + bl) * AF_S_STRIDE + col;
                    d[0] = acc[nt][0]; d[1] = acc[nt][1];
                }
                if (r_hi < rows_valid) {
                    float* d = s_sm + (r_hi * AF_MAX_RUN_BLOCKS + bl) * AF_S_STRIDE + col;
                    d[0] = acc[nt][2]; d[1] = acc[nt][3];
                }
            }
        }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (tid == 0) attn_stamp(3);

    // ---- B: the softmax of every (row, block), in the order the one-block-after-another kernel has it
    const bool has_task = tid < rows_valid * nb;
    const int t_row = has_task ? tid / nb : 0, t_bl = has_task ? tid % nb : 0;
    const float* s_row = s_sm + (t_row * AF_MAX_RUN_BLOCKS + t_bl) * AF_S_STRIDE;
    const int visible = p_first + (t_row >> gs) - (b_first + t_bl) * AP_BN;   // scores j <= visible count
    if (has_task) {
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < AP_BN; j += 4) {
#pragma unroll
            for (int u = 0; u < 4; ++u) mx[u] = fmaxf(mx[u], j + u > visible ? -INFINITY : s_row[j + u]);
        }
        mblk_sm[t_row * AF_MAX_RUN_BLOCKS + t_bl] = __fmul_rn(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), a.scale_log2);
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (tid < rows_valid) {
        float m_ref = -INFINITY;
        for (int bl = 0; bl < nb; ++bl) {
            const float m_blk = mblk_sm[tid * AF_MAX_RUN_BLOCKS + bl];
            float alpha = 1.f;
            if (m_blk > m_ref + AP_RESCALE_STEP) {
                alpha = exp2f(m_ref - m_blk);
                m_ref = m_blk;
            }
            alpha_sm[tid * AF_MAX_RUN_BLOCKS + bl] = alpha;
            negm_sm[tid * AF_MAX_RUN_BLOCKS + bl] = m_ref == -INFINITY ? 0.f : -m_ref;
        }
        mfin_sm[tid] = m_ref;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (has_task) {
        const float neg_m = negm_sm[t_row * AF_MAX_RUN_BLOCKS + t_bl];
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        uint8_t* prow = gbase + lay.p_off() + t_row * AF_P_ROW_BYTES;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            uint32_t w[4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int j = c * 8 + h * 4;
                const float p0 = ex2_hw(__fmaf_rn(j > visible ? -INFINITY : s_row[j], a.scale_log2, neg_m));
                const float p1 = ex2_hw(__fmaf_rn(j + 1 > visible ? -INFINITY : s_row[j + 1], a.scale_log2, neg_m));
                const float p2 = ex2_hw(__fmaf_rn(j + 2 > visible ? -INFINITY : s_row[j + 2], a.scale_log2, neg_m));
                const float p3 = ex2_hw(__fmaf_rn(j + 3 > visible ? -INFINITY : s_row[j + 3], a.scale_log2, neg_m));
                sum4[0] = __fadd_rn(sum4[0], p0); sum4[1] = __fadd_rn(sum4[1], p1);
                sum4[2] = __fadd_rn(sum4[2], p2); sum4[3] = __fadd_rn(sum4[3], p3);
                const __nv_bfloat162 pa = __floats2bfloat162_rn(p0, p1), pb = __floats2bfloat162_rn(p2, p3);
                w[2 * h] = *reinterpret_cast<const uint32_t*>(&pa);
                w[2 * h + 1] = *reinterpret_cast<const uint32_t*>(&pb);
            }
            const int chunk = t_bl * 8 + c;
            *reinterpret_cast<uint4*>(prow + ((chunk ^ (t_row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        rsum_sm[t_row * AF_MAX_RUN_BLOCKS + t_bl] = __fadd_rn(__fadd_rn(sum4[0], sum4[1]), __fadd_rn(sum4[2], sum4[3]));
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (tid == 0) attn_stamp(4);
    if (tid < rows_valid) {
        float l = 0.f;
        for (int bl = 0; bl < nb; ++bl)
            l = __fmaf_rn(l, alpha_sm[tid * AF_MAX_RUN_BLOCKS + bl], rsum_sm[tid * AF_MAX_RUN_BLOCKS + bl]);
        lfin_sm[tid] = l;
    }

    // ---- C: O = sum of P . V over the run's blocks; this warp has dims [warp * HD / 4, (warp + 1) * HD / 4)
    float o[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f; }
    {
        const int r_lo = gid, r_hi = gid + 8;
        // A fragments of P: lanes 0-7 rows 0-7 chunk c, 8-15 rows 8-15 chunk c, 16-23 rows 0-7 chunk c + 1, 24-31 rows 8-15 chunk c + 1
        const int a_row_raw = (lane & 7) + (((lane >> 3) & 1) << 3);
        const int a_row = a_row_raw < rows_valid ? a_row_raw : rows;   // (the zero row)
        const int a_sel = lane >> 4;
        const uint32_t a_row_addr = p_base + a_row * AF_P_ROW_BYTES;
        // B fragments of V (transposed on the way): lanes 0-7 keys k0.. dims d0, 8-15 keys k0 + 8.. dims d0, 16-23 keys k0.. dims d0 + 8, 24-31 keys k0 + 8.. dims d0 + 8
        const int v_key = (lane & 7) + (((lane >> 3) & 1) << 3);
        const int v_dsel = lane >> 4;
        const int d_warp = warp * (HD / 4);
        for (int bl = 0; bl < nb && ok; ++bl) {
            const int st = bl % stages;
            ok = mbar_wait(v_full(st), (bl / stages) & 1, abort_flag, &g_attn_tc_error);
            if (!ok) break;
            uint8_t* vgen = gbase + lay.v_off() + st * BLOCK_BYTES;
            const uint32_t vb = base + lay.v_off() + st * BLOCK_BYTES;
            const int key0 = (b_first + bl) * AP_BN;
            if (key0 + AP_BN > kv_len) {
                // rows of V past the sequence's end hold whatever the page held before: this warp zeroes its own dims of them
                const int first_bad = max(kv_len - key0, 0);
                constexpr int CH = HD / 32;                      // 16-byte pieces of a row that are this warp's
                for (int idx = lane; idx < (AP_BN - first_bad) * CH; idx += 32) {
                    const int key = first_bad + idx / CH, d = d_warp + (idx % CH) * 8;
                    const int chunk = (d & 63) >> 3;
                    *reinterpret_cast<uint4*>(vgen + (d >> 6) * (AP_BN * 128) + key * 128 + ((chunk ^ (key & 7)) << 4)) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
            if (bl > 0) {
                const float a_lo = r_lo < rows_valid ? alpha_sm[r_lo * AF_MAX_RUN_BLOCKS + bl] : 1.f;
                const float a_hi = r_hi < rows_valid ? alpha_sm[r_hi * AF_MAX_RUN_BLOCKS + bl] : 1.f;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    o[nt][0] = __fmul_rn(o[nt][0], a_lo); o[nt][1] = __fmul_rn(o[nt][1], a_lo);
                    o[nt][2] = __fmul_rn(o[nt][2], a_hi); o[nt][3] = __fmul_rn(o[nt][3], a_hi);
                }
            }
#pragma unroll
            for (int kk = 0; kk < AP_BN / 16; ++kk) {
                uint32_t pa[4];
                const int chunk = bl * 8 + kk * 2 + a_sel;
                af_ldmatrix_x4(pa, a_row_addr + ((chunk ^ (a_row & 7)) << 4));
                const int key = kk * 16 + v_key;
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    const int d = d_warp + np * 16 + v_dsel * 8;
                    const int vchunk = (d & 63) >> 3;
                    uint32_t bfr[4];
                    af_ldmatrix_x4_trans(bfr, vb + (d >> 6) * (AP_BN * 128) + key * 128 + ((vchunk ^ (key & 7)) << 4));
                    af_mma(o[2 * np], pa, bfr[0], bfr[1]);
                    af_mma(o[2 * np + 1], pa, bfr[2], bfr[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(v_empty(st));
        }
    }
    ok = __all_sync(0xffffffffu, ok);
    asm volatile("bar.sync 1, 128;" ::: "memory");               // (the runs' l are there)
    if (tid == 0) attn_stamp(40);

    // ---- D
    const int r_lo = gid, r_hi = gid + 8;
    if (n_runs > 1) {
        const int cap = a.rows_cap;
        const size_t part_floats = run_part_floats(cap, HD);
        float* part0 = a.parts + (size_t)(tile * n_hg + hg) * a.max_runs * part_floats;
        float* mine = part0 + (size_t)run * part_floats;
        if (ok) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int d = warp * (HD / 4) + nt * 8 + tig * 2;
                if (r_lo < rows_valid)
                    *reinterpret_cast<float2*>(mine + ((size_t)(d >> 2) * cap + r_lo) * 4 + (d & 3)) = make_float2(o[nt][0], o[nt][1]);
                if (r_hi < rows_valid)
                    *reinterpret_cast<float2*>(mine + ((size_t)(d >> 2) * cap + r_hi) * 4 + (d & 3)) = make_float2(o[nt][2], o[nt][3]);
            }
            if (tid < rows_valid) reinterpret_cast<float2*>(mine + (size_t)HD * cap)[tid] = make_float2(mfin_sm[tid], lfin_sm[tid]);
            __threadfence();
        }
        count_and_fold_runs<HD>(a, part0, part_floats, n_runs, rows_valid, tok0, head0, tile * n_hg + hg, last_flag, tid, ok);
        if (tid == 0) attn_stamp(41);
    } else if (ok) {
        // the tile's only run: folded onto nothing, then divided by the sum
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = half ? r_hi : r_lo;
            if (r >= rows_valid) continue;
            float M = -INFINITY, L = 0.f, a_, b_;
            fold_coeffs(M, L, mfin_sm[r], lfin_sm[r], a_, b_);
            const float inv = __fdiv_rn(1.0f, L);
            T* orow = a.out + ((size_t)(tok0 + (r >> gs)) * a.n_q + head0 + (r & (gp - 1))) * HD;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int d = warp * (HD / 4) + nt * 8 + tig * 2;
                const __nv_bfloat162 pk = __floats2bfloat162_rn(__fmul_rn(fold_value(0.f, a_, o[nt][2 * half], b_), inv),
                                                                __fmul_rn(fold_value(0.f, a_, o[nt][2 * half + 1], b_), inv));
                *reinterpret_cast<__nv_bfloat162*>(orow + d) = pk;
            }
        }
    }
    if (tid == 0) attn_stamp(42);
}

// The rings' depth and the block's shared memory for tiles of `rows` rows: two blocks per SM where the
// rings then still hold three key blocks and three value blocks, else one block with deeper rings.
static int attention_few_rows_plan(int hd, int rows, int* stages_out) {
    AttnFewLayout lay;
    lay.block_bytes = (hd / 64) * AP_BN * 128; lay.rows = rows; lay.stages = 0;
    const int fixed = lay.total();
    const int two_per_sm = (228 * 1024) / 2 - 1024, one_per_sm = 227 * 1024;
    int stages = (two_per_sm - fixed) / (2 * lay.block_bytes);
    if (stages < 3) stages = (one_per_sm - fixed) / (2 * lay.block_bytes);
    if (stages > AF_MAX_STAGES) stages = AF_MAX_STAGES;
    *stages_out = stages;
    lay.stages = stages;
    return lay.total();
}

static bool attention_few_rows_can(int hd, int rows_cap, int run_blocks, int max_runs) {
    return (hd == 64 || hd == 128) && rows_cap <= AF_MAX_ROWS && run_blocks <= AF_MAX_RUN_BLOCKS && max_runs > 0;
}

template <int HD>
static int launch_attention_few_rows(const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcArgs& a, const T* q,
                                     int n_tiles, cudaStream_t stream) {
    int stages = 0;
    const int bytes = attention_few_rows_plan(HD, a.rows_cap, &stages);
    IDM_REQUIRE(stages >= 2, "attention_few_rows: no room for the rings (%d rows)", a.rows_cap);
    static int configured = 0;
    if (configured < bytes) {
        cudaError_t e = cudaFuncSetAttribute(attention_few_rows_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        IDM_REQUIRE(e == cudaSuccess, "attention_few_rows: cannot get %d bytes of shared memory: %s", bytes, cudaGetErrorString(e));
        configured = bytes;
    }
    const int n_hg = a.n_q >> a.gp_shift;
    dim3 grid(n_hg * a.max_runs, n_tiles);
    idm_launch(attention_few_rows_kernel<HD>, dim3(grid), dim3(AF_THREADS), (size_t)bytes, stream, mk, mv, a, q, stages);
    IDM_LAUNCH_CHECK("attention_few_rows");
    return 0;
}
