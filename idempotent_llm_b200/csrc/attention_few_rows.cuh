// Attention for steps whose tiles have at most 16 rows (single tokens: the q-heads of one kv-head).
// Included by attention_tcgen05.cu, whose arithmetic it repeats row by row and bit for bit: the same
// scores (a chain of head_dim / 16 multiply-accumulate steps from zero), the same running maximum moved
// in the same blocks, the same 2^(s - m) with the same four-chain sum, p rounded to bfloat16, the same
// chain of P . V steps through a run's key blocks with the same rescaling between them, and the same
// fold of the runs (the code of it is shared).  What differs is the schedule.  The tcgen05 kernel walks
// a run's key blocks one after another, each through tensor memory and four hand-overs between warps:
// for 16 rows that is all latency.  Here the work item is one run of one tile and head group, and its
// blocks are worked on side by side with mma.sync fragments (whose chains give the same bits as tcgen05's):
//   A  scores of all blocks (the warps share them out) to shared memory, and each block's masked maximum
//   B  a thread per (row, block): where the running maximum stands in its block, p, its sum, P as
//      bfloat16 into shared memory
//   C  O = sum over blocks of P . V, each warp a quarter of head_dim, rescaled between blocks
//   D  the run's (m, l, O) to scratch and the count, or straight to the output if the tile has one run
// The blocks are persistent: each takes items from one counter until none is left, so that the keys
// and values of the next item are on their way while this one is finished, and the SMs stay level.
// A scheduler warp takes the items and looks up what they need (lengths, page numbers) ahead of time; a
// TMA warp requests an item's key blocks and then its value blocks, in that order, into one ring;
// four warps do the arithmetic.
// The reference's single-token path: src/detllm/ops/fused_attn.py:47-115.
#pragma once

#define AF_THREADS 192
#define AF_MAX_RUN_BLOCKS 8
#define AF_MAX_ROWS 16
#define AF_MAX_SLOTS 12
#define AF_QUEUE 2                         // items a block holds: the one being worked on and the next
#define AF_S_STRIDE 69                     // floats between a (row, block)'s scores and the next one's: spreads the threads of phase B over the banks
#define AF_P_ROW_BYTES (AF_MAX_RUN_BLOCKS * AP_BN * 2)
#define AF_WORK_COUNTER (AP_COUNTERS - 2)  // the last two arrival counters: items taken, blocks gone
#define AF_EXIT_COUNTER (AP_COUNTERS - 1)

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
// the working warps' barrier (named barrier 1, 128 threads) with a vote: true if any thread says so
__device__ __forceinline__ bool af_bar_any(bool mine) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbarrier.red.or.pred q, 1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(r) : "r"((uint32_t)mine) : "memory");
    return r != 0;
}
// one arrival more at a counter, with release and acquire at the scope of the GPU; the count before
__device__ __forceinline__ int af_count(int* counter) {
    int old;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
    return old;
}
__device__ __forceinline__ void af_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// A tile and head group whose runs have all arrived: to be folded
struct AttnFewFold {
    int n_runs;                            // 0: nothing to fold
    int tile, hg, rows_valid, tok0;
};
// What the scheduler warp hands on about an item, and with it up to two folds for the working warps
struct AttnFewItem {
    int item;                              // < 0: no more
    int tile, hg, run, n_runs;
    int tok0, rows_valid, p_first, kv_len;
    int b_first, nb, kv_head;
    int old_len;                           // the sequence's length before this step: blocks below it were written by earlier steps
    int pages[AF_MAX_RUN_BLOCKS];
    AttnFewFold fold[2];
    int pad[1];
};
static_assert(sizeof(AttnFewItem) == 128, "one item, 128 bytes");

// Shared memory of a block, from the first 1024-byte border on: the ring, the barriers, the items, P (a
// zero row behind the tile's rows), the scores, the per-(row, block) and per-row numbers.
struct AttnFewLayout {
    int block_bytes, slots, rows;
    __host__ __device__ int bar_off() const { return slots * block_bytes; }
    __host__ __device__ int item_off() const { return bar_off() + 512; }
    __host__ __device__ int p_off() const { return item_off() + AF_QUEUE * 128; }
    __host__ __device__ int s_off() const { return p_off() + (rows + 1) * AF_P_ROW_BYTES; }
    __host__ __device__ int stat_off() const { return s_off() + rows * AF_MAX_RUN_BLOCKS * AF_S_STRIDE * 4; }
    __host__ __device__ int need() const { return stat_off() + rows * (2 * AF_MAX_RUN_BLOCKS + 2) * 4; }
    __host__ __device__ int total() const { return need() + 1024; }
};

template <int HD>
__global__ void __launch_bounds__(AF_THREADS, 2)
attention_few_rows_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                          AttnTcArgs a, const T* __restrict__ q, int slots, int n_tiles) {
    constexpr int HT = HD / 64;
    constexpr int BLOCK_BYTES = HT * AP_BN * 128;
    constexpr int NT = HD / 32;                                  // 8-wide pieces of head_dim per warp in C
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    AttnFewLayout lay;
    lay.block_bytes = BLOCK_BYTES; lay.slots = slots; lay.rows = a.rows_cap;
    const uint32_t bars = base + lay.bar_off();
    auto full = [&](int i) { return bars + 8u * i; };            // a ring slot's block has arrived
    auto empty = [&](int i) { return bars + 128 + 8u * i; };     // ... has been used (four arrivals)
    auto q_full = [&](int i) { return bars + 256 + 8u * i; };    // an item is described
    auto q_empty = [&](int i) { return bars + 288 + 8u * i; };   // ... is finished with (four working warps and the TMA warp)
    auto d_done = [&](int i) { return bars + 304 + 8u * i; };    // an item's result is written (four working warps)
    volatile int* abort_flag = (volatile int*)(gbase + lay.bar_off() + 320);
    volatile AttnFewItem* items = (volatile AttnFewItem*)(gbase + lay.item_off());

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    if (threadIdx.x == 0) { attn_stamp(0); attn_item_stamp(0, 6); }
    const int gs = a.gp_shift, gp = 1 << gs;
    const int n_hg = a.n_q >> gs;
    const int R = a.run_blocks;

    if (threadIdx.x == 0) {
        for (int i = 0; i < slots; ++i) { mbar_init(full(i), 1); mbar_init(empty(i), 4); }
        for (int i = 0; i < AF_QUEUE; ++i) { mbar_init(q_full(i), 1); mbar_init(q_empty(i), 5); mbar_init(d_done(i), 4); }
        *abort_flag = 0;
        mbar_init_fence();
    }
    // the zero row of P (rows of the fragment beyond the tile's read it)
    if (threadIdx.x < AF_P_ROW_BYTES / 16)
        reinterpret_cast<uint4*>(gbase + lay.p_off() + a.rows_cap * AF_P_ROW_BYTES)[threadIdx.x] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    // The kernel before this one wrote q and the step's own keys and values.  What is older (the lengths
    // and page numbers, the key blocks below the step's first position) is looked up and asked for at
    // once; each role waits for that kernel where it first needs something of it.
    if (threadIdx.x == 0) attn_stamp(1);

    if (warp == 5) {
        // ------------------------------------------------------------------ scheduler
        // Items are numbered run by run up to the step's bound (then tile, then head group), so that the
        // runs few tiles have come last; runs beyond a tile's own last one are passed over.  A block's
        // first item is its own number, the others come from a counter.  (What is looked up here was
        // written before the step began.)
        const int total = n_tiles * n_hg * a.max_runs;
        bool ok = true, waited = false;
        AttnFewFold prev, pending;                               // the item whose arrival is still to be counted; a fold still to be handed on
        prev.n_runs = 0; pending.n_runs = 0;
        int prev_st = 0, prev_parity = 0;
        for (int qn = 0; ok; ++qn) {
            int item = -1, tile = 0, hg = 0, run = 0, seq = 0, tstart = 0, n_runs = 0, nb_tile = 0, toks_valid = 0, p_first = 0;
            for (;;) {
                if (qn == 0 && !waited && item == -1) {
                    item = blockIdx.x;
                } else {
                    if (!waited) { pdl_wait(); waited = true; }  // (the launch before has put the counter back to zero)
                    if (lane == 0) item = (int)gridDim.x + atomicAdd(a.counters + AF_WORK_COUNTER, 1);
                    item = __shfl_sync(0xffffffffu, item, 0);
                }
                if (item >= total) { item = -1; break; }
                run = item / (n_tiles * n_hg);
                tile = (item / n_hg) % n_tiles;
                hg = item % n_hg;
                seq = a.tile_seq[tile]; tstart = a.tile_start[tile];
                const int q_len = a.cu_q[seq + 1] - a.cu_q[seq];
                toks_valid = min(a.rows_cap >> gs, q_len - tstart);
                p_first = a.q_start[seq] + tstart;
                nb_tile = (p_first + toks_valid - 1) / AP_BN + 1;
                n_runs = (nb_tile + R - 1) / R;
                if (run < n_runs) break;
                item = -2;                                       // (passed over: the next one comes from the counter)
            }
            const int st = qn % AF_QUEUE;
            if (qn >= AF_QUEUE) {
                if (lane == 0) ok = mbar_wait(q_empty(st), ((qn / AF_QUEUE) - 1) & 1, abort_flag, &g_attn_tc_error);
                ok = __shfl_sync(0xffffffffu, (int)ok, 0);
                if (!ok) break;
            }
            // When the working warps have written an item's result, its arrival is counted here (they are
            // on the next item by then); if it was the last of its tile and head group to arrive, the fold
            // of the runs goes to the working warps with the next item described after that.  With the
            // last item of all, that is the notice that there is no more, which waits for it.
            auto complete = [&](AttnFewFold& job) -> bool {
                job.n_runs = 0;
                if (prev.n_runs == 0) return true;
                bool fine = true;
                if (lane == 0) fine = mbar_wait(d_done(prev_st), prev_parity, abort_flag, &g_attn_tc_error);
                fine = __shfl_sync(0xffffffffu, (int)fine, 0);
                if (fine && prev.n_runs > 1) {
                    if (!waited) { pdl_wait(); waited = true; }
                    int is_last = 0;
                    if (lane == 0) {
                        // (release: the working warps' stores, seen here through the barrier, come before the count;
                        // acquire: whoever counts last has the other blocks' results behind it, and so have the
                        // working warps it hands the fold to through the item's barrier)
                        int* counter = a.counters + prev.tile * n_hg + prev.hg;
                        is_last = af_count(counter) == prev.n_runs - 1;
                        if (is_last) *counter = 0;               // ready for the next launch
                    }
                    if (__shfl_sync(0xffffffffu, is_last, 0)) job = prev;
                }
                prev.n_runs = 0;
                return fine;
            };
            AttnFewFold now;
            now.n_runs = 0;
            if (item < 0) ok = complete(now);
            if (!ok) break;
            volatile AttnFewItem* d = items + st;
            if (item >= 0) {
                const int b_first = run * R, nb = min(R, nb_tile - b_first);
                if (lane < nb) d->pages[lane] = a.table[(size_t)a.slots[seq] * a.table_stride + b_first + lane];
                if (lane == 0) {
                    d->tile = tile; d->hg = hg; d->run = run; d->n_runs = n_runs;
                    d->tok0 = a.cu_q[seq] + tstart; d->rows_valid = toks_valid << gs; d->p_first = p_first;
                    d->kv_len = a.kv_len[seq]; d->b_first = b_first; d->nb = nb; d->old_len = a.q_start[seq];
                    d->kv_head = (hg << gs) / (a.n_q / a.n_kv);
                }
            }
            if (lane == 0) {
                d->item = item;
                d->fold[0].n_runs = pending.n_runs; d->fold[0].tile = pending.tile; d->fold[0].hg = pending.hg;
                d->fold[0].rows_valid = pending.rows_valid; d->fold[0].tok0 = pending.tok0;
                d->fold[1].n_runs = now.n_runs; d->fold[1].tile = now.tile; d->fold[1].hg = now.hg;
                d->fold[1].rows_valid = now.rows_valid; d->fold[1].tok0 = now.tok0;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full(st));
            if (item < 0) {
                // No more items for anybody.  The block whose scheduler comes here last puts the two counters of
                // the items back to zero for the next launch.  (After a wait that ran out counters may be left
                // standing: the caller, told by the status word, clears the scratch.)
                if (lane == 0 && atomicAdd(a.counters + AF_EXIT_COUNTER, 1) == (int)gridDim.x - 1) {
                    a.counters[AF_EXIT_COUNTER] = 0;
                    a.counters[AF_WORK_COUNTER] = 0;
                }
                break;
            }
            ok = complete(pending);
            prev.n_runs = n_runs; prev.tile = tile; prev.hg = hg; prev.rows_valid = toks_valid << gs; prev.tok0 = a.cu_q[seq] + tstart;
            prev_st = st; prev_parity = (qn / AF_QUEUE) & 1;
        }
        return;
    }
    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer
        // An item's key blocks, then its value blocks, one ring slot after another; a slot is asked for
        // again when its four users have arrived.
        int slot = 0, use = 0;
        bool ok = true, waited = false;
        for (int qn = 0; ok; ++qn) {
            const int st = qn % AF_QUEUE;
            if (lane == 0) ok = mbar_wait(q_full(st), (qn / AF_QUEUE) & 1, abort_flag, &g_attn_tc_error);
            ok = __shfl_sync(0xffffffffu, (int)ok, 0);
            if (!ok) break;
            volatile AttnFewItem* d = items + st;
            if (d->item < 0) break;
            const int nb = d->nb, g = d->kv_head;
            const int old_blocks = d->old_len / AP_BN - d->b_first;   // this many of the item's blocks hold nothing of this step
            const int my_page = lane < nb ? d->pages[lane] : 0;
            for (int r = 0; r < 2 * nb && ok; ++r) {
                const bool keys = r < nb;
                const int b = keys ? r : r - nb;
                const int page = __shfl_sync(0xffffffffu, my_page, b);
                if (!waited && b >= old_blocks) { pdl_wait(); waited = true; }
                if (lane == 0) {
                    if (use > 0) ok = mbar_wait(empty(slot), (use - 1) & 1, abort_flag, &g_attn_tc_error);
                    if (ok) {
                        const int row = (page * a.n_kv + g) * IDM_PAGE;
                        mbar_expect_tx(full(slot), BLOCK_BYTES);
                        for (int h = 0; h < HT; ++h)
                            tma_load_2d(base + slot * BLOCK_BYTES + h * AP_BN * 128, keys ? &map_k : &map_v, h * 64, row, full(slot));
                    }
                }
                ok = __shfl_sync(0xffffffffu, (int)ok, 0);
                if (++slot == slots) { slot = 0; ++use; }
            }
            if (ok && lane == 0) mbar_arrive(q_empty(st));
        }
        return;
    }

    // ---------------------------------------------------------------------- the four working warps
    const int tid = threadIdx.x;                                 // 0 .. 127
    const int gid = lane >> 2, tig = lane & 3;                   // the fragment's row (and row + 8) and column pair
    const int r_lo = gid, r_hi = gid + 8;
    float* s_sm = reinterpret_cast<float*>(gbase + lay.s_off());
    float* st_sm = reinterpret_cast<float*>(gbase + lay.stat_off());
    const int rows = a.rows_cap;
    float* mblk_sm = st_sm;                                      // [rows][8] the block's maximum (scaled)
    float* alpha_sm = st_sm + rows * AF_MAX_RUN_BLOCKS;          // [rows][8] what the context is scaled by before the block
    float* rsum_sm = alpha_sm + rows * AF_MAX_RUN_BLOCKS;        // [rows][8] the block's sum of p
    float* mfin_sm = rsum_sm + rows * AF_MAX_RUN_BLOCKS;         // [rows] the run's m
    float* lfin_sm = mfin_sm + rows;                             // [rows] the run's l
    const uint32_t p_base = base + lay.p_off();
    // ldmatrix addressing that does not change from item to item
    //   keys (B of the scores): lanes 0-7 keys n0.. chunk c, 8-15 the same keys chunk c + 1, 16-23 keys n0 + 8.. chunk c, 24-31 chunk c + 1
    const int key_in_pair = (lane & 7) + ((lane >> 4) << 3), chunk_sel = (lane >> 3) & 1;
    //   P (A of the context): lanes 0-7 rows 0-7 chunk c, 8-15 rows 8-15 chunk c, 16-23 rows 0-7 chunk c + 1, 24-31 rows 8-15 chunk c + 1
    const int a_row_raw = (lane & 7) + (((lane >> 3) & 1) << 3), a_sel = lane >> 4;
    //   values (B of the context, transposed on the way): lanes 0-7 keys k0.. dims d0, 8-15 keys k0 + 8.. dims d0, 16-23 keys k0.. dims d0 + 8, 24-31 keys k0 + 8.. dims d0 + 8
    const int v_key = (lane & 7) + (((lane >> 3) & 1) << 3), v_dsel = lane >> 4;
    const int d_warp = warp * (HD / 4);
    int pos_slot = 0, pos_use = 0;                               // the ring's slot and use of this item's first request

    // The first pass (qn == -1) is a rehearsal: while the kernel before this one still runs, the four
    // phases are walked once over a made-up item of one key block (whatever the ring's first slot holds;
    // no barrier of the ring is touched, nothing is read from or written to global memory), so that the
    // instructions are in the SM's cache when the first real item comes.  Fetching them from memory,
    // which the keys and values of every layer push them out of, was measured at several microseconds.
    // Then this role waits for that kernel (q, and the right to write results).
    for (int qn = -1;; ++qn) {
        const bool dry = qn < 0;
        const int qst = dry ? 0 : qn % AF_QUEUE;
        bool ok = true;
        int tile = 0, hg = 0, run = 0, n_runs = 2, tok0 = 0, rows_valid = rows, p_first = AP_BN - 1, kv_len = 1 << 30, b_first = 0, nb = 1;
        if (!dry) {
            ok = mbar_wait(q_full(qst), (qn / AF_QUEUE) & 1, abort_flag, &g_attn_tc_error);
            // (this barrier also parts the item before, whose P and numbers were read to its end, from this one)
            if (af_bar_any(!ok)) break;
            volatile AttnFewItem* d = items + qst;
            // folds that come with the item: tiles whose last run another of this block's items was
#pragma unroll 1
            for (int f = 0; f < 2; ++f) {
                const int f_runs = d->fold[f].n_runs;
                if (f_runs == 0) continue;
                const int f_tile = d->fold[f].tile, f_hg = d->fold[f].hg;
                const size_t part_floats = run_part_floats(a.rows_cap, HD);
                const float* part0 = a.parts + (size_t)(f_tile * n_hg + f_hg) * a.max_runs * part_floats;
                fold_runs_and_store<HD>(a, part0, part_floats, f_runs, d->fold[f].rows_valid, d->fold[f].tok0, f_hg << gs, tid, 128);
            }
            if (d->item < 0) break;
            tile = d->tile; hg = d->hg; run = d->run; n_runs = d->n_runs; tok0 = d->tok0;
            rows_valid = d->rows_valid; p_first = d->p_first; kv_len = d->kv_len; b_first = d->b_first; nb = d->nb;
        }
        const int head0 = hg << gs;
        if (tid == 0) { attn_stamp(2); attn_item_stamp(qn, 0); }

        // ---- A: scores, and the maximum of every row in every block
        {
            uint32_t qa[HD / 16][4];
            const T* q_lo = q + ((size_t)(tok0 + (r_lo >> gs)) * a.n_q + head0 + (r_lo & (gp - 1))) * HD;
            const T* q_hi = q + ((size_t)(tok0 + (r_hi >> gs)) * a.n_q + head0 + (r_hi & (gp - 1))) * HD;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                const int dd = kk * 16 + tig * 2;
                qa[kk][0] = (!dry && r_lo < rows_valid) ? *reinterpret_cast<const uint32_t*>(q_lo + dd) : 0u;
                qa[kk][1] = (!dry && r_hi < rows_valid) ? *reinterpret_cast<const uint32_t*>(q_hi + dd) : 0u;
                qa[kk][2] = (!dry && r_lo < rows_valid) ? *reinterpret_cast<const uint32_t*>(q_lo + dd + 8) : 0u;
                qa[kk][3] = (!dry && r_hi < rows_valid) ? *reinterpret_cast<const uint32_t*>(q_hi + dd + 8) : 0u;
            }
            // (a slot's key blocks always go to the same warp: a warp that skipped one of a barrier's phases
            // could take an earlier phase of the same parity for the one it waits for)
            if (tid == 0) attn_item_stamp(qn, 7);                 // (q asked for)
            int sl = pos_slot, use = pos_use;                     // (the ring's slot and use of the item's first key block)
            for (int bl = 0; bl < nb && ok; ++bl, sl = sl + 1 == slots ? 0 : sl + 1, use += sl == 0) {
                if ((sl & 3) != warp) continue;
                if (!dry) ok = mbar_wait(full(sl), use & 1, abort_flag, &g_attn_tc_error);
                if (!ok) break;
                if (lane == 0) attn_stamp(10 + 3 * warp);
                const uint32_t kb = base + sl * BLOCK_BYTES;
                float acc[8][4];
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) { acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f; }
                // (the fragments of step kk + 1 are asked for before the products of step kk are issued)
                uint32_t bfr[2][4][4];
                auto fetch = [&](int kk, uint32_t (&dst)[4][4]) {
                    const int chunk = (kk & 3) * 2 + chunk_sel;
#pragma unroll
                    for (int np = 0; np < 4; ++np) {             // two 8-key pieces at a time
                        const int key = np * 16 + key_in_pair;
                        af_ldmatrix_x4(dst[np], kb + (kk >> 2) * (AP_BN * 128) + key * 128 + ((chunk ^ (key & 7)) << 4));
                    }
                };
                fetch(0, bfr[0]);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    if (kk + 1 < HD / 16) fetch(kk + 1, bfr[(kk + 1) & 1]);
#pragma unroll
                    for (int np = 0; np < 4; ++np) {
                        af_mma(acc[2 * np], qa[kk], bfr[kk & 1][np][0], bfr[kk & 1][np][1]);
                        af_mma(acc[2 * np + 1], qa[kk], bfr[kk & 1][np][2], bfr[kk & 1][np][3]);
                    }
                }
                __syncwarp();
                if (!dry && lane < 4) mbar_arrive(empty(sl));
                if (lane == 0) attn_stamp(11 + 3 * warp);
                const int key0 = (b_first + bl) * AP_BN;
                const int vis_lo = p_first + (r_lo >> gs) - key0, vis_hi = p_first + (r_hi >> gs) - key0;   // columns up to here count
                float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    const int col = nt * 8 + tig * 2;
                    if (r_lo < rows_valid) {
                        float* dst = s_sm + (r_lo * AF_MAX_RUN_BLOCKS + bl) * AF_S_STRIDE + col;
                        dst[0] = acc[nt][0]; dst[1] = acc[nt][1];
                    }
                    if (r_hi < rows_valid) {
                        float* dst = s_sm + (r_hi * AF_MAX_RUN_BLOCKS + bl) * AF_S_STRIDE + col;
                        dst[0] = acc[nt][2]; dst[1] = acc[nt][3];
                    }
                    mx_lo = fmaxf(mx_lo, fmaxf(col > vis_lo ? -INFINITY : acc[nt][0], col + 1 > vis_lo ? -INFINITY : acc[nt][1]));
                    mx_hi = fmaxf(mx_hi, fmaxf(col > vis_hi ? -INFINITY : acc[nt][2], col + 1 > vis_hi ? -INFINITY : acc[nt][3]));
                }
                mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1)); mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
                mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1)); mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
                if (tig == 0) {
                    if (r_lo < rows_valid) mblk_sm[r_lo * AF_MAX_RUN_BLOCKS + bl] = __fmul_rn(mx_lo, a.scale_log2);
                    if (r_hi < rows_valid) mblk_sm[r_hi * AF_MAX_RUN_BLOCKS + bl] = __fmul_rn(mx_hi, a.scale_log2);
                }
                if (lane == 0) attn_stamp(12 + 3 * warp);
            }
        }
        af_bar();
        if (tid == 0) { attn_stamp(3); attn_item_stamp(qn, 1); }

        // ---- B: the softmax of every (row, block), in the order the one-block-after-another kernel has it.
        // A warp per row; in it four threads per block, one for each of the four sums that kernel keeps
        // side by side (scores j, j + 4, j + 8, .. in ascending order), which the first of them adds up as it does.
        for (int t_row = warp; t_row < rows_valid; t_row += 4) {
            const int u = lane & 3, t_bl = lane >> 2;
            const bool live = t_bl < nb;
            const float* s_row = s_sm + (t_row * AF_MAX_RUN_BLOCKS + (live ? t_bl : 0)) * AF_S_STRIDE;
            const int visible = p_first + (t_row >> gs) - (b_first + t_bl) * AP_BN;
            // where the running maximum stands when this block is reached, and whether this block moves it
            float mb[AF_MAX_RUN_BLOCKS];
#pragma unroll
            for (int i = 0; i < AF_MAX_RUN_BLOCKS; ++i) mb[i] = i < nb ? mblk_sm[t_row * AF_MAX_RUN_BLOCKS + i] : -INFINITY;
            float m_ref = -INFINITY, m_before = -INFINITY;
            bool moved = false;
#pragma unroll
            for (int i = 0; i < AF_MAX_RUN_BLOCKS; ++i) {
                if (i <= t_bl) {
                    moved = mb[i] > m_ref + AP_RESCALE_STEP;
                    m_before = m_ref;
                    if (moved) m_ref = mb[i];
                }
            }
            const float alpha = moved ? exp2f(m_before - m_ref) : 1.f;
            const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
            float sum = 0.f;
            __nv_bfloat16* prow = reinterpret_cast<__nv_bfloat16*>(gbase + lay.p_off() + t_row * AF_P_ROW_BYTES);
            // (four scores at a time, read before the four p are written; a short loop: the code stays small)
#pragma unroll 1
            for (int i0 = 0; i0 < AP_BN / 4; i0 += 4) {
                float sc[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) sc[i] = (live && 4 * (i0 + i) + u <= visible) ? s_row[4 * (i0 + i) + u] : -INFINITY;
                __nv_bfloat16 pb[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float pj = ex2_hw(__fmaf_rn(sc[i], a.scale_log2, neg_m));
                    sum = __fadd_rn(sum, pj);
                    pb[i] = __float2bfloat16_rn(pj);
                }
                if (live) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int j = 4 * (i0 + i) + u;
                        const int chunk = t_bl * 8 + (j >> 3);
                        prow[((chunk ^ (t_row & 7)) << 3) + (j & 7)] = pb[i];
                    }
                }
            }
            const float s1 = __shfl_down_sync(0xffffffffu, sum, 1), s2 = __shfl_down_sync(0xffffffffu, sum, 2),
                        s3 = __shfl_down_sync(0xffffffffu, sum, 3);
            const float row_sum = __fadd_rn(__fadd_rn(sum, s1), __fadd_rn(s2, s3));   // (in the first of the four)
            // the run's sum, block after block: l = l * alpha + the block's sum (every lane does it, the first keeps it)
            float al[AF_MAX_RUN_BLOCKS], rs[AF_MAX_RUN_BLOCKS];
#pragma unroll
            for (int i = 0; i < AF_MAX_RUN_BLOCKS; ++i) {
                al[i] = __shfl_sync(0xffffffffu, alpha, 4 * i);
                rs[i] = __shfl_sync(0xffffffffu, row_sum, 4 * i);
            }
            float l = 0.f;
#pragma unroll
            for (int i = 0; i < AF_MAX_RUN_BLOCKS; ++i)
                if (i < nb) l = __fmaf_rn(l, al[i], rs[i]);
            if (live && u == 0) {
                alpha_sm[t_row * AF_MAX_RUN_BLOCKS + t_bl] = alpha;
                if (t_bl == nb - 1) mfin_sm[t_row] = m_ref;
            }
            if (lane == 0) lfin_sm[t_row] = l;
        }
        af_bar();
        if (tid == 0) { attn_stamp(4); attn_item_stamp(qn, 2); }

        // ---- C: O = sum of P . V over the run's blocks; this warp has dims [warp * HD / 4, (warp + 1) * HD / 4)
        float o[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f; }
        {
            const int a_row = a_row_raw < rows_valid ? a_row_raw : rows;   // (the zero row)
            const uint32_t a_row_addr = p_base + a_row * AF_P_ROW_BYTES;
            // Half a block (32 keys) at a time; a half's fragments are asked for before the products of the
            // half before it are issued.
            constexpr int KH = AP_BN / 32;                       // 16-key steps of a half
            int v_slot = pos_slot + nb, v_use = pos_use;         // (the ring's slot and use of the item's first value block)
            while (v_slot >= slots) { v_slot -= slots; ++v_use; }
            uint32_t pa[2][KH][4], vfr[2][KH][NT / 2][4];
            auto fetch = [&](int step, uint32_t (&pd)[KH][4], uint32_t (&vd)[KH][NT / 2][4]) -> bool {
                const int bl = step >> 1, half = step & 1;
                const int sl = v_slot, use = v_use;
                if (half == 1) { v_slot = v_slot + 1 == slots ? 0 : v_slot + 1; v_use += v_slot == 0; }
                uint8_t* vgen = gbase + sl * BLOCK_BYTES;
                const uint32_t vb = base + sl * BLOCK_BYTES;
                if (half == 0) {
                    if (!dry && !mbar_wait(full(sl), use & 1, abort_flag, &g_attn_tc_error)) return false;
                    const int key0 = (b_first + bl) * AP_BN;
                    if (key0 + AP_BN > kv_len) {
                        // rows of V past the sequence's end hold whatever the page held before: this warp zeroes its own dims of them
                        const int first_bad = max(kv_len - key0, 0);
                        constexpr int CH = HD / 32;              // 16-byte pieces of a row that are this warp's
                        for (int idx = lane; idx < (AP_BN - first_bad) * CH; idx += 32) {
                            const int key = first_bad + idx / CH, dd = d_warp + (idx % CH) * 8;
                            const int chunk = (dd & 63) >> 3;
                            *reinterpret_cast<uint4*>(vgen + (dd >> 6) * (AP_BN * 128) + key * 128 + ((chunk ^ (key & 7)) << 4)) = make_uint4(0, 0, 0, 0);
                        }
                        __syncwarp();
                    }
                }
#pragma unroll
                for (int k2 = 0; k2 < KH; ++k2) {
                    const int kk = half * KH + k2;
                    const int chunk = bl * 8 + kk * 2 + a_sel;
                    af_ldmatrix_x4(pd[k2], a_row_addr + ((chunk ^ (a_row & 7)) << 4));
                    const int key = kk * 16 + v_key;
#pragma unroll
                    for (int np = 0; np < NT / 2; ++np) {
                        const int dd = d_warp + np * 16 + v_dsel * 8;
                        const int vchunk = (dd & 63) >> 3;
                        af_ldmatrix_x4_trans(vd[k2][np], vb + (dd >> 6) * (AP_BN * 128) + key * 128 + ((vchunk ^ (key & 7)) << 4));
                    }
                }
                if (half == 1) {
                    __syncwarp();
                    if (!dry && lane == 0) mbar_arrive(empty(sl));   // (the block is in registers)
                }
                return true;
            };
            auto products = [&](int step, const uint32_t (&pd)[KH][4], const uint32_t (&vd)[KH][NT / 2][4]) {
                const int bl = step >> 1;
                if (step >= 2 && (step & 1) == 0) {
                    const float a_lo = r_lo < rows_valid ? alpha_sm[r_lo * AF_MAX_RUN_BLOCKS + bl] : 1.f;
                    const float a_hi = r_hi < rows_valid ? alpha_sm[r_hi * AF_MAX_RUN_BLOCKS + bl] : 1.f;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        o[nt][0] = __fmul_rn(o[nt][0], a_lo); o[nt][1] = __fmul_rn(o[nt][1], a_lo);
                        o[nt][2] = __fmul_rn(o[nt][2], a_hi); o[nt][3] = __fmul_rn(o[nt][3], a_hi);
                    }
                }
#pragma unroll
                for (int k2 = 0; k2 < KH; ++k2) {
#pragma unroll
                    for (int np = 0; np < NT / 2; ++np) {
                        af_mma(o[2 * np], pd[k2], vd[k2][np][0], vd[k2][np][1]);
                        af_mma(o[2 * np + 1], pd[k2], vd[k2][np][2], vd[k2][np][3]);
                    }
                }
            };
            ok = fetch(0, pa[0], vfr[0]);
            for (int step = 0; step < 2 * nb && ok; step += 2) { // (two at a time: the buffers' numbers stay constants)
                ok = fetch(step + 1, pa[1], vfr[1]);
                if (!ok) break;
                products(step, pa[0], vfr[0]);
                if (step + 2 < 2 * nb) ok = fetch(step + 2, pa[0], vfr[0]);
                if (!ok) break;
                products(step + 1, pa[1], vfr[1]);
            }
        }
        if (af_bar_any(!ok)) break;                               // (the runs' l are there; a wait that ran out ends the block)
        if (!dry) {
            pos_slot += 2 * nb;
            while (pos_slot >= slots) { pos_slot -= slots; ++pos_use; }
        }
        if (tid == 0) { attn_stamp(40); attn_item_stamp(qn, 3); }

        // ---- D  (the rehearsal walks it with every store switched off)
        const int rv = dry ? 0 : rows_valid;
        if (n_runs > 1) {
            const int cap = a.rows_cap;
            const size_t part_floats = run_part_floats(cap, HD);
            float* part0 = a.parts + (size_t)(tile * n_hg + hg) * a.max_runs * part_floats;
            float* mine = part0 + (size_t)run * part_floats;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int dd = d_warp + nt * 8 + tig * 2;
                if (r_lo < rv)
                    *reinterpret_cast<float2*>(mine + ((size_t)(dd >> 2) * cap + r_lo) * 4 + (dd & 3)) = make_float2(o[nt][0], o[nt][1]);
                if (r_hi < rv)
                    *reinterpret_cast<float2*>(mine + ((size_t)(dd >> 2) * cap + r_hi) * 4 + (dd & 3)) = make_float2(o[nt][2], o[nt][3]);
            }
            if (tid < rv) reinterpret_cast<float2*>(mine + (size_t)HD * cap)[tid] = make_float2(mfin_sm[tid], lfin_sm[tid]);
            // (the scheduler warp, told through the barrier below, makes this visible, counts the arrival and folds if it was the last)
        } else {
            // the tile's only run: folded onto nothing, then divided by the sum
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = half ? r_hi : r_lo;
                if (r >= rv) continue;
                float M = -INFINITY, L = 0.f, a_, b_;
                fold_coeffs(M, L, mfin_sm[r], lfin_sm[r], a_, b_);
                const float inv = __fdiv_rn(1.0f, L);
                T* orow = a.out + ((size_t)(tok0 + (r >> gs)) * a.n_q + head0 + (r & (gp - 1))) * HD;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int dd = d_warp + nt * 8 + tig * 2;
                    const __nv_bfloat162 pk = __floats2bfloat162_rn(__fmul_rn(fold_value(0.f, a_, o[nt][2 * half], b_), inv),
                                                                    __fmul_rn(fold_value(0.f, a_, o[nt][2 * half + 1], b_), inv));
                    *reinterpret_cast<__nv_bfloat162*>(orow + dd) = pk;
                }
            }
        }
        if (dry) {
            pdl_wait();
            if (tid == 0) attn_item_stamp(0, 5);
            continue;
        }
        __syncwarp();
        if (lane == 0) { mbar_arrive(d_done(qst)); mbar_arrive(q_empty(qst)); }
        if (tid == 0) { attn_stamp(42); attn_item_stamp(qn, 4); }
    }
}

// The ring's depth and the block's shared memory for tiles of `rows` rows: two blocks per SM where the
// ring then still holds six key or value blocks and there are more work items than SMs; else one block
// per SM with a deeper ring (few items: every block has one, and what counts is how much of it is on its
// way at once).
static int attention_few_rows_plan(int hd, int rows, long long items, int n_sm, int* slots_out, int* per_sm_out) {
    AttnFewLayout lay;
    lay.block_bytes = (hd / 64) * AP_BN * 128; lay.rows = rows; lay.slots = 0;
    const int fixed = lay.total();
    const int two_per_sm = (228 * 1024) / 2 - 1024, one_per_sm = 227 * 1024;
    int slots = (two_per_sm - fixed) / lay.block_bytes, per_sm = 2;
    if (slots < 6 || items <= n_sm) { slots = (one_per_sm - fixed) / lay.block_bytes; per_sm = 1; }
    if (slots > AF_MAX_SLOTS) slots = AF_MAX_SLOTS;
    *slots_out = slots; *per_sm_out = per_sm;
    lay.slots = slots;
    return lay.total();
}

static bool attention_few_rows_can(int hd, int rows_cap, int run_blocks, int max_runs, long long groups) {
    return (hd == 64 || hd == 128) && rows_cap <= AF_MAX_ROWS && run_blocks <= AF_MAX_RUN_BLOCKS && max_runs > 0 &&
           groups <= AF_WORK_COUNTER;
}

template <int HD>
static int launch_attention_few_rows(const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcArgs& a, const T* q,
                                     int n_tiles, cudaStream_t stream) {
    static int configured = 0, n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        IDM_REQUIRE(n_sm > 0, "attention_few_rows: no SM count");
    }
    const long long items = (long long)n_tiles * (a.n_q >> a.gp_shift) * a.max_runs;
    IDM_REQUIRE(items < (1ll << 30), "attention_few_rows: %lld work items in one step", items);
    int slots = 0, per_sm = 0;
    const int bytes = attention_few_rows_plan(HD, a.rows_cap, items, n_sm, &slots, &per_sm);
    IDM_REQUIRE(slots >= 4, "attention_few_rows: no room for the ring (%d rows)", a.rows_cap);
    if (configured < bytes) {
        cudaError_t e = cudaFuncSetAttribute(attention_few_rows_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        IDM_REQUIRE(e == cudaSuccess, "attention_few_rows: cannot get %d bytes of shared memory: %s", bytes, cudaGetErrorString(e));
        configured = bytes;
    }
    const int grid = (int)(items < (long long)per_sm * n_sm ? items : (long long)per_sm * n_sm);
    idm_launch(attention_few_rows_kernel<HD>, dim3(grid), dim3(AF_THREADS), (size_t)bytes, stream, mk, mv, a, q, slots, n_tiles);
    IDM_LAUNCH_CHECK("attention_few_rows");
    return 0;
}
