// Causal attention over the paged cache on the tensor cores, for prompts and for single tokens alike.
//
// One kernel serves every step, so that a query's result does not depend on how its sequence was cut
// into steps.  A tile is 128 rows: the `gp` q-heads that share one kv-head, for 128 / gp consecutive
// tokens of one sequence (row = token * gp + head), so keys and values are fetched once per group.
// Keys come in blocks of 64 (one cache page) at absolute positions, fetched by TMA two blocks ahead.
// Per block:
//   S = Q . K^T        tcgen05.mma, both operands in shared memory, S [128 x 64] in tensor memory
//   softmax            one thread per row reads its row of S (tcgen05.ld): scale, causal mask, running
//                      maximum, p = 2^(s - m), running sum -- all 32-bit, no shuffles
//   O += P . V         P written to shared memory as bfloat16 in the MMA's swizzled layout, V read in
//                      place ([keys, head_dim] = MN-major operand); O stays in tensor memory
// The running maximum is only moved when the block's maximum exceeds it by more than 2^8 (then O and
// the sum are rescaled); p and the sum always use the same reference.
//
// Runs.  A row's keys are cut into runs of `run_blocks` key blocks at absolute positions (keys
// [64 R i, 64 R (i + 1))).  Every run starts from nothing (maximum, sum, context) and the runs' results
// (m, l, o) are folded in ascending order with one formula:
//   M' = max(M, m);  a = 2^(M - M'), b = 2^(m - M');  L = L a + l b;  O = O a + o b;   out = O / L.
// A step of few rows (single tokens) gives every run a block of its own; the runs go through scratch
// and the block that finishes last for a tile folds them, whoever it is.  A step of many rows lets one
// block walk a tile's runs and fold as it goes, keeping O in scratch of its own.  Either way a row is the
// same sequence of operations on the same numbers: the same bits (tests compare them).
//
// Masked keys give p = 0 exactly (select, not arithmetic); a row that sees no key of a run leaves that
// run out; rows of V past the sequence's length are zeroed in shared memory before they meet the MMA,
// so stale page contents cannot leak.  Rows of a tile beyond its tokens are not worked on.
// The reference's paths are src/detllm/model.py:382-402 (prompts: query-chunked integer GEMMs) and
// src/detllm/ops/fused_attn.py:47-115 (single tokens: one program per (batch, q-head)).
//
// Roles: warps 0-3 softmax + epilogue (thread = row = tensor-memory lane), warp 4 TMA, warp 5 MMA.
// All mbarrier waits are bounded; a wait that runs out sets the error word (idm_attention_tc_status).
#include "common.cuh"

#if defined(IDM_BF16)

#include "tcgen05.cuh"

#define AP_BM 128
#define AP_BN 64
#define AP_THREADS 192
#define AP_TMEM_COLS 256
#define AP_RESCALE_STEP 8.0f
#define AP_COUNTERS 65536           // arrival counters at the start of the scratch: one per (tile, head group)

__device__ int g_attn_tc_error = 0;

// -DIDM_TRACE: block (0, 0) leaves nanosecond stamps of its stages (a measuring aid, compiled out otherwise)
#if defined(IDM_TRACE)
__device__ unsigned long long g_attn_trace[64];
__device__ __forceinline__ void attn_stamp(int i) {
    if (blockIdx.x == 0 && blockIdx.y == 0 && i < 64) { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); g_attn_trace[i] = t; }
}
extern "C" int idm_attention_tc_trace_read(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_attn_trace, sizeof(unsigned long long) * 64);
}
// every block of the few-rows kernel: [block][item it worked on, up to 4][stamp]
__device__ unsigned long long g_attn_item_trace[512][4][8];
__device__ __forceinline__ void attn_item_stamp(int nth, int i) {
    if (blockIdx.x < 512 && nth >= 0 && nth < 4) { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); g_attn_item_trace[blockIdx.x][nth][i] = t; }
}
extern "C" int idm_attention_item_trace_read(unsigned long long* out, int clear) {
    if (clear) return (int)cudaMemcpyToSymbol(g_attn_item_trace, out, sizeof(unsigned long long) * 512 * 4 * 8);
    return (int)cudaMemcpyFromSymbol(out, g_attn_item_trace, sizeof(unsigned long long) * 512 * 4 * 8);
}
#else
__device__ __forceinline__ void attn_stamp(int) {}
__device__ __forceinline__ void attn_item_stamp(int, int) {}
#endif

struct AttnTcArgs {
    T* out;
    const int* tile_seq; const int* tile_start;
    const int* cu_q; const int* q_start; const int* kv_len; const int* slots;
    const int* table; int table_stride;
    int n_q, n_kv;
    int gp_shift;                                      // log2 of the q-heads that share a tile's rows
    float scale_log2;
    int run_blocks;                                    // key blocks of a run
    int max_runs;                                      // > 0: every run has a block of its own (grid.x = head groups x max_runs); 0: one block walks a tile's runs
    int rows_cap;                                      // the most rows any tile of the step has: what is fetched of q, and what the scratch holds of a run
    // one block per tile, but tiles with many key blocks shared by several: block `part` of a tile walks the runs
    // [part * runs_per_part, + runs_per_part) and leaves each run's result in the pool; the last to arrive folds
    const int* tile_pool;                              // per tile: its first slot in the pool (head group g: + g x its runs), or -1: one block has it alone
    int max_parts, runs_per_part;                      // max_parts == 0: no tile is shared
    float* pool;                                       // slots of rows_cap * (HD + 2) floats
    int* counters;                                     // [n_tiles * head groups] arrivals, zero between launches
    float* parts;                                      // runs through scratch: [n_tiles * head groups, max_runs] of rows_cap * (HD + 2) floats;
                                                       // one block per tile: [n_tiles * head groups] of 128 * HD floats (the context so far)
};

template <int HD>
struct AttnTcSmem {
    static constexpr int HT = HD / 64;                 // 64-wide tiles along head_dim
    static constexpr int Q_BYTES = HT * AP_BM * 128;
    static constexpr int K_BYTES = HT * AP_BN * 128;   // per stage, two stages
    static constexpr int V_BYTES = HT * AP_BN * 128;   // per stage, two stages
    static constexpr int P_BYTES = AP_BM * 128;
    static constexpr int Q_OFF = 0, K_OFF = Q_BYTES, V_OFF = K_OFF + 2 * K_BYTES, P_OFF = V_OFF + 2 * V_BYTES;
    static constexpr int BAR_OFF = P_OFF + P_BYTES;
    static constexpr int NEED = BAR_OFF + 256;         // from the first 1024-byte border on
    // two blocks per SM: 2 x (TOTAL + 1 KB the system keeps per block) must stay within 228 KB, which
    // leaves 512 bytes to reach the border (the array is declared with that alignment; the kernel checks)
    static constexpr int TOTAL = NEED + (HD == 128 ? 512 : 1024);
};

// One step of the fold of a run's (m, l) into the row's (M, L); a, b: what the contexts are scaled by.
// A run (or a start) without a key has m = -inf and drops out exactly.
__device__ __forceinline__ void fold_coeffs(float& M, float& L, float m, float l, float& a_, float& b_) {
    const float M_new = fmaxf(M, m);
    a_ = (M == -INFINITY) ? 0.f : exp2f(M - M_new);
    b_ = (m == -INFINITY) ? 0.f : exp2f(m - M_new);
    L = __fmaf_rn(L, a_, __fmul_rn(l, b_));
    M = M_new;
}
__device__ __forceinline__ float fold_value(float o_tot, float a_, float o_run, float b_) {
    return __fmaf_rn(o_tot, a_, __fmul_rn(o_run, b_));
}

// 16 finished values of a row as bfloat16: 32 bytes, two stores
__device__ __forceinline__ void store_out16(T* dst, const float (&o)[16], float inv) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const __nv_bfloat162 pk = __floats2bfloat162_rn(__fmul_rn(o[2 * i], inv), __fmul_rn(o[2 * i + 1], inv));
        w[i] = *reinterpret_cast<const uint32_t*>(&pk);
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
}

// Where run `run` of a tile and head group leaves its result: rows_cap rows of (HD + 2) floats, as
// [HD / 4][rows_cap] pieces of four dims and then [rows_cap] pairs (m, l).
__device__ __forceinline__ size_t run_part_floats(int rows_cap, int hd) {
    return ((size_t)rows_cap * (hd + 2) + 3) & ~(size_t)3;       // (16-byte pieces)
}

// All runs of a tile and head group folded in the order of the runs, divided by the sum, written to
// the output rows; `n_threads` threads (r = 0 .. n_threads - 1) share the tile's (row, two dims) pieces.
#define FOLD_BATCH 8
template <int HD>
__device__ __forceinline__ void fold_runs_and_store(const AttnTcArgs& a, const float* part0, size_t part_floats, int n_runs,
                                                    int rows_valid, int tok0, int head0, int r, int n_threads) {
    const int cap = a.rows_cap, gs = a.gp_shift, gp = 1 << gs;
    for (int w = r; w < (HD / 2) * cap; w += n_threads) {
        const int half = w & 1, row = (w >> 1) % cap, c4 = (w >> 1) / cap;
        if (row >= rows_valid) continue;
        const size_t at = ((size_t)c4 * cap + row) * 4 + 2 * half;
        float M = -INFINITY, L = 0.f;
        float2 acc = make_float2(0.f, 0.f);
        for (int i0 = 0; i0 < n_runs; i0 += FOLD_BATCH) {          // so many runs' loads are in flight together; the fold is a chain
            float2 ml[FOLD_BATCH], o[FOLD_BATCH];
#pragma unroll
            for (int u = 0; u < FOLD_BATCH; ++u) {
                if (i0 + u < n_runs) {
                    const float* pi = part0 + (size_t)(i0 + u) * part_floats;
                    ml[u] = __ldcg(reinterpret_cast<const float2*>(pi + (size_t)HD * cap) + row);
                    o[u] = __ldcg(reinterpret_cast<const float2*>(pi + at));
                }
            }
#pragma unroll
            for (int u = 0; u < FOLD_BATCH; ++u) {
                if (i0 + u < n_runs) {
                    float a_, b_;
                    fold_coeffs(M, L, ml[u].x, ml[u].y, a_, b_);
                    acc.x = fold_value(acc.x, a_, o[u].x, b_); acc.y = fold_value(acc.y, a_, o[u].y, b_);
                }
            }
        }
        const float inv = __fdiv_rn(1.0f, L);
        T* dst = a.out + ((size_t)(tok0 + (row >> gs)) * a.n_q + head0 + (row & (gp - 1))) * HD + c4 * 4 + 2 * half;
        *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(__fmul_rn(acc.x, inv), __fmul_rn(acc.y, inv));
    }
}

// The same fold for tiles of many rows: a thread per row (r = 0 .. 127), 16 dims at a time with four runs' loads in
// flight, so that the loads of a warp are whole lines and a row's (m, l) chain is walked by one thread.  The same
// operations in the same order as above: the same bits.
template <int HD>
__device__ __forceinline__ void fold_rows_and_store(const AttnTcArgs& a, const float* part0, size_t part_floats, int n_runs,
                                                    int rows_valid, int tok0, int head0, int r) {
    const int cap = a.rows_cap, gs = a.gp_shift, gp = 1 << gs;
    if (r >= rows_valid) return;
    T* dst = a.out + ((size_t)(tok0 + (r >> gs)) * a.n_q + head0 + (r & (gp - 1))) * HD;
#pragma unroll 1
    for (int c = 0; c < HD; c += 16) {
        float M = -INFINITY, L = 0.f;
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
#pragma unroll 1
        for (int i0 = 0; i0 < n_runs; i0 += 4) {
            float2 ml[4];
            float4 o[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (i0 + u < n_runs) {
                    const float* pi = part0 + (size_t)(i0 + u) * part_floats;
                    ml[u] = __ldcg(reinterpret_cast<const float2*>(pi + (size_t)HD * cap) + r);
#pragma unroll
                    for (int k = 0; k < 4; ++k) o[u][k] = __ldcg(reinterpret_cast<const float4*>(pi) + (size_t)(c / 4 + k) * cap + r);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (i0 + u < n_runs) {
                    float a_, b_;
                    fold_coeffs(M, L, ml[u].x, ml[u].y, a_, b_);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        acc[4 * k] = fold_value(acc[4 * k], a_, o[u][k].x, b_); acc[4 * k + 1] = fold_value(acc[4 * k + 1], a_, o[u][k].y, b_);
                        acc[4 * k + 2] = fold_value(acc[4 * k + 2], a_, o[u][k].z, b_); acc[4 * k + 3] = fold_value(acc[4 * k + 3], a_, o[u][k].w, b_);
                    }
                }
            }
        }
        store_out16(dst + c, acc, __fdiv_rn(1.0f, L));
    }
}

// The end of a block that has written its run's result to scratch, called by its 128 row threads
// (r = 0 .. 127; named barrier 1): the arrival is counted, and the block that comes last for the tile
// and head group folds all runs, whoever it is.  (A block whose wait ran out, ok == false, still counts:
// the error is reported, the result is wrong, and nobody waits for anybody for ever.)
template <int HD>
__device__ __forceinline__ void count_and_fold_runs(const AttnTcArgs& a, const float* part0, size_t part_floats, int n_runs,
                                                    int n_arrivals, int rows_valid, int tok0, int head0, int counter_index,
                                                    volatile int* last_flag, int r, bool ok) {
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (r == 0) {
        int* counter = a.counters + counter_index;
        const int is_last = atomicAdd(counter, 1) == n_arrivals - 1;
        if (is_last) *counter = 0;                                 // ready for the next launch
        *last_flag = is_last;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (!*last_flag || !ok) return;
    __threadfence();
    if (a.rows_cap > 32) fold_rows_and_store<HD>(a, part0, part_floats, n_runs, rows_valid, tok0, head0, r);
    else fold_runs_and_store<HD>(a, part0, part_floats, n_runs, rows_valid, tok0, head0, r, 128);
}

#include "attention_few_rows.cuh"

template <int HD>
__global__ void __launch_bounds__(AP_THREADS, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, AttnTcArgs a) {
    using S = AttnTcSmem<HD>;
    constexpr int HT = S::HT;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    if (base - smem_u32(smem_raw) + S::NEED > S::TOTAL) {        // (never seen: the array starts on a 1024-byte border)
        if (threadIdx.x == 0) atomicExch(&g_attn_tc_error, 2);
        return;
    }
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + S::BAR_OFF;
    // barriers (8 bytes each)
    const uint32_t q_full = bars, p_full = bars + 40, o_done = bars + 48;
    auto k_full = [&](int i) { return bars + 8 + 8u * i; };
    auto k_empty = [&](int i) { return bars + 24 + 8u * i; };
    auto v_full = [&](int i) { return bars + 56 + 8u * i; };
    auto v_empty = [&](int i) { return bars + 72 + 8u * i; };
    auto s_full = [&](int i) { return bars + 88 + 8u * i; };
    auto s_empty = [&](int i) { return bars + 104 + 8u * i; };
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gbase + S::BAR_OFF + 120);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    if (threadIdx.x == 0) attn_stamp(0);                         // block started

    // blocks start in this order: all head groups (and runs) of the longest tile first.  What is read
    // here was written before the step began, not by the kernel before this one.
    const bool through_scratch = a.max_runs > 0;
    const bool parted = !through_scratch && a.max_parts > 0;
    const int tile = blockIdx.y;
    const int hg = through_scratch ? blockIdx.x / a.max_runs : parted ? blockIdx.x / a.max_parts : blockIdx.x;
    const int run = through_scratch ? blockIdx.x % a.max_runs : 0;
    const int part = parted ? blockIdx.x % a.max_parts : 0;
    const int gs = a.gp_shift, gp = 1 << gs;
    const int seq = a.tile_seq[tile], tstart = a.tile_start[tile];
    const int head0 = hg << gs;                                  // the tile's first q-head
    const int g = head0 / (a.n_q / a.n_kv);                      // its kv-head
    const int tok0 = a.cu_q[seq] + tstart;                       // first token (packed row) of the tile
    const int q_len = a.cu_q[seq + 1] - a.cu_q[seq];
    const int toks_valid = min(AP_BM >> gs, q_len - tstart);
    const int rows_valid = toks_valid << gs;
    const int p_first = a.q_start[seq] + tstart;                 // position of row 0
    const int p_last = p_first + toks_valid - 1;
    const int kv_len = a.kv_len[seq];
    const int nb_tile = p_last / AP_BN + 1;                      // the tile's key blocks 0 .. nb_tile-1
    const int R = a.run_blocks;
    const int n_runs = (nb_tile + R - 1) / R;
    if (through_scratch && run >= n_runs) return;                // (the whole block, before anything is set up)
    const int pool_at = parted ? a.tile_pool[tile] : -1;
    const int n_parts = pool_at >= 0 ? (n_runs + a.runs_per_part - 1) / a.runs_per_part : 1;
    if (part >= n_parts) return;
    const bool shared = n_parts > 1;                             // this tile's runs go through the pool, several blocks walk them
    // this block's key blocks b_first .. b_first + nb - 1
    const int b_first = through_scratch ? run * R : shared ? part * a.runs_per_part * R : 0;
    const int nb = through_scratch ? min(R, nb_tile - b_first) : shared ? min(a.runs_per_part * R, nb_tile - b_first) : nb_tile;
    const int n_hg = a.n_q >> gs;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1); mbar_init(p_full, 4); mbar_init(o_done, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full(i), 1); mbar_init(k_empty(i), 1);
            mbar_init(v_full(i), 1); mbar_init(v_empty(i), 1); mbar_init(s_full(i), 1); mbar_init(s_empty(i), 4);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 5) tmem_alloc(smem_u32((const void*)tmem_slot), AP_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_o = tmem + 128;                          // S buffers at columns 0 and 64, O from 128
    pdl_wait();                                                  // set-up done; now the previous kernel's results
    if (threadIdx.x == 0) attn_stamp(1);                         // set-up done, the kernel before too

    // from here on b counts this block's own key blocks (buffers and barrier phases go by it); the block's
    // place among the sequence's keys is b_first + b, and a run starts wherever that is a multiple of R
    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer
        // (the whole warp walks the loop: its lanes fetch the page numbers of 32 key blocks at a time, so that
        // no request waits for a look-up of its own; lane 0 issues the requests)
        if (lane == 0) {
            // (only the rows that some tile of the step has are fetched; the rest of the tile is whatever was there,
            // makes rows of scores nobody reads, and gets p = 0)
            mbar_expect_tx(q_full, (uint32_t)(HT * a.rows_cap * 128));
            for (int h = 0; h < HT; ++h)
                tma_load_3d(base + S::Q_OFF + h * AP_BM * 128, &map_q, h * 64, head0, tok0, q_full);
        }
        const int* pages = a.table + (size_t)a.slots[seq] * a.table_stride + b_first;
        int my_page = 0;
        for (int b = 0; b < nb; ++b) {
            if ((b & 31) == 0) my_page = b + lane < nb ? pages[b + lane] : 0;
            const int page = __shfl_sync(0xffffffffu, my_page, b & 31);
            const int row = (page * a.n_kv + g) * IDM_PAGE;
            const int vb = b & 1;                                // this block's key and value buffers
            bool ok = true;
            if (lane == 0) {
                ok = b < 2 || mbar_wait(k_empty(vb), ((b >> 1) - 1) & 1, abort_flag, &g_attn_tc_error);
                if (ok) {
                    mbar_expect_tx(k_full(vb), S::K_BYTES);
                    for (int h = 0; h < HT; ++h)
                        tma_load_2d(base + S::K_OFF + vb * S::K_BYTES + h * AP_BN * 128, &map_k, h * 64, row, k_full(vb));
                    ok = b < 2 || mbar_wait(v_empty(vb), ((b >> 1) - 1) & 1, abort_flag, &g_attn_tc_error);
                }
                if (ok) {
                    mbar_expect_tx(v_full(vb), S::V_BYTES);
                    for (int h = 0; h < HT; ++h)
                        tma_load_2d(base + S::V_OFF + vb * S::V_BYTES + h * AP_BN * 128, &map_v, h * 64, row, v_full(vb));
                }
            }
            if (!__shfl_sync(0xffffffffu, (int)ok, 0)) break;
        }
    } else if (warp == 5) {
        // -------------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc(AP_BM, AP_BN);
            constexpr uint32_t idesc_o = umma_idesc(AP_BM, HD, true);
            auto mma_s = [&](int b) {                            // S[b % 2] = Q . K_b^T
                const uint32_t d = tmem + (uint32_t)(b & 1) * AP_BN;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint64_t ad = umma_desc_kmajor(base + S::Q_OFF + (kk / 4) * AP_BM * 128) + 2 * (kk % 4);
                    const uint64_t bd = umma_desc_kmajor(base + S::K_OFF + (b & 1) * S::K_BYTES + (kk / 4) * AP_BN * 128) + 2 * (kk % 4);
                    tc_mma_bf16(d, ad, bd, idesc_s, kk > 0 ? 1u : 0u);
                }
                tc_commit(s_full(b & 1));
                tc_commit(k_empty(b & 1));
            };
            bool ok = mbar_wait(q_full, 0, abort_flag, &g_attn_tc_error) &&
                      mbar_wait(k_full(0), 0, abort_flag, &g_attn_tc_error);
            if (ok) { tc_fence_after(); mma_s(0); }
            for (int b = 0; b < nb && ok; ++b) {
                if (b + 1 < nb) {
                    ok = mbar_wait(k_full((b + 1) & 1), ((b + 1) >> 1) & 1, abort_flag, &g_attn_tc_error);
                    if (ok && b + 1 >= 2)
                        ok = mbar_wait(s_empty((b + 1) & 1), (((b + 1) >> 1) - 1) & 1, abort_flag, &g_attn_tc_error);
                    if (!ok) break;
                    tc_fence_after();
                    mma_s(b + 1);
                }
                ok = mbar_wait(p_full, b & 1, abort_flag, &g_attn_tc_error) &&
                     mbar_wait(v_full(b & 1), (b >> 1) & 1, abort_flag, &g_attn_tc_error);
                if (!ok) break;
                tc_fence_after();
                const uint32_t vbase = base + S::V_OFF + (b & 1) * S::V_BYTES;
                const bool fresh = (b_first + b) % R == 0;       // a run's first block starts its context from nothing
#pragma unroll
                for (int kk = 0; kk < AP_BN / 16; ++kk) {        // O (+)= P . V_b
                    const uint64_t ad = umma_desc_kmajor(base + S::P_OFF) + 2 * kk;
                    const uint64_t bd = umma_desc_mnmajor(vbase + kk * 16 * 128, AP_BN * 128);
                    tc_mma_bf16(tmem_o, ad, bd, idesc_o, (!fresh || kk > 0) ? 1u : 0u);
                }
                tc_commit(o_done);
                tc_commit(v_empty(b & 1));
            }
        }
    } else {
        // ------------------------------------------------- softmax and epilogue (warps 0-3)
        const int r = warp * 32 + lane;                          // row = tensor-memory lane
        const bool row_live = r < rows_valid;
        const bool warp_live = warp * 32 < rows_valid;           // (a warp without rows keeps the barriers' count and no more)
        const int p_r = p_first + (r >> gs);
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        uint8_t* prow = gbase + S::P_OFF + r * 128;
        if (!row_live) {
            // the row's P stays zero: its part of O is never read, and nothing undefined meets the MMA
#pragma unroll
            for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(prow + (c << 4)) = make_uint4(0, 0, 0, 0);
        }
        // one block per tile, more than one run: the row's context so far lives in scratch of this block's own
        float* tot = (!through_scratch && !shared && n_runs > 1) ? a.parts + (size_t)(tile * n_hg + hg) * (AP_BM * HD) : nullptr;
        // where the runs of this tile and head group leave their results (a block per run, or a tile shared by several blocks)
        const int cap = a.rows_cap;
        const size_t part_floats = run_part_floats(cap, HD);
        float* part0 = through_scratch ? a.parts + (size_t)(tile * n_hg + hg) * a.max_runs * part_floats
                                       : shared ? a.pool + ((size_t)pool_at + (size_t)hg * n_runs) * part_floats : nullptr;
        // a finished run's (m, l) and context, from tensor memory to its slot (64 columns are asked for before the first is waited for)
        auto leave_run = [&](int which, float m_run, float l_run) {
            float4* mine = reinterpret_cast<float4*>(part0 + (size_t)which * part_floats);
#pragma unroll 1
            for (int c = 0; c < HD; c += 64) {
                uint32_t o[64];
#pragma unroll
                for (int u = 0; u < 64; u += 16) tc_ld16_issue(tmem_o + lane_base + c + u, o + u);
                tc_ld_wait();
                if (r < cap) {
#pragma unroll
                    for (int k = 0; k < 16; ++k)
                        mine[(c / 4 + k) * cap + r] = make_float4(__uint_as_float(o[4 * k]), __uint_as_float(o[4 * k + 1]),
                                                                  __uint_as_float(o[4 * k + 2]), __uint_as_float(o[4 * k + 3]));
                }
            }
            if (r < cap) reinterpret_cast<float2*>(part0 + (size_t)which * part_floats + (size_t)HD * cap)[r] = make_float2(m_run, l_run);
        };
        float m_ref = -INFINITY, l = 0.f;                        // the current run
        float M_tot = -INFINITY, L_tot = 0.f;                    // the runs folded so far
        bool ok = true;
        for (int b = 0; b < nb && ok; ++b) {
            ok = mbar_wait(s_full(b & 1), (b >> 1) & 1, abort_flag, &g_attn_tc_error);
            if (!ok) break;
            if (threadIdx.x == 0) attn_stamp(2 + 2 * b);         // scores of block b are there
            tc_fence_after();
            const bool run_start = b > 0 && (b_first + b) % R == 0;
            float m_prev = 0.f, l_prev = 0.f;
            if (run_start) { m_prev = m_ref; l_prev = l; m_ref = -INFINITY; l = 0.f; }
            uint32_t sr[AP_BN];
            if (warp_live) {
                tc_ld32_issue(tmem + lane_base + (uint32_t)(b & 1) * AP_BN, sr);
                tc_ld32_issue(tmem + lane_base + (uint32_t)(b & 1) * AP_BN + 32, sr + 32);
                tc_ld_wait();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty(b & 1));
            const int key0 = (b_first + b) * AP_BN;               // position of the block's first key
            float alpha = 1.f, row_sum = 0.f;
            uint32_t packed[AP_BN / 2];
            if (row_live) {
                const bool diagonal = key0 + AP_BN - 1 > p_first; // some key of the block lies past row 0's position
                if (diagonal) {
#pragma unroll
                    for (int j = 0; j < AP_BN; ++j)
                        if (key0 + j > p_r) sr[j] = 0xff800000u;  // -inf: p becomes 0 exactly
                }
                // the maximum of the raw scores (the scale is positive), four chains side by side
                // (the three-input maximum of sm_100: two scores per instruction)
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < AP_BN; j += 8) {
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        mx[u] = max3(mx[u], __uint_as_float(sr[j + 2 * u]), __uint_as_float(sr[j + 2 * u + 1]));
                }
                const float m_blk = __fmul_rn(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), a.scale_log2);
                if (m_blk > m_ref + AP_RESCALE_STEP) {             // (never for a block without a visible key: -inf)
                    alpha = exp2f(m_ref - m_blk);                  // 0 at a run's first visible key
                    m_ref = m_blk;
                }
                // p = 2^(s * scale - m_ref): one fused multiply-add and one exponential per score; before the
                // run's first visible key every score is -inf and p = 2^(-inf) = 0
                const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
                float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int j = 0; j < AP_BN; j += 4) {
                    const float p0 = ex2_hw(__fmaf_rn(__uint_as_float(sr[j]), a.scale_log2, neg_m));
                    const float p1 = ex2_hw(__fmaf_rn(__uint_as_float(sr[j + 1]), a.scale_log2, neg_m));
                    const float p2 = ex2_hw(__fmaf_rn(__uint_as_float(sr[j + 2]), a.scale_log2, neg_m));
                    const float p3 = ex2_hw(__fmaf_rn(__uint_as_float(sr[j + 3]), a.scale_log2, neg_m));
                    sum4[0] = __fadd_rn(sum4[0], p0); sum4[1] = __fadd_rn(sum4[1], p1);
                    sum4[2] = __fadd_rn(sum4[2], p2); sum4[3] = __fadd_rn(sum4[3], p3);
                    const __nv_bfloat162 pa = __floats2bfloat162_rn(p0, p1), pb = __floats2bfloat162_rn(p2, p3);
                    packed[j / 2] = *reinterpret_cast<const uint32_t*>(&pa);
                    packed[j / 2 + 1] = *reinterpret_cast<const uint32_t*>(&pb);
                }
                row_sum = __fadd_rn(__fadd_rn(sum4[0], sum4[1]), __fadd_rn(sum4[2], sum4[3]));
            }
            if (b >= 1) {
                ok = mbar_wait(o_done, (b - 1) & 1, abort_flag, &g_attn_tc_error);   // P is free, O is settled
                if (!ok) break;
                tc_fence_after();
                if (run_start && shared) {
                    // the run before this block is complete: its result goes to its slot (the MMA that starts the
                    // new run's context overwrites O only after this warp's arrival below)
                    if (warp_live) leave_run((b_first + b) / R - 1, m_prev, l_prev);
                } else if (run_start) {
                    // the run before this block is complete: fold it into the row's context so far (the MMA
                    // that starts the new run's context overwrites O only after this warp's arrival below)
                    if (warp_live) {
                        float a_, b_;
                        const bool first = (b_first + b) == R;     // it was the tile's first run: nothing to add to
                        fold_coeffs(M_tot, L_tot, m_prev, l_prev, a_, b_);
                        float4* mine = reinterpret_cast<float4*>(tot);
#pragma unroll 1
                        for (int c = 0; c < HD; c += 32) {           // 32 columns and their old values are asked for together
                            uint32_t o[32];
                            float4 t[8];
                            tc_ld16_issue(tmem_o + lane_base + c, o);
                            tc_ld16_issue(tmem_o + lane_base + c + 16, o + 16);
#pragma unroll
                            for (int k = 0; k < 8; ++k)
                                t[k] = (row_live && !first) ? mine[(c / 4 + k) * AP_BM + r] : make_float4(0.f, 0.f, 0.f, 0.f);
                            tc_ld_wait();
                            if (row_live) {
#pragma unroll
                                for (int k = 0; k < 8; ++k) {
                                    t[k].x = fold_value(t[k].x, a_, __uint_as_float(o[4 * k]), b_);
                                    t[k].y = fold_value(t[k].y, a_, __uint_as_float(o[4 * k + 1]), b_);
                                    t[k].z = fold_value(t[k].z, a_, __uint_as_float(o[4 * k + 2]), b_);
                                    t[k].w = fold_value(t[k].w, a_, __uint_as_float(o[4 * k + 3]), b_);
                                    mine[(c / 4 + k) * AP_BM + r] = t[k];
                                }
                            }
                        }
                    }
                } else if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
                    for (int c = 0; c < HD; c += 16) {
                        uint32_t o[16];
                        tc_ld16_issue(tmem_o + lane_base + c, o);
                        tc_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__fmul_rn(__uint_as_float(o[i]), alpha));
                        tc_st16(tmem_o + lane_base + c, o);
                    }
                    tc_st_wait();
                }
            }
            l = __fmaf_rn(l, alpha, row_sum);
            if (row_live) {
                // P row: 8 chunks of 16 bytes, chunk c stored at (c ^ (row & 7)) -- the 128-byte swizzle
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) =
                        make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
                }
            }
            // rows of V past the sequence's end hold whatever the page held before: zero them
            if (key0 + AP_BN > kv_len) {
                ok = mbar_wait(v_full(b & 1), (b >> 1) & 1, abort_flag, &g_attn_tc_error);
                if (!ok) break;
                const int first_bad = kv_len - key0;               // >= 1
                uint8_t* vb = gbase + S::V_OFF + (b & 1) * S::V_BYTES;
                for (int idx = r; idx < (AP_BN - first_bad) * HT * 8; idx += AP_BM) {
                    const int chunk = idx % 8, rest = idx / 8;
                    const int row = first_bad + rest % (AP_BN - first_bad), h = rest / (AP_BN - first_bad);
                    *reinterpret_cast<uint4*>(vb + h * AP_BN * 128 + row * 128 + chunk * 16) = make_uint4(0, 0, 0, 0);
                }
            }
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
            if (threadIdx.x == 0) attn_stamp(3 + 2 * b);         // p of block b handed over
        }
        if (ok) ok = mbar_wait(o_done, (nb - 1) & 1, abort_flag, &g_attn_tc_error);
        ok = __all_sync(0xffffffffu, ok);                          // (one answer per warp for what follows)
        if (threadIdx.x == 0) attn_stamp(40);                    // the last context is complete
        T* orow = a.out + ((size_t)(tok0 + (r >> gs)) * a.n_q + head0 + (r & (gp - 1))) * HD;
        if ((through_scratch || shared) && n_runs > 1) {
            // This block's (last) run's result goes to its place among the tile's; the block that comes last
            // folds them all, in the order of the runs whoever it is.  (A warp whose wait ran out skips the
            // work but not the two barriers and the count: the error is reported, the result is wrong, and
            // nobody waits for anybody for ever.)
            if (ok && warp_live) {
                tc_fence_after();
                leave_run(through_scratch ? run : (b_first + nb - 1) / R, m_ref, l);
                __threadfence();
            }
            count_and_fold_runs<HD>(a, part0, part_floats, n_runs, through_scratch ? n_runs : n_parts, rows_valid, tok0, head0,
                                    tile * n_hg + hg, (volatile int*)(gbase + S::BAR_OFF + 128), r, ok);
            if (threadIdx.x == 0) attn_stamp(41);                // this run's result is in scratch, counted, and folded if it was the last
        } else if (ok && warp_live) {
            // the last (or only) run folded onto what came before, then divided by the sum
            tc_fence_after();
            float a_, b_;
            const bool first = tot == nullptr;
            fold_coeffs(M_tot, L_tot, m_ref, l, a_, b_);
            const float inv = __fdiv_rn(1.0f, L_tot);
            const float4* mine = reinterpret_cast<const float4*>(tot);
#pragma unroll 1
            for (int c = 0; c < HD; c += 16) {
                float o[16];
                tc_ld16(tmem_o + lane_base + c, o);
                if (row_live) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (!first) t = mine[(c / 4 + k) * AP_BM + r];
                        o[4 * k] = fold_value(t.x, a_, o[4 * k], b_); o[4 * k + 1] = fold_value(t.y, a_, o[4 * k + 1], b_);
                        o[4 * k + 2] = fold_value(t.z, a_, o[4 * k + 2], b_); o[4 * k + 3] = fold_value(t.w, a_, o[4 * k + 3], b_);
                    }
                    store_out16(orow + c, o, inv);
                }
            }
        }
    }
    if (threadIdx.x == 0) attn_stamp(42);                        // done
    tc_fence_before();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem, AP_TMEM_COLS);
}

template <int HD>
static int launch_attention_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcArgs& a,
                               int n_tiles, cudaStream_t stream) {
    using S = AttnTcSmem<HD>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        IDM_REQUIRE(e == cudaSuccess, "attention_tc: cannot get %d bytes of shared memory: %s", S::TOTAL,
                    cudaGetErrorString(e));
        configured = true;
    }
    const int n_hg = a.n_q >> a.gp_shift;
    dim3 grid(n_hg * (a.max_runs > 0 ? a.max_runs : a.max_parts > 0 ? a.max_parts : 1), n_tiles);
    idm_launch(attention_tc_kernel<HD>, dim3(grid), dim3(AP_THREADS), S::TOTAL, stream, mq, mk, mv, a);
    IDM_LAUNCH_CHECK("attention_tc");
    return 0;
}

static int g_attn_few_rows = 1;

extern "C" int idm_attention_tc_supports(int hd) { return hd == 64 || hd == 128; }

// How many q-heads share a tile's rows: the largest power of two up to 16 that divides the group
// (q-heads per kv-head).  A tile then holds 128 / that many tokens.
extern "C" int idm_attention_tc_heads_per_tile(int n_q, int n_kv) {
    if (n_kv <= 0 || n_q % n_kv) return 1;
    const int group = n_q / n_kv;
    int gp = 1;
    while (gp < 16 && group % (gp * 2) == 0) gp *= 2;
    return gp;
}

// Floats of scratch: arrival counters (zero at the first launch, left at zero by every launch), then
// either the runs' results (max_runs > 0: rows_cap rows of every run of every tile and head group) or
// one context per tile and head group (max_runs == 0).
extern "C" long long idm_attention_tc_scratch_floats(int n_tiles, int n_q, int n_kv, int hd, int max_runs, int rows_cap) {
    const long long groups = (long long)n_tiles * (n_q / idm_attention_tc_heads_per_tile(n_q, n_kv));
    if (max_runs > 0) return (long long)AP_COUNTERS + groups * max_runs * (((long long)rows_cap * (hd + 2) + 3) / 4 * 4);
    return (long long)AP_COUNTERS + groups * AP_BM * hd;
}

// q [n_tokens, n_q, hd]; out [n_tokens, n_q * hd]; the cache entry's pools [n_pages, n_kv, 64, hd];
// tiles: (sequence, first token of the tile within the sequence's tokens of this step), a tile being
// 128 / heads_per_tile tokens, longest first; rows_cap: the most rows (tokens x heads_per_tile) any tile has.  max_runs > 0: every run of `run_blocks` key blocks is a
// block of its own and results meet in scratch; max_runs == 0:
// one block per tile and head group (`scratch` may be null if no tile has more than run_blocks key blocks).
extern "C" int idm_attention_tc(const void* q, void* out, const void* k_pool, const void* v_pool, int n_pages,
                                const int* table, int table_stride, const int* tile_seq, const int* tile_start,
                                int n_tiles, const int* cu_q, const int* q_start, const int* kv_len,
                                const int* slots, int n_tokens, int n_q, int n_kv, int hd, float scale,
                                int run_blocks, int max_runs, int rows_cap, float* scratch, const int* tile_pool,
                                int max_parts, int runs_per_part, cudaStream_t stream) {
    // (tile_pool / max_parts / runs_per_part, with max_runs == 0: tiles whose entry in tile_pool is not -1 are shared
    // by up to max_parts blocks of runs_per_part runs each; their runs' results lie in the scratch behind the
    // one-context-per-tile region, from the slot tile_pool names on, head group after head group)
    if (n_tiles == 0 || n_tokens == 0) return 0;
    IDM_REQUIRE(idm_attention_tc_supports(hd), "attention_tc: head_dim=%d has no kernel here", hd);
    IDM_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "attention_tc: bad head counts %d/%d", n_q, n_kv);
    IDM_REQUIRE(n_tiles <= 65535, "attention_tc: %d tiles in one step; at most 65535", n_tiles);
    IDM_REQUIRE(run_blocks >= 1, "attention_tc: a run has at least one key block, not %d", run_blocks);
    const int gp = idm_attention_tc_heads_per_tile(n_q, n_kv);
    int gs = 0;
    while ((1 << gs) < gp) ++gs;
    const long long groups = (long long)n_tiles * (n_q / gp);
    IDM_REQUIRE(rows_cap >= gp && rows_cap <= AP_BM && rows_cap % gp == 0,
                "attention_tc: rows_cap=%d must be a multiple of %d (the q-heads of a tile) up to %d", rows_cap, gp, AP_BM);
    IDM_REQUIRE(max_runs == 0 || (scratch != nullptr && groups <= AP_COUNTERS),
                "attention_tc: runs through scratch need scratch and at most %d tiles x head groups (got %lld)", AP_COUNTERS, groups);
    CUtensorMap mq, mk, mv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)n_q, (cuuint64_t)n_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)n_q * hd * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)gp, (cuuint32_t)(rows_cap / gp)};
        const int r = tc_make_map_bf16(&mq, q, 3, dims, strides, box);
        IDM_REQUIRE(r == 0, "attention_tc: tensor map for q failed (%d)", r);
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)n_pages * n_kv * IDM_PAGE};
        cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
        cuuint32_t box[2] = {64, AP_BN};
        int r = tc_make_map_bf16(&mk, k_pool, 2, dims, strides, box);
        IDM_REQUIRE(r == 0, "attention_tc: tensor map for k failed (%d)", r);
        r = tc_make_map_bf16(&mv, v_pool, 2, dims, strides, box);
        IDM_REQUIRE(r == 0, "attention_tc: tensor map for v failed (%d)", r);
    }
    AttnTcArgs a;
    a.out = (T*)out; a.tile_seq = tile_seq; a.tile_start = tile_start; a.cu_q = cu_q; a.q_start = q_start;
    a.kv_len = kv_len; a.slots = slots; a.table = table; a.table_stride = table_stride;
    a.n_q = n_q; a.n_kv = n_kv; a.gp_shift = gs; a.scale_log2 = scale * 1.4426950408889634f;
    a.run_blocks = run_blocks; a.max_runs = max_runs; a.rows_cap = rows_cap;
    a.counters = (int*)scratch; a.parts = scratch ? scratch + AP_COUNTERS : nullptr;
    a.tile_pool = tile_pool; a.max_parts = (max_runs == 0 && tile_pool != nullptr) ? max_parts : 0; a.runs_per_part = runs_per_part;
    a.pool = a.parts ? a.parts + groups * (long long)(AP_BM * hd) : nullptr;
    IDM_REQUIRE(a.max_parts == 0 || (scratch != nullptr && runs_per_part >= 1 && groups <= AP_COUNTERS),
                "attention_tc: shared tiles need scratch, runs_per_part >= 1 and at most %d tiles x head groups (got %lld)", AP_COUNTERS, groups);
    if (g_attn_few_rows && attention_few_rows_can(hd, rows_cap, run_blocks, max_runs, groups))
        return hd == 64 ? launch_attention_few_rows<64>(mk, mv, a, (const T*)q, n_tiles, stream)
                        : launch_attention_few_rows<128>(mk, mv, a, (const T*)q, n_tiles, stream);
    return hd == 64 ? launch_attention_tc<64>(mq, mk, mv, a, n_tiles, stream)
                    : launch_attention_tc<128>(mq, mk, mv, a, n_tiles, stream);
}

// 0: tiles of few rows go through the tcgen05 kernel as well (tests compare the two bit for bit); returns the old setting
extern "C" int idm_attention_tc_set_few_rows(int on) {
    const int old = g_attn_few_rows;
    g_attn_few_rows = on;
    return old;
}

extern "C" int idm_attention_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof(int));
    return v;
}

#endif  // IDM_BF16
