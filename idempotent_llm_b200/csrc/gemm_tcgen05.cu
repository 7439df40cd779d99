// out[t, f] = sum over k of x[t, k] * w[f, k]   (bfloat16 in, 32-bit out)
//
// The dense projections of the model (q/k/v, o, gate/up, down, lm_head) on the 5th-generation
// tensor cores: tcgen05.mma issued by one thread, operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle, no multicast), the accumulator in tensor memory, read
// back with tcgen05.ld.  The reference sends these products to a library (torch._int_mm,
// src/detllm/backends.py:88-135).
//
// One order of summation.  Every output element is ONE chain of MMA steps of 16 k each, in
// ascending k, into one accumulator that starts at zero; the inner axis is never split.  On this
// hardware the bits of such a chain do not depend on the instruction's shape, on what else is in the
// tile, or on which operand carries the tokens (tests/test_gpu_kernels.py pins all three), so a
// token's product is the same bits at 1, 64, 65, 300 or 2048 tokens in the step, whichever of the
// kernels below runs.  (Sums of partial chains differ from the one chain in the last bits, which is
// why nothing is split.)
//
// The kernels.
//   up to 128 tokens,   gemm_wide_kernel: 128 features on the lanes, the tokens along the columns, a block per 128
//   >= 16384 features   features (the lm_head).
//   up to 128 tokens    gemm_small_kernel: the MMA's M axis carries the step's tokens (an accumulator
//                       lane is a token), its N axis a narrow slice of 16 to 128 output features, so
//                       that even a matrix of 1024 rows is spread over 64 blocks; each block streams
//                       its slice of the weight once, all of it in flight before the kernel before
//                       this one has ended.  It also takes steps of more tokens, a block per 128 tokens
//                       and slice, where the kernels below would have too few tiles for the SMs.
//   more than 128       gemm_persistent_kernel: 128 features on the lanes, 128 or 256 tokens along the
//                       columns, one block per SM walking over tiles, two accumulators; the tiles in bands
//                       of the weight that stay in the L2.  gemm_pair_kernel: the same with the two blocks
//                       of a cluster on one tile of 256 features x 256 tokens (cta_group::2: each block
//                       fetches half of the token tile), for stored and residual products with tiles
//                       enough for every pair of SMs.
//   q/k/v, more than 128 gemm_qkv_tokens_kernel: tokens on the lanes, 256 features (whole heads) along
//                       the columns.
//
// Epilogues.  STORE (32-bit [M, N]), RESIDUAL (h[t, f] += result, the 32-bit residual sum), SWIGLU
// (bfloat16 y = silu(gate) * up; the weight's rows alternate: gate row of a feature, then its up
// row) and QKV (per-head q/k norm, rotation, q out and cache write by the thread that owns the token;
// head_dim 32, 64 or 128).  Each is one formula per element, the same in every kernel.
//
// Every wait on an mbarrier is bounded by a cycle count; a wait that runs out sets the error flag
// (idm_gemm_status), all roles leave their loops, tensor memory is freed and the block returns.
#include "common.cuh"

#if defined(IDM_BF16)

#include "tcgen05.cuh"
#include "qkv_finish.cuh"

#define GT_BM 128            // rows of the MMA's M axis
#define GT_BK 64             // k per stage: 64 bf16 = 128 bytes = one swizzle row
#define GT_UMMA_K 16

__device__ int g_gemm_error = 0;

// -DIDM_TRACE: block 0 of the kernel for few tokens leaves nanosecond stamps of its stages (a measuring aid,
// compiled out otherwise)
#if defined(IDM_TRACE)
__device__ unsigned long long g_gemm_trace[64];
__device__ int g_gemm_trace_base = 0;          // set by the kernel's first thread: 10 stamps per kind of product
__device__ __forceinline__ void trace_stamp(int i) {
    if (blockIdx.x == 0) { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); g_gemm_trace[(g_gemm_trace_base + i) & 63] = t; }
}
extern "C" int idm_gemm_trace_read(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_gemm_trace, sizeof(unsigned long long) * 64);
}
// per block of the last launch of each kind of product: wait over, first operands, accumulator ready, done, SM
__device__ unsigned long long g_gemm_block_trace[5][512][5];
__device__ __forceinline__ void block_stamp(int kind, int i) {
    if (blockIdx.x < 512) {
        unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        g_gemm_block_trace[kind][blockIdx.x][i] = t;
    }
}
extern "C" int idm_gemm_block_trace_read(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_gemm_block_trace, sizeof(g_gemm_block_trace));
}
// block 0's MMA thread: when each group's operands were there, and when its MMAs had been issued
__device__ unsigned long long g_gemm_mma_trace[5][64][2];
extern "C" int idm_gemm_mma_trace_read(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, g_gemm_mma_trace, sizeof(g_gemm_mma_trace));
}
// a log of block 0 of every launch, in order: kind, started, wait over, done
__device__ unsigned long long g_gemm_log[2048][4];
__device__ unsigned int g_gemm_log_n = 0;
extern "C" int idm_gemm_log_read(unsigned long long* out, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out, g_gemm_log, sizeof(g_gemm_log));
    unsigned int zero = 0;
    if (reset) cudaMemcpyToSymbol(g_gemm_log_n, &zero, sizeof(zero));
    return (int)e;
}
#else
__device__ __forceinline__ void trace_stamp(int) {}
__device__ __forceinline__ void block_stamp(int, int) {}
#endif

enum { EPI_STORE = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3, EPI_QKV = 4 };

struct GemmEpi {
    float* out;          // STORE: [M, N]; RESIDUAL: the residual stream [M, N]
    T* y; int inter;     // SWIGLU: y [M, inter]
    QkvArgs q;           // QKV
};

// ------------------------------------------------------------------- persistent kernel (many tokens)
// Above 256 tokens nothing is split and the product is bound by the tensor cores.  One block per SM
// walks over output tiles of 128 features x BN tokens (BN = 256, or 128 when that fills more SMs):
//   * warp 16 keeps the TMA ring full across tile borders;
//   * warp 17 issues the MMAs into one of TWO accumulators in tensor memory (2 x BN columns);
//   * warps 0-15 run the epilogue of the finished accumulator while the next tile's MMAs run: four
//     groups of four warps (a warp reads the 32 accumulator lanes of its number modulo 4), which take
//     the tile's chunks of 16 tokens in turn -- four warps per scheduler hide each other's latencies;
//     with one group the q/k/v epilogue took three times as long as the tile's MMAs.
// A 128 x 256 tile reads 12 KB of shared memory per 128 tensor-core cycles (128 x 128 reads 8 KB per
// 64, the whole shared-memory bandwidth).  The SwiGLU and q/k/v epilogues turn each chunk through an
// 8 KB buffer per group (the ring is never idle here), so that a thread ends up with consecutive
// features of one token.
#define GP_GROUPS 4
#define GP_EPI_WARPS (4 * GP_GROUPS)
#define GP_THREADS (32 * (GP_EPI_WARPS + 2))
#define GP_CHUNK 16
template <int BN, int STAGES>
struct PersistSmem {
    static constexpr int A_BYTES = GT_BM * GT_BK * 2;
    static constexpr int B_BYTES = BN * GT_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int XS_BYTES = GP_GROUPS * GP_CHUNK * GT_BM * 4;   // per group: [16 tokens][128 features] floats
    static constexpr int XS_OFF = STAGES * STAGE_BYTES;
    static constexpr int BAR_OFF = XS_OFF + XS_BYTES;
    static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ void group_sync(int g) { asm volatile("bar.sync %0, 128;" ::"r"(1 + g) : "memory"); }     // one group

// Where tile number `tile` of a persistent kernel lies: tiles are walked in bands of `band` feature tiles, inside a
// band token tile after token tile, so that the blocks at work together read a band of the weight that stays in the
// L2 (a weight of some hundred MB walked whole for every row of token tiles came from HBM every time: 33 GB for one
// product of 32B sizes with 16 384 tokens).
__device__ __forceinline__ void tile_place(int tile, int tiles_x, int n_tiles, int band, int& fx, int& ty) {
    const int tiles_y = n_tiles / tiles_x, per_band = band * tiles_y;
    const int b = tile / per_band, r = tile - b * per_band;
    const int width = min(band, tiles_x - b * band);               // the last band may be narrower
    ty = r / width;
    fx = b * band + r % width;
}

// The epilogue of one tile of the persistent kernels: the accumulator at `tmem_acc` (128 lanes = features f0 .., BN
// columns = tokens t0 ..) goes out as the EPI says.  Called by the 16 epilogue warps (group `grp`, accumulator
// lanes 32 `quarter` ..); `xs`: the group's buffer of [16 tokens][128 features] floats; `tx`: f0 / 128.
template <int BN, int EPI>
__device__ __forceinline__ void persistent_tile_epilogue(const GemmEpi& e, uint32_t tmem_acc, float* xs, int grp, int quarter,
                                                         int lane, int tx, int t0, int n_tokens, int n_features) {
    const int fl = quarter * 32 + lane;                            // feature within the tile = accumulator lane
    const int f0 = tx * GT_BM, f = f0 + fl;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    // the accumulator columns of a chunk are asked for while the chunk before is worked on (two sets of
    // registers in turn; the loop is unrolled so that which set is which is known at compile time)
    uint32_t raw[2][GP_CHUNK];
    if (t0 + grp * GP_CHUNK < n_tokens) tc_ld16_issue(tmem_acc + lane_base + (uint32_t)(grp * GP_CHUNK), raw[0]);
#pragma unroll
    for (int ci = 0; ci < BN / (GP_GROUPS * GP_CHUNK); ++ci) {
        const int c0 = grp * GP_CHUNK + ci * GP_GROUPS * GP_CHUNK;
        if (t0 + c0 >= n_tokens) break;                    // uniform over the group
        const int cols = min(GP_CHUNK, n_tokens - t0 - c0);
        float v[GP_CHUNK];
        tc_ld_wait();
#pragma unroll
        for (int j = 0; j < GP_CHUNK; ++j) v[j] = __uint_as_float(raw[ci & 1][j]);
        if (ci + 1 < BN / (GP_GROUPS * GP_CHUNK) && t0 + c0 + GP_GROUPS * GP_CHUNK < n_tokens)
            tc_ld16_issue(tmem_acc + lane_base + (uint32_t)(c0 + GP_GROUPS * GP_CHUNK), raw[(ci + 1) & 1]);
        if (EPI == EPI_STORE || EPI == EPI_RESIDUAL) {
            if (f < n_features) {
                float old[GP_CHUNK];
                if (EPI == EPI_RESIDUAL) {
#pragma unroll
                    for (int j = 0; j < GP_CHUNK; ++j)
                        old[j] = j < cols ? e.out[(size_t)(t0 + c0 + j) * n_features + f] : 0.f;
                }
#pragma unroll
                for (int j = 0; j < GP_CHUNK; ++j)
                    if (j < cols)
                        e.out[(size_t)(t0 + c0 + j) * n_features + f] = EPI == EPI_RESIDUAL ? old[j] + v[j] : v[j];
            }
        } else {
            // through shared memory, so that a thread ends up with consecutive features of one token
#pragma unroll
            for (int j = 0; j < GP_CHUNK; ++j) xs[j * GT_BM + fl] = v[j];
            group_sync(grp);
            if (EPI == EPI_SWIGLU) {
                // 8 consecutive features of y (16 tile rows: gate, up, gate, up, ...) per thread, one
                // 16-byte store; the group's 128 threads cover the chunk's 16 token rows
                const int j = fl >> 3, sub = fl & 7;
                if (j < cols) {
                    const float4* src = reinterpret_cast<const float4*>(xs + j * GT_BM + sub * 16);
                    const float4 p0 = src[0], p1 = src[1], p2 = src[2], p3 = src[3];
                    const float y8[8] = {silu_mul(p0.x, p0.y), silu_mul(p0.z, p0.w), silu_mul(p1.x, p1.y), silu_mul(p1.z, p1.w),
                                         silu_mul(p2.x, p2.y), silu_mul(p2.z, p2.w), silu_mul(p3.x, p3.y), silu_mul(p3.z, p3.w)};
                    const int fg = tx * 64 + sub * 8;
                    T* dst = e.y + (size_t)(t0 + c0 + j) * e.inter + fg;
                    if ((e.inter & 7) == 0 && fg + 8 <= e.inter) {
                        store8(dst, y8);
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            if (fg + i < e.inter) from_f32(dst[i], y8[i]);
                    }
                }
            }
            group_sync(grp);                               // the buffer is free for the group's next chunk
        }
    }
}

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(GP_THREADS) gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                     const __grid_constant__ CUtensorMap map_x,
                                                                     const GemmEpi e, int n_tokens, int n_features,
                                                                     int kb_total, int tiles_x, int n_tiles, int band) {
    using S = PersistSmem<BN, STAGES>;
    constexpr int TMEM_COLS = 2 * BN;                              // 256 or 512
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + S::BAR_OFF;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + S::BAR_OFF + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), GP_EPI_WARPS); }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == GP_EPI_WARPS + 1) tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_wait();

    if (warp == GP_EPI_WARPS) {
        if (lane == 0) {
            uint32_t cnt = 0;                                      // k-blocks issued so far, over all tiles
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                int fx, ty;
                tile_place(tile, tiles_x, n_tiles, band, fx, ty);
                const int f0 = fx * GT_BM, t0 = ty * BN;
                bool ok = true;
                for (int i = 0; i < kb_total && ok; ++i, ++cnt) {
                    const int s = cnt % STAGES;
                    ok = mbar_wait(empty_bar(s), ((cnt / STAGES) & 1) ^ 1, abort_flag, &g_gemm_error);
                    if (!ok) break;
                    mbar_expect_tx(full_bar(s), S::STAGE_BYTES);
                    const uint32_t a_dst = base + s * S::STAGE_BYTES;
                    tma_load_2d(a_dst, &map_w, i * GT_BK, f0, full_bar(s));
                    tma_load_2d(a_dst + S::A_BYTES, &map_x, i * GT_BK, t0, full_bar(s));
                }
                if (!ok) break;
            }
        }
    } else if (warp == GP_EPI_WARPS + 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(GT_BM, BN);
            uint32_t cnt = 0, it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
                const uint32_t acc = it & 1;
                ok = mbar_wait(tempty_bar(acc), ((it >> 1) & 1) ^ 1, abort_flag, &g_gemm_error);   // epilogue drained it
                if (!ok) break;
                tc_fence_after();
                // (the look at the next stage's barrier is issued before this stage's MMAs, so that its answer
                // is there when they have been issued: asking afterwards cost ~100 ns per k-block, a quarter
                // of the time the tensor core needs for it)
                bool ready = mbar_try(full_bar(cnt % STAGES), (cnt / STAGES) & 1);
                for (int i = 0; i < kb_total && ok; ++i, ++cnt) {
                    const int s = cnt % STAGES;
                    if (!ready) ok = mbar_wait(full_bar(s), (cnt / STAGES) & 1, abort_flag, &g_gemm_error);
                    if (!ok) break;
                    tc_fence_after();
                    ready = i + 1 < kb_total && mbar_try(full_bar((cnt + 1) % STAGES), ((cnt + 1) / STAGES) & 1);
                    const uint32_t a_addr = base + s * S::STAGE_BYTES;
                    const uint64_t a_desc = umma_desc_kmajor(a_addr), b_desc = umma_desc_kmajor(a_addr + S::A_BYTES);
#pragma unroll
                    for (int k = 0; k < GT_BK / GT_UMMA_K; ++k)
                        tc_mma_bf16(tmem + acc * BN, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    tc_commit(empty_bar(s));
                }
                if (ok) tc_commit(tfull_bar(acc));
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3, grp = warp >> 2;             // accumulator lanes 32 quarter ..; group 0 or 1
        float* xs = (float*)(gen_base + S::XS_OFF) + grp * (GP_CHUNK * GT_BM);
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
            int tx, ty;
            tile_place(tile, tiles_x, n_tiles, band, tx, ty);
            const int t0 = ty * BN;
            const uint32_t acc = it & 1;
            ok = mbar_wait(tfull_bar(acc), (it >> 1) & 1, abort_flag, &g_gemm_error);
            if (!ok) break;
            tc_fence_after();
            persistent_tile_epilogue<BN, EPI>(e, tmem + acc * BN, xs, grp, quarter, lane, tx, t0, n_tokens, n_features);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == GP_EPI_WARPS + 1) tmem_dealloc(tmem, TMEM_COLS);
}

// --------------------------------------------------- many tokens, a pair of blocks on one tile (cta_group::2)
// The persistent scheme above with tiles of 256 features x BN tokens worked by the two blocks of a cluster: block
// r holds features f0 + 128 r .. (its rows of w, its half of the accumulator) and fetches tokens t0 + BN/2 r ..
// (its half of the rows of x); block 0's MMA thread issues every MMA for both.  Per k-block a block fetches
// 128 + BN/2 rows for 128 x BN products, where the kernel above fetches 128 + BN: the way from the L2 to the SMs
// is what bounds these products.  Who waits for whom:
//   full[s]    in block 0: the bytes of both blocks' loads of stage s (each block's TMA counts there)
//   empty[s]   in each block: stage s has been read by the MMAs (a commit to both blocks)
//   tfull[a]   in each block: accumulator a is complete (a commit to both blocks)
//   tempty[a]  in block 0: the epilogue warps of BOTH blocks have read accumulator a
// Every wait is bounded; a block whose wait ran out falls through to the end, where both blocks meet before
// tensor memory is given back (the other block's waits then run out by themselves).
template <int BN, int STAGES>
struct PairSmem {
    static constexpr int A_BYTES = GT_BM * GT_BK * 2;
    static constexpr int B_BYTES = (BN / 2) * GT_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int XS_BYTES = GP_GROUPS * GP_CHUNK * GT_BM * 4;
    static constexpr int XS_OFF = STAGES * STAGE_BYTES;
    static constexpr int BAR_OFF = XS_OFF + XS_BYTES;
    static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(GP_THREADS) gemm_pair_kernel(const __grid_constant__ CUtensorMap map_w,
                                                               const __grid_constant__ CUtensorMap map_x,
                                                               const GemmEpi e, int n_tokens, int n_features,
                                                               int kb_total, int tiles_x, int n_tiles, int band) {
    using S = PairSmem<BN, STAGES>;
    constexpr int TMEM_COLS = 2 * BN;                              // 256 or 512
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + S::BAR_OFF;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + S::BAR_OFF + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                          // 0: issues the MMAs
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 2 * GP_EPI_WARPS); }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == GP_EPI_WARPS + 1) tmem_alloc_pair(smem_u32((const void*)tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                            // the other block's barriers exist before anything arrives there
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_wait();

    if (warp == GP_EPI_WARPS) {
        if (lane == 0) {
            uint32_t cnt = 0;                                      // k-blocks issued so far, over all tiles
            for (int tile = pair; tile < n_tiles; tile += n_pairs) {
                int fx, ty;
                tile_place(tile, tiles_x, n_tiles, band, fx, ty);
                const int f0 = fx * (2 * GT_BM) + (int)rank * GT_BM;
                const int t0 = ty * BN + (int)rank * (BN / 2);
                bool ok = true;
                for (int i = 0; i < kb_total && ok; ++i, ++cnt) {
                    const int s = cnt % STAGES;
                    ok = mbar_wait_cluster(empty_bar(s), ((cnt / STAGES) & 1) ^ 1, abort_flag, &g_gemm_error);
                    if (!ok) break;
                    if (rank == 0) mbar_expect_tx(full_bar(s), 2 * S::STAGE_BYTES);
                    const uint32_t a_dst = base + s * S::STAGE_BYTES;
                    const uint32_t full0 = mapa_u32(full_bar(s), 0);
                    tma_load_2d_pair(a_dst, &map_w, i * GT_BK, f0, full0);
                    tma_load_2d_pair(a_dst + S::A_BYTES, &map_x, i * GT_BK, t0, full0);
                }
                if (!ok) break;
            }
        }
    } else if (warp == GP_EPI_WARPS + 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = umma_idesc(2 * GT_BM, BN);
            uint32_t cnt = 0, it = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++it) {
                const uint32_t acc = it & 1;
                ok = mbar_wait_cluster(tempty_bar(acc), ((it >> 1) & 1) ^ 1, abort_flag, &g_gemm_error);   // both epilogues drained it
                if (!ok) break;
                tc_fence_after();
                for (int i = 0; i < kb_total && ok; ++i, ++cnt) {
                    const int s = cnt % STAGES;
                    ok = mbar_wait_cluster(full_bar(s), (cnt / STAGES) & 1, abort_flag, &g_gemm_error);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = base + s * S::STAGE_BYTES;
                    const uint64_t a_desc = umma_desc_kmajor(a_addr), b_desc = umma_desc_kmajor(a_addr + S::A_BYTES);
#pragma unroll
                    for (int k = 0; k < GT_BK / GT_UMMA_K; ++k)
                        tc_mma_bf16_pair(tmem + acc * BN, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(empty_bar(s), 3u);
                }
                if (ok) tc_commit_pair(tfull_bar(acc), 3u);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps (of both blocks)
        const int quarter = warp & 3, grp = warp >> 2;
        float* xs = (float*)(gen_base + S::XS_OFF) + grp * (GP_CHUNK * GT_BM);
        uint32_t it = 0;
        bool ok = true;
        for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++it) {
            int fx, ty;
            tile_place(tile, tiles_x, n_tiles, band, fx, ty);
            const int tx = fx * 2 + (int)rank, t0 = ty * BN;
            const uint32_t acc = it & 1;
            ok = mbar_wait_cluster(tfull_bar(acc), (it >> 1) & 1, abort_flag, &g_gemm_error);
            if (!ok) break;
            tc_fence_after();
            persistent_tile_epilogue<BN, EPI>(e, tmem + acc * BN, xs, grp, quarter, lane, tx, t0, n_tokens, n_features);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_u32(tempty_bar(acc), 0));
        }
    }
    // nobody leaves, and no tensor memory goes back, while the other block may still read this one's shared
    // memory, count at its barriers or run MMAs into its accumulators
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == GP_EPI_WARPS + 1) tmem_dealloc_pair(tmem, TMEM_COLS);
}

// ------------------------------------------------- q/k/v projection of many tokens, tokens on the lanes
// The same persistent scheme with the operands' roles exchanged: the MMA's M axis carries 128 tokens
// (rows of x), its N axis 256 features (rows of w: whole heads), so an accumulator lane is a token and
// a thread reads its token's whole head along the columns.  The per-head norm is then a sum inside the
// thread, the rotation partner (d, d + head_dim / 2) a register of the same thread: no shuffles, no
// turn through shared memory, no barrier between warps.  A head of a tile goes to one warp per 32
// tokens.  The epilogue is a chain of latencies (accumulator read ~900 cycles, the rotation table from
// L2, stores that touch 32 lines each), so it has few warps with many registers: a thread asks for its
// whole head (up to 128 columns) at once and for the next 16 dims' (cos, sin) while it works on these.
// With 16 warps of 112 registers, each reading 32 columns at a time and sharing heads through a
// barrier, a tile's epilogue took 9 us against 5.8 us for its MMAs.
#define GQ_BN 256
#define GQ_STAGES 4
#define GQ_EPI_WARPS 8
#define GQ_THREADS (32 * (GQ_EPI_WARPS + 2))
struct QkvTokensSmem {
    static constexpr int A_BYTES = GT_BM * GT_BK * 2;              // 128 tokens
    static constexpr int B_BYTES = GQ_BN * GT_BK * 2;              // 256 features
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFF = GQ_STAGES * STAGE_BYTES;
    static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

// One head of one token: norm, rotation, stores.  col0: the head's first accumulator column (with the
// warp's lanes); cs_row: the token's row of the rotation table; cs_dim: the same table by dim (the
// tokens of a dim side by side: two lines per request instead of 32), or null.
// (KEEP also says that gamma and cs_row may lie in shared memory: they are read with plain loads then)
template <int HD, bool KEEP = false>
__device__ __forceinline__ void qkv_tokens_head(const QkvArgs& a, uint32_t col0, const float* gamma, bool rotate,
                                                const float2* cs_row, const float2* cs_dim, int n_tokens,
                                                T* dst_a, T* dst_b) {
    constexpr int HALF = HD / 2;
    float cs4[4][8];                                               // (cos, sin) of 16 dims
    auto ask_cs = [&](int c) {
        if (!rotate) return;
        if (KEEP) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 u = *reinterpret_cast<const float4*>(cs_row + c + 4 * i), w = *reinterpret_cast<const float4*>(cs_row + c + 4 * i + 2);
                cs4[i][0] = u.x; cs4[i][1] = u.y; cs4[i][2] = u.z; cs4[i][3] = u.w;
                cs4[i][4] = w.x; cs4[i][5] = w.y; cs4[i][6] = w.z; cs4[i][7] = w.w;
            }
        } else if (cs_dim != nullptr) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float2 v = __ldg(cs_dim + (size_t)(c + i) * n_tokens);
                cs4[i / 4][2 * (i % 4)] = v.x; cs4[i / 4][2 * (i % 4) + 1] = v.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                load8_readonly(reinterpret_cast<const float*>(cs_row + c + 4 * i), cs4[i]);
        }
    };
    // KEEP (a block with few tokens and registers to spare): the whole head stays in registers after the sum of
    // squares, so the second pass reads no tensor memory again.  The arithmetic is the same either way.
    uint32_t all[KEEP ? HD : 1];
    uint32_t cur[32];                                              // 16 dims of each half: this step's, then the next's
    float inv = 1.f;
    {
        // the head's sum of squares (four chains), one half of the head at a time in registers (the whole
        // head at once leaves no room); the first step's columns of each half are kept
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t raw[HALF];
#pragma unroll
            for (int c = 0; c < HALF; c += 16) tc_ld16_issue(col0 + (uint32_t)(h * HALF + c), raw + c);
            if (h == 0) ask_cs(0);
            tc_ld_wait();
            if (gamma != nullptr) {
#pragma unroll
                for (int i = 0; i < HALF; ++i)
                    s4[i & 3] = __fmaf_rn(__uint_as_float(raw[i]), __uint_as_float(raw[i]), s4[i & 3]);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) cur[16 * h + i] = raw[i];
            if (KEEP) {
#pragma unroll
                for (int i = 0; i < HALF; ++i) all[h * HALF + i] = raw[i];
            }
        }
        if (gamma != nullptr) inv = head_inv_rms(a, (s4[0] + s4[1]) + (s4[2] + s4[3]));
    }
    // dims d and d + HALF together, 16 of each per step
    auto step = [&](int c, const uint32_t* lo_raw, const uint32_t* hi_raw) {
        float lo[16], hi[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) { lo[i] = __uint_as_float(lo_raw[i]); hi[i] = __uint_as_float(hi_raw[i]); }
        if (!KEEP && c + 16 < HALF) {
            tc_ld16_issue(col0 + (uint32_t)(c + 16), cur);
            tc_ld16_issue(col0 + (uint32_t)(HALF + c + 16), cur + 16);
        }
        if (gamma != nullptr) {
            // the norm weight four values a request (every lane asks for the same address)
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
                const float4 gl = KEEP ? *reinterpret_cast<const float4*>(gamma + c + i) : __ldg(reinterpret_cast<const float4*>(gamma + c + i));
                const float4 gh = KEEP ? *reinterpret_cast<const float4*>(gamma + HALF + c + i)
                                       : __ldg(reinterpret_cast<const float4*>(gamma + HALF + c + i));
                lo[i] = __fmul_rn(__fmul_rn(lo[i], inv), gl.x); lo[i + 1] = __fmul_rn(__fmul_rn(lo[i + 1], inv), gl.y);
                lo[i + 2] = __fmul_rn(__fmul_rn(lo[i + 2], inv), gl.z); lo[i + 3] = __fmul_rn(__fmul_rn(lo[i + 3], inv), gl.w);
                hi[i] = __fmul_rn(__fmul_rn(hi[i], inv), gh.x); hi[i + 1] = __fmul_rn(__fmul_rn(hi[i + 1], inv), gh.y);
                hi[i + 2] = __fmul_rn(__fmul_rn(hi[i + 2], inv), gh.z); hi[i + 3] = __fmul_rn(__fmul_rn(hi[i + 3], inv), gh.w);
            }
        }
        if (rotate) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float u = lo[i], w = hi[i];
                const float co = cs4[i / 4][2 * (i % 4)], si = cs4[i / 4][2 * (i % 4) + 1];
                lo[i] = __fmaf_rn(u, co, -__fmul_rn(w, si));
                hi[i] = __fmaf_rn(w, co, __fmul_rn(u, si));
            }
        }
        if (c + 16 < HALF) ask_cs(c + 16);                         // before this step's stores queue up
        if (dst_a) { store16(dst_a + c, lo); store16(dst_a + HALF + c, hi); }
        if (dst_b) { store16(dst_b + c, lo); store16(dst_b + HALF + c, hi); }
    };
    if (KEEP) {
#pragma unroll
        for (int c = 0; c < HALF; c += 16) step(c, all + c, all + HALF + c);
    } else {
        // the next step's columns are asked for before this step's arithmetic (the loop stays a loop: unrolled,
        // the compiler moves all steps' loads of the norm weight to the front and runs out of registers)
#pragma unroll 1
        for (int c = 0; c < HALF; c += 16) {
            if (c > 0) tc_ld_wait();
            step(c, cur, cur + 16);                                // (its values are taken before the next columns are asked into it)
        }
    }
}

__global__ void __launch_bounds__(GQ_THREADS) gemm_qkv_tokens_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                     const __grid_constant__ CUtensorMap map_x,
                                                                     const GemmEpi e, int n_tokens, int n_features,
                                                                     int kb_total, int tiles_x, int n_tiles, int band) {
    using S = QkvTokensSmem;
    constexpr int STAGES = GQ_STAGES, BN = GQ_BN;
    constexpr int TMEM_COLS = 2 * BN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + S::BAR_OFF;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + S::BAR_OFF + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), GQ_EPI_WARPS); }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == GQ_EPI_WARPS + 1) tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_wait();

    if (warp == GQ_EPI_WARPS) {
        if (lane == 0) {
            uint32_t cnt = 0;
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                int fx, ty;
                tile_place(tile, tiles_x, n_tiles, band, fx, ty);
                const int f0 = fx * BN, t0 = ty * GT_BM;
                bool ok = true;
                for (int i = 0; i < kb_total && ok; ++i, ++cnt) {
                    const int s = cnt % STAGES;
                    ok = mbar_wait(empty_bar(s), ((cnt / STAGES) & 1) ^ 1, abort_flag, &g_gemm_error);
                    if (!ok) break;
                    mbar_expect_tx(full_bar(s), S::STAGE_BYTES);
                    const uint32_t a_dst = base + s * S::STAGE_BYTES;
                    tma_load_2d(a_dst, &map_x, i * GT_BK, t0, full_bar(s));
                    tma_load_2d(a_dst + S::A_BYTES, &map_w, i * GT_BK, f0, full_bar(s));
                }
                if (!ok) break;
            }
        }
    } else if (warp == GQ_EPI_WARPS + 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(GT_BM, BN);
            uint32_t cnt = 0, it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
                const uint32_t acc = it & 1;
                ok = mbar_wait(tempty_bar(acc), ((it >> 1) & 1) ^ 1, abort_flag, &g_gemm_error);
                if (!ok) break;
                tc_fence_after();
                for (int i = 0; i < kb_total && ok; ++i, ++cnt) {
                    const int s = cnt % STAGES;
                    ok = mbar_wait(full_bar(s), (cnt / STAGES) & 1, abort_flag, &g_gemm_error);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = base + s * S::STAGE_BYTES;
                    const uint64_t a_desc = umma_desc_kmajor(a_addr), b_desc = umma_desc_kmajor(a_addr + S::A_BYTES);
#pragma unroll
                    for (int k = 0; k < GT_BK / GT_UMMA_K; ++k)
                        tc_mma_bf16(tmem + acc * BN, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    tc_commit(empty_bar(s));
                }
                if (ok) tc_commit(tfull_bar(acc));
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue warps
        const QkvArgs& a = e.q;
        const int quarter = warp & 3, grp = warp >> 2;             // accumulator lanes 32 quarter ..; heads grp, grp + 2, ...
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int hd = a.hd, half = hd >> 1, heads = a.n_q + 2 * a.n_kv, hpt = BN / hd;
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
            int tx, ty;
            tile_place(tile, tiles_x, n_tiles, band, tx, ty);
            const int f0 = tx * BN, t0 = ty * GT_BM;
            const uint32_t acc = it & 1;
            const int t = t0 + quarter * 32 + lane;                // this thread's token
            const bool live = t < n_tokens;
            // where the token's key/value rows lie in the cache (asked for before the accumulator is waited for)
            size_t place = 0;
            if (live && a.write_cache && f0 + BN > a.n_q * hd) {
                const int pos = a.positions[t];
                const int r = a.cache.ring ? pos % a.cache.ring : pos;
                const int page = a.cache.table[(size_t)a.slots[a.token_seq[t]] * a.cache.table_stride + r / IDM_PAGE];
                place = (size_t)page * a.n_kv * IDM_PAGE + r % IDM_PAGE;       // row of kv-head 0; kv-head g: + g * IDM_PAGE
            }
            const float2* cs_row = a.cs + (size_t)(live ? t : 0) * half;
            const float2* cs_dim = a.cs_by_dim ? a.cs_by_dim + (live ? t : 0) : nullptr;
            ok = mbar_wait(tfull_bar(acc), (it >> 1) & 1, abort_flag, &g_gemm_error);
            if (!ok) break;
            tc_fence_after();
            for (int hh = grp; hh < hpt; hh += GQ_EPI_WARPS / 4) {
                const int head = tx * hpt + hh;
                if (head >= heads) break;                          // the last tile may reach past the last head
                const uint32_t col0 = tmem + acc * BN + lane_base + (uint32_t)(hh * hd);
                const bool is_q = head < a.n_q, is_k = !is_q && head < a.n_q + a.n_kv;
                const float* gamma = is_q ? a.gq : (is_k ? a.gk : nullptr);
                T* dst_a = nullptr; T* dst_b = nullptr;
                if (live) {
                    if (is_q) {
                        dst_a = a.q_out + ((size_t)t * a.n_q + head) * hd;
                    } else {
                        const int g = is_k ? head - a.n_q : head - a.n_q - a.n_kv;
                        if (a.write_cache) dst_a = (is_k ? a.cache.k : a.cache.v) + (place + (size_t)g * IDM_PAGE) * hd;
                        T* packed = is_k ? a.k_new : a.v_new;
                        if (packed) dst_b = packed + ((size_t)t * a.n_kv + g) * hd;
                    }
                }
                const bool rotate = (is_q || is_k) && a.cs != nullptr;
                if (hd == 128) qkv_tokens_head<128>(a, col0, gamma, rotate, cs_row, cs_dim, n_tokens, dst_a, dst_b);
                else if (hd == 64) qkv_tokens_head<64>(a, col0, gamma, rotate, cs_row, cs_dim, n_tokens, dst_a, dst_b);
                else qkv_tokens_head<32>(a, col0, gamma, rotate, cs_row, cs_dim, n_tokens, dst_a, dst_b);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == GQ_EPI_WARPS + 1) tmem_dealloc(tmem, TMEM_COLS);
}

// Feature tiles per band of the persistent kernels' walk: as many as hold `g_gemm_band_mb` MB of the weight.
static int g_gemm_band_mb = 32;
extern "C" void idm_gemm_set_band_mb(int mb) { g_gemm_band_mb = mb < 1 ? 1 : mb; }
static int tile_band(int tile_rows, int kb_total, int tiles_x) {
    const long long tile_bytes = (long long)tile_rows * kb_total * GT_BK * 2;
    long long band = ((long long)g_gemm_band_mb << 20) / tile_bytes;
    if (band < 1) band = 1;
    return band > tiles_x ? tiles_x : (int)band;
}

static int launch_qkv_tokens(const CUtensorMap& mw, const CUtensorMap& mx, const GemmEpi& e, int M, int N, int kb_total,
                             cudaStream_t stream) {
    using S = QkvTokensSmem;
    static bool configured = false;
    static int n_sm = 0;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_qkv_tokens_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        IDM_REQUIRE(err == cudaSuccess, "gemm: cannot get %d bytes of shared memory: %s", S::TOTAL, cudaGetErrorString(err));
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        configured = true;
    }
    const int tiles_x = (N + GQ_BN - 1) / GQ_BN, tiles_y = (M + GT_BM - 1) / GT_BM;
    const int n_tiles = tiles_x * tiles_y;
    const int grid = n_tiles < n_sm ? n_tiles : n_sm;
    idm_launch(gemm_qkv_tokens_kernel, dim3(grid), dim3(GQ_THREADS), S::TOTAL, stream, mw, mx, e, M, N, kb_total, tiles_x,
               n_tiles, tile_band(GQ_BN, kb_total, tiles_x));
    IDM_LAUNCH_CHECK("gemm_qkv_tokens");
    return 0;
}

template <int BN, int STAGES, int EPI>
static int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mx, const GemmEpi& e, int M, int N, int kb_total,
                             cudaStream_t stream) {
    using S = PersistSmem<BN, STAGES>;
    static bool configured = false;
    static int n_sm = 0;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_persistent_kernel<BN, STAGES, EPI>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        IDM_REQUIRE(err == cudaSuccess, "gemm: cannot get %d bytes of shared memory: %s", S::TOTAL,
                    cudaGetErrorString(err));
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        configured = true;
    }
    const int tiles_x = (N + GT_BM - 1) / GT_BM, tiles_y = (M + BN - 1) / BN;
    const int n_tiles = tiles_x * tiles_y;
    const int grid = n_tiles < n_sm ? n_tiles : n_sm;
    idm_launch(gemm_persistent_kernel<BN, STAGES, EPI>, dim3(grid), dim3(GP_THREADS), S::TOTAL, stream, mw, mx, e, M, N,
               kb_total, tiles_x, n_tiles, tile_band(GT_BM, kb_total, tiles_x));
    IDM_LAUNCH_CHECK("gemm_persistent");
    return 0;
}
template <int BN, int STAGES, int EPI>
static int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, const GemmEpi& e, int M, int N, int kb_total,
                       cudaStream_t stream) {
    using S = PairSmem<BN, STAGES>;
    static bool configured = false;
    static int n_sm = 0;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_pair_kernel<BN, STAGES, EPI>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        IDM_REQUIRE(err == cudaSuccess, "gemm: cannot get %d bytes of shared memory: %s", S::TOTAL,
                    cudaGetErrorString(err));
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        configured = true;
    }
    const int tiles_x = (N + 2 * GT_BM - 1) / (2 * GT_BM), tiles_y = (M + BN - 1) / BN;
    const int n_tiles = tiles_x * tiles_y;
    const int pairs = n_tiles < n_sm / 2 ? n_tiles : n_sm / 2;
    // a cluster of two blocks along x: blocks 2 p and 2 p + 1 are pair p
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(GP_THREADS); cfg.dynamicSmemBytes = S::TOTAL; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = idm_pdl_enabled() ? 2 : 1;
    cudaError_t err = cudaLaunchKernelEx(&cfg, gemm_pair_kernel<BN, STAGES, EPI>, mw, mx, e, M, N, kb_total, tiles_x, n_tiles,
                                         tile_band(2 * GT_BM, kb_total, tiles_x));
    IDM_REQUIRE(err == cudaSuccess, "gemm_pair: launch failed: %s", cudaGetErrorString(err));
    IDM_LAUNCH_CHECK("gemm_pair");
    return 0;
}
// ------------------------------------------------------------------- few tokens (up to 128)
// The step's tokens on the accumulator's lanes (MMA M = 64 for up to 64 tokens, else 128: the rows of x,
// of which only the first `tbox` are fetched; what the other rows of the operand hold is whatever lies
// behind the slot in shared memory, and goes into accumulator lanes nobody reads), `bf` output features
// along its columns.  (An MMA of few columns costs what its operands' bytes cost to read from shared
// memory, about 64 a cycle, with a floor of ~46 cycles: hence as few rows as the tokens allow.)  A block owns features [bf * blockIdx.x, + bf) and walks the whole inner axis: one chain
// per element.  Warp 4 issues the TMA loads, `gk` k-blocks per request and barrier (a three-dimensional
// view of the matrices: k within a block, row, k-block) -- the weight slices of the first `stages`
// groups before the wait on the kernel before (no kernel writes weights), the activations after it;
// warp 5 issues the MMAs (a chain of K / 16 instructions of ~46 cycles each, whatever their width: the
// floor of this kernel); warps 0-3 read the accumulator (thread = token) and run the epilogue.
#define GS_THREADS 192
#define GS_MAX_STAGES 16
#define GS_BAR_BYTES 1024

// rows of the MMA's M axis: 64 for up to 64 tokens (half the operand bytes per instruction), else 128
__host__ __device__ inline int gs_mma_rows(int tbox) { return tbox <= 64 ? 64 : 128; }

__host__ __device__ inline uint32_t gs_data_bytes(int tbox, int bf, int gk, int stages) {
    const uint32_t a_slot = (uint32_t)tbox * 128u, b_slot = (uint32_t)bf * 128u;
    uint32_t data = (uint32_t)(stages * gk) * (a_slot + b_slot);
    const uint32_t reach = (uint32_t)(stages * gk - 1) * a_slot + (uint32_t)gs_mma_rows(tbox) * 128u;   // the MMA reads that many rows from every A slot
    if (reach > data) data = reach;
    return (data + 1023u) & ~1023u;
}

template <int EPI>
__global__ void __launch_bounds__(GS_THREADS) gemm_small_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_x,
                                                                const GemmEpi e, int n_tokens, int n_features,
                                                                int kb_total, int bf, int tbox, int gk, int grouped,
                                                                int stages, int tmem_cols) {
    pdl_launch_dependents();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_slot = (uint32_t)tbox * 128u, b_slot = (uint32_t)bf * 128u;      // one k-block of each operand
    const uint32_t a_base = base, b_base = base + (uint32_t)(stages * gk) * a_slot;
    const uint32_t bar_off = gs_data_bytes(tbox, bf, gk, stages);
    const uint32_t bars = base + bar_off;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (GS_MAX_STAGES + s); };
    const uint32_t accum_bar = bars + 8u * (2 * GS_MAX_STAGES);
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + bar_off + 8 * (2 * GS_MAX_STAGES + 1));
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = blockIdx.x * bf;
    const int t0 = blockIdx.y * 128;                             // more than 128 tokens: a block per 128 of them (and slice)
    const int n_groups = (kb_total + gk - 1) / gk;
    if (threadIdx.x == 0) block_stamp(EPI == EPI_RESIDUAL ? (kb_total > 32 ? 1 : 0) : EPI == EPI_SWIGLU ? 2 : EPI == EPI_QKV ? 3 : 4, 4);   // the block is there

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 5) tmem_alloc(smem_u32((const void*)tmem_slot), (uint32_t)tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;
#if defined(IDM_TRACE)
    // (stamps of the four fused products of a layer side by side: residual with a short / long inner axis, SwiGLU, q/k/v)
    if (blockIdx.x == 0 && threadIdx.x == 0) g_gemm_trace_base = EPI == EPI_RESIDUAL ? (kb_total > 32 ? 10 : 0) : EPI == EPI_SWIGLU ? 20 : EPI == EPI_QKV ? 30 : 40;
    __syncthreads();
#endif
    if (threadIdx.x == 0) trace_stamp(0);                        // set-up done
    const int trace_kind = EPI == EPI_RESIDUAL ? (kb_total > 32 ? 1 : 0) : EPI == EPI_SWIGLU ? 2 : EPI == EPI_QKV ? 3 : 4;

    if (warp == 4) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // a group's loads: one request per operand (grouped: the maps are three-dimensional), or one per k-block
            auto load_w = [&](int gi, int s) {
                const uint32_t dst = b_base + (uint32_t)(s * gk) * b_slot;
                if (grouped) { tma_load_3d(dst, &map_w, 0, f0, gi * gk, full_bar(s)); return; }
                for (int k = 0; k < gk && gi * gk + k < kb_total; ++k)
                    tma_load_2d(dst + k * b_slot, &map_w, (gi * gk + k) * GT_BK, f0, full_bar(s));
            };
            auto load_x = [&](int gi, int s) {
                const uint32_t dst = a_base + (uint32_t)(s * gk) * a_slot;
                if (grouped) { tma_load_3d(dst, &map_x, 0, t0, gi * gk, full_bar(s)); return; }
                for (int k = 0; k < gk && gi * gk + k < kb_total; ++k)
                    tma_load_2d(dst + k * a_slot, &map_x, (gi * gk + k) * GT_BK, t0, full_bar(s));
            };
            // (a grouped request always brings gk k-blocks: those past the end come as zeros)
            auto group_bytes = [&](int gi) { return (uint32_t)(grouped ? gk : min(gk, kb_total - gi * gk)) * (a_slot + b_slot); };
            const int early = min(n_groups, stages);
            for (int gi = 0; gi < early; ++gi) {
                mbar_expect_tx(full_bar(gi), group_bytes(gi));
                load_w(gi, gi);
            }
            trace_stamp(1);                                      // early weight loads issued
            pdl_wait();
            trace_stamp(2);                                      // the kernel before is done
            block_stamp(trace_kind, 0);
            for (int gi = 0; gi < early; ++gi) load_x(gi, gi);
            trace_stamp(3);                                      // early activation loads issued
            int s = 0; uint32_t phase = 0;                       // the ring goes round: stage and the parity of its use
            for (int gi = early; gi < n_groups; ++gi) {
                if (!mbar_wait(empty_bar(s), phase, abort_flag, &g_gemm_error)) break;
                mbar_expect_tx(full_bar(s), group_bytes(gi));
                load_w(gi, s);
                load_x(gi, s);
                if (++s == stages) { s = 0; phase ^= 1; }
            }
            trace_stamp(4);                                      // all loads issued
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(gs_mma_rows(tbox), bf);
            const uint64_t a_desc0 = umma_desc_kmajor(a_base), b_desc0 = umma_desc_kmajor(b_base);
            const uint32_t a_step = a_slot >> 4, b_step = b_slot >> 4;     // descriptors count in 16 bytes
            bool ok = true;
            int s = 0; uint32_t phase = 0, acc = 0;
            uint64_t a_desc = a_desc0, b_desc = b_desc0;
            for (int gi = 0; gi < n_groups && ok; ++gi) {
                ok = mbar_wait(full_bar(s), phase, abort_flag, &g_gemm_error);
                if (!ok) break;
                if (gi == 0) { trace_stamp(5); block_stamp(trace_kind, 1); }   // first operands landed
#if defined(IDM_TRACE)
                if (blockIdx.x == 0 && gi < 64) { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); g_gemm_mma_trace[trace_kind][gi][0] = t; }
#endif
                tc_fence_after();
                const int nk = min(gk, kb_total - gi * gk);
                uint64_t ad = a_desc, bd = b_desc;
#pragma unroll 4
                for (int k = 0; k < nk; ++k) {
                    tc_mma_bf16_kblock(tmem_d, ad, bd, idesc, acc);
                    acc = 1u;
                    ad += a_step; bd += b_step;
                }
#if defined(IDM_TRACE)
                if (blockIdx.x == 0 && gi < 64) { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); g_gemm_mma_trace[trace_kind][gi][1] = t; }
#endif
                if (gi + stages < n_groups) tc_commit(empty_bar(s));      // the stage is free once these MMAs have read it
                a_desc += (uint64_t)gk * a_step; b_desc += (uint64_t)gk * b_step;
                if (++s == stages) { s = 0; phase ^= 1; a_desc = a_desc0; b_desc = b_desc0; }
            }
            if (ok) tc_commit(accum_bar);         // the accumulator is complete once all MMAs are done
            trace_stamp(6);                       // all MMAs issued
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 0-3): thread = token
        // (an accumulator of 128 rows has row i on lane i; one of 64 rows has row i on lane 32 (i / 16) + i % 16:
        // sixteen tokens on the first sixteen lanes of each warp)
        const bool m64 = gs_mma_rows(tbox) == 64;
        const int tl = m64 ? warp * 16 + lane : warp * 32 + lane;   // the token within the block's 128, and in the step
        const int t = t0 + tl;
        const bool live = t < n_tokens && (!m64 || lane < 16);
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        pdl_wait();
        float* tab = reinterpret_cast<float*>(gen_base + bar_off + GS_BAR_BYTES);      // q/k/v: gq[hd], gk[hd], then a (cos, sin) row per token
        if (EPI == EPI_QKV) {
            // the norm weights and this block's tokens' rows of the rotation table go to shared memory while the
            // product is being made (all four warps carry them): the epilogue then waits for no load
            const QkvArgs& a = e.q;
            const int hd_ = a.hd, rows = min(n_tokens - t0, tbox);
            for (int i = threadIdx.x; i < hd_; i += 128) {
                tab[i] = a.gq ? a.gq[i] : 0.f;
                tab[hd_ + i] = a.gk ? a.gk[i] : 0.f;
            }
            if (a.cs != nullptr)
                for (int i = threadIdx.x; i < rows * hd_; i += 128)
                    tab[2 * hd_ + i] = reinterpret_cast<const float*>(a.cs)[(size_t)t0 * hd_ + i];   // rows of hd / 2 (cos, sin) pairs: hd floats each
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        if (t0 + (m64 ? warp * 16 : warp * 32) < n_tokens) {     // (a warp without tokens has nothing to read)
            size_t place = 0;
            if (EPI == EPI_QKV) {
                const QkvArgs& a = e.q;
                if (live && a.write_cache && f0 + bf > a.n_q * a.hd) {
                    const int pos = a.positions[t];
                    const int r = a.cache.ring ? pos % a.cache.ring : pos;
                    const int page = a.cache.table[(size_t)a.slots[a.token_seq[t]] * a.cache.table_stride + r / IDM_PAGE];
                    place = (size_t)page * a.n_kv * IDM_PAGE + r % IDM_PAGE;   // row of kv-head 0; kv-head g: + g * IDM_PAGE
                }
            }
            // RESIDUAL: the stream's old values of the first 16 features, asked for while the product is still being made
            float4 old4[4];
            const bool have_old = EPI == EPI_RESIDUAL && live && (n_features & 3) == 0 && f0 + 16 <= n_features;
            if (have_old) {
                const float4* p4 = reinterpret_cast<const float4*>(e.out + (size_t)t * n_features + f0);
#pragma unroll
                for (int i = 0; i < 4; ++i) old4[i] = __ldcg(p4 + i);
            }
            if (mbar_wait(accum_bar, 0, abort_flag, &g_gemm_error)) {
                if (threadIdx.x == 0) { trace_stamp(7); block_stamp(trace_kind, 2); }   // accumulator complete
                tc_fence_after();
                if (EPI == EPI_STORE || EPI == EPI_RESIDUAL) {
                    const bool vec = (n_features & 3) == 0;
#pragma unroll 1
                    for (int c0 = 0; c0 < bf; c0 += 16) {
                        if (f0 + c0 >= n_features) break;            // uniform over the block
                        float v[16];
                        tc_ld16(tmem_d + lane_base + (uint32_t)c0, v);
                        if (!live) continue;
                        float* p = e.out + (size_t)t * n_features + f0 + c0;
                        if (vec && f0 + c0 + 16 <= n_features) {
                            float4* p4 = reinterpret_cast<float4*>(p);
                            float4 o[4];
                            if (EPI == EPI_RESIDUAL) {
#pragma unroll
                                for (int i = 0; i < 4; ++i) o[i] = (c0 == 0 && have_old) ? old4[i] : p4[i];
                            }
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                float4 r = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                                if (EPI == EPI_RESIDUAL) { r.x = o[i].x + r.x; r.y = o[i].y + r.y; r.z = o[i].z + r.z; r.w = o[i].w + r.w; }
                                p4[i] = r;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (f0 + c0 + j < n_features) p[j] = EPI == EPI_RESIDUAL ? p[j] + v[j] : v[j];
                        }
                    }
                } else if (EPI == EPI_SWIGLU) {
                    // the tile's columns are gate, up, gate, up, ... of the features f0 / 2 ..; 32 columns are asked
                    // for before the first is waited for
#pragma unroll 1
                    for (int c0 = 0; c0 < bf; c0 += 32) {
                        if (((f0 + c0) >> 1) >= e.inter) break;
                        uint32_t raw[32];
                        tc_ld16_issue(tmem_d + lane_base + (uint32_t)c0, raw);
                        if (c0 + 16 < bf) tc_ld16_issue(tmem_d + lane_base + (uint32_t)(c0 + 16), raw + 16);
                        tc_ld_wait();
                        if (!live) continue;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int fg = (f0 + c0 + 16 * h) >> 1;
                            if (c0 + 16 * h >= bf || fg >= e.inter) break;
                            float y8[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                y8[i] = silu_mul(__uint_as_float(raw[16 * h + 2 * i]), __uint_as_float(raw[16 * h + 2 * i + 1]));
                            T* dst = e.y + (size_t)t * e.inter + fg;
                            if ((e.inter & 7) == 0 && fg + 8 <= e.inter) {
                                store8(dst, y8);
                            } else {
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    if (fg + i < e.inter) from_f32(dst[i], y8[i]);
                            }
                        }
                    }
                } else if (EPI == EPI_QKV) {
                    const QkvArgs& a = e.q;
                    const int hd = a.hd, heads = a.n_q + 2 * a.n_kv;
                    const float2* cs_row = reinterpret_cast<const float2*>(tab + 2 * hd + (live ? tl : 0) * hd);
                    for (int hh = 0; hh < bf / hd; ++hh) {
                        const int head = f0 / hd + hh;
                        if (head >= heads) break;
                        const uint32_t col0 = tmem_d + lane_base + (uint32_t)(hh * hd);
                        const bool is_q = head < a.n_q, is_k = !is_q && head < a.n_q + a.n_kv;
                        const float* gamma = is_q ? (a.gq ? tab : nullptr) : (is_k ? (a.gk ? tab + hd : nullptr) : nullptr);
                        T* dst_a = nullptr; T* dst_b = nullptr;
                        if (live) {
                            if (is_q) {
                                dst_a = a.q_out + ((size_t)t * a.n_q + head) * hd;
                            } else {
                                const int g = is_k ? head - a.n_q : head - a.n_q - a.n_kv;
                                if (a.write_cache) dst_a = (is_k ? a.cache.k : a.cache.v) + (place + (size_t)g * IDM_PAGE) * hd;
                                T* packed = is_k ? a.k_new : a.v_new;
                                if (packed) dst_b = packed + ((size_t)t * a.n_kv + g) * hd;
                            }
                        }
                        const bool rotate = (is_q || is_k) && a.cs != nullptr;
                        if (hd == 128) qkv_tokens_head<128, true>(a, col0, gamma, rotate, cs_row, nullptr, n_tokens, dst_a, dst_b);
                        else if (hd == 64) qkv_tokens_head<64, true>(a, col0, gamma, rotate, cs_row, nullptr, n_tokens, dst_a, dst_b);
                        else qkv_tokens_head<32, true>(a, col0, gamma, rotate, cs_row, nullptr, n_tokens, dst_a, dst_b);
                    }
                }
            }
        }
    }
    if (threadIdx.x == 0) { trace_stamp(8); block_stamp(trace_kind, 3); }   // epilogue done
#if defined(IDM_TRACE)
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        const unsigned int i = atomicAdd(&g_gemm_log_n, 1u) & 2047u;
        unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        g_gemm_log[i][0] = trace_kind; g_gemm_log[i][1] = g_gemm_trace[(g_gemm_trace_base + 0) & 63];
        g_gemm_log[i][2] = g_gemm_trace[(g_gemm_trace_base + 2) & 63]; g_gemm_log[i][3] = t;
    }
#endif
    tc_fence_before();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem_d, (uint32_t)tmem_cols);
}

// ------------------------------------------------------- few tokens, very many features (the lm_head)
// 128 output features on the accumulator's lanes, BN tokens along its columns, one block per 128 features,
// the whole inner axis in one chain.  With some thousand feature tiles there is no lack of blocks, and
// for one token the 32 lanes of a warp store 32 consecutive features: every thread of the four epilogue
// warps has work, where the kernel above would leave all of it to the few threads that own a token.
#define GW_THREADS 192
template <int BN, int STAGES>
struct WideSmem {
    static constexpr int A_BYTES = GT_BM * GT_BK * 2;
    static constexpr int B_BYTES = BN * GT_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 256 + 1024;   // barriers; slack to align to 1024
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(GW_THREADS) gemm_wide_kernel(const __grid_constant__ CUtensorMap map_w,
                                                               const __grid_constant__ CUtensorMap map_x,
                                                               float* out, int n_tokens, int n_features, int kb_total) {
    using S = WideSmem<BN, STAGES>;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    pdl_launch_dependents();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + STAGES * S::STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    const uint32_t accum_bar = bars + 8u * (2 * STAGES);
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + STAGES * S::STAGE_BYTES + 8 * (2 * STAGES + 1));
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = blockIdx.x * GT_BM, t0 = blockIdx.y * BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 5) tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;

    if (warp == 4) {
        if (lane == 0) {
            // weights are written by no kernel: the first stages' tiles are fetched before the wait on the kernel before
            const int early = min(kb_total, STAGES);
            for (int i = 0; i < early; ++i) {
                mbar_expect_tx(full_bar(i), S::STAGE_BYTES);
                tma_load_2d(base + i * S::STAGE_BYTES, &map_w, i * GT_BK, f0, full_bar(i));
            }
            pdl_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(base + i * S::STAGE_BYTES + S::A_BYTES, &map_x, i * GT_BK, t0, full_bar(i));
            int s = 0; uint32_t phase = 0;
            for (int i = early; i < kb_total; ++i) {
                if (!mbar_wait(empty_bar(s), phase, abort_flag, &g_gemm_error)) break;
                mbar_expect_tx(full_bar(s), S::STAGE_BYTES);
                const uint32_t a_dst = base + s * S::STAGE_BYTES;
                tma_load_2d(a_dst, &map_w, i * GT_BK, f0, full_bar(s));
                tma_load_2d(a_dst + S::A_BYTES, &map_x, i * GT_BK, t0, full_bar(s));
                if (++s == STAGES) { s = 0; phase ^= 1; }
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(GT_BM, BN);
            bool ok = true;
            int s = 0; uint32_t phase = 0;
            for (int i = 0; i < kb_total && ok; ++i) {
                ok = mbar_wait(full_bar(s), phase, abort_flag, &g_gemm_error);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = base + s * S::STAGE_BYTES;
                tc_mma_bf16_kblock(tmem_d, umma_desc_kmajor(a_addr), umma_desc_kmajor(a_addr + S::A_BYTES), idesc, i > 0 ? 1u : 0u);
                tc_commit(empty_bar(s));
                if (++s == STAGES) { s = 0; phase ^= 1; }
            }
            if (ok) tc_commit(accum_bar);
        }
    } else {
        pdl_wait();
        if (mbar_wait(accum_bar, 0, abort_flag, &g_gemm_error)) {
            tc_fence_after();
            const int f = f0 + warp * 32 + lane;                   // feature = accumulator lane
            const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (t0 + c0 >= n_tokens) break;                    // warp-uniform
                float v[16];
                tc_ld16(tmem_d + lane_base + (uint32_t)c0, v);
                if (f < n_features) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = t0 + c0 + j;
                        if (t < n_tokens) out[(size_t)t * n_features + f] = v[j];
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem_d, TMEM_COLS);
}

template <int BN, int STAGES>
static int launch_wide(const void* x, const void* w, float* out, int M, int N, int K, cudaStream_t stream);

// ------------------------------------------------------------------------------ host
// a [rows, k] bfloat16 row-major matrix, tiles of [box_rows, 64], 128-byte swizzle, zero fill outside
static int make_map(CUtensorMap* map, const void* ptr, int rows, int k, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    cuuint32_t box[2] = {GT_BK, (cuuint32_t)box_rows};
    const int r = tc_make_map_bf16(map, ptr, 2, dims, strides, box);
    IDM_REQUIRE(r == 0, "gemm: cuTensorMapEncodeTiled failed with %d (rows=%d k=%d box=%d)", r, rows, k, box_rows);
    return 0;
}

template <int BN, int STAGES>
static int launch_wide(const void* x, const void* w, float* out, int M, int N, int K, cudaStream_t stream) {
    using S = WideSmem<BN, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_wide_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        IDM_REQUIRE(err == cudaSuccess, "gemm: cannot get %d bytes of shared memory: %s", S::TOTAL, cudaGetErrorString(err));
        configured = true;
    }
    CUtensorMap mw, mx;
    if (make_map(&mw, w, N, K, GT_BM)) return 1;
    if (make_map(&mx, x, M, K, BN)) return 1;
    dim3 grid((N + GT_BM - 1) / GT_BM, (M + BN - 1) / BN);
    idm_launch(gemm_wide_kernel<BN, STAGES>, grid, dim3(GW_THREADS), S::TOTAL, stream, mw, mx, out, M, N, (K + GT_BK - 1) / GT_BK);
    IDM_LAUNCH_CHECK("gemm_wide");
    return 0;
}

static int device_sms() {
    static int n_sm = 0;
    if (n_sm == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        if (n_sm <= 0) n_sm = 148;
    }
    return n_sm;
}

// Features per block of the kernel for few tokens: the slice width that leaves the fullest SM the
// fewest bytes to fetch (its blocks' weight slices plus the activations each of them reads again).
// Wider than 128 features is never useful; the q/k/v epilogue needs whole heads.
static int small_slice(int N, int tbox, int unit, int token_tiles = 1) {
    const int sms = device_sms();
    int best = 0;
    long long best_cost = 0;
    for (int bf = 16; bf <= 128; bf += 16) {
        if (bf % unit) continue;
        const long long blocks = (long long)((N + bf - 1) / bf) * token_tiles;
        const long long cost = ((blocks + sms - 1) / sms) * (tbox + bf);
        if (best == 0 || cost < best_cost) { best = bf; best_cost = cost; }
    }
    return best ? best : unit;
}

// The same matrix as [k within a k-block (64), row, k-block]: a box of [64, box_rows, box_kb] brings
// box_kb k-blocks of box_rows rows with one request, each k-block's rows together in shared memory.
// Only for inner sizes that are whole k-blocks (a row's last, partial block would run into the next row).
static int make_map_grouped(CUtensorMap* map, const void* ptr, int rows, int k, int box_rows, int box_kb) {
    cuuint64_t dims[3] = {GT_BK, (cuuint64_t)rows, (cuuint64_t)(k / GT_BK)};
    cuuint64_t strides[2] = {(cuuint64_t)k * 2, GT_BK * 2};
    cuuint32_t box[3] = {GT_BK, (cuuint32_t)box_rows, (cuuint32_t)box_kb};
    const int r = tc_make_map_bf16(map, ptr, 3, dims, strides, box);
    IDM_REQUIRE(r == 0, "gemm: cuTensorMapEncodeTiled failed with %d (rows=%d k=%d box=%d x %d k-blocks)", r, rows, k, box_rows,
                box_kb);
    return 0;
}

static int g_small_bf = 0, g_small_budget = 200 * 1024, g_small_gk = 0;
// (for measurements: fix the slice width / the bytes of shared memory a block's ring may take / k-blocks per request)
extern "C" void idm_gemm_set_small(int bf, int ring_bytes, int gk) {
    g_small_bf = bf;
    if (ring_bytes > 0) g_small_budget = ring_bytes;
    g_small_gk = gk;
}

template <int EPI>
static int launch_small(const void* x, const void* w, const GemmEpi& e, int M, int N, int K, cudaStream_t stream) {
    const int kb_total = (K + GT_BK - 1) / GT_BK;
    const int tbox = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    int unit = 16;
    if (EPI == EPI_QKV) unit = e.q.hd < 16 ? 16 : e.q.hd;
    const int token_tiles = (M + 127) / 128;
    int bf = g_small_bf && g_small_bf % unit == 0 ? g_small_bf : small_slice(N, tbox, unit, token_tiles);
    if (EPI == EPI_QKV && bf < e.q.hd) bf = e.q.hd;
    const int kb_bytes = (tbox + bf) * 128;                       // one k-block of both operands
    // k-blocks per request and barrier: up to 64 KB, at most 8, and no more than half of the inner axis (the thread
    // that issues the MMAs spends ~0.2 us per barrier on waiting and bookkeeping, as much as eight MMAs take)
    int gk = g_small_gk ? g_small_gk : 64 * 1024 / kb_bytes;
    if (gk > 8) gk = 8;
    if (gk > kb_total / 2) gk = kb_total / 2;
    if (gk < 1) gk = 1;
    const int grouped = (K % GT_BK == 0 && gk > 1) ? 1 : 0;
    if (!grouped && K % GT_BK) gk = 1;
    const int n_groups = (kb_total + gk - 1) / gk;
    int stages = (g_small_budget - (EPI == EPI_QKV ? (2 + tbox) * e.q.hd * 4 : 0)) / (gk * kb_bytes);
    if (stages < 2) stages = 2;
    if (stages > n_groups) stages = n_groups;
    if (stages > GS_MAX_STAGES) stages = GS_MAX_STAGES;
    int tmem_cols = 32;
    while (tmem_cols < bf) tmem_cols *= 2;
    // behind the barriers: the q/k/v epilogue's tables (two norm weights, a row of the rotation table per token)
    const int tab_bytes = EPI == EPI_QKV ? (2 + tbox) * e.q.hd * 4 : 0;
    const int smem = (int)gs_data_bytes(tbox, bf, gk, stages) + GS_BAR_BYTES + tab_bytes + 1024;   // + slack to align to 1024
    IDM_REQUIRE(smem <= 227 * 1024, "gemm: %d bytes of shared memory for %d tokens x %d features a block", smem, tbox, bf);
    static int configured = 0;
    if (smem > configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_small_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        IDM_REQUIRE(err == cudaSuccess, "gemm: cannot get %d bytes of shared memory: %s", smem, cudaGetErrorString(err));
        configured = smem;
    }
    CUtensorMap mw, mx;
    if (grouped) {
        if (make_map_grouped(&mw, w, N, K, bf, gk)) return 1;
        if (make_map_grouped(&mx, x, M, K, tbox, gk)) return 1;
    } else {
        if (make_map(&mw, w, N, K, bf)) return 1;
        if (make_map(&mx, x, M, K, tbox)) return 1;
    }
    idm_launch(gemm_small_kernel<EPI>, dim3((N + bf - 1) / bf, token_tiles), dim3(GS_THREADS), (size_t)smem, stream, mw, mx, e, M, N,
               kb_total, bf, tbox, gk, grouped, stages, tmem_cols);
    IDM_LAUNCH_CHECK("gemm_small");
    return 0;
}

// Up to 128 tokens the kernel with the tokens on the lanes runs (fewer: for measurements).  Beyond that it
// takes a block per 128 tokens and slice, and runs where the persistent kernels would have no more than
// `g_gemm_small_tiles` tiles for their one block per SM (measured at 129-512 tokens: products of 1024
// features, 16-32 tiles, 18 -> 14 us and 22 -> 16 us, a whole prompt step of 0.6B sizes 2.2-2.6 -> 1.9-2.3 ms;
// 4096 features at 129-256 tokens, 64 tiles, 4 % of a step; with more tiles the persistent kernels win).
static int g_gemm_small_max = 128, g_gemm_small_tiles = 64;
extern "C" void idm_gemm_set_small_max(int tokens) { g_gemm_small_max = tokens < 0 ? 0 : tokens > 128 ? 128 : tokens; }
extern "C" void idm_gemm_set_small_tiles(int tiles) { g_gemm_small_tiles = tiles < 0 ? 0 : tiles; }
// Whether products of many tokens may run on pairs of blocks (cta_group::2), and from how many tiles of 256 x 256 on.
static int g_gemm_pair = 1, g_gemm_pair_tiles = 60;
extern "C" void idm_gemm_set_pair(int on, int tiles) {
    g_gemm_pair = on ? 1 : 0;
    if (tiles > 0) g_gemm_pair_tiles = tiles;
}
// From how many tiles of 256 tokens on the persistent kernel takes those instead of tiles of 128 tokens.
static int g_gemm_wide_tiles = 120;
extern "C" void idm_gemm_set_wide_tiles(int tiles) { g_gemm_wide_tiles = tiles < 1 ? 1 : tiles; }
// From how many output features on a plain product of few tokens runs with the features on the lanes.
static int g_gemm_wide_from = 16384;
extern "C" void idm_gemm_set_wide_from(int features) { g_gemm_wide_from = features; }

template <int EPI>
static int gemm_any(const void* x, const void* w, GemmEpi e, int M, int N, int K, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    IDM_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    IDM_REQUIRE(K % 8 == 0, "gemm: the inner size %d must be a multiple of 8 (rows start on 16-byte borders)", K);
    IDM_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm: operands must be 16-byte aligned");
    const int kb_total = (K + GT_BK - 1) / GT_BK;
    if (EPI == EPI_QKV) {
        auto on32 = [](const void* p) { return ((uintptr_t)p & 31) == 0; };   // (null counts: that output is not written)
        IDM_REQUIRE(e.q.hd == 32 || e.q.hd == 64 || e.q.hd == 128, "gemm_qkv: head_dim=%d has no fused epilogue (32, 64, 128)",
                    e.q.hd);
        IDM_REQUIRE(on32(e.q.q_out) && on32(e.q.k_new) && on32(e.q.v_new) && on32(e.q.cache.k) && on32(e.q.cache.v) &&
                    on32(e.q.cs) && on32(e.q.gq) && on32(e.q.gk), "gemm_qkv: outputs, tables and norm weights must lie on 32-byte borders");
    }
    const int token_tiles = (M + 127) / 128;
    const long long persistent_tiles = (long long)((N + (EPI == EPI_QKV ? 255 : 127)) / (EPI == EPI_QKV ? 256 : 128)) * token_tiles;
    if (M <= g_gemm_small_max || (M > 128 && persistent_tiles <= g_gemm_small_tiles)) {
        if (EPI == EPI_STORE && N >= g_gemm_wide_from && M <= 128) {
            // some hundred feature tiles: features on the lanes, every epilogue thread at work
            if (M <= 16) return launch_wide<16, 6>(x, w, e.out, M, N, K, stream);
            if (M <= 32) return launch_wide<32, 6>(x, w, e.out, M, N, K, stream);
            if (M <= 64) return launch_wide<64, 4>(x, w, e.out, M, N, K, stream);
            return launch_wide<128, 3>(x, w, e.out, M, N, K, stream);
        }
        return launch_small<EPI>(x, w, e, M, N, K, stream);
    }
    CUtensorMap mw, mx;
    if (EPI == EPI_QKV) {
        // many tokens: tokens on the accumulator's lanes, 256 features (whole heads) per tile
        if (make_map(&mw, w, N, K, GQ_BN)) return 1;
        if (make_map(&mx, x, M, K, GT_BM)) return 1;
        return launch_qkv_tokens(mw, mx, e, M, N, kb_total, stream);
    }
    // many tokens, a product that is stored or added to the stream, tiles enough for every pair of SMs: pairs of blocks
    // on tiles of 256 features x 256 tokens (measured at 8B sizes, 6 208 tokens: o 168 -> 151 us, down 485 -> 442 us;
    // at 32B sizes level; the SwiGLU product is as fast on single blocks once its walk stays in the L2, and products
    // of 1 024 features have too few such tiles)
    if constexpr (EPI == EPI_STORE || EPI == EPI_RESIDUAL) {
        if (g_gemm_pair && (long long)((N + 2 * GT_BM - 1) / (2 * GT_BM)) * ((M + 255) / 256) >= g_gemm_pair_tiles) {
            if (make_map(&mw, w, N, K, GT_BM)) return 1;
            if (make_map(&mx, x, M, K, 128)) return 1;
            return launch_pair<256, 6, EPI>(mw, mx, e, M, N, kb_total, stream);
        }
    }
    // many tokens: the persistent kernel; 256-token tiles unless 128 fill more of the SMs
    const int tiles_x = (N + GT_BM - 1) / GT_BM;
    const bool wide = (long long)tiles_x * ((M + 255) / 256) >= g_gemm_wide_tiles;
    if (make_map(&mw, w, N, K, GT_BM)) return 1;
    if (make_map(&mx, x, M, K, wide ? 256 : 128)) return 1;
    return wide ? launch_persistent<256, 4, EPI>(mw, mx, e, M, N, kb_total, stream)
                : launch_persistent<128, 6, EPI>(mw, mx, e, M, N, kb_total, stream);
}

// out [M, N] = x . w^T (32-bit)
extern "C" int idm_gemm_bf16(const void* x, const void* w, float* out, int M, int N, int K, cudaStream_t stream) {
    GemmEpi e = {};
    e.out = out;
    return gemm_any<EPI_STORE>(x, w, e, M, N, K, stream);
}

// h [M, N] += x . w^T (the 32-bit residual sum)
extern "C" int idm_gemm_bf16_residual(const void* x, const void* w, float* h, int M, int N, int K, cudaStream_t stream) {
    GemmEpi e = {};
    e.out = h;
    return gemm_any<EPI_RESIDUAL>(x, w, e, M, N, K, stream);
}

// y [M, inter] = silu(x . gate^T) * (x . up^T); w_tiled [tiles * 128, K]: rows 2 f and 2 f + 1 are the gate
// and the up row of feature f (rows past 2 * inter are zero)
extern "C" int idm_gemm_bf16_swiglu(const void* x, const void* w_tiled, void* y, int M, int inter, int K,
                                    cudaStream_t stream) {
    GemmEpi e = {};
    e.y = (T*)y; e.inter = inter;
    const int tiles = (inter + 63) / 64;
    return gemm_any<EPI_SWIGLU>(x, w_tiled, e, M, tiles * GT_BM, K, stream);
}

// The fused q/k/v projection with the per-head finish (norm, rotation, q out, cache write); head_dim 32, 64 or 128
extern "C" int idm_gemm_bf16_qkv(const void* x, const void* w, int M, int K, int n_q, int n_kv, int hd,
                                 const float* gq, const float* gk, float eps, const float* cs, const float* cs_by_dim,
                                 void* q_out, void* k_new, void* v_new, void* k_pool, void* v_pool, const int* table,
                                 int table_stride, int ring, const int* token_seq, const int* positions,
                                 const int* slots, cudaStream_t stream) {
    GemmEpi e = {};
    QkvArgs& a = e.q;
    a.qkv = nullptr; a.n_partials = 0; a.partial_stride = 0;
    a.n_tokens = M; a.n_q = n_q; a.n_kv = n_kv; a.hd = hd;
    a.gq = gq; a.gk = gk; a.eps = eps; a.inv_hd = 1.0f / (float)hd; a.cs = (const float2*)cs;
    a.cs_by_dim = (const float2*)cs_by_dim;
    a.q_out = (T*)q_out; a.k_new = (T*)k_new; a.v_new = (T*)v_new;
    a.cache = KVAddr{(T*)k_pool, (T*)v_pool, table, table_stride, ring, n_kv, hd};
    a.write_cache = k_pool != nullptr;
    a.token_seq = token_seq; a.positions = positions; a.slots = slots; a.tiles4 = 0;
    return gemm_any<EPI_QKV>(x, w, e, M, (n_q + 2 * n_kv) * hd, K, stream);
}

// ------------------------------------------------------------------- the bounded wait, by itself
// The wait every kernel here uses, made to run out: one block's roles wait on a barrier that nothing
// arrives at, with a limit of `limit_cycles` instead of the two seconds of real kernels.  The first role
// whose wait runs out sets the block's abort flag and the error word; the others see the flag and leave
// too; tensor memory is freed and the kernel ends normally (no trap, nothing left hanging).  out[0]: 1 if
// the wait was reported as run out, out[1]: cycles waited, out[2]: 1 if the second role left by the flag.
__global__ void __launch_bounds__(64) wait_probe_kernel(long long limit_cycles, int arrive, int* out) {
    __shared__ __align__(8) unsigned long long bar_mem;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const uint32_t bar = smem_u32(&bar_mem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) { mbar_init(bar, 1); abort_flag = 0; mbar_init_fence(); }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_slot), 32);          // held while waiting, as a real kernel holds it
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (arrive && threadIdx.x == 33) mbar_arrive(bar);            // (the same kernel with the arrival: the wait returns true)
    if (lane == 0) {
        const long long t0 = clock64();
        // warp 1's limit is far away: it leaves because warp 0 gave up, not because its own time ran out
        const bool ok = mbar_wait_limit(bar, 0, (volatile int*)&abort_flag, &g_gemm_error, warp == 0 ? limit_cycles : TC_WAIT_CYCLES);
        if (warp == 0) { out[0] = ok ? 0 : 1; out[1] = (int)min((long long)0x7fffffff, clock64() - t0); }
        else out[2] = ok ? 0 : 1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_slot, 32);
}

// Launches the probe; out: three words on the device (see above).  The library's error word is set when
// the wait runs out (idm_gemm_status reports and clears it).
extern "C" int idm_wait_probe(long long limit_cycles, int arrive, int* out, cudaStream_t stream) {
    IDM_REQUIRE(limit_cycles > 0 && limit_cycles <= 2000000000ll, "wait_probe: limit of %lld cycles (1 .. 2e9)", limit_cycles);
    IDM_REQUIRE(out != nullptr, "wait_probe: no place for the result");
    wait_probe_kernel<<<1, 64, 0, stream>>>(limit_cycles, arrive, out);
    IDM_LAUNCH_CHECK("wait_probe");
    return 0;
}

// 0, or 1 if any block's bounded wait ran out since the last call (reads the flag: synchronises)
extern "C" int idm_gemm_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    return v;
}

#endif  // IDM_BF16
