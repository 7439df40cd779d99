// out[p, t, f] = sum over the p-th slice of k of x[t, k] * w[f, k]   (bfloat16 in, 32-bit out)
//
// The dense projections of the model (q/k/v, o, gate/up, down, lm_head) on the 5th-generation
// tensor cores: tcgen05.mma issued by one thread, operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle, no multicast), the accumulator in tensor memory, read
// back with tcgen05.ld.  The reference sends these products to a library (torch._int_mm,
// src/detllm/backends.py:88-135).
//
// Roles in a block of 192 threads: warps 0-3 read the accumulator and store it (the epilogue),
// warp 4 issues TMA loads, warp 5 allocates tensor memory and issues the MMAs.
//
// Tiling.  The MMA's M axis carries 128 output features (rows of w), its N axis BN tokens
// (rows of x), so an accumulator lane is a feature and a column is a token: for one token the 32
// lanes of a warp store 32 consecutive features, 128 contiguous bytes, with no staging.  K is
// walked in blocks of 64 (one 128-byte swizzle row); the inner axis may be split over
// gridDim.z blocks, each writing its own partial sum to out[p] (the consumer adds them in
// ascending p).  How K is split depends on the layer's shape only, and an output element's value
// depends on its own row of x and row of w only.
//
// Epilogues.  PARTIAL stores each K-slice's 32-bit tile to out[p].  The fused epilogues produce the
// finished result inside the kernel: STORE (32-bit [M, N]), RESIDUAL (h[t, f] += result, the
// 32-bit residual sum), SWIGLU (bfloat16 y = silu(gate) * up; the weight's rows alternate: gate row
// of a feature, then its up row, so a 128-row tile holds 64 features) and QKV (per-head
// q/k norm, rotation, q out and cache write; a tile of 128 features must hold whole heads).  With K
// split, every slice writes its tile to a workspace and the block that arrives last for the tile
// (a counter it sets back to zero) adds the slices in ascending order and runs the epilogue, so the
// value does not depend on which block that is.  (Up to 64 tokens the slices are added inside a
// thread-block cluster instead; above 256 tokens nothing is split and the persistent kernels further
// down run: see there.)
//
// Every wait on an mbarrier is bounded by a cycle count; a wait that runs out sets the error flag
// (idm_gemm_status), all roles leave their loops, tensor memory is freed and the block returns.
#include "common.cuh"

#if defined(IDM_BF16)

#include "tcgen05.cuh"
#include "qkv_finish.cuh"

#define GT_BM 128            // features per tile (MMA M)
#define GT_BK 64             // k per stage: 64 bf16 = 128 bytes = one swizzle row
#define GT_UMMA_K 16
#define GT_THREADS 192
#define GT_COUNTER_SLOTS 65536

__device__ int g_gemm_error = 0;

enum { EPI_PARTIAL = 0, EPI_STORE = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3, EPI_QKV = 4 };

struct GemmEpi {
    float* out;          // PARTIAL: [splits, M, N]; STORE: [M, N]; RESIDUAL: the residual stream [M, N]
    float* ws;           // workspace [splits, M, N] of the fused epilogues when K is split
    int* counters;       // one per output tile, zero between launches
    T* y; int inter;     // SWIGLU: y [M, inter]
    QkvArgs q;           // QKV
};

__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // warps 0-3

// ---- thread-block clusters: all blocks of a cluster run together and can read each other's shared memory
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The finished row of 128 features of one token, four consecutive features per lane, through the
// fused epilogues (the cluster path: each block of a cluster finishes some of the tile's rows).
// What a row's epilogue reads besides the product, fetched while the product is still being made: the
// residual stream's old values (RESIDUAL) or the token's (cos, sin) (QKV).
struct RowOperand { float4 a, b; bool have; };
template <int EPI>
__device__ __forceinline__ RowOperand row_operand(const GemmEpi& e, const Tile4Lane& L, int t, int f0, int lane, int n_features) {
    RowOperand r;
    r.a = r.b = make_float4(0.f, 0.f, 0.f, 0.f);
    r.have = true;
    if (EPI == EPI_RESIDUAL) {
        const int f = f0 + lane * 4;
        if (f < n_features) r.a = __ldcg(reinterpret_cast<const float4*>(e.out + (size_t)t * n_features + f));
    } else if (EPI == EPI_QKV) {
        const float4* c4 = qkv_tile4_cs(e.q, L, t, f0, lane);
        if (c4) { r.a = __ldg(c4); r.b = __ldg(c4 + 1); }
    }
    return r;
}

template <int EPI>
__device__ __forceinline__ void epilogue_row(const GemmEpi& e, float4 v, int t, int f0, int tile_x, int lane,
                                             int n_features, const int* meta_row, const Tile4Lane& L, const RowOperand& pre) {
    const int f = f0 + lane * 4;
    if (EPI == EPI_STORE || EPI == EPI_RESIDUAL) {
        if (f < n_features) {
            float4* p = reinterpret_cast<float4*>(e.out + (size_t)t * n_features + f);
            if (EPI == EPI_RESIDUAL) { const float4 o = pre.a; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
            *p = v;
        }
    } else if (EPI == EPI_SWIGLU) {
        // a lane's four features of the tile are gate, up, gate, up of two features of y
        const int fg = tile_x * 64 + lane * 2;
        T* y = e.y + (size_t)t * e.inter + fg;
        if (fg + 0 < e.inter) from_f32(y[0], silu_mul(v.x, v.y));
        if (fg + 1 < e.inter) from_f32(y[1], silu_mul(v.z, v.w));
    } else if (EPI == EPI_QKV) {
        qkv_finish_tile4_pre(e.q, L, v, t, f0, lane, meta_row[0], meta_row[1], pre.a, pre.b);
    }
}

// ---------------------------------------------------------------------------- kernel
template <int BN, int STAGES, bool PUSH = false>
struct GemmSmem {
    static constexpr int A_BYTES = GT_BM * GT_BK * 2;
    static constexpr int B_BYTES = BN * GT_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BARRIER_BYTES = 2048;          // barriers and flags, then per-token cache rows (QKV)
    // PUSH (the cluster path): behind the barriers, the rows this block finishes, one copy per block of
    // the cluster (others write them while this block's ring may still be in use): S x ceil(BN / S) rows
    // of 128 floats for a cluster of S <= 16 blocks
    static constexpr int recv_rows() {
        int most = 0;
        for (int s = 2; s <= 16; ++s) { const int r = s * ((BN + s - 1) / s); most = r > most ? r : most; }
        return most;
    }
    static constexpr int RECV_BYTES = PUSH ? recv_rows() * GT_BM * 4 : 0;
    static constexpr int RECV_BAR = 512;                // offset of the arrival barrier inside the barrier area
    static constexpr int TOTAL = STAGES * STAGE_BYTES + BARRIER_BYTES + RECV_BYTES + 1024;   // + slack to align to 1024
};

template <int BN, int STAGES, int EPI, bool CL>
__global__ void __launch_bounds__(GT_THREADS) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                  const __grid_constant__ CUtensorMap map_x,
                                                                  const GemmEpi e, int n_tokens,
                                                                  int n_features, int kb_total, int kb_per_split) {
    constexpr bool PUSH = CL;
    using S = GemmSmem<BN, STAGES, PUSH>;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;          // allocation: a power of two >= 32
    pdl_launch_dependents();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + STAGES * S::STAGE_BYTES;
    // barriers: full[STAGES], empty[STAGES], accumulator ready; then the tensor-memory address and the abort flag
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    const uint32_t accum_bar = bars + 8u * (2 * STAGES);
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gen_base + STAGES * S::STAGE_BYTES + 8 * (2 * STAGES + 1));
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    const uint32_t recv_bar = bars + S::RECV_BAR;         // PUSH: all slices of this block's rows have arrived
    const uint32_t recv_base = bars + S::BARRIER_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = blockIdx.x * GT_BM, t0 = blockIdx.y * BN;
    const int kb0 = blockIdx.z * kb_per_split;
    const int kb_n = min(kb_per_split, kb_total - kb0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(accum_bar, 1);
        if (PUSH) {
            // the rows this block finishes arrive as bytes: 128 floats per row from every block of the cluster
            const int S_ = (int)gridDim.z, rank = (int)cluster_rank(), cols = min(BN, n_tokens - t0);
            mbar_init(recv_bar, 1);
            if (rank < cols) mbar_expect_tx(recv_bar, (uint32_t)(S_ * ((cols - rank + S_ - 1) / S_) * GT_BM * 4));
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (PUSH) cluster_sync_all();                         // every block's arrival barrier exists before anyone arrives there
    const uint32_t tmem_d = *tmem_slot;
    Tile4Lane tl4 = {};                                          // (cluster path, warps 0-3: see the epilogue)
    RowOperand pre = {};

    if (warp == 4) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // Weights are written by no kernel: the first stages' weight tiles are fetched before
            // the wait on the previous kernel; the activations follow after it.
            const int early = min(kb_n, STAGES);
            for (int i = 0; i < early; ++i) {
                mbar_expect_tx(full_bar(i), S::STAGE_BYTES);
                tma_load_2d(base + i * S::STAGE_BYTES, &map_w, (kb0 + i) * GT_BK, f0, full_bar(i));
            }
            pdl_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(base + i * S::STAGE_BYTES + S::A_BYTES, &map_x, (kb0 + i) * GT_BK, t0, full_bar(i));
            for (int i = early; i < kb_n; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait(empty_bar(s), ((i / STAGES) & 1) ^ 1, abort_flag, &g_gemm_error)) break;
                mbar_expect_tx(full_bar(s), S::STAGE_BYTES);
                const uint32_t a_dst = base + s * S::STAGE_BYTES;
                tma_load_2d(a_dst, &map_w, (kb0 + i) * GT_BK, f0, full_bar(s));
                tma_load_2d(a_dst + S::A_BYTES, &map_x, (kb0 + i) * GT_BK, t0, full_bar(s));
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(GT_BM, BN);
            bool ok = true;
            for (int i = 0; i < kb_n && ok; ++i) {
                const int s = i % STAGES;
                ok = mbar_wait(full_bar(s), (i / STAGES) & 1, abort_flag, &g_gemm_error);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_addr = base + s * S::STAGE_BYTES;
                const uint64_t a_desc = umma_desc_kmajor(a_addr), b_desc = umma_desc_kmajor(a_addr + S::A_BYTES);
#pragma unroll
                for (int k = 0; k < GT_BK / GT_UMMA_K; ++k) {
                    // 16 k = 32 bytes further along the swizzled row: +2 in units of 16 bytes
                    tc_mma_bf16(tmem_d, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit(empty_bar(s));          // the stage is free once these MMAs have read it
            }
            if (ok) tc_commit(accum_bar);         // the accumulator is complete once all MMAs are done
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 0-3)
        if (EPI == EPI_QKV) {
            // while the main loop runs: where each token's key/value row lies in the cache
            pdl_wait();
            int* meta = (int*)(gen_base + STAGES * S::STAGE_BYTES + 1024);
            const int tl = warp * 32 + lane;
            if (tl < BN && t0 + tl < n_tokens && e.q.write_cache) {
                const int t = t0 + tl;
                const int pos = e.q.positions[t];
                const int r = e.q.cache.ring ? pos % e.q.cache.ring : pos;
                meta[2 * tl] = e.q.cache.table[(size_t)e.q.slots[e.q.token_seq[t]] * e.q.cache.table_stride + r / IDM_PAGE];
                meta[2 * tl + 1] = r % IDM_PAGE;
            }
        }
        // cluster path: what the first row this warp will finish needs besides the product, asked for now
        if (CL && EPI != EPI_PARTIAL) {
            pdl_wait();
            if (EPI == EPI_QKV) tl4 = qkv_tile4_lane(e.q, lane);
            const int t_first = (int)cluster_rank() + (int)gridDim.z * warp;
            if (t_first < min(BN, n_tokens - t0)) pre = row_operand<EPI>(e, tl4, t0 + t_first, f0, lane, n_features);
        }
        if (mbar_wait(accum_bar, 0, abort_flag, &g_gemm_error)) {
            tc_fence_after();
            pdl_wait();                                           // (already satisfied: the activations came after it)
            const int fl = warp * 32 + lane;                      // feature within the tile = accumulator lane
            const int f = f0 + fl;
            const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
            const size_t mn = (size_t)n_tokens * n_features;
            const int splits = gridDim.z;
            if (EPI == EPI_PARTIAL) {
                float* dst = e.out + blockIdx.z * mn;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    if (t0 + c0 >= n_tokens) break;               // warp-uniform
                    float v[16];
                    tc_ld16(tmem_d + lane_base + (uint32_t)c0, v);
                    if (f < n_features) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int t = t0 + c0 + j;
                            if (t < n_tokens) dst[(size_t)t * n_features + f] = v[j];
                        }
                    }
                }
            } else if (PUSH) {
                // Cluster path (up to 64 tokens, K split).  Block r of the cluster finishes the token rows r, r + S, ...:
                // every block sends its K-slice of those rows into r's shared memory (copy number = the
                // sender's rank) with stores that count their bytes at r's barrier; r waits for the bytes
                // of its rows, adds the S copies in ascending order and runs the epilogue.  No block waits
                // for any other than through that barrier, and no sender waits at all.
                const int S_ = (int)gridDim.z, rank = (int)cluster_rank();
                const int cols = min(BN, n_tokens - t0);
                const int slots = (BN + S_ - 1) / S_;             // rows a block can own
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    if (c0 >= cols) break;
                    float v[16];
                    tc_ld16(tmem_d + lane_base + (uint32_t)c0, v);
                    int owner = c0 % S_, slot = c0 / S_;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (c0 + j < cols)
                            st_async_f32(recv_base + (uint32_t)(((rank * slots + slot) * GT_BM + fl) * 4), recv_bar, (uint32_t)owner, v[j]);
                        if (++owner == S_) { owner = 0; ++slot; }
                    }
                }
                if (rank < cols && mbar_wait_cluster(recv_bar, 0, abort_flag, &g_gemm_error)) {
                    const int* meta = (const int*)(gen_base + STAGES * S::STAGE_BYTES + 1024);
                    const float* recv = (const float*)(gen_base + STAGES * S::STAGE_BYTES + S::BARRIER_BYTES);
                    for (int slot = warp; rank + S_ * slot < cols; slot += 4) {
                        const int t = rank + S_ * slot;
                        const RowOperand op = (slot == warp && pre.have) ? pre : row_operand<EPI>(e, tl4, t0 + t, f0, lane, n_features);
                        float4 part[16];
#pragma unroll
                        for (int r = 0; r < 16; ++r)
                            if (r < S_) part[r] = *reinterpret_cast<const float4*>(recv + ((r * slots + slot) * GT_BM + lane * 4));
                        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int r = 0; r < 16; ++r)
                            if (r < S_) { acc.x += part[r].x; acc.y += part[r].y; acc.z += part[r].z; acc.w += part[r].w; }
                        epilogue_row<EPI>(e, acc, t0 + t, f0, blockIdx.x, lane, n_features, meta + 2 * t, tl4, op);
                    }
                }
            } else {
                float* xs = (float*)gen_base;                     // [BN][128] tile; the pipeline's stages are free now
                const int cols = min(BN, n_tokens - t0);
                bool last = true;
                if (splits > 1) {
                    float* dst = e.ws + blockIdx.z * mn;
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 16) {
                        if (t0 + c0 >= n_tokens) break;
                        float v[16];
                        tc_ld16(tmem_d + lane_base + (uint32_t)c0, v);
                        if (f < n_features) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int t = t0 + c0 + j;
                                if (t < n_tokens) dst[(size_t)t * n_features + f] = v[j];
                            }
                        }
                    }
                    __threadfence();
                    epi_sync();
                    volatile int* flag = (volatile int*)(tmem_slot + 2);
                    if (threadIdx.x == 0) {
                        int* ctr = e.counters + blockIdx.y * gridDim.x + blockIdx.x;
                        const int prev = atomicAdd(ctr, 1);
                        *flag = prev == splits - 1;
                        if (prev == splits - 1) *ctr = 0;
                    }
                    epi_sync();
                    last = *flag != 0;
                    if (last) {
                        // Add the slices' tiles in ascending order into the shared-memory tile.  A warp
                        // takes whole token rows; eight slices' loads are in flight together.
                        __threadfence();
                        if ((n_features & 3) == 0) {
                            const int f4 = f0 + lane * 4;
                            for (int t = warp; t < cols; t += 4) {
                                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                                if (f4 < n_features) {
                                    const float* src = e.ws + (size_t)(t0 + t) * n_features + f4;
                                    for (int z0 = 0; z0 < splits; z0 += 8) {
                                        float4 part[8];
#pragma unroll
                                        for (int i = 0; i < 8; ++i)
                                            if (z0 + i < splits) part[i] = __ldcg(reinterpret_cast<const float4*>(src + (z0 + i) * mn));
#pragma unroll
                                        for (int i = 0; i < 8; ++i)
                                            if (z0 + i < splits) {
                                                acc.x += part[i].x; acc.y += part[i].y; acc.z += part[i].z; acc.w += part[i].w;
                                            }
                                    }
                                }
                                *reinterpret_cast<float4*>(xs + t * GT_BM + lane * 4) = acc;
                            }
                        } else {
                            for (int t = warp; t < cols; t += 4)
                                for (int i = lane; i < GT_BM; i += 32) {
                                    float acc = 0.f;
                                    if (f0 + i < n_features)
                                        acc = add_partials(0.f, e.ws, splits, mn, (size_t)(t0 + t) * n_features + f0 + i);
                                    xs[t * GT_BM + i] = acc;
                                }
                        }
                        epi_sync();
                    }
                } else if (EPI == EPI_SWIGLU || EPI == EPI_QKV) {
                    // the tile from tensor memory into shared memory: these epilogues work across lanes
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 16) {
                        if (t0 + c0 >= n_tokens) break;
                        float v[16];
                        tc_ld16(tmem_d + lane_base + (uint32_t)c0, v);
#pragma unroll
                        for (int j = 0; j < 16; ++j) xs[(c0 + j) * GT_BM + fl] = v[j];
                    }
                    epi_sync();
                }
                if (last) {
                    if (EPI == EPI_STORE || EPI == EPI_RESIDUAL) {
                        if (splits > 1) {
                            if (f < n_features)
                                for (int c0 = 0; c0 < cols; c0 += 16) {            // 16 tokens' loads go out together
                                    float old[16];
#pragma unroll
                                    for (int j = 0; j < 16; ++j)
                                        old[j] = (EPI == EPI_RESIDUAL && c0 + j < cols)
                                                     ? e.out[(size_t)(t0 + c0 + j) * n_features + f] : 0.f;
#pragma unroll
                                    for (int j = 0; j < 16; ++j)
                                        if (c0 + j < cols)
                                            e.out[(size_t)(t0 + c0 + j) * n_features + f] = old[j] + xs[(c0 + j) * GT_BM + fl];
                                }
                        } else {
#pragma unroll 1
                            for (int c0 = 0; c0 < BN; c0 += 32) {     // 32 tokens at a time: their loads go out together
                                if (t0 + c0 >= n_tokens) break;
                                float v[32], old[32];
                                tc_ld16(tmem_d + lane_base + (uint32_t)c0, v);
                                if (BN > 16) tc_ld16(tmem_d + lane_base + (uint32_t)c0 + 16, v + 16);
                                if (f < n_features) {
                                    if (EPI == EPI_RESIDUAL) {
#pragma unroll
                                        for (int j = 0; j < (BN > 16 ? 32 : 16); ++j) {
                                            const int t = t0 + c0 + j;
                                            old[j] = t < n_tokens ? e.out[(size_t)t * n_features + f] : 0.f;
                                        }
                                    }
#pragma unroll
                                    for (int j = 0; j < (BN > 16 ? 32 : 16); ++j) {
                                        const int t = t0 + c0 + j;
                                        if (t < n_tokens)
                                            e.out[(size_t)t * n_features + f] = EPI == EPI_RESIDUAL ? old[j] + v[j] : v[j];
                                    }
                                }
                            }
                        }
                    } else if (EPI == EPI_SWIGLU) {
                        // rows 2 i and 2 i + 1 of the tile are the gate and up rows of feature i of this tile's 64
                        const int fg = blockIdx.x * 64 + (fl & 63);                // the feature of y
                        if (fg < e.inter)
                            for (int t = fl >> 6; t < cols; t += 2) {                  // two token rows at a time
                                const float g = xs[t * GT_BM + 2 * (fl & 63)], u = xs[t * GT_BM + 2 * (fl & 63) + 1];
                                from_f32(e.y[(size_t)(t0 + t) * e.inter + fg], silu_mul(g, u));
                            }
                    } else if (EPI == EPI_QKV) {
                        const int hpt = GT_BM / e.q.hd;           // heads per tile
                        const int heads = e.q.n_q + 2 * e.q.n_kv;
                        const int* meta = (const int*)(gen_base + STAGES * S::STAGE_BYTES + 1024);   // [BN][2]: page, row
                        for (int row = warp; row < cols * hpt; row += 4) {
                            const int c = row / hpt, hh = row % hpt;
                            const int head = f0 / e.q.hd + hh;
                            if (head < heads) {
                                const float* src = xs + c * GT_BM + hh * e.q.hd;
                                const int page = meta[2 * c], prow = meta[2 * c + 1];
                                qkv_finish_row(e.q, t0 + c, head, lane, [&](int j) { return src[j]; },
                                               [&](int g) {
                                                   return (((size_t)page * e.q.n_kv + g) * IDM_PAGE + prow) * (size_t)e.q.hd;
                                               });
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tmem_dealloc(tmem_d, TMEM_COLS);
    }
}

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
    static constexpr int META_BYTES = BN * 4;                      // per token: page * 64 + row
    static constexpr int XS_OFF = STAGES * STAGE_BYTES;
    static constexpr int META_OFF = XS_OFF + XS_BYTES;
    static constexpr int BAR_OFF = META_OFF + META_BYTES;
    static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ void group_sync(int g) { asm volatile("bar.sync %0, 128;" ::"r"(1 + g) : "memory"); }     // one group
__device__ __forceinline__ void groups_sync() {                                                                      // all epilogue warps
    asm volatile("bar.sync %0, %1;" ::"r"(1 + GP_GROUPS), "r"(32 * GP_EPI_WARPS) : "memory");
}

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(GP_THREADS) gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                     const __grid_constant__ CUtensorMap map_x,
                                                                     const GemmEpi e, int n_tokens, int n_features,
                                                                     int kb_total, int tiles_x, int n_tiles) {
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
                const int f0 = (tile % tiles_x) * GT_BM, t0 = (tile / tiles_x) * BN;
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
        int* meta = (int*)(gen_base + S::META_OFF);
        const int fl = quarter * 32 + lane;                        // feature within the tile = accumulator lane
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        uint32_t it = 0;
        bool ok = true;
        Tile4Lane tl4 = {};
        if (EPI == EPI_QKV) tl4 = qkv_tile4_lane(e.q, lane);
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
            const int tx = tile % tiles_x, f0 = tx * GT_BM, t0 = (tile / tiles_x) * BN;
            const int f = f0 + fl;
            const uint32_t acc = it & 1;
            if (EPI == EPI_QKV && e.q.write_cache) {
                groups_sync();                                     // the previous tile's readers of meta are done
                for (int tl = threadIdx.x; tl < BN; tl += 32 * GP_EPI_WARPS)
                    if (t0 + tl < n_tokens) {
                        const int t = t0 + tl;
                        const int pos = e.q.positions[t];
                        const int r = e.q.cache.ring ? pos % e.q.cache.ring : pos;
                        const int page = e.q.cache.table[(size_t)e.q.slots[e.q.token_seq[t]] * e.q.cache.table_stride + r / IDM_PAGE];
                        meta[tl] = page * IDM_PAGE + r % IDM_PAGE;
                    }
                groups_sync();
            }
            ok = mbar_wait(tfull_bar(acc), (it >> 1) & 1, abort_flag, &g_gemm_error);
            if (!ok) break;
            tc_fence_after();
            // the accumulator columns of a chunk are asked for while the chunk before is worked on (two sets of
            // registers in turn; the loop is unrolled so that which set is which is known at compile time)
            uint32_t raw[2][GP_CHUNK];
            if (t0 + grp * GP_CHUNK < n_tokens) tc_ld16_issue(tmem + acc * BN + lane_base + (uint32_t)(grp * GP_CHUNK), raw[0]);
#pragma unroll
            for (int ci = 0; ci < BN / (GP_GROUPS * GP_CHUNK); ++ci) {
                const int c0 = grp * GP_CHUNK + ci * GP_GROUPS * GP_CHUNK;
                if (t0 + c0 >= n_tokens) break;                    // uniform over the group
                const int cols = min(GP_CHUNK, n_tokens - t0 - c0);
                // q/k/v: the (cos, sin) of this warp's four token rows (rows quarter, quarter + 4, ...), asked for
                // before anything else waits
                float4 ca[GP_CHUNK / 4], cb[GP_CHUNK / 4];
                if (EPI == EPI_QKV) {
#pragma unroll
                    for (int r = 0; r < GP_CHUNK / 4; ++r) {
                        ca[r] = cb[r] = make_float4(0.f, 0.f, 0.f, 0.f);
                        const int row = quarter + 4 * r;
                        const float4* c4 = row < cols ? qkv_tile4_cs(e.q, tl4, t0 + c0 + row, f0, lane) : nullptr;
                        if (c4) { ca[r] = __ldg(c4); cb[r] = __ldg(c4 + 1); }
                    }
                }
                float v[GP_CHUNK];
                tc_ld_wait();
#pragma unroll
                for (int j = 0; j < GP_CHUNK; ++j) v[j] = __uint_as_float(raw[ci & 1][j]);
                if (ci + 1 < BN / (GP_GROUPS * GP_CHUNK) && t0 + c0 + GP_GROUPS * GP_CHUNK < n_tokens)
                    tc_ld16_issue(tmem + acc * BN + lane_base + (uint32_t)(c0 + GP_GROUPS * GP_CHUNK), raw[(ci + 1) & 1]);
                if (EPI == EPI_PARTIAL || EPI == EPI_STORE || EPI == EPI_RESIDUAL) {
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
                    } else if (EPI == EPI_QKV && f0 >= (e.q.n_q + e.q.n_kv) * e.q.hd) {
                        // a tile of value heads: nothing to norm or rotate, the rows go out as they are
                        const int g0 = f0 / e.q.hd - e.q.n_q - e.q.n_kv;          // first value head of the tile
#pragma unroll
                        for (int r = 0; r < GP_CHUNK / 4; ++r) {
                            const int row = quarter + 4 * r, t = t0 + c0 + row;
                            const int fv = g0 * e.q.hd + lane * 4;                // feature among the value features
                            if (row < cols && fv < e.q.n_kv * e.q.hd) {
                                const float4 v4 = *reinterpret_cast<const float4*>(xs + row * GT_BM + lane * 4);
                                const float y[4] = {v4.x, v4.y, v4.z, v4.w};
                                const int g = fv / e.q.hd, d = fv % e.q.hd;
                                if (e.q.write_cache) {
                                    const int place = meta[c0 + row];
                                    store4(e.q.cache.v + (((size_t)(place / IDM_PAGE) * e.q.n_kv + g) * IDM_PAGE + place % IDM_PAGE) *
                                                             (size_t)e.q.hd + d, y);
                                }
                                if (e.q.v_new) store4(e.q.v_new + (size_t)t * e.q.n_kv * e.q.hd + fv, y);
                            }
                        }
                    } else if (EPI == EPI_QKV) {
                        // a warp takes whole token rows of the tile (whole heads: 128 % head_dim == 0), four
                        // features per lane, as the separate kernel does
#pragma unroll
                        for (int r = 0; r < GP_CHUNK / 4; ++r) {
                            // the four rows' arithmetic is independent: no branch around it, only the
                            // stores of rows past the end are left out
                            const int row = quarter + 4 * r;
                            const float4 v4 = *reinterpret_cast<const float4*>(xs + row * GT_BM + lane * 4);
                            const int place = meta[c0 + row];
                            qkv_finish_tile4_pre(e.q, tl4, v4, t0 + c0 + row, f0, lane, place / IDM_PAGE, place % IDM_PAGE,
                                                 ca[r], cb[r], row < cols);
                        }
                    }
                    group_sync(grp);                               // the buffer is free for the group's next chunk
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == GP_EPI_WARPS + 1) tmem_dealloc(tmem, TMEM_COLS);
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
template <int HD>
__device__ __forceinline__ void qkv_tokens_head(const QkvArgs& a, uint32_t col0, const float* gamma, bool rotate,
                                                const float2* cs_row, const float2* cs_dim, int n_tokens,
                                                T* dst_a, T* dst_b) {
    constexpr int HALF = HD / 2;
    float cs4[4][8];                                               // (cos, sin) of 16 dims
    auto ask_cs = [&](int c) {
        if (!rotate) return;
        if (cs_dim != nullptr) {
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
        }
        if (gamma != nullptr) inv = head_inv_rms(a, (s4[0] + s4[1]) + (s4[2] + s4[3]));
    }
    // dims d and d + HALF together, 16 of each per step; the next step's columns are asked for before
    // this step's arithmetic (the loop stays a loop: unrolled, the compiler moves all steps' loads of the
    // norm weight to the front and runs out of registers)
#pragma unroll 1
    for (int c = 0; c < HALF; c += 16) {
        float lo[16], hi[16];
        if (c > 0) tc_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) { lo[i] = __uint_as_float(cur[i]); hi[i] = __uint_as_float(cur[16 + i]); }
        if (c + 16 < HALF) {
            tc_ld16_issue(col0 + (uint32_t)(c + 16), cur);
            tc_ld16_issue(col0 + (uint32_t)(HALF + c + 16), cur + 16);
        }
        if (gamma != nullptr) {
            // the norm weight four values a request (every lane asks for the same address)
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
                const float4 gl = __ldg(reinterpret_cast<const float4*>(gamma + c + i));
                const float4 gh = __ldg(reinterpret_cast<const float4*>(gamma + HALF + c + i));
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
    }
}

__global__ void __launch_bounds__(GQ_THREADS) gemm_qkv_tokens_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                     const __grid_constant__ CUtensorMap map_x,
                                                                     const GemmEpi e, int n_tokens, int n_features,
                                                                     int kb_total, int tiles_x, int n_tiles) {
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
                const int f0 = (tile % tiles_x) * BN, t0 = (tile / tiles_x) * GT_BM;
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
            const int tx = tile % tiles_x, f0 = tx * BN, t0 = (tile / tiles_x) * GT_BM;
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
               n_tiles);
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
               kb_total, tiles_x, n_tiles);
    IDM_LAUNCH_CHECK("gemm_persistent");
    return 0;
}

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

template <int BN, int STAGES, int EPI>
static int launch_gemm_cluster(const CUtensorMap& mw, const CUtensorMap& mx, const GemmEpi& e, int M, int N, int kb_total,
                               int kb_per_split, int splits, cudaStream_t stream) {
    using S = GemmSmem<BN, STAGES, true>;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, EPI, true>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        IDM_REQUIRE(err == cudaSuccess, "gemm: cannot get %d bytes of shared memory: %s", S::TOTAL,
                    cudaGetErrorString(err));
        err = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, EPI, true>,
                                   cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        IDM_REQUIRE(err == cudaSuccess, "gemm: clusters of up to 16 blocks are not allowed here: %s",
                    cudaGetErrorString(err));
        configured = true;
    }
    dim3 grid((N + GT_BM - 1) / GT_BM, 1, splits);
    cudaError_t err = idm_launch_cluster(gemm_tcgen05_kernel<BN, STAGES, EPI, true>, grid, dim3(GT_THREADS), S::TOTAL,
                                         stream, splits, mw, mx, e, M, N, kb_total, kb_per_split);
    IDM_REQUIRE(err == cudaSuccess, "gemm: cluster launch failed: %s", cudaGetErrorString(err));
    IDM_LAUNCH_CHECK("gemm_tcgen05 (cluster)");
    return 0;
}

template <int BN, int STAGES, int EPI>
static int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mx, const GemmEpi& e, int M, int N, int kb_total,
                       int kb_per_split, int splits, cudaStream_t stream) {
    using S = GemmSmem<BN, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, EPI, false>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        IDM_REQUIRE(err == cudaSuccess, "gemm: cannot get %d bytes of shared memory: %s", S::TOTAL,
                    cudaGetErrorString(err));
        configured = true;
    }
    dim3 grid((N + GT_BM - 1) / GT_BM, (M + BN - 1) / BN, splits);
    IDM_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "gemm: too many tiles (%u x %u)", grid.y, grid.z);
    IDM_REQUIRE(EPI == EPI_PARTIAL || splits == 1 || (long long)grid.x * grid.y <= GT_COUNTER_SLOTS,
                "gemm: %u x %u tiles exceed the %d counters", grid.x, grid.y, GT_COUNTER_SLOTS);
    idm_launch(gemm_tcgen05_kernel<BN, STAGES, EPI, false>, dim3(grid), dim3(GT_THREADS), S::TOTAL, stream, mw, mx, e, M, N,
               kb_total, kb_per_split);
    IDM_LAUNCH_CHECK("gemm_tcgen05");
    return 0;
}

// From how many tokens on a product runs unsplit in the persistent kernels.
static int g_gemm_many_from = 257;
extern "C" void idm_gemm_set_many_from(int tokens) { g_gemm_many_from = tokens < 65 ? 65 : tokens; }

// How many partial sums a product of this shape is split into.  Below that border the split depends
// on the layer (N, K) only, so a token's result is the same in any batch; from it on K is not split.
// Between 65 tokens and the border a layer whose unsplit product is short anyway (its tiles of 128
// tokens, counted for 256 tokens, times its k-blocks at 0.3 us: at most 16 us, about what the host
// needs to launch one more kernel) is not split either: it then runs with its epilogue fused, and a
// step of that size is bound by its launches, not by its kernels.
extern "C" int idm_gemm_bf16_splits(int M, int N, int K) {
    const int kb_total = (K + GT_BK - 1) / GT_BK;
    if (M >= g_gemm_many_from) return 1;
    if (M > 64) {
        const long long tiles256 = 2LL * ((N + GT_BM - 1) / GT_BM);
        const long long rounds = (tiles256 + 147) / 148;
        if (rounds * kb_total * 3 <= 160) return 1;
    }
    const int tiles = (N + GT_BM - 1) / GT_BM;
    int want = 296 / tiles;                       // about two blocks per SM
    if (want < 1) want = 1;
    if (want > kb_total) want = kb_total;
    if (want > 16) want = 16;
    const int per = (kb_total + want - 1) / want;
    return (kb_total + per - 1) / per;
}

// 32-bit words of workspace for a fused epilogue: the counters (a fixed place at the start, so that
// they are zero at every launch), then the slices' tiles
extern "C" long long idm_gemm_bf16_workspace_floats(int M, int N, int splits) {
    return (long long)GT_COUNTER_SLOTS + (splits > 1 ? (long long)splits * M * N : 0);
}

static int g_gemm_cluster = 1, g_gemm_persistent = 1;
extern "C" void idm_gemm_set_cluster(int on) { g_gemm_cluster = on ? 1 : 0; }
extern "C" void idm_gemm_set_persistent(int on) { g_gemm_persistent = on ? 1 : 0; }

template <int EPI>
static int gemm_any(const void* x, const void* w, GemmEpi e, float* workspace, int M, int N, int K, int splits,
                    cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    IDM_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    IDM_REQUIRE(K % 8 == 0, "gemm: the inner size %d must be a multiple of 8 (rows start on 16-byte borders)", K);
    IDM_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm: operands must be 16-byte aligned");
    const int kb_total = (K + GT_BK - 1) / GT_BK;
    IDM_REQUIRE(splits >= 1 && splits <= kb_total, "gemm: %d splits for %d k-blocks", splits, kb_total);
    const int per = (kb_total + splits - 1) / splits;
    IDM_REQUIRE((kb_total + per - 1) / per == splits, "gemm: %d splits leave one empty", splits);
    if (EPI != EPI_PARTIAL) {
        IDM_REQUIRE(splits == 1 || workspace != nullptr, "gemm: a split product with a fused epilogue needs a workspace");
        e.counters = (int*)workspace;
        e.ws = workspace ? workspace + GT_COUNTER_SLOTS : nullptr;
    }
    CUtensorMap mw, mx;
    auto on32 = [](const void* p) { return ((uintptr_t)p & 31) == 0; };   // (null counts: that output is not written)
    if (EPI == EPI_QKV && splits == 1 && M > 64 && g_gemm_persistent && (e.q.hd == 32 || e.q.hd == 64 || e.q.hd == 128) &&
        on32(e.q.q_out) && on32(e.q.k_new) && on32(e.q.v_new) && on32(e.q.cache.k) && on32(e.q.cache.v) && on32(e.q.cs) &&
        on32(e.q.gq) && on32(e.q.gk)) {
        // many tokens: tokens on the accumulator's lanes, 256 features (whole heads) per tile
        if (make_map(&mw, w, N, K, GQ_BN)) return 1;
        if (make_map(&mx, x, M, K, GT_BM)) return 1;
        return launch_qkv_tokens(mw, mx, e, M, N, kb_total, stream);
    }
    if (splits == 1 && M > 64 && g_gemm_persistent) {
        // many tokens: the persistent kernel; 256-token tiles unless 128 fill more of the SMs
        const int tiles_x = (N + GT_BM - 1) / GT_BM;
        const bool wide = (long long)tiles_x * ((M + 255) / 256) >= 120;
        if (make_map(&mw, w, N, K, GT_BM)) return 1;
        if (make_map(&mx, x, M, K, wide ? 256 : 128)) return 1;
        return wide ? launch_persistent<256, 4, EPI>(mw, mx, e, M, N, kb_total, stream)
                    : launch_persistent<128, 6, EPI>(mw, mx, e, M, N, kb_total, stream);
    }
    const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    if (make_map(&mw, w, N, K, GT_BM)) return 1;
    if (make_map(&mx, x, M, K, bn)) return 1;
    // up to 64 tokens with K split: the slices are added inside a thread-block cluster
    if (EPI != EPI_PARTIAL && splits > 1 && splits <= 16 && M <= 64 && N % 4 == 0 && g_gemm_cluster) {
        switch (bn) {
            case 16: return launch_gemm_cluster<16, 5, EPI>(mw, mx, e, M, N, kb_total, per, splits, stream);
            case 32: return launch_gemm_cluster<32, 4, EPI>(mw, mx, e, M, N, kb_total, per, splits, stream);
            default: return launch_gemm_cluster<64, 3, EPI>(mw, mx, e, M, N, kb_total, per, splits, stream);
        }
    }
    switch (bn) {
        case 16: return launch_gemm<16, 6, EPI>(mw, mx, e, M, N, kb_total, per, splits, stream);
        case 32: return launch_gemm<32, 6, EPI>(mw, mx, e, M, N, kb_total, per, splits, stream);
        case 64: return launch_gemm<64, 4, EPI>(mw, mx, e, M, N, kb_total, per, splits, stream);
        default: return launch_gemm<128, 3, EPI>(mw, mx, e, M, N, kb_total, per, splits, stream);
    }
}

// out [splits, M, N]: the slices' partial sums
extern "C" int idm_gemm_bf16(const void* x, const void* w, float* out, int M, int N, int K, int splits,
                             cudaStream_t stream) {
    GemmEpi e = {};
    e.out = out;
    return gemm_any<EPI_PARTIAL>(x, w, e, nullptr, M, N, K, splits, stream);
}

// out [M, N] = x . w^T (finished, 32-bit)
extern "C" int idm_gemm_bf16_store(const void* x, const void* w, float* out, float* workspace, int M, int N, int K,
                                   int splits, cudaStream_t stream) {
    GemmEpi e = {};
    e.out = out;
    return gemm_any<EPI_STORE>(x, w, e, workspace, M, N, K, splits, stream);
}

// h [M, N] += x . w^T (the 32-bit residual sum)
extern "C" int idm_gemm_bf16_residual(const void* x, const void* w, float* h, float* workspace, int M, int N, int K,
                                      int splits, cudaStream_t stream) {
    GemmEpi e = {};
    e.out = h;
    return gemm_any<EPI_RESIDUAL>(x, w, e, workspace, M, N, K, splits, stream);
}

// y [M, inter] = silu(x . gate^T) * (x . up^T); w_tiled [tiles * 128, K]: rows 128 j + 2 i and 128 j + 2 i + 1
// are the gate and the up row of feature 64 j + i (rows past `inter` are zero)
extern "C" int idm_gemm_bf16_swiglu(const void* x, const void* w_tiled, void* y, float* workspace, int M, int inter,
                                    int K, int splits, cudaStream_t stream) {
    GemmEpi e = {};
    e.y = (T*)y; e.inter = inter;
    const int tiles = (inter + 63) / 64;
    return gemm_any<EPI_SWIGLU>(x, w_tiled, e, workspace, M, tiles * GT_BM, K, splits, stream);
}

// The fused q/k/v projection with the per-head finish (see qkv_finish.cuh); 128 % head_dim must be 0
extern "C" int idm_gemm_bf16_qkv(const void* x, const void* w, float* workspace, int M, int K, int splits, int n_q,
                                 int n_kv, int hd, const float* gq, const float* gk, float eps, const float* cs,
                                 const float* cs_by_dim,
                                 void* q_out, void* k_new, void* v_new, void* k_pool, void* v_pool, const int* table,
                                 int table_stride, int ring, const int* token_seq, const int* positions,
                                 const int* slots, cudaStream_t stream) {
    IDM_REQUIRE(hd > 0 && GT_BM % hd == 0 && hd % 2 == 0, "gemm_qkv: head_dim=%d must divide %d", hd, GT_BM);
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
    return gemm_any<EPI_QKV>(x, w, e, workspace, M, (n_q + 2 * n_kv) * hd, K, splits, stream);
}

// 0, or 1 if any block's bounded wait ran out since the last call (reads the flag: synchronises)
extern "C" int idm_gemm_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    return v;
}

#endif  // IDM_BF16
