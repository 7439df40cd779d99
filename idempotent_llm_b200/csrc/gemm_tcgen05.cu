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
// Every wait on an mbarrier is bounded by a cycle count; a wait that runs out sets the error flag
// (idm_gemm_status), all roles leave their loops, tensor memory is freed and the block returns.
#include "common.cuh"

#if defined(IDM_BF16)

#include "tcgen05.cuh"

#define GT_BM 128            // features per tile (MMA M)
#define GT_BK 64             // k per stage: 64 bf16 = 128 bytes = one swizzle row
#define GT_UMMA_K 16
#define GT_THREADS 192

__device__ int g_gemm_error = 0;

// ---------------------------------------------------------------------------- kernel
template <int BN, int STAGES>
struct GemmSmem {
    static constexpr int A_BYTES = GT_BM * GT_BK * 2;
    static constexpr int B_BYTES = BN * GT_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BARRIER_BYTES = 1024;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + BARRIER_BYTES + 1024;   // + slack to align to 1024
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(GT_THREADS) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                  const __grid_constant__ CUtensorMap map_x,
                                                                  float* __restrict__ out, int n_tokens,
                                                                  int n_features, int kb_total, int kb_per_split) {
    using S = GemmSmem<BN, STAGES>;
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

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = blockIdx.x * GT_BM, t0 = blockIdx.y * BN;
    const int kb0 = blockIdx.z * kb_per_split;
    const int kb_n = min(kb_per_split, kb_total - kb0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 5) {
        tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;

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
        if (mbar_wait(accum_bar, 0, abort_flag, &g_gemm_error)) {
            tc_fence_after();
            pdl_wait();                                           // (already satisfied: the activations came after it)
            const int f = f0 + warp * 32 + lane;                  // this thread's feature (accumulator lane)
            float* dst = out + (size_t)blockIdx.z * n_tokens * n_features;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (t0 + c0 >= n_tokens) break;                   // warp-uniform
                float v[16];
                tc_ld16(tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
                if (f < n_features) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int t = t0 + c0 + j;
                        if (t < n_tokens) dst[(size_t)t * n_features + f] = v[j];
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
static int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mx, float* out, int M, int N, int kb_total,
                       int kb_per_split, int splits, cudaStream_t stream) {
    using S = GemmSmem<BN, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        IDM_REQUIRE(e == cudaSuccess, "gemm: cannot get %d bytes of shared memory: %s", S::TOTAL, cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid((N + GT_BM - 1) / GT_BM, (M + BN - 1) / BN, splits);
    IDM_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "gemm: too many tiles (%u x %u)", grid.y, grid.z);
    idm_launch(gemm_tcgen05_kernel<BN, STAGES>, dim3(grid), dim3(GT_THREADS), S::TOTAL, stream, mw, mx, out, M, N, kb_total, kb_per_split);
    IDM_LAUNCH_CHECK("gemm_tcgen05");
    return 0;
}

// How many partial sums a product of this shape is split into.  Up to 256 tokens the split depends
// on the layer (N, K) only, so a token's result is the same in any batch; beyond that K is not split.
extern "C" int idm_gemm_bf16_splits(int M, int N, int K) {
    const int kb_total = (K + GT_BK - 1) / GT_BK;
    if (M > 256) return 1;
    const int tiles = (N + GT_BM - 1) / GT_BM;
    int want = 296 / tiles;                       // about two blocks per SM
    if (want < 1) want = 1;
    if (want > kb_total) want = kb_total;
    if (want > 16) want = 16;
    const int per = (kb_total + want - 1) / want;
    return (kb_total + per - 1) / per;
}

extern "C" int idm_gemm_bf16(const void* x, const void* w, float* out, int M, int N, int K, int splits,
                             cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    IDM_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    IDM_REQUIRE(K % 8 == 0, "gemm: the inner size %d must be a multiple of 8 (rows start on 16-byte borders)", K);
    IDM_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm: operands must be 16-byte aligned");
    const int kb_total = (K + GT_BK - 1) / GT_BK;
    IDM_REQUIRE(splits >= 1 && splits <= kb_total, "gemm: %d splits for %d k-blocks", splits, kb_total);
    const int per = (kb_total + splits - 1) / splits;
    IDM_REQUIRE((kb_total + per - 1) / per == splits, "gemm: %d splits leave one empty", splits);
    CUtensorMap mw, mx;
    const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    if (make_map(&mw, w, N, K, GT_BM)) return 1;
    if (make_map(&mx, x, M, K, bn)) return 1;
    switch (bn) {
        case 16: return launch_gemm<16, 6>(mw, mx, out, M, N, kb_total, per, splits, stream);
        case 32: return launch_gemm<32, 6>(mw, mx, out, M, N, kb_total, per, splits, stream);
        case 64: return launch_gemm<64, 4>(mw, mx, out, M, N, kb_total, per, splits, stream);
        default: return launch_gemm<128, 3>(mw, mx, out, M, N, kb_total, per, splits, stream);
    }
}

// 0, or 1 if any block's bounded wait ran out since the last call (reads the flag: synchronises)
extern "C" int idm_gemm_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    return v;
}

#endif  // IDM_BF16
