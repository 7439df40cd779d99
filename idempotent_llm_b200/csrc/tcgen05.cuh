// Inline-PTX wrappers for the Blackwell (sm_100a) tensor-core path: mbarriers with bounded waits,
// TMA tile loads (no multicast), tensor-memory allocation, tcgen05.mma / commit / ld / st, and the
// shared-memory and instruction descriptors the MMA reads.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TC_WAIT_CYCLES 4000000000ll   // ~2 s: far beyond any real wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ------------------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false if it ran out (then *abort_flag and *error_word are set) or if another role of
// the block already gave up.  Callers leave their loops on false and fall through to the teardown.
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* error_word,
                                                long long limit_cycles) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit_cycles) {
            *abort_flag = 1;
            atomicExch(error_word, 1);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* error_word) {
    return mbar_wait_limit(bar, parity, abort_flag, error_word, TC_WAIT_CYCLES);
}

// The same for a barrier that blocks of other SMs of the cluster arrive at (acquire at cluster scope).
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* error_word) {
    if (mbar_try_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > TC_WAIT_CYCLES) {
            *abort_flag = 1;
            atomicExch(error_word, 1);
            return false;
        }
    }
}
// One float into the shared memory of block `rank` of the cluster (same address as here), counted in
// bytes at that block's barrier `bar`: who waits there sees the value, and the sender waits for nothing.
__device__ __forceinline__ void st_async_f32(uint32_t local_addr, uint32_t local_bar, uint32_t rank, float v) {
    uint32_t remote, remote_bar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(local_bar), "r"(rank));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];"
                 ::"r"(remote), "f"(v), "r"(remote_bar) : "memory");
}

// ----------------------------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
// writes made with ordinary stores become visible to the async proxy (TMA, tcgen05.mma operand reads)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ------------------------------------------------------------------------ tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem_addr, uint32_t cols) {       // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem_addr), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {              // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] . B[smem], kind::f16 (bf16 operands, 32-bit accumulate)
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// Four MMAs over one k-block of 64 (four steps of 16 k = 32 bytes = 2 descriptor units along the swizzled row),
// in ascending k, as one piece of code: the issuing thread spends no instructions between them.
__device__ __forceinline__ void tc_mma_bf16_kblock(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t accumulate_first) {
    asm volatile("{\n\t.reg .pred p, q;\n\t.reg .b64 a, b;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "setp.eq.b32 q, 0, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
                 "add.u64 a, %1, 2;\n\tadd.u64 b, %2, 2;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n\t"
                 "add.u64 a, %1, 4;\n\tadd.u64 b, %2, 4;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n\t"
                 "add.u64 a, %1, 6;\n\tadd.u64 b, %2, 6;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, q;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first) : "memory");
}

#define TC_REGS16(r) "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), \
                     "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
// 16 / 32 consecutive 32-bit columns of this warp's 32 lanes (issue only; tc_ld_wait before use)
__device__ __forceinline__ void tc_ld16_issue(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : TC_REGS16(r) : "r"(taddr));
}
__device__ __forceinline__ void tc_ld32_issue(uint32_t taddr, uint32_t* r) {
    tc_ld16_issue(taddr, r);
    tc_ld16_issue(taddr + 16, r + 16);
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    tc_ld16_issue(taddr, r);
    tc_ld_wait();
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------ a pair of blocks on one tile
// cta_group::2: the two blocks of a cluster work on one tile of 256 rows.  Each holds 128 rows of A and of the
// accumulator (in its own tensor memory, at the same address) and HALF of B's rows in its own shared memory
// (at the same offsets); the MMA is issued by block 0 alone and runs on both SMs, reading both halves of B.  So
// a block fetches 128 + N/2 rows per k-block for 128 x N products: operands shared between two SMs without any
// multicast load.  Loads of either block count their bytes at block 0's barrier; a commit with a mask of both
// blocks frees a stage, or hands over an accumulator, in both at once.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {             // every thread of every block of the cluster
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, uint32_t rank) {   // the same place in block `rank`
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {          // a barrier of any block of the cluster
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem_addr, uint32_t cols) {   // the same warp of both blocks
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem_addr), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {          // the same warp of both blocks
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// arrives at `bar` (the same offset) in every block of `mask` once the MMAs issued so far are done
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint32_t mask) {
    asm volatile("{\n\t.reg .b16 m;\n\tcvt.u16.u32 m, %1;\n\t"
                 "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
                 ::"r"(bar), "r"(mask) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// -------------------------------------------------------------------------- descriptors
// Shared-memory operand, 128-byte swizzle, descriptor version 1 (sm_100); addresses and offsets in
// units of 16 bytes.
//  K-major (rows of 64 bf16 = 128 bytes along K): groups of 8 rows lie 1024 bytes apart (stride
//  offset); the leading offset is unused.
__device__ __forceinline__ uint64_t umma_desc_kmajor(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
//  MN-major (rows of 64 bf16 = 128 bytes along M/N, one row per k): groups of 8 k-rows lie 1024 bytes
//  apart (stride offset); the next 64 elements along M/N lie `lead_bytes` further (leading offset).
__device__ __forceinline__ uint64_t umma_desc_mnmajor(uint32_t smem_addr, uint32_t lead_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lead_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor, kind::f16: D = F32 (bit 4), A = B = BF16 (bits 7, 10), B MN-major if asked
// (bit 16), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, bool b_mn_major = false) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// -------------------------------------------------------------------- tensor maps (host)
typedef CUresult (*TcEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static inline TcEncodeTiledFn tc_encode_fn() {
    static TcEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (TcEncodeTiledFn)p;
    }
    return fn;
}
// bf16 tensor of `rank` dims (dims[0] innermost, strides in bytes for dims 1..), 128-byte swizzle,
// zero fill outside.  Returns a CUresult (0 = success) or -1 if the driver lacks the entry point.
static inline int tc_make_map_bf16(CUtensorMap* map, const void* ptr, int rank, const cuuint64_t* dims,
                                   const cuuint64_t* strides, const cuuint32_t* box) {
    TcEncodeTiledFn fn = tc_encode_fn();
    if (!fn) return -1;
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    return (int)fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}
