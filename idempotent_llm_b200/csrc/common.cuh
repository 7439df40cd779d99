// Shared helpers of the hand-written sm_100a kernels.
//
// Each shared library is compiled for ONE storage type T (activations, weights
// and cache): -DIDM_BF16 gives __nv_bfloat16, -DIDM_F32 gives float.  All
// arithmetic (norm statistics, rotation, scores, softmax, residual sums) is in
// 32-bit whatever T is.  Entry points are plain C functions taking device
// pointers and a stream; they return 0 or record a message (idm_last_error)
// and return non-zero.  Nothing here allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#if defined(IDM_BF16)
typedef __nv_bfloat16 T;
#define IDM_DTYPE_NAME "bfloat16"
#elif defined(IDM_F32)
typedef float T;
#define IDM_DTYPE_NAME "float32"
#else
#error "compile with -DIDM_BF16 or -DIDM_F32"
#endif

#define IDM_PAGE 64          // tokens per cache page (must match cache/spec.py)
#define IDM_MAX_HEAD_DIM 256

// ---------------------------------------------------------------- errors
int idm_fail(const char* fmt, ...);   // records the message, returns 1

#define IDM_REQUIRE(cond, ...) \
    do { if (!(cond)) return idm_fail(__VA_ARGS__); } while (0)

#define IDM_LAUNCH_CHECK(name) \
    do { cudaError_t e_ = cudaGetLastError(); \
         if (e_ != cudaSuccess) return idm_fail("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
    } while (0)

// ------------------------------------------- programmatic dependent launch
// Every kernel of this library starts with pdl_launch_dependents() (but the one that moves a captured
// step's lengths and positions on, which lets nothing start before it is done) and executes pdl_wait()
// before its first access to global memory that an earlier kernel may have written (or may still read).
// Launched with the programmatic-serialization attribute, the next kernel's blocks are scheduled
// while this one still runs and do their set-up (and, in the matrix product, fetch weights, which
// no kernel writes) before the wait returns.  Without the attribute both instructions do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

int idm_pdl_enabled();   // runtime.cu: IDM_PDL=0 in the environment switches the attribute off
int idm_pdl_flag(const char* name, int dflt);   // per-kernel switches read once from the environment

template <typename... KArgs, typename... Args>
static inline cudaError_t idm_launch_opt(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl && idm_pdl_enabled()) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
static inline cudaError_t idm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args&&... args) {
    return idm_launch_opt(true, kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
}

// the same with a thread-block cluster of `cluster_z` blocks along z (distributed shared memory)
template <typename... KArgs, typename... Args>
static inline cudaError_t idm_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                             cudaStream_t stream, int cluster_z, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = cluster_z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = idm_pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ----------------------------------------------------------- conversions
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void from_f32(float& dst, float v) { dst = v; }
__device__ __forceinline__ void from_f32(__nv_bfloat16& dst, float v) { dst = __float2bfloat16_rn(v); }
// four consecutive elements as one store (the address on an 8-byte border in bfloat16, 16-byte in 32-bit);
// each value rounded as from_f32 rounds it
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

// 16-byte vector of T: 8 bfloat16 or 4 float
template <typename U> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    float4 raw;
    __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
    __device__ __forceinline__ float get(int i) const { return (&raw.x)[i]; }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    uint4 raw;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ float get(int i) const {
        uint32_t w = (&raw.x)[i >> 1];
        return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
    }
};

// 2^x by the hardware unit alone: relative error ~2e-7 * |x| rounding aside, results below 2^-126
// become 0.  (exp2f without fast-math wraps the same instruction in a range fix of three more.)
__device__ __forceinline__ float ex2_hw(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// max(a, b, c) in one instruction (sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// g * sigmoid(g) * u with the hardware exponential and division (relative error ~1e-6, far below the
// bfloat16 rounding of the result).  Every kernel that applies the activation uses this one formula,
// so fused and separate paths give the same bits.  (src/detllm/ops/di_swiglu.py:43-45)
__device__ __forceinline__ float silu_mul(float g, float u) {
#if defined(IDM_F32)
    return g / (1.0f + expf(-g)) * u;                       // the 32-bit path stays exact
#else
    return __fmul_rn(__fdividef(g, 1.0f + __expf(-g)), u);
#endif
}

// ------------------------------------------------------------ reductions
// Fixed-order reductions: xor butterflies inside a warp, then the warps' values
// added in ascending order.  The order depends on the block size only.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// all threads of the block get the sum; `scratch` holds >= 32 floats
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[w] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; ++i) t += scratch[i];
    return t;
}

// Sum of the partial results base[p * stride + idx], p = 0 .. n-1, added in ascending p onto `start`.
// The loads of a group of 8 are issued together (they do not wait on one another); only the adds
// are a chain.
__device__ __forceinline__ float add_partials(float start, const float* __restrict__ base, int n, size_t stride,
                                              size_t idx) {
    const float* p = base + idx;
    if (n == 1) return start + __ldg(p);                    // the common case: nothing was split
    float v = start;
    int left = n;
    while (left >= 8) {
        float part[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) part[i] = __ldg(p + (size_t)i * stride);
#pragma unroll
        for (int i = 0; i < 8; ++i) v += part[i];
        p += 8 * stride;
        left -= 8;
    }
    if (left > 0) {
        float part[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) part[i] = i < left ? __ldg(p + (size_t)i * stride) : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < left) v += part[i];
    }
    return v;
}

// ------------------------------------------------------- cache addressing
// One cache entry: pools [pages, kv_heads, IDM_PAGE, head_dim]; a sequence's
// pages through table[slot * table_stride + i]; key j sits at ring position
// (ring ? j % ring : j).
struct KVAddr {
    T* k;
    T* v;
    const int* table;
    int table_stride;
    int ring;
    int n_kv;
    int hd;
};
__device__ __forceinline__ size_t kv_offset(const KVAddr& c, int slot, int j, int kv_head) {
    const int r = c.ring ? (j % c.ring) : j;
    const int page = c.table[(size_t)slot * c.table_stride + (r / IDM_PAGE)];
    return (((size_t)page * c.n_kv + kv_head) * IDM_PAGE + (r % IDM_PAGE)) * (size_t)c.hd;
}
