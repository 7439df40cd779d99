// q/k norm + rotation + cache write for one (token, head) row of the fused q/k/v projection, done
// by one warp.  q and k heads: RMS norm over head_dim with a weight of shape [head_dim] shared by all
// heads (src/detllm/model.py:208-215), then rotation of pairs (d, d + hd/2) by the token's position
// (src/detllm/ops/rope.py:47-55); v heads are copied.  q goes to q_out [N, n_q, hd]; k and v go to
// the cache at the token's position and/or to packed buffers k_new, v_new [N, n_kv, hd].
// `load(j)` returns element j of the row in 32-bit (from partial sums in memory, or from a tile in
// shared memory when this runs as the epilogue of the matrix product).
#pragma once

#include "common.cuh"

// four consecutive elements, one store
__device__ __forceinline__ void store4(float* p, const float (&x)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&x)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b = __floats2bfloat162_rn(x[2], x[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

// eight consecutive elements, one store (16 bytes in bfloat16, two of 16 in 32-bit)
__device__ __forceinline__ void store8(float* p, const float (&x)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(x[4], x[5], x[6], x[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&x)[8]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b = __floats2bfloat162_rn(x[2], x[3]);
    const __nv_bfloat162 c = __floats2bfloat162_rn(x[4], x[5]), d = __floats2bfloat162_rn(x[6], x[7]);
    *reinterpret_cast<uint4*>(p) = make_uint4(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b),
                                              *reinterpret_cast<const uint32_t*>(&c), *reinterpret_cast<const uint32_t*>(&d));
}

// sixteen consecutive bfloat16 elements as one 32-byte store, and eight floats as one 32-byte load (the
// 256-bit forms of sm_100): a thread that walks a row of its own fills whole 32-byte sectors with one
// request each, where narrower accesses cost the memory pipeline two.  Addresses on 32-byte borders.
__device__ __forceinline__ void store16(__nv_bfloat16* p, const float (&x)[16]) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const __nv_bfloat162 t = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&t);
    }
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 :: "l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
}
__device__ __forceinline__ void load8_readonly(const float* p, float (&v)[8]) {
    asm volatile("ld.global.nc.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
                 : "l"(p));
}

struct QkvArgs {
    const float* qkv; int n_partials; size_t partial_stride;
    int n_tokens, n_q, n_kv, hd;
    const float* gq; const float* gk; float eps; float inv_hd;   // inv_hd = 1 / hd
    const float2* cs;
    const float2* cs_by_dim;                                     // the same table as [hd / 2, n_tokens], or null
    T* q_out; T* k_new; T* v_new;
    KVAddr cache; int write_cache;
    const int* token_seq; const int* positions; const int* slots;
    int tiles4;               // the separate kernel: 1 = work on tiles of 128 features, four per lane
};

// where the token's key/value row of kv-head g starts in the pools
struct QkvLocateFromTables {
    const QkvArgs& a; int t;
    __device__ __forceinline__ size_t operator()(int g) const {
        return kv_offset(a.cache, a.slots[a.token_seq[t]], a.positions[t], g);
    }
};

// 1 / sqrt(ss / hd + eps) for a head's sum of squares.  Every kernel that norms a head uses this one
// function, with its roundings pinned, so that fused and separate paths give the same bits.  The 32-bit
// library divides and takes the root exactly; the bfloat16 library uses the hardware's reciprocal square
// root (2 units in the last place of 32-bit, far below the rounding of the result), which is what keeps the
// tile epilogues of the projection from being bound by these instructions.
__device__ __forceinline__ float head_inv_rms(const QkvArgs& a, float ss) {
#if defined(IDM_F32)
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)a.hd), a.eps)));
#else
    return rsqrtf(__fmaf_rn(ss, a.inv_hd, a.eps));
#endif
}

template <typename Load, typename Locate>
__device__ __forceinline__ void qkv_finish_row(const QkvArgs& a, int t, int head, int lane, Load load, Locate locate) {
    const int half = a.hd >> 1;
    constexpr int MAXP = IDM_MAX_HEAD_DIM / 64;   // pairs per lane
    float x1[MAXP], x2[MAXP];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
        const int j = lane + 32 * i;
        x1[i] = x2[i] = 0.f;
        if (j < half) {
            x1[i] = load(j);
            x2[i] = load(j + half);
            ss = __fmaf_rn(x2[i], x2[i], __fmaf_rn(x1[i], x1[i], ss));
        }
    }
    const bool is_q = head < a.n_q, is_k = !is_q && head < a.n_q + a.n_kv;
    T* dst_a = nullptr; T* dst_b = nullptr;
    if (is_q) {
        dst_a = a.q_out + ((size_t)t * a.n_q + head) * a.hd;
    } else {
        const int g = is_k ? head - a.n_q : head - a.n_q - a.n_kv;
        if (a.write_cache) {
            const size_t off = locate(g);
            dst_a = (is_k ? a.cache.k : a.cache.v) + off;
        }
        T* packed = is_k ? a.k_new : a.v_new;
        if (packed) dst_b = packed + ((size_t)t * a.n_kv + g) * a.hd;
    }
    const float* gamma = is_q ? a.gq : (is_k ? a.gk : nullptr);
    float inv = 1.f;
    if (gamma) {
        ss = warp_sum(ss);
        inv = head_inv_rms(a, ss);
    }
    const bool rotate = (is_q || is_k) && a.cs != nullptr;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
        const int j = lane + 32 * i;
        if (j < half) {
            float u = x1[i], w = x2[i];
            // explicit roundings: the result must not depend on how the compiler contracts
            // multiplies and adds in the different kernels this is inlined into
            if (gamma) { u = __fmul_rn(__fmul_rn(u, inv), gamma[j]); w = __fmul_rn(__fmul_rn(w, inv), gamma[j + half]); }
            if (rotate) {
                const float2 c = a.cs[(size_t)t * half + j];
                const float ru = __fmaf_rn(u, c.x, -__fmul_rn(w, c.y));
                const float rw = __fmaf_rn(w, c.x, __fmul_rn(u, c.y));
                u = ru; w = rw;
            }
            if (dst_a) { from_f32(dst_a[j], u); from_f32(dst_a[j + half], w); }
            if (dst_b) { from_f32(dst_b[j], u); from_f32(dst_b[j + half], w); }
        }
    }
}

// The same for a tile of 128 consecutive features of the projection (whole heads: 128 % head_dim == 0)
// held by one warp, four consecutive features per lane (lane l: features f0 + 4 l .. + 3): norm over
// each head's lanes, rotation partner by shuffle, 8-byte stores.  page / prow: the token's place in
// the cache (page number, row inside the page).  Every lane of the warp must call it.
//
// What a lane needs that does not change from token to token (head_dim is a power of two here):
struct Tile4Lane {
    int sh;                   // log2(lanes per head)
    int d;                    // first of this lane's four dims within its head
    int cs_j;                 // first of its four (cos, sin) pairs in a token's row of the table
    bool first;               // its dims lie below head_dim / 2
    float4 gq, gk;            // the norm weights of its dims
};
__device__ __forceinline__ Tile4Lane qkv_tile4_lane(const QkvArgs& a, int lane) {
    Tile4Lane L;
    const int lph = a.hd >> 2;                        // lanes per head
    L.sh = 31 - __clz(lph);
    const int li = lane & (lph - 1);
    L.d = li * 4;
    L.first = li < (lph >> 1);
    L.cs_j = L.first ? L.d : L.d - (a.hd >> 1);
    L.gq = a.gq ? *reinterpret_cast<const float4*>(a.gq + L.d) : make_float4(0.f, 0.f, 0.f, 0.f);
    L.gk = a.gk ? *reinterpret_cast<const float4*>(a.gk + L.d) : make_float4(0.f, 0.f, 0.f, 0.f);
    return L;
}
// the lane's (cos, sin) of token t for the tile at feature f0, or nullptr if its head is not rotated
__device__ __forceinline__ const float4* qkv_tile4_cs(const QkvArgs& a, const Tile4Lane& L, int t, int f0, int lane) {
    const int head = (f0 >> (L.sh + 2)) + (lane >> L.sh);
    if (a.cs == nullptr || head >= a.n_q + a.n_kv) return nullptr;
    return reinterpret_cast<const float4*>(a.cs + (size_t)t * (a.hd >> 1) + L.cs_j);
}
// ca, cb: what qkv_tile4_cs points to (unused if it is nullptr)
// row_live = false: the arithmetic runs (the shuffles are warp-wide) but nothing is stored
__device__ __forceinline__ void qkv_finish_tile4_pre(const QkvArgs& a, const Tile4Lane& L, float4 v, int t, int f0, int lane,
                                                     int page, int prow, const float4& ca, const float4& cb,
                                                     bool row_live = true) {
    const int lph = 1 << L.sh;
    const int head = (f0 >> (L.sh + 2)) + (lane >> L.sh);
    const int heads = a.n_q + 2 * a.n_kv;
    const bool is_q = head < a.n_q, is_k = !is_q && head < a.n_q + a.n_kv, live = head < heads && row_live;
    const bool normed = is_q ? a.gq != nullptr : (is_k && a.gk != nullptr);
    float x[4] = {v.x, v.y, v.z, v.w};
    // (every lane runs the shuffles, whatever its head is: they are warp-wide)
    float ss = __fmaf_rn(x[3], x[3], __fmaf_rn(x[2], x[2], __fmaf_rn(x[1], x[1], __fmul_rn(x[0], x[0]))));
    for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (live && normed) {
        const float inv = head_inv_rms(a, ss);
        const float4 gm = is_q ? L.gq : L.gk;
        x[0] = __fmul_rn(__fmul_rn(x[0], inv), gm.x); x[1] = __fmul_rn(__fmul_rn(x[1], inv), gm.y);
        x[2] = __fmul_rn(__fmul_rn(x[2], inv), gm.z); x[3] = __fmul_rn(__fmul_rn(x[3], inv), gm.w);
    }
    float other[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) other[i] = __shfl_xor_sync(0xffffffffu, x[i], lph >> 1);   // the rotation partner
    if (live && (is_q || is_k) && a.cs != nullptr) {
        const float cs_[4][2] = {{ca.x, ca.y}, {ca.z, ca.w}, {cb.x, cb.y}, {cb.z, cb.w}};
#pragma unroll
        for (int i = 0; i < 4; ++i)
            x[i] = L.first ? __fmaf_rn(x[i], cs_[i][0], -__fmul_rn(other[i], cs_[i][1]))
                           : __fmaf_rn(x[i], cs_[i][0], __fmul_rn(other[i], cs_[i][1]));
    }
    if (live) {
        T* dst_a = nullptr; T* dst_b = nullptr;
        if (is_q) {
            dst_a = a.q_out + ((size_t)t * a.n_q + head) * a.hd + L.d;
        } else {
            const int g = is_k ? head - a.n_q : head - a.n_q - a.n_kv;
            if (a.write_cache)
                dst_a = (is_k ? a.cache.k : a.cache.v) +
                        (((size_t)page * a.n_kv + g) * IDM_PAGE + prow) * (size_t)a.hd + L.d;
            T* packed = is_k ? a.k_new : a.v_new;
            if (packed) dst_b = packed + ((size_t)t * a.n_kv + g) * a.hd + L.d;
        }
        if (dst_a) store4(dst_a, x);
        if (dst_b) store4(dst_b, x);
    }
}
__device__ __forceinline__ void qkv_finish_tile4(const QkvArgs& a, float4 v, int t, int f0, int lane, int page, int prow) {
    const Tile4Lane L = qkv_tile4_lane(a, lane);
    const float4* c4 = qkv_tile4_cs(a, L, t, f0, lane);
    float4 ca = make_float4(0.f, 0.f, 0.f, 0.f), cb = ca;
    if (c4) { ca = c4[0]; cb = c4[1]; }
    qkv_finish_tile4_pre(a, L, v, t, f0, lane, page, prow, ca, cb);
}
