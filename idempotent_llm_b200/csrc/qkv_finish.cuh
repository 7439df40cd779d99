// q/k norm + rotation + cache write for one (token, head) row of the fused q/k/v projection, done
// by one warp.  q and k heads: RMS norm over head_dim with a weight of shape [head_dim] shared by all
// heads (src/detllm/model.py:208-215), then rotation of pairs (d, d + hd/2) by the token's position
// (src/detllm/ops/rope.py:47-55); v heads are copied.  q goes to q_out [N, n_q, hd]; k and v go to
// the cache at the token's position and/or to packed buffers k_new, v_new [N, n_kv, hd].
// `load(j)` returns element j of the row in 32-bit (from partial sums in memory, or from a tile in
// shared memory when this runs as the epilogue of the matrix product).
#pragma once

#include "common.cuh"

struct QkvArgs {
    const float* qkv; int n_partials; size_t partial_stride;
    int n_tokens, n_q, n_kv, hd;
    const float* gq; const float* gk; float eps;
    const float2* cs;
    T* q_out; T* k_new; T* v_new;
    KVAddr cache; int write_cache;
    const int* token_seq; const int* positions; const int* slots;
};

// where the token's key/value row of kv-head g starts in the pools
struct QkvLocateFromTables {
    const QkvArgs& a; int t;
    __device__ __forceinline__ size_t operator()(int g) const {
        return kv_offset(a.cache, a.slots[a.token_seq[t]], a.positions[t], g);
    }
};

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
        inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)a.hd), a.eps)));
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
