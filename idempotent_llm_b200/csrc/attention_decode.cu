// Attention for steps of one token per sequence, bound by reading the cache.
//
// Grid (chunk, kv-head, sequence).  A chunk is 256 keys at absolute positions
// [256 c, 256 c + 256): four pages, one per warp.  A block serves all q-heads of its
// kv-head (GT at a time), so keys and values are read from memory once per group.
// Each row of head_dim elements is split over LPR lanes in 16-byte pieces; a warp-wide
// load covers 32 / LPR keys.  Scores, the running maximum, the exponentials and the
// context are 32-bit.  Every chunk writes an unnormalised partial (max, sum, context)
// to scratch; the block that finishes last for a (sequence, kv-head) -- found with a
// counter in scratch that it sets back to zero -- merges that sequence's chunks in
// ascending order, whichever block it is.  Which keys form a chunk and in which order
// everything is added depend on the sequence's length only: a sequence's result is the
// same alone or in any batch.
//
// Masked keys (beyond the length, or before the window) give p = 0 exactly and are left
// out of the maximum (src/detllm/ops/di_softmax.py:45-58 does this with an integer
// sentinel; ops/fused_attn.py:47-115 is the reference's own decode kernel: one program
// per (batch, q-head), three passes over a capacity-wide cache).
#include "common.cuh"

#ifndef AD_CHUNK
#define AD_CHUNK 256
#endif
#ifndef AD_WARPS
#define AD_WARPS (AD_CHUNK / 64)   // warps of a block; each takes AD_CHUNK / AD_WARPS consecutive keys (at most a page)
#endif
#define AD_WKEYS (AD_CHUNK / AD_WARPS)
#ifndef AD_ITERS
#define AD_ITERS 8            // warp-wide loads per group
#endif
#ifndef AD_PREFETCH
#define AD_PREFETCH 0         // 1: the next group's loads are issued before this group's arithmetic
#endif
#define AD_COUNTER_SLOTS 65536  // arrival counters at the start of scratch: a fixed place, so that they are
                                // zero at every launch whatever the sizes of earlier launches were

struct DecodeArgs {
    const T* q; T* out;
    KVAddr cache;
    const int* slots; const int* kv_len;
    float* part_o;            // [n_seqs, n_q, n_chunks, hd]
    float* part_ml;           // [n_seqs, n_q, n_chunks, 2]
    int* counters;            // [n_seqs, n_kv], zero between launches
    int n_seqs, n_q, n_kv, n_chunks;
    float scale_log2; int window;
    int early_trigger;        // 1: let the next kernel's blocks be scheduled as soon as this one's have started
};

// A sequence's length as this launch sees it: never beyond the chunks the grid has.  (A caller that passes a
// max_kv_len below some kv_len gets that sequence cut short, which is its own error; but every chunk that is
// counted on then arrives, so the arrival counters in scratch are back at zero when the launch ends -- they
// outlive the launch, and in the entry point without allocation they outlive every call of the process.)
__device__ __forceinline__ int decode_len(const DecodeArgs& a, int s) { return min(a.kv_len[s], a.n_chunks * AD_CHUNK); }

// out[s, head, :] = sum_c 2^(m_c - M) o_c / sum_c 2^(m_c - M) l_c over the sequence's chunks, ascending.
// One warp per (sequence, q-head).  Partials were written by other blocks: read around L1.
__device__ __forceinline__ void decode_merge_head(const DecodeArgs& a, int s, int head, int hd, int lane) {
    const int warp = s * a.n_q + head;
    const int len = decode_len(a, s);
    const int lo = a.window > 0 ? max(0, len - a.window) : 0;
    const int c0 = lo / AD_CHUNK, c1 = (len - 1) / AD_CHUNK;
    const size_t row0 = (size_t)warp * a.n_chunks;
    // lane c holds chunk c0 + c (+32, +64, ...): maxima and sums of up to 32 chunks at a time
    float M = -INFINITY;
    for (int c = c0 + lane; c <= c1; c += 32) M = fmaxf(M, __ldcg(a.part_ml + (row0 + c) * 2));
    M = warp_max(M);
    float L = 0.f;
    float acc[IDM_MAX_HEAD_DIM / 32];
#pragma unroll
    for (int i = 0; i < IDM_MAX_HEAD_DIM / 32; ++i) acc[i] = 0.f;
    for (int cb = c0; cb <= c1; cb += 32) {
        const int mine = cb + lane;
        float f_mine = 0.f, l_mine = 0.f;
        if (mine <= c1) {
            const float mc = __ldcg(a.part_ml + (row0 + mine) * 2);
            f_mine = mc == -INFINITY ? 0.f : exp2f(mc - M);
            l_mine = __ldcg(a.part_ml + (row0 + mine) * 2 + 1);
        }
        const int n_here = min(32, c1 - cb + 1);
        for (int j0 = 0; j0 < n_here; j0 += 4) {                   // four chunks' loads in flight together
            float f[4], o[4][IDM_MAX_HEAD_DIM / 32];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u;
                f[u] = __shfl_sync(0xffffffffu, f_mine, j & 31);
                const float lj = __shfl_sync(0xffffffffu, l_mine, j & 31);
                if (j < n_here) L += f[u] * lj;                    // ascending chunks
#pragma unroll
                for (int i = 0; i < IDM_MAX_HEAD_DIM / 32; ++i) {
                    const int d = lane + 32 * i;
                    o[u][i] = (j < n_here && d < hd) ? __ldcg(a.part_o + (row0 + cb + j) * hd + d) : 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (j0 + u < n_here) {
#pragma unroll
                    for (int i = 0; i < IDM_MAX_HEAD_DIM / 32; ++i) acc[i] += f[u] * o[u][i];
                }
        }
    }
    const float inv = 1.0f / L;
    T* orow = a.out + (size_t)warp * hd;
#pragma unroll
    for (int i = 0; i < IDM_MAX_HEAD_DIM / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) from_f32(orow[d], acc[i] * inv);
    }
}

// The same for head sizes of 64 and 128 with every load of up to 16 chunks asked for at once (the
// maxima and sums, and each chunk's context as one 8- or 16-byte piece per lane): the block that merges
// waits for memory once instead of once per four chunks.  Same order of additions, same bits.
template <int HD>
__device__ __forceinline__ void decode_merge_head_wide(const DecodeArgs& a, int s, int head, int lane) {
    constexpr int V = HD / 32;                               // consecutive dims per lane
    const int warp = s * a.n_q + head;
    const int len = decode_len(a, s);
    const int lo = a.window > 0 ? max(0, len - a.window) : 0;
    const int c0 = lo / AD_CHUNK, c1 = (len - 1) / AD_CHUNK;
    const size_t row0 = (size_t)warp * a.n_chunks;
    float M = -INFINITY;
    for (int c = c0 + lane; c <= c1; c += 32) M = fmaxf(M, __ldcg(a.part_ml + (row0 + c) * 2));
    float L = 0.f;
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    bool have_m = false;
    for (int cb = c0; cb <= c1; cb += 16) {
        // the contexts of chunks cb .. cb + 15 (they do not depend on the maximum: asked for first)
        float o[16][V];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
#pragma unroll
            for (int i = 0; i < V; ++i) o[u][i] = 0.f;
            if (cb + u <= c1) {
                const float* src = a.part_o + (row0 + cb + u) * HD + lane * V;
                if (V == 4) {
                    const float4 t = __ldcg(reinterpret_cast<const float4*>(src));
                    o[u][0] = t.x; o[u][1] = t.y; o[u][V > 2 ? 2 : 0] = t.z; o[u][V > 2 ? 3 : 1] = t.w;
                } else {
                    const float2 t = __ldcg(reinterpret_cast<const float2*>(src));
                    o[u][0] = t.x; o[u][1] = t.y;
                }
            }
        }
        const int mine = cb + (lane & 15);                   // lanes 0..15 (and their mirrors) hold chunk cb + lane
        float2 ml = make_float2(-INFINITY, 0.f);
        if (mine <= c1) ml = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (row0 + mine) * 2));
        if (!have_m) { M = warp_max(M); have_m = true; }
        const float f_mine = ml.x == -INFINITY ? 0.f : exp2f(ml.x - M);
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const float f = __shfl_sync(0xffffffffu, f_mine, u);
            const float lj = __shfl_sync(0xffffffffu, ml.y, u);
            if (cb + u <= c1) {
                L += f * lj;                                 // ascending chunks
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] += f * o[u][i];
            }
        }
    }
    const float inv = 1.0f / L;
    T* orow = a.out + (size_t)warp * HD + lane * V;
    if constexpr (V == 4) {
        store4(orow, acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
    } else {
#pragma unroll
        for (int i = 0; i < V; ++i) from_f32(orow[i], acc[i] * inv);
    }
}

template <int HD, int GT>
__global__ void __launch_bounds__(AD_WARPS * 32) attention_decode_kernel(DecodeArgs a) {
    if (a.early_trigger) pdl_launch_dependents();
    pdl_wait();
    constexpr int VEC = Vec16<T>::N;
    constexpr int LPR = HD / VEC;            // lanes per row
    constexpr int RPI = 32 / LPR;            // rows (keys) per warp-wide load
    constexpr int GROUP = AD_ITERS * RPI;    // keys per group
    static_assert(LPR >= 1 && LPR <= 32 && (LPR & (LPR - 1)) == 0, "head_dim / 16 bytes must be a power of two <= 32");
    static_assert(AD_WKEYS <= IDM_PAGE && IDM_PAGE % AD_WKEYS == 0, "a warp's keys lie inside one page");
    __shared__ float sm_m[AD_WARPS][GT], sm_l[AD_WARPS][GT];
    __shared__ float sm_o[AD_WARPS][GT][HD];

    const int chunk = blockIdx.x, g = blockIdx.y, s = blockIdx.z;
    const int len = decode_len(a, s);
    const int lo = a.window > 0 ? max(0, len - a.window) : 0;
    if (chunk * AD_CHUNK >= len || (chunk + 1) * AD_CHUNK <= lo) return;      // nothing to see here
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / LPR, li = lane % LPR;
    const int group_heads = a.n_q / a.n_kv;
    const int kb = chunk * AD_CHUNK + wib * AD_WKEYS;                        // this warp's keys (inside one page)
    const bool warp_live = kb < len && kb + AD_WKEYS > lo;
    const T* kpage = nullptr; const T* vpage = nullptr;
    if (warp_live) {
        const size_t off = kv_offset(a.cache, a.slots[s], kb, g);
        kpage = a.cache.k + off; vpage = a.cache.v + off;
    }
    for (int h0 = 0; h0 < group_heads; h0 += GT) {
        float q[GT][VEC], acc[GT][VEC], m[GT], l[GT];
#pragma unroll
        for (int h = 0; h < GT; ++h) {
            Vec16<T> qv; qv.load(a.q + ((size_t)s * a.n_q + g * group_heads + h0 + h) * HD + li * VEC);
#pragma unroll
            for (int e = 0; e < VEC; ++e) { q[h][e] = qv.get(e) * a.scale_log2; acc[h][e] = 0.f; }
            m[h] = -INFINITY; l[h] = 0.f;
        }
        if (warp_live) {
            constexpr int KEYS = AD_WKEYS;
            constexpr int NG = (KEYS + GROUP - 1) / GROUP;          // groups per page
            // Two register buffers: the next group's keys and values are on their way while this
            // group is worked on.  Every row of a live page is readable memory (rows past the
            // length hold stale data and are masked below).
            Vec16<T> kbuf[AD_PREFETCH + 1][AD_ITERS], vbuf[AD_PREFETCH + 1][AD_ITERS];
            auto fetch = [&](int grp, int buf) {
#pragma unroll
                for (int it = 0; it < AD_ITERS; ++it) {
                    const int r = grp * GROUP + it * RPI + sub;
                    if (r < KEYS) {
                        kbuf[buf][it].load(kpage + (size_t)r * HD + li * VEC);
                        vbuf[buf][it].load(vpage + (size_t)r * HD + li * VEC);
                    }
                }
            };
            if (AD_PREFETCH) fetch(0, 0);
#pragma unroll
            for (int grp = 0; grp < NG; ++grp) {
                const int cur = AD_PREFETCH ? (grp & 1) : 0;
                const int k0 = grp * GROUP;
                if (AD_PREFETCH) {
                    if (grp + 1 < NG) fetch(grp + 1, cur ^ 1);
                    if (kb + k0 >= len || kb + k0 + GROUP <= lo) continue;   // warp-uniform: no live key here
                } else {
                    if (kb + k0 >= len || kb + k0 + GROUP <= lo) continue;
                    fetch(grp, 0);
                }
                float sc[AD_ITERS][GT];
#pragma unroll
                for (int it = 0; it < AD_ITERS; ++it) {
                    const int r = k0 + it * RPI + sub;
                    const int j = kb + r;
                    const bool ok = r < KEYS && j < len && j >= lo;
#pragma unroll
                    for (int h = 0; h < GT; ++h) {
                        float d = 0.f;
                        if (r < KEYS) {
#pragma unroll
                            for (int e = 0; e < VEC; ++e) d = fmaf(q[h][e], kbuf[cur][it].get(e), d);
                        }
#pragma unroll
                        for (int o = LPR / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                        sc[it][h] = ok ? d : -INFINITY;
                    }
                }
#pragma unroll
                for (int h = 0; h < GT; ++h) {
                    float gm = sc[0][h];
#pragma unroll
                    for (int it = 1; it < AD_ITERS; ++it) gm = fmaxf(gm, sc[it][h]);
#pragma unroll
                    for (int o = LPR; o < 32; o <<= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, o));
                    const float m_new = fmaxf(m[h], gm);            // finite: the group holds a live key
                    const float alpha = exp2f(m[h] - m_new);
                    m[h] = m_new;
                    float ps = 0.f;
#pragma unroll
                    for (int e = 0; e < VEC; ++e) acc[h][e] *= alpha;
#pragma unroll
                    for (int it = 0; it < AD_ITERS; ++it) {
                        const float p = sc[it][h] == -INFINITY ? 0.f : exp2f(sc[it][h] - m_new);
                        ps += p;
                        if (p != 0.f) {
#pragma unroll
                            for (int e = 0; e < VEC; ++e) acc[h][e] = fmaf(p, vbuf[cur][it].get(e), acc[h][e]);
                        }
                    }
                    l[h] = l[h] * alpha + ps;
                }
            }
        }
        // lanes of different `sub` hold different keys of the same dims: add them up
#pragma unroll
        for (int h = 0; h < GT; ++h) {
#pragma unroll
            for (int o = LPR; o < 32; o <<= 1) {
                l[h] += __shfl_xor_sync(0xffffffffu, l[h], o);
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[h][e] += __shfl_xor_sync(0xffffffffu, acc[h][e], o);
            }
        }
        __syncthreads();                                  // previous pass's readers are done
        if (lane < LPR) {
#pragma unroll
            for (int h = 0; h < GT; ++h) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) sm_o[wib][h][li * VEC + e] = acc[h][e];
                if (lane == 0) { sm_m[wib][h] = m[h]; sm_l[wib][h] = l[h]; }
            }
        }
        __syncthreads();
        // merge the four warps in ascending order and write the chunk's partial
        for (int idx = threadIdx.x; idx < GT * HD; idx += AD_WARPS * 32) {
            const int h = idx / HD, d = idx % HD;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < AD_WARPS; ++w) M = fmaxf(M, sm_m[w][h]);
            float o = 0.f, L = 0.f;
#pragma unroll
            for (int w = 0; w < AD_WARPS; ++w) {
                const float f = sm_m[w][h] == -INFINITY ? 0.f : exp2f(sm_m[w][h] - M);
                o += f * sm_o[w][h][d];
                L += f * sm_l[w][h];
            }
            const size_t row = ((size_t)s * a.n_q + g * group_heads + h0 + h) * a.n_chunks + chunk;
            a.part_o[row * HD + d] = o;
            if (d == 0) { a.part_ml[row * 2] = M; a.part_ml[row * 2 + 1] = L; }
        }
    }
    // The block that arrives last for this (sequence, kv-head) merges the chunks.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int live = (len - 1) / AD_CHUNK - lo / AD_CHUNK + 1;
        const int prev = atomicAdd(&a.counters[s * a.n_kv + g], 1);
        is_last = prev == live - 1;
        if (is_last) a.counters[s * a.n_kv + g] = 0;             // ready for the next launch
    }
    __syncthreads();
    if (is_last) {
        __threadfence();
        for (int h = wib; h < group_heads; h += AD_WARPS) decode_merge_head(a, s, g * group_heads + h, HD, lane);
    }
}

#if defined(IDM_BF16)
// ------------------------------------------------------------- the same on mma.sync fragments
// For bfloat16 caches with head_dim 64 or 128 and up to 8 q-heads per kv-head.  The scalar kernel above
// spends its issue slots on FMAs and shuffles (a page of 64 keys costs a warp ~2 000 instructions);
// here q . k^T and p . v are m16n8k16 tensor-core products on registers (a page costs ~450):
//   * the 16 rows of the MMA tile are the group's q-heads (rows past the group are zero);
//   * a thread reads 16-byte pieces of key and value rows straight from the cache, coalesced; because
//     a dot product does not care in which order its terms come, the piece a thread holds is used as
//     the fragment of two k-steps (dims are permuted the same way for q and k);
//   * value fragments need keys along k: each 8 x 8 piece is transposed in registers with movmatrix;
//     the permutation makes a thread's output columns the same 8 consecutive dims it loads.
// Chunks, partials, the order of the merge and the masking rules are those of the scalar kernel.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}

template <int HD>
__global__ void __launch_bounds__(AD_WARPS * 32) attention_decode_mma_kernel(DecodeArgs a) {
    if (a.early_trigger) pdl_launch_dependents();
    pdl_wait();
    constexpr int NC = HD / 32;              // 32-dim pieces of a row: a thread holds 8 dims of each
    constexpr int GT = 8;                    // q-heads per block (rows 0..7 of the tile)
    __shared__ float sm_m[AD_WARPS][GT], sm_l[AD_WARPS][GT];
    __shared__ float sm_o[AD_WARPS][GT][HD];
    __shared__ int is_last;

    const int chunk = blockIdx.x, g = blockIdx.y, s = blockIdx.z;
    const int len = decode_len(a, s);
    const int lo = a.window > 0 ? max(0, len - a.window) : 0;
    if (chunk * AD_CHUNK >= len || (chunk + 1) * AD_CHUNK <= lo) return;
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;             // fragment row / column pair
    const int group_heads = a.n_q / a.n_kv;
    const int kb = chunk * AD_CHUNK + wib * IDM_PAGE;      // this warp's page of keys
    const bool warp_live = kb < len && kb + IDM_PAGE > lo;

    // q fragments: row gid = q-head gid of the group; piece c of the row feeds k-steps 2c and 2c + 1
    uint32_t qa[2 * NC][4];
    {
        const bool row_live = gid < group_heads;
        const T* qrow = a.q + ((size_t)s * a.n_q + g * group_heads + (row_live ? gid : 0)) * HD;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row_live) v = *reinterpret_cast<const uint4*>(qrow + 32 * c + tig * 8);
            qa[2 * c][0] = v.x; qa[2 * c][2] = v.y; qa[2 * c + 1][0] = v.z; qa[2 * c + 1][2] = v.w;
            qa[2 * c][1] = qa[2 * c][3] = qa[2 * c + 1][1] = qa[2 * c + 1][3] = 0;      // rows 8..15: none
        }
    }
    float o[4 * NC][4];                      // o[4 c + m]: dims 32 c + 8 tig + 2 m (+1) of row gid (and row gid + 8, unused)
#pragma unroll
    for (int i = 0; i < 4 * NC; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run = -INFINITY, l_run = 0.f;    // of row gid; l is this thread's share (keys 2 tig, 2 tig + 1 of each tile)

    if (warp_live) {
        const size_t off = kv_offset(a.cache, a.slots[s], kb, g);
        const T* kpage = a.cache.k + off;
        const T* vpage = a.cache.v + off;
        // scores of the page: 8 tiles of 8 keys
        float sc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
            const T* krow = kpage + (size_t)(8 * j + gid) * HD + tig * 8;
            uint4 kv[NC];
#pragma unroll
            for (int c = 0; c < NC; ++c) kv[c] = *reinterpret_cast<const uint4*>(krow + 32 * c);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                mma_bf16_16816(sc[j], qa[2 * c], kv[c].x, kv[c].y);
                mma_bf16_16816(sc[j], qa[2 * c + 1], kv[c].z, kv[c].w);
            }
        }
        // mask, scale, row maximum (row gid: this thread's 16 scores, then the 4 threads of the row)
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = kb + 8 * j + 2 * tig + e;
                const float v = (key < len && key >= lo) ? sc[j][e] * a.scale_log2 : -INFINITY;
                sc[j][e] = v;
                mx = fmaxf(mx, v);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        m_run = mx;                          // finite: the page holds a live key, and every row sees the same keys
        uint32_t pa[4][4];                   // p as A fragments: k-step t = key tiles 2t, 2t + 1
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float p0 = exp2f(sc[j][0] - m_run), p1 = exp2f(sc[j][1] - m_run);       // exp2(-inf) = 0
            l_run += p0 + p1;
            pa[j >> 1][(j & 1) * 2] = pack_bf16x2(p0, p1);
            pa[j >> 1][(j & 1) * 2 + 1] = 0;                                             // rows 8..15
        }
        // o = p . v
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            uint4 v0[NC], v1[NC];            // value rows of key tiles 2t and 2t + 1
            const int key0 = kb + 16 * t + gid, key1 = key0 + 8;
            const T* vrow = vpage + (size_t)(16 * t + gid) * HD + tig * 8;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                v0[c] = *reinterpret_cast<const uint4*>(vrow + 32 * c);
                v1[c] = *reinterpret_cast<const uint4*>(vrow + 8 * HD + 32 * c);
                // rows past the length (or before the window) hold stale data: p is 0 there, but 0 * NaN is not
                if (key0 >= len || key0 < lo) v0[c] = make_uint4(0, 0, 0, 0);
                if (key1 >= len || key1 < lo) v1[c] = make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const uint32_t r0[4] = {v0[c].x, v0[c].y, v0[c].z, v0[c].w};
                const uint32_t r1[4] = {v1[c].x, v1[c].y, v1[c].z, v1[c].w};
#pragma unroll
                for (int mth = 0; mth < 4; ++mth)
                    mma_bf16_16816(o[4 * c + mth], pa[t], movmatrix_trans(r0[mth]), movmatrix_trans(r1[mth]));
            }
        }
    }
    // the row's sum: the 4 threads of the row hold different keys
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (gid < GT) {
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int mth = 0; mth < 4; ++mth) {
                sm_o[wib][gid][32 * c + 8 * tig + 2 * mth] = o[4 * c + mth][0];
                sm_o[wib][gid][32 * c + 8 * tig + 2 * mth + 1] = o[4 * c + mth][1];
            }
        if (tig == 0) { sm_m[wib][gid] = m_run; sm_l[wib][gid] = l_run; }
    }
    __syncthreads();
    // merge the warps in ascending order and write the chunk's partial
    for (int idx = threadIdx.x; idx < group_heads * HD; idx += AD_WARPS * 32) {
        const int h = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) M = fmaxf(M, sm_m[w][h]);
        float ov = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) {
            const float f = sm_m[w][h] == -INFINITY ? 0.f : exp2f(sm_m[w][h] - M);
            ov += f * sm_o[w][h][d];
            L += f * sm_l[w][h];
        }
        const size_t row = ((size_t)s * a.n_q + g * group_heads + h) * a.n_chunks + chunk;
        a.part_o[row * HD + d] = ov;
        if (d == 0) { a.part_ml[row * 2] = M; a.part_ml[row * 2 + 1] = L; }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int live = (len - 1) / AD_CHUNK - lo / AD_CHUNK + 1;
        const int prev = atomicAdd(&a.counters[s * a.n_kv + g], 1);
        is_last = prev == live - 1;
        if (is_last) a.counters[s * a.n_kv + g] = 0;
    }
    __syncthreads();
    if (is_last) {
        __threadfence();
        for (int h = wib; h < group_heads; h += AD_WARPS) decode_merge_head_wide<HD>(a, s, g * group_heads + h, lane);
    }
}
#endif  // IDM_BF16

template <int HD>
static int launch_decode(const DecodeArgs& a, int group_heads, cudaStream_t stream) {
    dim3 grid(a.n_chunks, a.n_kv, a.n_seqs);
    // launched early, this kernel's waiting blocks (all registers of an SM) slow the product before it: measured
    static const bool pdl = idm_pdl_flag("IDM_PDL_ATTN", 0);
    static const bool early = idm_pdl_flag("IDM_PDL_ATTN_EARLY", 1);
    DecodeArgs b = a;
    b.early_trigger = early;
    if (group_heads % 4 == 0) idm_launch_opt(pdl, attention_decode_kernel<HD, 4>, dim3(grid), dim3(AD_WARPS * 32), 0, stream, b);
    else if (group_heads % 2 == 0) idm_launch_opt(pdl, attention_decode_kernel<HD, 2>, dim3(grid), dim3(AD_WARPS * 32), 0, stream, b);
    else idm_launch_opt(pdl, attention_decode_kernel<HD, 1>, dim3(grid), dim3(AD_WARPS * 32), 0, stream, b);
    return 0;
}

// 1 if this library has the kernel for the head size, else 0 (the caller then uses the general kernel)
extern "C" int idm_attention_decode_supports(int hd) {
    constexpr int VEC = Vec16<T>::N;
    return hd == VEC * 2 || hd == VEC * 4 || hd == VEC * 8 || hd == VEC * 16 || (hd == VEC * 32 && hd <= 256);
}

extern "C" int idm_attention_decode_chunk() { return AD_CHUNK; }

// floats of scratch for the partials: part_o then part_ml
extern "C" long long idm_attention_decode_scratch_floats(int n_seqs, int n_q, int n_chunks, int hd) {
    return (long long)AD_COUNTER_SLOTS + (long long)n_seqs * n_q * n_chunks * (hd + 2);   // counters + partials
}

extern "C" int idm_attention_decode(const void* q, void* out, void* k_pool, void* v_pool, const int* table,
                                    int table_stride, int ring, const int* slots, const int* kv_len,
                                    float* scratch, int n_seqs, int n_q, int n_kv, int hd, int max_kv_len,
                                    float scale, int window, cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    IDM_REQUIRE(idm_attention_decode_supports(hd), "attention_decode: head_dim=%d has no kernel here", hd);
    IDM_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "attention_decode: %d q-heads are no multiple of %d kv-heads", n_q, n_kv);
    IDM_REQUIRE(max_kv_len > 0 && n_seqs <= 65535 && n_kv <= 65535, "attention_decode: bad sizes");
    DecodeArgs a;
    a.q = (const T*)q; a.out = (T*)out;
    a.cache = KVAddr{(T*)k_pool, (T*)v_pool, table, table_stride, ring, n_kv, hd};
    a.slots = slots; a.kv_len = kv_len;
    a.n_seqs = n_seqs; a.n_q = n_q; a.n_kv = n_kv;
    a.n_chunks = (max_kv_len + AD_CHUNK - 1) / AD_CHUNK;
    IDM_REQUIRE((long long)n_seqs * n_kv <= AD_COUNTER_SLOTS, "attention_decode: %d sequences x %d kv-heads exceed %d",
                n_seqs, n_kv, AD_COUNTER_SLOTS);
    a.counters = (int*)scratch;
    a.part_o = scratch + AD_COUNTER_SLOTS;
    a.part_ml = a.part_o + (size_t)n_seqs * n_q * a.n_chunks * hd;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.window = window;
    const int gh = n_q / n_kv;
    constexpr int VEC = Vec16<T>::N;
#if defined(IDM_BF16)
    static const bool use_mma = idm_pdl_flag("IDM_DECODE_MMA", 1);
    if (use_mma && (hd == 64 || hd == 128) && gh <= 8 && AD_WARPS * IDM_PAGE == AD_CHUNK) {
        static const bool pdl = idm_pdl_flag("IDM_PDL_ATTN", 0);
        static const bool early = idm_pdl_flag("IDM_PDL_ATTN_EARLY", 1);
        a.early_trigger = early;
        dim3 grid(a.n_chunks, a.n_kv, a.n_seqs);
        if (hd == 128) idm_launch_opt(pdl, attention_decode_mma_kernel<128>, grid, dim3(AD_WARPS * 32), 0, stream, a);
        else idm_launch_opt(pdl, attention_decode_mma_kernel<64>, grid, dim3(AD_WARPS * 32), 0, stream, a);
        IDM_LAUNCH_CHECK("attention_decode_mma");
        return 0;
    }
#endif
    if (hd == VEC * 2) launch_decode<VEC * 2>(a, gh, stream);
    else if (hd == VEC * 4) launch_decode<VEC * 4>(a, gh, stream);
    else if (hd == VEC * 8) launch_decode<VEC * 8>(a, gh, stream);
    else if (hd == VEC * 16) launch_decode<VEC * 16>(a, gh, stream);
    else launch_decode<(VEC * 32 <= 256 ? VEC * 32 : 256)>(a, gh, stream);
    IDM_LAUNCH_CHECK("attention_decode");
    return 0;
}

// ------------------------------------------------------------------ entry point without allocation
// Declared and documented in idm_no_alloc.h.  The partial results of the chunks go to a fixed array
// that is part of the loaded library instead of caller-provided scratch.
#include "idm_no_alloc.h"

static __device__ __align__(256) float g_decode_scratch[IDM_NO_ALLOC_MAX_SCRATCH_FLOATS];

#define IDM_NO_ALLOC_MAX_DEVICES 64
static float* g_decode_scratch_ptr[IDM_NO_ALLOC_MAX_DEVICES];   // device address of the array, per device

extern "C" int idm_attention_decode_static(const void* q, void* out, void* k_pool, void* v_pool,
                                           const int* table, int table_stride, int ring, const int* slots,
                                           const int* kv_len, int n_seqs, int n_q, int n_kv, int hd,
                                           int max_kv_len, float scale, int window, cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    IDM_REQUIRE(n_seqs > 0 && n_q > 0 && hd > 0 && max_kv_len > 0, "attention_decode_static: bad sizes");
    const long long n_chunks = (max_kv_len + AD_CHUNK - 1) / AD_CHUNK;
    const long long need = idm_attention_decode_scratch_floats(n_seqs, n_q, (int)n_chunks, hd);
    IDM_REQUIRE(need <= (long long)IDM_NO_ALLOC_MAX_SCRATCH_FLOATS,
                "attention_decode_static: %d sequences x %d heads x %lld chunks x (%d + 2) = %lld floats of scratch; "
                "the built-in array holds %lld",
                n_seqs, n_q, n_chunks, hd, need, (long long)IDM_NO_ALLOC_MAX_SCRATCH_FLOATS);
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    IDM_REQUIRE(e == cudaSuccess, "attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    IDM_REQUIRE(dev >= 0 && dev < IDM_NO_ALLOC_MAX_DEVICES, "attention_decode_static: device %d out of range", dev);
    if (g_decode_scratch_ptr[dev] == nullptr) {
        // set-up, once per device, with that device current: the array's name is a host-side stand-in
        // here, not a device address; the address a kernel can use comes from the runtime
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_decode_scratch);
        IDM_REQUIRE(e == cudaSuccess && p != nullptr, "attention_decode_static: cudaGetSymbolAddress: %s",
                    cudaGetErrorString(e));
        g_decode_scratch_ptr[dev] = p;
    }
    // the partial results need no clearing (every chunk the merge reads was written by this call); the
    // arrival counters behind them must be zero at launch: the array starts as zeros and each launch
    // sets its counters back to zero before it ends
    return idm_attention_decode(q, out, k_pool, v_pool, table, table_stride, ring, slots, kv_len,
                                g_decode_scratch_ptr[dev], n_seqs, n_q, n_kv, hd, max_kv_len, scale, window, stream);
}
