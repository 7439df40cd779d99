// Attention over the cache for any head size (multiple of 8 up to 256), any number of
// heads and groups, with or without a window, for prompts and for single tokens:
// one warp per (token, q-head), all arithmetic in 32-bit.
//
// A query at position p of sequence s sees keys j with max(0, p - window + 1) <= j <= p
// (window <= 0: all j <= p), the slot-causal rule of src/detllm/model.py:259-266.
// Keys are walked in blocks of 32 aligned to absolute positions; inside a block lane i
// scores key j0 + i; masked lanes contribute exactly 0 and are left out of the maximum
// (the float analogue of the reference's integer sentinel, src/detllm/ops/di_softmax.py:45-58);
// the running (max, sum, context) is rescaled block by block.  The order of every sum
// depends on the query's position only, never on the step's batch or on how the
// sequence was cut into steps.
//
// Keys of the current step may come from packed buffers k_new/v_new instead of the
// cache (windowed layers, whose ring cannot hold a whole prompt).
#include "common.cuh"

struct AttnArgs {
    const T* q; T* out;
    KVAddr cache;
    const T* k_new; const T* v_new;
    const int* token_seq; const int* positions; const int* slots; const int* q_start; const int* cu_q;
    int n_tokens, n_q, n_kv, hd;
    float scale; int window;
};

#define AG_WARPS 4

__global__ void __launch_bounds__(AG_WARPS * 32) attention_generic_kernel(AttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float smem[];
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * AG_WARPS + wib;
    if (w >= (long long)a.n_tokens * a.n_q) return;            // whole warps leave; no block barrier below
    const int t = (int)(w / a.n_q), head = (int)(w % a.n_q);
    const int g = head / (a.n_q / a.n_kv);
    float* qs = smem + wib * a.hd;
    const T* qrow = a.q + ((size_t)t * a.n_q + head) * a.hd;
    for (int d = lane; d < a.hd; d += 32) qs[d] = to_f32(qrow[d]);
    __syncwarp();
    const int pos = a.positions[t], s = a.token_seq[t], slot = a.slots[s];
    const int first_new = a.k_new ? a.q_start[s] : 0x7fffffff, tok0 = a.cu_q[s];
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    float m = -INFINITY, l = 0.f;
    float acc[IDM_MAX_HEAD_DIM / 32];
#pragma unroll
    for (int i = 0; i < IDM_MAX_HEAD_DIM / 32; ++i) acc[i] = 0.f;
    for (int j0 = (lo / 32) * 32; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j >= lo && j <= pos;
        float sc = -INFINITY;
        const T* vrow = nullptr;
        if (valid) {
            const T* krow;
            if (j >= first_new) {
                const size_t off = ((size_t)(tok0 + j - first_new) * a.n_kv + g) * a.hd;
                krow = a.k_new + off; vrow = a.v_new + off;
            } else {
                const size_t off = kv_offset(a.cache, slot, j, g);
                krow = a.cache.k + off; vrow = a.cache.v + off;
            }
            float dot = 0.f;
            for (int d = 0; d < a.hd; d += Vec16<T>::N) {
                Vec16<T> kv; kv.load(krow + d);
#pragma unroll
                for (int e = 0; e < Vec16<T>::N; ++e) dot = fmaf(qs[d + e], kv.get(e), dot);
            }
            sc = dot * a.scale;
        }
        const float m_new = fmaxf(m, warp_max(sc));
        const float alpha = expf(m - m_new);
        const float p = valid ? expf(sc - m_new) : 0.f;
        l = l * alpha + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < IDM_MAX_HEAD_DIM / 32; ++i) acc[i] *= alpha;
        const unsigned live = __ballot_sync(0xffffffffu, valid);
        for (int jj = 0; jj < 32; ++jj) {
            if (!((live >> jj) & 1u)) continue;
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const T* vr = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)vrow, jj);
#pragma unroll
            for (int i = 0; i < IDM_MAX_HEAD_DIM / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < a.hd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
    }
    T* orow = a.out + ((size_t)t * a.n_q + head) * a.hd;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < IDM_MAX_HEAD_DIM / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < a.hd) from_f32(orow[d], acc[i] * inv);
    }
}

extern "C" int idm_attention_generic(const void* q, void* out, void* k_pool, void* v_pool, const int* table,
                                     int table_stride, int ring, const void* k_new, const void* v_new,
                                     const int* token_seq, const int* positions, const int* slots,
                                     const int* q_start, const int* cu_q, int n_tokens, int n_q, int n_kv,
                                     int hd, float scale, int window, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(hd > 0 && hd % Vec16<T>::N == 0 && hd <= IDM_MAX_HEAD_DIM,
                "attention: head_dim=%d must be a multiple of %d and at most %d", hd, Vec16<T>::N,
                IDM_MAX_HEAD_DIM);
    IDM_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "attention: %d q-heads are no multiple of %d kv-heads", n_q, n_kv);
    IDM_REQUIRE((k_new == nullptr) == (v_new == nullptr), "attention: k_new and v_new come together");
    AttnArgs a;
    a.q = (const T*)q; a.out = (T*)out;
    a.cache = KVAddr{(T*)k_pool, (T*)v_pool, table, table_stride, ring, n_kv, hd};
    a.k_new = (const T*)k_new; a.v_new = (const T*)v_new;
    a.token_seq = token_seq; a.positions = positions; a.slots = slots; a.q_start = q_start; a.cu_q = cu_q;
    a.n_tokens = n_tokens; a.n_q = n_q; a.n_kv = n_kv; a.hd = hd; a.scale = scale; a.window = window;
    const long long warps = (long long)n_tokens * n_q;
    idm_launch(attention_generic_kernel, dim3((unsigned)((warps + AG_WARPS - 1) / AG_WARPS)), dim3(AG_WARPS * 32), AG_WARPS * hd * sizeof(float), stream, a);
    IDM_LAUNCH_CHECK("attention_generic");
    return 0;
}
