// Embedding, residual-add + RMS norm, rotary table, q/k norm + rotation + cache
// write, ring write, SwiGLU.  Memory-bound kernels; everything that follows a
// matrix product reads its 32-bit partial sums and adds them in ascending order.
#include "common.cuh"
#include "qkv_finish.cuh"

// ------------------------------------------------------------------ embedding
// h[t, :] = table[tokens[t], :]  (a pure lookup, no scaling: src/detllm/model.py:246-249)
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                             float* __restrict__ h, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = table + (size_t)tokens[t] * hidden;
    float* out = h + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_f32(row[i]);
}

extern "C" int idm_embed(const int* tokens, const void* table, float* h, int n_tokens, int hidden,
                         cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(n_tokens > 0 && hidden > 0, "embed: bad sizes n_tokens=%d hidden=%d", n_tokens, hidden);
    idm_launch(embed_kernel, dim3(n_tokens), dim3(256), 0, stream, tokens, (const T*)table, h, hidden);
    IDM_LAUNCH_CHECK("embed");
    return 0;
}

// ------------------------------------------------------- residual add + RMSNorm
// rows == nullptr: for every token row r: h[r] += sum_p delta[p][r] (stored), x[r] = norm(h[r]).
// rows != nullptr: for i < n_rows: v = h[rows[i]] + sum_p delta[p][rows[i]] (not stored), x[i] = norm(v).
// norm(v) = v / sqrt(mean(v^2) + eps) * gamma, in 32-bit.  One block per row; the block
// size is fixed, so the reduction order depends on `hidden` only.
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta, int n_partials,
                                   size_t partial_stride, const float* __restrict__ gamma, float eps,
                                   T* __restrict__ x, const int* __restrict__ rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    extern __shared__ float vals[];            // the row, kept between the two passes
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* hr = h + (size_t)r * hidden;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = add_partials(hr[c], delta, n_partials, partial_stride, (size_t)r * hidden + c);
        if (!rows && n_partials) hr[c] = v;
        vals[c] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    T* xr = x + (size_t)i * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) from_f32(xr[c], vals[c] * inv * gamma[c]);
}

// The same for rows of at most 4 * 256 elements with hidden % 4 == 0: a thread owns four consecutive
// elements, and all of its loads (the stream and up to 16 partials) are in flight at once.
__global__ void __launch_bounds__(256) add_rmsnorm_vec4_kernel(float* __restrict__ h, const float* __restrict__ delta,
                                                               int n_partials, size_t partial_stride,
                                                               const float* __restrict__ gamma, float eps,
                                                               T* __restrict__ x, const int* __restrict__ rows,
                                                               int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    const int c = threadIdx.x * 4;
    const bool live = c < hidden;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
        const size_t idx = (size_t)r * hidden + c;
        v = *reinterpret_cast<const float4*>(h + idx);
        if (n_partials > 0) {
            float4 part[16];
#pragma unroll
            for (int p = 0; p < 16; ++p)
                if (p < n_partials) part[p] = *reinterpret_cast<const float4*>(delta + p * partial_stride + idx);
#pragma unroll
            for (int p = 0; p < 16; ++p)
                if (p < n_partials) { v.x += part[p].x; v.y += part[p].y; v.z += part[p].z; v.w += part[p].w; }
        }
        if (!rows && n_partials) *reinterpret_cast<float4*>(h + idx) = v;
    }
    const float total = block_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w, scratch);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    if (live) {
        const float4 gm = *reinterpret_cast<const float4*>(gamma + c);
        T* xr = x + (size_t)i * hidden + c;
        store4(xr, v.x * inv * gm.x, v.y * inv * gm.y, v.z * inv * gm.z, v.w * inv * gm.w);
    }
}

// Many rows with nothing to add (the residual was added by the product before): one warp per row, no
// block-wide barrier.  Lane l stands for the threads l, l + 32, ... of the kernel above (its warps
// 0 .. 7), sums each of those warps by the same butterfly and adds the eight totals in the same order:
// the same bits, whichever of the two kernels runs.
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ h, const float* __restrict__ gamma,
                                                           float eps, T* __restrict__ x, const int* __restrict__ rows,
                                                           int n_rows, int hidden) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= n_rows) return;
    const int r = rows ? rows[i] : i;
    const float* hr = h + (size_t)r * hidden;
    float4 v[8];
    float s[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const int c = (32 * w + lane) * 4;
        v[w] = c < hidden ? *reinterpret_cast<const float4*>(hr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        s[w] = v[w].x * v[w].x + v[w].y * v[w].y + v[w].z * v[w].z + v[w].w * v[w].w;
    }
#pragma unroll
    for (int w = 0; w < 8; ++w) s[w] = warp_sum(s[w]);
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += s[w];
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    T* xr = x + (size_t)i * hidden;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const int c = (32 * w + lane) * 4;
        if (c < hidden) {
            const float4 gm = *reinterpret_cast<const float4*>(gamma + c);
            store4(xr + c, v[w].x * inv * gm.x, v[w].y * inv * gm.y, v[w].z * inv * gm.z, v[w].w * inv * gm.w);
        }
    }
}

extern "C" int idm_add_rmsnorm(float* h, const float* delta, int n_partials, long long partial_stride,
                               const float* gamma, float eps, void* x, const int* rows, int n_rows,
                               int hidden, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    IDM_REQUIRE(hidden > 0 && n_rows > 0, "add_rmsnorm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    IDM_REQUIRE((size_t)hidden * 4 <= 160 * 1024, "add_rmsnorm: hidden=%d does not fit shared memory", hidden);
    if (hidden % 4 == 0 && hidden <= 1024 && (delta == nullptr || n_partials == 0) && n_rows >= 64) {
        idm_launch(rmsnorm_rows_kernel, dim3((n_rows + 7) / 8), dim3(256), 0, stream, (const float*)h, gamma, eps, (T*)x, rows,
                   n_rows, hidden);
        IDM_LAUNCH_CHECK("add_rmsnorm");
        return 0;
    }
    if (hidden % 4 == 0 && hidden <= 1024 && n_partials <= 16 && (partial_stride % 4) == 0) {
        // NOTE: the sum of squares is taken over the same values in a different thread layout than
        // the general kernel; which kernel runs depends on `hidden` and the number of partials only
        idm_launch(add_rmsnorm_vec4_kernel, dim3(n_rows), dim3(256), 0, stream, h, delta, delta ? n_partials : 0, (size_t)partial_stride,
                                                            gamma, eps, (T*)x, rows, hidden);
        IDM_LAUNCH_CHECK("add_rmsnorm");
        return 0;
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(add_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    idm_launch(add_rmsnorm_kernel, dim3(n_rows), dim3(256), smem, stream, h, delta, delta ? n_partials : 0,
                                                      (size_t)partial_stride, gamma, eps, (T*)x, rows, hidden);
    IDM_LAUNCH_CHECK("add_rmsnorm");
    return 0;
}

// ---------------------------------------------------------------- rotary table
// cs[t, j] = (cos, sin)(positions[t] * inv_freq[j]), angle and functions in 64-bit,
// rounded to 32-bit (src/detllm/ops/rope.py:25-35 builds its table the same way).
// cs_by_dim, if given, gets the same values as [half, n_tokens]: there the tokens of one dim lie side
// by side, which is how a kernel with one thread per token wants to read them.
__global__ void rope_table_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                  float2* __restrict__ cs, float2* __restrict__ cs_by_dim, int n_tokens, int half) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens * half) return;
    const int t = i / half, j = i % half;
    double s, c;
    sincos((double)positions[t] * inv_freq[j], &s, &c);
    cs[i] = make_float2((float)c, (float)s);
    if (cs_by_dim != nullptr) cs_by_dim[(size_t)j * n_tokens + t] = make_float2((float)c, (float)s);
}

extern "C" int idm_rope_table(const int* positions, const double* inv_freq, float* cs, float* cs_by_dim,
                              int n_tokens, int half, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(half > 0, "rope_table: bad half=%d", half);
    const int n = n_tokens * half;
    idm_launch(rope_table_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, positions, inv_freq, (float2*)cs,
               (float2*)cs_by_dim, n_tokens, half);
    IDM_LAUNCH_CHECK("rope_table");
    return 0;
}

// ------------------------------------------- q/k norm + rotation + cache write
// One warp per (token, head) over the n_q + 2 n_kv heads of the fused projection.
// q and k heads: RMS norm over head_dim with a weight of shape [head_dim] shared by
// all heads (src/detllm/model.py:208-215), then rotation of pairs (d, d + hd/2)
// by the token's position (src/detllm/ops/rope.py:47-55); v heads are copied.
// q goes to q_out [N, n_q, hd]; k and v go to the cache at the token's position
// and/or to packed buffers k_new, v_new [N, n_kv, hd].
__global__ void __launch_bounds__(128) qkv_finish_kernel(QkvArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    // one block per token: the token's place in the cache is looked up once, the warps share the heads
    __shared__ int place[2];
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = a.n_q + 2 * a.n_kv;
    if (threadIdx.x == 0 && a.write_cache) {
        const int pos = a.positions[t];
        const int r = a.cache.ring ? pos % a.cache.ring : pos;
        place[0] = a.cache.table[(size_t)a.slots[a.token_seq[t]] * a.cache.table_stride + r / IDM_PAGE];
        place[1] = r % IDM_PAGE;
    }
    __syncthreads();
    const int page = place[0], prow = place[1];
    if (a.tiles4) {
        // whole heads inside tiles of 128 features, four features per lane (qkv_finish_tile4)
        const int width = heads * a.hd;
        for (int f0 = warp * 128; f0 < width; f0 += 4 * 128) {
            const int f = f0 + lane * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (f < width) {
                const float* p = a.qkv + (size_t)t * width + f;
                for (int z = 0; z < a.n_partials; ++z) {
                    const float4 q4 = *reinterpret_cast<const float4*>(p + (size_t)z * a.partial_stride);
                    v.x += q4.x; v.y += q4.y; v.z += q4.z; v.w += q4.w;
                }
            }
            qkv_finish_tile4(a, v, t, f0, lane, page, prow);
        }
        return;
    }
    for (int head = warp; head < heads; head += 4) {
        const size_t row = (size_t)t * heads * a.hd + (size_t)head * a.hd;
        qkv_finish_row(a, t, head, lane,
                       [&](int j) { return add_partials(0.f, a.qkv, a.n_partials, a.partial_stride, row + j); },
                       [&](int g) { return (((size_t)page * a.n_kv + g) * IDM_PAGE + prow) * (size_t)a.hd; });
    }
}

extern "C" int idm_qkv_finish(const float* qkv, int n_partials, long long partial_stride, int n_tokens,
                              int n_q, int n_kv, int hd, const float* gq, const float* gk, float eps,
                              const float* cs, void* q_out, void* k_new, void* v_new,
                              void* k_pool, void* v_pool, const int* table, int table_stride, int ring,
                              const int* token_seq, const int* positions, const int* slots,
                              cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(hd > 0 && hd % 2 == 0 && hd <= IDM_MAX_HEAD_DIM,
                "qkv_finish: head_dim=%d must be even and at most %d", hd, IDM_MAX_HEAD_DIM);
    IDM_REQUIRE(n_q > 0 && n_kv >= 0 && n_partials >= 1, "qkv_finish: bad head counts %d/%d", n_q, n_kv);
    QkvArgs a;
    a.qkv = qkv; a.n_partials = n_partials; a.partial_stride = (size_t)partial_stride;
    a.n_tokens = n_tokens; a.n_q = n_q; a.n_kv = n_kv; a.hd = hd;
    a.gq = gq; a.gk = gk; a.eps = eps; a.inv_hd = 1.0f / (float)hd; a.cs = (const float2*)cs; a.cs_by_dim = nullptr;
    a.q_out = (T*)q_out; a.k_new = (T*)k_new; a.v_new = (T*)v_new;
    a.cache = KVAddr{(T*)k_pool, (T*)v_pool, table, table_stride, ring, n_kv, hd};
    a.write_cache = k_pool != nullptr;
    a.token_seq = token_seq; a.positions = positions; a.slots = slots;
    a.tiles4 = (128 % hd == 0 && hd >= 8 && (partial_stride % 4) == 0) ? 1 : 0;
    idm_launch(qkv_finish_kernel, dim3(n_tokens), dim3(128), 0, stream, a);
    IDM_LAUNCH_CHECK("qkv_finish");
    return 0;
}

// ------------------------------------------------------------------ ring write
// After a windowed layer's attention: the step's keys and values go into the ring.
// Only a sequence's last `ring` tokens are written (earlier ones would be overwritten
// by later ones of the same step; each ring position gets exactly one writer).
__global__ void kv_write_ring_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new, KVAddr c,
                                     const int* __restrict__ token_seq, const int* __restrict__ positions,
                                     const int* __restrict__ slots, const int* __restrict__ kv_len,
                                     int n_tokens) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n_tokens * c.n_kv) return;
    const int t = warp / c.n_kv, g = warp % c.n_kv;
    const int s = token_seq[t], pos = positions[t];
    if (c.ring && pos < kv_len[s] - c.ring) return;
    const size_t off = kv_offset(c, slots[s], pos, g);
    const size_t src = ((size_t)t * c.n_kv + g) * c.hd;
    for (int d = lane; d < c.hd; d += 32) { c.k[off + d] = k_new[src + d]; c.v[off + d] = v_new[src + d]; }
}

extern "C" int idm_kv_write_ring(const void* k_new, const void* v_new, void* k_pool, void* v_pool,
                                 const int* table, int table_stride, int ring, const int* token_seq,
                                 const int* positions, const int* slots, const int* kv_len, int n_tokens,
                                 int n_kv, int hd, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    KVAddr c{(T*)k_pool, (T*)v_pool, table, table_stride, ring, n_kv, hd};
    const long long warps = (long long)n_tokens * n_kv;
    idm_launch(kv_write_ring_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, stream, 
        (const T*)k_new, (const T*)v_new, c, token_seq, positions, slots, kv_len, n_tokens);
    IDM_LAUNCH_CHECK("kv_write_ring");
    return 0;
}

// ---------------------------------------------------------------------- SwiGLU
// y[t, i] = g * sigmoid(g) * u  (src/detllm/ops/di_swiglu.py:43-45; float form tests/test_ops.py:240-242).
// Plain layout: g = gu[t, i], u = gu[t, inter + i].  Tiled layout (the gate/up weight's rows in tiles
// alternating: gate row of a feature, then its up row; 64 features per 128-row tile, zero rows past
// the end): g = gu[t, 128 (i / 64) + 2 (i % 64)], u = the next column.
// grid (column blocks, tokens): no division by a runtime size per element.
__global__ void __launch_bounds__(256) swiglu_kernel(const float* __restrict__ gu, int n_partials, size_t partial_stride,
                                                     T* __restrict__ y, int inter, int width, int tiled) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= inter) return;
    const size_t t = blockIdx.y;
    const int gi = tiled ? ((c >> 6) << 7) + 2 * (c & 63) : c;
    const int ui = tiled ? gi + 1 : c + inter;
    const size_t base = t * (size_t)width;
    const float g = add_partials(0.f, gu, n_partials, partial_stride, base + gi);
    const float u = add_partials(0.f, gu, n_partials, partial_stride, base + ui);
    from_f32(y[t * (size_t)inter + c], silu_mul(g, u));
}

extern "C" int idm_swiglu(const float* gu, int n_partials, long long partial_stride, void* y, int n_tokens,
                          int inter, int tiled, cudaStream_t stream) {
    if (n_tokens == 0) return 0;
    IDM_REQUIRE(inter > 0 && n_partials >= 1, "swiglu: bad sizes");
    IDM_REQUIRE(n_tokens <= 65535 * 64, "swiglu: %d tokens in one launch", n_tokens);
    const int width = tiled ? ((inter + 63) / 64) * 128 : 2 * inter;
    for (int t0 = 0; t0 < n_tokens; t0 += 65535) {
        const int nt = n_tokens - t0 < 65535 ? n_tokens - t0 : 65535;
        idm_launch(swiglu_kernel, dim3((inter + 255) / 256, nt), dim3(256), 0, stream,
                   gu + (size_t)t0 * width, n_partials, (size_t)partial_stride, (T*)y + (size_t)t0 * inter, inter, width,
                   tiled);
        IDM_LAUNCH_CHECK("swiglu");
    }
    return 0;
}
