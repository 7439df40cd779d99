// Causal attention for steps that bring many tokens per sequence (prompts), on the tensor cores.
//
// One block per (tile of 128 consecutive query tokens of one sequence, q-head).  Keys and values
// come from the paged cache (the step's own keys were written before), one page of 64 keys per
// iteration, fetched by TMA two pages ahead (with one buffer for the keys each Q . K^T waited a whole
// trip to L2 for its operand).  Per iteration:
//   S = Q . K^T        tcgen05.mma, both operands in shared memory, S [128 x 64] in tensor memory
//   softmax            one thread per query row reads its row of S (tcgen05.ld): scale, causal
//                      mask, running maximum, p = 2^(s - m), running sum -- all 32-bit, no shuffles
//   O += P . V         P written to shared memory as bfloat16 in the MMA's swizzled layout,
//                      V read in place ([keys, head_dim] = MN-major operand); O stays in tensor
//                      memory for the whole tile
// The running maximum is only moved when the block's maximum exceeds it by more than 2^8 (then O
// and the sum are rescaled); p and the sum always use the same reference, so the result is exact
// up to rounding.  The next iteration's Q . K^T is issued before this iteration's P . V, so the
// tensor core works while the softmax threads do.  Blocks are aligned to absolute key positions:
// a token's result does not depend on the batch or on where its tile starts.
//
// Masked keys give p = 0 exactly (select, not arithmetic); rows of V past the sequence's length
// are zeroed in shared memory before they meet the MMA, so stale page contents cannot leak.
// The reference's prefill path is src/detllm/model.py:382-402 (query-chunked integer GEMMs).
//
// Roles: warps 0-3 softmax + epilogue (thread = query row = tensor-memory lane), warp 4 TMA, warp 5 MMA.
// All mbarrier waits are bounded; a wait that runs out sets the error word (idm_attention_prefill_status).
#include "common.cuh"

#if defined(IDM_BF16)

#include "tcgen05.cuh"

#define AP_BM 128
#define AP_BN 64
#define AP_THREADS 192
#define AP_TMEM_COLS 256
#define AP_RESCALE_STEP 8.0f
// A tile's key blocks may be cut into up to AP_MAX_SPLIT runs, each worked by a block of its own; a run
// has at least AP_MIN_RUN key blocks.  (At most three blocks at a tile's end hold masked keys, so with
// four every row sees the whole first block of every run: no run leaves a row without a key.)
#define AP_MAX_SPLIT 4
#define AP_MIN_RUN 4
#define AP_COUNTERS 2048

__device__ int g_attn_prefill_error = 0;

struct PrefillArgs {
    T* out;
    const int* tile_seq; const int* tile_start;
    const int* cu_q; const int* q_start; const int* kv_len; const int* slots;
    const int* table; int table_stride;
    int n_q, n_kv;
    float scale_log2;
    int max_split;                                     // runs a tile's key blocks may be cut into (1: never cut)
    int max_run;                                       // key blocks a run should not exceed
    int* counters;                                     // [n_tiles * n_q] arrivals, zero between launches
    float* parts;                                      // [n_tiles * n_q, max_split] partial results, PART floats each
};

template <int HD>
struct PrefillSmem {
    static constexpr int HT = HD / 64;                 // 64-wide tiles along head_dim
    static constexpr int Q_BYTES = HT * AP_BM * 128;
    static constexpr int K_BYTES = HT * AP_BN * 128;   // per stage, two stages
    static constexpr int V_BYTES = HT * AP_BN * 128;   // per stage, two stages
    static constexpr int P_BYTES = AP_BM * 128;
    static constexpr int Q_OFF = 0, K_OFF = Q_BYTES, V_OFF = K_OFF + 2 * K_BYTES, P_OFF = V_OFF + 2 * V_BYTES;
    static constexpr int BAR_OFF = P_OFF + P_BYTES;
    static constexpr int NEED = BAR_OFF + 256;         // from the first 1024-byte border on
    // two blocks per SM: 2 x (TOTAL + 1 KB the system keeps per block) must stay within 228 KB, which
    // leaves 512 bytes to reach the border (the array is declared with that alignment; the kernel checks)
    static constexpr int TOTAL = NEED + (HD == 128 ? 512 : 1024);
    // a run's partial result: the unnormalised output as [HD / 4][128 rows] float4, then (max, sum) per row
    static constexpr int PART = AP_BM * HD + 2 * AP_BM;
};

template <int HD>
__global__ void __launch_bounds__(AP_THREADS, 2)
attention_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, PrefillArgs a) {
    using S = PrefillSmem<HD>;
    constexpr int HT = S::HT;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    if (base - smem_u32(smem_raw) + S::NEED > S::TOTAL) {        // (never seen: the array starts on a 1024-byte border)
        if (threadIdx.x == 0) atomicExch(&g_attn_prefill_error, 2);
        return;
    }
    uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + S::BAR_OFF;
    // barriers (8 bytes each)
    const uint32_t q_full = bars, p_full = bars + 40, o_done = bars + 48;
    auto k_full = [&](int i) { return bars + 8 + 8u * i; };
    auto k_empty = [&](int i) { return bars + 24 + 8u * i; };
    auto v_full = [&](int i) { return bars + 56 + 8u * i; };
    auto v_empty = [&](int i) { return bars + 72 + 8u * i; };
    auto s_full = [&](int i) { return bars + 88 + 8u * i; };
    auto s_empty = [&](int i) { return bars + 104 + 8u * i; };
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(gbase + S::BAR_OFF + 120);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();

    // blocks start in this order: all heads (and runs) of the longest tile first.  What is read here was
    // written before the step began, not by the kernel before this one.
    const int tile = blockIdx.y, head = blockIdx.x / a.max_split, run = blockIdx.x % a.max_split;
    const int seq = a.tile_seq[tile], tstart = a.tile_start[tile];
    const int g = head / (a.n_q / a.n_kv);
    const int tok0 = a.cu_q[seq] + tstart;                       // first token (packed row) of the tile
    const int q_len = a.cu_q[seq + 1] - a.cu_q[seq];
    const int rows_valid = min(AP_BM, q_len - tstart);
    const int p_first = a.q_start[seq] + tstart;                 // position of row 0
    const int p_last = p_first + rows_valid - 1;
    const int kv_len = a.kv_len[seq];
    const int nb_tile = p_last / AP_BN + 1;                      // the tile's key blocks 0 .. nb_tile-1
    const int n_runs = min(a.max_split, max(1, min((nb_tile + a.max_run - 1) / a.max_run, nb_tile / AP_MIN_RUN)));
    if (run >= n_runs) return;                                   // (the whole block, before anything is set up)
    const int b_first = run * nb_tile / n_runs;                  // this block's run of key blocks
    const int nb = (run + 1) * nb_tile / n_runs - b_first;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1); mbar_init(p_full, 4); mbar_init(o_done, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full(i), 1); mbar_init(k_empty(i), 1);
            mbar_init(v_full(i), 1); mbar_init(v_empty(i), 1); mbar_init(s_full(i), 1); mbar_init(s_empty(i), 4);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 5) tmem_alloc(smem_u32((const void*)tmem_slot), AP_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_o = tmem + 128;                          // S buffers at columns 0 and 64, O from 128
    pdl_wait();                                                  // set-up done; now the previous kernel's results

    // from here on b counts the run's own key blocks (buffers and barrier phases go by it); the block's
    // place among the sequence's keys is b_first + b
    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_expect_tx(q_full, S::Q_BYTES);
            for (int h = 0; h < HT; ++h)
                tma_load_3d(base + S::Q_OFF + h * AP_BM * 128, &map_q, h * 64, head, tok0, q_full);
            const int slot = a.slots[seq];
            for (int b = 0; b < nb; ++b) {
                const int page = a.table[(size_t)slot * a.table_stride + b_first + b];
                const int row = (page * a.n_kv + g) * IDM_PAGE;
                const int vb = b & 1;                            // this block's key and value buffers
                if (b >= 2 && !mbar_wait(k_empty(vb), ((b >> 1) - 1) & 1, abort_flag, &g_attn_prefill_error)) break;
                mbar_expect_tx(k_full(vb), S::K_BYTES);
                for (int h = 0; h < HT; ++h)
                    tma_load_2d(base + S::K_OFF + vb * S::K_BYTES + h * AP_BN * 128, &map_k, h * 64, row, k_full(vb));
                if (b >= 2 && !mbar_wait(v_empty(vb), ((b >> 1) - 1) & 1, abort_flag, &g_attn_prefill_error)) break;
                mbar_expect_tx(v_full(vb), S::V_BYTES);
                for (int h = 0; h < HT; ++h)
                    tma_load_2d(base + S::V_OFF + vb * S::V_BYTES + h * AP_BN * 128, &map_v, h * 64, row, v_full(vb));
            }
        }
    } else if (warp == 5) {
        // -------------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc(AP_BM, AP_BN);
            constexpr uint32_t idesc_o = umma_idesc(AP_BM, HD, true);
            auto mma_s = [&](int b) {                            // S[b % 2] = Q . K_b^T
                const uint32_t d = tmem + (uint32_t)(b & 1) * AP_BN;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint64_t ad = umma_desc_kmajor(base + S::Q_OFF + (kk / 4) * AP_BM * 128) + 2 * (kk % 4);
                    const uint64_t bd = umma_desc_kmajor(base + S::K_OFF + (b & 1) * S::K_BYTES + (kk / 4) * AP_BN * 128) + 2 * (kk % 4);
                    tc_mma_bf16(d, ad, bd, idesc_s, kk > 0 ? 1u : 0u);
                }
                tc_commit(s_full(b & 1));
                tc_commit(k_empty(b & 1));
            };
            bool ok = mbar_wait(q_full, 0, abort_flag, &g_attn_prefill_error) &&
                      mbar_wait(k_full(0), 0, abort_flag, &g_attn_prefill_error);
            if (ok) { tc_fence_after(); mma_s(0); }
            for (int b = 0; b < nb && ok; ++b) {
                if (b + 1 < nb) {
                    ok = mbar_wait(k_full((b + 1) & 1), ((b + 1) >> 1) & 1, abort_flag, &g_attn_prefill_error);
                    if (ok && b + 1 >= 2)
                        ok = mbar_wait(s_empty((b + 1) & 1), (((b + 1) >> 1) - 1) & 1, abort_flag, &g_attn_prefill_error);
                    if (!ok) break;
                    tc_fence_after();
                    mma_s(b + 1);
                }
                ok = mbar_wait(p_full, b & 1, abort_flag, &g_attn_prefill_error) &&
                     mbar_wait(v_full(b & 1), (b >> 1) & 1, abort_flag, &g_attn_prefill_error);
                if (!ok) break;
                tc_fence_after();
                const uint32_t vbase = base + S::V_OFF + (b & 1) * S::V_BYTES;
#pragma unroll
                for (int kk = 0; kk < AP_BN / 16; ++kk) {        // O += P . V_b
                    const uint64_t ad = umma_desc_kmajor(base + S::P_OFF) + 2 * kk;
                    const uint64_t bd = umma_desc_mnmajor(vbase + kk * 16 * 128, AP_BN * 128);
                    tc_mma_bf16(tmem_o, ad, bd, idesc_o, (b > 0 || kk > 0) ? 1u : 0u);
                }
                tc_commit(o_done);
                tc_commit(v_empty(b & 1));
            }
        }
    } else {
        // ------------------------------------------------- softmax and epilogue (warps 0-3)
        const int r = warp * 32 + lane;                          // query row = tensor-memory lane
        const int p_r = p_first + r;
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int b = 0; b < nb && ok; ++b) {
            ok = mbar_wait(s_full(b & 1), (b >> 1) & 1, abort_flag, &g_attn_prefill_error);
            if (!ok) break;
            tc_fence_after();
            uint32_t sr[AP_BN];
            tc_ld32_issue(tmem + lane_base + (uint32_t)(b & 1) * AP_BN, sr);
            tc_ld32_issue(tmem + lane_base + (uint32_t)(b & 1) * AP_BN + 32, sr + 32);
            tc_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty(b & 1));
            const int key0 = (b_first + b) * AP_BN;               // position of the block's first key
            const bool diagonal = key0 + AP_BN - 1 > p_first;     // some key of the block lies past row 0's position
            if (diagonal) {
#pragma unroll
                for (int j = 0; j < AP_BN; ++j)
                    if (key0 + j > p_r) sr[j] = 0xff800000u;      // -inf: p becomes 0 exactly
            }
            // the maximum of the raw scores (the scale is positive), four chains side by side
            // (the three-input maximum of sm_100: two scores per instruction)
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < AP_BN; j += 8) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    mx[u] = max3(mx[u], __uint_as_float(sr[j + 2 * u]), __uint_as_float(sr[j + 2 * u + 1]));
            }
            const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * a.scale_log2;
            float alpha = 1.f;
            if (m_blk > m_ref + AP_RESCALE_STEP || m_ref == -INFINITY) {
                // (m_ref is -inf only before the run's first block, all of whose keys every row may see)
                alpha = exp2f(m_ref - m_blk);                      // 0 the first time
                m_ref = m_blk;
            }
            // p = 2^(s * scale - m_ref): one fused multiply-add and one exponential per score
            const float neg_m = -m_ref;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t packed[AP_BN / 2];
#pragma unroll
            for (int j = 0; j < AP_BN; j += 4) {
                const float p0 = ex2_hw(fmaf(__uint_as_float(sr[j]), a.scale_log2, neg_m));
                const float p1 = ex2_hw(fmaf(__uint_as_float(sr[j + 1]), a.scale_log2, neg_m));
                const float p2 = ex2_hw(fmaf(__uint_as_float(sr[j + 2]), a.scale_log2, neg_m));
                const float p3 = ex2_hw(fmaf(__uint_as_float(sr[j + 3]), a.scale_log2, neg_m));
                sum4[0] += p0; sum4[1] += p1; sum4[2] += p2; sum4[3] += p3;
                const __nv_bfloat162 pa = __floats2bfloat162_rn(p0, p1), pb = __floats2bfloat162_rn(p2, p3);
                packed[j / 2] = *reinterpret_cast<const uint32_t*>(&pa);
                packed[j / 2 + 1] = *reinterpret_cast<const uint32_t*>(&pb);
            }
            const float row_sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            if (b >= 1) {
                ok = mbar_wait(o_done, (b - 1) & 1, abort_flag, &g_attn_prefill_error);   // P is free, O is settled
                if (!ok) break;
                tc_fence_after();
                if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
                    for (int c = 0; c < HD; c += 16) {
                        uint32_t o[16];
                        tc_ld16_issue(tmem_o + lane_base + c, o);
                        tc_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tc_st16(tmem_o + lane_base + c, o);
                    }
                    tc_st_wait();
                }
            }
            l = l * alpha + row_sum;
            // P row: 8 chunks of 16 bytes, chunk c stored at (c ^ (row & 7)) -- the 128-byte swizzle
            uint8_t* prow = gbase + S::P_OFF + r * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) =
                    make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            }
            // rows of V past the sequence's end hold whatever the page held before: zero them
            if (key0 + AP_BN > kv_len) {
                ok = mbar_wait(v_full(b & 1), (b >> 1) & 1, abort_flag, &g_attn_prefill_error);
                if (!ok) break;
                const int first_bad = kv_len - key0;               // >= 1
                uint8_t* vb = gbase + S::V_OFF + (b & 1) * S::V_BYTES;
                for (int idx = r; idx < (AP_BN - first_bad) * HT * 8; idx += AP_BM) {
                    const int chunk = idx % 8, rest = idx / 8;
                    const int row = first_bad + rest % (AP_BN - first_bad), h = rest / (AP_BN - first_bad);
                    *reinterpret_cast<uint4*>(vb + h * AP_BN * 128 + row * 128 + chunk * 16) = make_uint4(0, 0, 0, 0);
                }
            }
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        if (ok) ok = mbar_wait(o_done, (nb - 1) & 1, abort_flag, &g_attn_prefill_error);
        T* orow = a.out + ((size_t)(tok0 + r) * a.n_q + head) * HD;
        ok = __all_sync(0xffffffffu, ok);                          // (one answer per warp for what follows)
        if (n_runs > 1) {
            // This run's result goes to its place among the tile's; the block that comes last adds them
            // all, in the order of the runs whoever it is, so the sum does not depend on who came last.
            // (A warp whose wait ran out skips the work but not the two barriers and the count: the
            // error is reported, the result is wrong, and nobody waits for anybody for ever.)
            float* part0 = a.parts + (size_t)(tile * a.n_q + head) * a.max_split * S::PART;
            float4* mine = reinterpret_cast<float4*>(part0 + (size_t)run * S::PART);
            if (ok) {
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD; c += 16) {
                    float o[16];
                    tc_ld16(tmem_o + lane_base + c, o);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        mine[(c / 4 + k) * AP_BM + r] = make_float4(o[4 * k], o[4 * k + 1], o[4 * k + 2], o[4 * k + 3]);
                }
                reinterpret_cast<float2*>(mine + (HD / 4) * AP_BM)[r] = make_float2(m_ref, l);
                __threadfence();
            }
            volatile int* last_flag = (volatile int*)(gbase + S::BAR_OFF + 128);
            asm volatile("bar.sync 1, 128;" ::: "memory");         // the four softmax warps
            if (r == 0) {
                int* counter = a.counters + tile * a.n_q + head;
                const int is_last = atomicAdd(counter, 1) == n_runs - 1;
                if (is_last) *counter = 0;                         // ready for the next launch
                *last_flag = is_last;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*last_flag && ok) {
                __threadfence();
                float f[AP_MAX_SPLIT], m_all = -INFINITY, l_all = 0.f;
#pragma unroll
                for (int i = 0; i < AP_MAX_SPLIT; ++i) {
                    f[i] = -INFINITY;
                    if (i < n_runs) {
                        f[i] = __ldcg(reinterpret_cast<const float2*>(part0 + (size_t)i * S::PART + AP_BM * HD) + r).x;
                        m_all = fmaxf(m_all, f[i]);
                    }
                }
#pragma unroll
                for (int i = 0; i < AP_MAX_SPLIT; ++i) {
                    if (i < n_runs) {
                        const float l_i = __ldcg(reinterpret_cast<const float2*>(part0 + (size_t)i * S::PART + AP_BM * HD) + r).y;
                        f[i] = exp2f(f[i] - m_all);
                        l_all += f[i] * l_i;
                    }
                }
                const float inv = 1.0f / l_all;
#pragma unroll 1
                for (int c = 0; c < HD; c += 16) {
                    float o[16];
#pragma unroll
                    for (int k = 0; k < 16; ++k) o[k] = 0.f;
#pragma unroll
                    for (int i = 0; i < AP_MAX_SPLIT; ++i) {
                        if (i < n_runs) {
                            const float4* src = reinterpret_cast<const float4*>(part0 + (size_t)i * S::PART);
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const float4 t = __ldcg(src + (c / 4 + k) * AP_BM + r);
                                o[4 * k] += f[i] * t.x; o[4 * k + 1] += f[i] * t.y;
                                o[4 * k + 2] += f[i] * t.z; o[4 * k + 3] += f[i] * t.w;
                            }
                        }
                    }
                    if (r < rows_valid) {
                        uint32_t w[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const __nv_bfloat162 pk = __floats2bfloat162_rn(o[2 * i] * inv, o[2 * i + 1] * inv);
                            w[i] = *reinterpret_cast<const uint32_t*>(&pk);
                        }
                        *reinterpret_cast<uint4*>(orow + c) = make_uint4(w[0], w[1], w[2], w[3]);
                        *reinterpret_cast<uint4*>(orow + c + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                    }
                }
            }
        } else if (ok) {
            tc_fence_after();
            const float inv = 1.0f / l;
#pragma unroll 1
            for (int c = 0; c < HD; c += 16) {
                float o[16];
                tc_ld16(tmem_o + lane_base + c, o);
                if (r < rows_valid) {
                    uint32_t w[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const __nv_bfloat162 pk = __floats2bfloat162_rn(o[2 * i] * inv, o[2 * i + 1] * inv);
                        w[i] = *reinterpret_cast<const uint32_t*>(&pk);
                    }
                    *reinterpret_cast<uint4*>(orow + c) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(orow + c + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem, AP_TMEM_COLS);
}

template <int HD>
static int launch_prefill(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillArgs& a,
                          int n_tiles, cudaStream_t stream) {
    using S = PrefillSmem<HD>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             S::TOTAL);
        IDM_REQUIRE(e == cudaSuccess, "attention_prefill: cannot get %d bytes of shared memory: %s", S::TOTAL,
                    cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid(a.n_q * a.max_split, n_tiles);
    idm_launch(attention_prefill_kernel<HD>, dim3(grid), dim3(AP_THREADS), S::TOTAL, stream, mq, mk, mv, a);
    IDM_LAUNCH_CHECK("attention_prefill");
    return 0;
}

extern "C" int idm_attention_prefill_supports(int hd) { return hd == 64 || hd == 128; }

// How many key blocks a run may have, for a step whose tiles have `key_blocks` in all (over all heads)
// and `longest` in the longest: a fair share of the work of the SMs' block slots and a quarter, so that
// only tiles that would keep one SM busy long after the others ended are cut.  A run's partial result
// goes through memory, which costs about as much as four key blocks.
extern "C" int idm_attention_prefill_max_run(long long key_blocks, int longest, int n_tiles, int n_q) {
    if ((long long)n_tiles * n_q > AP_COUNTERS) return longest;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;                               // (no answer from the device: the B200's count)
    const long long share = (key_blocks + 2 * sms - 1) / (2 * sms);
    const long long run = share + share / 4 + 2;
    return (int)(run < AP_MIN_RUN ? AP_MIN_RUN : run > longest ? longest : run);
}
// Floats of scratch for that: arrival counters (zero at the first launch, left at zero by every launch),
// then the runs' partial results.
extern "C" long long idm_attention_prefill_scratch_floats(int n_tiles, int n_q, int hd, int split) {
    if (split <= 1) return 0;
    return (long long)AP_COUNTERS + (long long)n_tiles * n_q * split * (AP_BM * hd + 2 * AP_BM);
}

// q [n_tokens, n_q, hd]; out [n_tokens, n_q * hd]; the cache entry's pools [n_pages, n_kv, 64, hd];
// tiles: (sequence, first token of the tile within the sequence's tokens of this step), longest first.
extern "C" int idm_attention_prefill(const void* q, void* out, const void* k_pool, const void* v_pool, int n_pages,
                                     const int* table, int table_stride, const int* tile_seq, const int* tile_start,
                                     int n_tiles, const int* cu_q, const int* q_start, const int* kv_len,
                                     const int* slots, int n_tokens, int n_q, int n_kv, int hd, float scale,
                                     int split, int max_run, float* scratch, cudaStream_t stream) {
    if (n_tiles == 0 || n_tokens == 0) return 0;
    IDM_REQUIRE(idm_attention_prefill_supports(hd), "attention_prefill: head_dim=%d has no kernel here", hd);
    IDM_REQUIRE(n_kv > 0 && n_q % n_kv == 0, "attention_prefill: bad head counts %d/%d", n_q, n_kv);
    IDM_REQUIRE(n_tiles <= 65535, "attention_prefill: %d tiles in one step; at most 65535", n_tiles);
    IDM_REQUIRE(split >= 1 && split <= AP_MAX_SPLIT && (split == 1 || (scratch && (long long)n_tiles * n_q <= AP_COUNTERS)),
                "attention_prefill: split=%d of %d tiles x %d heads (at most %d, with scratch, for at most %d of them)",
                split, n_tiles, n_q, AP_MAX_SPLIT, AP_COUNTERS);
    CUtensorMap mq, mk, mv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)n_q, (cuuint64_t)n_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)n_q * hd * 2};
        cuuint32_t box[3] = {64, 1, AP_BM};
        const int r = tc_make_map_bf16(&mq, q, 3, dims, strides, box);
        IDM_REQUIRE(r == 0, "attention_prefill: tensor map for q failed (%d)", r);
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)n_pages * n_kv * IDM_PAGE};
        cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
        cuuint32_t box[2] = {64, AP_BN};
        int r = tc_make_map_bf16(&mk, k_pool, 2, dims, strides, box);
        IDM_REQUIRE(r == 0, "attention_prefill: tensor map for k failed (%d)", r);
        r = tc_make_map_bf16(&mv, v_pool, 2, dims, strides, box);
        IDM_REQUIRE(r == 0, "attention_prefill: tensor map for v failed (%d)", r);
    }
    PrefillArgs a;
    a.out = (T*)out; a.tile_seq = tile_seq; a.tile_start = tile_start; a.cu_q = cu_q; a.q_start = q_start;
    a.kv_len = kv_len; a.slots = slots; a.table = table; a.table_stride = table_stride;
    a.n_q = n_q; a.n_kv = n_kv; a.scale_log2 = scale * 1.4426950408889634f;
    a.max_split = split; a.max_run = max_run < 1 ? 1 : max_run; a.counters = (int*)scratch; a.parts = scratch ? scratch + AP_COUNTERS : nullptr;
    return hd == 64 ? launch_prefill<64>(mq, mk, mv, a, n_tiles, stream)
                    : launch_prefill<128>(mq, mk, mv, a, n_tiles, stream);
}

extern "C" int idm_attention_prefill_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_prefill_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_attn_prefill_error, &zero, sizeof(int));
    return v;
}

#endif  // IDM_BF16
