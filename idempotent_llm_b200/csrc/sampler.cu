// Token choice from 32-bit logits: argmax (temperature 0) or Gumbel-max sampling from
// softmax(logits / T).  Ties go to the lowest token id (src/detllm/model.py:482-490).
// The uniform numbers are a pure function of (row key, token id), so a row's choice
// does not depend on the rest of the batch.  (max, lowest id) is associative and
// commutative, so the thread layout cannot change the result.
#include "common.cuh"

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__device__ __forceinline__ void better(float& bs, int& bi, float s, int i) {
    if (s > bs || (s == bs && i < bi)) { bs = s; bi = i; }
}

#define SP_SLICE 4096       // vocabulary entries per block
#define SP_THREADS 256

// grid (slices, rows).  Each block finds the best entry of its slice; the block that arrives last for
// a row (a counter in scratch, set back to zero) picks the best of the slices.
__global__ void __launch_bounds__(SP_THREADS) sample_kernel(const float* __restrict__ logits, int V, float temperature,
                                                            const long long* __restrict__ keys, int* __restrict__ out,
                                                            float* part_s, int* part_i, int* counters) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float ss[SP_THREADS / 32];
    __shared__ int si[SP_THREADS / 32];
    __shared__ int is_last;
    const int row = blockIdx.y, slice = blockIdx.x, n_slices = gridDim.x;
    const float* lg = logits + (size_t)row * V;
    const unsigned long long key = keys ? (unsigned long long)keys[row] : 0ull;
    const float inv_t = temperature > 0.f ? 1.0f / temperature : 1.0f;
    float bs = -INFINITY;
    int bi = 0x7fffffff;
    const int end = min(V, (slice + 1) * SP_SLICE);
    for (int v = slice * SP_SLICE + threadIdx.x; v < end; v += SP_THREADS) {
        float s = lg[v];
        if (s != s) s = -INFINITY;                      // a NaN never wins
        if (temperature > 0.f) {
            const unsigned long long bits = mix64(key ^ ((unsigned long long)v * 0xD1342543DE82EF95ull));
            // 23 bits: x + 0.5 is exact in 32-bit for x < 2^23, so u lies in [2^-24, 1 - 2^-24] and both
            // logarithms are finite (with 24 bits the largest x rounds up to u = 1 and the score to +inf)
            const float u = ((float)(bits >> 41) + 0.5f) * (1.0f / 8388608.0f);
            s = s * inv_t - logf(-logf(u));
        }
        better(bs, bi, s, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float os = __shfl_xor_sync(0xffffffffu, bs, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        better(bs, bi, os, oi);
    }
    if ((threadIdx.x & 31) == 0) { ss[threadIdx.x >> 5] = bs; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SP_THREADS / 32; ++w) better(bs, bi, ss[w], si[w]);
        part_s[(size_t)row * n_slices + slice] = bs;
        part_i[(size_t)row * n_slices + slice] = bi;
        __threadfence();
        const int prev = atomicAdd(&counters[row], 1);
        is_last = prev == n_slices - 1;
        if (is_last) counters[row] = 0;
    }
    __syncthreads();
    if (is_last && threadIdx.x < 32) {
        __threadfence();
        bs = -INFINITY; bi = 0x7fffffff;
        for (int c = threadIdx.x; c < n_slices; c += 32)
            better(bs, bi, __ldcg(part_s + (size_t)row * n_slices + c), __ldcg(part_i + (size_t)row * n_slices + c));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float os = __shfl_xor_sync(0xffffffffu, bs, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            better(bs, bi, os, oi);
        }
        if (threadIdx.x == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
    }
}

// 32-bit words of scratch: best score and index per (row, slice), one counter per row (zero between launches)
extern "C" long long idm_sample_scratch_floats(int n_rows, int V) {
    const long long n_slices = (V + SP_SLICE - 1) / SP_SLICE;
    return 65536 + 2 * n_rows * n_slices;      // counters first, at a fixed place
}

extern "C" int idm_sample(const float* logits, int n_rows, int V, float temperature, const long long* keys,
                          int* out, float* scratch, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    IDM_REQUIRE(V > 0, "sample: empty vocabulary");
    IDM_REQUIRE(n_rows <= 65535, "sample: %d rows in one launch", n_rows);
    IDM_REQUIRE(!(temperature > 0.f) || keys != nullptr, "sample: temperature > 0 needs row keys");
    const int n_slices = (V + SP_SLICE - 1) / SP_SLICE;
    int* counters = (int*)scratch;
    float* part_s = scratch + 65536;
    int* part_i = (int*)(part_s + (size_t)n_rows * n_slices);
    idm_launch(sample_kernel, dim3(n_slices, n_rows), dim3(SP_THREADS), 0, stream, logits, V, temperature, keys, out,
               part_s, part_i, counters);
    IDM_LAUNCH_CHECK("sample");
    return 0;
}

// After a captured single-token step: feed the chosen tokens back and move every sequence one
// position on, all on the device, so that steps can follow one another without the host
// (the reference's GraphedDecode keeps ids, positions and the write offset in device buffers the
// same way, src/detllm/graphed.py:111-132).  history[step, :] records the chosen tokens.
__global__ void decode_advance_kernel(int* tokens, int* positions, int* q_start, int* kv_len,
                                      const int* sampled, int* history, int* step_counter, int n_seqs,
                                      int max_history) {
    // (No early launch of what follows: the kernels of the next step read the lengths and positions
    // before their own wait for the kernel before them, as things that were there before the step began.
    // With this kernel finished before anything of the next step starts, they are.)
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int step = *step_counter;
    if (i < n_seqs) {
        const int t = sampled[i];
        tokens[i] = t;
        positions[i] += 1;
        q_start[i] += 1;
        kv_len[i] += 1;
        if (step < max_history) history[(size_t)step * n_seqs + i] = t;
    }
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x == 0) *step_counter = step + 1;   // grid is one block (n_seqs <= 1024)
}

extern "C" int idm_decode_advance(int* tokens, int* positions, int* q_start, int* kv_len, const int* sampled,
                                  int* history, int* step_counter, int n_seqs, int max_history,
                                  cudaStream_t stream) {
    IDM_REQUIRE(n_seqs > 0 && n_seqs <= 1024, "decode_advance: %d sequences (at most 1024)", n_seqs);
    idm_launch(decode_advance_kernel, dim3(1), dim3(1024), 0, stream, tokens, positions, q_start, kv_len, sampled, history,
                                                  step_counter, n_seqs, max_history);
    IDM_LAUNCH_CHECK("decode_advance");
    return 0;
}
