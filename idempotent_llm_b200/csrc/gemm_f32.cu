// out[M, N] = x[M, K] . w[N, K]^T in true 32-bit: plain FMA on CUDA cores, no tensor
// cores, no reduced-precision mode.  Each output element is one chain of FMAs over k
// in ascending order, so its value does not depend on M, on the tile it falls in, or
// on what else is in the batch.  (The reference's exact path is the CPU integer
// matmul of src/detllm/backends.py:95-96; this is its float counterpart.)
#include "common.cuh"

#define GB 64      // tile of outputs per block: GB x GB
#define GK 16      // inner-axis slab

__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                       float* __restrict__ out, int M, int N, int K) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float xs[GK][GB + 4];
    __shared__ float ws[GK][GB + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * GB, n0 = blockIdx.x * GB;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const int lr = threadIdx.x / 4;          // row of the tile this thread loads (0..63)
    const int lk = (threadIdx.x % 4) * 4;    // first of its 4 k
    for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int m = m0 + lr, n = n0 + lr;
            xs[lk + e][lr] = (m < M && k < K) ? x[(size_t)m * K + k] : 0.f;
            ws[lk + e][lr] = (n < N && k < K) ? w[(size_t)n * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) out[(size_t)m * N + n] = acc[i][j];
        }
    }
}

extern "C" int idm_gemm_f32(const float* x, const float* w, float* out, int M, int N, int K,
                            cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    IDM_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
    dim3 grid((N + GB - 1) / GB, (M + GB - 1) / GB);
    IDM_REQUIRE(grid.y <= 65535, "gemm_f32: M=%d is too large for one launch", M);
    idm_launch(gemm_f32_kernel, dim3(grid), dim3(256), 0, stream, x, w, out, M, N, K);
    IDM_LAUNCH_CHECK("gemm_f32");
    return 0;
}
