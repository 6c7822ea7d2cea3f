// out[M, N] = x[M, K] . w[N, K]^T in true FP32: FFMA on CUDA cores, no tensor-core mode.
//
// The reference calls cublasSgemm with the default math mode for every projection
// (src/op/kernels/cuda/matmul_kernel.cu:48-89).  This kernel keeps the FP32 path free of
// any library's choice of algorithm: each output element is one chain of fused
// multiply-adds over k = 0 .. K-1 in ascending order, whatever M is and wherever the
// element lies in a tile, so a token's result does not depend on its batch.
#include "common.cuh"

#define GF_BM 64
#define GF_BN 64
#define GF_BK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ out,
                int M, int N, int K) {
    __shared__ float xs[GF_BK][GF_BM + 4];
    __shared__ float ws[GF_BK][GF_BN + 4];
    const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GF_BK) {
        // 64 rows x 16 k of each operand: 1024 elements, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = threadIdx.x + 256 * e;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            xs[kk][r] = (m0 + r < M && k < K) ? x[(size_t)(m0 + r) * K + k] : 0.f;
            ws[kk][r] = (n0 + r < N && k < K) ? w[(size_t)(n0 + r) * K + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GF_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
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

NI_EXPORT int ni_gemm_f32(const float* x, const float* w, float* out, int M, int N, int K,
                          cudaStream_t stream) {
    if (M <= 0 || N <= 0) return NI_OK;
    if (K <= 0) return NI_ERR_BAD_ARGUMENT;
    dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
    if (grid.y > 65535) return NI_ERR_UNSUPPORTED_SIZE;
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(x, w, out, M, N, K);
    NI_RETURN_LAUNCH_STATUS();
}
