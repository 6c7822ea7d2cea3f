// Skinny matrix product for decode: y[M, N] = x[M, K] . W[N, K]^T with M <= 16 rows of
// activations against a large bfloat16 weight matrix - a bandwidth problem.
//
// "Swap AB": the weight rows are the M side of the tensor-core tile (mma.sync m16n8k16, bf16
// in, FP32 accumulate) and the batch is the 8-wide N side, so one pass over the weights serves
// the whole batch and the FP32 FMA pipes never become the limit (they would from about four
// rows on).  A block owns 8 or 16 weight rows; its 8 warps split K and stream their slices
// from global memory straight into MMA fragments with 16-byte loads (the contraction index is
// permuted identically in both operands, as in attention_decode.cu), several loads in flight
// per thread.  Partial sums meet in shared memory and are added in warp order, so a result
// never depends on timing.  The epilogue stores bfloat16, stores FP32 (logits) or adds into
// the FP32 residual stream.
//
// Reference counterpart: cublasSgemm on FP32 weights for every projection
// (src/op/kernels/cuda/matmul_kernel.cu:48-89) plus a separate add kernel for the residual.
#include "common.cuh"

#define GV_WARPS 8
#define GV_UNROLL 4

#define GV_STORE_BF16 0
#define GV_STORE_F32 1
#define GV_ADD_F32 2

__device__ __forceinline__ void gv_mma(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// RN: weight rows per block (8 or 16).  NT: batch tiles of 8 rows (1 or 2).
template <int RN, int NT>
__global__ void __launch_bounds__(GV_WARPS * 32)
gemv_bf16_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                 void* __restrict__ out, int M, int N, int K, int mode) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * RN;
    const int n_blocks = (K + 63) / 64;            // k-blocks of 64
    const uint4 zero = make_uint4(0, 0, 0, 0);

    const bool row_a_ok = n0 + g < N;
    const bool row_b_ok = RN == 16 && n0 + g + 8 < N;
    const __nv_bfloat16* wa = w + (size_t)(row_a_ok ? n0 + g : 0) * K;
    const __nv_bfloat16* wb = w + (size_t)(row_b_ok ? n0 + g + 8 : 0) * K;
    const __nv_bfloat16* xr[NT];
    bool x_ok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        x_ok[nt] = 8 * nt + g < M;
        xr[nt] = x + (size_t)(x_ok[nt] ? 8 * nt + g : 0) * K;
    }

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    for (int kb = warp; kb < n_blocks; kb += GV_WARPS * GV_UNROLL) {
        uint4 fa[GV_UNROLL][2], fb[GV_UNROLL][2], fx[GV_UNROLL][NT][2];
#pragma unroll
        for (int u = 0; u < GV_UNROLL; ++u) {
            const int k0 = (kb + u * GV_WARPS) * 64;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int k = k0 + 32 * h + 8 * t;
                const bool ok = k + 8 <= K;        // K is a multiple of 8
                fa[u][h] = (ok && row_a_ok) ? ld_stream(wa + k) : zero;
                fb[u][h] = (RN == 16 && ok && row_b_ok) ? ld_stream(wb + k) : zero;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    fx[u][nt][h] = (ok && x_ok[nt]) ? *reinterpret_cast<const uint4*>(xr[nt] + k) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < GV_UNROLL; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    gv_mma(acc[nt], fa[u][h].x, fb[u][h].x, fa[u][h].y, fb[u][h].y, fx[u][nt][h].x, fx[u][nt][h].y);
                    gv_mma(acc[nt], fa[u][h].z, fb[u][h].z, fa[u][h].w, fb[u][h].w, fx[u][nt][h].z, fx[u][nt][h].w);
                }
    }

    // partial sums of the 8 warps -> shared memory -> summed in warp order
    __shared__ float red[GV_WARPS][NT][16][8];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        red[warp][nt][g][2 * t] = acc[nt][0];
        red[warp][nt][g][2 * t + 1] = acc[nt][1];
        red[warp][nt][g + 8][2 * t] = acc[nt][2];
        red[warp][nt][g + 8][2 * t + 1] = acc[nt][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < NT * 8 * RN; idx += blockDim.x) {
        const int row = idx % RN;                  // weight row within the block: fastest, for coalescing
        const int m = idx / RN;                    // batch row
        const int n = n0 + row;
        if (m >= M || n >= N) continue;
        float s = 0.f;
#pragma unroll
        for (int wi = 0; wi < GV_WARPS; ++wi) s += red[wi][m >> 3][row][m & 7];
        const size_t o = (size_t)m * N + n;
        if (mode == GV_STORE_BF16) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(s);
        else if (mode == GV_STORE_F32) reinterpret_cast<float*>(out)[o] = s;
        else reinterpret_cast<float*>(out)[o] += s;
    }
}

// mode: 0 store bfloat16, 1 store float32, 2 add into float32.  M <= 16, K a multiple of 8.
NI_EXPORT int ni_gemv_bf16(const void* x, const void* w, void* out, int M, int N, int K, int mode,
                           cudaStream_t stream) {
    if (M <= 0 || N <= 0) return NI_OK;
    if (K <= 0 || mode < 0 || mode > 2) return NI_ERR_BAD_ARGUMENT;
    if (M > 16 || K % 8) return NI_ERR_UNSUPPORTED_SIZE;
    // 16 rows per block unless that leaves SMs idle
    const bool rn16 = (N + 15) / 16 >= 2 * 148;
    const int rn = rn16 ? 16 : 8;
    const int grid = (N + rn - 1) / rn;
#define LAUNCH(RN, NT)                                                                      \
    gemv_bf16_kernel<RN, NT><<<grid, GV_WARPS * 32, 0, stream>>>(                           \
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, out, M, N, K, mode)
    if (rn16) { if (M <= 8) LAUNCH(16, 1); else LAUNCH(16, 2); }
    else { if (M <= 8) LAUNCH(8, 1); else LAUNCH(8, 2); }
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}
