// Embedding gather, residual-add + RMSNorm, SwiGLU activation.
//
// Counterparts in the reference (all FP32, one launch per op, nothing fused):
// src/op/kernels/cuda/embedding_kernel.cu:30-48, rmsnorm_kernel.cu:49-104,
// add_kernel.cu:23-29, swiglu_kernel.cu:25-40.  Here the residual stream is FP32 in
// both precisions, the residual add is fused into the norm that follows it, and the
// norm's statistics are FP32.
#include "common.cuh"

// out[t, :] = table[tokens[t], :] as FP32.  Ids are validated on the host; an id out of
// range writes zeros instead of reading outside the table.
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                 float* __restrict__ out, int d, int vocab) {
    const int t = blockIdx.x;
    const int tok = tokens[t];
    const bool ok = tok >= 0 && tok < vocab;
    const T* row = table + (size_t)(ok ? tok : 0) * d;
    float* o = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = ok ? ni_to_float(row[i]) : 0.f;
}

NI_EXPORT int ni_embedding(const int* tokens, const void* table, int table_dtype, float* out,
                           int n_tokens, int d, int vocab, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (d <= 0 || vocab <= 0) return NI_ERR_BAD_ARGUMENT;
    const int threads = d >= 1024 ? 256 : 128;
    if (table_dtype == NI_DTYPE_F32)
        embedding_kernel<float><<<n_tokens, threads, 0, stream>>>(tokens, (const float*)table, out, d, vocab);
    else if (table_dtype == NI_DTYPE_BF16)
        embedding_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            tokens, (const __nv_bfloat16*)table, out, d, vocab);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// Row r of the output: src = rows ? rows[r] : r;  v = h[src] + delta[src];
// if rows == nullptr, h[src] = v is written back;  out[r] = v * rsqrt(mean(v^2) + eps) * gain.
// eps is added to the mean, inside the root (rmsnorm_kernel.cu:79).
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                   const float* __restrict__ gain, float eps,
                                   TO* __restrict__ out, const int* __restrict__ rows, int d) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* hr = h + (size_t)src * d;
    const TD* dr = delta ? delta + (size_t)src * d : nullptr;
    TO* o = out + (size_t)r * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = hr[i];
        if (dr) {
            v += ni_to_float(dr[i]);
            if (!rows) hr[i] = v;
        }
        ss += v * v;
    }
    ss = ni_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = hr[i];
        if (dr && rows) v += ni_to_float(dr[i]);
        o[i] = ni_from_float<TO>((v * inv) * gain[i]);
    }
}

NI_EXPORT int ni_add_rmsnorm(float* h, const void* delta, int delta_dtype, const float* gain,
                             float eps, void* out, int out_dtype, const int* rows, int n_rows,
                             int d, cudaStream_t stream) {
    if (n_rows <= 0) return NI_OK;
    if (d <= 0) return NI_ERR_BAD_ARGUMENT;
    const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
#define LAUNCH(TD, TO)                                                                         \
    add_rmsnorm_kernel<TD, TO><<<n_rows, threads, 0, stream>>>(h, (const TD*)delta, gain, eps, \
                                                                (TO*)out, rows, d)
    if (delta_dtype == NI_DTYPE_F32 && out_dtype == NI_DTYPE_F32) LAUNCH(float, float);
    else if (delta_dtype == NI_DTYPE_BF16 && out_dtype == NI_DTYPE_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (delta_dtype == NI_DTYPE_F32 && out_dtype == NI_DTYPE_BF16) LAUNCH(float, __nv_bfloat16);
    else if (delta_dtype == NI_DTYPE_BF16 && out_dtype == NI_DTYPE_F32) LAUNCH(__nv_bfloat16, float);
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}

// h[t, :] += delta[t, :]  (the last pending addition of a forward pass).
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ h, const TD* __restrict__ delta, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) h[i] += ni_to_float(delta[i]);
}

NI_EXPORT int ni_residual_add(float* h, const void* delta, int delta_dtype, long long n,
                              cudaStream_t stream) {
    if (n <= 0) return NI_OK;
    const int threads = 256;
    long long blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (delta_dtype == NI_DTYPE_F32)
        residual_add_kernel<float><<<(int)blocks, threads, 0, stream>>>(h, (const float*)delta, (size_t)n);
    else if (delta_dtype == NI_DTYPE_BF16)
        residual_add_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
            h, (const __nv_bfloat16*)delta, (size_t)n);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i], FP32 arithmetic with expf.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int n_tokens,
                              int inter) {
    const size_t total = (size_t)n_tokens * inter;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const size_t t = idx / inter;
        const int i = (int)(idx - t * inter);
        const float g = ni_to_float(gate_up[t * 2 * inter + i]);
        const float u = ni_to_float(gate_up[t * 2 * inter + inter + i]);
        out[idx] = ni_from_float<T>((g / (1.0f + expf(-g))) * u);
    }
}

NI_EXPORT int ni_swiglu(const void* gate_up, void* out, int dtype, int n_tokens, int inter,
                        cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (inter <= 0) return NI_ERR_BAD_ARGUMENT;
    const int threads = 256;
    long long blocks = ((long long)n_tokens * inter + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (dtype == NI_DTYPE_F32)
        swiglu_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, n_tokens, inter);
    else if (dtype == NI_DTYPE_BF16)
        swiglu_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, n_tokens, inter);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}
