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

// The same with 16-byte accesses and the row held in registers between the two passes:
// d a multiple of 4, at most VPT * 4 * blockDim.x.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
        return make_float4(__bfloat162float(a.x), __bfloat162float(a.y), __bfloat162float(b.x), __bfloat162float(b.y));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 r;
        r.x = *reinterpret_cast<uint32_t*>(&a);
        r.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = r;
    }
};

template <typename TD, typename TO, int VPT>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                       const float* __restrict__ gain, float eps, TO* __restrict__ out,
                                       const int* __restrict__ rows, int d) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* hr = h + (size_t)src * d;
    const TD* dr = delta ? delta + (size_t)src * d : nullptr;
    TO* o = out + (size_t)r * d;
    const int n4 = d >> 2;
    float4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n4) {
            v[i] = Vec4<float>::load(hr + 4 * c);
            if (dr) {
                const float4 dv = Vec4<TD>::load(dr + 4 * c);
                v[i].x += dv.x; v[i].y += dv.y; v[i].z += dv.z; v[i].w += dv.w;
                if (!rows) Vec4<float>::store(hr + 4 * c, v[i]);
            }
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    ss = ni_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n4) {
            const float4 gv = Vec4<float>::load(gain + 4 * c);
            Vec4<TO>::store(o + 4 * c, make_float4((v[i].x * inv) * gv.x, (v[i].y * inv) * gv.y,
                                                   (v[i].z * inv) * gv.z, (v[i].w * inv) * gv.w));
        }
    }
}

// One warp per row, the whole row in the lanes' registers (VPT float4 per lane: d = 128 * VPT):
// all of a row's loads are issued together and the statistics need no block barrier.  2,048 rows
// of 2,048: 10.7 us with one 512-thread block per row (one float4 per thread in flight), 50 MB of
// traffic that mostly lies in L2.
template <typename TD, typename TO, int VPT>
__global__ void __launch_bounds__(256, VPT <= 16 ? 2 : 1) add_rmsnorm_warp_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                                               const float* __restrict__ gain, float eps,
                                                               TO* __restrict__ out, const int* __restrict__ rows,
                                                               int n_rows, int d) {
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (r >= n_rows) return;
    const int src = rows ? rows[r] : r;
    float* hr = h + (size_t)src * d;
    const TD* dr = delta ? delta + (size_t)src * d : nullptr;
    TO* o = out + (size_t)r * d;
    float4 v[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) v[i] = Vec4<float>::load(hr + 4 * (lane + 32 * i));
    if (dr) {
#pragma unroll
        for (int i0 = 0; i0 < VPT; i0 += 4) {       // four loads at a time: the registers of a second whole row would halve the warps per SM
            float4 dv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) dv[j] = Vec4<TD>::load(dr + 4 * (lane + 32 * (i0 + j)));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = i0 + j;
                v[i].x += dv[j].x; v[i].y += dv[j].y; v[i].z += dv[j].z; v[i].w += dv[j].w;
                if (!rows) Vec4<float>::store(hr + 4 * (lane + 32 * i), v[i]);
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const float4 gv = Vec4<float>::load(gain + 4 * (lane + 32 * i));
        Vec4<TO>::store(o + 4 * (lane + 32 * i), make_float4((v[i].x * inv) * gv.x, (v[i].y * inv) * gv.y,
                                                             (v[i].z * inv) * gv.z, (v[i].w * inv) * gv.w));
    }
}

NI_EXPORT int ni_add_rmsnorm(float* h, const void* delta, int delta_dtype, const float* gain,
                             float eps, void* out, int out_dtype, const int* rows, int n_rows,
                             int d, cudaStream_t stream) {
    if (n_rows <= 0) return NI_OK;
    if (d <= 0) return NI_ERR_BAD_ARGUMENT;
    const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
    const bool vec = d % 4 == 0 && d <= 4 * 4 * threads;     // the row fits 4 float4 per thread
    const bool vec1 = vec && d <= 4 * threads;
    // FP32 activations: which kernel runs follows from d alone, never from the number of rows - a row's
    // result must not depend, to the last bit, on how many rows the step has.  bfloat16 activations
    // (whose results agree to rounding only): the warp-per-row kernel where it is faster, i.e. many
    // rows of up to 3,072 (2,048 x 2,048: 6.4 us against 7.7; 128 rows: 3.7 against 2.0; width 4,096,
    // one block per SM: 12.8 against 12.2).
    const bool many_rows = delta_dtype == NI_DTYPE_BF16 && out_dtype == NI_DTYPE_BF16 && n_rows >= 1024;
    const int vpt = (many_rows && d % 128 == 0 && d <= 3072) ? d / 128 : 0;
#define WARP(TD, TO, VPT)                                                                           \
    add_rmsnorm_warp_kernel<TD, TO, VPT><<<(n_rows + 7) / 8, 256, 0, stream>>>(h, (const TD*)delta, gain, eps, \
                                                                               (TO*)out, rows, n_rows, d)
#define LAUNCH(TD, TO)                                                                              \
    do {                                                                                            \
        if (vec1)                                                                                   \
            add_rmsnorm_vec_kernel<TD, TO, 1><<<n_rows, threads, 0, stream>>>(h, (const TD*)delta, gain, eps, \
                                                                             (TO*)out, rows, d);   \
        else if (vec)                                                                               \
            add_rmsnorm_vec_kernel<TD, TO, 4><<<n_rows, threads, 0, stream>>>(h, (const TD*)delta, gain, eps, \
                                                                             (TO*)out, rows, d);   \
        else                                                                                        \
            add_rmsnorm_kernel<TD, TO><<<n_rows, threads, 0, stream>>>(h, (const TD*)delta, gain, eps, \
                                                                        (TO*)out, rows, d);         \
    } while (0)
    if (vpt == 4) WARP(__nv_bfloat16, __nv_bfloat16, 4);
    else if (vpt == 8) WARP(__nv_bfloat16, __nv_bfloat16, 8);
    else if (vpt == 16) WARP(__nv_bfloat16, __nv_bfloat16, 16);
    else if (vpt == 24) WARP(__nv_bfloat16, __nv_bfloat16, 24);
    else if (delta_dtype == NI_DTYPE_F32 && out_dtype == NI_DTYPE_F32) LAUNCH(float, float);
    else if (delta_dtype == NI_DTYPE_BF16 && out_dtype == NI_DTYPE_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (delta_dtype == NI_DTYPE_F32 && out_dtype == NI_DTYPE_BF16) LAUNCH(float, __nv_bfloat16);
    else if (delta_dtype == NI_DTYPE_BF16 && out_dtype == NI_DTYPE_F32) LAUNCH(__nv_bfloat16, float);
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
#undef WARP
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
    if (blocks > ni_sm_count() * 16) blocks = ni_sm_count() * 16;
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

// The blocked layout: columns come in blocks of 16 = 8 gate values and their 8 up values, so
// that one thread turns two 16-byte loads into one 16-byte store (and so that a matrix-product
// epilogue finds a gate and its up value in the same tile).  out[t, 8b + r] =
// silu(gate_up[t, 16b + r]) * gate_up[t, 16b + 8 + r].  inter is a multiple of 8.
template <typename T>
__global__ void swiglu_blocked_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int n_tokens,
                                      int inter) {
    const int blocks_per_row = inter >> 3;
    const size_t total = (size_t)n_tokens * blocks_per_row;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < total; idx += stride) {
        const size_t t = idx / blocks_per_row;
        const int b = (int)(idx - t * blocks_per_row);
        const T* src = gate_up + t * 2 * inter + 16 * b;
        T* dst = out + t * inter + 8 * b;
        const float4 g0 = Vec4<T>::load(src), g1 = Vec4<T>::load(src + 4);
        const float4 u0 = Vec4<T>::load(src + 8), u1 = Vec4<T>::load(src + 12);
        Vec4<T>::store(dst, make_float4((g0.x / (1.0f + expf(-g0.x))) * u0.x, (g0.y / (1.0f + expf(-g0.y))) * u0.y,
                                        (g0.z / (1.0f + expf(-g0.z))) * u0.z, (g0.w / (1.0f + expf(-g0.w))) * u0.w));
        Vec4<T>::store(dst + 4, make_float4((g1.x / (1.0f + expf(-g1.x))) * u1.x, (g1.y / (1.0f + expf(-g1.y))) * u1.y,
                                            (g1.z / (1.0f + expf(-g1.z))) * u1.z, (g1.w / (1.0f + expf(-g1.w))) * u1.w));
    }
}

NI_EXPORT int ni_swiglu_blocked(const void* gate_up, void* out, int dtype, int n_tokens, int inter,
                                cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (inter <= 0 || inter % 8) return NI_ERR_BAD_ARGUMENT;
    const int threads = 256;
    long long blocks = ((long long)n_tokens * (inter / 8) + threads - 1) / threads;
    if (blocks > ni_sm_count() * 32) blocks = ni_sm_count() * 32;
    if (dtype == NI_DTYPE_F32)
        swiglu_blocked_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, n_tokens, inter);
    else if (dtype == NI_DTYPE_BF16)
        swiglu_blocked_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, n_tokens, inter);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

NI_EXPORT int ni_swiglu(const void* gate_up, void* out, int dtype, int n_tokens, int inter,
                        cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (inter <= 0) return NI_ERR_BAD_ARGUMENT;
    const int threads = 256;
    long long blocks = ((long long)n_tokens * inter + threads - 1) / threads;
    if (blocks > ni_sm_count() * 32) blocks = ni_sm_count() * 32;
    if (dtype == NI_DTYPE_F32)
        swiglu_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, n_tokens, inter);
    else if (dtype == NI_DTYPE_BF16)
        swiglu_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, n_tokens, inter);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}
