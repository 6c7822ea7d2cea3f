// Causal grouped-query attention over the paged cache, the plain way: one warp per
// (token, query head), keys visited one by one in ascending position with an online
// softmax in FP32.  Prompt portions and single decoded tokens are the same case: a
// token at position p sees keys [max(0, p - window + 1), p] of its own request.  An optional
// token list restricts the launch to some of the step's tokens (n_tokens = its length).
// An optional slope per query head adds slope * (key position - query position) to the scaled
// score: a position encoding that acts on the scores instead of rotating queries and keys.
//
// The result of a token depends only on its own keys and their order, never on how the
// step was cut or what else is in the batch, so this kernel is the FP32 path's attention
// and the yardstick beside the tensor-core kernels.
//
// Formula as in the reference (decode: src/op/kernels/cuda/paged_attention_kernel.cu:124-198,
// prefill: prefill_attention_kernel.cu:66-141): score = (q . k) * scale, softmax with the
// maximum subtracted, out = sum p_j v_j, kv head = q head / (Hq / Hkv).  The reference
// divides by (sum + 1e-6); this kernel divides by the sum.
#include "common.cuh"

#define ATT_MAX_REGS 8  // head_dim <= 256

template <typename T>
__global__ void attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                                         const T* __restrict__ v_pages, T* __restrict__ out,
                                         const int* __restrict__ token_list,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_token,
                                         const int* __restrict__ block_table, int bt_stride,
                                         int n_tokens, int n_q_heads, int n_kv_heads, int head_dim,
                                         int page_size, int window, float scale,
                                         const float* __restrict__ head_slopes) {
    const int warps_per_block = blockDim.x >> 5;
    const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    if (item >= (long long)n_tokens * n_q_heads) return;
    const int lane = threadIdx.x & 31;
    const int t_item = (int)(item / n_q_heads);
    const int head = (int)(item - (long long)t_item * n_q_heads);
    const int t = token_list ? token_list[t_item] : t_item;
    const int kvh = head / (n_q_heads / n_kv_heads);
    const int pos = positions[t];
    const int* table = block_table + (size_t)seq_of_token[t] * bt_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const float slope = head_slopes ? head_slopes[head] : 0.f;

    float qr[ATT_MAX_REGS], acc[ATT_MAX_REGS];
    const T* qrow = q + ((size_t)t * n_q_heads + head) * head_dim;
#pragma unroll
    for (int r = 0; r < ATT_MAX_REGS; ++r) {
        const int dim = lane + 32 * r;
        qr[r] = dim < head_dim ? ni_to_float(qrow[dim]) : 0.f;
        acc[r] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int j = lo; j <= pos; ++j) {
        const int page = table[j / page_size];
        const size_t off = (((size_t)page * n_kv_heads + kvh) * page_size + (j % page_size)) * head_dim;
        const T* krow = k_pages + off;
        const T* vrow = v_pages + off;
        float dot = 0.f;
#pragma unroll
        for (int r = 0; r < ATT_MAX_REGS; ++r) {
            const int dim = lane + 32 * r;
            if (dim < head_dim) dot += qr[r] * ni_to_float(krow[dim]);
        }
        dot = ni_warp_sum(dot);
        const float s = dot * scale + slope * (float)(j - pos);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int r = 0; r < ATT_MAX_REGS; ++r) {
            const int dim = lane + 32 * r;
            if (dim < head_dim) acc[r] = acc[r] * corr + p * ni_to_float(vrow[dim]);
        }
        m = m_new;
    }
    T* orow = out + ((size_t)t * n_q_heads + head) * head_dim;
    const float inv = 1.0f / l;
#pragma unroll
    for (int r = 0; r < ATT_MAX_REGS; ++r) {
        const int dim = lane + 32 * r;
        if (dim < head_dim) orow[dim] = ni_from_float<T>(acc[r] * inv);
    }
}

NI_EXPORT int ni_attention_generic(const void* q, int dtype, const void* k_pages,
                                   const void* v_pages, void* out, const int* token_list,
                                   const int* positions, const int* seq_of_token, const int* block_table, int bt_stride,
                                   int n_tokens, int n_q_heads, int n_kv_heads, int head_dim,
                                   int page_size, int window, float scale, const float* head_slopes,
                                   cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads || head_dim <= 0 || page_size <= 0)
        return NI_ERR_BAD_ARGUMENT;
    if (head_dim > 32 * ATT_MAX_REGS) return NI_ERR_UNSUPPORTED_SIZE;
    const int warps = 4;
    const long long items = (long long)n_tokens * n_q_heads;
    const long long blocks = (items + warps - 1) / warps;
    if (blocks > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
#define LAUNCH(T)                                                                                   \
    attention_generic_kernel<T><<<(int)blocks, warps * 32, 0, stream>>>(                            \
        (const T*)q, (const T*)k_pages, (const T*)v_pages, (T*)out, token_list, positions,         \
        seq_of_token,                                                                               \
        block_table, bt_stride, n_tokens, n_q_heads, n_kv_heads, head_dim, page_size, window, scale, head_slopes)
    if (dtype == NI_DTYPE_F32) LAUNCH(float);
    else if (dtype == NI_DTYPE_BF16) LAUNCH(__nv_bfloat16);
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}
