// Rotary position encoding of queries and keys, fused with the write of keys and values
// into their cache pages.
//
// The reference does this in three launches over FP32 tensors: rotation in place from a
// precomputed sin/cos table (src/op/kernels/cuda/rope_kernel.cu:32-84, table built at
// :95-132), then a paged write for decode (paged_kv_writed_kernel.cu:33-75) or for a
// prefill chunk (prefill_attention_kernel.cu:219-248).  Here one launch reads the fused
// QKV projection once: queries go rotated to a dense buffer, keys go rotated and values
// go unchanged straight to their page slots.  The angle is the FP32 product
// float(position) * inv_freq, as in the reference's table (rope_kernel.cu:127), and sin/cos
// are evaluated in FP32 per element instead of being read from a table of
// max_position rows.
//
// Page layout: [num_pages, num_kv_heads, page_size, head_dim]; the page of token t is
// block_table[seq_of_token[t] * bt_stride + position / page_size].
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token,
                                     const int* __restrict__ block_table, int bt_stride,
                                     const float* __restrict__ inv_freq, int n_q_heads,
                                     int n_kv_heads, int head_dim, int rotary_dim,
                                     int interleaved, int page_size, int write_cache) {
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = head_dim / 2;
    const int rot_half = rotary_dim / 2;
    const int row_width = (n_q_heads + 2 * n_kv_heads) * head_dim;
    const T* row = qkv + (size_t)t * row_width;
    size_t kv_base = 0;
    if (write_cache) {
        const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
        kv_base = ((size_t)page * n_kv_heads * page_size + (pos % page_size)) * head_dim;
    }
    const int n_pairs = (n_q_heads + 2 * n_kv_heads) * half;
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int head = p / half;
        const int i = p - head * half;
        int ia, ib;
        bool rotate = false;
        if (i < rot_half && head < n_q_heads + n_kv_heads) {
            rotate = true;
            if (interleaved) { ia = 2 * i; ib = 2 * i + 1; }
            else { ia = i; ib = i + rot_half; }
        } else if (head < n_q_heads + n_kv_heads) {
            // dimensions beyond rotary_dim pass through unchanged
            ia = rotary_dim + 2 * (i - rot_half); ib = ia + 1;
        } else {
            ia = 2 * i; ib = 2 * i + 1;
        }
        float a = ni_to_float(row[head * head_dim + ia]);
        float b = ni_to_float(row[head * head_dim + ib]);
        if (rotate) {
            float s, c;
            sincosf((float)pos * inv_freq[i], &s, &c);
            const float ra = a * c - b * s;
            const float rb = a * s + b * c;
            a = ra; b = rb;
        }
        T* dst;
        if (head < n_q_heads) {
            dst = q_out + ((size_t)t * n_q_heads + head) * head_dim;
        } else if (!write_cache) {
            continue;
        } else if (head < n_q_heads + n_kv_heads) {
            dst = k_pages + kv_base + (size_t)(head - n_q_heads) * page_size * head_dim;
        } else {
            dst = v_pages + kv_base + (size_t)(head - n_q_heads - n_kv_heads) * page_size * head_dim;
        }
        dst[ia] = ni_from_float<T>(a);
        dst[ib] = ni_from_float<T>(b);
    }
}

NI_EXPORT int ni_rope_kv_write(const void* qkv, int dtype, void* q_out, void* k_pages,
                               void* v_pages, const int* positions, const int* seq_of_token,
                               const int* block_table, int bt_stride, const float* inv_freq,
                               int n_tokens, int n_q_heads, int n_kv_heads, int head_dim,
                               int rotary_dim, int interleaved, int page_size, int write_cache,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (head_dim <= 0 || head_dim % 2 || rotary_dim < 0 || rotary_dim % 2 || rotary_dim > head_dim ||
        n_q_heads <= 0 || n_kv_heads <= 0 || page_size <= 0)
        return NI_ERR_BAD_ARGUMENT;
    const int n_pairs = (n_q_heads + 2 * n_kv_heads) * head_dim / 2;
    const int threads = n_pairs >= 1024 ? 256 : 128;
#define LAUNCH(T)                                                                                  \
    rope_kv_write_kernel<T><<<n_tokens, threads, 0, stream>>>(                                     \
        (const T*)qkv, (T*)q_out, (T*)k_pages, (T*)v_pages, positions, seq_of_token, block_table, \
        bt_stride, inv_freq, n_q_heads, n_kv_heads, head_dim, rotary_dim, interleaved, page_size, \
        write_cache)
    if (dtype == NI_DTYPE_F32) LAUNCH(float);
    else if (dtype == NI_DTYPE_BF16) LAUNCH(__nv_bfloat16);
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}
