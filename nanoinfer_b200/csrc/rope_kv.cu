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

// Adjacent-pair rotation with 16-byte accesses: one thread takes 8 consecutive elements (4
// rotary pairs) of one head of one token.  head_dim a multiple of 8.
template <typename T> struct Chunk8;
template <> struct Chunk8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float v[8]) {
        const uint4 r = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
            v[2 * i] = __bfloat162float(b.x);
            v[2 * i + 1] = __bfloat162float(b.y);
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float v[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&b);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <> struct Chunk8<float> {
    static __device__ __forceinline__ void load(const float* p, float v[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float v[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};

// Adjacent-pair rotation with 16-byte accesses.  A block takes one token at a time: the token's
// rotary_dim / 2 (cos, sin) pairs are computed once into shared memory (they are the same for all
// of its heads) and its page is looked up once; then every thread rotates 8-element chunks.
template <typename T>
__global__ void rope_kv_write_vec_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                         T* __restrict__ k_pages, T* __restrict__ v_pages,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_token,
                                         const int* __restrict__ block_table, int bt_stride,
                                         const float* __restrict__ inv_freq, int n_tokens, int n_q_heads,
                                         int n_kv_heads, int head_dim, int rotary_dim, int page_size,
                                         int write_cache) {
    extern __shared__ float rope_cs[];                 // [rotary_dim / 2][cos, sin]
    const int chunks_per_head = head_dim >> 3;
    const int heads = n_q_heads + 2 * n_kv_heads;
    const int items = heads * chunks_per_head;
    for (int t = blockIdx.x; t < n_tokens; t += gridDim.x) {
        const int pos = positions[t];
        __syncthreads();                               // the table of the token before is no longer read
        for (int i = threadIdx.x; i < (rotary_dim >> 1); i += blockDim.x) {
            float s, cs;
            sincosf((float)pos * inv_freq[i], &s, &cs);
            rope_cs[2 * i] = cs;
            rope_cs[2 * i + 1] = s;
        }
        __syncthreads();
        const int page = write_cache ? block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size] : 0;
        const int slot = pos % page_size;
        // four chunks per thread and pass: all loads are issued before the first store, since what
        // bounds this kernel is the number of bytes in flight
        for (int item0 = threadIdx.x; item0 < items; item0 += 4 * blockDim.x) {
            float v[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int item = item0 + u * blockDim.x;
                if (item < items) {
                    const int head = item / chunks_per_head, c = item - head * chunks_per_head;
                    Chunk8<T>::load(qkv + ((size_t)t * heads + head) * head_dim + 8 * c, v[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int item = item0 + u * blockDim.x;
                if (item >= items) continue;
                const int head = item / chunks_per_head, c = item - head * chunks_per_head;
                if (head < n_q_heads + n_kv_heads) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int d = 8 * c + 2 * i;
                        if (d < rotary_dim) {
                            const float cs = rope_cs[d], sn = rope_cs[d + 1];
                            const float a = v[u][2 * i], b = v[u][2 * i + 1];
                            v[u][2 * i] = a * cs - b * sn;
                            v[u][2 * i + 1] = a * sn + b * cs;
                        }
                    }
                }
                T* dst;
                if (head < n_q_heads) {
                    dst = q_out + ((size_t)t * n_q_heads + head) * head_dim + 8 * c;
                } else {
                    if (!write_cache) continue;
                    const bool is_k = head < n_q_heads + n_kv_heads;
                    const int kvh = is_k ? head - n_q_heads : head - n_q_heads - n_kv_heads;
                    dst = (is_k ? k_pages : v_pages) + (((size_t)page * n_kv_heads + kvh) * page_size + slot) * head_dim + 8 * c;
                }
                Chunk8<T>::store(dst, v[u]);
            }
        }
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
    if (interleaved && head_dim % 8 == 0) {
        const int items = (n_q_heads + 2 * n_kv_heads) * (head_dim / 8);
        const int threads = items >= 512 ? 256 : (items >= 256 ? 128 : 64);      // about four chunks per thread
        const int blocks = n_tokens < ni_sm_count() * 16 ? n_tokens : ni_sm_count() * 16;
#define LAUNCHV(T)                                                                                     \
    rope_kv_write_vec_kernel<T><<<blocks, threads, rotary_dim * sizeof(float), stream>>>(               \
        (const T*)qkv, (T*)q_out, (T*)k_pages, (T*)v_pages, positions, seq_of_token, block_table,     \
        bt_stride, inv_freq, n_tokens, n_q_heads, n_kv_heads, head_dim, rotary_dim, page_size, write_cache)
        if (dtype == NI_DTYPE_F32) LAUNCHV(float);
        else if (dtype == NI_DTYPE_BF16) LAUNCHV(__nv_bfloat16);
        else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCHV
        NI_RETURN_LAUNCH_STATUS();
    }
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
