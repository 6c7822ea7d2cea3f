// Split-K grouped-query attention for single query tokens over the paged bfloat16 cache.
//
// One thread block per (query token, kv head, split).  The G = Hq / Hkv query heads that
// share a kv head are the rows of a 16-row tensor-core tile (mma.sync m16n8k16, bf16 in, FP32
// accumulate), so every key and value is fetched once for all of them.  Each of the block's
// warps walks its own 32-key chunks of the split's key range with its own online-softmax state
// (FP32); K and V go from global memory straight into MMA fragments with 16-byte loads - no
// shared-memory staging, no barrier in the loop.  That works because the contraction index of
// an MMA may be permuted freely as long as both operands agree:
//   S = Q K^T: thread (g, t) takes dims [32p + 8t, 32p + 8t + 8) of key 8j + g in one load and
//              feeds them to two MMAs; Q's fragments are built with the same permutation.
//   O = P V:   output column (tile j, lane g) is dim 8g + j (hd 64), so a thread's B fragments
//              for all 8 column tiles of one key are one contiguous 16-byte load.
// Warps are merged through shared memory; the split's (max, sum, unnormalised O) goes to a
// scratch buffer; the block that arrives last for its (token, kv head) - counted with an atomic
// ticket - merges the splits in split order and writes the bfloat16 output.  No block waits for
// another, and the merge order is fixed, so results are reproducible.
//
// The grid does not depend on context lengths (they are read on the device), so a decode step
// can be captured in a CUDA graph and replayed as contexts grow.
//
// Reference counterpart: src/op/kernels/cuda/paged_attention_kernel.cu:111-199 (one block per
// (head, sequence), FP32 CUDA cores, all scores of a sequence in shared memory, no split).
#include "common.cuh"

#define DEC_WARPS 4
#define DEC_CHUNK 32  // keys per warp iteration

__device__ __forceinline__ void mma_bf16_16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// HD: head size (multiple of 32, <= 128).  Scratch per (token, q head, split): HD + 2 floats.
template <int HD>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                        const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ token_list, const int* __restrict__ positions,
                        const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                        int bt_stride, int n_q_heads, int n_kv_heads, int page_size, int window,
                        float scale_log2e, int n_splits, float* __restrict__ scratch,
                        int* __restrict__ tickets) {
    constexpr int KP = HD / 32;      // pairs of k-steps in Q K^T
    constexpr int NT_O = HD / 8;     // output column tiles in P V
    constexpr int VL = HD / 64 > 0 ? HD / 64 : 1;  // 16-byte V loads per key per thread (HD >= 64)
    static_assert(HD % 32 == 0 && HD <= 128, "head size");

    const int item = blockIdx.x;             // index into token_list
    const int kvh = blockIdx.y;
    const int split = blockIdx.z;
    const int t_idx = token_list ? token_list[item] : item;
    const int pos = positions[t_idx];
    const int* table = block_table + (size_t)seq_of_token[t_idx] * bt_stride;
    const int G = n_q_heads / n_kv_heads;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_keys = pos + 1 - lo;
    // the split's key range, in whole chunks
    const int chunks_total = (n_keys + DEC_CHUNK - 1) / DEC_CHUNK;
    const int chunks_per_split = (chunks_total + n_splits - 1) / n_splits;
    const int k_begin = lo + split * chunks_per_split * DEC_CHUNK;
    const int k_end = min(pos + 1, k_begin + chunks_per_split * DEC_CHUNK);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    // Q fragments (rows = heads of the group, zero beyond G), dims permuted as described above
    uint32_t qa[KP][2][4];
    {
        const __nv_bfloat16* qbase = q + ((size_t)t_idx * n_q_heads + (size_t)kvh * G) * HD;
#pragma unroll
        for (int p = 0; p < KP; ++p) {
            uint4 r0 = make_uint4(0, 0, 0, 0), r1 = make_uint4(0, 0, 0, 0);
            if (g < G) r0 = *reinterpret_cast<const uint4*>(qbase + (size_t)g * HD + 32 * p + 8 * t);
            if (g + 8 < G) r1 = *reinterpret_cast<const uint4*>(qbase + (size_t)(g + 8) * HD + 32 * p + 8 * t);
            qa[p][0][0] = r0.x; qa[p][0][1] = r1.x; qa[p][0][2] = r0.y; qa[p][0][3] = r1.y;
            qa[p][1][0] = r0.z; qa[p][1][1] = r1.z; qa[p][1][2] = r0.w; qa[p][1][3] = r1.w;
        }
    }

    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g + 8

    for (int c0 = k_begin + warp * DEC_CHUNK; c0 < k_end; c0 += DEC_WARPS * DEC_CHUNK) {
        // ---- S = Q K^T for 32 keys: 4 column tiles of 8 keys ----
        float s[4][4];
        uint4 kf[4][KP];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int key = c0 + 8 * j + g;
            key = key < k_end ? key : k_end - 1;       // clamp: masked below, never out of the table
            const int page = table[key / page_size];
            const __nv_bfloat16* krow =
                k_pages + (((size_t)page * n_kv_heads + kvh) * page_size + (key % page_size)) * HD;
#pragma unroll
            for (int p = 0; p < KP; ++p) kf[j][p] = *reinterpret_cast<const uint4*>(krow + 32 * p + 8 * t);
        }
        // V fragments for the same 32 keys: 2 k-steps of 16 keys; this thread's 4 keys per step
        uint4 vf[2][4][VL * (HD >= 64 ? 1 : 1)];
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int key = c0 + 16 * ks + 2 * t + (e & 1) + 8 * (e >> 1);
                key = key < k_end ? key : k_end - 1;
                const int page = table[key / page_size];
                const __nv_bfloat16* vrow =
                    v_pages + (((size_t)page * n_kv_heads + kvh) * page_size + (key % page_size)) * HD;
                if (HD >= 64) {
#pragma unroll
                    for (int x = 0; x < VL; ++x)
                        vf[ks][e][x] = *reinterpret_cast<const uint4*>(vrow + (HD / 8) * g + 8 * x);
                } else {  // HD == 32: 4 dims per lane group
                    const uint2 h = *reinterpret_cast<const uint2*>(vrow + 4 * g);
                    vf[ks][e][0] = make_uint4(h.x, h.y, 0, 0);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int p = 0; p < KP; ++p) {
                mma_bf16_16816(s[j], qa[p][0], kf[j][p].x, kf[j][p].y);
                mma_bf16_16816(s[j], qa[p][1], kf[j][p].z, kf[j][p].w);
            }
        }
        // ---- mask, online softmax (base 2) ----
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int key = c0 + 8 * j + 2 * t;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const bool ok = key + (e & 1) < k_end;
                s[j][e] = ok ? s[j][e] * scale_log2e : -INFINITY;
            }
            mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
            mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite: the chunk has >= 1 key
        const float corr0 = exp2f(m0 - mn0), corr1 = exp2f(m1 - mn1);
        m0 = mn0; m1 = mn1;
        float rs0 = 0.f, rs1 = 0.f;
        uint32_t pa[2][4];   // P as A fragments for the two 16-key k-steps
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float p0 = exp2f(s[j][0] - mn0), p1 = exp2f(s[j][1] - mn0);
            const float p2 = exp2f(s[j][2] - mn1), p3 = exp2f(s[j][3] - mn1);
            // the sum runs over the bfloat16-rounded probabilities that multiply V
            const __nv_bfloat162 r01 = __floats2bfloat162_rn(p0, p1), r23 = __floats2bfloat162_rn(p2, p3);
            rs0 += __bfloat162float(r01.x) + __bfloat162float(r01.y);
            rs1 += __bfloat162float(r23.x) + __bfloat162float(r23.y);
            pa[j >> 1][(j & 1) * 2 + 0] = *reinterpret_cast<const uint32_t*>(&r01);
            pa[j >> 1][(j & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&r23);
        }
        l0 = l0 * corr0 + rs0;
        l1 = l1 * corr1 + rs1;
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
            o[j][0] *= corr0; o[j][1] *= corr0; o[j][2] *= corr1; o[j][3] *= corr1;
        }
        // ---- O += P V ----
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                // column tile j, lane group g <-> dim (HD / 8) * g + j; B fragment: keys e = 0..3 of this thread
                const int x = j >> 3, w = j & 7;   // which 16-byte load, which element of it
                uint32_t b0, b1;
                const uint32_t* e0 = reinterpret_cast<const uint32_t*>(&vf[ks][0][x]);
                const uint32_t* e1 = reinterpret_cast<const uint32_t*>(&vf[ks][1][x]);
                const uint32_t* e2 = reinterpret_cast<const uint32_t*>(&vf[ks][2][x]);
                const uint32_t* e3 = reinterpret_cast<const uint32_t*>(&vf[ks][3][x]);
                // element w of each key's load: halves of 32-bit words
                const uint32_t w0 = e0[w >> 1], w1 = e1[w >> 1], w2 = e2[w >> 1], w3 = e3[w >> 1];
                if (w & 1) {
                    b0 = (w0 >> 16) | (w1 & 0xffff0000u);
                    b1 = (w2 >> 16) | (w3 & 0xffff0000u);
                } else {
                    b0 = (w0 & 0xffffu) | (w1 << 16);
                    b1 = (w2 & 0xffffu) | (w3 << 16);
                }
                mma_bf16_16816(o[j], pa[ks], b0, b1);
            }
        }
    }
    // row sums live in the 4 lanes of a row group
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // ---- merge the block's warps (fixed order) ----
    __shared__ float sm_m[DEC_WARPS][16], sm_l[DEC_WARPS][16];
    __shared__ float sm_o[DEC_WARPS][16][HD + 1];
    if (t == 0) { sm_m[warp][g] = m0; sm_m[warp][g + 8] = m1; sm_l[warp][g] = l0; sm_l[warp][g + 8] = l1; }
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
        // C fragment columns 2t, 2t+1 of tile j are lane groups 2t, 2t+1: dims (HD/8)*(2t) + j and (HD/8)*(2t+1) + j
        const int d0 = (HD / 8) * (2 * t) + j, d1 = (HD / 8) * (2 * t + 1) + j;
        sm_o[warp][g][d0] = o[j][0]; sm_o[warp][g][d1] = o[j][1];
        sm_o[warp][g + 8][d0] = o[j][2]; sm_o[warp][g + 8][d1] = o[j][3];
    }
    __syncthreads();
    const size_t rec = HD + 2;
    for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
        const int row = idx / HD, d = idx - row * HD;
        float mm = sm_m[0][row];
#pragma unroll
        for (int w = 1; w < DEC_WARPS; ++w) mm = fmaxf(mm, sm_m[w][row]);
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = sm_m[w][row] == -INFINITY ? 0.f : exp2f(sm_m[w][row] - mm);
            acc += sm_o[w][row][d] * f;
            ll += sm_l[w][row] * f;
        }
        float* dst = scratch + (((size_t)item * n_q_heads + (size_t)kvh * G + row) * n_splits + split) * rec;
        dst[2 + d] = acc;
        if (d == 0) { dst[0] = mm; dst[1] = ll; }
    }
    // ---- the last block of this (token, kv head) merges the splits ----
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* ticket = tickets + (size_t)item * n_kv_heads + kvh;
        const int prev = atomicAdd(ticket, 1);
        is_last = prev == n_splits - 1;
        if (is_last) *ticket = 0;   // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
        const int row = idx / HD, d = idx - row * HD;
        const float* src = scratch + ((size_t)item * n_q_heads + (size_t)kvh * G + row) * n_splits * rec;
        float mm = -INFINITY;
        for (int sidx = 0; sidx < n_splits; ++sidx) mm = fmaxf(mm, __ldcg(src + sidx * rec));
        float acc = 0.f, ll = 0.f;
        for (int sidx = 0; sidx < n_splits; ++sidx) {
            const float ms = __ldcg(src + sidx * rec);
            const float f = ms == -INFINITY ? 0.f : exp2f(ms - mm);
            acc += __ldcg(src + sidx * rec + 2 + d) * f;
            ll += __ldcg(src + sidx * rec + 1) * f;
        }
        out[((size_t)t_idx * n_q_heads + (size_t)kvh * G + row) * HD + d] = __float2bfloat16_rn(acc / ll);
    }
}

// Scratch floats needed: n_items * n_q_heads * n_splits * (head_dim + 2); tickets: n_items * n_kv_heads
// ints, zero before the first launch (the kernel leaves them zero).
NI_EXPORT int ni_attention_decode(const void* q, const void* k_pages, const void* v_pages, void* out,
                                  const int* token_list, int n_items, const int* positions,
                                  const int* seq_of_token, const int* block_table, int bt_stride,
                                  int n_q_heads, int n_kv_heads, int head_dim, int page_size, int window,
                                  float scale, int n_splits, float* scratch, int* tickets,
                                  cudaStream_t stream) {
    if (n_items <= 0) return NI_OK;
    if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads || page_size <= 0 || n_splits <= 0 ||
        n_splits > 65535 || n_kv_heads > 65535)
        return NI_ERR_BAD_ARGUMENT;
    if (n_q_heads / n_kv_heads > 16) return NI_ERR_UNSUPPORTED_SIZE;
    const float scale_log2e = scale * 1.4426950408889634f;
    dim3 grid(n_items, n_kv_heads, n_splits);
#define LAUNCH(HD)                                                                                    \
    attention_decode_kernel<HD><<<grid, DEC_WARPS * 32, 0, stream>>>(                                 \
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,       \
        (__nv_bfloat16*)out, token_list, positions, seq_of_token, block_table, bt_stride, n_q_heads, \
        n_kv_heads, page_size, window, scale_log2e, n_splits, scratch, tickets)
    switch (head_dim) {
        case 64: LAUNCH(64); break;
        case 128: LAUNCH(128); break;
        default: return NI_ERR_UNSUPPORTED_SIZE;
    }
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}

// ---- the variant that allocates nothing (see attention_decode_noalloc.h) ----------------------
#include "attention_decode_noalloc.h"

static __device__ __align__(256) float ni_noalloc_partials[NI_NOALLOC_MAX_PARTIAL_FLOATS];
static __device__ __align__(256) int ni_noalloc_tickets[NI_NOALLOC_MAX_TICKETS];

#define NI_NOALLOC_MAX_DEVICES 64
// Device addresses of the two arrays, looked up once per device.  In host code the array names
// above are host-side stand-ins; only cudaGetSymbolAddress yields what a kernel can use.
static float* noalloc_partials_addr[NI_NOALLOC_MAX_DEVICES];
static int* noalloc_tickets_addr[NI_NOALLOC_MAX_DEVICES];

NI_EXPORT int ni_attention_decode_noalloc(const void* q, const void* k_pages, const void* v_pages, void* out,
                                          const int* token_list, int n_items, const int* positions,
                                          const int* seq_of_token, const int* block_table, int bt_stride,
                                          int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                                          int window, float scale, int n_splits, cudaStream_t stream) {
    if (n_items <= 0) return NI_OK;
    if (n_q_heads <= 0 || n_kv_heads <= 0 || n_splits <= 0 || head_dim <= 0) return NI_ERR_BAD_ARGUMENT;
    const long long need_floats = (long long)n_items * n_q_heads * n_splits * (head_dim + 2);
    const long long need_tickets = (long long)n_items * n_kv_heads;
    if (need_floats > NI_NOALLOC_MAX_PARTIAL_FLOATS || need_tickets > NI_NOALLOC_MAX_TICKETS)
        return NI_ERR_STATIC_SCRATCH_TOO_SMALL;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NI_NOALLOC_MAX_DEVICES) return NI_ERR_BAD_ARGUMENT;
    if (noalloc_partials_addr[dev] == nullptr || noalloc_tickets_addr[dev] == nullptr) {
        // set-up, once per device, with that device current
        float* p = nullptr;
        int* t = nullptr;
        e = cudaGetSymbolAddress((void**)&p, ni_noalloc_partials);
        if (e != cudaSuccess) return (int)e;
        e = cudaGetSymbolAddress((void**)&t, ni_noalloc_tickets);
        if (e != cudaSuccess) return (int)e;
        noalloc_partials_addr[dev] = p;
        noalloc_tickets_addr[dev] = t;
    }
    // the tickets must start at zero; the partial results are written before they are read
    e = cudaMemsetAsync(noalloc_tickets_addr[dev], 0, (size_t)need_tickets * sizeof(int), stream);
    if (e != cudaSuccess) return (int)e;
    return ni_attention_decode(q, k_pages, v_pages, out, token_list, n_items, positions, seq_of_token,
                               block_table, bt_stride, n_q_heads, n_kv_heads, head_dim, page_size, window,
                               scale, n_splits, noalloc_partials_addr[dev], noalloc_tickets_addr[dev], stream);
}
