// Causal grouped-query attention for portions of prompts over the paged bfloat16 cache.
//
// Flash-style: one thread block per (128 query rows of one request, query head); keys and
// values are gathered from their pages 64 keys at a time into swizzled shared memory with
// cp.async (double buffered), scores and the P V product run on tensor cores (mma.sync
// m16n8k16 bf16, FP32 accumulate, fragments through ldmatrix), softmax is online in FP32.
// The score matrix never exists in memory.  A query at position p sees keys
// [max(0, p - window + 1), p] of its own request; keys written by this very step are
// already in the pages.  Work items (request, first row) come from the host, heaviest first.
//
// Reference counterpart: src/op/kernels/cuda/prefill_attention_kernel.cu:321-475 - gathers K
// and V to contiguous FP32 buffers, materialises the grouped heads and the whole
// [heads, chunk, context] score tensor in global memory, two cuBLAS batched SGEMMs and a
// softmax kernel in between, with seven stream-ordered allocations per layer per chunk.
#include "common.cuh"

#define PF_WARPS 8
#define PF_BM 128
#define PF_BN 128

__device__ __forceinline__ void pf_mma(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x with the hardware approximation (one MUFU instruction; about two units in the last place,
// far below the bfloat16 rounding of the probabilities it feeds); 2^-inf = 0.
__device__ __forceinline__ float pf_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void ldsm_x4(uint32_t r[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t r[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Element offset of (row, 16-byte chunk) in a tile of rows of HD bf16, chunks XOR-swizzled by row.
// The XOR stays inside the row: its mask is the largest power of two dividing the chunk count.
template <int HD> __device__ __forceinline__ int sw(int row, int chunk) {
    constexpr int CH = HD / 8;
    constexpr int MASK = ((CH & -CH) - 1) & 7;
    return row * HD + ((chunk ^ (row & MASK)) << 3);
}

template <int HD>
__global__ void __launch_bounds__(PF_WARPS * 32)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                         const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out,
                         const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
                         const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                         const int* __restrict__ block_table, int bt_stride, int n_q_heads,
                         int n_kv_heads, int page_size, int window, float scale_log2e) {
    constexpr int CH = HD / 8;        // 16-byte chunks per row
    constexpr int KS = HD / 16;       // k-steps over the head size
    constexpr int NT_O = HD / 8;      // output column tiles
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sK = sQ + PF_BM * HD;          // 2 stages
    __nv_bfloat16* sV = sK + 2 * PF_BN * HD;      // 2 stages

    // blocks are numbered tile-major (all heads of the tile with the most keys first): the hardware
    // hands them out in that order, longest job first over the whole launch
    const int tile_index = blockIdx.x / n_q_heads;
    const int seq = tile_seq[tile_index];
    const int row0 = tile_row0[tile_index];       // first query row of the tile within the portion
    const int head = blockIdx.x - tile_index * n_q_heads;
    const int kvh = head / (n_q_heads / n_kv_heads);
    const int tok0 = cu_q[seq];
    const int q_len = cu_q[seq + 1] - tok0;
    const int ctx = kv_len[seq];
    const int pos0 = ctx - q_len;                 // position of the portion's first token
    const int rows = min(PF_BM, q_len - row0);    // valid query rows of this tile
    const int* table = block_table + (size_t)seq * bt_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;

    // key range of the tile: up to the last row's position; from the first row's window start
    const int last_pos = pos0 + row0 + rows - 1;
    int key_lo = 0;
    if (window > 0) key_lo = max(0, pos0 + row0 - window + 1);
    key_lo = (key_lo / PF_BN) * PF_BN;
    const int n_tiles = (last_pos + 1 - key_lo + PF_BN - 1) / PF_BN;
    // keys before the first row's window may lie in pages that were already given back
    const int key_first = window > 0 ? max(0, pos0 + row0 - window + 1) : 0;

    // ---- load Q tile (rows beyond the portion: zeros) ----
    for (int idx = threadIdx.x; idx < PF_BM * CH; idx += blockDim.x) {
        const int r = idx / CH, c = idx - r * CH;
        __nv_bfloat16* dst = sQ + sw<HD>(r, c);
        if (r < rows)
            cp_async16(dst, q + ((size_t)(tok0 + row0 + r) * n_q_heads + head) * HD + c * 8);
        else
            *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    auto load_kv = [&](int tile, int stage) {
        const int k0 = key_lo + tile * PF_BN;
        __nv_bfloat16* dK = sK + stage * PF_BN * HD;
        __nv_bfloat16* dV = sV + stage * PF_BN * HD;
        for (int idx = threadIdx.x; idx < PF_BN * CH; idx += blockDim.x) {
            const int r = idx / CH, c = idx - r * CH;
            int key = k0 + r;
            key = (key <= last_pos && key >= key_first) ? key : last_pos;   // masked later, never off the table
            const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
            const int slot = page_shift >= 0 ? key & (page_size - 1) : key - pi * page_size;
            const size_t off = (((size_t)table[pi] * n_kv_heads + kvh) * page_size + slot) * HD + c * 8;
            cp_async16(dK + sw<HD>(r, c), k_pages + off);
            cp_async16(dV + sw<HD>(r, c), v_pages + off);
        }
    };
    load_kv(0, 0);
    cp_async_commit();

    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    uint32_t qa[KS][4];
    const int qrow_a = pos0 + row0 + warp * 16 + g;   // position of this thread's rows g and g + 8
    const int qrow_b = qrow_a + 8;

    for (int tile = 0; tile < n_tiles; ++tile) {
        const int stage = tile & 1;
        if (tile + 1 < n_tiles) load_kv(tile + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (tile == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
                ldsm_x4(qa[ks], sQ + sw<HD>(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), 2 * ks + (lane >> 4)));
        }
        const __nv_bfloat16* tK = sK + stage * PF_BN * HD;
        const __nv_bfloat16* tV = sV + stage * PF_BN * HD;
        const int k0 = key_lo + tile * PF_BN;
        // whole tile beyond this warp's rows (causal) or before their windows: nothing to add
        const int warp_last = pos0 + row0 + warp * 16 + 15;
        const int warp_first = pos0 + row0 + warp * 16;
        const bool skip = k0 > warp_last || (window > 0 && k0 + PF_BN - 1 < warp_first - window + 1);
        if (!skip) {
            float s[PF_BN / 8][4];
#pragma unroll
            for (int j = 0; j < PF_BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int jp = 0; jp < PF_BN / 16; ++jp) {
                    uint32_t b[4];
                    const int mi = lane >> 3;
                    ldsm_x4(b, tK + sw<HD>(16 * jp + (lane & 7) + 8 * (mi >> 1), 2 * ks + (mi & 1)));
                    pf_mma(s[2 * jp], qa[ks], b[0], b[1]);
                    pf_mma(s[2 * jp + 1], qa[ks], b[2], b[3]);
                }
            }
            // Scores stay unscaled; the scale rides in the exponent's FMA: p = 2^(s * scale - m).
            // Only tiles that touch the diagonal or a window's edge need the mask.
            const bool need_mask = k0 + PF_BN - 1 > warp_first || (window > 0 && k0 < warp_last - window + 1);
            if (need_mask) {
#pragma unroll
                for (int j = 0; j < PF_BN / 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = k0 + 8 * j + 2 * t + (e & 1);
                        const int qp = (e < 2) ? qrow_a : qrow_b;
                        bool ok = key <= qp;
                        if (window > 0) ok = ok && key > qp - window;
                        if (!ok) s[j][e] = -INFINITY;
                    }
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < PF_BN / 8; ++j) {
                mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
                mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            // m0, m1: running maxima of the SCALED scores (the scale is positive)
            const float mn0 = fmaxf(m0, mx0 * scale_log2e), mn1 = fmaxf(m1, mx1 * scale_log2e);
            // a row with no visible key so far keeps max = -inf: use 0 as the reference point
            const float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
            const bool rescale = mn0 != m0 || mn1 != m1;
            const float corr0 = pf_exp2(m0 - ref0), corr1 = pf_exp2(m1 - ref1);
            m0 = mn0; m1 = mn1;
            float rs0 = 0.f, rs1 = 0.f;
            uint32_t pa[PF_BN / 16][4];
#pragma unroll
            for (int j = 0; j < PF_BN / 8; ++j) {
                const float p0 = pf_exp2(fmaf(s[j][0], scale_log2e, -ref0)), p1 = pf_exp2(fmaf(s[j][1], scale_log2e, -ref0));
                const float p2 = pf_exp2(fmaf(s[j][2], scale_log2e, -ref1)), p3 = pf_exp2(fmaf(s[j][3], scale_log2e, -ref1));
                rs0 += p0 + p1;
                rs1 += p2 + p3;
                const __nv_bfloat162 r01 = __floats2bfloat162_rn(p0, p1), r23 = __floats2bfloat162_rn(p2, p3);
                pa[j >> 1][(j & 1) * 2 + 0] = *reinterpret_cast<const uint32_t*>(&r01);
                pa[j >> 1][(j & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&r23);
            }
            l0 = l0 * corr0 + rs0;
            l1 = l1 * corr1 + rs1;
            if (__any_sync(0xffffffffu, rescale)) {      // the maxima settle early: most tiles skip this
#pragma unroll
                for (int j = 0; j < NT_O; ++j) {
                    o[j][0] *= corr0; o[j][1] *= corr0; o[j][2] *= corr1; o[j][3] *= corr1;
                }
            }
#pragma unroll
            for (int ks = 0; ks < PF_BN / 16; ++ks) {
#pragma unroll
                for (int dp = 0; dp < NT_O / 2; ++dp) {
                    uint32_t b[4];
                    const int mi = lane >> 3;
                    ldsm_x4_trans(b, tV + sw<HD>(16 * ks + (lane & 7) + 8 * (mi & 1), 2 * dp + (mi >> 1)));
                    pf_mma(o[2 * dp], pa[ks], b[0], b[1]);
                    pf_mma(o[2 * dp + 1], pa[ks], b[2], b[3]);
                }
            }
        }
        __syncthreads();   // everyone is done with this stage before it is refilled
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    const int ra = row0 + warp * 16 + g, rb = ra + 8;
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
        const int d = 8 * j + 2 * t;
        if (ra < q_len) {
            __nv_bfloat162 v = __floats2bfloat162_rn(o[j][0] * inv0, o[j][1] * inv0);
            *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(tok0 + ra) * n_q_heads + head) * HD + d) = v;
        }
        if (rb < q_len) {
            __nv_bfloat162 v = __floats2bfloat162_rn(o[j][2] * inv1, o[j][3] * inv1);
            *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(tok0 + rb) * n_q_heads + head) * HD + d) = v;
        }
    }
}

template <int HD> static int launch_prefill(const void* q, const void* k_pages, const void* v_pages, void* out,
                                            const int* tile_seq, const int* tile_row0, int n_tiles,
                                            const int* cu_q, const int* kv_len, const int* block_table,
                                            int bt_stride, int n_q_heads, int n_kv_heads, int page_size,
                                            int window, float scale_log2e, cudaStream_t stream) {
    const size_t smem = (size_t)(PF_BM + 4 * PF_BN) * HD * sizeof(__nv_bfloat16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long long blocks = (long long)n_tiles * n_q_heads;
    if (blocks > 0x7fffffffLL) return NI_ERR_UNSUPPORTED_SIZE;
    dim3 grid((unsigned)blocks);
    attention_prefill_kernel<HD><<<grid, PF_WARPS * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
        (__nv_bfloat16*)out, tile_seq, tile_row0, cu_q, kv_len, block_table, bt_stride, n_q_heads,
        n_kv_heads, page_size, window, scale_log2e);
    NI_RETURN_LAUNCH_STATUS();
}

// tile_seq / tile_row0: int32 [n_tiles] on the device: request index and first query row (a
// multiple of 128 within the request's portion) of each tile.
NI_EXPORT int ni_attention_prefill(const void* q, const void* k_pages, const void* v_pages, void* out,
                                   const int* tile_seq, const int* tile_row0, int n_tiles, const int* cu_q,
                                   const int* kv_len, const int* block_table, int bt_stride, int n_q_heads,
                                   int n_kv_heads, int head_dim, int page_size, int window, float scale,
                                   cudaStream_t stream) {
    if (n_tiles <= 0) return NI_OK;
    if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads || page_size <= 0)
        return NI_ERR_BAD_ARGUMENT;
    const float sl = scale * 1.4426950408889634f;
#define GO(HD) return launch_prefill<HD>(q, k_pages, v_pages, out, tile_seq, tile_row0, n_tiles, cu_q, kv_len, \
                                         block_table, bt_stride, n_q_heads, n_kv_heads, page_size, window, sl, stream)
    switch (head_dim) {
        case 16: GO(16);
        case 32: GO(32);
        case 48: GO(48);
        case 64: GO(64);
        case 80: GO(80);
        case 96: GO(96);
        case 112: GO(112);
        case 128: GO(128);
        default: return NI_ERR_UNSUPPORTED_SIZE;
    }
#undef GO
}
