// Split-K grouped-query attention for single query tokens over the paged bfloat16 cache.
//
// One thread block per (query token, kv head, split).  The G = Hq / Hkv query heads that
// share a kv head are the rows of one 16-row tensor-core tile (mma.sync m16n8k16, bf16 in, FP32
// accumulate), so every key and value is fetched once for all of them.  A block walks its key
// range in segments of 128 keys with two shared-memory buffers: it asks for a whole segment at
// once with cp.async - page by page through the block table, 16 bytes at a time into
// XOR-swizzled shared memory - and the next segment streams in while the current one is used,
// so the memory system always sees a whole segment in flight instead of a chain of small
// dependent loads.  Each of the 4 warps takes a quarter of a segment: scores through ldmatrix +
// MMA, softmax in FP32 (base 2), P V through ldmatrix.trans + MMA.  Warps are merged through
// shared memory; the split's (max, sum, unnormalised O) goes to a scratch buffer; the block
// that arrives last for its (token, kv head) - counted with an atomic ticket - merges the
// splits in split order and writes the bfloat16 output.  No block waits for another, and the
// merge order is fixed, so results are reproducible.
//
// The splits of a (token, kv head) merge in one of two ways.  Through global memory: partial
// results to a scratch buffer, a fence, an atomic ticket, and the last arrival reads them back.
// Or, with 2 to 8 splits (up to 16 where the blocks are few), as a thread-block cluster (template parameter CL): partial results
// written into the first block's shared memory, one cluster barrier, merged there - about 1.5 us
// less per launch (batch 8, context 3,072: 17.0 -> 15.3 us).
//
// Launched with programmatic stream serialisation (the scratch variant): block tables, positions and all cached
// keys but the token's own (which the projection kernel just before writes) are requested
// before griddepcontrol.wait, so the first segment streams in while the projection drains.
// The kernel does not itself release its dependents early: measured on the decode step, letting
// the output projection's blocks take their places while attention still runs cost a third of
// the step's time, while the same early release between the projection kernels gains 6 %.
//
// The grid does not depend on context lengths (they are read on the device), so a decode step
// can be captured in a CUDA graph and replayed as contexts grow.
//
// Reference counterpart: src/op/kernels/cuda/paged_attention_kernel.cu:111-199 (one block per
// (head, sequence), FP32 CUDA cores, all scores of a sequence in shared memory, no split).
#include <cstdlib>

#include "common.cuh"

#define DEC_WARPS 4
// A token may attend to keys that the kernel before this one writes in the same step: its own,
// and those of the tokens before it in the same short portion of a prompt.  Only keys older
// than the last DEC_FRESH_KEYS are fetched before that kernel is known to have finished; callers
// send no token here whose portion has more tokens than this.
#define DEC_FRESH_KEYS 2

__device__ __forceinline__ void mma_bf16_16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x with the hardware approximation (one MUFU instruction; about two units in the last place,
// far below the bfloat16 rounding of the probabilities it feeds); 2^-inf = 0.
__device__ __forceinline__ float dec_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void dec_ldsm_x4(uint32_t r[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void dec_ldsm_x4_trans(uint32_t r[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void dec_cp_async16(void* smem, const void* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(gmem));
}
__device__ __forceinline__ void dec_pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

__device__ __forceinline__ void dec_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void dec_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
// stores v at the shared-memory address `p` of this block's layout, in block `rank` of the cluster
__device__ __forceinline__ void dec_st_cluster(const float* p, uint32_t rank, float v) {
    uint32_t local = (uint32_t)__cvta_generic_to_shared(p), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(remote), "f"(v) : "memory");
}

// Element offset of (row, 16-byte chunk) in a tile of rows of HD bf16, chunks XOR-swizzled by row.
template <int HD> __device__ __forceinline__ int dec_sw(int row, int chunk) {
    constexpr int CH = HD / 8;
    constexpr int MASK = ((CH & -CH) - 1) & 7;
    return row * HD + ((chunk ^ (row & MASK)) << 3);
}

// One warp's share of a request to bring [p, p + bytes) into L2 (p 16-byte aligned, bytes a multiple of 16).
__device__ __forceinline__ void dec_warm(const unsigned char* p, unsigned long long bytes) {
    if (!bytes) return;
    const unsigned int n_blocks = gridDim.x * gridDim.y * gridDim.z;
    const unsigned int bid = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    constexpr unsigned int PIECE = 8192;
    const unsigned int n_pieces = (unsigned int)((bytes + PIECE - 1) / PIECE);
    for (unsigned int i = bid + (threadIdx.x & 31) * n_blocks; i < n_pieces; i += 32 * n_blocks) {
        const unsigned long long off = (unsigned long long)i * PIECE;
        const unsigned int sz = bytes - off < PIECE ? (unsigned int)(bytes - off) : PIECE;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(p + off), "r"(sz) : "memory");
    }
}

// HD: head size (64 or 128).  SEG: keys a block holds in shared memory at a time (64 per warp
// pass).  Scratch per (token, q head, split): HD + 2 floats.
// CL: the splits of one (token, kv head) are the blocks of a thread-block cluster (2 to 8 of them):
// every split writes its partial result into the shared memory of the cluster's first block, one
// cluster barrier, and that block merges them in split order - no scratch in global memory, no
// fence, no ticket.
template <int HD, int SEG, bool CL>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                        const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ token_list, const int* __restrict__ positions,
                        const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                        int bt_stride, int n_q_heads, int n_kv_heads, int page_size, int window,
                        float scale_log2e, int n_splits, float* __restrict__ scratch,
                        int* __restrict__ tickets, const unsigned char* __restrict__ warm_a, unsigned long long warm_a_bytes,
                        const unsigned char* __restrict__ warm_b, unsigned long long warm_b_bytes) {
    // Weights that the kernels after this one will read (the caller's hint, up to two regions): asked
    // into L2 now, in pieces dealt over the blocks, while this kernel - which waits on latencies
    // more than on bandwidth - leaves the memory system room.  Nothing here depends on the kernel before.
    if (threadIdx.x >= (DEC_WARPS - 1) * 32) dec_warm(warm_a, warm_a_bytes);
    constexpr int CH = HD / 8;       // 16-byte chunks per row
    constexpr int KS = HD / 16;      // k-steps over the head size
    constexpr int NT_O = HD / 8;     // output column tiles
    constexpr int WK = SEG / DEC_WARPS;   // keys per warp per segment
    static_assert(WK % 16 == 0, "keys per warp");
    extern __shared__ __align__(128) unsigned char dec_smem[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(dec_smem);    // [16][HD]
    __nv_bfloat16* sKV = sQ + 16 * HD;                                  // 2 buffers of K [SEG][HD] + V [SEG][HD]
    float* cl_slots = reinterpret_cast<float*>(sKV + 4 * SEG * HD);     // CL: [n_splits][G][HD + 2], used in the first block
    if (CL) dec_cluster_arrive();                                       // "this block runs" (waited for before the first remote store)

    const int item = blockIdx.x;             // index into token_list
    const int kvh = blockIdx.y;
    const int split = blockIdx.z;
    const int t_idx = token_list ? token_list[item] : item;
    const int pos = positions[t_idx];
    const int* table = block_table + (size_t)seq_of_token[t_idx] * bt_stride;
    const int G = n_q_heads / n_kv_heads;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_keys = pos + 1 - lo;
    // the split's key range, in whole 64-key chunks
    const int chunks_total = (n_keys + 63) / 64;
    const int chunks_per_split = (chunks_total + n_splits - 1) / n_splits;
    const int k_begin = lo + split * chunks_per_split * 64;
    const int k_end = min(pos + 1, k_begin + chunks_per_split * 64);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;

    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g + 8
    uint32_t qa[KS][4];

    // Asks for the keys and values of segment [seg0, seg0 + SEG) into buffer `buf`.  The last
    // `fresh` keys up to the token's own may be written in this very step by the kernel before
    // this one (the token's own key, and the keys of the tokens before it in a short portion of
    // a prompt); `fresh_only` selects those rows, `skip_fresh` all other rows.
    const int first_fresh = pos - DEC_FRESH_KEYS + 1;
    auto request = [&](int seg0, int buf, bool fresh_only, bool skip_fresh) {
        const int seg_keys = min(SEG, k_end - seg0);
        const int rows = ((seg_keys + 15) / 16) * 16;            // rows that MMAs may touch
        __nv_bfloat16* sK = sKV + (size_t)buf * 2 * SEG * HD;
        __nv_bfloat16* sV = sK + SEG * HD;
        // Two passes over this thread's chunks: first all page look-ups, then all copies.  In one
        // pass every copy would wait for its own look-up before the next look-up is even issued.
        constexpr int ITERS = SEG * CH / (DEC_WARPS * 32);
        int page[ITERS];
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int idx = threadIdx.x + it * DEC_WARPS * 32;
            const int r = idx / CH;
            int key = seg0 + r;
            key = key < k_end ? key : k_end - 1;                 // masked below; never off the table
            const bool need = idx < rows * CH && !((fresh_only && key < first_fresh) || (skip_fresh && key >= first_fresh));
            const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
            page[it] = need ? table[pi] : -1;
        }
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            if (page[it] < 0) continue;
            const int idx = threadIdx.x + it * DEC_WARPS * 32;
            const int r = idx / CH, c = idx - r * CH;
            int key = seg0 + r;
            key = key < k_end ? key : k_end - 1;
            const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
            const int slot = page_shift >= 0 ? key & (page_size - 1) : key - pi * page_size;
            const size_t off = (((size_t)page[it] * n_kv_heads + kvh) * page_size + slot) * HD + c * 8;
            dec_cp_async16(sK + dec_sw<HD>(r, c), k_pages + off);
            dec_cp_async16(sV + dec_sw<HD>(r, c), v_pages + off);
        }
    };

    if (k_begin < k_end) {
        // everything but the fresh keys, which the projection before us may still be writing
        request(k_begin, 0, false, true);
    }
    dec_pdl_wait();                                              // the projection has finished
    if (k_begin < k_end) {
        request(k_begin, 0, true, false);
        for (int idx = threadIdx.x; idx < 16 * CH; idx += blockDim.x) {
            const int r = idx / CH, c = idx - r * CH;
            __nv_bfloat16* dst = sQ + dec_sw<HD>(r, c);
            if (r < G)
                dec_cp_async16(dst, q + ((size_t)t_idx * n_q_heads + (size_t)kvh * G + r) * HD + c * 8);
            else
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
    asm volatile("cp.async.commit_group;\n" ::);

    int buf = 0;
    for (int seg0 = k_begin; seg0 < k_end; seg0 += SEG, buf ^= 1) {
        const int seg_keys = min(SEG, k_end - seg0);
        const int rows = ((seg_keys + 15) / 16) * 16;
        const __nv_bfloat16* sK = sKV + (size_t)buf * 2 * SEG * HD;
        const __nv_bfloat16* sV = sK + SEG * HD;
        // the next segment streams in while this one is used
        if (seg0 + SEG < k_end) request(seg0 + SEG, buf ^ 1, false, false);
        asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group 1;\n" ::);
        __syncthreads();
        if (seg0 == k_begin) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
                dec_ldsm_x4(qa[ks], sQ + dec_sw<HD>((lane & 7) + 8 * ((lane >> 3) & 1), 2 * ks + (lane >> 4)));
        }
        const int w0 = warp * WK;                                // this warp's rows of the segment
        if (w0 < seg_keys) {
            // ---- S = Q K^T for WK keys ----
            float s[WK / 8][4];
#pragma unroll
            for (int j = 0; j < WK / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int jp = 0; jp < WK / 16; ++jp) {
                if (w0 + 16 * jp < rows) {
#pragma unroll
                    for (int ks = 0; ks < KS; ++ks) {
                        uint32_t b[4];
                        const int mi = lane >> 3;
                        dec_ldsm_x4(b, sK + dec_sw<HD>(w0 + 16 * jp + (lane & 7) + 8 * (mi >> 1), 2 * ks + (mi & 1)));
                        mma_bf16_16816(s[2 * jp], qa[ks], b[0], b[1]);
                        mma_bf16_16816(s[2 * jp + 1], qa[ks], b[2], b[3]);
                    }
                }
            }
            // ---- mask, online softmax (base 2) ----
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < WK / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const bool ok = w0 + 8 * j + 2 * t + (e & 1) < seg_keys;
                    s[j][e] = ok ? s[j][e] * scale_log2e : -INFINITY;
                }
                mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
                mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite: the warp has >= 1 key
            const float corr0 = dec_exp2(m0 - mn0), corr1 = dec_exp2(m1 - mn1);
            m0 = mn0; m1 = mn1;
            float rs0 = 0.f, rs1 = 0.f;
            uint32_t pa[WK / 16][4];
#pragma unroll
            for (int j = 0; j < WK / 8; ++j) {
                // the sum runs over the bfloat16-rounded probabilities that multiply V
                const __nv_bfloat162 r01 = __floats2bfloat162_rn(dec_exp2(s[j][0] - mn0), dec_exp2(s[j][1] - mn0));
                const __nv_bfloat162 r23 = __floats2bfloat162_rn(dec_exp2(s[j][2] - mn1), dec_exp2(s[j][3] - mn1));
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
            for (int ks = 0; ks < WK / 16; ++ks) {
                if (w0 + 16 * ks < rows) {
#pragma unroll
                    for (int dp = 0; dp < NT_O / 2; ++dp) {
                        uint32_t b[4];
                        const int mi = lane >> 3;
                        dec_ldsm_x4_trans(b, sV + dec_sw<HD>(w0 + 16 * ks + (lane & 7) + 8 * (mi & 1), 2 * dp + (mi >> 1)));
                        mma_bf16_16816(o[2 * dp], pa[ks], b[0], b[1]);
                        mma_bf16_16816(o[2 * dp + 1], pa[ks], b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();   // everyone is done with this buffer before it is refilled
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    // row sums live in the 4 lanes of a row group
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // ---- merge the block's warps (fixed order); the key/value tiles are no longer needed ----
    __shared__ float sm_m[DEC_WARPS][16], sm_l[DEC_WARPS][16];
    __syncthreads();
    float (*sm_o)[16][HD + 1] = reinterpret_cast<float (*)[16][HD + 1]>(dec_smem);
    static_assert(sizeof(float) * DEC_WARPS * 16 * (HD + 1) <= sizeof(__nv_bfloat16) * (16 + 4 * SEG) * HD, "merge buffer");
    if (t == 0) { sm_m[warp][g] = m0; sm_m[warp][g + 8] = m1; sm_l[warp][g] = l0; sm_l[warp][g + 8] = l1; }
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
        const int d = 8 * j + 2 * t;
        sm_o[warp][g][d] = o[j][0]; sm_o[warp][g][d + 1] = o[j][1];
        sm_o[warp][g + 8][d] = o[j][2]; sm_o[warp][g + 8][d + 1] = o[j][3];
    }
    // the block's own stream has ended: the second region is asked for under the merges (here, where
    // the accumulators are no longer live, it costs the kernel no registers)
    if (threadIdx.x >= (DEC_WARPS - 1) * 32) dec_warm(warm_b, warm_b_bytes);
    __syncthreads();
    const size_t rec = HD + 2;
    if (CL) dec_cluster_wait();     // every block of the cluster runs: the first one's shared memory may be written
    for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
        const int row = idx / HD, d = idx - row * HD;
        float mm = sm_m[0][row];
#pragma unroll
        for (int w = 1; w < DEC_WARPS; ++w) mm = fmaxf(mm, sm_m[w][row]);
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float f = sm_m[w][row] == -INFINITY ? 0.f : dec_exp2(sm_m[w][row] - mm);
            acc += sm_o[w][row][d] * f;
            ll += sm_l[w][row] * f;
        }
        if (n_splits == 1) {   // nothing to merge with: this is the result
            out[((size_t)t_idx * n_q_heads + (size_t)kvh * G + row) * HD + d] = __float2bfloat16_rn(acc / ll);
            continue;
        }
        if (CL) {
            const float* dst = cl_slots + ((size_t)split * G + row) * rec;
            dec_st_cluster(dst + 2 + d, 0, acc);
            if (d == 0) { dec_st_cluster(dst, 0, mm); dec_st_cluster(dst + 1, 0, ll); }
            continue;
        }
        float* dst = scratch + (((size_t)item * n_q_heads + (size_t)kvh * G + row) * n_splits + split) * rec;
        dst[2 + d] = acc;
        if (d == 0) { dst[0] = mm; dst[1] = ll; }
    }
    if (n_splits == 1) return;
    if (CL) {
        // ---- the cluster's first block merges the splits, from its own shared memory ----
        dec_cluster_arrive();   // this block's partial results are written
        dec_cluster_wait();     // ... and everyone else's
        if (split != 0) return;
    } else {
        // ---- the last block of this (token, kv head) merges the splits ----
        __shared__ int is_last;
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();   // the block's partial results (ordered before by the barrier) become visible
            int* ticket = tickets + (size_t)item * n_kv_heads + kvh;
            const int prev = atomicAdd(ticket, 1);
            is_last = prev == n_splits - 1;
            if (is_last) *ticket = 0;   // ready for the next launch
        }
        __syncthreads();
        if (!is_last) return;
        __threadfence();
    }
    for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
        const int row = idx / HD, d = idx - row * HD;
        // the splits' records of this row: rec floats apart in the scratch, G * rec apart in the cluster's slots
        const float* src = CL ? cl_slots + (size_t)row * rec
                              : scratch + ((size_t)item * n_q_heads + (size_t)kvh * G + row) * n_splits * rec;
        const size_t step = CL ? (size_t)G * rec : rec;
        // Eight splits at a time: their 24 loads are issued together (one after the other, each
        // followed by its use, they cost a memory round trip per split), then merged in split order.
        float mm = -INFINITY, acc = 0.f, ll = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += 8) {
            float ms[8], ls[8], as[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool ok = s0 + j < n_splits;
                const float* r = src + (size_t)(ok ? s0 + j : s0) * step;
                ms[j] = CL ? r[0] : __ldcg(r);
                ls[j] = CL ? r[1] : __ldcg(r + 1);
                as[j] = CL ? r[2 + d] : __ldcg(r + 2 + d);
                if (!ok) ms[j] = -INFINITY;
            }
            float cm = mm;
#pragma unroll
            for (int j = 0; j < 8; ++j) cm = fmaxf(cm, ms[j]);
            const float f0 = mm == -INFINITY ? 0.f : dec_exp2(mm - cm);
            acc *= f0;
            ll *= f0;
            mm = cm;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float f = ms[j] == -INFINITY ? 0.f : dec_exp2(ms[j] - cm);
                acc += as[j] * f;
                ll += ls[j] * f;
            }
        }
        out[((size_t)t_idx * n_q_heads + (size_t)kvh * G + row) * HD + d] = __float2bfloat16_rn(acc / ll);
    }
}

// ---- the balanced variant: keys dealt evenly over a fixed set of blocks ---------------------------
//
// With many (token, kv head) pairs - more than about one per SM - no split count fills the GPU
// evenly: 256 pairs are 1.7 fat blocks per SM, or 3.5 lean ones in two splits, and requests of
// different lengths make it worse (every pair is cut into the same number of splits, whatever its
// length).  Here the grid is fixed: gridDim.x blocks per kv head, three resident per SM in all.
// For one kv head the keys of all tokens, in 64-key chunks, form one long line, and every block
// takes an equal stretch of it: the tail of a token that an earlier block began, whole tokens,
// the head of a token that the next block continues.  A token that lies inside one block is
// finished there.  A token that spans blocks leaves one partial result per block in a scratch
// slot (a block has two: one for a stretch that continues a token, one for a stretch that begins
// one), and the block that arrives last for it (atomic ticket) merges them in the order of the
// line.  The chunk counts come from the positions on the device (a scan in shared memory by every
// block), so the launch does not depend on the context lengths and can be replayed from a graph.
#define DEC_BAL_MAX_ITEMS 1024

template <int HD, int SEG>
__global__ void __launch_bounds__(DEC_WARPS * 32, 3)
attention_decode_balanced_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                                 const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out,
                                 const int* __restrict__ token_list, int n_items, const int* __restrict__ positions,
                                 const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                 int bt_stride, int n_q_heads, int n_kv_heads, int page_size, int window,
                                 float scale_log2e, float* __restrict__ scratch, int* __restrict__ tickets,
                                 const unsigned char* __restrict__ warm_a, unsigned long long warm_a_bytes,
                                 const unsigned char* __restrict__ warm_b, unsigned long long warm_b_bytes) {
    if (threadIdx.x >= (DEC_WARPS - 1) * 32) dec_warm(warm_a, warm_a_bytes);
    constexpr int CH = HD / 8;
    constexpr int KS = HD / 16;
    constexpr int NT_O = HD / 8;
    constexpr int WK = SEG / DEC_WARPS;
    extern __shared__ __align__(128) unsigned char dec_smem[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(dec_smem);
    __nv_bfloat16* sKV = sQ + 16 * HD;
    __shared__ int s_prefix[DEC_BAL_MAX_ITEMS + 1];      // chunks before item i; [n_items] = all chunks
    __shared__ int s_warp_sum[DEC_WARPS];
    __shared__ int s_first_item;
    __shared__ float sm_m[DEC_WARPS][16], sm_l[DEC_WARPS][16];
    __shared__ int is_last;

    const int kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int G = n_q_heads / n_kv_heads;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    const size_t rec = HD + 2;

    // ---- every token's chunk count, and their running sum (step metadata: not written by the kernel before) ----
    int running = 0;
    for (int base = 0; base < n_items; base += DEC_WARPS * 32) {
        const int i = base + threadIdx.x;
        int c = 0;
        if (i < n_items) {
            const int pos = positions[token_list ? token_list[i] : i];
            const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
            c = (pos + 1 - lo + 63) >> 6;
        }
        int incl = c;                                     // inclusive scan inside the warp
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += v;
        }
        if (lane == 31) s_warp_sum[warp] = incl;
        __syncthreads();
        int before = running;
        for (int w = 0; w < warp; ++w) before += s_warp_sum[w];
        if (i < n_items) s_prefix[i] = before + incl - c;
        int all = 0;
        for (int w = 0; w < DEC_WARPS; ++w) all += s_warp_sum[w];
        running += all;
        __syncthreads();
    }
    if (threadIdx.x == 0) s_prefix[n_items] = running;
    const int total = running;
    const int quota = (total + (int)gridDim.x - 1) / (int)gridDim.x;
    const int g_begin = (int)blockIdx.x * quota;
    const int g_end = min(total, g_begin + quota);
    // (asking for old keys before this wait, as the kernel above does, changed nothing here: the scan
    // already covers the projection's tail)
    dec_pdl_wait();                                      // the projection has finished: queries and fresh keys are there
    if (g_begin >= g_end) return;                        // (block-uniform) more blocks than chunks
    __syncthreads();
    // the token whose chunks contain g_begin
    for (int i = threadIdx.x; i < n_items; i += DEC_WARPS * 32)
        if (s_prefix[i] <= g_begin && g_begin < s_prefix[i + 1]) s_first_item = i;
    __syncthreads();

    int gpos = g_begin;
    for (int item = s_first_item; gpos < g_end; ++item) {
        const int pre = s_prefix[item], c_item = s_prefix[item + 1] - pre;
        const int c0 = gpos - pre;
        const int take = min(g_end - gpos, c_item - c0);
        gpos += take;
        const int t_idx = token_list ? token_list[item] : item;
        const int pos = positions[t_idx];
        const int* table = block_table + (size_t)seq_of_token[t_idx] * bt_stride;
        const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        const int k_begin = lo + c0 * 64;
        const int k_end = min(pos + 1, k_begin + take * 64);

        float o[NT_O][4];
#pragma unroll
        for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
        uint32_t qa[KS][4];

        auto request = [&](int seg0, int buf) {
            const int seg_keys = min(SEG, k_end - seg0);
            const int rows = ((seg_keys + 15) / 16) * 16;
            __nv_bfloat16* sK = sKV + (size_t)buf * 2 * SEG * HD;
            __nv_bfloat16* sV = sK + SEG * HD;
            constexpr int ITERS = SEG * CH / (DEC_WARPS * 32);
            int page[ITERS];
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                const int idx = threadIdx.x + it * DEC_WARPS * 32;
                const int r = idx / CH;
                int key = seg0 + r;
                key = key < k_end ? key : k_end - 1;
                const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
                page[it] = idx < rows * CH ? table[pi] : -1;
            }
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                if (page[it] < 0) continue;
                const int idx = threadIdx.x + it * DEC_WARPS * 32;
                const int r = idx / CH, c = idx - r * CH;
                int key = seg0 + r;
                key = key < k_end ? key : k_end - 1;
                const int pi = page_shift >= 0 ? key >> page_shift : key / page_size;
                const int slot = page_shift >= 0 ? key & (page_size - 1) : key - pi * page_size;
                const size_t off = (((size_t)page[it] * n_kv_heads + kvh) * page_size + slot) * HD + c * 8;
                dec_cp_async16(sK + dec_sw<HD>(r, c), k_pages + off);
                dec_cp_async16(sV + dec_sw<HD>(r, c), v_pages + off);
            }
        };

        __syncthreads();      // the buffers and the merge area of the token before are no longer in use
        request(k_begin, 0);
        for (int idx = threadIdx.x; idx < 16 * CH; idx += blockDim.x) {
            const int r = idx / CH, c = idx - r * CH;
            __nv_bfloat16* dst = sQ + dec_sw<HD>(r, c);
            if (r < G)
                dec_cp_async16(dst, q + ((size_t)t_idx * n_q_heads + (size_t)kvh * G + r) * HD + c * 8);
            else
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("cp.async.commit_group;\n" ::);

        int buf = 0;
        for (int seg0 = k_begin; seg0 < k_end; seg0 += SEG, buf ^= 1) {
            const int seg_keys = min(SEG, k_end - seg0);
            const int rows = ((seg_keys + 15) / 16) * 16;
            const __nv_bfloat16* sK = sKV + (size_t)buf * 2 * SEG * HD;
            const __nv_bfloat16* sV = sK + SEG * HD;
            if (seg0 + SEG < k_end) request(seg0 + SEG, buf ^ 1);
            asm volatile("cp.async.commit_group;\n" ::);
            asm volatile("cp.async.wait_group 1;\n" ::);
            __syncthreads();
            if (seg0 == k_begin) {
#pragma unroll
                for (int ks = 0; ks < KS; ++ks)
                    dec_ldsm_x4(qa[ks], sQ + dec_sw<HD>((lane & 7) + 8 * ((lane >> 3) & 1), 2 * ks + (lane >> 4)));
            }
            const int w0 = warp * WK;
            if (w0 < seg_keys) {
                float sc[WK / 8][4];
#pragma unroll
                for (int j = 0; j < WK / 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
                for (int jp = 0; jp < WK / 16; ++jp) {
                    if (w0 + 16 * jp < rows) {
#pragma unroll
                        for (int ks = 0; ks < KS; ++ks) {
                            uint32_t b[4];
                            const int mi = lane >> 3;
                            dec_ldsm_x4(b, sK + dec_sw<HD>(w0 + 16 * jp + (lane & 7) + 8 * (mi >> 1), 2 * ks + (mi & 1)));
                            mma_bf16_16816(sc[2 * jp], qa[ks], b[0], b[1]);
                            mma_bf16_16816(sc[2 * jp + 1], qa[ks], b[2], b[3]);
                        }
                    }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int j = 0; j < WK / 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const bool ok = w0 + 8 * j + 2 * t + (e & 1) < seg_keys;
                        sc[j][e] = ok ? sc[j][e] * scale_log2e : -INFINITY;
                    }
                    mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
                    mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
                }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
                const float corr0 = dec_exp2(m0 - mn0), corr1 = dec_exp2(m1 - mn1);
                m0 = mn0; m1 = mn1;
                float rs0 = 0.f, rs1 = 0.f;
                uint32_t pa[WK / 16][4];
#pragma unroll
                for (int j = 0; j < WK / 8; ++j) {
                    const __nv_bfloat162 r01 = __floats2bfloat162_rn(dec_exp2(sc[j][0] - mn0), dec_exp2(sc[j][1] - mn0));
                    const __nv_bfloat162 r23 = __floats2bfloat162_rn(dec_exp2(sc[j][2] - mn1), dec_exp2(sc[j][3] - mn1));
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
#pragma unroll
                for (int ks = 0; ks < WK / 16; ++ks) {
                    if (w0 + 16 * ks < rows) {
#pragma unroll
                        for (int dp = 0; dp < NT_O / 2; ++dp) {
                            uint32_t b[4];
                            const int mi = lane >> 3;
                            dec_ldsm_x4_trans(b, sV + dec_sw<HD>(w0 + 16 * ks + (lane & 7) + 8 * (mi & 1), 2 * dp + (mi >> 1)));
                            mma_bf16_16816(o[2 * dp], pa[ks], b[0], b[1]);
                            mma_bf16_16816(o[2 * dp + 1], pa[ks], b[2], b[3]);
                        }
                    }
                }
            }
            __syncthreads();
        }
        asm volatile("cp.async.wait_group 0;\n" ::);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

        // ---- merge the block's warps (fixed order) ----
        __syncthreads();
        float (*sm_o)[16][HD + 1] = reinterpret_cast<float (*)[16][HD + 1]>(dec_smem);
        static_assert(sizeof(float) * DEC_WARPS * 16 * (HD + 1) <= sizeof(__nv_bfloat16) * (16 + 4 * SEG) * HD, "merge buffer");
        if (t == 0) { sm_m[warp][g] = m0; sm_m[warp][g + 8] = m1; sm_l[warp][g] = l0; sm_l[warp][g + 8] = l1; }
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
            const int d = 8 * j + 2 * t;
            sm_o[warp][g][d] = o[j][0]; sm_o[warp][g][d + 1] = o[j][1];
            sm_o[warp][g + 8][d] = o[j][2]; sm_o[warp][g + 8][d + 1] = o[j][3];
        }
        __syncthreads();
        // where this token's stretches lie on the line of blocks
        const int first_block = pre / quota, last_block = (pre + c_item - 1) / quota;
        const int n_parts = last_block - first_block + 1;
        // a block's two slots: 0 for a stretch that continues a token, 1 for one that begins a token
        float* my_slot = scratch + ((((size_t)kvh * gridDim.x + blockIdx.x) * 2 + (c0 == 0 ? 1 : 0)) * G) * rec;
        for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
            const int row = idx / HD, d = idx - row * HD;
            float mm = sm_m[0][row];
#pragma unroll
            for (int w = 1; w < DEC_WARPS; ++w) mm = fmaxf(mm, sm_m[w][row]);
            float acc = 0.f, ll = 0.f;
#pragma unroll
            for (int w = 0; w < DEC_WARPS; ++w) {
                const float f = sm_m[w][row] == -INFINITY ? 0.f : dec_exp2(sm_m[w][row] - mm);
                acc += sm_o[w][row][d] * f;
                ll += sm_l[w][row] * f;
            }
            if (n_parts == 1) {
                out[((size_t)t_idx * n_q_heads + (size_t)kvh * G + row) * HD + d] = __float2bfloat16_rn(acc / ll);
                continue;
            }
            float* dst = my_slot + (size_t)row * rec;
            dst[2 + d] = acc;
            if (d == 0) { dst[0] = mm; dst[1] = ll; }
        }
        if (n_parts == 1) continue;
        // ---- the last block to arrive for this token merges its stretches, in the order of the line ----
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            int* ticket = tickets + (size_t)item * n_kv_heads + kvh;
            const int prev = atomicAdd(ticket, 1);
            is_last = prev == n_parts - 1;
            if (is_last) *ticket = 0;
        }
        __syncthreads();
        if (!is_last) continue;
        __threadfence();
        for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
            const int row = idx / HD, d = idx - row * HD;
            float mm = -INFINITY, acc = 0.f, ll = 0.f;
            for (int s0 = 0; s0 < n_parts; s0 += 8) {
                float ms[8], ls[8], as[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const bool ok = s0 + j < n_parts;
                    const int part = ok ? s0 + j : s0;
                    // part 0 began the token in block first_block (slot 1); the others continue it (slot 0)
                    const float* r = scratch + ((((size_t)kvh * gridDim.x + first_block + part) * 2 + (part == 0 ? 1 : 0)) * G + row) * rec;
                    ms[j] = __ldcg(r);
                    ls[j] = __ldcg(r + 1);
                    as[j] = __ldcg(r + 2 + d);
                    if (!ok) ms[j] = -INFINITY;
                }
                float cm = mm;
#pragma unroll
                for (int j = 0; j < 8; ++j) cm = fmaxf(cm, ms[j]);
                const float f0 = mm == -INFINITY ? 0.f : dec_exp2(mm - cm);
                acc *= f0;
                ll *= f0;
                mm = cm;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float f = ms[j] == -INFINITY ? 0.f : dec_exp2(ms[j] - cm);
                    acc += as[j] * f;
                    ll += ls[j] * f;
                }
            }
            out[((size_t)t_idx * n_q_heads + (size_t)kvh * G + row) * HD + d] = __float2bfloat16_rn(acc / ll);
        }
    }
    if (threadIdx.x >= (DEC_WARPS - 1) * 32) dec_warm(warm_b, warm_b_bytes);
}

// Blocks per kv head of the balanced kernel: three resident per SM, shared among the kv heads.
static int dec_balanced_blocks(int n_kv_heads) {
    const int b = (3 * ni_sm_count()) / n_kv_heads;
    return b < 1 ? 1 : b;
}

template <int HD, int SEG>
static int launch_decode_balanced(const void* q, const void* k_pages, const void* v_pages, void* out,
                                  const int* token_list, int n_items, const int* positions, const int* seq_of_token,
                                  const int* block_table, int bt_stride, int n_q_heads, int n_kv_heads, int page_size,
                                  int window, float scale_log2e, float* scratch, int* tickets, const void* warm_a,
                                  unsigned long long warm_a_bytes, const void* warm_b, unsigned long long warm_b_bytes,
                                  cudaStream_t stream) {
    const size_t smem = (size_t)(16 + 4 * SEG) * HD * sizeof(__nv_bfloat16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_balanced_kernel<HD, SEG>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(dec_balanced_blocks(n_kv_heads), n_kv_heads);
    cfg.blockDim = dim3(DEC_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_decode_balanced_kernel<HD, SEG>, (const __nv_bfloat16*)q,
                                       (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
                                       (__nv_bfloat16*)out, token_list, n_items, positions, seq_of_token, block_table,
                                       bt_stride, n_q_heads, n_kv_heads, page_size, window, scale_log2e, scratch,
                                       tickets, (const unsigned char*)warm_a, warm_a_bytes, (const unsigned char*)warm_b,
                                       warm_b_bytes);
    return e == cudaSuccess ? NI_OK : (int)e;
}

// Scratch floats of the balanced kernel: two slots per block of G x (head_dim + 2); tickets: n_items * n_kv_heads.
NI_EXPORT long long ni_attention_decode_balanced_scratch(int n_q_heads, int n_kv_heads, int head_dim) {
    if (n_kv_heads <= 0 || n_q_heads <= 0) return 0;
    return 2LL * dec_balanced_blocks(n_kv_heads) * n_kv_heads * (n_q_heads / n_kv_heads) * (head_dim + 2);
}

NI_EXPORT int ni_attention_decode_balanced(const void* q, const void* k_pages, const void* v_pages, void* out,
                                           const int* token_list, int n_items, const int* positions,
                                           const int* seq_of_token, const int* block_table, int bt_stride,
                                           int n_q_heads, int n_kv_heads, int head_dim, int page_size, int window,
                                           float scale, float* scratch, int* tickets, const void* warm_a,
                                           long long warm_a_bytes, const void* warm_b, long long warm_b_bytes,
                                           cudaStream_t stream) {
    if (n_items <= 0) return NI_OK;
    if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads || page_size <= 0 || n_kv_heads > 65535)
        return NI_ERR_BAD_ARGUMENT;
    if (warm_a_bytes < 0 || (warm_a_bytes & 15) || (warm_a_bytes && (!warm_a || ((uintptr_t)warm_a & 15)))) return NI_ERR_BAD_ARGUMENT;
    if (warm_b_bytes < 0 || (warm_b_bytes & 15) || (warm_b_bytes && (!warm_b || ((uintptr_t)warm_b & 15)))) return NI_ERR_BAD_ARGUMENT;
    if (n_q_heads / n_kv_heads > 16 || n_items > DEC_BAL_MAX_ITEMS) return NI_ERR_UNSUPPORTED_SIZE;
    const float scale_log2e = scale * 1.4426950408889634f;
    switch (head_dim) {
        case 64:
            return launch_decode_balanced<64, 128>(q, k_pages, v_pages, out, token_list, n_items, positions, seq_of_token,
                                                   block_table, bt_stride, n_q_heads, n_kv_heads, page_size, window,
                                                   scale_log2e, scratch, tickets, warm_a, (unsigned long long)warm_a_bytes,
                                                   warm_b, (unsigned long long)warm_b_bytes, stream);
        case 128:
            return launch_decode_balanced<128, 64>(q, k_pages, v_pages, out, token_list, n_items, positions, seq_of_token,
                                                   block_table, bt_stride, n_q_heads, n_kv_heads, page_size, window,
                                                   scale_log2e, scratch, tickets, warm_a, (unsigned long long)warm_a_bytes,
                                                   warm_b, (unsigned long long)warm_b_bytes, stream);
        default: return NI_ERR_UNSUPPORTED_SIZE;
    }
}

template <int HD, int SEG, bool CL>
static int launch_decode_cl(const void* q, const void* k_pages, const void* v_pages, void* out, const int* token_list,
                         int n_items, const int* positions, const int* seq_of_token, const int* block_table,
                         int bt_stride, int n_q_heads, int n_kv_heads, int page_size, int window,
                         float scale_log2e, int n_splits, float* scratch, int* tickets, const void* warm_a,
                         unsigned long long warm_a_bytes, const void* warm_b, unsigned long long warm_b_bytes,
                         cudaStream_t stream) {
    const size_t kv_smem = (size_t)(16 + 4 * SEG) * HD * sizeof(__nv_bfloat16);
    const size_t smem = kv_smem + (CL ? (size_t)n_splits * (n_q_heads / n_kv_heads) * (HD + 2) * sizeof(float) : 0);
    static size_t configured = 0;
    if (configured < smem) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD, SEG, CL>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        if (CL) {   // clusters of 9 to 16 blocks (a lone request's many splits) are beyond the portable size
            e = cudaFuncSetAttribute(attention_decode_kernel<HD, SEG, CL>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            if (e != cudaSuccess) return (int)e;
        }
        configured = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_items, n_kv_heads, n_splits);
    cfg.blockDim = dim3(DEC_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = n_splits;
    // A cluster launch is not made a programmatic dependent: clusters that start under the tail of the
    // kernel before take whatever six slots of one GPC are free at that moment, and the step got slower
    // (batch 8, context 2,048: 0.850 ms against 0.814 with the scratch merge; context 8,192: 1.27 against
    // 1.13).  Started after its predecessor, the cluster variant wins (0.804; batch 4: 0.801 -> 0.773).
    cfg.attrs = CL ? attr + 1 : attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_decode_kernel<HD, SEG, CL>, (const __nv_bfloat16*)q,
                                       (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
                                       (__nv_bfloat16*)out, token_list, positions, seq_of_token, block_table,
                                       bt_stride, n_q_heads, n_kv_heads, page_size, window, scale_log2e, n_splits,
                                       scratch, tickets, (const unsigned char*)warm_a, warm_a_bytes,
                                       (const unsigned char*)warm_b, warm_b_bytes);
    return e == cudaSuccess ? NI_OK : (int)e;
}

// The splits of a (token, kv head) merge inside a cluster when there are 2 to 8 of them and the
// partial results fit beside the key/value buffers without costing a resident block
// (DEC_CLUSTER_SLOT_BYTES), or there are so few blocks that two per SM hold them all; else through
// the scratch and the tickets.
#define DEC_CLUSTER_SLOT_BYTES 6400
static int dec_cluster_merge = 1;
NI_EXPORT int ni_attention_decode_set_cluster_merge(int on) { dec_cluster_merge = on; return NI_OK; }

template <int HD, int SEG>
static int launch_decode(const void* q, const void* k_pages, const void* v_pages, void* out, const int* token_list,
                         int n_items, const int* positions, const int* seq_of_token, const int* block_table,
                         int bt_stride, int n_q_heads, int n_kv_heads, int page_size, int window,
                         float scale_log2e, int n_splits, float* scratch, int* tickets, const void* warm_a,
                         unsigned long long warm_a_bytes, const void* warm_b, unsigned long long warm_b_bytes,
                         cudaStream_t stream) {
    const size_t slot_bytes = (size_t)n_splits * (n_q_heads / n_kv_heads) * (HD + 2) * sizeof(float);
    const bool few_blocks = (long long)n_items * n_kv_heads * n_splits <= 2LL * ni_sm_count() && slot_bytes <= 65536;
    if (dec_cluster_merge && n_splits >= 2 && ((n_splits <= 8 && slot_bytes <= DEC_CLUSTER_SLOT_BYTES) || (n_splits <= 16 && few_blocks)))
        return launch_decode_cl<HD, SEG, true>(q, k_pages, v_pages, out, token_list, n_items, positions, seq_of_token,
                                               block_table, bt_stride, n_q_heads, n_kv_heads, page_size, window,
                                               scale_log2e, n_splits, scratch, tickets, warm_a, warm_a_bytes, warm_b,
                                               warm_b_bytes, stream);
    return launch_decode_cl<HD, SEG, false>(q, k_pages, v_pages, out, token_list, n_items, positions, seq_of_token,
                                            block_table, bt_stride, n_q_heads, n_kv_heads, page_size, window,
                                            scale_log2e, n_splits, scratch, tickets, warm_a, warm_a_bytes, warm_b,
                                            warm_b_bytes, stream);
}

// Scratch floats needed: n_items * n_q_heads * n_splits * (head_dim + 2); tickets: n_items * n_kv_heads
// ints, zero before the first launch (the kernel leaves them zero).
NI_EXPORT int ni_attention_decode_fresh_keys() { return DEC_FRESH_KEYS; }

NI_EXPORT int ni_attention_decode(const void* q, const void* k_pages, const void* v_pages, void* out,
                                  const int* token_list, int n_items, const int* positions,
                                  const int* seq_of_token, const int* block_table, int bt_stride,
                                  int n_q_heads, int n_kv_heads, int head_dim, int page_size, int window,
                                  float scale, int n_splits, float* scratch, int* tickets,
                                  const void* warm_a, long long warm_a_bytes, const void* warm_b,
                                  long long warm_b_bytes, cudaStream_t stream) {
    if (n_items <= 0) return NI_OK;
    if (warm_a_bytes < 0 || (warm_a_bytes & 15) || (warm_a_bytes && (!warm_a || ((uintptr_t)warm_a & 15)))) return NI_ERR_BAD_ARGUMENT;
    if (warm_b_bytes < 0 || (warm_b_bytes & 15) || (warm_b_bytes && (!warm_b || ((uintptr_t)warm_b & 15)))) return NI_ERR_BAD_ARGUMENT;
    if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads || page_size <= 0 || n_splits <= 0 ||
        n_splits > 65535 || n_kv_heads > 65535)
        return NI_ERR_BAD_ARGUMENT;
    if (n_q_heads / n_kv_heads > 16) return NI_ERR_UNSUPPORTED_SIZE;
    const float scale_log2e = scale * 1.4426950408889634f;
    switch (head_dim) {
        case 64:
            // while all blocks fit the GPU at 3 per SM: fat blocks with 128-key buffers; beyond that
            // (large batches with one block per token and kv head, middle batches in two or three
            // splits): 64-key buffers, so that 4 fit an SM and 512 to 592 blocks are still one wave
            if ((long long)n_items * n_kv_heads * n_splits <= 3LL * ni_sm_count())
                return launch_decode<64, 128>(q, k_pages, v_pages, out, token_list, n_items, positions, seq_of_token,
                                              block_table, bt_stride, n_q_heads, n_kv_heads, page_size, window,
                                              scale_log2e, n_splits, scratch, tickets, warm_a, (unsigned long long)warm_a_bytes, warm_b,
                                              (unsigned long long)warm_b_bytes, stream);
            return launch_decode<64, 64>(q, k_pages, v_pages, out, token_list, n_items, positions, seq_of_token,
                                          block_table, bt_stride, n_q_heads, n_kv_heads, page_size, window,
                                          scale_log2e, n_splits, scratch, tickets, warm_a, (unsigned long long)warm_a_bytes, warm_b,
                                              (unsigned long long)warm_b_bytes, stream);
        case 128:
            return launch_decode<128, 64>(q, k_pages, v_pages, out, token_list, n_items, positions, seq_of_token,
                                           block_table, bt_stride, n_q_heads, n_kv_heads, page_size, window,
                                           scale_log2e, n_splits, scratch, tickets, warm_a, (unsigned long long)warm_a_bytes, warm_b,
                                              (unsigned long long)warm_b_bytes, stream);
        default: return NI_ERR_UNSUPPORTED_SIZE;
    }
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
                               scale, n_splits, noalloc_partials_addr[dev], noalloc_tickets_addr[dev], nullptr, 0, nullptr, 0, stream);
}
