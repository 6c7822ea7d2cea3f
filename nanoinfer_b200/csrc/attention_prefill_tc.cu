// Causal grouped-query attention for portions of prompts over the paged bfloat16 cache, on the
// fifth-generation tensor cores: S = Q K^T and O += P V are tcgen05.mma instructions with their
// accumulators in tensor memory; Q, K and V tiles come into 128-byte-swizzled shared memory by TMA
// (one box per cache page and kv head: a page's keys of one head are contiguous); the softmax
// runs in FP32 on CUDA cores, two threads per query row, between the two products.
//
// One block works on 128 query rows of one request for TWO query heads that share a kv head
// (streams 0 and 1).  Both streams use the same K/V tiles, and while the softmax warps of one
// stream turn its scores into probabilities the tensor core runs the other stream's products.
//
//   warp 0      TMA: Q once, then K and V tiles through rings of shared-memory stages
//   warp 1      issues every MMA and commits it to mbarriers; owns the tensor memory
//   warps 2-9   softmax of stream 0: two warps per quarter of the 128 TMEM lanes (= rows), each with
//               half of a tile's columns
//   warps 10-17 softmax of stream 1
//
// Tensor memory (512 columns).  The A operand of P V is read from tensor memory, where the softmax
// threads leave the probabilities as bfloat16 pairs.  64-wide heads: scores of stream s in columns
// [128 s, +128), probabilities in [256 + 64 s, +64), outputs in [384 + 64 s, +64); since scores and
// probabilities do not share columns, the scores of the next tile are computed while the
// exponentials of this one run, and no product is on a stream's critical path.  128-wide heads:
// the probabilities overwrite the scores, outputs in [256 + 128 s, +128).
//
// The unit that computes exponentials bounds a tile's time (128 x 128 of them per stream against
// about 600 tensor-core cycles), so the two streams take turns at it instead of sharing it.
//
// The running maximum of a row is only raised when it grows by more than 8 (a factor 256 in
// the probabilities, harmless in FP32 sums and bfloat16 products); only then is the output
// accumulator rescaled, which is rare after the first tiles.
//
// The MMA warp runs its loop with all lanes and lets one elected lane issue, so that descriptors
// and addresses stay warp-uniform values; descriptors are built once and advanced by additions.
//
// Every wait on an mbarrier is bounded (about a second) and watches a block-wide abort flag;
// a wait that runs out records a code in the error word, and the block frees its tensor memory
// and returns.
//
// Takes head sizes 64 and 128, two or more query heads per kv head, and page sizes 8 to
// 128 that divide 128; everything else is the business of attention_prefill.cu.
//
// Reference counterpart: src/op/kernels/cuda/prefill_attention_kernel.cu:321-475 (gathered FP32
// copies of K and V, the whole score tensor in global memory, two cuBLAS batched SGEMMs).
#include <cuda.h>

#include <mutex>

#include "common.cuh"

#define AT_BM 128
#define AT_BN 128
#define AT_THREADS 576
#define AT_RESCALE_STEP 8.0f


#define AT_ERR_PRODUCER 11
#define AT_ERR_MMA 12
#define AT_ERR_SOFTMAX 13

__device__ __forceinline__ uint32_t at_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(at_smem(bar)), "r"(count));
}
__device__ __forceinline__ void at_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(at_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void at_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(at_smem(bar)) : "memory");
}
// Waits for the phase of the given parity.  False if the wait ran out or another thread of the
// block gave up (the abort flag); the first to run out sets the flag and the error word.
// SLEEP: pause between tries (for the loader, which runs ahead and whose polls would only take
// issue slots from the softmax warps); the others poll in a short loop, since every hand-over
// between the MMA thread and the softmax warps is on the critical path of a tile.
// The limit in clock ticks (set by ni_attention_prefill_tc_set_wait), and a switch for the tests: with
// it the softmax warps wait once more at the end, for a phase that nothing completes.
__constant__ long long at_wait_limit = 2000000000LL;
__constant__ int at_extra_wait = 0;

template <bool SLEEP>
__device__ __forceinline__ bool at_wait_impl(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* error, int code) {
    const uint32_t addr = at_smem(bar);
    long long start = 0;
    for (int iter = 0;; ++iter) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.b32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (SLEEP) __nanosleep(200);
        if ((iter & (SLEEP ? 255 : 4095)) == (SLEEP ? 255 : 4095)) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (start == 0) start = now;
            if (now - start > at_wait_limit) {
                *abort_flag = 1;
                atomicExch(error, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* error, int code) {
    return at_wait_impl<false>(bar, parity, abort_flag, error, code);
}
__device__ __forceinline__ bool at_wait_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* error, int code) {
    return at_wait_impl<true>(bar, parity, abort_flag, error, code);
}
__device__ __forceinline__ void at_tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(at_smem(dst)), "l"(map), "r"(at_smem(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void at_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void at_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// Shared-memory descriptors, 128-byte swizzle, tiles of rows of 128 bytes (64 bf16), 8-row
// groups 1024 bytes apart.  K-major: the contraction runs along a row (Q and K for Q K^T).
// MN-major: the contraction runs down the rows (V for P V: rows are keys); `lbo` is the distance
// between the 64-column halves of a wider tile.
__device__ __forceinline__ uint64_t at_desc(const void* tile, uint32_t lbo_bytes) {
    const uint32_t addr = at_smem(tile);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// BF16 x BF16 -> FP32, M = 128, N = n; b_mn: the B operand is MN-major.
__host__ __device__ constexpr uint32_t at_idesc(int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(AT_BM >> 4) << 24);
}
__device__ __forceinline__ void at_mma_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void at_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void at_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ void at_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void at_ld32_async(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void at_ld32(uint32_t taddr, uint32_t r[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void at_st32(uint32_t taddr, const uint32_t r[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void at_st16(uint32_t taddr, const uint32_t r[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void at_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ bool at_elect() {
    uint32_t pred;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.b32 %0, 1, 0, p;\n}\n" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ float at_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t at_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct AtParams {
    __nv_bfloat16* out;            // [n_tokens, Hq * HD]
    const int* tile_seq;
    const int* tile_row0;
    const int* cu_q;
    const int* kv_len;
    const int* block_table;
    int bt_stride, n_q_heads, n_kv_heads, page_size, window;
    float scale_log2e;
    int* error;
};

template <int HD, int STAGES>
__global__ void __launch_bounds__(AT_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const AtParams p) {
    constexpr int HALVES = HD / 64;
    constexpr int HALF_BYTES = AT_BN * 128;              // a [128][64] bf16 tile: 16 KB
    constexpr int TILE_BYTES = HALVES * HALF_BYTES;      // Q of one stream, or K, or V
    // Tensor-memory columns.  With 64-wide heads there is room to keep the probabilities beside the
    // scores, so the next tile's scores are computed while this tile's exponentials run; with
    // 128-wide heads the probabilities overwrite the scores (ALIAS).
    constexpr bool ALIAS = HD > 64;
    constexpr uint32_t P_COL = ALIAS ? 0 : 256;          // + 128 s (alias) or + 64 s
    constexpr uint32_t P_STRIDE = ALIAS ? AT_BN : 64;
    constexpr uint32_t O_COL = ALIAS ? 256 : 384;
    extern __shared__ uint8_t at_smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)at_smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = base;                                   // [2 streams][HALVES][128][64]
    uint8_t* sK = sQ + 2 * TILE_BYTES;                    // [STAGES][HALVES][128][64]
    uint8_t* sV = sK + STAGES * TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + STAGES * TILE_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* k_empty = k_full + STAGES;
    uint64_t* v_full = k_empty + STAGES;
    uint64_t* v_empty = v_full + STAGES;
    uint64_t* s_full = v_empty + STAGES;                  // [2] scores of a stream are in tensor memory
    uint64_t* p_full = s_full + 2;                        // [2] its probabilities are (256 arrivals)
    uint64_t* o_done = p_full + 2;                        // [2] its P V product has finished
    uint64_t* turn = o_done + 2;                          // [2] stream s may use the exponential unit (256 arrivals)
    uint64_t* s_free = turn + 2;                          // [2] its scores are in registers (256 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // row maxima (per tile) and row sums (at the end) that the two halves of a row exchange
    float (*row_max)[2][2][AT_BM] = reinterpret_cast<float (*)[2][2][AT_BM]>(tmem_slot + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- the tile's place ----
    // Blocks are numbered tile-major: all head pairs of the tile with the most keys first, then all
    // of the next one.  The hardware hands blocks out in the order of their numbers, so this is
    // "longest job first" over the whole launch (with the tiles on the grid's fast axis every head
    // pair's light tiles came before the next pair's heavy ones: 2,048 tokens took 25 tile-times
    // of the heaviest block's 16, against 16 to 18 this way).
    const int pairs = p.n_kv_heads * ((p.n_q_heads / p.n_kv_heads + 1) / 2);
    const int tile_index = blockIdx.x / pairs, pair_index = blockIdx.x - tile_index * pairs;
    const int seq = p.tile_seq[tile_index];
    const int row0 = p.tile_row0[tile_index];
    const int q_begin = p.cu_q[seq];
    const int q_len = p.cu_q[seq + 1] - q_begin;
    const int kvl = p.kv_len[seq];
    const int kv_start = kvl - q_len;                     // position of the request's first query row
    const int rows = min(AT_BM, q_len - row0);
    const int first_pos = kv_start + row0, last_pos = first_pos + rows - 1;
    const int j_end = last_pos / AT_BN + 1;
    const int j_begin = p.window > 0 ? max(0, first_pos - p.window + 1) / AT_BN : 0;
    const int n_tiles = j_end - j_begin;
    const int G = p.n_q_heads / p.n_kv_heads;
    // A kv head's group of query heads is cut into blocks of two (the two streams).  The last
    // block of an odd group has one head left: its second stream runs that head again, so that
    // the streams' hand-offs stay as they are, and stores nothing.
    const int blocks_per_kv = (G + 1) / 2;
    const int kvh = pair_index / blocks_per_kv;
    const int first = 2 * (pair_index - kvh * blocks_per_kv);
    const int head0 = kvh * G + first;
    const int head1 = first + 1 < G ? head0 + 1 : head0;

    if (threadIdx.x == 0) {
        at_mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            at_mbar_init(&k_full[s], 1); at_mbar_init(&k_empty[s], 1);
            at_mbar_init(&v_full[s], 1); at_mbar_init(&v_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            at_mbar_init(&s_full[s], 1); at_mbar_init(&p_full[s], 256); at_mbar_init(&o_done[s], 1);
            at_mbar_init(&turn[s], 256); at_mbar_init(&s_free[s], 256);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_v) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(at_smem(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    at_fence_before();
    __syncthreads();
    at_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer: lane 0 waits and announces the bytes, lane g copies page g of a tile ----
        if (lane == 0) {
            at_mbar_expect_tx(q_full, 2 * TILE_BYTES);
            for (int s = 0; s < 2; ++s)
                for (int h = 0; h < HALVES; ++h)
                    at_tma_2d(sQ + s * TILE_BYTES + h * HALF_BYTES, &map_q, (s ? head1 : head0) * HD + h * 64, q_begin + row0, q_full);
        }
        const int* table = p.block_table + (size_t)seq * p.bt_stride;
        const int pages_held = (kvl + p.page_size - 1) / p.page_size;
        const int pages_per_tile = AT_BN / p.page_size;      // at most 16
        const int page_bytes = p.page_size * 128;
        // first cache row of this lane's page of tile i; pages past the request's own hold keys
        // that every row masks: any page will do
        auto row_of_page = [&](int i) {
            const int idx = (j_begin + i) * pages_per_tile + lane;
            int page = (lane < pages_per_tile && i < n_tiles && idx < pages_held) ? table[idx] : 0;
            page = page < 0 ? 0 : page;
            return (page * p.n_kv_heads + kvh) * p.page_size;
        };
        int y_next = row_of_page(0);
        int issued = 0;
        for (int i = 0; i < n_tiles; ++i) {
            const int stage = i % STAGES;
            const uint32_t phase = (uint32_t)(i / STAGES) & 1u;
            const int y = y_next;
            y_next = row_of_page(i + 1);                      // in flight while this tile's stage is awaited
            bool ok = true;
            for (int kv = 0; kv < 2 && ok; ++kv) {
                uint64_t* full = kv == 0 ? &k_full[stage] : &v_full[stage];
                uint64_t* empty = kv == 0 ? &k_empty[stage] : &v_empty[stage];
                uint8_t* dst = (kv == 0 ? sK : sV) + stage * TILE_BYTES;
                const CUtensorMap* map = kv == 0 ? &map_k : &map_v;
                if (lane == 0) {
                    ok = at_wait_relaxed(empty, phase ^ 1, abort_flag, p.error, AT_ERR_PRODUCER);
                    if (ok) at_mbar_expect_tx(full, TILE_BYTES);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (ok && lane < pages_per_tile)
                    for (int h = 0; h < HALVES; ++h)
                        at_tma_2d(dst + h * HALF_BYTES + lane * page_bytes, map, h * 64, y, full);
            }
            if (!ok) break;
            issued = i + 1;
        }
        // copies still in flight must land before the block may end
        if (lane == 0)
            for (int i = max(0, issued - STAGES); i < issued; ++i) {
                at_wait(&k_full[i % STAGES], (uint32_t)(i / STAGES) & 1u, abort_flag, p.error, AT_ERR_PRODUCER);
                at_wait(&v_full[i % STAGES], (uint32_t)(i / STAGES) & 1u, abort_flag, p.error, AT_ERR_PRODUCER);
            }
        __syncwarp();
    } else if (warp == 1) {
        // ---- MMA issuer: the whole warp runs the loop (so that addresses and descriptors stay
        // warp-uniform values), one elected lane issues ----
        {
            constexpr uint32_t idesc_s = at_idesc(AT_BN, false);
            constexpr uint32_t idesc_o = at_idesc(HD, true);
            const bool leader = at_elect();
            auto wait_all = [&](uint64_t* bar, uint32_t parity) {
                return __all_sync(0xffffffffu, at_wait(bar, parity, abort_flag, p.error, AT_ERR_MMA)) != 0;
            };
            bool ok = wait_all(q_full, 0);
            // descriptors are built once; a tile further on is an addition to the address field
            // (in 16-byte units; the field cannot overflow within shared memory)
            const uint64_t dq0 = at_desc(sQ, 1024), dk0 = at_desc(sK, 1024);
            const uint64_t dv0 = at_desc(sV, HALVES > 1 ? HALF_BYTES : 1024);
            auto scores = [&](int s, int i) {      // S_s = Q_s K_i^T
                const uint64_t dq = dq0 + (uint64_t)((s * TILE_BYTES) >> 4);
                const uint64_t dk = dk0 + (uint64_t)(((i % STAGES) * TILE_BYTES) >> 4);
                if (leader) {
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            at_mma_ss(tmem_base + s * AT_BN, dq + (uint64_t)((h * HALF_BYTES + kk * 32) >> 4),
                                      dk + (uint64_t)((h * HALF_BYTES + kk * 32) >> 4), idesc_s, (h | kk) != 0 ? 1u : 0u);
                    at_commit(&s_full[s]);
                }
            };
            if (ok) ok = wait_all(&k_full[0], 0);
            if (ok) {
                at_fence_after();
                scores(0, 0);
                scores(1, 0);
                if (leader) at_commit(&k_empty[0]);
            }
            auto outputs = [&](int s, int i) {     // O_s += P_s V_i, 16 keys at a time
                const uint64_t dv = dv0 + (uint64_t)(((i % STAGES) * TILE_BYTES) >> 4);
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < AT_BN / 16; ++kk)
                        at_mma_ts(tmem_base + O_COL + s * HD, tmem_base + P_COL + s * P_STRIDE + kk * 8,
                                  dv + (uint64_t)((kk * 2048) >> 4), idesc_o, (i | kk) != 0 ? 1u : 0u);
                    at_commit(&o_done[s]);
                }
            };
            if (ALIAS) {
                // per stream: P V of tile i, then the scores of tile i + 1 over the same columns
                for (int i = 0; i < n_tiles && ok; ++i) {
                    const int stage = i % STAGES;
                    const uint32_t par = (uint32_t)i & 1u;
                    for (int s = 0; s < 2 && ok; ++s) {
                        if (!wait_all(&p_full[s], par)) { ok = false; break; }
                        if (s == 0 && !wait_all(&v_full[stage], (uint32_t)(i / STAGES) & 1u)) { ok = false; break; }
                        at_fence_after();
                        outputs(s, i);
                        if (s == 1 && leader) at_commit(&v_empty[stage]);
                        if (i + 1 < n_tiles) {
                            if (s == 0 && !wait_all(&k_full[(i + 1) % STAGES], (uint32_t)((i + 1) / STAGES) & 1u)) { ok = false; break; }
                            at_fence_after();
                            scores(s, i + 1);
                            if (s == 1 && leader) at_commit(&k_empty[(i + 1) % STAGES]);
                        }
                    }
                }
            } else {
                // The softmax warps free a stream's score columns early in a tile (once the scores
                // are in registers) and fill its probability columns at the tile's end, and the two
                // streams run half a tile apart; the events therefore come in this order:
                // scores of 0 free, probabilities of 1 (tile before), scores of 1 free, probabilities of 0.
                for (int i = 0; i < n_tiles && ok; ++i) {
                    const uint32_t par = (uint32_t)i & 1u;
                    const bool more = i + 1 < n_tiles;
                    const int next = (i + 1) % STAGES;
                    if (more) {
                        if (!wait_all(&s_free[0], par) || !wait_all(&k_full[next], (uint32_t)((i + 1) / STAGES) & 1u)) { ok = false; break; }
                        at_fence_after();
                        scores(0, i + 1);
                    }
                    if (i > 0) {
                        if (!wait_all(&p_full[1], par ^ 1u)) { ok = false; break; }
                        at_fence_after();
                        outputs(1, i - 1);
                        if (leader) at_commit(&v_empty[(i - 1) % STAGES]);
                    }
                    if (more) {
                        if (!wait_all(&s_free[1], par)) { ok = false; break; }
                        at_fence_after();
                        scores(1, i + 1);
                        if (leader) at_commit(&k_empty[next]);
                    }
                    if (!wait_all(&p_full[0], par) || !wait_all(&v_full[i % STAGES], (uint32_t)(i / STAGES) & 1u)) { ok = false; break; }
                    at_fence_after();
                    outputs(0, i);
                }
                if (ok && wait_all(&p_full[1], (uint32_t)(n_tiles - 1) & 1u)) {
                    at_fence_after();
                    outputs(1, n_tiles - 1);
                    if (leader) at_commit(&v_empty[(n_tiles - 1) % STAGES]);
                }
            }
            __syncwarp();
        }
    } else {
        // ---- softmax of one stream: TWO threads per query row, each with half of a tile's columns
        // (one warp alone cannot issue a row's 128 exponentials fast enough; the halves exchange
        // their row maxima through shared memory and meet at a named barrier of their 64 threads) ----
        const int sw = warp - 2;                            // warps 2..17; any four in a row cover the four lane quarters
        const int s = sw >> 3;                              // stream
        const int half = (sw >> 2) & 1;                     // which 64 of a tile's 128 columns
        const int quarter = warp & 3;                       // which 32 of the 128 rows (= this warp's TMEM lanes)
        const int r = quarter * 32 + lane;
        const int pos = first_pos + r;
        const int pair_bar = 2 + s * 4 + quarter;           // named barrier of the two warps that share these rows
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t t_s = lane_base + s * AT_BN + 64 * half;
        const uint32_t t_p = lane_base + P_COL + s * P_STRIDE + 32 * half;
        const uint32_t t_o = lane_base + O_COL + s * HD + (HD / 2) * half;
        const float sc = p.scale_log2e;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n_tiles && ok; ++i) {
            const uint32_t par = (uint32_t)i & 1u;
            // (the collective tensor-memory loads below need the whole warp: decide as one)
            if (!__all_sync(0xffffffffu, at_wait(&s_full[s], par, abort_flag, p.error, AT_ERR_SOFTMAX))) { ok = false; break; }
            at_fence_after();
            const int kbase = (j_begin + i) * AT_BN + 64 * half;        // key of this thread's column 0
            // visible columns of this row among its 64: [c_lo, c_hi)
            const int c_hi = min(64, pos - kbase + 1);
            const int c_lo = p.window > 0 ? max(0, pos - p.window + 1 - kbase) : 0;
            const int tile_k0 = (j_begin + i) * AT_BN;
            const bool masked = (tile_k0 + AT_BN - 1 > first_pos) || (p.window > 0 && tile_k0 < last_pos - p.window + 1);
            // the row's 64 scores of this half, read once
            uint32_t v[64];
            at_ld32_async(t_s, v);
            at_ld32_async(t_s + 32, v + 32);
            at_wait_ld();
            if (!ALIAS) {                                // the score columns may be written again
                at_fence_before();
                at_mbar_arrive(&s_free[s]);
            }
            bool o_waited = false;                       // P V of the tile before is known to have finished
            float mx = -INFINITY;
            if (masked) {
#pragma unroll
                for (int e = 0; e < 64; ++e)
                    mx = fmaxf(mx, (e >= c_lo && e < c_hi) ? __uint_as_float(v[e]) : -INFINITY);
            } else {
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int e = 0; e < 64; e += 8) {
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        m4[u] = at_max3(m4[u], __uint_as_float(v[e + 2 * u]), __uint_as_float(v[e + 2 * u + 1]));
                }
                mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            }
            // the other half's maximum of the same row (buffers alternate by tile, so a value is
            // never overwritten before its reader has passed the next barrier)
            row_max[par][s][half][r] = mx;
            asm volatile("bar.sync %0, 64;\n" ::"r"(pair_bar) : "memory");
            mx = fmaxf(mx, row_max[par][s][half ^ 1][r]);
            mx *= sc;                                    // sc > 0
            const bool raise = mx > m_used + AT_RESCALE_STEP || (m_used == -INFINITY && mx > -INFINITY);
            float alpha = 1.0f;
            if (raise) {
                alpha = at_exp2(m_used - mx);            // 0 while nothing has been seen
                m_used = mx;
                l *= alpha;
            }
            if (i > 0 && __any_sync(0xffffffffu, raise)) {
                // the accumulator of the rows whose maximum rose is scaled down (each half its own
                // columns); P V of the tile before this one must have finished
                if (!__all_sync(0xffffffffu, at_wait(&o_done[s], par ^ 1u, abort_flag, p.error, AT_ERR_SOFTMAX))) { ok = false; break; }
                at_fence_after();
                o_waited = true;
#pragma unroll 1
                for (int c = 0; c < HD / 64; ++c) {
                    uint32_t o[32];
                    at_ld32(t_o + 32 * c, o);
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                    at_st32(t_o + 32 * c, o);
                }
            }
            // The exponentials of the two streams take turns (0, 1, 0, 1, ...), so that one
            // stream's products always run beside the other stream's softmax.
            if (s == 1 || i > 0) {
                const uint32_t turn_par = s == 1 ? par : par ^ 1u;     // stream 1 follows 0's tile i; 0 follows 1's tile i - 1
                if (!__all_sync(0xffffffffu, at_wait(&turn[s], turn_par, abort_flag, p.error, AT_ERR_SOFTMAX))) { ok = false; break; }
            }
            // probabilities, written as bfloat16 pairs (pair e lands in v[e / 2], whose score has
            // been used by then)
            const float m_ref = m_used == -INFINITY ? 0.f : m_used;     // a row that sees nothing yet
            float sum0 = 0.f, sum1 = 0.f;
            if (masked) {       // (two copies of the loop: the common one carries no mask arithmetic)
#pragma unroll
                for (int e = 0; e < 64; e += 2) {
                    float p0 = at_exp2(fmaf(__uint_as_float(v[e]), sc, -m_ref));
                    float p1 = at_exp2(fmaf(__uint_as_float(v[e + 1]), sc, -m_ref));
                    p0 = (e >= c_lo && e < c_hi) ? p0 : 0.f;
                    p1 = (e + 1 >= c_lo && e + 1 < c_hi) ? p1 : 0.f;
                    sum0 += p0;
                    sum1 += p1;
                    v[e >> 1] = at_pack(p0, p1);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 64; e += 2) {
                    const float p0 = at_exp2(fmaf(__uint_as_float(v[e]), sc, -m_ref));
                    const float p1 = at_exp2(fmaf(__uint_as_float(v[e + 1]), sc, -m_ref));
                    sum0 += p0;
                    sum1 += p1;
                    v[e >> 1] = at_pack(p0, p1);
                }
            }
            l += sum0 + sum1;
            at_mbar_arrive(&turn[s ^ 1]);
            if (!ALIAS && i > 0 && !o_waited) {
                // the probability columns are still being read by P V of the tile before (long
                // finished in practice: it was issued a whole tile ago)
                if (!__all_sync(0xffffffffu, at_wait(&o_done[s], par ^ 1u, abort_flag, p.error, AT_ERR_SOFTMAX))) { ok = false; break; }
                at_fence_after();
            }
            at_st32(t_p, v);
            at_wait_st();
            at_fence_before();
            at_mbar_arrive(&p_full[s]);
        }
        // ---- the finished rows: O / l -> bfloat16; the row's sum is the two halves' together ----
        row_max[0][s][half][r] = l;                        // (the buffer of an even tile; see below)
        if (ok && n_tiles > 0 &&
            __all_sync(0xffffffffu, at_wait(&o_done[s], (uint32_t)(n_tiles - 1) & 1u, abort_flag, p.error, AT_ERR_SOFTMAX))) {
            at_fence_after();
            // Both warps of the pair pass this barrier after their last tile's exchange, whichever
            // buffer that used; the sums go through buffer 0, written above after the last read of it.
            asm volatile("bar.sync %0, 64;\n" ::"r"(pair_bar) : "memory");
            const float inv = 1.0f / (l + row_max[0][s][half ^ 1][r]);
            __nv_bfloat16* orow = p.out + (size_t)(q_begin + row0 + r) * ((size_t)p.n_q_heads * HD) +
                                  (size_t)(s ? head1 : head0) * HD + (HD / 2) * half;
            const bool stores = r < rows && (s == 0 || head1 != head0);
#pragma unroll 1
            for (int c = 0; c < HD / 64; ++c) {
                uint32_t o[32];
                at_ld32(t_o + 32 * c, o);
                if (stores) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        uint4 w;
                        w.x = at_pack(__uint_as_float(o[e]) * inv, __uint_as_float(o[e + 1]) * inv);
                        w.y = at_pack(__uint_as_float(o[e + 2]) * inv, __uint_as_float(o[e + 3]) * inv);
                        w.z = at_pack(__uint_as_float(o[e + 4]) * inv, __uint_as_float(o[e + 5]) * inv);
                        w.w = at_pack(__uint_as_float(o[e + 6]) * inv, __uint_as_float(o[e + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + 32 * c + e) = w;
                    }
                }
            }
        }
        if (at_extra_wait)                                     // tests: a phase that never completes
            at_wait(&o_done[s], (uint32_t)n_tiles & 1u, abort_flag, p.error, AT_ERR_SOFTMAX);
    }
    at_fence_before();
    __syncthreads();
    if (warp == 1) {
        at_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------------
typedef CUresult (*AtEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// ticks: how long a wait inside the kernel may last, in clock ticks (<= 0: the default of about a
// second); extra_wait != 0: the softmax warps wait once more for a phase that never completes (for
// the test of the give-up path).  Holds for the current device until set again.
NI_EXPORT int ni_attention_prefill_tc_set_wait(long long ticks, int extra_wait) {
    if (ticks <= 0) ticks = 2000000000LL;
    cudaError_t e = cudaMemcpyToSymbol(at_wait_limit, &ticks, sizeof(ticks));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(at_extra_wait, &extra_wait, sizeof(extra_wait));
    return e == cudaSuccess ? NI_OK : (int)e;
}

static AtEncodeTiledFn at_encode_tiled() {
    static AtEncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<AtEncodeTiledFn>(sym);
    });
    return fn;
}

// Tensor map of a row-major bf16 matrix [rows, cols] with boxes of [box_rows, 64], 128-byte swizzle.
static int at_make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, int box_rows) {
    AtEncodeTiledFn enc = at_encode_tiled();
    if (!enc) return NI_ERR_BAD_ARGUMENT;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NI_OK : NI_ERR_BAD_ARGUMENT;
}

template <int HD, int STAGES>
static int launch_at(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AtParams& p,
                     int n_tiles, cudaStream_t stream) {
    constexpr size_t tile = (size_t)(HD / 64) * AT_BN * 128;
    constexpr size_t smem = 1024 + (2 + 2 * STAGES) * tile + 512 + 2 * 2 * 2 * AT_BM * sizeof(float);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long long blocks = (long long)n_tiles * p.n_kv_heads * ((p.n_q_heads / p.n_kv_heads + 1) / 2);
    if (blocks > 0x7fffffffLL) return NI_ERR_UNSUPPORTED_SIZE;
    dim3 grid((unsigned)blocks);
    attention_prefill_tc_kernel<HD, STAGES><<<grid, AT_THREADS, smem, stream>>>(mq, mk, mv, p);
    NI_RETURN_LAUNCH_STATUS();
}

// 1 if this kernel takes the case, else 0 (the caller then uses the mma.sync kernel).
NI_EXPORT int ni_attention_prefill_tc_supports(int n_q_heads, int n_kv_heads, int head_dim, int page_size) {
    if (n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads) return 0;
    const int group = n_q_heads / n_kv_heads;
    if (group == 1) return 0;                 // two streams on one head would do every product twice
    if (head_dim != 64 && head_dim != 128) return 0;
    if (page_size < 8 || page_size > 128 || 128 % page_size) return 0;
    return 1;
}

// q, out: bf16 [n_tokens, Hq * hd]; k_pages, v_pages: bf16 [n_pages, Hkv, page_size, hd], all 16-byte
// aligned.  tile_seq / tile_row0 [n_tiles]: request and first query row of each block's 128 rows.
// error: a device int, zero on entry; non-zero afterwards if a wait inside the kernel ran out.
NI_EXPORT int ni_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages, void* out, int n_tokens,
                                      int n_pages, const int* tile_seq, const int* tile_row0, int n_tiles,
                                      const int* cu_q, const int* kv_len, const int* block_table, int bt_stride,
                                      int n_q_heads, int n_kv_heads, int head_dim, int page_size, int window,
                                      float scale, int* error, cudaStream_t stream) {
    if (n_tiles <= 0) return NI_OK;
    if (n_tokens <= 0 || n_pages <= 0 || error == nullptr) return NI_ERR_BAD_ARGUMENT;
    if (!ni_attention_prefill_tc_supports(n_q_heads, n_kv_heads, head_dim, page_size)) return NI_ERR_UNSUPPORTED_SIZE;
    if (((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || ((uintptr_t)out & 15))
        return NI_ERR_UNSUPPORTED_SIZE;
    CUtensorMap mq, mk, mv;
    int rc = at_make_map(&mq, q, n_tokens, (long long)n_q_heads * head_dim, AT_BM);
    if (rc != NI_OK) return rc;
    const long long cache_rows = (long long)n_pages * n_kv_heads * page_size;
    rc = at_make_map(&mk, k_pages, cache_rows, head_dim, page_size);
    if (rc != NI_OK) return rc;
    rc = at_make_map(&mv, v_pages, cache_rows, head_dim, page_size);
    if (rc != NI_OK) return rc;
    AtParams p;
    p.out = (__nv_bfloat16*)out; p.tile_seq = tile_seq; p.tile_row0 = tile_row0; p.cu_q = cu_q; p.kv_len = kv_len;
    p.block_table = block_table; p.bt_stride = bt_stride; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
    p.page_size = page_size; p.window = window; p.scale_log2e = scale * 1.4426950408889634f; p.error = error;
    if (head_dim == 64) return launch_at<64, 4>(mq, mk, mv, p, n_tiles, stream);
    return launch_at<128, 2>(mq, mk, mv, p, n_tiles, stream);
}
