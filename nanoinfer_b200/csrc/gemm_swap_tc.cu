// out[M, N] = x[M, K] . w[N, K]^T for a MODERATE number of activation rows (9 .. 128: decode
// batches beyond the skinny kernel, short prompt portions) - a bandwidth problem over the
// weights - on the fifth-generation tensor cores with the operands swapped: the 128 lanes of the
// tcgen05 tile are WEIGHT rows, the batch is the tile's N side (32, 64 or 128 columns), so the
// weights stream through TMA exactly once and no tensor-core row is wasted on padding.
//
// A block is persistent and warp-specialised like gemm_tc.cu: warp 0 drives TMA through a deep
// ring of stages (16 KB of weights + the matching activation columns each), warp 1 issues the MMAs
// (warp-uniform loop, elected lane), warps 2-5 read the accumulator from tensor memory (two
// accumulators alternate).  A work unit is (128 weight rows, a slice of K).  A projection with few
// weight rows (2,048 rows are 16 tiles for 148 SMs) is split along K over the blocks of a THREAD-
// BLOCK CLUSTER (up to 8): every block multiplies its slice, leaves its partial tile in its own
// shared memory, and after a cluster barrier each block adds, in block order, all partial tiles
// for ITS share of the batch rows - read through distributed shared memory - and runs the
// epilogue.  No global scratch, no atomics, a fixed order of sums.
//
// The kernel is launched with programmatic stream serialisation: a block requests its first
// stages of WEIGHTS (which depend on nothing) before griddepcontrol.wait and the activations after
// it, so the weight stream of a projection starts under the tail of the kernel before it.
//
// Epilogues (a thread owns one weight row = one output column of every batch row): store
// bfloat16 | store FP32 | add into the FP32 residual stream | SwiGLU over the blocked gate/up
// layout (lanes l and l + 8 of a 16-row group exchange by shuffle) | rotary encoding of adjacent
// row pairs (lanes l and l ^ 1) and the paged K/V write of a fused QKV projection.
//
// Every wait on an mbarrier is bounded (about a second); a wait that runs out records a code in
// the error word, and the block frees its tensor memory and returns.
//
// Reference counterparts: cublasSgemm (src/op/kernels/cuda/matmul_kernel.cu:48-89) with separate
// kernels for RoPE, the cache write, SwiGLU and the residual add (src/model/llama.cpp:324-379).
#include <cuda.h>

#include <mutex>

#include "common.cuh"

#define SW_BK 64
#define SW_ROWS 128            // weight rows per tile
#define SW_THREADS 320           // loader, MMA issuer, 8 epilogue warps: two per quarter of the lanes, half the batch columns each

#define SW_STORE_BF16 0
#define SW_STORE_F32 1
#define SW_ADD_F32 2
#define SW_SWIGLU 3
#define SW_ROPE_KV 4

#define SW_ERR_PRODUCER 21
#define SW_ERR_MMA 22
#define SW_ERR_EPILOGUE 23

__device__ __forceinline__ uint32_t sw_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void sw_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(sw_smem(bar)), "r"(count));
}
__device__ __forceinline__ void sw_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(sw_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void sw_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(sw_smem(bar)) : "memory");
}
// How long a wait on an mbarrier may last, in clock ticks (about a second), and a switch for the
// tests: with it the epilogue warps wait once more at the end, for a phase that nothing completes.
// Set by ni_gemm_swap_tc_set_wait.
__constant__ long long sw_wait_limit = 2000000000LL;
__constant__ int sw_extra_wait = 0;

__device__ __forceinline__ bool sw_wait(uint64_t* bar, uint32_t parity, int* error, int code) {
    const uint32_t addr = sw_smem(bar);
    long long start = 0;
    for (int iter = 0;; ++iter) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.b32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((iter & 1023) == 1023) {
            const long long now = clock64();
            if (start == 0) start = now;
            if (now - start > sw_wait_limit) {
                atomicExch(error, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void sw_tma_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(sw_smem(dst)), "l"(map), "r"(sw_smem(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void sw_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void sw_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ uint64_t sw_desc(const void* tile) {   // K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
    const uint32_t addr = sw_smem(tile);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__host__ __device__ constexpr uint32_t sw_idesc(int n) {          // BF16 x BF16 -> FP32, M = 128, N = n
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(SW_ROWS >> 4) << 24);
}
__device__ __forceinline__ void sw_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void sw_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(sw_smem(bar)) : "memory");
}
__device__ __forceinline__ void sw_ld32(uint32_t taddr, uint32_t r[32]) {
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

__device__ __forceinline__ void sw_ld8(uint32_t taddr, uint32_t r[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

__device__ __forceinline__ void sw_pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void sw_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }
__device__ __forceinline__ void sw_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t sw_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// Stores a float at the same shared-memory offset in block `rank` of this cluster.
__device__ __forceinline__ void sw_st_cluster(const float* mine, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(sw_smem(mine)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(remote), "f"(v) : "memory");
}

struct SwParams {
    void* out;
    int M, N, K, mode;
    int splits;               // slices of K per tile of weight rows = blocks of a cluster
    int* error;
    long long* trace;         // optional: block 0 stamps the time (ns) of its milestones here
    // SW_ROPE_KV
    const int* positions;
    const int* seq_of_token;
    const int* block_table;
    const float* inv_freq;
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
    int bt_stride, n_q_heads, n_kv_heads, head_dim, rotary_dim, page_size, write_cache;
};

// The finished sum v of (weight row n, batch row m) goes through the epilogue.  All 32 lanes of a
// warp call this together (lanes = consecutive weight rows), whatever n and m are.
template <int MODE>
__device__ __forceinline__ void sw_epilogue(const SwParams& p, int n, int m, float v, int lane) {
    const bool ok = n < p.N && m < p.M;
    if (MODE == SW_STORE_BF16) {
        if (ok) reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.N + n] = __float2bfloat16_rn(v);
    } else if (MODE == SW_STORE_F32) {
        if (ok) reinterpret_cast<float*>(p.out)[(size_t)m * p.N + n] = v;
    } else if (MODE == SW_ADD_F32) {
        if (ok) reinterpret_cast<float*>(p.out)[(size_t)m * p.N + n] += v;
    } else if (MODE == SW_SWIGLU) {
        // rows come in groups of 16: 8 gate rows, then their 8 up rows
        const float up = __shfl_down_sync(0xffffffffu, v, 8);
        if (ok && (n & 8) == 0)
            reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * (p.N >> 1) + ((n >> 4) << 3) + (n & 7)] =
                __float2bfloat16_rn(__fdividef(v, 1.0f + __expf(-v)) * up);
    } else {  // SW_ROPE_KV: rows 2i and 2i + 1 are a rotary pair
        const float other = __shfl_xor_sync(0xffffffffu, v, 1);
        if (!ok) return;
        const int hd = p.head_dim, nq = p.n_q_heads, nkv = p.n_kv_heads;
        const int head = n / hd, d = n - head * hd;
        const int pos = p.positions[m];
        float r = v;
        if (head < nq + nkv && d < p.rotary_dim) {
            float sn, cs;
            sincosf((float)pos * p.inv_freq[d >> 1], &sn, &cs);
            r = (n & 1) ? other * sn + v * cs : v * cs - other * sn;
        }
        __nv_bfloat16* dst;
        if (head < nq) {
            dst = reinterpret_cast<__nv_bfloat16*>(p.out) + ((size_t)m * nq + head) * hd + d;
        } else {
            if (!p.write_cache) return;
            const int page = p.block_table[(size_t)p.seq_of_token[m] * p.bt_stride + pos / p.page_size];
            const int kvh = head < nq + nkv ? head - nq : head - nq - nkv;
            __nv_bfloat16* base = head < nq + nkv ? p.k_pages : p.v_pages;
            dst = base + (((size_t)page * nkv + kvh) * p.page_size + (pos % p.page_size)) * hd + d;
        }
        *dst = __float2bfloat16_rn(r);
    }
}

// Stages of the ring: as many as fit shared memory, since bytes in flight set the streaming rate.
__device__ __forceinline__ void sw_stamp(const SwParams& p, int i) {
    if (p.trace != nullptr && blockIdx.x == 0) {
        long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.trace[i] = t;
    }
}

template <int BT> struct SwStages { static constexpr int value = BT <= 32 ? 10 : (BT <= 64 ? 7 : 4); };

template <int BT, int MODE>
__global__ void __launch_bounds__(SW_THREADS, 1)
gemm_swap_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const SwParams p) {
    constexpr int A_BYTES = SW_ROWS * SW_BK * 2;     // weights: 16 KB
    constexpr int B_BYTES = BT * SW_BK * 2;          // activations
    constexpr int ACC_COLS = 2 * BT < 32 ? 32 : 2 * BT;
    constexpr int SW_STAGES = SwStages<BT>::value;
    extern __shared__ uint8_t sw_smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)sw_smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = base;
    uint8_t* sB = base + SW_STAGES * A_BYTES;
    float* slots = reinterpret_cast<float*>(sB + SW_STAGES * B_BYTES);     // split sums: [slices][rows owned][128] FP32, <= BT rows in all
    uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(slots) + (BT + 8) * SW_ROWS * 4);
    uint64_t* empty = full + SW_STAGES;
    uint64_t* acc_full = empty + SW_STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    int* pre_kb = reinterpret_cast<int*>(tmem_slot + 1);       // [SW_STAGES] k-blocks whose weights were requested ahead

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) sw_stamp(p, 0);
    const int k_blocks = (p.K + SW_BK - 1) / SW_BK;
    const int tiles = (p.N + SW_ROWS - 1) / SW_ROWS;
    const int splits = p.splits;                    // > 1: one unit per block, the tile's units form a cluster
    const int n_units = tiles * splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SW_STAGES; ++s) { sw_mbar_init(&full[s], 1); sw_mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { sw_mbar_init(&acc_full[a], 1); sw_mbar_init(&acc_empty[a], 256); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_x) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(sw_smem(tmem_slot)), "r"(ACC_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    sw_fence_before();
    __syncthreads();
    sw_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    sw_pdl_launch_dependents();                     // the kernel after this one may begin its own prologue
    if (splits > 1) sw_cluster_sync();              // every block of the cluster runs: its shared memory may be stored into
    if (threadIdx.x == 0) sw_stamp(p, 1);

    if (warp == 0) {
        // ---- TMA producer ----
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true, released = false;
            int issued = 0;                         // loads of this block so far
            for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
                const int tile = unit / splits, split = unit - tile * splits;
                const int kb0 = k_blocks * split / splits, kb1 = k_blocks * (split + 1) / splits;   // (never empty: splits <= k_blocks)
                // Every block needs the same activation columns for a k-block.  Blocks therefore walk
                // their slice of K from different starting points (a fixed function of the tile), or
                // they would all ask the same few L2 lines for them at the same moment.
                const int span = kb1 - kb0, start = (tile * 5) % span;
                for (int i = 0; i < span; ++i) {
                    const int kb = kb0 + (start + i < span ? start + i : start + i - span);
                    if (!released && issued == SW_STAGES) {
                        // The ring is full of weights, which depend on nothing.  Now wait for the kernel
                        // before this one, whose results the activations are, and send them after.
                        sw_pdl_wait();
                        released = true;
                        for (int j = 0; j < SW_STAGES; ++j) sw_tma_2d(sB + j * B_BYTES, &map_x, pre_kb[j] * SW_BK, 0, &full[j]);
                    }
                    if (!sw_wait(&empty[stage], phase ^ 1, p.error, SW_ERR_PRODUCER)) { ok = false; break; }
                    sw_mbar_expect_tx(&full[stage], A_BYTES + B_BYTES);
                    sw_tma_2d(sA + stage * A_BYTES, &map_w, kb * SW_BK, tile * SW_ROWS, &full[stage]);
                    if (released) sw_tma_2d(sB + stage * B_BYTES, &map_x, kb * SW_BK, 0, &full[stage]);
                    else pre_kb[issued] = kb;
                    ++issued;
                    if (++stage == SW_STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!released) {                        // fewer loads than stages: all weights are on their way
                sw_pdl_wait();
                for (int j = 0; j < issued; ++j) sw_tma_2d(sB + j * B_BYTES, &map_x, pre_kb[j] * SW_BK, 0, &full[j]);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: warp-uniform loop, one elected lane issues ----
        constexpr uint32_t idesc = sw_idesc(BT);
        uint32_t elected;
        asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.b32 %0, 1, 0, p;\n}\n" : "=r"(elected));
        const bool leader = elected != 0;
        const uint64_t da0 = sw_desc(sA), db0 = sw_desc(sB);
        int stage = 0, acc = 0;
        uint32_t phase = 0, acc_phase = 0;
        bool ok = true;
        for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
            const int tile = unit / splits, split = unit - tile * splits;
            const int kb0 = k_blocks * split / splits, kb1 = k_blocks * (split + 1) / splits;
            if (!__all_sync(0xffffffffu, sw_wait(&acc_empty[acc], acc_phase ^ 1, p.error, SW_ERR_MMA))) break;
            sw_fence_after();
            const uint32_t tmem_d = tmem_base + acc * BT;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!__all_sync(0xffffffffu, sw_wait(&full[stage], phase, p.error, SW_ERR_MMA))) { ok = false; break; }
                sw_fence_after();
                const uint64_t da = da0 + (uint64_t)((stage * A_BYTES) >> 4);
                const uint64_t db = db0 + (uint64_t)((stage * B_BYTES) >> 4);
                if (leader) {
#pragma unroll
                    for (int k = 0; k < SW_BK / 16; ++k)
                        sw_mma(tmem_d, da + (uint64_t)((k * 32) >> 4), db + (uint64_t)((k * 32) >> 4), idesc,
                               (kb > kb0 || k > 0) ? 1u : 0u);
                    sw_commit(&empty[stage]);
                }
                if (++stage == SW_STAGES) { stage = 0; phase ^= 1; }
            }
            if (!ok) break;
            if (leader) sw_commit(&acc_full[acc]);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        __syncwarp();
    } else {
        // ---- epilogue: warps 2..9; a warp reads the lanes of its quarter (warp & 3, as tensor memory
        // demands), and of the two warps of a quarter each takes half of the batch columns ----
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane;               // weight row within the tile
        const int c_lo = half * (BT / 2), c_hi = c_lo + BT / 2;
        int acc = 0;
        uint32_t acc_phase = 0;
        sw_pdl_wait();                                      // the epilogues read and write what earlier kernels wrote
        for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
            const int tile = unit / splits;
            const int n = tile * SW_ROWS + row;
            if (threadIdx.x == 64) sw_stamp(p, 2);
            if (!__all_sync(0xffffffffu, sw_wait(&acc_full[acc], acc_phase, p.error, SW_ERR_EPILOGUE))) break;
            sw_fence_after();
            if (threadIdx.x == 64) sw_stamp(p, 3);
            const uint32_t t_acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BT;
            // (Short loop bodies: a tile's epilogue code runs once per tile, so it has to stay small
            // enough for the instruction cache - fully unrolled it was the kernel's largest cost.)
            if (splits == 1) {
#pragma unroll 1
                for (int c0 = c_lo; c0 < c_hi && c0 < p.M; c0 += 8) {
                    uint32_t v[8];
                    sw_ld8(t_acc + c0, v);
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        if (c0 + c < p.M) sw_epilogue<MODE>(p, n, c0 + c, __uint_as_float(v[c]), lane);   // (uniform over the warp)
                }
            } else {
                // This slice's partial sums go straight to the block that owns the batch row (block r of
                // the cluster owns rows r * per .. ), into slot [slice][row of that block][128] of ITS
                // shared memory, a region apart from the ring (which a neighbour's MMAs may still be
                // reading).  Stores to a neighbour's shared memory do not make the storing thread wait;
                // loads from it, tried first, did: 64 round trips per thread.
                const int per = (p.M + splits - 1) / splits;
                const uint32_t me = sw_cluster_rank();
                float* dst = slots + (size_t)me * per * SW_ROWS + row;
                int owner = c_lo / per, local = c_lo - owner * per;      // of batch row c_lo; advanced without dividing
#pragma unroll 1
                for (int c0 = c_lo; c0 < c_hi && c0 < p.M; c0 += 8) {
                    uint32_t v[8];
                    sw_ld8(t_acc + c0, v);
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        if (c0 + c < p.M) sw_st_cluster(dst + local * SW_ROWS, (uint32_t)owner, __uint_as_float(v[c]));
                        if (++local == per) { local = 0; ++owner; }
                    }
                }
            }
            sw_fence_before();
            sw_mbar_arrive(&acc_empty[acc]);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            if (threadIdx.x == 64) sw_stamp(p, 4);
        }
        if (sw_extra_wait) sw_wait(&acc_full[acc], acc_phase, p.error, SW_ERR_EPILOGUE);   // tests: a phase that never completes
    }
    if (splits > 1) {
        // ---- the slices' partial sums are added, in slice order, by the block that owns the batch row ----
        sw_cluster_sync();                                  // all partial sums have arrived in their owners' slots
        if (threadIdx.x == 64) sw_stamp(p, 5);
        if (warp >= 2) {
            const int quarter = warp & 3, half = (warp - 2) >> 2;
            const int row = quarter * 32 + lane;
            const int n = (blockIdx.x / splits) * SW_ROWS + row;
            const int per = (p.M + splits - 1) / splits;
            const int me = (int)sw_cluster_rank();
            const float* mine = slots + row;
#pragma unroll 1
            for (int l = half; l < per && me * per + l < p.M; l += 2) {     // the quarter's two warps take rows in turn
                float v = 0.f;
                for (int sp = 0; sp < splits; ++sp) v += mine[((size_t)sp * per + l) * SW_ROWS];
                sw_epilogue<MODE>(p, n, me * per + l, v, lane);
            }
        }
        // (nothing remote is touched after the barrier above: the blocks may leave one by one)
    }
    if (threadIdx.x == 64) sw_stamp(p, 6);
    sw_fence_before();
    __syncthreads();
    if (warp == 1) {
        sw_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(ACC_COLS) : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------------
typedef CUresult (*SwEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static SwEncodeTiledFn sw_encode_tiled() {
    static SwEncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<SwEncodeTiledFn>(sym);
    });
    return fn;
}

// ticks: how long a wait inside the kernel may last, in clock ticks (<= 0: the default of about a
// second); extra_wait != 0: the epilogue warps wait once more for a phase that never completes (for
// the test of the give-up path).  Holds for the current device until set again.
NI_EXPORT int ni_gemm_swap_tc_set_wait(long long ticks, int extra_wait) {
    if (ticks <= 0) ticks = 2000000000LL;
    cudaError_t e = cudaMemcpyToSymbol(sw_wait_limit, &ticks, sizeof(ticks));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(sw_extra_wait, &extra_wait, sizeof(extra_wait));
    return e == cudaSuccess ? NI_OK : (int)e;
}

static long long* sw_trace_ptr = nullptr;
// For looking at where a launch's time goes: block 0 writes the time of its milestones (start, set-up
// done, epilogue starts waiting, accumulator complete, accumulator read, sums arrived, end) to ptr.
NI_EXPORT void ni_gemm_swap_tc_set_trace(long long* ptr) { sw_trace_ptr = ptr; }

static int sw_make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    SwEncodeTiledFn enc = sw_encode_tiled();
    if (!enc) return NI_ERR_BAD_ARGUMENT;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {SW_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NI_OK : NI_ERR_BAD_ARGUMENT;
}

static int sw_n_sms() { return ni_sm_count(); }

template <int BT, int MODE>
static int launch_sw_mode(const CUtensorMap& mw, const CUtensorMap& mx, const SwParams& p, cudaStream_t stream) {
    constexpr size_t smem = 1024 + (size_t)SwStages<BT>::value * (SW_ROWS * SW_BK * 2 + BT * SW_BK * 2) +
                            (size_t)(BT + 8) * SW_ROWS * 4 + 256;
    static_assert(smem <= 232448, "shared memory of the swapped-operand product");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_swap_tc_kernel<BT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int units = ((p.N + SW_ROWS - 1) / SW_ROWS) * p.splits;
    // split: one unit per block, a tile's units are one cluster; whole tiles: persistent blocks
    const int grid = p.splits > 1 ? units : (units < sw_n_sms() ? units : sw_n_sms());
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(SW_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    int n_attr = 1;
    if (p.splits > 1) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = p.splits;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        n_attr = 2;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_swap_tc_kernel<BT, MODE>, mw, mx, p);
    return e == cudaSuccess ? NI_OK : (int)e;
}

template <int BT>
static int launch_sw(const CUtensorMap& mw, const CUtensorMap& mx, const SwParams& p, cudaStream_t stream) {
    switch (p.mode) {
        case SW_STORE_BF16: return launch_sw_mode<BT, SW_STORE_BF16>(mw, mx, p, stream);
        case SW_STORE_F32: return launch_sw_mode<BT, SW_STORE_F32>(mw, mx, p, stream);
        case SW_ADD_F32: return launch_sw_mode<BT, SW_ADD_F32>(mw, mx, p, stream);
        case SW_SWIGLU: return launch_sw_mode<BT, SW_SWIGLU>(mw, mx, p, stream);
        default: return launch_sw_mode<BT, SW_ROPE_KV>(mw, mx, p, stream);
    }
}

// How many slices of K a product is cut into - the blocks of one cluster per tile of 128 weight rows -
// so that about every SM has a unit: 1 when whole tiles already keep three quarters of the SMs busy,
// else up to 8 (the portable cluster size), never more than there are 64-column blocks of K.
NI_EXPORT int ni_gemm_swap_tc_splits(int M, int N, int K) {
    const int tiles = (N + SW_ROWS - 1) / SW_ROWS;
    const int k_blocks = (K + SW_BK - 1) / SW_BK;
    if (tiles * 4 >= sw_n_sms() * 3) return 1;
    int splits = sw_n_sms() / tiles;
    if (splits > 8) splits = 8;
    if (splits > k_blocks) splits = k_blocks;
    return splits < 1 ? 1 : splits;
}
// Global scratch the product needs: none (the slices of K meet in the cluster's shared memory).
NI_EXPORT long long ni_gemm_swap_tc_scratch(int M, int N, int K) { return 0; }

// x: bf16 [M, K], 9 <= M <= 128 (fewer rows work too); w: bf16 [N, K]; K a multiple of 8; 16-byte aligned.
// mode 0 store bf16 [M, N], 1 store FP32, 2 add into FP32 [M, N], 3 SwiGLU over blocked rows -> bf16
// [M, N / 2], 4 rotary encoding + paged K/V write of a fused QKV projection (out = q, bf16 [M, Hq * hd]).
// partials, tickets: unused (kept in the signature; earlier versions combined the slices of K through them).
NI_EXPORT int ni_gemm_swap_tc(const void* x, const void* w, void* out, int M, int N, int K, int mode, float* partials,
                              int* tickets, const int* positions, const int* seq_of_token, const int* block_table,
                              int bt_stride, const float* inv_freq, void* k_pages, void* v_pages, int n_q_heads,
                              int n_kv_heads, int head_dim, int rotary_dim, int page_size, int* error,
                              cudaStream_t stream) {
    if (M <= 0 || N <= 0) return NI_OK;
    if (K <= 0 || mode < 0 || mode > SW_ROPE_KV || error == nullptr) return NI_ERR_BAD_ARGUMENT;
    if (M > 128 || K % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return NI_ERR_UNSUPPORTED_SIZE;
    if (mode == SW_SWIGLU && N % 16) return NI_ERR_UNSUPPORTED_SIZE;
    if (mode == SW_ROPE_KV && (head_dim % 2 || rotary_dim % 2 || N != (n_q_heads + 2 * n_kv_heads) * head_dim))
        return NI_ERR_BAD_ARGUMENT;
    SwParams p = {};
    p.out = out; p.M = M; p.N = N; p.K = K; p.mode = mode; p.error = error;
    p.splits = ni_gemm_swap_tc_splits(M, N, K);
    p.trace = sw_trace_ptr;
    (void)partials; (void)tickets;
    p.positions = positions; p.seq_of_token = seq_of_token; p.block_table = block_table; p.inv_freq = inv_freq;
    p.k_pages = (__nv_bfloat16*)k_pages; p.v_pages = (__nv_bfloat16*)v_pages; p.bt_stride = bt_stride;
    p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.rotary_dim = rotary_dim;
    p.page_size = page_size; p.write_cache = (k_pages != nullptr && v_pages != nullptr) ? 1 : 0;
    const int bt = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
    CUtensorMap mw, mx;
    int rc = sw_make_map(&mw, w, N, K, SW_ROWS);
    if (rc != NI_OK) return rc;
    rc = sw_make_map(&mx, x, M, K, bt);
    if (rc != NI_OK) return rc;
    if (bt == 32) return launch_sw<32>(mw, mx, p, stream);
    if (bt == 64) return launch_sw<64>(mw, mx, p, stream);
    return launch_sw<128>(mw, mx, p, stream);
}
