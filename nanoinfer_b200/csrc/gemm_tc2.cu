// C[M, N] = A[M, K] . B[N, K]^T for bfloat16 operands on the fifth-generation tensor cores, two SMs
// to a tile: the blocks of a cluster of two share one 256 x 256 output tile (tcgen05.mma with
// cta_group::2).  Each block holds its own 128 rows of A and HALF of the B tile in shared memory
// and its own 128 x 256 accumulator in tensor memory; the MMA, issued by one thread of the
// cluster's first block, reads B from both blocks' shared memory.  A block thus takes in 32 KB per
// 64-wide k-block instead of the 48 KB of a single-SM 128 x 256 tile, and that intake, not the
// tensor pipe, is what bounds the single-SM kernel (gemm_tc.cu).  No TMA load uses multicast: each
// block loads what it holds.
//
// Roles per block as in gemm_tc.cu: warp 0 TMA producer, warp 1 MMA issuer (first block only;
// warp-uniform loop, elected lane), warps 2-5 epilogue.  Barriers that span the pair: a stage's
// "full" barrier lives in the first block and counts both producers' bytes (the second block's
// loads signal it through the cluster address); "empty" and "accumulator full" are signalled in
// both blocks at once by tcgen05.commit with a block mask; "accumulator empty" in the first block
// counts the epilogue threads of both.  Epilogues as in gemm_tc.cu.
//
// Every wait on an mbarrier is bounded: after about two seconds a waiter records where it gave up
// in the error word and leaves its loop; the blocks then meet at the cluster barrier, free their
// tensor memory and return.
//
// Reference counterpart: cublasSgemm in FP32 for every projection
// (src/op/kernels/cuda/matmul_kernel.cu:48-89) with separate SwiGLU and add kernels behind it.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define TC_STORE_BF16 0
#define TC_STORE_F32 1
#define TC_ADD_F32 2
#define TC_SWIGLU 3

#define TC_ERR_TIMEOUT_PRODUCER 1
#define TC_ERR_TIMEOUT_MMA 2
#define TC_ERR_TIMEOUT_EPILOGUE 3

__device__ __forceinline__ uint32_t tc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(tc_smem(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(tc_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc_smem(bar)) : "memory");
}
// How long a wait on an mbarrier may last, in clock ticks (about two seconds), and a switch for the
// tests: with it the epilogue warps wait once more at the end, for a phase that nothing completes, so
// that a wait runs out, the kernel records it and returns.  Set by ni_gemm_tc2_set_wait.
__constant__ long long tc_wait_limit = 4000000000LL;
__constant__ int tc_extra_wait = 0;

// Waits for the phase with the given parity; false if the wait ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = tc_smem(bar);
    const long long start = clock64();
    for (;;) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.b32 %0, 1, 0, p;\n}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (clock64() - start > tc_wait_limit) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(tc_smem(dst)), "l"(map), "r"(tc_smem(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// The shared::cluster address of `local` (an address in this block's shared memory) in block `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_expect_tx_at(uint32_t cluster_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;\n" ::"r"(cluster_addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_at(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// A load into this block's shared memory whose bytes are counted by a barrier that may live in the
// other block of the pair (cluster address).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(tc_smem(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes,
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
    const uint32_t addr = tc_smem(tile);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);          // start address
    d |= (uint64_t)1 << 16;                           // leading byte offset (unused for this layout)
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                           // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                           // 128-byte swizzle
    return d;
}
// Instruction descriptor: BF16 x BF16 -> FP32, both operands K-major, M = 256 over the pair, N = bn.
__host__ __device__ constexpr uint32_t umma_idesc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)((2 * TC_BM) >> 4) << 24);
}
__device__ __forceinline__ void umma_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, once the MMAs issued so far have finished, on the barrier at this offset in BOTH blocks.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(tc_smem(bar)), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t r[32]) {
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

struct TcParams {
    void* out;
    int M, N, K, mode;
    int* error;       // device word: 0, or where a wait gave up
};

// One row's 32 consecutive accumulator columns [col, col + 32) through the epilogue.
__device__ __forceinline__ void tc_epilogue_row(const TcParams& p, int row, int col, const uint32_t v[32]) {
    const int N = p.N;
    if (row >= p.M || col >= N) return;
    const bool full = col + 32 <= N;
    if (p.mode == TC_STORE_BF16) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)row * N + col;
        if (full && (N & 7) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 w;
                uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]), __uint_as_float(v[8 * i + 2 * j + 1]));
                    wp[j] = *reinterpret_cast<uint32_t*>(&b);
                }
                *reinterpret_cast<uint4*>(o + 8 * i) = w;
            }
        } else {
            for (int i = 0; i < 32 && col + i < N; ++i) o[i] = __float2bfloat16_rn(__uint_as_float(v[i]));
        }
    } else if (p.mode == TC_STORE_F32 || p.mode == TC_ADD_F32) {
        float* o = reinterpret_cast<float*>(p.out) + (size_t)row * N + col;
        const bool add = p.mode == TC_ADD_F32;
        if (full && (N & 3) == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float4 w = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                       __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                if (add) {
                    const float4 h = *reinterpret_cast<const float4*>(o + 4 * i);
                    w.x += h.x; w.y += h.y; w.z += h.z; w.w += h.w;
                }
                *reinterpret_cast<float4*>(o + 4 * i) = w;
            }
        } else {
            for (int i = 0; i < 32 && col + i < N; ++i) o[i] = (add ? o[i] : 0.f) + __uint_as_float(v[i]);
        }
    } else {  // TC_SWIGLU: two blocks of 8 gate + 8 up columns -> 16 outputs; N is a multiple of 16
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)row * (N >> 1) + (col >> 1);
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            if (col + 16 * b >= N) break;
            uint4 w;
            uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float g0 = __uint_as_float(v[16 * b + 2 * j]), g1 = __uint_as_float(v[16 * b + 2 * j + 1]);
                const float u0 = __uint_as_float(v[16 * b + 8 + 2 * j]), u1 = __uint_as_float(v[16 * b + 8 + 2 * j + 1]);
                __nv_bfloat162 r = __floats2bfloat162_rn((g0 / (1.0f + expf(-g0))) * u0, (g1 / (1.0f + expf(-g1))) * u1);
                wp[j] = *reinterpret_cast<uint32_t*>(&r);
            }
            *reinterpret_cast<uint4*>(o + 8 * b) = w;
        }
    }
}

#define TC2_STAGES 6

// BN: columns of the pair's tile (128, 192 or 256; each block holds BN / 2 rows of B): narrower
// tiles give small products more tiles than there are pairs of SMs.  ACCS: accumulators per block
// (2: the epilogue of a tile overlaps the next tile's products).
template <int BN, int ACCS>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcParams p) {
    constexpr int STAGES = TC2_STAGES;
    constexpr int A_BYTES = TC_BM * TC_BK * 2;            // this block's rows of A: 16 KB
    constexpr int B_BYTES = (BN / 2) * TC_BK * 2;         // this block's half of B: 16 KB
    constexpr int ACC_COLS = ACCS * BN <= 128 ? 128 : (ACCS * BN <= 256 ? 256 : 512);
    static_assert(ACCS * BN <= 512 && BN % 32 == 0, "tensor memory columns");
    extern __shared__ uint8_t tc_smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>(((uintptr_t)tc_smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = base;
    uint8_t* sB = base + STAGES * A_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(sB + STAGES * B_BYTES);   // used in the first block
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;                                    // used in the first block
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                 // 0: issues the MMAs; 1: its peer
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int k_blocks = (p.K + TC_BK - 1) / TC_BK;
    const int tiles_m = (p.M + 2 * TC_BM - 1) / (2 * TC_BM);
    const int tiles_n = (p.N + BN - 1) / BN;
    const int n_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 2); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 256); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_b) : "memory");
    }
    if (warp == 1) {
        // one warp of EACH block of the pair takes part in the allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(tc_smem(tmem_slot)), "r"(ACC_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                   // both blocks' barriers exist before anyone signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA producer (both blocks): own rows of A, own half of B; bytes counted in the first block ----
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
                const int m0 = (tile % tiles_m) * 2 * TC_BM + (int)rank * TC_BM;
                const int n0 = (tile / tiles_m) * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1)) { atomicExch(p.error, TC_ERR_TIMEOUT_PRODUCER); ok = false; break; }
                    const uint32_t full_first = map_to_rank(tc_smem(&full[stage]), 0);
                    mbar_expect_tx_at(full_first, A_BYTES + B_BYTES);
                    tma_load_2d_pair(sA + stage * A_BYTES, &map_a, kb * TC_BK, m0, full_first);
                    tma_load_2d_pair(sB + stage * B_BYTES, &map_b, kb * TC_BK, n0, full_first);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer (first block only): warp-uniform loop, one elected lane issues ----
        if (rank == 0) {
            constexpr uint32_t idesc = umma_idesc(BN);
            uint32_t elected;
            asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.b32 %0, 1, 0, p;\n}\n" : "=r"(elected));
            const bool leader = elected != 0;
            const uint64_t da0 = umma_desc(sA), db0 = umma_desc(sB);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
                if (!__all_sync(0xffffffffu, mbar_wait(&acc_empty[acc], acc_phase ^ 1))) {
                    if (leader) atomicExch(p.error, TC_ERR_TIMEOUT_MMA);
                    break;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!__all_sync(0xffffffffu, mbar_wait(&full[stage], phase))) {
                        if (leader) atomicExch(p.error, TC_ERR_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t da = da0 + (uint64_t)((stage * A_BYTES) >> 4);
                    const uint64_t db = db0 + (uint64_t)((stage * B_BYTES) >> 4);
                    if (leader) {
#pragma unroll
                        for (int k = 0; k < TC_BK / 16; ++k)
                            umma_mma(tmem_d, da + (uint64_t)((k * 32) >> 4), db + (uint64_t)((k * 32) >> 4), idesc,
                                     (kb | k) != 0 ? 1u : 0u);
                        umma_commit_pair(&empty[stage]);      // the stage is free in both blocks once these MMAs have read it
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (leader) umma_commit_pair(&acc_full[acc]); // the accumulator halves are complete in both blocks
                if (ACCS == 2) { if (++acc == 2) { acc = 0; acc_phase ^= 1; } } else acc_phase ^= 1;
            }
            __syncwarp();
        }
    } else {
        // ---- epilogue (both blocks): warps 2..5, each its own quarter of this block's 128 accumulator lanes ----
        const int quarter = warp & 3;
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = pair; tile < n_tiles; tile += n_pairs) {
            const int m0 = (tile % tiles_m) * 2 * TC_BM + (int)rank * TC_BM, n0 = (tile / tiles_m) * BN;
            if (!mbar_wait(&acc_full[acc], acc_phase)) { atomicExch(p.error, TC_ERR_TIMEOUT_EPILOGUE); break; }
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + c0, v);
                tc_epilogue_row(p, row, n0 + c0, v);
            }
            tc_fence_before();
            mbar_arrive_at(map_to_rank(tc_smem(&acc_empty[acc]), 0));
            if (ACCS == 2) { if (++acc == 2) { acc = 0; acc_phase ^= 1; } } else acc_phase ^= 1;
        }
        if (tc_extra_wait && !mbar_wait(&acc_full[acc], acc_phase))     // tests: a phase that never completes
            atomicExch(p.error, TC_ERR_TIMEOUT_EPILOGUE);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                   // nobody signals the other block's barriers after this
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(ACC_COLS) : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// Tensor map of a row-major bf16 matrix [rows, K] with boxes of [box_rows, 64] and 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return NI_ERR_BAD_ARGUMENT;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NI_OK : NI_ERR_BAD_ARGUMENT;
}

template <int BN, int ACCS>
static int launch_tc2(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, cudaStream_t stream) {
    constexpr size_t smem = 1024 + (size_t)TC2_STAGES * (TC_BM * TC_BK * 2 + (BN / 2) * TC_BK * 2) + 256;
    static bool configured = false;
    static int n_sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel<BN, ACCS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
        configured = true;
    }
    const int tiles = ((p.M + 2 * TC_BM - 1) / (2 * TC_BM)) * ((p.N + BN - 1) / BN);
    const int pairs = tiles < n_sms / 2 ? tiles : n_sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<BN, ACCS>, ma, mb, p);
    return e == cudaSuccess ? NI_OK : (int)e;
}

// ticks: how long a wait inside the kernel may last, in clock ticks (<= 0: the default of about two
// seconds); extra_wait != 0: the epilogue warps of both blocks wait once more for a phase that never
// completes (for the test of the give-up path).  Holds for the current device until set again.
NI_EXPORT int ni_gemm_tc2_set_wait(long long ticks, int extra_wait) {
    if (ticks <= 0) ticks = 4000000000LL;
    cudaError_t e = cudaMemcpyToSymbol(tc_wait_limit, &ticks, sizeof(ticks));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(tc_extra_wait, &extra_wait, sizeof(extra_wait));
    return e == cudaSuccess ? NI_OK : (int)e;
}

// a: bf16 [M, K]; b: bf16 [N, K]; K a multiple of 8; both 16-byte aligned.  mode 0 store bf16 [M, N],
// 1 store FP32, 2 add into FP32 [M, N], 3 SwiGLU over blocked columns -> bf16 [M, N / 2].
// error: a device int, zero on entry; non-zero afterwards if a wait inside the kernel ran out.
// accumulators: 1 or 2 per block.  tile_n: 128, 192 or 256 columns per tile, or 0: as many as give every
// pair of SMs about two tiles.
NI_EXPORT int ni_gemm_tc2(const void* a, const void* b, void* out, int M, int N, int K, int mode, int accumulators,
                          int tile_n, int* error, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return NI_OK;
    if (K <= 0 || mode < 0 || mode > TC_SWIGLU || error == nullptr) return NI_ERR_BAD_ARGUMENT;
    if (K % 8 || ((uintptr_t)a & 15) || ((uintptr_t)b & 15)) return NI_ERR_UNSUPPORTED_SIZE;
    if (mode == TC_SWIGLU && N % 16) return NI_ERR_UNSUPPORTED_SIZE;
    if (tile_n == 0) {
        const long long tiles_m = (M + 2 * TC_BM - 1) / (2 * TC_BM);
        tile_n = 256;
        if (tiles_m * ((N + 255) / 256) < 2 * 74) tile_n = 192;
        if (tiles_m * ((N + 191) / 192) < 2 * 74) tile_n = 128;
    }
    if (tile_n != 128 && tile_n != 192 && tile_n != 256) return NI_ERR_BAD_ARGUMENT;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, a, M, K, TC_BM);
    if (rc != NI_OK) return rc;
    rc = make_map(&mb, b, N, K, tile_n / 2);
    if (rc != NI_OK) return rc;
    TcParams p;
    p.out = out; p.M = M; p.N = N; p.K = K; p.mode = mode; p.error = error;
    const bool one = accumulators == 1;
    if (tile_n == 128) return one ? launch_tc2<128, 1>(ma, mb, p, stream) : launch_tc2<128, 2>(ma, mb, p, stream);
    if (tile_n == 192) return one ? launch_tc2<192, 1>(ma, mb, p, stream) : launch_tc2<192, 2>(ma, mb, p, stream);
    return one ? launch_tc2<256, 1>(ma, mb, p, stream) : launch_tc2<256, 2>(ma, mb, p, stream);
}
