// Skinny matrix product for decode with a long contraction: y[M, N] = x[M, K] . W[N, K]^T,
// M <= 8, K of several thousand (the down projection of a feed-forward) - K split over the blocks
// of a thread-block cluster.
//
// The register-streaming kernel of gemv_bf16.cu keeps a warp's activations in registers only when
// one pass of the block covers K (K <= 2,048 at two blocks per SM).  Beyond that it re-reads the
// activations from L2 for every tile of 8 weight rows: as many bytes again as the weights (8 rows
// of activations per 8 rows of weights), and an SM then has to take in twice what the memory
// system delivers to it.  Here a cluster of S = ceil(K / 2,048) blocks shares each row tile: block r
// owns the r-th slice of K, keeps its 8 x (K / S) activations in registers for all the row tiles it
// walks, and the slices' sums meet in the shared memory of the cluster's first block (written
// there through distributed shared memory, added in slice order - a result never depends on
// timing).  The activations are read once per block, not once per tile.
//
// As in gemv_bf16.cu: weights on the 16-row side of mma.sync m16n8k16 (two tiles of 8 rows, or one
// of 16), the batch on the 8-wide side; 16-byte streaming loads straight into MMA fragments with
// the contraction index permuted alike in both operands; the next tile's weights requested right
// after this tile's MMAs; programmatic launch with the first weights requested before
// griddepcontrol.wait.  Blocks wait for one another only inside their cluster (hardware cluster
// barrier, whose blocks are co-scheduled).
//
// Reference counterpart: cublasSgemm on FP32 weights (src/op/kernels/cuda/matmul_kernel.cu:48-89)
// followed by a separate residual add (src/model/llama.cpp:376-379).
#include <cstdint>

#include "common.cuh"

#define KS_WARPS 8
#define KS_U 4                                   // k-blocks of 64 per warp: a slice is at most 64 * 8 * 4 = 2,048
#define KS_SLICE_BLOCKS (KS_WARPS * KS_U)
#define KS_MAX_SPLITS 8                          // portable cluster size
#define KS_MAX_SLOT_FLOATS (10 * 1024)           // 40 KB of partial sums in the first block

#define KS_STORE_BF16 0
#define KS_STORE_F32 1
#define KS_ADD_F32 2

struct KsParams {
    const __nv_bfloat16* x;   // [M, K]
    const __nv_bfloat16* w;   // [N, K]
    void* out;
    int M, N, K, mode;
    int splits, slice_blocks, tiles_per_cluster;
    const unsigned char* warm;
    unsigned long long warm_bytes;
    // with mode KS_ADD_F32: also prepare the norm that follows - next_x = bf16(out * next_gain) and per row
    // tile and row the sum of out^2 (next_ssq[row][tile]); see gemv_bf16.cu
    const float* next_gain;
    __nv_bfloat16* next_x;
    float* next_ssq;          // [8 rows][next_parts]
    int next_parts;
};

__device__ __forceinline__ void ks_mma(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ks_ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void ks_pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void ks_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }
__device__ __forceinline__ uint32_t ks_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void ks_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void ks_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
// the address of `p` (a shared-memory address of this block) in block `rank` of the cluster
__device__ __forceinline__ uint32_t ks_map(const void* p, uint32_t rank) {
    uint32_t local = (uint32_t)__cvta_generic_to_shared(p), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ void ks_st_cluster(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}

// RN: weight rows per tile (8 or 16).  WARM: the kernel ends with its share of the request to bring
// p.warm into L2 (see gemv_bf16.cu).
// NEXT: the adding epilogue also prepares the norm that follows (KsParams::next_*).
template <int RN, bool WARM, bool NEXT>
__global__ void __launch_bounds__(KS_WARPS * 32, 2) gemv_ksplit_kernel(const KsParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int M = p.M, N = p.N, K = p.K;
    const int splits = p.splits, tpc = p.tiles_per_cluster;
    const uint32_t rank = ks_cluster_rank();
    const int cluster = blockIdx.x / splits;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    ks_pdl_launch_dependents();
    ks_cluster_arrive();        // "this block runs" (waited for before the first write into another block)

    __shared__ float red[KS_WARPS][16][8];
    // partial sums of every slice and tile of the cluster; only the first block's copy is used
    extern __shared__ __align__(16) float slots[];   // [splits][tiles_per_cluster][8 * RN]

    // this block's slice of K: k-blocks [kb_lo, kb_hi)
    const int kb_lo = (int)rank * p.slice_blocks;
    const int kb_hi = min((K + 63) / 64, kb_lo + p.slice_blocks);

    uint4 fa[KS_U][2], fb[KS_U][2], fx[KS_U][2];
    auto load_weights = [&](int n0) {
        const bool row_a_ok = n0 + g < N;
        const bool row_b_ok = RN == 16 && n0 + g + 8 < N;
        const __nv_bfloat16* wa = p.w + (size_t)(row_a_ok ? n0 + g : 0) * K;
        const __nv_bfloat16* wb = p.w + (size_t)(row_b_ok ? n0 + g + 8 : 0) * K;
#pragma unroll
        for (int u = 0; u < KS_U; ++u) {
            const int kb = kb_lo + warp + u * KS_WARPS;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int k = kb * 64 + 32 * h + 8 * t;
                const bool ok = kb < kb_hi && k + 8 <= K;        // K is a multiple of 8
                fa[u][h] = (ok && row_a_ok) ? ks_ld_stream(wa + k) : zero;
                fb[u][h] = (RN == 16 && ok && row_b_ok) ? ks_ld_stream(wb + k) : zero;
            }
        }
    };

    const int tile0 = cluster * tpc;
    const int n_tiles = (N + RN - 1) / RN;
    if (tile0 < n_tiles) load_weights(tile0 * RN);
    ks_pdl_wait();              // what follows reads the activations, which the kernel before this one wrote
    {
        const bool x_ok = g < M;
        const __nv_bfloat16* xr = p.x + (size_t)(x_ok ? g : 0) * K;
#pragma unroll
        for (int u = 0; u < KS_U; ++u) {
            const int kb = kb_lo + warp + u * KS_WARPS;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int k = kb * 64 + 32 * h + 8 * t;
                fx[u][h] = (x_ok && kb < kb_hi && k + 8 <= K) ? *reinterpret_cast<const uint4*>(xr + k) : zero;
            }
        }
    }
    ks_cluster_wait();          // every block of the cluster runs: its shared memory may be written

    for (int ti = 0; ti < tpc; ++ti) {
        const int n0 = (tile0 + ti) * RN;
        if (n0 >= N) break;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int u = 0; u < KS_U; ++u)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                ks_mma(acc, fa[u][h].x, fb[u][h].x, fa[u][h].y, fb[u][h].y, fx[u][h].x, fx[u][h].y);
                ks_mma(acc, fa[u][h].z, fb[u][h].z, fa[u][h].w, fb[u][h].w, fx[u][h].z, fx[u][h].w);
            }
        if (ti + 1 < tpc && n0 + RN < N) load_weights(n0 + RN);   // in flight during the reduction below

        // the 8 warps' sums -> shared memory -> added in warp order -> the first block's slot of this slice
        red[warp][g][2 * t] = acc[0];
        red[warp][g][2 * t + 1] = acc[1];
        red[warp][g + 8][2 * t] = acc[2];
        red[warp][g + 8][2 * t + 1] = acc[3];
        __syncthreads();
        if (threadIdx.x < 8 * RN) {
            const int row = threadIdx.x % RN, m = threadIdx.x / RN;
            float s = 0.f;
#pragma unroll
            for (int wi = 0; wi < KS_WARPS; ++wi) s += red[wi][row][m];
            float* slot = slots + ((size_t)rank * tpc + ti) * (8 * RN) + threadIdx.x;
            ks_st_cluster(ks_map(slot, 0), s);
        }
        __syncthreads();        // red is free for the next tile
    }
    if (WARM && warp == KS_WARPS - 1) {
        constexpr unsigned int PIECE = 8192;
        const unsigned int n_pieces = (unsigned int)((p.warm_bytes + PIECE - 1) / PIECE);
        for (unsigned int i = blockIdx.x + lane * gridDim.x; i < n_pieces; i += 32 * gridDim.x) {
            const unsigned long long off = (unsigned long long)i * PIECE;
            const unsigned int sz = p.warm_bytes - off < PIECE ? (unsigned int)(p.warm_bytes - off) : PIECE;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(p.warm + off), "r"(sz) : "memory");
        }
    }
    ks_cluster_arrive();        // this block's sums are written
    ks_cluster_wait();          // ... and everyone else's
    if (rank != 0) return;

    // the first block adds the slices in slice order and writes the result
    const int mode = p.mode;
    if (NEXT) {
        // ... and what the next norm needs; whole warps take part (a tile's 8 * RN sums are a multiple of 64 threads)
        for (int idx = threadIdx.x; idx < tpc * 8 * RN; idx += blockDim.x) {
            const int ti = idx / (8 * RN), e = idx - ti * (8 * RN);
            const int row = e % RN, m = e / RN, n = (tile0 + ti) * RN + row;
            float s = 0.f;
            for (int r = 0; r < splits; ++r) s += slots[((size_t)r * tpc + ti) * (8 * RN) + e];
            float v = 0.f;
            if (m < M && n < N) {
                const size_t o = (size_t)m * N + n;
                v = reinterpret_cast<float*>(p.out)[o] + s;
                reinterpret_cast<float*>(p.out)[o] = v;
                p.next_x[o] = __float2bfloat16_rn(v * p.next_gain[n]);
            }
            float sq = v * v;
#pragma unroll
            for (int off = RN / 2; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
            if (row == 0 && tile0 + ti < n_tiles) p.next_ssq[(size_t)m * p.next_parts + tile0 + ti] = sq;
        }
        return;
    }
    for (int idx = threadIdx.x; idx < tpc * 8 * RN; idx += blockDim.x) {
        const int ti = idx / (8 * RN), e = idx - ti * (8 * RN);
        const int row = e % RN, m = e / RN, n = (tile0 + ti) * RN + row;
        if (m >= M || n >= N) continue;
        float s = 0.f;
        for (int r = 0; r < splits; ++r) s += slots[((size_t)r * tpc + ti) * (8 * RN) + e];
        const size_t o = (size_t)m * N + n;
        if (mode == KS_STORE_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(s);
        else if (mode == KS_STORE_F32) reinterpret_cast<float*>(p.out)[o] = s;
        else reinterpret_cast<float*>(p.out)[o] += s;
    }
}

struct KsPlan {
    int rn, splits, slice_blocks, tiles_per_cluster, clusters;
    size_t smem;
};

// How a product is cut: slices of K of equal size (at most 2,048); row tiles of 16 weight rows (64 KB
// of a tile's weights in flight per block: measured 8.5 us against 9.2 us with tiles of 8 rows on
// N 2,048 x K 8,192) unless N is so small that half the cluster slots would idle; as many tiles per
// cluster as leave two blocks per SM.
static bool ks_plan(int N, int K, KsPlan* plan) {
    const int k_blocks = (K + 63) / 64;
    const int splits = (k_blocks + KS_SLICE_BLOCKS - 1) / KS_SLICE_BLOCKS;
    if (splits < 2 || splits > KS_MAX_SPLITS) return false;
    const int slots = (2 * ni_sm_count()) / splits;               // clusters resident at once
    if (slots < 1) return false;
    const int rn = 2 * ((N + 15) / 16) >= slots ? 16 : 8;
    const int tiles = (N + rn - 1) / rn;
    const int tpc = (tiles + slots - 1) / slots;
    plan->rn = rn;
    plan->splits = splits;
    plan->slice_blocks = (k_blocks + splits - 1) / splits;
    plan->tiles_per_cluster = tpc;
    plan->clusters = (tiles + tpc - 1) / tpc;
    plan->smem = (size_t)splits * tpc * 8 * rn * sizeof(float);
    return plan->smem <= KS_MAX_SLOT_FLOATS * sizeof(float);
}

template <int RN, bool WARM, bool NEXT>
static int launch_ksplit(const KsParams& p, const KsPlan& plan, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.clusters * plan.splits);
    cfg.blockDim = dim3(KS_WARPS * 32);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = plan.splits;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_ksplit_kernel<RN, WARM, NEXT>, p);
    return e == cudaSuccess ? NI_OK : (int)e;
}

// 1 if ni_gemv_ksplit takes the product (M <= 8 rows, K a multiple of 8 that needs 2 to 8 slices of
// at most 2,048), else 0.
NI_EXPORT int ni_gemv_ksplit_supports(int M, int N, int K) {
    KsPlan plan;
    return M >= 1 && M <= 8 && N >= 1 && K >= 8 && K % 8 == 0 && ks_plan(N, K, &plan) ? 1 : 0;
}

// Row tiles of the output for these sizes (= partial sums per row of a handed-over norm), 0 if unsupported.
NI_EXPORT int ni_gemv_ksplit_out_tiles(int N, int K) {
    KsPlan plan;
    if (N < 1 || K < 8 || K % 8 || !ks_plan(N, K, &plan)) return 0;
    return (N + plan.rn - 1) / plan.rn;
}

// x bf16 [M, K], w bf16 [N, K].  mode: 0 store bf16 [M, N], 1 store FP32, 2 add into FP32.
// warm / warm_bytes: optional stretch of memory that the kernel asks into L2 on its way out.
// next_gain / next_x / next_ssq: with mode 2, also prepare the norm that follows (null: off).
NI_EXPORT int ni_gemv_ksplit(const void* x, const void* w, void* out, int M, int N, int K, int mode,
                             const void* warm, long long warm_bytes, const float* next_gain, void* next_x,
                             float* next_ssq, int next_parts, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return NI_OK;
    if (mode < KS_STORE_BF16 || mode > KS_ADD_F32) return NI_ERR_BAD_ARGUMENT;
    if (next_gain && (mode != KS_ADD_F32 || !next_x || !next_ssq)) return NI_ERR_BAD_ARGUMENT;
    if (warm_bytes < 0 || (warm_bytes & 15) || (warm_bytes && (!warm || ((uintptr_t)warm & 15)))) return NI_ERR_BAD_ARGUMENT;
    KsPlan plan;
    if (M > 8 || K <= 0 || K % 8 || !ks_plan(N, K, &plan)) return NI_ERR_UNSUPPORTED_SIZE;
    KsParams p = {};
    p.x = (const __nv_bfloat16*)x; p.w = (const __nv_bfloat16*)w; p.out = out;
    p.M = M; p.N = N; p.K = K; p.mode = mode;
    p.splits = plan.splits; p.slice_blocks = plan.slice_blocks; p.tiles_per_cluster = plan.tiles_per_cluster;
    p.warm = (const unsigned char*)warm; p.warm_bytes = (unsigned long long)warm_bytes;
    p.next_gain = next_gain; p.next_x = (__nv_bfloat16*)next_x; p.next_ssq = next_ssq; p.next_parts = next_parts;
    if (next_gain && (next_parts % 4 || next_parts < (N + plan.rn - 1) / plan.rn)) return NI_ERR_BAD_ARGUMENT;
#define KS_GO(RN)                                                                       \
    do {                                                                                \
        if (next_gain) {                                                                \
            if (warm_bytes) return launch_ksplit<RN, true, true>(p, plan, stream);      \
            return launch_ksplit<RN, false, true>(p, plan, stream);                     \
        }                                                                               \
        if (warm_bytes) return launch_ksplit<RN, true, false>(p, plan, stream);         \
        return launch_ksplit<RN, false, false>(p, plan, stream);                        \
    } while (0)
    if (plan.rn == 16) KS_GO(16);
    KS_GO(8);
#undef KS_GO
}
