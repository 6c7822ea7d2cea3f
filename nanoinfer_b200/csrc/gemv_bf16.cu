// Skinny matrix product for decode: y[M, N] = x[M, K] . W[N, K]^T with M <= 16 rows of
// activations against a large bfloat16 weight matrix - a bandwidth problem - with the
// neighbouring element-wise work fused into its two ends.
//
// "Swap AB": the weight rows are the M side of the tensor-core tile (mma.sync m16n8k16, bf16
// in, FP32 accumulate) and the batch is the 8-wide N side, so one pass over the weights serves
// the whole batch and the FP32 FMA pipes never become the limit.  A block owns 8 or 16 weight
// rows; its 8 warps split K and stream their slices from global memory straight into MMA
// fragments with 16-byte loads (the contraction index is permuted identically in both
// operands), several loads in flight per thread.  Partial sums meet in shared memory and are
// added in warp order, so a result never depends on timing.
//
// Input side:  bfloat16 activations, or the FP32 residual stream with RMSNorm fused in: the
//   gain is applied while the fragments are built, the sum of squares of each row is collected
//   from the very loads that feed the MMAs, and 1/rms is applied to the finished sums (it is a
//   per-row scalar, so it commutes with the product).  An index list can pick the rows.
// Output side: store bfloat16 | store FP32 (logits) | add into the FP32 residual stream |
//   SwiGLU (weight rows come in blocks of 8 gate rows + their 8 up rows) | rotary encoding and
//   the paged K/V write of a fused QKV projection (weight rows ordered so that the two
//   elements of a rotary pair are adjacent).
//
// The kernels are launched with programmatic stream serialisation: the first weight fragments
// are requested before griddepcontrol.wait, so a kernel's weight stream starts while the
// kernel before it drains; nothing that depends on the previous kernel is touched before the wait.
//
// Reference counterparts: cublasSgemm on FP32 weights for every projection
// (src/op/kernels/cuda/matmul_kernel.cu:48-89) and separate kernels for RMSNorm, RoPE, the cache
// write, SwiGLU and the residual add (src/model/llama.cpp:324-379).
#include "common.cuh"

#define GV_WARPS 8

#define GV_STORE_BF16 0
#define GV_STORE_F32 1
#define GV_ADD_F32 2
#define GV_SWIGLU 3
#define GV_ROPE_KV 4

struct GemvParams {
    const void* x;            // bf16 [M, K], or FP32 [*, K] with the norm fused
    const float* gain;        // norm: [K]
    const int* rows;          // norm: optional source row of each of the M rows
    float eps;
    const __nv_bfloat16* w;   // [N, K]
    void* out;
    int M, N, K, mode;
    // GV_ROPE_KV
    const int* positions;
    const int* seq_of_token;
    const int* block_table;
    const float* inv_freq;
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
    int bt_stride, n_q_heads, n_kv_heads, head_dim, rotary_dim, page_size, write_cache;
    // A norm handed from kernel to kernel (up to 8 rows; template parameter HAND).  Producer (HAND 2,
    // mode GV_ADD_F32): after out += product it also stores next_x = bf16(out * next_gain) and, per
    // tile of output columns and row, the sum of out^2 over the tile (next_ssq[row][tile]).  Consumer
    // (HAND 1; its bfloat16 input is such a next_x): 1/rms of each row from the pre_parts partial
    // sums, applied to the finished products (a per-row scalar commutes with the product).  Together
    // they are RMSNorm without a kernel of its own and without the consumer reading the FP32 stream.
    const float* next_gain;
    __nv_bfloat16* next_x;
    float* next_ssq;          // [8 rows][next_parts]: a row's partial sums lie together (parts: a multiple of 4; what no tile writes stays 0)
    int next_parts;
    const float* pre_ssq;     // [8 rows][pre_parts]
    int pre_parts;
    float pre_eps;
    // optional: bytes that kernels after this one read (weights), asked into L2 once this block has
    // issued its own last loads - they fill the gap between this kernel's tail and the next one's start
    const unsigned char* warm;
    unsigned long long warm_bytes;
};

__device__ __forceinline__ void gv_mma(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

// This block's share of the request to bring [p.warm, +p.warm_bytes) into L2, issued by one warp
// (addresses and sizes are multiples of 16 bytes).
__device__ __forceinline__ void gv_warm(const GemvParams& p) {
    constexpr unsigned int PIECE = 8192;
    const unsigned int n_pieces = (unsigned int)((p.warm_bytes + PIECE - 1) / PIECE);
    for (unsigned int i = blockIdx.x + (threadIdx.x & 31) * gridDim.x; i < n_pieces; i += 32 * gridDim.x) {
        const unsigned long long off = (unsigned long long)i * PIECE;
        const unsigned int sz = p.warm_bytes - off < PIECE ? (unsigned int)(p.warm_bytes - off) : PIECE;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(p.warm + off), "r"(sz) : "memory");
    }
}

// One lane's share of the sum of a row of n floats (n a multiple of 4, the row 16-byte aligned).
__device__ __forceinline__ float gv_row_sum(const float* row, int n, int lane) {
    float q = 0.f;
    for (int i = 4 * lane; i < n; i += 128) {
        const float4 v = *reinterpret_cast<const float4*>(row + i);
        q += (v.x + v.y) + (v.z + v.w);
    }
    return q;
}

// Builds the B fragment (8 activations of one batch row at k .. k+7) and, with the norm fused,
// adds their squares to ssq.
template <bool NORM>
__device__ __forceinline__ uint4 load_x8(const void* xrow, const float* gain8, int k, float& ssq) {
    if (NORM) {   // gain8: the gains of elements k .. k+7
        const float4 h0 = *reinterpret_cast<const float4*>((const float*)xrow + k);
        const float4 h1 = *reinterpret_cast<const float4*>((const float*)xrow + k + 4);
        const float4 g0 = *reinterpret_cast<const float4*>(gain8);
        const float4 g1 = *reinterpret_cast<const float4*>(gain8 + 4);
        ssq += h0.x * h0.x + h0.y * h0.y + h0.z * h0.z + h0.w * h0.w +
               h1.x * h1.x + h1.y * h1.y + h1.z * h1.z + h1.w * h1.w;
        return make_uint4(pack2(h0.x * g0.x, h0.y * g0.y), pack2(h0.z * g0.z, h0.w * g0.w),
                          pack2(h1.x * g1.x, h1.y * g1.y), pack2(h1.z * g1.z, h1.w * g1.w));
    }
    return *reinterpret_cast<const uint4*>((const __nv_bfloat16*)xrow + k);
}

// RN: weight rows per tile (8 or 16).  NT: batch tiles of 8 rows (1 or 2).  NORM: FP32 input +
// RMSNorm.  U: k-blocks of 64 a warp has in flight per pass (a pass of the block covers
// 64 * GV_WARPS * U of K).  KEEP: one pass covers K, the activations of a warp's K slice stay in
// registers and the block walks `tiles_per_block` consecutive row tiles with them, so that
// activations are read and normalised once per block, not once per 16 weight rows (U = 4 for K
// <= 2048 with two blocks per SM; U = 6 and 8 for K up to 3072 and 4096 with one).
// WARM: the kernel ends with its share of the request for p.warm (a variant of its own: the mere
// presence of that code after the loop made the gate/up kernel, which runs at its register limit,
// 6 % slower, whether or not it ran).
// HAND: 0, or 1 / 2 for the reader / the writer of a handed-over norm (see GemvParams) - variants of
// their own for the same reason.
template <int RN, int NT, bool NORM, bool KEEP, int U, bool WARM, int HAND>
__global__ void __launch_bounds__(GV_WARPS * 32, (NT == 1 && U <= 4) ? 2 : 1) gemv_bf16_kernel(const GemvParams p, int tiles_per_block, int long_blocks) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int M = p.M, N = p.N, K = p.K;
    const int n_blocks = (K + 63) / 64;            // k-blocks of 64
    const uint4 zero = make_uint4(0, 0, 0, 0);
    pdl_launch_dependents();

    __shared__ float red[GV_WARPS][NT][16][8];
    __shared__ float ss_red[GV_WARPS][NT * 8];
    __shared__ float tile[NT * 8][17];
    __shared__ float inv_rms[NT * 8];

    // KEEP with the norm fused: the gain does not depend on the kernel before this one, so each
    // warp stages the gains of its own K slice in shared memory before the wait; afterwards only
    // the residual rows come from memory.
    __shared__ __align__(16) float s_gain[(NORM && KEEP) ? GV_WARPS : 1][(NORM && KEEP) ? U * 64 : 4];
    static_assert(!KEEP || NT * U <= 8, "activation registers");
    if (NORM && KEEP) {
        for (int i = lane; i < U * 16; i += 32) {
            const int u = i >> 4, k = (warp + u * GV_WARPS) * 64 + 4 * (i & 15);
            if (k + 4 <= K) *reinterpret_cast<float4*>(&s_gain[warp][4 * i]) = *reinterpret_cast<const float4*>(p.gain + k);
        }
        __syncwarp();
    }

    // Fused QKV projection: the position and the cache page of every batch row are step metadata
    // (not written by the kernel before this one), so they are fetched now; in the epilogue the
    // chain position -> block-table entry -> address would cost two memory round trips.
    __shared__ int s_pos[NT * 8], s_page[NT * 8];
    if (p.mode == GV_ROPE_KV && threadIdx.x < NT * 8) {
        const int m = threadIdx.x;
        int pos = 0, page = 0;
        if (m < M) {
            pos = p.positions[m];
            if (p.write_cache) page = p.block_table[(size_t)p.seq_of_token[m] * p.bt_stride + pos / p.page_size];
        }
        s_pos[m] = pos;
        s_page[m] = page;
    }

    uint4 fx[U][NT][2];     // KEEP: this warp's activations, loaded once
    float ssq[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) ssq[nt] = 0.f;
    bool waited = false;
    float pre_q = 0.f;      // HAND 1: this lane's share of row `warp`'s partial sums of squares

    // This warp's weight fragments of one pass over K (U k-blocks of 64).
    uint4 fa[U][2], fb[U][2];
    auto load_weights = [&](int n0, int kb) {
        const bool row_a_ok = n0 + g < N;
        const bool row_b_ok = RN == 16 && n0 + g + 8 < N;
        const __nv_bfloat16* wa = p.w + (size_t)(row_a_ok ? n0 + g : 0) * K;
        const __nv_bfloat16* wb = p.w + (size_t)(row_b_ok ? n0 + g + 8 : 0) * K;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k0 = (kb + u * GV_WARPS) * 64;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int k = k0 + 32 * h + 8 * t;
                const bool ok = k + 8 <= K;        // K is a multiple of 8
                fa[u][h] = (ok && row_a_ok) ? ld_stream(wa + k) : zero;
                fb[u][h] = (RN == 16 && ok && row_b_ok) ? ld_stream(wb + k) : zero;
            }
        }
    };
    // KEEP: one pass covers K, so a tile is one batch of loads per warp; the batch of the NEXT tile
    // is issued right after this tile's MMAs (into the same registers), so that it is in flight
    // while this tile's partial sums go through shared memory and the epilogue.
    bool prefetched = false;

    // The first `long_blocks` blocks walk tiles_per_block row tiles, the others one fewer: with two
    // blocks per SM an SM then gets a long and a short block (the hardware fills every SM's first
    // slot before any second one) instead of some SMs two long ones and others a single block.
    const bool is_long = (int)blockIdx.x < long_blocks;
    // (kept as first row and end row: one register fewer than a tile counter and a tile count, and
    // this kernel's gate/up instance runs at its register limit)
    const int n_first = (is_long ? (int)blockIdx.x * tiles_per_block
                                 : long_blocks * tiles_per_block + ((int)blockIdx.x - long_blocks) * (tiles_per_block - 1)) * RN;
    const int n_end = min(N, n_first + (is_long ? tiles_per_block : tiles_per_block - 1) * RN);
    bool first_tile = true;
    for (int n0 = n_first; n0 < n_end; n0 += RN) {
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

        for (int kb = warp; kb < n_blocks; kb += GV_WARPS * U) {
            if (!prefetched) load_weights(n0, kb);
            prefetched = false;
            if (!waited) {
                // everything above reads weights (and the gain) only; what follows depends on the kernel before
                pdl_wait();
                waited = true;
                // a norm prepared by that kernel: this warp's share of its row's partial sums, requested
                // together with the activations below (its latency hides behind theirs)
                if (HAND == 1)
                    pre_q += gv_row_sum(p.pre_ssq + (size_t)warp * p.pre_parts, p.pre_parts, lane);
            }
            if (!KEEP || first_tile) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int m = 8 * nt + g;
                    const bool x_ok = m < M;
                    const int src = (NORM && p.rows && x_ok) ? p.rows[m] : (x_ok ? m : 0);
                    const void* xr = NORM ? (const void*)((const float*)p.x + (size_t)src * K)
                                          : (const void*)((const __nv_bfloat16*)p.x + (size_t)src * K);
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int k0 = (kb + u * GV_WARPS) * 64;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int k = k0 + 32 * h + 8 * t;
                            const float* gain8 = (NORM && KEEP) ? &s_gain[warp][u * 64 + 32 * h + 8 * t] : p.gain + k;
                            fx[u][nt][h] = (k + 8 <= K && x_ok) ? load_x8<NORM>(xr, gain8, k, ssq[nt]) : zero;
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        gv_mma(acc[nt], fa[u][h].x, fb[u][h].x, fa[u][h].y, fb[u][h].y, fx[u][nt][h].x, fx[u][nt][h].y);
                        gv_mma(acc[nt], fa[u][h].z, fb[u][h].z, fa[u][h].w, fb[u][h].w, fx[u][nt][h].z, fx[u][nt][h].w);
                    }
            if (KEEP && n0 + RN < n_end) {
                load_weights(n0 + RN, kb);      // (KEEP: this is the warp's only pass over K)
                prefetched = true;
            }
        }
        if (!waited) {                                // a warp without work must not run ahead either
            pdl_wait();
            waited = true;
            if (HAND == 1)
                pre_q += gv_row_sum(p.pre_ssq + (size_t)warp * p.pre_parts, p.pre_parts, lane);
        }
        // partial sums of the 8 warps -> shared memory -> summed in warp order
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            red[warp][nt][g][2 * t] = acc[nt][0];
            red[warp][nt][g][2 * t + 1] = acc[nt][1];
            red[warp][nt][g + 8][2 * t] = acc[nt][2];
            red[warp][nt][g + 8][2 * t + 1] = acc[nt][3];
            if (NORM && first_tile) {
                float s = ssq[nt];
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                if (t == 0) ss_red[warp][nt * 8 + g] = s;
            }
        }
        if (HAND == 1 && first_tile) {
            // warp w holds row w's partial sums (lanes took them in turn): a fixed shuffle tree adds them
            // up, in time for the barrier that the warps' partial products need anyway
            float q = pre_q;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) q += __shfl_xor_sync(0xffffffffu, q, off);
            if (lane == 0) inv_rms[warp] = 1.0f / sqrtf(q / (float)K + p.pre_eps);
        }
        __syncthreads();
        if (NORM && first_tile) {
            if (threadIdx.x < NT * 8) {
                float q = 0.f;
#pragma unroll
                for (int wi = 0; wi < GV_WARPS; ++wi) q += ss_red[wi][threadIdx.x];
                inv_rms[threadIdx.x] = 1.0f / sqrtf(q / (float)K + p.eps);
            }
            __syncthreads();
        }
        for (int idx = threadIdx.x; idx < NT * 8 * RN; idx += blockDim.x) {
            const int row = idx % RN;                  // weight row within the tile
            const int m = idx / RN;                    // batch row
            float s = 0.f;
#pragma unroll
            for (int wi = 0; wi < GV_WARPS; ++wi) s += red[wi][m >> 3][row][m & 7];
            if (NORM || HAND == 1) s *= inv_rms[m];
            tile[m][row] = s;
        }
        __syncthreads();

        const int mode = p.mode;
        if (HAND == 2) {
            // the addition, and with it what the next norm needs (see GemvParams); whole warps take part
            for (int idx = threadIdx.x; idx < 8 * RN; idx += blockDim.x) {
                const int row = idx % RN, m = idx / RN, n = n0 + row;
                const bool ok = m < M && n < N;
                float v = 0.f;
                if (ok) {
                    const size_t o = (size_t)m * N + n;
                    v = reinterpret_cast<float*>(p.out)[o] + tile[m][row];
                    reinterpret_cast<float*>(p.out)[o] = v;
                    p.next_x[o] = __float2bfloat16_rn(v * p.next_gain[n]);
                }
                float sq = v * v;
#pragma unroll
                for (int off = RN / 2; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
                if (row == 0) p.next_ssq[(size_t)m * p.next_parts + n0 / RN] = sq;
            }
        } else if (mode <= GV_ADD_F32) {
            for (int idx = threadIdx.x; idx < NT * 8 * RN; idx += blockDim.x) {
                const int row = idx % RN, m = idx / RN, n = n0 + row;
                if (m >= M || n >= N) continue;
                const float s = tile[m][row];
                const size_t o = (size_t)m * N + n;
                if (mode == GV_STORE_BF16) reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(s);
                else if (mode == GV_STORE_F32) reinterpret_cast<float*>(p.out)[o] = s;
                else reinterpret_cast<float*>(p.out)[o] += s;
            }
        } else if (mode == GV_SWIGLU) {
            // rows 0..7 of the tile: gate; rows 8..15: the matching up rows (RN == 16)
            for (int idx = threadIdx.x; idx < NT * 8 * 8; idx += blockDim.x) {
                const int r = idx & 7, m = idx >> 3;
                if (m >= M || n0 + r + 8 >= N) continue;
                const float gt = tile[m][r], up = tile[m][r + 8];
                reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * (N / 2) + (n0 >> 1) + r] =
                    __float2bfloat16_rn((gt / (1.0f + expf(-gt))) * up);
            }
        } else {  // GV_ROPE_KV: rows come in adjacent rotary pairs; a tile never straddles a head
            const int hd = p.head_dim, nq = p.n_q_heads, nkv = p.n_kv_heads;
            for (int idx = threadIdx.x; idx < NT * 8 * (RN / 2); idx += blockDim.x) {
                const int pr = idx % (RN / 2), m = idx / (RN / 2);
                const int n = n0 + 2 * pr;
                if (m >= M || n + 1 >= N) continue;
                const int head = n / hd, d = n - head * hd;
                float a = tile[m][2 * pr], b = tile[m][2 * pr + 1];
                const int pos = s_pos[m];
                if (head < nq + nkv && d < p.rotary_dim) {
                    float sn, cs;
                    sincosf((float)pos * p.inv_freq[d >> 1], &sn, &cs);
                    const float ra = a * cs - b * sn, rb = a * sn + b * cs;
                    a = ra; b = rb;
                }
                __nv_bfloat16* dst;
                if (head < nq) {
                    dst = reinterpret_cast<__nv_bfloat16*>(p.out) + ((size_t)m * nq + head) * hd + d;
                } else {
                    if (!p.write_cache) continue;
                    const int page = s_page[m];
                    const int kvh = head < nq + nkv ? head - nq : head - nq - nkv;
                    __nv_bfloat16* base = head < nq + nkv ? p.k_pages : p.v_pages;
                    dst = base + (((size_t)page * nkv + kvh) * p.page_size + (pos % p.page_size)) * hd + d;
                }
                *reinterpret_cast<uint32_t*>(dst) = pack2(a, b);
            }
        }
        first_tile = false;
    }
    if (!waited) pdl_wait();
    if (WARM && warp == GV_WARPS - 1) gv_warm(p);
}

template <int RN, int NT, bool NORM, bool KEEP, int U, bool WARM, int HAND>
static int launch_gemv_w(const GemvParams& p, int tiles_per_block, cudaStream_t stream) {
    const int tiles = (p.N + RN - 1) / RN;
    // as many blocks as fit the GPU at once (the dispatcher sized tiles_per_block for that), the
    // tiles dealt as evenly as they go: `long_blocks` blocks take tiles_per_block, the rest one fewer
    // (gate/up of the 1B sizes: 136 blocks of 4 tiles and 160 of 3 instead of 256 of 4; decode step at
    // batch 8 0.806 -> 0.796 ms, 3B 2.226 -> 2.194, 8B 3.746 -> 3.669; batch 1 0.728 -> 0.735)
    int grid = (tiles + tiles_per_block - 1) / tiles_per_block, long_blocks = grid;
    if (KEEP && tiles_per_block > 1) {
        const int slots = ((NT == 1 && U <= 4) ? 2 : 1) * ni_sm_count();
        grid = tiles < slots ? tiles : slots;
        long_blocks = tiles - grid * (tiles_per_block - 1);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(GV_WARPS * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_bf16_kernel<RN, NT, NORM, KEEP, U, WARM, HAND>, p, tiles_per_block, long_blocks);
    return e == cudaSuccess ? NI_OK : (int)e;
}

// True for the template instances that exist with HAND != 0: up to 8 rows of bfloat16 activations kept
// in registers; the reader with 16-row tiles (gate/up, fused QKV), the writer with K <= 2,048 (longer
// contractions add through gemv_ksplit.cu).
template <int RN, int NT, bool NORM, bool KEEP, int U> constexpr bool gv_reads_handoff() { return NT == 1 && !NORM && KEEP && RN == 16; }
template <int RN, int NT, bool NORM, bool KEEP, int U> constexpr bool gv_writes_handoff() { return NT == 1 && !NORM && KEEP && U == 4; }

template <int RN, int NT, bool NORM, bool KEEP, int U>
static int launch_gemv(const GemvParams& p, int tiles_per_block, cudaStream_t stream) {
    if (p.pre_ssq) {
        if (!gv_reads_handoff<RN, NT, NORM, KEEP, U>()) return NI_ERR_UNSUPPORTED_SIZE;
        return launch_gemv_w<RN, NT, NORM, KEEP, U, false, gv_reads_handoff<RN, NT, NORM, KEEP, U>() ? 1 : 0>(p, tiles_per_block, stream);
    }
    if (p.next_gain) {
        if (!gv_writes_handoff<RN, NT, NORM, KEEP, U>() || p.mode != GV_ADD_F32) return NI_ERR_UNSUPPORTED_SIZE;
        constexpr int H = gv_writes_handoff<RN, NT, NORM, KEEP, U>() ? 2 : 0;
        if (p.warm_bytes) return launch_gemv_w<RN, NT, NORM, KEEP, U, H == 2, H>(p, tiles_per_block, stream);
        return launch_gemv_w<RN, NT, NORM, KEEP, U, false, H>(p, tiles_per_block, stream);
    }
    // the variant that asks for p.warm exists for up to 8 rows of bfloat16 activations (what the
    // engine's hints go to: a mixer's output projection, a down projection); elsewhere the hint is dropped
    if (NT == 1 && !NORM && p.warm_bytes) return launch_gemv_w<RN, NT, NORM, KEEP, U, NT == 1 && !NORM, 0>(p, tiles_per_block, stream);
    return launch_gemv_w<RN, NT, NORM, KEEP, U, false, 0>(p, tiles_per_block, stream);
}

static int dispatch_gemv(const GemvParams& p, bool norm, cudaStream_t stream) {
    if (p.M <= 0 || p.N <= 0) return NI_OK;
    if (p.K <= 0 || p.mode < 0 || p.mode > GV_ROPE_KV) return NI_ERR_BAD_ARGUMENT;
    if (p.M > 16 || p.K % 8) return NI_ERR_UNSUPPORTED_SIZE;
    // 16 rows per tile unless that leaves SMs idle; the fused epilogues need whole 16-row tiles
    const bool rn16 = p.mode >= GV_SWIGLU || (p.N + 15) / 16 >= 2 * ni_sm_count();
    if (p.mode == GV_SWIGLU && p.N % 16) return NI_ERR_UNSUPPORTED_SIZE;
    if (p.mode == GV_ROPE_KV && (p.head_dim % 16 || p.rotary_dim % 2 ||
                                 p.N != (p.n_q_heads + 2 * p.n_kv_heads) * p.head_dim))
        return NI_ERR_BAD_ARGUMENT;
    const bool one = p.M <= 8;
    // Activations stay in registers when one unrolled pass covers K: up to 2048 with four k-blocks
    // per warp in flight (two blocks per SM; one with two batch tiles, whose registers allow no
    // more), up to 3072 and 4096 with six and eight (one batch tile, one block per SM).  Then a
    // block takes several row tiles, as many as leave that many blocks per SM, and reads and
    // normalises the activations once.
    const int unroll = p.K <= 64 * GV_WARPS * 4 ? 4 : p.K <= 64 * GV_WARPS * 6 ? 6 : 8;
    const bool keep = p.K <= 64 * GV_WARPS * 4 || (one && p.K <= 64 * GV_WARPS * 8);
    int tpb = 1;
    if (keep) {
        const int tiles = (p.N + (rn16 ? 16 : 8) - 1) / (rn16 ? 16 : 8);
        const int blocks = ((one && unroll == 4) ? 2 : 1) * ni_sm_count();
        tpb = (tiles + blocks - 1) / blocks;
        if (tpb < 1) tpb = 1;
    }
#define GO(RN, NT, NORM, KEEP, U) return launch_gemv<RN, NT, NORM, KEEP, U>(p, tpb, stream)
#define GO_KEEP1(U)                                                                              \
    do {                                                                                         \
        if (norm) { if (rn16) GO(16, 1, true, true, U); else GO(8, 1, true, true, U); }          \
        else { if (rn16) GO(16, 1, false, true, U); else GO(8, 1, false, true, U); }             \
    } while (0)
    if (keep && one) {
        if (unroll == 4) GO_KEEP1(4);
        if (unroll == 6) GO_KEEP1(6);
        GO_KEEP1(8);
    }
    if (keep) {
        if (norm) { if (rn16) GO(16, 2, true, true, 4); else GO(8, 2, true, true, 4); }
        else { if (rn16) GO(16, 2, false, true, 4); else GO(8, 2, false, true, 4); }
    }
    if (norm) {
        if (rn16) { if (one) GO(16, 1, true, false, 4); else GO(16, 2, true, false, 4); }
        else { if (one) GO(8, 1, true, false, 4); else GO(8, 2, true, false, 4); }
    }
    if (rn16) { if (one) GO(16, 1, false, false, 4); else GO(16, 2, false, false, 4); }
    if (one) GO(8, 1, false, false, 4); else GO(8, 2, false, false, 4);
#undef GO_KEEP1
#undef GO
}

// x bf16 [M, K].  mode: 0 store bf16 [M, N], 1 store FP32, 2 add into FP32, 3 SwiGLU -> bf16 [M, N / 2].
static bool gv_warm_ok(const void* warm, long long bytes) {
    return bytes >= 0 && !(bytes & 15) && (bytes == 0 || (warm && !((uintptr_t)warm & 15)));
}

// Row tiles of ni_gemv_bf16's output (= partial sums per row that the writer of a handed-over norm stores).
NI_EXPORT int ni_gemv_bf16_out_tiles(int N, int mode) {
    const bool rn16 = mode >= GV_SWIGLU || (N + 15) / 16 >= 2 * ni_sm_count();
    return rn16 ? (N + 15) / 16 : (N + 7) / 8;
}
// 1 if ni_gemv_bf16 can write a handed-over norm while adding [M, N] (inner size K) / read one on an input of width K.
NI_EXPORT int ni_gemv_bf16_writes_handoff(int M, int N, int K) { return M >= 1 && M <= 8 && N >= 1 && K >= 8 && K % 8 == 0 && K <= 64 * GV_WARPS * 4; }
NI_EXPORT int ni_gemv_bf16_reads_handoff(int M, int K) { return M >= 1 && M <= 8 && K >= 8 && K % 8 == 0 && K <= 64 * GV_WARPS * 8; }

// next_gain / next_x / next_ssq: with mode 2, also prepare the norm that follows (see GemvParams);
// pre_ssq / pre_parts / pre_eps: x is such a prepared input.  Null pointers switch either off; sizes for
// which the variant does not exist are refused (-2).
NI_EXPORT int ni_gemv_bf16(const void* x, const void* w, void* out, int M, int N, int K, int mode,
                           const void* warm, long long warm_bytes, const float* next_gain, void* next_x,
                           float* next_ssq, int next_parts, const float* pre_ssq, int pre_parts, float pre_eps,
                           cudaStream_t stream) {
    if (mode == GV_ROPE_KV || !gv_warm_ok(warm, warm_bytes)) return NI_ERR_BAD_ARGUMENT;
    if (next_gain && (mode != GV_ADD_F32 || !next_x || !next_ssq || pre_ssq || next_parts % 4 ||
                      next_parts < ni_gemv_bf16_out_tiles(N, mode)))
        return NI_ERR_BAD_ARGUMENT;
    if (pre_ssq && (pre_parts <= 0 || pre_parts % 4 || ((uintptr_t)pre_ssq & 15))) return NI_ERR_BAD_ARGUMENT;
    if (pre_ssq && mode != GV_SWIGLU && (N + 15) / 16 < 2 * ni_sm_count()) return NI_ERR_UNSUPPORTED_SIZE;   // (the reader has 16-row tiles)
    GemvParams p = {};
    p.next_gain = next_gain; p.next_x = (__nv_bfloat16*)next_x; p.next_ssq = next_ssq; p.next_parts = next_parts;
    p.pre_ssq = pre_ssq; p.pre_parts = pre_parts; p.pre_eps = pre_eps;
    p.warm = (const unsigned char*)warm; p.warm_bytes = (unsigned long long)warm_bytes;
    p.x = x; p.w = (const __nv_bfloat16*)w; p.out = out; p.M = M; p.N = N; p.K = K; p.mode = mode;
    return dispatch_gemv(p, false, stream);
}

// h FP32 [*, K] with RMSNorm fused: y = (norm(h[rows]) * gain) . w^T.  rows may be null (rows 0..M-1).
NI_EXPORT int ni_gemv_norm_bf16(const float* h, const float* gain, float eps, const int* rows, const void* w,
                                void* out, int M, int N, int K, int mode, const void* warm, long long warm_bytes,
                                cudaStream_t stream) {
    if (mode == GV_ROPE_KV || !gv_warm_ok(warm, warm_bytes)) return NI_ERR_BAD_ARGUMENT;
    GemvParams p = {};
    p.warm = (const unsigned char*)warm; p.warm_bytes = (unsigned long long)warm_bytes;
    p.x = h; p.gain = gain; p.eps = eps; p.rows = rows; p.w = (const __nv_bfloat16*)w; p.out = out;
    p.M = M; p.N = N; p.K = K; p.mode = mode;
    return dispatch_gemv(p, true, stream);
}

// Fused QKV projection of single tokens with RMSNorm in front and rotary encoding + paged K/V
// write behind: q (rotated) -> q_out bf16 [M, Hq * hd]; k (rotated), v -> their page slots.
// The weight rows of q and k must be ordered with rotary pairs adjacent (2i, 2i + 1).
// h may instead be bf16 activations when gain is null (no norm).
NI_EXPORT int ni_gemv_qkv_rope(const void* x, const float* gain, float eps, const void* w, void* q_out,
                               void* k_pages, void* v_pages, const int* positions, const int* seq_of_token,
                               const int* block_table, int bt_stride, const float* inv_freq, int M, int K,
                               int n_q_heads, int n_kv_heads, int head_dim, int rotary_dim, int page_size,
                               int write_cache, const void* warm, long long warm_bytes, const float* pre_ssq,
                               int pre_parts, float pre_eps, cudaStream_t stream) {
    if (!gv_warm_ok(warm, warm_bytes)) return NI_ERR_BAD_ARGUMENT;
    if (pre_ssq && (gain != nullptr || pre_parts <= 0 || pre_parts % 4 || ((uintptr_t)pre_ssq & 15))) return NI_ERR_BAD_ARGUMENT;
    GemvParams p = {};
    p.pre_ssq = pre_ssq; p.pre_parts = pre_parts; p.pre_eps = pre_eps;
    p.warm = (const unsigned char*)warm; p.warm_bytes = (unsigned long long)warm_bytes;
    p.x = x; p.gain = gain; p.eps = eps; p.w = (const __nv_bfloat16*)w; p.out = q_out;
    p.M = M; p.N = (n_q_heads + 2 * n_kv_heads) * head_dim; p.K = K; p.mode = GV_ROPE_KV;
    p.positions = positions; p.seq_of_token = seq_of_token; p.block_table = block_table; p.bt_stride = bt_stride;
    p.inv_freq = inv_freq; p.k_pages = (__nv_bfloat16*)k_pages; p.v_pages = (__nv_bfloat16*)v_pages;
    p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.rotary_dim = rotary_dim;
    p.page_size = page_size; p.write_cache = write_cache;
    return dispatch_gemv(p, gain != nullptr, stream);
}
