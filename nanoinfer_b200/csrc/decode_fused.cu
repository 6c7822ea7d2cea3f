// One decode step of a pre-norm attention + SwiGLU decoder as ONE persistent kernel: embedding,
// every layer (RMSNorm -> fused QKV projection -> rotary encoding + paged K/V write -> split-K
// grouped-query attention over the paged cache -> output projection + residual -> RMSNorm ->
// gate/up projection + SwiGLU -> down projection + residual), final norm and the projection onto
// the vocabulary, for up to 8 single query tokens.
//
// Why one kernel: at these sizes a decode step is a chain of ~80 products of 3-15 us each, and what
// it costs is not bandwidth inside the kernels but the ramp and the tail of every one of them.
// Here the weights of ALL layers are one stream that never stops:
//
//   * one block per SM (cooperative launch), 8 consumer warps + 1 loader warp;
//   * every weight matrix is cut by rows into one contiguous share per block (+-1 unit, so every
//     SM streams the same number of bytes); the loader warp walks its block's shares of all
//     matrices of all layers in order and copies them, 16 rows x 512 columns at a time, with
//     cp.async.bulk (TMA, no tensor map needed for contiguous row segments) into a ring of shared-
//     memory stages guarded by mbarriers.  It runs ahead of the consumers by the depth of the ring
//     (150 KB per SM, 22 MB over the GPU), across layer and phase boundaries: while the consumers
//     sit at a grid barrier or run attention, the next projections' weights are already landing;
//   * the consumer warps split a stage's columns, multiply with mma.sync (weights on the 16-row
//     side, the batch on the 8-wide side, FP32 accumulate), add their partial sums in warp order
//     through shared memory and run the epilogue (rotary + cache write, residual add, SwiGLU,
//     logits).  Each output element is owned by one block: no atomics on data, results do not
//     depend on timing;
//   * activations pass from phase to phase through global memory (L2) and a grid barrier: a
//     counter that every block increments and polls (bounded).  Attention runs between two such
//     barriers on the same blocks: the (token, kv head) pairs' keys are cut into 64-key units, each
//     block takes a contiguous run of units, partial results of a pair are merged, in order, by
//     the block that finishes last (atomic ticket, no waiting).
//
// Every wait (grid barrier, ring stages) is bounded in clock ticks; a wait that runs out writes a
// code to the error word, raises the block's abort flag, the loader waits (bounded) for its copies
// in flight, and the kernel returns.  Blocks wait for each other only inside this one cooperative
// launch, which guarantees that they are all resident.
//
// Reference counterpart: the per-layer loop of src/model/llama.cpp:297-389, one cuBLAS call or
// element-wise kernel per line of it, FP32.
#include <cooperative_groups.h>

#include "common.cuh"

#define FD_CONSUMER_WARPS 8
#define FD_CONSUMERS (FD_CONSUMER_WARPS * 32)
#define FD_THREADS (FD_CONSUMERS + 32)
#define FD_KT 512                                  // columns of a ring tile
#define FD_ROW_BYTES (FD_KT * 2 + 16)              // padded: ldmatrix rows fall into different banks
#define FD_STAGE_BYTES (16 * FD_ROW_BYTES)
#define FD_STAGES 9
#define FD_RING_BYTES (FD_STAGES * FD_STAGE_BYTES)
#define FD_WORK_BYTES (68 * 1024)                  // activations of a phase / K and V segments / merge buffer
#define FD_RED_FLOATS (2 * FD_CONSUMER_WARPS * 16 * 8)
#define FD_SMEM_BYTES (FD_RING_BYTES + FD_WORK_BYTES + FD_RED_FLOATS * 4 + 512)
#define FD_MAX_ROWS 8
#define FD_MAX_GROUPS 4

#define FD_ERR_BARRIER 31
#define FD_ERR_LOADER 32
#define FD_ERR_CONSUMER 33

typedef __nv_bfloat16 bf16;

// Pointers first, then 4-byte fields: the Python side mirrors these two records with ctypes.
struct FdLayer {
    const bf16* w_qkv;      // [(Hq + 2 Hkv) hd, d], rotary pairs adjacent
    const bf16* w_o;        // [d, Hq hd]
    const bf16* w_gate_up;  // [2 I, d], blocks of 8 gate rows + their 8 up rows
    const bf16* w_down;     // [d, I]
    const float* gain_mixer;
    const float* gain_ffn;
    bf16* k_pages;          // [P, Hkv, page, hd]
    bf16* v_pages;
    float eps_mixer, eps_ffn;
    int write_cache;        // 0: this run reads another run's cache
    int group;              // which block table
};

struct FdParams {
    const FdLayer* layers;
    const float* inv_freq;       // [rotary_dim / 2]
    const bf16* embedding;       // [V, d]
    const bf16* lm_head;         // [V, d]
    const float* gain_final;
    const int* tokens;           // [M]
    const int* positions;        // [M]
    const int* seq_of_token;     // [M]
    const int* logit_rows;       // [R] rows of the step whose logits are wanted
    const int* tables[FD_MAX_GROUPS];
    float* h;                    // [M, d] residual stream
    bf16* q;                     // [M, Hq hd]
    bf16* att;                   // [M, Hq hd]
    bf16* act;                   // [M, I]
    float* logits;               // [R, V]
    float* partials;             // attention: (blocks + M Hkv) x 16 x (hd + 2)
    int* tickets;                // attention: M Hkv (zeroed by the kernel)
    unsigned* barrier;           // one word; set to zero before the launch
    int* error;
    long long wait_limit;        // clock ticks
    int bt_stride[FD_MAX_GROUPS];
    int n_layers, M, R, d, n_q_heads, n_kv_heads, head_dim, rotary_dim, inter, vocab, page_size, window;
    float scale_log2e, eps_final;
    int skip_arrive_at;          // tests: block 0 leaves out its arrival at this barrier (-1: never)
};

// ---- small PTX helpers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t fd_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fd_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(fd_smem(bar)), "r"(count));
}
__device__ __forceinline__ void fd_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(fd_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fd_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(fd_smem(bar)) : "memory");
}
__device__ __forceinline__ bool fd_mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(fd_smem(bar)), "r"(parity) : "memory");
    return done != 0;
}
// Bounded wait; also gives up when the block's abort flag is up.  false: gave up.
__device__ __forceinline__ bool fd_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, long long limit) {
    if (fd_mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    long long start = 0;
    for (int iter = 1;; ++iter) {
        if (fd_mbar_try(bar, parity)) return true;
        if ((iter & 255) == 0) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (start == 0) start = now;
            if (now - start > limit) return false;
        }
    }
}
__device__ __forceinline__ void fd_bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(fd_smem(dst)), "l"(src), "r"(bytes), "r"(fd_smem(bar)) : "memory");
}
__device__ __forceinline__ void fd_bar() { asm volatile("bar.sync 1, %0;\n" ::"n"(FD_CONSUMERS) : "memory"); }
__device__ __forceinline__ void fd_cp16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(fd_smem(smem)), "l"(gmem));
}
__device__ __forceinline__ void fd_cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void fd_cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void fd_ldsm_x4(uint32_t r[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void fd_ldsm_x2(uint32_t r[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void fd_ldsm_x1(uint32_t& r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x1.shared.b16 {%0}, [%1];\n" : "=r"(r) : "r"(addr));
}
__device__ __forceinline__ void fd_ldsm_x4_trans(uint32_t r[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void fd_mma16(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void fd_mma8(float c[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ float fd_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned fd_ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t fd_pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---- how a matrix is shared out --------------------------------------------------------------------
// Rows [r0, r1) of an [N, K] matrix for block b of nb: N / gran units, as even as integers allow.
__device__ __forceinline__ void fd_rows(int N, int gran, int b, int nb, int& r0, int& r1) {
    const long long units = N / gran;
    r0 = (int)(units * b / nb) * gran;
    r1 = (int)(units * (b + 1) / nb) * gran;
}
// Columns of activations kept in shared memory at a time: all of K when 8 padded rows of it fit
// the work area, else 2048 in each of two buffers.
__device__ __forceinline__ int fd_chunk(int K) { return 8 * (K * 2 + 16) <= FD_WORK_BYTES ? K : 2048; }

struct FdShared {
    unsigned char* ring;
    unsigned char* work;
    float* red;              // [2][warps][16][8]
    uint64_t* full;          // [FD_STAGES]
    uint64_t* empty;
    float* rstd;             // [8]
    volatile int* abort_flag;
    int* flag;               // "this block arrived last" of the attention merge
};

struct FdRing {              // a consumer's or the loader's place in the ring
    int stage;
    uint32_t phase;
    __device__ __forceinline__ void advance() { if (++stage == FD_STAGES) { stage = 0; phase ^= 1; } }
};

// ---- the loader warp -------------------------------------------------------------------------------
__device__ bool fd_load_matrix(const FdParams& p, const FdShared& s, FdRing& ring, const bf16* W, int N, int K, int gran,
                               int lane) {
    int r0, r1;
    fd_rows(N, gran, blockIdx.x, gridDim.x, r0, r1);
    for (int rg = r0; rg < r1; rg += 16) {
        const int rows = min(16, r1 - rg);
        for (int k0 = 0; k0 < K; k0 += FD_KT) {
            const int cols = min(FD_KT, K - k0);
            if (!fd_mbar_wait(&s.empty[ring.stage], ring.phase ^ 1, s.abort_flag, p.wait_limit)) {
                if (lane == 0 && !*s.abort_flag) { atomicCAS(p.error, 0, FD_ERR_LOADER); *s.abort_flag = 1; }
                return false;
            }
            if (lane == 0) fd_mbar_expect_tx(&s.full[ring.stage], (uint32_t)(rows * cols * 2));
            __syncwarp();
            if (lane < rows)
                fd_bulk_copy(s.ring + (size_t)ring.stage * FD_STAGE_BYTES + lane * FD_ROW_BYTES,
                             W + (size_t)(rg + lane) * K + k0, (uint32_t)(cols * 2), &s.full[ring.stage]);
            ring.advance();
        }
    }
    return true;
}

__device__ void fd_loader(const FdParams& p, const FdShared& s, int lane) {
    FdRing ring = {0, 0};
    const int qkv_rows = (p.n_q_heads + 2 * p.n_kv_heads) * p.head_dim, q_dim = p.n_q_heads * p.head_dim;
    bool ok = true;
    for (int l = 0; l < p.n_layers && ok; ++l) {
        const FdLayer& L = p.layers[l];
        ok = fd_load_matrix(p, s, ring, L.w_qkv, qkv_rows, p.d, 2, lane) &&
             fd_load_matrix(p, s, ring, L.w_o, p.d, q_dim, 1, lane) &&
             fd_load_matrix(p, s, ring, L.w_gate_up, 2 * p.inter, p.d, 16, lane) &&
             fd_load_matrix(p, s, ring, L.w_down, p.d, p.inter, 1, lane);
    }
    if (ok && p.R > 0) ok = fd_load_matrix(p, s, ring, p.lm_head, p.vocab, p.d, 1, lane);
    if (!ok) {
        // Gave up: the copies already issued still land in this block's shared memory.  Wait (bounded) until
        // every stage's pending fill has completed before the block may end.  A stage whose current
        // phase has no fill pending completes nothing; its wait simply runs out of tries at once.
        for (int st = 0; st < FD_STAGES; ++st) {
            const uint32_t par = st < ring.stage ? ring.phase : ring.phase ^ 1;   // parity of the stage's last fill
            long long start = clock64();
            while (!fd_mbar_try(&s.full[st], par)) {
                if (clock64() - start > p.wait_limit) break;
            }
        }
    }
}

// ---- consumers: grid barrier -------------------------------------------------------------------------
// Every block's consumers arrive; the counter only grows within a launch (the host zeroes it
// before), so barrier number i is passed when it reaches (i + 1) * blocks.  A block that gave up goes straight through.
__device__ void fd_grid_sync(const FdParams& p, const FdShared& s, int& n_passed) {
    fd_bar();
    if (threadIdx.x == 0 && !*s.abort_flag) {
        const unsigned target = (unsigned)(n_passed + 1) * gridDim.x;
        __threadfence();
        if (!(blockIdx.x == 0 && p.skip_arrive_at == n_passed)) atomicAdd(p.barrier, 1u);
        long long start = 0;
        for (int iter = 0; fd_ld_acquire(p.barrier) < target; ++iter) {
            if ((iter & 63) == 63) {
                const long long now = clock64();
                if (start == 0) start = now;
                if (now - start > p.wait_limit || *reinterpret_cast<volatile int*>(p.error) != 0) {
                    atomicCAS(p.error, 0, FD_ERR_BARRIER);
                    *s.abort_flag = 1;
                    break;
                }
            }
        }
        __threadfence();
    }
    ++n_passed;
    fd_bar();
}

// ---- consumers: activations of a phase into shared memory ---------------------------------------------
// 1 / rms of each of the phase's rows (one warp per row), from the FP32 residual stream.
__device__ void fd_row_rstd(const FdParams& p, const FdShared& s, const int* rows, int n_rows, float eps, int warp, int lane) {
    if (warp < n_rows) {
        const float* src = p.h + (size_t)(rows ? rows[warp] : warp) * p.d;
        float ss = 0.f;
        for (int i = lane * 4; i < p.d; i += 128) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + i));
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = ni_warp_sum(ss);
        if (lane == 0) s.rstd[warp] = rsqrtf(ss / (float)p.d + eps);
    }
}
// norm(h[rows])[:, c0 : c0 + n] * gain as bfloat16 into buffer `dst` (row stride `stride` bytes).
__device__ void fd_act_norm(const FdParams& p, const FdShared& s, unsigned char* dst, int stride, const int* rows, int n_rows,
                            const float* gain, int c0, int n, int warp, int lane) {
    if (warp < n_rows) {
        const float* src = p.h + (size_t)(rows ? rows[warp] : warp) * p.d + c0;
        const float r = s.rstd[warp];
        for (int i = lane * 4; i < n; i += 128) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + i));
            const float4 g = *reinterpret_cast<const float4*>(gain + c0 + i);
            uint2 o;
            o.x = fd_pack2(v.x * r * g.x, v.y * r * g.y);
            o.y = fd_pack2(v.z * r * g.z, v.w * r * g.w);
            *reinterpret_cast<uint2*>(dst + (size_t)warp * stride + i * 2) = o;
        }
    }
}
// src[0 .. n_rows)[c0 : c0 + n] (bfloat16, row length K) into buffer `dst`, asynchronously.
__device__ void fd_act_copy(unsigned char* dst, int stride, const bf16* src, int K, int n_rows, int c0, int n) {
    const int per_row = n / 8;                     // 16-byte pieces
    for (int i = threadIdx.x; i < n_rows * per_row; i += FD_CONSUMERS) {
        const int r = i / per_row, c = i - r * per_row;
        fd_cp16(dst + (size_t)r * stride + c * 16, src + (size_t)r * K + c0 + c * 8);
    }
}

enum { FD_IN_NORM = 0, FD_IN_BF16 = 1 };
enum { FD_OUT_QKV = 0, FD_OUT_ADD = 1, FD_OUT_SWIGLU = 2, FD_OUT_LOGITS = 3 };

struct FdInput {
    int kind;
    const bf16* src;       // FD_IN_BF16: [n_rows, K]
    const int* rows;       // FD_IN_NORM: optional row list
    const float* gain;
    float eps;
    int n_rows;
};

// ---- consumers: one projection ---------------------------------------------------------------------
// A wait that runs out does not change the control flow: the warp records the error, raises the
// block's abort flag and goes on through the same loops and block barriers without data (every
// later wait returns at once), so that no warp is ever left alone at a barrier.
template <int OUT>
__device__ void fd_project(const FdParams& p, const FdShared& s, FdRing& ring, int& red_buf, const FdInput& in,
                           const FdLayer* L, int N, int K, int gran) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    int r0, r1;
    fd_rows(N, gran, blockIdx.x, gridDim.x, r0, r1);
    const int Kc = fd_chunk(K);
    const bool chunked = Kc < K;
    const int stride = Kc * 2 + 16;
    if (in.kind == FD_IN_NORM) {
        fd_row_rstd(p, s, in.rows, in.n_rows, in.eps, warp, lane);
        __syncwarp();
    }
    int resident = -1;                                        // chunk that lies in the work area
    for (int rg = r0; rg < r1; rg += 16) {
        const int rows = min(16, r1 - rg);
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        for (int c0 = 0; c0 < K; c0 += Kc) {
            const int chunk = c0 / Kc, cn = min(Kc, K - c0);
            unsigned char* act = s.work + (chunked ? (chunk & 1) * 8 * stride : 0);
            if (chunk != resident) {
                // (chunked: every warp is past the chunk before last, whose buffer the prefetch overwrites)
                if (chunked) fd_bar();
                if (in.kind == FD_IN_NORM) {
                    fd_act_norm(p, s, act, stride, in.rows, in.n_rows, in.gain, c0, cn, warp, lane);
                } else {
                    if (!chunked || resident < 0 || chunk != resident + 1) { fd_act_copy(act, stride, in.src, K, in.n_rows, c0, cn); fd_cp_commit(); }
                    if (chunked && c0 + Kc < K) {             // the next chunk streams in under this one
                        fd_act_copy(s.work + ((chunk + 1) & 1) * 8 * stride, stride, in.src, K, in.n_rows, c0 + Kc, min(Kc, K - c0 - Kc));
                        fd_cp_commit();
                        fd_cp_wait<1>();
                    } else {
                        fd_cp_wait<0>();
                    }
                }
                fd_bar();
                resident = chunk;
            }
            for (int k0 = c0; k0 < c0 + cn; k0 += FD_KT) {
                const int cols = min(FD_KT, c0 + cn - k0);
                const bool landed = fd_mbar_wait(&s.full[ring.stage], ring.phase, s.abort_flag, p.wait_limit);
                if (!landed && lane == 0 && !*s.abort_flag) { atomicCAS(p.error, 0, FD_ERR_CONSUMER); *s.abort_flag = 1; }
                const int kw = warp * 64;
                if (landed && kw < cols) {
                    const int n = min(64, cols - kw);
                    const uint32_t a_base = fd_smem(s.ring + (size_t)ring.stage * FD_STAGE_BYTES + (lane & 15) * FD_ROW_BYTES) +
                                            (kw + (lane >> 4) * 8) * 2;
                    const uint32_t b_base = fd_smem(act + (size_t)(lane & 7) * stride) + ((k0 - c0) + kw + ((lane >> 3) & 1) * 8) * 2;
                    int kk = 0;
#pragma unroll 4
                    for (; kk + 16 <= n; kk += 16) {
                        uint32_t a[4], b[2];
                        fd_ldsm_x4(a, a_base + kk * 2);
                        fd_ldsm_x2(b, b_base + kk * 2);
                        fd_mma16(c, a, b[0], b[1]);
                    }
                    if (kk < n) {                             // K = 8 (mod 16): one step of eight columns
                        uint32_t a[2], b;
                        fd_ldsm_x2(a, fd_smem(s.ring + (size_t)ring.stage * FD_STAGE_BYTES + (lane & 15) * FD_ROW_BYTES) + (kw + kk) * 2);
                        fd_ldsm_x1(b, fd_smem(act + (size_t)(lane & 7) * stride) + ((k0 - c0) + kw + kk) * 2);
                        fd_mma8(c, a[0], a[1], b);
                    }
                }
                __syncwarp();
                if (lane == 0) fd_mbar_arrive(&s.empty[ring.stage]);
                ring.advance();
            }
        }
        // ---- the warps' partial sums meet in shared memory; added in warp order ----
        float* red = s.red + red_buf * (FD_CONSUMER_WARPS * 128);
        red_buf ^= 1;
        float* mine = red + warp * 128;
        mine[g * 8 + 2 * t] = c[0];
        mine[g * 8 + 2 * t + 1] = c[1];
        mine[(g + 8) * 8 + 2 * t] = c[2];
        mine[(g + 8) * 8 + 2 * t + 1] = c[3];
        fd_bar();
        auto total = [&](int row, int tok) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < FD_CONSUMER_WARPS; ++w) v += red[w * 128 + row * 8 + tok];
            return v;
        };
        if (OUT == FD_OUT_QKV) {
            if (tid < 64) {
                const int row = 2 * (tid >> 3), tok = tid & 7;
                if (row < rows && tok < p.M) {
                    float v0 = total(row, tok), v1 = total(row + 1, tok);
                    const int n = rg + row, hd = p.head_dim;
                    const int q_dim = p.n_q_heads * hd, kv_dim = p.n_kv_heads * hd;
                    const int pos = p.positions[tok];
                    const int dh = n % hd;
                    if (n < q_dim + kv_dim && dh < p.rotary_dim) {
                        float sn, cs;
                        sincosf((float)pos * p.inv_freq[dh >> 1], &sn, &cs);
                        const float a = v0 * cs - v1 * sn, b = v0 * sn + v1 * cs;
                        v0 = a;
                        v1 = b;
                    }
                    if (n < q_dim) {
                        *reinterpret_cast<uint32_t*>(p.q + (size_t)tok * q_dim + n) = fd_pack2(v0, v1);
                    } else if (L->write_cache) {
                        const int kv = n - q_dim;
                        const bool is_v = kv >= kv_dim;
                        const int idx = is_v ? kv - kv_dim : kv;
                        const int head = idx / hd;
                        const int page = p.tables[L->group][(size_t)p.seq_of_token[tok] * p.bt_stride[L->group] + pos / p.page_size];
                        const size_t off = (((size_t)page * p.n_kv_heads + head) * p.page_size + pos % p.page_size) * hd + dh;
                        *reinterpret_cast<uint32_t*>((is_v ? L->v_pages : L->k_pages) + off) = fd_pack2(v0, v1);
                    }
                }
            }
        } else if (OUT == FD_OUT_ADD) {
            if (tid < 128) {
                const int tok = tid >> 4, row = tid & 15;
                if (row < rows && tok < p.M) {
                    float* dst = p.h + (size_t)tok * p.d + rg + row;
                    *dst = __ldcg(dst) + total(row, tok);
                }
            }
        } else if (OUT == FD_OUT_SWIGLU) {
            if (tid < 64) {
                const int tok = tid >> 3, j = tid & 7;
                if (tok < p.M) {                                // (gran 16: a group is 8 gate rows + their 8 up rows)
                    const float gate = total(j, tok), up = total(8 + j, tok);
                    p.act[(size_t)tok * p.inter + (rg >> 1) + j] = __float2bfloat16_rn(gate / (1.0f + __expf(-gate)) * up);
                }
            }
        } else {
            if (tid < 128) {
                const int tok = tid >> 4, row = tid & 15;
                if (row < rows && tok < p.R) p.logits[(size_t)tok * p.vocab + rg + row] = total(row, tok);
            }
        }
    }
}

// ---- consumers: attention of the step's tokens over the paged cache ------------------------------------
// Element offset of (row, 16-byte piece) in a tile of rows of HD bf16, pieces XOR-swizzled by row.
template <int HD> __device__ __forceinline__ int fd_sw(int row, int piece) {
    constexpr int CH = HD / 8;
    constexpr int MASK = ((CH & -CH) - 1) & 7;
    return row * HD + ((piece ^ (row & MASK)) << 3);
}

// The block's share of one (token, kv head) pair: keys [k_begin, k_end).  Result: (max, sum,
// unnormalised output) per query head of the group, either final (-> att) or a partial record.
template <int HD>
__device__ void fd_attend_range(const FdParams& p, const FdShared& s, const FdLayer& L, int tok, int kvh, int k_begin, int k_end,
                                bool final_result, float* record) {
    constexpr int SEG = HD == 64 ? 128 : 64;      // keys per buffer
    constexpr int MW = SEG / 16;                   // warps that do the arithmetic (16 keys each per segment)
    constexpr int CH = HD / 8, KS = HD / 16, NT_O = HD / 8;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    bf16* sQ = reinterpret_cast<bf16*>(s.work);                       // [16][HD]
    bf16* sKV = sQ + 16 * HD;                                         // 2 x (K [SEG][HD] + V [SEG][HD])
    const int G = p.n_q_heads / p.n_kv_heads;
    const int* table = p.tables[L.group] + (size_t)p.seq_of_token[tok] * p.bt_stride[L.group];
    const int page_size = p.page_size;

    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    uint32_t qa[KS][4];

    auto request = [&](int seg0, int buf) {
        const int seg_keys = min(SEG, k_end - seg0);
        const int rows = ((seg_keys + 15) / 16) * 16;
        bf16* sK = sKV + (size_t)buf * 2 * SEG * HD;
        bf16* sV = sK + SEG * HD;
        constexpr int ITERS = SEG * CH / FD_CONSUMERS;
        int page[ITERS];
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {                          // all look-ups first, then all copies
            const int idx = tid + it * FD_CONSUMERS;
            int key = seg0 + idx / CH;
            key = key < k_end ? key : k_end - 1;
            page[it] = idx < rows * CH ? table[key / page_size] : -1;
        }
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            if (page[it] < 0) continue;
            const int idx = tid + it * FD_CONSUMERS;
            const int r = idx / CH, c = idx - r * CH;
            int key = seg0 + r;
            key = key < k_end ? key : k_end - 1;
            const size_t off = (((size_t)page[it] * p.n_kv_heads + kvh) * page_size + key % page_size) * HD + c * 8;
            fd_cp16(sK + fd_sw<HD>(r, c), L.k_pages + off);
            fd_cp16(sV + fd_sw<HD>(r, c), L.v_pages + off);
        }
    };

    request(k_begin, 0);
    for (int idx = tid; idx < 16 * CH; idx += FD_CONSUMERS) {
        const int r = idx / CH, c = idx - r * CH;
        bf16* dst = sQ + fd_sw<HD>(r, c);
        if (r < G) fd_cp16(dst, p.q + ((size_t)tok * p.n_q_heads + (size_t)kvh * G + r) * HD + c * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    fd_cp_commit();

    int buf = 0;
    for (int seg0 = k_begin; seg0 < k_end; seg0 += SEG, buf ^= 1) {
        const int seg_keys = min(SEG, k_end - seg0);
        const int rows = ((seg_keys + 15) / 16) * 16;
        const bf16* sK = sKV + (size_t)buf * 2 * SEG * HD;
        const bf16* sV = sK + SEG * HD;
        if (seg0 + SEG < k_end) request(seg0 + SEG, buf ^ 1);
        fd_cp_commit();
        fd_cp_wait<1>();
        fd_bar();
        if (seg0 == k_begin) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
                fd_ldsm_x4(qa[ks], fd_smem(sQ + fd_sw<HD>((lane & 7) + 8 * ((lane >> 3) & 1), 2 * ks + (lane >> 4))));
        }
        const int w0 = warp * 16;                                    // this warp's keys of the segment
        if (warp < MW && w0 < seg_keys) {
            float sc[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t b[4];
                const int mi = lane >> 3;
                fd_ldsm_x4(b, fd_smem(sK + fd_sw<HD>(w0 + (lane & 7) + 8 * (mi >> 1), 2 * ks + (mi & 1))));
                fd_mma16(sc[0], qa[ks], b[0], b[1]);
                fd_mma16(sc[1], qa[ks], b[2], b[3]);
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const bool ok = w0 + 8 * j + 2 * t + (e & 1) < seg_keys;
                    sc[j][e] = ok ? sc[j][e] * p.scale_log2e : -INFINITY;
                }
                mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
                mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite: the warp has at least one key
            const float corr0 = fd_exp2(m0 - mn0), corr1 = fd_exp2(m1 - mn1);
            m0 = mn0;
            m1 = mn1;
            float rs0 = 0.f, rs1 = 0.f;
            uint32_t pa[4];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                // the sum runs over the bfloat16-rounded probabilities that multiply V
                const __nv_bfloat162 r01 = __floats2bfloat162_rn(fd_exp2(sc[j][0] - mn0), fd_exp2(sc[j][1] - mn0));
                const __nv_bfloat162 r23 = __floats2bfloat162_rn(fd_exp2(sc[j][2] - mn1), fd_exp2(sc[j][3] - mn1));
                rs0 += __bfloat162float(r01.x) + __bfloat162float(r01.y);
                rs1 += __bfloat162float(r23.x) + __bfloat162float(r23.y);
                pa[j * 2 + 0] = *reinterpret_cast<const uint32_t*>(&r01);
                pa[j * 2 + 1] = *reinterpret_cast<const uint32_t*>(&r23);
            }
            l0 = l0 * corr0 + rs0;
            l1 = l1 * corr1 + rs1;
#pragma unroll
            for (int j = 0; j < NT_O; ++j) {
                o[j][0] *= corr0; o[j][1] *= corr0; o[j][2] *= corr1; o[j][3] *= corr1;
            }
            if (w0 < rows) {
#pragma unroll
                for (int dp = 0; dp < NT_O / 2; ++dp) {
                    uint32_t b[4];
                    const int mi = lane >> 3;
                    fd_ldsm_x4_trans(b, fd_smem(sV + fd_sw<HD>(w0 + (lane & 7) + 8 * (mi & 1), 2 * dp + (mi >> 1))));
                    fd_mma16(o[2 * dp], pa, b[0], b[1]);
                    fd_mma16(o[2 * dp + 1], pa, b[2], b[3]);
                }
            }
        }
        fd_bar();   // everyone is done with this buffer before it is refilled
    }
    fd_cp_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // ---- merge the warps (fixed order); the key/value tiles are no longer needed ----
    float* sm_m = s.red;                                           // [MW][16]  (the projections' buffer is idle here)
    float* sm_l = s.red + MW * 16;
    float (*sm_o)[16][HD + 1] = reinterpret_cast<float (*)[16][HD + 1]>(s.work);
    static_assert(sizeof(float) * MW * 16 * (HD + 1) <= FD_WORK_BYTES, "merge buffer");
    if (warp < MW) {
        if (t == 0) { sm_m[warp * 16 + g] = m0; sm_m[warp * 16 + g + 8] = m1; sm_l[warp * 16 + g] = l0; sm_l[warp * 16 + g + 8] = l1; }
#pragma unroll
        for (int j = 0; j < NT_O; ++j) {
            const int d = 8 * j + 2 * t;
            sm_o[warp][g][d] = o[j][0]; sm_o[warp][g][d + 1] = o[j][1];
            sm_o[warp][g + 8][d] = o[j][2]; sm_o[warp][g + 8][d + 1] = o[j][3];
        }
    }
    fd_bar();
    for (int idx = tid; idx < G * HD; idx += FD_CONSUMERS) {
        const int row = idx / HD, d = idx - row * HD;
        float mm = sm_m[row];
#pragma unroll
        for (int w = 1; w < MW; ++w) mm = fmaxf(mm, sm_m[w * 16 + row]);
        float acc = 0.f, ll = 0.f;
#pragma unroll
        for (int w = 0; w < MW; ++w) {
            const float f = sm_m[w * 16 + row] == -INFINITY ? 0.f : fd_exp2(sm_m[w * 16 + row] - mm);
            acc += sm_o[w][row][d] * f;
            ll += sm_l[w * 16 + row] * f;
        }
        if (final_result) {
            p.att[((size_t)tok * p.n_q_heads + (size_t)kvh * G + row) * HD + d] = __float2bfloat16_rn(acc / ll);
        } else {
            float* dst = record + (size_t)row * (HD + 2);
            dst[2 + d] = acc;
            if (d == 0) { dst[0] = mm; dst[1] = ll; }
        }
    }
    fd_bar();   // the work area may be overwritten by the next range
}

template <int HD>
__device__ void fd_attention(const FdParams& p, const FdShared& s, const FdLayer& L) {
    const int tid = threadIdx.x;
    const int nb = gridDim.x, b = blockIdx.x;
    const int G = p.n_q_heads / p.n_kv_heads;
    // units of 64 keys, pairs in (token, kv head) order
    int chunks[FD_MAX_ROWS], lo[FD_MAX_ROWS];
    long long U = 0;
    for (int i = 0; i < p.M; ++i) {
        const int pos = p.positions[i];
        lo[i] = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
        chunks[i] = (pos + 1 - lo[i] + 63) / 64;
        U += (long long)chunks[i] * p.n_kv_heads;
    }
    const long long u_begin = U * b / nb, u_end = U * (b + 1) / nb;
    auto block_of = [&](long long u) { return (int)(((u + 1) * nb - 1) / U); };
    long long pu0 = 0;
    for (int i = 0; i < p.M; ++i) {
        for (int kvh = 0; kvh < p.n_kv_heads; ++kvh, pu0 += chunks[i]) {
            const long long pu1 = pu0 + chunks[i];
            if (pu1 <= u_begin || pu0 >= u_end) continue;
            const int pair = i * p.n_kv_heads + kvh;
            const int cb = (int)(max(pu0, u_begin) - pu0), ce = (int)(min(pu1, u_end) - pu0);
            const int pos = p.positions[i];
            const int k_begin = lo[i] + cb * 64, k_end = min(pos + 1, lo[i] + ce * 64);
            const int first = block_of(pu0), last = block_of(pu1 - 1);
            const int n_seg = last - first + 1;
            float* record = p.partials + ((size_t)(b + pair) * 16) * (HD + 2);
            fd_attend_range<HD>(p, s, L, i, kvh, k_begin, k_end, n_seg == 1, record);
            if (n_seg == 1) continue;
            // ---- whoever finishes this pair last merges its records, in block order ----
            if (tid == 0) {
                __threadfence();
                int* ticket = p.tickets + pair;
                const int prev = atomicAdd(ticket, 1);
                const int is_last = prev == n_seg - 1;
                if (is_last) *ticket = 0;
                *s.flag = is_last;
            }
            fd_bar();
            const bool is_last = *s.flag != 0;
            if (is_last) {
                __threadfence();
                for (int idx = tid; idx < G * HD; idx += FD_CONSUMERS) {
                    const int row = idx / HD, d = idx - row * HD;
                    const float* src = p.partials + ((size_t)(first + pair) * 16 + row) * (HD + 2);
                    const size_t step = (size_t)16 * (HD + 2);
                    float mm = -INFINITY, acc = 0.f, ll = 0.f;
                    for (int s0 = 0; s0 < n_seg; s0 += 4) {          // four records at a time: their loads overlap
                        float ms[4], ls[4], as[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const bool ok = s0 + j < n_seg;
                            const float* r = src + (size_t)(ok ? s0 + j : s0) * step;
                            ms[j] = __ldcg(r);
                            ls[j] = __ldcg(r + 1);
                            as[j] = __ldcg(r + 2 + d);
                            if (!ok) ms[j] = -INFINITY;
                        }
                        float cm = mm;
#pragma unroll
                        for (int j = 0; j < 4; ++j) cm = fmaxf(cm, ms[j]);
                        const float f0 = mm == -INFINITY ? 0.f : fd_exp2(mm - cm);
                        acc *= f0;
                        ll *= f0;
                        mm = cm;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float f = ms[j] == -INFINITY ? 0.f : fd_exp2(ms[j] - cm);
                            acc += as[j] * f;
                            ll += ls[j] * f;
                        }
                    }
                    p.att[((size_t)i * p.n_q_heads + (size_t)kvh * G + row) * HD + d] = __float2bfloat16_rn(acc / ll);
                }
            }
            fd_bar();   // the flag is read before it is written again
        }
    }
}

// ---- the kernel --------------------------------------------------------------------------------------
__global__ void __launch_bounds__(FD_THREADS, 1) decode_fused_kernel(const __grid_constant__ FdParams p) {
    extern __shared__ __align__(128) unsigned char fd_smem_raw[];
    FdShared s;
    s.ring = fd_smem_raw;
    s.work = fd_smem_raw + FD_RING_BYTES;
    s.red = reinterpret_cast<float*>(s.work + FD_WORK_BYTES);
    unsigned char* tail = reinterpret_cast<unsigned char*>(s.red + FD_RED_FLOATS);
    s.full = reinterpret_cast<uint64_t*>(tail);
    s.empty = s.full + FD_STAGES;
    s.rstd = reinterpret_cast<float*>(s.empty + FD_STAGES);
    s.abort_flag = reinterpret_cast<volatile int*>(s.rstd + 8);
    s.flag = const_cast<int*>(s.abort_flag) + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < FD_STAGES; ++i) { fd_mbar_init(&s.full[i], 1); fd_mbar_init(&s.empty[i], FD_CONSUMER_WARPS); }
        *s.abort_flag = 0;
        *s.flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    if (warp == FD_CONSUMER_WARPS) {
        fd_loader(p, s, lane);
    } else {
        FdRing ring = {0, 0};
        int red_buf = 0, n_passed = 0;
        const int qkv_rows = (p.n_q_heads + 2 * p.n_kv_heads) * p.head_dim, q_dim = p.n_q_heads * p.head_dim;
        // embedding: row i of the residual stream by block i (mod blocks)
        for (int i = blockIdx.x; i < p.M; i += gridDim.x) {
            const bf16* src = p.embedding + (size_t)p.tokens[i] * p.d;
            for (int c = tid * 8; c < p.d; c += FD_CONSUMERS * 8) {
                const uint4 v = *reinterpret_cast<const uint4*>(src + c);
                const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&v);
                float4 a, b2;
                a.x = __bfloat162float(e[0].x); a.y = __bfloat162float(e[0].y); a.z = __bfloat162float(e[1].x); a.w = __bfloat162float(e[1].y);
                b2.x = __bfloat162float(e[2].x); b2.y = __bfloat162float(e[2].y); b2.z = __bfloat162float(e[3].x); b2.w = __bfloat162float(e[3].y);
                *reinterpret_cast<float4*>(p.h + (size_t)i * p.d + c) = a;
                *reinterpret_cast<float4*>(p.h + (size_t)i * p.d + c + 4) = b2;
            }
        }
        // the attention merge's tickets start from zero whatever an earlier launch that gave up left there
        if (blockIdx.x == 0) for (int i = tid; i < p.M * p.n_kv_heads; i += FD_CONSUMERS) p.tickets[i] = 0;
        fd_grid_sync(p, s, n_passed);
        for (int l = 0; l < p.n_layers; ++l) {
            const FdLayer* L = p.layers + l;
            FdInput in;
            in.kind = FD_IN_NORM; in.src = nullptr; in.rows = nullptr; in.gain = L->gain_mixer; in.eps = L->eps_mixer; in.n_rows = p.M;
            fd_project<FD_OUT_QKV>(p, s, ring, red_buf, in, L, qkv_rows, p.d, 2);
            fd_grid_sync(p, s, n_passed);
            if (p.head_dim == 64) fd_attention<64>(p, s, *L); else fd_attention<128>(p, s, *L);
            fd_grid_sync(p, s, n_passed);
            in.kind = FD_IN_BF16; in.src = p.att;
            fd_project<FD_OUT_ADD>(p, s, ring, red_buf, in, L, p.d, q_dim, 1);
            fd_grid_sync(p, s, n_passed);
            in.kind = FD_IN_NORM; in.src = nullptr; in.gain = L->gain_ffn; in.eps = L->eps_ffn;
            fd_project<FD_OUT_SWIGLU>(p, s, ring, red_buf, in, L, 2 * p.inter, p.d, 16);
            fd_grid_sync(p, s, n_passed);
            in.kind = FD_IN_BF16; in.src = p.act;
            fd_project<FD_OUT_ADD>(p, s, ring, red_buf, in, L, p.d, p.inter, 1);
            fd_grid_sync(p, s, n_passed);
        }
        if (p.R > 0) {
            FdInput in;
            in.kind = FD_IN_NORM; in.src = nullptr; in.rows = p.logit_rows; in.gain = p.gain_final; in.eps = p.eps_final; in.n_rows = p.R;
            fd_project<FD_OUT_LOGITS>(p, s, ring, red_buf, in, nullptr, p.vocab, p.d, 1);
        }
    }
    __syncthreads();
}

// ---- host side -------------------------------------------------------------------------------------
NI_EXPORT int ni_decode_fused_max_rows() { return FD_MAX_ROWS; }
NI_EXPORT int ni_decode_fused_max_groups() { return FD_MAX_GROUPS; }
NI_EXPORT int ni_decode_fused_blocks() { return ni_sm_count(); }
NI_EXPORT long long ni_decode_fused_params_size() { return (long long)sizeof(FdParams); }
NI_EXPORT long long ni_decode_fused_layer_size() { return (long long)sizeof(FdLayer); }

// 1 if the kernel takes these sizes.
NI_EXPORT int ni_decode_fused_supports(int M, int d, int n_q_heads, int n_kv_heads, int head_dim, int rotary_dim, int inter,
                                       int vocab, int page_size) {
    if (M <= 0 || M > FD_MAX_ROWS || d <= 0 || inter <= 0 || vocab <= 0 || page_size <= 0) return 0;
    if (head_dim != 64 && head_dim != 128) return 0;
    if (n_kv_heads <= 0 || n_q_heads % n_kv_heads || n_q_heads / n_kv_heads > 16) return 0;
    if (d % 8 || inter % 8 || rotary_dim % 2 || rotary_dim < 0 || rotary_dim > head_dim) return 0;
    return 1;
}

// Floats of `partials` and ints of `tickets` the attention merge needs.
NI_EXPORT long long ni_decode_fused_partials(int M, int n_kv_heads, int head_dim) {
    return (long long)(ni_sm_count() + M * n_kv_heads) * 16 * (head_dim + 2);
}

NI_EXPORT int ni_decode_fused(const FdParams* hp, cudaStream_t stream) {
    if (hp == nullptr) return NI_ERR_BAD_ARGUMENT;
    FdParams p = *hp;
    if (!ni_decode_fused_supports(p.M, p.d, p.n_q_heads, p.n_kv_heads, p.head_dim, p.rotary_dim, p.inter, p.vocab, p.page_size))
        return NI_ERR_UNSUPPORTED_SIZE;
    if (p.R < 0 || p.R > FD_MAX_ROWS || p.n_layers < 0 || p.barrier == nullptr || p.error == nullptr) return NI_ERR_BAD_ARGUMENT;
    if (p.wait_limit <= 0) p.wait_limit = 4000000000LL;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FD_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_fused_kernel, FD_THREADS, FD_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        if (per_sm < 1) return NI_ERR_UNSUPPORTED_SIZE;
        configured = true;
    }
    cudaError_t e = cudaMemsetAsync(p.barrier, 0, sizeof(unsigned), stream);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ni_sm_count());
    cfg.blockDim = dim3(FD_THREADS);
    cfg.dynamicSmemBytes = FD_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // all blocks resident at once: they wait for each other
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, decode_fused_kernel, p);
    return e == cudaSuccess ? NI_OK : (int)e;
}
