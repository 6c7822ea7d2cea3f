// One decode step of a pre-norm attention + SwiGLU decoder as ONE persistent kernel: embedding,
// every layer (RMSNorm -> fused QKV projection -> rotary encoding + paged K/V write -> split-K
// grouped-query attention over the paged cache -> output projection + residual -> RMSNorm ->
// gate/up projection + SwiGLU -> down projection + residual), final norm and the projection onto
// the vocabulary, for up to 8 single query tokens.
//
// Why one kernel: at these sizes a decode step is a chain of ~80 products of 3-15 us each, and what
// it costs is not bandwidth inside the kernels but the ramp and the tail of every one of them.
// Here the weights of ALL layers are one stream:
//
//   * one block per SM (cooperative launch), 8 consumer warps + 1 loader warp;
//   * every weight matrix is cut by rows into one contiguous share per block (+-1 unit, so every
//     SM streams the same number of bytes); the loader warp walks its block's shares of all
//     matrices of all layers in order and copies them, 8 rows x 2048 columns at a time, one
//     cp.async.bulk (TMA, no tensor map needed for contiguous row segments) of up to 4 KB per row,
//     into a ring of shared-memory stages guarded by mbarriers.  It runs ahead of the consumers by
//     the depth of the ring (128 KB per SM, 19 MB over the GPU), across layer and phase boundaries;
//   * the consumer warps split a stage's columns, multiply with mma.sync (two stages = the 16 rows
//     of the A operand, the batch on the 8-wide side, FP32 accumulate), add their partial sums in
//     warp order through shared memory and run the epilogue (rotary + cache write, residual add,
//     SwiGLU, logits).  Each output element is owned by one block: no atomics on data, results do
//     not depend on timing;
//   * activations pass from phase to phase through global memory (L2) and a grid barrier: a
//     counter that every block increments and polls (bounded).  Attention runs between two such
//     barriers on the same blocks: the (token, kv head) pairs' keys are cut into 64-key units, each
//     block takes a contiguous run of units, partial results of a pair are merged, in order, by
//     the block that finishes last (atomic ticket, no waiting).
//
// Where it stands (1B sizes, context 2,048, time of one step seen by block 0): batch 8: 1.68 ms
// (projections 0.79, attention 0.48, the 81 grid barriers 0.29, output projection 0.12); batch 1:
// 1.19 ms - against 0.86 and 0.81 ms for the chain of per-part kernels, so the engine does not use
// it unless asked (ModelRunner(fused_decode=True)).  What was learned on the way: the copy engine
// takes about 90 clocks per bulk copy, so 1 KB copies ran the stream at half the HBM rate (the
// output projection alone: 166 us with 1 KB copies, 95 us with 2 KB, 82 us = HBM rate with 4 KB);
// the legacy mma.sync pipe delivers one m16n8k16 per ~60 clocks per scheduler here, so with two
// warps per scheduler the arithmetic (2,000 clocks per 64 KB) is slower than the stream; with nine
// warps per block a thread gets at most 168 registers (a scheduler's third warp); and a grid barrier
// costs 1.8-7 us (3.5 on average: two trips to L2 plus the skew of 148 blocks), five per layer,
// on the consumers' critical path where the ring (2.9 us of stream) cannot hide it.
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
#define FD_TILE_ROWS 8                             // weight rows of a ring stage
#define FD_KT 2048                                 // columns of a ring stage: 4 KB per row and copy
#define FD_ROW_BYTES (FD_KT * 2 + 16)              // padded: ldmatrix rows fall into different banks
#define FD_STAGE_BYTES (FD_TILE_ROWS * FD_ROW_BYTES)
#define FD_STAGES 4
#define FD_RING_BYTES (FD_STAGES * FD_STAGE_BYTES)
#define FD_WORK_BYTES (68 * 1024)                  // activations of a phase / K and V segments / merge buffer
#define FD_RED_FLOATS (2 * FD_CONSUMER_WARPS * 128)
#define FD_SMEM_BYTES (FD_RING_BYTES + FD_WORK_BYTES + FD_RED_FLOATS * 4 + 1024 + 512)
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
    long long* trace;            // optional: block 0 writes the time (ns) at which it passes each phase boundary
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
    float* ssq;              // [warps][8] partial sums of squares
    int* pos;                // [8] the tokens' positions
    int* seq;                // [8] the tokens' rows of the block tables
    int* page;               // [groups][8] the page that receives each token's key and value
    volatile int* abort_flag;
    int* flag;               // "this block arrived last" of the attention merge
};

// Shared memory: the ring, the work area, the reduction buffers, then the small things - among them
// a copy of the kernel's arguments.  Functions that are not inlined find all of it through these two
// accessors instead of through references to the kernel's own variables (which would live in local
// memory, and every use of them would be a load from there).
extern __shared__ __align__(128) unsigned char fd_smem_raw[];
#define FD_TAIL_OFFSET (FD_RING_BYTES + FD_WORK_BYTES + FD_RED_FLOATS * 4)
#define FD_TAIL_BYTES 1024                          // barriers, statistics, positions, pages, flags: 552 bytes used
#define FD_PARAMS_OFFSET (FD_TAIL_OFFSET + FD_TAIL_BYTES)

__device__ __forceinline__ FdShared fd_shared() {
    FdShared s;
    s.ring = fd_smem_raw;
    s.work = fd_smem_raw + FD_RING_BYTES;
    s.red = reinterpret_cast<float*>(s.work + FD_WORK_BYTES);
    unsigned char* tail = fd_smem_raw + FD_TAIL_OFFSET;
    s.full = reinterpret_cast<uint64_t*>(tail);
    s.empty = s.full + FD_STAGES;
    s.rstd = reinterpret_cast<float*>(s.empty + FD_STAGES);
    s.ssq = s.rstd + 8;
    s.pos = reinterpret_cast<int*>(s.ssq + FD_CONSUMER_WARPS * 8);
    s.seq = s.pos + 8;
    s.page = s.seq + 8;
    s.abort_flag = reinterpret_cast<volatile int*>(s.page + FD_MAX_GROUPS * 8);
    s.flag = const_cast<int*>(s.abort_flag) + 1;
    static_assert(2 * FD_STAGES * 8 + (8 + FD_CONSUMER_WARPS * 8 + 8 + 8 + FD_MAX_GROUPS * 8 + 2) * 4 <= FD_TAIL_BYTES, "tail of the shared memory");
    static_assert(sizeof(FdParams) <= 512, "room for the arguments' copy");
    return s;
}
__device__ __forceinline__ const FdParams& fd_params() { return *reinterpret_cast<const FdParams*>(fd_smem_raw + FD_PARAMS_OFFSET); }

struct FdRing {              // a consumer's or the loader's place in the ring
    int stage;
    uint32_t phase;
    __device__ __forceinline__ void advance() { if (++stage == FD_STAGES) { stage = 0; phase ^= 1; } }
};

// ---- the loader warp -------------------------------------------------------------------------------
// The order in which a block's share of a matrix passes through the ring (the consumers walk the
// same order): groups of up to 16 rows; within a group the 2048-column tiles one after the other;
// within a tile the group's first 8 rows, then the rest.  One stage = up to 8 rows of one tile; each
// row is one bulk copy of up to 4 KB (copies of this size keep the copy engine's request rate, about
// one per 90 clocks, off the critical path; at 1 KB per copy the stream ran at half the HBM rate).
__device__ bool fd_load_matrix(const FdParams& p, const FdShared& s, FdRing& ring, const bf16* W, int N, int K, int gran,
                               int lane) {
    int r0, r1;
    fd_rows(N, gran, blockIdx.x, gridDim.x, r0, r1);
    for (int rg = r0; rg < r1; rg += 16) {
        const int sg_rows = min(16, r1 - rg);
        for (int k0 = 0; k0 < K; k0 += FD_KT) {
            const int cols = min(FD_KT, K - k0);
            for (int sub = 0; sub * 8 < sg_rows; ++sub) {
                const int rows = min(8, sg_rows - sub * 8);
                if (!fd_mbar_wait(&s.empty[ring.stage], ring.phase ^ 1, s.abort_flag, p.wait_limit)) {
                    if (lane == 0 && !*s.abort_flag) { atomicCAS(p.error, 0, FD_ERR_LOADER); *s.abort_flag = 1; }
                    return false;
                }
                if (lane == 0) fd_mbar_expect_tx(&s.full[ring.stage], (uint32_t)(rows * cols * 2));
                __syncwarp();
                if (lane < rows)
                    fd_bulk_copy(s.ring + (size_t)ring.stage * FD_STAGE_BYTES + lane * FD_ROW_BYTES,
                                 W + (size_t)(rg + sub * 8 + lane) * K + k0, (uint32_t)(cols * 2), &s.full[ring.stage]);
                ring.advance();
            }
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
// norm(h[rows]) * gain as bfloat16 into the work area, for a projection whose K (= d) fits it in one
// piece.  All consumer threads share every row (thread j takes the 16-byte pieces j, j + 256, ...),
// so that all loads of the phase are in flight at once: one trip to L2 instead of one per piece.
// With d <= 2048 the values stay in registers between the statistics and the scaling; wider rows are
// read a second time.
__device__ __noinline__ void fd_act_norm_whole(unsigned char* dst, int stride, const int* rows, int n_rows, const float* gain,
                                               float eps) {
    const FdParams& p = fd_params();
    const FdShared s = fd_shared();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pieces = p.d / 4;                                  // float4 per row
    const bool keep = pieces <= 2 * FD_CONSUMERS;
    float4 v[16];
    float ss[FD_MAX_ROWS];
#pragma unroll
    for (int r = 0; r < FD_MAX_ROWS; ++r) ss[r] = 0.f;
    if (keep) {
#pragma unroll
        for (int r = 0; r < FD_MAX_ROWS; ++r) {
            const float* src = p.h + (size_t)(r < n_rows ? (rows ? rows[r] : r) : 0) * p.d;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int idx = tid + c * FD_CONSUMERS;
                v[r * 2 + c] = (r < n_rows && idx < pieces) ? __ldcg(reinterpret_cast<const float4*>(src) + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int r = 0; r < FD_MAX_ROWS; ++r)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const float4 x = v[r * 2 + c];
                ss[r] += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
            }
    } else {
        for (int base = 0; base < pieces; base += 2 * FD_CONSUMERS) {
#pragma unroll
            for (int r = 0; r < FD_MAX_ROWS; ++r) {
                const float* src = p.h + (size_t)(r < n_rows ? (rows ? rows[r] : r) : 0) * p.d;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int idx = base + tid + c * FD_CONSUMERS;
                    v[r * 2 + c] = (r < n_rows && idx < pieces) ? __ldcg(reinterpret_cast<const float4*>(src) + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int r = 0; r < FD_MAX_ROWS; ++r)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const float4 x = v[r * 2 + c];
                    ss[r] += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
                }
        }
    }
#pragma unroll
    for (int r = 0; r < FD_MAX_ROWS; ++r) {
        const float t = ni_warp_sum(ss[r]);
        if (lane == 0) s.ssq[warp * 8 + r] = t;
    }
    fd_bar();
    float rstd[FD_MAX_ROWS];
#pragma unroll
    for (int r = 0; r < FD_MAX_ROWS; ++r) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < FD_CONSUMER_WARPS; ++w) t += s.ssq[w * 8 + r];
        rstd[r] = rsqrtf(t / (float)p.d + eps);
    }
    for (int base = 0; base < pieces; base += 2 * FD_CONSUMERS) {
        if (!keep) {
#pragma unroll
            for (int r = 0; r < FD_MAX_ROWS; ++r) {
                const float* src = p.h + (size_t)(r < n_rows ? (rows ? rows[r] : r) : 0) * p.d;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int idx = base + tid + c * FD_CONSUMERS;
                    v[r * 2 + c] = (r < n_rows && idx < pieces) ? __ldcg(reinterpret_cast<const float4*>(src) + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int idx = base + tid + c * FD_CONSUMERS;
            if (idx < pieces) {
                const float4 g = *(reinterpret_cast<const float4*>(gain) + idx);
#pragma unroll
                for (int r = 0; r < FD_MAX_ROWS; ++r) {
                    if (r < n_rows) {
                        const float4 x = v[r * 2 + c];
                        uint2 o;
                        o.x = fd_pack2(x.x * rstd[r] * g.x, x.y * rstd[r] * g.y);
                        o.y = fd_pack2(x.z * rstd[r] * g.z, x.w * rstd[r] * g.w);
                        *reinterpret_cast<uint2*>(dst + (size_t)r * stride + (size_t)idx * 8) = o;
                    }
                }
            }
        }
    }
}
// The same piece by piece, for rows too wide for the work area: 1 / rms of every row first (one warp per row).
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
// The epilogue of a group of up to 16 weight rows: the warps' partial sums (in `red`) are added in warp
// order and go where the projection's kind says.  A function of its own, so that what it needs in
// registers (rotary angles, page addresses) does not weigh on the loop that streams the weights.
__device__ __noinline__ void fd_epilogue(const int OUT, const FdLayer* L, const float* red, int rg, int sg_rows) {
    const FdParams& p = fd_params();
    const FdShared s = fd_shared();
    const int tid = threadIdx.x;
        auto total = [&](int row, int tok) {                  // row: 0 .. 15 within the group
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < FD_CONSUMER_WARPS; ++w) v += red[w * 128 + (row >> 3) * 64 + tok * 8 + (row & 7)];
            return v;
        };
        if (OUT == FD_OUT_QKV) {
            if (tid < 64) {
                const int row = 2 * (tid >> 3), tok = tid & 7;
                if (row < sg_rows && tok < p.M) {
                    float v0 = total(row, tok), v1 = total(row + 1, tok);
                    const int n_row = rg + row, hd = p.head_dim;
                    const int q_dim = p.n_q_heads * hd, kv_dim = p.n_kv_heads * hd;
                    const int pos = s.pos[tok];
                    const int dh = n_row % hd;
                    if (n_row < q_dim + kv_dim && dh < p.rotary_dim) {
                        float sn, cs;
                        sincosf((float)pos * p.inv_freq[dh >> 1], &sn, &cs);
                        const float a = v0 * cs - v1 * sn, b = v0 * sn + v1 * cs;
                        v0 = a;
                        v1 = b;
                    }
                    if (n_row < q_dim) {
                        *reinterpret_cast<uint32_t*>(p.q + (size_t)tok * q_dim + n_row) = fd_pack2(v0, v1);
                    } else if (L->write_cache) {
                        const int kv = n_row - q_dim;
                        const bool is_v = kv >= kv_dim;
                        const int idx = is_v ? kv - kv_dim : kv;
                        const int head = idx / hd;
                        const int page = s.page[L->group * 8 + tok];
                        const size_t off = (((size_t)page * p.n_kv_heads + head) * p.page_size + pos % p.page_size) * hd + dh;
                        *reinterpret_cast<uint32_t*>((is_v ? L->v_pages : L->k_pages) + off) = fd_pack2(v0, v1);
                    }
                }
            }
        } else if (OUT == FD_OUT_ADD) {
            if (tid < 128) {
                const int tok = tid >> 4, row = tid & 15;
                if (row < sg_rows && tok < p.M) {
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
                if (row < sg_rows && tok < p.R) p.logits[(size_t)tok * p.vocab + rg + row] = total(row, tok);
            }
        }
}

// A warp's share of a group's stages when it is narrower than 256 columns (K is not a multiple of 2048: the
// last tile of a row, or a small model): steps of 16 columns and at most one of 8, activations read
// from shared memory as they are needed.  x_base / w0_base / w1_base: this lane's row of the
// activations / of the group's first and second stage (0: there is none), at the warp's first column.
__device__ __noinline__ void fd_narrow_tile(float c[4], uint32_t x_base, uint32_t w0_base, uint32_t w1_base, int n, int lane) {
    int kk = 0;
    for (; kk + 16 <= n; kk += 16) {
        uint32_t lo[2], hi[2] = {0u, 0u}, x[2];
        fd_ldsm_x2(lo, w0_base + (kk + ((lane >> 3) & 1) * 8) * 2);
        if (w1_base) fd_ldsm_x2(hi, w1_base + (kk + ((lane >> 3) & 1) * 8) * 2);
        fd_ldsm_x2(x, x_base + (kk + ((lane >> 3) & 1) * 8) * 2);
        const uint32_t a[4] = {lo[0], hi[0], lo[1], hi[1]};
        fd_mma16(c, a, x[0], x[1]);
    }
    if (kk < n) {
        uint32_t lo, hi = 0u, x;
        fd_ldsm_x1(lo, w0_base + kk * 2);
        if (w1_base) fd_ldsm_x1(hi, w1_base + kk * 2);
        fd_ldsm_x1(x, x_base + kk * 2);
        fd_mma8(c, lo, hi, x);
    }
}

// A wait that runs out does not change the control flow: the warp records the error, raises the
// block's abort flag and goes on through the same loops and block barriers without data (every
// later wait returns at once), so that no warp is ever left alone at a barrier.
//
// The weights are the A operand of the MMA (a group's two 8-row stages are the halves of its 16
// rows), the batch its 8 columns.  The 8 warps split a stage's columns, 256 each; a warp's activation
// fragments for its columns of the current tile stay in registers (for K <= 2048: for the whole
// phase), so shared memory carries the weights only.  (The legacy mma.sync pipe is slow on this
// part: with the weights as the 8-wide operand, twice as many MMAs, the arithmetic took longer
// than the stream - 4,900 clocks per 32 KB stage.)
//
// One function for all four projections (the epilogue is chosen at run time): the hot loop exists
// once in the instruction cache, and it is short - the general code for tiles narrower than a
// warp's 256 columns (odd sizes) is kept out of it.
struct FdConsumer {          // what a consumer thread carries from projection to projection
    FdRing ring;
    int red_buf;
};

__device__ __noinline__ FdConsumer fd_project(const int OUT, FdConsumer state, const FdInput in, const FdLayer* L, int N, int K,
                                              int gran) {
    const FdParams& p = fd_params();
    const FdShared s = fd_shared();
    FdRing ring = state.ring;
    int red_buf = state.red_buf;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    int r0, r1;
    fd_rows(N, gran, blockIdx.x, gridDim.x, r0, r1);
    const int Kc = fd_chunk(K);
    const bool chunked = Kc < K;                              // then Kc == FD_KT: a chunk is a tile
    const int stride = Kc * 2 + 16;
    int resident = -1;                                        // chunk that lies in the work area
    if (in.kind == FD_IN_NORM) {
        if (!chunked) {                                       // the usual case: the whole normalised rows, loaded at once
            fd_act_norm_whole(s.work, stride, in.rows, in.n_rows, in.gain, in.eps);
            fd_bar();
            resident = 0;
        } else {
            fd_row_rstd(p, s, in.rows, in.n_rows, in.eps, warp, lane);
            __syncwarp();
        }
    }
    uint32_t af[16][2];                                       // A fragments of this warp's 256 columns of a tile
    int frag_k0 = -1;
    const int kw = warp * 256;
    for (int rg = r0; rg < r1; rg += 16) {
        const int sg_rows = min(16, r1 - rg);
        float c[2][4];                                        // two chains (even and odd steps) of the same 16 rows x 8 tokens
#pragma unroll
        for (int j = 0; j < 2; ++j) c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f;
        for (int k0 = 0; k0 < K; k0 += FD_KT) {
            const int cols = min(FD_KT, K - k0);
            const int chunk = chunked ? k0 / FD_KT : 0, c0 = chunked ? k0 : 0;
            unsigned char* act = s.work + (chunked ? (chunk & 1) * 8 * stride : 0);
            if (chunk != resident) {
                // (chunked: every warp is past the chunk before last, whose buffer the prefetch overwrites)
                if (chunked) fd_bar();
                if (in.kind == FD_IN_NORM) {
                    fd_act_norm(p, s, act, stride, in.rows, in.n_rows, in.gain, c0, cols, warp, lane);
                } else {
                    if (!chunked || resident < 0 || chunk != resident + 1) {
                        fd_act_copy(act, stride, in.src, K, in.n_rows, c0, chunked ? cols : K);
                        fd_cp_commit();
                    }
                    if (chunked && k0 + FD_KT < K) {          // the next chunk streams in under this one
                        fd_act_copy(s.work + ((chunk + 1) & 1) * 8 * stride, stride, in.src, K, in.n_rows, k0 + FD_KT,
                                    min(FD_KT, K - k0 - FD_KT));
                        fd_cp_commit();
                        fd_cp_wait<1>();
                    } else {
                        fd_cp_wait<0>();
                    }
                }
                fd_bar();
                resident = chunk;
                frag_k0 = -1;
            }
            const int n = min(256, cols - kw);                // this warp's columns of the tile (may be <= 0)
            const bool whole = n == 256;
            const uint32_t a_base = fd_smem(act + (size_t)(lane & 7) * stride) + ((k0 - c0) + kw) * 2;
            if (whole && frag_k0 != k0) {
                frag_k0 = k0;
#pragma unroll
                for (int i2 = 0; i2 < 8; ++i2) {
                    uint32_t r[4];
                    fd_ldsm_x4(r, a_base + (i2 * 32 + (lane >> 3) * 8) * 2);
                    af[2 * i2][0] = r[0]; af[2 * i2][1] = r[1]; af[2 * i2 + 1][0] = r[2]; af[2 * i2 + 1][1] = r[3];
                }
            }
            // The group's two 8-row stages of this tile are the two halves of the MMA's 16 rows.
            const bool two = sg_rows > 8;
            const int st0 = ring.stage;
            bool landed = fd_mbar_wait(&s.full[st0], ring.phase, s.abort_flag, p.wait_limit);
            ring.advance();
            const int st1 = ring.stage;
            if (two) {
                landed = fd_mbar_wait(&s.full[st1], ring.phase, s.abort_flag, p.wait_limit) && landed;
                ring.advance();
            }
            if (!landed && lane == 0 && !*s.abort_flag) { atomicCAS(p.error, 0, FD_ERR_CONSUMER); *s.abort_flag = 1; }
            const uint32_t w0_row = fd_smem(s.ring + (size_t)st0 * FD_STAGE_BYTES + (lane & 7) * FD_ROW_BYTES) + kw * 2;
            const uint32_t w1_row = fd_smem(s.ring + (size_t)st1 * FD_STAGE_BYTES + (lane & 7) * FD_ROW_BYTES) + kw * 2;
            if (landed && whole) {
#pragma unroll
                for (int i2 = 0; i2 < 8; ++i2) {
                    uint32_t lo[4], hi[4] = {0u, 0u, 0u, 0u};
                    fd_ldsm_x4(lo, w0_row + (i2 * 32 + (lane >> 3) * 8) * 2);
                    if (two) fd_ldsm_x4(hi, w1_row + (i2 * 32 + (lane >> 3) * 8) * 2);
                    const uint32_t a0[4] = {lo[0], hi[0], lo[1], hi[1]};
                    const uint32_t a1[4] = {lo[2], hi[2], lo[3], hi[3]};
                    fd_mma16(c[0], a0, af[2 * i2][0], af[2 * i2][1]);
                    fd_mma16(c[1], a1, af[2 * i2 + 1][0], af[2 * i2 + 1][1]);
                }
            } else if (landed && n > 0) {
                fd_narrow_tile(c[0], a_base, w0_row, two ? w1_row : 0u, n, lane);
            }
            __syncwarp();
            if (lane == 0) {
                fd_mbar_arrive(&s.empty[st0]);
                if (two) fd_mbar_arrive(&s.empty[st1]);
            }
        }
        // ---- the warps' partial sums meet in shared memory; added in warp order ----
        // c[sub][0..1]: token g, weight rows 2t and 2t + 1 of the group's rows sub * 8 ..
        float* red = s.red + red_buf * (FD_CONSUMER_WARPS * 128);
        red_buf ^= 1;
        float* mine = red + warp * 128;
        // rows g (first stage) and g + 8 (second stage) of the group, tokens 2t and 2t + 1
        mine[2 * t * 8 + g] = c[0][0] + c[1][0];
        mine[(2 * t + 1) * 8 + g] = c[0][1] + c[1][1];
        mine[64 + 2 * t * 8 + g] = c[0][2] + c[1][2];
        mine[64 + (2 * t + 1) * 8 + g] = c[0][3] + c[1][3];
        fd_bar();
        fd_epilogue(OUT, L, red, rg, sg_rows);
    }
    state.ring = ring;
    state.red_buf = red_buf;
    return state;
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
    constexpr int SEG = 4096 / HD;                 // keys per buffer: K and V of a segment are 8 KB each
    constexpr int NBUF = 4;                        // three segments in flight while one is used
    constexpr int MW = SEG / 16;                   // warps that do the arithmetic (16 keys each per segment)
    constexpr int CH = HD / 8, KS = HD / 16, NT_O = HD / 8;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    bf16* sQ = reinterpret_cast<bf16*>(s.work);                       // [16][HD]
    bf16* sKV = sQ + 16 * HD;                                         // NBUF x (K [SEG][HD] + V [SEG][HD])
    static_assert((16 + NBUF * 2 * SEG) * HD * 2 <= FD_WORK_BYTES, "attention buffers");
    const int G = p.n_q_heads / p.n_kv_heads;
    const int* table = p.tables[L.group] + (size_t)s.seq[tok] * p.bt_stride[L.group];
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
        static_assert(ITERS * FD_CONSUMERS == SEG * CH, "segment pieces per thread");
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

    const int n_segs = (k_end - k_begin + SEG - 1) / SEG;
    for (int idx = tid; idx < 16 * CH; idx += FD_CONSUMERS) {
        const int r = idx / CH, c = idx - r * CH;
        bf16* dst = sQ + fd_sw<HD>(r, c);
        if (r < G) fd_cp16(dst, p.q + ((size_t)tok * p.n_q_heads + (size_t)kvh * G + r) * HD + c * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < NBUF - 1; ++i) {                              // (a group may be empty: the counting stays the same)
        if (i < n_segs) request(k_begin + i * SEG, i);
        fd_cp_commit();
    }

    for (int i = 0; i < n_segs; ++i) {
        const int seg0 = k_begin + i * SEG;
        const int buf = i % NBUF;
        const int seg_keys = min(SEG, k_end - seg0);
        const int rows = ((seg_keys + 15) / 16) * 16;
        const bf16* sK = sKV + (size_t)buf * 2 * SEG * HD;
        const bf16* sV = sK + SEG * HD;
        if (i + NBUF - 1 < n_segs) request(seg0 + (NBUF - 1) * SEG, (i + NBUF - 1) % NBUF);
        fd_cp_commit();
        fd_cp_wait<NBUF - 1>();                                       // segment i (and Q) have landed
        fd_bar();
        if (i == 0) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks)
                fd_ldsm_x4(qa[ks], fd_smem(sQ + fd_sw<HD>((lane & 7) + 8 * ((lane >> 3) & 1), 2 * ks + (lane >> 4))));
        }
        const int w0 = warp * 16;                                    // this warp's keys of the segment
        if (warp < MW && w0 < seg_keys) {
            float sc[2][4], sc2[2][4];                               // two chains per tile: an MMA's result takes long to come back
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
                sc2[j][0] = sc2[j][1] = sc2[j][2] = sc2[j][3] = 0.f;
            }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t b[4];
                const int mi = lane >> 3;
                fd_ldsm_x4(b, fd_smem(sK + fd_sw<HD>(w0 + (lane & 7) + 8 * (mi >> 1), 2 * ks + (mi & 1))));
                fd_mma16((ks & 1) ? sc2[0] : sc[0], qa[ks], b[0], b[1]);
                fd_mma16((ks & 1) ? sc2[1] : sc[1], qa[ks], b[2], b[3]);
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[j][e] += sc2[j][e];
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
__device__ __noinline__ void fd_attention(const FdLayer* layer) {
    const FdParams& p = fd_params();
    const FdShared s = fd_shared();
    const FdLayer& L = *layer;
    const int tid = threadIdx.x;
    const int nb = gridDim.x, b = blockIdx.x;
    const int G = p.n_q_heads / p.n_kv_heads;
    // units of 64 keys, pairs in (token, kv head) order
    int chunks[FD_MAX_ROWS], lo[FD_MAX_ROWS];
    long long U = 0;
    for (int i = 0; i < p.M; ++i) {
        const int pos = s.pos[i];
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
            const int pos = s.pos[i];
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

__device__ __forceinline__ void fd_trace(const FdParams& p, int& n) {
    if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.trace[n] = t;
    }
    ++n;
}

// ---- the kernel --------------------------------------------------------------------------------------
__global__ void __launch_bounds__(FD_THREADS, 1) decode_fused_kernel(const __grid_constant__ FdParams kernel_params) {
    const FdShared s = fd_shared();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    {   // the arguments' copy in shared memory
        const int* src = reinterpret_cast<const int*>(&kernel_params);
        int* dst = reinterpret_cast<int*>(fd_smem_raw + FD_PARAMS_OFFSET);
        for (int i = tid; i < (int)(sizeof(FdParams) / 4); i += FD_THREADS) dst[i] = src[i];
    }
    const FdParams& p = fd_params();
    if (tid == 0) {
        for (int i = 0; i < FD_STAGES; ++i) { fd_mbar_init(&s.full[i], 1); fd_mbar_init(&s.empty[i], FD_CONSUMER_WARPS); }
        *s.abort_flag = 0;
        *s.flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (tid < FD_MAX_ROWS) {                                      // what every phase asks of the step's tokens
        const bool live = tid < kernel_params.M;
        const int pos = live ? kernel_params.positions[tid] : 0, seq = live ? kernel_params.seq_of_token[tid] : 0;
        s.pos[tid] = pos;
        s.seq[tid] = seq;
        for (int g = 0; g < FD_MAX_GROUPS; ++g)
            s.page[g * 8 + tid] = (live && kernel_params.tables[g] != nullptr)
                                      ? kernel_params.tables[g][(size_t)seq * kernel_params.bt_stride[g] + pos / kernel_params.page_size] : 0;
    }
    __syncthreads();

    if (warp == FD_CONSUMER_WARPS) {
        fd_loader(p, s, lane);
    } else {
        FdConsumer st;
        st.ring.stage = 0; st.ring.phase = 0; st.red_buf = 0;
        int n_passed = 0;
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
        int n_trace = 0;
        fd_trace(p, n_trace);
        fd_grid_sync(p, s, n_passed);
        fd_trace(p, n_trace);
        for (int l = 0; l < p.n_layers; ++l) {
            const FdLayer* L = p.layers + l;
            FdInput in;
            in.kind = FD_IN_NORM; in.src = nullptr; in.rows = nullptr; in.gain = L->gain_mixer; in.eps = L->eps_mixer; in.n_rows = p.M;
            st = fd_project(FD_OUT_QKV, st, in, L, qkv_rows, p.d, 2);
            fd_trace(p, n_trace);
            fd_grid_sync(p, s, n_passed);
            fd_trace(p, n_trace);
            if (p.head_dim == 64) fd_attention<64>(L); else fd_attention<128>(L);
            fd_trace(p, n_trace);
            fd_grid_sync(p, s, n_passed);
            fd_trace(p, n_trace);
            in.kind = FD_IN_BF16; in.src = p.att;
            st = fd_project(FD_OUT_ADD, st, in, L, p.d, q_dim, 1);
            fd_trace(p, n_trace);
            fd_grid_sync(p, s, n_passed);
            fd_trace(p, n_trace);
            in.kind = FD_IN_NORM; in.src = nullptr; in.gain = L->gain_ffn; in.eps = L->eps_ffn;
            st = fd_project(FD_OUT_SWIGLU, st, in, L, 2 * p.inter, p.d, 16);
            fd_trace(p, n_trace);
            fd_grid_sync(p, s, n_passed);
            fd_trace(p, n_trace);
            in.kind = FD_IN_BF16; in.src = p.act;
            st = fd_project(FD_OUT_ADD, st, in, L, p.d, p.inter, 1);
            fd_trace(p, n_trace);
            fd_grid_sync(p, s, n_passed);
            fd_trace(p, n_trace);
        }
        if (p.R > 0) {
            FdInput in;
            in.kind = FD_IN_NORM; in.src = nullptr; in.rows = p.logit_rows; in.gain = p.gain_final; in.eps = p.eps_final; in.n_rows = p.R;
            st = fd_project(FD_OUT_LOGITS, st, in, nullptr, p.vocab, p.d, 1);
            fd_trace(p, n_trace);
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

// Blocks of the kernel that fit one SM at once (1 is what the launch needs; 0: it cannot be launched
// here), or a negative CUDA error code.
NI_EXPORT int ni_decode_fused_occupancy() {
    cudaError_t e = cudaFuncSetAttribute(decode_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FD_SMEM_BYTES);
    if (e != cudaSuccess) return -(int)e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_fused_kernel, FD_THREADS, FD_SMEM_BYTES);
    if (e != cudaSuccess) return -(int)e;
    return per_sm;
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
