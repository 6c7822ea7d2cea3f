// Next-token selection from FP32 logits: arg-max, and repetition penalty -> temperature ->
// top-k -> top-p -> multinomial draw, one thread block per row.
//
// The reference does this in up to five launches with host round trips for mixed batches
// (src/sampler/configurable_sampler.cpp:65-174; kernels in
// src/op/kernels/cuda/argmax_kernel.cu:40-102 and sampling_kernel.cu:38-398).  Its top-k and
// top-p thresholds come from 16 steps of bisection (approximate), its uniform number is drawn
// from Philox with the row index as the subsequence and offset 0, so a fixed seed repeats
// the same number every step and depends on the row's place in the batch.
//
// Here:
//  * the row's own parameters decide (temperature <= 0: arg-max, ties to the lowest id);
//  * top-k and top-p thresholds are exact: a radix select over the ordered bit patterns of
//    the scaled logits (k-th largest), and over probability mass (the smallest set of most
//    probable tokens whose mass exceeds p; tokens equal to the threshold are all kept);
//  * probability mass is summed in 64-bit fixed point, so every sum is exact and independent
//    of the order in which threads add: the same logits give the same token, always;
//  * the uniform number is Philox4x32-10 keyed by the request's seed with the index of the
//    generated token as counter: it does not depend on batching;
//  * the draw walks the vocabulary in id order: first id whose inclusive mass exceeds u * total.
#include "common.cuh"

#define SAMPLE_THREADS 1024
#define MASS_SCALE 274877906944.0f  // 2^38: exp(z - max) <= 1 in fixed point; sums fit 64 bits

__device__ __forceinline__ uint32_t ordered_key(float z) {
    const uint32_t b = __float_as_uint(z);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long mass_of(float e) {
    return (unsigned long long)(e * MASS_SCALE);
}

// Philox4x32-10 (Salmon et al. 2011); returns the first output word.
__device__ __forceinline__ uint32_t philox_first_word(unsigned long long seed, unsigned long long ctr) {
    uint32_t c0 = (uint32_t)ctr, c1 = (uint32_t)(ctr >> 32), c2 = 0u, c3 = 0u;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const unsigned long long p0 = (unsigned long long)0xD2511F53u * c0;
        const unsigned long long p1 = (unsigned long long)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        const uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return c0;
}

// Adds `val` of every active lane to bin `bin` of this warp's own histogram.  (All threads of a block
// adding to one shared histogram serialise on the few bins that the leading byte of similar numbers
// falls into: the first radix pass over 128 K logits took over a millisecond that way.  With a
// histogram per warp only a warp's own lanes can meet in a bin.  Taking the bins that occur in the
// warp one after the other and adding their lanes up by shuffles - no atomics at all - was slower
// again in the later passes, where every lane has a bin of its own: 94 us against 76 us for top-k; a
// fast path for warps whose lanes all agree on the bin changed nothing.)
__device__ __forceinline__ void warp_hist_add(unsigned long long* hist, uint32_t bin, unsigned long long val, bool active) {
    if (active) atomicAdd(&hist[bin], val);
}

struct BlockScratch {
    unsigned long long hist[256];
    unsigned long long red[32];
    float fred[32];
    unsigned long long chosen_u64;
    uint32_t chosen_u32;
    int chosen_int;
};

__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, BlockScratch& s) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s.red[threadIdx.x >> 5] = v;
    __syncthreads();
    unsigned long long t = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += s.red[w];
    return t;
}

// Row-wise arg-max with ties to the lowest index.
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    __shared__ float vals[32];
    __shared__ int idxs[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((threadIdx.x & 31) == 0) { vals[threadIdx.x >> 5] = best; idxs[threadIdx.x >> 5] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (vals[w] > best || (vals[w] == best && idxs[w] < best_i)) { best = vals[w]; best_i = idxs[w]; }
        out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
    }
}

// Wide rows, few of them: many blocks per row.  Each block folds its slice into one 64-bit key
// (ordered bits of the value above, 2^32 - 1 - index below, so that the larger value wins and,
// among equals, the lower index) and merges it with atomicMax: the result does not depend on
// the order of arrival.  A second tiny kernel unpacks the winners and leaves the keys at zero.
#define ARGMAX_SLICE 4096

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, unsigned long long* __restrict__ keys, int vocab) {
    const float* row = logits + (size_t)blockIdx.y * vocab;
    const int begin = blockIdx.x * ARGMAX_SLICE;
    const int end = min(vocab, begin + ARGMAX_SLICE);
    unsigned long long best = 0ull;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const unsigned long long key = ((unsigned long long)ordered_key(row[i]) << 32) | (0xffffffffu - (uint32_t)i);
        best = key > best ? key : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0 && best != 0ull) atomicMax(keys + blockIdx.y, best);
}

__global__ void argmax_finish_kernel(unsigned long long* __restrict__ keys, int* __restrict__ out, int n_rows) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    out[r] = (int)(0xffffffffu - (uint32_t)(keys[r] & 0xffffffffull));
    keys[r] = 0ull;
}

// keys: n_rows 64-bit words, zero before the first call (left zero), or null for the
// one-block-per-row kernel.
NI_EXPORT int ni_argmax(const float* logits, int* out, int n_rows, int vocab, unsigned long long* keys,
                        cudaStream_t stream) {
    if (n_rows <= 0) return NI_OK;
    if (vocab <= 0) return NI_ERR_BAD_ARGUMENT;
    if (keys == nullptr || vocab <= 2 * ARGMAX_SLICE || n_rows > 65535) {
        argmax_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, out, vocab);
        NI_RETURN_LAUNCH_STATUS();
    }
    dim3 grid((vocab + ARGMAX_SLICE - 1) / ARGMAX_SLICE, n_rows);
    argmax_partial_kernel<<<grid, 256, 0, stream>>>(logits, keys, vocab);
    argmax_finish_kernel<<<(n_rows + 127) / 128, 128, 0, stream>>>(keys, out, n_rows);
    NI_RETURN_LAUNCH_STATUS();
}

// logits[row, id] = l > 0 ? l / penalty : l * penalty for every listed id (each id once;
// the list is padded with -1).  Formula of sampling_kernel.cu:38-60.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, const int* __restrict__ ids,
                                          const float* __restrict__ penalties, int vocab, int max_ids) {
    const float p = penalties[blockIdx.x];
    if (p == 1.0f) return;
    float* row = logits + (size_t)blockIdx.x * vocab;
    const int* list = ids + (size_t)blockIdx.x * max_ids;
    for (int i = threadIdx.x; i < max_ids; i += blockDim.x) {
        const int id = list[i];
        if (id < 0 || id >= vocab) continue;
        const float l = row[id];
        row[id] = l > 0.f ? l / p : l * p;
    }
}

NI_EXPORT int ni_repetition_penalty(float* logits, const int* ids, const float* penalties, int n_rows,
                                    int vocab, int max_ids, cudaStream_t stream) {
    if (n_rows <= 0 || max_ids <= 0) return NI_OK;
    repetition_penalty_kernel<<<n_rows, 256, 0, stream>>>(logits, ids, penalties, vocab, max_ids);
    NI_RETURN_LAUNCH_STATUS();
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int* __restrict__ out,
              const float* __restrict__ temperatures, const int* __restrict__ top_ks,
              const float* __restrict__ top_ps, const unsigned long long* __restrict__ seeds,
              const unsigned long long* __restrict__ counters, int vocab) {
    __shared__ BlockScratch s;
    extern __shared__ unsigned long long warp_hists[];      // [warps][256]: one histogram per warp
    const int r = blockIdx.x;
    const int tid = threadIdx.x;
    const int n_warps = blockDim.x >> 5;
    unsigned long long* my_hist = warp_hists + (size_t)(tid >> 5) * 256;
    const int vocab_up = (vocab + 31) & ~31;                // whole warps walk the vocabulary
    const float* row = logits + (size_t)r * vocab;
    const float temp = temperatures[r];

    if (temp <= 0.f) {  // greedy row
        float best = -INFINITY;
        int best_i = 0x7fffffff;
        for (int i = tid; i < vocab; i += blockDim.x) {
            const float v = row[i];
            if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        __shared__ float vals[32];
        __shared__ int idxs[32];
        if ((tid & 31) == 0) { vals[tid >> 5] = best; idxs[tid >> 5] = best_i; }
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
                if (vals[w] > best || (vals[w] == best && idxs[w] < best_i)) { best = vals[w]; best_i = idxs[w]; }
            out[r] = best_i == 0x7fffffff ? 0 : best_i;
        }
        return;
    }

    const float inv_t = 1.0f / temp;
    // maximum of the scaled logits
    float m = -INFINITY;
    for (int i = tid; i < vocab; i += blockDim.x) m = fmaxf(m, row[i] * inv_t);
    m = ni_block_max(m, s.fred);

    // ---- top-k: ordered key of the k-th largest scaled logit (exact) ----
    uint32_t key_floor = 0u;  // keep keys >= key_floor
    const int k = top_ks[r];
    if (k > 0 && k < vocab) {
        uint32_t prefix = 0u, mask = 0u;
        unsigned long long remaining = (unsigned long long)k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256 * n_warps; b += blockDim.x) warp_hists[b] = 0ull;
            __syncthreads();
            for (int i = tid; i < vocab_up; i += blockDim.x) {
                const uint32_t key = i < vocab ? ordered_key(row[i] * inv_t) : 0u;
                warp_hist_add(my_hist, (key >> shift) & 255u, 1ull, i < vocab && (key & mask) == prefix);
            }
            __syncthreads();
            for (int b = tid; b < 256; b += blockDim.x) {
                unsigned long long t = 0ull;
                for (int w = 0; w < n_warps; ++w) t += warp_hists[w * 256 + b];
                s.hist[b] = t;
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long above = 0ull;
                int d = 255;
                for (; d > 0; --d) {
                    if (above + s.hist[d] >= remaining) break;
                    above += s.hist[d];
                }
                s.chosen_u32 = (uint32_t)d;
                s.chosen_u64 = remaining - above;
            }
            __syncthreads();
            prefix |= s.chosen_u32 << shift;
            mask |= 255u << shift;
            remaining = s.chosen_u64;
            __syncthreads();
        }
        key_floor = prefix;
    }

    // ---- mass of the tokens that survive top-k ----
    unsigned long long local = 0ull;
    for (int i = tid; i < vocab; i += blockDim.x) {
        const float z = row[i] * inv_t;
        if (ordered_key(z) >= key_floor) local += mass_of(expf(z - m));
    }
    unsigned long long total = block_sum_u64(local, s);

    // ---- top-p: smallest set of most probable tokens whose mass exceeds p * total ----
    uint32_t e_floor = 0u;  // keep tokens whose exp bits >= e_floor (exp >= 0: bits are ordered)
    const float p = top_ps[r];
    if (p > 0.f && p < 1.f) {
        unsigned long long remaining = (unsigned long long)((double)p * (double)total);
        uint32_t prefix = 0u, mask = 0u;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256 * n_warps; b += blockDim.x) warp_hists[b] = 0ull;
            __syncthreads();
            for (int i = tid; i < vocab_up; i += blockDim.x) {
                const float z = i < vocab ? row[i] * inv_t : 0.f;
                const float e = expf(z - m);
                const uint32_t bits = __float_as_uint(e);
                const bool in = i < vocab && ordered_key(z) >= key_floor && (bits & mask) == prefix;
                warp_hist_add(my_hist, (bits >> shift) & 255u, mass_of(e), in);
            }
            __syncthreads();
            for (int b = tid; b < 256; b += blockDim.x) {
                unsigned long long t = 0ull;
                for (int w = 0; w < n_warps; ++w) t += warp_hists[w * 256 + b];
                s.hist[b] = t;
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long above = 0ull;
                int d = 255;
                for (; d > 0; --d) {
                    if (above + s.hist[d] > remaining) break;
                    above += s.hist[d];
                }
                s.chosen_u32 = (uint32_t)d;
                s.chosen_u64 = remaining - above;
            }
            __syncthreads();
            prefix |= s.chosen_u32 << shift;
            mask |= 255u << shift;
            remaining = s.chosen_u64;
            __syncthreads();
        }
        e_floor = prefix;
        local = 0ull;
        for (int i = tid; i < vocab; i += blockDim.x) {
            const float z = row[i] * inv_t;
            if (ordered_key(z) < key_floor) continue;
            const float e = expf(z - m);
            if (__float_as_uint(e) >= e_floor) local += mass_of(e);
        }
        total = block_sum_u64(local, s);
    }

    // ---- draw: first id (in id order) whose inclusive mass exceeds u * total ----
    const uint32_t word = philox_first_word(seeds[r], counters[r]);
    const double u = ((double)(word >> 8) + 0.5) * (1.0 / 16777216.0);  // (0, 1)
    unsigned long long target = (unsigned long long)(u * (double)total);
    if (total > 0ull && target >= total) target = total - 1ull;

    // every warp owns a stretch of the vocabulary (a multiple of 32 ids) and reads it lane by lane;
    // the warp whose stretch holds the target then walks it 32 ids at a time
    const int lane = tid & 31, warp = tid >> 5;
    const int stretch = ((vocab + n_warps - 1) / n_warps + 31) & ~31;
    const int lo = warp * stretch;
    const int hi = min(vocab, lo + stretch);
    auto kept_mass = [&](int i) -> unsigned long long {
        if (i >= hi) return 0ull;
        const float z = row[i] * inv_t;
        if (ordered_key(z) < key_floor) return 0ull;
        const float e = expf(z - m);
        return __float_as_uint(e) >= e_floor ? mass_of(e) : 0ull;
    };
    local = 0ull;
    for (int i = lo + lane; i < hi; i += 32) local += kept_mass(i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    __syncthreads();
    if (lane == 0) s.red[warp] = local;
    if (tid == 0) s.chosen_int = vocab;  // "not found"
    __syncthreads();
    unsigned long long before = 0ull;
    for (int w = 0; w < warp; ++w) before += s.red[w];
    if (local > 0ull && before <= target && target < before + local) {      // (warp-uniform)
        unsigned long long acc = before;
        for (int i0 = lo; i0 < hi; i0 += 32) {
            const unsigned long long mine = kept_mass(i0 + lane);
            unsigned long long incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long n = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += n;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, acc + incl > target);
            if (hit) {
                if (lane == 0) s.chosen_int = i0 + __ffs(hit) - 1;
                break;
            }
            acc += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    __syncthreads();
    if (tid == 0) {
        int pick = s.chosen_int;
        if (pick >= vocab) pick = 0;  // only if every mass rounded to zero
        out[r] = pick;
    }
}

// ---- the same selection by a thread-block cluster per row -----------------------------------------
//
// One block per row walks 128 K logits several times from L2 with one SM's load rate: 92 us for a plain
// temperature draw, 0.5-0.7 ms with top-k or top-p - as long as a whole decode step of a small batch,
// while the other SMs idle.  Here a row belongs to a cluster of SC_RANKS blocks.  Each block keeps its
// eighth of the scaled logits in shared memory, so every pass after the first reads shared memory;
// what the passes reduce (the maximum, the 256-bin histograms of the radix selects, the kept mass)
// every block sends to all blocks of the cluster through distributed shared memory (an all-gather,
// one cluster barrier per pass), and every block draws the same conclusion from the same numbers.
// Sums are the same 64-bit fixed-point sums, the draw the same walk in id order: the result is bit
// for bit that of the one-block kernel.
#define SC_RANKS 8
#define SC_THREADS 512
#define SC_WARPS (SC_THREADS / 32)
#define SC_HISTS (SC_WARPS / 2)  // histograms per block: one per pair of warps (16 KB; with one per warp a second block would not fit an SM)
#define SC_MAX_SLICE 40960      // floats of a block's slice (160 KB): vocabularies up to 327,680

__device__ __forceinline__ uint32_t sc_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void sc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void sc_st_remote(const unsigned long long* local_addr, uint32_t rank, unsigned long long v) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(local_addr), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(a), "r"(rank));
    asm volatile("st.shared::cluster.u64 [%0], %1;\n" ::"r"(remote), "l"(v) : "memory");
}
// Every block's `count` values (src) end up in every block's buf[rank][0..count): buf is [SC_RANKS][256].
__device__ __forceinline__ void sc_all_gather(unsigned long long* buf, const unsigned long long* src, int count, uint32_t my_rank) {
    for (int idx = threadIdx.x; idx < count * SC_RANKS; idx += blockDim.x) {
        const int dst = idx / count, j = idx - dst * count;
        sc_st_remote(buf + my_rank * 256 + j, (uint32_t)dst, src[j]);
    }
    sc_cluster_sync();
}

struct ScScratch {
    unsigned long long hist[256];        // this block's histogram of a pass / values to send
    unsigned long long red[SC_WARPS];
    unsigned long long digit_rest[2];    // the chosen digit and what is left of the count or mass
    int chosen;
};

__global__ void __launch_bounds__(SC_THREADS, 2)
sample_cluster_kernel(const float* __restrict__ logits, int* __restrict__ out,
                      const float* __restrict__ temperatures, const int* __restrict__ top_ks,
                      const float* __restrict__ top_ps, const unsigned long long* __restrict__ seeds,
                      const unsigned long long* __restrict__ counters, int vocab, int slice) {
    extern __shared__ __align__(16) unsigned char sc_smem[];
    float* z = reinterpret_cast<float*>(sc_smem);                                              // [slice]
    unsigned long long* warp_hists = reinterpret_cast<unsigned long long*>(z + slice);       // [SC_HISTS][256]
    unsigned long long* gather = warp_hists + SC_HISTS * 256;                                 // [2][SC_RANKS][256]
    __shared__ ScScratch s;
    const int r = blockIdx.x / SC_RANKS;
    const uint32_t rank = sc_rank();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned long long* my_hist = warp_hists + (size_t)(warp >> 1) * 256;
    const float* row = logits + (size_t)r * vocab;
    const int lo = (int)rank * slice;
    const int n = max(0, min(vocab, lo + slice) - lo);       // this block's ids: lo .. lo + n
    const int n_up = (n + 31) & ~31;
    const float temp = temperatures[r];
    const bool greedy = temp <= 0.f;
    const float inv_t = greedy ? 1.0f : 1.0f / temp;
    sc_cluster_sync();                                       // every block of the cluster runs: its shared memory may be written
    int pass = 0;                                            // which of the two gather buffers is next
    auto next_buf = [&]() { unsigned long long* b = gather + (size_t)(pass & 1) * SC_RANKS * 256; ++pass; return b; };

    // ---- the slice into shared memory; its maximum (with the lowest id that has it) ----
    unsigned long long best = 0ull;                          // (ordered key << 32) | (0xffffffff - id): larger is better
    for (int i = tid; i < n; i += blockDim.x) {
        const float v = row[lo + i] * inv_t;
        z[i] = v;
        // (-0 and +0 are one value to a comparison, but not to the ordered key)
        const unsigned long long cand = ((unsigned long long)ordered_key(v == 0.f ? 0.f : v) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)(lo + i));
        best = cand > best ? cand : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other > best ? other : best;
    }
    if (lane == 0) s.red[warp] = best;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < SC_WARPS; ++w) best = s.red[w] > best ? s.red[w] : best;
        s.hist[0] = best;
    }
    __syncthreads();
    unsigned long long* g = next_buf();
    sc_all_gather(g, s.hist, 1, rank);
    best = g[0];
    for (int c = 1; c < SC_RANKS; ++c) best = g[c * 256] > best ? g[c * 256] : best;
    if (greedy) {
        if (rank == 0 && tid == 0) out[r] = (best >> 32) == 0ull ? 0 : (int)(0xffffffffu - (uint32_t)best);
        return;
    }
    const uint32_t max_key = (uint32_t)(best >> 32);
    const float m = __uint_as_float((max_key & 0x80000000u) ? (max_key & 0x7fffffffu) : ~max_key);

    // One radix select over this cluster's kept tokens: `by_mass` false counts tokens by the ordered
    // key of z (top-k), true sums masses by the bits of exp(z - m) (top-p).  Returns the 32-bit floor.
    auto radix_select = [&](bool by_mass, uint32_t key_floor, unsigned long long remaining, bool strict) -> uint32_t {
        uint32_t prefix = 0u, mask = 0u;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256 * SC_HISTS; b += blockDim.x) warp_hists[b] = 0ull;
            __syncthreads();
            for (int i = tid; i < n_up; i += blockDim.x) {
                const float v = i < n ? z[i] : 0.f;
                uint32_t bits;
                unsigned long long val;
                bool in = i < n;
                if (by_mass) {
                    const float e = expf(v - m);
                    bits = __float_as_uint(e);
                    val = mass_of(e);
                    in = in && ordered_key(v) >= key_floor;
                } else {
                    bits = ordered_key(v);
                    val = 1ull;
                }
                warp_hist_add(my_hist, (bits >> shift) & 255u, val, in && (bits & mask) == prefix);
            }
            __syncthreads();
            for (int b = tid; b < 256; b += blockDim.x) {
                unsigned long long t = 0ull;
                for (int w = 0; w < SC_HISTS; ++w) t += warp_hists[w * 256 + b];
                s.hist[b] = t;
            }
            __syncthreads();
            unsigned long long* gb = next_buf();
            sc_all_gather(gb, s.hist, 256, rank);
            for (int b = tid; b < 256; b += blockDim.x) {
                unsigned long long t = 0ull;
                for (int c = 0; c < SC_RANKS; ++c) t += gb[c * 256 + b];
                s.hist[b] = t;
            }
            __syncthreads();
            // the digit: the largest d >= 1 whose bin, with all bins above it, reaches what is left (else 0).
            // Thread b holds bin b and the sum of the bins above it (a suffix scan over the 256 bins).
            if (tid < 256) {
                const unsigned long long mine = s.hist[tid];
                unsigned long long incl = mine;                       // inclusive suffix sum inside the warp
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned long long nb = __shfl_down_sync(0xffffffffu, incl, o);
                    if (lane + o < 32) incl += nb;
                }
                if (lane == 0) s.red[warp] = incl;                    // the warp's total (8 warps hold the 256 bins)
                asm volatile("bar.sync 1, 256;\n" ::: "memory");
                unsigned long long above = incl - mine;
                for (int w = warp + 1; w < 8; ++w) above += s.red[w];
                const bool reach = strict ? above + mine > remaining : above + mine >= remaining;
                const bool reached_above = strict ? above > remaining : above >= remaining;
                if (tid == 0) { s.digit_rest[0] = 0ull; s.digit_rest[1] = remaining - (above + mine - s.hist[0]); }
                asm volatile("bar.sync 1, 256;\n" ::: "memory");
                if (tid >= 1 && reach && !reached_above) {
                    s.digit_rest[0] = (unsigned long long)tid;
                    s.digit_rest[1] = remaining - above;
                }
            }
            __syncthreads();
            prefix |= (uint32_t)s.digit_rest[0] << shift;
            mask |= 255u << shift;
            remaining = s.digit_rest[1];
            __syncthreads();
        }
        return prefix;
    };
    // The kept mass of this block's slice, every block's share of it (shares[c]) and the total.
    unsigned long long shares[SC_RANKS];
    auto kept_total = [&](uint32_t key_floor, uint32_t e_floor) -> unsigned long long {
        unsigned long long local = 0ull;
        for (int i = tid; i < n; i += blockDim.x) {
            const float v = z[i];
            if (ordered_key(v) < key_floor) continue;
            const float e = expf(v - m);
            if (__float_as_uint(e) >= e_floor) local += mass_of(e);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
        __syncthreads();
        if (lane == 0) s.red[warp] = local;
        __syncthreads();
        if (tid == 0) {
            unsigned long long t = 0ull;
            for (int w = 0; w < SC_WARPS; ++w) t += s.red[w];
            s.hist[0] = t;
        }
        __syncthreads();
        unsigned long long* gb = next_buf();
        sc_all_gather(gb, s.hist, 1, rank);
        unsigned long long total = 0ull;
        for (int c = 0; c < SC_RANKS; ++c) { shares[c] = gb[c * 256]; total += shares[c]; }
        return total;
    };

    uint32_t key_floor = 0u, e_floor = 0u;
    const int k = top_ks[r];
    if (k > 0 && k < vocab) key_floor = radix_select(false, 0u, (unsigned long long)k, false);
    unsigned long long total = kept_total(key_floor, 0u);
    const float p = top_ps[r];
    if (p > 0.f && p < 1.f) {
        e_floor = radix_select(true, key_floor, (unsigned long long)((double)p * (double)total), true);
        total = kept_total(key_floor, e_floor);
    }

    // ---- draw: first id (in id order) whose inclusive mass exceeds u * total ----
    const uint32_t word = philox_first_word(seeds[r], counters[r]);
    const double u = ((double)(word >> 8) + 0.5) * (1.0 / 16777216.0);
    unsigned long long target = (unsigned long long)(u * (double)total);
    if (total > 0ull && target >= total) target = total - 1ull;
    if (total == 0ull) {                                     // only if every mass rounded to zero
        if (rank == 0 && tid == 0) out[r] = 0;
        return;
    }
    unsigned long long before_me = 0ull;
    for (int c = 0; c < (int)rank; ++c) before_me += shares[c];
    if (!(before_me <= target && target < before_me + shares[rank])) return;     // (block-uniform) another block's ids
    // this block holds the id: every warp sums a stretch of the slice, the warp with the target walks it
    auto kept_mass = [&](int i, int end) -> unsigned long long {
        if (i >= end) return 0ull;
        const float v = z[i];
        if (ordered_key(v) < key_floor) return 0ull;
        const float e = expf(v - m);
        return __float_as_uint(e) >= e_floor ? mass_of(e) : 0ull;
    };
    const int stretch = ((n + SC_WARPS - 1) / SC_WARPS + 31) & ~31;
    const int w_lo = min(n, warp * stretch), w_hi = min(n, w_lo + stretch);
    unsigned long long local = 0ull;
    for (int i = w_lo + lane; i < w_hi; i += 32) local += kept_mass(i, w_hi);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    __syncthreads();
    if (lane == 0) s.red[warp] = local;
    __syncthreads();
    unsigned long long before = before_me;
    for (int w = 0; w < warp; ++w) before += s.red[w];
    if (local > 0ull && before <= target && target < before + local) {           // (warp-uniform)
        unsigned long long acc = before;
        for (int i0 = w_lo; i0 < w_hi; i0 += 32) {
            unsigned long long incl = kept_mass(i0 + lane, w_hi);
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long nb = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += nb;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, acc + incl > target);
            if (hit) {
                if (lane == 0) out[r] = lo + i0 + __ffs(hit) - 1;
                break;
            }
            acc += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
}

// One launch for a batch with per-row parameters.  temperatures[r] <= 0 selects arg-max.
// top_ks[r] <= 0 or >= vocab: no top-k; top_ps[r] outside (0, 1): no top-p.
static int sample_by_cluster = 1;
// 0: always the one-block-per-row kernel (for comparisons); 1: a cluster per row where it fits (the default).
NI_EXPORT int ni_sample_set_cluster(int on) { sample_by_cluster = on; return NI_OK; }

NI_EXPORT int ni_sample(const float* logits, int* out, const float* temperatures, const int* top_ks,
                        const float* top_ps, const unsigned long long* seeds,
                        const unsigned long long* counters, int n_rows, int vocab, cudaStream_t stream) {
    if (n_rows <= 0) return NI_OK;
    if (vocab <= 0) return NI_ERR_BAD_ARGUMENT;
    if (vocab > (1 << 25)) return NI_ERR_UNSUPPORTED_SIZE;  // fixed-point mass would overflow
    // a cluster per row while a block's slice of the vocabulary fits its shared memory
    const int slice = (((vocab + SC_RANKS - 1) / SC_RANKS) + 31) & ~31;
    if (sample_by_cluster && vocab >= 4096 && slice <= SC_MAX_SLICE) {
        const size_t sc_smem = (size_t)slice * sizeof(float) + (size_t)(SC_HISTS + 2 * SC_RANKS) * 256 * sizeof(unsigned long long);
        static size_t sc_configured = 0;
        if (sc_configured < sc_smem) {
            cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sc_smem);
            if (e != cudaSuccess) return (int)e;
            sc_configured = sc_smem;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)n_rows * SC_RANKS);
        cfg.blockDim = dim3(SC_THREADS);
        cfg.dynamicSmemBytes = sc_smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = SC_RANKS;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, sample_cluster_kernel, logits, out, temperatures, top_ks, top_ps, seeds,
                                           counters, vocab, slice);
        return e == cudaSuccess ? NI_OK : (int)e;
    }
    const size_t smem = (size_t)(SAMPLE_THREADS / 32) * 256 * sizeof(unsigned long long);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    sample_kernel<<<n_rows, SAMPLE_THREADS, smem, stream>>>(logits, out, temperatures, top_ks, top_ps,
                                                           seeds, counters, vocab);
    NI_RETURN_LAUNCH_STATUS();
}
