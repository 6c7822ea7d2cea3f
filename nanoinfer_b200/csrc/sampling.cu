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
    const int r = blockIdx.x;
    const int tid = threadIdx.x;
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
            for (int b = tid; b < 256; b += blockDim.x) s.hist[b] = 0ull;
            __syncthreads();
            for (int i = tid; i < vocab; i += blockDim.x) {
                const uint32_t key = ordered_key(row[i] * inv_t);
                if ((key & mask) == prefix) atomicAdd(&s.hist[(key >> shift) & 255u], 1ull);
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
            for (int b = tid; b < 256; b += blockDim.x) s.hist[b] = 0ull;
            __syncthreads();
            for (int i = tid; i < vocab; i += blockDim.x) {
                const float z = row[i] * inv_t;
                if (ordered_key(z) < key_floor) continue;
                const float e = expf(z - m);
                const uint32_t bits = __float_as_uint(e);
                if ((bits & mask) == prefix) atomicAdd(&s.hist[(bits >> shift) & 255u], mass_of(e));
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

    const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
    const int lo = tid * chunk;
    const int hi = min(vocab, lo + chunk);
    local = 0ull;
    for (int i = lo; i < hi; ++i) {
        const float z = row[i] * inv_t;
        if (ordered_key(z) < key_floor) continue;
        const float e = expf(z - m);
        if (__float_as_uint(e) >= e_floor) local += mass_of(e);
    }
    // exclusive scan of the chunk sums over the block (warp scan, then warp totals)
    unsigned long long incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long n = __shfl_up_sync(0xffffffffu, incl, o);
        if ((tid & 31) >= o) incl += n;
    }
    __syncthreads();
    if ((tid & 31) == 31) s.red[tid >> 5] = incl;
    if (tid == 0) s.chosen_int = vocab;  // "not found"
    __syncthreads();
    unsigned long long before = 0ull;
    for (int w = 0; w < (tid >> 5); ++w) before += s.red[w];
    const unsigned long long excl = before + incl - local;
    if (local > 0ull && excl <= target && target < excl + local) {
        unsigned long long acc = excl;
        for (int i = lo; i < hi; ++i) {
            const float z = row[i] * inv_t;
            if (ordered_key(z) < key_floor) continue;
            const float e = expf(z - m);
            if (__float_as_uint(e) < e_floor) continue;
            acc += mass_of(e);
            if (acc > target) { s.chosen_int = i; break; }
        }
    }
    __syncthreads();
    if (tid == 0) {
        int pick = s.chosen_int;
        if (pick >= vocab) pick = 0;  // only if every mass rounded to zero
        out[r] = pick;
    }
}

// One launch for a batch with per-row parameters.  temperatures[r] <= 0 selects arg-max.
// top_ks[r] <= 0 or >= vocab: no top-k; top_ps[r] outside (0, 1): no top-p.
NI_EXPORT int ni_sample(const float* logits, int* out, const float* temperatures, const int* top_ks,
                        const float* top_ps, const unsigned long long* seeds,
                        const unsigned long long* counters, int n_rows, int vocab, cudaStream_t stream) {
    if (n_rows <= 0) return NI_OK;
    if (vocab <= 0) return NI_ERR_BAD_ARGUMENT;
    if (vocab > (1 << 25)) return NI_ERR_UNSUPPORTED_SIZE;  // fixed-point mass would overflow
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, out, temperatures, top_ks, top_ps,
                                                        seeds, counters, vocab);
    NI_RETURN_LAUNCH_STATUS();
}
