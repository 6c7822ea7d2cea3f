"""Makes tests/golden/reference_cpu_kernels.npz: outputs of the reference project's own C++ CPU
kernels, compiled here unchanged, for the formulas that its Python model (tools/model.py) does
not contain:

  * sin_cos_cache_calc_cpu and rope_kernel_cpu (src/op/kernels/cpu/rope_kernel.cpp:39-153):
    the llama3 frequency rule with all three branches taken, and the rotation of adjacent pairs;
  * paged_attention_kernel_cpu (src/op/kernels/cpu/paged_attention_kernel.cpp:44-135): single
    query tokens over a paged cache with a shuffled block table;
  * prefill_attention_kernel_cpu (src/op/kernels/cpu/prefill_attention_kernel.cpp:47-159): a
    portion of a prompt that starts in the middle of a sequence, written into pages first.

Run once by hand from the repository root, with the reference project's path:
    python tests/golden/make_kernel_golden.py /path/to/NanoInfer

The reference's sources are compiled from where they lie (nothing is copied): the three kernel
files with src/tensor/tensor.cpp and src/base/*.cpp, against two stub headers written to a
temporary folder - a glog/logging.h that provides CHECK / LOG as no-op streams, and an empty
armadillo (rope_kernel.cpp includes it without using it) - and linked with the CUDA runtime
library that tensor.cpp names (no CUDA call is made).  tests/test_reference_kernels.py compares
the plain implementation with the stored outputs, and rebuilds them when NANOINFER_REFERENCE is set.
"""
import ctypes
import os
import subprocess
import sys
import tempfile

import numpy as np

GLOG_STUB = r"""
#pragma once
#include <cstdlib>
#include <iostream>
#include <sstream>
struct NiNullStream {
    template <typename T> NiNullStream& operator<<(const T&) { return *this; }
    NiNullStream& operator<<(std::ostream& (*)(std::ostream&)) { return *this; }
};
struct NiFatalStream {
    std::ostringstream s;
    template <typename T> NiFatalStream& operator<<(const T& v) { s << v; return *this; }
    ~NiFatalStream() { std::cerr << "CHECK failed: " << s.str() << std::endl; std::abort(); }
};
struct NiVoidify { void operator&(const NiNullStream&) {} void operator&(const NiFatalStream&) {} };
#define LOG(level) NiNullStream()
#define LOG_IF(level, c) NiNullStream()
#define VLOG(n) NiNullStream()
#define DLOG(level) NiNullStream()
#define CHECK(c) (c) ? (void)0 : NiVoidify() & NiFatalStream() << #c << " "
#define CHECK_OP_(a, b, op) CHECK((a) op (b))
#define CHECK_EQ(a, b) CHECK_OP_(a, b, ==)
#define CHECK_NE(a, b) CHECK_OP_(a, b, !=)
#define CHECK_LT(a, b) CHECK_OP_(a, b, <)
#define CHECK_LE(a, b) CHECK_OP_(a, b, <=)
#define CHECK_GT(a, b) CHECK_OP_(a, b, >)
#define CHECK_GE(a, b) CHECK_OP_(a, b, >=)
#define DCHECK(c) CHECK(c)
namespace google { inline void InitGoogleLogging(const char*) {} }
"""

HARNESS = r"""
#include <cstdint>
#include <memory>
#include "nanoinfer/base/alloc.h"
#include "nanoinfer/tensor/tensor.h"

namespace kernel {
void rope_kernel_cpu(int32_t dim, int32_t kv_dim, int32_t head_size, const tensor::Tensor& input_q,
                     const tensor::Tensor& input_k, const tensor::Tensor& input_pos, const tensor::Tensor& sin_cache,
                     const tensor::Tensor& cos_cache, void* stream);
void sin_cos_cache_calc_cpu(int32_t head_size, int32_t max_seq_len, const tensor::Tensor& sin_cache,
                            const tensor::Tensor& cos_cache, float rope_theta, bool has_rope_scaling,
                            float scaling_factor, float low_freq_factor, float high_freq_factor,
                            int32_t original_max_pos, void* stream);
void paged_attention_kernel_cpu(const tensor::Tensor& query, const tensor::Tensor& output, const tensor::Tensor& k_cache,
                                const tensor::Tensor& v_cache, const tensor::Tensor& block_table,
                                const tensor::Tensor& context_lens, int32_t max_context_len, int32_t num_heads,
                                int32_t num_kv_heads, int32_t head_size, int32_t block_size, float scale, void* stream);
void prefill_attention_kernel_cpu(const tensor::Tensor& query, const tensor::Tensor& key, const tensor::Tensor& value,
                                  const tensor::Tensor& output, const tensor::Tensor& k_cache, const tensor::Tensor& v_cache,
                                  const tensor::Tensor& block_table, const tensor::Tensor& positions, int32_t num_heads,
                                  int32_t num_kv_heads, int32_t head_size, int32_t block_size, int32_t context_len,
                                  void* stream);
}

static tensor::Tensor wrap_f(float* p, std::vector<int32_t> dims) {
    tensor::Tensor t(base::DataType::kDataTypeFp32, dims, false, nullptr, p);
    t.set_device_type(base::DeviceType::kDeviceCPU);
    return t;
}
static tensor::Tensor wrap_i(int32_t* p, std::vector<int32_t> dims) {
    tensor::Tensor t(base::DataType::kDataTypeInt32, dims, false, nullptr, p);
    t.set_device_type(base::DeviceType::kDeviceCPU);
    return t;
}

extern "C" {
void ref_sin_cos(int head, int max_len, float* sin, float* cos, float theta, int has, float factor, float low,
                 float high, int orig) {
    kernel::sin_cos_cache_calc_cpu(head, max_len, wrap_f(sin, {max_len, head}), wrap_f(cos, {max_len, head}), theta,
                                   has != 0, factor, low, high, orig, nullptr);
}
void ref_rope(int dim, int kv_dim, int head, float* q, float* k, int32_t* pos, int n, float* sin, float* cos, int max_len) {
    kernel::rope_kernel_cpu(dim, kv_dim, head, wrap_f(q, {n, dim}), wrap_f(k, {n, kv_dim}), wrap_i(pos, {n}),
                            wrap_f(sin, {max_len, head}), wrap_f(cos, {max_len, head}), nullptr);
}
void ref_paged_attention(float* q, float* out, float* kc, float* vc, int32_t* table, int32_t* lens, int batch,
                         int max_blocks, int n_blocks, int heads, int kv_heads, int head, int block, float scale) {
    kernel::paged_attention_kernel_cpu(wrap_f(q, {batch, heads * head}), wrap_f(out, {batch, heads * head}),
                                       wrap_f(kc, {n_blocks, block, kv_heads, head}), wrap_f(vc, {n_blocks, block, kv_heads, head}),
                                       wrap_i(table, {batch, max_blocks}), wrap_i(lens, {batch}), 0, heads, kv_heads, head,
                                       block, scale, nullptr);
}
void ref_prefill_attention(float* q, float* k, float* v, float* out, float* kc, float* vc, int32_t* table,
                           int32_t* pos, int chunk, int max_blocks, int n_blocks, int heads, int kv_heads, int head,
                           int block, int context_len) {
    kernel::prefill_attention_kernel_cpu(wrap_f(q, {chunk, heads * head}), wrap_f(k, {chunk, kv_heads * head}),
                                         wrap_f(v, {chunk, kv_heads * head}), wrap_f(out, {chunk, heads * head}),
                                         wrap_f(kc, {n_blocks, block, kv_heads, head}),
                                         wrap_f(vc, {n_blocks, block, kv_heads, head}), wrap_i(table, {1, max_blocks}),
                                         wrap_i(pos, {chunk}), heads, kv_heads, head, block, context_len, nullptr);
}
}
"""


def build(ref_root: str, work: str) -> ctypes.CDLL:
    """Compile the reference's CPU kernels (unchanged, from ``ref_root``) with the harness."""
    stub = os.path.join(work, "stub")
    os.makedirs(os.path.join(stub, "glog"), exist_ok=True)
    with open(os.path.join(stub, "glog", "logging.h"), "w") as f:
        f.write(GLOG_STUB)
    with open(os.path.join(stub, "armadillo"), "w") as f:
        f.write("#pragma once\n")
    harness = os.path.join(work, "harness.cpp")
    with open(harness, "w") as f:
        f.write(HARNESS)
    src = os.path.join(ref_root, "src")
    files = [os.path.join(src, "op/kernels/cpu", n) for n in
             ("rope_kernel.cpp", "paged_attention_kernel.cpp", "prefill_attention_kernel.cpp")]
    files += [os.path.join(src, "tensor/tensor.cpp")]
    files += [os.path.join(src, "base", n) for n in sorted(os.listdir(os.path.join(src, "base"))) if n.endswith(".cpp")]
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    lib = os.path.join(work, "libref_kernels.so")
    cmd = ["g++", "-O1", "-std=c++17", "-fPIC", "-shared", "-w", "-include", "cstring", "-include", "cfloat",
           "-I", stub, "-I", os.path.join(ref_root, "include"), "-I", src, "-I", os.path.join(cuda, "include"),
           harness] + files + ["-L", os.path.join(cuda, "lib64"), "-lcudart", "-Wl,-rpath," + os.path.join(cuda, "lib64"),
                               "-o", lib]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("the reference's CPU kernels did not compile:\n" + proc.stderr[-4000:])
    return ctypes.CDLL(lib)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


# (name, head size, theta, scaling or None, positions): Tiny B's and the 1B shape's parameters
# (all three branches of the rule occur in both), one without scaling, one with factor 8.
ROPE_CASES = [
    ("tiny_b", 32, 500000.0, (32.0, 1.0, 4.0, 64), 512),
    ("llama_1b", 64, 500000.0, (32.0, 1.0, 4.0, 8192), 4096),
    ("plain", 16, 10000.0, None, 128),
    ("factor8_hd128", 128, 500000.0, (8.0, 1.0, 4.0, 8192), 1024),
]
# (name, query heads, kv heads, head size, block size, context lengths)
DECODE_CASES = [("gqa", 4, 2, 16, 16, [1, 17, 48, 100]), ("mqa_odd", 3, 1, 32, 8, [7, 8, 9, 130])]
# (name, query heads, kv heads, head size, block size, start position, portion length)
PREFILL_CASES = [("from_zero", 4, 2, 16, 16, 0, 37), ("mid_sequence", 6, 2, 32, 8, 29, 24)]


def generate(lib) -> dict:
    out = {}
    rng = np.random.default_rng(0)
    for name, hd, theta, sc, n_pos in ROPE_CASES:
        sin = np.zeros((n_pos, hd), dtype=np.float32)
        cos = np.zeros((n_pos, hd), dtype=np.float32)
        f, lo, hi, orig = sc if sc else (1.0, 1.0, 1.0, 1)
        lib.ref_sin_cos(hd, n_pos, _p(sin), _p(cos), ctypes.c_float(theta), 1 if sc else 0, ctypes.c_float(f),
                        ctypes.c_float(lo), ctypes.c_float(hi), orig)
        out[f"rope/{name}/sin"], out[f"rope/{name}/cos"] = sin, cos
        n, heads, kv = 9, 3, 1
        q = rng.standard_normal((n, heads * hd)).astype(np.float32)
        k = rng.standard_normal((n, kv * hd)).astype(np.float32)
        pos = rng.integers(0, min(n_pos, 128), n).astype(np.int32)     # small angles: FP32 agrees to 1e-5 there
        out[f"rope/{name}/q_in"], out[f"rope/{name}/k_in"], out[f"rope/{name}/pos"] = q.copy(), k.copy(), pos
        lib.ref_rope(heads * hd, kv * hd, hd, _p(q), _p(k), _p(pos), n, _p(sin), _p(cos), n_pos)
        out[f"rope/{name}/q_out"], out[f"rope/{name}/k_out"] = q, k
    for name, hq, hkv, hd, bs, lens in DECODE_CASES:
        batch = len(lens)
        max_blocks = max(-(-l // bs) for l in lens)
        n_blocks = sum(-(-l // bs) for l in lens) + 3
        perm = rng.permutation(n_blocks).astype(np.int32)
        table = np.full((batch, max_blocks), -1, dtype=np.int32)
        at = 0
        for b, l in enumerate(lens):
            nb = -(-l // bs)
            table[b, :nb] = perm[at:at + nb]
            at += nb
        kc = rng.standard_normal((n_blocks, bs, hkv, hd)).astype(np.float32)
        vc = rng.standard_normal((n_blocks, bs, hkv, hd)).astype(np.float32)
        q = rng.standard_normal((batch, hq * hd)).astype(np.float32)
        o = np.zeros_like(q)
        cl = np.asarray(lens, dtype=np.int32)
        lib.ref_paged_attention(_p(q), _p(o), _p(kc), _p(vc), _p(table), _p(cl), batch, max_blocks, n_blocks, hq, hkv, hd,
                                bs, ctypes.c_float(1.0 / np.sqrt(hd)))
        for key, val in (("q", q), ("out", o), ("k_cache", kc), ("v_cache", vc), ("table", table), ("lens", cl)):
            out[f"decode/{name}/{key}"] = val
    for name, hq, hkv, hd, bs, start, chunk in PREFILL_CASES:
        ctx = start + chunk
        max_blocks = -(-ctx // bs)
        n_blocks = max_blocks + 2
        table = rng.permutation(n_blocks)[:max_blocks].astype(np.int32).reshape(1, max_blocks)
        kc = np.zeros((n_blocks, bs, hkv, hd), dtype=np.float32)
        vc = np.zeros((n_blocks, bs, hkv, hd), dtype=np.float32)
        k_all = rng.standard_normal((ctx, hkv * hd)).astype(np.float32)
        v_all = rng.standard_normal((ctx, hkv * hd)).astype(np.float32)
        for t in range(start):                                   # what earlier portions left in the cache
            kc[table[0, t // bs], t % bs] = k_all[t].reshape(hkv, hd)
            vc[table[0, t // bs], t % bs] = v_all[t].reshape(hkv, hd)
        q = rng.standard_normal((chunk, hq * hd)).astype(np.float32)
        k, v = np.ascontiguousarray(k_all[start:]), np.ascontiguousarray(v_all[start:])
        o = np.zeros_like(q)
        pos = np.arange(start, ctx, dtype=np.int32)
        lib.ref_prefill_attention(_p(q), _p(k), _p(v), _p(o), _p(kc), _p(vc), _p(table), _p(pos), chunk, max_blocks,
                                  n_blocks, hq, hkv, hd, bs, ctx)
        for key, val in (("q", q), ("k_all", k_all), ("v_all", v_all), ("out", o), ("k_cache_after", kc), ("table", table)):
            out[f"prefill/{name}/{key}"] = val
    return out


def main() -> int:
    if len(sys.argv) != 2:
        print(__doc__)
        return 2
    with tempfile.TemporaryDirectory() as work:
        lib = build(sys.argv[1], work)
        data = generate(lib)
    # float16-free, compressed: a few hundred KB (the sin/cos tables are kept at the positions a test reads)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_cpu_kernels.npz")
    slim = {}
    for k, v in data.items():
        if k.endswith("/sin") or k.endswith("/cos"):
            rows = sorted(set(list(range(0, 40)) + list(range(v.shape[0] - 8, v.shape[0])) + list(range(0, v.shape[0], 97))))
            slim[k + "_rows"] = np.asarray(rows, dtype=np.int32)
            slim[k] = v[rows]
        else:
            slim[k] = v
    np.savez_compressed(path, **slim)
    print(f"wrote {path}: {len(slim)} arrays, {os.path.getsize(path) / 1024:.0f} KB")
    return 0


if __name__ == "__main__":
    sys.exit(main())
