"""Each kernel alone against a plain FP32 computation of the same op, at sizes other than
the engine tests': widths and vocabularies that are no power of two, head sizes in steps of
16, odd head counts and page sizes."""
import math

import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dtype):
    # float32: rounding in a different order.  bfloat16: the kernels compute in FP32 and round
    # the result once: one unit in the last place of bfloat16 (2^-8) plus cancellation slack.
    return dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=4e-3, atol=1e-3)


def _randn(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,vocab", [(64, 100), (120, 1000), (2056, 333)])
def test_embedding(dtype, d, vocab):
    from nanoinfer_b200.kernels import ops
    table = _randn(vocab, d, dtype=dtype)
    tokens = torch.randint(0, vocab, (37,), generator=torch.Generator().manual_seed(1)).int().to(DEV)
    out = torch.empty(37, d, dtype=torch.float32, device=DEV)
    ops.embedding(tokens, table, out)
    assert torch.equal(out.cpu(), plain.embedding(table.cpu(), tokens.cpu()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,eps", [(64, 1e-5), (120, 1e-6), (2056, 1e-5), (8200, 1e-3)])
def test_add_rmsnorm(dtype, d, eps):
    from nanoinfer_b200.kernels import ops
    n = 19
    h = _randn(n, d, seed=1)
    delta = _randn(n, d, dtype=dtype, seed=2)
    gain = _randn(d, seed=3) + 1.0
    want_h = h.cpu() + delta.cpu().float()
    want = plain.rms_norm(want_h, gain.cpu(), eps)
    out = torch.empty(n, d, dtype=dtype, device=DEV)
    h1 = h.clone()
    ops.add_rmsnorm(h1, delta, gain, eps, out)
    torch.testing.assert_close(h1.cpu(), want_h, rtol=0, atol=0)
    torch.testing.assert_close(out.cpu().float(), want, **_tol(dtype))
    # without an addition
    h2 = h.clone()
    ops.add_rmsnorm(h2, None, gain, eps, out)
    assert torch.equal(h2, h)
    torch.testing.assert_close(out.cpu().float(), plain.rms_norm(h.cpu(), gain.cpu(), eps), **_tol(dtype))
    # selected rows only: h untouched, rows may repeat
    rows = torch.tensor([18, 0, 7, 7], dtype=torch.int32, device=DEV)
    out_r = torch.empty(4, d, dtype=dtype, device=DEV)
    h3 = h.clone()
    ops.add_rmsnorm(h3, delta, gain, eps, out_r, rows)
    assert torch.equal(h3, h)
    torch.testing.assert_close(out_r.cpu().float(), want[rows.cpu().long()], **_tol(dtype))


@pytest.mark.parametrize("d", [512, 1024, 2048, 3072])
def test_add_rmsnorm_of_many_rows(d):
    """Many bfloat16 rows of a width that is a multiple of 128 take the warp-per-row kernel; a last
    block with fewer rows than warps, selected rows, and the same result as the few-row kernel up
    to the order of the sum of squares."""
    from nanoinfer_b200.kernels import ops
    n, eps = 1027, 1e-5
    h = _randn(n, d, seed=1)
    delta = _randn(n, d, dtype=torch.bfloat16, seed=2)
    gain = _randn(d, seed=3) + 1.0
    want_h = h.cpu() + delta.cpu().float()
    want = plain.rms_norm(want_h, gain.cpu(), eps)
    out = torch.empty(n, d, dtype=torch.bfloat16, device=DEV)
    h1 = h.clone()
    ops.add_rmsnorm(h1, delta, gain, eps, out)
    torch.testing.assert_close(h1.cpu(), want_h, rtol=0, atol=0)
    torch.testing.assert_close(out.cpu().float(), want, **_tol(torch.bfloat16))
    few = torch.empty(40, d, dtype=torch.bfloat16, device=DEV)
    h2 = h[:40].clone()
    ops.add_rmsnorm(h2, delta[:40].contiguous(), gain, eps, few)
    torch.testing.assert_close(few.float(), out[:40].float(), rtol=8e-3, atol=1e-6)     # one bfloat16 step at most
    rows = torch.randperm(n, generator=torch.Generator().manual_seed(4))[:1024].int().to(DEV)
    out_r = torch.empty(1024, d, dtype=torch.bfloat16, device=DEV)
    h3 = h.clone()
    ops.add_rmsnorm(h3, delta, gain, eps, out_r, rows)
    assert torch.equal(h3, h)
    assert torch.equal(out_r, out[rows.long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [192, 200, 8200])
def test_swiglu(dtype, inter):
    from nanoinfer_b200.kernels import ops
    gu = _randn(11, 2 * inter, dtype=dtype, scale=3.0)
    out = torch.empty(11, inter, dtype=dtype, device=DEV)
    ops.swiglu(gu, out)
    g, u = gu.cpu().float()[:, :inter], gu.cpu().float()[:, inter:]
    torch.testing.assert_close(out.cpu().float(), (g / (1 + torch.exp(-g))) * u, **_tol(dtype))


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (7, 100, 120), (65, 333, 200), (130, 64, 2056)])
def test_gemm_f32(m, n, k):
    from nanoinfer_b200.kernels import ops
    x, w = _randn(m, k, seed=1), _randn(n, k, seed=2)
    out = torch.empty(m, n, dtype=torch.float32, device=DEV)
    ops.gemm_f32(x, w, out)
    want = (x.cpu().double() @ w.cpu().double().t()).float()
    torch.testing.assert_close(out.cpu(), want, rtol=1e-5, atol=1e-5 * math.sqrt(k))
    # a row's result does not depend on the rows beside it
    out1 = torch.empty(1, n, dtype=torch.float32, device=DEV)
    ops.gemm_f32(x[m - 1:m].contiguous(), w, out1)
    assert torch.equal(out1[0], out[m - 1])


def _paged_setup(T_per_seq, n_kv, hd, page, dtype, seed):
    """Random k/v for sequences of the given lengths, scattered over shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    n_seq = len(T_per_seq)
    width = max(-(-t // page) for t in T_per_seq)
    n_pages = sum(-(-t // page) for t in T_per_seq) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((n_seq, width), -1, dtype=torch.int32)
    ks, vs = [], []
    k_pages = torch.zeros(n_pages, n_kv, page, hd, dtype=dtype)
    v_pages = torch.zeros_like(k_pages)
    for s, t in enumerate(T_per_seq):
        k = (torch.randn(t, n_kv, hd, generator=g)).to(dtype)
        v = (torch.randn(t, n_kv, hd, generator=g)).to(dtype)
        ks.append(k); vs.append(v)
        for j in range(t):
            if j % page == 0:
                table[s, j // page] = perm.pop()
            p = table[s, j // page]
            k_pages[p, :, j % page] = k[j]
            v_pages[p, :, j % page] = v[j]
    return table, k_pages, v_pages, ks, vs


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,hd,page,window", [(4, 2, 16, 16, None), (3, 1, 32, 8, None),
                                                      (6, 3, 48, 4, 20), (5, 5, 80, 16, None),
                                                      (8, 2, 128, 32, 100), (2, 1, 256, 16, None)])
def test_attention_generic(dtype, n_q, n_kv, hd, page, window):
    from nanoinfer_b200.kernels import ops
    lens = [37, 1, 150]
    table, k_pages, v_pages, ks, vs = _paged_setup(lens, n_kv, hd, page, dtype, seed=hd)
    # queries: the last 5 tokens of seq 0, the only token of seq 1, tokens 100..149 of seq 2
    spans = [(32, 37), (0, 1), (100, 150)]
    g = torch.Generator().manual_seed(5)
    qs = [torch.randn(t, n_q, hd, generator=g).to(dtype) for t in lens]
    q = torch.cat([qs[s][a:b] for s, (a, b) in enumerate(spans)]).reshape(-1, n_q * hd)
    positions = torch.cat([torch.arange(a, b) for a, b in spans]).int()
    seq_of = torch.cat([torch.full((b - a,), s) for s, (a, b) in enumerate(spans)]).int()
    out = torch.empty_like(q).to(DEV)
    scale = 1.0 / math.sqrt(hd)
    ops.attention_generic(q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), out, positions.to(DEV),
                          seq_of.to(DEV), table.to(DEV), n_q, n_kv, hd, page, window, scale)
    want = torch.cat([plain.attention(qs[s], ks[s], vs[s], scale, window)[a:b]
                      for s, (a, b) in enumerate(spans)]).reshape(-1, n_q * hd)
    torch.testing.assert_close(out.cpu().float(), want, **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,hd,page,window", [(6, 2, 48, 4, None), (5, 1, 80, 16, 33)])
def test_attention_generic_with_a_slope_per_head(dtype, n_q, n_kv, hd, page, window):
    """score = q.k * scale + slope[h] * (key position - query position), over pages, for a span of
    queries in the middle of a sequence; the plain side is written out here."""
    from nanoinfer_b200.kernels import ops
    lens = [150, 9]
    table, k_pages, v_pages, ks, vs = _paged_setup(lens, n_kv, hd, page, dtype, seed=hd + 1)
    spans = [(90, 150), (8, 9)]
    g = torch.Generator().manual_seed(6)
    qs = [torch.randn(t, n_q, hd, generator=g).to(dtype) for t in lens]
    slopes = torch.rand(n_q, generator=g) * 0.5
    q = torch.cat([qs[s][a:b] for s, (a, b) in enumerate(spans)]).reshape(-1, n_q * hd)
    positions = torch.cat([torch.arange(a, b) for a, b in spans]).int()
    seq_of = torch.cat([torch.full((b - a,), s) for s, (a, b) in enumerate(spans)]).int()
    out = torch.empty_like(q).to(DEV)
    scale = 1.0 / math.sqrt(hd)
    ops.attention_generic(q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), out, positions.to(DEV),
                          seq_of.to(DEV), table.to(DEV), n_q, n_kv, hd, page, window, scale,
                          head_slopes=slopes.to(DEV))
    want = []
    for s, (a, b) in enumerate(spans):
        t = lens[s]
        i = torch.arange(t)
        mask = i[None, :] <= i[:, None]
        if window is not None:
            mask &= i[None, :] > i[:, None] - window
        o = torch.empty(t, n_q, hd)
        for h in range(n_q):
            kh, vh = ks[s][:, h // (n_q // n_kv)].float(), vs[s][:, h // (n_q // n_kv)].float()
            sc = (qs[s][:, h].float() @ kh.t()) * scale + slopes[h] * (i[None, :] - i[:, None]).float()
            o[:, h] = torch.softmax(sc.masked_fill(~mask, float("-inf")), dim=-1) @ vh
        want.append(o[a:b])
    torch.testing.assert_close(out.cpu().float(), torch.cat(want).reshape(-1, n_q * hd), **_tol(dtype))
    with pytest.raises(ops.KernelError, match="one slope per query head"):
        ops.attention_generic(q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), out, positions.to(DEV),
                              seq_of.to(DEV), table.to(DEV), n_q, n_kv, hd, page, window, scale,
                              head_slopes=slopes[:-1].to(DEV))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pairing", ["half", "interleaved"])
@pytest.mark.parametrize("n_q,n_kv,hd,rot,page", [(4, 2, 16, 16, 16), (3, 1, 32, 32, 8), (6, 3, 48, 32, 4),
                                                  (5, 5, 80, 80, 16)])
def test_rope_kv_write(dtype, pairing, n_q, n_kv, hd, rot, page):
    from nanoinfer_b200.kernels import ops
    lens = [9, 70]
    starts = [4, 60]          # tokens [start, len) of each sequence are in this step
    width = max(-(-t // page) for t in lens)
    n_pages = 2 * width + 2
    g = torch.Generator().manual_seed(rot)
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.tensor([[perm.pop() for _ in range(width)] for _ in lens], dtype=torch.int32)
    positions = torch.cat([torch.arange(s, t) for s, t in zip(starts, lens)]).int()
    seq_of = torch.cat([torch.full((t - s,), i) for i, (s, t) in enumerate(zip(starts, lens))]).int()
    T = positions.numel()
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, generator=g).to(dtype)
    inv_freq = plain.rope_inv_freq(rot, 10000.0, None)
    q_out = torch.empty(T, n_q * hd, dtype=dtype, device=DEV)
    k_pages = torch.full((n_pages, n_kv, page, hd), 7.0, dtype=dtype, device=DEV)
    v_pages = torch.full((n_pages, n_kv, page, hd), 7.0, dtype=dtype, device=DEV)
    ops.rope_kv_write(qkv.to(DEV), q_out, k_pages, v_pages, positions.to(DEV), seq_of.to(DEV),
                      table.to(DEV), inv_freq.to(DEV), n_q, n_kv, hd, rot, pairing == "interleaved", page)
    qf = qkv.float()
    q = plain.rope(qf[:, :n_q * hd].view(T, n_q, hd), positions, inv_freq, pairing)
    k = plain.rope(qf[:, n_q * hd:(n_q + n_kv) * hd].view(T, n_kv, hd), positions, inv_freq, pairing)
    v = qf[:, (n_q + n_kv) * hd:].view(T, n_kv, hd)
    torch.testing.assert_close(q_out.cpu().float().view(T, n_q, hd), q, **_tol(dtype))
    touched = torch.zeros(n_pages, page, dtype=torch.bool)
    kp, vp = k_pages.cpu().float(), v_pages.cpu().float()
    for t in range(T):
        p, slot = table[seq_of[t], positions[t] // page], positions[t] % page
        torch.testing.assert_close(kp[p, :, slot], k[t], **_tol(dtype))
        torch.testing.assert_close(vp[p, :, slot], v[t].to(dtype).float(), rtol=0, atol=0)
        touched[p, slot] = True
    # nothing else was written
    assert torch.all(kp.permute(0, 2, 1, 3)[~touched] == 7.0)
    assert torch.all(vp.permute(0, 2, 1, 3)[~touched] == 7.0)


@pytest.mark.parametrize("mode", ["bf16", "f32", "add"])
@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (3, 100, 120), (8, 4800, 2048), (9, 333, 200), (16, 520, 8200),
                                   (5, 2048, 8192), (7, 1000, 3072), (8, 600, 4096), (2, 328, 2056),
                                   (3, 200, 3080), (9, 200, 3072)])
def test_gemv_bf16(m, n, k, mode):
    from nanoinfer_b200.kernels import ops
    x = _randn(m, k, dtype=torch.bfloat16, seed=1)
    w = _randn(n, k, dtype=torch.bfloat16, seed=2, scale=0.05)
    want = x.cpu().double() @ w.cpu().double().t()
    if mode == "bf16":
        out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
        ops.gemv_bf16(x, w, out, ops.STORE_BF16)
        torch.testing.assert_close(out.cpu().double(), want, rtol=4e-3, atol=1e-3)
    elif mode == "f32":
        out = torch.empty(m, n, dtype=torch.float32, device=DEV)
        ops.gemv_bf16(x, w, out, ops.STORE_F32)
        torch.testing.assert_close(out.cpu().double(), want, rtol=1e-5, atol=1e-5 * math.sqrt(k))
    else:
        h = _randn(m, n, seed=3)
        out = h.clone()
        ops.gemv_bf16(x, w, out, ops.ADD_F32)
        torch.testing.assert_close(out.cpu().double(), h.cpu().double() + want, rtol=1e-5, atol=1e-5 * math.sqrt(k))
    # a row's result does not depend on the rows beside it
    if mode == "f32" and m > 1:
        one = torch.empty(1, n, dtype=torch.float32, device=DEV)
        ops.gemv_bf16(x[m - 1:m].contiguous(), w, one, ops.STORE_F32)
        assert torch.equal(one[0], out[m - 1])


@pytest.mark.parametrize("mode", ["bf16", "f32", "add"])
@pytest.mark.parametrize("m,n,k", [(8, 2048, 8192), (3, 200, 4104), (1, 77, 16384), (8, 4096, 14336), (5, 264, 2056),
                                   (7, 1000, 6152)])
def test_gemv_with_k_split_over_a_cluster(m, n, k, mode):
    """Long contractions: 2 to 8 slices of K in the blocks of a cluster, sums added in slice order;
    sizes with ragged last slices, last k-blocks and last row tiles."""
    from nanoinfer_b200.kernels import ops
    assert ops.gemv_ksplit_supports(m, n, k)
    x = _randn(m, k, dtype=torch.bfloat16, seed=1)
    w = _randn(n, k, dtype=torch.bfloat16, seed=2, scale=0.05)
    w[n // 2, k - 8:] = 4.0                      # the very last k-block of a row must be read
    want = x.cpu().double() @ w.cpu().double().t()
    if mode == "bf16":
        out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
        ops.gemv_ksplit(x, w, out, ops.STORE_BF16)
        torch.testing.assert_close(out.cpu().double(), want, rtol=4e-3, atol=1e-3 * math.sqrt(k / 2048))
    elif mode == "f32":
        out = torch.empty(m, n, dtype=torch.float32, device=DEV)
        ops.gemv_ksplit(x, w, out, ops.STORE_F32)
        torch.testing.assert_close(out.cpu().double(), want, rtol=1e-5, atol=1e-5 * math.sqrt(k))
        again = torch.empty_like(out)
        ops.gemv_ksplit(x, w, again, ops.STORE_F32)
        assert torch.equal(out, again)           # fixed order of addition
        if m > 1:                                # a row's result does not depend on the rows beside it
            one = torch.empty(1, n, dtype=torch.float32, device=DEV)
            ops.gemv_ksplit(x[m - 1:m].contiguous(), w, one, ops.STORE_F32)
            assert torch.equal(one[0], out[m - 1])
    else:
        h = _randn(m, n, seed=3)
        out = h.clone()
        ops.gemv_ksplit(x, w, out, ops.ADD_F32)
        torch.testing.assert_close(out.cpu().double(), h.cpu().double() + want, rtol=1e-5, atol=1e-5 * math.sqrt(k))
    ops.check_device_errors()


def test_gemv_k_split_refuses_what_it_cannot_take():
    from nanoinfer_b200.kernels import ops
    assert not ops.gemv_ksplit_supports(8, 2048, 2048)       # one slice: the other kernel's business
    assert not ops.gemv_ksplit_supports(9, 2048, 8192)       # more than 8 rows
    assert not ops.gemv_ksplit_supports(8, 2048, 8 * 2048 + 64)   # more than 8 slices
    assert not ops.gemv_ksplit_supports(4, 128256, 8192)     # too many row tiles per cluster for its shared memory
    with pytest.raises(ops.KernelError, match="not supported"):
        ops.gemv_ksplit(_randn(8, 2048, dtype=torch.bfloat16), _randn(64, 2048, dtype=torch.bfloat16),
                        torch.empty(8, 64, dtype=torch.float32, device=DEV), ops.STORE_F32)
    # the dispatcher of the engine's products falls back to the streaming kernel there
    x, w = _randn(4, 8192, dtype=torch.bfloat16, seed=1), _randn(40000, 8192, dtype=torch.bfloat16, seed=2, scale=0.05)
    if not ops.gemv_ksplit_supports(4, 40000, 8192):
        out = ops.linear_bf16(x, w, torch.float32)
        torch.testing.assert_close(out.cpu().double(), x.cpu().double() @ w.cpu().double().t(), rtol=1e-5, atol=1e-3)


@pytest.mark.parametrize("m,d,k_in", [(8, 2048, 8192), (3, 264, 2048), (1, 2048, 2048), (5, 520, 4104), (8, 3072, 3072)])
def test_a_norm_handed_from_the_adding_product_to_its_reader(m, d, k_in):
    """The product that adds into the residual stream (either skinny kernel) also stores
    bfloat16(h * gain) and partial sums of h^2; the reader scales its products by 1/rms.  Compared
    with the plain formulas, and with the reader that runs the norm inside itself."""
    from nanoinfer_b200.kernels import ops
    eps, inter = 1e-5, 400
    act = _randn(m, k_in, dtype=torch.bfloat16, seed=1)
    w_add = _randn(d, k_in, dtype=torch.bfloat16, seed=2, scale=0.03)
    h0 = _randn(m, d, seed=3, scale=1.5)
    gain = _randn(d, seed=4, scale=0.2) + 1.0

    class Norm:                                                   # what a norm part shows of itself
        fused_kind = "rmsnorm"
    norm = Norm()
    norm.gain, norm.eps = gain, eps
    tiles = ops.gemv_out_tiles(m, d, k_in)
    hand = ops.NormHandoff(norm, gain, eps, m, d, tiles, DEV)
    h = h0.clone()
    assert ops.linear_bf16(act, w_add, torch.float32, residual=h, handoff=hand) is None
    want_h = h0.cpu().double() + act.cpu().double() @ w_add.cpu().double().t()
    torch.testing.assert_close(h.cpu().double(), want_h, rtol=1e-5, atol=1e-5 * math.sqrt(k_in))
    # the prepared input is bfloat16(h * gain) of the very h that was stored, and the partial sums add up to sum(h^2)
    assert torch.equal(hand.x, (h * gain).to(torch.bfloat16))
    torch.testing.assert_close(hand.ssq[:m].sum(1).cpu(), (h.cpu() ** 2).sum(-1), rtol=1e-5, atol=0)
    # readers: gate/up with SwiGLU, and a plain store
    gate = _randn(inter, d, dtype=torch.bfloat16, seed=5, scale=0.05)
    up = _randn(inter, d, dtype=torch.bfloat16, seed=6, scale=0.05)
    w13 = torch.stack([gate.view(inter // 8, 8, d), up.view(inter // 8, 8, d)], dim=1).reshape(2 * inter, d).contiguous()
    got = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    ops.gemv_bf16(hand.x, w13, got, ops.SWIGLU_BF16, pre=hand)
    fused = torch.empty_like(got)
    ops.gemv_norm_bf16(h, gain, eps, None, w13, fused, ops.SWIGLU_BF16)
    x = plain.rms_norm(h.cpu(), gain.cpu(), eps)
    want = plain.swiglu_ffn(x, gate.cpu(), up.cpu(), torch.eye(inter))       # the activation alone (identity down projection)
    scale = want.abs().max().item()
    assert (got.cpu().float() - want).abs().max().item() <= 1e-2 * scale
    assert (got.float() - fused.float()).abs().max().item() <= 4e-3 * scale       # the same roundings, another order of sums
    # the fused QKV projection as a reader (rotation and cache write behind it), against itself with the norm inside
    n_q, n_kv, hd, page = 4, 2, 32, 8
    if True:
        w_qkv = _randn((n_q + 2 * n_kv) * hd, d, dtype=torch.bfloat16, seed=7, scale=0.05)
        positions = torch.arange(3, 3 + m, dtype=torch.int32, device=DEV)
        seq_of = torch.arange(m, dtype=torch.int32, device=DEV)
        table = torch.arange(m * 2, dtype=torch.int32, device=DEV).view(m, 2)
        inv_freq = plain.rope_inv_freq(hd, 10000.0, None).to(DEV)
        outs = []
        for pre in (hand, None):
            q_out = torch.zeros(m, n_q * hd, dtype=torch.bfloat16, device=DEV)
            kp = torch.zeros(m * 2, n_kv, page, hd, dtype=torch.bfloat16, device=DEV)
            vp = torch.zeros_like(kp)
            if pre is not None:
                ops.gemv_qkv_rope(hand.x, None, 0.0, w_qkv, q_out, kp, vp, positions, seq_of, table, inv_freq, n_q, n_kv, hd, hd, page, pre=hand)
            else:
                ops.gemv_qkv_rope(h, gain, eps, w_qkv, q_out, kp, vp, positions, seq_of, table, inv_freq, n_q, n_kv, hd, hd, page)
            outs.append((q_out, kp, vp))
        for a, b in zip(*outs):
            assert (a.float() - b.float()).abs().max().item() <= 1e-2 * b.float().abs().max().item()
    # a reader without 16-row tiles (a plain store of few columns) has no such variant: refused, not wrong
    with pytest.raises(ops.KernelError, match="not supported"):
        ops.gemv_bf16(hand.x, w13, torch.empty(m, 2 * inter, dtype=torch.float32, device=DEV), ops.STORE_F32, pre=hand)
    # what cannot be handed over is refused
    with pytest.raises(ops.KernelError, match="at most 8 rows"):
        ops.gemv_bf16(_randn(9, d, dtype=torch.bfloat16), w13, torch.empty(9, 2 * inter, dtype=torch.float32, device=DEV),
                      ops.STORE_F32, pre=hand)
    with pytest.raises(ops.KernelError, match="does not fit"):
        ops.gemv_bf16(act, w_add, torch.empty(m, d, dtype=torch.float32, device=DEV), ops.STORE_F32, handoff=hand)


def test_a_request_to_warm_l2_changes_no_result():
    """The skinny products and the decode attention may be handed a stretch of memory to ask into
    L2 on their way (weights that later kernels read).  Results are the same bit for bit, for
    stretches of any size and offset (cut to the tensor and to 16 bytes); nothing is written there."""
    from nanoinfer_b200.kernels import ops
    later = _randn(300, 1000, dtype=torch.bfloat16, seed=9)             # 600,000 bytes: no multiple of a piece
    keep = later.clone()
    x = _randn(5, 2048, dtype=torch.bfloat16, seed=1)
    w = _randn(264, 2048, dtype=torch.bfloat16, seed=2, scale=0.05)
    plain_out = torch.empty(5, 264, dtype=torch.float32, device=DEV)
    ops.gemv_bf16(x, w, plain_out, ops.STORE_F32)
    for hint in [(later, 0, 1 << 30), (later, 4096 + 8, 100_000), (later, 599_000, 5000), (later, 10**7, 64), None]:
        out = torch.empty_like(plain_out)
        ops.gemv_bf16(x, w, out, ops.STORE_F32, warm=hint)
        assert torch.equal(out, plain_out)
    assert ops.warm_region((later, 8, 100)) == (later.data_ptr(), 96)      # first byte and size cut to 16 bytes
    assert ops.warm_region((later, 600_000, 64)) == (None, 0) and ops.warm_region(None) == (None, 0)
    # the decode attention takes two stretches
    lens = [300, 40]
    spans = [(t - 1, t) for t in lens]
    table, k_pages, v_pages, ks, vs, qs, q, positions, seq_of = _attention_case(lens, spans, 8, 2, 64, 16, 77)
    outs = []
    for hints in [(), ((later, 0, 1 << 30), (w, 0, 1 << 20)), ((later, 16, 48), None)]:
        out = torch.zeros_like(q).to(DEV)
        scratch = torch.empty(2 * 8 * 3 * 66, dtype=torch.float32, device=DEV)
        tickets = torch.zeros(4, dtype=torch.int32, device=DEV)
        ops.attention_decode(q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), out, None, 2, positions.to(DEV), seq_of.to(DEV),
                             table.to(DEV), 8, 2, 64, 16, None, 0.125, 3, scratch, tickets, warm=hints)
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    torch.cuda.synchronize()
    assert torch.equal(later, keep)


def test_gemv_refuses_what_it_cannot_take():
    from nanoinfer_b200.kernels import ops
    x = _randn(17, 64, dtype=torch.bfloat16)
    w = _randn(8, 64, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError, match="at most 16 rows"):
        ops.gemv_bf16(x, w, torch.empty(17, 8, dtype=torch.bfloat16, device=DEV), ops.STORE_BF16)
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        ops.gemv_bf16(_randn(2, 60, dtype=torch.bfloat16), _randn(8, 60, dtype=torch.bfloat16),
                      torch.empty(2, 8, dtype=torch.bfloat16, device=DEV), ops.STORE_BF16)


def _attention_case(lens, spans, n_q, n_kv, hd, page, seed, far_key=None):
    """Paged k/v for sequences of the given lengths and queries for the spans [a, b) of each.
    ``far_key`` = (seq, key index): that key is made to dominate the last query's scores."""
    dtype = torch.bfloat16
    table, k_pages, v_pages, ks, vs = _paged_setup(lens, n_kv, hd, page, dtype, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    qs = [torch.randn(t, n_q, hd, generator=g).to(dtype) for t in lens]
    if far_key is not None:
        s_i, j = far_key
        # make one far key stand out for the last query of that sequence: all heads of a group
        # share one query vector and the key is three times that vector, so its score
        # (3 sqrt(hd) after scaling) dwarfs the rest; a kernel that skips or misplaces that key
        # cannot pass
        rep = n_q // n_kv
        base = torch.randn(n_kv, hd, generator=g).to(dtype)
        qs[s_i][-1] = base.repeat_interleave(rep, dim=0)
        ks[s_i][j] = (base.float() * 3.0).to(dtype)
        p, slot = table[s_i, j // page], j % page
        k_pages[p, :, slot] = ks[s_i][j]
        vs[s_i][j] = torch.full((n_kv, hd), 5.0, dtype=dtype)
        v_pages[p, :, slot] = vs[s_i][j]
    q = torch.cat([qs[s][a:b] for s, (a, b) in enumerate(spans)]).reshape(-1, n_q * hd)
    positions = torch.cat([torch.arange(a, b) for a, b in spans]).int()
    seq_of = torch.cat([torch.full((b - a,), s) for s, (a, b) in enumerate(spans)]).int()
    return table, k_pages, v_pages, ks, vs, qs, q, positions, seq_of


@pytest.mark.parametrize("n_splits", [1, 3, 7, 12])     # 12: a cluster beyond the portable size where the blocks are few
@pytest.mark.parametrize("n_q,n_kv,hd,page,window", [(32, 8, 64, 16, None), (8, 8, 64, 8, None), (24, 8, 128, 16, None),
                                                      (16, 1, 64, 4, 100), (6, 2, 128, 32, 33), (16, 2, 64, 16, None)])
@pytest.mark.parametrize("cluster", [True, False])
def test_attention_decode(n_q, n_kv, hd, page, window, n_splits, cluster):
    """``cluster``: the splits merge inside a thread-block cluster where the kernel can (2 to 8 splits
    whose partial results fit its shared memory), else through the scratch and the tickets; off: always the latter."""
    from nanoinfer_b200.kernels import ops
    ops.attention_decode_cluster_merge(cluster)
    lens = [700, 1, 33, 257]
    spans = [(t - 1, t) for t in lens]          # the last token of each sequence
    far = (0, 5) if window is None else None    # a far key among hundreds must be found
    table, k_pages, v_pages, ks, vs, qs, q, positions, seq_of = _attention_case(lens, spans, n_q, n_kv, hd, page, hd + n_q, far)
    scale = 1.0 / math.sqrt(hd)
    n = q.shape[0]
    out = torch.zeros_like(q).to(DEV)
    scratch = torch.empty(n * n_q * n_splits * (hd + 2), dtype=torch.float32, device=DEV)
    tickets = torch.zeros(n * n_kv, dtype=torch.int32, device=DEV)
    args = (positions.to(DEV), seq_of.to(DEV), table.to(DEV), n_q, n_kv, hd, page, window, scale, n_splits,
            scratch, tickets)
    ops.attention_decode(q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), out, None, n, *args)
    want = torch.cat([plain.attention(qs[s], ks[s], vs[s], scale, window)[a:b]
                      for s, (a, b) in enumerate(spans)]).reshape(-1, n_q * hd)
    # bfloat16 probabilities multiply V (2^-9 relative each) and the output is rounded once
    torch.testing.assert_close(out.cpu().float(), want, rtol=8e-3, atol=4e-3)
    assert torch.all(tickets == 0)              # left ready for the next launch
    if far is not None:
        assert out.cpu().float()[0].mean() > 4.0    # the far key's value dominates
    # a token list picks some tokens; the others are left alone
    out2 = torch.full_like(out, 9.0)
    pick = torch.tensor([2, 0], dtype=torch.int32, device=DEV)
    ops.attention_decode(q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), out2, pick, 2, *args)
    assert torch.equal(out2[0], out[0]) and torch.equal(out2[2], out[2])
    assert torch.all(out2[1] == 9.0) and torch.all(out2[3] == 9.0)
    ops.attention_decode_cluster_merge(True)


@pytest.mark.parametrize("n_q,n_kv,hd,page,window", [(32, 8, 64, 16, None), (8, 2, 64, 8, 130), (24, 8, 128, 16, None),
                                                      (16, 1, 64, 4, None), (6, 2, 128, 32, 77)])
def test_attention_decode_balanced(n_q, n_kv, hd, page, window):
    """The kernel that deals the keys of all tokens evenly over a fixed grid: contexts from one key
    to thousands, so that blocks hold whole tokens, tails, heads, and one token spans many blocks;
    a far key that must be found; a token list; twice the same result (fixed merge order)."""
    from nanoinfer_b200.kernels import ops
    lens = [3000, 1, 33, 257, 64, 65, 700, 2, 128, 1500, 17, 900]
    spans = [(t - 1, t) for t in lens]
    far = (0, 5) if window is None else None
    table, k_pages, v_pages, ks, vs, qs, q, positions, seq_of = _attention_case(lens, spans, n_q, n_kv, hd, page, hd + n_q, far)
    scale = 1.0 / math.sqrt(hd)
    n = q.shape[0]
    scratch = torch.full((ops.attention_decode_balanced_scratch(n_q, n_kv, hd),), float("nan"), dtype=torch.float32, device=DEV)
    tickets = torch.zeros(n * n_kv, dtype=torch.int32, device=DEV)
    args = (positions.to(DEV), seq_of.to(DEV), table.to(DEV), n_q, n_kv, hd, page, window, scale, scratch, tickets)
    out = torch.zeros_like(q).to(DEV)
    ops.attention_decode_balanced(q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), out, None, n, *args)
    want = torch.cat([plain.attention(qs[s], ks[s], vs[s], scale, window)[a:b]
                      for s, (a, b) in enumerate(spans)]).reshape(-1, n_q * hd)
    torch.testing.assert_close(out.cpu().float(), want, rtol=8e-3, atol=4e-3)
    assert torch.all(tickets == 0)
    if far is not None:
        assert out.cpu().float()[0].mean() > 4.0
    again = torch.zeros_like(out)
    ops.attention_decode_balanced(q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), again, None, n, *args)
    assert torch.equal(again, out)
    # a token list: those tokens only, in the list's order of work, the others left alone
    out2 = torch.full_like(out, 9.0)
    pick = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    ops.attention_decode_balanced(q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), out2, pick, 3, *args)
    for i in range(n):
        if i in (6, 0, 3):
            torch.testing.assert_close(out2[i].float(), out[i].float(), rtol=8e-3, atol=4e-3)   # cut elsewhere: rounding only
        else:
            assert torch.all(out2[i] == 9.0)
    ops.check_device_errors()


@pytest.mark.parametrize("n_q,n_kv,hd,page,window", [(4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 3, 48, 4, 70),
                                                      (32, 8, 64, 16, None), (5, 5, 80, 16, None), (4, 1, 96, 16, 64),
                                                      (2, 2, 112, 8, None), (8, 2, 128, 16, 129)])
def test_attention_prefill(n_q, n_kv, hd, page, window):
    from nanoinfer_b200.kernels import ops
    lens = [300, 70, 5, 130]
    spans = [(100, 300), (0, 70), (2, 5), (127, 130)]   # portions: late and longer than a tile, whole, tiny, at a page edge
    far = (0, 3) if window is None else None
    table, k_pages, v_pages, ks, vs, qs, q, positions, seq_of = _attention_case(lens, spans, n_q, n_kv, hd, page, hd, far)
    scale = 1.0 / math.sqrt(hd)
    q_lens = [b - a for a, b in spans]
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    kv_len = torch.tensor([b for _, b in spans], dtype=torch.int32)
    tiles = [(s, r0) for s, ql in enumerate(q_lens) for r0 in range(0, ql, ops.PREFILL_TILE_ROWS)]
    tile_seq = torch.tensor([t[0] for t in tiles], dtype=torch.int32)
    tile_row0 = torch.tensor([t[1] for t in tiles], dtype=torch.int32)
    out = torch.zeros_like(q).to(DEV)
    ops.attention_prefill(q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), out, tile_seq.to(DEV), tile_row0.to(DEV),
                          len(tiles), cu_q.to(DEV), kv_len.to(DEV), table.to(DEV), n_q, n_kv, hd, page, window, scale)
    want = torch.cat([plain.attention(qs[s], ks[s], vs[s], scale, window)[a:b]
                      for s, (a, b) in enumerate(spans)]).reshape(-1, n_q * hd)
    torch.testing.assert_close(out.cpu().float(), want, rtol=8e-3, atol=4e-3)
    if far is not None:
        assert out.cpu().float()[199].mean() > 4.0      # last row of sequence 0 found key 3


@pytest.mark.parametrize("far_at", [3, 640])
@pytest.mark.parametrize("n_q,n_kv,hd,page,window", [(32, 8, 64, 16, None), (4, 2, 64, 8, None), (8, 2, 128, 16, 129),
                                                      (2, 1, 128, 32, None), (16, 2, 64, 64, 300), (4, 1, 64, 128, None),
                                                      (6, 1, 128, 8, None), (6, 2, 128, 16, None), (5, 1, 64, 16, 200),
                                                      (9, 3, 64, 32, None)])
def test_attention_prefill_tensor_core(n_q, n_kv, hd, page, window, far_at):
    """The tcgen05 kernel: several key tiles per query tile, a portion that starts late, tiny and
    page-edge portions, and a dominant key either in the first tile or in a late one (there the
    running maximum jumps and the accumulator in tensor memory is rescaled)."""
    from nanoinfer_b200.kernels import ops
    assert ops.attention_prefill_tc_supports(n_q, n_kv, hd, page)
    lens = [700, 70, 5, 130, 513]
    spans = [(100, 700), (0, 70), (2, 5), (127, 130), (0, 513)]
    far = (0, far_at) if window is None else None
    table, k_pages, v_pages, ks, vs, qs, q, positions, seq_of = _attention_case(lens, spans, n_q, n_kv, hd, page, hd + page, far)
    scale = 1.0 / math.sqrt(hd)
    q_lens = [b - a for a, b in spans]
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    kv_len = torch.tensor([b for _, b in spans], dtype=torch.int32)
    tiles = [(s, r0) for s, ql in enumerate(q_lens) for r0 in range(0, ql, ops.PREFILL_TILE_ROWS)]
    tile_seq = torch.tensor([t[0] for t in tiles], dtype=torch.int32)
    tile_row0 = torch.tensor([t[1] for t in tiles], dtype=torch.int32)
    out = torch.full_like(q, 7.0).to(DEV)
    ops.attention_prefill(q.to(DEV), k_pages.to(DEV), v_pages.to(DEV), out, tile_seq.to(DEV), tile_row0.to(DEV),
                          len(tiles), cu_q.to(DEV), kv_len.to(DEV), table.to(DEV), n_q, n_kv, hd, page, window, scale,
                          kernel="tc")
    ops.check_device_errors()
    want = torch.cat([plain.attention(qs[s], ks[s], vs[s], scale, window)[a:b]
                      for s, (a, b) in enumerate(spans)]).reshape(-1, n_q * hd)
    torch.testing.assert_close(out.cpu().float(), want, rtol=8e-3, atol=4e-3)
    if far is not None:
        assert out.cpu().float()[599].mean() > 4.0      # last row of sequence 0 found the far key


def test_attention_prefill_tensor_core_declines_what_it_cannot_take():
    from nanoinfer_b200.kernels import ops
    assert not ops.attention_prefill_tc_supports(5, 5, 64, 16)      # one query head per kv head
    assert not ops.attention_prefill_tc_supports(8, 2, 96, 16)      # head size
    assert not ops.attention_prefill_tc_supports(8, 2, 64, 4)       # page size
    assert not ops.attention_prefill_tc_supports(8, 2, 64, 48)
    q = torch.zeros(4, 5 * 64, dtype=torch.bfloat16, device=DEV)
    kp = torch.zeros(2, 5, 16, 64, dtype=torch.bfloat16, device=DEV)
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(ops.KernelError):
        ops.attention_prefill(q, kp, kp, q.clone(), z, z, 1, z, z, z.view(1, 2), 5, 5, 64, 16, None, 0.125, kernel="tc")


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (4, 336, 120), (8, 4800, 2048), (13, 200, 264), (16, 1000, 8200),
                                   (8, 5120, 3072), (5, 1000, 4096), (3, 264, 2600), (6, 200, 4104)])
def test_gemv_with_fused_norm(m, n, k):
    """RMSNorm (on picked rows of the FP32 residual stream) inside the skinny product."""
    from nanoinfer_b200.kernels import ops
    h = _randn(m + 5, k, seed=1, scale=2.0)
    gain = _randn(k, seed=2, scale=0.2) + 1.0
    w = _randn(n, k, dtype=torch.bfloat16, seed=3, scale=0.05)
    rows = torch.randperm(m + 5, generator=torch.Generator().manual_seed(4))[:m].int().to(DEV)
    eps = 1e-5
    x = plain.rms_norm(h.cpu()[rows.cpu().long()], gain.cpu(), eps)
    want = x.double() @ w.cpu().double().t()
    out = torch.empty(m, n, dtype=torch.float32, device=DEV)
    ops.gemv_norm_bf16(h, gain, eps, rows, w, out, ops.STORE_F32)
    # the kernel rounds h * gain to bfloat16 before the product (2^-9 relative per element,
    # averaging out over K), the statistics are exact FP32
    scale = want.abs().max().item()
    assert (out.cpu().double() - want).abs().max().item() <= 4e-3 * scale
    # without a row list: rows 0..m-1
    out2 = torch.empty(m, n, dtype=torch.float32, device=DEV)
    ops.gemv_norm_bf16(h[:m].contiguous(), gain, eps, None, w, out2, ops.STORE_F32)
    want2 = plain.rms_norm(h.cpu()[:m], gain.cpu(), eps).double() @ w.cpu().double().t()
    assert (out2.cpu().double() - want2).abs().max().item() <= 4e-3 * want2.abs().max().item()


@pytest.mark.parametrize("m,inter,k", [(1, 64, 64), (7, 200, 120), (8, 8192, 2048), (16, 264, 160), (8, 4096, 3072),
                                       (4, 2048, 4096)])
def test_gemv_with_swiglu_epilogue(m, inter, k):
    from nanoinfer_b200.kernels import ops
    x = _randn(m, k, dtype=torch.bfloat16, seed=1)
    gate = _randn(inter, k, dtype=torch.bfloat16, seed=2, scale=0.08)
    up = _randn(inter, k, dtype=torch.bfloat16, seed=3, scale=0.08)
    w13 = torch.stack([gate.view(inter // 8, 8, k), up.view(inter // 8, 8, k)], dim=1).reshape(2 * inter, k).contiguous()
    out = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    ops.gemv_bf16(x, w13, out, ops.SWIGLU_BF16)
    g = x.cpu().double() @ gate.cpu().double().t()
    u = x.cpu().double() @ up.cpu().double().t()
    want = (g / (1 + torch.exp(-g))) * u
    torch.testing.assert_close(out.cpu().double(), want, rtol=4e-3, atol=1e-3)
    # the activation kernel on the same blocked layout (the path of longer portions)
    gu = (x.cpu().float() @ w13.cpu().float().t()).to(torch.bfloat16).to(DEV)
    out2 = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    ops.swiglu(gu, out2, blocked=True)
    gf = gu.cpu().float().view(m, inter // 8, 2, 8)
    want2 = ((gf[:, :, 0] / (1 + torch.exp(-gf[:, :, 0]))) * gf[:, :, 1]).reshape(m, inter)
    torch.testing.assert_close(out2.cpu().float(), want2, rtol=4e-3, atol=1e-3)


@pytest.mark.parametrize("with_norm", [False, True])
@pytest.mark.parametrize("n_q,n_kv,hd,rot,page,d", [(4, 2, 16, 16, 16, 64), (3, 1, 32, 32, 8, 96), (6, 3, 48, 32, 4, 120),
                                                     (32, 8, 64, 64, 16, 2048), (24, 8, 128, 128, 16, 3072), (8, 2, 128, 128, 16, 4096)])
def test_gemv_qkv_rope(n_q, n_kv, hd, rot, page, d, with_norm):
    """Projection + (norm) + adjacent-pair rotation + paged write in one launch, against the
    plain steps."""
    from nanoinfer_b200.kernels import ops
    m = 9
    g = torch.Generator().manual_seed(hd)
    n = (n_q + 2 * n_kv) * hd
    w = (torch.randn(n, d, generator=g) * 0.06).to(torch.bfloat16)
    h = torch.randn(m, d, generator=g) * 1.5
    gain = torch.randn(d, generator=g) * 0.1 + 1.0
    positions = torch.tensor([0, 1, 15, 16, 17, 40, 63, 64, 100][:m], dtype=torch.int32)
    seq_of = torch.arange(m, dtype=torch.int32)
    width = 128 // page
    perm = torch.randperm(m * width + 3, generator=g)
    table = perm[:m * width].view(m, width).int()
    n_pages = m * width + 3
    inv_freq = plain.rope_inv_freq(rot, 10000.0, None)
    q_out = torch.empty(m, n_q * hd, dtype=torch.bfloat16, device=DEV)
    k_pages = torch.full((n_pages, n_kv, page, hd), 7.0, dtype=torch.bfloat16, device=DEV)
    v_pages = torch.full((n_pages, n_kv, page, hd), 7.0, dtype=torch.bfloat16, device=DEV)
    if with_norm:
        x_in, x_ref = h.to(DEV), plain.rms_norm(h, gain, 1e-5)
        gain_dev = gain.to(DEV)
    else:
        x_in, gain_dev = h.to(torch.bfloat16).to(DEV), None
        x_ref = h.to(torch.bfloat16).float()
    ops.gemv_qkv_rope(x_in, gain_dev, 1e-5, w.to(DEV), q_out, k_pages, v_pages, positions.to(DEV), seq_of.to(DEV),
                      table.to(DEV), inv_freq.to(DEV), n_q, n_kv, hd, rot, page)
    qkv = x_ref @ w.float().t()
    q = plain.rope(qkv[:, :n_q * hd].view(m, n_q, hd), positions, inv_freq, "interleaved")
    k = plain.rope(qkv[:, n_q * hd:(n_q + n_kv) * hd].view(m, n_kv, hd), positions, inv_freq, "interleaved")
    v = qkv[:, (n_q + n_kv) * hd:].view(m, n_kv, hd)
    scale = qkv.abs().max().item()
    tol = 6e-3 * scale
    assert (q_out.cpu().float().view(m, n_q, hd) - q).abs().max().item() <= tol
    kp, vp = k_pages.cpu().float(), v_pages.cpu().float()
    touched = torch.zeros(n_pages, page, dtype=torch.bool)
    for t in range(m):
        p, slot = table[t, positions[t] // page], positions[t] % page
        assert (kp[p, :, slot] - k[t]).abs().max().item() <= tol
        assert (vp[p, :, slot] - v[t]).abs().max().item() <= tol
        touched[p, slot] = True
    assert torch.all(kp.permute(0, 2, 1, 3)[~touched] == 7.0) and torch.all(vp.permute(0, 2, 1, 3)[~touched] == 7.0)


@pytest.mark.parametrize("kernel", ["single", "pair"])
@pytest.mark.parametrize("mode", ["bf16", "f32", "add", "swiglu"])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (2048, 512, 2048), (200, 336, 200), (17, 4800, 2048), (300, 128, 8200),
                                   (1, 48, 64), (130, 1000, 120), (2048, 8192, 512), (2048, 4608, 128)])
def test_gemm_tc(m, n, k, mode, kernel):
    """The tcgen05/TMEM product against a float64 product: full tiles, ragged edges in M, N and
    K, every epilogue; one SM per tile and two SMs per tile (cta_group::2)."""
    from nanoinfer_b200.kernels import ops
    if mode == "swiglu" and n % 16:
        n = n - n % 16
    a = _randn(m, k, dtype=torch.bfloat16, seed=1)
    b = _randn(n, k, dtype=torch.bfloat16, seed=2, scale=0.05)
    want = a.cpu().double() @ b.cpu().double().t()
    tol = 1e-5 * math.sqrt(k)
    if mode == "bf16":
        out = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=DEV)
        ops.gemm_tc(a, b, out, ops.STORE_BF16, kernel=kernel)
        torch.testing.assert_close(out.cpu().double(), want, rtol=4e-3, atol=1e-3)
    elif mode == "f32":
        out = torch.full((m, n), 7.0, dtype=torch.float32, device=DEV)
        ops.gemm_tc(a, b, out, ops.STORE_F32, kernel=kernel)
        torch.testing.assert_close(out.cpu().double(), want, rtol=1e-5, atol=tol)
    elif mode == "add":
        h = _randn(m, n, seed=3)
        out = h.clone()
        ops.gemm_tc(a, b, out, ops.ADD_F32, kernel=kernel)
        torch.testing.assert_close(out.cpu().double(), h.cpu().double() + want, rtol=1e-5, atol=tol)
    else:
        out = torch.full((m, n // 2), 7.0, dtype=torch.bfloat16, device=DEV)
        ops.gemm_tc(a, b, out, ops.SWIGLU_BF16, kernel=kernel)
        w4 = want.view(m, n // 16, 2, 8)
        ref = ((w4[:, :, 0] / (1 + torch.exp(-w4[:, :, 0]))) * w4[:, :, 1]).reshape(m, n // 2)
        torch.testing.assert_close(out.cpu().double(), ref, rtol=4e-3, atol=1e-3)
    ops.check_device_errors()


def _swap_scratch(ops, m, n, k):
    need = ops.gemm_swap_scratch(m, n, k)
    scratch = torch.full((max(need, 1),), float("nan"), dtype=torch.float32, device=DEV)
    tickets = torch.zeros(-(-n // 128), dtype=torch.int32, device=DEV)
    return scratch, tickets


@pytest.mark.parametrize("mode", ["bf16", "f32", "add", "swiglu"])
@pytest.mark.parametrize("m,n,k", [(9, 256, 64), (64, 16384, 2048), (33, 2048, 2048), (100, 1008, 200), (128, 2048, 8192),
                                   (17, 4800, 2056), (1, 48, 64), (32, 128, 640)])
def test_gemm_swap_tc(m, n, k, mode):
    """The swapped-operand tcgen05 product (weights on the tile's lanes, the batch on its columns)
    against a float64 product: every batch-tile width, ragged N and K, K cut into slices that a
    ticket combines, every epilogue; the second launch finds the tickets at zero again."""
    from nanoinfer_b200.kernels import ops
    x = _randn(m, k, dtype=torch.bfloat16, seed=1)
    w = _randn(n, k, dtype=torch.bfloat16, seed=2, scale=0.05)
    want = x.cpu().double() @ w.cpu().double().t()
    tol = 1e-5 * math.sqrt(k)
    scratch, tickets = _swap_scratch(ops, m, n, k)
    for _ in range(2):
        if mode == "bf16":
            out = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=DEV)
            ops.gemm_swap_tc(x, w, out, ops.STORE_BF16, scratch, tickets)
            torch.testing.assert_close(out.cpu().double(), want, rtol=4e-3, atol=1e-3)
        elif mode == "f32":
            out = torch.full((m, n), 7.0, dtype=torch.float32, device=DEV)
            ops.gemm_swap_tc(x, w, out, ops.STORE_F32, scratch, tickets)
            torch.testing.assert_close(out.cpu().double(), want, rtol=1e-5, atol=tol)
        elif mode == "add":
            h = _randn(m, n, seed=3)
            out = h.clone()
            ops.gemm_swap_tc(x, w, out, ops.ADD_F32, scratch, tickets)
            torch.testing.assert_close(out.cpu().double(), h.cpu().double() + want, rtol=1e-5, atol=tol)
        else:
            out = torch.full((m, n // 2), 7.0, dtype=torch.bfloat16, device=DEV)
            ops.gemm_swap_tc(x, w, out, ops.SWIGLU_BF16, scratch, tickets)
            w4 = want.view(m, n // 16, 2, 8)
            ref = ((w4[:, :, 0] / (1 + torch.exp(-w4[:, :, 0]))) * w4[:, :, 1]).reshape(m, n // 2)
            torch.testing.assert_close(out.cpu().double(), ref, rtol=4e-3, atol=1e-3)
        ops.check_device_errors()
        assert torch.all(tickets == 0)


@pytest.mark.parametrize("n_q,n_kv,hd,rot,page,d,m", [(4, 2, 32, 32, 16, 128, 9), (32, 8, 64, 64, 16, 2048, 64),
                                                      (6, 3, 48, 32, 8, 200, 33), (8, 1, 128, 128, 32, 512, 128)])
def test_gemm_swap_tc_qkv_rope(n_q, n_kv, hd, rot, page, d, m):
    """Fused QKV projection + adjacent-pair rotation + paged K/V write for 9..128 rows."""
    from nanoinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(hd + m)
    n = (n_q + 2 * n_kv) * hd
    w = (torch.randn(n, d, generator=g) * 0.06).to(torch.bfloat16)
    x = torch.randn(m, d, generator=g).to(torch.bfloat16)
    positions = torch.randint(0, 128, (m,), generator=g).int()
    seq_of = torch.arange(m, dtype=torch.int32)
    width = 128 // page
    n_pages = m * width + 3
    table = torch.randperm(n_pages, generator=g)[:m * width].view(m, width).int()
    inv_freq = plain.rope_inv_freq(rot, 10000.0, None)
    q_out = torch.empty(m, n_q * hd, dtype=torch.bfloat16, device=DEV)
    k_pages = torch.full((n_pages, n_kv, page, hd), 7.0, dtype=torch.bfloat16, device=DEV)
    v_pages = torch.full((n_pages, n_kv, page, hd), 7.0, dtype=torch.bfloat16, device=DEV)
    scratch, tickets = _swap_scratch(ops, m, n, d)
    ops.gemm_swap_tc(x.to(DEV), w.to(DEV), q_out, ops.ROPE_KV, scratch, tickets,
                     rope=(positions.to(DEV), seq_of.to(DEV), table.to(DEV), inv_freq.to(DEV), k_pages, v_pages,
                           n_q, n_kv, hd, rot, page))
    ops.check_device_errors()
    qkv = x.float() @ w.float().t()
    q = plain.rope(qkv[:, :n_q * hd].view(m, n_q, hd), positions, inv_freq, "interleaved")
    k = plain.rope(qkv[:, n_q * hd:(n_q + n_kv) * hd].view(m, n_kv, hd), positions, inv_freq, "interleaved")
    v = qkv[:, (n_q + n_kv) * hd:].view(m, n_kv, hd)
    tol = 6e-3 * qkv.abs().max().item()
    assert (q_out.cpu().float().view(m, n_q, hd) - q).abs().max().item() <= tol
    kp, vp = k_pages.cpu().float(), v_pages.cpu().float()
    touched = torch.zeros(n_pages, page, dtype=torch.bool)
    for t in range(m):
        p, slot = table[t, positions[t] // page], positions[t] % page
        assert (kp[p, :, slot] - k[t]).abs().max().item() <= tol
        assert (vp[p, :, slot] - v[t]).abs().max().item() <= tol
        touched[p, slot] = True
    assert torch.all(kp.permute(0, 2, 1, 3)[~touched] == 7.0) and torch.all(vp.permute(0, 2, 1, 3)[~touched] == 7.0)
    assert torch.all(tickets == 0)


@pytest.mark.parametrize("hd", [64, 128])
def test_attention_kernels_at_a_long_context(hd):
    """A late portion of a 4,500-token sequence: the prefill kernels walk 36 key tiles per query tile
    (their stage rings and barrier phases wrap many times), the decode kernel splits 4,500 keys; one
    key among the first hundred is made to dominate the last query."""
    from nanoinfer_b200.kernels import ops
    n_q, n_kv, page = 4, 2, 16
    lens, spans = [4500], [(4000, 4500)]
    table, k_pages, v_pages, ks, vs, qs, q, positions, seq_of = _attention_case(lens, spans, n_q, n_kv, hd, page, 3 * hd, (0, 70))
    scale = 1.0 / math.sqrt(hd)
    want = plain.attention(qs[0], ks[0], vs[0], scale, None)[4000:4500].reshape(-1, n_q * hd)
    dev = [t.to(DEV) for t in (q, k_pages, v_pages, table)]
    cu_q = torch.tensor([0, 500], dtype=torch.int32, device=DEV)
    kv_len = torch.tensor([4500], dtype=torch.int32, device=DEV)
    rows = list(range(0, 500, ops.PREFILL_TILE_ROWS))
    tile_seq = torch.zeros(len(rows), dtype=torch.int32, device=DEV)
    tile_row0 = torch.tensor(rows, dtype=torch.int32, device=DEV)
    for kernel in ("tc", "mma"):
        out = torch.full_like(dev[0], 7.0)
        ops.attention_prefill(dev[0], dev[1], dev[2], out, tile_seq, tile_row0, len(rows), cu_q, kv_len, dev[3],
                              n_q, n_kv, hd, page, None, scale, kernel=kernel)
        ops.check_device_errors()
        torch.testing.assert_close(out.cpu().float(), want, rtol=8e-3, atol=4e-3)
        assert out.cpu().float()[499].mean() > 4.0
    # the last token alone, through the decode kernel
    n_splits = 12
    q1 = dev[0][499:500].contiguous()
    out1 = torch.zeros_like(q1)
    scratch = torch.empty(n_q * n_splits * (hd + 2), dtype=torch.float32, device=DEV)
    tickets = torch.zeros(n_kv, dtype=torch.int32, device=DEV)
    ops.attention_decode(q1, dev[1], dev[2], out1, None, 1, torch.tensor([4499], dtype=torch.int32, device=DEV),
                         torch.zeros(1, dtype=torch.int32, device=DEV), dev[3], n_q, n_kv, hd, page, None, scale, n_splits,
                         scratch, tickets)
    torch.testing.assert_close(out1.cpu().float(), want[499:500], rtol=8e-3, atol=4e-3)
