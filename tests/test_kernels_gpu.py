"""Each CUDA kernel alone against its plain torch statement (tests/kernel_refs.py),
in float32 and bfloat16, at sizes other than the engine's: widths that are no
power of two, odd vocabularies, head sizes 16..256, several page sizes, groups
of 1, 3 and 8 query heads per kv head."""
import math

import pytest
import torch

import kernel_refs as ref
from arle_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-3)


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,H,T", [(300, 72, 5), (1000, 4096, 33), (17, 8, 1)])
def test_embedding(dtype, V, H, T):
    table = rnd(V, H, dtype=dtype)
    ids = torch.randint(0, V, (T,), dtype=torch.int32, device=DEV)
    out = torch.empty(T, H, device=DEV)
    exp = torch.empty(T, H, device=DEV)
    ops.embedding(ids, table, out)
    ref.embedding(ids, table, exp)
    assert torch.equal(out, exp)


def test_embedding_bad_id_sets_flag_and_writes_zeros():
    table = rnd(10, 16)
    ids = torch.tensor([3, 11, -1], dtype=torch.int32, device=DEV)
    out = torch.full((3, 16), 7.0, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embedding(ids, table, out, err)
    assert err.item() == 1 and torch.equal(out[0], table[3]) and out[1:].abs().sum().item() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,H", [(1, 64), (7, 260), (19, 4096), (3, 12288), (5, 100)])
@pytest.mark.parametrize("with_delta", [False, True])
def test_rmsnorm(dtype, N, H, with_delta):
    resid = rnd(N, H, scale=3.0, seed=1)
    delta = rnd(N, H, dtype=dtype, seed=2) if with_delta else None
    w = 1.0 + 0.2 * rnd(H, seed=3)
    r1, r2 = resid.clone(), resid.clone()
    out = torch.empty(N, H, dtype=dtype, device=DEV)
    exp = torch.empty(N, H, dtype=dtype, device=DEV)
    ops.rmsnorm(r1, delta, None, w, 1e-5, out, with_delta)
    ref.rmsnorm(r2, delta, None, w, 1e-5, exp, with_delta)
    torch.testing.assert_close(out.float(), exp.float(), **tol(dtype))
    torch.testing.assert_close(r1, r2, rtol=0, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_rows_leave_residual(dtype):
    N, H = 11, 200
    resid, delta = rnd(N, H, seed=4), rnd(N, H, dtype=dtype, seed=5)
    w = 1.0 + 0.1 * rnd(H, seed=6)
    rows = torch.tensor([10, 0, 3], dtype=torch.int32, device=DEV)
    before = resid.clone()
    out = torch.empty(3, H, dtype=dtype, device=DEV)
    exp = torch.empty(3, H, dtype=dtype, device=DEV)
    ops.rmsnorm(resid, delta, rows, w, 1e-6, out, False)
    ref.rmsnorm(before.clone(), delta, rows, w, 1e-6, exp, False)
    torch.testing.assert_close(out.float(), exp.float(), **tol(dtype))
    assert torch.equal(resid, before)


@pytest.mark.parametrize("dtype", DTYPES)
def test_residual_add(dtype):
    resid, delta = rnd(9, 130, seed=1), rnd(9, 130, dtype=dtype, seed=2)
    exp = resid + delta.float()
    ops.residual_add(resid, delta)
    assert torch.equal(resid, exp)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(1, 100), (6, 176), (33, 12288)])
def test_silu_mul(dtype, T, I):
    gu = rnd(T, 2 * I, dtype=dtype, scale=2.0)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    exp = torch.empty(T, I, dtype=dtype, device=DEV)
    ops.silu_mul(gu, out)
    ref.silu_mul(gu, exp)
    torch.testing.assert_close(out.float(), exp.float(), **tol(dtype))


@pytest.mark.parametrize("wdtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 301, 72), (70, 130, 100), (129, 65, 17), (3, 500, 96)])
def test_gemm_f32_true_32bit(wdtype, M, N, K):
    x = rnd(M, K, seed=1)
    w = rnd(N, K, dtype=wdtype, seed=2)
    out = torch.empty(M, N, device=DEV)
    ops.gemm(x, w, out)
    exp = (x.double() @ w.double().t())
    # float32 products and sums: error of a K-term dot product, far below TF32's 1e-3
    assert (out.double() - exp).abs().max().item() < 2e-6 * math.sqrt(K) * 4


def test_gemm_f32_rows_do_not_depend_on_batch():
    x, w = rnd(77, 200, seed=3), rnd(150, 200, seed=4)
    full = torch.empty(77, 150, device=DEV)
    ops.gemm(x, w, full)
    for rows in ([0], [5, 6, 7], list(range(64, 77))):
        part = torch.empty(len(rows), 150, device=DEV)
        ops.gemm(x[rows].contiguous(), w, part)
        assert torch.equal(part, full[rows])


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (8, 4096, 1024), (130, 304, 72)])
def test_gemm_bf16(M, N, K):
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, seed=2)
    exp = x.float() @ w.float().t()
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm(x, w, out)
    torch.testing.assert_close(out.float(), exp, rtol=2e-2, atol=2e-2 * math.sqrt(K) / 8)
    out32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.gemm(x, w, out32)
    torch.testing.assert_close(out32, exp, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 16, 32), (1, 4096, 4096), (8, 6144, 4096), (3, 1000, 192), (5, 37, 320),
                                   (8, 301, 256), (7, 500, 12288), (8, 200, 12288), (8, 4100, 12288), (2, 151936, 128),
                                   # K split over a cluster and more than sixteen tiles per cluster: several reductions
                                   (4, 20000, 8192), (8, 12000, 16384)])
def test_gemm_skinny_weight_streaming(M, N, K, out_dtype):
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=2)
    assert ops.skinny_gemm_supported(x, w, torch.empty(M, N, dtype=out_dtype, device=DEV))
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.gemm(x, w, out)
    exp = x.double() @ w.double().t()
    err = (out.double() - exp).abs().max().item()
    scale = exp.abs().max().item()
    assert err <= (2e-5 if out_dtype == torch.float32 else 6e-3) * max(scale, 1.0), (err, scale)
    again = torch.empty_like(out)
    ops.gemm(x, w, again)
    assert torch.equal(out, again)              # fixed summation order: bit-identical from run to run
    ops.check_errors(DEV)                       # no bounded wait ran out


@pytest.mark.parametrize("M,N,K", [(1, 64, 32), (8, 4096, 4096), (8, 4096, 12288), (3, 992, 192), (5, 160, 320), (8, 1024, 3072),
                                   (7, 5120, 25600), (2, 20000, 8192)])
def test_gemm_with_residual_sink_and_row_scale(M, N, K):
    """The two fusions that take the norm kernels out of a decode step.  A product with a sink adds its
    sums into the float32 residual and leaves bfloat16(residual * gain) and the rows' sums of squares;
    a product over those rows multiplies its sums by rsqrt(mean square + eps): together they equal
    residual sum, RMSNorm and product done one after the other."""
    eps = 1e-5
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=2)
    resid0 = rnd(M, N, dtype=torch.float32, seed=3)
    gain = (1.0 + 0.2 * rnd(N, dtype=torch.float32, seed=4)).contiguous()
    resid = resid0.clone()
    xs = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ss = torch.full(ops.SS_TABLE_SHAPE, float("nan"), dtype=torch.float32, device=DEV)
    sink = ops.ResidualSink(resid, gain, eps, xs, ss)
    assert ops.fused_gemm_shape_ok(M, w) and ops.gemm(x, w, None, sink=sink) is True and sink.filled
    ops.check_errors(DEV)
    want_r = resid0.double() + x.double() @ w.double().t()
    scale = want_r.abs().max().item()
    assert (resid.double() - want_r).abs().max().item() <= 2e-5 * max(scale, 1.0)
    assert (xs.double() - want_r * gain.double()).abs().max().item() <= 6e-3 * max(scale, 1.0)
    assert not ss.isnan().any() and (ss[M:] == 0).all()
    want_ss = (want_r * want_r).sum(dim=1)
    assert ((ss.double().sum(dim=1)[:M] - want_ss).abs() / want_ss).max().item() < 1e-5
    again_r, again_ss = resid0.clone(), torch.empty_like(ss)
    ops.gemm(x, w, None, sink=ops.ResidualSink(again_r, gain, eps, torch.empty_like(xs), again_ss))
    assert torch.equal(again_r, resid) and torch.equal(again_ss, ss)          # no atomics: the same bits every time
    # the reader: a product over the unscaled rows equals the product over the normalised rows
    w2 = rnd(300, N, dtype=torch.bfloat16, scale=0.05, seed=5)
    rows = ops.ScaledRows(xs, ss, eps)
    normed = want_r * torch.rsqrt((want_r * want_r).mean(dim=1, keepdim=True) + eps) * gain.double()
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.full((M, 300), float("nan"), dtype=out_dtype, device=DEV)
        assert ops.gemm(rows, w2, out) is False
        exp = normed @ w2.double().t()
        assert (out.double() - exp).abs().max().item() <= 1.2e-2 * max(exp.abs().max().item(), 1.0)
    if ops.gated_gemm_fits(N):
        w3 = rnd(2 * 150, N, dtype=torch.bfloat16, scale=0.08, seed=6)
        act = torch.full((M, 150), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.gemm_silu_mul(rows, w3, torch.empty(M, 300, dtype=torch.bfloat16, device=DEV), act)
        g, u = normed @ w3[0::2].double().t(), normed @ w3[1::2].double().t()
        exp = g / (1 + torch.exp(-g)) * u
        assert (act.double() - exp).abs().max().item() <= 2e-2 * max(exp.abs().max().item(), 1.0)
    ops.check_errors(DEV)


def test_a_sink_is_left_alone_when_the_shapes_do_not_allow_the_fused_kernel():
    x, w = rnd(9, 64, dtype=torch.bfloat16, seed=1), rnd(32, 64, dtype=torch.bfloat16, seed=2)      # nine rows
    resid = rnd(9, 32, dtype=torch.float32, seed=3)
    keep = resid.clone()
    sink = ops.ResidualSink(resid, torch.ones(32, device=DEV), 1e-6, torch.empty(9, 32, dtype=torch.bfloat16, device=DEV),
                            torch.empty(ops.SS_TABLE_SHAPE, device=DEV))
    out = torch.empty(9, 32, dtype=torch.bfloat16, device=DEV)
    assert ops.gemm(x, w, out, sink=sink) is False and not sink.filled and torch.equal(resid, keep)
    assert (out.double() - x.double() @ w.double().t()).abs().max().item() < 0.1
    with pytest.raises(ops.KernelError):
        ops.gemm(ops.ScaledRows(x, torch.zeros(ops.SS_TABLE_SHAPE, device=DEV), 1e-6), w, out)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,I,K", [(1, 8, 32), (8, 12288, 4096), (3, 500, 192), (5, 37, 320), (8, 2050, 4096), (7, 100, 4608),
                                   (9, 64, 64), (40, 176, 96), (2, 64, 8192), (8, 300, 5120), (4, 128, 5376)])
def test_gemm_silu_mul(M, I, K, out_dtype):
    """Gate and up rows interleaved in one weight; few rows of x take the fused launch, more rows
    (or a K too long for one CTA) the product and the gate kernel: same numbers either way."""
    x = rnd(M, K, dtype=torch.bfloat16, seed=1)
    w = rnd(2 * I, K, dtype=torch.bfloat16, scale=0.08, seed=2)
    gu = torch.full((M, 2 * I), float("nan"), dtype=torch.bfloat16, device=DEV)
    out = torch.full((M, I), float("nan"), dtype=out_dtype, device=DEV)
    fused = M <= 8 and ops.gated_gemm_fits(K)
    before = ops.launch_count()
    if out_dtype == torch.float32 and not fused:
        pytest.skip("the two-kernel path writes the activation type")
    ops.gemm_silu_mul(x, w, gu, out)
    assert ops.launch_count() - before == (1 if fused else (2 if M <= 8 else 1))
    ops.check_errors(DEV)
    g = x.double() @ w[0::2].double().t()
    u = x.double() @ w[1::2].double().t()
    exp = g / (1 + torch.exp(-g)) * u
    err = (out.double() - exp).abs().max().item()
    scale = exp.abs().max().item()
    assert err <= (3e-5 if out_dtype == torch.float32 else 1.5e-2) * max(scale, 1.0), (err, scale)
    if fused:
        assert gu.isnan().all()                    # the product itself was never written


def test_gemm_skinny_takes_row_views():
    big = rnd(8, 512, dtype=torch.bfloat16, seed=3)
    x, w = big[:, :256], rnd(70, 256, dtype=torch.bfloat16, seed=4)      # row stride 512, unit inner stride
    out = torch.empty(8, 70, dtype=torch.bfloat16, device=DEV)
    ops.gemm(x, w, out)
    torch.testing.assert_close(out.float(), x.float() @ w.float().t(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 128, 128), (256, 512, 4096), (2048, 6144, 4096), (100, 300, 72),
                                   (1, 256, 64), (129, 257, 200), (64, 4096, 12288), (300, 1000, 136), (2048, 4096, 4096)])
def test_gemm_tcgen05(M, N, K, out_dtype):
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=2)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.gemm_tcgen05(x, w, out)
    ops.check_errors(DEV)
    exp = x.double() @ w.double().t()
    err = (out.double() - exp).abs().max().item()
    scale = exp.abs().max().item()
    assert err <= (3e-5 if out_dtype == torch.float32 else 6e-3) * max(scale, 1.0), (err, scale)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (257, 512, 128), (300, 1000, 328), (2048, 4096, 4096), (511, 6144, 1024),
                                   (1024, 768, 12288), (129, 260, 72), (5000, 520, 256)])
def test_gemm_tcgen05_pair(M, N, K, out_dtype):
    """Two SMs to a 256 x 256 tile: rows and columns that fill no tile, a K that fills no block, few and many tiles."""
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=2)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.gemm_tcgen05_pair(x, w, out)
    ops.check_errors(DEV)
    exp = x.double() @ w.double().t()
    err = (out.double() - exp).abs().max().item()
    assert err <= (2e-5 if out_dtype == torch.float32 else 6e-3) * max(exp.abs().max().item(), 1.0), err
    again = torch.empty_like(out)
    ops.gemm_tcgen05_pair(x, w, again)
    assert torch.equal(out, again)


@pytest.mark.parametrize("M,I,K", [(256, 128, 64), (300, 500, 192), (2048, 12288, 4096), (777, 1536, 1024)])
def test_gemm_tcgen05_pair_gated(M, I, K):
    x = rnd(M, K, dtype=torch.bfloat16, seed=1)
    w = rnd(2 * I, K, dtype=torch.bfloat16, scale=0.08, seed=2)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tcgen05_pair(x, w, out, gated=True)
    ops.check_errors(DEV)
    g, u = x.double() @ w[0::2].double().t(), x.double() @ w[1::2].double().t()
    exp = g / (1 + torch.exp(-g)) * u
    assert (out.double() - exp).abs().max().item() <= 1.5e-2 * max(exp.abs().max().item(), 1.0)


def _paged_setup(dtype, nq, nkv, hd, ps, lens, q_lens, seed=0):
    """Random cache contents for requests of the given lengths, scattered pages."""
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    pages_per = [-(-n // ps) for n in lens]
    total_pages = sum(pages_per) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    width = max(pages_per)
    bt = torch.full((R, width), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(pages_per):
        bt[r, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    kc = (torch.randn(total_pages, nkv, ps, hd, generator=g)).to(dtype).to(DEV)
    vc = (torch.randn(total_pages, nkv, ps, hd, generator=g)).to(dtype).to(DEV)
    positions, rows = [], []
    for r, (n, ql) in enumerate(zip(lens, q_lens)):
        positions += list(range(n - ql, n))
        rows += [r] * ql
    T = len(positions)
    q = (torch.randn(T, nq * hd, generator=g)).to(dtype).to(DEV)
    return (q, kc, vc, torch.tensor(positions, dtype=torch.int32, device=DEV),
            torch.tensor(rows, dtype=torch.int32, device=DEV), bt.to(DEV))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,ps,window", [(4, 2, 16, 4, None), (6, 1, 32, 8, None), (3, 3, 48, 16, 21),
                                                  (8, 1, 128, 16, None), (2, 2, 256, 32, 40), (5, 5, 80, 3, 7)])
def test_paged_attention_plain(dtype, nq, nkv, hd, ps, window):
    lens, q_lens = [1, 37, 150, 64], [1, 5, 1, 64]
    q, kc, vc, pos, rows, bt = _paged_setup(dtype, nq, nkv, hd, ps, lens, q_lens)
    out = torch.empty(q.shape[0], nq * hd, dtype=dtype, device=DEV)
    exp = torch.empty_like(out).cpu()
    ops.paged_attention(q, out, kc, vc, pos, rows, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), window)
    ref.paged_attention(q.cpu(), exp, kc.cpu(), vc.cpu(), pos.cpu(), rows.cpu(), bt.cpu(), nq, nkv, hd, ps,
                        1 / math.sqrt(hd), window)
    torch.testing.assert_close(out.float().cpu(), exp.float(), **tol(dtype))


def test_paged_attention_finds_a_far_key():
    """One key among hundreds, far back, is made to dominate: the output must be
    that key's value row (a kernel that drops or misplaces a page would miss it)."""
    nq, nkv, hd, ps = 4, 2, 64, 16
    for far in (0, 15, 16, 333, 511):
        q, kc, vc, pos, rows, bt = _paged_setup(torch.float32, nq, nkv, hd, ps, [600], [1], seed=far)
        page, off = int(bt[0, far // ps]), far % ps
        kc[page, :, off] = 0
        kc[page, 0, off, :] = q[0, :hd] * 50           # kv head 0 serves q heads 0,1; align with q head 0
        out = torch.empty(1, nq * hd, device=DEV)
        ops.paged_attention(q, out, kc, vc, pos, rows, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), None)
        torch.testing.assert_close(out[0, :hd], vc[page, 0, off], rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,hd,ps,rot,norm", [(4, 2, 16, 4, 16, True), (6, 1, 32, 8, 32, True),
                                                    (3, 3, 48, 16, 48, True), (8, 2, 128, 16, 128, True),
                                                    (2, 1, 64, 16, 32, False), (2, 2, 256, 8, 0, True)])
@pytest.mark.parametrize("T", [23, 70])
def test_attention_prep(dtype, nq, nkv, hd, ps, rot, norm, T):
    pages = -(-T // ps) + 6
    width = (nq + 2 * nkv) * hd
    qkv = rnd(T, width, dtype=dtype, scale=2.0, seed=1)
    pos = torch.randint(0, 5000, (T,), dtype=torch.int32, device=DEV)
    slots = torch.randperm(pages * ps)[:T].to(torch.int32).to(DEV)
    slots[3] = -1
    qw = (1.0 + 0.2 * rnd(hd, seed=2)) if norm else None
    kw = (1.0 + 0.2 * rnd(hd, seed=3)) if norm else None
    inv = torch.pow(torch.tensor(1e4), -2.0 * torch.arange(rot // 2) / max(rot, 1)).float().to(DEV) if rot else None
    kc = torch.zeros(pages, nkv, ps, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    a, b = qkv.clone(), qkv.clone()
    kc2, vc2 = kc.clone(), vc.clone()
    ops.attention_prep(a, pos, slots, qw, kw, 1e-6, inv, rot, kc, vc, nq, nkv, hd, ps)
    ref.attention_prep(b, pos, slots, qw, kw, 1e-6, inv, rot, kc2, vc2, nq, nkv, hd, ps)
    t = dict(rtol=3e-5, atol=3e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(a[:, :nq * hd].float(), b[:, :nq * hd].float(), **t)
    torch.testing.assert_close(kc.float(), kc2.float(), **t)
    assert torch.equal(vc, vc2)


@pytest.mark.parametrize("nq,nkv,hd", [(32, 8, 128), (56, 8, 128), (5, 1, 128), (5, 1, 64), (9, 3, 64), (120, 12, 64)])
@pytest.mark.parametrize("norm", [True, False, "q"])
def test_attention_prep_token_kernel(nq, nkv, hd, norm):
    """The kernel for prompt portions (a block per token, 16-byte lanes, several heads to a warp at once): more heads
    than the block takes in one round, head counts that leave lanes of a warp without a head, both head sizes."""
    T, ps = 70, 16
    pages = -(-T // ps) + 6
    qkv = rnd(T, (nq + 2 * nkv) * hd, dtype=torch.bfloat16, scale=2.0, seed=1)
    pos = torch.randint(0, 40000, (T,), dtype=torch.int32, device=DEV)
    slots = torch.randperm(pages * ps)[:T].to(torch.int32).to(DEV)
    slots[3] = -1
    qw = (1.0 + 0.2 * rnd(hd, seed=2)) if norm else None
    kw = (1.0 + 0.2 * rnd(hd, seed=3)) if norm is True else None          # "q": a query head and a key head of one warp differ
    inv = torch.pow(torch.tensor(1e6), -2.0 * torch.arange(hd // 2) / hd).float().to(DEV)
    kc = torch.zeros(pages, nkv, ps, hd, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    a, b = qkv.clone(), qkv.clone()
    kc2, vc2 = kc.clone(), vc.clone()
    ops.attention_prep(a, pos, slots, qw, kw, 1e-6, inv, hd, kc, vc, nq, nkv, hd, ps)
    ref.attention_prep(b, pos, slots, qw, kw, 1e-6, inv, hd, kc2, vc2, nq, nkv, hd, ps)
    torch.testing.assert_close(a[:, :nq * hd].float(), b[:, :nq * hd].float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(kc.float(), kc2.float(), rtol=2e-2, atol=2e-2)
    assert torch.equal(vc, vc2)
    assert torch.equal(a[:, nq * hd:], qkv[:, nq * hd:])            # keys and values of the projection output stay
    # the kernel for a few tokens (a warp per token and head), 16 tokens at a call: the same bits, so a key has the
    # same bits whether its token came in a prompt portion or alone
    d = qkv.clone()
    kc4, vc4 = torch.zeros_like(kc), torch.zeros_like(vc)
    for lo in range(0, T, 16):
        ops.attention_prep(d[lo:lo + 16], pos[lo:lo + 16], slots[lo:lo + 16], qw, kw, 1e-6, inv, hd, kc4, vc4, nq, nkv, hd, ps)
    assert torch.equal(d, a) and torch.equal(kc4, kc) and torch.equal(vc4, vc)
    # with the step's table of cosines and sines: the same bits as with the angles evaluated in the kernel
    assert ops.attention_prep_takes_angles(qkv, hd, hd)
    angles = torch.empty(T, hd // 2, 2, device=DEV)
    ops.rotary_angles(pos, inv, angles)
    got = angles.double()
    assert (got[..., 0] - torch.cos((pos.float()[:, None] * inv[None, :]).double())).abs().max() < 1e-6
    assert (got[..., 1] - torch.sin((pos.float()[:, None] * inv[None, :]).double())).abs().max() < 1e-6
    c = qkv.clone()
    kc3, vc3 = torch.zeros_like(kc), torch.zeros_like(vc)
    ops.attention_prep(c, pos, slots, qw, kw, 1e-6, inv, hd, kc3, vc3, nq, nkv, hd, ps, angles=angles)
    assert torch.equal(c, a) and torch.equal(kc3, kc) and torch.equal(vc3, vc)


def test_attention_prep_q_only():
    nq, hd, T = 4, 32, 6
    q = rnd(T, nq * hd, seed=1)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    qw = 1.0 + 0.1 * rnd(hd, seed=2)
    inv = torch.pow(torch.tensor(1e6), -2.0 * torch.arange(hd // 2) / hd).float().to(DEV)
    a, b = q.clone(), q.clone()
    ops.attention_prep(a, pos, None, qw, None, 1e-6, inv, hd, None, None, nq, 0, hd, 16)
    ref.attention_prep(b, pos, None, qw, None, 1e-6, inv, hd, None, None, nq, 0, hd, 16)
    torch.testing.assert_close(a, b, rtol=3e-5, atol=3e-5)


@pytest.mark.parametrize("V", [256, 301, 151936])
def test_sample_greedy_lowest_index_on_ties(V):
    logits = rnd(5, V, seed=1)
    logits[1, 7] = logits[1, V - 3] = 50.0
    logits[2, :] = 0.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.sample(logits, None, None, None, None, None, None, out)
    exp = torch.empty(5, dtype=torch.int32)
    ref.sample(logits.cpu(), None, None, None, None, None, None, exp)
    assert out.cpu().tolist() == exp.tolist() and out[1].item() == 7 and out[2].item() == 0


@pytest.mark.parametrize("R,V", [(1, 40), (3, 301), (9, 151936)])
def test_argmax_split_kernel(R, V):
    logits = rnd(R, V, seed=7)
    logits[0, V - 1] = logits[0, 5] = 99.0
    if R > 1:
        logits[1] = -3.0
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.argmax(logits, torch.empty(R * 64, device=DEV), out)
    assert out.tolist() == torch.argmax(logits, dim=1).tolist() and out[0].item() == 5
    if R > 1:
        assert out[1].item() == 0


@pytest.mark.parametrize("V,shift", [(1003, 0), (1003, 1), (1003, 3), (4096, 2), (151936, 0)])
def test_argmax_at_every_edge_of_its_parts(V, shift):
    """The maximum at the first and last places of the 32 parts that the rows are cut into, in rows that start at
    any alignment (the kernel reads 16 bytes at a time between ragged ends), and a tie across two parts."""
    per = -(-V // 32)
    places = sorted({p for k in range(32) for p in (k * per - 1, k * per, k * per + 1, k * per + 2, k * per + 3)
                     if 0 <= p < V} | {V - 1, V - 2})
    R = len(places) + 1
    store = rnd(R, V + 8, seed=3)
    logits = store[:, shift:shift + V]
    for r, pl in enumerate(places):
        logits[r, pl] = 60.0
    logits[R - 1, per + 5] = logits[R - 1, per - 2] = logits[R - 1, 7 * per] = 70.0
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.argmax(logits, torch.empty(R * 64, device=DEV), out)
    assert out.tolist() == places + [per - 2]


@pytest.mark.parametrize("V", [257, 5000])
def test_sample_temperature_top_k_top_p(V):
    R = 8
    logits = rnd(R, V, scale=3.0, seed=2)
    temp = torch.tensor([0.7, 1.0, 0.0, 1.3, 0.5, 1.0, 1.0, 0.9], device=DEV)
    top_k = torch.tensor([-1, 5, -1, 1, 40, -1, 3, -1], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1.0, 1.0, 1.0, 1.0, 0.8, 0.5, 0.9, 1.0], device=DEV)
    min_p = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.1], device=DEV)
    for trial in range(6):
        u = torch.rand(R, generator=torch.Generator().manual_seed(trial)).to(DEV)
        scratch = torch.empty(R, V, device=DEV)
        out = torch.empty(R, dtype=torch.int32, device=DEV)
        ops.sample(logits, temp, top_k, top_p, min_p, u, scratch, out)
        exp = torch.empty(R, dtype=torch.int32)
        ref.sample(logits.cpu(), temp.cpu(), top_k.cpu(), top_p.cpu(), min_p.cpu(), u.cpu(), None, exp)
        got = out.cpu().tolist()
        for r in range(R):
            if got[r] != exp[r].item():
                # only a draw that falls within rounding of a CDF step may differ, by one kept token
                p = torch.softmax(logits[r].double().cpu() / max(float(temp[r]), 1e-9), 0)
                assert abs(got[r] - exp[r].item()) >= 1 and p[got[r]] > 0, (r, got[r], exp[r].item())
                c = torch.cumsum(scratch[r].double().cpu(), 0)
                assert abs(float(c[min(got[r], exp[r].item())]) - float(u[r]) * float(c[-1])) < 1e-5


def test_sample_draws_follow_the_distribution():
    V, n = 50, 4000
    logits = rnd(1, V, scale=2.0, seed=5).repeat(n, 1)
    u = torch.rand(n, generator=torch.Generator().manual_seed(1)).to(DEV)
    ones = torch.ones(n, device=DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, ones, torch.full((n,), -1, dtype=torch.int32, device=DEV), ones, 0 * ones, u,
               torch.empty(n, V, device=DEV), out)
    freq = torch.bincount(out.long().cpu(), minlength=V).double() / n
    p = torch.softmax(logits[0].double().cpu(), 0)
    assert (freq - p).abs().max().item() < 0.03


def test_refuses_cpu_tensors_loudly():
    with pytest.raises(ops.KernelError):
        ops.silu_mul(torch.zeros(2, 8), torch.zeros(2, 4))


# ----------------------------------------------------- tensor-core attention kernels
def _fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=0, scale_q=1.0):
    q, kc, vc, pos, rows, bt = _paged_setup(torch.bfloat16, nq, nkv, hd, ps, lens, q_lens, seed)
    q = (q.float() * scale_q).to(torch.bfloat16)
    qi = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    kv = torch.tensor(lens, dtype=torch.int32, device=DEV)
    return q, kc, vc, pos, rows, bt, qi, kv


def _ref_attn(q, kc, vc, pos, rows, bt, nq, nkv, hd, ps, window):
    exp = torch.empty(q.shape[0], nq * hd, dtype=torch.bfloat16)
    ref.paged_attention(q.cpu(), exp, kc.cpu(), vc.cpu(), pos.cpu(), rows.cpu(), bt.cpu(), nq, nkv, hd, ps,
                        1 / math.sqrt(hd), window)
    return exp.float()


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
@pytest.mark.parametrize("nq,nkv,hd,ps,window", [(32, 8, 128, 16, None), (6, 1, 64, 8, None), (16, 1, 128, 32, None),
                                                  (4, 4, 128, 16, 100), (8, 2, 64, 4, 33), (3, 1, 128, 5, None)])
def test_decode_attention_kernel(nq, nkv, hd, ps, window, splits):
    lens = [1, 63, 64, 65, 700, 2049, 17]
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, [1] * len(lens), seed=3)
    R = len(lens)
    out = torch.zeros(R, nq * hd, dtype=torch.bfloat16, device=DEV)
    po = torch.full((R * nq * splits * hd,), float("nan"), device=DEV)       # stale scratch must not leak
    pml = torch.full((R * nq * splits * 2,), float("nan"), device=DEV)
    cnt = torch.zeros(R * nkv, dtype=torch.int32, device=DEV)
    exp = _ref_attn(q, kc, vc, pos, rows, bt, nq, nkv, hd, ps, window)
    for _ in range(2):                      # twice: the counters must be back at zero after a launch
        out.zero_()
        ops.paged_attention_decode(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), window, splits, po, pml, cnt)
        torch.testing.assert_close(out.float().cpu(), exp, rtol=2e-2, atol=1e-2)
        assert cnt.abs().sum().item() == 0


def _stream_decode(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, window, ctas, scratch=None):
    R = kv.numel()
    slots = (ctas + R * nkv) * (nq // nkv)
    if scratch is None:
        scratch = (torch.full((slots * hd,), float("nan"), device=DEV), torch.full((slots * 2,), float("nan"), device=DEV),
                   torch.zeros(R * nkv, dtype=torch.int32, device=DEV))
    ops.paged_attention_decode_stream(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), window, *scratch, ctas)
    ops.check_errors(DEV)
    return scratch


@pytest.mark.parametrize("ctas", [1, 3, 37, 148, 400])
@pytest.mark.parametrize("nq,nkv,hd,ps,window", [(32, 8, 128, 16, None), (6, 1, 64, 16, None), (16, 1, 128, 32, None),
                                                  (4, 4, 128, 16, 100), (8, 2, 64, 48, 33), (3, 1, 128, 64, 700),
                                                  (10, 2, 64, 16, 64)])
def test_decode_attention_stream_kernel(nq, nkv, hd, ps, window, ctas):
    """Every way of sharing the tiles among CTAs (one CTA alone, pieces of several pairs in one
    CTA, a pair spread over many CTAs, more CTAs than tiles) gives the same attention."""
    lens = [1, 63, 64, 65, 700, 2049, 17, 128]
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, [1] * len(lens), seed=3)
    out = torch.zeros(len(lens), nq * hd, dtype=torch.bfloat16, device=DEV)
    exp = _ref_attn(q, kc, vc, pos, rows, bt, nq, nkv, hd, ps, window)
    scratch = None
    for _ in range(2):                      # twice: the counters must be back at zero after a launch
        out.zero_()
        scratch = _stream_decode(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, window, ctas, scratch)
        torch.testing.assert_close(out.float().cpu(), exp, rtol=2e-2, atol=1e-2)
        assert scratch[2].abs().sum().item() == 0


@pytest.mark.parametrize("norm,rot", [(True, True), (False, True), (True, False)])
@pytest.mark.parametrize("nq,nkv,hd,ps,window,lens", [
    (32, 8, 128, 16, None, [2049] * 8), (32, 8, 128, 16, None, [1, 63, 64, 65, 700, 2049, 17, 128]),
    (6, 1, 64, 16, None, [5, 300, 1024]), (16, 1, 128, 32, None, [2000]), (4, 4, 128, 16, 100, [1, 99, 100, 101, 640]),
    (8, 2, 64, 48, 33, [97, 48, 49, 1]), (2, 1, 128, 64, None, [64 * k + d for k in (1, 3) for d in (-1, 0, 1)]),
    (8, 8, 64, 16, None, [int(x) for x in torch.randint(1, 500, (70,), generator=torch.Generator().manual_seed(5))])])
def test_decode_attention_with_fused_preparation(nq, nkv, hd, ps, window, lens, norm, rot):
    """One launch that norms and rotates the queries and the new keys, stores the new keys and values and
    attends, against the preparation kernel followed by the attention kernel: the same arithmetic in the
    same order, so the same bits in the output and in the cache (also at the first token of a sequence, at
    the edges of tiles and pages, and with pieces of several rows in one CTA).  Without a rotation the separate
    preparation runs on the general kernel, which adds the squares of a head in another order: equal within
    rounding there (one draw in twenty of random shapes differs in a bit), bit for bit with the rotation."""
    from types import SimpleNamespace
    from arle_b200.engine import Workspace

    R, eps = len(lens), 1e-5
    _, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, [1] * R, seed=3)
    qkv = rnd(R, (nq + 2 * nkv) * hd + 8, dtype=torch.bfloat16, seed=7)[:, : (nq + 2 * nkv) * hd]     # rows with a stride of their own
    qw = (1 + 0.2 * rnd(hd, seed=8)).contiguous() if norm else None
    kw = (1 + 0.2 * rnd(hd, seed=9)).contiguous() if norm else None
    inv_freq = torch.pow(torch.tensor(1e4), -torch.arange(hd // 2, dtype=torch.float32) * 2 / hd).to(DEV) if rot else None
    last = kv.long() - 1
    slots = (bt[torch.arange(R, device=DEV), last // ps].long() * ps + last % ps).to(torch.int32)
    assert torch.equal(pos.long(), last)
    # the two-kernel way
    qkv_a, kc_a, vc_a = qkv.clone(), kc.clone(), vc.clone()
    ops.attention_prep(qkv_a, pos, slots, qw, kw, eps, inv_freq, hd if rot else 0, kc_a, vc_a, nq, nkv, hd, ps)
    want = torch.zeros(R, nq * hd, dtype=torch.bfloat16, device=DEV)
    _stream_decode(qkv_a[:, : nq * hd], want, kc_a, vc_a, qi, kv, bt, nq, nkv, hd, ps, window, ops.sm_count(DEV))
    # the one-kernel way
    kc_b, vc_b = kc.clone(), vc.clone()
    batch = SimpleNamespace(max_q_len=1, num_rows=R, ws=Workspace(DEV), q_indptr=qi, kv_lens=kv)
    assert ops.fused_decode_supported(qkv, batch, kc.dtype, nq, nkv, hd, ps, hd if rot else 0)
    got = torch.full((R, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    for _ in range(2):
        ops.decode_attention_with_prep(qkv, got, kc_b, vc_b, slots, qw, kw, eps, inv_freq, bt, nq, nkv, hd, ps,
                                       1 / math.sqrt(hd), window, batch)
        ops.check_errors(DEV)
        if rot:
            assert torch.equal(kc_b, kc_a) and torch.equal(vc_b, vc_a)
            assert torch.equal(got, want)
        else:
            torch.testing.assert_close(kc_b.float(), kc_a.float(), rtol=1e-2, atol=1e-2)
            torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=1e-2)
            assert torch.equal(vc_b, vc_a)
    # with the step's plan (shares and first pages worked out once, kept in the step's memo): the same bits, twice
    # (the second launch finds the plan in the memo)
    batch.memo = {}
    kc_c, vc_c = kc.clone(), vc.clone()
    for _ in range(2):
        again = torch.full((R, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.decode_attention_with_prep(qkv, again, kc_c, vc_c, slots, qw, kw, eps, inv_freq, bt, nq, nkv, hd, ps,
                                       1 / math.sqrt(hd), window, batch)
        ops.check_errors(DEV)
        assert torch.equal(again, got) and torch.equal(kc_c, kc_b) and torch.equal(vc_c, vc_b)
    assert len(batch.memo) == 1


@pytest.mark.parametrize("ctas", [7, 148])
def test_decode_attention_stream_many_rows(ctas):
    """More rows than one warp scans at once, lengths of every kind, prompt rows in between."""
    g = torch.Generator().manual_seed(11)
    R = 77
    lens = [int(v) for v in torch.randint(1, 400, (R,), generator=g)]
    q_lens = [1] * R
    for r in (3, 40, 41, 76):                      # rows of a prompt portion: left alone
        q_lens[r] = min(lens[r], 5)
    nq, nkv, hd, ps = 4, 2, 64, 16
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=12)
    out = torch.full((q.shape[0], nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    _stream_decode(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, None, ctas)
    exp = _ref_attn(q, kc, vc, pos, rows, bt, nq, nkv, hd, ps, None)
    single = torch.tensor([int(qi[r]) for r in range(R) if q_lens[r] == 1])
    multi = torch.tensor([t for r in range(R) if q_lens[r] > 1 for t in range(int(qi[r]), int(qi[r + 1]))])
    assert out[multi.to(DEV)].isnan().all()
    torch.testing.assert_close(out[single.to(DEV)].float().cpu(), exp[single], rtol=2e-2, atol=1e-2)


def test_decode_attention_stream_skips_prompt_rows_and_stale_slots():
    """Rows with several queries are left alone, and cache slots beyond a request's last
    key, holding huge values, do not leak through P = 0."""
    nq, nkv, hd, ps = 8, 2, 128, 16
    lens, q_lens = [100, 40, 7, 300, 1], [1, 40, 1, 11, 1]
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=5)
    used = torch.zeros(kc.shape[0], ps, dtype=torch.bool)
    for r, n in enumerate(lens):
        for j in range(n):
            used[int(bt[r, j // ps]), j % ps] = True
    vc[~used.to(DEV)[:, None, :].expand(-1, nkv, -1)] = 3.0e38
    kc[~used.to(DEV)[:, None, :].expand(-1, nkv, -1)] = 3.0e38
    out = torch.full((q.shape[0], nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    _stream_decode(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, None, 148)
    single = torch.tensor([0, 41, 53])
    assert out[1:41].isnan().all() and out[42:53].isnan().all()
    exp = _ref_attn(q, kc, vc, pos, rows, bt, nq, nkv, hd, ps, None)
    assert torch.isfinite(out[single.to(DEV)].float()).all()
    torch.testing.assert_close(out[single.to(DEV)].float().cpu(), exp[single], rtol=2e-2, atol=1e-2)


def test_decode_attention_stream_refuses_small_pages():
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(4, 2, 128, 8, [30], [1], seed=1)
    out = torch.zeros(1, 4 * 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ops.KernelError):
        _stream_decode(q, out, kc, vc, qi, kv, bt, 4, 2, 128, 8, None, 8)
    assert ops.stream_decode_supported(64, 16, 8) and not ops.stream_decode_supported(64, 16, 17)


@pytest.mark.parametrize("nq,nkv,hd,R,n", [(64, 8, 128, 64, 2048), (16, 1, 128, 64, 2048), (32, 8, 128, 40, 3000),
                                           (14, 2, 64, 64, 1500)])
def test_decode_attention_stream_long_runs(nq, nkv, hd, R, n):
    """Many rows of long contexts: every CTA walks a hundred tiles and more, across several pairs,
    with HBM saturated, so that copies land far out of the order they were issued in.  The ring's
    depth (which the shared memory left beside the merge scratch decides, and which must be even for
    the two consumer groups' waits to tell a stage's phases apart) differs between these shapes."""
    ps = 16
    lens = [n - (r % 5) * 13 for r in range(R)]
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, [1] * R, seed=21)
    exp = _ref_attn(q, kc, vc, pos, rows, bt, nq, nkv, hd, ps, None)
    out = torch.zeros(R, nq * hd, dtype=torch.bfloat16, device=DEV)
    scratch = None
    for _ in range(3):
        out.zero_()
        scratch = _stream_decode(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, None, 148, scratch)
        torch.testing.assert_close(out.float().cpu(), exp, rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("nq,nkv,hd,ps,window", [(32, 8, 128, 16, None), (6, 1, 64, 8, None), (4, 4, 128, 16, 70),
                                                  (8, 2, 64, 4, 33), (3, 1, 128, 5, 64), (2, 1, 128, 64, 65)])
def test_prefill_attention_kernel(nq, nkv, hd, ps, window):
    lens, q_lens = [130, 300, 64, 65, 9, 200], [130, 2, 64, 3, 1, 77]
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=4)
    out = torch.zeros(q.shape[0], nq * hd, dtype=torch.bfloat16, device=DEV)
    ops.paged_attention_prefill(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), window, max(q_lens))
    exp = _ref_attn(q, kc, vc, pos, rows, bt, nq, nkv, hd, ps, window)
    torch.testing.assert_close(out.float().cpu(), exp, rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("nq,nkv,ps,window", [(2, 1, 16, None), (8, 2, 16, None), (32, 8, 16, None), (4, 4, 32, 70), (3, 1, 64, 129),
                                               (2, 2, 16, 500)])
def test_prefill_attention_tcgen05_kernel(nq, nkv, ps, window):
    hd = 128
    lens, q_lens = [130, 300, 128, 129, 9, 700, 1000], [130, 2, 128, 3, 1, 333, 1000]
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=6)
    out = torch.zeros(q.shape[0], nq * hd, dtype=torch.bfloat16, device=DEV)
    ops.paged_attention_prefill_tc(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), window, max(q_lens))
    ops.check_errors(DEV)
    exp = _ref_attn(q, kc, vc, pos, rows, bt, nq, nkv, hd, ps, window)
    torch.testing.assert_close(out.float().cpu(), exp, rtol=2e-2, atol=1e-2)


def test_prefill_attention_tcgen05_random_shapes_one_after_another():
    """Sixty launches of random shapes in a row, each against the mma.sync kernel: fewer blocks than SMs and several
    times more, rows whose last block is nearly empty, rows of one query, windows, and after each launch the
    counter that the resident CTAs draw their blocks from must be back at zero for the next one."""
    import random
    rng = random.Random(11)
    hd = 128
    for case in range(60):
        nkv = rng.choice([1, 2, 3, 8])
        nq = nkv * rng.choice([1, 2, 4, 5])
        ps = rng.choice([16, 32, 64])
        R = rng.randint(1, 6)
        q_lens = [rng.choice([1, 2, 17, 128, 255, 256, 257, rng.randint(1, 900)]) for _ in range(R)]
        lens = [n + rng.choice([0, 0, 5, 128, rng.randint(0, 600)]) for n in q_lens]
        window = rng.choice([None, None, 33, 128, 300])
        q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=100 + case)
        got = torch.full((q.shape[0], nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        want = torch.zeros_like(got)
        ops.paged_attention_prefill_tc(q, got, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), window, max(q_lens))
        ops.paged_attention_prefill(q, want, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), window, max(q_lens))
        ops.check_errors(DEV)
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=1e-2,
                                   msg=lambda m: f"case {case}: nq {nq} nkv {nkv} page {ps} q {q_lens} kv {lens} window {window}: {m}")


def test_prefill_attention_tcgen05_sharp_scores_and_stale_rows():
    """Scores far apart (the lazy rescaling of the accumulator must kick in) and a cache
    whose unused slots hold huge values (they must not leak through P = 0)."""
    nq, nkv, hd, ps = 4, 2, 128, 16
    lens, q_lens = [520, 77], [520, 77]
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=7, scale_q=6.0)
    used = torch.zeros(kc.shape[0], ps, dtype=torch.bool)
    for r, n in enumerate(lens):
        for j in range(n):
            used[int(bt[r, j // ps]), j % ps] = True
    vc[~used.to(DEV)[:, None, :].expand(-1, nkv, -1)] = 3.0e38
    out = torch.zeros(q.shape[0], nq * hd, dtype=torch.bfloat16, device=DEV)
    ops.paged_attention_prefill_tc(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), None, max(q_lens))
    ops.check_errors(DEV)
    exp = _ref_attn(q, kc, vc, pos, rows, bt, nq, nkv, hd, ps, None)
    assert torch.isfinite(out.float()).all()
    torch.testing.assert_close(out.float().cpu(), exp, rtol=3e-2, atol=2e-2)


def test_prefill_and_decode_kernels_split_a_mixed_step():
    nq, nkv, hd, ps = 8, 2, 128, 16
    lens, q_lens = [100, 40, 7, 300], [1, 40, 1, 11]
    q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=5)
    out = torch.full((q.shape[0], nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.paged_attention_prefill(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), None, 40, skip_single=True)
    assert out[0].isnan().all() and out[41].isnan().all() and not out[1:41].isnan().any()
    ops.paged_attention_decode(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), None, 1)
    exp = _ref_attn(q, kc, vc, pos, rows, bt, nq, nkv, hd, ps, None)
    torch.testing.assert_close(out.float().cpu(), exp, rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("kernel", ["decode", "stream", "prefill"])
def test_fast_attention_sees_one_far_key_and_the_windows_edge(kernel):
    """Peaked attention: the query is aligned with exactly one key far back, so the
    output must be that key's value; with a window that ends one key short of it,
    the key must be invisible."""
    nq, nkv, hd, ps = 4, 1, 128, 16
    n = 1000
    for far in (0, 63, 64, 500, 998):
        lens, q_lens = ([n], [3]) if kernel == "prefill" else ([n], [1])
        q, kc, vc, pos, rows, bt, qi, kv = _fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=far)
        page, off = int(bt[0, far // ps]), far % ps
        unit = torch.zeros(hd)
        unit[far % hd] = 1.0
        kc[page, 0, off] = (unit * 40).to(torch.bfloat16).to(DEV)
        q[-1, :hd] = (unit * 40).to(torch.bfloat16).to(DEV)           # last query, head 0
        for window, visible in ((None, True), (n - far, True), (n - far - 1, False)):
            out = torch.zeros(q.shape[0], nq * hd, dtype=torch.bfloat16, device=DEV)
            if kernel == "decode":
                ops.paged_attention_decode(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), window, 4,
                                           torch.empty(nq * 4 * hd, device=DEV), torch.empty(nq * 8, device=DEV),
                                           torch.zeros(nkv, dtype=torch.int32, device=DEV))
            elif kernel == "stream":
                _stream_decode(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, window, 5)
            else:
                ops.paged_attention_prefill(q, out, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), window, 3)
            close = (out[-1, :hd].float() - vc[page, 0, off].float()).abs().max().item() < 2e-2
            assert close == visible, (far, window)
