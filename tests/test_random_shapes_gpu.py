"""Tests over random shapes.  Differential tests of the fast attention kernels: the streaming decode
kernel against the split-KV kernel, and the tcgen05 prefill kernel against the mma.sync one.
Each pair shares no code beyond the cache layout, and each is compared with the plain reference
at fixed shapes elsewhere; here the shapes are drawn at random (numbers of rows, heads and groups,
page sizes, windows, lengths around the tile edges, prompt portions beside decoded rows, grid
sizes), which is where the ways of sharing the work out among CTAs meet their corner cases.
And the weight-streaming product against float64 over random row counts, widths and depths
(depths beside the edges of its stages, widths beside the number of SMs, depths long enough for
a cluster together with many output rows)."""
import math
import random

import pytest
import torch

import test_kernels_gpu as tk
from arle_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("seed", [1, 2])
def test_stream_decode_equals_split_kv_on_random_shapes(seed):
    rng = random.Random(seed)
    for it in range(30):
        nkv = rng.choice([1, 2, 4, 8])
        group = rng.choice([1, 2, 3, 4, 7, 8, 16])
        nq = nkv * group
        hd, ps = rng.choice([64, 128]), rng.choice([16, 32, 48, 64])
        R = rng.choice([1, 2, 3, 5, 8, 13, 18, 19, 30, 40])
        kind = rng.choice(["short", "mixed", "long", "equal"])
        if kind == "short":
            lens = [rng.randint(1, 130) for _ in range(R)]
        elif kind == "mixed":
            lens = [rng.choice([1, 17, 64, 65, 300, 1000, 2500]) + rng.randint(0, 5) for _ in range(R)]
        elif kind == "long":
            lens = [rng.randint(1500, 3000) for _ in range(R)]
        else:
            lens = [rng.choice([64, 700, 2048])] * R
        if sum(lens) * nkv * hd > 40_000_000:                 # keep the host-side setup small
            lens = [min(n, 600) for n in lens]
        q_lens = [1 if rng.random() < 0.85 else min(n, rng.randint(2, 6)) for n in lens]
        window = rng.choice([None, None, 33, 100, 700])
        ctas = rng.choice([148, 148, 148, 37, 5])
        q, kc, vc, pos, rows, bt, qi, kv = tk._fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=1000 * seed + it)
        a = torch.zeros(q.shape[0], nq * hd, dtype=torch.bfloat16, device=DEV)
        b = torch.zeros_like(a)
        tk._stream_decode(q, a, kc, vc, qi, kv, bt, nq, nkv, hd, ps, window, ctas)
        splits = rng.choice([1, 3, 8])
        po = torch.empty(R * nq * splits * hd, device=DEV)
        pml = torch.empty(R * nq * splits * 2, device=DEV)
        cnt = torch.zeros(R * nkv, dtype=torch.int32, device=DEV)
        ops.paged_attention_decode(q, b, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), window, splits, po, pml, cnt)
        ops.check_errors(DEV)
        single = [int(qi[r]) for r in range(R) if q_lens[r] == 1]
        if not single:
            continue
        idx = torch.tensor(single, device=DEV)
        what = dict(nq=nq, nkv=nkv, hd=hd, ps=ps, R=R, window=window, ctas=ctas, lens=lens[:8])
        assert torch.isfinite(a[idx].float()).all(), what
        torch.testing.assert_close(a[idx].float(), b[idx].float(), rtol=2e-2, atol=1e-2, msg=lambda m: f"{m}\n{what}")


@pytest.mark.parametrize("seed", [1, 2])
def test_tcgen05_prefill_equals_mma_sync_prefill_on_random_shapes(seed):
    rng = random.Random(seed)
    hd = 128
    for it in range(25):
        nkv = rng.choice([1, 2, 4])
        nq = nkv * rng.choice([1, 2, 4, 5])
        ps = rng.choice([16, 32, 48, 64])
        lens, q_lens = [], []
        for _ in range(rng.choice([1, 2, 3, 5])):
            # portions whose ends fall on and beside the edges of the 128-row query tiles and the 256-row blocks
            n = rng.choice([1, 2, 3, 127, 128, 129, 200, 255, 256, 257, 300, 384, 385, 511, 512, 513, 700, 1025])
            past = rng.choice([0, 0, 1, 63, 64, 100, 128, 129, 500])
            q_lens.append(n)
            lens.append(n + past)
        window = rng.choice([None, None, 1, 2, 64, 127, 128, 129, 130, 255, 256, 257, 300, 600])
        q, kc, vc, pos, rows, bt, qi, kv = tk._fast_setup(nq, nkv, hd, ps, lens, q_lens, seed=2000 * seed + it)
        a = torch.zeros(q.shape[0], nq * hd, dtype=torch.bfloat16, device=DEV)
        b = torch.zeros_like(a)
        ops.paged_attention_prefill_tc(q, a, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), window, max(q_lens))
        ops.paged_attention_prefill(q, b, kc, vc, qi, kv, bt, nq, nkv, hd, ps, 1 / math.sqrt(hd), window, max(q_lens))
        ops.check_errors(DEV)
        what = dict(nq=nq, nkv=nkv, ps=ps, q_lens=q_lens, lens=lens, window=window)
        assert torch.isfinite(a.float()).all(), what
        torch.testing.assert_close(a.float(), b.float(), rtol=3e-2, atol=2e-2, msg=lambda m: f"{m}\n{what}")


@pytest.mark.parametrize("seed", [1, 2])
def test_weight_streaming_gemm_on_random_shapes(seed):
    rng = random.Random(seed)
    for it in range(40):
        M = rng.randint(1, 8)
        K = 32 * rng.choice([1, 2, 3, 7, 16, 31, 32, 33, 64, 100, 128, 129, 160, 200, 256, 300, 384, 512])
        N = rng.choice([1, 2, 15, 16, 17, 33, 100, 147, 148, 149, 296, 1000, 2368, 2369, 4096, 5000, 20000])
        out_dtype = rng.choice([torch.bfloat16, torch.float32])
        gated = rng.random() < 0.3
        g = torch.Generator().manual_seed(100 * seed + it)
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
        what = dict(M=M, N=N, K=K, gated=gated, out=str(out_dtype))
        if gated:
            inter = max(1, N // 2)
            w = (torch.randn(2 * inter, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
            gate_up = torch.empty(M, 2 * inter, dtype=torch.bfloat16, device=DEV)
            out = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
            ops.gemm_silu_mul(x, w, gate_up, out)
            gate, up = x.double() @ w[0::2].double().t(), x.double() @ w[1::2].double().t()
            exp = gate / (1 + torch.exp(-gate)) * up
            bound = 1.5e-2
        else:
            w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
            out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
            ops.gemm(x, w, out)
            exp = x.double() @ w.double().t()
            bound = 2e-5 if out_dtype == torch.float32 else 6e-3
        ops.check_errors(DEV)                                  # no bounded wait ran out
        err = (out.double() - exp).abs().max().item()
        assert err <= bound * max(exp.abs().max().item(), 1.0), (what, err)
