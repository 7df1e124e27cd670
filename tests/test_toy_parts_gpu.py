"""Parts that no model of the package has, defined here, registered here and run through the
package's model, cache, step function and kernels without a change to the package: a
feed-forward that routes each token to two of several experts, and a position encoding with
frequencies and a rotated span of its own.  They sit in one model beside the package's own
attention (one layer with a window) and gated feed-forward, so the model has a different mixer
setting and a different feed-forward in each layer.  The toy feed-forward is written with torch
operations: it tests the framework's interfaces, not a kernel.  Compared with a whole-sequence
computation in float64 written out below."""
import math
from dataclasses import dataclass
from typing import ClassVar

import pytest
import torch

import plain_qwen3 as plain
from arle_b200.config import ModelSpec, ScheduleEntry
from arle_b200.engine import ModelRunner, StepEntry
from arle_b200.parts import (AttentionSpec, DecoderModel, GatedMlpSpec, PreNormBlockSpec, RmsNormSpec, WeightDecl,
                             build_model, register_model, register_part)
from arle_b200.parts.base import CacheNeed, FeedForward, Mixer, PositionEncoding
from arle_b200.weights import random_tensors

pytestmark = pytest.mark.gpu
DEV = "cuda"


# ------------------------------------------------------------------ a routed feed-forward
@dataclass(frozen=True)
class RoutedFfnSpec:
    prefix: str
    hidden_size: int
    expert_size: int
    num_experts: int
    top_k: int
    kind: ClassVar[str] = "test_routed_ffn"


class RoutedFfn(FeedForward):
    """Router logits and their softmax in float32; the top_k experts of a token, their
    probabilities renormalised to sum to one, each expert a small gated feed-forward."""

    def __init__(self, spec):
        self.spec = spec

    def weight_decls(self):
        s, p = self.spec, self.spec.prefix
        decls = [WeightDecl(p + "router.weight", (s.num_experts, s.hidden_size))]
        for e in range(s.num_experts):
            decls += [WeightDecl(p + f"experts.{e}.gate.weight", (s.expert_size, s.hidden_size)),
                      WeightDecl(p + f"experts.{e}.up.weight", (s.expert_size, s.hidden_size)),
                      WeightDecl(p + f"experts.{e}.down.weight", (s.hidden_size, s.expert_size))]
        return tuple(decls)

    def load(self, tensors, dtype, device):
        s, p = self.spec, self.spec.prefix
        self.router = tensors[p + "router.weight"].to(device=device, dtype=torch.float32)
        self.experts = [tuple(tensors[p + f"experts.{e}.{n}.weight"].to(device=device, dtype=dtype) for n in ("gate", "up", "down"))
                        for e in range(s.num_experts)]

    def weight_bytes(self):
        return self.router.numel() * 4 + sum(t.numel() * t.element_size() for ex in self.experts for t in ex)

    def forward(self, x, ctx):
        prob = torch.softmax(x.float() @ self.router.t(), dim=-1)
        top_p, top_e = prob.topk(self.spec.top_k, dim=-1)
        top_p = top_p / top_p.sum(dim=-1, keepdim=True)
        out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
        for e, (wg, wu, wd) in enumerate(self.experts):
            rows, which = (top_e == e).nonzero(as_tuple=True)
            if rows.numel() == 0:
                continue
            xe = x[rows]
            g = (xe @ wg.t()).float()
            act = (g / (1.0 + torch.exp(-g)) * (xe @ wu.t()).float()).to(x.dtype)
            out.index_add_(0, rows, (act @ wd.t()).float() * top_p[rows, which][:, None])
        return out.to(x.dtype)


def plain_routed_ffn(x, w, p, spec):
    prob = torch.softmax(x @ w[p + "router.weight"].T, dim=-1)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        top = torch.argsort(prob[t], descending=True)[: spec.top_k]
        norm = prob[t][top].sum()
        for e in top.tolist():
            g = x[t] @ w[p + f"experts.{e}.gate.weight"].T
            u = x[t] @ w[p + f"experts.{e}.up.weight"].T
            out[t] += prob[t][e] / norm * ((g / (1.0 + torch.exp(-g)) * u) @ w[p + f"experts.{e}.down.weight"].T)
    return out


# ------------------------------------------------------------------ another position encoding
@dataclass(frozen=True)
class PowerLawRotarySpec:
    rotary_dim: int                 # only the first rotary_dim elements of a head turn
    exponent: float
    kind: ClassVar[str] = "test_power_law_rotary"


class PowerLawRotary(PositionEncoding):
    """Rotation with inv_freq_i = (i + 1)^-exponent over the first rotary_dim elements of a head
    (pairs i, i + rotary_dim/2); the rest of the head is left as it is."""

    def __init__(self, spec):
        self.spec = spec

    def load(self, tensors, dtype, device):
        i = torch.arange(self.spec.rotary_dim // 2, dtype=torch.float64)
        self.inv_freq = torch.pow(i + 1.0, -self.spec.exponent).to(torch.float32).to(device)

    def rotary(self):
        return self.inv_freq, self.spec.rotary_dim


def plain_power_law_rotation(x, positions, spec):
    rd, half = spec.rotary_dim, spec.rotary_dim // 2
    inv = torch.pow(torch.arange(half, dtype=torch.float64) + 1.0, -spec.exponent)
    ang = positions.double()[:, None] * inv[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    lo, hi = x[..., :half], x[..., half:rd]
    return torch.cat([lo * cos - hi * sin, lo * sin + hi * cos, x[..., rd:]], dim=-1)


# ------------------------------------------------------------------ the model around them
H, V, NQ, NKV, HD, EPS = 96, 211, 6, 2, 32, 1e-5
ROUTED = RoutedFfnSpec("layers.0.moe.", H, 40, 5, 2)
POWER = PowerLawRotarySpec(16, 1.3)
WINDOW = 24


def _model_spec(routed):
    def attn(i, position, window):
        return AttentionSpec(f"layers.{i}.attn.", H, NQ, NKV, HD, 1.0 / math.sqrt(HD), EPS, position, window)

    def norm(name):
        return RmsNormSpec(name, H, EPS)

    first = ROUTED if routed else GatedMlpSpec("layers.0.mlp.", H, 56)
    blocks = (PreNormBlockSpec(norm("layers.0.n1.weight"), attn(0, POWER, None), norm("layers.0.n2.weight"), first),
              PreNormBlockSpec(norm("layers.1.n1.weight"), attn(1, POWER, WINDOW), norm("layers.1.n2.weight"),
                               GatedMlpSpec("layers.1.mlp.", H, 72)))
    return ModelSpec("ToyPartsForTests", V, H, blocks, (ScheduleEntry(0), ScheduleEntry(1)), norm("norm.weight"),
                     "embed.weight", None, 4096)


def plain_forward(w, tokens, routed):
    wd = {k: v.double() for k, v in w.items()}
    T = len(tokens)
    pos = torch.arange(T)
    x = wd["embed.weight"][torch.tensor(tokens)]
    for i, window in ((0, None), (1, WINDOW)):
        p = f"layers.{i}."
        h = plain.rms_norm(x, wd[p + "n1.weight"], EPS)
        q = plain.rms_norm((h @ wd[p + "attn.q_proj.weight"].T).view(T, NQ, HD), wd[p + "attn.q_norm.weight"], EPS)
        k = plain.rms_norm((h @ wd[p + "attn.k_proj.weight"].T).view(T, NKV, HD), wd[p + "attn.k_norm.weight"], EPS)
        v = (h @ wd[p + "attn.v_proj.weight"].T).view(T, NKV, HD)
        q, k = plain_power_law_rotation(q, pos, POWER), plain_power_law_rotation(k, pos, POWER)
        o = plain.causal_attention(q, k, v, 1.0 / math.sqrt(HD), window)
        x = x + o.reshape(T, NQ * HD) @ wd[p + "attn.o_proj.weight"].T
        h = plain.rms_norm(x, wd[p + "n2.weight"], EPS)
        x = x + (plain_routed_ffn(h, wd, p + "moe.", ROUTED) if i == 0 and routed else plain.swiglu_mlp(h, wd, p + "mlp."))
    return plain.rms_norm(x, wd["norm.weight"], EPS) @ wd["embed.weight"].T


# In bfloat16 a token whose second and third expert are nearly tied may go to another expert than
# in the float64 computation, and the later tokens see its keys: the routed model is compared in
# 32-bit, the position encoding in both.
@pytest.mark.parametrize("dtype,routed", [(torch.float32, True), (torch.float32, False), (torch.bfloat16, False)])
def test_toy_routed_feed_forward_and_position_encoding_in_one_model(dtype, routed):
    register_part(RoutedFfnSpec.kind, RoutedFfn)
    register_part(PowerLawRotarySpec.kind, PowerLawRotary)
    model = DecoderModel(_model_spec(routed))
    # two layers of attention with different windows: two groups of pages
    assert len(model.cache_needs) == 2 and model.state_needs == []
    w = random_tensors(model.weight_decls(), 9, sigma=0.25, dtype=torch.float32)
    if dtype == torch.bfloat16:
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}          # both sides see the same weights
    model.load(w, dtype, DEV)
    runner = ModelRunner(model, 16, 12, 3, device=DEV)
    g = torch.Generator().manual_seed(2)
    a = torch.randint(0, V, (70,), generator=g).tolist()
    b = torch.randint(0, V, (45,), generator=g).tolist()
    want_a, want_b = plain_forward(w, a, routed), plain_forward(w, b, routed)
    got_a, got_b = [], []
    got_a.append(runner.step([StepEntry("a", a[:33], range(33))]).clone())
    lg = runner.step([StepEntry("a", a[33:34], (0,)), StepEntry("b", b[:20], range(20))]).clone()
    got_a.append(lg[:1]); got_b.append(lg[1:])
    lg = runner.step([StepEntry("b", b[20:22], (0, 1)), StepEntry("a", a[34:60], range(26))]).clone()
    got_b.append(lg[:2]); got_a.append(lg[2:])
    at_a, at_b = 60, 22
    while at_a < len(a) or at_b < len(b):
        entries = []
        if at_a < len(a):
            entries.append(StepEntry("a", a[at_a:at_a + 1], (0,)))
        if at_b < len(b):
            n = min(3, len(b) - at_b)
            entries.append(StepEntry("b", b[at_b:at_b + n], range(n)))
        lg = runner.step(entries).clone()
        if at_a < len(a):
            got_a.append(lg[:1]); lg = lg[1:]; at_a += 1
        if at_b < len(b):
            got_b.append(lg); at_b += n
    # the engine tests' bounds (2e-5 and 4e-2 on logits of magnitude 1.5), as fractions of this model's largest logit
    frac = 2e-5 if dtype == torch.float32 else 2.7e-2
    for got, want in ((got_a, want_a), (got_b, want_b)):
        tol = frac * want.abs().max().item()
        err = (torch.cat(got).double().cpu() - want).abs().max(dim=1).values
        assert err.max().item() < tol, f"first wrong position {int((err >= tol).nonzero()[0])}: {err.max().item()}"
    runner.end_request("a")
    runner.end_request("b")


# ------------------------------------------------------------------ a mixer with one compressed vector per token
@dataclass(frozen=True)
class LatentMixerSpec:
    prefix: str
    hidden_size: int
    latent: int
    kind: ClassVar[str] = "test_latent_mixer"


class LatentMixer(Mixer):
    """Keeps ONE vector of ``latent`` numbers per token in the paged cache (not keys and values of
    equal shape): c_t = x_t Wc.  A query q_t = x_t Wq scores the vectors of its request up to its own
    position, and the output is (softmax(q c^T / sqrt(latent)) c) Wo.  Written with torch operations
    over the cache manager's pages, block table and slot mapping."""

    def __init__(self, spec):
        self.spec = spec

    def weight_decls(self):
        s, p = self.spec, self.spec.prefix
        return (WeightDecl(p + "wc.weight", (s.latent, s.hidden_size)), WeightDecl(p + "wq.weight", (s.latent, s.hidden_size)),
                WeightDecl(p + "wo.weight", (s.hidden_size, s.latent)))

    def load(self, tensors, dtype, device):
        p = self.spec.prefix
        self.wc, self.wq, self.wo = (tensors[p + n + ".weight"].to(device=device, dtype=torch.float32) for n in ("wc", "wq", "wo"))

    def cache_need(self):
        return CacheNeed(streams=((1, self.spec.latent),))

    def forward(self, x, ctx, cache, state):
        L = self.spec.latent
        assert len(cache.streams) == 1 and tuple(cache.streams[0].shape[1:]) == (1, cache.page_size, L)
        pages = cache.streams[0]
        flat = pages.view(-1, L)                                     # one head: token slot = page * page_size + offset
        xf = x.float()
        flat[cache.slot_mapping.long()] = (xf @ self.wc.t()).to(pages.dtype)
        q = xf @ self.wq.t()
        out = torch.zeros(x.shape[0], L, device=x.device)
        at = 0
        for r, (n, kv) in enumerate(zip(ctx.q_lens, ctx.kv_lens_host)):
            held = cache.block_table[r, : -(-kv // cache.page_size)].long()
            c = pages[held, 0].reshape(-1, L)[:kv].float()
            sc = q[at:at + n] @ c.t() / math.sqrt(L)
            pos = torch.arange(kv - n, kv, device=x.device)[:, None]
            sc = sc.masked_fill(torch.arange(kv, device=x.device)[None, :] > pos, float("-inf"))
            out[at:at + n] = torch.softmax(sc, dim=-1) @ c
            at += n
        return (out @ self.wo.t()).to(x.dtype)


# ------------------------------------------------------------------ a model class of another arrangement
class ScaledCappedDecoder(DecoderModel):
    """The embedding times a constant, and logits capped smoothly: cap * tanh(logits / cap)."""

    MULT, CAP = 3.0, 4.0

    def embed_tokens(self, ctx):
        resid = super().embed_tokens(ctx)
        resid.mul_(self.MULT)
        return resid

    def logits_at_wanted(self, stream, ctx):
        logits = super().logits_at_wanted(stream, ctx)
        return torch.tanh(logits / self.CAP) * self.CAP


def test_toy_latent_cache_mixer_and_a_model_class_of_its_own():
    register_part(LatentMixerSpec.kind, LatentMixer)
    register_model("test_scaled_capped_decoder", ScaledCappedDecoder)
    LAT = 24

    def norm(name):
        return RmsNormSpec(name, H, EPS)

    blocks = (PreNormBlockSpec(norm("layers.0.n1.weight"), LatentMixerSpec("layers.0.mix.", H, LAT), norm("layers.0.n2.weight"),
                               GatedMlpSpec("layers.0.mlp.", H, 56)),
              PreNormBlockSpec(norm("layers.1.n1.weight"),
                               AttentionSpec("layers.1.attn.", H, NQ, NKV, HD, 1.0 / math.sqrt(HD), EPS, POWER, None),
                               norm("layers.1.n2.weight"), GatedMlpSpec("layers.1.mlp.", H, 72)))
    spec = ModelSpec("ToyLatentForTests", V, H, blocks, (ScheduleEntry(0), ScheduleEntry(1)), norm("norm.weight"),
                     "embed.weight", None, 4096, kind="test_scaled_capped_decoder")
    model = build_model(spec)
    assert type(model) is ScaledCappedDecoder
    # two groups of pages: one array of [1, LAT] per token, and keys and values of [NKV, HD]
    assert [n.arrays() for n in model.cache_needs] == [((1, LAT),), ((NKV, HD), (NKV, HD))]
    w = random_tensors(model.weight_decls(), 13, sigma=0.25, dtype=torch.float32)
    model.load(w, torch.float32, DEV)
    runner = ModelRunner(model, 8, 20, 3, device=DEV)
    assert [len(g.arrays) for g in runner.cache.groups] == [1, 2]
    assert runner.cache.bytes_per_token() == (LAT + 2 * NKV * HD) * 4

    def plain_model(tokens):
        wd = {k: v.double() for k, v in w.items()}
        T = len(tokens)
        x = wd["embed.weight"][torch.tensor(tokens)] * ScaledCappedDecoder.MULT
        h = plain.rms_norm(x, wd["layers.0.n1.weight"], EPS)
        c, q = h @ wd["layers.0.mix.wc.weight"].T, h @ wd["layers.0.mix.wq.weight"].T
        sc = (q @ c.T / math.sqrt(LAT)).masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        x = x + (torch.softmax(sc, dim=-1) @ c) @ wd["layers.0.mix.wo.weight"].T
        x = x + plain.swiglu_mlp(plain.rms_norm(x, wd["layers.0.n2.weight"], EPS), wd, "layers.0.mlp.")
        p = "layers.1."
        h = plain.rms_norm(x, wd[p + "n1.weight"], EPS)
        qq = plain.rms_norm((h @ wd[p + "attn.q_proj.weight"].T).view(T, NQ, HD), wd[p + "attn.q_norm.weight"], EPS)
        kk = plain.rms_norm((h @ wd[p + "attn.k_proj.weight"].T).view(T, NKV, HD), wd[p + "attn.k_norm.weight"], EPS)
        vv = (h @ wd[p + "attn.v_proj.weight"].T).view(T, NKV, HD)
        pos = torch.arange(T)
        o = plain.causal_attention(plain_power_law_rotation(qq, pos, POWER), plain_power_law_rotation(kk, pos, POWER), vv,
                                   1.0 / math.sqrt(HD), None)
        x = x + o.reshape(T, NQ * HD) @ wd[p + "attn.o_proj.weight"].T
        x = x + plain.swiglu_mlp(plain.rms_norm(x, wd[p + "n2.weight"], EPS), wd, p + "mlp.")
        lg = plain.rms_norm(x, wd["norm.weight"], EPS) @ wd["embed.weight"].T
        return torch.tanh(lg / ScaledCappedDecoder.CAP) * ScaledCappedDecoder.CAP

    g = torch.Generator().manual_seed(4)
    a = torch.randint(0, V, (50,), generator=g).tolist()
    b = torch.randint(0, V, (31,), generator=g).tolist()
    want_a, want_b = plain_model(a), plain_model(b)
    got_a = [runner.step([StepEntry("a", a[:19], range(19))]).clone()]
    lg = runner.step([StepEntry("b", b[:9], range(9)), StepEntry("a", a[19:20], (0,))]).clone()
    got_b = [lg[:9]]
    got_a.append(lg[9:])
    at_a, at_b = 20, 9
    while at_a < len(a) or at_b < len(b):
        entries = []
        na, nb = min(7, len(a) - at_a), min(1, len(b) - at_b)
        if na:
            entries.append(StepEntry("a", a[at_a:at_a + na], range(na)))
        if nb:
            entries.append(StepEntry("b", b[at_b:at_b + 1], (0,)))
        lg = runner.step(entries).clone()
        if na:
            got_a.append(lg[:na]); lg = lg[na:]; at_a += na
        if nb:
            got_b.append(lg); at_b += 1
    for got, want in ((got_a, want_a), (got_b, want_b)):
        err = (torch.cat(got).double().cpu() - want).abs().max(dim=1).values
        tol = 2e-5 * want.abs().max().item()
        assert err.max().item() < tol, f"first wrong position {int((err >= tol).nonzero()[0])}: {err.max().item()}"
    runner.end_request("a")
    runner.end_request("b")
    runner.cache.check()
    assert runner.cache.free_pages() == runner.cache.total_pages()
