"""Each part alone on the GPU against the plain model's function for it, the layer
schedule as data (a block named twice; a block that reads another's cache), the first
tokens of a sequence, a far key made to matter in the whole engine, and a toy mixer
with state of its own that is registered, built and stepped without touching the
package."""
import math
from dataclasses import dataclass
from typing import ClassVar

import pytest
import torch

import plain_qwen3 as plain
import traces
from arle_b200 import ops
from arle_b200.cache import CacheManager
from arle_b200.config import ModelSpec, ScheduleEntry, config_from_dict
from arle_b200.engine import ModelRunner, StepEntry, load_model
from arle_b200.engine.batch import StepContext, Workspace
from arle_b200.parts import (AttentionSpec, DecoderModel, GatedMlpSpec, Mixer, PreNormBlockSpec, ResidualStream,
                             RmsNormSpec, RotarySpec, StateNeed, WeightDecl, build_part, register_part)
from arle_b200.weights import SafetensorsFile, random_tensors, write_safetensors
from tiny_models import CONFIGS, PAGE_SIZES, make_model_dir

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 3e-5, torch.bfloat16: 3e-2}


def _ctx_for(cache, entries, starts):
    ws = Workspace(DEV)
    cache.append([(e.request, len(e.tokens)) for e in entries])
    return StepContext(cache, ws).build(entries, starts)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_norm_part_alone(dtype):
    part = build_part(RmsNormSpec("n.weight", 200, 1e-5))
    w = random_tensors(part.weight_decls(), 1, gain_jitter=0.3)
    part.load(w, dtype, DEV)
    x = torch.randn(9, 200, device=DEV)
    out = torch.empty(9, 200, dtype=dtype, device=DEV)
    part.apply(x.clone(), None, None, out, False)
    want = plain.rms_norm(x.double().cpu(), w["n.weight"].double(), 1e-5)
    assert (out.double().cpu() - want).abs().max() < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
def test_feed_forward_part_alone(dtype):
    spec = GatedMlpSpec("m.", 96, 176)
    part = build_part(spec)
    w = random_tensors(part.weight_decls(), 2, sigma=0.1)
    part.load(w, dtype, DEV)
    cm = CacheManager([], [], 16, 4, 2, 64, dtype, DEV)
    ctx = _ctx_for(cm, [], []) if False else type("C", (), {"ws": Workspace(DEV), "num_tokens": 7})()
    x = torch.randn(7, 96).to(dtype)
    out = part.forward(x.to(DEV), ctx)
    want = plain.swiglu_mlp(x.double(), {k: v.double() for k, v in w.items()}, "m.")
    assert (out.double().cpu() - want).abs().max() < TOL[dtype] * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("nq,nkv,hd,window", [(4, 2, 16, None), (6, 1, 32, 9), (4, 2, 64, None), (2, 1, 128, 40)])
def test_attention_part_alone_prefill_then_decode(dtype, nq, nkv, hd, window):
    H, ps, T = 72, 8, 50
    spec = AttentionSpec("a.", H, nq, nkv, hd, 1 / math.sqrt(hd), 1e-6, RotarySpec(hd, 1e4), window)
    part = build_part(spec)
    w = random_tensors(part.weight_decls(), 3, sigma=0.15, gain_jitter=0.2)
    part.load(w, dtype, DEV)
    cm = CacheManager([part.cache_need()], [], ps, 16, 2, 256, dtype, DEV)
    cm.add_request("r")
    x = torch.randn(T, H).to(dtype)
    cfg = dict(num_attention_heads=nq, num_key_value_heads=nkv, head_dim=hd, rms_norm_eps=1e-6, rope_theta=1e4)
    want, _ = plain.attention_mixer(x.double(), {k: v.double() for k, v in w.items()}, "a.", cfg, torch.arange(T), window)
    got = []
    at = 0
    for n in (37, 1, 1, 9, 1, 1):                    # a portion, decoded tokens, another portion, decoded tokens
        e = [StepEntry("r", list(range(n)), ())]
        ctx = _ctx_for(cm, e, [at])
        got.append(part.forward(x[at:at + n].to(DEV), ctx, ctx.cache_view(0), None).clone())
        at += n
    got = torch.cat(got).double().cpu()
    assert (got - want).abs().max() < TOL[dtype] * max(1.0, want.abs().max().item())


def _spec_with_schedule(cfg, schedule):
    base = config_from_dict(cfg).to_model_spec()
    return ModelSpec(**{**base.__dict__, "schedule": tuple(schedule)})


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("schedule", [[(0, None), (1, None), (0, None), (1, None)],     # blocks named twice
                                       [(0, None), (1, 0), (1, None), (0, 2)]],          # blocks that read another's cache
                         ids=["twice", "shared-cache"])
def test_layer_schedule_is_data(dtype, schedule, tmp_path):
    d = make_model_dir("A", seed=5, root=str(tmp_path))
    cfg, w = plain.read_config(d), plain.read_weights(d)
    toks = torch.randint(0, 256, (41,), generator=torch.Generator().manual_seed(1)).tolist()
    want = plain.forward(w, cfg, toks, schedule=schedule)
    spec = _spec_with_schedule(CONFIGS["A"], [ScheduleEntry(b, k) for b, k in schedule])
    model = DecoderModel(spec)
    f = SafetensorsFile(str(tmp_path / "A" / "model.safetensors"))
    model.load({n: f.tensor(n) for n in f.names()}, dtype, DEV)
    assert len(model.cache_needs) == sum(1 for _, k in schedule if k is None)
    runner = ModelRunner(model, 4, 64, 2, device=DEV)
    got = []
    for chunk in (toks[:17], toks[17:18], toks[18:40], toks[40:]):
        got.append(runner.step([StepEntry("r", chunk, range(len(chunk)))]).clone())
    err = (torch.cat(got).double().cpu() - want).abs().max().item()
    assert err < (2e-5 if dtype == torch.float32 else 4e-2)


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "D", "E"])
def test_first_tokens_of_a_sequence(name, dtype, tmp_path):
    d = make_model_dir(name, seed=8, root=str(tmp_path))
    cfg, w = plain.read_config(d), plain.read_weights(d)
    toks = [7, 7, 3, 250, 1]
    want = plain.forward(w, cfg, toks)
    runner = ModelRunner(load_model(d, dtype, DEV), PAGE_SIZES[name], 8, 2, device=DEV)
    one_by_one = torch.cat([runner.step([StepEntry("a", [t], (0,))]).clone() for t in toks])
    together = runner.step([StepEntry("b", toks, range(5))]).clone()
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    assert (one_by_one.double().cpu() - want).abs().max() < tol and (together.double().cpu() - want).abs().max() < tol


@pytest.mark.parametrize("dtype", DTYPES, ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["B", "D", "E", "F"])
def test_a_far_token_decides_the_logits(name, dtype, tmp_path):
    """Random weights make attention nearly uniform, which hides a lost page or a wrong
    position.  Here the q and k projections of layer 0 are scaled up so that attention
    is sharp, and the sequence is long enough to span many pages and several key tiles;
    the engine, cut into portions and decoded tokens, must still agree with the plain
    model, whose logits then depend strongly on single far tokens."""
    d = make_model_dir(name, seed=9, root=str(tmp_path))
    path = str(tmp_path / name / "model.safetensors")
    f = SafetensorsFile(path)
    t = {n: f.tensor(n).clone() for n in f.names()}
    for n in ("q_proj", "k_proj"):
        t[f"model.layers.0.self_attn.{n}.weight"] = (t[f"model.layers.0.self_attn.{n}.weight"].float() * 6).to(torch.bfloat16)
    t["model.layers.0.self_attn.q_norm.weight"] = (t["model.layers.0.self_attn.q_norm.weight"].float() * 3).to(torch.bfloat16)
    write_safetensors(path, t)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, cfg["vocab_size"], (330,), generator=g).tolist()
    want = plain.forward(w, cfg, toks)
    # the sharpened layer must really look far back: moving one early token changes late logits
    moved = list(toks)
    moved[5] = (moved[5] + 1) % cfg["vocab_size"]
    assert (plain.forward(w, cfg, moved)[-1] - want[-1]).abs().max() > 1e-3
    runner = ModelRunner(load_model(d, dtype, DEV), PAGE_SIZES[name], 48, 2, device=DEV)
    got, at = [], 0
    for n in (130, 1, 1, 64, 2, 99, 1, 1) + (1,) * 31:
        got.append(runner.step([StepEntry("r", toks[at:at + n], range(n))]).clone())
        at += n
    assert at == 330
    err = (torch.cat(got).double().cpu() - want).abs()
    tol = 5e-5 if dtype == torch.float32 else 8e-2
    assert err.max().item() < tol, f"first wrong position {int((err.max(dim=1).values > tol).nonzero()[0])}"


# ------------------------------------------------------------------ a toy mixer with state of its own
@dataclass(frozen=True)
class DecayMixerSpec:
    prefix: str
    hidden_size: int
    decay: float
    kind: ClassVar[str] = "test_decay_mixer"


class DecayMixer(Mixer):
    """s_t = decay * s_{t-1} + x_t W_in ; y_t = s_t W_out.  The state s lives in the
    per-request state slot; there is no paged cache.  Written with torch operations:
    it is a test of the framework's interfaces, not a kernel."""

    def __init__(self, spec):
        self.spec = spec

    def weight_decls(self):
        h = self.spec.hidden_size
        return (WeightDecl(self.spec.prefix + "in.weight", (h, h)), WeightDecl(self.spec.prefix + "out.weight", (h, h)))

    def load(self, tensors, dtype, device):
        self.w_in = tensors[self.spec.prefix + "in.weight"].to(device=device, dtype=torch.float32)
        self.w_out = tensors[self.spec.prefix + "out.weight"].to(device=device, dtype=torch.float32)

    def state_need(self):
        return StateNeed((self.spec.hidden_size,), torch.float32)

    def forward(self, x, ctx, cache, state):
        assert cache is None
        u = x.float() @ self.w_in.t()
        if ctx.max_q_len == 1:
            # one token a row: no loop over rows and nothing read back to the host, so that the step can be
            # captured in a CUDA graph
            slots = ctx.state_slots.long()
            s = self.spec.decay * state[slots] + u
            state.index_copy_(0, slots, s)
            return (s @ self.w_out.t()).to(x.dtype)
        out = torch.empty_like(u)
        at = 0
        for r, n in enumerate(ctx.q_lens):
            slot = int(ctx.state_slots[r])
            s = state[slot]
            for i in range(at, at + n):
                s = self.spec.decay * s + u[i]
                out[i] = s
            state[slot] = s
            at += n
        return (out @ self.w_out.t()).to(x.dtype)


def test_toy_mixer_with_state_registers_builds_and_steps():
    register_part(DecayMixerSpec.kind, DecayMixer)
    H, V = 32, 50
    blocks = []
    for i in range(2):
        p = f"layers.{i}."
        blocks.append(PreNormBlockSpec(RmsNormSpec(p + "n1.weight", H, 1e-6), DecayMixerSpec(p + "mix.", H, 0.9),
                                       RmsNormSpec(p + "n2.weight", H, 1e-6), GatedMlpSpec(p + "mlp.", H, 48)))
    spec = ModelSpec("ToyForTests", V, H, tuple(blocks), (ScheduleEntry(0), ScheduleEntry(1)),
                     RmsNormSpec("norm.weight", H, 1e-6), "embed.weight", None, 512)
    model = DecoderModel(spec)
    assert model.cache_needs == [] and len(model.state_needs) == 2
    w = random_tensors(model.weight_decls(), 4, sigma=0.2, dtype=torch.float32)
    model.load(w, torch.float32, DEV)
    runner = ModelRunner(model, 16, 4, 3, device=DEV)

    def plain_toy(tokens):
        wd = {k: v.double() for k, v in w.items()}
        x = wd["embed.weight"][torch.tensor(tokens)]
        for i in range(2):
            p = f"layers.{i}."
            h = plain.rms_norm(x, wd[p + "n1.weight"], 1e-6) @ wd[p + "mix.in.weight"].T
            s, ys = torch.zeros(H, dtype=torch.float64), []
            for t in range(len(tokens)):
                s = 0.9 * s + h[t]
                ys.append(s)
            x = x + torch.stack(ys) @ wd[p + "mix.out.weight"].T
            x = x + plain.swiglu_mlp(plain.rms_norm(x, wd[p + "n2.weight"], 1e-6), wd, p + "mlp.")
        return plain.rms_norm(x, wd["norm.weight"], 1e-6) @ wd["embed.weight"].T

    a, b = [3, 9, 1, 44, 7, 7, 12, 30, 2], [5, 6, 7, 8]
    got_a, got_b = [], []
    got_a.append(runner.step([StepEntry("a", a[:4], range(4))]).clone())
    lg = runner.step([StepEntry("a", a[4:5], (0,)), StepEntry("b", b[:3], range(3))]).clone()     # mixed step
    got_a.append(lg[:1]); got_b.append(lg[1:])
    lg = runner.step([StepEntry("b", b[3:], (0,)), StepEntry("a", a[5:], range(4))]).clone()
    got_b.append(lg[:1]); got_a.append(lg[1:])
    assert (torch.cat(got_a).double().cpu() - plain_toy(a)).abs().max() < 1e-4
    assert (torch.cat(got_b).double().cpu() - plain_toy(b)).abs().max() < 1e-4
    runner.end_request("a")
    got_c = runner.step([StepEntry("c", a, range(len(a)))]).clone()       # takes a's slot: the state starts at zero again
    assert (got_c.double().cpu() - plain_toy(a)).abs().max() < 1e-4
    runner.end_request("b")
    runner.end_request("c")
    # decode steps as CUDA graphs: the step in which a graph is captured must advance the state once, not twice
    runner.enable_graphs()
    seqs = {"d": [int(t) for t in torch.randint(0, V, (30,), generator=torch.Generator().manual_seed(1))],
            "e": [int(t) for t in torch.randint(0, V, (26,), generator=torch.Generator().manual_seed(2))]}
    got = {r: [runner.step([StepEntry(r, t[:6], range(6))]).clone()] for r, t in seqs.items()}
    for i in range(6, 30):
        rows = [r for r, t in seqs.items() if i < len(t)]
        lg = runner.step([StepEntry(r, seqs[r][i:i + 1], (0,)) for r in rows]).clone()
        for k, r in enumerate(rows):
            got[r].append(lg[k:k + 1])
    assert runner.graph_steps == 24 and len(runner._graphs) == 2          # graphs of two rows and of one row
    for r, t in seqs.items():
        assert (torch.cat(got[r]).double().cpu() - plain_toy(t)).abs().max() < 1e-4
