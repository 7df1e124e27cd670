"""The assembled engine at the layer sizes the benchmark times, against the plain model: two
layers of Qwen3-8B's widths (hidden 4096, 32 query and 8 kv heads of 128, feed-forward 12288)
and of Qwen3-0.6B's (hidden 1024, 16 and 8 heads of 128, so that the query width differs from
the hidden width; feed-forward 3072; tied output), with the vocabulary cut to a few thousand
entries (no power of two) and pages of 16.  At these widths the bfloat16 engine runs the
gated weight-streaming product, the streaming decode attention with four (two) query heads per
kv head and the tensor-core prefill with 32 (16) heads; the tiny models reach none of these
shapes.  All four cuttings, float32 and bfloat16."""
import pytest
import torch

import plain_qwen3 as plain
import traces
from arle_b200.engine import ModelRunner, load_model, random_model
from arle_b200.weights import write_random_model

pytestmark = pytest.mark.gpu

WIDE = {
    "8b": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=4096, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=3001, rope_theta=1000000.0,
               rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096, hidden_act="silu",
               bos_token_id=0, eos_token_id=1),
    "0.6b": dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=1024, num_attention_heads=16,
                 num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=2999, rope_theta=1000000.0,
                 rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096, hidden_act="silu",
                 bos_token_id=0, eos_token_id=1),
}
LENGTHS = [3, 70, 150, 40, 97]
# Logits here have a spread of about 1.3, like the tiny models', but every sum is 4,096 to 12,288
# terms long instead of 64 to 416, and float32 rounding of a sum grows with the square root of its
# length (a factor of 5 to 8): the float32 bound is 1e-4 of the spread of the logits.  What
# bfloat16 storage of the activations costs at these widths is measured, not guessed: the plain
# model is run once more with every stored activation rounded to bfloat16 (``plain.bf16_round``),
# and the engine may be one and a half times as far from the exact logits as that run is at its
# worst (measured: 1.0 to 1.2 times).
REL_F32 = 1e-4

_made = {}


def setup(size, tmp_path_factory):
    if size not in _made:
        d = str(tmp_path_factory.mktemp(f"wide{size}"))
        write_random_model(d, WIDE[size], seed=3, sigma=0.02, gain_jitter=0.1, device="cuda")
        cfg, w = plain.read_config(d), plain.read_weights(d)
        reqs = traces.make_requests(cfg["vocab_size"], LENGTHS, seed=6)
        oracle = {r: plain.forward(w, cfg, t) for r, t in reqs.items()}
        rounded = max((plain.forward(w, cfg, t, rnd=plain.bf16_round) - oracle[r]).abs().max().item() for r, t in reqs.items())
        del w
        _made[size] = (d, reqs, oracle, rounded)
    return _made[size]


@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("size", ["8b", "0.6b"])
def test_cuttings_at_benchmark_widths(size, dtype, cut, tmp_path_factory):
    d, reqs, oracle, rounded = setup(size, tmp_path_factory)
    steps = traces.mixed(reqs, seed=5) if cut == "mixed" else getattr(traces, cut)(reqs)
    model = load_model(d, dtype, "cuda")
    runner = ModelRunner(model, 16, traces.peak_tokens(steps) // 16, 4)
    got = traces.run_trace(runner, steps)
    runner.cache.check()
    assert runner.cache.free_pages() == runner.cache.total_pages()
    from arle_b200 import ops
    ops.check_errors("cuda")
    for r, want in oracle.items():
        err = (got[r].double() - want).abs().max(dim=1).values
        tol = REL_F32 * float(want.std()) if dtype == torch.float32 else 1.5 * rounded
        bad = (err > tol).nonzero()
        assert bad.numel() == 0, (f"{size} {cut} {dtype}: request {r} first wrong position {int(bad[0])} of {len(reqs[r])}, "
                                  f"error {err.max().item():.3g} (allowed {tol:.3g}; logits spread {float(want.std()):.3g})")


def test_random_model_on_the_device_is_the_model_the_folder_holds(tmp_path_factory):
    """The same configuration and seed give the same weights whether they are made on the GPU
    (the benchmark's way) or written to a folder and loaded."""
    d = setup("0.6b", tmp_path_factory)[0]
    a = load_model(d, torch.bfloat16, "cuda")
    b = random_model(WIDE["0.6b"], 3, torch.bfloat16, "cuda", sigma=0.02, gain_jitter=0.1)
    assert torch.equal(a.embed, b.embed)
    for x, y in zip(a.blocks, b.blocks):
        assert torch.equal(x.mixer.w_qkv, y.mixer.w_qkv) and torch.equal(x.mixer.w_o, y.mixer.w_o)
        assert torch.equal(x.mixer.q_norm, y.mixer.q_norm) and torch.equal(x.ffn.w_gate_up, y.ffn.w_gate_up)
        assert torch.equal(x.ffn.w_down, y.ffn.w_down) and torch.equal(x.mixer_norm.weight, y.mixer_norm.weight)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_a_far_token_decides_the_logits_at_8b_widths(dtype, tmp_path):
    """Random weights make attention nearly uniform, which hides a lost page or a wrong position.  Here the gain of
    layer 0's query norm is tripled, so that its attention is sharp, on two layers of Qwen3-8B's widths; a sequence of
    330 tokens is cut into portions and decoded tokens (tensor-core prefill, the streaming decode kernel with its
    own preparation, the gated weight-streaming product) and must agree with the plain model, whose late logits
    depend on single early tokens."""
    from arle_b200.engine import StepEntry
    from arle_b200.weights.safetensors_io import SafetensorsFile, write_safetensors

    d = str(tmp_path / "sharp8b")
    write_random_model(d, WIDE["8b"], seed=5, sigma=0.02, gain_jitter=0.1, device="cuda")
    path = d + "/model.safetensors"
    f = SafetensorsFile(path)
    t = {n: f.tensor(n).clone() for n in f.names()}
    name = "model.layers.0.self_attn.q_norm.weight"
    t[name] = (t[name].float() * 3).to(t[name].dtype)
    write_safetensors(path, t)
    del t, f
    cfg, w = plain.read_config(d), plain.read_weights(d)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, cfg["vocab_size"], (330,), generator=g).tolist()
    want = plain.forward(w, cfg, toks)
    moved = list(toks)
    moved[5] = (moved[5] + 1) % cfg["vocab_size"]
    assert (plain.forward(w, cfg, moved)[-1] - want[-1]).abs().max() > 1e-3      # the last logits see token 5
    tol = REL_F32 * float(want.std()) if dtype == torch.float32 else \
        1.5 * (plain.forward(w, cfg, toks, rnd=plain.bf16_round) - want).abs().max().item()
    del w
    runner = ModelRunner(load_model(d, dtype, "cuda"), 16, 48, 2)
    got, at = [], 0
    for n in (130, 1, 1, 64, 2, 99, 1, 1) + (1,) * 31:
        got.append(runner.step([StepEntry("r", toks[at:at + n], range(n))]).clone())
        at += n
    assert at == 330
    err = (torch.cat(got).double().cpu() - want).abs().max(dim=1).values
    bad = (err > tol).nonzero()
    assert bad.numel() == 0, f"first wrong position {int(bad[0])}: error {err.max().item():.3g}, allowed {tol:.3g}"
