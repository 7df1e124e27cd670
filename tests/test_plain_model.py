"""The plain implementation checked against itself: properties any correct statement
of the formulas has, so that the oracle is not trusted blindly."""
import math

import pytest
import torch

import plain_qwen3 as plain
from arle_b200.sampling import SamplingParams
from tiny_models import make_model_dir


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    out = {}
    for name in ("A", "C"):
        d = make_model_dir(name, seed=2, root=str(tmp_path_factory.mktemp(f"plain{name}")))
        out[name] = (plain.read_config(d), plain.read_weights(d))
    return out


def test_rms_norm_closed_form():
    x = torch.tensor([[3.0, 4.0]], dtype=plain.DT)
    y = plain.rms_norm(x, torch.tensor([2.0, 0.5], dtype=plain.DT), 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]], dtype=plain.DT))


def test_rope_is_a_rotation_of_half_split_pairs_and_relative():
    x = torch.randn(5, 2, 8, dtype=plain.DT)
    pos = torch.tensor([0, 1, 7, 100, 4000])
    y = plain.rope_half_split(x, pos, 10000.0)
    assert torch.allclose(y[0], x[0])                                      # position 0: identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))                  # rotations keep lengths
    pair = lambda t, i: torch.stack([t[..., i], t[..., i + 4]], -1)
    assert torch.allclose(pair(y, 1).norm(dim=-1), pair(x, 1).norm(dim=-1))   # pairs (i, i + hd/2)
    q, k = torch.randn(1, 1, 8, dtype=plain.DT), torch.randn(1, 1, 8, dtype=plain.DT)
    dot = lambda a, b: (plain.rope_half_split(q, torch.tensor([a]), 1e4) * plain.rope_half_split(k, torch.tensor([b]), 1e4)).sum()
    assert torch.allclose(dot(10, 3), dot(107, 100))                        # scores depend on the distance only


def test_attention_is_causal_grouped_and_windowed():
    T, nq, nkv, hd = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n, hd, dtype=plain.DT) for n in (nq, nkv, nkv))
    out = plain.causal_attention(q, k, v, 0.3)
    k2, v2 = k.clone(), v.clone()
    k2[6:], v2[6:] = 0, 7
    assert torch.allclose(plain.causal_attention(q, k2, v2, 0.3)[:6], out[:6])      # later keys do not matter
    assert torch.allclose(out[0], v[0].repeat_interleave(2, dim=0))                 # first token sees itself only; head h -> kv head h // 2
    win = plain.causal_attention(q, k, v, 0.3, window=3)
    k3, v3 = k.clone(), v.clone()
    k3[:4], v3[:4] = 5, -5
    assert torch.allclose(plain.causal_attention(q, k3, v3, 0.3, window=3)[6:], win[6:])   # position 6 sees keys 4, 5, 6
    assert not torch.allclose(plain.causal_attention(q, k3, v3, 0.3, window=4)[6], win[6])


def test_whole_model_is_causal_and_windows_are_read_from_config(tiny):
    cfg, w = tiny["A"]
    a = [5, 9, 200, 31, 77, 12]
    b = a[:4] + [1, 2]
    la, lb = plain.forward(w, cfg, a), plain.forward(w, cfg, b)
    assert torch.allclose(la[:4], lb[:4]) and not torch.allclose(la[4], lb[4])
    cfg_c, w_c = tiny["C"]
    assert plain.layer_windows(cfg_c) == [None, None, 21, 21]
    toks = list(range(3, 60))
    full = plain.forward(w_c, dict(cfg_c, use_sliding_window=False), toks)
    wind = plain.forward(w_c, cfg_c, toks)
    assert torch.allclose(full[:21], wind[:21]) and not torch.allclose(full[40], wind[40])


def test_tied_output_uses_the_embedding_table(tiny):
    cfg, w = tiny["A"]
    assert cfg["tie_word_embeddings"] and "lm_head.weight" not in w
    x = torch.randn(2, cfg["hidden_size"], dtype=plain.DT)
    f = plain.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    assert torch.allclose(plain.output_logits(x, w, cfg), f @ w["model.embed_tokens.weight"].T)


def test_greedy_ties_and_sampling_filters():
    assert plain.greedy(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1
    lg = torch.tensor([2.0, 1.0, 0.0, -1.0, -2.0])
    p = plain.sampling_distribution(lg, 1.0)
    assert torch.allclose(p.sum(), torch.tensor(1.0, dtype=plain.DT)) and (p[:-1] > p[1:]).all()
    assert (plain.sampling_distribution(lg, 1.0, top_k=2) > 0).tolist() == [True, True, False, False, False]
    pp = plain.sampling_distribution(lg, 1.0, top_p=0.7)          # 0.636 + 0.234 >= 0.7: two tokens
    assert (pp > 0).tolist() == [True, True, False, False, False] and abs(pp.sum().item() - 1) < 1e-12
    cold = plain.sampling_distribution(lg, 0.05)
    assert cold[0] > 0.999
    assert plain.sample_from(p, 0.0) == 0 and plain.sample_from(p, 0.999999) == 4
    assert plain.sample_from(torch.tensor([0.5, 0.0, 0.5]), 0.5) == 2


def test_sampling_params_follow_the_reference_rules():
    assert SamplingParams().is_greedy() and SamplingParams(temperature=0.8, top_k=1).is_greedy()
    assert not SamplingParams(temperature=0.8).is_greedy() and not SamplingParams(top_p=0.9).is_greedy()
    with pytest.raises(ValueError):
        SamplingParams(repetition_penalty=1.1)
    with pytest.raises(ValueError):
        SamplingParams(top_p=0.0)
