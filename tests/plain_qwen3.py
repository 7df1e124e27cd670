"""Plain, slow statement of the Qwen3 dense forward pass, whole sequences, no cache.

This file is the oracle that the engine's tests compare against.  It shares no
code with the package: it reads ``config.json`` as a plain dict, reads the
weights with the ``safetensors`` library, and computes every part with
elementary tensor arithmetic in float64 (or float32 on request).

It rests on the formulas of cklxx/arle's Qwen3 path, not on running that code:
the reference model is Rust driving CUDA kernels (no Rust toolchain and no GPU
where these tests are written; its CPU backend returns canned text), so it can
be neither imported nor compiled on the CPU.  Each function cites the reference
file and lines that give its formula.  Two independent statements of the same
layer in the reference were cross-read: the inference kernels and the f32
training model in ``crates/train/src/qwen3.rs:90-157``.

One extension beyond the reference: a per-layer key window (``sliding_window``
config keys, which the reference ignores).  A query at position p then sees keys
j with p - window < j <= p.
"""
from __future__ import annotations

import json
import math
import os

import torch

DT = torch.float64


# --------------------------------------------------------------------------- io
def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def read_weights(model_dir: str, dtype=DT) -> dict:
    from safetensors.torch import load_file

    raw = load_file(os.path.join(model_dir, "model.safetensors"))
    return {k: v.to(dtype) for k, v in raw.items()}


def layer_windows(cfg: dict) -> list:
    """Per-layer key window (None = all keys) from the config.json keys
    ``layer_types`` / ``use_sliding_window`` / ``sliding_window`` /
    ``max_window_layers``.  The reference ignores these keys
    (crates/qwen3-spec/src/lib.rs:95-108 lists the fields it reads)."""
    n = cfg["num_hidden_layers"]
    types = cfg.get("layer_types")
    win = cfg.get("sliding_window")
    if types is None:
        use = bool(cfg.get("use_sliding_window", False)) and win is not None
        first = cfg.get("max_window_layers", n)
        types = ["sliding_attention" if (use and i >= first) else "full_attention" for i in range(n)]
    return [win if t == "sliding_attention" else None for t in types]


# ------------------------------------------------------------------------ parts
def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """x0[t,:] = E[id_t,:], a pure gather without scale.
    infer/src/model/common.rs:64-80;
    crates/cuda-kernels/csrc/misc/elementwise_basic.cu:186-209."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """n_i = x_i / sqrt(mean(x^2) + eps) * w_i over the last axis; plain weight
    (no 1 + w).  crates/cuda-kernels/csrc/misc/norm.cu:221-300 (sum :234-262,
    inverse :266, product :281-285); the same kernel body serves the per-head
    q/k norm in csrc/attention/prefill_attention_paged_prep.cu:33-58."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(ms + eps) * w


def rope_inv_freq(rotary_dim: int, theta: float) -> torch.Tensor:
    """inv_freq_i = theta^(-2i/rotary_dim), i < rotary_dim/2.
    infer/src/weight_loader.rs:963-965."""
    i = torch.arange(rotary_dim // 2, dtype=DT)
    return theta ** (-2.0 * i / rotary_dim)


def rope_half_split(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Half-split rotation of whole heads.  x: [T, heads, hd]; pairs (i, i+hd/2):
    out_i = x_i cos - x_{i+hd/2} sin ; out_{i+hd/2} = x_i sin + x_{i+hd/2} cos,
    angle = position * inv_freq_i.
    infer/src/weight_loader.rs:955-989 (table);
    crates/cuda-kernels/csrc/attention/prefill_attention_paged_prep.cu:60-78."""
    hd = x.shape[-1]
    half = hd // 2
    ang = positions.to(DT)[:, None] * rope_inv_freq(hd, theta)[None, :]  # [T, half]
    cos = torch.cos(ang)[:, None, :].to(x.dtype)
    sin = torch.sin(ang)[:, None, :].to(x.dtype)
    lo, hi = x[..., :half], x[..., half:]
    return torch.cat([lo * cos - hi * sin, lo * sin + hi * cos], dim=-1)


def _same(x):
    return x


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    """x rounded to bfloat16 (nearest even) and widened again.  Passed as ``rnd`` to the functions
    below it marks the places where a bfloat16 engine stores an activation in 16 bits (outputs
    of norms, projections, the gate and attention, and the attention probabilities before P.V,
    crates/cuda-kernels/tools/tilelang/batch_prefill_paged_hd128.py:213-232), so that the
    size of bfloat16 rounding at a given width can be measured instead of guessed.  The
    residual stays unrounded, as in the engine."""
    return x.to(torch.bfloat16).to(x.dtype)


def causal_attention(q, k, v, scale: float, window=None, rnd=_same) -> torch.Tensor:
    """q: [T, nq, hd]; k, v: [T, nkv, hd]; query head h reads kv head h // (nq/nkv).
    s_tj = (q_t . k_j) * scale, keys j <= t (and j > t - window when a window is
    given), softmax over j, o_t = sum_j p_tj v_j.
    crates/cuda-kernels/tools/tilelang/batch_prefill_paged_hd128.py:46 (kv head),
    :103 (scale applied in the exponent), :170-232 (mask, online softmax, P.V);
    infer/src/ops/attention.rs:636 (scale = 1/sqrt(head_dim))."""
    T, nq, hd = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    out = torch.empty_like(q)
    t_idx = torch.arange(T)
    mask = t_idx[None, :] <= t_idx[:, None]
    if window is not None:
        mask &= t_idx[None, :] > (t_idx[:, None] - window)
    for h in range(nq):
        s = (q[:, h, :] @ k[:, h // g, :].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        if rnd is not _same:
            # the kernels round the unnormalised exp(s - max) and divide by the unrounded sum afterwards
            e = torch.exp(s - s.max(dim=-1, keepdim=True).values)
            out[:, h, :] = (rnd(e) @ v[:, h // g, :]) / e.sum(dim=-1, keepdim=True)
        else:
            out[:, h, :] = p @ v[:, h // g, :]
    return out


def attention_mixer(x, w: dict, pre: str, cfg: dict, positions, window=None, shared_kv=None, rnd=_same):
    """q/k/v projections without bias, per-head RMSNorm of q and k (one weight of
    head_dim shared by all heads, the layer's eps), rotation after the norm, V
    untouched, causal attention, output projection.  Returns the output and the
    (k, v) it attended over; with ``shared_kv`` it computes only q and attends
    over the given keys and values.
    infer/src/model/qwen3/prefill.rs:652-654 (projections), :674 (eps), :718-722
    (o_proj); crates/train/src/qwen3.rs:90-140."""
    T = x.shape[0]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q = rnd(x @ w[pre + "q_proj.weight"].T).view(T, nq, hd)
    q = rms_norm(q, w[pre + "q_norm.weight"], cfg["rms_norm_eps"])
    q = rnd(rope_half_split(q, positions, cfg["rope_theta"]))
    if shared_kv is None:
        k = rnd(x @ w[pre + "k_proj.weight"].T).view(T, nkv, hd)
        v = rnd(x @ w[pre + "v_proj.weight"].T).view(T, nkv, hd)
        k = rms_norm(k, w[pre + "k_norm.weight"], cfg["rms_norm_eps"])
        k = rnd(rope_half_split(k, positions, cfg["rope_theta"]))
    else:
        k, v = shared_kv
    o = rnd(causal_attention(q, k, v, 1.0 / math.sqrt(hd), window, rnd))
    return rnd(o.reshape(T, nq * hd) @ w[pre + "o_proj.weight"].T), (k, v)


def swiglu_mlp(x, w: dict, pre: str, rnd=_same) -> torch.Tensor:
    """d = (silu(x Wg^T) * (x Wu^T)) Wd^T, silu(g) = g / (1 + exp(-g)); no bias.
    infer/src/model/qwen3/prefill.rs:291-337;
    crates/cuda-kernels/csrc/misc/elementwise_basic.cu:18-24."""
    g = rnd(x @ w[pre + "gate_proj.weight"].T)
    u = rnd(x @ w[pre + "up_proj.weight"].T)
    return rnd(rnd(g / (1.0 + torch.exp(-g)) * u) @ w[pre + "down_proj.weight"].T)


def decoder_block(x, w: dict, layer: int, cfg: dict, positions, window=None, shared_kv=None, rnd=_same):
    """Pre-norm block: x1 = x + attn(norm(x)); x2 = x1 + mlp(norm(x1)).  Returns
    x2 and the block's (k, v).
    infer/src/model/qwen3/prefill.rs:618-776 (norm :644, add :737, norm :746,
    add :766)."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    h = rnd(rms_norm(x, w[p + "input_layernorm.weight"], eps))
    a, kv = attention_mixer(h, w, p + "self_attn.", cfg, positions, window, shared_kv, rnd)
    x = x + a
    h = rnd(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps))
    return x + swiglu_mlp(h, w, p + "mlp.", rnd), kv


def output_logits(x, w: dict, cfg: dict, rnd=_same) -> torch.Tensor:
    """Final RMSNorm then projection with lm_head.weight, or with the embedding
    table when tie_word_embeddings; no bias and no scaling of the logits.
    infer/src/model/qwen3/prefill.rs:426-455; infer/src/model/qwen3/weights.rs:305-316."""
    f = rnd(rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]))
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return f @ head.T


def forward(w: dict, cfg: dict, tokens, schedule=None, rnd=_same) -> torch.Tensor:
    """Logits [T, vocab] for one whole sequence starting at position 0.

    ``schedule`` lists the layers in running order as (layer, keys_of) pairs:
    ``keys_of`` is None when the entry computes its own keys and values, or the
    index of an earlier entry whose keys and values it attends over instead.
    The default runs layers 0..L-1 once each.  Only the default is a Qwen3
    model; other lists exist for the tests of the engine's layer schedule.
    ``rnd=bf16_round`` rounds every stored activation to bfloat16 (see there)."""
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(ids.numel())
    x = embedding(w["model.embed_tokens.weight"], ids)
    wins = layer_windows(cfg)
    order = schedule if schedule is not None else [(i, None) for i in range(cfg["num_hidden_layers"])]
    kvs = []
    for layer, keys_of in order:
        shared = kvs[keys_of] if keys_of is not None else None
        x, kv = decoder_block(x, w, layer, cfg, positions, wins[layer], shared, rnd)
        kvs.append(kv)
    return output_logits(x, w, cfg, rnd)


# --------------------------------------------------------------------- sampling
def greedy(logits: torch.Tensor) -> int:
    """Index of the largest logit; ties go to the lowest index.
    crates/cuda-kernels/csrc/misc/sampling.cu:16-26, :208-215."""
    best, idx = None, 0
    for i, val in enumerate(logits.tolist()):
        if best is None or val > best:
            best, idx = val, i
    return idx


def sampling_distribution(logits: torch.Tensor, temperature: float, top_k: int = -1,
                          top_p: float = 1.0) -> torch.Tensor:
    """p = softmax(logits / T); keep the top_k most probable (top_k <= 0: all) and
    renormalise; then keep the most probable tokens whose mass first reaches
    top_p and renormalise.  crates/cuda-kernels/csrc/misc/sampling.cu:327-594
    (the reference finds both thresholds by 32 bisection steps; this is the
    exact set it converges to when no two probabilities tie at the threshold)."""
    p = torch.softmax(logits.to(DT) / temperature, dim=-1)
    if 0 < top_k < p.numel():
        kth = torch.sort(p, descending=True).values[top_k - 1]
        p = torch.where(p >= kth, p, torch.zeros_like(p))
        p = p / p.sum()
    if top_p < 1.0:
        sp, order = torch.sort(p, descending=True)
        csum = torch.cumsum(sp, 0)
        keep_n = int((csum < top_p).sum().item()) + 1
        thr = sp[min(keep_n, sp.numel()) - 1]
        p = torch.where(p >= thr, p, torch.zeros_like(p))
        p = p / p.sum()
    return p


def sample_from(p: torch.Tensor, u: float) -> int:
    """First index whose cumulative probability exceeds u, in index order; the
    last index with non-zero probability if rounding leaves none.
    crates/cuda-kernels/csrc/misc/sampling.cu:569-593."""
    c = 0.0
    last = 0
    for i, val in enumerate(p.tolist()):
        if val > 0.0:
            last = i
        c += val
        if u < c:
            return i
    return last


def generate_greedy(w: dict, cfg: dict, prompt, steps: int) -> list:
    """Greedy continuation by re-running the whole sequence at every step."""
    toks = list(prompt)
    out = []
    for _ in range(steps):
        nxt = greedy(forward(w, cfg, toks)[-1])
        out.append(nxt)
        toks.append(nxt)
    return out
