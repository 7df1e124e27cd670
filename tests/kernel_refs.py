"""Plain torch statements of each CUDA kernel of the package, one function per
kernel with the kernel's own signature (see ``arle_b200/ops/__init__.py``).

Two uses: the GPU tests compare every kernel alone against its function here, at
sizes other than the engine's; and the CPU tests put these functions in the place
of the kernels (fixture ``cpu_kernels`` in conftest.py) so that everything around
the kernels (cache manager, block tables, step function, scheduler) runs and is
compared with the plain model without a GPU.  They are test code only: the
package itself has no CPU path.
"""
from __future__ import annotations

import math

import torch

F32 = torch.float32


def embedding(ids, table, out, err=None, last_token=None, slot_of_token=None):
    ids = ids.long()
    if last_token is not None:
        ids = torch.where(ids < 0, last_token[slot_of_token.long()].long(), ids)
    out.copy_(table[ids].to(F32))


def rmsnorm(resid, delta, rows, weight, eps, out, write_resid):
    idx = rows.long() if rows is not None else torch.arange(resid.shape[0], device=resid.device)
    x = resid[idx].to(F32)
    if delta is not None:
        x = x + delta[idx].to(F32)
    if write_resid:
        resid[idx] = x
    inv = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    out.copy_((x * inv * weight).to(out.dtype))


def residual_add(resid, delta):
    resid += delta.to(F32)


def gemm(x, w, out, sink=None):
    """``sink`` is never taken here (the parts are told so by ``fused_gemm_shape_ok``): False."""
    out.copy_((x.to(F32) @ w.to(F32).t()).to(out.dtype))
    return False


def fused_gemm_shape_ok(rows, w, gated=False):
    return False


def fused_decode_supported(*args, **kwargs):
    return False


def attention_prep_takes_angles(*args, **kwargs):
    return False


def attention_prep(qkv, positions, slot_mapping, q_weight, k_weight, eps, inv_freq, rotary_dim, k_cache, v_cache,
                   nq, nkv, hd, page_size, angles=None):
    T = qkv.shape[0]
    heads = qkv[:, : (nq + 2 * nkv) * hd].view(T, nq + 2 * nkv, hd)

    def norm_rope(x, w):
        x = x.to(F32)
        if w is not None:
            x = x * (1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)) * w
        if rotary_dim:
            half = rotary_dim // 2
            ang = positions.to(F32)[:, None] * inv_freq[None, :]
            cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            lo, hi = x[..., :half], x[..., half:rotary_dim]
            x = torch.cat([lo * cos - hi * sin, lo * sin + hi * cos, x[..., rotary_dim:]], dim=-1)
        return x

    q = norm_rope(heads[:, :nq], q_weight)
    heads[:, :nq] = q.to(qkv.dtype)
    if nkv:
        k = norm_rope(heads[:, nq:nq + nkv], k_weight).to(qkv.dtype)
        v = heads[:, nq + nkv:]
        keep = slot_mapping >= 0
        page = (slot_mapping[keep] // page_size).long()
        off = (slot_mapping[keep] % page_size).long()
        k_cache[page, :, off] = k[keep]
        v_cache[page, :, off] = v[keep]


def paged_attention(q, out, k_cache, v_cache, positions, row_of_token, block_table, nq, nkv, hd, page_size, scale,
                    window, batch=None):
    T = q.shape[0]
    g = nq // nkv
    for t in range(T):
        p = int(positions[t])
        lo = max(0, p - window + 1) if window else 0
        js = torch.arange(lo, p + 1)
        pages = block_table[int(row_of_token[t]), js // page_size].long()
        offs = js % page_size
        k = k_cache[pages, :, offs].to(F32)          # [n, nkv, hd]
        v = v_cache[pages, :, offs].to(F32)
        qt = q[t].view(nq, hd).to(F32)
        for h in range(nq):
            s = (k[:, h // g] @ qt[h]) * scale
            pr = torch.softmax(s, dim=0)
            out[t, h * hd:(h + 1) * hd] = (pr @ v[:, h // g]).to(out.dtype)


def silu_mul(gate_up, out):
    g, u = gate_up[:, 0::2].to(F32), gate_up[:, 1::2].to(F32)          # rows 2i, 2i + 1 of the packed weight: gate_i, up_i
    out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))


def gemm_silu_mul(x, w, gate_up, out):
    gemm(x, w, gate_up)
    silu_mul(gate_up, out)


def argmax(logits, scratch, out, scatter=None, last_token=None):
    out[: logits.shape[0]] = torch.argmax(logits, dim=1).to(out.dtype)      # torch returns the first maximal index
    if scatter is not None:
        last_token[scatter[: logits.shape[0]].long()] = out[: logits.shape[0]]


def scatter_tokens(tokens, scatter, last_token):
    last_token[scatter.long()] = tokens[: scatter.numel()]


def sample(logits, temperature, top_k, top_p, min_p, uniform, scratch, out):
    R, V = logits.shape
    for r in range(R):
        x = logits[r].to(F32)
        t = float(temperature[r]) if temperature is not None else 0.0
        k = int(top_k[r]) if top_k is not None else -1
        if not t > 0 or k == 1:
            out[r] = int(torch.argmax(x))          # torch returns the first maximal index
            continue
        p = torch.softmax(x / t, dim=0)
        mp = float(min_p[r])
        if mp > 0:
            p = torch.where(p >= mp * p.max(), p, torch.zeros_like(p))
            p = p / p.sum()
        if 0 < k < V:
            kth = torch.sort(p, descending=True).values[k - 1]
            p = torch.where(p >= kth, p, torch.zeros_like(p))
            p = p / p.sum()
        tp = float(top_p[r])
        if tp < 1:
            sp = torch.sort(p, descending=True).values
            n = int((torch.cumsum(sp, 0) < tp).sum()) + 1
            thr = sp[min(n, V) - 1]
            p = torch.where(p >= thr, p, torch.zeros_like(p))
            p = p / p.sum()
        c = torch.cumsum(p, 0)
        target = float(uniform[r]) * float(c[-1])
        hit = torch.nonzero(c > target)
        out[r] = int(hit[0]) if hit.numel() else int(torch.nonzero(p > 0)[-1])


ALL = ("embedding", "rmsnorm", "residual_add", "gemm", "fused_gemm_shape_ok", "fused_decode_supported", "attention_prep_takes_angles", "attention_prep", "paged_attention", "silu_mul", "gemm_silu_mul", "argmax", "scatter_tokens", "sample")
