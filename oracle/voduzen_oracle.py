"""Plain, slow restatement of the Voduzen decoder: one function per mechanism, whole sequences only, no cache, no batching.

Test infrastructure: the product never imports this file. Everything runs on the CPU in one floating-point type (float64 by
default) with keys and values materialised per head, which is the opposite of what the product does (latent cache, absorbed
projections, packed batches), so the two share neither code nor structure.

Notation. A layer updates the residual stream x as x <- x + N1(mixer(x)); x <- x + N2(ff(x)) with N(y) = y / rms(y) * (1 + g):
the norm sits on the sublayer's OUTPUT and the sublayers read x itself. rms(y) = sqrt(mean(y^2) + eps).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


def rms_unit(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def norm_zero_centred(y, g, eps):
    """Weight stored around zero: y / rms(y) * (1 + g)."""
    return rms_unit(y, eps) * (1.0 + g)


def norm_plain(y, g, eps):
    return rms_unit(y, eps) * g


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_angles(rot: dict, n_pos: int):
    """(cos, sin) [n_pos, dims/2] for pair index i: a = p * f_i, f_i = base^(-2i/dims); with `scaling` the frequencies are
    blended between f_i and f_i / factor by a linear ramp over the pair index and both tables are multiplied by
    0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=DT)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def corr(t):
            return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo = max(math.floor(corr(float(sc["fast"]))), 0)
        hi = min(math.ceil(corr(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    ang = torch.arange(n_pos, dtype=DT)[:, None] * f[None, :]
    return ang.cos() * mult, ang.sin() * mult


def rotate_interleaved(v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """v [T, ..., D]; the first 2 * cos.shape[1] dims are rotated pairwise (2i, 2i + 1), the rest pass unchanged.
    cos / sin [T, dims/2] are broadcast over the middle axes."""
    n = cos.shape[1] * 2
    out = v.clone()
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [n // 2]
    c, s = cos.reshape(shape), sin.reshape(shape)
    a, b = v[..., 0:n:2], v[..., 1:n:2]
    out[..., 0:n:2] = a * c - b * s
    out[..., 1:n:2] = b * c + a * s
    return out


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, p: str) -> torch.Tensor:
    """Both latent-attention mixers. Present tensors / keys decide the branches: '.dq' -> queries through a normed latent;
    '.sink' -> one extra term exp(sink_h) in the softmax denominator; rot['scaling'] -> blended frequencies."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    if p + "dq" in w:
        cq = norm_plain(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
        q = cq @ w[p + "uq"].T
    else:
        q = h @ w[p + "q"].T
    q = q.view(T, H, dn + dr)
    dkv = h @ w[p + "dkv"].T
    c = norm_plain(dkv[:, :r], w[p + "dkv.norm"], eps)
    k_rot = dkv[:, r:]                                       # [T, dr], shared by the heads
    cos, sin = rotary_angles(m["rot"], T)
    q_n, q_r = q[..., :dn], rotate_interleaved(q[..., dn:].contiguous(), cos, sin)
    k_r = rotate_interleaved(k_rot.contiguous(), cos, sin)
    k_n = (c @ w[p + "uk"].T).view(T, H, dn)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q_n, k_n) + torch.einsum("ihd,jd->hij", q_r, k_r)) * m["scale"]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    if p + "sink" in w:
        sink = w[p + "sink"].view(H, 1, 1).expand(H, T, 1)
        full = torch.cat([s, sink], dim=-1)
        pr = torch.softmax(full, dim=-1)[..., :T]           # the sink takes probability and gives nothing back
    else:
        pr = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", pr, v).reshape(T, H * dv)
    return o @ w[p + "o"].T


def router_choice(h, w, spec, p):
    """-> (ids [T, top], weights [T, top]) over experts + identity outputs: softmax scores s, choice by s + correction,
    weights = s of the chosen, not renormalised."""
    z = h @ w[p + "router"].T
    s = torch.softmax(z, dim=-1)
    ch = s + w[p + "correction"] if p + "correction" in w else s
    ids = torch.topk(ch, spec["router"]["top"], dim=-1).indices
    return ids, torch.gather(s, 1, ids)


def expert_ff(h, up, down):
    return (torch.relu(h @ up.T) ** 2) @ down.T


def moe_ff(h, w, spec, p):
    E = spec["router"]["experts"]
    ids, wt = router_choice(h, w, spec, p)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), wt[t]):
            if e >= E:                                       # identity expert: the input itself
                out[t] += a * h[t]
            else:
                out[t] += a * expert_ff(h[t], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
    if spec.get("shared"):
        g = torch.sigmoid(h @ w[p + "shared.sg"].T)         # [T, 1]
        out = out + g * expert_ff(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], collect: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; `collect` receives the residual stream after every layer."""
    w = {k: v.to(DT) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens)] * float(cfg["embedding"]["scale"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] not in ("latent_attention", "latent_attention_2"):
            raise ValueError(layer["type"])
        y = latent_attention(x, w, layer["mixer"], eps, p + "mix.")
        x = x + norm_zero_centred(y, w[p + "norm1"], eps)
        if layer.get("mlp"):
            y = moe_ff(x, w, layer["mlp"], p + "mlp.")
            x = x + norm_zero_centred(y, w[p + "norm2"], eps)
        if collect is not None:
            collect.append(x.clone())
    x = norm_zero_centred(x, w["final.norm"], eps)
    return (x @ w["head"].T) * float(cfg.get("logit_scale", 1.0))
