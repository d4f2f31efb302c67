"""Plain, slow restatement of the Tifisun decoder: one function per mechanism, whole sequences only, token-by-token loops.

Test infrastructure: the product never imports this file. Everything runs on the CPU in float64; recurrences are written as the
literal per-token update, attention materialises the whole score matrix, convolutions loop over taps. The product does the
opposite (packed steps, paged keys, state slots, fused kernels), so the two share neither code nor structure.

Notation. x is the residual stream [T, C]. A layer with residual factor m:
    x <- x + m * Nb1(mixer(Na1(x)));   x <- x + m * Nb2(ff(Na2(x)))       N(y) = y / sqrt(mean(y^2) + eps) * (1 + g)
Mixers: 'delta' (gated delta rule, one decay per head), 'channel_delta' (one decay per head and key channel, low-rank decay and
gate projections), 'parallel' (windowed soft-capped attention with a bucketed distance bias beside a constant-decay linear
attention, averaged after a norm each).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


def unit_rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def norm_zero_centred(y, g, eps):
    return unit_rms(y, eps) * (1.0 + g)


def norm_plain(y, g, eps):
    return unit_rms(y, eps) * g


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + z.clamp(min=0.0)


def causal_conv(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, ch], w [ch, taps]; the last tap multiplies the current token, earlier taps the tokens before it, zeros before
    the sequence starts."""
    T, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1 - j)
            if s >= 0:
                y[t] += w[:, j] * x[s]
    return y


def unit_vectors(x: torch.Tensor, heads: int) -> torch.Tensor:
    """[T, heads * d] -> every head's slice divided by sqrt(sum of squares + 1e-6)."""
    T = x.shape[0]
    xh = x.view(T, heads, -1)
    return (xh / torch.sqrt((xh * xh).sum(-1, keepdim=True) + 1e-6)).reshape(T, -1)


def delta_rule(q, k, v, g, beta):
    """One head. q, k [T, d]; v [T, dv]; g [T, d] (decay of every key channel; a per-head decay is a constant row); beta [T].
    S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t."""
    T, d = q.shape
    S = torch.zeros(d, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.T @ q[t])
    return torch.stack(out)


def decayed_outer_sum(q, k, v, decay: float):
    """One head of constant-decay linear attention: S <- decay * S + k_t v_t^T; o_t = S^T q_t."""
    S = torch.zeros(q.shape[1], v.shape[1], dtype=q.dtype)
    out = []
    for t in range(q.shape[0]):
        S = decay * S + torch.outer(k[t], v[t])
        out.append(S.T @ q[t])
    return torch.stack(out)


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Distances below rows/2 have a row each; larger ones share logarithmically spaced rows up to `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def windowed_attention(q, k, v, heads, kv_heads, scale, softcap, rel, far, window):
    """q [T, heads * d], k [T, kv_heads * d], v [T, kv_heads * dv], rel [rows, heads]. Position i sees j with 0 <= i - j < window."""
    T = q.shape[0]
    d, dv = q.shape[1] // heads, v.shape[1] // kv_heads
    rep = heads // kv_heads
    out = torch.zeros(T, heads * dv, dtype=q.dtype)
    for h in range(heads):
        qh = q[:, h * d:(h + 1) * d]
        kh = k[:, (h // rep) * d:(h // rep + 1) * d]
        vh = v[:, (h // rep) * dv:(h // rep + 1) * dv]
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (kh[lo:i + 1] @ qh[i]) * scale
            s = softcap * torch.tanh(s / softcap)
            s = s + torch.stack([rel[distance_bucket(i - j, rel.shape[0], far), h] for j in range(lo, i + 1)])
            p = torch.softmax(s, dim=0)
            out[i, h * dv:(h + 1) * dv] = p @ vh[lo:i + 1]
    return out


# --------------------------------------------------------------------------------------------------------------------- mixers
def mixer_delta(h, P: Dict[str, torch.Tensor], m: dict, eps: float, per_channel: bool):
    """P: this layer's 'mix.*' tensors by their short names."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ P["q"].T, P["q.conv"]))
    k = silu(causal_conv(h @ P["k"].T, P["k.conv"]))
    v = silu(causal_conv(h @ P["v"].T, P["v.conv"]))
    q = unit_vectors(q, G) * d ** -0.5
    k = unit_vectors(k, G)
    beta = torch.sigmoid(h @ P["b"].T)                                    # [T, H]
    if per_channel:
        a = (h @ P["a1"].T) @ P["a2"].T                                     # [T, H * d]
        g = torch.exp(-torch.exp(P["A_log"])[None, :, None] * softplus(a + P["dt_bias"]).view(T, H, d))
        gate = torch.sigmoid((h @ P["g1"].T) @ P["g2"].T)
    else:
        a = h @ P["a"].T                                                    # [T, H]
        g = torch.exp(-torch.exp(P["A_log"]) * softplus(a + P["dt_bias"]))[:, :, None].expand(T, H, d)
        gate = silu(h @ P["g"].T)
    rep = H // G
    outs = []
    for hh in range(H):
        kv = hh // rep
        o = delta_rule(q[:, kv * d:(kv + 1) * d], k[:, kv * d:(kv + 1) * d], v[:, hh * dv:(hh + 1) * dv], g[:, hh], beta[:, hh])
        outs.append(norm_plain(o, P["norm"], eps))
    y = torch.cat(outs, dim=1) * gate
    return y @ P["o"].T


def mixer_parallel(h, P: Dict[str, torch.Tensor], m: dict, eps: float):
    L, R = m["left"], m["right"]
    q = norm_plain(h @ P["left.q"].T, P["left.q.norm"], eps)
    k = norm_plain(h @ P["left.k"].T, P["left.k.norm"], eps)
    v = h @ P["left.v"].T
    a = windowed_attention(q, k, v, L["heads"], L["kv_heads"], L["scale"], L["softcap"], P["left.rel"], L["bias_max"], L["mask"]["size"])
    left = a @ P["left.o"].T
    H, d, dv = R["heads"], R["dim"], R["vdim"]
    rq, rk, rv = silu(h @ P["right.q"].T), silu(h @ P["right.k"].T), silu(h @ P["right.v"].T)
    o = torch.cat([decayed_outer_sum(rq[:, i * d:(i + 1) * d], rk[:, i * d:(i + 1) * d], rv[:, i * dv:(i + 1) * dv], float(R["decay"][i]))
                   for i in range(H)], dim=1)
    right = (norm_plain(o, P["right.norm"], eps) * torch.sigmoid(h @ P["right.g"].T)) @ P["right.o"].T
    return 0.5 * (norm_plain(left, P["left.out"], eps) + norm_plain(right, P["right.out"], eps))


def dense_ff(h, P: Dict[str, torch.Tensor]):
    return (gelu_tanh(h @ P["gate"].T + P["gate.b"]) * (h @ P["up"].T + P["up.b"])) @ P["down"].T + P["down.b"]


# ---------------------------------------------------------------------------------------------------------------------- model
def _sub(sd, prefix):
    return {k[len(prefix):]: v.to(DT) for k, v in sd.items() if k.startswith(prefix)}


def forward(cfg: dict, sd: Dict[str, torch.Tensor], tokens, collect: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; collect receives the residual stream after every layer."""
    eps, m = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = sd["embed"].to(DT)[torch.as_tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    for i, ld in enumerate(cfg["layers"]):
        src = ld.get("weights_of", i)
        P = _sub(sd, f"l{src}.")
        h = norm_zero_centred(x, P["norm1"], eps)
        mix = _sub(P, "mix.")
        if ld["type"] == "parallel":
            y = mixer_parallel(h, mix, ld["mixer"], eps)
        elif ld["type"] in ("delta", "channel_delta"):
            y = mixer_delta(h, mix, ld["mixer"], eps, ld["type"] == "channel_delta")
        else:
            raise ValueError(ld["type"])
        x = x + m * norm_zero_centred(y, P["norm1b"], eps)
        if ld.get("mlp"):
            y = dense_ff(norm_zero_centred(x, P["norm2"], eps), _sub(P, "mlp."))
            x = x + m * norm_zero_centred(y, P["norm2b"], eps)
        if collect is not None:
            collect.append(x.clone())
    return norm_zero_centred(x, sd["final.norm"].to(DT), eps) @ sd["head"].to(DT).T
