"""Tifisun: a decoder-only language model whose mixers carry a fixed-size state - gated delta-rule layers (one decay per head, or one
per head and key channel) and 'parallel' layers that run sliding-window attention beside a constant-decay linear attention.

A layer with residual factor m:  x <- x + m * Nb1(mixer(Na1(x)));  x <- x + m * Nb2(ff(Na2(x)))  with N(y) = y / rms(y) * (1 + g) on
both sides of every sublayer; the residual stream x is fp32 on the device. Layers may share another layer's tensors (config
`weights_of`) while keeping a cache and state of their own. Feed-forward: gelu_tanh(W_g x + b) * (W_u x + b) -> W_d + b.

Like the other sequence-step decoder (model/voduzen.py) the model owns no cache and no loop: `step()` runs ONE packed batch of rows -
portions of prompts beside single decoded tokens, each row addressed by (slot, position) - against a PagedStateCache that the
caller (serving.StepScheduler) manages: pages of keys and values for the windowed attention, per-slot fp32 states for the
recurrences and the convolutions' last inputs. `generate()` goes through that scheduler.

Kernels (csrc/state_mixers.cu, window_attention.cu, rownorm32.cu, linear_any.cu): one stacked input projection per mixer, causal
convolution + silu + unit vectors, the linear-state recurrence (delta rule or plain outer-product sum; decays, sigmoid and softplus
evaluated in fp32 inside it), gated RMS norm, query/key norm + cache append, windowed soft-capped attention with a distance-bias table,
and one kernel that turns a sublayer's output into the residual update AND the next sublayer's normed input.

Compute dtype bfloat16: bf16 matrix operands with fp32 accumulation, bf16 keys / values; norms, softmax, residual, recurrent state
and everything that enters a recurrence after the projections in fp32. Compute dtype float32: everything in fp32 on the FMA pipe.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .. import lib, seqlib
from ..config import DeltaRuleSpec, ParallelMixerSpec, TifisunConfig, WindowAttentionSpec
from .paged_cache import PagedStateCache
from .seq_linear import dense_linear


# ------------------------------------------------------------------------------------------------------------------- weights
@dataclass
class DeltaW:
    w_in: torch.Tensor             # [q | k | v | beta | decay (or its first factor) | gate (or its first factor) | zero rows, C]
    cols: Dict[str, slice]         # column ranges of the stacked projection's output
    conv: torch.Tensor             # [q + k + v channels, taps]
    A_log: torch.Tensor            # fp32 [H]
    dt_bias: torch.Tensor          # fp32 [H] or [H * dim]
    a2: Optional[torch.Tensor]     # [H * dim, decay_rank] (per-channel decay)
    g2: Optional[torch.Tensor]     # [H * vdim, gate_rank]
    norm: torch.Tensor             # [vdim]
    o: torch.Tensor                # [C, H * vdim]


@dataclass
class ParallelW:
    w_in: torch.Tensor             # [left q | left k | left v | right q | right k | right v | right gate | zero rows, C]
    cols: Dict[str, slice]
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    dist_bias: torch.Tensor        # fp32 [window, H]: the learned table expanded by distance
    left_o: torch.Tensor
    decay: torch.Tensor            # fp32 [right heads]
    right_norm: torch.Tensor
    right_o: torch.Tensor
    left_out: torch.Tensor         # [C]
    right_out: torch.Tensor


@dataclass
class DenseMlpW:
    gate_up: torch.Tensor          # [2 * ff, C]
    gate_up_b: torch.Tensor
    down: torch.Tensor
    down_b: torch.Tensor


@dataclass
class TifisunLayerW:
    norm1: torch.Tensor
    norm1b: torch.Tensor
    norm2: Optional[torch.Tensor]
    norm2b: Optional[torch.Tensor]
    mix: object
    mlp: Optional[DenseMlpW]


@dataclass
class TifisunW:
    embed: torch.Tensor
    final_norm: torch.Tensor
    head: torch.Tensor
    layers: List[TifisunLayerW]    # one entry per layer; layers that share tensors share the entry


def _stack(parts: Sequence[tuple], device, dtype):
    """[(name, matrix [n_i, C])] -> (stacked matrix with zero rows up to a multiple of 8, {name: column slice of its output})."""
    cols, rows, at = {}, [], 0
    for name, m in parts:
        cols[name] = slice(at, at + m.shape[0])
        at += m.shape[0]
        rows.append(m)
    if at % 8:   # the tensor-core GEMMs take N % 8 == 0; the extra outputs are never read
        rows.append(torch.zeros(8 - at % 8, rows[0].shape[1], device=device, dtype=dtype))
    return torch.cat(rows, dim=0).contiguous(), cols


def distance_bias_table(rel: torch.Tensor, spec: WindowAttentionSpec) -> torch.Tensor:
    """rel [rows, H] -> fp32 [window, H]: row n is the bias of a key n positions back."""
    idx = [WindowAttentionSpec.bucket(n, rel.shape[0], spec.bias_max) for n in range(spec.window)]
    return rel.to(torch.float32)[torch.tensor(idx, dtype=torch.long, device=rel.device)].contiguous()


def weights_from_state_dict(sd: Dict[str, torch.Tensor], cfg: TifisunConfig, device, dtype: torch.dtype) -> TifisunW:
    """Checkpoint names: 'embed', 'final.norm', 'head', per layer i 'l<i>.norm1|norm1b|norm2|norm2b', 'l<i>.mix.*', 'l<i>.mlp.*';
    linear weights [out, in]. A layer with weights_of = j has no tensors and uses layer j's entry. Load-time re-layouts: the
    mixer's input projections are stacked into one matrix, gate and up likewise, the distance-bias table is expanded."""
    def g(name, dt=dtype):
        if name not in sd:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        return sd[name].to(device=device, dtype=dt).contiguous()

    C, f32 = cfg.hidden_size, torch.float32
    built: Dict[int, TifisunLayerW] = {}

    def owner(i: int) -> int:
        seen = set()
        while cfg.layers[i].weights_of is not None:
            if i in seen:
                raise ValueError("weights_of forms a cycle")
            seen.add(i)
            i = cfg.layers[i].weights_of
        return i

    def build(i: int) -> TifisunLayerW:
        spec, p = cfg.layers[i], f"l{i}.mix."
        m = spec.mixer
        if isinstance(m, DeltaRuleSpec):
            parts = [("q", g(p + "q")), ("k", g(p + "k")), ("v", g(p + "v")), ("beta", g(p + "b"))]
            if m.channel_decay:
                parts += [("a", g(p + "a1")), ("g", g(p + "g1"))]
            else:
                parts += [("a", g(p + "a")), ("g", g(p + "g"))]
            w_in, cols = _stack(parts, device, dtype)
            nqk = m.kv_heads * m.dim
            for name, n in (("q", nqk), ("k", nqk), ("v", m.heads * m.vdim), ("beta", m.heads)):
                if cols[name].stop - cols[name].start != n:
                    raise ValueError(f"layer {i}: projection {name!r} has {cols[name].stop - cols[name].start} outputs, config says {n}")
            mix = DeltaW(w_in=w_in, cols=cols, conv=torch.cat([g(p + "q.conv"), g(p + "k.conv"), g(p + "v.conv")], dim=0).contiguous(),
                         A_log=g(p + "A_log", f32), dt_bias=g(p + "dt_bias", f32),
                         a2=g(p + "a2") if m.channel_decay else None, g2=g(p + "g2") if m.channel_decay else None,
                         norm=g(p + "norm"), o=g(p + "o"))
            if mix.conv.shape[1] != m.conv or mix.dt_bias.numel() != (m.heads * m.dim if m.channel_decay else m.heads):
                raise ValueError(f"layer {i}: convolution taps or decay bias do not fit the config")
        else:
            assert isinstance(m, ParallelMixerSpec)
            L, R = m.left, m.right
            parts = [("lq", g(p + "left.q")), ("lk", g(p + "left.k")), ("lv", g(p + "left.v")), ("rq", g(p + "right.q")),
                     ("rk", g(p + "right.k")), ("rv", g(p + "right.v")), ("rg", g(p + "right.g"))]
            w_in, cols = _stack(parts, device, dtype)
            rel = g(p + "left.rel", f32)
            if rel.shape[1] != L.heads:
                raise ValueError(f"layer {i}: the distance-bias table has {rel.shape[1]} columns for {L.heads} heads")
            mix = ParallelW(w_in=w_in, cols=cols, q_norm=g(p + "left.q.norm"), k_norm=g(p + "left.k.norm"),
                            dist_bias=distance_bias_table(rel, L), left_o=g(p + "left.o"),
                            decay=torch.tensor(R.decay, dtype=f32, device=device), right_norm=g(p + "right.norm"),
                            right_o=g(p + "right.o"), left_out=g(p + "left.out"), right_out=g(p + "right.out"))
        mlp = None
        if spec.mlp is not None:
            q = f"l{i}.mlp."
            mlp = DenseMlpW(gate_up=torch.cat([g(q + "gate"), g(q + "up")], dim=0).contiguous(),
                            gate_up_b=torch.cat([g(q + "gate.b"), g(q + "up.b")], dim=0).contiguous(),
                            down=g(q + "down"), down_b=g(q + "down.b"))
            if mlp.gate_up.shape[0] != 2 * spec.mlp.ff:
                raise ValueError(f"layer {i}: feed-forward width does not fit the config")
        return TifisunLayerW(norm1=g(f"l{i}.norm1"), norm1b=g(f"l{i}.norm1b"), norm2=g(f"l{i}.norm2") if mlp else None,
                             norm2b=g(f"l{i}.norm2b") if mlp else None, mix=mix, mlp=mlp)

    layers = []
    for i in range(len(cfg.layers)):
        j = owner(i)
        if j not in built:
            built[j] = build(j)
        layers.append(built[j])
    return TifisunW(embed=g("embed"), final_norm=g("final.norm"), head=g("head"), layers=layers)


def random_state_dict(cfg: TifisunConfig, seed: int = 0, decay_rank: int = 16, gate_rank: int = 16, bias_rows: int = 32) -> Dict[str, torch.Tensor]:
    """Random bf16 weights under the checkpoint names (benchmarks, tests)."""
    gen = torch.Generator().manual_seed(seed)

    def rn(*shape, s=1.0, mean=0.0):
        return (torch.randn(*shape, generator=gen) * s + mean).to(torch.bfloat16)

    C, sd = cfg.hidden_size, {}
    sd["embed"] = rn(cfg.vocab_size, C, s=1.0 / max(cfg.embedding_scale, 1e-6))
    sd["final.norm"] = rn(C, s=0.2)
    sd["head"] = rn(cfg.vocab_size, C, s=C ** -0.5)
    for i, spec in enumerate(cfg.layers):
        if spec.weights_of is not None:
            continue
        m, p = spec.mixer, f"l{i}.mix."
        for n in ("norm1", "norm1b"):
            sd[f"l{i}.{n}"] = rn(C, s=0.2)
        if isinstance(m, DeltaRuleSpec):
            nqk, nv = m.kv_heads * m.dim, m.heads * m.vdim
            for name, n in (("q", nqk), ("k", nqk), ("v", nv)):
                sd[p + name] = rn(n, C, s=C ** -0.5)
                sd[p + name + ".conv"] = rn(n, m.conv, s=0.6)
            sd[p + "b"] = rn(m.heads, C, s=C ** -0.5)
            sd[p + "A_log"] = rn(m.heads, s=1.0, mean=-2.0)
            sd[p + "norm"] = rn(m.vdim, s=0.2, mean=1.0)
            if m.channel_decay:
                sd[p + "a1"] = rn(decay_rank, C, s=C ** -0.5)
                sd[p + "a2"] = rn(m.heads * m.dim, decay_rank, s=decay_rank ** -0.5)
                sd[p + "dt_bias"] = rn(m.heads * m.dim, s=0.8, mean=-2.0)
                sd[p + "g1"] = rn(gate_rank, C, s=C ** -0.5)
                sd[p + "g2"] = rn(nv, gate_rank, s=gate_rank ** -0.5)
            else:
                sd[p + "a"] = rn(m.heads, C, s=C ** -0.5)
                sd[p + "dt_bias"] = rn(m.heads, s=0.5, mean=-2.0)
                sd[p + "g"] = rn(nv, C, s=C ** -0.5)
            sd[p + "o"] = rn(C, nv, s=nv ** -0.5)
        else:
            L, R = m.left, m.right
            sd[p + "left.q"] = rn(L.heads * L.dim, C, s=C ** -0.5)
            sd[p + "left.k"] = rn(L.kv_heads * L.dim, C, s=C ** -0.5)
            sd[p + "left.v"] = rn(L.kv_heads * L.vdim, C, s=C ** -0.5)
            sd[p + "left.q.norm"] = rn(L.heads * L.dim, s=0.3, mean=1.2)
            sd[p + "left.k.norm"] = rn(L.kv_heads * L.dim, s=0.3, mean=1.2)
            sd[p + "left.rel"] = rn(bias_rows, L.heads, s=1.0)
            sd[p + "left.o"] = rn(C, L.heads * L.vdim, s=(L.heads * L.vdim) ** -0.5)
            sd[p + "right.q"] = rn(R.heads * R.dim, C, s=C ** -0.5)
            sd[p + "right.k"] = rn(R.heads * R.dim, C, s=C ** -0.5)
            sd[p + "right.v"] = rn(R.heads * R.vdim, C, s=C ** -0.5)
            sd[p + "right.g"] = rn(R.heads * R.vdim, C, s=C ** -0.5)
            sd[p + "right.norm"] = rn(R.heads * R.vdim, s=0.2, mean=1.0)
            sd[p + "right.o"] = rn(C, R.heads * R.vdim, s=(R.heads * R.vdim) ** -0.5)
            sd[p + "left.out"] = rn(C, s=0.15, mean=0.9)
            sd[p + "right.out"] = rn(C, s=0.15, mean=0.9)
        if spec.mlp is not None:
            q, ff = f"l{i}.mlp.", spec.mlp.ff
            for n in ("norm2", "norm2b"):
                sd[f"l{i}.{n}"] = rn(C, s=0.2)
            sd[q + "gate"], sd[q + "gate.b"] = rn(ff, C, s=C ** -0.5), rn(ff, s=0.1)
            sd[q + "up"], sd[q + "up.b"] = rn(ff, C, s=C ** -0.5), rn(ff, s=0.1)
            sd[q + "down"], sd[q + "down.b"] = rn(C, ff, s=ff ** -0.5), rn(C, s=0.1)
    return sd


# ------------------------------------------------------------------------------------------------------------------- decoder
PREP_MIN_ROWS = 32   # average rows per request from which silu / decays of a recurrence's inputs are a pass of their own


class TifisunDecoder:
    def __init__(self, cfg: TifisunConfig, w: TifisunW, dtype: torch.dtype):
        self.cfg, self.w, self.dtype = cfg, w, dtype
        self.device = w.embed.device
        self.C = cfg.hidden_size
        self.eps = cfg.norm_eps
        self.tensor_gemm = dtype == torch.bfloat16
        self._graphs = {}         # (rows, id(cache)) -> captured decode-only step
        self._arange = None       # int32 [n + 1]: portion starts of a step whose rows are one request each
        self.use_graph = True
        self.tensor_attention = True    # False: the plain attention kernel for every shape (A/B, tests)

    # ---- cache
    def cache_widths(self) -> List[int]:
        """Cached numbers per token and layer: keys and values of the windowed attention; 0 for layers that only carry state."""
        return [l.mixer.left.kv_heads * (l.mixer.left.dim + l.mixer.left.vdim) if isinstance(l.mixer, ParallelMixerSpec) else 0
                for l in self.cfg.layers]

    def state_shapes(self) -> List[dict]:
        out = []
        for l in self.cfg.layers:
            m = l.mixer
            if isinstance(m, DeltaRuleSpec):
                s = {"S": (m.heads, m.dim, m.vdim)}
                if m.conv > 1:
                    s["conv"] = (m.conv - 1, 2 * m.kv_heads * m.dim + m.heads * m.vdim)
            else:
                s = {"S": (m.right.heads, m.right.dim, m.right.vdim)}
            out.append(s)
        return out

    def new_cache(self, n_pages: int, n_slots: int, max_pages_per_slot: int = 0) -> PagedStateCache:
        return PagedStateCache(self.cache_widths(), self.state_shapes(), n_pages, n_slots, self.cfg.kv_page_size, self.dtype,
                               self.device, max_pages_per_slot)

    def _linear(self, x, w, out_dtype, act: int = seqlib.ACT_NONE, bias=None):
        return dense_linear(x, w, out_dtype, tensor_gemm=self.tensor_gemm, act=act, bias=bias)

    # ---- mixers: compute-dtype rows [T, C] -> fp32 [T, C] (two tensors for the parallel mixer)
    def _delta(self, li: int, xb, pos, slot, cache: PagedStateCache, row_begin, n_portions: int):
        m: DeltaRuleSpec = self.cfg.layers[li].mixer
        mw: DeltaW = self.w.layers[li].mix
        st = cache.states[li]
        T, f32, dev = xb.shape[0], torch.float32, xb.device
        H, G, d, dv = m.heads, m.kv_heads, m.dim, m.vdim
        z = self._linear(xb, mw.w_in, f32)                              # [T, q | k | v | beta | a | g]
        nqk = G * d
        qkv = torch.empty(T, 2 * nqk + H * dv, device=dev, dtype=f32)
        seqlib.causal_conv_silu(z[:, :2 * nqk + H * dv], mw.conv, pos, slot, st.get("conv"), qkv, unit_channels=2 * nqk, unit_group=d,
                                unit_eps=1e-6, scaled_channels=nqk, unit_mult=d ** -0.5, single_rows=n_portions == T)
        a, gate = z[:, mw.cols["a"]], z[:, mw.cols["g"]]
        if m.channel_decay:
            a = self._linear(a, mw.a2, f32)                              # [T, H * d]
            gate = self._linear(gate, mw.g2, f32)                        # [T, H * dv]
        o = torch.empty(T, H * dv, device=dev, dtype=f32)
        # long portions: the per-channel decays in one pass instead of in every CTA that shares a head (the same function either way)
        prep = m.channel_decay and T >= PREP_MIN_ROWS * n_portions
        if prep:
            seqlib.map_rows(a, seqlib.MAP_DECAY, mw.A_log, mw.dt_bias, d)
        seqlib.linear_state_scan(qkv[:, :nqk], qkv[:, nqk:2 * nqk], qkv[:, 2 * nqk:], st["S"], o, row_begin, n_portions, pos, slot, H, G, d, dv,
                                 a=a, A_log=mw.A_log, dt_bias=mw.dt_bias, channel_decay=m.channel_decay, beta=z[:, mw.cols["beta"]],
                                 decay_given=prep)
        on = torch.empty(T, H * dv, device=dev, dtype=self.dtype)
        seqlib.gated_rms_rows(o, H, dv, mw.norm, self.eps, gate, seqlib.GATE_SIGMOID if m.channel_decay else seqlib.GATE_SILU, on)
        return self._linear(on, mw.o, f32)

    def _parallel(self, li: int, xb, pos, slot, cache: PagedStateCache, row_begin, n_portions: int, plans: Optional[dict] = None):
        m: ParallelMixerSpec = self.cfg.layers[li].mixer
        mw: ParallelW = self.w.layers[li].mix
        L, R = m.left, m.right
        T, f32, dev = xb.shape[0], torch.float32, xb.device
        z = self._linear(xb, mw.w_in, f32)
        c = mw.cols
        # left: windowed attention over the paged keys / values
        pool = cache.pools[li]
        q = torch.empty(T, L.heads * L.dim, device=dev, dtype=self.dtype)
        seqlib.qk_norm_kv_store(z[:, c["lq"]], mw.q_norm, z[:, c["lk"]], mw.k_norm, z[:, c["lv"]], self.eps, pos, slot, cache.block_table,
                                cache.page_size, pool, q)
        att = torch.empty(T, L.heads * L.vdim, device=dev, dtype=self.dtype)
        if plans is not None and self.tensor_attention and seqlib.window_attn_mma_ok(L.heads, L.kv_heads, L.dim, L.vdim, self.dtype):
            rep = L.heads // L.kv_heads
            if plans["portions"] is None:        # one row per request: the kernel reads positions and slots itself
                items = None
            else:
                items = plans.get(rep)
                if items is None:
                    items = plans[rep] = seqlib.window_attn_items(plans["portions"], rep, dev)
            seqlib.window_attn_mma(q, L.heads, L.kv_heads, L.dim, L.vdim, pool, cache.block_table, cache.page_size, items, pos, slot,
                                   L.window, L.scale, L.softcap, mw.dist_bias, att)
        else:
            seqlib.window_attn(q, L.heads, L.kv_heads, L.dim, L.vdim, pool, cache.block_table, cache.page_size, pos, slot, L.window, L.scale,
                               L.softcap, mw.dist_bias, att)
        left = self._linear(att, mw.left_o, f32)
        # right: constant-decay outer-product state
        o = torch.empty(T, R.heads * R.vdim, device=dev, dtype=f32)
        prep = T >= PREP_MIN_ROWS * n_portions
        if prep:   # q | k | v are neighbours in the stacked projection: one pass of silu over the three
            seqlib.map_rows(z[:, c["rq"].start:c["rv"].stop], seqlib.MAP_SILU)
        seqlib.linear_state_scan(z[:, c["rq"]], z[:, c["rk"]], z[:, c["rv"]], cache.states[li]["S"], o, row_begin, n_portions, pos, slot,
                                 R.heads, R.heads, R.dim, R.vdim, silu_in=not prep, decay_const=mw.decay)
        on = torch.empty(T, R.heads * R.vdim, device=dev, dtype=self.dtype)
        seqlib.gated_rms_rows(o, 1, R.heads * R.vdim, mw.right_norm, self.eps, z[:, c["rg"]], seqlib.GATE_SIGMOID, on)
        right = self._linear(on, mw.right_o, f32)
        return left, right

    def _row_begin(self, T: int, slot: torch.Tensor, portions: Optional[Sequence]):
        """Device int32 [P + 1] with the first row of every request's portion (and T), and P."""
        if portions is None:   # one row per request, or derive it from the slots (a host round trip: tests, debugging)
            s = slot.cpu()
            starts = [0] + [i for i in range(1, T) if s[i] != s[i - 1]]
        else:
            starts = [p[0] for p in portions]
        if len(starts) == T:
            if self._arange is None or self._arange.numel() < T + 1:
                self._arange = torch.arange(max(T + 1, 65), device=self.device, dtype=torch.int32)
            return self._arange, T
        rb = torch.tensor(starts + [T], dtype=torch.int32)
        if self.device.type == "cuda":
            rb = rb.pin_memory().to(self.device, non_blocking=True)
        return rb, len(starts)

    # ---- the step
    @torch.no_grad()
    def step(self, tokens: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, cache: PagedStateCache,
             want_rows: Optional[torch.Tensor] = None, collect: Optional[list] = None,
             portions: Optional[Sequence] = None, one_row_each: bool = False) -> Optional[torch.Tensor]:
        """tokens / pos / slot: int32 [T] on the device - row t is token tokens[t] at position pos[t] of the request in slot slot[t];
        rows of one request are consecutive and ascending in position, and a request's rows continue where its previous step
        ended. Appends every row to the cache, advances the states and returns fp32 logits [len(want_rows), vocab] (None when no
        row is asked for). collect: receives the residual stream after every layer. portions: the same batch as the host knows
        it, [(first_row, n_rows, slot, first_pos)] per request. one_row_each: every row is a request of its own (decode)."""
        T, dev, f32 = tokens.numel(), self.device, torch.float32
        if one_row_each:
            portions = None
            if self._arange is None or self._arange.numel() < T + 1:
                self._arange = torch.arange(max(T + 1, 65), device=dev, dtype=torch.int32)
            row_begin, n_portions = self._arange, T
        else:
            row_begin, n_portions = self._row_begin(T, slot, portions)
        # work lists of the tensor-core attention kernel, built once per step and head grouping; without the host's view of the
        # batch (portions) the plain kernel runs
        plans = {"portions": None} if one_row_each else ({"portions": list(portions)} if portions is not None else None)
        layers, mult = self.w.layers, self.cfg.residual_mult
        h32 = torch.empty(T, self.C, device=dev, dtype=f32)
        xb = torch.empty(T, self.C, device=dev, dtype=self.dtype)
        seqlib.embed_scale(tokens, self.w.embed, self.cfg.embedding_scale, h32, None)
        seqlib.rms_rows(h32, layers[0].norm1, self.eps, xb, one_plus=True)
        for li, lw in enumerate(layers):
            last = li + 1 == len(layers)
            nxt = None if last else layers[li + 1].norm1
            after_mixer = lw.norm2 if lw.mlp is not None else nxt
            xb_out = xb if (lw.mlp is not None or not last) else None
            if isinstance(self.cfg.layers[li].mixer, DeltaRuleSpec):
                y = self._delta(li, xb, pos, slot, cache, row_begin, n_portions)
                seqlib.post_norm_residual(y, lw.norm1b, self.eps, mult, h32, after_mixer, xb_out)
            else:
                yl, yr = self._parallel(li, xb, pos, slot, cache, row_begin, n_portions, plans)
                seqlib.post_norm_residual(yl, lw.norm1b, self.eps, mult, h32, after_mixer, xb_out, y2=yr, wa=lw.mix.left_out,
                                          wb=lw.mix.right_out)
            if lw.mlp is not None:
                ff = lw.mlp.down.shape[1]
                z = self._linear(xb, lw.mlp.gate_up, self.dtype, bias=lw.mlp.gate_up_b)   # gate | up in the compute dtype
                act = seqlib.glu_mul(z, ff, seqlib.ACT_GELU_TANH, torch.empty(T, ff, device=dev, dtype=self.dtype))
                y = self._linear(act, lw.mlp.down, f32, bias=lw.mlp.down_b)
                seqlib.post_norm_residual(y, lw.norm2b, self.eps, mult, h32, nxt, None if last else xb)
            if collect is not None:
                collect.append(h32.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        hw = h32.index_select(0, want_rows)
        xf = seqlib.rms_rows(hw, self.w.final_norm, self.eps, torch.empty(hw.shape[0], self.C, device=dev, dtype=self.dtype), one_plus=True)
        return self._linear(xf, self.w.head, f32)

    class _Graph:
        pass

    @torch.no_grad()
    def decode_step(self, meta_host: torch.Tensor, cache: PagedStateCache, max_keys: int) -> torch.Tensor:
        """A decode-only step: meta_host int32 [3, B] (tokens, positions, slots; pinned host memory), one row per request. The
        step is captured once per (B, cache) in a CUDA graph and replayed - every kernel takes positions and slots from device
        memory and no launch shape depends on the contexts' lengths. Returns fp32 logits [B, vocab] (a static buffer,
        overwritten by the next call)."""
        B = meta_host.shape[1]
        key = (B, id(cache))
        g = self._graphs.get(key)
        if g is not None and g.cache is not cache:
            g = None
        if g is None:
            if len(self._graphs) >= 16:
                self._graphs.pop(next(iter(self._graphs)))
            g = TifisunDecoder._Graph()
            g.cache = cache
            g.meta = torch.zeros(3, B, device=self.device, dtype=torch.int32)
            g.want = torch.arange(B, device=self.device)
            g.graph = None
            self._graphs[key] = g
            if self.use_graph:
                # Capture needs a warmed-up step (kernel attributes, workspaces), but a step ADVANCES the states, so the warm-up
                # and the capture's dry run must not touch live slots: they run on a scratch cache of the same shapes.
                scratch = self.new_cache(2, cache.n_slots, 1)
                dummy = torch.zeros(3, B, device=self.device, dtype=torch.int32)
                dummy[2] = torch.arange(B, device=self.device, dtype=torch.int32) % cache.n_slots
                self.step(dummy[0], dummy[1], dummy[2], scratch, g.want, one_row_each=True)
                torch.cuda.synchronize()
                del scratch, dummy
                n0 = lib.launch_count()
                g.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g.graph):
                    g.logits = self.step(g.meta[0], g.meta[1], g.meta[2], cache, g.want, one_row_each=True)
                g.launches = lib.launch_count() - n0
                lib.add_launches(-g.launches)   # the capture does not execute
        g.meta.copy_(meta_host, non_blocking=True)
        if g.graph is None:
            return self.step(g.meta[0], g.meta[1], g.meta[2], cache, g.want, one_row_each=True)
        g.graph.replay()
        lib.add_launches(g.launches)
        return g.logits


# ------------------------------------------------------------------------------------------------------------------- model
class TifisunForCausalLM:
    """Entry point: from_pretrained / from_state_dict, step() for serving loops, generate() for greedy generation."""
    config_class = TifisunConfig

    def __init__(self, config: TifisunConfig, weights: TifisunW, dtype: torch.dtype = torch.bfloat16):
        if not torch.cuda.is_available():
            raise lib.OmcError("omchat_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        seqlib.load()
        self.config, self.weights, self.dtype = config, weights, dtype
        self.device = weights.embed.device
        self.decoder = TifisunDecoder(config, weights, dtype)
        self.vocab_size = config.vocab_size

    @classmethod
    def from_state_dict(cls, sd, config: TifisunConfig, device="cuda", dtype: torch.dtype = torch.bfloat16, **unused):
        if not torch.cuda.is_available():
            raise lib.OmcError("omchat_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("compute dtype must be torch.bfloat16 or torch.float32")
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        return cls(config, weights_from_state_dict(sd, config, device, dtype), dtype)

    @classmethod
    def from_pretrained(cls, path: str, config: Optional[TifisunConfig] = None, device="cuda", dtype: torch.dtype = torch.bfloat16, **kw):
        from .checkpoint import load_checkpoint
        sd, cfg = load_checkpoint(path, config)
        if not isinstance(cfg, TifisunConfig):
            raise ValueError(f"{path} is not a Tifisun checkpoint")
        return cls.from_state_dict(sd, cfg, device=device, dtype=dtype)

    def eval(self):
        return self

    def step(self, tokens, pos, slot, cache, want_rows=None, collect=None, portions=None):
        with torch.cuda.device(self.device):
            return self.decoder.step(tokens, pos, slot, cache, want_rows, collect, portions)

    def decode_step(self, meta_host, cache, max_keys: int):
        """Decode-only batch (one token per request) through the captured CUDA graph; see TifisunDecoder.decode_step."""
        with torch.cuda.device(self.device):
            return self.decoder.decode_step(meta_host, cache, max_keys)

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens: int = 32, eos_token_id: Optional[int] = None, do_sample: bool = False,
                 slots: int = 4, chunk: int = 512, **unused) -> List[torch.Tensor]:
        """Greedy generation of a batch of prompts (a [b, S] tensor or a list of 1-D id sequences of unequal length) through
        serving.StepScheduler: prompts are prefilled in portions of `chunk` tokens beside the decode rows of the requests that
        are already generating. Returns one LongTensor per prompt: the prompt followed by the generated ids."""
        if do_sample:
            raise NotImplementedError("only greedy decoding (do_sample=False) is on the accelerated path")
        from ..serving import StepScheduler
        prompts = [torch.as_tensor(p).view(-1).tolist() for p in input_ids]
        ps = self.config.kv_page_size
        need = sorted((-(-(len(p) + max_new_tokens) // ps) * ps for p in prompts), reverse=True)
        sched = StepScheduler(self, max_tokens=sum(need[:slots]), slots=slots, chunk=chunk)
        eos = self.config.eos_token_id if eos_token_id is None else eos_token_id
        rids = [sched.submit(p, max_new_tokens, eos) for p in prompts]
        res = sched.run()
        return [torch.tensor(p + res[r], dtype=torch.int64) for p, r in zip(prompts, rids)]
