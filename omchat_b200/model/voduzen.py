"""Voduzen: a decoder-only language model of latent-attention layers with mixture-of-experts feed-forwards.

A layer is x <- x + N1(mixer(x)); x <- x + N2(ff(x)) with the norm on the sublayer's OUTPUT, N(y) = y / rms(y) * (1 + g), and
the sublayers reading x itself. The residual stream x is fp32 on the device; sublayers read its rounding to the compute dtype.

Mixers (config.LatentAttentionSpec): keys / values are up-projections of a cached latent c (kv_rank wide, RMS-normed) plus one
rotated key part shared by the heads; queries are projected directly or through a normed latent of their own (q_rank); the
softmax may carry a per-head sink term. The up-projections are absorbed (csrc/latent_attention.cu): the unrotated query goes
through W_uk^T into latent space, attention runs against the cached rows, W_uv maps the weighted latent sum to the head's value.
Feed-forward (config.RouterMoeSpec): softmax router over experts + identity outputs, choice by score + correction, weights =
uncorrected scores, relu^2 experts, a sigmoid-gated shared expert.

The model owns no cache and no loop: `step()` runs ONE packed batch of rows - portions of prompts beside single decoded tokens,
each row addressed by (cache slot, position) - against a PagedLatentCache that the caller (serving.StepScheduler) manages, and
returns fp32 logits for the rows asked for. `generate()` goes through that scheduler.

Compute dtype bfloat16: bf16 storage and matrix operands with fp32 accumulation; softmax, norms, router, residual in fp32.
Compute dtype float32: everything in fp32 on the FMA pipe (csrc/linear_any.cu), no reduced-precision matrix mode.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .. import lib, seqlib
from ..config import LatentAttentionSpec, RouterMoeSpec, VoduzenConfig
from .paged_cache import PagedLatentCache
from .seq_linear import TENSOR_GEMM_MIN_WEIGHT, dense_linear


# ------------------------------------------------------------------------------------------------------------------- weights
@dataclass
class LatentAttnW:
    q: Optional[torch.Tensor]       # [H * (dn + dr), C]        (direct queries)
    dq: Optional[torch.Tensor]      # [q_rank, C]               (latent queries)
    dq_norm: Optional[torch.Tensor]
    uq: Optional[torch.Tensor]      # [H * (dn + dr), q_rank]
    dkv: torch.Tensor               # [kv_rank + dr, C]
    dq_dkv: Optional[torch.Tensor]  # [q_rank + kv_rank + dr, C]: dq stacked on dkv (latent queries)
    dkv_norm: torch.Tensor          # [kv_rank]
    uk_t: torch.Tensor              # [H, kv_rank, dn]: per head W_uk^T, the absorbing projection of the unrotated query
    uv: torch.Tensor                # [H * dv, kv_rank]
    o: torch.Tensor                 # [C, H * dv]
    sink: Optional[torch.Tensor]    # fp32 [H]
    rot_cs: torch.Tensor = None     # fp32 [positions, dims / 2, 2], grown on demand


@dataclass
class RouterMoeW:
    router_cat: torch.Tensor            # [E_tot (+ 1) rounded up to 8, C]: router rows, the shared expert's gate row, zero rows
    correction: Optional[torch.Tensor]  # fp32 [E_tot]
    up: Optional[torch.Tensor]          # [E, ff, C]
    down: Optional[torch.Tensor]        # [E, C, ff]
    shared_up: Optional[torch.Tensor]   # [ffs, C]
    shared_down: Optional[torch.Tensor]  # [C, ffs]


@dataclass
class VoduzenLayerW:
    norm1: torch.Tensor
    norm2: Optional[torch.Tensor]
    mix: LatentAttnW
    mlp: Optional[RouterMoeW]


@dataclass
class VoduzenW:
    embed: torch.Tensor
    final_norm: torch.Tensor
    head: torch.Tensor
    layers: List[VoduzenLayerW]


def weights_from_state_dict(sd: Dict[str, torch.Tensor], cfg: VoduzenConfig, device, dtype: torch.dtype) -> VoduzenW:
    """Checkpoint names: 'embed', 'final.norm', 'head', and per layer i 'l<i>.norm1|norm2', 'l<i>.mix.*', 'l<i>.mlp.*' with
    linear weights stored [out, in]. Load-time re-layouts: W_uk is transposed per head, the experts are stacked, the shared
    expert's gate row is appended to the router matrix."""
    def g(name, dt=dtype):
        if name not in sd:
            raise KeyError(f"checkpoint has no tensor {name!r}")
        return sd[name].to(device=device, dtype=dt).contiguous()

    layers = []
    for i, spec in enumerate(cfg.layers):
        p, m = f"l{i}.mix.", spec.mixer
        H, dn, r = m.heads, m.dim, m.kv_rank
        uk = g(p + "uk")                                               # [H * dn, r]
        mix = LatentAttnW(
            q=g(p + "q") if m.q_rank is None else None,
            dq=g(p + "dq") if m.q_rank is not None else None,
            dq_norm=g(p + "dq.norm") if m.q_rank is not None else None,
            uq=g(p + "uq") if m.q_rank is not None else None,
            dkv=g(p + "dkv"), dkv_norm=g(p + "dkv.norm"),
            dq_dkv=torch.cat([g(p + "dq"), g(p + "dkv")], dim=0).contiguous() if m.q_rank is not None else None,
            uk_t=uk.view(H, dn, r).transpose(1, 2).contiguous(),
            uv=g(p + "uv"), o=g(p + "o"),
            sink=g(p + "sink", torch.float32) if m.sink else None)
        mlp = None
        if spec.mlp is not None:
            q, s = f"l{i}.mlp.", spec.mlp
            router = g(q + "router")
            if router.shape[0] != s.experts + s.identity:
                raise ValueError(f"layer {i}: router has {router.shape[0]} outputs, config says {s.experts} + {s.identity}")
            rows = [router]
            if s.shared_ff:
                rows.append(g(q + "shared.sg").view(1, -1))
            n_rows = sum(x.shape[0] for x in rows)
            if n_rows % 8:   # zero rows up to a multiple of 8: the tensor-core GEMMs take the matrix, the extra logits are never read
                rows.append(torch.zeros(8 - n_rows % 8, router.shape[1], device=device, dtype=dtype))
            mlp = RouterMoeW(
                router_cat=torch.cat(rows, dim=0).contiguous(),
                correction=g(q + "correction", torch.float32) if (q + "correction") in sd else None,
                up=torch.stack([g(f"{q}e{e}.up") for e in range(s.experts)]) if s.experts else None,
                down=torch.stack([g(f"{q}e{e}.down") for e in range(s.experts)]) if s.experts else None,
                shared_up=g(q + "shared.up") if s.shared_ff else None,
                shared_down=g(q + "shared.down") if s.shared_ff else None)
        layers.append(VoduzenLayerW(norm1=g(f"l{i}.norm1"), norm2=g(f"l{i}.norm2") if mlp is not None else None, mix=mix, mlp=mlp))
    return VoduzenW(embed=g("embed"), final_norm=g("final.norm"), head=g("head"), layers=layers)


def random_state_dict(cfg: VoduzenConfig, seed: int = 0, std: float = 0.05) -> Dict[str, torch.Tensor]:
    """Random bf16 weights under the checkpoint names (benchmarks, tests)."""
    gen = torch.Generator().manual_seed(seed)

    def rn(*shape, s=std):
        return (torch.randn(*shape, generator=gen) * s).to(torch.bfloat16)

    C, sd = cfg.hidden_size, {}
    sd["embed"] = rn(cfg.vocab_size, C, s=1.0 / max(cfg.embedding_scale, 1e-6))
    sd["final.norm"] = rn(C, s=0.1)
    sd["head"] = rn(cfg.vocab_size, C, s=C ** -0.5)
    for i, spec in enumerate(cfg.layers):
        m, p = spec.mixer, f"l{i}.mix."
        qw = m.heads * (m.dim + m.rot_dim)
        sd[f"l{i}.norm1"] = rn(C, s=0.1)
        if m.q_rank is None:
            sd[p + "q"] = rn(qw, C, s=C ** -0.5)
        else:
            sd[p + "dq"] = rn(m.q_rank, C, s=C ** -0.5)
            sd[p + "dq.norm"] = 1.0 + rn(m.q_rank, s=0.1)
            sd[p + "uq"] = rn(qw, m.q_rank, s=m.q_rank ** -0.5)
        sd[p + "dkv"] = rn(m.kv_rank + m.rot_dim, C, s=C ** -0.5)
        sd[p + "dkv.norm"] = 1.0 + rn(m.kv_rank, s=0.1)
        sd[p + "uk"] = rn(m.heads * m.dim, m.kv_rank, s=m.kv_rank ** -0.5)
        sd[p + "uv"] = rn(m.heads * m.vdim, m.kv_rank, s=m.kv_rank ** -0.5)
        sd[p + "o"] = rn(C, m.heads * m.vdim, s=(m.heads * m.vdim) ** -0.5)
        if m.sink:
            sd[p + "sink"] = rn(m.heads, s=1.0)
        s = spec.mlp
        if s is not None:
            q = f"l{i}.mlp."
            sd[f"l{i}.norm2"] = rn(C, s=0.1)
            sd[q + "router"] = rn(s.experts + s.identity, C, s=C ** -0.5)
            sd[q + "correction"] = rn(s.experts + s.identity, s=0.02)
            for e in range(s.experts):
                sd[f"{q}e{e}.up"] = rn(s.expert_ff, C, s=C ** -0.5)
                sd[f"{q}e{e}.down"] = rn(C, s.expert_ff, s=s.expert_ff ** -0.5)
            if s.shared_ff:
                sd[q + "shared.up"] = rn(s.shared_ff, C, s=C ** -0.5)
                sd[q + "shared.down"] = rn(C, s.shared_ff, s=s.shared_ff ** -0.5)
                sd[q + "shared.sg"] = rn(1, C, s=C ** -0.5)
    return sd


# ------------------------------------------------------------------------------------------------------------------- decoder
SMALL_STEP_ROWS = 4    # steps of up to this many rows sort their rows by expert in one single-CTA launch (32 rows: 0.07 ms per layer slower than the two kernels)


class VoduzenDecoder:
    def __init__(self, cfg: VoduzenConfig, w: VoduzenW, dtype: torch.dtype):
        self.cfg, self.w, self.dtype = cfg, w, dtype
        self.device = w.embed.device
        self.C = cfg.hidden_size
        self.eps = cfg.norm_eps
        self.tensor_gemm = dtype == torch.bfloat16
        self.tensor_attention = True    # False: the plain attention kernel for every shape (A/B, tests)
        self._moe_ws = {}
        self._decode_plans = {}   # (rows, heads, parts) -> seqlib.DecodeAttnPlan
        self._graphs = {}         # (rows, parts, id(cache)) -> captured decode-only step
        self.use_graph = True

    # ---- cache
    def cache_widths(self) -> List[int]:
        return [l.mixer.kv_rank + l.mixer.rot_dim for l in self.cfg.layers]

    def new_cache(self, n_pages: int, n_slots: int, max_pages_per_slot: int = 0) -> PagedLatentCache:
        return PagedLatentCache(self.cache_widths(), n_pages, n_slots, self.cfg.kv_page_size, self.dtype, self.device,
                                max_pages_per_slot)

    def _rot_table(self, mw: LatentAttnW, spec: LatentAttentionSpec, positions: int) -> torch.Tensor:
        """fp32 (cos, sin) [positions, dims / 2, 2]: angles and functions evaluated in double precision on the host, once."""
        t = mw.rot_cs
        if t is None or t.shape[0] < positions:
            n = max(positions, 1024)
            f, mult = spec.rot.frequencies()
            ang = torch.arange(n, dtype=torch.float64)[:, None] * torch.tensor(f, dtype=torch.float64)[None, :]
            t = (torch.stack([ang.cos(), ang.sin()], dim=-1) * mult).to(torch.float32).contiguous().to(self.device)
            if t.numel() == 0:   # no rotated dimensions: the kernels still want a valid pointer
                t = torch.zeros(n, 1, 2, device=self.device)
            mw.rot_cs = t
        return t

    # ---- linear layers
    def _linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, act: int = seqlib.ACT_NONE, alpha: float = 1.0):
        """act(alpha * x @ w^T) -> [rows, N] of out_dtype."""
        return dense_linear(x, w, out_dtype, tensor_gemm=self.tensor_gemm, act=act, alpha=alpha)

    # ---- sublayers
    def _mixer(self, li: int, xb: torch.Tensor, pos, slot, cache: PagedLatentCache, plans: Optional[dict] = None) -> torch.Tensor:
        """-> fp32 [T, C], the mixer's output before its norm."""
        spec, mw = self.cfg.layers[li].mixer, self.w.layers[li].mix
        T = xb.shape[0]
        H, dn, dr, dv, r = spec.heads, spec.dim, spec.rot_dim, spec.vdim, spec.kv_rank
        f32 = torch.float32
        # bf16: q, the absorbed query and the weighted latent sum are bf16 matrix operands (tensor-pipe GEMMs on both sides);
        # fp32: they stay fp32 throughout
        qdt = self.dtype
        if spec.q_rank is not None:
            # both down-projections read the same rows and want fp32 outputs: one product over the stacked matrix
            both = self._linear(xb, mw.dq_dkv, f32)
            cq32, dkv32 = both[:, :spec.q_rank], both[:, spec.q_rank:]
            cq = seqlib.rms_rows(cq32, mw.dq_norm, self.eps, torch.empty(T, spec.q_rank, device=xb.device, dtype=self.dtype))
            q = self._linear(cq, mw.uq, qdt)
        else:
            q = self._linear(xb, mw.q, qdt)
            dkv32 = self._linear(xb, mw.dkv, f32)
        cs = self._rot_table(mw, spec, cache.capacity)
        pool = cache.pools[li]
        qcat = torch.empty(T, H, r + dr, device=xb.device, dtype=self.dtype)
        # latent norm + key rotation + cache append + query rotation in one launch
        seqlib.latent_rope_store(dkv32, r, dr, mw.dkv_norm, self.eps, cs, spec.rot.dims, pos, slot, cache.block_table, cache.page_size,
                                 pool, q, H, dn, qcat)
        # absorbed keys: qcat[t, h, :r] = q[t, h, :dn] @ W_uk,h  (one problem per head, column slices of both buffers)
        seqlib.linear(q, mw.uk_t, qcat, M=T, N=r, K=dn, ldx=q.stride(0), sx=dn + dr, ldw=dn, sw=r * dn, ldy=H * (r + dr),
                      sy=r + dr, batch=H)
        use_mma = plans is not None and self.tensor_attention and seqlib.latent_attn_mma_ok(H, r, dr, self.dtype)
        olat = torch.empty(T, H, r, device=xb.device, dtype=self.dtype if use_mma else f32)
        if use_mma:
            plan = plans.get(H)
            if plan is None:
                if "decode_parts" in plans:       # decode-only step: the list is written on the device from pos / slot
                    plan = self._decode_plans.get((T, H, plans["decode_parts"]))
                    if plan is None:
                        plan = self._decode_plans[(T, H, plans["decode_parts"])] = seqlib.DecodeAttnPlan(T, H, plans["decode_parts"], xb.device)
                    plan.fill(pos, slot)
                else:
                    plan = seqlib.LatentAttnPlan(plans["portions"], H, xb.device)
                plans[H] = plan
            seqlib.latent_attn_mma(qcat, r, dr, pool, cache.block_table, cache.page_size, plan, mw.sink, spec.scale, olat)
        else:
            seqlib.latent_attn(qcat, r, dr, pool, cache.block_table, cache.page_size, pos, slot, mw.sink, spec.scale, olat)
        # values: attn[t, h*dv:(h+1)*dv] = W_uv,h @ olat[t, h]
        attn = torch.empty(T, H * dv, device=xb.device, dtype=self.dtype)
        seqlib.linear(olat, mw.uv, attn, M=T, N=dv, K=r, ldx=H * r, sx=r, ldw=r, sw=dv * r, ldy=H * dv, sy=dv, batch=H)
        return self._linear(attn, mw.o, f32)

    class _MoeWs:
        pass

    def _grouped_tensor_gemm(self, s: RouterMoeSpec) -> bool:
        """Experts on the grouped tcgen05 GEMM (128-row tiles): bf16, tile-aligned widths, matrices large enough to matter."""
        return (self.tensor_gemm and s.experts > 0 and s.expert_ff % 128 == 0 and self.C % 128 == 0
                and s.expert_ff * self.C >= TENSOR_GEMM_MIN_WEIGHT // 4)

    def _moe_workspace(self, T: int, s: RouterMoeSpec, tile: int):
        bucket = 1 << max(T - 1, 0).bit_length()
        key = (bucket, s.experts, s.identity, s.top, s.expert_ff, tile)
        ws = self._moe_ws.get(key)
        if ws is None:
            dev, i32 = self.device, torch.int32
            ws = VoduzenDecoder._MoeWs()
            ws.max_tiles = seqlib.moe_max_tiles(bucket, s.top, max(s.experts, 1), tile)
            rows = ws.max_tiles * tile
            ws.ids = torch.empty(bucket, s.top, device=dev, dtype=i32)
            ws.w = torch.empty(bucket, s.top, device=dev, dtype=torch.float32)
            ws.gate = torch.empty(bucket, device=dev, dtype=torch.float32)
            ws.counts = torch.zeros(max(s.experts, 1), device=dev, dtype=i32)
            ws.cursor = torch.zeros(max(s.experts, 1), device=dev, dtype=i32)
            ws.seg_start = torch.zeros(max(s.experts, 1) + 1, device=dev, dtype=i32)
            ws.tile_group = torch.empty(ws.max_tiles, device=dev, dtype=i32)
            ws.slot_of = torch.empty(bucket, s.top, device=dev, dtype=i32)
            ws.xs = torch.zeros(rows, self.C, device=dev, dtype=self.dtype)
            ws.act = torch.empty(rows, max(s.expert_ff, 1), device=dev, dtype=self.dtype)
            ws.ys = torch.empty(rows, self.C, device=dev, dtype=torch.float32)
            self._moe_ws[key] = ws
        return ws

    def _moe(self, li: int, xb: torch.Tensor, h32: torch.Tensor, xb_out: Optional[torch.Tensor]):
        """The feed-forward half of layer li, its output norm and the residual add: updates h32 (and xb_out) in place."""
        s, mw, lw = self.cfg.layers[li].mlp, self.w.layers[li].mlp, self.w.layers[li]
        T = xb.shape[0]
        grouped = self._grouped_tensor_gemm(s)
        tile = 128 if grouped else seqlib.LINEAR_TILE
        ws = self._moe_workspace(T, s, tile)
        e_tot = s.experts + s.identity
        z32 = self._linear(xb, mw.router_cat, torch.float32)
        has_gate = s.shared_ff is not None
        seqlib.router_topk(z32, e_tot, s.experts, s.top, mw.correction, has_gate, ws.ids, ws.w, ws.gate, ws.counts)
        ys = None
        if s.experts:
            max_tiles = seqlib.moe_max_tiles(T, s.top, s.experts, tile)
            if T <= SMALL_STEP_ROWS:
                seqlib.moe_plan_scatter_small(ws.counts, s.experts, tile, max_tiles, ws.seg_start, ws.tile_group, xb, ws.ids, s.top,
                                              ws.slot_of, ws.xs)
            else:
                seqlib.moe_plan_tiles(ws.counts, s.experts, tile, max_tiles, ws.seg_start, ws.cursor, ws.tile_group)
                seqlib.moe_scatter_rows(xb, ws.ids, s.top, s.experts, ws.seg_start, ws.cursor, ws.slot_of, ws.xs)
            rows = max_tiles * tile
            if grouped:
                hint = min(max_tiles, T * s.top)
                lib.gemm_grouped(ws.xs[:rows], mw.up, ws.tile_group, ws.act[:rows], lib.EPI_RELU2, hint)
                lib.gemm_grouped(ws.act[:rows], mw.down, ws.tile_group, ws.ys[:rows], lib.EPI_NONE, hint)
            else:
                seqlib.linear(ws.xs, mw.up, ws.act, M=rows, N=s.expert_ff, K=self.C, ldw=self.C, act=seqlib.ACT_RELU2,
                              tile_group=ws.tile_group, group_stride=s.expert_ff * self.C)
                seqlib.linear(ws.act, mw.down, ws.ys, M=rows, N=self.C, K=s.expert_ff, ldw=s.expert_ff, tile_group=ws.tile_group,
                              group_stride=self.C * s.expert_ff)
            ys = ws.ys
        else:
            ws.slot_of.fill_(-1)
        ysh = None
        if has_gate:
            sact = self._linear(xb, mw.shared_up, self.dtype, act=seqlib.ACT_RELU2)
            ysh = self._linear(sact, mw.shared_down, torch.float32)
        seqlib.moe_combine_norm(ys, ws.slot_of, ws.w, s.top, ws.gate if has_gate else None, ysh, lw.norm2, self.eps, h32, xb_out)

    # ---- the step
    @torch.no_grad()
    def step(self, tokens: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, cache: PagedLatentCache,
             want_rows: Optional[torch.Tensor] = None, collect: Optional[list] = None,
             portions: Optional[Sequence] = None, decode_parts: Optional[int] = None) -> Optional[torch.Tensor]:
        """tokens / pos / slot: int32 [T] on the device - row t is token tokens[t] at position pos[t] of the request in cache
        slot slot[t]; rows of one request are consecutive and ascending in position. Appends every row to the cache and returns
        fp32 logits [len(want_rows), vocab] (None when no row is asked for). collect: receives the residual stream after
        every layer (debugging / tests). portions: the same batch as the host knows it, [(first_row, n_rows, slot, first_pos)]
        per request - the tensor-core attention kernel's work list is built from it; without it the plain kernel runs."""
        T = tokens.numel()
        dev = self.device
        plans = {"portions": list(portions)} if portions is not None else None
        if decode_parts is not None:   # every row is a single decoded token of its own request
            plans = {"decode_parts": decode_parts}
        h32 = torch.empty(T, self.C, device=dev, dtype=torch.float32)
        xb = torch.empty(T, self.C, device=dev, dtype=self.dtype)
        seqlib.embed_scale(tokens, self.w.embed, self.cfg.embedding_scale, h32, xb)
        for li, lw in enumerate(self.w.layers):
            y32 = self._mixer(li, xb, pos, slot, cache, plans)
            seqlib.norm_residual(y32, lw.norm1, self.eps, h32, xb)
            if lw.mlp is not None:
                self._moe(li, xb, h32, xb)
            if collect is not None:
                collect.append(h32.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        hw = h32.index_select(0, want_rows)
        xf = seqlib.rms_rows(hw, self.w.final_norm, self.eps, torch.empty(hw.shape[0], self.C, device=dev, dtype=self.dtype),
                             one_plus=True)
        return self._linear(xf, self.w.head, torch.float32, alpha=self.cfg.logit_scale)


    class _Graph:
        pass

    @torch.no_grad()
    def decode_step(self, meta_host: torch.Tensor, cache: PagedLatentCache, max_keys: int) -> torch.Tensor:
        """A decode-only step: meta_host int32 [3, B] (tokens, positions, slots; pinned host memory), one row per request.
        The step is captured once per (B, key-range count, cache) in a CUDA graph and replayed: embedding, all layers against
        the cache (the attention work list is rebuilt on the device from the positions) and the logits of all B rows.
        Returns fp32 logits [B, vocab] (a static buffer, overwritten by the next call)."""
        B = meta_host.shape[1]
        parts = seqlib.DecodeAttnPlan.parts_for(B, max_keys)
        key = (B, parts, id(cache))
        g = self._graphs.get(key)
        if g is not None and g.cache is not cache:
            g = None
        if g is None:
            if len(self._graphs) >= 16:
                self._graphs.pop(next(iter(self._graphs)))
            g = VoduzenDecoder._Graph()
            g.cache = cache
            g.meta = torch.zeros(3, B, device=self.device, dtype=torch.int32)
            g.want = torch.arange(B, device=self.device)
            g.meta.copy_(meta_host, non_blocking=True)
            if not self.use_graph:
                g.graph = None
            else:
                # one eager run first: workspaces, rotary tables and kernel attributes are set up outside the capture (it writes
                # the same cache rows the replay writes again)
                self.step(g.meta[0], g.meta[1], g.meta[2], cache, g.want, decode_parts=parts)
                torch.cuda.synchronize()
                n0 = lib.launch_count()
                g.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g.graph):
                    g.logits = self.step(g.meta[0], g.meta[1], g.meta[2], cache, g.want, decode_parts=parts)
                g.launches = lib.launch_count() - n0
                lib.add_launches(-g.launches)   # the capture does not execute
            self._graphs[key] = g
        else:
            g.meta.copy_(meta_host, non_blocking=True)
        if g.graph is None:
            return self.step(g.meta[0], g.meta[1], g.meta[2], cache, g.want, decode_parts=parts)
        g.graph.replay()
        lib.add_launches(g.launches)
        return g.logits


# ------------------------------------------------------------------------------------------------------------------- model
class VoduzenForCausalLM:
    """Entry point: from_pretrained / from_state_dict, step() for serving loops, generate() for greedy generation."""
    config_class = VoduzenConfig

    def __init__(self, config: VoduzenConfig, weights: VoduzenW, dtype: torch.dtype = torch.bfloat16):
        if not torch.cuda.is_available():
            raise lib.OmcError("omchat_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        seqlib.load()
        self.config, self.weights, self.dtype = config, weights, dtype
        self.device = weights.embed.device
        self.decoder = VoduzenDecoder(config, weights, dtype)
        self.vocab_size = config.vocab_size

    @classmethod
    def from_state_dict(cls, sd, config: VoduzenConfig, device="cuda", dtype: torch.dtype = torch.bfloat16, **unused):
        if not torch.cuda.is_available():
            raise lib.OmcError("omchat_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("compute dtype must be torch.bfloat16 or torch.float32")
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        return cls(config, weights_from_state_dict(sd, config, device, dtype), dtype)

    @classmethod
    def from_pretrained(cls, path: str, config: Optional[VoduzenConfig] = None, device="cuda", dtype: torch.dtype = torch.bfloat16, **kw):
        from .checkpoint import load_checkpoint
        sd, cfg = load_checkpoint(path, config)
        if not isinstance(cfg, VoduzenConfig):
            raise ValueError(f"{path} is not a Voduzen checkpoint")
        return cls.from_state_dict(sd, cfg, device=device, dtype=dtype)

    def eval(self):
        return self

    def step(self, tokens, pos, slot, cache, want_rows=None, collect=None, portions=None):
        with torch.cuda.device(self.device):
            return self.decoder.step(tokens, pos, slot, cache, want_rows, collect, portions)

    def decode_step(self, meta_host, cache, max_keys: int):
        """Decode-only batch (one token per request) through the captured CUDA graph; see VoduzenDecoder.decode_step."""
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
