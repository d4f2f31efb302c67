#!/usr/bin/env python
"""Voduzen decoder at sizes that resemble a real model's layers (random weights), beside the framework's closest existing model,
the Qwen2-MoE decoder, at equal width, depth, heads, experts, top-k, expert and shared widths and vocabulary.

Per size: prefill of `--prefill` x 1024-token prompts as ONE packed step through serving.StepScheduler (tokens/s), decode steps at
batch B and context ctx through the same scheduler (ms/step, tokens/s), and the new kernels timed alone on one layer's shapes
against their rooflines, each beside the like kernel of the Qwen2-MoE path:
  latent attention (tensor-core kernel)  prefill: FLOPs = rows x visible keys x heads x 2 (2 r + dr) against the measured bf16 peak;
                                         decode:  bytes = batch x ctx x (r + dr) x 2 against the measured copy bandwidth
  omc_norm_residual / omc_moe_combine_norm, omc_router_topk: bytes read + written against the copy bandwidth
python tools/bench_voduzen.py --size s --size m
"""
import argparse
import json
import math
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from omchat_b200 import lib, seqlib  # noqa: E402
from omchat_b200.config import VoduzenConfig  # noqa: E402
from omchat_b200.model.voduzen import VoduzenForCausalLM, random_state_dict  # noqa: E402
from omchat_b200.serving import StepScheduler  # noqa: E402

# width, layers, heads, dim, rot_dim, vdim, kv_rank, q_rank, experts, identity, top, expert ff, shared ff, vocab
SIZES = {
    "s": dict(C=2048, L=4, H=16, dn=128, dr=64, dv=128, r=512, qr=1536, E=60, I=4, top=4, ff=1408, sff=5632, V=32768),
    "m": dict(C=4096, L=4, H=32, dn=128, dr=64, dv=128, r=512, qr=1536, E=32, I=2, top=4, ff=2048, sff=4096, V=65536),
}


def config_dict(z):
    def mixer(kind):
        m = {"dim": z["dn"], "heads": z["H"], "kv_rank": z["r"], "rot_dim": z["dr"], "vdim": z["dv"],
             "scale": 1.0 / math.sqrt(z["dn"] + z["dr"]), "rot": {"base": 1e6, "dims": z["dr"]}}
        if kind == "latent_attention_2":
            m["q_rank"] = z["qr"]
        else:
            m["rot"]["scaling"] = {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}
        return m
    mlp = {"kind": "moe", "expert": {"ff": z["ff"]}, "router": {"experts": z["E"], "identity": z["I"], "top": z["top"]},
           "shared": {"ff": z["sff"]}}
    kinds = ["latent_attention", "latent_attention_2"]
    return {"architecture": "Voduzen", "vocab": z["V"], "width": z["C"], "embedding": {"scale": math.sqrt(z["C"])},
            "logit_scale": 1.0, "norm": {"eps": 1e-6},
            "layers": [{"type": kinds[i % 2], "mixer": mixer(kinds[i % 2]), "mlp": mlp} for i in range(z["L"])]}


def peaks():
    hbm, tf = 6535.4, 1400.0
    try:
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        hbm, tf = pk.get("hbm_gbs", hbm), pk.get("bf16_tflops_sustained", pk.get("bf16_tflops", tf))
    except Exception:
        pass
    return hbm, tf


_flush = None


def timed(fn, reps=10, warm=3):
    """Median CUDA-event time of fn() in ms; a 256 MB write between launches evicts L2."""
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(reps):
        _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2]


def kernels(z, n_seq, L, B, ctx):
    """The new kernels alone on one layer's shapes, each beside the like kernel of the Qwen2-MoE path."""
    hbm, tf = peaks()
    dev, bf, f32, i32 = "cuda", torch.bfloat16, torch.float32, torch.int32
    H, r, dr, C = z["H"], z["r"], z["dr"], z["C"]
    D, page = r + dr, 64
    out = {}
    # ---- prefill attention: n_seq x L rows, causal
    T = n_seq * L
    pages_per = L // page
    pool = (torch.randn(n_seq * pages_per + 1, page, D, device=dev) * 0.3).to(bf)
    table = (torch.arange(n_seq * pages_per, dtype=i32, device=dev) + 1).view(n_seq, pages_per).contiguous()
    q = (torch.randn(T, H, D, device=dev) * 0.3).to(bf)
    o = torch.empty(T, H, r, device=dev, dtype=f32)
    plan = seqlib.LatentAttnPlan([(s * L, L, s, 0) for s in range(n_seq)], H, dev)
    ms = timed(lambda: seqlib.latent_attn_mma(q, r, dr, pool, table, page, plan, None, 0.07, o))
    flops = n_seq * H * (L * (L + 1) / 2) * 2 * (2 * r + dr)
    out["latent_attn_prefill"] = {"ms": ms, "tflops": flops / ms / 1e9, "frac_tensor": flops / ms / 1e9 / tf}
    qkv = (torch.randn(T, 3 * H * 128, device=dev) * 0.3).to(bf)
    att = torch.empty(T, H * 128, device=dev, dtype=bf)
    cu = torch.arange(0, T + 1, L, dtype=i32, device=dev)
    ms = timed(lambda: lib.attention(qkv[:, :H * 128], qkv[:, H * 128:2 * H * 128], qkv[:, 2 * H * 128:], att, cu, L, H, H, True, 0.088))
    flops = n_seq * H * (L * (L + 1) / 2) * 4 * 128
    out["qwen2_attn_prefill"] = {"ms": ms, "tflops": flops / ms / 1e9, "frac_tensor": flops / ms / 1e9 / tf}
    del pool, q, o, qkv, att
    # ---- decode attention: B rows, each over ctx cached entries
    pages_per = -(-(ctx + 1) // page)
    pool = (torch.randn(B * pages_per + 1, page, D, device=dev) * 0.3).to(bf)
    table = (torch.arange(B * pages_per, dtype=i32, device=dev) + 1).view(B, pages_per).contiguous()
    q = (torch.randn(B, H, D, device=dev) * 0.3).to(bf)
    o = torch.empty(B, H, r, device=dev, dtype=f32)
    plan = seqlib.LatentAttnPlan([(b, 1, b, ctx) for b in range(B)], H, dev)
    ms = timed(lambda: seqlib.latent_attn_mma(q, r, dr, pool, table, page, plan, None, 0.07, o))
    nbytes = B * (ctx + 1) * D * 2
    out["latent_attn_decode"] = {"batch": B, "ctx": ctx, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm,
                                 "ctas": plan.n_items}
    kvp = (torch.randn(B * pages_per + 1, 2, H, page, 128, device=dev) * 0.3).to(bf)
    qkv = (torch.randn(B, 3 * H * 128, device=dev) * 0.3).to(bf)
    att = torch.empty(B, H * 128, device=dev, dtype=bf)
    lens = torch.full((B,), ctx + 1, dtype=i32, device=dev)
    splits = lib.decode_attn_splits(B, H, ctx + 1)
    ws = lib.decode_attn_workspace(B, H, H, splits, dev)
    inv = torch.ones(64, device=dev)
    ms = timed(lambda: lib.paged_decode_attn(qkv, inv, kvp, table, page, lens, H, H, splits, 0.088, att, ws))
    nbytes = B * (ctx + 1) * 2 * H * 128 * 2
    out["qwen2_attn_decode"] = {"batch": B, "ctx": ctx, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm}
    del pool, q, o, kvp, qkv, att
    # ---- row kernels at prefill size
    y = torch.randn(T, C, device=dev)
    h = torch.randn(T, C, device=dev)
    xb = torch.empty(T, C, device=dev, dtype=bf)
    w = torch.zeros(C, device=dev, dtype=bf)
    ms = timed(lambda: seqlib.norm_residual(y, w, 1e-6, h, xb))
    nbytes = T * C * (4 + 4 + 4 + 2)
    out["norm_residual"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm}
    xin = torch.randn(T, C, device=dev).to(bf)
    xo = torch.empty_like(xin)
    ms = timed(lambda: lib.rmsnorm(xin, w, 1e-6, out=xo))
    nbytes = T * C * 4
    out["qwen2_rmsnorm"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm}
    return out


def measure(size="s", batches=(1, 32), ctx=1024, steps=32, prefill=4, with_kernels=True, with_qwen2=True):
    z = SIZES[size]
    hbm, tf = peaks()
    cfg = VoduzenConfig.from_dict(config_dict(z))
    model = VoduzenForCausalLM.from_state_dict(random_state_dict(cfg, seed=0), cfg, device="cuda:0")
    V, L = z["V"], 1024
    g = torch.Generator().manual_seed(0)
    rec = {"size": size, "dims": z}
    # ---- prefill: `prefill` prompts of 1024 tokens as one packed step
    n0 = lib.launch_count()

    def prefill_once():
        sched = StepScheduler(model, max_tokens=prefill * L, slots=prefill)
        entries = [(f"p{i}", torch.randint(0, V, (L,), generator=g).tolist(), [L - 1]) for i in range(prefill)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        sched.run_step(entries)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)
    for _ in range(2):
        prefill_once()
    n0 = lib.launch_count()
    ms = sorted(prefill_once() for _ in range(3))[1]
    T = prefill * L
    rec["prefill"] = {"tokens": T, "ms": ms, "tokens_per_sec": T / ms * 1e3, "launches": (lib.launch_count() - n0) // 3}
    # ---- decode: B requests at context ctx, one token each per step
    rec["decode"] = []
    for B in batches:
        sched = StepScheduler(model, max_tokens=B * (ctx + steps + 80), slots=B)
        for lo in range(0, B, 8):     # contexts are filled by prefill steps of 8 prompts
            sched.run_step([(f"d{i}", torch.randint(0, V, (ctx,), generator=g).tolist(), []) for i in range(lo, min(B, lo + 8))])
        toks = torch.randint(0, V, (B,), generator=g).tolist()
        for _ in range(3):
            sched.run_step([(f"d{i}", [toks[i]], [0]) for i in range(B)])
        torch.cuda.synchronize()
        n0 = lib.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            lg = sched.run_step([(f"d{i}", [toks[i]], [0]) for i in range(B)])
            toks = lib.argmax(lg).tolist()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        rec["decode"].append({"batch": B, "ctx": ctx, "ms_per_step": ms, "tokens_per_sec": B / ms * 1e3,
                              "launches_per_step": (lib.launch_count() - n0) // steps})
        del sched
    del model
    torch.cuda.empty_cache()
    if with_kernels:
        rec["kernels"] = kernels(z, prefill, L, max(batches), ctx)
    if with_qwen2:
        from tools.bench_moe import measure as measure_moe
        kw = dict(hidden_size=z["C"], num_attention_heads=z["H"], num_key_value_heads=z["H"], num_experts=z["E"],
                  num_experts_per_tok=z["top"], moe_intermediate_size=z["ff"], shared_expert_intermediate_size=z["sff"],
                  vocab_size=z["V"], intermediate_size=z["sff"])
        try:
            rec["qwen2_moe_equal_size"] = measure_moe(layers=z["L"], batches=batches, ctx=ctx, steps=steps, prefill=prefill, cfg_kw=kw)
        except Exception as e:  # noqa: BLE001
            rec["qwen2_moe_equal_size"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", action="append", choices=sorted(SIZES))
    ap.add_argument("--batch", type=int, action="append")
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--prefill", type=int, default=4)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    for s in a.size or ["s"]:
        print(json.dumps(measure(s, tuple(a.batch or [1, 32]), a.ctx, a.steps, a.prefill)), flush=True)


if __name__ == "__main__":
    main()
