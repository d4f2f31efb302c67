#!/usr/bin/env python
"""Tifisun decoder at sizes that resemble a real model's layers (random weights), beside the framework's closest existing model, the
dense Qwen2 decoder (model/decoder.py), at equal width, depth, query / key-value heads, feed-forward width and vocabulary.

Per size: prefill of `--prefill` x 1024-token prompts as ONE packed step through serving.StepScheduler (tokens/s), decode steps at
batch B and context ctx through the same scheduler (ms/step, tokens/s), and the new kernels timed alone on one layer's shapes
against their rooflines, each beside the like kernel of the Qwen2 path:
  omc_linear_state_scan  prefill: FLOPs = rows x heads x 6 dim vdim on the fp32 FMA pipe (nominal 148 SMs x 128 lanes x 2 x clock) and
                         bytes of q, k, v, decay, output against the measured copy bandwidth; decode: the states read and written
  omc_window_attn        prefill: FLOPs = rows x visible keys x heads x 2 (dim + vdim) against the measured bf16 peak (the Qwen2 kernel
                         is the causal tcgen05 flash attention); decode: bytes of the visible keys and values against the copy bandwidth
  omc_post_norm_residual, omc_causal_conv_silu, omc_gated_rms_rows: bytes read + written against the copy bandwidth (like kernel: omc_rmsnorm)
python tools/bench_tifisun.py --size s --size m
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from omchat_b200 import lib, seqlib  # noqa: E402
from omchat_b200.config import TifisunConfig  # noqa: E402
from omchat_b200.model.tifisun import TifisunForCausalLM, random_state_dict  # noqa: E402
from omchat_b200.serving import StepScheduler  # noqa: E402
from tools.bench_voduzen import peaks, timed  # noqa: E402

# width, layers, heads, key/value heads of the windowed attention (and query/key heads of the delta layers), head widths, window, ff, vocab
SIZES = {
    "s": dict(C=2048, L=6, H=16, G=4, d=128, dv=128, conv=4, window=512, rank=64, ff=5632, V=32768),
    "m": dict(C=4096, L=6, H=32, G=8, d=128, dv=128, conv=4, window=512, rank=128, ff=8192, V=65536),
}
FMA_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12   # nominal fp32 FMA peak of the part: what the recurrence runs on


def config_dict(z):
    mlp = {"ff": z["ff"], "kind": "dense"}
    dl = {"conv": z["conv"], "dim": z["d"], "heads": z["H"], "kv_heads": z["H"] // 2, "vdim": z["dv"]}
    cd = {"conv": z["conv"], "dim": z["d"], "heads": z["H"], "kv_heads": z["H"], "vdim": z["dv"]}
    par = {"left": {"bias_max": z["window"], "dim": z["d"], "heads": z["H"], "kv_heads": z["G"], "mask": {"size": z["window"]},
                    "scale": z["d"] ** -0.5, "softcap": 50.0, "vdim": z["dv"]},
           "right": {"decay": [1.0 - 2.0 ** (-3 - 6 * i / z["H"]) for i in range(z["H"])], "dim": z["d"], "heads": z["H"], "vdim": z["dv"]}}
    kinds = [("delta", dl), ("parallel", par), ("channel_delta", cd)]
    return {"architecture": "Tifisun", "vocab": z["V"], "width": z["C"], "embedding": {"scale": 1.0}, "residual_mult": 0.5,
            "norm": {"eps": 1e-5}, "layers": [{"type": kinds[i % 3][0], "mixer": kinds[i % 3][1], "mlp": mlp} for i in range(z["L"])]}


def kernels(z, n_seq, L, B, ctx):
    """The new kernels alone on one layer's shapes, each beside the like kernel of the Qwen2 path."""
    hbm, tf = peaks()
    dev, bf, f32, i32 = "cuda", torch.bfloat16, torch.float32, torch.int32
    H, G, d, dv, C, W = z["H"], z["G"], z["d"], z["dv"], z["C"], z["window"]
    page, out = 64, {}
    T = n_seq * L
    pos = torch.arange(L, dtype=i32, device=dev).repeat(n_seq)
    slot = torch.arange(n_seq, dtype=i32, device=dev).repeat_interleave(L)
    rb = torch.arange(0, T + 1, L, dtype=i32, device=dev)
    # ---- recurrence, prefill: one decay per head / per channel / constant
    q, k = torch.randn(T, H * d, device=dev) * d ** -0.5, torch.nn.functional.normalize(torch.randn(T, H, d, device=dev), dim=-1).view(T, -1)
    v, o = torch.randn(T, H * dv, device=dev), torch.empty(T, H * dv, device=dev)
    a1, a2, beta = torch.randn(T, H, device=dev), torch.randn(T, H * d, device=dev), torch.randn(T, H, device=dev)
    A_log, dt1, dt2 = torch.full((H,), -2.0, device=dev), torch.full((H,), -2.0, device=dev), torch.full((H * d,), -2.0, device=dev)
    consts = torch.full((H,), 0.99, device=dev)
    state = torch.zeros(max(n_seq, B), H, d, dv, device=dev)
    flops = T * H * 6.0 * d * dv
    for name, kw, extra in (("head", dict(a=a1, A_log=A_log, dt_bias=dt1, beta=beta), T * H * 8),
                            ("channel", dict(a=a2, A_log=A_log, dt_bias=dt2, channel_decay=True, beta=beta), T * H * (d + 1) * 4),
                            ("const", dict(decay_const=consts, silu_in=True), 0)):
        ms = timed(lambda: seqlib.linear_state_scan(q, k, v, state, o, rb, n_seq, pos, slot, H, H, d, dv, **kw))
        nbytes = T * H * (2 * d + 2 * dv) * 4 + extra + 2 * n_seq * H * d * dv * 4
        out[f"state_scan_prefill_{name}"] = {"ms": ms, "tflops": flops / ms / 1e9, "frac_fp32_fma": flops / ms / 1e9 / FMA_TFLOPS,
                                             "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm}
    # the same with silu / the per-channel decays applied by one pass in front (what a step with long portions does)
    ms_map = timed(lambda: seqlib.map_rows(a2, seqlib.MAP_DECAY, A_log, dt2, d))
    a2.uniform_(0.9, 1.0)
    ms = timed(lambda: seqlib.linear_state_scan(q, k, v, state, o, rb, n_seq, pos, slot, H, H, d, dv, a=a2, beta=beta, decay_given=True))
    out["state_scan_prefill_channel_prepared"] = {"ms": ms, "ms_decay_pass": ms_map, "tflops": flops / ms / 1e9, "frac_fp32_fma": flops / ms / 1e9 / FMA_TFLOPS}
    qkv3 = torch.randn(T, 2 * H * d + H * dv, device=dev)
    ms_map = timed(lambda: seqlib.map_rows(qkv3, seqlib.MAP_SILU))
    ms = timed(lambda: seqlib.linear_state_scan(q, k, v, state, o, rb, n_seq, pos, slot, H, H, d, dv, decay_const=consts))
    out["state_scan_prefill_const_prepared"] = {"ms": ms, "ms_silu_pass": ms_map, "tflops": flops / ms / 1e9, "frac_fp32_fma": flops / ms / 1e9 / FMA_TFLOPS}
    del qkv3
    a2.normal_()
    # ---- recurrence, decode: B rows, each reads and writes its states
    posd = torch.full((B,), ctx, dtype=i32, device=dev)
    slotd = torch.arange(B, dtype=i32, device=dev)
    rbd = torch.arange(B + 1, dtype=i32, device=dev)
    ms = timed(lambda: seqlib.linear_state_scan(q[:B], k[:B], v[:B], state, o[:B], rbd, B, posd, slotd, H, H, d, dv, a=a2[:B], A_log=A_log,
                                                dt_bias=dt2, channel_decay=True, beta=beta[:B]))
    nbytes = 2.0 * B * H * d * dv * 4
    out["state_scan_decode"] = {"batch": B, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm}
    del state
    # ---- windowed attention, prefill
    pages_per = L // page
    pool = (torch.randn(n_seq * pages_per + 1, page, G * (d + dv), device=dev) * 0.3).to(bf)
    table = (torch.arange(n_seq * pages_per, dtype=i32, device=dev) + 1).view(n_seq, pages_per).contiguous()
    qb = (torch.randn(T, H * d, device=dev) * 0.3).to(bf)
    att = torch.empty(T, H * dv, device=dev, dtype=bf)
    bias = torch.randn(W, H, device=dev)
    ms = timed(lambda: seqlib.window_attn(qb, H, G, d, dv, pool, table, page, pos, slot, W, d ** -0.5, 50.0, bias, att), reps=5, warm=2)
    visible = n_seq * sum(min(p + 1, W) for p in range(L))
    flops = visible * H * 2.0 * (d + dv)
    out["window_attn_plain_prefill"] = {"ms": ms, "tflops": flops / ms / 1e9, "frac_tensor": flops / ms / 1e9 / tf}
    items = seqlib.window_attn_items([(s_ * L, L, s_, 0) for s_ in range(n_seq)], H // G, dev)
    ms = timed(lambda: seqlib.window_attn_mma(qb, H, G, d, dv, pool, table, page, items, pos, slot, W, d ** -0.5, 50.0, bias, att))
    out["window_attn_prefill"] = {"ms": ms, "tflops": flops / ms / 1e9, "frac_tensor": flops / ms / 1e9 / tf, "ctas": int(items.shape[0]) * G}
    qkv = (torch.randn(T, (H + 2 * G) * 128, device=dev) * 0.3).to(bf)
    cu = torch.arange(0, T + 1, L, dtype=i32, device=dev)
    ms = timed(lambda: lib.attention(qkv[:, :H * 128], qkv[:, H * 128:(H + G) * 128], qkv[:, (H + G) * 128:], att, cu, L, H, G, True, 0.088))
    flops = n_seq * H * (L * (L + 1) / 2) * 4 * 128
    out["qwen2_attn_prefill"] = {"ms": ms, "tflops": flops / ms / 1e9, "frac_tensor": flops / ms / 1e9 / tf}
    del pool, qkv
    # ---- windowed attention, decode
    pages_per = -(-(ctx + 1) // page)
    pool = (torch.randn(B * pages_per + 1, page, G * (d + dv), device=dev) * 0.3).to(bf)
    table = (torch.arange(B * pages_per, dtype=i32, device=dev) + 1).view(B, pages_per).contiguous()
    ms = timed(lambda: seqlib.window_attn(qb[:B], H, G, d, dv, pool, table, page, posd, slotd, W, d ** -0.5, 50.0, bias, att[:B]))
    nbytes = B * min(ctx + 1, W) * G * (d + dv) * 2
    out["window_attn_plain_decode"] = {"batch": B, "ctx": ctx, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm}
    ms = timed(lambda: seqlib.window_attn_mma(qb[:B], H, G, d, dv, pool, table, page, None, posd, slotd, W, d ** -0.5, 50.0, bias, att[:B]))
    out["window_attn_decode"] = {"batch": B, "ctx": ctx, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm, "ctas": B * G}
    kvp = (torch.randn(B * pages_per + 1, 2, G, page, 128, device=dev) * 0.3).to(bf)
    qkv = (torch.randn(B, (H + 2 * G) * 128, device=dev) * 0.3).to(bf)
    lens = torch.full((B,), ctx + 1, dtype=i32, device=dev)
    splits = lib.decode_attn_splits(B, H, ctx + 1)
    ws = lib.decode_attn_workspace(B, H, G, splits, dev)
    inv = torch.ones(64, device=dev)
    try:
        ms = timed(lambda: lib.paged_decode_attn(qkv, inv, kvp, table, page, lens, H, G, splits, 0.088, att[:B], ws))
        nbytes = B * (ctx + 1) * 2 * G * 128 * 2
        out["qwen2_attn_decode"] = {"batch": B, "ctx": ctx, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm}
    except Exception as e:  # noqa: BLE001
        out["qwen2_attn_decode"] = {"error": f"{type(e).__name__}: {e}"[:200]}
    del pool, kvp, qkv
    # ---- row kernels at prefill size
    y, h = torch.randn(T, C, device=dev), torch.randn(T, C, device=dev)
    xb = torch.empty(T, C, device=dev, dtype=bf)
    w = torch.zeros(C, device=dev, dtype=bf)
    ms = timed(lambda: seqlib.post_norm_residual(y, w, 1e-5, 0.7, h, w, xb))
    nbytes = T * C * (4 + 4 + 4 + 2)
    out["post_norm_residual"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm}
    ms = timed(lambda: seqlib.post_norm_residual(y, w, 1e-5, 0.7, h, w, xb, y2=y, wa=w, wb=w))
    out["post_norm_residual_pair"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm}
    xin = torch.randn(T, C, device=dev).to(bf)
    xo = torch.empty_like(xin)
    ms = timed(lambda: lib.rmsnorm(xin, w, 1e-6, out=xo))
    nbytes = T * C * 4
    out["qwen2_rmsnorm"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm}
    ch = (H + H) * d + H * dv
    xz, yz = torch.randn(T, ch, device=dev), torch.empty(T, ch, device=dev)
    cw = torch.randn(ch, z["conv"], device=dev).to(bf)
    cst = torch.zeros(n_seq, z["conv"] - 1, ch, device=dev)
    ms = timed(lambda: seqlib.causal_conv_silu(xz, cw, pos, slot, cst, yz, unit_channels=2 * H * d, unit_group=d, scaled_channels=H * d, unit_mult=d ** -0.5))
    nbytes = T * ch * 8
    out["causal_conv_silu"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm}
    on = torch.empty(T, H * dv, device=dev, dtype=bf)
    nw = torch.ones(dv, device=dev, dtype=bf)
    ms = timed(lambda: seqlib.gated_rms_rows(o, H, dv, nw, 1e-5, v, seqlib.GATE_SILU, on))
    nbytes = T * H * dv * (4 + 4 + 2)
    out["gated_rms_rows"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / hbm}
    return out


def qwen2_dense(z, batches, ctx, steps, prefill):
    """The dense Qwen2 decoder at equal sizes: prefill of `prefill` x 1024 tokens and greedy decode steps (its own serving path)."""
    from omchat_b200.config import OmChatQwen2Config
    from omchat_b200.model.decoder import Qwen2Decoder
    from omchat_b200.model.weights import random_init
    lib.load()
    cfg = OmChatQwen2Config(num_hidden_layers=z["L"], mm_vision_tower=None, hidden_size=z["C"], num_attention_heads=z["C"] // 128,
                            num_key_value_heads=z["G"], intermediate_size=z["ff"], vocab_size=z["V"])
    w = random_init(cfg, device="cuda:0", vision=False)
    dec = Qwen2Decoder(cfg, w.llm)
    out = []
    n, L, C = prefill, 1024, z["C"]
    T = n * L
    emb = (torch.randn(T, C, device="cuda") * 0.5).to(torch.bfloat16)
    pos = torch.arange(L, dtype=torch.int32, device="cuda").repeat(n)
    seq = torch.arange(n, dtype=torch.int32, device="cuda").repeat_interleave(L)
    offs = [i * L for i in range(n + 1)]
    cache = dec.new_cache(n, L + 16)
    for _ in range(2):
        dec.prefill(emb.clone(), pos, seq, offs, cache, logits="last")
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        dec.prefill(emb.clone(), pos, seq, offs, cache, logits="last")
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 3
    out.append({"phase": "prefill", "tokens": T, "ms": ms, "tokens_per_sec": T / ms * 1e3})
    del cache, emb
    for B in batches:
        try:
            cache = dec.new_cache(B, ctx + 2 * steps + 16)
            cache.host_lens = [ctx] * B
            cache.ctx_lens.fill_(ctx)
            cache.pool.normal_(0, 0.5)
            toks = torch.randint(0, cfg.vocab_size, (B,), device="cuda:0")
            dec.generate_greedy(toks, cache, 8)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dec.generate_greedy(toks, cache, steps)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
            out.append({"phase": "decode", "batch": B, "ctx": ctx, "ms_per_step": ms, "tokens_per_sec": B / ms * 1e3})
            del cache
        except Exception as e:  # noqa: BLE001  (a decode path of that model that does not take these sizes)
            out.append({"phase": "decode", "batch": B, "error": f"{type(e).__name__}: {e}"[:200]})
    dec.release()
    return out


def measure(size="s", batches=(1, 32), ctx=1024, steps=32, prefill=4, with_kernels=True, with_qwen2=True):
    z = SIZES[size]
    cfg = TifisunConfig.from_dict(config_dict(z))
    model = TifisunForCausalLM.from_state_dict(random_state_dict(cfg, seed=0, decay_rank=z["rank"], gate_rank=z["rank"], bias_rows=32), cfg,
                                               device="cuda:0")
    V, L = z["V"], 1024
    g = torch.Generator().manual_seed(0)
    rec = {"size": size, "dims": z}

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
        try:
            rec["qwen2_equal_size"] = qwen2_dense(z, batches, ctx, steps, prefill)
        except Exception as e:  # noqa: BLE001
            rec["qwen2_equal_size"] = {"error": f"{type(e).__name__}: {e}"[:300]}
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
