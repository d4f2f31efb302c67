"""Tifisun on the GPU against the plain restatement in oracle/tifisun_oracle.py (float64, whole sequences, token-by-token loops).

Small configurations of their own, random weights, and engineered weights or inputs where random ones would hide a fault: a key
that dominates just inside / just outside the attention window, decays close to one so that a token hundreds of positions back
still shows in the state, states poisoned with NaN before a slot is used again.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():  # collected on the CPU box too
    pytest.skip("needs a CUDA device", allow_module_level=True)

from omchat_b200 import seqlib  # noqa: E402
from omchat_b200.config import TifisunConfig  # noqa: E402
from omchat_b200.model.tifisun import TifisunForCausalLM, random_state_dict  # noqa: E402
from omchat_b200.serving import StepScheduler  # noqa: E402
from oracle import tifisun_oracle as O  # noqa: E402

DEV = "cuda:0"
F64 = torch.float64


def delta(heads, kv_heads, dim, vdim, conv, ff=40, channel=False, **extra):
    d = {"type": "channel_delta" if channel else "delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim},
         "mlp": {"ff": ff, "kind": "dense"} if ff else None}
    d.update(extra)
    return d


def parallel(heads, kv_heads, dim, vdim, window, rheads, rdim, rvdim, decay, softcap=12.0, bias_max=50, ff=40, **extra):
    d = {"type": "parallel", "mixer": {
        "left": {"bias_max": bias_max, "dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window}, "scale": dim ** -0.5,
                 "softcap": softcap, "vdim": vdim},
        "right": {"decay": decay, "dim": rdim, "heads": rheads, "vdim": rvdim}}, "mlp": {"ff": ff, "kind": "dense"} if ff else None}
    d.update(extra)
    return d


def config_a(page=16):
    """Every mixer kind, a shared layer, a layer without feed-forward, widths that are no multiples of 32, grouped heads."""
    return {"architecture": "Tifisun", "vocab": 150, "width": 96, "embedding": {"scale": 2.5}, "residual_mult": 0.6, "norm": {"eps": 1e-5},
            "kv_page_size": page, "layers": [
                delta(4, 2, 24, 40, 4),
                parallel(6, 2, 20, 12, 19, 3, 24, 20, [0.7, 0.97, 0.999]),
                delta(2, 1, 40, 24, 2, channel=True, ff=56),
                delta(4, 2, 24, 40, 4, weights_of=0),
                parallel(6, 2, 20, 12, 19, 3, 24, 20, [0.7, 0.97, 0.999], ff=0)]}


def config_b(page=32):
    """Ones and equal values: one head everywhere, a convolution of one tap (no ring), a window of one key, value width = key width."""
    return {"architecture": "Tifisun", "vocab": 67, "width": 64, "embedding": {"scale": 1.0}, "residual_mult": 1.0, "norm": {"eps": 1e-6},
            "kv_page_size": page, "layers": [
                parallel(1, 1, 16, 16, 1, 1, 16, 16, [0.9], softcap=50.0, bias_max=4),
                delta(1, 1, 16, 16, 1, ff=0),
                delta(1, 1, 8, 8, 5, channel=True, ff=24)]}


def config_c(page=16):
    """Wide heads (key widths above 64 and above 128), a window longer than several pages, parallel layer first."""
    return {"architecture": "Tifisun", "vocab": 90, "width": 80, "embedding": {"scale": 4.0}, "residual_mult": 0.8, "norm": {"eps": 1e-5},
            "kv_page_size": page, "layers": [
                parallel(2, 1, 72, 40, 70, 2, 136, 24, [0.5, 0.995], softcap=5.0, bias_max=64),
                delta(3, 3, 72, 33, 3),
                delta(2, 2, 136, 16, 3, channel=True, ff=0, ),
                parallel(2, 1, 72, 40, 70, 2, 136, 24, [0.5, 0.995], softcap=5.0, bias_max=64, weights_of=0)]}


def config_d(page=16):
    """Attention shapes the tensor-core kernel takes (bf16): grouped heads, a window over several key tiles, two such layers."""
    return {"architecture": "Tifisun", "vocab": 110, "width": 64, "embedding": {"scale": 3.5}, "residual_mult": 0.75, "norm": {"eps": 1e-5},
            "kv_page_size": page, "layers": [
                parallel(4, 2, 32, 16, 75, 2, 16, 32, [0.9, 0.99], softcap=20.0, bias_max=80),
                delta(2, 2, 32, 32, 4),
                parallel(8, 1, 16, 64, 9, 1, 32, 16, [0.97], softcap=20.0, bias_max=20, ff=0)]}


def build(cfg_dict, dtype, seed=0, edit=None, bias_rows=10):
    cfg = TifisunConfig.from_dict(cfg_dict)
    sd = random_state_dict(cfg, seed=seed, decay_rank=12, gate_rank=20, bias_rows=bias_rows)
    if edit:
        edit(sd)
    return TifisunForCausalLM.from_state_dict(sd, cfg, device=DEV, dtype=dtype), sd


def oracle_logits(cfg_dict, sd, tokens, collect=None):
    return O.forward(cfg_dict, sd, tokens, collect)


def rel_err(got, want):
    """RMS difference of mean-free logits relative to the RMS of the reference row."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)).max())


def tokens_for(cfg_dict, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg_dict["vocab"], (n,), generator=g).tolist()


TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


def run_schedule(model, steps, max_tokens, slots=4):
    """steps: [[(key, tokens, want)], end-keys]. Returns {key: [logit rows in the order they came]}."""
    sched = StepScheduler(model, max_tokens=max_tokens, slots=slots)
    out = {}
    for entries, end in steps:
        lg = sched.run_step(entries, end)
        at = 0
        for key, _, want in entries:
            for _ in want:
                out.setdefault(key, []).append(lg[at].float().cpu().clone())
                at += 1
    return out, sched


# ------------------------------------------------------------------------------------------------------- each mechanism alone
def _dev(t, dt=torch.float32):
    return t.to(device=DEV, dtype=dt).contiguous()


def _rows(portions):
    """[(slot, first_pos, n)] -> pos, slot, row_begin (device int32) of the packed rows."""
    pos, slot, rb = [], [], [0]
    for s, p0, n in portions:
        pos += range(p0, p0 + n)
        slot += [s] * n
        rb.append(rb[-1] + n)
    i32 = dict(device=DEV, dtype=torch.int32)
    return torch.tensor(pos, **i32), torch.tensor(slot, **i32), torch.tensor(rb, **i32)


@pytest.mark.parametrize("taps,ch,group", [(4, 48, 12), (2, 40, 8), (1, 24, 24), (7, 36, 0)])
def test_causal_conv_alone_and_in_portions(taps, ch, group):
    g = torch.Generator().manual_seed(taps)
    T = 23
    x = torch.randn(2, T, ch, generator=g, dtype=F64)
    w = torch.randn(ch, taps, generator=g, dtype=F64)
    unit = (ch // group // 2) * group * 2 if group else 0      # the leading `unit` channels become unit vectors, half of them scaled
    want = []
    for b in range(2):
        y = O.silu(O.causal_conv(x[b], w))
        if unit:
            u = O.unit_vectors(y[:, :unit], unit // group)
            u[:, :unit // 2] *= 0.37
            y = torch.cat([u, y[:, unit:]], dim=1)
        want.append(y)
    state = torch.full((3, max(taps - 1, 1), ch), float("nan"), device=DEV) if taps > 1 else None   # stale contents must never be read
    got = [torch.zeros(T, ch, dtype=F64), torch.zeros(T, ch, dtype=F64)]
    # request 0 in slot 2 in portions of 2, 1, 9, 11 tokens; request 1 in slot 0 as 20 + 3; the steps interleave them
    plan = [[(2, 0, 0, 2), (0, 1, 0, 20)], [(2, 0, 2, 1)], [(0, 1, 20, 3), (2, 0, 3, 9)], [(2, 0, 12, 11)]]
    for step in plan:
        pos, slot, _ = _rows([(s, p0, n) for s, _, p0, n in step])
        xin = torch.cat([x[b, p0:p0 + n] for _, b, p0, n in step])
        xin = torch.cat([_dev(xin), torch.zeros(xin.shape[0], 5, device=DEV)], dim=1)          # a column slice of a wider buffer
        y = torch.empty(xin.shape[0], ch, device=DEV)
        seqlib.causal_conv_silu(xin[:, :ch], _dev(w), pos, slot, state, y, unit_channels=unit, unit_group=group, unit_eps=1e-6,
                                scaled_channels=unit // 2, unit_mult=0.37, single_rows=all(n == 1 for _, _, _, n in step))
        at = 0
        for _, b, p0, n in step:
            got[b][p0:p0 + n] = y[at:at + n].double().cpu()
            at += n
    for b in range(2):
        assert torch.allclose(got[b], want[b], atol=2e-5, rtol=1e-5), (got[b] - want[b]).abs().max()


@pytest.mark.parametrize("dim,vdim,H,G,mode", [(24, 40, 4, 2, "head"), (72, 33, 3, 3, "channel"), (136, 16, 2, 1, "channel"), (16, 64, 2, 2, "const"),
                                               (200, 8, 1, 1, "head"), (8, 8, 1, 1, "const")])
def test_linear_state_scan_against_token_loop(dim, vdim, H, G, mode):
    g = torch.Generator().manual_seed(dim + vdim)
    T = 37
    q = torch.randn(T, G * dim, generator=g, dtype=F64) * 0.5
    k = torch.randn(T, G * dim, generator=g, dtype=F64)
    if mode != "const":     # the delta rule is a contraction only for keys of at most unit length (the model feeds it unit vectors)
        k = O.unit_vectors(k, G)
    v = torch.randn(T, H * vdim, generator=g, dtype=F64)
    A_log = torch.randn(H, generator=g, dtype=F64) - 1.5
    a = torch.randn(T, H * dim if mode == "channel" else H, generator=g, dtype=F64)
    dtb = torch.randn(H * dim if mode == "channel" else H, generator=g, dtype=F64) - 1.0
    beta_raw = torch.randn(T, H, generator=g, dtype=F64)
    consts = torch.rand(H, generator=g, dtype=F64) * 0.5 + 0.5
    want = torch.zeros(T, H * vdim, dtype=F64)
    for h in range(H):
        kv = h // (H // G)
        qh, kh, vh = q[:, kv * dim:(kv + 1) * dim], k[:, kv * dim:(kv + 1) * dim], v[:, h * vdim:(h + 1) * vdim]
        if mode == "const":
            want[:, h * vdim:(h + 1) * vdim] = O.decayed_outer_sum(O.silu(qh), O.silu(kh), O.silu(vh), float(consts[h]))
        else:
            if mode == "channel":
                gd = torch.exp(-torch.exp(A_log[h]) * O.softplus(a[:, h * dim:(h + 1) * dim] + dtb[h * dim:(h + 1) * dim]))
            else:
                gd = torch.exp(-torch.exp(A_log[h]) * O.softplus(a[:, h] + dtb[h]))[:, None].expand(T, dim)
            want[:, h * vdim:(h + 1) * vdim] = O.delta_rule(qh, kh, vh, gd, torch.sigmoid(beta_raw[:, h]))
    state = torch.full((3, H, dim, vdim), float("nan"), device=DEV)
    got = torch.zeros(T, H * vdim, dtype=F64)
    cuts = [0, 1, 3, 19, 20, 36, 37]       # portions of 1, 2, 16, 1, 16, 1 tokens: chunk edges of the kernel's staging included
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        # the request in slot 1 beside a one-token request that starts fresh in slot 0 every step (it must not disturb slot 1)
        pos, slot, rb = _rows([(0, 0, 1), (1, lo, hi - lo)])
        pad = lambda t: torch.cat([_dev(t[:1]), _dev(t[lo:hi])])
        out = torch.empty(1 + hi - lo, H * vdim, device=DEV)
        kw = dict(decay_const=_dev(consts), silu_in=True) if mode == "const" else dict(
            a=pad(a), A_log=_dev(A_log), dt_bias=_dev(dtb), channel_decay=mode == "channel", beta=pad(beta_raw))
        seqlib.linear_state_scan(pad(q), pad(k), pad(v), state, out, rb, 2, pos, slot, H, G, dim, vdim, **kw)
        got[lo:hi] = out[1:].double().cpu()
    assert torch.allclose(got, want, atol=3e-5, rtol=2e-5), (got - want).abs().max()


@pytest.mark.parametrize("groups,n,act", [(4, 40, 1), (1, 60, 2), (11, 7, 0)])
def test_gated_rms_rows(groups, n, act):
    g = torch.Generator().manual_seed(n)
    x, gate, w = torch.randn(9, groups * n, generator=g, dtype=F64), torch.randn(9, groups * n, generator=g, dtype=F64), torch.randn(n, generator=g, dtype=F64)
    a = {0: gate, 1: O.silu(gate), 2: torch.sigmoid(gate)}[act]
    want = (O.norm_plain(x.view(9, groups, n), w, 1e-5) * a.view(9, groups, n)).reshape(9, -1)
    out = torch.empty(9, groups * n, device=DEV)
    seqlib.gated_rms_rows(_dev(x), groups, n, _dev(w), 1e-5, _dev(gate), act, out)
    assert torch.allclose(out.double().cpu(), want, atol=1e-5, rtol=1e-5)


def test_post_norm_residual_single_and_pair():
    g = torch.Generator().manual_seed(5)
    C, T = 70, 6
    y1, y2, h = (torch.randn(T, C, generator=g, dtype=F64) for _ in range(3))
    wa, wb, wp, wn = (torch.randn(C, generator=g, dtype=F64) * 0.3 for _ in range(4))
    for pair in (False, True):
        y = 0.5 * (O.norm_plain(y1, wa, 1e-5) + O.norm_plain(y2, wb, 1e-5)) if pair else y1
        h_want = h + 0.7 * O.norm_zero_centred(y, wp, 1e-5)
        for nxt in (False, True):
            hd, xb = _dev(h), torch.empty(T, C, device=DEV)
            seqlib.post_norm_residual(_dev(y1), _dev(wp), 1e-5, 0.7, hd, _dev(wn) if nxt else None, xb, y2=_dev(y2) if pair else None,
                                      wa=_dev(wa) if pair else None, wb=_dev(wb) if pair else None)
            assert torch.allclose(hd.double().cpu(), h_want, atol=1e-5)
            assert torch.allclose(xb.double().cpu(), O.norm_zero_centred(h_want, wn, 1e-5) if nxt else h_want, atol=1e-5)


def test_linear_bias_and_gated_halves():
    g = torch.Generator().manual_seed(6)
    x, w, b = torch.randn(70, 33, generator=g), torch.randn(2 * 19, 33, generator=g), torch.randn(2 * 19, generator=g)
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        xd, wd, bd = _dev(x, dt), _dev(w, dt), _dev(b, dt)
        z = seqlib.linear(xd, wd, torch.empty(70, 38, device=DEV), bias=bd)
        want = xd.double().cpu() @ wd.double().cpu().T + bd.double().cpu()
        assert torch.allclose(z.double().cpu(), want, atol=tol, rtol=tol)
        z = z.to(dt)                                        # the gated halves are read in either dtype
        out = seqlib.glu_mul(z, 19, seqlib.ACT_GELU_TANH, torch.empty(70, 19, device=DEV))
        zz = z.double().cpu()
        assert torch.allclose(out.double().cpu(), O.gelu_tanh(zz[:, :19]) * zz[:, 19:], atol=1e-5, rtol=1e-5)
    # four columns per thread when the halves are a multiple of four wide
    for dt in (torch.float32, torch.bfloat16):
        z = _dev(torch.randn(33, 2 * 24, generator=g), dt)
        for odt in (torch.float32, torch.bfloat16):
            out = seqlib.glu_mul(z, 24, seqlib.ACT_GELU_TANH, torch.empty(33, 24, device=DEV, dtype=odt))
            zz = z.double().cpu()
            assert torch.allclose(out.double().cpu(), O.gelu_tanh(zz[:, :24]) * zz[:, 24:], atol=1e-5 if odt == torch.float32 else 2e-2, rtol=1e-2)
    # the aligned bf16 shape takes the tensor-core kernel of the library: same check there
    x, w, b = torch.randn(130, 64, generator=g), torch.randn(136, 64, generator=g), torch.randn(136, generator=g)
    xd, wd, bd = _dev(x, torch.bfloat16), _dev(w, torch.bfloat16), _dev(b, torch.bfloat16)
    z = seqlib.linear(xd, wd, torch.empty(130, 136, device=DEV), bias=bd, act=seqlib.ACT_GELU_TANH)
    want = O.gelu_tanh(xd.double().cpu() @ wd.double().cpu().T + bd.double().cpu())
    assert torch.allclose(z.double().cpu(), want, atol=2e-3, rtol=2e-3)


def _window_case(H, G, d, dv, window, page, softcap, dtype, q, k, v, rel, far, cuts, wq=None, wk=None, mma=False):
    """Runs store + attention over `cuts` portions of one request on shuffled pages; returns [T, H * dv] float64. mma: the
    tensor-core kernel (portions of one token go through its list-free decode form)."""
    T = q.shape[0]
    n_pages = -(-T // page) + 2
    pool = torch.full((n_pages, page, G * (d + dv)), float("nan"), device=DEV, dtype=dtype)
    table = torch.zeros(3, n_pages, dtype=torch.int32)
    table[2, :n_pages - 1] = torch.tensor(list(range(n_pages - 1, 0, -1)), dtype=torch.int32)    # descending page ids, page 0 unused
    table = table.to(DEV)
    from omchat_b200.config import WindowAttentionSpec
    idx = [WindowAttentionSpec.bucket(n, rel.shape[0], far) for n in range(window)]
    bias = _dev(rel)[torch.tensor(idx, device=DEV)].contiguous()
    wq = torch.ones(H * d, dtype=F64) if wq is None else wq
    wk = torch.ones(G * d, dtype=F64) if wk is None else wk
    out = torch.zeros(T, H * dv, dtype=F64)
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        pos, slot, _ = _rows([(2, lo, hi - lo)])
        qo = torch.empty(hi - lo, H * d, device=DEV, dtype=dtype)
        seqlib.qk_norm_kv_store(_dev(q[lo:hi]), _dev(wq, dtype), _dev(k[lo:hi]), _dev(wk, dtype), _dev(v[lo:hi]), 1e-5, pos, slot, table, page, pool, qo)
        o = torch.empty(hi - lo, H * dv, device=DEV, dtype=dtype)
        if mma:
            items = None if hi - lo == 1 else seqlib.window_attn_items([(0, hi - lo, 2, lo)], H // G, DEV)
            seqlib.window_attn_mma(qo, H, G, d, dv, pool, table, page, items, pos, slot, window, d ** -0.5, softcap, bias, o)
        else:
            seqlib.window_attn(qo, H, G, d, dv, pool, table, page, pos, slot, window, d ** -0.5, softcap, bias, o)
        out[lo:hi] = o.double().cpu()
    return out


@pytest.mark.parametrize("H,G,d,dv,window,page", [(6, 2, 20, 12, 19, 16), (1, 1, 16, 16, 1, 8), (2, 1, 72, 40, 70, 16), (4, 4, 8, 200, 5, 4)])
def test_window_attention_random(H, G, d, dv, window, page):
    g = torch.Generator().manual_seed(window)
    T = 83
    q, k, v = torch.randn(T, H * d, generator=g, dtype=F64), torch.randn(T, G * d, generator=g, dtype=F64), torch.randn(T, G * dv, generator=g, dtype=F64)
    wq, wk = torch.rand(H * d, generator=g, dtype=F64) + 0.5, torch.rand(G * d, generator=g, dtype=F64) + 0.5
    rel = torch.randn(10, H, generator=g, dtype=F64)
    want = O.windowed_attention(O.norm_plain(q, wq, 1e-5), O.norm_plain(k, wk, 1e-5), v, H, G, d ** -0.5, 7.0, rel, 40.0, window)
    got = _window_case(H, G, d, dv, window, page, 7.0, torch.float32, q, k, v, rel, 40.0, [0, 1, 3, 40, 41, 83], wq, wk)
    assert torch.allclose(got, want, atol=3e-5, rtol=1e-4), (got - want).abs().max()
    got = _window_case(H, G, d, dv, window, page, 7.0, torch.bfloat16, q, k, v, rel, 40.0, [0, 83], wq, wk)
    assert torch.allclose(got, want, atol=6e-2, rtol=6e-2)


@pytest.mark.parametrize("H,G,d,dv,window,page", [(4, 2, 32, 16, 37, 16), (2, 2, 64, 64, 70, 8), (8, 1, 16, 128, 100, 32), (16, 4, 128, 128, 130, 64),
                                                  (1, 1, 48, 32, 64, 16), (64, 1, 16, 16, 5, 16)])
def test_window_attention_tensor_core(H, G, d, dv, window, page):
    assert seqlib.window_attn_mma_ok(H, G, d, dv, torch.bfloat16) and not seqlib.window_attn_mma_ok(H, G, d + 4, dv, torch.bfloat16)
    g = torch.Generator().manual_seed(window + H)
    T = 150
    q, k, v = torch.randn(T, H * d, generator=g, dtype=F64), torch.randn(T, G * d, generator=g, dtype=F64), torch.randn(T, G * dv, generator=g, dtype=F64)
    rel = torch.randn(10, H, generator=g, dtype=F64)
    # bf16-rounded inputs on both sides: what is left is the rounding of the probabilities and the hardware tanh
    r16 = lambda t: t.to(torch.bfloat16).double()
    ones_q, ones_k = torch.ones(H * d, dtype=F64), torch.ones(G * d, dtype=F64)
    want = O.windowed_attention(r16(O.norm_plain(q, ones_q, 1e-5)), r16(O.norm_plain(k, ones_k, 1e-5)), r16(v), H, G, d ** -0.5, 7.0, rel, 40.0, window)
    for cuts in ([0, T], [0, 1, 3, 70, 71, 72, 149, 150]):     # whole; portions with single decoded tokens between them
        got = _window_case(H, G, d, dv, window, page, 7.0, torch.bfloat16, q, k, v, rel, 40.0, cuts, mma=True)
        assert torch.allclose(got, want, atol=2.5e-2, rtol=2.5e-2), (cuts, (got - want).abs().max())


@pytest.mark.parametrize("edge", ["inside", "outside"])
@pytest.mark.parametrize("decoded", [False, True])
def test_window_edge_key_on_the_tensor_core_kernel(edge, decoded):
    H, G, d, dv, window, page, T = 2, 1, 16, 16, 70, 16, 200          # the window spans more than one key tile
    g = torch.Generator().manual_seed(3)
    k = torch.randn(T, d, generator=g, dtype=F64) * 0.05
    v = torch.randn(T, dv, generator=g, dtype=F64)
    q = torch.randn(T, H * d, generator=g, dtype=F64) * 0.05
    i = T - 1
    j = i - window + 1 if edge == "inside" else i - window
    e = torch.zeros(d, dtype=F64)
    e[3] = 1.0
    k[:, 3] = 0.0
    k[j] = e
    q[i] = torch.cat([e, e])
    rel = torch.zeros(10, H, dtype=F64)
    wq = torch.full((H * d,), 5.0, dtype=F64)
    got = _window_case(H, G, d, dv, window, page, 1000.0, torch.bfloat16, q, k, v, rel, 40.0, [0, T - 1, T] if decoded else [0, T], wq=wq, mma=True)
    if edge == "inside":
        assert torch.allclose(got[i, :dv], v[j], atol=0.05)
    else:
        assert (got[i, :dv] - v[j]).abs().max() > 0.3


@pytest.mark.parametrize("edge", ["inside", "outside"])
@pytest.mark.parametrize("decoded", [False, True])
def test_window_edge_key_dominates_or_is_unseen(edge, decoded):
    """The key `window - 1` back is the last one seen: when it carries the query's direction it takes the whole softmax; the key
    one further back carries it in the other case and must not matter at all."""
    H, G, d, dv, window, page, T = 2, 1, 16, 8, 21, 16, 64
    g = torch.Generator().manual_seed(3)
    k = torch.randn(T, d, generator=g, dtype=F64) * 0.05
    v = torch.randn(T, dv, generator=g, dtype=F64)
    q = torch.randn(T, H * d, generator=g, dtype=F64) * 0.05
    i = T - 1
    j = i - window + 1 if edge == "inside" else i - window
    e = torch.zeros(d, dtype=F64)
    e[3] = 1.0
    k[:, 3] = 0.0                 # every other key is orthogonal to the query: score 0
    k[j] = e
    q[i] = torch.cat([e, e])      # after the norms: one component of 4 in the query's heads and in that key; the weight makes it 20
    rel = torch.zeros(10, H, dtype=F64)
    cuts = [0, T - 1, T] if decoded else [0, T]
    wq = torch.full((H * d,), 5.0, dtype=F64)
    got = _window_case(H, G, d, dv, window, page, 1000.0, torch.float32, q, k, v, rel, 40.0, cuts, wq=wq)
    want = O.windowed_attention(O.norm_plain(q, wq, 1e-5), O.norm_plain(k, torch.ones(d, dtype=F64), 1e-5), v, H, G,
                                d ** -0.5, 1000.0, rel, 40.0, window)
    assert torch.allclose(got[i], want[i], atol=1e-4)
    if edge == "inside":
        assert torch.allclose(got[i, :dv], v[j], atol=0.15)       # the softmax sits on that key
    else:
        assert (got[i, :dv] - v[j]).abs().max() > 0.3             # an unseen key leaves no trace


def test_distance_bias_buckets_show_in_the_scores():
    """A bias of +20 on one bucket puts the softmax on the keys of exactly that distance range."""
    from omchat_b200.config import WindowAttentionSpec
    H, G, d, dv, window, page, T = 1, 1, 8, 8, 40, 16, 60
    rows, far = 12, 36.0
    g = torch.Generator().manual_seed(4)
    q, k = torch.randn(T, d, generator=g, dtype=F64) * 0.01, torch.randn(T, d, generator=g, dtype=F64) * 0.01
    v = torch.randn(T, dv, generator=g, dtype=F64)
    for b in (0, 5, 6, 9, 11):
        rel = torch.zeros(rows, H, dtype=F64)
        rel[b] = 20.0
        got = _window_case(H, G, d, dv, window, page, 30.0, torch.float32, q, k, v, rel, far, [0, 50, T])
        want = O.windowed_attention(O.norm_plain(q, torch.ones(d, dtype=F64), 1e-5), O.norm_plain(k, torch.ones(d, dtype=F64), 1e-5), v, H, G,
                                    d ** -0.5, 30.0, rel, far, window)
        assert torch.allclose(got, want, atol=1e-4), b
        assert [O.distance_bucket(n, rows, far) for n in range(window)] == [WindowAttentionSpec.bucket(n, rows, far) for n in range(window)]


# --------------------------------------------------------------------------------------------------------------- whole model
CONFIGS = {"a": config_a, "b": config_b, "c": config_c, "d": config_d}


@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layers_and_logits_against_oracle(name, dtype):
    cd = CONFIGS[name]()
    model, sd = build(cd, dtype, seed=1)
    toks = tokens_for(cd, 90, 2)
    want_layers = []
    want = oracle_logits(cd, sd, toks, want_layers)
    T = len(toks)
    cache = model.decoder.new_cache(8, 2)
    cache.set_pages(1, 0, [5, 2, 7, 1, 3, 6][:-(-T // cache.page_size)])
    cache.sync()
    cache.poison_slot(1)
    i32 = dict(device=DEV, dtype=torch.int32)
    got_layers = []
    lg = model.step(torch.tensor(toks, **i32), torch.arange(T, **i32), torch.full((T,), 1, **i32), cache, torch.arange(T, device=DEV),
                    collect=got_layers, portions=[(0, T, 1, 0)])
    assert len(got_layers) == len(want_layers) == len(cd["layers"])
    for i, (gl, wl) in enumerate(zip(got_layers, want_layers)):
        err = float((gl.double().cpu() - wl).abs().max() / wl.abs().max())
        assert err < (1e-4 if dtype == torch.float32 else 8e-2), (i, err)
    assert rel_err(lg, want) < TOL[dtype]


@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prefill_portions_and_token_by_token_agree_with_oracle(name, dtype):
    cd = CONFIGS[name]()
    model, sd = build(cd, dtype, seed=3)
    toks = tokens_for(cd, 100 if name == "d" else 75, 4)       # d: past its window of 75
    want = oracle_logits(cd, sd, toks)
    T = len(toks)
    every = list(range(T))
    # whole; token by token (through the captured decode step from the second token on); portions of 2, 1, 17, 2, 30, 3, 20
    whole, _ = run_schedule(model, [([("w", toks, every)], ["w"])], 128)
    single, _ = run_schedule(model, [([("s", [t], [0])], ["s"] if i == T - 1 else []) for i, t in enumerate(toks)], 128)
    cuts = [0, 2, 3, 20, 22, 52, 55, 75] + ([100] if T == 100 else [])
    parts, _ = run_schedule(model, [([("p", toks[lo:hi], list(range(hi - lo)))], []) for lo, hi in zip(cuts[:-1], cuts[1:])], 128)
    for got in (whole["w"], single["s"], parts["p"]):
        assert len(got) == T
        assert rel_err(torch.stack(got), want) < TOL[dtype]
    if dtype == torch.float32:   # the same instructions in the same order: cuts change nothing but the last bits of the matrix products
        assert rel_err(torch.stack(parts["p"]), torch.stack(whole["w"])) < 2e-6
        assert rel_err(torch.stack(single["s"]), torch.stack(whole["w"])) < 2e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mixed_batches_reused_pages_and_slots(dtype):
    """Five requests of unequal length through two slots and a pool of six pages: portions of some beside single tokens of others,
    every request checked against the oracle run alone. Freed pages and slots are taken again; their states are poisoned first."""
    cd = config_a(page=16)
    model, sd = build(cd, dtype, seed=5)
    lens = {"r0": 41, "r1": 30, "r2": 7, "r3": 48, "r4": 1}
    toks = {k: tokens_for(cd, n, 10 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: oracle_logits(cd, sd, v) for k, v in toks.items()}
    sched = StepScheduler(model, max_tokens=96, slots=2)
    fed = {k: 0 for k in toks}
    got = {k: [] for k in toks}

    def step(plan):
        entries, end = [], []
        for k, n in plan:
            part = toks[k][fed[k]:fed[k] + n]
            entries.append((k, part, list(range(len(part)))))
            fed[k] += len(part)
            if fed[k] == lens[k]:
                end.append(k)
        lg = sched.run_step(entries)
        at = 0
        for k, part, w in entries:
            got[k] += [lg[at + i].float().cpu().clone() for i in range(len(part))]
            at += len(part)
        for k in end:
            slot = sched.live[k].slot
            sched.release(k)
            sched.cache.poison_slot(slot)

    step([("r0", 17), ("r1", 2)])
    step([("r0", 1), ("r1", 20)])
    step([("r1", 1), ("r0", 2)])
    step([("r0", 21), ("r1", 7)])          # both end: 3 + 2 pages and both slots go back
    assert sched.pages.available() == 6 and len(sched.free_slots) == 2
    step([("r2", 5), ("r3", 3)])
    step([("r3", 30), ("r2", 1)])
    step([("r2", 1), ("r3", 1)])           # r2 ends, its slot goes to r4
    step([("r4", 1), ("r3", 14)])
    for k in toks:
        assert len(got[k]) == lens[k]
        assert rel_err(torch.stack(got[k]), want[k]) < TOL[dtype], k


def test_wide_layers_take_the_tensor_core_gemms():
    """Width 1024: the stacked projections, gate | up (with bias) and down go through the tcgen05 GEMM in prompt portions and through
    the skinny GEMM in decode rows; both against the oracle, and against each other."""
    cd = {"architecture": "Tifisun", "vocab": 520, "width": 1024, "embedding": {"scale": 2.0}, "residual_mult": 0.6, "norm": {"eps": 1e-5},
          "kv_page_size": 64, "layers": [delta(8, 4, 64, 128, 4, ff=1024), parallel(8, 2, 64, 64, 48, 4, 64, 128, [0.9, 0.95, 0.99, 0.999], ff=1024),
                                         delta(8, 8, 64, 64, 3, channel=True, ff=1024)]}
    model, sd = build(cd, torch.bfloat16, seed=17)
    toks = tokens_for(cd, 80, 18)
    want = oracle_logits(cd, sd, toks)
    whole, _ = run_schedule(model, [([("w", toks, list(range(80)))], ["w"])], 128)
    assert rel_err(torch.stack(whole["w"]), want) < TOL[torch.bfloat16]
    steps = [([("p", toks[:70], [69])], [])] + [([("p", [t], [0])], []) for t in toks[70:]]
    parts, _ = run_schedule(model, steps, 128)
    assert rel_err(torch.stack(parts["p"]), want[69:]) < TOL[torch.bfloat16]


def test_more_requests_than_slots_is_refused_and_pool_exhaustion_is_reported():
    cd = config_b(page=32)
    model, _ = build(cd, torch.float32)
    sched = StepScheduler(model, max_tokens=64, slots=1)
    sched.run_step([("x", [1, 2, 3], [])])
    with pytest.raises(RuntimeError):
        sched.run_step([("y", [1], [])])
    with pytest.raises(RuntimeError):
        sched.run_step([("x", list(range(62)), [])])


def _slow_decay(sd):
    for k in list(sd):
        if k.endswith("A_log"):
            sd[k] = torch.full_like(sd[k], -9.0)          # decay = exp(-e^-9 softplus(.)) ~ 0.9999 per token
        if k.endswith(".mix.b"):
            sd[k] = sd[k] * 0.0                           # beta = 1/2 everywhere: every token writes


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_far_tokens_stay_in_the_state_and_long_decoding(dtype):
    """Decays close to one: a token 300 positions back still shapes the output, so a state that is lost, reset or mixed up between
    slots shows. 260 tokens in portions, then 70 decoded one by one (past the attention window, through several pages)."""
    cd = config_a(page=16)
    cd["layers"][1]["mixer"]["right"]["decay"] = [0.9999, 0.97, 0.9995]
    model, sd = build(cd, dtype, seed=7, edit=_slow_decay)
    toks = tokens_for(cd, 330, 8)
    want = oracle_logits(cd, sd, toks)
    other = tokens_for(cd, 330, 9)
    # the far token matters: the reference itself changes when token 5 changes
    changed = list(toks)
    changed[5] = (changed[5] + 1) % cd["vocab"]
    assert rel_err(oracle_logits(cd, sd, changed)[-1:], want[-1:]) > 100 * TOL[torch.float32]     # far above what float32 is held to
    steps, at = [], 0
    for n in (100, 61, 2, 97):
        steps.append(([("m", toks[at:at + n], [n - 1]), ("o", other[at:at + n], [])], []))
        at += n
    for i in range(at, 330):
        steps.append(([("o", [other[i]], []), ("m", [toks[i]], [0])], ["m", "o"] if i == 329 else []))
    got, _ = run_schedule(model, steps, 704)
    idx = [99, 160, 162, 259] + list(range(260, 330))
    assert rel_err(torch.stack(got["m"]), want[idx]) < TOL[dtype]


def test_first_tokens_of_a_sequence():
    """Positions 0..taps-2 have fewer convolution inputs than taps, position 0 has an empty state and a window of one key."""
    cd = config_a()
    model, sd = build(cd, torch.float32, seed=11)
    toks = tokens_for(cd, 6, 12)
    want = oracle_logits(cd, sd, toks)
    for cuts in ([0, 6], [0, 1, 2, 3, 4, 5, 6], [0, 2, 6], [0, 1, 6]):
        got, _ = run_schedule(model, [([("f", toks[lo:hi], list(range(hi - lo)))], []) for lo, hi in zip(cuts[:-1], cuts[1:])], 64)
        assert rel_err(torch.stack(got["f"]), want) < TOL[torch.float32], cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_the_scheduler(dtype):
    cd = config_a()
    model, sd = build(cd, dtype, seed=13)
    prompts = [tokens_for(cd, n, 20 + n) for n in (5, 23, 1, 40, 12)]
    outs = model.generate(prompts, max_new_tokens=12, slots=3, chunk=16)
    for p, o in zip(prompts, outs):
        o = o.tolist()
        assert o[:len(p)] == p and len(o) == len(p) + 12
        # every generated token is the oracle's choice given the same prefix (near-ties within the rounding error may go either way)
        lg = oracle_logits(cd, sd, o[:-1])
        for i in range(len(p) - 1, len(o) - 1):
            row = lg[i]
            assert row[o[i + 1]] >= row.max() - (1e-3 if dtype == torch.float32 else 0.15) * float(row.std()), (i, dtype)


def test_config_json_round_trip_and_registry(tmp_path):
    from omchat_b200.model import registry
    from omchat_b200.model.checkpoint import save_checkpoint
    cd = config_c()
    cfg = TifisunConfig.from_dict(cd)
    sd = random_state_dict(cfg, seed=2, decay_rank=12, gate_rank=20, bias_rows=10)
    save_checkpoint(sd, cfg, str(tmp_path))
    model = registry.load_model(str(tmp_path), device=DEV, dtype=torch.float32)
    assert type(model).__name__ == "TifisunForCausalLM" and model.config == cfg
    toks = tokens_for(cd, 20, 1)
    got, _ = run_schedule(model, [([("x", toks, [19])], ["x"])], 64)
    assert rel_err(torch.stack(got["x"]), oracle_logits(cd, sd, toks)[19:]) < TOL[torch.float32]
