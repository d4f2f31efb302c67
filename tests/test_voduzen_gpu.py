"""Voduzen on the GPU against the plain restatement in oracle/voduzen_oracle.py (float64, whole sequences, no cache).

Small configurations of their own (sizes that are not multiples of 32, a rotation narrower than the rotated part, top-1 and
top-3 routers, layers without identity experts / shared expert / feed-forward), random weights, and engineered weights or
inputs where random ones would hide a fault (one dominant far key, a dominant sink, a dominant key just past the causal edge).
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():  # collected on the CPU box too
    pytest.skip("needs a CUDA device", allow_module_level=True)

from omchat_b200 import seqlib  # noqa: E402
from omchat_b200.config import VoduzenConfig  # noqa: E402
from omchat_b200.model.voduzen import VoduzenForCausalLM, random_state_dict  # noqa: E402
from omchat_b200.serving import StepScheduler  # noqa: E402
from oracle import voduzen_oracle as O  # noqa: E402

DEV = "cuda:0"


def layer(kind, heads, dim, rot_dim, vdim, kv_rank, q_rank=None, dims=None, scaling=None, base=10000.0, mlp="full", experts=5,
          identity=2, top=3, ff=40, shared=72):
    rot = {"base": base, "dims": dims or rot_dim}
    if scaling:
        rot["scaling"] = scaling
    m = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "rot": rot, "rot_dim": rot_dim, "scale": 1.0 / math.sqrt(dim + rot_dim),
         "vdim": vdim}
    if q_rank:
        m["q_rank"] = q_rank
    f = None
    if mlp:
        f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top},
             "shared": {"ff": shared} if shared else None}
    return {"type": kind, "mixer": m, "mlp": f}


YARN = {"factor": 8.0, "fast": 16.0, "original": 64, "slow": 2.0}


def config_a(page=16):
    """Four layers that differ in everything the design lets differ."""
    return {"architecture": "Voduzen", "vocab": 160, "width": 96, "embedding": {"scale": 9.0}, "logit_scale": 0.5,
            "norm": {"eps": 1e-5}, "kv_page_size": page, "layers": [
                layer("latent_attention", 3, 16, 8, 24, 40, scaling=YARN, base=5000.0),
                layer("latent_attention_2", 2, 24, 16, 8, 48, q_rank=56, dims=8, identity=0, top=1, shared=None),
                layer("latent_attention", 5, 8, 24, 16, 24, dims=24, mlp=None),
                layer("latent_attention_2", 1, 32, 8, 32, 72, q_rank=24, experts=3, identity=3, top=4, ff=24, shared=16)]}


def config_b(page=32):
    """One head, one expert beside one identity output, top 1 - values that tend to hide indexing faults when equal or 1."""
    return {"architecture": "Voduzen", "vocab": 97, "width": 64, "embedding": {"scale": 1.0}, "logit_scale": 3.0,
            "norm": {"eps": 1e-6}, "kv_page_size": page, "layers": [
                layer("latent_attention", 1, 8, 8, 8, 8, experts=1, identity=1, top=1, ff=8, shared=8),
                layer("latent_attention_2", 2, 40, 24, 40, 104, q_rank=40, scaling=None, experts=7, identity=0, top=2, ff=56)]}


def config_c(page=16):
    """Shapes the tensor-core attention kernel takes (latent and rotated widths multiples of 16), one per register tier."""
    return {"architecture": "Voduzen", "vocab": 120, "width": 80, "embedding": {"scale": 4.0}, "logit_scale": 1.5,
            "norm": {"eps": 1e-6}, "kv_page_size": page, "layers": [
                layer("latent_attention", 3, 16, 16, 24, 32, scaling=YARN, experts=4, identity=1, top=2, ff=32, shared=40),
                layer("latent_attention_2", 5, 24, 32, 16, 272, q_rank=48, mlp=None),
                layer("latent_attention", 2, 8, 16, 8, 160, dims=8, mlp=None),
                layer("latent_attention_2", 7, 8, 48, 8, 96, q_rank=32, experts=2, identity=0, top=2, ff=16, shared=None)]}


def build(cfg_dict, dtype, seed=0, edit=None):
    cfg = VoduzenConfig.from_dict(cfg_dict)
    sd = random_state_dict(cfg, seed=seed)
    for k in sd:                      # spread the router logits: near-ties that bf16 rounding could flip become rare
        if k.endswith(".router"):
            sd[k] = (sd[k].float() * 6).to(torch.bfloat16)
    if edit:
        edit(sd)
    return VoduzenForCausalLM.from_state_dict(sd, cfg, device=DEV, dtype=dtype), {k: v.float() for k, v in sd.items()}


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def run_schedule(model, schedule, max_tokens, slots=4):
    """schedule: list of steps, each a list of (key, token list); a key's last appearance ends it. Returns {key: logits [n, V]}."""
    last = {}
    for i, step in enumerate(schedule):
        for key, _ in step:
            last[key] = i
    sched = StepScheduler(model, max_tokens=max_tokens, slots=slots)
    out = {}
    for i, step in enumerate(schedule):
        entries = [(k, ids, list(range(len(ids)))) for k, ids in step]
        lg = sched.run_step(entries, [k for k, _ in step if last[k] == i]).cpu()
        at = 0
        for k, ids in step:
            out.setdefault(k, []).append(lg[at:at + len(ids)])
            at += len(ids)
    assert sched.pages.available() == sched.pages.count and len(sched.free_slots) == slots  # everything was given back
    return {k: torch.cat(v) for k, v in out.items()}, sched


def rel_err(got, want):
    want = want.detach().cpu().to(torch.float64)
    return ((got.detach().cpu().to(torch.float64) - want).abs().max() / want.abs().max().clamp_min(1e-9)).item()


def rms_err(got, want):
    want = want.detach().cpu().to(torch.float64)
    d = got.detach().cpu().to(torch.float64) - want
    return (d.pow(2).mean().sqrt() / want.pow(2).mean().sqrt().clamp_min(1e-9)).item()


TOL = {torch.float32: 2e-4, torch.bfloat16: 4e-2}


def close(got, want, dtype):
    """fp32: largest deviation against the largest value. bf16: per row, the root mean square of the deviation against that of
    the values; rounding can flip a near-tie of the router for a token, which changes that row by far more than rounding does,
    and through attention
    the rows after it by a little, so a minority of the rows may exceed the bound - a fault of the path shows in most rows."""
    if dtype == torch.float32:
        return rel_err(got, want) < TOL[dtype]
    want = want.detach().cpu().to(torch.float64)
    d = got.detach().cpu().to(torch.float64) - want
    rows = d.pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-9)
    over = int((rows > TOL[dtype]).sum())
    return over <= max(1, int(0.3 * rows.numel())) and float(rows.median()) < TOL[dtype]


# ------------------------------------------------------------------------------------------------- kernels, one at a time
@pytest.mark.parametrize("xdt,wdt,ydt", [(torch.float32, torch.float32, torch.float32), (torch.float32, torch.bfloat16, torch.bfloat16),
                                         (torch.bfloat16, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (67, 130, 33), (130, 64, 200)])
def test_linear_any_shape(xdt, wdt, ydt, M, N, K):
    g = torch.Generator().manual_seed(M * N + K)
    x = torch.randn(M, K, generator=g).to(xdt).to(DEV)
    w = torch.randn(N, K, generator=g).to(wdt).to(DEV)
    for act, f in ((seqlib.ACT_NONE, lambda z: z), (seqlib.ACT_RELU2, lambda z: torch.relu(z) ** 2), (seqlib.ACT_GELU_TANH, O.gelu_tanh)):
        y = seqlib.linear(x, w, torch.empty(M, N, device=DEV, dtype=ydt), alpha=0.5, act=act)
        want = f(0.5 * (x.double() @ w.double().T))
        assert rel_err(y, want) < (1e-5 if ydt == torch.float32 else 1e-2)


def test_linear_heads_are_column_slices_and_groups_pick_their_matrix():
    g = torch.Generator().manual_seed(3)
    T, H, dn, dr, r = 37, 3, 10, 6, 20
    q = torch.randn(T, H * (dn + dr), generator=g).to(DEV)
    wt = torch.randn(H, r, dn, generator=g).to(DEV)
    out = torch.zeros(T, H, r + dr, device=DEV)
    seqlib.linear(q, wt, out, M=T, N=r, K=dn, ldx=q.stride(0), sx=dn + dr, ldw=dn, sw=r * dn, ldy=H * (r + dr), sy=r + dr, batch=H)
    want = torch.einsum("thd,hrd->thr", q.view(T, H, dn + dr)[..., :dn].double(), wt.double())
    assert rel_err(out[..., :r], want) < 1e-5 and float(out[..., r:].abs().max()) == 0.0
    # grouped: 64-row tiles, tile i uses matrix group[i]; tiles with group < 0 are left alone
    E, N, K = 3, 12, 9
    x = torch.randn(4 * 64, K, generator=g).to(DEV)
    w = torch.randn(E, N, K, generator=g).to(DEV)
    group = torch.tensor([2, -1, 0, 1], dtype=torch.int32, device=DEV)
    y = torch.full((4 * 64, N), 7.0, device=DEV)
    seqlib.linear(x, w, y, M=4 * 64, N=N, K=K, ldw=K, tile_group=group, group_stride=N * K)
    for i, e in enumerate(group.tolist()):
        blk = y[i * 64:(i + 1) * 64]
        if e < 0:
            assert float((blk - 7.0).abs().max()) == 0.0
        else:
            assert rel_err(blk, x[i * 64:(i + 1) * 64].double() @ w[e].double().T) < 1e-5


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_norm_kernels(dt):
    g = torch.Generator().manual_seed(5)
    T, C, eps = 9, 100, 1e-3
    y = (torch.randn(T, C, generator=g) * 3).to(DEV)
    w = (torch.randn(C, generator=g) * 0.3).to(dt).to(DEV)
    h = torch.randn(T, C, generator=g).to(DEV)
    out = seqlib.rms_rows(y, w, eps, torch.empty(T, 60, device=DEV, dtype=dt), n=60)
    assert rel_err(out, O.norm_plain(y[:, :60].double().cpu(), w[:60].double().cpu(), eps)) < (1e-5 if dt == torch.float32 else 1e-2)
    out = seqlib.rms_rows(y, w, eps, torch.empty(T, C, device=DEV, dtype=dt), one_plus=True)
    assert rel_err(out, O.norm_zero_centred(y.double().cpu(), w.double().cpu(), eps)) < (1e-5 if dt == torch.float32 else 1e-2)
    want = h.double().cpu() + O.norm_zero_centred(y.double().cpu(), w.double().cpu(), eps)
    xb = torch.empty(T, C, device=DEV, dtype=dt)
    seqlib.norm_residual(y, w, eps, h, xb)
    assert rel_err(h, want) < 1e-5          # the residual stream itself is fp32 whatever the compute dtype
    assert rel_err(xb, want) < (1e-5 if dt == torch.float32 else 1e-2)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_fused_rope_store_equals_the_two_kernels_and_the_plain_formulas(dt):
    g = torch.Generator().manual_seed(17)
    T, H, dn, dr, r, dims, page = 23, 3, 10, 12, 20, 8, 8
    dkv = torch.randn(T, r + dr, generator=g).to(DEV)
    q = torch.randn(T, H * (dn + dr), generator=g).to(dt).to(DEV)
    w = (1 + 0.1 * torch.randn(r, generator=g)).to(dt).to(DEV)
    rot = {"dims": dims, "base": 100.0}
    cos, sin = O.rotary_angles(rot, 64)
    cs = torch.stack([cos, sin], dim=-1).float().contiguous().to(DEV)
    pos = torch.arange(5, 5 + T, dtype=torch.int32, device=DEV)
    slot = torch.zeros(T, dtype=torch.int32, device=DEV)
    table = torch.tensor([[3, 1, 4, 2, 0]], dtype=torch.int32, device=DEV)
    pools = [torch.zeros(5, page, r + dr, device=DEV, dtype=dt) for _ in range(2)]
    qcats = [torch.zeros(T, H, r + dr, device=DEV, dtype=dt) for _ in range(2)]
    seqlib.latent_kv_store(dkv, r, dr, w, 1e-5, cs, dims, pos, slot, table, page, pools[0])
    seqlib.rotary_q(q, H, dn, dr, cs, dims, pos, qcats[0], r)
    seqlib.latent_rope_store(dkv, r, dr, w, 1e-5, cs, dims, pos, slot, table, page, pools[1], q, H, dn, qcats[1])
    assert torch.equal(pools[0], pools[1]) and torch.equal(qcats[0], qcats[1])
    tol = 1e-5 if dt == torch.float32 else 1e-2
    p = pos.cpu().long()
    want_c = O.norm_plain(dkv[:, :r].double().cpu(), w.double().cpu(), 1e-5)
    want_k = O.rotate_interleaved(dkv[:, r:].double().cpu().contiguous(), cos[p], sin[p])
    rows = pools[1][table[0].long()].reshape(-1, r + dr)[5:5 + T]
    assert rel_err(rows[:, :r], want_c) < tol and rel_err(rows[:, r:], want_k) < tol
    want_q = O.rotate_interleaved(q.double().cpu().view(T, H, dn + dr)[..., dn:].contiguous(), cos[p], sin[p])
    assert rel_err(qcats[1][..., r:], want_q) < tol and float(qcats[1][..., :r].abs().max()) == 0.0


def test_small_step_row_sort_equals_plan_and_scatter():
    g = torch.Generator().manual_seed(19)
    T, C, E, top, tile = 9, 24, 5, 3, 64
    x = torch.randn(T, C, generator=g).to(DEV)
    ids = torch.stack([torch.randperm(E + 2, generator=g)[:top] for _ in range(T)]).to(torch.int32).to(DEV)   # ids >= E: identity
    counts = torch.tensor([int((ids == e).sum()) for e in range(E)], dtype=torch.int32, device=DEV)
    mt = seqlib.moe_max_tiles(T, top, E, tile)
    outs = []
    for fused in (False, True):
        cnt, cur = counts.clone(), torch.zeros(E, dtype=torch.int32, device=DEV)
        seg, grp = torch.zeros(E + 1, dtype=torch.int32, device=DEV), torch.zeros(mt, dtype=torch.int32, device=DEV)
        slot_of, xs = torch.zeros(T, top, dtype=torch.int32, device=DEV), torch.zeros(mt * tile, C, device=DEV)
        if fused:
            seqlib.moe_plan_scatter_small(cnt, E, tile, mt, seg, grp, x, ids, top, slot_of, xs)
        else:
            seqlib.moe_plan_tiles(cnt, E, tile, mt, seg, cur, grp)
            seqlib.moe_scatter_rows(x, ids, top, E, seg, cur, slot_of, xs)
        assert int(cnt.abs().sum()) == 0                                  # counters are left zeroed for the next call
        outs.append((seg.cpu(), grp.cpu()))
        for t in range(T):                                                 # every copy sits in its expert's segment and holds the row
            for k in range(top):
                e, sl = int(ids[t, k]), int(slot_of[t, k])
                if e >= E:
                    assert sl == -1
                else:
                    assert int(seg[e]) <= sl < int(seg[e]) + int(counts[e]) and torch.equal(xs[sl], x[t]) and int(grp[sl // tile]) == e
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


def test_router_matches_plain_choice_and_counts():
    g = torch.Generator().manual_seed(11)
    T, E, I, top = 50, 6, 3, 4
    z = torch.randn(T, E + I + 1, generator=g) * 2
    corr = torch.randn(E + I, generator=g) * 0.3      # large enough to change the choice against the plain scores
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    w = torch.empty(T, top, device=DEV)
    gate = torch.empty(T, device=DEV)
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    seqlib.router_topk(z.to(DEV), E + I, E, top, corr.to(DEV), True, ids, w, gate, counts)
    s = torch.softmax(z[:, :E + I].double(), -1)
    want_ids = torch.topk(s + corr.double(), top, dim=-1).indices
    assert (s.argmax(-1) != (s + corr.double()).argmax(-1)).any()  # the correction matters in this test
    assert torch.equal(ids.cpu().long().sort(-1).values, want_ids.sort(-1).values)
    assert rel_err(w.cpu(), torch.gather(s, 1, ids.cpu().long())) < 1e-5      # weights are the UNcorrected scores
    assert rel_err(gate.cpu(), torch.sigmoid(z[:, -1].double())) < 1e-5
    assert counts.cpu().tolist() == [int((want_ids == e).sum()) for e in range(E)]  # identity outputs take no rows


# ------------------------------------------------------------------------------------------------- mechanisms through the model
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfgf", [config_a, config_b, config_c])
def test_every_layer_against_the_plain_model(cfgf, dtype):
    cfg = cfgf()
    model, sd = build(cfg, dtype, seed=1)
    toks = tokens(75, cfg["vocab"], 2)
    states = []
    want = O.forward(cfg, sd, toks, states)
    sched = StepScheduler(model, max_tokens=128)
    r = sched._admit("a")
    sched._grow(r, len(toks))
    sched.cache.sync()
    n = len(toks)
    got_states = []
    lg = model.step(torch.tensor(toks, dtype=torch.int32, device=DEV), torch.arange(n, dtype=torch.int32, device=DEV),
                    torch.full((n,), r.slot, dtype=torch.int32, device=DEV), sched.cache, torch.arange(n, device=DEV), got_states,
                    portions=[(0, n, r.slot, 0)])
    for i, (a, b) in enumerate(zip(got_states, states)):
        assert close(a, b, dtype), f"residual stream after layer {i}"
    assert close(lg, want, dtype)


def test_mixers_alone_in_fp32():
    """Each mixer against the plain one on a sequence that spans several pages (no feed-forward in between)."""
    cfg = config_a(page=16)
    for l in cfg["layers"]:
        l["mlp"] = None
    model, sd = build(cfg, torch.float32, seed=4)
    toks = tokens(70, cfg["vocab"], 5)
    states, got = [], []
    O.forward(cfg, sd, toks, states)
    sched = StepScheduler(model, max_tokens=80)
    r = sched._admit("a")
    sched._grow(r, 70)
    sched.cache.host_lens[r.slot] = 70
    sched.cache.sync()
    model.step(torch.tensor(toks, dtype=torch.int32, device=DEV), torch.arange(70, dtype=torch.int32, device=DEV),
               torch.full((70,), r.slot, dtype=torch.int32, device=DEV), sched.cache, None, got)
    for a, b in zip(got, states):
        assert rel_err(a.cpu(), b) < 1e-4
    # what the cache holds is the normed latent and the rotated key part of the plain formulas
    m = cfg["layers"][0]["mixer"]
    x0 = sd["embed"].double()[torch.tensor(toks)] * cfg["embedding"]["scale"]
    dkv = x0 @ sd["l0.mix.dkv"].double().T
    c = O.norm_plain(dkv[:, :m["kv_rank"]], sd["l0.mix.dkv.norm"].double(), cfg["norm"]["eps"])
    cos, sin = O.rotary_angles(m["rot"], 70)
    kr = O.rotate_interleaved(dkv[:, m["kv_rank"]:].contiguous(), cos, sin)
    rows = sched.cache.gather(0, r.slot).cpu()
    assert rel_err(rows[:, :m["kv_rank"]], c) < 1e-5 and rel_err(rows[:, m["kv_rank"]:], kr) < 1e-5


# ------------------------------------------------------------------------------------------------- schedules
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfgf", [config_a, config_c])
def test_prefill_decode_portions_and_mixed_batches_agree(cfgf, dtype):
    cfg = cfgf(page=16)
    model, sd = build(cfg, dtype, seed=7)
    V = cfg["vocab"]
    reqs = {"a": tokens(83, V, 1), "b": tokens(5, V, 2), "c": tokens(40, V, 3), "d": tokens(1, V, 4), "e": tokens(33, V, 5)}
    gold = {k: O.forward(cfg, sd, v) for k, v in reqs.items()}
    # whole prompts, one request per step
    got, _ = run_schedule(model, [[(k, v)] for k, v in reqs.items()], max_tokens=96)
    for k in reqs:
        assert close(got[k], gold[k], dtype), f"whole {k}"
    # token by token (every row is a decode row, first tokens included)
    got, _ = run_schedule(model, [[("a", [t])] for t in reqs["a"]], max_tokens=96)
    assert close(got["a"], gold["a"], dtype)
    # portions of changing size down to two tokens, cut inside pages
    cuts = [2, 14, 3, 17, 2, 30, 15]
    sch, at = [], 0
    for c in cuts:
        sch.append([("a", reqs["a"][at:at + c])])
        at += c
    assert at == 83
    got, _ = run_schedule(model, sch, max_tokens=96)
    assert close(got["a"], gold["a"], dtype)
    # unequal requests in one batch: portions beside single tokens; more requests than slots over time, so that slots and
    # pages are given back and used again (pool: 12 pages of 16 for at most 3 live requests)
    sch = [[("a", reqs["a"][:20]), ("b", reqs["b"][:1]), ("c", reqs["c"][:33])],
           [("a", reqs["a"][20:22]), ("b", reqs["b"][1:2]), ("c", reqs["c"][33:34])],
           [("b", reqs["b"][2:5]), ("c", reqs["c"][34:40])],
           [("a", reqs["a"][22:70]), ("d", reqs["d"]), ("e", reqs["e"][:31])],
           [("a", reqs["a"][70:71]), ("e", reqs["e"][31:32])],
           [("a", reqs["a"][71:83]), ("e", reqs["e"][32:33])]]
    got, sched = run_schedule(model, sch, max_tokens=12 * 16, slots=3)
    for k in reqs:
        assert close(got[k], gold[k], dtype), f"mixed {k}"


def test_pages_and_slots_are_reused_without_leaking_state():
    """A pool of 3 pages and one slot serves five requests in a row; each must come out as if it ran alone."""
    cfg = config_b(page=32)
    model, sd = build(cfg, torch.float32, seed=9)
    sched = StepScheduler(model, max_tokens=96, slots=1)
    for i in range(5):
        toks = tokens(96 - 7 * i, cfg["vocab"], 20 + i)
        lg = sched.run_step([(f"r{i}", toks[:50], list(range(50)))], [])
        lg2 = sched.run_step([(f"r{i}", toks[50:], list(range(len(toks) - 50)))], [f"r{i}"])
        assert rel_err(torch.cat([lg, lg2]).cpu(), O.forward(cfg, sd, toks)) < 2e-4
    assert sched.pages.available() == 3


def test_long_decoding_in_fp32():
    cfg = config_b(page=32)
    model, sd = build(cfg, torch.float32, seed=12)
    toks = tokens(260, cfg["vocab"], 31)
    got, _ = run_schedule(model, [[("a", toks[:4])]] + [[("a", [t])] for t in toks[4:]], max_tokens=288)
    assert rel_err(got["a"], O.forward(cfg, sd, toks)) < 2e-4


def test_long_decoding_in_bf16_through_growing_key_ranges():
    """Decode-only steps replay a CUDA graph whose attention work list is rebuilt on the device; as the context passes 128, 256
    and 512 tokens the rows are cut into 1, 2, 4 and 8 key ranges (new graphs) that the merge kernel combines."""
    cfg = config_c(page=16)
    model, sd = build(cfg, torch.bfloat16, seed=15)
    toks = tokens(560, cfg["vocab"], 33)
    got, _ = run_schedule(model, [[("a", toks[:100])]] + [[("a", [t])] for t in toks[100:]], max_tokens=576)
    assert len(model.decoder._graphs) >= 3
    assert close(got["a"], O.forward(cfg, sd, toks), torch.bfloat16)
    # two requests decoding side by side at different lengths, against each alone
    a, b = tokens(300, cfg["vocab"], 34), tokens(140, cfg["vocab"], 35)
    sch = [[("a", a[:270]), ("b", b[:110])]] + [[("a", [a[270 + i]]), ("b", [b[110 + i]])] for i in range(30)]
    got, _ = run_schedule(model, sch, max_tokens=512)
    assert close(got["a"], O.forward(cfg, sd, a), torch.bfloat16) and close(got["b"], O.forward(cfg, sd, b), torch.bfloat16)


# ------------------------------------------------------------------------------------------------- engineered cases
def one_layer(page, sink_value=None):
    l = layer("latent_attention", 2, 8, 8, 8, 16, mlp=None)
    return {"architecture": "Voduzen", "vocab": 64, "width": 32, "embedding": {"scale": 1.0}, "logit_scale": 1.0,
            "norm": {"eps": 1e-6}, "kv_page_size": page, "layers": [l]}


def run_attn(impl, q, r, dr, pool, table, page, pos, slot, sink, scale):
    """impl 'plain': fp32 kernel; 'mma': the tensor-core kernel on bf16 copies (with the split of long contexts into key ranges
    that a small batch triggers)."""
    T, H = q.shape[0], q.shape[1]
    out = torch.empty(T, H, r, device=DEV)
    sk = sink.to(DEV) if sink is not None else None
    if impl == "plain":
        seqlib.latent_attn(q.contiguous().to(DEV), r, dr, pool.to(DEV), table.to(DEV), page, pos.to(DEV), slot.to(DEV), sk, scale, out)
    else:
        assert seqlib.latent_attn_mma_ok(H, r, dr, torch.bfloat16)
        portions, t = [], 0
        while t < T:                       # consecutive rows of one slot with ascending positions form a portion
            e = t + 1
            while e < T and slot[e] == slot[t] and pos[e] == pos[e - 1] + 1:
                e += 1
            portions.append((t, e - t, int(slot[t]), int(pos[t])))
            t = e
        plan = seqlib.LatentAttnPlan(portions, H, DEV)
        seqlib.latent_attn_mma(q.contiguous().to(torch.bfloat16).to(DEV), r, dr, pool.to(torch.bfloat16).to(DEV), table.to(DEV), page,
                               plan, sk, scale, out)
    return out.cpu()


KERNELS = [("plain", 16, 8), ("plain", 32, 16), ("mma", 32, 16), ("mma", 144, 16), ("mma", 288, 32)]  # mma: 1, 2 and 4 warps per row group


def attn_case(page, n, qpos, hot, decode, impl="plain", r=16, dr=8):
    """Attention kernel alone with one dominant key: the cache row at position `hot` has a large entry that only the query at
    `qpos` looks at. Returns the kernel's output row for (qpos, head 0) and the cached latents."""
    H = 2
    g = torch.Generator().manual_seed(100 + hot)
    rows = torch.randn(n, r + dr, generator=g) * 0.3
    rows[hot, 3] = 40.0
    q = torch.randn(n, H, r + dr, generator=g) * 0.3
    q[qpos, 0, 3] = 5.0
    pages = -(-n // page)
    pool = torch.zeros(pages + 3, page, r + dr)
    order = list(range(pages + 2, 2, -1))                     # pages in descending, non-contiguous order
    for j in range(n):
        pool[order[j // page], j % page] = rows[j]
    table = torch.zeros(2, pages, dtype=torch.int32)
    table[1] = torch.tensor(order, dtype=torch.int32)
    if decode:
        qs, pos = q[qpos:qpos + 1], torch.tensor([qpos], dtype=torch.int32)
    else:
        qs, pos = q, torch.arange(n, dtype=torch.int32)
    out = run_attn(impl, qs, r, dr, pool, table, page, pos, torch.ones(qs.shape[0], dtype=torch.int32), None, 1.0)
    return out[0 if decode else qpos, 0], rows[:, :r]


@pytest.mark.parametrize("impl,r,dr", KERNELS)
@pytest.mark.parametrize("decode", [False, True])
def test_a_far_key_is_found_wherever_it_lies(decode, impl, r, dr):
    page, n, qpos = 16, 600, 599
    for hot in (0, 1, 15, 16, 17, 31, 32, 63, 64, 65, 150, 255, 256, 511, 512, 598, 599):   # first tokens, page, tile and key-range borders, the row itself
        got, lat = attn_case(page, n, qpos, hot, decode, impl, r, dr)
        assert (got - lat[hot]).abs().max() < (1e-3 if impl == "plain" else 2e-2), f"key {hot}"


@pytest.mark.parametrize("impl,r,dr", KERNELS)
def test_a_key_past_the_causal_edge_is_not_seen(impl, r, dr):
    """The dominant key sits one position AFTER the query, in the same step and the same page: the query must ignore it."""
    page, n = 16, 140
    for qpos in (0, 14, 15, 16, 31, 32, 63, 64, 127, 138):
        got, lat = attn_case(page, n, qpos, qpos + 1, False, impl, r, dr)
        assert (got - lat[qpos + 1]).abs().max() > 0.05
        # and equals plain softmax attention over keys 0..qpos
        g = torch.Generator().manual_seed(100 + qpos + 1)
        rows = torch.randn(n, r + dr, generator=g) * 0.3
        rows[qpos + 1, 3] = 40.0
        q = torch.randn(n, 2, r + dr, generator=g) * 0.3
        q[qpos, 0, 3] = 5.0
        p = torch.softmax(rows[:qpos + 1].double() @ q[qpos, 0].double(), 0)
        assert (got.double() - p @ rows[:qpos + 1, :r].double()).abs().max() < (1e-5 if impl == "plain" else 2e-2)


@pytest.mark.parametrize("impl,r,dr", KERNELS)
def test_sink_takes_probability_and_returns_nothing(impl, r, dr):
    H, n, page = 2, 20, 16
    g = torch.Generator().manual_seed(1)
    rows = torch.randn(n, r + dr, generator=g)
    q = torch.randn(1, H, r + dr, generator=g)
    pool = torch.zeros(3, page, r + dr)
    pool[1, :16], pool[2, :4] = rows[:16], rows[16:]
    table = torch.tensor([[1, 2]], dtype=torch.int32)
    sink = torch.tensor([3.0, -30.0])
    rows, q = rows.to(torch.bfloat16).float() * 0.5, q.to(torch.bfloat16).float() * 0.5   # representable in both kernels' storage
    pool[1, :16], pool[2, :4] = rows[:16], rows[16:]
    pos, slot = torch.tensor([n - 1], dtype=torch.int32), torch.zeros(1, dtype=torch.int32)
    out = run_attn(impl, q, r, dr, pool, table, page, pos, slot, sink, 0.5)
    tol = 1e-5 if impl == "plain" else 1e-2
    for h in range(H):
        s = (rows.double() @ q[0, h].double()) * 0.5
        e = torch.exp(s - s.max())
        want = (e[:, None] * rows[:, :r].double()).sum(0) / (e.sum() + math.exp(float(sink[h]) - float(s.max())))
        assert (out[0, h].double() - want).abs().max() < tol
    plain = run_attn(impl, q, r, dr, pool, table, page, pos, slot, None, 0.5)
    assert (plain[0, 0] - out[0, 0]).abs().max() > 2e-2      # sink 3.0 shrinks head 0 ...
    assert (plain[0, 1] - out[0, 1]).abs().max() < 1e-6      # ... sink -30 leaves head 1 alone


def test_model_with_dominant_sink_and_far_key():
    """Model level: a large sink must change the logits exactly as the plain model says, and so must a rotated-key weight scaled
    so that far positions dominate."""
    cfg = one_layer(16)

    def edit(sd):
        sd["l0.mix.sink"] = torch.tensor([4.0, -2.0]).to(torch.bfloat16)
        sd["l0.mix.dkv"] = (sd["l0.mix.dkv"].float() * 6).to(torch.bfloat16)
        sd["l0.mix.q"] = (sd["l0.mix.q"].float() * 6).to(torch.bfloat16)
    model, sd = build(cfg, torch.float32, seed=3, edit=edit)
    toks = tokens(150, 64, 8)
    gold = O.forward(cfg, sd, toks)
    got, _ = run_schedule(model, [[("a", toks[:100])], [("a", toks[100:149])], [("a", toks[149:])]], max_tokens=160)
    assert rel_err(got["a"], gold) < 2e-4
    sd2 = dict(sd)
    sd2["l0.mix.sink"] = torch.tensor([-20.0, -20.0])
    assert rel_err(O.forward(cfg, sd2, toks), gold) > 1e-3   # the sink is visible in this model's logits


# ------------------------------------------------------------------------------------------------- tensor-core paths at width
def test_tcgen05_gemms_and_grouped_experts_match_the_plain_kernels():
    """A width at which the bf16 model takes the tcgen05 GEMMs (dense, skinny, grouped with the relu^2 epilogue) and the
    tensor-core attention: same schedule with those switched off (FMA kernels, plain attention) and against the plain model."""
    l1 = layer("latent_attention", 8, 64, 32, 64, 256, scaling=YARN, experts=6, identity=2, top=3, ff=512, shared=1024)
    l2 = layer("latent_attention_2", 4, 128, 64, 128, 128, q_rank=1024, experts=6, identity=0, top=2, ff=512, shared=None)
    cfg = {"architecture": "Voduzen", "vocab": 2048, "width": 1024, "embedding": {"scale": 32.0}, "logit_scale": 0.25,
           "norm": {"eps": 1e-6}, "kv_page_size": 64, "layers": [l1, l2]}
    model, sd = build(cfg, torch.bfloat16, seed=13)
    assert model.decoder._grouped_tensor_gemm(model.config.layers[0].mlp)
    toks = tokens(300, 2048, 3)
    sch = [[("a", toks[:200])], [("a", toks[200:290])]] + [[("a", [t])] for t in toks[290:]]
    fast, _ = run_schedule(model, sch, max_tokens=320)
    model.decoder.tensor_gemm = model.decoder.tensor_attention = False
    slow, _ = run_schedule(model, sch, max_tokens=320)
    assert close(fast["a"], slow["a"].double(), torch.bfloat16)
    assert close(fast["a"], O.forward(cfg, sd, toks), torch.bfloat16)


# ------------------------------------------------------------------------------------------------- generation
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_greedy_generation_through_the_scheduler(dtype):
    cfg = config_a(page=16)
    model, sd = build(cfg, dtype, seed=21)
    prompts = [tokens(n, cfg["vocab"], 40 + n) for n in (3, 50, 21, 1, 34, 9)]
    outs = model.generate(prompts, max_new_tokens=12, slots=3, chunk=16)
    clear = missed = 0
    for p, o in zip(prompts, outs):
        o = o.tolist()
        assert o[:len(p)] == p and len(o) == len(p) + 12
        # teacher-forced check: a generated token is the plain model's argmax wherever its top-1 margin is clear (in bf16 a
        # flipped router near-tie may move one logit row by more than the margin: a few misses are let through there)
        lg = O.forward(cfg, sd, o[:-1])
        for i in range(len(p) - 1, len(o) - 1):
            top2 = torch.topk(lg[i], 2).values
            if float(top2[0] - top2[1]) > (1e-3 if dtype == torch.float32 else 0.15) * float(lg[i].abs().max()):
                clear += 1
                missed += o[i + 1] != int(lg[i].argmax())
    assert clear >= 20 and missed <= (0 if dtype == torch.float32 else clear // 10)
