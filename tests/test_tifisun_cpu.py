"""Host-side parts of the Tifisun path that need no GPU: configuration parsing, the distance buckets, the state-slot cache, and the
oracle's recurrences against closed forms."""
import math

import pytest
import torch

from omchat_b200.config import DeltaRuleSpec, ParallelMixerSpec, TifisunConfig, WindowAttentionSpec
from omchat_b200.model import registry
from omchat_b200.model.checkpoint import config_from_dict
from omchat_b200.model.paged_cache import PagedStateCache
from oracle import tifisun_oracle as O


def small_config():
    left = {"bias_max": 50, "dim": 20, "heads": 6, "kv_heads": 2, "mask": {"size": 19}, "scale": 0.2, "softcap": 12.0, "vdim": 12}
    right = {"decay": [0.7, 0.97, 0.999], "dim": 24, "heads": 3, "vdim": 20}
    return {"architecture": "Tifisun", "vocab": 150, "width": 96, "embedding": {"scale": 2.5}, "residual_mult": 0.6, "norm": {"eps": 1e-5},
            "layers": [
                {"type": "delta", "mixer": {"conv": 4, "dim": 24, "heads": 4, "kv_heads": 2, "vdim": 40}, "mlp": {"ff": 40, "kind": "dense"}},
                {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": None},
                {"type": "channel_delta", "mixer": {"conv": 2, "dim": 40, "heads": 2, "kv_heads": 1, "vdim": 24}, "mlp": {"ff": 56, "kind": "dense"}},
                {"type": "delta", "mixer": {"conv": 4, "dim": 24, "heads": 4, "kv_heads": 2, "vdim": 40}, "mlp": {"ff": 40, "kind": "dense"},
                 "weights_of": 0}]}


def test_config_is_read_from_the_dictionary_and_round_trips():
    cfg = config_from_dict(small_config())
    assert isinstance(cfg, TifisunConfig) and cfg.vocab_size == 150 and cfg.hidden_size == 96 and cfg.residual_mult == 0.6
    a, b, c, d = cfg.layers
    assert isinstance(a.mixer, DeltaRuleSpec) and not a.mixer.channel_decay and a.mixer.conv == 4 and a.mixer.kv_heads == 2
    assert isinstance(b.mixer, ParallelMixerSpec) and b.mixer.left.window == 19 and b.mixer.left.softcap == 12.0 and b.mlp is None
    assert b.mixer.right.decay == [0.7, 0.97, 0.999] and c.mixer.channel_decay and c.mlp.ff == 56
    assert d.weights_of == 0 and a.weights_of is None
    assert TifisunConfig.from_dict(cfg.to_dict()) == cfg
    assert registry.MODEL_CLASSES[TifisunConfig][1] == "TifisunForCausalLM"
    for breakage in (lambda x: x["layers"][0].update(type="something_else"), lambda x: x["layers"][3].update(weights_of=1),
                     lambda x: x["layers"][3].update(weights_of=9), lambda x: x["layers"][0]["mixer"].update(kv_heads=3),
                     lambda x: x["layers"][1]["mixer"]["right"].update(decay=[0.5])):
        bad = small_config()
        breakage(bad)
        with pytest.raises(ValueError):
            config_from_dict(bad)


@pytest.mark.parametrize("rows,far", [(10, 40.0), (16, 128.0), (12, 36.0), (4, 1000.0), (32, 256.0)])
def test_distance_buckets(rows, far):
    half = rows // 2
    b = [WindowAttentionSpec.bucket(n, rows, far) for n in range(int(far) + 50)]
    assert b[:half] == list(range(half)) and b[half] == half
    assert all(x <= y for x, y in zip(b[:-1], b[1:])) and max(b) == rows - 1
    assert b[int(far)] == rows - 1 and b[-1] == rows - 1
    assert b == [O.distance_bucket(n, rows, far) for n in range(len(b))]
    for n in range(half, int(far)):     # a distance lies in the bucket whose logarithmic bounds enclose it
        lo = half * (far / half) ** ((b[n] - half) / (rows - half))
        assert n >= lo * (1 - 1e-9)


def test_state_cache_shapes_and_poison():
    c = PagedStateCache([0, 64, 0], [{"S": (2, 4, 8), "conv": (3, 10)}, {"S": (1, 4, 4)}, {}], n_pages=5, n_slots=3, page_size=16,
                        dtype=torch.float32, device="cpu")
    assert c.pools[0] is None and c.pools[2] is None and c.pools[1].shape == (5, 16, 64)
    assert c.states[0]["S"].shape == (3, 2, 4, 8) and c.states[0]["conv"].shape == (3, 3, 10) and c.states[2] == {}
    assert c.state_bytes_per_slot() == 4 * (64 + 30 + 16)
    c.poison_slot(1)
    assert torch.isnan(c.states[0]["S"][1]).all() and not torch.isnan(c.states[0]["S"][0]).any() and not torch.isnan(c.states[1]["S"][2]).any()


def test_oracle_recurrences_against_closed_forms():
    g = torch.Generator().manual_seed(0)
    T, d, dv = 9, 5, 4
    q, k, v = (torch.randn(T, n, generator=g, dtype=torch.float64) for n in (d, d, dv))
    # constant decay: o_t = sum_{s <= t} decay^(t - s) (q_t . k_s) v_s
    o = O.decayed_outer_sum(q, k, v, 0.8)
    for t in range(T):
        want = sum(0.8 ** (t - s) * (q[t] @ k[s]) * v[s] for s in range(t + 1))
        assert torch.allclose(o[t], want)
    # delta rule with beta = 1, no decay and orthonormal keys stores each value exactly: reading with k_s returns v_s
    keys = torch.linalg.qr(torch.randn(d, d, generator=g, dtype=torch.float64))[0][:4]
    vals = torch.randn(4, dv, generator=g, dtype=torch.float64)
    o = O.delta_rule(keys, keys, vals, torch.ones(4, d, dtype=torch.float64), torch.ones(4, dtype=torch.float64))
    assert torch.allclose(o, vals)
    # writing the same key twice with beta = 1 replaces the value
    kk = torch.stack([keys[0], keys[0]])
    o = O.delta_rule(kk, kk, vals[:2], torch.ones(2, d, dtype=torch.float64), torch.ones(2, dtype=torch.float64))
    assert torch.allclose(o[1], vals[1])
    # convolution: one tap is the identity scale, taps look back only
    x = torch.randn(6, 3, generator=g, dtype=torch.float64)
    assert torch.allclose(O.causal_conv(x, torch.full((3, 1), 2.0, dtype=torch.float64)), 2 * x)
    w = torch.zeros(3, 3, dtype=torch.float64)
    w[:, 0] = 1.0
    y = O.causal_conv(x, w)
    assert torch.allclose(y[2:], x[:-2]) and float(y[:2].abs().max()) == 0.0
