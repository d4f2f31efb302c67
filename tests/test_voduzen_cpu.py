"""Host-side parts of the Voduzen path that need no GPU: configuration parsing, rotary frequencies, the page free list and the
step scheduler's bookkeeping (driven with a stand-in model that records what it is given)."""
import math

import pytest
import torch

from omchat_b200.config import RotarySpec, VoduzenConfig
from omchat_b200.model.checkpoint import config_from_dict
from omchat_b200.model.paged_cache import PageAllocator, PagedLatentCache
from omchat_b200.model import registry
from omchat_b200.serving import StepScheduler
from oracle import voduzen_oracle as O


def small_config():
    mix1 = {"dim": 16, "heads": 3, "kv_rank": 40, "rot": {"base": 5000.0, "dims": 8, "scaling": {"factor": 8.0, "fast": 16.0,
            "original": 64, "slow": 2.0}}, "rot_dim": 8, "scale": 0.2, "vdim": 24}
    mix2 = {"dim": 24, "heads": 2, "kv_rank": 48, "q_rank": 56, "rot": {"base": 10000.0, "dims": 8}, "rot_dim": 16, "scale": 0.15,
            "vdim": 8}
    mlp = {"kind": "moe", "expert": {"ff": 40}, "router": {"experts": 5, "identity": 2, "top": 3}, "shared": {"ff": 72}}
    return {"architecture": "Voduzen", "vocab": 160, "width": 96, "embedding": {"scale": 9.0}, "logit_scale": 0.5,
            "norm": {"eps": 1e-5}, "layers": [{"type": "latent_attention", "mixer": mix1, "mlp": mlp},
                                              {"type": "latent_attention_2", "mixer": mix2, "mlp": None}]}


def test_config_is_read_from_the_dictionary_and_round_trips():
    cfg = config_from_dict(small_config())
    assert isinstance(cfg, VoduzenConfig) and cfg.vocab_size == 160 and cfg.hidden_size == 96 and cfg.norm_eps == 1e-5
    a, b = cfg.layers
    assert a.mixer.sink and a.mixer.q_rank is None and a.mixer.rot.scaling["factor"] == 8.0
    assert not b.mixer.sink and b.mixer.q_rank == 56 and b.mixer.rot.dims == 8 and b.mixer.rot_dim == 16 and b.mlp is None
    assert a.mlp.experts == 5 and a.mlp.identity == 2 and a.mlp.top == 3 and a.mlp.shared_ff == 72
    assert VoduzenConfig.from_dict(cfg.to_dict()) == cfg
    assert registry.MODEL_CLASSES[VoduzenConfig][1] == "VoduzenForCausalLM"
    bad = small_config()
    bad["layers"][0]["type"] = "something_else"
    with pytest.raises(ValueError):
        config_from_dict(bad)


@pytest.mark.parametrize("scaling", [None, {"factor": 8.0, "fast": 16.0, "original": 64, "slow": 2.0},
                                     {"factor": 2.0, "fast": 4.0, "original": 4096, "slow": 4.0}])
def test_rotary_frequencies_match_the_plain_tables(scaling):
    rot = {"dims": 12, "base": 777.0}
    if scaling:
        rot["scaling"] = scaling
    f, mult = RotarySpec(dims=12, base=777.0, scaling=scaling).frequencies()
    cos, sin = O.rotary_angles(rot, 50)
    ang = torch.arange(50, dtype=torch.float64)[:, None] * torch.tensor(f, dtype=torch.float64)[None]
    assert torch.allclose(ang.cos() * mult, cos, atol=1e-12) and torch.allclose(ang.sin() * mult, sin, atol=1e-12)
    if scaling:
        assert mult == pytest.approx(0.1 * math.log(scaling["factor"]) + 1.0)
        assert f[0] == pytest.approx(1.0) or f[0] == pytest.approx(1.0 / scaling["factor"])


def test_page_allocator_hands_freed_pages_out_first():
    a = PageAllocator(5, first=1)
    x = a.take(3)
    assert x == [1, 2, 3] and a.available() == 2
    a.give([2])
    assert a.take(2) == [2, 4]
    with pytest.raises(RuntimeError):
        a.take(2)


class _Recorder:
    """Stands in for a model: keeps the batches it is given and answers with the position of each wanted row."""

    class _Dec:
        def __init__(self, outer):
            self.outer = outer

        def new_cache(self, n_pages, n_slots, max_pages_per_slot=0):
            return PagedLatentCache([4], n_pages, n_slots, self.outer.config.kv_page_size, torch.float32, "cpu", max_pages_per_slot)

    def __init__(self, page):
        self.config = VoduzenConfig(kv_page_size=page)
        self.device = torch.device("cpu")
        self.decoder = _Recorder._Dec(self)
        self.batches = []

    def step(self, tokens, pos, slot, cache, want_rows=None, collect=None, portions=None):
        self.batches.append((tokens.tolist(), pos.tolist(), slot.tolist(), cache.table_host.clone()))
        if want_rows is None:
            return None
        return torch.stack([pos[want_rows].float(), slot[want_rows].float()], dim=1)


def test_scheduler_positions_slots_and_page_reuse():
    m = _Recorder(page=4)
    s = StepScheduler(m, max_tokens=24, slots=2)
    assert s.pages.count == 6
    out = s.run_step([("a", [7, 8, 9, 10, 11], [4]), ("b", [1], [0])])
    toks, pos, slot, table = m.batches[-1]
    assert toks == [7, 8, 9, 10, 11, 1] and pos == [0, 1, 2, 3, 4, 0] and slot[:5] == [slot[0]] * 5 and slot[5] != slot[0]
    assert out[:, 0].tolist() == [4.0, 0.0]
    pa = table[slot[0], :2].tolist()
    assert len(set(pa)) == 2 and 0 not in pa                        # two pages for five tokens, never the scratch page
    s.run_step([("a", [12, 13, 14], [])])                           # b skips a step; a goes on inside its second page
    assert m.batches[-1][1] == [5, 6, 7] and s.live["a"].pages == pa
    s.run_step([("a", [15], [0]), ("b", [2, 3], [1])], end=["a"])   # a crosses into a third page, then ends
    assert m.batches[-1][1] == [8, 1, 2] and "a" not in s.live
    with pytest.raises(RuntimeError):                                # a third request while two are live: no slot
        s.run_step([("b", [4], []), ("c", [1], []), ("d", [1], [])])
    s.release("c")
    freed_slot = slot[0]
    s.run_step([("e", list(range(9)), [8])])                         # takes a's slot and its pages again
    assert m.batches[-1][2] == [freed_slot] * 9 and set(pa) <= set(s.live["e"].pages)
    s.release("b")
    s.release("e")
    assert s.pages.available() == 6 and len(s.free_slots) == 2
    with pytest.raises(RuntimeError):                                # more tokens than the pool holds
        s.run_step([("f", list(range(25)), [])])
