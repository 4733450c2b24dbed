"""Kibotar without a GPU: the configuration's keys and refusals, the run order of a span that runs several times, what
the parts ask of the cache manager (rows per block of positions beside windowed pages), and the plain implementation's
functions on cases done by hand."""
import copy
import math

import pytest
import torch

import plain_kibotar as plain
import tiny_kibotar as tk
from atom_b200.cache import CacheManager
from atom_b200.config.model_config import ConfigError, config_from_dict
from atom_b200.models.kibotar import KibotarConfig, build_kibotar_spec
from atom_b200.models.model import EMBEDDING_CACHE, Model
from atom_b200.parts.spec import CacheEntry, CacheNeed


def _cfg(name):
    return KibotarConfig.from_dict(copy.deepcopy(tk.CONFIGS[name]))


@pytest.mark.parametrize("name", list(tk.CONFIGS))
def test_config_round_trip_and_run_order(name):
    cfg = _cfg(name)
    assert KibotarConfig.from_dict(cfg.to_dict()) == cfg
    assert config_from_dict(cfg.to_dict(), None) == cfg
    raw = tk.CONFIGS[name]
    want = plain.run_order(raw)
    got = cfg.run_order()
    assert [(i, t) for i, _, t in got] == [(i, t if (t is not None and i == raw["loop"]["start"]) else None) for i, t in want]
    assert sorted(slot for _, slot, _ in got) == list(range(len(got)))          # a cache of its own for every run
    spec = build_kibotar_spec(cfg)
    assert [(e.layer, e.cache, e.add_step) for e in spec.run_order] == got
    model = Model(spec)
    needs = model.cache_needs()
    assert set(needs) == {EMBEDDING_CACHE} | set(range(len(got)))
    assert needs[EMBEDDING_CACHE].states[0].dtype == "int32"


def test_sizes_come_from_shapes_and_keys():
    raw = tk.folder_config(tk.CONFIGS["A"])
    with pytest.raises(ConfigError, match="rank"):
        KibotarConfig.from_dict(copy.deepcopy(raw))                            # no checkpoint and no key
    shapes = {"l2.mix.a1": (7, 64)}
    cfg = KibotarConfig.from_dict(copy.deepcopy(raw), shapes)
    assert cfg.layers[2].mixer.rank == 7
    with pytest.raises(ConfigError, match="a1"):
        KibotarConfig.from_dict(copy.deepcopy(raw), {})


@pytest.mark.parametrize("path,value,match", [
    (("layers", 1, "mixer", "heads"), 3, "multiple of kv_heads"),
    (("layers", 1, "mixer", "rot", "dims"), 18, "rot.dims"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 1, "mixer", "mask", "size"), 0, "size"),
    (("layers", 2, "mixer", "tau"), 0.0, "tau"),
    (("layers", 0, "type"), "conv", "not supported"),
    (("layers", 0, "mlp"), {"kind": "moe"}, "dense"),
    (("loop", "stop"), 9, "loop"),
    (("loop", "times"), 0, "times"),
    (("embedding", "bigram", "buckets"), 0, "buckets"),
    (("norm", "eps"), 0.0, "eps"),
])
def test_what_cannot_run_is_refused_with_the_keys_name(path, value, match):
    raw = copy.deepcopy(tk.CONFIGS["A"])
    d = raw
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError, match=match):
        KibotarConfig.from_dict(raw)


def test_absent_keys_leave_their_step_out():
    raw = copy.deepcopy(tk.CONFIGS["A"])
    del raw["loop"]
    del raw["layers"][1]["mixer"]["rot"]
    raw["layers"][1]["mixer"]["mask"] = {"size": 9, "pool": 0}
    cfg = KibotarConfig.from_dict(raw)
    m = cfg.layers[1].mixer
    assert cfg.loop is None and m.rot_base is None and m.window == 9 and m.pool is None
    spec = build_kibotar_spec(cfg)
    assert spec.stream_steps is None and all(e.add_step is None for e in spec.run_order)
    need = Model(spec).cache_needs()[1]
    assert need.window == 9 and not need.block_entries
    raw["loop"] = {"start": 2, "stop": 2, "times": 5}                          # an empty span
    assert KibotarConfig.from_dict(raw).loop is None


def test_cache_needs_of_the_mixers():
    needs = Model(build_kibotar_spec(_cfg("C"))).cache_needs()
    att = needs[2]                   # a window of 5 behind blocks of 16: the cache keeps a block's length
    assert att.kind == "pages" and att.window == 16 and att.block == 16
    assert [e.name for e in att.block_entries] == ["pk", "pv"] and [e.name for e in att.states] == ["shift.last"]
    first = needs[0]                 # a window of one token, blocks of 2
    assert first.window == 2 and first.block == 2
    assert needs[4].window == 33 and needs[4].block == 0
    gla = needs[1]
    assert gla.kind == "state" and {e.name: e.shape for e in gla.states} == {"shift.last": (44,), "mixer.S": (1, 12, 20)}
    lat = needs[3]
    assert lat.kind == "pages" and lat.window is None and lat.entries[0].shape == (24,)


def test_rows_per_block_live_in_a_group_of_their_own():
    """Pages of pooled rows: one row per whole block, page_size rows a page, never given back by the window."""
    e = (CacheEntry("k", (2, 8)), CacheEntry("v", (2, 8)))
    b = (CacheEntry("pk", (2, 8)), CacheEntry("pv", (2, 8)))
    need = CacheNeed("pages", window=24, entries=e, block=4, block_entries=b)
    m = CacheManager({0: need, 1: need, 2: CacheNeed("pages", window=24, entries=e)}, 8, 40, 3)
    assert len(m.groups) == 2 and m.groups[0].slots == [0, 1, 2] and m.groups[1].slots == [0, 1] and m.groups[1].block == 4
    assert m.slot_block_group == {0: 1, 1: 1}
    assert m.groups[1].pool.num_pages == 40 // 4 + 3
    m.admit("a")
    m.extend("a", 3)
    assert [len(m.requests["a"].tables[g]) for g in (0, 1)] == [1, 0]         # no whole block yet
    m.commit("a", 3)
    m.extend("a", 4)
    assert len(m.requests["a"].tables[1]) == 1                                  # the first block's row
    m.commit("a", 4)
    m.extend("a", 131)
    m.commit("a", 131)
    t0, t1 = m.requests["a"].tables[0], m.requests["a"].tables[1]
    assert len(t0) == 17 and len(t1) == 4 == -(-(131 // 4) // 8)
    assert sum(p != -1 for p in t0) == 4 and all(p != -1 for p in t1)          # the window's pages; every pooled page
    assert m.peak_pages(131, 16)[1] == 4
    m.check()
    m.admit("b")
    m.extend("b", 40)
    m.release("a")
    m.check()
    assert m.groups[1].pool.num_used == 2
    m.release("b")
    assert all(g.pool.num_used == 0 for g in m.groups)
    with pytest.raises(ValueError):
        CacheNeed("pages", entries=e, block=4)
    with pytest.raises(ValueError):
        CacheNeed("state", block=4, block_entries=b)


def test_wavelength_frequencies_by_hand():
    from atom_b200.parts.rope import wavelength_frequencies
    f = wavelength_frequencies(8, 10000.0, 8.0, 64.0, 1.0, 4.0)
    base = [10000.0 ** (-2 * i / 8) for i in range(4)]
    assert f[0] == base[0]                                  # wavelength 6.3 < 64 / 4: kept
    assert f[2] == base[2] / 8.0 and f[3] == base[3] / 8.0  # wavelengths 628 and 6283 > 64: stretched
    wave = 2 * math.pi / base[1]                            # 62.8: between the two
    s = (64.0 / wave - 1.0) / 3.0
    assert abs(f[1] - ((1 - s) * base[1] / 8.0 + s * base[1])) < 1e-15 and base[1] / 8 < f[1] < base[1]
    assert plain.scaled_frequencies({"dims": 8, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0,
                                                                         "original": 64}}).tolist() == pytest.approx(f, rel=1e-15)


def test_plain_functions_by_hand():
    # embedding: the first token takes the last row of the pair table, later ones the hashed row
    table, pairs = torch.arange(12, dtype=plain.F).view(6, 2), torch.arange(8, dtype=plain.F).view(4, 2) * 100
    e = {"scale": 0.5, "bigram": {"buckets": 3, "mul_prev": 5, "mul_cur": 2}}
    x = plain.embed_tokens([4, 1, 3], table, pairs, e)
    assert x.tolist() == [[4 + 600, 4.5 + 700], [1 + 200, 1.5 + 300], [3 + 400, 3.5 + 500]]     # rows 3, (20+2)%3=1, (5+6)%3=2
    # token shift
    h = torch.tensor([[1.0, 2.0], [3.0, 6.0]], dtype=plain.F)
    assert plain.token_shift(h, torch.tensor([0.5, 0.0], dtype=plain.F)).tolist() == [[0.5, 2.0], [2.0, 6.0]]
    # gated linear attention: one head, one key channel, two value columns; decay sigmoid(0)^(1/2) = 2^(-1/2).  Column 1
    # gets its only value at token 0, column 0 at token 2: at token 2 the state holds (1, decay^2) = (1, 1/2)
    m = {"heads": 1, "dim": 1, "vdim": 2, "tau": 2.0}
    hh = torch.tensor([[1.0, 0.0, 1.0], [1.0, 0.0, 0.0], [1.0, 1.0, 0.0]], dtype=plain.F)
    const = torch.tensor([[1.0, 0.0, 0.0]], dtype=plain.F)
    P = {"q": const, "k": const, "v": torch.tensor([[0.0, 1.0, 0.0], [0.0, 0.0, 1.0]], dtype=plain.F),
         "g": torch.cat([const, const]) * 50.0, "o": torch.eye(2, dtype=plain.F), "a1": const * 0.0,
         "a2": torch.ones(1, 1, dtype=plain.F), "a2.b": torch.zeros(1, dtype=plain.F), "norm": torch.ones(2, dtype=plain.F)}
    y = plain.gated_linear_attention(hh, P, m, 0.0)
    rms = math.sqrt((1 + 0.25) / 2)
    assert y[2].tolist() == pytest.approx([50.0 / rms, 25.0 / rms])
    assert y[0].tolist() == pytest.approx([0.0, 50.0 * math.sqrt(2)])
    one = torch.ones(1, 1, dtype=plain.F)
    # attention: a window of 2 and blocks of 2, the sink in the denominator; zero queries give uniform weights
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "scale": 1.0, "mask": {"size": 2, "pool": 2}}
    z = torch.zeros(1, 1, dtype=plain.F)
    P = {"q": z, "q.b": torch.zeros(1, dtype=plain.F), "k": one, "k.b": torch.zeros(1, dtype=plain.F), "v": one,
         "v.b": torch.zeros(1, dtype=plain.F), "talk": one * 2.0, "g": z, "o": one, "o.b": torch.zeros(1, dtype=plain.F)}
    x = torch.tensor([[1.0], [2.0], [4.0], [8.0], [16.0]], dtype=plain.F)
    y = plain.pooled_window_attention(x, P, m)[:, 0]
    # position 3 sees tokens 2, 3 and block 0 (positions 0, 1: mean 1.5): (4 + 8 + 1.5) / 4, mixed by 2, gated by 1/2
    # position 2 sees tokens 1, 2 only (block 0 ends at 1 > 2 - 2): (2 + 4) / 3
    # position 4 sees tokens 3, 4 and block 0 (block 1 ends at 3 > 4 - 2)
    assert y.tolist() == pytest.approx([1 / 2, 3 / 3, 6 / 3, 13.5 / 4, 25.5 / 4])
