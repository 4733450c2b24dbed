"""Simivik's configuration and model description, on the CPU: every size and constant comes from config.json, a layer
that runs another's tensors has a cache of its own, the pages of a window's kept first tokens stay while the others go
back, and what cannot run is refused with the key's name."""
import copy

import pytest
import torch

import plain_simivik as plain
import tiny_simivik as ts
from atom_b200.cache.manager import NO_PAGE, CacheManager
from atom_b200.config.model_config import ConfigError, config_from_dict
from atom_b200.models.model import Model
from atom_b200.models.registry import build_model_spec
from atom_b200.parts.spec import CacheNeed
from atom_b200.weights.loader import expected_tensors


@pytest.mark.parametrize("name", list(ts.CONFIGS))
def test_config_round_trip_and_tensor_names(name):
    cfg = config_from_dict(ts.CONFIGS[name])
    assert cfg.architecture == "Simivik"
    assert config_from_dict(cfg.to_dict()) == cfg
    model = Model(build_model_spec(cfg))
    want = expected_tensors(model)
    have = ts.random_tensors(ts.CONFIGS[name], 1)
    assert set(want) == set(have)
    for n, (_, _, _, shape, _) in want.items():
        assert tuple(have[n].shape) == tuple(shape), n


def test_layers_on_anothers_tensors_have_their_own_cache():
    spec = build_model_spec(config_from_dict(ts.CONFIGS["A"]))
    assert len(spec.layers) == 2                                       # two layers' tensors, run twice each
    assert [(e.layer, e.cache) for e in spec.run_order] == [(0, 0), (1, 1), (0, 2), (1, 3)]
    needs = Model(spec).cache_needs()
    assert needs[0].kind == needs[2].kind == "pages" and needs[0].window == 24 and needs[0].keep_first == 5
    assert {e.name: e.shape for e in needs[0].entries} == {"k": (2, 16), "v": (2, 24)}
    assert {e.name: e.shape for e in needs[0].states} == {"conv": (2, (4 + 2) * 16 + 2 * 24)}
    assert needs[1].kind == needs[3].kind == "state" and {e.name: e.shape for e in needs[1].states} == {"S": (2, 16, 24)}
    assert needs[1].states[0].dtype == "float32"


def test_one_decay_for_all_heads():
    c = copy.deepcopy(ts.CONFIGS["A"])
    c["layers"][1]["mixer"]["decay"] = 0.75
    c["layers"][3]["mixer"]["decay"] = 0.75
    assert config_from_dict(c).layers[1].mixer.decay == (0.75, 0.75)


def test_zero_stands_for_an_option_left_out():
    c = copy.deepcopy(ts.CONFIGS["B"])
    m = c["layers"][2]["mixer"]
    m.update(softcap=0, conv=0)
    m["rot"]["dims"] = 0
    layer = config_from_dict(c).layers[2]
    assert layer.mixer.softcap is None and layer.mixer.taps is None and layer.mixer.rot_dims == 0
    spec = build_model_spec(config_from_dict(c))
    assert spec.layers[2].parts["mixer"].args["position"] is None and spec.layers[2].parts["mixer"].args["taps"] is None


def test_options_left_out_of_the_config():
    needs = Model(build_model_spec(config_from_dict(ts.CONFIGS["B"]))).cache_needs()
    assert needs[1].window is None and needs[1].keep_first == 0 and not needs[1].states      # no window, no convolution
    assert needs[2].window == 7 and needs[2].keep_first == 0 and needs[2].states[0].shape == (1, 3 * 8 + 3 * 8 + 3 * 40)
    needs = Model(build_model_spec(config_from_dict(ts.CONFIGS["C"]))).cache_needs()
    assert needs[0].window == 1 and needs[0].keep_first == 1 and not needs[0].states         # one tap keeps no rows
    assert needs[2].keep_first == 40 and needs[2].window == 33


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),                 # itself
    (lambda c: c["layers"][2].update(weights_of=9), "weights_of"),                 # no such layer
    (lambda c: c["layers"][2]["mixer"].update(dim=32), "other sizes"),             # not the sizes of the tensors' owner
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),        # more than the head holds
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),         # odd
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1].update(type="lstm"), "type"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "router.top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "mlp.kind"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=-1.0), "softcap"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.'size'"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_refusals_name_the_key(edit, word):
    c = copy.deepcopy(ts.CONFIGS["A"])
    edit(c)
    with pytest.raises(ConfigError, match=word.replace(".", r"\.")):
        config_from_dict(c)


def test_pages_of_kept_first_tokens_stay_while_the_window_moves():
    """Window 20 keeping the first 11 positions over pages of 8: the first two pages stay for the request's life, the
    others go back once the window has passed them, and all of them when the request ends."""
    need = CacheNeed("pages", num_kv_heads=2, head_dim=16, window=20, keep_first=11)
    cm = CacheManager({0: need}, page_size=8, num_pages=7, max_requests=2)
    cm.admit("a")
    first_two = None
    for n in range(1, 200):
        cm.extend("a", n)
        cm.commit("a", n)
        table = cm.table("a", 0)
        if n == 16:
            first_two = table[:2]
        if n >= 16:
            assert table[:2] == first_two and NO_PAGE not in first_two
        live = [p for p in table if p != NO_PAGE]
        assert len(live) <= 2 + 4                                  # the kept pages and the window's
        oldest = max(0, n - 20 + 1) // 8
        assert all(table[i] == NO_PAGE for i in range(2, min(oldest, len(table))))
        cm.check()
    cm.release("a")
    assert cm.num_free_pages(0) == 7
    # without kept tokens the same pool serves with two pages fewer
    cm = CacheManager({0: CacheNeed("pages", num_kv_heads=2, head_dim=16, window=20)}, page_size=8, num_pages=5, max_requests=2)
    cm.admit("b")
    for n in range(1, 100):
        cm.extend("b", n)
        cm.commit("b", n)
    assert sum(p != NO_PAGE for p in cm.table("b", 0)) <= 4


def test_groups_differ_by_kept_tokens_and_peak_counts_them():
    a = CacheNeed("pages", num_kv_heads=1, head_dim=8, window=16, keep_first=4)
    b = CacheNeed("pages", num_kv_heads=1, head_dim=8, window=16, keep_first=0)
    c = CacheNeed("pages", num_kv_heads=1, head_dim=8, window=16, keep_first=4)
    cm = CacheManager({0: a, 1: b, 2: c}, page_size=4, num_pages=32, max_requests=2)
    assert cm.slot_group[0] == cm.slot_group[2] != cm.slot_group[1]
    peak = cm.peak_pages(1000, 8)
    assert peak[cm.slot_group[0]] == peak[cm.slot_group[1]] + 1


def test_plain_mechanisms_are_what_the_formulas_say():
    """The plain implementation itself on cases small enough to do by hand."""
    F = torch.float64
    seen = plain.visible(6, 2, 1)
    assert seen.int().tolist() == [[1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0], [1, 0, 1, 1, 0, 0],
                                   [1, 0, 0, 1, 1, 0], [1, 0, 0, 0, 1, 1]]
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=F)
    assert plain.short_conv(u, torch.tensor([[10.0, 1.0]], dtype=F)).flatten().tolist() == [1.0, 12.0, 23.0]
    q = k = torch.ones(3, 1, 1, dtype=F)
    v = torch.tensor([1.0, 2.0, 4.0], dtype=F).view(3, 1, 1)
    assert plain.decayed_state(q, k, v, [0.5]).flatten().tolist() == [1.0, 2.5, 5.25]
    x = torch.tensor([[3.0, 4.0]], dtype=F)
    assert torch.allclose(plain.rms_norm(x, torch.tensor([1.0, 0.0], dtype=F), 0.0, around_zero=True),
                          torch.tensor([[6.0, 4.0]], dtype=F) / 12.5 ** 0.5)
    r = plain.rotate_front(torch.tensor([[[1.0, 0.0, 5.0]], [[1.0, 0.0, 5.0]]], dtype=F), 2, 100.0)
    assert torch.allclose(r[1, 0], torch.tensor([0.5403023058681398, 0.8414709848078965, 5.0], dtype=F))
