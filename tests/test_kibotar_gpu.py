"""Kibotar on the GPU against the plain implementation (tests/plain_kibotar.py): every mechanism's part alone through
the cache manager (requests of unequal lengths side by side, whole, in portions down to two tokens and token by token,
on pages and state slots that held other requests before), single keys made to stand out at every edge of the window
and of the pooled blocks, the sink, the mixing of the heads' weights, then whole models under every way of cutting the
work, long decoding, captured steps, and greedy generation through the engine's entry point."""
import math

import numpy as np
import pytest
import torch

import plain_kibotar as plain
import tiny_kibotar as tk
import traces
from test_simivik_gpu import (DEV, F64, Harness, _bind, _close, _compare, _dt, _i32, _junk_first, _replay, _rounded, _rt,
                              _runner, _schedules)

pytestmark = pytest.mark.gpu


# ============================================================================= token shift, embedding by pairs, norms

class _Echo:
    """A mixer that hands its input on, to see what a wrapper feeds it."""
    graph_safe = True
    defers_output = False

    def __init__(self, hidden_size):
        self.hidden_size = hidden_size

    def params(self):
        return {}

    def cache_need(self):
        return None

    def bind(self, tensors, rt):
        self.rt = rt

    def after_load(self):
        pass

    def launch_plan(self, step):
        pass

    def forward(self, x, step, cache, writes_cache):
        return x.clone()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_shift_carries_the_last_row_from_step_to_step(dtype):
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec
    registry.register("mixer", "test_echo")(_Echo)
    W = 44
    part = registry.build("mixer", PartSpec("token_shifted", {"hidden_size": W, "member": PartSpec("test_echo", {"hidden_size": W})}))
    g = torch.Generator().manual_seed(3)
    held = _bind(part, {"mu": torch.rand(1, W, generator=g)}, _rt(dtype))
    lens = {"a": 37, "b": 2, "c": 18}
    x = {r: _rounded(torch.randn(n, W, generator=g), dtype) for r, n in lens.items()}
    want = {r: plain.token_shift(x[r], held["mu"][0]) for r in lens}
    assert float((want["a"][0] - x["a"][0] * (1 - held["mu"][0])).abs().max()) < 1e-12      # zeros before the first row
    for what, sched in _schedules(lens):
        h = Harness(part, dtype)
        _junk_first(h, W)
        got = h.run(x, sched)
        for r in lens:
            _close(got[r], want[r], dtype, f"{what}, request {r}", f32=1e-6, bf16=8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(53, 31, 5), (1, 9, 4), (1019, 1 << 40, 999983), (7, 0, 1)])
def test_pair_embedding_remembers_the_previous_token(dtype, buckets, mul_prev, mul_cur):
    """The row of the pair table depends on the token before, also across steps and after the slot held another
    request; a request's first token takes the table's last row."""
    from atom_b200.cache import CacheManager
    from atom_b200.cache.storage import CacheStorage
    from atom_b200.engine.batch import StepBuilder, StepEntry
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec
    V, W, scale = 97, 40, 0.37
    part = registry.build("embedding", PartSpec("pair_embedding", dict(vocab_size=V, hidden_size=W, buckets=buckets,
                                                                       mul_prev=mul_prev, mul_cur=mul_cur, scale=scale)))
    g = torch.Generator().manual_seed(buckets)
    held = _bind(part, {"weight": torch.randn(V, W, generator=g), "pairs": torch.randn(buckets + 1, W, generator=g)}, _rt(dtype))
    e = {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}
    rng = np.random.default_rng(5)
    toks = {r: rng.integers(0, V, size=n).tolist() for r, n in (("a", 30), ("b", 1), ("c", 11))}
    want = {r: plain.embed_tokens(t, held["weight"], held["pairs"], e) for r, t in toks.items()}
    manager = CacheManager({-1: part.cache_need()}, 8, 16, 2)
    storage = CacheStorage(manager, _dt(dtype), torch.device(DEV))
    builder = StepBuilder(manager, DEV, V, torch.zeros(1, dtype=torch.int32, device=DEV))
    done = {r: 0 for r in toks}
    got = {r: [] for r in toks}
    # a and b side by side in ragged portions; c comes later into a slot that b has left
    for portions in ({"a": 4, "b": 1}, {"a": 1}, {"a": 2, "c": 5}, {"c": 1, "a": 20}, {"a": 3, "c": 5}):
        entries, targets = [], []
        for r, n in portions.items():
            if r not in manager.requests:
                manager.admit(r)
            entries.append(StepEntry(r, toks[r][done[r]:done[r] + n], ()))
            targets.append(done[r] + n)
        ctx = builder.build(entries, targets)
        y = part.forward(ctx.token_ids, ctx.num_tokens, ctx, storage.view(-1)).double().cpu()
        o = 0
        for (r, n), t in zip(portions.items(), targets):
            got[r].append(y[o:o + n])
            o += n
            done[r] = t
            manager.commit(r, t)
            if t == len(toks[r]):
                manager.release(r)
    for r in toks:
        _close(torch.cat(got[r]), want[r], "float32", f"request {r}", f32=1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W", [44, 200, 1000])
def test_norm_after_a_sub_block_fused_with_the_next_norm(dtype, W):
    """residual += rmsnorm(delta; w1); out = rmsnorm(residual; w2) in one kernel, also on picked rows."""
    from atom_b200 import native
    g = torch.Generator().manual_seed(W)
    T, eps = 9, 1e-5
    dt = _dt(dtype)
    res = torch.randn(T, W, generator=g) * 3
    delta = _rounded(torch.randn(T, W, generator=g) * 5, dtype)
    w1, w2 = _rounded(torch.rand(W, generator=g) + 0.5, dtype), _rounded(torch.rand(W, generator=g) + 0.5, dtype)
    want_res = res.double() + plain.rms_norm(delta, w1, eps)
    want_out = plain.rms_norm(want_res, w2, eps)
    r = res.to(DEV).contiguous()
    out = torch.empty(T, W, dtype=dt, device=DEV)
    native.normed_add_rmsnorm(out, r, delta.to(dt).to(DEV), w1.to(dt).to(DEV), eps, w2.to(dt).to(DEV), eps)
    _close(r, want_res, "float32", "residual", f32=2e-6)
    _close(out, want_out, dtype, "normalised rows", f32=2e-6, bf16=8e-3)
    rows = [7, 0, 3]
    r2 = res.to(DEV).contiguous()
    out2 = torch.empty(3, W, dtype=dt, device=DEV)
    native.normed_add_rmsnorm(out2, r2, delta.to(dt).to(DEV), w1.to(dt).to(DEV), eps, w2.to(dt).to(DEV), eps, _i32(rows), 3)
    _close(out2, want_out[rows], dtype, "picked rows", f32=2e-6, bf16=8e-3)
    assert torch.equal(r2.cpu(), res)                      # picked rows leave the stream as it is


# ============================================================================= gated linear attention

GLA_CASES = [  # H, dk, dv, tau, rank, lens
    (2, 16, 24, 8.0, 4, (70, 9, 41)),
    (3, 8, 40, 2.0, 8, (37, 5, 18)),
    (1, 12, 20, 1.0, 3, (50, 2, 31)),
    (4, 4, 8, 32.0, 1, (33, 64, 65)),
    (2, 64, 64, 16.0, 16, (300, 40, 131)),
    (2, 128, 96, 16.0, 8, (130, 3, 70)),
    (5, 32, 48, 12.0, 12, (2100, 7, 200)),
]


def _gla_part(case, dtype, width=72):
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    H, dk, dv, tau, rank, lens = case
    eps = 1e-5
    part = registry.build("mixer", PartSpec("gated_linear_attention", dict(
        hidden_size=width, num_heads=H, key_dim=dk, value_dim=dv, decay_rank=rank, tau=tau, norm_eps=eps)))
    g = torch.Generator().manual_seed(H * dk + dv)
    mats = [torch.randn(n, width, generator=g) * 1.5 / width ** 0.5 for n in (H * dk, H * dk, H * dv, H * dv, rank)]
    held = _bind(part, {"in.weight": torch.cat(mats), "a2.weight": torch.randn(H * dk, rank, generator=g) * 2.0 / rank ** 0.5,
                        "a2.bias": torch.rand(H * dk, generator=g) * 4.0, "norm": torch.rand(dv, generator=g) * 0.6 + 0.7,
                        "o.weight": torch.randn(width, H * dv, generator=g) / (H * dv) ** 0.5}, _rt(dtype))
    a, b, c = H * dk, 2 * H * dk, 2 * H * dk + H * dv
    w = held["in.weight"]
    P = {"q": w[:a], "k": w[a:b], "v": w[b:c], "g": w[c:c + H * dv], "a1": w[c + H * dv:], "a2": held["a2.weight"],
         "a2.b": held["a2.bias"], "norm": held["norm"], "o": held["o.weight"]}
    return part, {"heads": H, "dim": dk, "vdim": dv, "tau": tau}, P, eps, width


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", GLA_CASES)
def test_gla_part_under_every_cut(case, dtype):
    """The state goes from step to step in the request's slot, whatever the cut; steps of many rows take the form that
    sums runs of rows up side by side, and give the same numbers."""
    part, m, P, eps, W = _gla_part(case, dtype)
    lens = dict(zip("abc", case[5]))
    g = torch.Generator().manual_seed(sum(case[5]))
    x = {r: _rounded(torch.randn(n, W, generator=g), dtype) for r, n in lens.items()}
    want = {r: plain.gated_linear_attention(x[r], P, m, eps) for r in lens}
    for what, sched in _schedules(lens):
        if what == "pairs" and max(lens.values()) > 400:
            continue
        h = Harness(part, dtype)
        _junk_first(h, W)
        got = h.run(x, sched)
        for r in lens:
            _close(got[r], want[r], dtype, f"{what}, request {r}", f32=5e-5, bf16=4e-2)


def test_gla_state_remembers_a_far_token():
    """With decays of almost one a key written at the first token is still read 600 tokens later, through 600 single
    steps; with a short memory it is gone."""
    from atom_b200 import native
    H, dk, dv, T = 1, 16, 16, 600
    for bias, tau, stays in ((12.0, 16.0, True), (-2.0, 1.0, False)):
        q = torch.zeros(T, H * dk)
        k = torch.zeros(T, H * dk)
        v = torch.zeros(T, H * dv)
        k[0, 3], v[0, 5] = 1.0, 1.0
        q[:, 3] = 1.0
        z = torch.zeros(T, H * dk)
        state = torch.zeros(1, H, dk, dv, device=DEV)
        outs = []
        for t in range(T):
            o = torch.zeros(1, H * dv, device=DEV)
            native.gla_scan(o, q[t:t + 1].to(DEV), k[t:t + 1].to(DEV), v[t:t + 1].to(DEV), z[t:t + 1].to(DEV),
                            torch.full((H * dk,), bias, device=DEV), tau, 1.0, state, None, None, _i32([0, 1]), _i32([0]), 1,
                            H, dk, dv)
            outs.append(float(o[0, 5]))
        want = math.exp(-math.log1p(math.exp(-bias)) / tau * (T - 1))
        assert abs(outs[-1] - want) <= 1e-4 * max(want, 1e-3) and (outs[-1] > 0.9) == stays and outs[0] == 1.0


# ============================================================================= latent attention without positions

LAT_CASES = [  # H, dn, dv, R, lens, page
    (3, 8, 12, 64, (70, 9, 41), 16),
    (2, 16, 8, 64, (37, 5, 18), 8),
    (1, 28, 12, 24, (50, 2, 31), 16),
    (6, 48, 64, 128, (300, 40, 131), 16),
    (4, 64, 32, 128, (130, 3, 70), 32),
]


def _latent_part(case, dtype, width=72):
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    H, dn, dv, R, lens, page = case
    eps, scale = 1e-5, 1.7 / dn ** 0.5
    part = registry.build("mixer", PartSpec("latent_attention", dict(
        hidden_size=width, num_heads=H, head_dim=dn, rot_dim=0, value_dim=dv, q_rank=None, kv_rank=R, scale=scale,
        norm_eps=eps, position=None, gate="head")))
    g = torch.Generator().manual_seed(H * dn + dv)
    mats = [torch.randn(n, width, generator=g) * s / width ** 0.5 for n, s in ((H * dn, 2.0), (R, 1.0), (H, 2.0))]
    held = _bind(part, {"in.weight": torch.cat(mats), "dkv.norm": torch.rand(R, generator=g) * 0.6 + 0.7,
                        "uk.weight": torch.randn(H * dn, R, generator=g) * 2.0 / R ** 0.5,
                        "uv.weight": torch.randn(H * dv, R, generator=g) / R ** 0.5,
                        "o.weight": torch.randn(width, H * dv, generator=g) / (H * dv) ** 0.5}, _rt(dtype))
    w = held["in.weight"]
    P = {"q": w[:H * dn], "dkv": w[H * dn:H * dn + R], "g": w[H * dn + R:], "dkv.norm": held["dkv.norm"],
         "uk": held["uk.weight"], "uv": held["uv.weight"], "o": held["o.weight"]}
    return part, {"heads": H, "dim": dn, "vdim": dv, "kv_rank": R, "scale": scale}, P, eps, width


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "bfloat16-plain"])
@pytest.mark.parametrize("case", LAT_CASES)
def test_latent_part_under_every_cut(case, dtype, monkeypatch):
    from atom_b200 import native
    if dtype.endswith("-plain"):
        if not native.latent_attention_tc_supports(case[0], case[3], 0, torch.bfloat16):
            pytest.skip("these sizes run the plain kernel anyway")
        monkeypatch.setattr(native, "LATENT_TC", False)
        dtype = "bfloat16"
    part, m, P, eps, W = _latent_part(case, dtype)
    lens, page = dict(zip("abc", case[4])), case[5]
    g = torch.Generator().manual_seed(sum(case[4]))
    x = {r: _rounded(torch.randn(n, W, generator=g), dtype) for r, n in lens.items()}
    want = {r: plain.latent_attention(x[r], P, m, eps) for r in lens}
    for what, sched in _schedules(lens):
        h = Harness(part, dtype, page=page, pages=3 * (max(lens.values()) // page + 3))
        _junk_first(h, W)
        got = h.run(x, sched)
        for r in lens:
            _close(got[r], want[r], dtype, f"{what}, request {r}", f32=3e-5, bf16=3e-2)
        assert all(gr.pool.num_used == 0 for gr in h.manager.groups) and h.manager.state_slots.num_free == 4


# ============================================================================= attention over a window and pooled blocks

ATT_CASES = [  # H, G, dk, dv, (base, dims, scaling), (window, pool), page, lens
    (4, 2, 16, 24, (10000.0, 8, (8.0, 1.0, 4.0, 64)), (24, 4), 16, (70, 9, 41)),
    (2, 1, 24, 16, (500.0, 24, None), None, 8, (50, 3, 27)),
    (3, 3, 8, 40, (77.0, 4, (2.0, 0.5, 2.0, 16)), (7, 1), 8, (40, 17, 2)),
    (5, 5, 20, 12, (1000.0, 12, None), (1, 2), 16, (33, 5, 20)),
    (6, 1, 12, 28, None, (5, 16), 16, (90, 48, 7)),
    (2, 2, 16, 16, (10000.0, 16, None), (33, None), 8, (64, 65, 63)),
    (8, 2, 64, 48, (200000.0, 32, (8.0, 1.0, 2.0, 512)), (120, 24), 16, (400, 40, 153)),
    (8, 4, 128, 128, (100000.0, 32, None), (50, 8), 32, (140, 60, 10)),
    (16, 4, 32, 64, (10000.0, 32, None), (17, 16), 16, (64, 33, 3)),
]


def _attention_part(case, dtype, width=72, zero_sink=True, talk=True, gate=True, bias=True):
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    H, G, dk, dv, rot, mask, page, lens = case
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "scale": 1.7 / dk ** 0.5}
    position = None
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        scaling = None
        if rot[2] is not None:
            scaling = dict(zip(("factor", "low", "high", "original"), rot[2]))
            m["rot"]["scaling"] = scaling
        position = PartSpec("rope_wavelength", {"rotary_dim": rot[1], "theta": rot[0], "scaling": scaling})
    if mask is not None:
        m["mask"] = {"size": mask[0]}
        if mask[1]:
            m["mask"]["pool"] = mask[1]
    part = registry.build("mixer", PartSpec("pooled_window_attention", dict(
        hidden_size=width, num_heads=H, num_kv_heads=G, key_dim=dk, value_dim=dv, scale=m["scale"], position=position,
        window=mask[0] if mask else None, pool=mask[1] if mask else None, zero_sink=zero_sink, talk=talk, gate=gate,
        bias=bias)))
    g = torch.Generator().manual_seed(H * dk + dv)
    rows = [(H * dk, 1.6), (G * dk, 1.6), (G * dv, 1.0)] + ([(H * dv, 2.0)] if gate else [])
    t = {"in.weight": torch.cat([torch.randn(n, width, generator=g) * s / width ** 0.5 for n, s in rows]),
         "o.weight": torch.randn(width, H * dv, generator=g) / (H * dv) ** 0.5}
    if bias:
        t["qkv.bias"] = torch.randn((H + G) * dk + G * dv, generator=g) * 0.3
        t["o.bias"] = torch.randn(width, generator=g) * 0.2
    if talk:
        t["talk"] = torch.eye(H) * 0.7 + torch.randn(H, H, generator=g) * 0.3
    held = _bind(part, t, _rt(dtype))
    nq, nk, nv = H * dk, G * dk, G * dv
    w = held["in.weight"]
    P = {"q": w[:nq], "k": w[nq:nq + nk], "v": w[nq + nk:nq + nk + nv], "o": held["o.weight"]}
    zeros = lambda n: torch.zeros(n, dtype=F64)
    b = held.get("qkv.bias")
    P.update({"q.b": b[:nq] if bias else zeros(nq), "k.b": b[nq:nq + nk] if bias else zeros(nk),
              "v.b": b[nq + nk:] if bias else zeros(nv), "o.b": held["o.bias"] if bias else zeros(width),
              "talk": held["talk"] if talk else torch.eye(H, dtype=F64),
              "g": w[nq + nk + nv:] if gate else None})
    return part, m, P, width


def _plain_attention(x, P, m, zero_sink=True, gate=True):
    """The plain function with the options a part may leave out (no sink: an ordinary softmax; no gate)."""
    if zero_sink and gate:
        return plain.pooled_window_attention(x, P, m)
    Q = dict(P)
    if not gate:
        Q["g"] = torch.zeros(m["heads"] * m["vdim"], x.shape[1], dtype=F64)
    y = plain.pooled_window_attention(x, Q, m)
    assert zero_sink, "the plain function always holds the sink"
    return (y - P["o.b"]) * 2.0 + P["o.b"] if not gate else y        # (sigmoid(0) = 1/2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "bfloat16-plain", "float32-whole"])
@pytest.mark.parametrize("case", ATT_CASES)
def test_attention_part_under_every_cut(case, dtype, monkeypatch):
    """(bfloat16 runs the tensor-core kernel where it takes the sizes; "bfloat16-plain" the plain kernel there too;
    steps of few tokens share their keys out among CTAs, "float32-whole" leaves that form out.)"""
    from atom_b200 import native
    if dtype.endswith("-plain"):
        if not native.pooled_attention_tc_supports(case[0], case[1], case[2], case[3], torch.bfloat16):
            pytest.skip("these sizes run the plain kernel anyway")
        monkeypatch.setattr(native, "POOLED_TC", False)
        dtype = "bfloat16"
    if dtype.endswith("-whole"):
        monkeypatch.setattr(native, "POOLED_SPLIT_ROWS", 0)
        dtype = "float32"
    part, m, P, W = _attention_part(case, dtype)
    page, lens = case[6], dict(zip("abc", case[7]))
    g = torch.Generator().manual_seed(sum(case[7]))
    x = {r: _rounded(torch.randn(n, W, generator=g), dtype) for r, n in lens.items()}
    want = {r: plain.pooled_window_attention(x[r], P, m) for r in lens}
    for what, sched in _schedules(lens):
        h = Harness(part, dtype, page=page, pages=3 * (max(lens.values()) // page + 3))
        _junk_first(h, W)
        got = h.run(x, sched)
        for r in lens:
            _close(got[r], want[r], dtype, f"{what}, request {r}", f32=3e-5, bf16=3e-2)
        assert all(gr.pool.num_used == 0 for gr in h.manager.groups) and h.manager.state_slots.num_free == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_part_without_gate_and_bias(dtype):
    case = (4, 2, 16, 24, (10000.0, 8, None), (24, 4), 16, (70, 9, 41))
    part, m, P, W = _attention_part(case, dtype, gate=False, bias=False, talk=False)
    lens = dict(zip("abc", case[7]))
    g = torch.Generator().manual_seed(1)
    x = {r: _rounded(torch.randn(n, W, generator=g), dtype) for r, n in lens.items()}
    want = {r: _plain_attention(x[r], P, m, gate=False) for r in lens}
    h = Harness(part, dtype, page=16, pages=24)
    got = h.run(x, list(_schedules(lens))[2][1])
    for r in lens:
        _close(got[r], want[r], dtype, f"request {r}", f32=3e-5, bf16=3e-2)


def _pages(n_rows, G, page, d, dtype, seed, extra=3):
    g = torch.Generator().manual_seed(seed)
    n_pages = max(1, -(-n_rows // page))
    order = torch.randperm(n_pages + extra, generator=g)[:n_pages]
    table = order.to(torch.int32).view(1, -1).to(DEV)
    return table, torch.full((n_pages + extra, G, page, d), float("nan"), dtype=_dt(dtype), device=DEV)


def _kernels(H, G, dk, dv, dtype):
    """The kernels that take these sizes: the plain one always, the tensor-core one where it does."""
    from atom_b200 import native
    out = ["plain"]
    if native.pooled_attention_split_supports(H, G, dk, dv):
        out += ["split1", "split3", "split7"]          # the keys of every token alone, and shared out among 3 and 7 CTAs
    return out + (["tc"] if native.pooled_attention_tc_supports(H, G, dk, dv, _dt(dtype)) else [])


def _run_pooled_attention(q, k, v, scale, window, pool, dtype, page, cuts, sink=True, mix=None, kernel="plain"):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] of ONE request, keys and values laid into scrambled pages and the
    blocks' means formed by the pooling kernel as the tokens come; the queries are run in portions ``cuts``."""
    from atom_b200 import native

    T, H, dk = q.shape
    G, dv = k.shape[1], v.shape[2]
    dt = _dt(dtype)
    table, kp = _pages(T, G, page, dk, dtype, T)
    _, vp = _pages(T, G, page, dv, dtype, T)
    ptable, pkp = _pages(T // pool if pool else 1, G, page, dk, dtype, T + 1)
    _, pvp = _pages(T // pool if pool else 1, G, page, dv, dtype, T + 1)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.zeros(T, H * dv, dtype=dt, device=DEV)
    mixd = None if mix is None else mix.float().to(DEV).contiguous()
    at = 0
    for n in cuts:
        n = min(n, T - at)
        if n <= 0:
            continue
        j = torch.arange(at, at + n, device=DEV)
        pg = table[0].long()[j // page]
        kp[pg, :, j % page] = k[at:at + n].to(dt).to(DEV)
        vp[pg, :, j % page] = v[at:at + n].to(dt).to(DEV)
        pos, seq = _i32(range(at, at + n)), _i32([0] * n)
        if pool:
            native.pool_blocks(kp, vp, pkp, pvp, table, ptable, page, pos, seq, n, pool, status)
        o = torch.zeros(n, H * dv, dtype=dt, device=DEV)
        qd = q[at:at + n].reshape(n, H * dk).to(dt).to(DEV).contiguous()
        if kernel.startswith("split"):
            ns = int(kernel[5:])
            scratch = torch.full((native.pooled_attention_scratch_elems(n, H, G, dv, ns),), float("nan"),
                                 dtype=torch.float32, device=DEV)
            native.pooled_attention_split(o, scratch, qd, kp, vp, pkp if pool else None, pvp if pool else None, table,
                                          ptable if pool else None, page, pos, seq, H, scale, window, pool, sink, mixd,
                                          None, ns)
        elif kernel == "tc":
            native.pooled_attention_tc(o, qd, kp, vp, pkp if pool else None, pvp if pool else None, table,
                                       ptable if pool else None, page, pos, _i32([0, n]), 1, H, scale, window, pool, sink,
                                       mixd, None)
        else:
            native.pooled_attention(o, qd, kp, vp, pkp if pool else None, pvp if pool else None, table,
                                    ptable if pool else None, page, pos, seq, H, scale, window, pool, sink, mixd, None)
        out[at:at + n] = o
        at += n
    assert at == T and int(status.item()) == 0
    return out.double().cpu().view(T, H, dv)


def _plain_weights(q, k, v, scale, window, pool, sink=True, mix=None):
    T, H, _ = q.shape
    G = k.shape[1]
    nb = T // pool if pool else 0
    if nb:
        k = torch.cat([k, k[:nb * pool].view(nb, pool, G, -1).mean(1)], 0)
        v = torch.cat([v, v[:nb * pool].view(nb, pool, G, -1).mean(1)], 0)
    per = H // G
    kk, vv = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) & ((i - j < window) if window else (j <= i))
    if nb:
        seen = torch.cat([seen, torch.arange(nb)[None, :] * pool + pool - 1 <= i - window], 1)
    e = torch.exp(s.masked_fill(~seen[None], -math.inf))
    a = e / ((1.0 if sink else 0.0) + e.sum(-1, keepdim=True))
    if mix is not None:
        a = torch.einsum("hg,gij->hij", mix, a)
    return torch.einsum("hij,jhd->ihd", a, vv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,pool", [(1, 1), (2, 3), (16, 4), (17, 16), (40, 8), (64, 64), (120, 24), (300, 7), (5, 32)])
def test_single_keys_at_the_windows_edge_and_in_pooled_blocks(window, pool, dtype):
    """One key row in the middle of the request carries a mark that only it has and a score far above all others.  It is
    seen as a token at distance window - 1 and not at distance window; from the position at which its block lies wholly
    before the window it is seen again, as a pool-th of the block's mean; in between it is not seen at all.  In a
    prompt, across portions that end at every place around the edges and a page's border, and decoded one by one."""
    H, G, dk, dv, page, T = 4, 2, 32, 16, 16, 520
    needle = 181
    g = torch.Generator().manual_seed(window * 100 + pool)
    k = torch.randn(T, G, dk, generator=g) * 0.1
    v = torch.randn(T, G, dv, generator=g) * 0.1
    q = torch.randn(T, H, dk, generator=g) * 0.1
    v[:, :, 0] = 0.0
    k[:, :, 0] = 0.0
    q[:, :, 0] = 3.0
    v[needle, :, 0] = 1.0
    k[needle, :, 0] = 4.0 * min(pool, 16)     # also its block's mean scores 3 to 12 against a few hundredths
    q, k, v = _rounded(q, dtype), _rounded(k, dtype), _rounded(v, dtype)
    want = _plain_weights(q, k, v, 1.0, window, pool)
    block_end = (needle // pool) * pool + pool - 1
    as_token = lambda i: 0 <= i - needle < window
    as_block = lambda i: block_end <= i - window
    assert all((want[i, :, 0].min() > 0.05 / pool) == (as_token(i) or as_block(i)) for i in range(T))
    assert all(float(want[i, :, 0].abs().max()) == 0 for i in range(T) if not (as_token(i) or as_block(i)))
    edge, first = needle + window, block_end + window
    cut_sets = [[T], [edge - 1, 1, 1, 1, T], [edge, T], [edge + 1, T], [needle, 2, window, 2, T], [first - 1, 1, 1, 2, T],
                [first, T], [first + 1, T], [block_end, 1, 1, T], [block_end + 1, T]]
    if window <= 64:
        cut_sets.append([needle + 1] + [1] * (first - needle + 3) + [T])
    for cuts in cut_sets:
      for kernel in _kernels(H, G, dk, dv, dtype):
        if kernel in ("split3", "split7") and len(cuts) > 20:
            continue
        got = _run_pooled_attention(q, k, v, 1.0, window, pool, dtype, page, cuts, kernel=kernel)
        what = f"{kernel}, window {window}, pool {pool}, cuts {cuts[:4]}"
        for i in range(T):
            if as_token(i) or as_block(i):
                assert float(got[i, :, 0].min()) > 0.05 / pool, f"{what}: key {needle} is lost at {i}"
            else:
                assert float(got[i, :, 0].abs().max()) == 0, f"{what}: key {needle} is seen from {i}"
        _close(got, want, dtype, what, f32=2e-5, bf16=1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_of_score_zero_and_weights_mixed_after_the_softmax(dtype):
    """Two keys whose scores are 0 and s: with the sink the second one's weight is e^s / (2 + e^s), without it
    e^s / (1 + e^s); mixing adds other heads' weights, not their scores, and leaves the sink's share alone."""
    H, G, dk, dv = 3, 1, 16, 16
    k = torch.zeros(2, G, dk, dtype=F64)
    k[1, 0, 0] = 1.0
    v = torch.zeros(2, G, dv, dtype=F64)
    v[1, 0, 0] = 1.0
    q = torch.zeros(2, H, dk, dtype=F64)
    s = torch.tensor([0.5, 4.0, -3.0], dtype=F64)
    q[1, :, 0] = s
    e = torch.exp(s)
    for kernel in _kernels(H, G, dk, dv, dtype):
        for sink in (True, False):
            p = e / ((2.0 if sink else 1.0) + e)
            got = _run_pooled_attention(q, k, v, 1.0, 0, 0, dtype, 8, [2], sink=sink, kernel=kernel)
            _close(got[1, :, 0], p, dtype, f"{kernel}, sink {sink}", scale=1.0, f32=1e-6, bf16=4e-3)
            mix = torch.tensor([[1.0, 0.5, 0.0], [0.0, -1.0, 2.0], [0.25, 0.25, 0.25]], dtype=F64)
            got = _run_pooled_attention(q, k, v, 1.0, 0, 0, dtype, 8, [2], sink=sink, mix=mix, kernel=kernel)
            _close(got[1, :, 0], mix @ p, dtype, f"{kernel}, mixed, sink {sink}", scale=1.0, f32=1e-6, bf16=4e-3)
        # the first token sees itself and the sink only
        got = _run_pooled_attention(q, k, v, 1.0, 5, 2, dtype, 8, [1, 1], kernel=kernel)
        assert float(got[0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_block_among_hundreds(dtype):
    """A block 2,000 tokens back holds the one key that matters: its mean must reach the last token, from a prompt and
    token by token."""
    H, G, dk, dv, page, T, window, pool = 2, 1, 16, 8, 16, 2300, 64, 8
    g = torch.Generator().manual_seed(8)
    k = torch.randn(T, G, dk, generator=g) * 0.05
    v = torch.randn(T, G, dv, generator=g) * 0.05
    q = torch.randn(T, H, dk, generator=g) * 0.05
    k[:, :, 0] = 0.0
    v[:, :, 0] = 0.0
    q[:, :, 0] = 3.0
    k[203, :, 0], v[203, :, 0] = 4.0 * pool, 1.0
    q, k, v = _rounded(q, dtype), _rounded(k, dtype), _rounded(v, dtype)
    want = _plain_weights(q, k, v, 1.0, window, pool)
    for cuts in ([T], [T - 40] + [1] * 40, [700, 3, 900, T]):
        for kernel in _kernels(H, G, dk, dv, dtype):
            got = _run_pooled_attention(q, k, v, 1.0, window, pool, dtype, page, cuts, kernel=kernel)
            assert float(got[-1, :, 0].min()) > 0.5 / pool
            _close(got[-60:], want[-60:], dtype, f"{kernel}, cuts {cuts[:3]}", f32=2e-5, bf16=1e-2)


TC_CASES = [  # H, G, dk, dv, window, pool, page, T, talk
    (4, 2, 16, 32, 24, 4, 16, 200, True), (8, 2, 64, 48, 120, 24, 16, 333, True), (6, 3, 80, 48, 90, 7, 16, 300, True),
    (4, 1, 128, 128, 0, 0, 16, 270, False), (2, 2, 256, 16, 65, 64, 8, 200, True), (3, 1, 48, 112, 1, 1, 16, 150, True),
    (5, 5, 32, 80, 200, 0, 64, 520, False), (16, 4, 128, 128, 100, 32, 16, 600, True), (16, 8, 32, 32, 17, 16, 16, 210, True),
]


@pytest.mark.parametrize("case", TC_CASES)
def test_tensor_core_attention_against_plain_weights(case):
    """The tensor-core kernel on sharp random scores: prompts of several tiles, portions that start in the middle of a
    tile of keys or of a block, and single tokens."""
    from atom_b200 import native
    H, G, dk, dv, window, pool, page, T, talk = case
    assert native.pooled_attention_tc_supports(H, G, dk, dv, torch.bfloat16)
    g = torch.Generator().manual_seed(T + dk)
    q = _rounded(torch.randn(T, H, dk, generator=g), "bfloat16")
    k = _rounded(torch.randn(T, G, dk, generator=g), "bfloat16")
    v = _rounded(torch.randn(T, G, dv, generator=g), "bfloat16")
    mix = _rounded(torch.eye(H) * 0.7 + torch.randn(H, H, generator=g) * 0.3, "bfloat16") if talk else None
    scale = 3.0 / dk ** 0.5
    want = _plain_weights(q, k, v, scale, window, pool, mix=mix)
    for cuts in ([T], [T - 9] + [1] * 9, [13, 64, 5, 2, 129, 2, 70, 3, 17] * 8):
        got = _run_pooled_attention(q, k, v, scale, window, pool, "bfloat16", page, cuts, mix=mix, kernel="tc")
        _close(got, want, "bfloat16", f"cuts {cuts[:3]}", bf16=1e-2)


# ============================================================================= whole models

LENGTHS = {"A": [150, 9, 1, 83, 47, 2], "B": [120, 30, 3, 71, 1, 58], "C": [131, 64, 5, 90, 17, 33], "D": [300, 130, 2, 77]}
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for name, cfg in tk.CONFIGS.items():
        d = str(tmp_path_factory.mktemp(f"kibotar_{name}"))
        tk.write_model(cfg, d, tk.SEEDS[name])
        out[name] = d
    return out


_plain_memo = {}


def _plain_logits(model_dir, seqs):
    if model_dir not in _plain_memo:
        _plain_memo[model_dir] = tk.read_model(model_dir) + ({},)
    cfg, w, memo = _plain_memo[model_dir]
    out = {}
    for rid, toks in seqs.items():
        key = tuple(toks)
        if key not in memo:
            memo[key] = plain.forward(cfg, w, list(toks)).numpy()
        out[rid] = memo[key]
    return out


def _seqs(name):
    ps = tk.prompts(tk.CONFIGS[name], LENGTHS[name], seed=len(name) + ord(name))
    return {f"r{i}": p for i, p in enumerate(ps)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_layer_by_layer_against_plain(dirs, name, dtype):
    """The residual stream after every layer run of a short prompt (a layer of the span that runs several times counts
    each time), from two portions."""
    from atom_b200.engine.batch import StepEntry
    from atom_b200.parts.linear import resolve
    cfg, w = tk.read_model(dirs[name])
    p = tk.prompts(tk.CONFIGS[name], [45], seed=2)[0]
    want = plain.forward(cfg, w, p, return_layers=True)[1]
    runner = _runner(dirs[name], dtype, 64, tk.PAGE[name])
    seen = []
    for b in runner.model.blocks:
        def run(residual, delta, step, cache, wc, _o=b.run):
            out = _o(residual, delta, step, cache, wc)
            seen.append(residual.double() + resolve(out).double())
            return out
        b.run = run
    runner.step([StepEntry("a", p[:31], [0])])
    first = [s.cpu() for s in seen]
    seen.clear()
    runner.step([StepEntry("a", p[31:], [0])])
    runner.check_status()
    assert len(seen) == len(want) == len(plain.run_order(cfg))
    for i, (g0, g1, r) in enumerate(zip(first, seen, want)):
        _close(torch.cat([g0, g1.cpu()]), r, dtype, f"after layer run {i}", f32=3e-5, bf16=3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tk.CONFIGS))
def test_every_cut_matches_plain(dirs, name, dtype):
    """Whole; the last 48 tokens one by one (every window of these models passes over decoded tokens); portions of
    changing size down to two tokens; pairs of tokens throughout; up to four live requests with portions beside single
    tokens in a pool so small that pages and state slots are used again."""
    seqs = _seqs(name)
    ref = _plain_logits(dirs[name], seqs)
    budget = 512 if name == "D" else 320
    mixed, peak = traces.mixed(seqs, max_live=4, budget_tokens=budget)
    assert peak <= budget < sum(-(-len(t) // 64) * 64 for t in seqs.values())
    runner = _runner(dirs[name], dtype, budget, tk.PAGE[name], max_num_seqs=4)
    for what, steps in (("whole", traces.whole(seqs)), ("tail", traces.tail_by_token(seqs, 48)),
                        ("ragged", traces.ragged(seqs)), ("pairs", traces.ragged(seqs, sizes=(2,))), ("mixed", mixed)):
        if what == "pairs":
            steps = [s for s in steps if s["entries"][0]["id"] in ("r1", "r3")]       # (two requests are enough)
            sub = {r: ref[r] for r in ("r1", "r3")}
            _compare(traces.collect(steps, _replay(runner, steps)), sub, dtype, f"{name}/{what}")
            continue
        _compare(traces.collect(steps, _replay(runner, steps)), ref, dtype, f"{name}/{what}")
        assert all(g.pool.num_used == 0 for g in runner.cache.groups) and runner.cache.state_slots.num_free == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_request_freed_half_way_and_fed_again(dirs, name, dtype):
    """What preemption by recomputation does: pages and the state slot go back, another request takes them, and the
    victim starts over on whatever slot is free, with a state, a shifted row and a previous token of zeros."""
    seqs = _seqs(name)
    ref = _plain_logits(dirs[name], seqs)
    ids = list(seqs)
    steps, peak = traces.mixed_refeed(seqs, [ids[0], ids[3]], max_live=3, budget_tokens=384)
    runner = _runner(dirs[name], dtype, peak, tk.PAGE[name], max_num_seqs=3)
    rows = traces.collect_rows(steps, _replay(runner, steps))
    scale = max(float(np.abs(r).max()) for r in ref.values())
    tol = TOL[dtype] * max(1.0, scale)
    for rid, got in rows.items():
        assert {p for p, _ in got} == set(range(len(seqs[rid])))
        errs = [float(np.abs(row.astype(np.float64) - ref[rid][p]).max()) for p, row in got]
        assert max(errs) <= tol, f"{name}/{dtype}: {rid}: worst {max(errs):.3e} > {tol:.3e}"
    assert all(g.pool.num_used == 0 for g in runner.cache.groups) and runner.cache.state_slots.num_free == 3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_of_unequal_requests_equals_each_alone(dirs, dtype):
    """The same rows, computed alone and beside three other requests of other lengths, differ by rounding at most."""
    name = "D"
    ps = tk.prompts(tk.CONFIGS[name], [50, 3, 27, 64], seed=99)
    runner = _runner(dirs[name], dtype, 1024, tk.PAGE[name])
    from atom_b200.engine.batch import StepEntry
    alone = []
    for i, p in enumerate(ps):
        alone.append(runner.step([StepEntry(("a", i), p, list(range(len(p))))]).float().cpu().numpy())
        runner.finish(("a", i))
    both = runner.step([StepEntry(("b", i), p, list(range(len(p)))) for i, p in enumerate(ps)]).float().cpu().numpy()
    at = 0
    for i, p in enumerate(ps):
        part = both[at:at + len(p)]
        at += len(p)
        scale = float(np.abs(alone[i]).max())
        assert np.abs(part - alone[i]).max() <= (1e-4 if dtype == "float32" else 4e-2) * scale
    runner.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_token_by_token(dirs, name, dtype):
    """300 tokens decoded one by one after a prompt of three: pages fill, follow one another and are given back as
    the windows pass while the pooled rows' pages stay; the recurrent state, the shifted row and the previous token are
    read and written 300 times."""
    p = tk.prompts(tk.CONFIGS[name], [303], seed=4)[0]
    seqs = {"long": p}
    ref = _plain_logits(dirs[name], seqs)
    steps = traces.tail_by_token(seqs, 300)
    runner = _runner(dirs[name], dtype, 320, tk.PAGE[name])
    _compare(traces.collect(steps, _replay(runner, steps)), ref, dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_steps_match_plain(dirs, dtype):
    """Decode steps and small mixed steps replayed from CUDA graphs, with padding rows and padding requests."""
    name = "A"
    seqs = _seqs(name)
    ref = _plain_logits(dirs[name], seqs)
    runner = _runner(dirs[name], dtype, 1024, tk.PAGE[name], max_num_seqs=8, enforce_eager=False,
                     cudagraph_capture_sizes=[1, 2, 4], max_model_len=256)
    for what, steps in (("tail", traces.tail_by_token(seqs, 32)), ("mixed", traces.mixed(seqs, max_live=3, tail=40)[0]),
                        ("ragged", traces.ragged(seqs))):
        _compare(traces.collect(steps, _replay(runner, steps)), ref, dtype, f"graphs/{what}")
    assert runner.graph_replays > 50
    assert all(g.pool.num_used == 0 for g in runner.cache.groups)


def _plain_greedy(cfg, w, prompt, n_new):
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(plain.forward(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.parametrize("name,chunk", [("A", 8), ("C", 13)])
def test_greedy_generation_through_the_engine_fp32(dirs, name, chunk):
    from atom_b200 import LLMEngine, SamplingParams
    cfg, w = tk.read_model(dirs[name])
    prompts = tk.prompts(tk.CONFIGS[name], [1, 7, 16, 33], seed=21)
    eng = LLMEngine(dirs[name], dtype="float32", kv_cache_block_size=tk.PAGE[name], num_kvcache_blocks=64,
                    enforce_eager=(name == "C"), max_num_batched_tokens=chunk + 4, long_prefill_token_threshold=chunk,
                    max_num_seqs=4)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o["num_tokens_output"] == 10
        assert o["token_ids"] == _plain_greedy(cfg, w, p, 10)
    assert all(g.pool.num_used == 0 for g in eng.runner.cache.groups)


def test_greedy_generation_bf16_with_preemption(dirs):
    """A pool so small that requests are preempted and computed again; every token stays within rounding of the
    plain implementation's best."""
    from atom_b200 import LLMEngine, SamplingParams
    name = "B"          # (its latent layers keep every row, so pages do run out)
    cfg, w = tk.read_model(dirs[name])
    prompts = tk.prompts(tk.CONFIGS[name], [3, 5, 12, 29], seed=5)
    eng = LLMEngine(dirs[name], dtype="bfloat16", kv_cache_block_size=8, num_kvcache_blocks=14, max_num_batched_tokens=24,
                    max_num_seqs=4, enforce_eager=True)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))
    assert eng.stats()["preemptions"] > 0
    for p, o in zip(prompts, outs):
        full = list(p) + o["token_ids"]
        logits = plain.forward(cfg, w, full[:-1]).numpy()
        for i, tok in enumerate(o["token_ids"]):
            row = logits[len(p) - 1 + i]
            assert row[tok] >= row.max() - 0.03 * np.abs(logits).max(), f"token {i}: logit {row[tok]:.3f} against {row.max():.3f}"
    eng.runner.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program_on_a_kibotar_folder(dirs, tmp_path, dtype):
    """bin/trace_run as a user runs it (a child process, steps on standard input, one file of logits per step): the
    model class is chosen by config.json; four state slots and a pool smaller than the requests' sum."""
    import json
    import os
    import subprocess
    import sys

    name = "A"
    seqs = _seqs(name)
    steps, peak = traces.mixed(seqs, max_live=4, budget_tokens=320)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / f"out_{dtype}"
    text = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", dirs[name], "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(peak)], input=text, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(l.split()[1]) for l in p.stdout.splitlines() if l.startswith("done ")] == [s["step"] for s in steps]
    V = tk.CONFIGS[name]["vocab"]
    outputs = {}
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        if n:
            a = np.fromfile(out / f"{s['step']}.f32", dtype="<f4")
            assert a.size == n * V
            outputs[s["step"]] = a.reshape(n, V)
    _compare(traces.collect(steps, outputs), _plain_logits(dirs[name], seqs), dtype, f"trace_run/{dtype}")
