"""Simivik on the GPU against the plain implementation (tests/plain_simivik.py): every mechanism's part alone through
the cache manager (requests of unequal lengths side by side, whole, in portions down to two tokens and token by token,
on pages and state slots that held other requests before), single keys made to stand out at every edge of the mask,
then whole models under every way of cutting the work, long decoding, captured steps, and greedy generation through
the engine's entry point."""
import math

import numpy as np
import pytest
import torch

import plain_simivik as plain
import tiny_simivik as ts
import traces

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64


def _dt(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def _close(got, want, dtype, what, scale=None, f32=2e-5, bf16=2e-2):
    got, want = got.detach().double().cpu(), want.double()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} against {tuple(want.shape)}"
    scale = float(want.abs().max()) if scale is None else scale
    tol = (f32 if dtype == "float32" else bf16) * max(scale, 1e-3)
    err = float((got - want).abs().max())
    assert math.isfinite(err) and err <= tol, f"{what}: max abs error {err:.3e} > {tol:.3e}"


def _rounded(t, dtype):
    """The values as a kernel gets them (inputs are stored in the activation type)."""
    return t.to(_dt(dtype)).double()


def _i32(x):
    return torch.as_tensor(x, dtype=torch.int32, device=DEV)


def _rt(dtype):
    from atom_b200.parts.base import Runtime, Workspace
    return Runtime(_dt(dtype), torch.device(DEV), Workspace(torch.device(DEV)))


def _bind(part, tensors, rt):
    """Gives the part its tensors (matrices in the compute type, vectors as a checkpoint stores them) and returns
    what it holds, widened, under the names of a model folder's tensors."""
    dev = {}
    for k, v in tensors.items():
        spec = part.params()[k]
        dt = rt.dtype if spec.role == "matrix" else (torch.float32 if rt.dtype == torch.float32 else torch.bfloat16)
        dev[k] = v.to(dt).to(DEV).contiguous()
    held = {k: v.double().cpu() for k, v in dev.items()}
    part.bind(dev, rt)
    part.after_load()
    return held


class Harness:
    """A cache manager, its storage and a step builder around one mixer; feeds requests' rows by a schedule."""

    def __init__(self, part, dtype, page=8, pages=96, max_requests=4):
        from atom_b200.cache import CacheManager
        from atom_b200.cache.storage import CacheStorage
        from atom_b200.engine.batch import StepBuilder

        self.part, self.dtype = part, _dt(dtype)
        self.manager = CacheManager({0: part.cache_need()}, page, pages, max_requests)
        self.storage = CacheStorage(self.manager, self.dtype, torch.device(DEV))
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.builder = StepBuilder(self.manager, DEV, 1 << 30, self.status)

    def run(self, x, schedule, keep=()):
        """x: request -> rows [n, width]; schedule: list of {request: number of new rows}.  Returns request -> the
        mixer's output rows.  A request is released after its last row unless named in ``keep``."""
        from atom_b200.engine.batch import StepEntry

        done = {r: 0 for r in x}
        outs = {r: [] for r in x}
        for portions in schedule:
            entries, targets = [], []
            for rid, n in portions.items():
                if rid not in self.manager.requests:
                    self.manager.admit(rid)
                t = done[rid] + n
                self.manager.extend(rid, t)
                entries.append(StepEntry(rid, [0] * n, ()))
                targets.append(t)
            ctx = self.builder.build(entries, targets)
            xs = torch.cat([x[r][done[r]:done[r] + n] for r, n in portions.items()]).to(self.dtype).to(DEV)
            y = self.part.forward(xs, ctx, self.storage.view(0), True).double().cpu()
            assert int(self.status.item()) == 0
            o = 0
            for (rid, n), t in zip(portions.items(), targets):
                self.manager.commit(rid, t)
                outs[rid].append(y[o:o + n])
                done[rid] = t
                o += n
                if t == x[rid].shape[0] and rid not in keep:
                    self.manager.release(rid)
            self.manager.check()
        assert all(done[r] == x[r].shape[0] for r in x)
        return {r: torch.cat(v) for r, v in outs.items()}


def _schedules(lens):
    """Ways of cutting the same requests: all whole in one batch; most of each whole and the last 9 rows one by one,
    all requests side by side; portions of changing size down to two rows, requests entering one step after another."""
    ids = list(lens)
    yield "whole", [dict(lens)]
    tail = {r: min(9, n - 1) for r, n in lens.items()}
    sched = [{r: n - tail[r] for r, n in lens.items()}]
    for i in range(max(tail.values())):
        sched.append({r: 1 for r in ids if i < tail[r]})
    yield "tail", sched
    sizes = (13, 5, 2, 29, 2, 8, 3, 17, 64, 2)
    left, sched, k = dict(lens), [], 0
    while any(left.values()):
        step = {}
        for j, r in enumerate(ids):
            if left[r] and len(sched) >= j:
                n = min(sizes[k % len(sizes)], left[r])
                k += 1
                step[r] = n
                left[r] -= n
        sched.append(step)
    yield "ragged", sched
    yield "pairs", [{r: min(2, n - 2 * i) for r, n in lens.items() if n > 2 * i} for i in range((max(lens.values()) + 1) // 2)]


def _junk_first(h, width, n=21):
    """A request that fills pages and a state slot with other numbers and goes away before the real ones come."""
    g = torch.Generator().manual_seed(99)
    h.run({"junk": torch.randn(n, width, generator=g) * 3}, [{"junk": n}])


# ============================================================================= attention behind a convolution

ATT_CASES = [  # H, G, dk, dv, taps, (base, dims), (window, keep), cap, page, lens
    (4, 2, 16, 24, 3, (10000.0, 8), (24, 5), 5.0, 16, (70, 9, 41)),
    (2, 1, 24, 16, None, (500.0, 24), None, None, 8, (50, 3, 27)),
    (3, 3, 8, 40, 2, (77.0, 4), (7, 0), 30.0, 8, (40, 17, 2)),
    (5, 5, 20, 12, 1, (1000.0, 12), (1, 1), 8.0, 16, (33, 5, 20)),
    (6, 1, 12, 28, 8, None, (33, 40), 1.5, 16, (90, 48, 7)),
    (8, 2, 64, 64, 4, (100000.0, 32), (128, 16), 30.0, 32, (300, 40, 131)),
    (4, 4, 32, 128, 3, (10000.0, 32), (64, 4), None, 16, (150, 70, 4)),
    (8, 4, 128, 128, 4, (1000000.0, 128), (50, 3), 20.0, 16, (140, 60, 10)),
    (2, 2, 80, 48, 5, (10000.0, 40), (17, 16), 4.0, 8, (64, 65, 63)),
    (2, 2, 32, 16, None, (10000.0, 32), (20, 2), None, 8, (40, 9, 3)),
    (4, 1, 16, 8, 1, None, None, 2.0, 8, (30, 2, 11)),
    (2, 1, 48, 24, 8, (300.0, 16), (9, 1), 6.0, 16, (70, 20, 5)),
    (3, 3, 24, 40, 7, (5000.0, 16), (40, 0), None, 16, (50, 33, 6)),
]


def _attention_part(case, dtype, width=72, seed=0):
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    H, G, dk, dv, taps, rot, mask, cap, page, lens = case
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "scale": 1.7 / dk ** 0.5}
    position = None
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
        position = PartSpec("rope_yarn", {"rotary_dim": rot[1], "theta": rot[0], "scaling": None})
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if cap is not None:
        m["softcap"] = cap
    if taps is not None:
        m["conv"] = taps
    part = registry.build("mixer", PartSpec("conv_window_attention", dict(
        hidden_size=width, num_heads=H, num_kv_heads=G, key_dim=dk, value_dim=dv, scale=m["scale"], softcap=cap, taps=taps,
        position=position, window=mask[0] if mask else None, keep_first=mask[1] if mask else 0)))
    g = torch.Generator().manual_seed(seed + H * dk + dv)
    sharp = 2.2
    q, k, v = (torch.randn(n, width, generator=g) * s / width ** 0.5 for n, s in ((H * dk, sharp), (G * dk, sharp), (G * dv, 1.0)))
    t = {"qkv.weight": torch.cat([q, k, v]), "o.weight": torch.randn(width, H * dv, generator=g) / (H * dv) ** 0.5}
    if taps is not None:
        cw = torch.randn((H + G) * dk + G * dv, taps, generator=g) * (0.5 / taps ** 0.5)
        cw[:, -1] += 0.8
        t["conv.weight"] = cw
    held = _bind(part, t, _rt(dtype))
    nq, nk = H * dk, G * dk
    P = {"q": held["qkv.weight"][:nq], "k": held["qkv.weight"][nq:nq + nk], "v": held["qkv.weight"][nq + nk:], "o": held["o.weight"]}
    if taps is not None:
        c = held["conv.weight"]
        P.update({"q.conv": c[:nq], "k.conv": c[nq:nq + nk], "v.conv": c[nq + nk:]})
    return part, m, P, width


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "bfloat16-plain"])
@pytest.mark.parametrize("case", ATT_CASES)
def test_attention_part_under_every_cut(case, dtype, monkeypatch):
    """(bfloat16 runs the tensor-core kernel where it takes the sizes; "bfloat16-plain" the plain kernel there too.)"""
    from atom_b200 import native
    if dtype.endswith("-plain"):
        if not native.window_attention_tc_supports(case[2], case[3], torch.bfloat16):
            pytest.skip("these sizes run the plain kernel anyway")
        monkeypatch.setattr(native, "WINDOW_TC", False)
        dtype = "bfloat16"
    part, m, P, W = _attention_part(case, dtype)
    page, lens = case[8], dict(zip("abc", case[9]))
    g = torch.Generator().manual_seed(sum(case[9]))
    x = {r: _rounded(torch.randn(n, W, generator=g), dtype) for r, n in lens.items()}
    want = {r: plain.capped_attention(x[r], P, m) for r in lens}
    for what, sched in _schedules(lens):
        h = Harness(part, dtype, page=page, pages=3 * (max(lens.values()) // page + 3))
        _junk_first(h, W)
        got = h.run(x, sched)
        for r in lens:
            _close(got[r], want[r], dtype, f"{what}, request {r}", f32=3e-5, bf16=3e-2)
        assert all(gr.pool.num_used == 0 for gr in h.manager.groups) and h.manager.state_slots.num_free == 4


def _win_pages(T, G, page, dk, dv, dtype, seed=0, extra=5):
    g = torch.Generator().manual_seed(seed)
    n_pages = -(-T // page)
    order = torch.randperm(n_pages + extra, generator=g)[:n_pages]
    table = order.to(torch.int32).view(1, -1).to(DEV)
    kp = torch.full((n_pages + extra, G, page, dk), float("nan"), dtype=_dt(dtype), device=DEV)
    vp = torch.full((n_pages + extra, G, page, dv), float("nan"), dtype=_dt(dtype), device=DEV)
    return table, kp, vp


def _kernels(dk, dv, dtype):
    """The kernels that take these sizes: the plain one always; the tensor-core one where it does, alone on a tile's
    keys and with the keys shared out among three and among seven CTAs."""
    from atom_b200 import native
    return ["plain", "tc1", "tc3", "tc7"] if native.window_attention_tc_supports(dk, dv, _dt(dtype)) else ["plain"]


def _run_window_attention(q, k, v, scale, cap, window, keep, dtype, page, cuts, kernel="plain"):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] of ONE request, keys and values laid into scrambled pages; the queries
    are run in portions ``cuts`` (the keys of later portions are not in the pages yet)."""
    from atom_b200 import native

    T, H, dk = q.shape
    G, dv = k.shape[1], v.shape[2]
    dt = _dt(dtype)
    table, kp, vp = _win_pages(T, G, page, dk, dv, dtype, seed=T)
    out = torch.zeros(T, H * dv, dtype=dt, device=DEV)
    at = 0
    for n in cuts:
        n = min(n, T - at)
        if n <= 0:
            continue
        j = torch.arange(at, at + n, device=DEV)
        pg = table[0].long()[j // page]
        kp[pg, :, j % page] = k[at:at + n].to(dt).to(DEV)
        vp[pg, :, j % page] = v[at:at + n].to(dt).to(DEV)
        o = torch.zeros(n, H * dv, dtype=dt, device=DEV)
        qd = q[at:at + n].reshape(n, H * dk).to(dt).to(DEV).contiguous()
        if kernel.startswith("tc"):
            ns = int(kernel[2:])
            scratch = torch.full((native.attention_mixed_scratch_elems(n, H, dv, ns),), float("nan"), dtype=torch.float32,
                                 device=DEV) if ns > 1 else None
            # (a step of one token also runs the form whose rows are the query heads of a key head)
            native.window_attention_tc(o, qd, kp, vp, table, _i32(range(at, at + n)), _i32([0] * n), _i32([0, n]), 1, H, G,
                                       dk, dv, scale, cap, window, keep, ns, scratch, heads_rows=(n == 1 and at % 2 == 0))
        else:
            native.window_attention(o, qd, kp, vp, table, _i32(range(at, at + n)), _i32([0] * n), H, G, dk, dv, scale,
                                    cap, window, keep)
        out[at:at + n] = o
        at += n
    assert at == T
    return out.double().cpu().view(T, H, dv)


def _plain_scores(q, k, v, scale, cap, window, keep):
    T, H, _ = q.shape
    per = H // k.shape[1]
    kk, vv = k.repeat_interleave(per, dim=1), v.repeat_interleave(per, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    s = s.masked_fill(~plain.visible(T, window or None, keep)[None], -math.inf)
    return torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), vv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window,keep", [(1, 0), (2, 1), (16, 3), (17, 16), (40, 17), (64, 1), (300, 33)])
def test_single_keys_at_the_windows_edge_and_among_the_kept_tokens(window, keep, dtype):
    """Three key rows carry a mark each that only they have, and a score far above all others: one in the middle of the
    request (seen at distance window - 1, not at distance window), the last kept token (seen from everywhere after it)
    and the first token that is not kept (seen only while the window reaches it).  In a prompt, across portions that end
    at every place around the edges and a page's border, and decoded one by one."""
    H, G, dk, dv, page, T = 4, 2, 32, 16, 16, 420
    needle = 177
    marks = {0: needle, 2: keep}            # value column -> the key's position
    if keep:
        marks[1] = keep - 1
    g = torch.Generator().manual_seed(window)
    k = torch.randn(T, G, dk, generator=g) * 0.1
    v = torch.randn(T, G, dv, generator=g) * 0.1
    q = torch.randn(T, H, dk, generator=g) * 0.1
    v[:, :, :3] = 0.0
    k[:, :, :3] = 0.0
    q[:, :, :3] = 3.0
    for col, pos in marks.items():
        v[pos, :, col] = 1.0
        k[pos, :, col] = 4.0               # a score of 12 against a few tenths
    q, k, v = _rounded(q, dtype), _rounded(k, dtype), _rounded(v, dtype)
    want = _plain_scores(q, k, v, 1.0, 0.0, window, keep)
    sees = lambda i, j: j <= i and (i - j < window or j < keep)
    for col, pos in marks.items():
        assert all((want[i, :, col].min() > 0.25) == sees(i, pos) for i in range(T))
        assert all(float(want[i, :, col].abs().max()) == 0 for i in range(T) if not sees(i, pos))
    edge = needle + window
    cut_sets = [[T], [edge - 1, 1, 1, 1, T], [edge, T], [edge + 1, T], [needle, 2, window, 2, T], [keep + window - 1, 1, 1, 2, T],
                [max(keep, 1), T]]
    if window <= 64:
        cut_sets.append([needle + 1] + [1] * (T - needle - 1))
        cut_sets.append([1] * (keep + window + 3) + [T])
    for cuts in cut_sets:
        for kernel in _kernels(dk, dv, dtype):
            if kernel in ("tc3", "tc7") and len(cuts) > 20:
                continue
            got = _run_window_attention(q, k, v, 1.0, 0.0, window, keep, dtype, page, cuts, kernel)
            what = f"{kernel}, window {window}, kept {keep}, cuts {cuts[:4]}"
            for col, pos in marks.items():
                for i in range(T):
                    if sees(i, pos):
                        assert float(got[i, :, col].min()) > 0.25, f"{what}: key {pos} is lost at {i}"
                    else:
                        assert float(got[i, :, col].abs().max()) == 0, f"{what}: key {pos} is seen from {i}"
            _close(got, want, dtype, what, f32=2e-5, bf16=1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scores_are_capped_before_the_softmax(dtype):
    """Two keys whose scores are 0 and s: the second one's weight is 1 / (1 + exp(-cap tanh(s / cap))), which stops
    growing with s; without a cap it is the logistic function of s."""
    H, G, dk, dv = 3, 1, 16, 8
    k = torch.zeros(2, G, dk, dtype=F64)
    k[1, 0, 0] = 1.0
    v = torch.zeros(2, G, dv, dtype=F64)
    v[1, 0, 0] = 1.0
    q = torch.zeros(2, H, dk, dtype=F64)
    q[1, :, 0] = torch.tensor([0.5, 4.0, 64.0], dtype=F64)
    for cap, scale in ((2.0, 1.0), (0.0, 0.25), (7.5, 0.5)):
        s = q[1, :, 0] * scale
        want = torch.sigmoid(cap * torch.tanh(s / cap) if cap else s)
        for kernel in _kernels(dk, dv, dtype):
            got = _run_window_attention(q, k, v, scale, cap, 0, 0, dtype, 8, [2], kernel)
            _close(got[1, :, 0], want, dtype, f"{kernel}, cap {cap}", scale=1.0, f32=1e-6, bf16=4e-3)
            assert cap == 0 or float(got[1, 2, 0]) < 1 / (1 + math.exp(-cap)) + 1e-3


TC_CASES = [  # H, G, dk, dv, window, keep, cap, page, T
    (4, 2, 16, 32, 24, 5, 5.0, 16, 200), (8, 2, 64, 64, 128, 16, 30.0, 32, 333), (6, 3, 80, 48, 90, 70, 40.0, 16, 300),
    (4, 1, 128, 128, 0, 0, 0.0, 16, 270), (2, 2, 256, 16, 65, 64, 3.0, 8, 200), (3, 1, 48, 112, 1, 1, 0.0, 16, 150),
    (5, 5, 32, 80, 200, 130, 10.0, 64, 520), (16, 4, 128, 128, 100, 3, 20.0, 16, 600),
]


@pytest.mark.parametrize("case", TC_CASES)
def test_tensor_core_attention_against_plain_scores(case):
    """The tensor-core kernel on sharp random scores: prompts of several tiles, portions that start in the middle of a
    tile of keys, single tokens, and the keys shared out among CTAs (also more CTAs than there are key tiles)."""
    H, G, dk, dv, window, keep, cap, page, T = case
    g = torch.Generator().manual_seed(T + dk)
    q = _rounded(torch.randn(T, H, dk, generator=g), "bfloat16")
    k = _rounded(torch.randn(T, G, dk, generator=g), "bfloat16")
    v = _rounded(torch.randn(T, G, dv, generator=g), "bfloat16")
    scale = 3.0 / dk ** 0.5
    want = _plain_scores(q, k, v, scale, cap, window, keep)
    kernels = _kernels(dk, dv, "bfloat16")
    assert "tc1" in kernels
    for kernel in kernels:
        for cuts in ([T], [T - 9] + [1] * 9, [13, 64, 5, 2, 129, 2, 70, 3, 17] * 8):
            got = _run_window_attention(q, k, v, scale, cap, window, keep, "bfloat16", page, cuts, kernel)
            _close(got, want, "bfloat16", f"{kernel}, cuts {cuts[:3]}", bf16=1e-2)


# ============================================================================= lightning attention

LIGHT_CASES = [  # H, dk, dv, decay, lens
    (2, 16, 24, (0.9, 0.995), (70, 9, 41)),
    (3, 8, 40, (0.5, 0.97, 0.9999), (37, 5, 18)),
    (1, 12, 20, (1.0,), (50, 2, 31)),
    (5, 4, 4, (0.3, 0.8, 0.95, 0.99, 0.999), (33, 64, 65)),
    (4, 64, 32, (0.8, 0.95, 0.99, 0.999), (300, 40, 131)),
    (2, 128, 128, (0.99, 0.9), (130, 3, 70)),
    (3, 32, 96, (0.999, 0.5, 0.97), (5000, 7, 200)),
]


def _lightning_part(case, dtype, width=72):
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    H, dk, dv, decay, lens = case
    eps = 1e-5
    part = registry.build("mixer", PartSpec("lightning_attention", dict(
        hidden_size=width, num_heads=H, key_dim=dk, value_dim=dv, decay=decay, norm_eps=eps)))
    g = torch.Generator().manual_seed(H * dk + dv)
    mats = [torch.randn(n, width, generator=g) * 1.5 / width ** 0.5 for n in (H * dk, H * dk, H * dv, H * dv)]
    held = _bind(part, {"qkvg.weight": torch.cat(mats), "norm": torch.rand(H * dv, generator=g) * 0.6 + 0.7,
                        "o.weight": torch.randn(width, H * dv, generator=g) / (H * dv) ** 0.5}, _rt(dtype))
    a, b = H * dk, 2 * H * dk
    w = held["qkvg.weight"]
    P = {"q": w[:a], "k": w[a:b], "v": w[b:b + H * dv], "g": w[b + H * dv:], "norm": held["norm"], "o": held["o.weight"]}
    # the decays as the kernel holds them
    m = {"heads": H, "dim": dk, "vdim": dv, "decay": [float(torch.tensor(d, dtype=torch.float32)) for d in decay]}
    return part, m, P, eps, width


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", LIGHT_CASES)
def test_lightning_part_under_every_cut(case, dtype):
    """The state goes from step to step in the request's slot, whatever the cut; steps of many rows take the form that
    sums runs of rows up side by side, and give the same numbers."""
    part, m, P, eps, W = _lightning_part(case, dtype)
    lens = dict(zip("abc", case[4]))
    g = torch.Generator().manual_seed(sum(case[4]))
    x = {r: _rounded(torch.randn(n, W, generator=g), dtype) for r, n in lens.items()}
    want = {r: plain.lightning(x[r], P, m, eps) for r in lens}
    for what, sched in _schedules(lens):
        if what == "pairs" and max(lens.values()) > 1000:
            continue
        h = Harness(part, dtype)
        _junk_first(h, W)
        got = h.run(x, sched)
        for r in lens:
            _close(got[r], want[r], dtype, f"{what}, request {r}", f32=5e-5, bf16=3e-2)
        assert h.manager.state_slots.num_free == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lightning_state_after_six_hundred_single_steps(dtype):
    """One key and value at step 2, then the same query for 600 steps of one token: the output falls as decay^n, in
    32-bit whatever the activations' type (a state kept in 16 bits would stop falling, or fall to zero at once)."""
    from atom_b200 import native

    H, dk, dv, n = 3, 16, 8, 600
    dt = _dt(dtype)
    decay = torch.tensor([0.999, 0.97, 1.0], dtype=torch.float32)
    state = torch.full((2, H, dk, dv), 7.0, dtype=torch.float32, device=DEV)
    state[1].zero_()                                                     # (the request's slot, zeroed at admission)
    z = 3.0
    silu = z / (1 + math.exp(-z))
    outs = []
    for t in range(n):
        proj = torch.full((1, 2 * H * dk + H * dv), -30.0, dtype=dt, device=DEV)      # silu(-30) = 0
        proj[:, :H * dk] = z                                                             # the query
        if t == 2:
            proj[:, H * dk:] = z                                                         # key and value
        o = torch.empty(1, H * dv, dtype=torch.float32, device=DEV)
        native.lightning_scan(o, proj, decay.to(DEV), state, None, _i32([0, 1]), _i32([1]), 1, H, dk, dv, True)
        outs.append(o[0].double().cpu().view(H, dv))
    assert float(outs[1].abs().max()) < 1e-9
    want = decay.double() ** (n - 3) * dk * silu ** 3
    assert 0.5 < float(want[0]) < float(want[2]) and float(want[1]) < 1e-5
    _close(outs[-1][:, 0], want, "float32", "after 600 steps", f32=2e-4)
    assert bool((state[0] == 7.0).all())                                  # another request's slot is left alone


# ============================================================================= feed-forwards and the norm


def _plain_experts(x, P, E, top, score, renormalize, weight_on, shared, shared_gate):
    z = x @ P["router"].T
    s = torch.sigmoid(z) if score == "sigmoid" else torch.softmax(z, -1)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        chosen = torch.topk(s[t], top).indices.tolist()
        w = s[t, chosen]
        if renormalize:
            w = w / w.sum()
        for e, we in zip(chosen, w):
            if weight_on == "input":
                out[t] += plain.gated_expert((we * x[t])[None], P, f"e{e}.")[0]
            else:
                out[t] += we * plain.gated_expert(x[t][None], P, f"e{e}.")[0]
    if shared:
        sh = plain.gated_expert(x, P, "shared.")
        out = out + (torch.sigmoid(x @ P["shared.sg"].T) * sh if shared_gate else sh)
    return out


EXPERT_CASES = [  # width, E, top, ff, shared, score, renormalize, weight_on, shared_gate, T
    (64, 6, 2, 32, 48, "sigmoid", False, "input", True, 45),
    (96, 5, 3, 40, None, "sigmoid", False, "input", False, 33),
    (100, 3, 3, 28, 36, "sigmoid", False, "input", True, 7),
    (256, 8, 2, 128, 256, "sigmoid", False, "input", True, 300),
    (72, 12, 1, 20, 24, "sigmoid", False, "input", True, 1),
    (72, 40, 4, 24, None, "softmax", True, "output", False, 130),
    (80, 7, 2, 52, 16, "softmax", False, "output", False, 50),
    (128, 16, 5, 64, None, "sigmoid", True, "input", False, 2),
    (192, 4, 2, 200, 72, "sigmoid", False, "input", True, 700),
    (136, 3, 1, 48, None, "sigmoid", False, "input", False, 260),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "bfloat16-plain"])
@pytest.mark.parametrize("case", EXPERT_CASES)
def test_routed_experts_part(case, dtype, monkeypatch):
    """Scores, choice, weights on the way in (or out), the shared expert and its gate; rows of one step go to experts
    in any numbers, some experts get none.  (bfloat16 runs the experts' products on the tensor cores where the sizes
    are multiples of 8, "bfloat16-plain" on plain FMAs there too.)"""
    from atom_b200 import native
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    W, E, top, ff, shared, score, renorm, weight_on, sgate, T = case
    if dtype.endswith("-plain"):
        monkeypatch.setattr(native, "MOE_TC", False)
        dtype = "bfloat16"
    part = registry.build("ffn", PartSpec("routed_experts", dict(
        hidden_size=W, num_experts=E, top=top, intermediate_size=ff, shared_size=shared, score=score, renormalize=renorm,
        weight_on=weight_on, shared_gate=sgate)))
    g = torch.Generator().manual_seed(W + E)
    mat = lambda o, i, gain=1.0: torch.randn(o, i, generator=g) * gain / i ** 0.5
    router = mat(E, W, 2.0)
    t = {"router.weight": torch.cat([router, mat(1, W, 2.0)]) if sgate else router,
         "gate_up.weight": torch.cat([mat(ff, W, 1.5) for _ in range(2 * E)]),
         "down.weight": torch.cat([mat(W, ff, 1.5) for _ in range(E)])}
    if shared:
        t["shared.gate_up.weight"] = torch.cat([mat(shared, W, 1.5), mat(shared, W)])
        t["shared.down.weight"] = mat(W, shared, 1.5)
    held = _bind(part, t, _rt(dtype))
    P = {"router": held["router.weight"][:E]}
    if sgate:
        P["shared.sg"] = held["router.weight"][E:]
    for e in range(E):
        P[f"e{e}.gate"] = held["gate_up.weight"][2 * e * ff:(2 * e + 1) * ff]
        P[f"e{e}.up"] = held["gate_up.weight"][(2 * e + 1) * ff:(2 * e + 2) * ff]
        P[f"e{e}.down"] = held["down.weight"][e * W:(e + 1) * W]
    if shared:
        P["shared.gate"], P["shared.up"] = held["shared.gate_up.weight"][:shared], held["shared.gate_up.weight"][shared:]
        P["shared.down"] = held["shared.down.weight"]
    x = _rounded(torch.randn(T, W, generator=g), dtype)
    if T > 40:
        x[5:25] = x[5]                        # twenty rows with the same choice: an expert with many rows
    want = _plain_experts(x, P, E, top, score, renorm, weight_on, shared, sgate)
    if score == "sigmoid" and not renorm and weight_on == "input" and (sgate or not shared):
        mlp = {"router": {"experts": E, "top": top}, "shared": {"ff": shared} if shared else None}
        assert torch.allclose(plain.routed_experts(x, P, mlp), want, rtol=1e-12, atol=1e-12)
    from types import SimpleNamespace
    step = SimpleNamespace(seq_of_token=_i32([0] * T), num_tokens=T, num_seqs=1)
    for _ in range(2):                        # twice: what the first call leaves in the workspace does not leak
        got = part.forward(x.to(_dt(dtype)).to(DEV), step)
        _close(got, want, dtype, "routed experts", f32=3e-5, bf16=3e-2)


def test_router_choice_kernel():
    """The chosen experts are the largest scores, each once, with their scores as weights; the counts add up."""
    from atom_b200 import native

    g = torch.Generator().manual_seed(5)
    for E, top, T in ((12, 1, 40), (6, 2, 9), (64, 8, 300), (5, 5, 3), (200, 32, 17)):
        logits = torch.randn(T, E + 3, generator=g) * 2
        ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
        wts = torch.empty(T, top, dtype=torch.float32, device=DEV)
        counts = torch.zeros(1024, dtype=torch.int32, device=DEV)
        native.moe_route(logits.to(DEV), E, top, "sigmoid", False, _i32([0] * T), ids, wts, counts)
        s = torch.sigmoid(logits[:, :E].double())
        ref = torch.topk(s, top).indices
        assert torch.equal(ids.cpu().long().sort(-1).values, ref.sort(-1).values)
        _close(wts, torch.gather(s, 1, ids.cpu().long()), "float32", "weights", f32=1e-6)
        assert torch.equal(counts[:E].cpu().long(), torch.bincount(ref.flatten(), minlength=E))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [3, 70])
def test_dense_relu_squared_part_and_norm_around_zero(dtype, T):
    from atom_b200.parts import registry
    from atom_b200.parts.spec import PartSpec

    W, ff, eps = 104, 76, 3e-5
    rt = _rt(dtype)
    g = torch.Generator().manual_seed(T)
    ffn = registry.build("ffn", PartSpec("dense_relu2", {"hidden_size": W, "intermediate_size": ff}))
    held = _bind(ffn, {"up.weight": torch.randn(ff, W, generator=g) / W ** 0.5, "down.weight": torch.randn(W, ff, generator=g) / ff ** 0.5}, rt)
    x = _rounded(torch.randn(T, W, generator=g), dtype)
    got = ffn.forward(x.to(_dt(dtype)).to(DEV), None)
    _close(got, plain.dense_relu2(x, {"up": held["up.weight"], "down": held["down.weight"]}), dtype, "relu squared")

    norm = registry.build("norm", PartSpec("rmsnorm", {"size": W, "eps": eps, "weight_offset": 1.0}))
    w = torch.rand(W, generator=g) * 0.6 - 0.3
    stored = _bind(norm, {"weight": w}, rt)["weight"]
    res = torch.randn(T, W, generator=g)
    delta = _rounded(torch.randn(T, W, generator=g), dtype)
    rd = res.to(DEV).contiguous()
    out = norm.add_norm(rd, delta.to(_dt(dtype)).to(DEV), "t")
    r = res.double() + delta
    _close(rd, r, "float32", "residual", f32=1e-6)
    _close(out, plain.rms_norm(r, stored, eps, around_zero=True), dtype, "norm with 1 + w")


# ============================================================================= whole models

LENGTHS = {"A": [1, 2, 9, 41, 100, 70], "B": [3, 17, 64, 131, 30], "C": [5, 33, 90, 48, 70], "D": [4, 70, 150, 33]}
TOL = {"float32": 2e-4, "bfloat16": 8e-2}
RMS_TOL_BF16 = 1.5e-2


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for name, cfg in ts.CONFIGS.items():
        d = str(tmp_path_factory.mktemp(f"simivik_{name}"))
        ts.write_model(cfg, d, ts.SEEDS[name])
        out[name] = d
    return out


_plain_memo = {}


def _plain_logits(model_dir, seqs):
    if model_dir not in _plain_memo:
        _plain_memo[model_dir] = ts.read_model(model_dir) + ({},)
    cfg, w, memo = _plain_memo[model_dir]
    out = {}
    for rid, toks in seqs.items():
        key = tuple(toks)
        if key not in memo:
            memo[key] = plain.forward(cfg, w, list(toks)).numpy()
        out[rid] = memo[key]
    return out


def _runner(model_dir, dtype, max_tokens, page, max_num_seqs=4, **kw):
    from atom_b200.config import EngineConfig
    from atom_b200.engine.runner import ModelRunner

    kw.setdefault("enforce_eager", True)
    return ModelRunner(EngineConfig(model=model_dir, dtype=dtype, kv_cache_block_size=page,
                                    num_kvcache_blocks=max(1, -(-max_tokens // page)), max_num_seqs=max_num_seqs, **kw))


def _replay(runner, steps):
    from atom_b200.engine.batch import StepEntry

    out = {}
    for s in steps:
        logits = runner.step([StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in s["entries"]])
        runner.check_status()
        if logits.shape[0]:
            out[s["step"]] = logits.float().cpu().numpy()
        for rid in s.get("end", []):
            runner.finish(rid)
        runner.cache.check()
    return out


def _compare(got, ref, dtype, what):
    scale = max(float(np.abs(r).max()) for r in ref.values())
    tol = TOL[dtype] * max(1.0, scale)
    for rid, r in ref.items():
        g = got[rid]
        assert g.shape == r.shape and np.isfinite(g).all(), f"{what}: {rid}"
        e = np.abs(g.astype(np.float64) - r).max(axis=1)
        assert e.max() <= tol, f"{what}: {rid}[{int(e.argmax())}] off by {e.max():.3e} > {tol:.3e}"
        if dtype == "bfloat16":
            rms = float(np.sqrt(((g - r) ** 2).mean()))
            assert rms <= RMS_TOL_BF16 * scale, f"{what}: rms error {rms:.3e} in {rid}"
        else:
            assert (g.argmax(1) == r.argmax(1)).all(), f"{what}: greedy token differs in {rid}"


def _seqs(name):
    ps = ts.prompts(ts.CONFIGS[name], LENGTHS[name], seed=len(name) + ord(name))
    return {f"r{i}": p for i, p in enumerate(ps)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_layer_by_layer_against_plain(dirs, name, dtype):
    """The residual stream after every layer of a short prompt (what the next norm reads); a layer that runs another's
    tensors counts on its own."""
    from atom_b200.engine.batch import StepEntry
    cfg, w = ts.read_model(dirs[name])
    p = ts.prompts(ts.CONFIGS[name], [45], seed=2)[0]
    want = plain.forward(cfg, w, p, return_layers=True)[1]
    runner = _runner(dirs[name], dtype, 64, ts.PAGE[name])
    seen = []
    for b in runner.model.blocks:
        def run(residual, delta, step, cache, wc, delta_scale=None, _o=b.run, _b=b):
            out = _o(residual, delta, step, cache, wc, delta_scale=delta_scale)
            seen.append(residual.double() + _b.delta_scale * out.double())
            return out
        b.run = run
    runner.step([StepEntry("a", p, [0])])
    runner.check_status()
    assert len(seen) == len(want) == len(cfg["layers"])
    for i, (g, r) in enumerate(zip(seen, want)):
        _close(g, r, dtype, f"after layer {i}", f32=2e-5, bf16=2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ts.CONFIGS))
def test_every_cut_matches_plain(dirs, name, dtype):
    """Whole; the last 48 tokens one by one (every window of these models passes over decoded tokens); portions of
    changing size down to two tokens; pairs of tokens throughout; up to four live requests with portions beside single
    tokens in a pool so small that pages and state slots are used again."""
    seqs = _seqs(name)
    ref = _plain_logits(dirs[name], seqs)
    mixed, peak = traces.mixed(seqs, max_live=4, budget_tokens=320)
    assert peak <= 320 < sum(-(-len(t) // 64) * 64 for t in seqs.values())
    runner = _runner(dirs[name], dtype, 320, ts.PAGE[name], max_num_seqs=4)
    for what, steps in (("whole", traces.whole(seqs)), ("tail", traces.tail_by_token(seqs, 48)),
                        ("ragged", traces.ragged(seqs)), ("pairs", traces.ragged(seqs, sizes=(2,))), ("mixed", mixed)):
        if what == "pairs":
            steps = [s for s in steps if s["entries"][0]["id"] in ("r1", "r2")]       # (two short requests are enough)
            sub = {r: ref[r] for r in ("r1", "r2")}
            _compare(traces.collect(steps, _replay(runner, steps)), sub, dtype, f"{name}/{what}")
            continue
        _compare(traces.collect(steps, _replay(runner, steps)), ref, dtype, f"{name}/{what}")
        assert all(g.pool.num_used == 0 for g in runner.cache.groups) and runner.cache.state_slots.num_free == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_request_freed_half_way_and_fed_again(dirs, name, dtype):
    """What preemption by recomputation does: pages and the state slot go back, another request takes them, and the
    victim starts over on whatever slot is free, with a state and a convolution tail of zeros."""
    seqs = _seqs(name)
    ref = _plain_logits(dirs[name], seqs)
    ids = list(seqs)
    steps, peak = traces.mixed_refeed(seqs, [ids[-1], ids[-2]], max_live=3, budget_tokens=384)
    runner = _runner(dirs[name], dtype, peak, ts.PAGE[name], max_num_seqs=3)
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
    ps = ts.prompts(ts.CONFIGS[name], [50, 3, 27, 64], seed=99)
    runner = _runner(dirs[name], dtype, 1024, ts.PAGE[name])
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
    the windows pass while the pages of the kept first tokens stay; the lightning state and the convolution's tail are
    read and written 300 times."""
    p = ts.prompts(ts.CONFIGS[name], [303], seed=4)[0]
    seqs = {"long": p}
    ref = _plain_logits(dirs[name], seqs)
    steps = traces.tail_by_token(seqs, 300)
    runner = _runner(dirs[name], dtype, 128, ts.PAGE[name])          # (a pool that only the windows' and kept pages fit into)
    _compare(traces.collect(steps, _replay(runner, steps)), ref, dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_steps_match_plain(dirs, dtype):
    """Decode steps and small mixed steps replayed from CUDA graphs, with padding rows and padding requests."""
    name = "B"
    seqs = _seqs(name)
    ref = _plain_logits(dirs[name], seqs)
    runner = _runner(dirs[name], dtype, 1024, ts.PAGE[name], max_num_seqs=8, enforce_eager=False,
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
    cfg, w = ts.read_model(dirs[name])
    prompts = ts.prompts(ts.CONFIGS[name], [1, 7, 16, 33], seed=21)
    eng = LLMEngine(dirs[name], dtype="float32", kv_cache_block_size=ts.PAGE[name], num_kvcache_blocks=64,
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
    name = "B"          # (its second layer keeps every row, so pages do run out)
    cfg, w = ts.read_model(dirs[name])
    prompts = ts.prompts(ts.CONFIGS[name], [3, 5, 12, 29], seed=5)
    eng = LLMEngine(dirs[name], dtype="bfloat16", kv_cache_block_size=8, num_kvcache_blocks=14, max_num_batched_tokens=24,
                    max_num_seqs=4, enforce_eager=True)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))
    assert eng.stats()["preemptions"] > 0
    for p, o in zip(prompts, outs):
        full = list(p) + o["token_ids"]
        logits = plain.forward(cfg, w, full[:-1]).numpy()
        for i, tok in enumerate(o["token_ids"]):
            row = logits[len(p) - 1 + i]
            assert row[tok] >= row.max() - 0.02 * np.abs(logits).max(), f"token {i}: logit {row[tok]:.3f} against {row.max():.3f}"
    eng.runner.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program_on_a_simivik_folder(dirs, tmp_path, dtype):
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
    V = ts.CONFIGS[name]["vocab"]
    outputs = {}
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        if n:
            a = np.fromfile(out / f"{s['step']}.f32", dtype="<f4")
            assert a.size == n * V
            outputs[s["step"]] = a.reshape(n, V)
    _compare(traces.collect(steps, outputs), _plain_logits(dirs[name], seqs), dtype, f"trace_run/{dtype}")
