"""Prefill and decode throughput of the Nurinex, Mugulorn, Simivik and Kibotar designs beside Qwen3 dense at equal sizes.

    python -m atom_b200.benchmarks.designs [--sizes 1024x8,2048x16] [--layers 4] [--prefill 2048]
                                           [--batch 8] [--context 2048] [--kernels] [--only qwen3,kibotar]

For each size (width x attention heads; head size 128, four query heads to a kv head, feed-forward three
times the width, vocabulary 32768) two engines are built with random bfloat16 weights and the same number
of layers: Qwen3 dense, and Nurinex whose attention has the same heads and whose recurrence has width / 64
heads of 64 channels; and Mugulorn, whose layers alternate attention through a latent (the same heads,
128 + 64 numbers per head, values of 128, a latent of width / 4, queries through width / 2, a window of 1024;
every second attention layer reads the cache of the one before) with a gated linear recurrence of the width's
channels in as many blocks as heads behind a convolution of 4 taps; and Simivik, whose layers are attention behind
a convolution of 4 taps (the same heads, all 128 numbers rotated, scores capped at 30, a window of 1024 that keeps the
first 64 tokens) with a dense relu-squared feed-forward, lightning attention (the same heads, 128 numbers per key and
value) with 16 experts of the width's size of which 2 are used beside a shared one (three times the width per token,
as the dense ones), attention with the dense feed-forward, attention with the experts, and so on; and Kibotar, whose
layers (norms before and after every sub-block, a token shift before every mixer, dense relu-squared feed-forwards) are
attention through a latent of width / 4 (the same heads, 128 numbers per key and value, a gate per head), attention
over a window of 1024 and pooled blocks of 64 (the same heads, all 128 numbers rotated with stretched frequencies, a
sink, mixed weights, an output gate, biases), which runs twice in a row, and gated linear attention (the same heads,
128 numbers per key and value, a decay of rank 64), so that as many layers run as the other designs have.  Measured on the device with CUDA events: one prompt of ``--prefill`` tokens through
one step, and decode steps of ``--batch`` requests whose caches hold ``--context`` tokens (captured graphs,
as the engine runs them).  With ``--kernels`` the kernels of one prefill step and of one decode step are
listed with their summed device time (the engine's profiler hook), which is what the per-kernel rooflines
in the design notes are computed from.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import re
import statistics
from typing import Dict, List

import numpy as np
import torch

VOCAB = 32768
PAGE = 16


def qwen3_config(width: int, heads: int, layers: int) -> dict:
    return {"architectures": ["Qwen3ForCausalLM"], "hidden_size": width, "num_hidden_layers": layers,
            "num_attention_heads": heads, "num_key_value_heads": max(1, heads // 4), "head_dim": 128,
            "intermediate_size": 3 * width, "vocab_size": VOCAB, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
            "max_position_embeddings": 40960, "hidden_act": "silu", "tie_word_embeddings": False,
            "attention_bias": False}


def nurinex_config(width: int, heads: int, layers: int) -> dict:
    left = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
            "bias_max": 4096, "bias_rows": 32, "q_temp": {"coef": 0.5, "every": 64}}
    right = {"heads": width // 64, "dim": 64, "decay_rank": 64}
    layer = {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": {"kind": "dense", "ff": 3 * width}}
    return {"architecture": "Nurinex", "vocab": VOCAB, "width": width, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-5}, "layers": [layer] * layers}


def mugulorn_config(width: int, heads: int, layers: int) -> dict:
    def att(kv_from=None):
        m = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": width // 2, "kv_rank": width // 4,
             "scale": 192 ** -0.5, "mask": {"size": 1024},
             "rot": {"base": 1000000.0, "dims": 64, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return {"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": 3 * width}}

    rec = {"type": "rglru", "mixer": {"width": width, "blocks": heads, "conv": 4}, "mlp": {"kind": "dense", "ff": 3 * width}}
    out, owner = [], None
    for i in range(layers):
        if i % 2:
            out.append(rec)
        elif owner is None:
            out.append(att())
            owner = i
        else:
            out.append(att(kv_from=owner))
            owner = None
    return {"architecture": "Mugulorn", "vocab": VOCAB, "width": width, "residual_mult": 0.5, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-5}, "layers": out}


def simivik_config(width: int, heads: int, layers: int) -> dict:
    att = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 30.0,
           "conv": 4, "rot": {"base": 1000000.0, "dims": 128}, "mask": {"size": 1024, "keep_first": 64}}
    lin = {"heads": heads, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** -(3 + 7 * h / max(1, heads - 1)) for h in range(heads)]}
    dense = {"kind": "dense", "ff": 3 * width}
    moe = {"kind": "moe", "router": {"experts": 16, "top": 2}, "expert": {"ff": width}, "shared": {"ff": width}}
    kinds = [("attention", att, dense), ("lightning", lin, moe), ("attention", att, dense), ("attention", att, moe)]
    return {"architecture": "Simivik", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-5},
            "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in (kinds[i % 4] for i in range(layers))]}


def kibotar_config(width: int, heads: int, layers: int) -> dict:
    dense = {"kind": "dense", "ff": 3 * width}
    lat = {"type": "latent_attention", "mlp": dense,
           "mixer": {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": width // 4, "scale": 128 ** -0.5}}
    att = {"type": "attention", "mlp": dense,
           "mixer": {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                     "rot": {"base": 1000000.0, "dims": 128,
                             "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}},
                     "mask": {"size": 1024, "pool": 64}}}
    gla = {"type": "gla", "mlp": dense, "mixer": {"heads": heads, "dim": 128, "vdim": 128, "tau": 8.0, "rank": 64}}
    kinds = [lat, att, gla]
    unique = max(2, layers - 1)          # the second layer runs twice: ``layers`` layer runs in all
    return {"architecture": "Kibotar", "vocab": VOCAB, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"scale": 1.0, "bigram": {"buckets": 4093, "mul_prev": 257, "mul_cur": 11}},
            "loop": {"start": 1, "stop": 2, "times": 2}, "layers": [kinds[i % 3] for i in range(unique)]}


def _runner(cfg: dict, pages: int, max_len: int, batch: int):
    from atom_b200.config import EngineConfig, config_from_dict
    from atom_b200.engine.runner import ModelRunner

    ecfg = EngineConfig(model="", dtype="bfloat16", load_dummy="random", seed=3, kv_cache_block_size=PAGE,
                        num_kvcache_blocks=pages, max_num_seqs=max(batch, 4), max_num_batched_tokens=8192,
                        max_model_len=max_len, cudagraph_capture_sizes=[batch], cudagraph_mixed_steps=False)
    return ModelRunner(ecfg, config_from_dict(cfg))


def _short(name: str) -> str:
    return re.sub(r"\(.*", "", name).replace("atom::", "").replace("void ", "")[:60]


def _kernels(fn, runner=None) -> Dict[str, float]:
    """Kernel name -> summed device time (us) over one call of fn.  With ``runner`` the call runs eagerly and with
    plain launches: under dependent launch a kernel's time holds its wait for the kernel before it, and a captured
    graph keeps the launches it was recorded with."""
    from torch.profiler import ProfilerActivity, profile

    from atom_b200 import native

    graphs = None
    if runner is not None:
        graphs, runner.graphs_enabled = runner.graphs_enabled, False
        native.set_option("pdl", 0)
        fn()                              # (buffers of the eager path are made outside the listing)
        torch.cuda.synchronize()
    try:
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            fn()
            torch.cuda.synchronize()
    finally:
        if runner is not None:
            runner.graphs_enabled = graphs
            native.set_option("pdl", 1)
    out: Dict[str, float] = {}
    for e in prof.events():
        if e.device_type is not None and str(e.device_type).endswith("CUDA") and e.device_time > 0 and not e.name.startswith("Memcpy"):
            out[_short(e.name)] = out.get(_short(e.name), 0.0) + float(e.device_time)
    return dict(sorted(out.items(), key=lambda kv: -kv[1]))


def measure(cfg: dict, n_prefill: int, batch: int, context: int, kernels: bool) -> dict:
    from atom_b200.engine.batch import StepEntry

    max_len = max(n_prefill, context + 64)
    pages = (batch * (context + 64) + n_prefill) // PAGE + 64
    runner = _runner(cfg, pages, max_len, batch)
    rng = np.random.default_rng(5)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def prefill_once():
        runner.step([StepEntry("p", prompt, (n_prefill - 1,))])

    prompt = rng.integers(0, VOCAB, size=n_prefill).tolist()
    times = []
    for i in range(3 + 5):
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        prefill_once()
        b.record()
        torch.cuda.synchronize()
        runner.finish("p")
        if i >= 3:
            times.append(a.elapsed_time(b))
    out = {"prefill_ms": round(statistics.median(times), 3),
           "prefill_tokens_per_s": round(n_prefill / (statistics.median(times) * 1e-3), 1)}
    if kernels:
        def prefill_and_finish():
            prefill_once()
            runner.finish("p")
        out["prefill_kernels_us"] = {k: round(v, 1) for k, v in _kernels(prefill_and_finish, runner).items()}

    ids = [f"d{i}" for i in range(batch)]
    start = context - 24
    for rid in ids:
        toks = rng.integers(0, VOCAB, size=start).tolist()
        for s in range(0, start, 4096):
            runner.step([StepEntry(rid, toks[s:s + 4096], ())])

    def decode_once():
        runner.step([StepEntry(rid, [int(rng.integers(0, VOCAB))], (0,)) for rid in ids])

    for _ in range(4):
        decode_once()
    torch.cuda.synchronize()
    a, b = ev(), ev()
    a.record()
    K = 16
    for _ in range(K):
        decode_once()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / K
    out.update(decode_ms_per_step=round(ms, 4), decode_tokens_per_s=round(batch / (ms * 1e-3), 1),
               decode_graph=bool(runner.graph_replays))
    if kernels:
        out["decode_kernels_us"] = {k: round(v, 1) for k, v in _kernels(decode_once, runner).items()}
    runner.check_status()
    out["weight_gb"] = round(runner.weight_bytes / 1e9, 3)
    del runner
    torch.cuda.empty_cache()
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--sizes", default="1024x8,2048x16", help="comma-separated width x attention heads")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--prefill", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--kernels", action="store_true", help="list the kernels of one prefill and one decode step")
    ap.add_argument("--only", default="qwen3,nurinex,mugulorn,simivik,kibotar", help="the designs to measure, comma-separated")
    args = ap.parse_args(argv)
    configs = {"qwen3": qwen3_config, "nurinex": nurinex_config, "mugulorn": mugulorn_config, "simivik": simivik_config,
               "kibotar": kibotar_config}
    chosen = [d for d in args.only.split(",") if d]
    if any(d not in configs for d in chosen):
        ap.error(f"--only takes {sorted(configs)}")
    results: List[dict] = []
    for item in args.sizes.split(","):
        width, heads = (int(x) for x in item.lower().split("x"))
        row = {"width": width, "heads": heads, "kv_heads": max(1, heads // 4), "head_dim": 128, "ff": 3 * width,
               "layers": args.layers}
        for d in chosen:
            row[d] = measure(configs[d](width, heads, args.layers), args.prefill, args.batch, args.context, args.kernels)
        results.append(row)
    print(json.dumps({"bench": "designs", "dtype": "bf16", "data": "synthetic", "prefill_tokens": args.prefill,
                      "decode_batch": args.batch, "decode_context": args.context, "vocab": VOCAB, "sizes": results}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
