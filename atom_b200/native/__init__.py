"""ctypes binding of the sm_100a kernel library.

``lib()`` builds the library on first use (see ``build.py``) and loads it; every kernel
wrapper below takes torch tensors, passes raw device pointers and the current stream, and
raises if the kernel refuses its arguments.  There is no fallback: without the library the
product path does not run.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

from .build import NativeBuildError, build, build_variant

F32, BF16 = 0, 1
_ERR = {1: "argument the kernel does not take", 2: "CUDA launch failed", 3: "library call failed"}

_lib = None
_lock = threading.Lock()
launches = 0        # launches of this library's own kernels made by this process
library_gemms = 0   # calls into the vendor GEMM library (counted apart from own kernels)


class NativeError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise NativeError(f"kernels take float32 or bfloat16, not {dt}")


def lib():
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = build()
                try:
                    _lib = ctypes.CDLL(path)
                except OSError as e:  # pragma: no cover
                    raise NativeBuildError(f"cannot load {path}: {e}") from e
                _declare(_lib)
    return _lib


def lib_path() -> str:
    return build(verbose=False)


_vp, _i, _i64, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t

_SIGNATURES = {
    "atom_embedding": [_vp, _vp, _i, _vp, _i, _i, _i, _f, _vp],
    "atom_pair_embedding": [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i64, _i64, _f, _i, _vp],
    "atom_add_row": [_vp, _vp, _i, _i, _i, _vp],
    "atom_normed_add_rmsnorm": [_vp, _i, _vp, _vp, _vp, _f, _vp, _i, _f, _vp, _i, _i, _vp],
    "atom_head_gate": [_vp, _vp, _i, _i64, _i, _i, _i, _vp],
    "atom_gla_supports": [_i, _i],
    "atom_gla_scan": [_vp, _vp, _vp, _vp, _i, _i64, _vp, _i64, _vp, _i, _f, _f, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                      _i, _i, _i, _vp],
    "atom_gla_gate_norm": [_vp, _vp, _vp, _i, _i64, _vp, _i, _i, _i, _i, _f, _vp, _vp],
    "atom_pooled_attention_supports": [_i, _i, _i, _i],
    "atom_pooled_attention_split_supports": [_i, _i, _i, _i],
    "atom_pooled_attention_split": [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i,
                                    _i, _i, _f, _i, _i, _i, _vp, _vp, _i64, _i, _vp],
    "atom_pool_blocks": [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _i64, _i64, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "atom_pooled_attention": [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i,
                              _f, _i, _i, _i, _vp, _vp, _i64, _vp],
    "atom_xielu": [_vp, _vp, _i, _i64, _f, _f, _vp],
    "atom_tanh": [_vp, _i, _i64, _vp],
    "atom_pair_rmsnorm_add": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _f, _i, _i, _vp],
    "atom_token_shift_mix": [_vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "atom_wkv": [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp],
    "atom_kv_write": [_vp, _i, _i64, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _i, _i, _vp, _vp, _i64, _vp, _vp],
    "atom_attention_mixed": [_vp, _vp, _i64, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _f, _i,
                             _vp, _i, _vp, _i, _vp, _vp, _f, _i, _i, _vp, _vp],
    "atom_attention_mixed_merge": [_vp, _i, _vp, _vp, _i, _i, _i, _i, _vp],
    "atom_add_rmsnorm": [_vp, _i, _vp, _vp, _vp, _i, _f, _vp, _i, _i, _f, _vp],
    "atom_latent_prepare": [_vp, _vp, _i, _i64, _i, _i, _vp, _i, _i, _i, _i, _vp, _i, _f, _vp, _f, _vp, _vp, _vp, _i, _i,
                            _vp, _i64, _vp, _i, _vp],
    "atom_rotate_pairs": [_vp, _i64, _i, _i, _vp, _i, _i64, _i, _i, _i, _i, _i, _vp, _f, _vp, _vp, _i, _vp],
    "atom_latent_attention_supports": [_i, _i, _i],
    "atom_latent_attention_head_group": [_i, _i, _i],
    "atom_latent_attention": [_vp, _vp, _vp, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _f, _i, _vp, _i, _vp],
    "atom_latent_attention_tc_supports": [_i, _i, _i],
    "atom_latent_attention_tc": [_vp, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _vp, _vp, _i, _i, _vp],
    "atom_latent_merge": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _vp, _vp],
    "atom_causal_conv": [_vp, _vp, _i, _i64, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "atom_rglru_scan": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i64, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                        _f, _i, _vp],
    "atom_sigmoid_mul": [_vp, _vp, _i, _i64, _i, _i, _vp],
    "atom_gelu_mul": [_vp, _vp, _i, _i, _i, _vp],
    "atom_gemm_f32_batched": [_vp, _vp, _vp, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _vp],
    "atom_gemm_bf16_batched": [_vp, _i, _vp, _vp, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _vp, _sz, _vp],
    "atom_relu2": [_vp, _i, _i64, _vp],
    "atom_conv_rope_write": [_vp, _vp, _i, _i64, _i, _i, _i, _i, _i, _vp, _i, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i,
                             _i, _vp, _vp, _i64, _vp, _vp],
    "atom_conv_state_update": [_vp, _vp, _i, _i64, _i, _i, _vp, _vp, _i, _vp],
    "atom_window_attention_merge": [_vp, _i, _vp, _vp, _i, _i, _i, _i, _vp],
    "atom_window_attention": [_vp, _vp, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _f, _f, _i, _i, _vp],
    "atom_lightning_supports": [_i, _i],
    "atom_lightning_scan": [_vp, _vp, _i, _i64, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "atom_lightning_gate_norm": [_vp, _vp, _vp, _i, _i64, _vp, _i, _i, _i, _f, _vp, _vp],
    "atom_moe_route": [_vp, _i64, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp],
    "atom_moe_place": [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "atom_moe_gemm": [_vp, _vp, _i, _i64, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "atom_moe_combine": [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _i64, _i, _i, _vp, _vp],
    "atom_rmsnorm": [_vp, _vp, _i, _vp, _i, _f, _i, _i, _vp],
    "atom_silu_mul": [_vp, _vp, _i, _i, _i, _vp],
    "atom_qknorm_rope_kvwrite": [_vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _f, _vp, _i, _i, _vp, _vp,
                                 _vp, _i, _i, _vp, _vp, _i64, _vp, _vp],
    "atom_qk_headnorm": [_vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _f, _vp, _vp],
    "atom_paged_attention_generic": [_vp, _vp, _i64, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i,
                                     _i, _i, _f, _i, _vp],
    "atom_gemm_f32": [_vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i64, _vp],
    "atom_gemm_bf16": [_vp, _i, _vp, _vp, _i, _i, _i, _i64, _vp, _sz, _vp],
    "atom_add_bias": [_vp, _i, _vp, _i, _i, _i, _vp],
    "atom_gemm_rows": [_vp, _i, _vp, _vp],
    "atom_gemm_rows_grid": [],
    "atom_gemm_rows_supports": [_i, _i, _i, _i64],
    "atom_gemm_pairs": [_vp, _i64, _vp, _vp, _i64, _i, _i, _i, _i, _vp, _vp],
    "atom_gemm_pairs_resident": [],
    "atom_gemm_pairs_supports": [_i, _i, _i, _i64, _i64],
    "atom_set_option": [_i, _i],
    "atom_copy_rows_h2d": [_vp, _i64, _vp, _i64, _i64, _i64, _vp],
}


def _declare(l) -> None:
    for name, args in _SIGNATURES.items():
        if not hasattr(l, name):
            continue  # optional kernels are declared by the module that owns them
        fn = getattr(l, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int64 if name.endswith("_bytes") else ctypes.c_int


def declare(name: str, args) -> None:
    """Declares the signature of one more exported function (used by kernel modules)."""
    _SIGNATURES[name] = args
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int


# Choices the launch code otherwise makes by itself (csrc/common.cuh, ATOM_OPT_*): for measurements
# and for tests of both sides of a choice.  They hold for launches made after the call; a captured
# graph keeps what it was recorded with.
OPTIONS = {"pdl": 0, "decode_tma": 1, "decode_ktw": 2}
_option_values = {}


def set_option(name: str, value: int) -> None:
    """Sets an option in every loaded library of the package (and in those loaded later)."""
    key = OPTIONS[name]
    _option_values[key] = int(value)
    if lib().atom_set_option(key, int(value)) != 0:
        raise NativeError(f"option {name!r} was refused")
    for l in _flash_libs.values():
        l.atom_flash_set_option(key, int(value))
    for l in _mixtc_libs.values():
        l.atom_mixtc_set_option(key, int(value))
    for l in _pwtc_libs.values():
        l.atom_pwtc_set_option(key, int(value))


def reset_options() -> None:
    for name, default in (("pdl", 1), ("decode_tma", 1), ("decode_ktw", 0)):
        set_option(name, default)
    _option_values.clear()


def copy_rows_h2d(dst: torch.Tensor, dst_pitch: int, src: torch.Tensor, src_pitch: int, row_elems: int,
                  rows: int) -> None:
    """rows x row_elems elements from pinned host memory (rows src_pitch elements apart) to the device
    (rows dst_pitch elements apart), asynchronously on the current stream."""
    es = dst.element_size()
    assert dst.is_cuda and not src.is_cuda and src.element_size() == es     # (src: pinned memory)
    assert rows == 0 or (dst.numel() >= (rows - 1) * dst_pitch + row_elems and src.numel() >= (rows - 1) * src_pitch + row_elems)
    code = lib().atom_copy_rows_h2d(dst.data_ptr(), dst_pitch * es, src.data_ptr(), src_pitch * es, row_elems * es,
                                    rows, _stream())
    if code != 0:
        raise NativeError(f"copy_rows_h2d: {_ERR.get(code, code)}")


def _check(code: int, name: str, own: bool = True) -> None:
    global launches, library_gemms
    if own:
        launches += 1
    else:
        library_gemms += 1
    if code != 0:
        raise NativeError(f"{name}: {_ERR.get(code, f'error {code}')}")


def add_launches(n: int) -> None:
    """Counts kernels that ran without passing through the wrappers (a replayed CUDA graph)."""
    global launches
    launches += n


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of the current CUDA stream of the current device (the raw query is an order of
    magnitude cheaper than building a torch.cuda.Stream object for every launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NativeError("kernels take CUDA tensors only (there is no CPU path)")


# --------------------------------------------------------------------------- wrappers

GATE_ACTS = {"silu": 1, "gelu_tanh": 2}      # the activation on the gate of a gated product (gemm_rows, gemm_pairs)


def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0) -> None:
    """out[t] = table[ids[t]] * scale widened to float32.  out [T,H] f32, table [V,H], ids [T] i32."""
    _cuda(out, table, ids)
    T, H = out.shape
    assert out.dtype == torch.float32 and ids.dtype == torch.int32 and table.shape[1] == H
    assert out.is_contiguous() and table.is_contiguous() and ids.numel() >= T
    _check(lib().atom_embedding(out.data_ptr(), table.data_ptr(), dtype_code(table.dtype),
                                ids.data_ptr(), T, H, table.shape[0], float(scale), _stream()), "embedding")


def add_rmsnorm(out: torch.Tensor, residual: torch.Tensor, delta: Optional[torch.Tensor],
                weight: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None, delta_scale: float = 1.0) -> None:
    """residual (+= delta_scale * delta); out = rmsnorm(residual) * weight.  With ``rows`` (int32 indices)
    only those rows are normalised, written densely to ``out``, and residual is left as is."""
    _cuda(out, residual, delta, weight, rows)
    H = residual.shape[-1]
    assert residual.dtype == torch.float32 and residual.is_contiguous() and out.is_contiguous()
    assert weight.numel() == H and (delta is None or (delta.dtype == out.dtype and delta.is_contiguous()))
    n = (rows.numel() if n_rows is None else n_rows) if rows is not None else residual.shape[0]
    assert out.shape[0] >= n and out.shape[-1] == H
    _check(lib().atom_add_rmsnorm(out.data_ptr(), dtype_code(out.dtype), residual.data_ptr(),
                                  _ptr(delta), weight.data_ptr(), dtype_code(weight.dtype),
                                  float(eps), _ptr(rows), n, H, float(delta_scale), _stream()), "add_rmsnorm")


def rmsnorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    _cuda(out, x, weight)
    H = x.shape[-1]
    assert x.is_contiguous() and out.is_contiguous() and out.dtype == x.dtype and weight.numel() == H
    _check(lib().atom_rmsnorm(out.data_ptr(), x.data_ptr(), dtype_code(x.dtype), weight.data_ptr(),
                              dtype_code(weight.dtype), float(eps), x.numel() // H, H, _stream()),
           "rmsnorm")


def xielu(out: torch.Tensor, x: torch.Tensor, ap: float, aq: float) -> None:
    """out = xIELU(x) elementwise: ap z^2 + z/2 for z > 0, (1/2 + aq)(exp(z) - 1 - z) + z/2 otherwise."""
    _cuda(out, x)
    assert out.shape == x.shape and out.dtype == x.dtype and out.is_contiguous() and x.is_contiguous()
    _check(lib().atom_xielu(out.data_ptr(), x.data_ptr(), dtype_code(x.dtype), x.numel(), float(ap), float(aq),
                            _stream()), "xielu")


def tanh_(x: torch.Tensor) -> None:
    """x = tanh(x) in place."""
    _cuda(x)
    assert x.is_contiguous()
    _check(lib().atom_tanh(x.data_ptr(), dtype_code(x.dtype), x.numel(), _stream()), "tanh")


def pair_rmsnorm_add(residual: torch.Tensor, a: torch.Tensor, wa: Optional[torch.Tensor], b: Optional[torch.Tensor],
                     wb: Optional[torch.Tensor], c: Optional[torch.Tensor], eps: float) -> None:
    """residual += 0.5 * (rmsnorm(a; wa) + rmsnorm(b; wb)) (+ c) in 32-bit; with b None: += rmsnorm(a; wa) (+ c);
    with wa None as well: += a (+ c)."""
    _cuda(residual, a, wa, b, wb, c)
    M, H = a.shape
    assert residual.dtype == torch.float32 and residual.is_contiguous() and residual.shape[0] >= M and residual.shape[1] == H
    assert a.is_contiguous() and (wa is None or wa.numel() == H)
    for t in (b, c):
        assert t is None or (t.shape == a.shape and t.dtype == a.dtype and t.is_contiguous())
    assert (b is None) == (wb is None) and (wb is None or (wa is not None and wb.numel() == H and wb.dtype == wa.dtype))
    _check(lib().atom_pair_rmsnorm_add(residual.data_ptr(), a.data_ptr(), _ptr(wa), _ptr(b), _ptr(wb),
                                       dtype_code(wa.dtype) if wa is not None else F32, _ptr(c), dtype_code(a.dtype),
                                       float(eps), M, H, _stream()), "pair_rmsnorm_add")


def token_shift_mix(out: torch.Tensor, h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor,
                    seq_of_token: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor,
                    write_state: bool = True) -> None:
    """out[m, t] = h[t] + (h[t-1] - h[t]) * mu[m] within each request; a request's first token of the step takes
    h[t-1] from its row of ``state`` [slots, W], which then takes the h of the request's last token."""
    _cuda(out, h, mu, state, seq_of_token, cu_q, state_slots)
    T, W = h.shape
    n = mu.shape[0]
    assert out.shape == (n, T, W) and out.dtype == h.dtype == state.dtype and mu.shape == (n, W)
    assert out.is_contiguous() and h.is_contiguous() and mu.is_contiguous() and state.is_contiguous()
    assert state.shape[1] == W and seq_of_token.dtype == cu_q.dtype == state_slots.dtype == torch.int32
    _check(lib().atom_token_shift_mix(out.data_ptr(), h.data_ptr(), dtype_code(h.dtype), mu.data_ptr(),
                                      dtype_code(mu.dtype), state.data_ptr(), seq_of_token.data_ptr(),
                                      cu_q.data_ptr(), state_slots.data_ptr(), T, W, n, int(write_state),
                                      _stream()), "token_shift_mix")


def wkv_supports(dk: int, dv: int) -> bool:
    return 0 < dk <= 128 and 0 < dv <= 128


def wkv(y: torch.Tensor, r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, d: torch.Tensor, gate: torch.Tensor,
        w0: torch.Tensor, u: torch.Tensor, norm_w: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor,
        state_slots: torch.Tensor, num_seqs: int, heads: int, dk: int, dv: int, eps: float,
        write_state: bool = True) -> None:
    """The decayed linear recurrence with bonus of csrc/wkv.cu over every request's tokens of the step, followed by
    the per-head unit norm, the channel weights and silu(gate).  state: [slots, heads, dk, dv] float32."""
    _cuda(y, r, k, v, d, gate, w0, u, norm_w, state, cu_q, state_slots)
    T = r.shape[0]
    for t_, n_ in ((r, dk), (k, dk), (d, dk), (v, dv), (gate, dv), (y, dv)):
        assert t_.shape == (T, heads * n_) and t_.is_contiguous()
    assert r.dtype == k.dtype == v.dtype == gate.dtype == y.dtype and d.dtype in (r.dtype, torch.float32)
    assert w0.dtype == u.dtype == norm_w.dtype and w0.numel() == u.numel() == heads * dk and norm_w.numel() == heads * dv
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dk, dv)
    _check(lib().atom_wkv(y.data_ptr(), r.data_ptr(), k.data_ptr(), v.data_ptr(), dtype_code(r.dtype), d.data_ptr(),
                          dtype_code(d.dtype), gate.data_ptr(), w0.data_ptr(), u.data_ptr(), norm_w.data_ptr(),
                          dtype_code(w0.dtype), state.data_ptr(), cu_q.data_ptr(), state_slots.data_ptr(), num_seqs,
                          heads, dk, dv, float(eps), int(write_state), _stream()), "wkv")


def kv_write(qkv: torch.Tensor, k_off: int, v_off: int, nkv: int, dk: int, dv: int, vnorm: bool, eps: float,
             positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int,
             k_pages: torch.Tensor, v_pages: torch.Tensor, status: torch.Tensor) -> None:
    """Writes the step's keys (columns k_off...) and values (columns v_off...) of the packed projection to their
    pages; vnorm: every value head is first divided by its root mean square."""
    _cuda(qkv, positions, seq_of_token, block_table, k_pages, v_pages, status)
    assert qkv.stride(1) == 1 and k_pages.dtype == v_pages.dtype == qkv.dtype
    assert tuple(k_pages.shape[1:]) == (nkv, page_size, dk) and tuple(v_pages.shape[1:]) == (nkv, page_size, dv)
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and block_table.dtype == torch.int32
    assert block_table.dim() == 2 and block_table.is_contiguous() and k_pages.shape[0] == v_pages.shape[0]
    _check(lib().atom_kv_write(qkv.data_ptr(), dtype_code(qkv.dtype), qkv.stride(0), k_off, v_off, qkv.shape[0], nkv,
                               dk, dv, int(vnorm), float(eps), positions.data_ptr(), seq_of_token.data_ptr(),
                               block_table.data_ptr(), block_table.shape[1], page_size, k_pages.data_ptr(),
                               v_pages.data_ptr(), k_pages.shape[0], status.data_ptr(), _stream()), "kv_write")


def attention_mixed(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                    block_table: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, nh: int, nkv: int,
                    dk: int, dv: int, scale: float, window: int = 0, rel: Optional[torch.Tensor] = None,
                    half: int = 0, thresholds: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
                    sink: Optional[torch.Tensor] = None, temp_coef: float = 0.0, temp_every: int = 0,
                    nsplit: int = 1, scratch: Optional[torch.Tensor] = None) -> None:
    """Causal paged attention whose heads' scores are mixed before the softmax (csrc/attention_mixed.cu), with a
    bias by distance, a sink per head and a query temperature, each optional.  q: [T, >= nh * dk] (row stride
    taken from the tensor); out: [T, nh * dv]; rel [rows, nh], mix [nh, nh], sink [nh] float32; thresholds int32.
    nsplit > 1: every token's keys are shared out among nsplit blocks (steps of few tokens and long contexts);
    scratch: float32, at least ``attention_mixed_scratch_elems`` elements."""
    _cuda(out, q, k_pages, v_pages, block_table, positions, seq_of_token, rel, thresholds, mix, sink)
    T = out.shape[0]
    page_size = k_pages.shape[2]
    assert out.is_contiguous() and out.shape[1] == nh * dv and q.stride(1) == 1 and out.dtype == q.dtype == k_pages.dtype
    assert tuple(k_pages.shape[1:]) == (nkv, page_size, dk) and tuple(v_pages.shape[1:]) == (nkv, page_size, dv)
    assert k_pages.is_contiguous() and v_pages.is_contiguous()
    n_thr = 0 if thresholds is None else thresholds.numel()
    for t_ in (rel, mix, sink):
        assert t_ is None or (t_.dtype == torch.float32 and t_.is_contiguous())
    assert rel is None or (rel.shape[1] == nh and rel.shape[0] >= half + n_thr + (1 if n_thr else 0))
    assert thresholds is None or thresholds.dtype == torch.int32
    assert nsplit == 1 or (scratch is not None and scratch.dtype == torch.float32 and scratch.is_cuda
                           and scratch.numel() >= attention_mixed_scratch_elems(T, nh, dv, nsplit))
    _check(lib().atom_attention_mixed(
        out.data_ptr(), q.data_ptr(), q.stride(0), dtype_code(q.dtype), k_pages.data_ptr(), v_pages.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], page_size, positions.data_ptr(), seq_of_token.data_ptr(), T,
        nh, nkv, dk, dv, float(scale), int(window), _ptr(rel), int(half), _ptr(thresholds), n_thr, _ptr(mix),
        _ptr(sink), float(temp_coef), int(temp_every), int(nsplit), _ptr(scratch) if nsplit > 1 else None, _stream()),
        "attention_mixed")
    if nsplit > 1:
        add_launches(1)      # (the kernel that puts the shares together)


SM_COUNT = 148      # B200


def attention_mixed_scratch_elems(T: int, nh: int, dv: int, nsplit: int) -> int:
    return T * nsplit * nh * (dv + 2)


def attention_mixed_splits(units: int, max_ctx_len: int, per_sm: int = 2, min_share: int = 256) -> int:
    """Into how many shares the attention with mixed heads cuts the keys of every unit of work (a token for the
    plain kernel, a tile of 16 tokens for the tensor-core kernel): ``per_sm`` CTAs per SM fill the device (and even
    out the unequal lengths of a prompt's tiles); below that the keys are shared out, in shares of at least
    ``min_share``."""
    if units >= per_sm * SM_COUNT:
        return 1
    return max(1, min(-(-per_sm * SM_COUNT // max(units, 1)), -(-max_ctx_len // min_share), 64))


# ---- the same attention on the tensor cores (csrc/attention_mixed_tc.cu), compiled per (heads, kv heads, key size,
# value size) on first use
_mixtc_libs = {}
_MIXTC_SIG = [_vp, _vp, _i64, _vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _f, _i, _vp, _i, _vp, _i, _vp, _vp, _f, _i, _i,
              _vp, _vp]
MIXED_TC = True      # False: the plain kernel also where the tensor-core kernel takes the sizes (measurements, tests)


def attention_mixed_tc_supports(nh: int, nkv: int, dk: int, dv: int, n_thr: int, mixing: bool, dtype: torch.dtype) -> bool:
    """bfloat16; key and value sizes in steps of 16; at most 16 heads whose output tiles (16 rows x heads x value
    size, 32-bit) fit the registers of a CTA's 16 warps; everything in 227 KB of shared memory."""
    if dtype != torch.bfloat16 or dk % 16 or dv % 16 or nh % nkv or not 1 <= nh <= 16 or n_thr > 256:
        return False
    group = nh // nkv
    if nkv * (-(-(group * (dv // 16)) // 16)) * 8 > 64:
        return False
    smem = 2 * (nh * 16 * (dk + 8) + 2 * 64 * (max(dk, dv) + 8)) + 4 * nh * 16 * 72 + 4 * nh * nh \
        + 4 * (3 * nh * 16 + 16) + 4 * (2 * 64 + 256) + 256
    return smem <= 226 * 1024


def mixtc_lib(nh: int, nkv: int, dk: int, dv: int):
    key = (nh, nkv, dk, dv)
    l = _mixtc_libs.get(key)
    if l is None:
        with _lock:
            l = _mixtc_libs.get(key)
            if l is None:
                path = build_variant("attention_mixed_tc.cu", {"ATOM_MH_NH": nh, "ATOM_MH_NKV": nkv, "ATOM_MH_DK": dk,
                                                               "ATOM_MH_DV": dv})
                l = ctypes.CDLL(path)
                l.atom_attention_mixed_tc.argtypes = _MIXTC_SIG
                l.atom_attention_mixed_tc.restype = ctypes.c_int
                l.atom_mixtc_set_option.argtypes = [_i, _i]
                l.atom_mixtc_set_option.restype = ctypes.c_int
                got = [ctypes.c_int() for _ in range(4)]
                l.atom_mixtc_sizes(*[ctypes.byref(g) for g in got])
                if tuple(g.value for g in got) != key:
                    raise NativeBuildError(f"{path} was built for other sizes")
                for k, v in _option_values.items():
                    l.atom_mixtc_set_option(k, v)
                _mixtc_libs[key] = l
    return l


def attention_mixed_tc(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                       block_table: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                       cu_q: torch.Tensor, num_seqs: int, nh: int, nkv: int, dk: int, dv: int, scale: float,
                       window: int = 0, rel: Optional[torch.Tensor] = None, half: int = 0,
                       thresholds: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
                       sink: Optional[torch.Tensor] = None, temp_coef: float = 0.0, temp_every: int = 0,
                       nsplit: int = 1, scratch: Optional[torch.Tensor] = None) -> None:
    """``attention_mixed`` on the tensor cores: tiles of 16 consecutive tokens of a request (cu_q: [num_seqs + 1]
    first token row of every request).  Sizes as ``attention_mixed_tc_supports`` says."""
    _cuda(out, q, k_pages, v_pages, block_table, positions, seq_of_token, cu_q, rel, thresholds, mix, sink)
    T = out.shape[0]
    page_size = k_pages.shape[2]
    assert out.is_contiguous() and out.shape[1] == nh * dv and q.stride(1) == 1
    assert out.dtype == q.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16
    assert tuple(k_pages.shape[1:]) == (nkv, page_size, dk) and tuple(v_pages.shape[1:]) == (nkv, page_size, dv)
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and cu_q.numel() >= num_seqs + 1
    n_thr = 0 if thresholds is None else thresholds.numel()
    for t_ in (rel, mix, sink):
        assert t_ is None or (t_.dtype == torch.float32 and t_.is_contiguous())
    assert rel is None or (rel.shape[1] == nh and rel.shape[0] >= half + n_thr + (1 if n_thr else 0))
    assert nsplit == 1 or (scratch is not None and scratch.dtype == torch.float32
                           and scratch.numel() >= attention_mixed_scratch_elems(T, nh, dv, nsplit))
    tiles = -(-T // 16) + num_seqs
    _check(mixtc_lib(nh, nkv, dk, dv).atom_attention_mixed_tc(
        out.data_ptr(), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], page_size, positions.data_ptr(), cu_q.data_ptr(), num_seqs, tiles, float(scale),
        int(window), _ptr(rel), int(half), _ptr(thresholds), n_thr, _ptr(mix), _ptr(sink), float(temp_coef),
        int(temp_every), int(nsplit), _ptr(scratch) if nsplit > 1 else None, _stream()), "attention_mixed_tc")
    if nsplit > 1:
        _check(lib().atom_attention_mixed_merge(out.data_ptr(), dtype_code(out.dtype), scratch.data_ptr(),
                                                seq_of_token.data_ptr(), T, nh, dv, nsplit, _stream()),
               "attention_mixed_merge")


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _cuda(out, gate_up)
    T, I2 = gate_up.shape
    assert I2 % 2 == 0 and out.shape == (T, I2 // 2) and out.dtype == gate_up.dtype
    assert out.is_contiguous() and gate_up.is_contiguous()
    _check(lib().atom_silu_mul(out.data_ptr(), gate_up.data_ptr(), dtype_code(out.dtype), T, I2 // 2,
                               _stream()), "silu_mul")


def qknorm_rope_kvwrite(qkv: torch.Tensor, nh: int, nkv: int, hd: int,
                        q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                        eps: float, cos_sin: Optional[torch.Tensor], rotary_dim: int,
                        positions: torch.Tensor, seq_of_token: torch.Tensor,
                        block_table: torch.Tensor, page_size: int,
                        k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                        status: torch.Tensor) -> None:
    """Per-head q/k norm, rotation and cache write for the packed [T, (nh+2nkv)*hd] projection."""
    _cuda(qkv, q_weight, k_weight, cos_sin, positions, seq_of_token, block_table, k_pages, v_pages, status)
    T = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * hd
    assert (q_weight is None) == (k_weight is None)
    wd = dtype_code(q_weight.dtype) if q_weight is not None else F32
    if q_weight is not None:
        assert k_weight.dtype == q_weight.dtype and q_weight.numel() == hd and k_weight.numel() == hd
    if cos_sin is not None:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] == rotary_dim
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    num_pages = 0
    if k_pages is not None:
        assert k_pages.dtype == qkv.dtype and k_pages.is_contiguous() and v_pages.is_contiguous()
        assert tuple(k_pages.shape[1:]) == (nkv, page_size, hd) and v_pages.shape == k_pages.shape
        num_pages = k_pages.shape[0]
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
    assert positions.dtype == torch.int32 and seq_of_token.dtype == torch.int32
    assert status.dtype == torch.int32
    _check(lib().atom_qknorm_rope_kvwrite(
        qkv.data_ptr(), dtype_code(qkv.dtype), T, nh, nkv, hd, _ptr(q_weight), _ptr(k_weight), wd,
        float(eps), _ptr(cos_sin), rotary_dim, max_pos, positions.data_ptr(), seq_of_token.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], page_size, _ptr(k_pages), _ptr(v_pages),
        num_pages, status.data_ptr(), _stream()), "qknorm_rope_kvwrite")


def qk_headnorm(qkv: torch.Tensor, nh: int, nkv: int, hd: int, q_weight: torch.Tensor, k_weight: torch.Tensor,
                eps: float, seq_of_token: torch.Tensor) -> None:
    """Per-head RMSNorm of the q and k heads of the packed [T, (nh+2nkv)*hd] projection, in place."""
    _cuda(qkv, q_weight, k_weight, seq_of_token)
    assert qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * hd
    assert k_weight.dtype == q_weight.dtype and q_weight.numel() == hd and k_weight.numel() == hd
    _check(lib().atom_qk_headnorm(qkv.data_ptr(), dtype_code(qkv.dtype), qkv.shape[0], nh, nkv, hd,
                                  q_weight.data_ptr(), k_weight.data_ptr(), dtype_code(q_weight.dtype), float(eps),
                                  seq_of_token.data_ptr(), _stream()), "qk_headnorm")


def paged_attention_generic(out: torch.Tensor, q: torch.Tensor, q_stride: int,
                            k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                            positions: torch.Tensor, seq_of_token: torch.Tensor, T: int, nh: int,
                            nkv: int, hd: int, scale: float, window: int) -> None:
    """out[T, nh*hd]: causal attention of every token over its request's pages (any sizes)."""
    _cuda(out, q, k_pages, v_pages, block_table, positions, seq_of_token)
    page_size = k_pages.shape[2]
    assert out.is_contiguous() and out.dtype == q.dtype == k_pages.dtype
    assert tuple(k_pages.shape[1:]) == (nkv, page_size, hd) and k_pages.is_contiguous() and v_pages.is_contiguous()
    _check(lib().atom_paged_attention_generic(
        out.data_ptr(), q.data_ptr(), q_stride, dtype_code(q.dtype), k_pages.data_ptr(),
        v_pages.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size,
        positions.data_ptr(), seq_of_token.data_ptr(), T, nh, nkv, hd, float(scale), int(window),
        _stream()), "paged_attention_generic")


def gemm_f32(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T (+ bias) in true 32-bit arithmetic."""
    _cuda(out, a, w, bias)
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == w.dtype == out.dtype == torch.float32 and w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous()
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == N)
    _check(lib().atom_gemm_f32(out.data_ptr(), a.data_ptr(), w.data_ptr(), _ptr(bias), M, N, K,
                               a.stride(0), out.stride(0), _stream()), "gemm_f32")


_workspaces = {}


def _workspace(device: torch.device) -> torch.Tensor:
    """The library's scratch memory: one per device and stream, since products on two streams may run at once."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.empty(32 << 20, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def gemm_bf16(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """out[M,N] (bf16 or f32) = a[M,K] @ w[N,K]^T, bf16 operands, 32-bit accumulation (cuBLAS)."""
    _cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == w.dtype == torch.bfloat16 and w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and out.is_contiguous() and w.is_contiguous()
    ws = _workspace(out.device)
    _check(lib().atom_gemm_bf16(out.data_ptr(), dtype_code(out.dtype), a.data_ptr(), w.data_ptr(), M, N,
                                K, a.stride(0), ws.data_ptr(), ws.numel(), _stream()), "gemm_bf16",
           own=False)


def gemm_batched(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> None:
    """out[:, b, :] = a[:, b, :] @ w[b]^T for every b: a [M, B, K] and out [M, B, N] may be views (rows and
    batches any distance apart, the last axis dense), w [B, N, K] dense.  bfloat16 operands through the GEMM library
    with 32-bit sums (out bfloat16 or float32); float32 on the FMA kernel."""
    _cuda(out, a, w)
    M, B, K = a.shape
    N = w.shape[1]
    assert w.shape == (B, N, K) and out.shape == (M, B, N) and w.is_contiguous() and a.dtype == w.dtype
    assert a.stride(2) == 1 and out.stride(2) == 1
    if a.dtype == torch.float32:
        assert out.dtype == torch.float32
        _check(lib().atom_gemm_f32_batched(out.data_ptr(), a.data_ptr(), w.data_ptr(), B, M, N, K, a.stride(0),
                                           out.stride(0), a.stride(1), N * K, out.stride(1), _stream()), "gemm_f32_batched")
        return
    assert a.dtype == torch.bfloat16
    ws = _workspace(out.device)
    _check(lib().atom_gemm_bf16_batched(out.data_ptr(), dtype_code(out.dtype), a.data_ptr(), w.data_ptr(), B, M, N, K,
                                        a.stride(0), out.stride(0), a.stride(1), N * K, out.stride(1), ws.data_ptr(),
                                        ws.numel(), _stream()), "gemm_bf16_batched", own=False)


def latent_prepare(cq: Optional[torch.Tensor], proj: torch.Tensor, q_off: int, wq: Optional[torch.Tensor], eps: float,
                   positions: torch.Tensor, seq_of_token: torch.Tensor, kv_off: int = 0, kv_rank: int = 0,
                   rot_dim: int = 0, rot_dims: int = 0, wkv: Optional[torch.Tensor] = None,
                   freq: Optional[torch.Tensor] = None, mag: float = 1.0, block_table: Optional[torch.Tensor] = None,
                   page_size: int = 0, pages: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> None:
    """Per token: cq = rmsnorm(proj[:, q_off : q_off + Rq]; wq); with ``pages``, the row [rmsnorm(first kv_rank
    numbers at kv_off; wkv) | the next rot_dim numbers, the first rot_dims of them rotated by position * freq and
    scaled by mag] goes to the token's place in the pages [pages, page size, kv_rank + rot_dim].  cq None: only the
    page row is made (queries that pass no latent of their own)."""
    _cuda(cq, proj, wq, positions, seq_of_token, wkv, freq, block_table, pages, status)
    T, Rq = (cq.shape if cq is not None else (proj.shape[0], 0))
    assert proj.stride(1) == 1
    assert cq is None or (proj.dtype == cq.dtype and cq.is_contiguous() and wq.numel() == Rq)
    if pages is not None:
        assert pages.dtype == proj.dtype and pages.is_contiguous() and tuple(pages.shape[1:]) == (page_size, kv_rank + rot_dim)
        assert wkv.numel() == kv_rank and (wq is None or wkv.dtype == wq.dtype)
        assert rot_dims == 0 or (freq.dtype == torch.float32 and freq.numel() >= rot_dims // 2)
        assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
    _check(lib().atom_latent_prepare(
        _ptr(cq), proj.data_ptr(), dtype_code(proj.dtype), proj.stride(0), q_off, Rq, _ptr(wq), kv_off,
        kv_rank, rot_dim, rot_dims, _ptr(wkv), dtype_code((wq if wq is not None else wkv).dtype), float(eps), _ptr(freq),
        float(mag),
        positions.data_ptr(), seq_of_token.data_ptr(), _ptr(block_table),
        block_table.shape[1] if block_table is not None else 0, page_size, _ptr(pages),
        pages.shape[0] if pages is not None else 0, _ptr(status), T, _stream()), "latent_prepare")


def rotate_pairs(out: torch.Tensor, out_off: int, x: torch.Tensor, x_off: int, length: int, dims: int,
                 freq: torch.Tensor, mag: float, positions: torch.Tensor, seq_of_token: torch.Tensor) -> None:
    """For every token t and vector n: out[t, n, out_off : out_off + length] = x[t, n, x_off : x_off + length] with
    its first ``dims`` numbers rotated (pairs (i, i + dims/2)) by positions[t] * freq[i], times mag.  out is float32."""
    _cuda(out, x, freq, positions, seq_of_token)
    T, n_vec = x.shape[0], x.shape[1]
    assert out.dtype == torch.float32 and out.shape[:2] == x.shape[:2] and out.stride(2) == 1 and x.stride(2) == 1
    assert freq.dtype == torch.float32 and freq.numel() >= dims // 2
    _check(lib().atom_rotate_pairs(out.data_ptr(), out.stride(0), out.stride(1), out_off, x.data_ptr(),
                                   dtype_code(x.dtype), x.stride(0), x.stride(1), x_off, n_vec, length, dims,
                                   freq.data_ptr(), float(mag), positions.data_ptr(), seq_of_token.data_ptr(), T,
                                   _stream()), "rotate_pairs")


def latent_attention_supports(heads: int, kv_rank: int, rot_dim: int) -> bool:
    return bool(lib().atom_latent_attention_supports(heads, kv_rank, rot_dim))


def latent_attention_head_group(heads: int, kv_rank: int, rot_dim: int) -> int:
    """Heads that a CTA of the plain kernel takes together."""
    return max(1, int(lib().atom_latent_attention_head_group(heads, kv_rank, rot_dim)))


def latent_attention_scratch_elems(T: int, heads: int, kv_rank: int, nsplit: int) -> int:
    return T * heads * nsplit * (kv_rank + 2)


def latent_attention(out: torch.Tensor, q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                     positions: torch.Tensor, seq_of_token: torch.Tensor, kv_rank: int, rot_dim: int, scale: float,
                     window: int, sink: Optional[torch.Tensor], nsplit: int = 1,
                     scratch: Optional[torch.Tensor] = None) -> None:
    """out[t, h, :] = sum_j a[t, h, j] * pages[row(j)][:kv_rank], a the softmax over the keys j of the token's
    request with 0 <= pos(t) - j < window (window 0: all) of scale * q[t, h] . pages[row(j)], with exp(sink[h])
    one more term of the denominator.  q [T, heads, kv_rank + rot_dim] float32; pages [pages, page, kv_rank + rot_dim]."""
    _cuda(out, q, pages, block_table, positions, seq_of_token, sink, scratch)
    T, H, Dk = q.shape
    assert q.dtype == torch.float32 and q.is_contiguous() and Dk == kv_rank + rot_dim
    assert out.shape == (T, H, kv_rank) and out.is_contiguous() and out.dtype == pages.dtype
    assert pages.is_contiguous() and pages.shape[2] == Dk and block_table.dtype == torch.int32 and block_table.is_contiguous()
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == H)
    assert nsplit == 1 or (scratch is not None and scratch.dtype == torch.float32
                           and scratch.numel() >= latent_attention_scratch_elems(T, H, kv_rank, nsplit))
    _check(lib().atom_latent_attention(out.data_ptr(), _ptr(scratch), q.data_ptr(), pages.data_ptr(),
                                       dtype_code(pages.dtype), block_table.data_ptr(), block_table.shape[1],
                                       pages.shape[1], positions.data_ptr(), seq_of_token.data_ptr(), T, H, kv_rank,
                                       rot_dim, float(scale), int(window), _ptr(sink), nsplit, _stream()),
           "latent_attention")
    if nsplit > 1:
        global launches
        launches += 1


LATENT_TC = True      # False: the plain kernel also where the tensor-core kernel takes the sizes (measurements, tests)


def latent_attention_tc_supports(heads: int, kv_rank: int, rot_dim: int, dtype: torch.dtype) -> bool:
    return dtype == torch.bfloat16 and bool(lib().atom_latent_attention_tc_supports(heads, kv_rank, rot_dim))


def latent_attention_tc_tile_tokens(heads: int, rows: int = 64) -> int:
    """Consecutive tokens of a request in one tile of the tensor-core kernel (``rows`` = tokens x heads)."""
    return max(1, rows // min(heads, rows))


def latent_attention_tc(out: torch.Tensor, q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor,
                        positions: torch.Tensor, cu_q: torch.Tensor, num_seqs: int, kv_rank: int, rot_dim: int,
                        scale: float, window: int, sink: Optional[torch.Tensor], nsplit: int = 1,
                        scratch: Optional[torch.Tensor] = None, seq_of_token: Optional[torch.Tensor] = None,
                        rows: int = 64) -> None:
    """``latent_attention`` on the tensor cores (bfloat16 pages and output): a CTA is a few consecutive tokens of a
    request with a group of heads (``rows`` = 64 query rows, or 16 for steps of single tokens), found from cu_q on
    the device.  With ``nsplit`` > 1 every CTA walks one share of
    its tokens' keys and the merge kernel puts the shares together (``scratch`` as for the plain kernel;
    ``seq_of_token`` marks padding rows)."""
    _cuda(out, q, pages, block_table, positions, cu_q, sink, scratch, seq_of_token)
    T, H, Dk = q.shape
    assert q.dtype == torch.float32 and q.is_contiguous() and Dk == kv_rank + rot_dim
    assert out.shape == (T, H, kv_rank) and out.is_contiguous() and out.dtype == pages.dtype == torch.bfloat16
    assert pages.is_contiguous() and pages.shape[2] == Dk and block_table.dtype == torch.int32 and block_table.is_contiguous()
    assert sink is None or (sink.dtype == torch.float32 and sink.numel() == H)
    _check(lib().atom_latent_attention_tc(out.data_ptr(), q.data_ptr(), pages.data_ptr(), block_table.data_ptr(),
                                          block_table.shape[1], pages.shape[1], cu_q.data_ptr(), positions.data_ptr(),
                                          num_seqs, T, H, kv_rank, rot_dim, float(scale), int(window), _ptr(sink),
                                          _ptr(scratch), int(nsplit), int(rows), _stream()), "latent_attention_tc")
    if nsplit > 1:
        assert scratch is not None and scratch.dtype == torch.float32 and seq_of_token is not None
        assert scratch.numel() >= latent_attention_scratch_elems(T, H, kv_rank, nsplit)
        _check(lib().atom_latent_merge(out.data_ptr(), scratch.data_ptr(), dtype_code(out.dtype), seq_of_token.data_ptr(),
                                       T, H, kv_rank, int(nsplit), _ptr(sink), _stream()), "latent_merge")


def causal_conv(u: torch.Tensor, x: torch.Tensor, bx: torch.Tensor, w: torch.Tensor, bc: torch.Tensor,
                conv_state: torch.Tensor, seq_of_token: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor) -> None:
    """u[t, c] = bc[c] + sum_k w[c, k] * v[t - taps + 1 + k, c] within each request, v = x + bx; values before the
    step's first token of a request come from its row of conv_state [slots, taps - 1, W] (read only)."""
    _cuda(u, x, bx, w, bc, conv_state, seq_of_token, cu_q, state_slots)
    T, W = u.shape
    taps = w.shape[1]
    assert x.shape == (T, W) and x.stride(1) == 1 and u.is_contiguous() and x.dtype == u.dtype == conv_state.dtype
    assert w.shape == (W, taps) and w.is_contiguous() and bx.numel() == bc.numel() == W and bx.dtype == w.dtype == bc.dtype
    assert conv_state.is_contiguous() and tuple(conv_state.shape[1:]) == (max(taps - 1, 0), W)
    _check(lib().atom_causal_conv(u.data_ptr(), x.data_ptr(), dtype_code(x.dtype), x.stride(0), bx.data_ptr(),
                                  w.data_ptr(), bc.data_ptr(), dtype_code(w.dtype), conv_state.data_ptr(),
                                  seq_of_token.data_ptr(), cu_q.data_ptr(), state_slots.data_ptr(), T, W, taps,
                                  _stream()), "causal_conv")


def rglru_scan(out: torch.Tensor, gates: torch.Tensor, gate_b: torch.Tensor, lam: torch.Tensor, u: torch.Tensor,
               y: torch.Tensor, x: torch.Tensor, by: torch.Tensor, bx: torch.Tensor, state: torch.Tensor,
               conv_state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, num_seqs: int, taps: int,
               decay_c: float, write_state: bool = True) -> None:
    """The gated linear recurrence of csrc/rglru.cu over every request's tokens of the step.  gates [T, blocks, 2 bw]
    float32 (sums of r, then of i, per block), gate_b [blocks, 2 bw]; y, x [T, W] views of the branches before their
    biases; state [slots, W] float32; conv_state [slots, taps - 1, W]."""
    _cuda(out, gates, gate_b, lam, u, y, x, by, bx, state, conv_state, cu_q, state_slots)
    T, W = out.shape
    blocks, bw2 = gates.shape[1], gates.shape[2]
    assert gates.dtype == torch.float32 and gates.is_contiguous() and blocks * bw2 == 2 * W and gate_b.numel() == 2 * W
    assert u.shape == (T, W) and u.is_contiguous() and out.is_contiguous() and y.shape == x.shape == (T, W)
    assert y.stride(1) == x.stride(1) == 1 and y.stride(0) == x.stride(0) and out.dtype == u.dtype == y.dtype == x.dtype
    assert gate_b.dtype == lam.dtype == by.dtype == bx.dtype and gate_b.is_contiguous()
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == W
    assert conv_state.dtype == out.dtype and conv_state.is_contiguous() and tuple(conv_state.shape[1:]) == (taps - 1, W)
    _check(lib().atom_rglru_scan(out.data_ptr(), gates.data_ptr(), gate_b.data_ptr(), lam.data_ptr(), u.data_ptr(),
                                 y.data_ptr(), x.data_ptr(), dtype_code(out.dtype), y.stride(0), by.data_ptr(),
                                 bx.data_ptr(), dtype_code(lam.dtype), state.data_ptr(), conv_state.data_ptr(),
                                 cu_q.data_ptr(), state_slots.data_ptr(), num_seqs, T, W, bw2 // 2, taps, float(decay_c),
                                 int(write_state), _stream()), "rglru_scan")


def sigmoid_mul(x: torch.Tensor, g: torch.Tensor) -> None:
    """x *= sigmoid(g) elementwise; x [T, n] dense, g [T, n] a view whose rows may lie further apart."""
    _cuda(x, g)
    assert x.shape == g.shape and x.dtype == g.dtype and x.is_contiguous() and g.stride(1) == 1
    _check(lib().atom_sigmoid_mul(x.data_ptr(), g.data_ptr(), dtype_code(x.dtype), g.stride(0), x.shape[0], x.shape[1],
                                  _stream()), "sigmoid_mul")


def gelu_mul(out: torch.Tensor, gate_up: torch.Tensor) -> None:
    """out = gelu_tanh(gate_up[:, :I]) * gate_up[:, I:]."""
    _cuda(out, gate_up)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.is_contiguous() and out.is_contiguous() and out.dtype == gate_up.dtype
    _check(lib().atom_gelu_mul(out.data_ptr(), gate_up.data_ptr(), dtype_code(out.dtype), T, I, _stream()), "gelu_mul")


def relu2_(x: torch.Tensor) -> None:
    """x = relu(x)^2 in place."""
    _cuda(x)
    assert x.is_contiguous()
    _check(lib().atom_relu2(x.data_ptr(), dtype_code(x.dtype), x.numel(), _stream()), "relu2")


def conv_rope_write(q_out: torch.Tensor, qkv: torch.Tensor, H: int, G: int, dk: int, dv: int,
                    conv_w: Optional[torch.Tensor], conv_state: Optional[torch.Tensor], freq: Optional[torch.Tensor],
                    rot_dims: int, positions: torch.Tensor, seq_of_token: torch.Tensor, cu_q: torch.Tensor,
                    state_slots: torch.Tensor, block_table: torch.Tensor, page_size: int,
                    k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], status: torch.Tensor) -> None:
    """Per token of the packed projection [q (H dk) | k (G dk) | v (G dv)]: the short causal convolution over time on
    every channel (conv_w [C, taps]; rows before the step from conv_state [slots, taps - 1, C], which is only read),
    rotation of the first rot_dims numbers of every query and key head by position * freq, queries to q_out
    [T, H dk], keys and values to their pages (csrc/window_attention.cu).  conv_w None: no convolution."""
    _cuda(q_out, qkv, conv_w, conv_state, freq, positions, seq_of_token, cu_q, state_slots, block_table, k_pages,
          v_pages, status)
    T = qkv.shape[0]
    C = (H + G) * dk + G * dv
    taps = 0 if conv_w is None else conv_w.shape[1]
    assert qkv.stride(1) == 1 and qkv.shape[1] >= C and q_out.is_contiguous() and q_out.shape == (T, H * dk)
    assert q_out.dtype == qkv.dtype and block_table.dtype == torch.int32 and block_table.is_contiguous()
    assert conv_w is None or (tuple(conv_w.shape) == (C, taps) and conv_w.is_contiguous())
    assert taps <= 1 or (conv_state is not None and conv_state.is_contiguous() and conv_state.dtype == qkv.dtype
                         and tuple(conv_state.shape[1:]) == (taps - 1, C))
    assert rot_dims == 0 or (freq is not None and freq.dtype == torch.float32 and freq.numel() >= rot_dims // 2)
    if k_pages is not None:
        assert tuple(k_pages.shape[1:]) == (G, page_size, dk) and tuple(v_pages.shape[1:]) == (G, page_size, dv)
        assert k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.dtype == v_pages.dtype == qkv.dtype
    _check(lib().atom_conv_rope_write(
        q_out.data_ptr(), qkv.data_ptr(), dtype_code(qkv.dtype), qkv.stride(0), T, H, G, dk, dv, _ptr(conv_w),
        dtype_code(conv_w.dtype) if conv_w is not None else F32, taps, _ptr(conv_state) if taps > 1 else None,
        _ptr(freq), rot_dims, positions.data_ptr(), seq_of_token.data_ptr(), cu_q.data_ptr(), state_slots.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], page_size, _ptr(k_pages), _ptr(v_pages),
        k_pages.shape[0] if k_pages is not None else 0, status.data_ptr(), _stream()), "conv_rope_write")


def conv_state_update(conv_state: torch.Tensor, qkv: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor,
                      num_seqs: int) -> None:
    """conv_state [slots, taps - 1, C] <- every request's last taps - 1 rows of (what it held, then the step's rows)."""
    _cuda(conv_state, qkv, cu_q, state_slots)
    taps, C = conv_state.shape[1] + 1, conv_state.shape[2]
    assert conv_state.is_contiguous() and qkv.stride(1) == 1 and qkv.shape[1] >= C and qkv.dtype == conv_state.dtype
    _check(lib().atom_conv_state_update(conv_state.data_ptr(), qkv.data_ptr(), dtype_code(qkv.dtype), qkv.stride(0), C,
                                        taps, cu_q.data_ptr(), state_slots.data_ptr(), num_seqs, _stream()),
           "conv_state_update")


def window_attention(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     block_table: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, nh: int, nkv: int,
                     dk: int, dv: int, scale: float, softcap: float = 0.0, window: int = 0, keep_first: int = 0) -> None:
    """Causal paged attention, key j seen from position p if j <= p and (p - j < window or j < keep_first); scores
    scale * q.k, then softcap * tanh(score / softcap) if softcap > 0.  q [T, nh dk], out [T, nh dv], any sizes, both
    precisions (csrc/window_attention.cu)."""
    _cuda(out, q, k_pages, v_pages, block_table, positions, seq_of_token)
    T = q.shape[0]
    page_size = k_pages.shape[2]
    assert q.is_contiguous() and out.is_contiguous() and q.shape == (T, nh * dk) and out.shape == (T, nh * dv)
    assert out.dtype == q.dtype == k_pages.dtype == v_pages.dtype and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert tuple(k_pages.shape[1:]) == (nkv, page_size, dk) and tuple(v_pages.shape[1:]) == (nkv, page_size, dv)
    assert block_table.dtype == torch.int32 and block_table.is_contiguous()
    _check(lib().atom_window_attention(
        out.data_ptr(), q.data_ptr(), dtype_code(q.dtype), k_pages.data_ptr(), v_pages.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], page_size, positions.data_ptr(), seq_of_token.data_ptr(), T, nh,
        nkv, dk, dv, float(scale), float(softcap or 0.0), int(window or 0), int(keep_first), _stream()),
        "window_attention")


# ---- the same attention on the tensor cores (csrc/window_attention_tc.cu), compiled per (key size, value size) on
# first use
_watc_libs = {}
_WATC_SIG = [_vp, _vp, _i64, _vp, _vp, _i64, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _i, _i, _i, _vp, _i, _vp]
WINDOW_TC = True     # False: the plain kernel also where the tensor-core kernel takes the sizes (measurements, tests)
WINDOW_TC_ROWS = 64  # query rows of a tile


def window_attention_tc_supports(dk: int, dv: int, dtype: torch.dtype) -> bool:
    """bfloat16; key and value sizes in steps of 16, keys up to 256 and values up to 128 numbers (a warp keeps its
    16 x value size output in registers)."""
    return dtype == torch.bfloat16 and dk % 16 == 0 and dv % 16 == 0 and 16 <= dk <= 256 and 16 <= dv <= 128


def watc_lib(dk: int, dv: int):
    key = (dk, dv)
    l = _watc_libs.get(key)
    if l is None:
        with _lock:
            l = _watc_libs.get(key)
            if l is None:
                path = build_variant("window_attention_tc.cu", {"ATOM_WA_DK": dk, "ATOM_WA_DV": dv})
                l = ctypes.CDLL(path)
                l.atom_window_attention_tc.argtypes = _WATC_SIG
                l.atom_window_attention_tc.restype = ctypes.c_int
                got = [ctypes.c_int() for _ in range(2)]
                l.atom_watc_sizes(*[ctypes.byref(g) for g in got])
                if tuple(g.value for g in got) != key:
                    raise NativeBuildError(f"{path} was built for other sizes")
                _watc_libs[key] = l
    return l


def window_attention_tc(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                        block_table: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                        cu_q: torch.Tensor, num_seqs: int, nh: int, nkv: int, dk: int, dv: int, scale: float,
                        softcap: float = 0.0, window: int = 0, keep_first: int = 0, nsplit: int = 1,
                        scratch: Optional[torch.Tensor] = None, heads_rows: bool = False) -> None:
    """``window_attention`` on the tensor cores: tiles of 64 consecutive tokens of a request and one head (cu_q:
    [num_seqs + 1] first token row of every request); with nsplit > 1 a tile's keys are shared out among nsplit
    CTAs and put together by a merge kernel.  heads_rows (only for steps in which every request brings ONE token, and
    at most 64 query heads to a key head): a CTA's rows are the query heads of one key head for one token, so the
    keys and values are read once per key head.  Sizes as ``window_attention_tc_supports``."""
    _cuda(out, q, k_pages, v_pages, block_table, positions, seq_of_token, cu_q, scratch)
    T = q.shape[0]
    page_size = k_pages.shape[2]
    assert q.stride(1) == 1 and q.shape[1] == nh * dk and out.is_contiguous() and out.shape == (T, nh * dv)
    assert out.dtype == q.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16
    assert tuple(k_pages.shape[1:]) == (nkv, page_size, dk) and tuple(v_pages.shape[1:]) == (nkv, page_size, dv)
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and cu_q.numel() >= num_seqs + 1
    assert block_table.dtype == torch.int32 and block_table.is_contiguous()
    assert nsplit == 1 or (scratch is not None and scratch.dtype == torch.float32
                           and scratch.numel() >= attention_mixed_scratch_elems(T, nh, dv, nsplit))
    assert not heads_rows or nh // nkv <= WINDOW_TC_ROWS
    units = T if heads_rows else -(-T // WINDOW_TC_ROWS) + num_seqs
    _check(watc_lib(dk, dv).atom_window_attention_tc(
        out.data_ptr(), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
        block_table.data_ptr(), block_table.shape[1], page_size, positions.data_ptr(), seq_of_token.data_ptr(),
        cu_q.data_ptr(), num_seqs, units, nh, nkv, float(scale), float(softcap or 0.0), int(window or 0),
        int(keep_first), int(nsplit), _ptr(scratch) if nsplit > 1 else None, int(heads_rows), _stream()),
        "window_attention_tc")
    if nsplit > 1:
        _check(lib().atom_window_attention_merge(out.data_ptr(), dtype_code(out.dtype), scratch.data_ptr(),
                                                 seq_of_token.data_ptr(), T, nh, dv, nsplit, _stream()),
               "window_attention_merge")


def lightning_supports(dk: int, dv: int) -> bool:
    return bool(lib().atom_lightning_supports(dk, dv))


LIGHTNING_RUN = 64        # rows per run of the lightning scan in steps of more rows than this


def lightning_run(T: int) -> int:
    """Rows per run for a step of T rows (0: every request is walked once)."""
    if T <= LIGHTNING_RUN:
        return 0
    return LIGHTNING_RUN if T <= 64 * LIGHTNING_RUN else -(-T // 64)


def lightning_scratch_elems(T: int, num_seqs: int, H: int, dk: int, dv: int) -> int:
    run = lightning_run(T)
    return 1 if run == 0 else (-(-T // run) + num_seqs) * H * dk * dv


def lightning_scan(out: torch.Tensor, proj: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
                   scratch: Optional[torch.Tensor], cu_q: torch.Tensor, state_slots: torch.Tensor, num_seqs: int,
                   H: int, dk: int, dv: int, write_state: bool = True) -> None:
    """out[t] (float32 [T, H dv]) = S_t^T silu(q_t) with S_t = decay_h S_(t-1) + silu(k_t) silu(v_t)^T per head, over
    every request's rows; proj rows are [q (H dk) | k (H dk) | v (H dv) | ...]; state [slots, H, dk, dv] float32."""
    _cuda(out, proj, decay, state, scratch, cu_q, state_slots)
    T = proj.shape[0]
    run = lightning_run(T)
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, H * dv) and proj.stride(1) == 1
    assert proj.shape[1] >= 2 * H * dk + H * dv and decay.dtype == torch.float32 and decay.numel() == H
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, dk, dv)
    assert run == 0 or (scratch is not None and scratch.dtype == torch.float32
                        and scratch.numel() >= lightning_scratch_elems(T, num_seqs, H, dk, dv))
    _check(lib().atom_lightning_scan(out.data_ptr(), proj.data_ptr(), dtype_code(proj.dtype), proj.stride(0),
                                     decay.data_ptr(), state.data_ptr(), _ptr(scratch) if run else None,
                                     cu_q.data_ptr(), state_slots.data_ptr(), num_seqs, T, H, dk, dv, run,
                                     int(write_state), _stream()), "lightning_scan")
    if run:
        add_launches(2)      # (the runs' sums, the prefix over the runs, the outputs)


def lightning_gate_norm(y: torch.Tensor, o: torch.Tensor, g: torch.Tensor, w: torch.Tensor, eps: float,
                        seq_of_token: torch.Tensor) -> None:
    """y = o / rms(o over the whole row) * w * sigmoid(g); o float32 [T, n], g a view of n columns of the projection."""
    _cuda(y, o, g, w, seq_of_token)
    T, n = o.shape
    assert o.dtype == torch.float32 and o.is_contiguous() and y.is_contiguous() and y.shape == (T, n)
    assert g.shape == (T, n) and g.stride(1) == 1 and g.dtype == y.dtype and w.numel() == n and w.is_contiguous()
    _check(lib().atom_lightning_gate_norm(y.data_ptr(), o.data_ptr(), g.data_ptr(), dtype_code(y.dtype), g.stride(0),
                                          w.data_ptr(), dtype_code(w.dtype), T, n, float(eps), seq_of_token.data_ptr(),
                                          _stream()), "lightning_gate_norm")


def moe_route(logits: torch.Tensor, E: int, top: int, score: str, renormalize: bool, seq_of_token: torch.Tensor,
              ids: torch.Tensor, wts: torch.Tensor, counts: torch.Tensor) -> None:
    """Per row: the ``top`` experts with the largest scores (sigmoid or softmax of logits[:, :E], float32), their
    scores as weights (divided by their sum if renormalize), and the experts' row counts added to ``counts``."""
    _cuda(logits, seq_of_token, ids, wts, counts)
    T = logits.shape[0]
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and logits.shape[1] >= E
    assert ids.dtype == counts.dtype == torch.int32 and wts.dtype == torch.float32 and ids.is_contiguous()
    assert wts.is_contiguous() and ids.shape == wts.shape == (T, top) and counts.numel() >= E
    _check(lib().atom_moe_route(logits.data_ptr(), logits.stride(0), T, E, top, int(score == "softmax"),
                                int(renormalize), seq_of_token.data_ptr(), ids.data_ptr(), wts.data_ptr(),
                                counts.data_ptr(), _stream()), "moe_route")


def moe_place(ids: torch.Tensor, wts: torch.Tensor, E: int, counts: torch.Tensor, offsets: torch.Tensor,
              row_token: torch.Tensor, row_w: torch.Tensor, pair_pos: torch.Tensor) -> None:
    """Sorts the (row, choice) pairs by expert: offsets [E + 1] (first place of every expert), for every place the
    row it came from and its weight, for every pair its place.  ``counts`` goes back to zero."""
    _cuda(ids, wts, counts, offsets, row_token, row_w, pair_pos)
    pairs, top = ids.numel(), ids.shape[1]
    assert offsets.numel() >= E + 1 and row_token.numel() >= pairs and row_w.numel() >= pairs and pair_pos.numel() >= pairs
    assert offsets.dtype == row_token.dtype == pair_pos.dtype == torch.int32 and row_w.dtype == torch.float32
    _check(lib().atom_moe_place(ids.data_ptr(), wts.data_ptr(), pairs, top, E, counts.data_ptr(), offsets.data_ptr(),
                                row_token.data_ptr(), row_w.data_ptr(), pair_pos.data_ptr(), _stream()), "moe_place")


MOE_TC = True        # False: the plain product also in bfloat16 (measurements, tests)


def moe_gemm(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, gated: bool = False,
             row_token: Optional[torch.Tensor] = None, row_w: Optional[torch.Tensor] = None) -> None:
    """out[r] = A[r] w[e]^T for the places r of every expert e (offsets [E + 1]); w [E, N or 2 N, K].  With row_token
    and row_w, A[r] = row_w[r] * a[row_token[r]] (rows picked from the step's rows, weighted on the way in); else
    A = a by place.  gated: w[e] = [gate ; up], out = silu(gate) * up.  bfloat16 with K and the row stride in steps
    of 8 runs on the tensor cores, everything else on plain FMAs."""
    _cuda(out, a, w, offsets, row_token, row_w)
    R, N = out.shape
    E, K = w.shape[0], w.shape[2]
    assert w.shape[1] == (2 * N if gated else N) and w.is_contiguous() and out.is_contiguous() and a.stride(1) == 1
    assert a.shape[1] == K and out.dtype == a.dtype == w.dtype and (row_token is not None or a.shape[0] >= R)
    _check(lib().atom_moe_gemm(out.data_ptr(), a.data_ptr(), dtype_code(a.dtype), a.stride(0), w.data_ptr(),
                               offsets.data_ptr(), _ptr(row_token), _ptr(row_w), R, E, N, K, int(gated),
                               int(row_token is not None), int(MOE_TC), _stream()), "moe_gemm")


def moe_combine(out: torch.Tensor, y: torch.Tensor, pair_pos: torch.Tensor, top: int,
                pair_w: Optional[torch.Tensor], shared: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                seq_of_token: torch.Tensor) -> None:
    """out[t] = sum over t's choices k of (pair_w[t, k] *) y[pair_pos[t, k]] (+ sigmoid(gate[t]) * shared[t]);
    gate: a float32 column view (one logit per row) or None (the shared part is added as it is)."""
    _cuda(out, y, pair_pos, pair_w, shared, gate, seq_of_token)
    T, n = out.shape
    assert out.is_contiguous() and y.is_contiguous() and y.shape[1] == n and out.dtype == y.dtype
    assert shared is None or (shared.is_contiguous() and shared.shape == (T, n) and shared.dtype == out.dtype)
    assert gate is None or (gate.dtype == torch.float32 and gate.shape[0] == T)
    _check(lib().atom_moe_combine(out.data_ptr(), y.data_ptr(), dtype_code(out.dtype), pair_pos.data_ptr(),
                                  _ptr(pair_w), top, _ptr(shared), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                  T, n, seq_of_token.data_ptr(), _stream()), "moe_combine")


_device_flags = {}


def device_flags(device: torch.device) -> torch.Tensor:
    """Two device ints that kernels raise and the host reads after a step (0: all well):
    [0] a bounded wait ran out, [1] a token position had no cache page."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    f = _device_flags.get(key)
    if f is None:
        f = _device_flags[key] = torch.zeros(2, dtype=torch.int32, device=device)
    return f


def error_flag(device: torch.device) -> torch.Tensor:
    """The device int that kernels with bounded waits set when a wait ran out."""
    return device_flags(device)[0:1]


def status_flag(device: torch.device) -> torch.Tensor:
    """The device int that kernels set when they meet a token position without a cache page."""
    return device_flags(device)[1:2]


FLAG_MESSAGES = ("a kernel's bounded wait ran out", "a kernel found a token position without a cache page")


def flash_has_tc(hd: int) -> bool:
    """Whether the attention library of this head size has the tcgen05 kernel for long portions."""
    return flash_supports(hd, torch.bfloat16) and bool(flash_lib(hd).atom_flash_has_tc())


def check_error_flags() -> None:
    """Raises if a kernel gave up a bounded wait or met a position without a page (synchronises the
    device); the flags are cleared, so the next check speaks of what ran after this one."""
    for f in _device_flags.values():
        v = f.tolist()
        if any(v):
            f.zero_()
            raise NativeError("; ".join(m for m, x in zip(FLAG_MESSAGES, v) if x))
    for hd, l in _flash_libs.items():      # (a device on which the library still uses its own flag)
        if l.atom_flash_take_error() != 0:
            raise NativeError(f"a bounded wait of the attention kernels (head size {hd}) ran out")


class _RowsOpC(ctypes.Structure):
    """csrc/gemm_rows.h: AtomRowsOp."""
    _fields_ = [("X", _vp), ("lda", _i64), ("W", _vp), ("out", _vp), ("out_dtype", _i), ("ldc", _i64),
                ("bias", _vp), ("bias_dtype", _i), ("N", _i), ("K", _i), ("gated", _i),
                ("ssq_in", _vp), ("ssq_parts", _i), ("norm_size", _i), ("norm_eps", _f),
                ("residual", _vp), ("norm_w", _vp), ("norm_w_dtype", _i), ("xout", _vp), ("ssq_out", _vp),
                ("res_scale", _f)]


ROWS_M = 16     # rows up to which the weight-streaming product is used (parts/linear.py: streams)


def gemm_rows_grid() -> int:
    """CTAs of a ``gemm_rows`` launch: a residual product writes one part of the rows' sums of squares per CTA."""
    return int(lib().atom_gemm_rows_grid())


def gemm_rows_supports(M: int, N: int, K: int, lda: int) -> bool:
    return bool(lib().atom_gemm_rows_supports(M, N, K, lda))


def gemm_rows(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
              bias: Optional[torch.Tensor] = None, gated: bool = False, ssq_in: Optional[torch.Tensor] = None,
              norm_size: int = 0, norm_eps: float = 0.0, residual: Optional[torch.Tensor] = None,
              norm_w: Optional[torch.Tensor] = None, xout: Optional[torch.Tensor] = None,
              ssq_out: Optional[torch.Tensor] = None, act: str = "silu", res_scale: float = 1.0) -> None:
    """out[M, N] = x[M, K] w[N, K]^T for at most 16 rows of bf16 x, with one of the epilogues of
    csrc/gemm_rows.h: plain (+ bias; out bf16 or float32); ``gated`` (w = [gate ; up] of 2N rows, ``act`` "silu" or
    "gelu_tanh" on the gate);
    ``residual`` (float32 [M, N], += ``res_scale`` * product in place, with ``xout`` = bf16(residual * norm_w) and the CTAs'
    sums of squares in ``ssq_out`` [gemm_rows_grid(), 16]).  ``ssq_in`` (such sums, of ``norm_size`` columns):
    every output row is first multiplied by its rstd."""
    M, K = x.shape
    res = residual is not None
    N = residual.shape[1] if res else out.shape[1]
    _cuda(x, w, out, bias, ssq_in, residual, norm_w, xout, ssq_out)
    assert x.dtype == w.dtype == torch.bfloat16 and w.shape[1] == K and w.is_contiguous() and x.stride(1) == 1
    assert w.shape[0] == (2 * N if gated else N)
    c = _RowsOpC()
    if res:
        assert residual.dtype == torch.float32 and residual.is_contiguous() and residual.shape[0] == M
        assert xout.dtype == torch.bfloat16 and xout.is_contiguous() and xout.shape == residual.shape
        assert ssq_out.dtype == torch.float32 and ssq_out.shape == (gemm_rows_grid(), 16) and ssq_out.is_contiguous()
        assert norm_w.numel() == N and norm_w.is_contiguous()
    else:
        assert out.shape[0] == M and out.stride(1) == 1
    if ssq_in is not None:
        assert ssq_in.dtype == torch.float32 and ssq_in.is_contiguous() and ssq_in.shape[-1] == 16
    c.X, c.lda, c.W = x.data_ptr(), x.stride(0), w.data_ptr()
    c.out = _ptr(out)
    c.out_dtype = dtype_code(out.dtype) if out is not None else BF16
    c.ldc = out.stride(0) if out is not None else 0
    c.bias, c.bias_dtype = _ptr(bias), (dtype_code(bias.dtype) if bias is not None else F32)
    c.N, c.K, c.gated = N, K, (GATE_ACTS[act] if gated else 0)
    c.ssq_in = _ptr(ssq_in)
    c.ssq_parts = ssq_in.numel() // 16 if ssq_in is not None else 0
    c.norm_size, c.norm_eps = int(norm_size), float(norm_eps)
    c.residual, c.norm_w = _ptr(residual), _ptr(norm_w)
    c.norm_w_dtype = dtype_code(norm_w.dtype) if norm_w is not None else F32
    c.xout, c.ssq_out = _ptr(xout), _ptr(ssq_out)
    c.res_scale = float(res_scale)
    _check(lib().atom_gemm_rows(ctypes.byref(c), M, error_flag(x.device).data_ptr(), _stream()), "gemm_rows")


def gemm_pairs_supports(M: int, N: int, K: int, lda: int, ldc: int) -> bool:
    return bool(lib().atom_gemm_pairs_supports(M, N, K, lda, ldc)) and gemm_pairs_resident() > 0


_pairs_resident = None


def gemm_pairs_resident() -> int:
    """Pairs of CTAs of a ``gemm_pairs`` launch: as many as the device holds at once."""
    global _pairs_resident
    if _pairs_resident is None:
        _pairs_resident = int(lib().atom_gemm_pairs_resident())
    return _pairs_resident


def gemm_pairs_waves(M: int, N: int, gated: bool) -> float:
    """How well the tiles of a ``gemm_pairs`` product fill the device: tiles / (waves x pairs), where the
    last, ragged wave counts 0.72 when it is handed out in halves (csrc/gemm_pairs.cu: plan_items; a half
    tile runs at about 0.72 of a whole one's time)."""
    pairs = gemm_pairs_resident()
    if pairs < 1:
        return 0.0
    tiles = -(-M // 256) * (-(-N // 256) if gated else -(-N // 512))
    full, rem = divmod(tiles, pairs)
    waves = full + (0.0 if rem == 0 else (0.72 if full > 0 and 2 * rem <= pairs else 1.0))
    return tiles / (waves * pairs)


def gemm_pairs(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False, act: str = "silu") -> None:
    """out[M, N] = x[M, K] w[N, K]^T in bf16 on tcgen05 with two CTAs to a tile; ``gated``: w = [gate ; up]
    of 2N rows, out = act(x gate^T) * (x up^T), ``act`` "silu" or "gelu_tanh" (csrc/gemm_pairs.cu)."""
    M, K = x.shape
    N = out.shape[1]
    _cuda(x, w, out)
    assert x.dtype == w.dtype == out.dtype == torch.bfloat16 and w.shape[1] == K and w.is_contiguous()
    assert x.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == M and w.shape[0] == (2 * N if gated else N)
    _check(lib().atom_gemm_pairs(x.data_ptr(), x.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0), M, N, K,
                                 GATE_ACTS[act] if gated else 0, error_flag(x.device).data_ptr(), _stream()), "gemm_pairs")


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    _cuda(out, bias)
    M, N = out.shape
    assert out.is_contiguous() and bias.numel() == N
    _check(lib().atom_add_bias(out.data_ptr(), dtype_code(out.dtype), bias.data_ptr(),
                               dtype_code(bias.dtype), M, N, _stream()), "add_bias")


# --------------------------------------------------------------------------- tensor-core attention

_flash_libs = {}
_FLASH_SIG = [_vp, _vp, _i64, _vp, _vp, _i64, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _i,
              _i, _vp, _vp]
_FLASH_ROT_SIG = [_vp, _vp, _i64, _vp, _vp, _i64, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _i, _vp,
                  _vp, _vp, _i, _i, _vp, _vp, _i, _f, _i, _vp, _vp]
LONG_ROWS = 128    # packed rows from which a request runs on the tcgen05 attention kernel
ROTATE_IN_DECODE = True    # decode steps leave q/k norm, rotation and cache write to the attention kernel where it takes them


def flash_supports(hd: int, dtype: torch.dtype) -> bool:
    """The tensor-core attention takes bfloat16 and head sizes that are multiples of 16 up to 256."""
    return dtype == torch.bfloat16 and hd % 16 == 0 and 16 <= hd <= 256


def flash_lib(hd: int):
    """The attention library compiled for this head size (built on first use)."""
    l = _flash_libs.get(hd)
    if l is None:
        with _lock:
            l = _flash_libs.get(hd)
            if l is None:
                path = build_variant("attention_flash.cu", {"ATOM_HD": hd})
                l = ctypes.CDLL(path)
                l.atom_flash_attention.argtypes = _FLASH_SIG
                l.atom_flash_attention.restype = ctypes.c_int
                l.atom_flash_scratch_bytes.argtypes = [_i, _i, _i]
                l.atom_flash_scratch_bytes.restype = ctypes.c_int64
                l.atom_flash_attention_rotating.argtypes = _FLASH_ROT_SIG
                l.atom_flash_attention_rotating.restype = ctypes.c_int
                l.atom_flash_rotating_supports.argtypes = [_i, _i64, _i, _i, _i]
                l.atom_flash_rotating_supports.restype = ctypes.c_int
                l.atom_flash_take_error.restype = ctypes.c_int
                l.atom_flash_has_tc.restype = ctypes.c_int
                if l.atom_flash_head_dim() != hd:
                    raise NativeBuildError(f"{path} was built for another head size")
                # bounded waits of this library report into the device's shared flag word, which the
                # engine reads back with every step's tokens (other devices keep the library's own flag)
                l.atom_flash_set_option.argtypes = [_i, _i]
                l.atom_flash_set_option.restype = ctypes.c_int
                for k, v in _option_values.items():
                    l.atom_flash_set_option(k, v)
                l.atom_flash_set_error_flag.argtypes = [_vp]
                l.atom_flash_set_error_flag.restype = ctypes.c_int
                if torch.cuda.is_available():
                    l.atom_flash_set_error_flag(error_flag(torch.device("cuda", torch.cuda.current_device())).data_ptr())
                _flash_libs[hd] = l
    return l


_sm_counts = {}


def sm_count() -> int:
    dev = torch.cuda.current_device()
    if dev not in _sm_counts:
        _sm_counts[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sm_counts[dev]


def flash_plan(q_lens, group: int, nkv: int, max_ctx: int, sms: Optional[int] = None, long_rows: int = 0):
    """Host-side launch plan: (64-row tiles of the mid-size requests, any short request?,
    splits[, 128-row tiles of the long requests when long_rows > 0]).

    Short requests (at most 16 packed rows) are split along their keys.  Two CTAs fit an SM.
    Measured on B200: one wave of CTAs (at most 2 per SM) is best, with splits no shorter than
    256 keys; when even one split per (request, kv head) is more than a wave, a larger split
    count (up to 8) only where it fills whole waves at least 15 % better (every split costs a
    pass of the merge kernel over its partial sums)."""
    sms = sms or sm_count()
    tiles, short, long_tiles = 0, 0, 0
    for n in q_lens:
        rows = n * group
        if long_rows and rows >= long_rows:
            long_tiles += -(-rows // 128)
        elif rows > 16:
            tiles += -(-rows // 64)
        elif rows > 0:
            short += 1
    splits = 1
    if short:
        slots = 2 * sms
        pairs = max(1, len(q_lens) * nkv)
        longest = max(1, -(-max_ctx // 256))
        if pairs <= slots:
            splits = max(1, min(slots // pairs, longest, 64))
        else:
            best = 0.0
            for s in range(1, min(8, longest) + 1):
                ctas = pairs * s
                eff = ctas / (-(-ctas // slots) * slots)
                if eff > best * 1.15:
                    best, splits = eff, s
    if long_rows:
        return tiles, short > 0, splits, long_tiles
    return tiles, short > 0, splits


def flash_plan_for_any(tokens: int, seqs: int, group: int, nkv: int, max_ctx: int, sms: Optional[int] = None,
                       long_rows: int = 0):
    """A launch plan that holds for every batch of at most ``tokens`` tokens in at most ``seqs`` requests
    (for a step recorded once and replayed for batches of other makeups): tile counts are upper bounds
    (the kernels find their tile from the step's arrays; a CTA without one leaves at once), short
    requests are always provided for, with the splits of ``seqs`` short requests."""
    rows = tokens * group
    n_long = min(seqs, rows // long_rows) if long_rows else 0
    long_tiles = rows // 128 + 1 + n_long if long_rows else 0
    tiles = rows // 64 + 1 + min(seqs, max(1, rows // 17))
    splits = flash_plan([1] * seqs, group, nkv, max_ctx, sms)[2]
    if long_rows:
        return tiles, True, splits, long_tiles
    return tiles, True, splits


def flash_attention(out: torch.Tensor, q: torch.Tensor, q_stride: int, k_pages: torch.Tensor,
                    v_pages: torch.Tensor, block_table: torch.Tensor, cu_q: torch.Tensor,
                    ctx_len: torch.Tensor, seq_of_token: torch.Tensor, T: int, num_seqs: int, nh: int,
                    nkv: int, hd: int, scale: float, window: int, plan, scratch: Optional[torch.Tensor]) -> None:
    """out[T, nh*hd] (bf16): causal attention of every token over its request's pages, on the
    tensor cores.  ``plan`` comes from ``flash_plan``; ``scratch`` (float32) must hold
    ``flash_scratch_elems`` elements when the plan has more than one split."""
    _cuda(out, q, k_pages, v_pages, block_table, cu_q, ctx_len, seq_of_token, scratch)
    page_size = k_pages.shape[2]
    assert out.dtype == q.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16
    assert out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert tuple(k_pages.shape[1:]) == (nkv, page_size, hd) and v_pages.shape == k_pages.shape
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
    assert cu_q.dtype == ctx_len.dtype == seq_of_token.dtype == torch.int32
    tiles, has_short, splits = plan[:3]
    long_tiles = plan[3] if len(plan) > 3 else 0
    if splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32
        assert scratch.numel() >= flash_scratch_elems(T, nh, hd, splits)
    l = flash_lib(hd)
    _check(l.atom_flash_attention(
        out.data_ptr(), q.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
        block_table.data_ptr(), block_table.shape[1], page_size, cu_q.data_ptr(), ctx_len.data_ptr(),
        seq_of_token.data_ptr(), T, num_seqs, nh, nkv, hd, float(scale), int(window), int(long_tiles),
        LONG_ROWS, int(tiles), int(has_short), int(splits), _ptr(scratch), _stream()), "flash_attention")
    # (one kernel for the long portions, one for the others, one for the short requests, one that merges their splits)
    add_launches(int(long_tiles > 0) + int(tiles > 0) + int(bool(has_short)) + int(bool(has_short) and splits > 1) - 1)


def flash_rotating_supports(hd: int, page_size: int, num_pages: int, nh: int, nkv: int, rotary_dim: int) -> bool:
    """A decode step of these sizes can leave the heads' norm, the rotation and the cache write of its new
    tokens to the decode attention kernel (``flash_attention_rotating``)."""
    return ROTATE_IN_DECODE and flash_supports(hd, torch.bfloat16) and bool(
        flash_lib(hd).atom_flash_rotating_supports(page_size, num_pages, nh, nkv, rotary_dim))


def flash_attention_rotating(out: torch.Tensor, qkv: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                             block_table: torch.Tensor, cu_q: torch.Tensor, ctx_len: torch.Tensor,
                             seq_of_token: torch.Tensor, T: int, num_seqs: int, nh: int, nkv: int, hd: int,
                             scale: float, window: int, splits: int, scratch: Optional[torch.Tensor],
                             table: torch.Tensor, rotary_dim: int, rows: torch.Tensor,
                             q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                             write_cache: bool, status: torch.Tensor) -> None:
    """Decode attention of a step in which every request brings one token, over the raw projection
    qkv[T, (nh + 2 nkv) * hd]: the kernel normalises each query and key head (weights or None), rotates it
    by row rows[t] of ``table`` [positions, rotary_dim] (cos, then sin), stores the new key and value in the
    token's page (``write_cache``; a token without a page sets ``status``) and attends.  out[T, nh*hd]."""
    _cuda(out, qkv, k_pages, v_pages, block_table, cu_q, ctx_len, seq_of_token, scratch, table, rows, q_weight,
          k_weight, status)
    page_size = k_pages.shape[2]
    assert out.dtype == qkv.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16 and T == num_seqs
    assert out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous() and qkv.stride(1) == 1
    assert qkv.shape[1] == (nh + 2 * nkv) * hd
    assert tuple(k_pages.shape[1:]) == (nkv, page_size, hd) and v_pages.shape == k_pages.shape
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
    assert cu_q.dtype == ctx_len.dtype == seq_of_token.dtype == rows.dtype == status.dtype == torch.int32
    assert table.dtype == torch.float32 and table.is_contiguous() and table.shape[1] == rotary_dim
    w = q_weight if q_weight is not None else k_weight
    if w is not None:
        assert all(x is None or (x.dtype == w.dtype and x.numel() == hd and x.is_contiguous()) for x in (q_weight, k_weight))
    if splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32
        assert scratch.numel() >= flash_scratch_elems(T, nh, hd, splits)
    l = flash_lib(hd)
    _check(l.atom_flash_attention_rotating(
        out.data_ptr(), qkv.data_ptr(), qkv.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
        block_table.data_ptr(), block_table.shape[1], page_size, cu_q.data_ptr(), ctx_len.data_ptr(),
        seq_of_token.data_ptr(), T, num_seqs, nh, nkv, hd, float(scale), int(window), int(splits), _ptr(scratch),
        table.data_ptr(), rows.data_ptr(), int(rotary_dim), table.shape[0], _ptr(q_weight), _ptr(k_weight),
        dtype_code(w.dtype) if w is not None else F32, float(eps), int(write_cache), status.data_ptr(), _stream()),
        "flash_attention_rotating")
    add_launches(int(splits > 1))      # (the kernel that merges the splits)


def flash_scratch_elems(T: int, nh: int, hd: int, splits: int) -> int:
    return 0 if splits <= 1 else T * nh * splits * (hd + 2)


# ------------------------------------------------------------------ embedding with a table of token pairs, stream steps

def pair_embedding(out: torch.Tensor, table: torch.Tensor, pairs: torch.Tensor, ids: torch.Tensor,
                   positions: torch.Tensor, seq_of_token: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor,
                   prev_state: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int, scale: float = 1.0,
                   write_state: bool = True) -> None:
    """out[t] = table[id] * scale + pairs[(previous id * mul_prev + id * mul_cur) mod buckets] in float32; a request's
    first token takes pairs[buckets].  prev_state [slots] int32 carries a request's last id from step to step."""
    _cuda(out, table, pairs, ids, positions, seq_of_token, cu_q, state_slots, prev_state)
    T, H = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous() and pairs.is_contiguous()
    assert table.dtype == pairs.dtype and table.shape[1] == H and tuple(pairs.shape) == (buckets + 1, H)
    assert prev_state.dtype == torch.int32 and prev_state.is_contiguous() and ids.dtype == torch.int32
    _check(lib().atom_pair_embedding(out.data_ptr(), table.data_ptr(), pairs.data_ptr(), dtype_code(table.dtype),
                                     ids.data_ptr(), positions.data_ptr(), seq_of_token.data_ptr(), cu_q.data_ptr(),
                                     state_slots.data_ptr(), prev_state.data_ptr(), T, H, table.shape[0], int(buckets),
                                     int(mul_prev), int(mul_cur), float(scale), int(write_state), _stream()),
           "pair_embedding")


def add_row(residual: torch.Tensor, vec: torch.Tensor) -> None:
    """residual[t] += vec for every row (float32 sums)."""
    _cuda(residual, vec)
    T, H = residual.shape
    assert residual.dtype == torch.float32 and residual.is_contiguous() and vec.is_contiguous() and vec.numel() == H
    _check(lib().atom_add_row(residual.data_ptr(), vec.data_ptr(), dtype_code(vec.dtype), T, H, _stream()), "add_row")


def normed_add_rmsnorm(out: torch.Tensor, residual: torch.Tensor, delta: torch.Tensor, delta_weight: torch.Tensor,
                       delta_eps: float, weight: torch.Tensor, eps: float, rows: Optional[torch.Tensor] = None,
                       n_rows: Optional[int] = None) -> None:
    """residual += rmsnorm(delta; delta_weight); out = rmsnorm(residual; weight), one kernel, 32-bit.  With ``rows``
    only those rows, written densely, and residual is left as it is."""
    _cuda(out, residual, delta, delta_weight, weight, rows)
    H = residual.shape[-1]
    assert residual.dtype == torch.float32 and residual.is_contiguous() and out.is_contiguous()
    assert delta.dtype == out.dtype and delta.is_contiguous() and delta.shape[-1] == H
    assert weight.numel() == H and delta_weight.numel() == H and weight.dtype == delta_weight.dtype
    n = (rows.numel() if n_rows is None else n_rows) if rows is not None else residual.shape[0]
    _check(lib().atom_normed_add_rmsnorm(out.data_ptr(), dtype_code(out.dtype), residual.data_ptr(), delta.data_ptr(),
                                         delta_weight.data_ptr(), float(delta_eps), weight.data_ptr(),
                                         dtype_code(weight.dtype), float(eps), _ptr(rows), n, H, _stream()),
           "normed_add_rmsnorm")


def head_gate(x: torch.Tensor, g: torch.Tensor) -> None:
    """x[t, h, :] *= sigmoid(g[t, h]); x [T, H, n] dense, g [T, H] a view whose rows may lie further apart."""
    _cuda(x, g)
    T, H, n = x.shape
    assert x.is_contiguous() and g.shape == (T, H) and g.stride(1) == 1 and g.dtype == x.dtype
    _check(lib().atom_head_gate(x.data_ptr(), g.data_ptr(), dtype_code(x.dtype), g.stride(0), T, H, n, _stream()),
           "head_gate")


# ------------------------------------------------------------------ gated linear attention

def gla_supports(dk: int, dv: int) -> bool:
    return bool(lib().atom_gla_supports(dk, dv))


GLA_RUN = 64        # rows per run of the scan in steps of more rows than this


def gla_run(T: int) -> int:
    """Rows per run for a step of T rows (0: every request is walked once)."""
    if T <= GLA_RUN:
        return 0
    return GLA_RUN if T <= 64 * GLA_RUN else -(-T // 64)


def gla_scratch_elems(T: int, num_seqs: int, H: int, dk: int, dv: int):
    """(floats of the runs' sums, floats of the runs' decay products)."""
    run = gla_run(T)
    if run == 0:
        return 0, 0
    slots = -(-T // run) + num_seqs
    return slots * H * dk * dv, slots * H * dk


def gla_scan(out: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, z_bias: torch.Tensor,
             tau: float, q_scale: float, state: torch.Tensor, scratch_b: Optional[torch.Tensor],
             scratch_a: Optional[torch.Tensor], cu_q: torch.Tensor, state_slots: torch.Tensor, num_seqs: int, H: int,
             dk: int, dv: int, write_state: bool = True) -> None:
    """out[t] (float32 [T, H dv]) = S_t^T (q_t q_scale), S_t = diag(a_t) S_(t-1) + k_t v_t^T per head with
    a_t = sigmoid(z_t + z_bias)^(1 / tau), over every request's rows.  q, k [T, H dk] and v [T, H dv] are views of one
    array of rows (equal row stride); z [T, H dk] float32 (steps that are cut into runs leave the decays in it);
    state [slots, H, dk, dv] float32."""
    _cuda(out, q, k, v, z, z_bias, state, scratch_a, scratch_b, cu_q, state_slots)
    T = q.shape[0]
    run = gla_run(T)
    assert out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, H * dv)
    assert q.stride(0) == k.stride(0) == v.stride(0) and q.stride(1) == k.stride(1) == v.stride(1) == 1
    assert q.dtype == k.dtype == v.dtype and q.shape[1] == k.shape[1] == H * dk and v.shape[1] == H * dv
    assert z.dtype == torch.float32 and z.stride(1) == 1 and z.shape == (T, H * dk) and z_bias.numel() == H * dk
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, dk, dv)
    if run:
        nb, na = gla_scratch_elems(T, num_seqs, H, dk, dv)
        assert scratch_b is not None and scratch_a is not None and scratch_b.dtype == scratch_a.dtype == torch.float32
        assert scratch_b.numel() >= nb and scratch_a.numel() >= na
    _check(lib().atom_gla_scan(out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), dtype_code(q.dtype), q.stride(0),
                               z.data_ptr(), z.stride(0), z_bias.data_ptr(), dtype_code(z_bias.dtype), float(tau),
                               float(q_scale), state.data_ptr(), _ptr(scratch_b) if run else None,
                               _ptr(scratch_a) if run else None, cu_q.data_ptr(), state_slots.data_ptr(), num_seqs, T, H,
                               dk, dv, run, int(write_state), _stream()), "gla_scan")
    if run:
        add_launches(3)      # (the decays, the runs' sums, the prefix over the runs, the outputs)


def gla_gate_norm(y: torch.Tensor, o: torch.Tensor, g: torch.Tensor, w: torch.Tensor, eps: float, H: int, dv: int,
                  seq_of_token: torch.Tensor) -> None:
    """y[t, h] = o[t, h] / rms(o[t, h]) * w * silu(g[t, h]): the norm runs over one head's columns, w [dv] is shared by
    the heads.  o float32 [T, H dv]; g a view whose rows may lie further apart."""
    _cuda(y, o, g, w, seq_of_token)
    T = o.shape[0]
    assert o.dtype == torch.float32 and o.is_contiguous() and y.is_contiguous() and y.shape == o.shape == (T, H * dv)
    assert g.dtype == y.dtype and g.stride(1) == 1 and g.shape == (T, H * dv) and w.numel() == dv
    _check(lib().atom_gla_gate_norm(y.data_ptr(), o.data_ptr(), g.data_ptr(), dtype_code(y.dtype), g.stride(0),
                                    w.data_ptr(), dtype_code(w.dtype), T, H, dv, float(eps), seq_of_token.data_ptr(),
                                    _stream()), "gla_gate_norm")


# ------------------------------------------------------------------ attention over a window and pooled blocks

def pooled_attention_supports(H: int, G: int, dk: int, dv: int) -> bool:
    return bool(lib().atom_pooled_attention_supports(H, G, dk, dv))


def pool_blocks(k_pages: torch.Tensor, v_pages: torch.Tensor, pk_pages: torch.Tensor, pv_pages: torch.Tensor,
                block_table: torch.Tensor, pool_table: torch.Tensor, page_size: int, positions: torch.Tensor,
                seq_of_token: torch.Tensor, T: int, pool: int, status: torch.Tensor) -> None:
    """For every token of the step that ends a block of ``pool`` positions: the means of the block's cached keys and
    values go to the block's row of the pooled pages.  Pages [pages, kv heads, page, size]."""
    _cuda(k_pages, v_pages, pk_pages, pv_pages, block_table, pool_table, positions, seq_of_token, status)
    G, dk, dv = k_pages.shape[1], k_pages.shape[3], v_pages.shape[3]
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and pk_pages.is_contiguous() and pv_pages.is_contiguous()
    assert k_pages.dtype == v_pages.dtype == pk_pages.dtype == pv_pages.dtype
    assert tuple(pk_pages.shape[1:]) == (G, page_size, dk) and tuple(pv_pages.shape[1:]) == (G, page_size, dv)
    assert block_table.dtype == pool_table.dtype == torch.int32 and block_table.is_contiguous() and pool_table.is_contiguous()
    _check(lib().atom_pool_blocks(k_pages.data_ptr(), v_pages.data_ptr(), pk_pages.data_ptr(), pv_pages.data_ptr(),
                                  dtype_code(k_pages.dtype), block_table.data_ptr(), block_table.shape[1],
                                  pool_table.data_ptr(), pool_table.shape[1], page_size, k_pages.shape[0],
                                  pk_pages.shape[0], positions.data_ptr(), seq_of_token.data_ptr(), T, G, dk, dv,
                                  int(pool), status.data_ptr(), _stream()), "pool_blocks")


def pooled_attention(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     pk_pages: Optional[torch.Tensor], pv_pages: Optional[torch.Tensor], block_table: torch.Tensor,
                     pool_table: Optional[torch.Tensor], page_size: int, positions: torch.Tensor,
                     seq_of_token: torch.Tensor, H: int, scale: float, window: int, pool: int, sink: bool,
                     mix: Optional[torch.Tensor], gate: Optional[torch.Tensor]) -> None:
    """out[t, h] = sum_x w_h[x] v[x] over the tokens of the window and the pooled blocks before it (see
    csrc/pooled_attention.cu), times sigmoid(gate[t, h]) with a gate.  q [T, H dk] (rows may lie apart), out [T, H dv]
    dense, mix [H, H] float32 or None, gate [T, H dv] (rows may lie apart) or None."""
    _cuda(out, q, k_pages, v_pages, pk_pages, pv_pages, block_table, pool_table, positions, seq_of_token, mix, gate)
    T = q.shape[0]
    G, dk, dv = k_pages.shape[1], k_pages.shape[3], v_pages.shape[3]
    assert out.is_contiguous() and out.shape == (T, H * dv) and q.shape[1] == H * dk and q.stride(1) == 1
    assert out.dtype == q.dtype == k_pages.dtype == v_pages.dtype and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert mix is None or (mix.dtype == torch.float32 and mix.is_contiguous() and tuple(mix.shape) == (H, H))
    assert gate is None or (gate.dtype == out.dtype and gate.shape == out.shape and gate.stride(1) == 1)
    assert block_table.dtype == torch.int32 and block_table.is_contiguous()
    if pool and window:
        assert pk_pages is not None and pv_pages is not None and pool_table is not None and pool_table.is_contiguous()
        assert pk_pages.dtype == pv_pages.dtype == out.dtype and pk_pages.is_contiguous() and pv_pages.is_contiguous()
    _check(lib().atom_pooled_attention(out.data_ptr(), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
                                       _ptr(pk_pages), _ptr(pv_pages), dtype_code(out.dtype), block_table.data_ptr(),
                                       block_table.shape[1], _ptr(pool_table),
                                       pool_table.shape[1] if pool_table is not None else 0, page_size,
                                       positions.data_ptr(), seq_of_token.data_ptr(), T, H, G, dk, dv, float(scale),
                                       int(window), int(pool), int(bool(sink)), _ptr(mix), _ptr(gate),
                                       gate.stride(0) if gate is not None else 0, _stream()), "pooled_attention")


def pooled_attention_split_supports(H: int, G: int, dk: int, dv: int) -> bool:
    return bool(lib().atom_pooled_attention_split_supports(H, G, dk, dv))


POOLED_SPLIT_ROWS = 64      # steps of up to this many tokens share every token's keys out among CTAs (0: never)


def pooled_attention_splits(T: int, longest: int) -> int:
    """Into how many shares a step of T tokens cuts every token's keys (``longest``: the most keys a token sees): two
    CTAs per SM fill the device, in shares of at least 64 keys."""
    return max(1, min(-(-2 * SM_COUNT // max(T, 1)), -(-longest // 64), 64))


def pooled_attention_scratch_elems(T: int, H: int, G: int, dv: int, nsplit: int) -> int:
    return T * nsplit * (2 * H + H * G * dv)


def pooled_attention_split(out: torch.Tensor, scratch: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor,
                           v_pages: torch.Tensor, pk_pages: Optional[torch.Tensor], pv_pages: Optional[torch.Tensor],
                           block_table: torch.Tensor, pool_table: Optional[torch.Tensor], page_size: int,
                           positions: torch.Tensor, seq_of_token: torch.Tensor, H: int, scale: float, window: int,
                           pool: int, sink: bool, mix: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                           nsplit: int) -> None:
    """``pooled_attention`` for steps of few tokens: every token's keys are shared out among ``nsplit`` CTAs, which
    leave unnormalised sums per (head, kv head) in ``scratch``; a merge kernel puts them together, divides and mixes
    the heads (csrc/pooled_attention.cu)."""
    _cuda(out, scratch, q, k_pages, v_pages, pk_pages, pv_pages, block_table, pool_table, positions, seq_of_token, mix, gate)
    T = q.shape[0]
    G, dk, dv = k_pages.shape[1], k_pages.shape[3], v_pages.shape[3]
    assert out.is_contiguous() and out.shape == (T, H * dv) and q.shape[1] == H * dk and q.stride(1) == 1
    assert out.dtype == q.dtype == k_pages.dtype == v_pages.dtype and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert mix is None or (mix.dtype == torch.float32 and mix.is_contiguous() and tuple(mix.shape) == (H, H))
    assert gate is None or (gate.dtype == out.dtype and gate.shape == out.shape and gate.stride(1) == 1)
    assert block_table.dtype == torch.int32 and block_table.is_contiguous()
    assert scratch.dtype == torch.float32 and scratch.numel() >= pooled_attention_scratch_elems(T, H, G, dv, nsplit)
    if pool and window:
        assert pk_pages is not None and pv_pages is not None and pool_table is not None and pool_table.is_contiguous()
        assert pk_pages.dtype == pv_pages.dtype == out.dtype and pk_pages.is_contiguous() and pv_pages.is_contiguous()
    _check(lib().atom_pooled_attention_split(
        out.data_ptr(), scratch.data_ptr(), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
        _ptr(pk_pages), _ptr(pv_pages), dtype_code(out.dtype), block_table.data_ptr(), block_table.shape[1],
        _ptr(pool_table), pool_table.shape[1] if pool_table is not None else 0, page_size, positions.data_ptr(),
        seq_of_token.data_ptr(), T, H, G, dk, dv, float(scale), int(window), int(pool), int(bool(sink)), _ptr(mix),
        _ptr(gate), gate.stride(0) if gate is not None else 0, int(nsplit), _stream()), "pooled_attention_split")
    add_launches(1)      # (the merge)


_PWTC_SIG = [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _i, _f, _i, _i, _i, _vp, _vp, _i64, _vp]
POOLED_TC = True     # False: the plain kernel also where the tensor-core kernel takes the sizes (measurements, tests)
_pwtc_libs = {}


def pooled_attention_tc_supports(nh: int, nkv: int, dk: int, dv: int, dtype: torch.dtype) -> bool:
    """Sizes the tensor-core kernel takes: bfloat16, up to 16 heads, key and value sizes in steps of 16, a warp's output
    tiles within its registers, everything within an SM's shared memory."""
    if dtype != torch.bfloat16 or nh > 16 or nkv <= 0 or nh % nkv or dk % 16 or dv % 16 or dk <= 0 or dv <= 0:
        return False
    group = nh // nkv
    tpg = -(-(group * (dv // 16)) // 16)
    if nkv * tpg * 8 > 64:
        return False
    smem = 2 * (nh * 16 * (dk + 8) + 2 * 64 * (max(dk, dv) + 8)) + 4 * nh * 16 * 72 + 4 * nh * nh + 4 * 2 * nh * 16 + 4 * 2 * 64
    return smem <= 226 * 1024


def pwtc_lib(nh: int, nkv: int, dk: int, dv: int):
    key = (nh, nkv, dk, dv)
    l = _pwtc_libs.get(key)
    if l is None:
        with _lock:
            l = _pwtc_libs.get(key)
            if l is None:
                path = build_variant("pooled_attention_tc.cu", {"ATOM_PW_NH": nh, "ATOM_PW_NKV": nkv, "ATOM_PW_DK": dk,
                                                                "ATOM_PW_DV": dv})
                l = ctypes.CDLL(path)
                l.atom_pooled_attention_tc.argtypes = _PWTC_SIG
                l.atom_pooled_attention_tc.restype = ctypes.c_int
                l.atom_pwtc_set_option.argtypes = [_i, _i]
                l.atom_pwtc_set_option.restype = ctypes.c_int
                got = [ctypes.c_int() for _ in range(4)]
                l.atom_pwtc_sizes(*[ctypes.byref(g) for g in got])
                if tuple(g.value for g in got) != key:
                    raise NativeBuildError(f"{path} was built for other sizes")
                for k, v in _option_values.items():
                    l.atom_pwtc_set_option(k, v)
                _pwtc_libs[key] = l
    return l


def pooled_attention_tc(out: torch.Tensor, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                        pk_pages: Optional[torch.Tensor], pv_pages: Optional[torch.Tensor], block_table: torch.Tensor,
                        pool_table: Optional[torch.Tensor], page_size: int, positions: torch.Tensor, cu_q: torch.Tensor,
                        num_seqs: int, H: int, scale: float, window: int, pool: int, sink: bool,
                        mix: Optional[torch.Tensor], gate: Optional[torch.Tensor]) -> None:
    """``pooled_attention`` on the tensor cores (bfloat16): tiles of 16 consecutive tokens of a request with all heads
    (cu_q: [num_seqs + 1] first token row of every request).  Sizes as ``pooled_attention_tc_supports`` says."""
    _cuda(out, q, k_pages, v_pages, pk_pages, pv_pages, block_table, pool_table, positions, cu_q, mix, gate)
    T = q.shape[0]
    G, dk, dv = k_pages.shape[1], k_pages.shape[3], v_pages.shape[3]
    assert out.is_contiguous() and out.shape == (T, H * dv) and q.shape[1] == H * dk and q.stride(1) == 1
    assert out.dtype == q.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16
    assert k_pages.is_contiguous() and v_pages.is_contiguous() and cu_q.numel() >= num_seqs + 1
    assert tuple(k_pages.shape[1:]) == (G, page_size, dk) and tuple(v_pages.shape[1:]) == (G, page_size, dv)
    assert mix is None or (mix.dtype == torch.float32 and mix.is_contiguous() and tuple(mix.shape) == (H, H))
    assert gate is None or (gate.dtype == out.dtype and gate.shape == out.shape and gate.stride(1) == 1)
    assert block_table.dtype == torch.int32 and block_table.is_contiguous()
    if pool and window:
        assert pk_pages is not None and pv_pages is not None and pool_table is not None and pool_table.is_contiguous()
        assert pk_pages.dtype == pv_pages.dtype == out.dtype and pk_pages.is_contiguous() and pv_pages.is_contiguous()
    tiles = -(-T // 16) + num_seqs
    _check(pwtc_lib(H, G, dk, dv).atom_pooled_attention_tc(
        out.data_ptr(), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), _ptr(pk_pages), _ptr(pv_pages),
        block_table.data_ptr(), block_table.shape[1], _ptr(pool_table),
        pool_table.shape[1] if pool_table is not None else 0, page_size, positions.data_ptr(), cu_q.data_ptr(), num_seqs,
        tiles, float(scale), int(window), int(pool), int(bool(sink)), _ptr(mix), _ptr(gate),
        gate.stride(0) if gate is not None else 0, _stream()), "pooled_attention_tc")
