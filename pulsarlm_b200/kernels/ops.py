"""Python face of the CUDA kernel library: one function per entry point.

The library is loaded with ctypes on first use (and built first if stale). There
is no fallback: if it cannot be built or loaded, or the device is not sm_100,
the call raises. Every function launches on torch's current CUDA stream and
takes torch tensors on the device; shapes and dtypes are checked here, sizes a
kernel refuses come back as KernelError with the kernel's message.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

from . import build

_I32 = ctypes.c_int
_I64 = ctypes.c_int64
_F32 = ctypes.c_float
_PTR = ctypes.c_void_p

_lib = None
_lock = threading.Lock()

ABI_VERSION = 28

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    """A kernel refused its arguments or failed to launch."""


_SIGNATURES = {
    "pl_embed": [_PTR, _PTR, _PTR, _I32, _I32, _I32, _F32, _I32, _PTR, _PTR],
    "pl_add_normed_rmsnorm": [_PTR, _PTR, _PTR, _PTR, _F32, _F32, _PTR, _F32, _PTR, _PTR, _I32, _I32, _PTR, _PTR, _PTR,
                              _I32, _I32, _PTR],
    "pl_bias_act": [_PTR, _I64, _PTR, _PTR, _I32, _I32, _I32, _I32, _PTR],
    "pl_short_conv": [_PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _PTR],
    "pl_short_conv_state": [_PTR, _PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _PTR],
    "pl_delta_rule": [_PTR, _PTR, _PTR, _PTR, _PTR, _I64, _PTR, _I64, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR,
                      _PTR, _I64, _I32, _I32, _I32, _I32, _F32, _F32, _F32, _I32, _PTR],
    "pl_norm_write_paged": [_PTR, _I64, _PTR, _F32, _PTR, _PTR, _PTR, _I32, _PTR, _I64, _I32, _I32, _I32, _I32, _I32,
                            _PTR, _PTR],
    "pl_take_tokens": [_PTR, _PTR, _PTR, _I32, _I32, _PTR, _PTR],
    "pl_add_rmsnorm": [_PTR, _PTR, _PTR, _I32, _PTR, _PTR, _I32, _I32, _F32, _I32, _PTR],
    "pl_swiglu": [_PTR, _PTR, _I32, _I32, _I32, _PTR],
    "pl_bf16_to_f32": [_PTR, _PTR, _I64, _PTR],
    "pl_gemm_f32": [_PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _PTR],
    "pl_rope_kv_write": [_PTR, _PTR, _PTR, _I64, _PTR, _PTR, _PTR, _I32, _PTR, _PTR, _I64, _I64, _I32, _I32,
                         _PTR, _I32, _I32, _I32, _I32, _I32, _I32, _PTR, _PTR, _F32, _PTR, _PTR],
    "pl_attention_simt": [_PTR, _I64, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _PTR, _PTR, _I64,
                          _I32, _I32, _I32, _I32, _I32, _F32, _F32, _I32, _PTR, _PTR, _PTR, _PTR, _PTR, _I64, _PTR,
                          _I32, _PTR, _PTR],
    "pl_attention_decode": [_PTR, _I64, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _PTR, _PTR, _I64,
                            _I32, _I32, _I32, _I32, _I32, _F32, _I32, _PTR, _PTR, _PTR, _PTR],
    "pl_attention_decode_mass": [_PTR, _I64, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _PTR, _PTR, _I64,
                                 _I32, _I32, _I32, _I32, _I32, _F32, _I32, _PTR, _PTR, _I32, _PTR, _PTR, _F32, _PTR,
                                 _PTR],
    "pl_attention_decode_items": [_PTR, _I64, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _PTR, _PTR, _I64,
                                  _I32, _I32, _I32, _I32, _I32, _F32, _PTR, _I32, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR],
    "pl_attention_decode_ctas_per_sm": [_I32],
    "pl_layer_forward": [_PTR, _PTR, _PTR],
    "pl_gemm_bf16_skinny_gated_in": [_PTR, _PTR, _PTR, _I32, _I32, _I32, _I64, _I64, _I64, _I32, _PTR, _PTR],
    "pl_gemm_bf16_skinny_act_in": [_PTR, _PTR, _PTR, _PTR, _I32, _I32, _I32, _I64, _I64, _I64, _I32, _I32, _PTR, _PTR],
    "pl_fill_random": [_PTR, _I64, _I32, ctypes.c_uint64, ctypes.c_uint64, _F32, _F32, _PTR],
    "pl_attention_decode_supports": [_I32, _I32, _I32, _I32],
    "pl_attention_prefill": [_PTR, _I64, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _I32, _PTR, _I64,
                             _I32, _I32, _I32, _I32, _F32, _PTR, _PTR, _PTR],
    "pl_attention_decode_extras": [_PTR, _I64, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _PTR, _PTR, _I64,
                                   _I32, _I32, _I32, _I32, _I32, _F32, _I32, _PTR, _PTR, _PTR, _PTR],
    "pl_attention_prefill_supports": [_I32, _I32, _I32],
    "pl_attention_prefill_tcgen05": [_PTR, _I64, _I32, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _I32,
                                     _PTR, _I64, _I32, _I32, _I32, _I32, _F32, _I32, _PTR, _I32, _PTR, _PTR, _PTR],
    "pl_attention_prefill_tcgen05_bias": [_PTR, _I64, _I32, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR, _I32, _PTR, _I32,
                                          _PTR, _I64, _I32, _I32, _I32, _I32, _F32, _I32, _PTR, _PTR, _I32, _PTR, _PTR],
    "pl_attention_prefill_tcgen05_tile_rows": [_I32],
    "pl_attention_prefill_tcgen05_supports": [_I32, _I32, _I32, _I64, _I64, _I64, _I32],
    "pl_attention_prefill_tile_rows": [],
    "pl_gemm_bf16_pair_supports": [_I32, _I32, _I32, _I64, _I64],
    "pl_gemm_bf16_skinny": [_PTR, _PTR, _PTR, _I32, _I32, _I32, _I64, _I64, _I64, _I32, _PTR, _PTR],
    "pl_gemm_bf16_skinny_max_tokens": [],
    "pl_gemm_bf16_pair": [_PTR, _PTR, _PTR, _I32, _I32, _I32, _I64, _I64, _I64, _I32, _I32, _PTR, _PTR],
    "pl_attention_decode_resident_clusters": [_I32, _I32, _I32],
    "pl_gemm_bf16_skinny_splits": [_I32, _I32, _I32],
    "pl_pair_residual_norm": [_PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _I32, _I32, _F32, _I32,
                              _PTR],
    "pl_rope_maps_write": [_PTR, _PTR, _PTR, _I64, _PTR, _PTR, _PTR, _I32, _PTR, _PTR, _I64, _I64, _I32, _I32, _PTR,
                           _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _PTR, _I32, _PTR, _PTR],
    "pl_diff_combine": [_PTR, _PTR, _I32, _I32, _I32, _I32, _F32, _F32, _F32, _I32, _PTR],
    "pl_short_conv_act": [_PTR, _I64, _PTR, _PTR, _PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _I32, _I32, _PTR],
    "pl_short_conv_single": [_PTR, _I64, _PTR, _PTR, _PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _I32, _I32, _PTR],
    "pl_short_conv_state_strided": [_PTR, _I64, _PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _PTR],
    "pl_gated_delta": [_PTR, _PTR, _PTR, _I64, _PTR, _I64, _PTR, _I64, _PTR, _I64, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR,
                       _PTR, _PTR, _PTR, _I64, _I32, _I32, _I32, _I32, _I32, _I32, _F32, _F32, _F32, _I32, _PTR],
    "pl_moe_route": [_PTR, _I64, _PTR, _PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32,
                     _PTR],
    "pl_moe_up": [_PTR, _I64, _PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _I32, _I32, _PTR],
    "pl_pair_embed": [_PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _I64, _I64, _I32, _I32,
                      _PTR, _PTR],
    "pl_pair_embed_state": [_PTR, _PTR, _PTR, _PTR, _I32, _PTR],
    "pl_norm_rope_mix_write": [_PTR, _PTR, _PTR, _I64, _PTR, _I64, _F32, _PTR, _PTR, _PTR, _PTR, _I32, _PTR, _PTR,
                               _I64, _I64, _I32, _I32, _PTR, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _I32, _PTR,
                               _PTR, _F32, _I32, _PTR, _PTR],
    "pl_moe_gate_up": [_PTR, _I64, _PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _I32, _I32, _PTR],
    "pl_moe_down": [_PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _I32, _I32, _PTR],
    "pl_moe_sort": [_PTR, _I32, _I32, _PTR, _PTR, _PTR, _PTR],
    "pl_moe_gather": [_PTR, _I64, _PTR, _PTR, _I32, _I32, _I32, _I32, _PTR],
    "pl_moe_combine": [_PTR, _PTR, _PTR, _PTR, _PTR, _I32, _I32, _I32, _I32, _PTR],
    "pl_add_layernorm": [_PTR, _PTR, _PTR, _PTR, _F32, _PTR, _PTR, _PTR, _F32, _PTR, _I32, _I32, _I32, _I32, _PTR],
    "pl_gated_act": [_PTR, _PTR, _I32, _I32, _I32, _I32, _PTR],
    "pl_sigmoid_gate": [_PTR, _I64, _PTR, _I64, _I32, _I32, _I32, _PTR],
    "pl_sigmoid_gate_heads": [_PTR, _I64, _PTR, _I64, _I32, _I32, _I32, _I32, _PTR],
    "pl_conv_norm_rope_write": [_PTR, _I64, _PTR, _PTR, _I32, _PTR, _PTR, _I32, _PTR, _PTR, _F32, _PTR, _I32, _I32, _F32,
                                _PTR, _PTR, _PTR, _I32, _PTR, _I64, _PTR, _PTR, _I64, _I64, _I32, _I32, _I32, _I32, _I32,
                                _I32, _I32, _PTR, _PTR],
    "pl_latent_rope_write": [_PTR, _I64, _I32, _I32, _PTR, _I64, _PTR, _I64, _PTR, _F32, _I32, _I32, _PTR, _I32, _F32,
                             _PTR, _PTR, _PTR, _I32, _PTR, _I64, _I32, _I32, _I32, _I32, _PTR, _PTR],
    "pl_sample": [_PTR, _I64, _I32, _I32, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR],
}


def library() -> ctypes.CDLL:
    """The loaded kernel library; builds it on first use."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = build.library_path(build=True)
        lib = ctypes.CDLL(path)
        lib.pl_last_error.restype = ctypes.c_char_p
        lib.pl_abi_version.restype = _I32
        if lib.pl_abi_version() != ABI_VERSION:
            raise KernelError(f"{path}: ABI version {lib.pl_abi_version()} does not match the package's "
                              f"{ABI_VERSION}; delete the build folder and try again")
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _I32
        lib.pl_device_arch.restype = _I32
        lib.pl_attention_decode_scratch_floats.argtypes = [_I32, _I32, _I32, _I32]
        lib.pl_attention_decode_scratch_floats.restype = _I64
        lib.pl_attention_prefill_scratch_floats.argtypes = [_I32, _I32, _I32, _I32]
        lib.pl_attention_prefill_scratch_floats.restype = _I64
        lib.pl_set_overlap.argtypes = [_I32]
        lib.pl_set_overlap.restype = _I32
        if os.environ.get("PULSARLM_B200_OVERLAP", "1") == "0":
            lib.pl_set_overlap(0)
        _lib = lib
    return _lib


def set_overlap(enabled: bool) -> bool:
    """Lets consecutive kernels of a stream overlap (programmatic dependent launch:
    a kernel's set-up and weight loads run under its predecessor's tail). On by
    default; `PULSARLM_B200_OVERLAP=0` starts with it off. Returns the old setting."""
    return bool(library().pl_set_overlap(int(enabled)))


_device_checked = False


def require_device() -> None:
    """Raises unless a CUDA device of compute capability 10.x is current."""
    global _device_checked
    if _device_checked:
        return
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: the engine runs on a B200 (sm_100) only and has no CPU path")
    torch.cuda.init()
    arch = library().pl_device_arch()
    if arch // 10 != 10:
        raise KernelError(f"the kernels are built for sm_100a; the current device is sm_{arch}")
    _device_checked = True


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (torch's; inside a graph capture, the capturing stream).
    Asked through torch's C entry point when it has one: the Python object costs 15 us a
    call, which a step of a few hundred launches notices."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_launches = 0


def launch_count() -> int:
    """How many kernel entry points of this library have been called so far."""
    return _launches


def _call(name: str, *args) -> None:
    global _launches
    _launches += 1
    code = getattr(library(), name)(*args)
    if code != 0:
        raise KernelError(library().pl_last_error().decode("utf-8", "replace"))


def call_native(name: str, *args, launches: int = 1) -> None:
    """Calls an entry point that takes structs and the stream (the caller has checked what
    the structs point at); `launches`: how many of the library's kernels it launches."""
    global _launches
    _launches += launches - 1
    _call(name, *args, _stream())


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {dtype}; the kernels take float32 and bfloat16") from None


def _dev(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must be CUDA tensors")


# ----------------------------------------------------------------------------- ops

def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, status: torch.Tensor | None = None,
          scale: float = 1.0) -> None:
    """out[t] (fp32 [T, H]) = table[tokens[t]] * scale; tokens int32 [T]."""
    _dev(table, tokens, out, status)
    assert table.is_contiguous() and out.is_contiguous() and out.dtype == torch.float32
    assert tokens.dtype == torch.int32 and tokens.is_contiguous()
    vocab, hidden = table.shape
    _call("pl_embed", _p(table), _p(tokens), _p(out), tokens.numel(), hidden, vocab, float(scale), _code(table.dtype),
          _p(status), _stream())


def take_tokens(tokens: torch.Tensor, source: torch.Tensor, ids: torch.Tensor,
                status: torch.Tensor | None = None) -> None:
    """tokens[i] = ids[source[i]] for the rows with source[i] >= 0 (all int32, on the
    device): the tokens of entries that go on from a step whose ids are still being drawn."""
    _dev(tokens, source, ids, status)
    assert tokens.dtype == source.dtype == ids.dtype == torch.int32
    assert tokens.is_contiguous() and source.is_contiguous() and ids.is_contiguous()
    assert source.numel() <= tokens.numel()
    _call("pl_take_tokens", _p(tokens), _p(source), _p(ids), source.numel(), ids.numel(), _p(status), _stream())


def pair_embed(table: torch.Tensor, pairs: torch.Tensor, tokens: torch.Tensor, pos: torch.Tensor, entry: torch.Tensor,
               slots: torch.Tensor, last_token: torch.Tensor, out: torch.Tensor, mul_prev: int, mul_cur: int,
               single_tokens: bool, status: torch.Tensor | None = None) -> None:
    """out[t] (fp32 [T, H]) = table[tokens[t]] + pairs[(before * mul_prev + tokens[t] * mul_cur) mod buckets], with
    pairs [buckets + 1, H] and its last row for a token at position 0. The token before row t is the row above it
    where that is the same entry's, else last_token[slots[entry[t]]] (int32, one per request slot), which afterwards
    holds the entry's last token (single_tokens: every entry brings one token and one launch does both)."""
    _dev(table, pairs, tokens, pos, entry, slots, last_token, out, status)
    assert table.is_contiguous() and pairs.is_contiguous() and out.is_contiguous() and out.dtype == torch.float32
    assert table.dtype == pairs.dtype and table.shape[1] == pairs.shape[1] == out.shape[1] and pairs.shape[0] >= 2
    for t in (tokens, pos, entry, slots, last_token):
        assert t.dtype == torch.int32 and t.is_contiguous()
    n = tokens.numel()
    assert pos.numel() == n and entry.numel() == n and out.shape[0] == n
    vocab, hidden = table.shape
    _call("pl_pair_embed", _p(table), _p(pairs), _p(tokens), _p(pos), _p(entry), _p(slots), _p(last_token), _p(out), n,
          hidden, vocab, pairs.shape[0] - 1, int(mul_prev), int(mul_cur), int(bool(single_tokens)), _code(table.dtype),
          _p(status), _stream())
    if not single_tokens:
        _call("pl_pair_embed_state", _p(tokens), _p(entry), _p(slots), _p(last_token), n, _stream())


NORM_MODES = {"none": 0, "per_head": 1, "whole": 2, "unit_after": 3}


def norm_rope_mix_write(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, v_first: torch.Tensor | None, lam: float,
                        q_out: torch.Tensor, pos: torch.Tensor, entry: torch.Tensor, table: torch.Tensor,
                        k_pool: torch.Tensor, v_pool: torch.Tensor, page_size: int, inv_freq: torch.Tensor | None,
                        rotary: int, mode: str, q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
                        eps: float, status: torch.Tensor | None = None, row_stride: int | None = None,
                        v_first_stride: int | None = None) -> None:
    """q [T, nh, dim], k [T, nkv, dim], v [T, nkv, vdim] (slices of one projection's output: equal row
    strides; `row_stride`, and `v_first_stride` for v_first, name them where a step of one token would hide them:
    the kernel chosen depends on them) are normed (mode: "none", "per_head" with weights fp32 [dim], "whole" over the whole projection with
    weights fp32 [nh * dim] and [nkv * dim], "unit_after": per head, no weights, after the rotation), rotated over
    the first `rotary` columns of every head (inv_freq fp64 [rotary / 2] or None), v mixed with v_first [T, nkv,
    vdim] as (1 - lam) v + lam v_first (None: not), and written: q to q_out [T, nh, row], k and v into the pools
    [pages, nkv, page_size, row], all with zeros past their own columns."""
    _dev(q, k, v, v_first, q_out, pos, entry, table, k_pool, v_pool, inv_freq, q_weight, k_weight, status)
    tokens, n_heads, dim = q.shape
    n_kv, vdim = v.shape[1], v.shape[2]
    row = q_out.shape[2]
    n_pages = k_pool.shape[0]
    assert k.shape == (tokens, n_kv, dim) and v.shape[0] == tokens
    for t_, size in ((q, dim), (k, dim), (v, vdim)):
        assert t_.stride(2) == 1 and t_.stride(1) == size and (tokens == 1 or t_.stride(0) == q.stride(0))
        assert t_.dtype == q.dtype
    assert q_out.shape == (tokens, n_heads, row) and q_out.is_contiguous() and q_out.dtype == q.dtype
    assert k_pool.shape == (n_pages, n_kv, page_size, row) == v_pool.shape and k_pool.dtype == q.dtype == v_pool.dtype
    assert k_pool.stride() == v_pool.stride() and k_pool.stride(3) == 1 and k_pool.stride(2) == row
    if v_first is not None:
        assert v_first.shape == v.shape and v_first.dtype == q.dtype and v_first.stride(2) == 1
        assert v_first.stride(1) == vdim
        v_first_stride = v_first.stride(0) if v_first_stride is None else int(v_first_stride)
    else:
        v_first_stride = 0
    n_q, n_k = (n_heads * dim, n_kv * dim) if mode == "whole" else (dim, dim)
    for w_, n_ in ((q_weight, n_q), (k_weight, n_k)):
        assert w_ is None or (w_.dtype == torch.float32 and w_.numel() == n_ and w_.is_contiguous())
    assert pos.dtype == torch.int32 and entry.dtype == torch.int32 and table.dtype == torch.int32
    assert pos.numel() == tokens and entry.numel() == tokens and table.dim() == 2 and table.is_contiguous()
    if inv_freq is not None:
        assert inv_freq.dtype == torch.float64 and inv_freq.numel() == rotary // 2 and inv_freq.is_contiguous()
    _call("pl_norm_rope_mix_write", _p(q), _p(k), _p(v), q.stride(0) if row_stride is None else int(row_stride),
          _p(v_first), v_first_stride, float(lam),
          _p(q_out), _p(pos), _p(entry), _p(table), table.shape[1], _p(k_pool), _p(v_pool), k_pool.stride(0),
          k_pool.stride(1), page_size, n_pages, _p(inv_freq), int(rotary) if inv_freq is not None else 0, tokens,
          n_heads, n_kv, dim, vdim, row, NORM_MODES[mode], _p(q_weight), _p(k_weight), float(eps), _code(q.dtype),
          _p(status), _stream())


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: torch.Tensor | None = None) -> None:
    """x fp32 [T, H] residual stream; x += delta (when rows is None); out = norm(x + delta) * weight.
    With rows (int32 [R]), output row r is made from source row rows[r] and x is left as it was."""
    _dev(x, delta, weight, out, rows)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    hidden = x.shape[-1]
    n_rows = rows.numel() if rows is not None else x.shape[0]
    assert out.shape == (n_rows, hidden) and weight.shape == (hidden,) and weight.is_contiguous()
    if delta is not None:
        assert delta.shape == x.shape and delta.dtype == out.dtype and delta.is_contiguous()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.is_contiguous()
    _call("pl_add_rmsnorm", _p(x), _p(delta), _p(weight), _code(weight.dtype), _p(out), _p(rows), n_rows, hidden,
          float(eps), _code(out.dtype), _stream())


def add_normed_rmsnorm(x: torch.Tensor, y: torch.Tensor, y_weight: torch.Tensor, mult: float, y_eps: float,
                       weight: torch.Tensor | None, eps: float, out: torch.Tensor | None,
                       rows: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                       conv: tuple | None = None) -> None:
    """x fp32 [T, H] += mult * rmsnorm(y + bias) * y_weight (in place unless rows is given); out =
    rmsnorm(x) * weight when out is given. y, bias and out in the engine's dtype, the weights fp32.
    With rows (int32 [R]), output row r is made from source row rows[r] and x is left as it was.
    conv = (weight fp32 [H, taps], state [slots, taps - 1, H], slots int32 [T]): in a step whose
    entries bring one token each (row t is entry t), the short convolution over time rides along:
    out = short_conv(normed row) and every entry's state slot moves on (see short_conv)."""
    _dev(x, y, y_weight, weight, out, rows, bias)
    conv_weight = conv_state = conv_slots = None
    taps = 0
    if conv is not None:
        conv_weight, conv_state, conv_slots = conv
        _dev(conv_weight, conv_state, conv_slots)
        taps = conv_weight.shape[1]
        assert rows is None and out is not None and conv_weight.dtype == torch.float32 and conv_weight.is_contiguous()
        assert conv_weight.shape[0] == x.shape[-1] and conv_slots.dtype == torch.int32 and conv_slots.numel() >= x.shape[0]
        assert conv_state.dtype == y.dtype and conv_state.is_contiguous() and conv_state.shape[1:] == (taps - 1, x.shape[-1])
    hidden = x.shape[-1]
    assert x.dtype == torch.float32 and x.is_contiguous() and y.shape == x.shape and y.is_contiguous()
    assert y_weight.dtype == torch.float32 and y_weight.shape == (hidden,) and y_weight.is_contiguous()
    n_rows = rows.numel() if rows is not None else x.shape[0]
    if out is not None:
        assert weight is not None and weight.dtype == torch.float32 and weight.shape == (hidden,)
        assert weight.is_contiguous() and out.shape == (n_rows, hidden) and out.is_contiguous() and out.dtype == y.dtype
    if bias is not None:
        assert bias.dtype == y.dtype and bias.shape == (hidden,) and bias.is_contiguous()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.is_contiguous()
    _call("pl_add_normed_rmsnorm", _p(x), _p(y), _p(bias), _p(y_weight), float(mult), float(y_eps), _p(weight),
          float(eps), _p(out), _p(rows), n_rows, hidden, _p(conv_weight), _p(conv_state), _p(conv_slots), taps,
          _code(y.dtype), _stream())


BIAS_ACT = {"none": 0, "relu2": 1, "tanh": 2}


def bias_act(x: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor, act: str = "none") -> None:
    """out = act(x + bias) over [T, N]; act "none", "relu2" (the square of relu) or "tanh". x may be
    columns of a wider matrix (row stride free); out is dense and may be x."""
    _dev(x, bias, out)
    tokens, width = x.shape
    assert out.shape == x.shape and out.dtype == x.dtype and x.stride(1) == 1 and out.is_contiguous()
    if bias is not None:
        assert bias.shape == (width,) and bias.dtype == x.dtype and bias.is_contiguous()
    _call("pl_bias_act", _p(x), x.stride(0) if tokens > 1 else width, _p(bias), _p(out), tokens, width, BIAS_ACT[act],
          _code(x.dtype), _stream())


def short_conv(h: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, entry: torch.Tensor, slots: torch.Tensor,
               out: torch.Tensor) -> None:
    """out = h + causal convolution of h over time per channel; h, out [T, W], weight fp32 [W, taps],
    state [slots, taps - 1, W] the inputs before this step's rows (read only)."""
    _dev(h, weight, state, entry, slots, out)
    tokens, width = h.shape
    taps = weight.shape[1]
    assert weight.dtype == torch.float32 and weight.shape == (width, taps) and weight.is_contiguous()
    assert h.is_contiguous() and out.is_contiguous() and out.shape == h.shape and out.dtype == h.dtype == state.dtype
    assert state.is_contiguous() and state.shape[1:] == (taps - 1, width) and out.data_ptr() != h.data_ptr()
    assert entry.dtype == torch.int32 and slots.dtype == torch.int32 and entry.numel() == tokens
    _call("pl_short_conv", _p(h), _p(weight), _p(state), _p(entry), _p(slots), _p(out), tokens, width, taps,
          _code(h.dtype), _stream())


def short_conv_state(h: torch.Tensor, entry: torch.Tensor, slots: torch.Tensor, state: torch.Tensor) -> None:
    """state[slot] <- the last taps - 1 inputs of each entry's sequence after this step's rows h."""
    _dev(h, entry, slots, state)
    tokens, width = h.shape
    taps = state.shape[1] + 1
    assert h.is_contiguous() and state.is_contiguous() and state.dtype == h.dtype and state.shape[2] == width
    _call("pl_short_conv_state", _p(h), _p(entry), _p(slots), _p(state), tokens, width, taps, _code(h.dtype),
          _stream())


def delta_rule(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, a_pre: torch.Tensor,
               w_pre: torch.Tensor, w0: torch.Tensor, a0: torch.Tensor, norm: torch.Tensor, state: torch.Tensor,
               first_rows: torch.Tensor, counts: torch.Tensor, slots: torch.Tensor, out: torch.Tensor, n_heads: int,
               dim: int, decay_scale: float, unit_eps: float, eps: float) -> None:
    """The generalized delta rule over each entry's rows in order (see csrc/delta_rule.cu). r, k, v,
    g, a_pre [T, heads * dim] share one row stride; state fp32 [slots, heads, dim, dim] is updated."""
    _dev(r, k, v, g, a_pre, w_pre, w0, a0, norm, state, first_rows, counts, slots, out)
    width = n_heads * dim
    stride = r.stride(0)
    for t in (r, k, v, g, a_pre):
        assert t.shape[1] == width and t.stride(1) == 1 and t.stride(0) == stride and t.dtype == out.dtype
    assert w_pre.shape[1] == width and w_pre.stride(1) == 1 and w_pre.dtype == out.dtype
    for t in (w0, a0, norm):
        assert t.dtype == torch.float32 and t.shape == (width,) and t.is_contiguous()
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (n_heads, dim, dim)
    assert out.shape[1] == width and out.stride(1) == 1
    n_entries = first_rows.numel()
    tokens = r.shape[0]
    assert counts.numel() == n_entries and slots.numel() >= n_entries
    o_raw = torch.empty((tokens, width), dtype=torch.float32, device=out.device)  # (the scan's output before the norm)
    _call("pl_delta_rule", _p(r), _p(k), _p(v), _p(g), _p(a_pre), stride, _p(w_pre), w_pre.stride(0), _p(w0), _p(a0),
          _p(norm), _p(state), _p(first_rows), _p(counts), _p(slots), _p(o_raw), _p(out), out.stride(0), tokens,
          n_entries, n_heads, dim, float(decay_scale), float(unit_eps), float(eps), _code(out.dtype), _stream())
    global _launches
    _launches += 1  # (two kernels)


def pair_residual_norm(x: torch.Tensor, y1: torch.Tensor | None, s1: torch.Tensor | None, y2: torch.Tensor | None,
                       s2: torch.Tensor | None, also: torch.Tensor | None, w1: torch.Tensor | None,
                       w2: torch.Tensor | None, h1: torch.Tensor | None, h2: torch.Tensor | None, eps: float,
                       rows: torch.Tensor | None = None) -> None:
    """x += s1 * y1 + s2 * y2 + also (each optional), then h1 = rmsnorm(x) * w1 and h2 = rmsnorm(x) * w2
    (see csrc/parallel_norm.cu). x fp32 [T, H]; y1, y2, h1, h2 in the engine's dtype; s1, s2, w1, w2, also
    fp32. With `rows` only those rows are normed and x is left as it is."""
    _dev(x, y1, s1, y2, s2, also, w1, w2, h1, h2, rows)
    tokens, hidden = x.shape
    outs = [h for h in (h1, h2) if h is not None]
    assert outs and x.dtype == torch.float32 and x.is_contiguous()
    dtype = outs[0].dtype
    n_rows = rows.numel() if rows is not None else tokens
    for y in (y1, y2):
        assert y is None or (y.shape == (tokens, hidden) and y.is_contiguous() and y.dtype == dtype)
    for v in (s1, s2, w1, w2):
        assert v is None or (v.dtype == torch.float32 and v.shape == (hidden,) and v.is_contiguous())
    assert also is None or (also.dtype == torch.float32 and also.shape == x.shape and also.is_contiguous())
    for h in outs:
        assert h.shape == (n_rows, hidden) and h.is_contiguous() and h.dtype == dtype
    assert rows is None or rows.dtype == torch.int32
    _call("pl_pair_residual_norm", _p(x), _p(y1), _p(s1), _p(y2), _p(s2), _p(also), _p(w1), _p(w2), _p(h1), _p(h2),
          _p(rows), n_rows, hidden, float(eps), _code(dtype), _stream())


def rope_maps_write(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos: torch.Tensor, entry: torch.Tensor,
                    table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_size: int,
                    inv_freq: torch.Tensor | None, rotary: int, n_heads: int, n_kv_heads: int, maps: int, dim: int,
                    vdim: int, q_out: torch.Tensor, status: torch.Tensor | None) -> None:
    """Lays the score maps of every head out as heads of their own, rotates q and k (neighbouring
    pairs within each map's first `rotary` columns) and writes k and v rows into their pages (see
    csrc/rope_maps.cu). q [T, heads * maps * dim], k [T, kv_heads * maps * dim], v [T, kv_heads * vdim]
    with one row stride; q_out [T, heads * maps, padded]; pools [pages, kv_heads, page_size, padded]."""
    _dev(q, k, v, pos, entry, table, k_pool, v_pool, inv_freq, q_out, status)
    tokens = q.shape[0]
    padded = q_out.shape[2]
    assert q.shape[1] == n_heads * maps * dim and k.shape[1] == n_kv_heads * maps * dim and v.shape[1] == n_kv_heads * vdim
    assert q.stride(1) == k.stride(1) == v.stride(1) == 1 and q.stride(0) == k.stride(0) == v.stride(0)
    assert q_out.is_contiguous() and q_out.shape == (tokens, n_heads * maps, padded) and q_out.dtype == q.dtype
    assert k_pool.dtype == q.dtype and k_pool.shape[1:] == (n_kv_heads, page_size, padded) and v_pool.shape == k_pool.shape
    assert k_pool.stride() == v_pool.stride() and k_pool.stride(3) == 1 and k_pool.stride(2) == padded
    assert inv_freq is None or (inv_freq.dtype == torch.float64 and inv_freq.numel() == rotary // 2)
    _call("pl_rope_maps_write", _p(q), _p(k), _p(v), q.stride(0), _p(pos), _p(entry), _p(table), table.shape[1],
          _p(k_pool), _p(v_pool), k_pool.stride(0), k_pool.stride(1), page_size, k_pool.shape[0], _p(inv_freq),
          rotary if inv_freq is not None else 0, tokens, n_heads, n_kv_heads, maps, dim, vdim, padded, _p(q_out),
          _code(q.dtype), _p(status), _stream())


def diff_combine(a: torch.Tensor, out: torch.Tensor, n_heads: int, vdim: int, lam: float, eps: float,
                 mult: float) -> None:
    """out[t, h] = mult * unit_rms(a[t, h, 0] - lam * a[t, h, 1]) over the first vdim columns; a [T, heads * 2,
    padded], out [T, heads * vdim]."""
    _dev(a, out)
    tokens, rows, padded = a.shape
    assert rows == 2 * n_heads and a.is_contiguous() and out.is_contiguous() and out.shape == (tokens, n_heads * vdim)
    assert a.dtype == out.dtype
    _call("pl_diff_combine", _p(a), _p(out), tokens, n_heads, vdim, padded, float(lam), float(eps), float(mult),
          _code(a.dtype), _stream())


def short_conv_act(h: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, entry: torch.Tensor,
                   slots: torch.Tensor, out: torch.Tensor, residual: bool, act: str) -> None:
    """out = act(conv(h) [+ h]) per channel over time; h [T, W] may be columns of a wider matrix (unit column
    stride); act "none" or "silu". The state [slots, taps - 1, W] is read only."""
    _dev(h, weight, state, entry, slots, out)
    tokens, width = h.shape
    taps = weight.shape[1]
    assert weight.dtype == torch.float32 and weight.shape == (width, taps) and weight.is_contiguous()
    assert h.stride(1) == 1 and out.is_contiguous() and out.shape == h.shape and out.dtype == h.dtype == state.dtype
    assert state.is_contiguous() and state.shape[1:] == (taps - 1, width) and out.data_ptr() != h.data_ptr()
    _call("pl_short_conv_act", _p(h), h.stride(0) if tokens > 1 else width, _p(weight), _p(state), _p(entry),
          _p(slots), _p(out), tokens, width, taps, int(bool(residual)), {"none": 0, "silu": 1}[act], _code(h.dtype),
          _stream())


def short_conv_single(h: torch.Tensor, weight: torch.Tensor, state: torch.Tensor, entry: torch.Tensor,
                      slots: torch.Tensor, out: torch.Tensor, residual: bool, act: str) -> bool:
    """short_conv_act and the state's update in one launch, for a step in which every entry brings
    exactly one row. False (nothing launched) when the sizes are not the ones this form takes."""
    _dev(h, weight, state, entry, slots, out)
    tokens, width = h.shape
    taps = weight.shape[1]
    assert weight.dtype == torch.float32 and weight.shape == (width, taps) and weight.is_contiguous()
    assert h.stride(1) == 1 and out.is_contiguous() and out.shape == h.shape and out.dtype == h.dtype == state.dtype
    assert state.is_contiguous() and state.shape[1:] == (taps - 1, width) and out.data_ptr() != h.data_ptr()
    global _launches
    code = library().pl_short_conv_single(_p(h), h.stride(0) if tokens > 1 else width, _p(weight), _p(state),
                                          _p(entry), _p(slots), _p(out), tokens, width, taps, int(bool(residual)),
                                          {"none": 0, "silu": 1}[act], _code(h.dtype), _stream())
    if code == 1:
        return False
    if code != 0:
        raise KernelError(library().pl_last_error().decode("utf-8", "replace"))
    _launches += 1
    return True


def short_conv_state_strided(h: torch.Tensor, entry: torch.Tensor, slots: torch.Tensor, state: torch.Tensor) -> None:
    """short_conv_state for rows of h that are columns of a wider matrix."""
    _dev(h, entry, slots, state)
    tokens, width = h.shape
    taps = state.shape[1] + 1
    assert h.stride(1) == 1 and state.is_contiguous() and state.dtype == h.dtype and state.shape[2] == width
    _call("pl_short_conv_state_strided", _p(h), h.stride(0) if tokens > 1 else width, _p(entry), _p(slots), _p(state),
          tokens, width, taps, _code(h.dtype), _stream())


def gated_delta(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, b_pre: torch.Tensor, a_pre: torch.Tensor,
                gate_pre: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor, norm: torch.Tensor,
                state: torch.Tensor, first_rows: torch.Tensor, counts: torch.Tensor, slots: torch.Tensor,
                out: torch.Tensor, n_heads: int, qk_heads: int, dim: int, vdim: int, unit_eps: float, q_scale: float,
                eps: float) -> None:
    """The gated delta rule with a decay per key channel over each entry's rows in order (see
    csrc/gated_delta.cu). q, k [T, qk_heads * dim] and v [T, heads * vdim] share one row stride; state fp32
    [slots, heads, dim, vdim] is updated."""
    _dev(q, k, v, b_pre, a_pre, gate_pre, a_log, dt_bias, norm, state, first_rows, counts, slots, out)
    tokens = q.shape[0]
    assert q.shape[1] == k.shape[1] == qk_heads * dim and v.shape[1] == n_heads * vdim
    assert q.stride(0) == k.stride(0) == v.stride(0) and q.stride(1) == k.stride(1) == v.stride(1) == 1
    for t, width in ((b_pre, n_heads), (a_pre, n_heads * dim), (gate_pre, n_heads * vdim), (out, n_heads * vdim)):
        assert t.shape == (tokens, width) and t.stride(1) == 1 and t.dtype == q.dtype
    assert a_log.dtype == dt_bias.dtype == norm.dtype == torch.float32
    assert a_log.shape == (n_heads,) and dt_bias.shape == (n_heads * dim,) and norm.shape == (vdim,)
    assert a_log.is_contiguous() and dt_bias.is_contiguous() and norm.is_contiguous()
    assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1:] == (n_heads, dim, vdim)
    n_entries = first_rows.numel()
    assert counts.numel() == n_entries and slots.numel() >= n_entries
    o_raw = torch.empty((tokens, n_heads * vdim), dtype=torch.float32, device=out.device)

    def stride(t):
        return t.stride(0) if tokens > 1 else t.shape[1]

    _call("pl_gated_delta", _p(q), _p(k), _p(v), stride(q), _p(b_pre), stride(b_pre), _p(a_pre), stride(a_pre),
          _p(gate_pre), stride(gate_pre), _p(a_log), _p(dt_bias), _p(norm), _p(state), _p(first_rows), _p(counts),
          _p(slots), _p(o_raw), _p(out), stride(out), tokens, n_entries, n_heads, qk_heads, dim, vdim, float(unit_eps),
          float(q_scale), float(eps), _code(out.dtype), _stream())
    global _launches
    _launches += 1  # (two kernels)


def moe_route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor | None, top: int, n_groups: int,
              keep: int, sigmoid_scores: bool = False, group_top: int = 1,
              renormalise: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """(ids int32 [T, top], weights fp32 [T, top]) of the experts each token's router chooses (see csrc/moe.cu).
    sigmoid_scores: scores are sigmoids of the logits instead of their softmax; group_top: how many of a
    group's largest choice scores add up to its score; renormalise: the chosen scores over their sum."""
    _dev(h, router, correction)
    tokens, hidden = h.shape
    n_experts = router.shape[0]
    assert router.dtype == torch.float32 and router.shape == (n_experts, hidden) and router.is_contiguous()
    assert correction is None or (correction.dtype == torch.float32 and correction.shape == (n_experts,))
    assert h.stride(1) == 1
    ids = torch.empty((tokens, top), dtype=torch.int32, device=h.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=h.device)
    _call("pl_moe_route", _p(h), h.stride(0) if tokens > 1 else hidden, _p(router), _p(correction), _p(ids),
          _p(weights), tokens, hidden, n_experts, top, n_groups, keep, int(bool(sigmoid_scores)), int(group_top),
          int(bool(renormalise)), _code(h.dtype), _stream())
    return ids, weights


def moe_up(h: torch.Tensor, up: torch.Tensor, ids: torch.Tensor, act: torch.Tensor) -> None:
    """act[t * top + j] = relu(Wu h_t)^2 with the weights of expert ids[t, j]; up [E, ff, H] (experts without a gate)."""
    _dev(h, up, ids, act)
    tokens, hidden = h.shape
    n_experts, ff, _ = up.shape
    top = ids.shape[1]
    assert up.is_contiguous() and up.shape[2] == hidden and up.dtype == h.dtype == act.dtype
    assert act.is_contiguous() and act.shape == (tokens * top, ff) and ids.is_contiguous() and h.stride(1) == 1
    _call("pl_moe_up", _p(h), h.stride(0) if tokens > 1 else hidden, _p(up), _p(ids), _p(act), tokens, hidden, ff, top,
          n_experts, _code(h.dtype), _stream())


def moe_gate_up(h: torch.Tensor, gate_up: torch.Tensor, ids: torch.Tensor, act: torch.Tensor) -> None:
    """act[t * top + j] = silu(Wg h_t) * (Wu h_t) with the weights of expert ids[t, j]; gate_up [E, 2 * ff, H]."""
    _dev(h, gate_up, ids, act)
    tokens, hidden = h.shape
    n_experts, two_ff, _ = gate_up.shape
    top = ids.shape[1]
    assert gate_up.is_contiguous() and gate_up.shape[2] == hidden and gate_up.dtype == h.dtype == act.dtype
    assert act.is_contiguous() and act.shape == (tokens * top, two_ff // 2) and ids.is_contiguous() and h.stride(1) == 1
    _call("pl_moe_gate_up", _p(h), h.stride(0) if tokens > 1 else hidden, _p(gate_up), _p(ids), _p(act), tokens,
          hidden, two_ff // 2, top, n_experts, _code(h.dtype), _stream())


def moe_down(act: torch.Tensor, down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
             also: torch.Tensor | None, out: torch.Tensor) -> None:
    """out[t] = sum_j weights[t, j] * W_down,ids[t, j] act[t * top + j] + also[t]; down [E, H, ff]."""
    _dev(act, down, ids, weights, also, out)
    tokens, hidden = out.shape
    n_experts, _, ff = down.shape
    top = ids.shape[1]
    assert down.is_contiguous() and down.shape[1] == hidden and down.dtype == act.dtype == out.dtype
    assert act.is_contiguous() and act.shape == (tokens * top, ff) and out.is_contiguous()
    assert weights.dtype == torch.float32 and weights.is_contiguous() and weights.shape == ids.shape
    assert also is None or (also.shape == out.shape and also.is_contiguous() and also.dtype == out.dtype)
    _call("pl_moe_down", _p(act), _p(down), _p(ids), _p(weights), _p(also), _p(out), tokens, hidden, ff, top,
          n_experts, _code(out.dtype), _stream())


def moe_sort(ids: torch.Tensor, n_experts: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The (token, expert) pairs in expert order: (ends int32 [E]: the row after each expert's last,
    row_of_pair int32 [pairs], pair_of_row int32 [pairs])."""
    _dev(ids)
    pairs = ids.numel()
    assert ids.dtype == torch.int32 and ids.is_contiguous()
    ends = torch.empty(n_experts, dtype=torch.int32, device=ids.device)
    row_of_pair = torch.empty(pairs, dtype=torch.int32, device=ids.device)
    pair_of_row = torch.empty(pairs, dtype=torch.int32, device=ids.device)
    _call("pl_moe_sort", _p(ids), pairs, n_experts, _p(ends), _p(row_of_pair), _p(pair_of_row), _stream())
    return ends, row_of_pair, pair_of_row


def moe_gather(x: torch.Tensor, pair_of_row: torch.Tensor, top: int) -> torch.Tensor:
    """Rows of x in expert order: out[r] = x[pair_of_row[r] // top]."""
    _dev(x, pair_of_row)
    assert x.stride(1) == 1
    pairs = pair_of_row.numel()
    out = torch.empty((pairs, x.shape[1]), dtype=x.dtype, device=x.device)
    _call("pl_moe_gather", _p(x), x.stride(0) if x.shape[0] > 1 else x.shape[1], _p(pair_of_row), _p(out), pairs,
          x.shape[1], top, _code(x.dtype), _stream())
    return out


def moe_combine(y: torch.Tensor, row_of_pair: torch.Tensor, weights: torch.Tensor, also: torch.Tensor | None,
                out: torch.Tensor) -> None:
    """out[t] = sum_j weights[t, j] * y[row_of_pair[t * top + j]] + also[t]."""
    _dev(y, row_of_pair, weights, also, out)
    tokens, hidden = out.shape
    top = weights.shape[1]
    assert y.is_contiguous() and y.shape == (tokens * top, hidden) and y.dtype == out.dtype and out.is_contiguous()
    assert weights.dtype == torch.float32 and weights.is_contiguous()
    assert also is None or (also.shape == out.shape and also.is_contiguous() and also.dtype == out.dtype)
    _call("pl_moe_combine", _p(y), _p(row_of_pair), _p(weights), _p(also), _p(out), tokens, hidden, top,
          _code(out.dtype), _stream())


def norm_write_paged(z: torch.Tensor, weight: torch.Tensor, eps: float, pos: torch.Tensor, entry: torch.Tensor,
                     table: torch.Tensor, pool: torch.Tensor, page_size: int,
                     status: torch.Tensor | None = None) -> None:
    """pool[page of (entry, pos)] <- rmsnorm(z) * weight; z [T, rank] (row stride free), weight fp32
    [rank], pool [pages, 1, page_size, rank]."""
    _dev(z, weight, pos, entry, table, pool, status)
    tokens, rank = z.shape
    assert z.stride(1) == 1 and weight.dtype == torch.float32 and weight.shape == (rank,) and weight.is_contiguous()
    assert pool.dtype == z.dtype and pool.shape[1:] == (1, page_size, rank) and pool.stride(3) == 1
    assert pool.stride(2) == rank and table.dim() == 2 and table.is_contiguous()
    _call("pl_norm_write_paged", _p(z), z.stride(0), _p(weight), float(eps), _p(pos), _p(entry), _p(table),
          table.shape[1], _p(pool), pool.stride(0), page_size, pool.shape[0], rank, tokens, _code(z.dtype),
          _p(status), _stream())


def add_layernorm(x: torch.Tensor, y: torch.Tensor | None, y_weight: torch.Tensor | None,
                  y_bias: torch.Tensor | None, y_eps: float, out: torch.Tensor | None,
                  weight: torch.Tensor | None = None, bias: torch.Tensor | None = None, eps: float = 0.0,
                  rows: torch.Tensor | None = None) -> None:
    """x fp32 [T, H] += layernorm(y) * y_weight + y_bias (in place unless rows is given; nothing when
    y is None); then out = the stream rounded to the engine's dtype, or with weight and bias its
    layer norm. y and out in the engine's dtype, weights and biases fp32. With rows (int32 [R]),
    output row r is made from source row rows[r] and x is left as it was."""
    _dev(x, y, y_weight, y_bias, out, weight, bias, rows)
    hidden = x.shape[-1]
    assert x.dtype == torch.float32 and x.is_contiguous()
    dtype = out.dtype if out is not None else y.dtype
    if y is not None:
        assert y.shape == x.shape and y.is_contiguous() and y.dtype == dtype
        for v in (y_weight, y_bias):
            assert v.dtype == torch.float32 and v.shape == (hidden,) and v.is_contiguous()
    n_rows = rows.numel() if rows is not None else x.shape[0]
    if out is not None:
        assert out.shape == (n_rows, hidden) and out.is_contiguous()
    if weight is not None:
        for v in (weight, bias):
            assert v.dtype == torch.float32 and v.shape == (hidden,) and v.is_contiguous()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.is_contiguous()
    _call("pl_add_layernorm", _p(x), _p(y), _p(y_weight), _p(y_bias), float(y_eps), _p(out), _p(weight), _p(bias),
          float(eps), _p(rows), n_rows, hidden, int(weight is not None), _code(dtype), _stream())


GATED_ACT = {"silu": 0, "gelu_tanh": 1}


def gated_act(gate_up: torch.Tensor, out: torch.Tensor, act: str) -> None:
    """out[t, i] = act(gate_up[t, i]) * gate_up[t, I + i]; act "silu" or "gelu_tanh" (the tanh form)."""
    _dev(gate_up, out)
    tokens, two_i = gate_up.shape
    assert two_i % 2 == 0 and out.shape == (tokens, two_i // 2) and out.dtype == gate_up.dtype
    assert gate_up.is_contiguous() and out.is_contiguous()
    _call("pl_gated_act", _p(gate_up), _p(out), tokens, two_i // 2, GATED_ACT[act], _code(out.dtype), _stream())


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor) -> None:
    """x[t, i] *= sigmoid(gate[t, i]) in place; both [T, W] with free row strides (columns of wider matrices)."""
    _dev(x, gate)
    tokens, width = x.shape
    assert gate.shape == x.shape and gate.dtype == x.dtype and x.stride(1) == 1 and gate.stride(1) == 1
    _call("pl_sigmoid_gate", _p(x), x.stride(0) if tokens > 1 else width, _p(gate),
          gate.stride(0) if tokens > 1 else width, tokens, width, _code(x.dtype), _stream())


def sigmoid_gate_heads(x: torch.Tensor, gate: torch.Tensor) -> None:
    """x[t, h, :] *= sigmoid(gate[t, h]) in place; x [T, nh, row] (rows of a head dense, row stride free), gate
    [T, nh] logits (row stride free)."""
    _dev(x, gate)
    tokens, n_heads, row = x.shape
    assert gate.shape == (tokens, n_heads) and gate.dtype == x.dtype and gate.stride(1) == 1
    assert x.stride(2) == 1 and x.stride(1) == row
    _call("pl_sigmoid_gate_heads", _p(x), x.stride(0) if tokens > 1 else n_heads * row, _p(gate),
          gate.stride(0) if tokens > 1 else n_heads, tokens, n_heads, row, _code(x.dtype), _stream())


def conv_norm_rope_write(proj: torch.Tensor, bias: torch.Tensor | None, conv_weight: torch.Tensor | None,
                         conv_state: torch.Tensor | None, slots: torch.Tensor | None, update_state: bool,
                         q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, eps: float,
                         inv_freq: torch.Tensor | None, rotary: int, interleaved: bool, amplitude: float,
                         pos: torch.Tensor, entry: torch.Tensor, table: torch.Tensor, q_out: torch.Tensor,
                         k_pool: torch.Tensor, v_pool: torch.Tensor, page_size: int, n_heads: int, n_kv: int,
                         head_dim: int, status: torch.Tensor | None = None) -> None:
    """From a token's projected q and k channels (proj [T, (n_heads + n_kv) * head_dim], columns of a
    wider matrix allowed) to the rotated query rows q_out [T, n_heads * head_dim] and the token's
    page: bias, causal convolution over time (conv_weight fp32 [channels, taps], conv_state [slots,
    taps - 1, channels] the projected rows before this step's), one RMS norm over all q channels and
    one over all k channels (q_norm, k_norm fp32), rotation of the first `rotary` columns of every
    head (interleaved: neighbouring pairs; else halves), K page <- rotated normed key, V page <- the
    filtered key before norm and rotation. update_state: every entry brings one token and its slot
    moves on in the same launch."""
    _dev(proj, bias, conv_weight, conv_state, slots, q_norm, k_norm, inv_freq, pos, entry, table, q_out, k_pool,
         v_pool, status)
    tokens, channels = proj.shape
    q_width, k_width = n_heads * head_dim, n_kv * head_dim
    assert channels == q_width + k_width and proj.stride(1) == 1 and q_out.shape == (tokens, q_width)
    assert q_out.stride(1) == 1 and q_out.dtype == proj.dtype == k_pool.dtype == v_pool.dtype
    taps = 1
    if conv_weight is not None:
        taps = conv_weight.shape[1]
        assert conv_weight.dtype == torch.float32 and conv_weight.shape == (channels, taps) and conv_weight.is_contiguous()
    if taps > 1:
        assert conv_state.dtype == proj.dtype and conv_state.is_contiguous() and conv_state.shape[1:] == (taps - 1, channels)
        assert slots.dtype == torch.int32
    for v, n in ((bias, channels), (q_norm, q_width), (k_norm, k_width)):
        assert v is None or (v.dtype == torch.float32 and v.shape == (n,) and v.is_contiguous())
    if rotary:
        assert inv_freq.dtype == torch.float64 and inv_freq.numel() == rotary // 2 and inv_freq.is_contiguous()
    n_pages = k_pool.shape[0]
    assert k_pool.shape == (n_pages, n_kv, page_size, head_dim) == v_pool.shape and k_pool.stride() == v_pool.stride()
    assert k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim and table.dim() == 2 and table.is_contiguous()
    assert pos.dtype == torch.int32 and entry.dtype == torch.int32 and table.dtype == torch.int32
    _call("pl_conv_norm_rope_write", _p(proj), proj.stride(0) if tokens > 1 else channels, _p(bias), _p(conv_weight),
          taps, _p(conv_state) if taps > 1 else None, _p(slots), int(bool(update_state)), _p(q_norm), _p(k_norm),
          float(eps), _p(inv_freq), int(rotary), int(bool(interleaved)), float(amplitude), _p(pos), _p(entry),
          _p(table), table.shape[1], _p(q_out), q_out.stride(0) if tokens > 1 else q_width, _p(k_pool), _p(v_pool),
          k_pool.stride(0), k_pool.stride(1), page_size, n_pages, tokens, n_heads, n_kv, head_dim,
          _code(proj.dtype), _p(status), _stream())


def latent_rope_write(q: torch.Tensor, q_out: torch.Tensor, z: torch.Tensor | None, weight: torch.Tensor | None,
                      eps: float, rank: int, rot: int, inv_freq: torch.Tensor | None, interleaved: bool,
                      amplitude: float, pos: torch.Tensor, entry: torch.Tensor, table: torch.Tensor,
                      pool: torch.Tensor, page_size: int, status: torch.Tensor | None = None) -> None:
    """The rows a latent-attention layer with a rotated key part caches, and the rotated part of its
    queries. q [T, nh, dim + rot] (the last rot columns of every head are rotated into q_out [T, nh,
    rank + rot] at columns rank...); z [T, rank + rot] (row stride free; None: nothing is cached):
    pool row <- [rmsnorm(z[:rank]) * weight | rotate(z[rank:])]; pool [pages, 1, page_size, rank + rot]."""
    _dev(q, q_out, z, weight, inv_freq, pos, entry, table, pool, status)
    tokens, n_heads, q_row = q.shape
    dim = q_row - rot
    assert dim >= 0 and q.stride(2) == 1 and q.stride(1) == q_row and q_out.shape == (tokens, n_heads, rank + rot)
    assert q_out.stride(2) == 1 and q_out.stride(1) == rank + rot and q_out.dtype == q.dtype == pool.dtype
    if z is not None:
        assert z.shape == (tokens, rank + rot) and z.stride(1) == 1 and z.dtype == q.dtype
        assert weight.dtype == torch.float32 and weight.shape == (rank,) and weight.is_contiguous()
    if rot:
        assert inv_freq.dtype == torch.float64 and inv_freq.numel() == rot // 2 and inv_freq.is_contiguous()
    assert pool.shape[1:] == (1, page_size, rank + rot) and pool.stride(3) == 1 and pool.stride(2) == rank + rot
    assert table.dim() == 2 and table.is_contiguous() and table.dtype == torch.int32
    _call("pl_latent_rope_write", _p(q), q.stride(0), n_heads, dim, _p(q_out), q_out.stride(0), _p(z),
          z.stride(0) if z is not None else 0, _p(weight), float(eps), rank, rot, _p(inv_freq),
          int(bool(interleaved)), float(amplitude), _p(pos), _p(entry), _p(table), table.shape[1], _p(pool),
          pool.stride(0), page_size, pool.shape[0], tokens, _code(q.dtype), _p(status), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _dev(gate_up, out)
    tokens, two_i = gate_up.shape
    assert two_i % 2 == 0 and out.shape == (tokens, two_i // 2) and out.dtype == gate_up.dtype
    assert gate_up.is_contiguous() and out.is_contiguous()
    _call("pl_swiglu", _p(gate_up), _p(out), tokens, two_i // 2, _code(out.dtype), _stream())


def fill_random(out: torch.Tensor, seed: int, tensor_hash: int, scale: float, offset: float = 0.0) -> None:
    """out = offset + scale * noise(seed, tensor_hash, element index): random weights drawn in
    place, the same bits as the host core draws (weights/random_init.py)."""
    _dev(out)
    assert out.is_contiguous()
    _call("pl_fill_random", _p(out), out.numel(), _code(out.dtype), seed, tensor_hash, float(scale), float(offset),
          _stream())


def bf16_to_f32(src: torch.Tensor, dst: torch.Tensor) -> None:
    _dev(src, dst)
    assert src.dtype == torch.bfloat16 and dst.dtype == torch.float32 and src.numel() == dst.numel()
    assert src.is_contiguous() and dst.is_contiguous()
    _call("pl_bf16_to_f32", _p(src), _p(dst), src.numel(), _stream())


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out[M, N] (+)= a[M, K] @ w[N, K]^T in true fp32 (CUDA-core FMA)."""
    _dev(a, w, out)
    assert a.dtype == w.dtype == out.dtype == torch.float32
    assert a.dim() == 2 and w.dim() == 2 and out.dim() == 2
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and out.shape == (m, n)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _call("pl_gemm_f32", _p(a), _p(w), _p(out), m, n, k, a.stride(0) if m > 1 else k, w.stride(0) if n > 1 else k,
          out.stride(0) if m > 1 else n, int(accumulate), _stream())


def gemm_bf16_supports(t: int, n: int, k: int, ldx: int, ldw: int) -> bool:
    """True when the tcgen05 products take these sizes: rows of both operands must start
    on 16 bytes (k and the leading dimensions multiples of 8)."""
    return bool(library().pl_gemm_bf16_pair_supports(t, n, k, ldx, ldw))


GEMM_SKINNY_MAX_TOKENS = 64


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor | None = None,
              kernel: str | None = None, gated: bool = False) -> None:
    """out[T, N] (bf16 or fp32) = x[T, K] @ w[N, K]^T on the tcgen05 tensor cores.

    Two kernels: "skinny" for up to 64 tokens (one tile and part of k per CTA, the parts
    added inside a thread-block cluster) and "pair" (256 x 256 tiles on pairs of SMs,
    any token count, meant for prompts). `kernel=None` picks by the token count.

    gated (pair only): w is [2N, K], a gate matrix over an up matrix, and
    out = silu(x gate^T) * (x up^T), both products rounded to bfloat16 first."""
    _dev(x, w, out, status)
    assert x.dtype == w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
    t, k = x.shape
    n = w.shape[0] // 2 if gated else w.shape[0]
    assert w.shape[1] == k and out.shape == (t, n) and (not gated or w.shape[0] == 2 * n)
    assert x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    ldx = x.stride(0) if t > 1 else k
    ldw = w.stride(0) if w.shape[0] > 1 else k
    if kernel is None:
        kernel = "skinny" if t <= GEMM_SKINNY_MAX_TOKENS and not gated else "pair"
    if kernel == "skinny":
        assert not gated, "only the pair kernel has the gated epilogue"
        _call("pl_gemm_bf16_skinny", _p(x), _p(w), _p(out), t, n, k, ldx, ldw, out.stride(0) if t > 1 else n,
              int(out.dtype == torch.float32), _p(status), _stream())
        return
    if kernel == "pair":
        _call("pl_gemm_bf16_pair", _p(x), _p(w), _p(out), t, n, k, ldx, ldw, out.stride(0) if t > 1 else n,
              int(out.dtype == torch.float32), int(gated), _p(status), _stream())
        return
    raise ValueError(f"gemm_bf16: unknown kernel {kernel!r}")

GEMM_GATED_IN_MAX_TOKENS = 16


def gemm_bf16_gated_in(gate_up: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
                       status: torch.Tensor | None = None) -> None:
    """out[T, N] = (silu(g) * u) @ w[N, K]^T for gate_up = [g | u] of [T, 2K] (a gate/up
    projection's output): the skinny kernel forms the gated activation as it reads it
    (fp32, one rounding, the SwiGLU kernel's expression) and never writes it. T <= 16."""
    _dev(gate_up, w, out, status)
    assert gate_up.dtype == w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
    t, two_k = gate_up.shape
    n, k = w.shape
    assert two_k == 2 * k and out.shape == (t, n) and t <= GEMM_GATED_IN_MAX_TOKENS
    assert gate_up.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _call("pl_gemm_bf16_skinny_gated_in", _p(gate_up), _p(w), _p(out), t, n, k,
          gate_up.stride(0) if t > 1 else two_k, w.stride(0) if n > 1 else k, out.stride(0) if t > 1 else n,
          int(out.dtype == torch.float32), _p(status), _stream())


def gemm_bf16_act_in(z: torch.Tensor, bias: torch.Tensor | None, w: torch.Tensor, out: torch.Tensor, act: str,
                     status: torch.Tensor | None = None) -> None:
    """out[T, N] = act(z + bias) @ w[N, K]^T for z [T, K] (a projection's output, row stride free), act
    "relu2" or "tanh": the skinny kernel forms the activation as it reads z (fp32, one rounding, the
    bits of bias_act) and never writes it. T <= 16."""
    _dev(z, bias, w, out, status)
    assert z.dtype == w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
    t, k = z.shape
    n = w.shape[0]
    assert w.shape[1] == k and out.shape == (t, n) and t <= GEMM_GATED_IN_MAX_TOKENS and act in ("relu2", "tanh")
    assert z.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.shape == (k,) and bias.is_contiguous()
    _call("pl_gemm_bf16_skinny_act_in", _p(z), _p(bias), _p(w), _p(out), t, n, k, z.stride(0) if t > 1 else k,
          w.stride(0) if n > 1 else k, out.stride(0) if t > 1 else n, BIAS_ACT[act], int(out.dtype == torch.float32),
          _p(status), _stream())


def rope_kv_write(q: torch.Tensor, k: torch.Tensor | None, v: torch.Tensor | None, pos: torch.Tensor,
                  entry: torch.Tensor, table: torch.Tensor, k_pool: torch.Tensor | None,
                  v_pool: torch.Tensor | None, page_size: int, inv_freq: torch.Tensor | None, rotary: int,
                  status: torch.Tensor | None = None, q_norm: torch.Tensor | None = None,
                  k_norm: torch.Tensor | None = None, norm_eps: float = 0.0) -> None:
    """Rotates q [T, nh, hd] in place and writes rotated k and v [T, nkv, hd] into
    the pools [pages, nkv, page_size, hd] (views of one layer's K and V). q_norm and
    k_norm (fp32 [hd]): each head of q, of k, is first normalised over its hd
    (x * rsqrt(mean(x^2) + norm_eps) * scale) in fp32."""
    _dev(q, k, v, pos, entry, table, k_pool, v_pool, inv_freq, status, q_norm, k_norm)
    for scale_ in (q_norm, k_norm):
        if scale_ is not None:
            assert scale_.dtype == torch.float32 and scale_.shape == (q.shape[2],) and scale_.is_contiguous()
    tokens, n_heads, head_dim = q.shape
    assert q.stride(2) == 1 and q.stride(1) == head_dim
    row_stride = q.stride(0)
    n_kv = n_heads
    page_stride = head_stride = n_pages = 0
    if k_pool is not None:
        assert k is not None and v is not None and v_pool is not None
        n_kv = k.shape[1]
        for t in (k, v):
            assert t.shape == (tokens, n_kv, head_dim) and t.stride(2) == 1 and t.stride(1) == head_dim
            assert (tokens == 1 or t.stride(0) == row_stride) and t.dtype == q.dtype
        n_pages = k_pool.shape[0]
        assert k_pool.shape == (n_pages, n_kv, page_size, head_dim) == v_pool.shape
        assert k_pool.stride() == v_pool.stride() and k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim
        assert k_pool.dtype == q.dtype == v_pool.dtype
        page_stride, head_stride = k_pool.stride(0), k_pool.stride(1)
    assert pos.dtype == torch.int32 and entry.dtype == torch.int32 and table.dtype == torch.int32
    assert pos.numel() == tokens and entry.numel() == tokens and table.dim() == 2 and table.is_contiguous()
    if inv_freq is not None:
        assert inv_freq.dtype == torch.float64 and inv_freq.numel() == rotary // 2 and inv_freq.is_contiguous()
    _call("pl_rope_kv_write", _p(q), _p(k), _p(v), row_stride, _p(pos), _p(entry), _p(table), table.shape[1],
          _p(k_pool), _p(v_pool), page_stride, head_stride, page_size, n_pages, _p(inv_freq), rotary, tokens,
          n_heads, n_kv, head_dim, _code(q.dtype), _p(q_norm), _p(k_norm), float(norm_eps), _p(status), _stream())


def attention_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor,
                   pos: torch.Tensor, entry: torch.Tensor, out: torch.Tensor, page_size: int, window: int | None,
                   scale: float, status: torch.Tensor | None = None, mass_sum: torch.Tensor | None = None,
                   weight_sum: torch.Tensor | None = None, query_weights: torch.Tensor | None = None,
                   softcap: float = 0.0, sinks: torch.Tensor | None = None, gate: torch.Tensor | None = None,
                   distance_bias: torch.Tensor | None = None) -> None:
    """Causal paged attention; q and out [T, nh, hd] (row strides free), pools
    [pages, nkv, page_size, hd]. With mass_sum fp32 [pages, nh] and weight_sum fp32
    [pages], the attention mass of every attended page is added to them
    (query_weights fp32 [T], all 1 when None). softcap > 0: scaled scores pass through
    softcap * tanh(s / softcap) before the softmax. sinks fp32 [nh]: exp(sinks[h]) joins head
    h's softmax denominator (a term with no key and no value). gate [T, nh] logits (row
    stride free): head h's output for token t is multiplied by sigmoid(gate[t, h]). distance_bias
    fp32 [nh, rows]: entry min(distance, rows - 1) of a head's row is added to its scaled scores of a
    key `distance` tokens before the query."""
    _dev(q, k_pool, v_pool, table, pos, entry, out, status, mass_sum, weight_sum, query_weights, sinks, gate,
         distance_bias)
    if distance_bias is not None:
        assert distance_bias.dtype == torch.float32 and distance_bias.dim() == 2 and distance_bias.is_contiguous()
        assert distance_bias.shape[0] == q.shape[1] and distance_bias.shape[1] > 0
    if sinks is not None:
        assert sinks.dtype == torch.float32 and sinks.shape == (q.shape[1],) and sinks.is_contiguous()
    if gate is not None:
        assert gate.dtype == q.dtype and gate.shape == (q.shape[0], q.shape[1]) and gate.stride(1) == 1
    if mass_sum is not None:
        assert mass_sum.dtype == torch.float32 and mass_sum.shape == (k_pool.shape[0], q.shape[1])
        assert mass_sum.is_contiguous() and weight_sum is not None and weight_sum.dtype == torch.float32
        assert weight_sum.shape == (k_pool.shape[0],) and weight_sum.is_contiguous()
        if query_weights is not None:
            assert query_weights.dtype == torch.float32 and query_weights.numel() == q.shape[0]
            assert query_weights.is_contiguous()
    tokens, n_heads, head_dim = q.shape
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    assert q.stride(2) == 1 and q.stride(1) == head_dim and out.stride(2) == 1 and out.stride(1) == head_dim
    assert out.shape == q.shape and out.dtype == q.dtype == k_pool.dtype == v_pool.dtype
    assert k_pool.shape == (n_pages, n_kv, page_size, head_dim) == v_pool.shape
    assert k_pool.stride() == v_pool.stride() and k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim
    assert pos.dtype == torch.int32 and entry.dtype == torch.int32 and table.dtype == torch.int32
    assert table.dim() == 2 and table.is_contiguous()
    _call("pl_attention_simt", _p(q), q.stride(0), _p(k_pool), _p(v_pool), k_pool.stride(0), k_pool.stride(1),
          page_size, n_pages, _p(table), table.shape[1], _p(pos), _p(entry), _p(out), out.stride(0), tokens,
          n_heads, n_kv, head_dim, int(window or 0), float(scale), float(softcap or 0.0), _code(q.dtype),
          _p(mass_sum), _p(weight_sum), _p(query_weights), _p(sinks), _p(gate),
          gate.stride(0) if gate is not None else 0, _p(distance_bias),
          distance_bias.shape[1] if distance_bias is not None else 0, _p(status), _stream())


def attention_decode_supports(head_dim: int, group: int, page_size: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core decode kernel takes this shape."""
    return bool(library().pl_attention_decode_supports(head_dim, group, page_size, DTYPE_CODE.get(dtype, -1)))


def attention_decode_scratch_floats(n_tokens: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return int(library().pl_attention_decode_scratch_floats(n_tokens, n_heads, head_dim, n_splits))


class _DecodeRope(ctypes.Structure):
    _fields_ = [("k_new", _PTR), ("v_new", _PTR), ("inv_freq", _PTR), ("rotary", _I32)]


def _decode_rope(rope: tuple | None, q: torch.Tensor, n_kv: int):
    """The PlDecodeRope argument of the decode attention calls from (k_new, v_new,
    inv_freq, rotary), or None. k_new, v_new [T, nkv, hd] share q's row stride (slices of
    one projection output); None for both when the layer writes no keys."""
    if rope is None:
        return None
    k_new, v_new, inv_freq, rotary = rope
    tokens, _, head_dim = q.shape
    _dev(k_new, v_new, inv_freq)
    assert rotary == head_dim and inv_freq.dtype == torch.float64 and inv_freq.numel() == rotary // 2
    assert inv_freq.is_contiguous()
    for t in (k_new, v_new):
        if t is not None:
            assert t.dtype == q.dtype and t.shape == (tokens, n_kv, head_dim) and t.stride(2) == 1
            assert t.stride(1) == head_dim and (tokens == 1 or t.stride(0) == q.stride(0))
    return ctypes.byref(_DecodeRope(_p(k_new), _p(v_new), _p(inv_freq), int(rotary)))


_DECODE_COUNTERS: dict[torch.device, torch.Tensor] = {}
DECODE_COUNTERS = 1 << 20


def attention_decode_counters(device: torch.device) -> torch.Tensor:
    """The zeroed counters attention_decode_items works with (int32, DECODE_COUNTERS of
    them, one set per device: launches on one stream share it, each leaves it zero)."""
    device = torch.device(device)
    if device not in _DECODE_COUNTERS:
        _DECODE_COUNTERS[device] = torch.zeros(DECODE_COUNTERS, dtype=torch.int32, device=device)
    return _DECODE_COUNTERS[device]


def attention_decode_items(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor,
                           pos: torch.Tensor, entry: torch.Tensor, out: torch.Tensor, page_size: int,
                           window: int | None, scale: float, items: torch.Tensor, token_slot: torch.Tensor,
                           scratch: torch.Tensor, status: torch.Tensor | None = None,
                           rope: tuple | None = None) -> None:
    """bf16 attention of single decode tokens over a work list (shapes as
    attention_decode). items: int32 [n, 4] rows {token, first 16-key tile, tiles, split |
    splits << 12}, rows of no tiles are padding; the rows of a token cover its tiles once.
    token_slot int32 [tokens]: first slot of a token's partial results in `scratch`
    (fp32, n * n_heads * (head_dim + 2) floats). The CTA that finishes a token's kv head
    last merges its splits in split order. `rope` as in attention_decode."""
    _dev(q, k_pool, v_pool, table, pos, entry, out, items, token_slot, scratch, status)
    tokens, n_heads, head_dim = q.shape
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    assert q.dtype == torch.bfloat16 == k_pool.dtype == out.dtype
    assert k_pool.shape == v_pool.shape and k_pool.stride() == v_pool.stride()
    assert k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim
    assert q.stride(2) == 1 and q.stride(1) == head_dim and out.stride(2) == 1 and out.stride(1) == head_dim
    assert table.dtype == torch.int32 and table.is_contiguous() and pos.dtype == torch.int32 == entry.dtype
    assert pos.numel() == tokens == entry.numel() == token_slot.numel()
    assert items.dtype == torch.int32 == token_slot.dtype and items.dim() == 2 and items.shape[1] == 4
    assert items.is_contiguous() and token_slot.is_contiguous()
    n_items = items.shape[0]
    assert scratch.dtype == torch.float32 and scratch.is_contiguous()
    assert scratch.numel() >= n_items * n_heads * (head_dim + 2)
    if 2 + tokens * n_kv > DECODE_COUNTERS:
        raise KernelError(f"attention_decode_items: {tokens} tokens x {n_kv} kv heads need more than "
                          f"{DECODE_COUNTERS} counters")
    counters = attention_decode_counters(q.device)
    _call("pl_attention_decode_items", _p(q), q.stride(0), _p(k_pool), _p(v_pool), k_pool.stride(0),
          k_pool.stride(1), page_size, n_pages, _p(table), table.shape[1], _p(pos), _p(entry), _p(out),
          out.stride(0), tokens, n_heads, n_kv, head_dim, int(window or 0), float(scale), _p(items), n_items,
          _p(token_slot), _p(scratch), _p(counters), _decode_rope(rope, q, n_kv), _p(status), _stream())


def attention_decode_ctas_per_sm(head_dim: int) -> int:
    """How many CTAs of the decode attention kernel an SM holds at once."""
    return int(library().pl_attention_decode_ctas_per_sm(head_dim))


class _AttentionExtras(ctypes.Structure):
    _fields_ = [("sinks", _PTR), ("gate", _PTR), ("gate_row_stride", _I64), ("split_weights", _I32),
                ("softcap", _F32), ("distance_bias", _PTR), ("bias_rows", _I32)]


def attention_extras(q: torch.Tensor, sinks: torch.Tensor | None, gate: torch.Tensor | None,
                     split_weights: bool, softcap: float = 0.0,
                     distance_bias: torch.Tensor | None = None) -> "_AttentionExtras | None":
    """What the tensor-core attention kernels take beyond plain softmax attention (the struct
    PlAttentionExtras): sinks fp32 [nh] (exp(sinks[h]) joins head h's denominator), gate [T, nh]
    logits in q's dtype (outputs times their sigmoid), split_weights (softmax weights enter the
    value product as two bfloat16 terms), softcap (> 0: scaled scores pass through softcap *
    tanh(s / softcap)), distance_bias fp32 [nh, rows] (entry min(distance, rows - 1) of a head's row joins
    its scaled scores of a key `distance` tokens before the query). None when nothing is asked for. The tensors
    must outlive the call that takes the struct."""
    if sinks is None and gate is None and not split_weights and not softcap and distance_bias is None:
        return None
    _dev(sinks, gate, distance_bias)
    if distance_bias is not None:
        assert distance_bias.dtype == torch.float32 and distance_bias.dim() == 2 and distance_bias.is_contiguous()
        assert distance_bias.shape[0] == q.shape[1] and distance_bias.shape[1] > 0
    if sinks is not None:
        assert sinks.dtype == torch.float32 and sinks.shape == (q.shape[1],) and sinks.is_contiguous()
    if gate is not None:
        assert gate.dtype == q.dtype and gate.shape == (q.shape[0], q.shape[1]) and gate.stride(1) == 1
    return _AttentionExtras(_p(sinks), _p(gate), gate.stride(0) if gate is not None else 0, int(bool(split_weights)),
                            float(softcap or 0.0), _p(distance_bias),
                            distance_bias.shape[1] if distance_bias is not None else 0)


def attention_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor,
                     pos: torch.Tensor, entry: torch.Tensor, out: torch.Tensor, page_size: int, window: int | None,
                     scale: float, n_splits: int, scratch: torch.Tensor | None,
                     status: torch.Tensor | None = None, mass: tuple | None = None,
                     rope: tuple | None = None, extras: "_AttentionExtras | None" = None) -> None:
    """bf16 attention of single decode tokens, split over the keys `n_splits` ways;
    shapes as attention_simt. `scratch`: fp32, attention_decode_scratch_floats long.
    `mass` = (tile_max, mass_sum, weight_sum, decay): also measures attention mass.
    tile_max is fp32 scratch of tokens * heads * (table width * page_size / 16) floats;
    mass_sum fp32 [pages, nh] and weight_sum fp32 [pages] are the running accumulators:
    what the request's pages hold is scaled by 1 - decay (the page the token opens
    restarts at zero) and decay * (the token's largest scaled score in the page), per
    head, and decay, per page, are added.
    `rope` = (k_new, v_new, inv_freq, rotary): q is unrotated; the kernel rotates it as it
    loads it, and rotates and stores each token's new key (with its value) at the token's
    place in the pools before reading it: the position encoding and the cache write
    folded into the attention (whole-head rotation only; not together with `mass`)."""
    _dev(q, k_pool, v_pool, table, pos, entry, out, scratch, status)
    tokens, n_heads, head_dim = q.shape
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    assert q.dtype == torch.bfloat16 == out.dtype == k_pool.dtype == v_pool.dtype
    assert q.stride(2) == 1 and q.stride(1) == head_dim and out.stride(2) == 1 and out.stride(1) == head_dim
    assert out.shape == q.shape
    assert k_pool.shape == (n_pages, n_kv, page_size, head_dim) == v_pool.shape
    assert k_pool.stride() == v_pool.stride() and k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim
    assert pos.dtype == torch.int32 and entry.dtype == torch.int32 and table.dtype == torch.int32
    assert table.dim() == 2 and table.is_contiguous() and pos.numel() == tokens == entry.numel()
    if n_splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
        assert scratch.numel() >= attention_decode_scratch_floats(tokens, n_heads, head_dim, n_splits)
    if mass is not None:
        assert rope is None, "the mass-measuring call does not fold the position encoding in"
        tile_max, mass_sum, weight_sum, decay = mass
        max_tiles = table.shape[1] * page_size // 16
        _dev(tile_max, mass_sum, weight_sum)
        assert tile_max.dtype == torch.float32 and tile_max.is_contiguous()
        assert tile_max.numel() >= tokens * n_heads * max_tiles
        assert mass_sum.dtype == torch.float32 and mass_sum.shape == (n_pages, n_heads) and mass_sum.is_contiguous()
        assert weight_sum.dtype == torch.float32 and weight_sum.shape == (n_pages,) and weight_sum.is_contiguous()
        _call("pl_attention_decode_mass", _p(q), q.stride(0), _p(k_pool), _p(v_pool), k_pool.stride(0),
              k_pool.stride(1), page_size, n_pages, _p(table), table.shape[1], _p(pos), _p(entry), _p(out),
              out.stride(0), tokens, n_heads, n_kv, head_dim, int(window or 0), float(scale), int(n_splits),
              _p(scratch), _p(tile_max), max_tiles, _p(mass_sum), _p(weight_sum), float(decay), _p(status),
              _stream())
        return
    if extras is not None:
        assert rope is None, "sinks, gates and split weights: not together with the folded position encoding"
        _call("pl_attention_decode_extras", _p(q), q.stride(0), _p(k_pool), _p(v_pool), k_pool.stride(0),
              k_pool.stride(1), page_size, n_pages, _p(table), table.shape[1], _p(pos), _p(entry), _p(out),
              out.stride(0), tokens, n_heads, n_kv, head_dim, int(window or 0), float(scale), int(n_splits),
              _p(scratch), ctypes.byref(extras), _p(status), _stream())
        return
    _call("pl_attention_decode", _p(q), q.stride(0), _p(k_pool), _p(v_pool), k_pool.stride(0), k_pool.stride(1),
          page_size, n_pages, _p(table), table.shape[1], _p(pos), _p(entry), _p(out), out.stride(0), tokens,
          n_heads, n_kv, head_dim, int(window or 0), float(scale), int(n_splits), _p(scratch),
          _decode_rope(rope, q, n_kv), _p(status),
          _stream())


def attention_prefill_supports(head_dim: int, page_size: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core kernel for prompt portions takes this shape."""
    return bool(library().pl_attention_prefill_supports(head_dim, page_size, DTYPE_CODE.get(dtype, -1)))


def attention_prefill_tile_rows() -> int:
    return int(library().pl_attention_prefill_tile_rows())


def attention_prefill(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor,
                      tiles: torch.Tensor, out: torch.Tensor, page_size: int, window: int | None, scale: float,
                      status: torch.Tensor | None = None, extras: "_AttentionExtras | None" = None) -> None:
    """bf16 causal attention of prompt portions. tiles int32 [n, 4]: {first token
    row, rows, position of the first row, block-table row}; q, out [T, nh, hd]. extras: see
    attention_extras."""
    _dev(q, k_pool, v_pool, table, tiles, out, status)
    tokens, n_heads, head_dim = q.shape
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    assert q.dtype == torch.bfloat16 == out.dtype == k_pool.dtype == v_pool.dtype
    assert q.stride(2) == 1 and q.stride(1) == head_dim and out.stride(2) == 1 and out.stride(1) == head_dim
    assert out.shape == q.shape
    assert k_pool.shape == (n_pages, n_kv, page_size, head_dim) == v_pool.shape
    assert k_pool.stride() == v_pool.stride() and k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    assert tiles.dtype == torch.int32 and tiles.dim() == 2 and tiles.shape[1] == 4 and tiles.is_contiguous()
    _call("pl_attention_prefill", _p(q), q.stride(0), _p(k_pool), _p(v_pool), k_pool.stride(0), k_pool.stride(1),
          page_size, n_pages, _p(table), table.shape[1], _p(tiles), tiles.shape[0], _p(out), out.stride(0),
          n_heads, n_kv, head_dim, int(window or 0), float(scale),
          ctypes.byref(extras) if extras is not None else None, _p(status), _stream())


def attention_prefill_tcgen05_supports(q: torch.Tensor, k_pool: torch.Tensor, page_size: int) -> bool:
    """Whether the tcgen05 kernel for prompt portions takes this shape and cache layout."""
    return bool(library().pl_attention_prefill_tcgen05_supports(
        q.shape[2], page_size, k_pool.shape[1], k_pool.stride(0), k_pool.stride(1), q.stride(0),
        DTYPE_CODE.get(q.dtype, -1)))


PREFILL_SPLITS_MAX = 32


def attention_prefill_scratch_floats(n_tokens: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return int(library().pl_attention_prefill_scratch_floats(n_tokens, n_heads, head_dim, n_splits))


def attention_prefill_tcgen05_tile_rows(group: int) -> int:
    """The most rows of a tile that attention_prefill_tcgen05 takes with `wide=True` for
    this GQA group: 256 when the group is odd (a CTA then works on one head, and the
    two halves of a tile share its keys), else 128."""
    return int(library().pl_attention_prefill_tcgen05_tile_rows(group))


class _PrefillMass(ctypes.Structure):
    _fields_ = [("query_weights", _PTR), ("scratch", _PTR), ("pages", _I32), ("table_rows", _I32),
                ("step_mass", _PTR), ("step_weight", _PTR)]


def attention_prefill_tcgen05_measures_mass(group: int, page_size: int, wide: bool) -> bool:
    """Whether attention_prefill_tcgen05 can measure attention mass for this shape: two
    heads (an even group) or two halves of a wide tile per CTA, pages of 16, 32 or 64."""
    return (group % 2 == 0 or wide) and page_size in (16, 32, 64)


def attention_prefill_tcgen05(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table: torch.Tensor,
                              tiles: torch.Tensor, out: torch.Tensor, page_size: int, window: int | None,
                              scale: float, status: torch.Tensor | None = None, n_splits: int = 1,
                              scratch: torch.Tensor | None = None, wide: bool = False,
                              mass: tuple | None = None, distance_bias: torch.Tensor | None = None) -> None:
    """As attention_prefill, on the tcgen05 tensor cores. `distance_bias` fp32 [nh, rows] (even GQA groups, no
    wide tiles, no mass): entry min(distance, rows - 1) of a head's row joins its scaled scores. With n_splits > 1 every tile's
    keys are shared out over that many CTAs and merged through `scratch` (float32,
    attention_prefill_scratch_floats elements): for few tiles over many keys. `wide`: the
    tiles have up to attention_prefill_tcgen05_tile_rows(group) rows instead of 128.
    `mass` = (query_weights fp32 [T], step_mass fp32 [pages, nh], step_weight fp32
    [pages]): also adds to the step's attention mass: per page and head the sum over the
    query rows of weight * (the row's largest scaled score among the page's keys it
    attends), and per page the sum of the weights of the rows that attend it; the rows'
    sums are added in a fixed order (see attention_prefill_tcgen05_measures_mass)."""
    _dev(q, k_pool, v_pool, table, tiles, out, status, scratch)
    mass_arg = None
    if mass is not None:
        query_weights, step_mass, step_weight = mass
        _dev(query_weights, step_mass, step_weight)
        assert query_weights.dtype == torch.float32 and query_weights.numel() >= q.shape[0]
        assert query_weights.is_contiguous() and step_mass.is_contiguous() and step_weight.is_contiguous()
        assert step_mass.dtype == torch.float32 and step_mass.shape == (k_pool.shape[0], q.shape[1])
        assert step_weight.dtype == torch.float32 and step_weight.shape == (k_pool.shape[0],)
        pages = table.shape[1]
        mass_scratch = torch.zeros(tiles.shape[0] * q.shape[1] * 8 * pages, dtype=torch.float32, device=q.device)
        mass_arg = ctypes.byref(_PrefillMass(_p(query_weights), _p(mass_scratch), pages, table.shape[0],
                                             _p(step_mass), _p(step_weight)))
    if n_splits > 1:
        need = attention_prefill_scratch_floats(q.shape[0], q.shape[1], q.shape[2], n_splits)
        assert scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need
    tokens, n_heads, head_dim = q.shape
    n_pages, n_kv = k_pool.shape[0], k_pool.shape[1]
    assert q.dtype == torch.bfloat16 == out.dtype == k_pool.dtype == v_pool.dtype
    assert q.stride(2) == 1 and q.stride(1) == head_dim and out.stride(2) == 1 and out.stride(1) == head_dim
    assert out.shape == q.shape
    assert k_pool.shape == (n_pages, n_kv, page_size, head_dim) == v_pool.shape
    assert k_pool.stride() == v_pool.stride() and k_pool.stride(3) == 1 and k_pool.stride(2) == head_dim
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    assert tiles.dtype == torch.int32 and tiles.dim() == 2 and tiles.shape[1] == 4 and tiles.is_contiguous()
    if distance_bias is not None:
        _dev(distance_bias)
        assert mass is None and not wide and (n_heads // n_kv) % 2 == 0
        assert distance_bias.dtype == torch.float32 and distance_bias.is_contiguous()
        assert distance_bias.dim() == 2 and distance_bias.shape[0] == n_heads and distance_bias.shape[1] > 0
        _call("pl_attention_prefill_tcgen05_bias", _p(q), q.stride(0), tokens, _p(k_pool), _p(v_pool), k_pool.stride(0),
              k_pool.stride(1), page_size, n_pages, _p(table), table.shape[1], _p(tiles), tiles.shape[0], _p(out),
              out.stride(0), n_heads, n_kv, head_dim, int(window or 0), float(scale), int(n_splits), _p(scratch),
              _p(distance_bias), distance_bias.shape[1], _p(status), _stream())
        return
    _call("pl_attention_prefill_tcgen05", _p(q), q.stride(0), tokens, _p(k_pool), _p(v_pool), k_pool.stride(0),
          k_pool.stride(1), page_size, n_pages, _p(table), table.shape[1], _p(tiles), tiles.shape[0], _p(out),
          out.stride(0), n_heads, n_kv, head_dim, int(window or 0), float(scale), int(n_splits), _p(scratch),
          int(wide), mass_arg, _p(status), _stream())


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor | None,
           top_p: torch.Tensor | None, seed: torch.Tensor, draw_count: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] (int32) = a token drawn from row r of fp32 logits [R, V]."""
    _dev(logits, temperature, top_k, top_p, seed, draw_count, out)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and temperature.numel() == rows
    assert seed.dtype == torch.int64 and draw_count.dtype == torch.int64 and out.dtype == torch.int32
    assert seed.numel() == rows and draw_count.numel() == rows and out.numel() == rows
    if top_k is not None:
        assert top_k.dtype == torch.int32 and top_k.numel() == rows
    if top_p is not None:
        assert top_p.dtype == torch.float32 and top_p.numel() == rows
    _call("pl_sample", _p(logits), logits.stride(0) if rows > 1 else vocab, rows, vocab, _p(temperature),
          _p(top_k), _p(top_p), _p(seed), _p(draw_count), _p(out), _stream())
