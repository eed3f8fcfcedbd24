"""Python face of the CUDA library: one function per kernel, taking torch tensors.

Each wrapper checks device, dtype, contiguity and sizes, then calls the exported C entry
point with raw device pointers on torch's current stream.  There is no CPU path and no
fallback: a tensor that is not on a CUDA device, or a library that cannot be built or
loaded, raises.  Library matrix products (cuBLAS through torch) stand in for the bf16
linear layers, as the reference uses a library for them (kvcore/model/layer/linear.py:6-12).
"""
from __future__ import annotations

import ctypes
import os
from typing import Any

import torch

from . import build as _build

_F32, _BF16 = 0, 1
_lib: ctypes.CDLL | None = None
_vp = ctypes.c_void_p
_int = ctypes.c_int
_ll = ctypes.c_longlong
_float = ctypes.c_float


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or its launch failed."""


def ensure_built(verbose: bool = False) -> str:
    """Build (if needed) and load the CUDA library; returns its path."""
    global _lib
    if _lib is not None:
        return _lib._name
    path = _build.build(verbose=verbose)
    lib = ctypes.CDLL(str(path))
    lib.kvb_last_error.restype = ctypes.c_char_p
    lib.kvb_status_word.restype = _vp
    signatures: dict[str, list[Any]] = {
        "kvb_gather_rows": [_vp, _vp, _vp, _int, _int, _int, _int, _vp],
        "kvb_rmsnorm": [_vp, _vp, _vp, _vp, _int, _int, _float, _int, _int, _vp],
        "kvb_silu_mul": [_vp, _vp, _int, _int, _int, _int, _vp],
        "kvb_rope_table": [_vp, _vp, _vp, _int, _int, _vp],
        "kvb_rope_kv_write": [_vp, _ll, _vp, _vp, _vp, _vp, _int, _vp, _vp, _int, _int, _int, _int,
                              _int, _int, _int, _vp],
        "kvb_paged_attention_rows": [_vp, _int, _vp, _int, _vp, _vp, _vp, _int, _vp, _vp, _int, _int,
                                     _int, _int, _int, _int, _float, _int, _int, _int, _vp],
        "kvb_layer_norm": [_vp, _vp, _vp, _vp, _int, _int, _float, _int, _int, _int, _vp],
        "kvb_stream_add": [_vp, _vp, _int, _vp, _vp, _ll, _int, _vp],
        "kvb_qk_prepare": [_vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _int, _vp, _vp, _int, _int, _int, _int, _int,
                           _int, _int, _float, _int, _int, _int, _int, _vp],
        "kvb_glu_clamped": [_vp, _vp, _int, _int, _float, _float, _float, _int, _vp],
        "kvb_moe_route": [_vp, _vp, _vp, _vp, _ll, _vp, _vp, _int, _int, _int, _int, _int, _int, _int, _vp, _int, _int,
                          _float, _int, _vp],
        "kvb_moe_align": [_vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _int, _vp],
        "kvb_moe_gemv": [_vp, _vp, _ll, _int, _vp, _vp, _vp, _int, _int, _int, _int, _int, _vp],
        "kvb_moe_gemv_rows": [_vp, _vp, _ll, _int, _vp, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _vp],
        "kvb_moe_gather": [_vp, _vp, _ll, _int, _vp, _vp, _vp, _int, _int, _vp, _int, _int, _vp],
        "kvb_moe_gemm": [_vp, _vp, _ll, _int, _vp, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _int, _vp],
        "kvb_moe_combine": [_vp, _vp, _int, _int, _vp, _vp, _vp, _vp, _int, _int, _int, _vp],
        "kvb_flash_paged_attention": [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _int, _vp, _vp, _int, _int, _int,
                                      _int, _int, _int, _int, _float, _int, _int, _vp, _vp, _vp],
        "kvb_kept_first_merge": [_vp, _int, _vp, _vp, _int, _vp, _vp, _vp, _int, _vp, _vp, _int, _int, _int, _int,
                                 _int, _int, _float, _int, _int, _int, _vp],
        "kvb_make_kv_tensor_map": [_vp, _vp, _ll, _int, _int, _int],
        "kvb_flash_decode_tma": [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _int, _vp, _vp, _int, _int, _int, _int,
                                 _int, _int, _int, _float, _int, _int, _vp, _vp, _vp, _vp, _vp, _int, _vp, _vp],
        "kvb_make_kv_half_tensor_map": [_vp, _vp, _ll, _int, _int, _int],
        "kvb_flash_prefill_tc5": [_vp, _ll, _vp, _ll, _vp, _vp, _vp, _int, _vp, _vp, _int, _int, _int, _int, _int,
                                  _int, _int, _int, _float, _int, _vp, _vp],
        "kvb_gemm_f32": [_vp, _vp, _vp, _vp, _int, _int, _int, _ll, _ll, _vp],
        "kvb_rms_norm_shift": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _float, _int, _int, _int, _vp],
        "kvb_stream_add_norm": [_vp, _vp, _vp, _vp, _int, _int, _float, _vp, _vp, _ll, _vp, _int, _vp, _int, _int, _vp],
        "kvb_attention_dims_rows": [_vp, _ll, _ll, _int, _vp, _ll, _ll, _vp, _ll, _ll, _ll, _vp, _ll, _ll, _ll, _vp,
                                    _int, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _int, _int, _int, _int, _float,
                                    _int, _int, _vp],
        "kvb_flash_dims_attention": [_vp, _ll, _ll, _int, _vp, _ll, _ll, _vp, _ll, _ll, _ll, _vp, _ll, _ll, _ll, _vp,
                                     _int, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _int, _int, _int, _int, _int,
                                     _float, _int, _int, _vp, _vp],
        "kvb_latent_prepare": [_vp, _ll, _vp, _float, _vp, _int, _vp, _vp, _vp, _int, _vp, _int, _int, _int, _vp,
                               _ll, _ll, _int, _vp, _ll, _ll, _vp, _int, _int, _int, _int, _int, _int, _vp],
        "kvb_gather_cached_rows": [_vp, _ll, _ll, _int, _vp, _int, _int, _int, _vp, _vp, _int, _vp, _int, _int,
                                   _int, _int, _vp],
        "kvb_head_norm_kv_write": [_vp, _ll, _vp, _vp, _float, _vp, _vp, _vp, _int, _vp, _int, _int, _int, _int,
                                   _int, _int, _int, _int, _int, _vp],
        "kvb_maps_combine": [_vp, _vp, _ll, _int, _float, _float, _float, _int, _vp],
        "kvb_sigmoid_gate_mul": [_vp, _vp, _ll, _ll, _vp, _ll, _int, _int, _int, _int, _vp],
        "kvb_gemm_stream_bf16": [_vp, _int, _ll, _vp, _ll, _vp, _vp, _int, _int, _int, _int, _vp, _int, _float, _vp,
                                 _int, _vp, _vp, _vp, _int, _vp],
        "kvb_gla_scan": [_vp, _vp, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _ll, _ll, _vp, _vp, _int, _int, _int, _int, _int,
                         _float, _float, _int, _vp],
        "kvb_delta_scan": [_vp, _vp, _vp, _ll, _ll, _vp, _vp, _int, _int, _int, _int, _int, _int, _vp],
        "kvb_conv_prepare": [_vp, _vp, _ll, _vp, _int, _vp, _ll, _ll, _vp, _vp, _vp, _vp, _vp, _int, _int, _int, _int,
                             _int, _int, _int, _int, _float, _float, _int, _vp],
        "kvb_gated_rms_norm": [_vp, _ll, _vp, _vp, _ll, _vp, _int, _int, _int, _float, _float, _int, _int, _vp],
        "kvb_lightning_scan": [_vp, _vp, _vp, _vp, _vp, _ll, _vp, _vp, _ll, _ll, _vp, _vp, _int, _int, _int, _int, _int,
                               _float, _int, _vp],
        "kvb_gelu_mul": [_vp, _vp, _vp, _ll, _int, _int, _int, _int, _vp],
        "kvb_turn_norm_kv_write": [_vp, _ll, _vp, _int, _vp, _vp, _int, _float, _vp, _vp, _vp, _int, _vp, _int, _int,
                                   _int, _int, _int, _int, _int, _int, _float, _int, _vp, _ll, _vp, _int, _vp],
        "kvb_head_gate": [_vp, _ll, _vp, _vp, _ll, _int, _int, _int, _float, _int, _vp],
        "kvb_embed_scaled": [_vp, _vp, _vp, _int, _int, _int, _float, _int, _vp],
        "kvb_sample": [_vp, _vp, _vp, _int, _int, _float, _vp],
        "kvb_feed_tokens": [_vp, _vp, _vp, _int, _int, _vp],
        "kvb_read_status": [_int, ctypes.POINTER(ctypes.c_int)],
    }
    for name, argtypes in signatures.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _int
    lib.kvb_set_pdl.argtypes = [_int]
    lib.kvb_set_pdl.restype = None
    lib.kvb_peek_status.argtypes = []
    lib.kvb_peek_status.restype = _int
    # Kernels of this library overlap their start with the end of the kernel in front of them
    # (programmatic dependent launch); KVCORE_B200_SERIAL_LAUNCH=1 switches that off.
    lib.kvb_set_pdl(0 if os.environ.get("KVCORE_B200_SERIAL_LAUNCH") == "1" else 1)
    lib.kvb_gemm_stream_scratch_floats.argtypes = [_int]
    lib.kvb_gemm_stream_scratch_floats.restype = _ll
    lib.kvb_gemm_stream_norm_max_k.argtypes = []
    lib.kvb_gemm_stream_norm_max_k.restype = _int
    lib.kvb_gemm_stream_scratch_marker.argtypes = []
    lib.kvb_gemm_stream_scratch_marker.restype = ctypes.c_uint
    lib.kvb_moe_tile_rows.argtypes = []
    lib.kvb_moe_tile_rows.restype = _int
    _lib = lib
    return str(path)


def library_is_loaded() -> bool:
    return _lib is not None


def require_device(device: torch.device | str) -> None:
    """Fail loudly unless ``device`` is a usable CUDA device and the library loads."""
    device = torch.device(device)
    if device.type != "cuda":
        raise KernelError(f"kvcore_b200 runs on CUDA devices only, got device {device}")
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available; kvcore_b200 has no CPU path")
    ensure_built()
    with torch.cuda.device(device):
        if not _lib.kvb_status_word():
            raise KernelError("cannot allocate the device status word")


launch_count = 0  # kernels of this library launched so far (read by the benchmark)


def _call(name: str, *args: Any, kernels: int = 1) -> None:
    """Run entry point ``name``, which launches ``kernels`` kernels."""
    global launch_count
    if _lib is None:
        ensure_built()
    launch_count += kernels
    code = getattr(_lib, name)(*args)
    if code != 0:
        raise KernelError(f"{name}: {_lib.kvb_last_error().decode()}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise KernelError(f"unsupported tensor dtype {t.dtype}: kernels take float32 or bfloat16")


def _check(t: torch.Tensor, name: str, *, dtype: torch.dtype | None = None, contiguous: bool = True) -> None:
    if t.device.type != "cuda":
        raise KernelError(f"{name} must be on a CUDA device, got {t.device}: there is no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def read_status(reset: bool = True) -> int:
    """Status bits set by kernels (1 bad token id, 2 bad page id, 4 bounded wait ran out)."""
    out = ctypes.c_int(0)
    _call("kvb_read_status", int(reset), ctypes.byref(out))
    if out.value & 4:
        # a kernel gave up a wait: the hand-over areas of the streaming kernels may hold parts that
        # nobody took; put them back into their state between launches
        for scratch in _stream_scratch.values():
            scratch.view(torch.int32).fill_(int(_lib.kvb_gemm_stream_scratch_marker()))
        for counters in _decode_work_counters.values():
            counters.zero_()
    return out.value


STATUS_BITS = {1: "a token id outside the vocabulary", 2: "a page id outside the cache",
               4: "a bounded wait inside a kernel ran out"}


def peek_status() -> int:
    """The status bits reported by the kernels that have finished, without waiting for any: free to
    call after the caller has synchronised on its own (0 when the library is not loaded)."""
    if _lib is None:
        return 0
    return int(_lib.kvb_peek_status())


def raise_on_status() -> None:
    """Raise ``KernelError`` if a finished kernel reported a problem (and clear the report)."""
    if peek_status():
        bits = read_status(reset=True)
        what = "; ".join(text for bit, text in STATUS_BITS.items() if bits & bit) or f"status {bits}"
        raise KernelError(f"a kernel reported: {what}")


# ---- shape policy -------------------------------------------------------------------------------
def check_attention_shape(num_heads: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype) -> None:
    """Refuse, with a clear error, head shapes the attention kernels do not take."""
    if head_dim <= 0 or head_dim % 2 or head_dim > 256:
        raise ValueError(f"head_dim must be even and at most 256, got {head_dim}")
    if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads:
        raise ValueError(
            f"num_heads {num_heads} must be a positive multiple of num_kv_heads {num_kv_heads}"
        )
    if dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"attention runs in float32 or bfloat16, got {dtype}")


# ---- kernels --------------------------------------------------------------------------------------
def gather_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[i] = table[ids[i]]`` for int32 ``ids``; used for the embedding and for logits rows."""
    _check(table, "table")
    _check(ids, "ids", dtype=torch.int32)
    if table.dim() != 2:
        raise KernelError(f"table must be [rows, width], got {tuple(table.shape)}")
    count, (rows, width) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((count, width), dtype=table.dtype, device=table.device)
    _call("kvb_gather_rows", out.data_ptr(), table.data_ptr(), ids.data_ptr(), count, width, rows,
          _dtype_code(table), _stream())
    return out


def feed_tokens(token_ids: torch.Tensor, source: torch.Tensor, sampled: torch.Tensor) -> None:
    """``token_ids[t] = sampled[source[t]]`` wherever ``source[t] >= 0`` (all int32, in place): the
    ids of a step that was packed before the step in front had been read back."""
    _check(token_ids, "token_ids", dtype=torch.int32)
    _check(source, "source", dtype=torch.int32)
    _check(sampled, "sampled", dtype=torch.int32)
    if source.numel() != token_ids.numel():
        raise KernelError(f"one source per token id is needed, got {source.numel()} for {token_ids.numel()}")
    _call("kvb_feed_tokens", token_ids.data_ptr(), source.data_ptr(), sampled.data_ptr(), token_ids.numel(),
          sampled.numel(), _stream())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    _check(x, "x")
    _check(weight, "weight")
    rows, width = x.shape
    if weight.numel() != width:
        raise KernelError(f"norm weight has {weight.numel()} entries for rows of width {width}")
    out = torch.empty_like(x)
    _call("kvb_rmsnorm", out.data_ptr(), None, x.data_ptr(), weight.data_ptr(), rows, width,
          float(eps), _dtype_code(x), _dtype_code(weight), _stream())
    return out


def add_rmsnorm(h: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``residual += h`` in place, returns ``norm(residual) * weight``."""
    _check(h, "h")
    _check(residual, "residual", dtype=h.dtype)
    _check(weight, "weight")
    if h.shape != residual.shape:
        raise KernelError(f"h {tuple(h.shape)} and residual {tuple(residual.shape)} differ in shape")
    rows, width = h.shape
    if weight.numel() != width:
        raise KernelError(f"norm weight has {weight.numel()} entries for rows of width {width}")
    out = torch.empty_like(h)
    _call("kvb_rmsnorm", out.data_ptr(), residual.data_ptr(), h.data_ptr(), weight.data_ptr(), rows,
          width, float(eps), _dtype_code(h), _dtype_code(weight), _stream())
    return out


def silu_mul(gate_up: torch.Tensor, group: int = 0) -> torch.Tensor:
    """``silu(gate) * up`` of a packed ``[T, 2I]`` tensor.

    ``group == 0``: gate is ``gate_up[:, :I]``, up is ``gate_up[:, I:]``.  ``group > 0``: gate and
    up columns alternate in runs of ``group`` (gate 0..g-1, up 0..g-1, gate g..2g-1, ...)."""
    _check(gate_up, "gate_up")
    rows, two_inter = gate_up.shape
    if two_inter % 2:
        raise KernelError(f"gate_up must have an even width, got {two_inter}")
    inter = two_inter // 2
    if group < 0 or (group and inter % group):
        raise KernelError(f"silu_mul: group {group} does not divide the width {inter}")
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    _call("kvb_silu_mul", out.data_ptr(), gate_up.data_ptr(), rows, inter, group, _dtype_code(gate_up), _stream())
    return out


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """``[T, D/2, 2]`` float32 (cos, sin) of ``float(position) * inv_freq``: made once per step."""
    _check(positions, "positions", dtype=torch.int32)
    _check(inv_freq, "inv_freq", dtype=torch.float32)
    tokens, half = positions.numel(), inv_freq.numel()
    table = torch.empty((tokens, half, 2), dtype=torch.float32, device=positions.device)
    _call("kvb_rope_table", table.data_ptr(), positions.data_ptr(), inv_freq.data_ptr(), tokens, half, _stream())
    return table


def rope_kv_write(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    req_index: torch.Tensor,
    cos_sin: torch.Tensor | None,
    table: torch.Tensor | None,
    k_cache: torch.Tensor | None,
    v_cache: torch.Tensor | None,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    *,
    write_kv: bool = True,
) -> None:
    """Rotate q and k of ``qkv [T, (H+2KVH)*D]`` in place with the ``rope_table`` values
    ``cos_sin`` (``None``: no rotation) and write k, v into their pages."""
    _check(qkv, "qkv", contiguous=False)
    _check(positions, "positions", dtype=torch.int32)
    _check(req_index, "req_index", dtype=torch.int32)
    tokens = qkv.shape[0]
    if qkv.stride(1) != 1:
        raise KernelError("qkv rows must be contiguous")
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"qkv width {qkv.shape[1]} does not match the head layout")
    if cos_sin is not None:
        _check(cos_sin, "cos_sin", dtype=torch.float32)
        if tuple(cos_sin.shape) != (tokens, head_dim // 2, 2):
            raise KernelError(f"cos_sin has shape {tuple(cos_sin.shape)} for {tokens} tokens of head_dim {head_dim}")
    k_ptr = v_ptr = table_ptr = None
    table_stride = page_size = num_pages = 0
    if write_kv:
        if k_cache is None or v_cache is None or table is None:
            raise KernelError("a cache write needs k_cache, v_cache and a block table")
        _check(k_cache, "k_cache", dtype=qkv.dtype)
        _check(v_cache, "v_cache", dtype=qkv.dtype)
        _check(table, "block table", dtype=torch.int32, contiguous=False)
        num_pages, kvh, page_size, d = k_cache.shape
        if (kvh, d) != (num_kv_heads, head_dim) or v_cache.shape != k_cache.shape:
            raise KernelError(f"cache shape {tuple(k_cache.shape)} does not match the head layout")
        if table.stride(1) != 1:
            raise KernelError("block table rows must be contiguous")
        k_ptr, v_ptr, table_ptr = k_cache.data_ptr(), v_cache.data_ptr(), table.data_ptr()
        table_stride = table.stride(0)
    if cos_sin is None and not write_kv:
        return
    _call("kvb_rope_kv_write", qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), req_index.data_ptr(),
          None if cos_sin is None else cos_sin.data_ptr(), table_ptr, table_stride, k_ptr, v_ptr,
          tokens, num_heads, num_kv_heads, head_dim, page_size, num_pages, _dtype_code(qkv), _stream())


def rope_inplace(q: torch.Tensor, k: torch.Tensor | None, positions: torch.Tensor, inv_freq: torch.Tensor) -> None:
    """Rotate ``q [T, H, D]`` (and ``k [T, KVH, D]``) in place without touching a cache; rows may
    be views into a wider buffer as long as heads are contiguous."""
    cos_sin = rope_table(positions, inv_freq)
    for x in (q, k):
        if x is None:
            continue
        _check(x, "q/k", contiguous=False)
        tokens, heads, head_dim = x.shape
        if x.stride(2) != 1 or x.stride(1) != head_dim:
            raise KernelError("rope_inplace: heads must be contiguous within a row")
        if inv_freq.numel() != head_dim // 2:
            raise KernelError(f"inv_freq has {inv_freq.numel()} entries for head_dim {head_dim}")
        _call("kvb_rope_kv_write", x.data_ptr(), x.stride(0), positions.data_ptr(), positions.data_ptr(),
              cos_sin.data_ptr(), None, 0, None, None, tokens, heads, 0, head_dim, 0, 0,
              _dtype_code(x), _stream())


_sm_counts: dict[int, int] = {}
_FLASH_CTAS_PER_SM = 3


def sm_count(device: torch.device | str | int | None = None) -> int:
    """Multiprocessors of ``device`` (default: the current CUDA device), asked from the driver once
    per device.  Grids, split counts and the scratch of the streaming kernels are sized from it."""
    if device is None:
        index = torch.cuda.current_device()
    elif isinstance(device, int):
        index = device
    else:
        device = torch.device(device)
        if device.type != "cuda":
            raise KernelError(f"kvcore_b200 runs on CUDA devices only, got device {device}")
        index = torch.cuda.current_device() if device.index is None else device.index
    count = _sm_counts.get(index)
    if count is None:
        count = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return count


def flash_attention_supported(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether the tensor-core kernel takes this shape (else the general kernel runs)."""
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128


def decode_splits(num_reqs: int, num_kv_heads: int, max_seq_len: int, sms: int | None = None) -> int:
    """How many chunks each request's keys are cut into so that the GPU (``sms`` multiprocessors,
    default: the current device's) is filled."""
    blocks = max(1, num_reqs * num_kv_heads)
    wanted = -(-(sms or sm_count()) * _FLASH_CTAS_PER_SM // blocks)
    longest = max(1, -(-max_seq_len // 256))  # a split of fewer than 256 keys is not worth a block
    return max(1, min(wanted, longest, 64))


def tma_decode_supported(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Whether the TMA-fed decode kernel takes this cache shape."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size in (8, 16, 32, 64)


def decode_splits_tma(num_reqs: int, num_kv_heads: int, max_seq_len: int, sms: int | None = None) -> int:
    """Splits for the TMA decode kernel, which keeps two blocks per SM (measured inside whole steps
    on B200; ``sms``: multiprocessors, default the current device's).

    Up to half a wave of (request, kv head) pairs: as many splits as still fit one wave of blocks,
    at most 16 (the merge grows with them) and at least two 64-key tiles a split (batch 1 at 1,024
    tokens gains 3.6 % with 8 splits over 2, loses with 16; at 8,192 tokens 16 beat 24, 32 and 37).

    More pairs than that: the kernel is bound by memory as long as the last wave is not sparse
    (64 requests x 8 heads = 1.73 waves run at 0.97 of the copy bandwidth unsplit, and 4 splits
    are 1.3 % slower), but a last wave of a few blocks runs no faster than ~0.45 of a full one
    (48 requests at 8,192 tokens: 3 splits -11 % a step; 40 at 4,096: 4 splits -9 %).  So the
    cost of 1 to 4 splits is estimated as full waves + max(rest, 0.45), half a percent a split for
    the merge, and the cheapest is taken."""
    base = max(1, num_reqs * num_kv_heads)
    tiles = max(1, -(-max_seq_len // 64))
    wave = (sms or sm_count()) * TMA_DECODE_BLOCKS_PER_SM
    if base * 2 <= wave:
        return max(1, min(wave // base, tiles // 2, 16))
    best, best_cost = 1, float("inf")
    for splits in (1, 2, 3, 4):
        if splits > 1 and tiles // splits < 4:
            break
        full, rest = divmod(base * splits, wave)
        cost = (full + (max(rest / wave, 0.45) if rest else 0.0)) / splits * (1.0 + 0.005 * (splits - 1))
        if cost < best_cost - 1e-9:
            best, best_cost = splits, cost
    return best


TMA_DECODE_BLOCKS_PER_SM = 2
# more (request, kv head, split) items than blocks fit the GPU at once: blocks stay and share the items
# (KVCORE_B200_DECODE_SHARED_WORK=0: one block an item, whatever their number)
TMA_DECODE_SHARED_WORK = os.environ.get("KVCORE_B200_DECODE_SHARED_WORK", "1") != "0"
_decode_work_counters: dict[torch.device, torch.Tensor] = {}


def _decode_work(device: torch.device) -> torch.Tensor:
    """Two counters through which the blocks of the TMA decode kernel share out their work when there
    is more of it than blocks that fit the GPU at once (zero between launches: the kernel's last
    block puts them back)."""
    counters = _decode_work_counters.get(device)
    if counters is None:
        counters = _decode_work_counters[device] = torch.zeros(2, dtype=torch.int32, device=device)
    return counters

_kv_tensor_maps: dict[tuple, tuple] = {}


def _kv_tensor_map_pair(k_cache: torch.Tensor, v_cache: torch.Tensor, kind: str = "page") -> tuple:
    """Host-side TMA descriptors of one layer's K and V cache, made once per tensor.  ``kind``:
    "page" = one contiguous box per page and head (decode), "half" = boxes of one 64-column half
    of a page (operand tiles of the tcgen05 prefill kernel)."""
    key = (kind, k_cache.data_ptr(), v_cache.data_ptr(), tuple(k_cache.shape))
    maps = _kv_tensor_maps.get(key)
    if maps is None:
        num_pages, kvh, page_size, d = k_cache.shape
        maps = (ctypes.create_string_buffer(128), ctypes.create_string_buffer(128))
        maker = "kvb_make_kv_tensor_map" if kind == "page" else "kvb_make_kv_half_tensor_map"
        for buffer, cache in zip(maps, (k_cache, v_cache)):
            _call(maker, ctypes.addressof(buffer), cache.data_ptr(), num_pages, kvh, page_size, d)
        _kv_tensor_maps[key] = maps
    return maps


def tc5_prefill_supported(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill kernel takes this cache shape."""
    return dtype == torch.bfloat16 and head_dim == 128 and page_size in (8, 16, 32, 64)


def paged_attention(
    qkv: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    table: torch.Tensor,
    ctx,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    scale: float,
    window: int | None,
    *,
    force_general: bool = False,
    num_splits: int | None = None,
    use_tma: bool = True,
    use_tc5: bool = True,
    cos_sin: torch.Tensor | None = None,
    write_kv: bool | None = None,
    keep_first: int = 0,
) -> torch.Tensor:
    """Attention of the step's queries (the first ``H*D`` columns of ``qkv``) over the cache.

    Returns ``[T, H*D]``.  ``ctx`` describes the batch: positions and request rows of the
    tokens, and per request its query start and cached length.  bfloat16 with a head size in
    steps of 16 up to 128 runs on the tensor-core kernel (split over the keys for decode
    batches); everything else, and all of float32, runs on the general kernel.

    ``write_kv=None``: q and k in ``qkv`` are rotated already and the cache holds this step's
    keys and values.  Otherwise this call also rotates q and k with the ``rope_table`` values
    ``cos_sin`` (``None``: no rotation) and, if ``write_kv``, writes this step's k and v into
    their pages: inside the decode kernel where that one runs (``qkv`` is then left as it
    was), through ``rope_kv_write`` in front of the other kernels.
    """
    if write_kv is not None:
        group = num_heads // num_kv_heads
        fused = (not force_general and not keep_first and use_tma and flash_attention_supported(qkv.dtype, head_dim)
                 and qkv.stride(0) % 8 == 0 and ctx.max_query_len * group <= 16
                 and tma_decode_supported(qkv.dtype, head_dim, k_cache.shape[2]))
        if not fused:
            rope_kv_write(qkv, ctx.positions, ctx.req_index, cos_sin, table, k_cache, v_cache,
                          num_heads, num_kv_heads, head_dim, write_kv=write_kv)
            cos_sin, write_kv = None, None
        elif cos_sin is not None:
            _check(cos_sin, "cos_sin", dtype=torch.float32)
            if tuple(cos_sin.shape) != (qkv.shape[0], head_dim // 2, 2):
                raise KernelError(f"cos_sin has shape {tuple(cos_sin.shape)} for {qkv.shape[0]} tokens "
                                  f"of head_dim {head_dim}")
    _check(qkv, "qkv", contiguous=False)
    _check(k_cache, "k_cache", dtype=qkv.dtype)
    _check(v_cache, "v_cache", dtype=qkv.dtype)
    _check(table, "block table", dtype=torch.int32, contiguous=False)
    tokens = qkv.shape[0]
    num_pages, kvh, page_size, d = k_cache.shape
    if (kvh, d) != (num_kv_heads, head_dim):
        raise KernelError(f"cache shape {tuple(k_cache.shape)} does not match the head layout")
    if keep_first < 0 or (keep_first and not window):
        raise KernelError(f"kept first positions ({keep_first}) need a window")
    out = torch.empty((tokens, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    if not force_general and flash_attention_supported(qkv.dtype, head_dim) and qkv.stride(0) % 8 == 0:
        group = num_heads // num_kv_heads
        geometry = (num_heads, num_kv_heads, head_dim, float(scale), int(window or 0))
        # Kept first positions: the windowed kernels also leave each row's log-sum, and a small kernel
        # behind them adds the kept keys that lie behind the row's window.
        lse = (torch.empty((tokens, num_heads), dtype=torch.float32, device=qkv.device)
               if keep_first and write_kv is None else None)

        def add_kept_first() -> None:
            if lse is not None:
                _call("kvb_kept_first_merge", out.data_ptr(), out.stride(0), lse.data_ptr(), qkv.data_ptr(),
                      qkv.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), table.data_ptr(), table.stride(0),
                      ctx.positions.data_ptr(), ctx.req_index.data_ptr(), tokens, num_heads, num_kv_heads, head_dim,
                      page_size, num_pages, float(scale), int(window), int(keep_first), _dtype_code(qkv), _stream())

        # A mixed step (portions of prompts beside single decoded tokens) is two kinds of work: the
        # portions fill query tiles of 128 rows, a decoded token has at most 16 rows a kv head and would
        # leave such a tile almost empty while walking all its keys.  When the batch says how long each
        # request's portion is and stands longest first (the step function packs it so), the two runs of
        # requests go to the kernel made for each.
        lens = getattr(ctx, "host_query_lens", None)
        contexts = getattr(ctx, "host_context_lens", None)
        if (write_kv is None and num_splits is None and lens and contexts and len(lens) == ctx.num_reqs
                and ctx.max_query_len * group > 16):
            long_count = sum(1 for n in lens if n * group > 16)
            if 0 < long_count < ctx.num_reqs and all(n * group > 16 for n in lens[:long_count]):
                for begin, end in ((0, long_count), (long_count, ctx.num_reqs)):
                    part = _RequestRun(ctx, begin, end)
                    _flash_attention_into(out, qkv, k_cache, v_cache, table[begin:end], part, geometry,
                                          None, use_tma, use_tc5, None, None, lse)
                add_kept_first()
                return out
        _flash_attention_into(out, qkv, k_cache, v_cache, table, ctx, geometry, num_splits, use_tma, use_tc5,
                              cos_sin, write_kv, lse)
        add_kept_first()
        return out
    _call("kvb_paged_attention_rows", out.data_ptr(), out.stride(0), qkv.data_ptr(), qkv.stride(0),
          k_cache.data_ptr(), v_cache.data_ptr(), table.data_ptr(), table.stride(0),
          ctx.positions.data_ptr(), ctx.req_index.data_ptr(), tokens, num_heads, num_kv_heads,
          head_dim, page_size, num_pages, float(scale), int(window or 0), int(keep_first), _dtype_code(qkv),
          _stream())
    return out


class _RequestRun:
    """Requests ``[begin, end)`` of a step's batch, as the attention kernels need a batch described:
    views of the per-request arrays (query starts are token offsets into the whole step, so outputs
    land in the rows of the whole step's tensors) and the lengths that size the launch."""

    def __init__(self, ctx, begin: int, end: int) -> None:
        lens, contexts = ctx.host_query_lens[begin:end], ctx.host_context_lens[begin:end]
        self.num_reqs = end - begin
        self.max_query_len = max(lens)
        self.max_seq_len = max(c + n for c, n in zip(contexts, lens))
        self.max_seq_len_bound = 0
        self.query_start = ctx.query_start[begin : end + 1]
        self.context_lens = ctx.context_lens[begin:end]
        self.host_query_lens, self.host_context_lens = lens, contexts


def _flash_attention_into(out, qkv, k_cache, v_cache, table, ctx, geometry, num_splits, use_tma, use_tc5,
                          cos_sin, write_kv, lse=None) -> None:
    """The tensor-core attention kernels on one batch (or one run of requests of a batch): the TMA
    decode kernel for at most 16 rows a kv head, the tcgen05 kernel for portions of prompts, the
    ``mma.sync`` kernel for the shapes those two do not take."""
    num_heads, num_kv_heads, head_dim, scale, window = geometry
    num_pages, _, page_size, _ = k_cache.shape
    lse_ptr = None if lse is None else lse.data_ptr()    # [tokens, H] rows of the whole step, as ``out``
    group = num_heads // num_kv_heads
    split_mode = ctx.max_query_len * group <= 16
    bound = getattr(ctx, "max_seq_len_bound", 0) or ctx.max_seq_len
    if split_mode and use_tma and tma_decode_supported(qkv.dtype, head_dim, page_size):
        sms = sm_count(qkv.device)
        splits = num_splits or decode_splits_tma(ctx.num_reqs, num_kv_heads, bound, sms)
        scratch = None
        if splits > 1:
            scratch = torch.empty(ctx.num_reqs * num_kv_heads * splits * 16 * (head_dim + 2),
                                  dtype=torch.float32, device=qkv.device)
        k_map, v_map = _kv_tensor_map_pair(k_cache, v_cache)
        _call("kvb_flash_decode_tma", out.data_ptr(), out.stride(0), qkv.data_ptr(), qkv.stride(0),
              ctypes.addressof(k_map), ctypes.addressof(v_map), table.data_ptr(), table.stride(0),
              ctx.query_start.data_ptr(), ctx.context_lens.data_ptr(), ctx.num_reqs, ctx.max_query_len,
              num_heads, num_kv_heads, head_dim, page_size, num_pages, scale, window,
              splits, None if scratch is None else scratch.data_ptr(),
              None if cos_sin is None else cos_sin.data_ptr(),
              k_cache.data_ptr() if write_kv else None, v_cache.data_ptr() if write_kv else None,
              _decode_work(qkv.device).data_ptr() if TMA_DECODE_SHARED_WORK else None,
              sms * TMA_DECODE_BLOCKS_PER_SM, lse_ptr, _stream(),
              kernels=2 if splits > 1 else 1)   # the splits are merged by a second kernel
        return
    if (not split_mode and use_tc5 and tc5_prefill_supported(qkv.dtype, head_dim, page_size)
            and out.stride(0) % 8 == 0):
        k_map, v_map = _kv_tensor_map_pair(k_cache, v_cache, "half")
        _call("kvb_flash_prefill_tc5", out.data_ptr(), out.stride(0), qkv.data_ptr(), qkv.stride(0),
              ctypes.addressof(k_map), ctypes.addressof(v_map), table.data_ptr(), table.stride(0),
              ctx.query_start.data_ptr(), ctx.context_lens.data_ptr(), ctx.num_reqs, ctx.max_query_len,
              qkv.shape[0], num_heads, num_kv_heads, head_dim, page_size, num_pages, scale, window,
              lse_ptr, _stream())
        return
    splits = 1
    if split_mode:
        splits = num_splits or decode_splits(ctx.num_reqs, num_kv_heads, bound, sm_count(qkv.device))
    scratch = None
    if splits > 1:
        scratch = torch.empty(ctx.num_reqs * num_kv_heads * splits * 16 * (head_dim + 2),
                              dtype=torch.float32, device=qkv.device)
    _call("kvb_flash_paged_attention", out.data_ptr(), out.stride(0), qkv.data_ptr(), qkv.stride(0),
          k_cache.data_ptr(), v_cache.data_ptr(), table.data_ptr(), table.stride(0),
          ctx.query_start.data_ptr(), ctx.context_lens.data_ptr(), ctx.num_reqs, ctx.max_query_len,
          num_heads, num_kv_heads, head_dim, page_size, num_pages, scale, window,
          splits, None if scratch is None else scratch.data_ptr(), lse_ptr, _stream(),
          kernels=2 if splits > 1 else 1)


_mm_out_dtype_ok: bool | None = None
# bf16 layers of at most STREAM_AUTO_ROWS tokens (K a multiple of 64) go to this library's own
# weight-streaming kernel (in a whole decode step it measured level with the library product on
# B200 at Llama 3.1 8B shapes, ahead at batch 1); larger batches go to the library product.
# KVCORE_B200_STREAM_ROWS overrides the bound (0: never).
STREAM_MAX_ROWS = 16
STREAM_AUTO_ROWS = int(os.environ.get("KVCORE_B200_STREAM_ROWS", "16"))
_stream_scratch: dict[int, torch.Tensor] = {}


TRACE_TAGS = {27: "rms_norm_shift", 28: "stream_add_norm", 29: "attention_dims_rows", 30: "latent_prepare",
              31: "head_norm_kv_write", 32: "maps_combine", 33: "sigmoid_gate_mul", 34: "flash_dims",
              35: "flash_dims_combine", 36: "gather_cached_rows", 37: "gla_scan", 38: "delta_scan", 39: "conv_prepare",
              40: "gated_rms_norm", 41: "turn_norm_kv_write", 42: "head_gate", 43: "embed_scaled", 44: "gla_prepare", 45: "gelu_mul", 46: "lightning_prepare", 47: "lightning_scan", 25: "kept_first_merge", 26: "moe_gather", 17: "layer_norm", 18: "stream_add", 19: "qk_prepare", 20: "glu_clamped", 21: "moe_route",
              22: "moe_align", 23: "moe_gemm", 24: "moe_combine", 1: "gather_rows", 2: "rmsnorm", 3: "silu_mul", 4: "rope_table", 5: "rope_kv_write", 6: "attention_rows",
              7: "flash_paged", 8: "flash_combine", 9: "flash_decode_tma", 10: "flash_decode_combine",
              11: "flash_prefill_tc5", 12: "gemm_f32", 13: "gemm_stream", 14: "sample", 16: "feed_tokens"}
_TRACE_UNITS = ("elementwise", "attention_decode_tma", "attention_flash", "attention_generic",
                "attention_prefill_tc5", "gemm_f32", "sampling", "gemm_stream", "layer_norm", "qk_prepare", "moe", "attention_kept_first",
                "stream_norm", "attention_dims", "mixer_prepare", "attention_flash_dims", "recurrence", "turn_norm")
_trace_buffer: torch.Tensor | None = None


def _trace_set(pointer: int | None) -> None:
    for unit in _TRACE_UNITS:
        fn = getattr(_lib, f"kvb_trace_set_{unit}")
        fn.argtypes = [_vp]
        fn.restype = _int
        if fn(pointer) != 0:
            raise KernelError(f"kvb_trace_set_{unit} failed")


def trace_start(device: torch.device | str = "cuda:0", capacity: int = 1 << 16, every_block: bool = False) -> None:
    """Start the kernel timeline trace: the first and last block of every kernel of this library
    (``every_block``: all of them) record when they entered, when the kernel in front had finished,
    and when they left."""
    global _trace_buffer
    ensure_built()
    torch.cuda.synchronize(device)
    buffer = torch.zeros(2 + 4 * capacity, dtype=torch.int64, device=device)
    buffer[1] = capacity | (-(1 << 63) if every_block else 0)
    with torch.cuda.device(device):
        _trace_set(buffer.data_ptr())
    _trace_buffer = buffer


def trace_stop() -> list[dict]:
    """Stop the trace; events sorted by entry time: kernel, block ("first"/"last"/"other"), sm, index
    (linear block index), entry, waited, exit (ns)."""
    global _trace_buffer
    if _trace_buffer is None:
        return []
    buffer = _trace_buffer
    torch.cuda.synchronize(buffer.device)
    with torch.cuda.device(buffer.device):
        _trace_set(None)
    host = buffer.cpu().tolist()
    _trace_buffer = None
    count = min(host[0], host[1] & ((1 << 63) - 1))
    events = []
    for i in range(count):
        tag, entry, waited, leave = host[2 + 4 * i: 6 + 4 * i]
        events.append({"kernel": TRACE_TAGS.get(tag & 0xFF, str(tag & 0xFF)),
                       "block": ("first", "last", "other")[min((tag >> 8) & 3, 2)], "sm": (tag >> 12) & 0x3FF,
                       "index": (tag >> 32) & 0xFFFFFFFF, "entry": entry, "waited": waited, "exit": leave})
    events.sort(key=lambda e: e["entry"])
    return events


def set_overlapped_launch(enabled: bool) -> None:
    """Switch programmatic dependent launch on or off for this library's kernels."""
    ensure_built()
    _lib.kvb_set_pdl(1 if enabled else 0)


def linear_stream(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, *,
                  out_dtype: torch.dtype | None = None, silu_pairs: bool = False) -> torch.Tensor:
    """``x @ weight.T`` for a decode-sized batch of bf16 ``x`` (at most 16 rows), K a multiple of 64: a
    balanced weight-streaming kernel (one block per SM, every block the same number of bytes).

    ``silu_pairs``: the rows of ``weight`` alternate in runs of 8 gate rows and 8 up rows; the
    result is ``[M, N/2]``, ``silu(gate) * up``, with the roundings of the unfused path."""
    _check(x, "x", dtype=torch.bfloat16, contiguous=False)
    _check(weight, "weight", dtype=torch.bfloat16)
    m, k = x.shape
    n = weight.shape[0]
    if not 0 < m <= STREAM_MAX_ROWS or k % 64 or x.stride(1) != 1 or x.stride(0) % 8:
        raise KernelError(f"linear_stream: unsupported shape x {tuple(x.shape)} strides {x.stride()}")
    if bias is not None:
        _check(bias, "bias", dtype=torch.bfloat16)
    if silu_pairs and (n % 16 or out_dtype not in (None, torch.bfloat16)):
        raise KernelError("linear_stream: gated pairs need an output width that is a multiple of 16 and a bf16 result")
    out = torch.empty((m, n // 2 if silu_pairs else n), dtype=out_dtype or torch.bfloat16, device=x.device)
    _stream_call(x.device, out.data_ptr(), int(out.dtype == torch.float32), out.stride(0),
                 x.data_ptr(), x.stride(0), weight.data_ptr(), None if bias is None else bias.data_ptr(),
                 m, n, k, int(silu_pairs), None, 0, 0.0, None, 0, None, None)
    return out


def linear(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None = None,
    *,
    out_dtype: torch.dtype | None = None,
) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` for ``x [M, K]``, ``weight [N, K]``.

    float32: this package's own FMA kernel (no tensor cores, fixed summation order).
    bfloat16: the library matrix product with 32-bit accumulation.
    ``out_dtype=float32`` keeps the accumulator's precision in the result (the logits).
    """
    global _mm_out_dtype_ok
    _check(x, "x", contiguous=False)
    _check(weight, "weight", dtype=x.dtype)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
        raise KernelError(f"linear: x {tuple(x.shape)} does not match weight {tuple(weight.shape)}")
    if x.stride(1) != 1:
        x = x.contiguous()
    m, k = x.shape
    n = weight.shape[0]
    if x.dtype == torch.float32:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
        _call("kvb_gemm_f32", out.data_ptr(), x.data_ptr(), weight.data_ptr(),
              None if bias is None else bias.data_ptr(), m, n, k, x.stride(0), out.stride(0), _stream())
        return out
    # Decode-sized batches: the layer is one pass over the weights, which this library's own
    # streaming kernel does, overlapping its start with the kernels in front of it.
    if _stream_ok(x, weight):
        return linear_stream(x, weight, bias, out_dtype=out_dtype)
    if out_dtype == torch.float32:
        if _mm_out_dtype_ok is None:
            try:
                torch.mm(x[:1], weight[:1].t(), out_dtype=torch.float32)
                _mm_out_dtype_ok = True
            except (TypeError, RuntimeError):
                _mm_out_dtype_ok = False
        if _mm_out_dtype_ok:
            out = torch.mm(x, weight.t(), out_dtype=torch.float32)
        else:
            out = torch.mm(x, weight.t()).float()
        if bias is not None:
            out = out + bias.float()
        return out
    return torch.nn.functional.linear(x, weight, bias)


def _stream_buffers(device: torch.device) -> torch.Tensor:
    """Scratch of the streaming kernel; kept for good, since a captured graph holds its address.  Every
    word holds a marker between launches."""
    index = device.index or 0
    scratch = _stream_scratch.get(index)
    if scratch is None:
        floats = int(_lib.kvb_gemm_stream_scratch_floats(sm_count(device)))
        marker = int(_lib.kvb_gemm_stream_scratch_marker())
        words = torch.full((floats,), marker, dtype=torch.int32, device=device)
        scratch = _stream_scratch[index] = words.view(torch.float32)
    return scratch


def _stream_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether the streaming kernel takes ``x @ weight.T`` (at most STREAM_AUTO_ROWS tokens); otherwise
    the library product does.  A streaming kernel on tcgen05 for 17 to 128 tokens existed and was
    taken out: in whole decode steps at Llama 3.1 8B layer sizes it was 29 % slower than the library
    product at 20 and 32 tokens and 39 to 47 % slower at 48 and 64."""
    m, k = x.shape
    return (x.dtype == torch.bfloat16 and k % 64 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and weight.is_contiguous() and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and 0 < m <= min(STREAM_AUTO_ROWS, STREAM_MAX_ROWS))


_STREAM_PIECE = 64   # columns of the residual whose squares one piece of ``sumsq`` holds


def _stream_call(device: torch.device, *args) -> None:
    """``kvb_gemm_stream_bf16`` with ``args`` up to ``sumsq_out``; scratch, SM count and stream are appended."""
    _call("kvb_gemm_stream_bf16", *args, _stream_buffers(device).data_ptr(), sm_count(device), _stream())


def linear_silu_mul(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, *,
                    group: int = 0) -> torch.Tensor:
    """The first half of a gated feed-forward: ``silu(gate(x)) * up(x)`` for a packed ``[2I, E]``
    matrix whose gate and up rows are halves (``group == 0``) or alternate in runs of ``group``.
    Decode-sized bf16 batches with runs of 8 take the streaming kernel with the activation in
    its epilogue; everything else is the matrix product followed by ``silu_mul``."""
    _check(x, "x", contiguous=False)
    _check(weight, "weight", dtype=x.dtype)
    if group == 8 and x.dim() == 2 and _stream_ok(x, weight) and weight.shape[0] % 16 == 0:
        return linear_stream(x, weight, bias, silu_pairs=True)
    return silu_mul(linear(x, weight, bias), group)


def norm_linear(h: torch.Tensor | None, residual: torch.Tensor | None, norm_weight: torch.Tensor, eps: float,
                weight: torch.Tensor, bias: torch.Tensor | None = None, *, silu_group: int | None = None,
                sumsq: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """A sub-layer's entry: ``x = rmsnorm(h + residual)``, then ``x @ weight.T`` (``silu_group`` None)
    or the gated ``silu(gate(x)) * up(x)`` (``silu_group`` as in ``linear_silu_mul``).

    Returns ``(out, residual)`` with ``residual`` now holding the sum (``residual`` None: the sum is
    ``h`` itself).  ``h`` None means the sub-layer in front has already added its output into
    ``residual`` (see ``linear_add_residual``); if it also left the rows' squares in ``sumsq``, a
    decode-sized bf16 batch runs as ONE kernel: a warp of the streaming product scales each stage's
    token rows by ``norm_weight * rsqrt(mean + eps)`` before they are used.  Everything else is
    the norm kernel followed by the product."""
    if h is None:
        if residual is None:
            raise KernelError("norm_linear: nothing to normalise")
        _check(residual, "residual", contiguous=False)
        m, k = residual.shape
        weight_bytes = 4 if norm_weight.dtype == torch.float32 else 2
        if (sumsq is not None and _stream_ok(residual, weight)
                and k * weight_bytes <= 4 * int(_lib.kvb_gemm_stream_norm_max_k())
                and norm_weight.dtype in (torch.bfloat16, torch.float32) and norm_weight.is_contiguous()
                and norm_weight.data_ptr() % 16 == 0
                and sumsq.dtype == torch.float32 and sumsq.is_contiguous() and sumsq.shape[0] == m
                and (silu_group is None or (silu_group == 8 and weight.shape[0] % 16 == 0))):
            _check(weight, "weight", dtype=torch.bfloat16)
            if bias is not None:
                _check(bias, "bias", dtype=torch.bfloat16)
            n = weight.shape[0]
            out = torch.empty((m, n // 2 if silu_group else n), dtype=torch.bfloat16, device=residual.device)
            _stream_call(residual.device, out.data_ptr(), 0, out.stride(0), residual.data_ptr(),
                         residual.stride(0), weight.data_ptr(), None if bias is None else bias.data_ptr(), m, n, k,
                         int(bool(silu_group)), norm_weight.data_ptr(), int(norm_weight.dtype == torch.float32),
                         float(eps), sumsq.data_ptr(), sumsq.shape[1], None, None)
            return out, residual
        x = rmsnorm(residual, norm_weight, eps)
    elif residual is None:
        x, residual = rmsnorm(h, norm_weight, eps), h
    else:
        x = add_rmsnorm(h, residual, norm_weight, eps)
    out = linear(x, weight, bias) if silu_group is None else linear_silu_mul(x, weight, bias, group=silu_group)
    return out, residual


def linear_add_residual(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                        residual: torch.Tensor | None) -> tuple[torch.Tensor | None, torch.Tensor | None]:
    """A sub-layer's exit: ``out = x @ weight.T (+ bias)`` on its way into the residual stream.

    Decode-sized bf16 batches: the streaming product adds its (bf16-rounded) result into ``residual``
    in place and returns ``(None, sumsq)``, ``sumsq [T, ceil(N / 64)]`` being the squares of the new
    rows of ``residual``, 64 columns a piece, for the norm that follows.  Otherwise returns
    ``(out, None)``: the sum is left to that norm, as the deferred-residual scheme has it."""
    if (residual is not None and x.dim() == 2 and _stream_ok(x, weight)
            and weight.shape[0] % 8 == 0 and residual.dtype == torch.bfloat16 and residual.is_contiguous()
            and tuple(residual.shape) == (x.shape[0], weight.shape[0]) and residual.data_ptr() % 16 == 0):
        _check(weight, "weight", dtype=torch.bfloat16)
        if bias is not None:
            _check(bias, "bias", dtype=torch.bfloat16)
        m, k = x.shape
        n = weight.shape[0]
        sumsq = torch.empty((m, -(-n // _STREAM_PIECE)), dtype=torch.float32, device=x.device)
        _stream_call(x.device, None, 0, n, x.data_ptr(), x.stride(0), weight.data_ptr(),
                     None if bias is None else bias.data_ptr(), m, n, k, 0, None, 0, 0.0, None, 0,
                     residual.data_ptr(), sumsq.data_ptr())
        return None, sumsq
    return linear(x, weight, bias), None


# ---- parts of layers that keep a 32-bit residual stream -------------------------------------------
def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, eps: float,
               out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``(x - mean) / sqrt(var + eps) * weight (+ bias)`` over the last axis of ``x [rows, width]`` with
    32-bit statistics; ``x`` may be the 32-bit stream of a bfloat16 model, ``out_dtype`` the activations'."""
    _check(x, "x")
    _check(weight, "weight")
    rows, width = x.shape
    if weight.numel() != width or (bias is not None and (bias.numel() != width or bias.dtype != weight.dtype)):
        raise KernelError(f"layer_norm: weight/bias do not match rows of width {width}")
    out = torch.empty((rows, width), dtype=out_dtype or x.dtype, device=x.device)
    _call("kvb_layer_norm", out.data_ptr(), x.data_ptr(), weight.data_ptr(), None if bias is None else bias.data_ptr(),
          rows, width, float(eps), _dtype_code(x), _dtype_code(out), _dtype_code(weight), _stream())
    return out


def stream_add(base: torch.Tensor, a: torch.Tensor | None = None, b: torch.Tensor | None = None,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """The 32-bit residual stream: ``base + (a + b)`` summed in 32-bit.  A 32-bit ``base`` is updated in
    place and returned; a ``base`` of the activation type (the embedded tokens) is widened into a new stream
    (into ``out`` when given: a 32-bit tensor of the same shape)."""
    _check(base, "base")
    for name, t in (("a", a), ("b", b)):
        if t is not None:
            _check(t, name)
            if t.shape != base.shape:
                raise KernelError(f"stream_add: {name} {tuple(t.shape)} does not match the stream {tuple(base.shape)}")
    if b is not None and (a is None or a.dtype != b.dtype):
        raise KernelError("stream_add: the two addends must have one type")
    if out is not None:
        _check(out, "out", dtype=torch.float32)
        if out.shape != base.shape:
            raise KernelError(f"stream_add: out {tuple(out.shape)} does not match the stream {tuple(base.shape)}")
    elif base.dtype == torch.float32:
        out = base
    else:
        out = torch.empty(base.shape, dtype=torch.float32, device=base.device)
    if a is None and out is base:
        return out
    addend = a if a is not None else base
    _call("kvb_stream_add", out.data_ptr(), base.data_ptr(), _dtype_code(base), None if a is None else a.data_ptr(),
          None if b is None else b.data_ptr(), base.numel(), _dtype_code(addend), _stream())
    return out


def rms_norm_shift(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype | None = None, *,
                   shift: torch.Tensor | None = None, state: torch.Tensor | None = None, ctx=None) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * weight`` over the rows of ``x [rows, width]`` (the 32-bit stream of a
    bfloat16 model, or rows of the activation type) into ``out_dtype``.  With ``shift`` (``[width]``) every
    normed row ``y_t`` becomes ``y_t + (y_{t-1} - y_t) * shift`` with ``y_{t-1}`` the normed row of the
    request's token in front: the row before inside the step, else the request's row of ``state``
    (``[slots, width]`` 32-bit, addressed by ``ctx.state_slots``), which this call also brings up to date."""
    _check(x, "x")
    _check(weight, "weight")
    rows, width = x.shape
    if weight.numel() != width:
        raise KernelError(f"rms_norm_shift: weight has {weight.numel()} entries for rows of width {width}")
    out = torch.empty((rows, width), dtype=out_dtype or x.dtype, device=x.device)
    pointers = (None, None, None, None, None)
    if shift is not None:
        _check(shift, "shift", dtype=weight.dtype)
        if state is None or ctx is None:
            raise KernelError("rms_norm_shift: a token shift needs the state rows and the step's context")
        _check(state, "state", dtype=torch.float32)
        if shift.numel() != width or state.dim() != 2 or state.shape[1] != width:
            raise KernelError(f"rms_norm_shift: shift {tuple(shift.shape)} / state {tuple(state.shape)} do not "
                              f"match rows of width {width}")
        pointers = (shift.data_ptr(), state.data_ptr(), ctx.req_index.data_ptr(), ctx.query_start.data_ptr(),
                    ctx.state_slots.data_ptr())
    _call("kvb_rms_norm_shift", out.data_ptr(), x.data_ptr(), weight.data_ptr(), *pointers, rows, width, float(eps),
          _dtype_code(x), _dtype_code(out), _dtype_code(weight), _stream())
    return out


def stream_add_norm(x: torch.Tensor, a: torch.Tensor, weight: torch.Tensor, eps: float, *,
                    out: torch.Tensor | None = None, stack: torch.Tensor | None = None, depth: int = 0,
                    coeffs: torch.Tensor | None = None, rounded: torch.dtype | None = None) -> tuple:
    """``X = x + a * rsqrt(mean(a^2) + eps) * weight`` on the 32-bit stream ``x [rows, width]`` (``a``: a
    sub-layer's output), into ``out`` (default: in place).  With ``coeffs`` (``[depth + 1]``) it also returns
    the weighted average ``sum_{j < depth} coeffs[j] * stack[j] + coeffs[depth] * X`` over the results in
    front (``stack [>= depth, rows, width]`` 32-bit); returns ``(X, average or None)``.  With ``rounded``
    (the type of ``a``) it also leaves ``X`` in that type, for a matrix product that reads the stream itself,
    and returns ``(X, average or None, X in that type)``."""
    _check(x, "x", dtype=torch.float32)
    _check(a, "a")
    _check(weight, "weight")
    rows, width = x.shape
    if a.shape != x.shape or weight.numel() != width:
        raise KernelError(f"stream_add_norm: a {tuple(a.shape)} / weight do not match the stream {tuple(x.shape)}")
    out = x if out is None else out
    _check(out, "out", dtype=torch.float32)
    if out.shape != x.shape:
        raise KernelError("stream_add_norm: out does not match the stream")
    avg = None
    extra = (None, None, 0, None, 0)
    if coeffs is not None:
        _check(coeffs, "coeffs", dtype=weight.dtype)
        if coeffs.numel() != depth + 1:
            raise KernelError(f"stream_add_norm: {coeffs.numel()} coefficients for {depth} results in front and one new")
        if depth:
            if stack is None:
                raise KernelError("stream_add_norm: the results in front are missing")
            _check(stack, "stack", dtype=torch.float32)
            if stack.dim() != 3 or stack.shape[0] < depth or tuple(stack.shape[1:]) != (rows, width):
                raise KernelError(f"stream_add_norm: stack {tuple(stack.shape)} does not hold {depth} x {tuple(x.shape)}")
        avg = torch.empty_like(x)
        extra = (avg.data_ptr(), None if not depth else stack.data_ptr(), rows * width, coeffs.data_ptr(), depth)
    narrow = None
    if rounded is not None:
        if rounded != a.dtype:
            raise KernelError(f"stream_add_norm: the stream is also left in the type of a ({a.dtype}), not {rounded}")
        narrow = torch.empty(x.shape, dtype=rounded, device=x.device)
    _call("kvb_stream_add_norm", out.data_ptr(), x.data_ptr(), a.data_ptr(), weight.data_ptr(), rows, width,
          float(eps), *extra, None if narrow is None else narrow.data_ptr(), _dtype_code(a), _dtype_code(weight),
          _stream())
    return (out, avg) if rounded is None else (out, avg, narrow)


def attention_dims(q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, table: torch.Tensor, ctx, *,
                   value_heads: int, group: int, maps: int, key_width: int, value_width: int, page_size: int,
                   num_pages: int, key_strides: tuple[int, int, int], value_strides: tuple[int, int, int], scale: float,
                   sink: torch.Tensor | None = None, window: int | None = None,
                   out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
                   force_general: bool = False, num_splits: int | None = None,
                   slopes: torch.Tensor | None = None) -> torch.Tensor:
    """Paged attention with a key width and a value width of their own.

    ``q [T, HQ, key_width]`` (a view; last stride 1) with ``HQ = value_heads * group * maps``: query head
    ``hq`` reads value head ``hq // (group * maps)`` and key head ``vh * maps + hq % maps``.  ``keys`` and
    ``values`` are tensors inside the paged cache (they may be views of one plane, and ``values`` may be a
    view of ``keys``); ``key_strides`` / ``value_strides`` give their (page, head, row) strides in elements;
    page ``p`` slot ``s`` head ``h`` starts at ``p * page + h * head + s * row``.  ``sink [HQ]`` (32-bit):
    a logit per query head that joins the softmax's denominator.  ``slopes [HQ]`` (32-bit): query head ``hq``'s
    score of the key at position ``j`` for the query at position ``i`` is lowered by ``slopes[hq] * (i - j)``.  Returns ``[T, HQ, value_width]`` in
    ``out_dtype`` (32-bit or the cache's type; default the cache's) or fills ``out`` (a view with last
    stride 1).  bfloat16 shapes the tensor-core kernel takes run there; everything else, and all of float32,
    on the general kernel."""
    _check(q, "q", contiguous=False)
    _check(keys, "keys", dtype=q.dtype, contiguous=False)
    _check(values, "values", dtype=q.dtype, contiguous=False)
    _check(table, "block table", dtype=torch.int32, contiguous=False)
    tokens, hq, dk = q.shape
    if dk != key_width or hq != value_heads * group * maps or q.stride(2) != 1:
        raise KernelError(f"attention_dims: q {tuple(q.shape)} does not match {value_heads} x {group} x {maps} heads "
                          f"of width {key_width}")
    if out is None:
        out = torch.empty((tokens, hq, value_width), dtype=out_dtype or q.dtype, device=q.device)
    if tuple(out.shape) != (tokens, hq, value_width) or out.stride(2) != 1 or out.dtype not in (torch.float32, q.dtype):
        raise KernelError(f"attention_dims: out {tuple(out.shape)} {out.dtype} does not fit")
    if sink is not None:
        _check(sink, "sink", dtype=torch.float32)
        if sink.numel() != hq:
            raise KernelError(f"attention_dims: {sink.numel()} sinks for {hq} query heads")
    if slopes is not None:
        _check(slopes, "slopes", dtype=torch.float32)
        if slopes.numel() != hq:
            raise KernelError(f"attention_dims: {slopes.numel()} slopes for {hq} query heads")
    if tokens == 0:
        return out
    if (not force_general and flash_dims_supported(q, out, key_width, value_width, page_size, key_strides,
                                                    value_strides, keys, values, maps)):
        _flash_dims(out, q, keys, values, table, ctx, value_heads, group, maps, key_width, value_width, page_size,
                    num_pages, key_strides, value_strides, scale, sink, window, num_splits, slopes)
        return out
    _call("kvb_attention_dims_rows", out.data_ptr(), out.stride(0), out.stride(1), int(out.dtype == torch.float32),
          q.data_ptr(), q.stride(0), q.stride(1), keys.data_ptr(), *key_strides, values.data_ptr(), *value_strides,
          table.data_ptr(), table.stride(0), ctx.positions.data_ptr(), ctx.req_index.data_ptr(),
          None if sink is None else sink.data_ptr(), None if slopes is None else slopes.data_ptr(), tokens, hq,
          group * maps, maps, key_width, value_width, page_size, num_pages, float(scale), int(window or 0),
          _dtype_code(q), _stream())
    return out


def _flash_dims_geometry(key_width: int, value_width: int, tile_rows: int, values_in_keys: bool):
    """(value width a block accumulates, slices of the value width, shared-memory bytes) of the tensor-core
    kernel for separate key and value widths, or None when it does not take them.  ``tile_rows``: 64 for
    prompt tiles, 16 or 32 for the few-row form of decode steps."""
    split_mode = tile_rows < 64
    if key_width % 16 or not 16 <= key_width <= 1024 or value_width % 8 or not 8 <= value_width <= 1024:
        return None
    slices = -(-value_width // 256)
    each = -(-value_width // slices)
    block = next((w for w in (32, 64, 96, 128, 192, 256) if w >= each), None)
    if block is None:
        return None
    values_in_keys = values_in_keys and slices * block <= key_width
    tile_m = tile_rows

    def tiles_bytes(keys_per_tile: int) -> int:
        total = 4 * keys_per_tile * 8 + (tile_m + 2 * keys_per_tile) * (key_width + 8) * 2
        return total if values_in_keys else total + 2 * keys_per_tile * (block + 8) * 2

    # prompts: tiles of 64 keys while three blocks of them fit a multiprocessor's shared memory, else of 32
    keys_per_tile = 64 if split_mode or tiles_bytes(64) <= 75 * 1024 else 32
    smem = tiles_bytes(keys_per_tile)
    if split_mode:
        smem = max(smem, 4 * keys_per_tile * 8 + tile_m * (key_width + 8) * 2 + (4 * 16 * block + 128) * 4)
    return (block, slices, smem) if smem <= 227 * 1024 else None


def flash_dims_supported(q, out, key_width, value_width, page_size, key_strides, value_strides, keys, values,
                         maps: int = 1) -> bool:
    """Whether the tensor-core kernel for separate key and value widths takes this call: bfloat16, widths in
    steps of 16 (keys) and 8 (values), every row on a 16-byte boundary, tiles that fit in shared memory."""
    if q.dtype != torch.bfloat16:
        return False
    strides = (*key_strides, *value_strides, q.stride(0), q.stride(1))
    if any(stride % 8 for stride in strides) or any(t.data_ptr() % 16 for t in (q, keys, values)):
        return False
    if out.stride(0) % 2 or out.stride(1) % 2 or out.data_ptr() % 8:
        return False
    alias = (keys.data_ptr() == values.data_ptr() and tuple(key_strides) == tuple(value_strides) and maps == 1)
    return all(_flash_dims_geometry(key_width, value_width, rows, alias) is not None for rows in (64, 32, 16))


def _flash_dims(out, q, keys, values, table, ctx, value_heads, group, maps, key_width, value_width, page_size,
                num_pages, key_strides, value_strides, scale, sink, window, num_splits, slopes=None) -> None:
    """The tensor-core kernel on the step's batch.  A mixed step (portions of prompts beside single decoded
    tokens, longest first as the step function packs them) goes as two runs of requests, so that the
    decoded tokens take the shape made for few rows and have their keys cut into chunks."""
    lens = getattr(ctx, "host_query_lens", None)
    contexts = getattr(ctx, "host_context_lens", None)
    runs = [(ctx, table)]
    if num_splits is None and lens and contexts and len(lens) == ctx.num_reqs and ctx.max_query_len * group > 32:
        long_count = sum(1 for n in lens if n * group > 32)
        if 0 < long_count < ctx.num_reqs and all(n * group > 32 for n in lens[:long_count]):
            runs = [(_RequestRun(ctx, begin, end), table[begin:end])
                    for begin, end in ((0, long_count), (long_count, ctx.num_reqs))]
    for run, run_table in runs:
        max_rows = run.max_query_len * group
        split_mode = max_rows <= 32                 # the few-row form: 16 or 32 rows a key head
        tile_m = 16 if max_rows <= 16 else 32 if split_mode else 64
        alias = keys.data_ptr() == values.data_ptr() and tuple(key_strides) == tuple(value_strides) and maps == 1
        block, slices, _ = _flash_dims_geometry(key_width, value_width, tile_m, alias)
        splits = num_splits
        if splits is None:
            splits = 1
            if run.max_query_len == 1:       # decoded tokens only: fill the GPU by cutting the keys
                bound = getattr(run, "max_seq_len_bound", 0) or run.max_seq_len
                tiles = 1 if split_mode else -(-max_rows // 64)
                # Measured in whole steps (batch 8 and 64 at 2,048 tokens, both cache layouts): beyond one wave
                # of blocks (two fit a multiprocessor, as of the TMA decode kernel) that kernel's policy of
                # evening out the last wave; below it the fewer chunks of the two policies (every chunk costs a
                # block's start, a partial result and a share of the combine)
                sms = sm_count(q.device)
                items, heads_here = run.num_reqs * tiles, value_heads * maps * slices
                splits = decode_splits_tma(items, heads_here, bound, sms)
                if items * heads_here * 2 <= sms * TMA_DECODE_BLOCKS_PER_SM:
                    splits = min(splits, decode_splits(items, heads_here, bound, sms))
        scratch = None
        if splits > 1:
            tiles = 1 if split_mode else -(-max_rows // 64)
            scratch = torch.empty(run.num_reqs * value_heads * maps * slices * tiles * splits * tile_m * (block + 2),
                                  dtype=torch.float32, device=q.device)
        _call("kvb_flash_dims_attention", out.data_ptr(), out.stride(0), out.stride(1),
              int(out.dtype == torch.float32), q.data_ptr(), q.stride(0), q.stride(1), keys.data_ptr(), *key_strides,
              values.data_ptr(), *value_strides, run_table.data_ptr(), run_table.stride(0),
              run.query_start.data_ptr(), run.context_lens.data_ptr(), None if sink is None else sink.data_ptr(),
              None if slopes is None else slopes.data_ptr(), run.num_reqs, run.max_query_len, value_heads, group, maps, key_width, value_width, page_size,
              num_pages, float(scale), int(window or 0), splits, None if scratch is None else scratch.data_ptr(),
              _stream(), kernels=2 if splits > 1 else 1)


def latent_prepare(kv_rows: torch.Tensor, norm_weight: torch.Tensor, eps: float, inv_freq: torch.Tensor, dims: int,
                   ctx, table: torch.Tensor, cache: torch.Tensor, q: torch.Tensor, q_width: int,
                   q_out: torch.Tensor, *, q_latent: torch.Tensor | None = None, write: bool = True) -> None:
    """Between the projections and the attention of a mixer that caches one latent vector a token.

    ``kv_rows [T, rank + rot]`` (a view): the first ``rank`` entries get an RMS norm with ``norm_weight``, the
    first ``dims`` of the last ``rot`` are turned by the token's position (entry 2i with 2i+1, angle
    ``position * inv_freq[i]``); the row goes into the token's place of ``cache [pages, 1, page, rank + rot]``
    if ``write``.  ``q [T, H, q_width + rot]`` (a view): its last ``rot`` entries, turned the same way, go
    behind the first ``lead`` entries of ``q_out [T, H, lead + rot]``; those first entries are copied from
    ``q_latent [T, H, lead]`` (a view) when given.  ``lead`` is ``rank`` when the attention runs in the latent
    space (``q_latent``: the query carried there), or ``q_width`` when it runs on keys of ``q_width + rot``
    entries (``q_latent``: the unturned part of ``q`` itself)."""
    _check(kv_rows, "kv_rows", contiguous=False)
    _check(q, "q", dtype=kv_rows.dtype, contiguous=False)
    _check(q_out, "q_out", dtype=kv_rows.dtype)
    _check(cache, "cache", dtype=kv_rows.dtype)
    _check(norm_weight, "norm_weight", dtype=kv_rows.dtype)
    if ctx.positions.numel() != q_out.shape[0]:
        raise KernelError(f"latent_prepare: {ctx.positions.numel()} positions for {q_out.shape[0]} tokens")
    _check(inv_freq, "inv_freq", dtype=torch.float32)
    tokens, heads, q_row = q_out.shape
    rank = norm_weight.numel()
    num_pages, one, page_size, width = cache.shape
    rot = width - rank
    lead = q_row - rot
    row = width
    if (one != 1 or lead not in (rank, q_width) or tuple(kv_rows.shape) != (tokens, row)
            or tuple(q.shape) != (tokens, heads, q_width + rot)):
        raise KernelError(f"latent_prepare: shapes kv_rows {tuple(kv_rows.shape)}, q {tuple(q.shape)}, q_out "
                          f"{tuple(q_out.shape)}, cache {tuple(cache.shape)} do not fit")
    if kv_rows.stride(1) != 1 or q.stride(2) != 1 or inv_freq.numel() * 2 < dims:
        raise KernelError("latent_prepare: rows must be contiguous in their last axis")
    latent = (None, 0, 0)
    if q_latent is not None:
        _check(q_latent, "q_latent", dtype=kv_rows.dtype, contiguous=False)
        if tuple(q_latent.shape) != (tokens, heads, lead) or q_latent.stride(2) != 1:
            raise KernelError(f"latent_prepare: q_latent {tuple(q_latent.shape)} does not fit")
        latent = (q_latent.data_ptr(), q_latent.stride(0), q_latent.stride(1))
    _call("kvb_latent_prepare", kv_rows.data_ptr(), kv_rows.stride(0), norm_weight.data_ptr(), float(eps),
          inv_freq.data_ptr(), int(dims), ctx.positions.data_ptr(), ctx.req_index.data_ptr(), table.data_ptr(),
          table.stride(0), cache.data_ptr(), page_size, num_pages, int(write), q.data_ptr(), q.stride(0), q.stride(1),
          int(q_width), *latent, q_out.data_ptr(), tokens, heads, rank, rot, lead, _dtype_code(kv_rows), _stream())


def gather_cached_rows(cache: torch.Tensor, table: torch.Tensor, src_req: torch.Tensor, src_pos: torch.Tensor,
                       col0: int, cols: int, out: torch.Tensor, *, copies: int = 1, head_stride: int = 0) -> None:
    """Columns ``[col0, col0 + cols)`` of the cached rows of the tokens ``(src_req[n], src_pos[n])`` (request row
    of ``table``, position) of ``cache [pages, 1, page, width]`` into ``out``: row ``n`` of ``out`` (a 2-D view,
    last stride 1) gets them at its start, and again every ``head_stride`` entries, ``copies`` times."""
    _check(cache, "cache")
    _check(out, "out", dtype=cache.dtype, contiguous=False)
    _check(src_req, "src_req", dtype=torch.int32)
    _check(src_pos, "src_pos", dtype=torch.int32)
    num_pages, one, page_size, width = cache.shape
    count = src_req.numel()
    if one != 1 or out.dim() != 2 or out.stride(1) != 1 or out.shape[0] < count or src_pos.numel() != count:
        raise KernelError(f"gather_cached_rows: cache {tuple(cache.shape)} / out {tuple(out.shape)} do not fit")
    if (copies - 1) * head_stride + cols > out.shape[1]:
        raise KernelError("gather_cached_rows: the copies do not fit a row of out")
    _call("kvb_gather_cached_rows", out.data_ptr(), out.stride(0), int(head_stride), int(copies), cache.data_ptr(),
          width, int(col0), int(cols), src_req.data_ptr(), src_pos.data_ptr(), count, table.data_ptr(),
          table.stride(0), page_size, num_pages, _dtype_code(cache), _stream())


def head_norm_kv_write(rows: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor | None, eps: float, ctx,
                       table: torch.Tensor, cache: torch.Tensor, *, q_vectors: int, k_vectors: int, dim: int,
                       value_width: int, write: bool = True) -> None:
    """``rows [T, (q_vectors + k_vectors) * dim + value_width]`` (a view; without the k and v part when not
    ``write``): every q and k vector of ``dim`` entries gets an RMS norm of its own (weights ``[dim]``, shared);
    q in place, the normed k vectors and the values side by side into the token's row of
    ``cache [pages, 1, page, k_vectors * dim + value_width]``."""
    _check(rows, "rows", contiguous=False)
    _check(q_weight, "q_weight", dtype=rows.dtype)
    _check(cache, "cache", dtype=rows.dtype)
    tokens = rows.shape[0]
    num_pages, one, page_size, width = cache.shape
    need = q_vectors * dim + ((k_vectors * dim + value_width) if write else 0)
    if rows.stride(1) != 1 or rows.shape[1] < need or (one, width) != (1, k_vectors * dim + value_width):
        raise KernelError(f"head_norm_kv_write: rows {tuple(rows.shape)} / cache {tuple(cache.shape)} do not fit")
    if write:
        _check(k_weight, "k_weight", dtype=rows.dtype)
    _call("kvb_head_norm_kv_write", rows.data_ptr(), rows.stride(0), q_weight.data_ptr(),
          None if k_weight is None else k_weight.data_ptr(), float(eps), ctx.positions.data_ptr(),
          ctx.req_index.data_ptr(), table.data_ptr(), table.stride(0), cache.data_ptr(), page_size, num_pages,
          int(write), tokens, q_vectors, k_vectors, dim, value_width, _dtype_code(rows), _stream())


def maps_combine(a: torch.Tensor, lam: float, eps: float, out_scale: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``a [T, H, 2, width]`` (32-bit: the outputs of a head's two score maps) -> ``[T, H * width]`` in
    ``out_dtype``: ``o = a[..., 0, :] - lam * a[..., 1, :]``, divided by its root mean square over ``width``
    (eps inside the root), times ``out_scale``."""
    _check(a, "a", dtype=torch.float32)
    tokens, heads, two, width = a.shape
    if two != 2:
        raise KernelError(f"maps_combine: two maps a head, got {tuple(a.shape)}")
    out = torch.empty((tokens, heads * width), dtype=out_dtype, device=a.device)
    _call("kvb_maps_combine", out.data_ptr(), a.data_ptr(), tokens * heads, width, float(lam), float(eps),
          float(out_scale), _dtype_code(out), _stream())
    return out


def sigmoid_gate_mul(o: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """``o [T, H, width]`` (a view) times ``sigmoid(gate [T, H * width])`` (a view of rows) -> ``[T, H * width]``."""
    _check(o, "o", contiguous=False)
    _check(gate, "gate", dtype=o.dtype, contiguous=False)
    tokens, heads, width = o.shape
    if o.stride(2) != 1 or gate.stride(1) != 1 or tuple(gate.shape) != (tokens, heads * width):
        raise KernelError(f"sigmoid_gate_mul: o {tuple(o.shape)} and gate {tuple(gate.shape)} do not fit")
    out = torch.empty((tokens, heads * width), dtype=o.dtype, device=o.device)
    _call("kvb_sigmoid_gate_mul", out.data_ptr(), o.data_ptr(), o.stride(0), o.stride(1), gate.data_ptr(),
          gate.stride(0), tokens, heads, width, _dtype_code(o), _stream())
    return out


def heads_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """A product per head: ``x [T, H, K]`` (a view; last stride 1) with ``weight [H, N, K]`` -> ``[T, H, N]``
    (a view when the batched library product made it; into ``out``, a view with last stride 1, on the 32-bit
    path).  float32: this package's own FMA kernel, head by head; bfloat16: one batched library product."""
    _check(x, "x", contiguous=False)
    _check(weight, "weight", dtype=x.dtype)
    tokens, heads, k = x.shape
    if weight.dim() != 3 or weight.shape[0] != heads or weight.shape[2] != k or x.stride(2) != 1:
        raise KernelError(f"heads_linear: x {tuple(x.shape)} does not match weight {tuple(weight.shape)}")
    n = weight.shape[1]
    if x.dtype == torch.float32:
        if out is None:
            out = torch.empty((tokens, heads, n), dtype=torch.float32, device=x.device)
        if tuple(out.shape) != (tokens, heads, n) or out.stride(2) != 1:
            raise KernelError(f"heads_linear: out {tuple(out.shape)} does not fit")
        for h in range(heads):
            _call("kvb_gemm_f32", out[:, h].data_ptr(), x[:, h].data_ptr(), weight[h].data_ptr(), None, tokens, n, k,
                  x.stride(0), out.stride(0), _stream())
        return out
    result = torch.bmm(x.transpose(0, 1), weight.transpose(1, 2)).transpose(0, 1)
    if out is not None:
        out.copy_(result)
        return out
    return result


QK_NORM_MODES = {None: 0, "none": 0, "projection": 1, "head": 2}


# ---- mixers with a matrix state per request and head, and attention with turned, normed q and k ------------
def embed_scaled(table: torch.Tensor, ids: torch.Tensor, scale: float) -> torch.Tensor:
    """``table[ids] * scale`` as the first value of a 32-bit residual stream ``[T, width]``."""
    _check(table, "table")
    _check(ids, "ids", dtype=torch.int32)
    out = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    _call("kvb_embed_scaled", out.data_ptr(), table.data_ptr(), ids.data_ptr(), ids.numel(), table.shape[0],
          table.shape[1], float(scale), _dtype_code(table), _stream())
    return out


def turn_norm_kv_write(rows: torch.Tensor, inv_freq: torch.Tensor | None, rot: int, ctx, table: torch.Tensor,
                       cache: torch.Tensor, *, q_heads: int, k_heads: int, dim: int, value_width: int,
                       norm: bool = True, eps: float = 0.0, q_weight: torch.Tensor | None = None,
                       k_weight: torch.Tensor | None = None, write: bool = True, q_temp: tuple | None = None,
                       mix_values: torch.Tensor | None = None, mix_weight: torch.Tensor | None = None) -> None:
    """q ``[q_heads, dim]`` and k ``[k_heads, dim]`` at the start of each row of ``rows`` (a view; last stride 1),
    then ``value_width`` value entries.  The first ``rot`` entries of every head turn in neighbouring pairs
    (2i, 2i+1) by ``position * inv_freq[i]``; then (``norm``) every head is divided by
    ``sqrt(mean(x^2) + eps)`` (times ``q_weight`` / ``k_weight [dim]`` when given).  ``q_temp = (coef, every)``:
    q is then multiplied by ``1 + coef * ln(floor((position + 1) / every) + 1)``.  q is replaced in place;
    with ``write`` the keys and the values go side by side into the token's row of ``cache``
    ``[pages, 1, page, k_heads * dim + value_width]``; with ``mix_values [T, value_width]`` (a view) and
    ``mix_weight`` (one 32-bit number ``lambda``) the cached values are
    ``(1 - lambda) * values + lambda * mix_values``."""
    _check(rows, "rows", contiguous=False)
    _check(cache, "cache", dtype=rows.dtype)
    _check(table, "block table", dtype=torch.int32, contiguous=False)
    tokens = rows.shape[0]
    if rows.stride(1) != 1 or rows.shape[1] < (q_heads + k_heads) * dim + value_width:
        raise KernelError(f"turn_norm_kv_write: rows {tuple(rows.shape)} do not hold the heads and the values")
    rot = int(rot) if inv_freq is not None else 0
    if rot:
        _check(inv_freq, "inv_freq", dtype=torch.float32)
        if rot % 2 or rot > dim or inv_freq.numel() < rot // 2:
            raise KernelError(f"turn_norm_kv_write: {rot} turned entries of {dim} with {inv_freq.numel()} frequencies")
    for name, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            _check(w, name, dtype=rows.dtype)
            if w.numel() != dim:
                raise KernelError(f"turn_norm_kv_write: {name} has {w.numel()} entries for heads of {dim}")
    num_pages, one, page_size, width = cache.shape
    if one != 1 or width != k_heads * dim + value_width or table.stride(1) != 1:
        raise KernelError(f"turn_norm_kv_write: cache {tuple(cache.shape)} does not hold rows of "
                          f"{k_heads} x {dim} + {value_width}")
    if q_temp is not None and int(q_temp[1]) <= 0:
        raise KernelError(f"turn_norm_kv_write: the temperature's period must be positive, got {q_temp[1]}")
    if mix_values is not None:
        _check(mix_values, "mix_values", dtype=rows.dtype, contiguous=False)
        if tuple(mix_values.shape) != (tokens, value_width) or (tokens and mix_values.stride(1) != 1):
            raise KernelError(f"turn_norm_kv_write: values to mix in {tuple(mix_values.shape)} are not "
                              f"[{tokens}, {value_width}]")
        if mix_weight is None:
            raise KernelError("turn_norm_kv_write: values to mix in need their weight")
        _check(mix_weight, "mix_weight", dtype=torch.float32)
    _call("kvb_turn_norm_kv_write", rows.data_ptr(), rows.stride(0), None if not rot else inv_freq.data_ptr(), rot,
          None if q_weight is None else q_weight.data_ptr(), None if k_weight is None else k_weight.data_ptr(),
          int(bool(norm)), float(eps), ctx.positions.data_ptr(), ctx.req_index.data_ptr(), table.data_ptr(),
          table.stride(0), cache.data_ptr(), page_size, num_pages, int(bool(write)), tokens, q_heads, k_heads, dim,
          value_width, 0.0 if q_temp is None else float(q_temp[0]), 0 if q_temp is None else int(q_temp[1]),
          None if mix_values is None else mix_values.data_ptr(), 0 if mix_values is None else mix_values.stride(0),
          None if mix_values is None else mix_weight.data_ptr(), _dtype_code(rows), _stream())


def head_gate(o: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``out[t, h * V + j] = o[t, h, j] * sigmoid(gate[t, h]) * scale``: ``o [T, H, V]`` 32-bit, ``gate [T, H]``
    and ``out [T, H * V]`` views of the activation type (last stride 1).  ``gate`` None: the scale alone."""
    _check(o, "o", dtype=torch.float32)
    _check(out, "out", contiguous=False)
    tokens, heads, width = o.shape
    if tuple(out.shape) != (tokens, heads * width) or (tokens and out.stride(1) != 1):
        raise KernelError(f"head_gate: out {tuple(out.shape)} does not fit o {tuple(o.shape)}")
    if gate is not None:
        _check(gate, "gate", dtype=out.dtype, contiguous=False)
        if tuple(gate.shape) != (tokens, heads) or (tokens and gate.stride(1) != 1):
            raise KernelError(f"head_gate: gate {tuple(gate.shape)} does not fit o {tuple(o.shape)}")
    _call("kvb_head_gate", out.data_ptr(), out.stride(0), o.data_ptr(), None if gate is None else gate.data_ptr(),
          0 if gate is None else gate.stride(0), tokens, heads, width, float(scale), _dtype_code(out), _stream())
    return out


def _state_row(state: torch.Tensor, offset: int, need: int) -> None:
    _check(state, "state", dtype=torch.float32)
    if state.dim() != 2 or offset < 0 or offset + need > state.shape[1]:
        raise KernelError(f"state {tuple(state.shape)} has no room for {need} entries at {offset}")


def gla_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, state: torch.Tensor, ctx, *,
             heads: int, dim: int, value_dim: int, q_scale: float, tau: float, state_offset: int = 0) -> torch.Tensor:
    """Gated linear attention over the step's tokens, request by request in order:
    ``S <- diag(a_t) S + k_t v_t^T``, ``o_t = S^T (q_t * q_scale)`` with ``a_t = sigmoid(z_t)^(1/tau)``.
    ``q, k [T, heads * dim]`` and ``v [T, heads * value_dim]`` are views of one tensor of projected rows,
    ``z [T, heads * dim]`` the decay's logits; ``state [slots, n]`` (32-bit) holds each request's
    ``S`` column by column (``[heads, value_dim, dim]``) at ``state_offset`` of its slot's row and is brought up
    to date.
    Returns ``o [T, heads, value_dim]`` 32-bit."""
    for name, t in (("q", q), ("k", k), ("v", v), ("z", z)):
        _check(t, name, dtype=q.dtype, contiguous=False)
        if t.stride(1) != 1 or t.shape[0] != q.shape[0]:
            raise KernelError(f"gla_scan: {name} {tuple(t.shape)} is not a view of the step's rows")
    if q.stride(0) != k.stride(0) or q.stride(0) != v.stride(0):
        raise KernelError("gla_scan: q, k and v must be views of one tensor of rows")
    if q.shape[1] != heads * dim or k.shape[1] != heads * dim or v.shape[1] != heads * value_dim or z.shape[1] != heads * dim:
        raise KernelError("gla_scan: widths do not match the head layout")
    _state_row(state, state_offset, heads * dim * value_dim)
    out = torch.empty((q.shape[0], heads, value_dim), dtype=torch.float32, device=q.device)
    # what the scan reads a token, 32-bit: q times its scale, k, the decays
    prepared = torch.empty((q.shape[0], 3 * heads * dim), dtype=torch.float32, device=q.device)
    _call("kvb_gla_scan", out.data_ptr(), prepared.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0),
          z.data_ptr(), z.stride(0), state.data_ptr(), state.stride(0), state_offset, ctx.query_start.data_ptr(),
          ctx.state_slots.data_ptr(), q.shape[0], ctx.num_reqs, heads, dim, value_dim, float(q_scale), float(tau),
          _dtype_code(q), _stream())
    return out


def conv_prepare(rows: torch.Tensor, taps: torch.Tensor, state: torch.Tensor, ctx, a_log: torch.Tensor,
                 dt_bias: torch.Tensor, *, heads: int, kv_heads: int, dim: int, value_dim: int, b_col: int, a_col: int,
                 q_scale: float, unit_eps: float, state_offset: int) -> torch.Tensor:
    """What a delta-rule mixer does to its projections before the scan.  ``rows`` (a view; last stride 1): q and k
    ``[kv_heads, dim]`` each, v ``[heads, value_dim]`` in the first columns (the convolved channels), one column a
    head at ``b_col`` and at ``a_col``.  Channels pass a causal convolution over time (``taps [channels, C]``, the
    last tap on the current token; the ``C - 1`` inputs in front of a portion are the request's
    ``state[slot, state_offset:][channels, C - 1]``, brought up to date by this call) and SiLU; q and k become
    unit vectors per head (``x / sqrt(sum(x^2) + unit_eps)``, q times ``q_scale``); ``beta = sigmoid(b)``;
    ``gate = exp(-exp(a_log) * softplus(a + dt_bias))``.  Returns 32-bit ``[T, q | k | v | beta | gate]``."""
    _check(rows, "rows", contiguous=False)
    _check(taps, "taps", dtype=rows.dtype)
    _check(a_log, "a_log", dtype=rows.dtype)
    _check(dt_bias, "dt_bias", dtype=rows.dtype)
    channels = 2 * kv_heads * dim + heads * value_dim
    if rows.stride(1) != 1 or taps.dim() != 2 or taps.shape[0] != channels or not 1 <= taps.shape[1] <= 9:
        raise KernelError(f"conv_prepare: taps {tuple(taps.shape)} for {channels} channels (1 to 9 taps)")
    if max(b_col, a_col) + heads > rows.shape[1] or min(b_col, a_col) < channels or a_log.numel() != heads or dt_bias.numel() != heads:
        raise KernelError("conv_prepare: the per-head columns do not fit the rows")
    _state_row(state, state_offset, channels * (taps.shape[1] - 1))
    tokens = rows.shape[0]
    out = torch.empty((tokens, channels + 2 * heads), dtype=torch.float32, device=rows.device)
    _call("kvb_conv_prepare", out.data_ptr(), rows.data_ptr(), rows.stride(0), taps.data_ptr(), taps.shape[1],
          state.data_ptr(), state.stride(0), state_offset, ctx.req_index.data_ptr(), ctx.query_start.data_ptr(),
          ctx.state_slots.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(), tokens, ctx.num_reqs, heads, kv_heads, dim,
          value_dim, b_col, a_col, float(q_scale), float(unit_eps), _dtype_code(rows), _stream(),
          kernels=2 if taps.shape[1] > 1 else 1)
    return out


def delta_scan(prepared: torch.Tensor, state: torch.Tensor, ctx, *, heads: int, kv_heads: int, dim: int,
               value_dim: int, state_offset: int = 0) -> torch.Tensor:
    """The gated delta rule over the step's tokens, request by request in order, on what ``conv_prepare`` left:
    ``S <- g_t S``; ``u = beta_t (v_t - S^T k_t)``; ``S <- S + k_t u^T``; ``o_t = S^T q_t`` (head ``h`` reads
    q/k head ``h // (heads / kv_heads)``).  ``state [slots, n]`` holds ``S`` column by column
    (``[heads, value_dim, dim]``) at ``state_offset``.  Returns ``o [T, heads, value_dim]`` 32-bit."""
    _check(prepared, "prepared", dtype=torch.float32)
    if prepared.dim() != 2 or prepared.shape[1] != 2 * kv_heads * dim + heads * value_dim + 2 * heads:
        raise KernelError(f"delta_scan: prepared rows {tuple(prepared.shape)} do not match the head layout")
    _state_row(state, state_offset, heads * dim * value_dim)
    out = torch.empty((prepared.shape[0], heads, value_dim), dtype=torch.float32, device=prepared.device)
    _call("kvb_delta_scan", out.data_ptr(), prepared.data_ptr(), state.data_ptr(), state.stride(0), state_offset,
          ctx.query_start.data_ptr(), ctx.state_slots.data_ptr(), prepared.shape[0], ctx.num_reqs, heads, kv_heads,
          dim, value_dim, _stream())
    return out


def gated_rms_norm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                   scale: float = 1.0, *, gate_act: str = "silu") -> torch.Tensor:
    """``out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * silu(gate[t, h, :]) * scale``:
    ``o [T, H, V]`` 32-bit, ``gate`` and ``out [T, H * V]`` views of the activation type, ``weight [V]``.
    ``gate_act="sigmoid"``: ``sigmoid(gate)`` in place of ``silu(gate)``.  (A norm over all heads together is
    the case ``H = 1``.)"""
    if gate_act not in ("silu", "sigmoid"):
        raise KernelError(f"gated_rms_norm: the gate passes silu or sigmoid, not {gate_act!r}")
    _check(o, "o", dtype=torch.float32)
    _check(gate, "gate", contiguous=False)
    _check(out, "out", dtype=gate.dtype, contiguous=False)
    _check(weight, "weight", dtype=gate.dtype)
    tokens, heads, width = o.shape
    if (tuple(gate.shape) != (tokens, heads * width) or tuple(out.shape) != (tokens, heads * width)
            or weight.numel() != width or (tokens and (gate.stride(1) != 1 or out.stride(1) != 1))):
        raise KernelError(f"gated_rms_norm: gate {tuple(gate.shape)} / out {tuple(out.shape)} / weight do not fit "
                          f"o {tuple(o.shape)}")
    _call("kvb_gated_rms_norm", out.data_ptr(), out.stride(0), o.data_ptr(), gate.data_ptr(), gate.stride(0),
          weight.data_ptr(), tokens, heads, width, float(eps), float(scale), int(gate_act == "sigmoid"),
          _dtype_code(out), _stream())
    return out


def lightning_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, ctx, *,
                   heads: int, dim: int, value_dim: int, q_scale: float = 1.0, state_offset: int = 0) -> torch.Tensor:
    """Linear attention with one fixed decay a head over the step's tokens, request by request in order:
    ``S <- decay[h] S + k_t v_t^T``, ``o_t = S^T q_t`` with ``q_t = silu(q) * q_scale``, ``k_t = silu(k)``,
    ``v_t = silu(v)``.  ``q, k [T, heads * dim]`` and ``v [T, heads * value_dim]`` are views of one tensor of
    projected rows, ``decay [heads]`` 32-bit; ``state [slots, n]`` (32-bit) holds each request's ``S`` column by
    column (``[heads, value_dim, dim]``) at ``state_offset`` of its slot's row and is brought up to date.
    Returns ``o [T, heads, value_dim]`` 32-bit."""
    for name, t in (("q", q), ("k", k), ("v", v)):
        _check(t, name, dtype=q.dtype, contiguous=False)
        if t.stride(1) != 1 or t.shape[0] != q.shape[0]:
            raise KernelError(f"lightning_scan: {name} {tuple(t.shape)} is not a view of the step's rows")
    if q.stride(0) != k.stride(0) or q.stride(0) != v.stride(0):
        raise KernelError("lightning_scan: q, k and v must be views of one tensor of rows")
    if q.shape[1] != heads * dim or k.shape[1] != heads * dim or v.shape[1] != heads * value_dim:
        raise KernelError("lightning_scan: widths do not match the head layout")
    _check(decay, "decay", dtype=torch.float32)
    if decay.numel() != heads:
        raise KernelError(f"lightning_scan: {decay.numel()} decays for {heads} heads")
    _state_row(state, state_offset, heads * dim * value_dim)
    out = torch.empty((q.shape[0], heads, value_dim), dtype=torch.float32, device=q.device)
    # what the scan reads a token, 32-bit: silu(q) times its scale, silu(k), silu(v)
    prepared = torch.empty((q.shape[0], 2 * heads * dim + heads * value_dim), dtype=torch.float32, device=q.device)
    _call("kvb_lightning_scan", out.data_ptr(), prepared.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
          q.stride(0), decay.data_ptr(), state.data_ptr(), state.stride(0), state_offset, ctx.query_start.data_ptr(),
          ctx.state_slots.data_ptr(), q.shape[0], ctx.num_reqs, heads, dim, value_dim, float(q_scale),
          _dtype_code(q), _stream(), kernels=2)
    return out


def gelu_mul(z: torch.Tensor, rows: torch.Tensor, column: int) -> torch.Tensor:
    """``gelu_tanh(z) * rows[:, column:column + dim]`` for ``z [T, dim]``, in 32-bit with one rounding;
    ``rows [T, n]`` of the same type (a table's rows of the step's tokens)."""
    _check(z, "z")
    _check(rows, "rows", dtype=z.dtype, contiguous=False)
    tokens, dim = z.shape
    if rows.dim() != 2 or rows.shape[0] != tokens or column < 0 or column + dim > rows.shape[1] or rows.stride(1) != 1:
        raise KernelError(f"gelu_mul: rows {tuple(rows.shape)} have no columns [{column}, {column + dim}) for z {tuple(z.shape)}")
    out = torch.empty_like(z)
    _call("kvb_gelu_mul", out.data_ptr(), z.data_ptr(), rows.data_ptr(), rows.stride(0), int(column), tokens, dim,
          _dtype_code(z), _stream())
    return out


def qk_prepare(rows: torch.Tensor, positions: torch.Tensor, req_index: torch.Tensor, cos_sin: torch.Tensor | None,
               table: torch.Tensor | None, k_cache: torch.Tensor | None, v_cache: torch.Tensor | None,
               num_heads: int, num_kv_heads: int, head_dim: int, *, rotary_dim: int | None = None,
               norm: str | None = None, q_norm_weight: torch.Tensor | None = None,
               k_norm_weight: torch.Tensor | None = None, eps: float = 0.0, value_from_key: bool = False,
               write_kv: bool = True) -> None:
    """Norm of q and k (``norm``: None, "projection" = one root mean square over all heads of q and one
    over all heads of k, "head" = one per head), rotation of the first ``rotary_dim`` entries of every head
    with the ``[T, rotary_dim/2, 2]`` table ``cos_sin``, and the write of keys and values into their pages;
    q and k of ``rows [T, (H+KVH(+KVH))*D]`` are replaced in place.  ``value_from_key``: the values are the
    keys as projected (before norm and rotation) and ``rows`` has no value section."""
    _check(rows, "rows", contiguous=False)
    _check(positions, "positions", dtype=torch.int32)
    _check(req_index, "req_index", dtype=torch.int32)
    tokens = rows.shape[0]
    if rows.stride(1) != 1:
        raise KernelError("qk_prepare: rows must be contiguous")
    sections = num_heads + num_kv_heads * (1 if value_from_key else 2)
    if rows.shape[1] != sections * head_dim:
        raise KernelError(f"qk_prepare: row width {rows.shape[1]} does not match the head layout")
    rot = head_dim if rotary_dim is None else int(rotary_dim)
    if cos_sin is None:
        rot = 0
    else:
        _check(cos_sin, "cos_sin", dtype=torch.float32)
        if tuple(cos_sin.shape) != (tokens, rot // 2, 2):
            raise KernelError(f"cos_sin has shape {tuple(cos_sin.shape)} for {tokens} tokens and {rot} rotated entries")
    mode = QK_NORM_MODES[norm]
    weight_code = _dtype_code(rows)
    if mode:
        expect_q = num_heads * head_dim if mode == 1 else head_dim
        expect_k = num_kv_heads * head_dim if mode == 1 else head_dim
        _check(q_norm_weight, "q_norm_weight")
        _check(k_norm_weight, "k_norm_weight", dtype=q_norm_weight.dtype)
        if q_norm_weight.numel() != expect_q or k_norm_weight.numel() != expect_k:
            raise KernelError("qk_prepare: norm weights do not match the head layout")
        weight_code = _dtype_code(q_norm_weight)
    k_ptr = v_ptr = table_ptr = None
    table_stride = page_size = num_pages = 0
    if write_kv:
        if k_cache is None or v_cache is None or table is None:
            raise KernelError("a cache write needs k_cache, v_cache and a block table")
        _check(k_cache, "k_cache", dtype=rows.dtype)
        _check(v_cache, "v_cache", dtype=rows.dtype)
        _check(table, "block table", dtype=torch.int32, contiguous=False)
        num_pages, kvh, page_size, d = k_cache.shape
        if (kvh, d) != (num_kv_heads, head_dim) or v_cache.shape != k_cache.shape or table.stride(1) != 1:
            raise KernelError(f"cache shape {tuple(k_cache.shape)} does not match the head layout")
        k_ptr, v_ptr, table_ptr, table_stride = k_cache.data_ptr(), v_cache.data_ptr(), table.data_ptr(), table.stride(0)
    _call("kvb_qk_prepare", rows.data_ptr(), rows.stride(0), positions.data_ptr(), req_index.data_ptr(),
          None if cos_sin is None else cos_sin.data_ptr(),
          None if not mode else q_norm_weight.data_ptr(), None if not mode else k_norm_weight.data_ptr(),
          table_ptr, table_stride, k_ptr, v_ptr, tokens, num_heads, num_kv_heads, head_dim, rot, mode,
          int(bool(value_from_key)), float(eps), page_size, num_pages, _dtype_code(rows), weight_code, _stream())


def glu_clamped(gate_up: torch.Tensor, *, alpha: float, limit: float, shift: float) -> torch.Tensor:
    """``g * sigmoid(alpha * g) * (u + shift)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``
    of a packed ``[T, 2I]`` tensor (gate columns first)."""
    _check(gate_up, "gate_up")
    rows, two_inter = gate_up.shape
    if two_inter % 2:
        raise KernelError(f"gate_up must have an even width, got {two_inter}")
    out = torch.empty((rows, two_inter // 2), dtype=gate_up.dtype, device=gate_up.device)
    _call("kvb_glu_clamped", out.data_ptr(), gate_up.data_ptr(), rows, two_inter // 2, float(alpha), float(limit),
          float(shift), _dtype_code(gate_up), _stream())
    return out


MOE_SCORE_MODES = {"sigmoid": 0, "softmax": 1}


def moe_route(x: torch.Tensor, router: torch.Tensor, top: int, *, score: str = "sigmoid", renormalize: bool = False,
              gate_rows: torch.Tensor | None = None, correction: torch.Tensor | None = None, group_count: int = 1,
              group_keep: int = 1, weight_scale: float = 1.0) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor | None]:
    """Router of a mixture of experts on ``x [T, K]``: 32-bit logits with the 32-bit matrix ``router [E, K]``,
    scores by ``score``, the ``top`` largest per token.  ``correction [E]`` (32-bit): the choice goes by
    ``score + correction``, the weights stay the scores.  ``group_count`` / ``group_keep``: the experts form
    equal groups of neighbours, a group's score is its largest choice score, and only experts of the
    ``group_keep`` best groups can be chosen.  ``weight_scale`` multiplies the weights.  Returns ``(ids [T, top] int32, weights [T, top] float32,
    gates)``; ``gates [T, R]`` = ``sigmoid(gate_rows @ x)`` for the 32-bit rows ``gate_rows [R, K]``, else None."""
    _check(x, "x", contiguous=False)
    _check(router, "router", dtype=torch.float32)
    tokens, k = x.shape
    experts = router.shape[0]
    if router.shape[1] != k or x.stride(1) != 1:
        raise KernelError(f"moe_route: x {tuple(x.shape)} does not match the router {tuple(router.shape)}")
    ids = torch.empty((tokens, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=x.device)
    gates, extra = None, 0
    if gate_rows is not None:
        _check(gate_rows, "gate_rows", dtype=torch.float32)
        if gate_rows.dim() != 2 or gate_rows.shape[1] != k:
            raise KernelError(f"moe_route: gate rows {tuple(gate_rows.shape)} do not match x")
        extra = gate_rows.shape[0]
        gates = torch.empty((tokens, extra), dtype=torch.float32, device=x.device)
    if correction is not None:
        _check(correction, "correction", dtype=torch.float32)
        if correction.numel() != experts:
            raise KernelError(f"moe_route: {correction.numel()} corrections for {experts} experts")
    if (group_count <= 0 or experts % group_count or not 0 < group_keep <= group_count
            or group_keep * (experts // group_count) < top):
        raise KernelError(f"moe_route: {group_keep} of {group_count} groups of {experts} experts must hold {top} experts")
    _call("kvb_moe_route", ids.data_ptr(), weights.data_ptr(), None if gates is None else gates.data_ptr(),
          x.data_ptr(), x.stride(0), router.data_ptr(), None if gate_rows is None else gate_rows.data_ptr(),
          tokens, experts, extra, k, int(top), MOE_SCORE_MODES[score], int(bool(renormalize)),
          None if correction is None else correction.data_ptr(), int(group_count), int(group_keep), float(weight_scale),
          _dtype_code(x), _stream())
    return ids, weights, gates


# bf16 batches of at most this many (token, expert) pairs take the kernel that streams each chosen expert's
# matrices once; larger ones take library products over each expert's run of rows
MOE_GEMV_MAX_PAIRS = int(os.environ.get("KVCORE_B200_MOE_GEMV_PAIRS", "512"))
# up to this many pairs, or fewer than four pairs an expert, each pair streams its expert alone; otherwise
# the pairs are grouped by expert first
MOE_GEMV_SINGLE_PAIRS = int(os.environ.get("KVCORE_B200_MOE_GEMV_SINGLE_PAIRS", "16"))


class ExpertRows:
    """What ``moe_experts`` leaves for ``moe_combine``: the experts' outputs ``rows [R, N]``, where the row of
    pair ``t * top + s`` is that index itself (``row_of_pair`` None) or ``row_of_pair[t * top + s]``, and
    weights still to be applied (``pending_weights`` [T * top], or None)."""

    __slots__ = ("rows", "row_of_pair", "pending_weights")

    def __init__(self, rows, row_of_pair=None, pending_weights=None):
        self.rows, self.row_of_pair, self.pending_weights = rows, row_of_pair, pending_weights


class ExpertGrouping:
    """The (token, expert) pairs of a batch laid out expert by expert (``moe_group``), with the experts' row
    counts on their way to the host: ``begins()`` waits for that copy alone, not for the stream."""

    __slots__ = ("sorted_pairs", "tile_expert", "meta", "row_of_pair", "expert_begin", "max_tiles", "capacity",
                 "_host", "_ready")

    def begins(self) -> list[int]:
        self._ready.synchronize()
        return self._host.tolist()


def moe_group(ids: torch.Tensor, experts: int, *, for_library: bool) -> ExpertGrouping:
    """Group the pairs ``t * top + s`` of ``ids [T, top]`` by expert.  ``for_library``: also the row of every
    pair and where each expert's run begins, the latter copied to pinned host memory behind an event, so that
    a caller who has other work to launch first (a layer whose mixer runs beside its feed-forward) finds the
    counts there when it comes back, without draining the stream."""
    _check(ids, "ids", dtype=torch.int32)
    pairs = ids.numel()
    tile = int(_lib.kvb_moe_tile_rows())
    g = ExpertGrouping()
    g.max_tiles = min(-(-(pairs + experts * (tile - 1)) // tile), pairs)
    g.capacity = g.max_tiles * tile
    g.sorted_pairs = torch.empty(g.capacity, dtype=torch.int32, device=ids.device)
    g.tile_expert = torch.empty(g.max_tiles, dtype=torch.int32, device=ids.device)
    g.meta = torch.empty(4, dtype=torch.int32, device=ids.device)
    g.row_of_pair = torch.empty(pairs, dtype=torch.int32, device=ids.device) if for_library else None
    g.expert_begin = torch.empty(experts + 1, dtype=torch.int32, device=ids.device) if for_library else None
    g._host = g._ready = None
    _call("kvb_moe_align", g.sorted_pairs.data_ptr(), g.tile_expert.data_ptr(), g.meta.data_ptr(),
          None if g.row_of_pair is None else g.row_of_pair.data_ptr(),
          None if g.expert_begin is None else g.expert_begin.data_ptr(), ids.data_ptr(), pairs, experts, g.capacity,
          _stream())
    if for_library:
        g._host = torch.empty(experts + 1, dtype=torch.int32, pin_memory=True)
        g._host.copy_(g.expert_begin, non_blocking=True)
        g._ready = torch.cuda.Event()
        g._ready.record()
    return g


def moe_path(x: torch.Tensor, pairs: int, ff: int) -> str:
    """Which way ``moe_experts`` takes for a batch of ``pairs`` (token, expert) pairs of ``x``'s type."""
    if x.dtype != torch.bfloat16:
        return "tiles"
    if pairs <= MOE_GEMV_MAX_PAIRS and x.shape[1] % 8 == 0 and ff % 8 == 0 and x.stride(0) % 8 == 0:
        return "stream"
    return "library" if not torch.cuda.is_current_stream_capturing() else "tiles"


def moe_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, gate_up: torch.Tensor,
                down: torch.Tensor, *, weight_on_input: bool, path: str | None = None,
                grouping: ExpertGrouping | None = None) -> ExpertRows:
    """The chosen experts of every token: for pair ``t * top + s`` with ``e = ids[t, s]``,
    ``down[e] @ (silu(gate[e] @ a) * (up[e] @ a))``.  ``weight_on_input``: ``a = weights[t, s] * x[t]``
    (rounded to the storage type).  Otherwise ``a = x[t]`` and the weight multiplies the output (the rows
    that enter the last product, or the sum in ``moe_combine``: that product is linear).
    ``gate_up [E, 2F, K]`` (gate rows first), ``down [E, N, F]``.

    Three ways, by ``path`` (default: by type and size).  "tiles": grouped products of this library, one
    accumulator per output in ascending k (all of float32: bit-equal under any batching).  "stream": bf16,
    a handful of pairs, one pass over each chosen expert's matrices.  "library": bf16 prompts, the pairs'
    rows gathered expert by expert at a common stride and one batched library product per matrix over all
    experts (the experts' row counts are read back from the device once per call)."""
    _check(x, "x", contiguous=False)
    _check(ids, "ids", dtype=torch.int32)
    _check(weights, "weights", dtype=torch.float32)
    _check(gate_up, "gate_up", dtype=x.dtype)
    _check(down, "down", dtype=x.dtype)
    tokens, k = x.shape
    top = ids.shape[1]
    experts, two_ff, _ = gate_up.shape
    ff = two_ff // 2
    n = down.shape[1]
    if gate_up.shape[2] != k or down.shape != (experts, n, ff) or x.stride(1) != 1:
        raise KernelError("moe_experts: the experts' matrices do not match the input")
    pairs = tokens * top
    code = _dtype_code(x)
    if path is None:
        path = moe_path(x, pairs, ff)
    if path == "stream" and pairs > MOE_GEMV_SINGLE_PAIRS and pairs >= 4 * experts:
        # enough pairs that experts are shared: the pairs of an expert take one pass over its matrices together
        g = grouping if grouping is not None else moe_group(ids, experts, for_library=False)
        hidden = torch.empty((pairs, ff), dtype=x.dtype, device=x.device)
        _call("kvb_moe_gemv_rows", hidden.data_ptr(), x.data_ptr(), x.stride(0), top,
              weights.data_ptr() if weight_on_input else None, gate_up.data_ptr(), g.sorted_pairs.data_ptr(),
              g.tile_expert.data_ptr(), g.meta.data_ptr(), g.max_tiles, ff, k, 1, _stream())
        out = torch.empty((pairs, n), dtype=x.dtype, device=x.device)
        _call("kvb_moe_gemv_rows", out.data_ptr(), hidden.data_ptr(), hidden.stride(0), 1,
              None if weight_on_input else weights.data_ptr(), down.data_ptr(), g.sorted_pairs.data_ptr(),
              g.tile_expert.data_ptr(), g.meta.data_ptr(), g.max_tiles, n, ff, 0, _stream())
        return ExpertRows(out)
    if path == "stream":
        hidden = torch.empty((pairs, ff), dtype=x.dtype, device=x.device)
        _call("kvb_moe_gemv", hidden.data_ptr(), x.data_ptr(), x.stride(0), top,
              weights.data_ptr() if weight_on_input else None, gate_up.data_ptr(), ids.data_ptr(), pairs, experts,
              ff, k, 1, _stream())
        out = torch.empty((pairs, n), dtype=x.dtype, device=x.device)
        _call("kvb_moe_gemv", out.data_ptr(), hidden.data_ptr(), hidden.stride(0), 1,
              None if weight_on_input else weights.data_ptr(), down.data_ptr(), ids.data_ptr(), pairs, experts,
              n, ff, 0, _stream())
        return ExpertRows(out)
    library = path == "library"
    if grouping is None or (library and grouping.expert_begin is None):
        grouping = moe_group(ids, experts, for_library=library)
    tile = int(_lib.kvb_moe_tile_rows())
    sorted_pairs, tile_expert, meta = grouping.sorted_pairs, grouping.tile_expert, grouping.meta
    row_of_pair, expert_begin = grouping.row_of_pair, grouping.expert_begin
    max_tiles, capacity = grouping.max_tiles, grouping.capacity
    if library:
        begins = grouping.begins()                # the one read-back: how many rows each expert got
        # the common stride: the fullest expert's rows, rounded up to 64 so that the library sees few
        # different shapes (it chooses a kernel anew for every shape it has not met: about a millisecond)
        stride = -(-max(begins[e + 1] - begins[e] for e in range(experts)) // 64) * 64
        gathered = torch.empty((experts, stride, k), dtype=x.dtype, device=x.device)
        _call("kvb_moe_gather", gathered.data_ptr(), x.data_ptr(), x.stride(0), top,
              weights.data_ptr() if weight_on_input else None, sorted_pairs.data_ptr(), expert_begin.data_ptr(),
              experts, stride, row_of_pair.data_ptr(), k, code, _stream())
        # every expert's rows at one stride: two batched library products over all experts (an expert with
        # fewer pairs multiplies zero rows; with one expert far fuller than the rest, expert by expert instead)
        if experts * stride <= 2 * capacity + experts * 64:
            both = torch.bmm(gathered, gate_up.transpose(1, 2))
            hidden = silu_mul(both.view(experts * stride, two_ff), 0).view(experts, stride, ff)
            out = torch.bmm(hidden, down.transpose(1, 2)).view(experts * stride, n)
        else:
            # an expert's rows rounded up to 64 as well (the rows beyond its pairs are zeros): few shapes again
            counts = [min(stride, -(-(begins[e + 1] - begins[e]) // 64) * 64) for e in range(experts)]
            both = torch.zeros((experts, stride, two_ff), dtype=x.dtype, device=x.device)
            for e in range(experts):
                if counts[e]:
                    torch.mm(gathered[e, : counts[e]], gate_up[e].t(), out=both[e, : counts[e]])
            hidden = silu_mul(both.view(experts * stride, two_ff), 0).view(experts, stride, ff)
            out = torch.empty((experts, stride, n), dtype=x.dtype, device=x.device)
            for e in range(experts):
                if counts[e]:
                    torch.mm(hidden[e, : counts[e]], down[e].t(), out=out[e, : counts[e]])
            out = out.view(experts * stride, n)
        return ExpertRows(out, row_of_pair, None if weight_on_input else weights.reshape(-1))
    hidden = torch.empty((pairs, ff), dtype=x.dtype, device=x.device)
    _call("kvb_moe_gemm", hidden.data_ptr(), x.data_ptr(), x.stride(0), top,
          weights.data_ptr() if weight_on_input else None, gate_up.data_ptr(), sorted_pairs.data_ptr(),
          tile_expert.data_ptr(), meta.data_ptr(), max_tiles, ff, k, 1, code, _stream())
    out = torch.empty((pairs, n), dtype=x.dtype, device=x.device)
    _call("kvb_moe_gemm", out.data_ptr(), hidden.data_ptr(), hidden.stride(0), 1,
          None if weight_on_input else weights.data_ptr(), down.data_ptr(), sorted_pairs.data_ptr(),
          tile_expert.data_ptr(), meta.data_ptr(), max_tiles, n, ff, 0, code, _stream())
    return ExpertRows(out)


def moe_combine(expert_out, tokens: int, top: int, shared: torch.Tensor | None = None,
                gates: torch.Tensor | None = None) -> torch.Tensor:
    """``y[t] = sum_s rows[row of pair t * top + s] (+ gates[t, 0] * shared[t])``, summed in 32-bit in slot
    order; ``expert_out`` is what ``moe_experts`` returned (or a plain ``[T * top, N]`` tensor)."""
    if not isinstance(expert_out, ExpertRows):
        expert_out = ExpertRows(expert_out)
    rows = expert_out.rows
    _check(rows, "expert_out")
    width = rows.shape[1]
    if expert_out.row_of_pair is None and rows.shape[0] != tokens * top:
        raise KernelError("moe_combine: one row per (token, slot) is needed")
    if shared is not None:
        _check(shared, "shared", dtype=rows.dtype)
        if tuple(shared.shape) != (tokens, width):
            raise KernelError("moe_combine: the shared expert's rows do not match")
    if gates is not None:
        _check(gates, "gates", dtype=torch.float32)
        if shared is None or gates.shape[0] != tokens:
            raise KernelError("moe_combine: gates need the shared rows they multiply")
    out = torch.empty((tokens, width), dtype=rows.dtype, device=rows.device)
    _call("kvb_moe_combine", out.data_ptr(), rows.data_ptr(), tokens, top,
          None if expert_out.row_of_pair is None else expert_out.row_of_pair.data_ptr(),
          None if expert_out.pending_weights is None else expert_out.pending_weights.data_ptr(),
          None if shared is None else shared.data_ptr(), None if gates is None else gates.data_ptr(),
          0 if gates is None else gates.stride(0), width, _dtype_code(rows), _stream())
    return out


def sample(logits: torch.Tensor, packed_params: torch.Tensor, eps: float) -> torch.Tensor:
    """One token per row of ``logits [S, V]`` float32; ``packed_params [S, 6]`` float64 (on the
    device already, or on the host: then copied): temperature, top_k, top_p, seed low 32 bits, seed
    high 32 bits, index of the sampled token."""
    _check(logits, "logits", dtype=torch.float32)
    rows, vocab = logits.shape
    params = packed_params.to(device=logits.device, dtype=torch.float64, non_blocking=False).contiguous()
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _call("kvb_sample", out.data_ptr(), logits.data_ptr(), params.data_ptr(), rows, vocab, float(eps), _stream())
    return out


__all__ = [
    "KernelError",
    "add_rmsnorm",
    "check_attention_shape",
    "ensure_built",
    "feed_tokens",
    "decode_splits",
    "decode_splits_tma",
    "flash_attention_supported",
    "tc5_prefill_supported",
    "tma_decode_supported",
    "gather_rows",
    "glu_clamped",
    "layer_norm",
    "library_is_loaded",
    "moe_combine",
    "moe_experts",
    "moe_group",
    "moe_path",
    "moe_route",
    "qk_prepare",
    "stream_add",
    "linear",
    "linear_add_residual",
    "linear_silu_mul",
    "linear_stream",
    "norm_linear",
    "set_overlapped_launch",
    "sm_count",
    "trace_start",
    "trace_stop",
    "paged_attention",
    "read_status",
    "peek_status",
    "raise_on_status",
    "require_device",
    "rmsnorm",
    "rope_inplace",
    "rope_kv_write",
    "rope_table",
    "sample",
    "silu_mul",
]
