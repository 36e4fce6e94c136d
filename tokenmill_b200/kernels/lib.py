"""ctypes binding of the compiled kernel library.

There is no other implementation behind these calls: if the library cannot be built or loaded, or a
launch reports an error, an exception is raised. ``launch_count`` counts every kernel entry point
called, which is what the benchmark reports as its own launches.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p

from . import build as _build


class KernelError(RuntimeError):
    pass


_REFUSALS = {
    90001: "unsupported shape for this kernel",
    90002: "unsupported dtype for this kernel",
    90003: "scratch buffer missing or too small",
    90004: "size beyond the entry point's fixed scratch capacity",
    90005: "device-side wait ran out (kernel gave up and reported instead of hanging)",
    90006: "tensor map could not be encoded",
}

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None
launch_count = 0

_P, _I, _F, _LL = c_void_p, c_int, c_float, c_longlong

# name -> argument types (the trailing stream pointer included)
_SIGNATURES: dict[str, list] = {
    "tm_add_rmsnorm": [_I, _P, _P, _P, _I, _LL, _P, _P, _P, _P, _F, _P, _I, _I, _P],
    "tm_qkv_rope_write": [_I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    "tm_kv_cache_write": [_I, _P, _P, _P, _P, _P, _I, _I, _P],
    "tm_paged_attention": [_I, _P, _P, _P, _P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I,
                           _I, _P],
    "tm_attention_combine": [_I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "tm_decode_attention_bf16": [_P, _P, _P, _P, _I, _P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P],
    "tm_decode_attention_units_bf16": [_P, _P, _P, _LL, _P, _I, _P, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I,
                                       _I, _P, _P],
    "tm_decode_attention_units_rope_bf16": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _LL, _P, _I, _P, _P, _P, _P, _I, _I, _P, _P, _P,
                                            _P, _I, _I, _I, _I, _F, _I, _I, _P, _P],
    "tm_decode_attention_units_slots": [_I, _I],
    "tm_prefill_attention_bf16": [_P, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P],
    "tm_prefill_attention_tc_timing": [_P],
    "tm_decode_attention_units_timing": [_P],
    "tm_prefill_attention_tc_bf16": [_P, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P, _P],
    "tm_swiglu": [_I, _P, _P, _I, _I, _P],
    "tm_skinny_linear": [_P, _I, _P, _P, _P, _I, _I, _P, _I, _I, _I, _I, _I, _P],
    "tm_skinny_qkv_rope_write": [_P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "tm_skinny_gate_up_swiglu": [_P, _I, _P, _P, _I, _I, _I, _I, _P],
    "tm_tc_linear": [_P, _I, _P, _P, _I, _I, _I, _I, _P, _P],
    "tm_tc_linear_add_f32": [_P, _I, _P, _P, _I, _I, _I, _I, _P, _P],
    "tm_tc_gate_up_swiglu": [_P, _I, _P, _P, _I, _I, _I, _I, _P, _P],
    "tm_tc_qkv_rope_write": [_P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "tm_decode_fused": [_P, _P],
    "tm_decode_fused_max_tokens": [_I, _I, _I, _I, _I, _I],
    "tm_lm_head_bf16": [_P, _P, _P, _I, _I, _I, _P, _P],
    "tm_stream_linear_bf16": [_P, _P, _P, _I, _I, _I, _P, _P],
    "tm_lm_head_argmax_bf16": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P],
    "tm_stream_linear_slices": [_I],
    "tm_swiglu_partials": [_P, _I, _LL, _P, _I, _I, _P],
    "tm_gemm_f32_nt": [_P, _I, _P, _P, _P, _I, _I, _I, _I, _P],
    "tm_argmax": [_P, _I, _I, _LL, _P, _P, _P, _P],
    "tm_sample": [_P, _I, _I, _LL, _P, _P, _P, _P, _P, _P, _I, _P, _P],
}


def register_signature(name: str, argtypes: list) -> None:
    """Declare one more exported entry point (used by kernel files added later)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        _bind(_lib, name, argtypes)


def _bind(lib: ctypes.CDLL, name: str, argtypes: list) -> None:
    try:
        fn = getattr(lib, name)
    except AttributeError:
        raise KernelError(f"the kernel library lacks the entry point {name}") from None
    fn.argtypes = argtypes
    fn.restype = c_int


def load() -> ctypes.CDLL:
    """Build (if needed) and load the library. Raises if that is impossible."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.build()
            lib = ctypes.CDLL(str(path))
            for name, argtypes in _SIGNATURES.items():
                _bind(lib, name, argtypes)
            _lib = lib
    return _lib


def library_file() -> str:
    return str(_build.library_path())


def call(name: str, *args) -> None:
    """Call an entry point; a non-zero status raises."""
    global launch_count
    lib = load()
    status = getattr(lib, name)(*args)
    launch_count += 1
    if status != 0:
        reason = _REFUSALS.get(status)
        if reason is None:
            reason = f"CUDA error {status}"
            try:
                import torch

                reason += f" ({torch.cuda.cudart().cudaGetErrorString(status)})"  # type: ignore[attr-defined]
            except Exception:
                pass
        raise KernelError(f"{name}: {reason}")
