"""Loading the native libraries (building them at first use).

``cuda()`` is the ctypes handle of ``libaxon_cuda.so``; ``host()`` is the
``axon_host`` extension module.  There is no fallback: when a library cannot be
built or loaded the error says so and nothing runs.
"""

from __future__ import annotations

import ctypes
import importlib.util
import threading
from ctypes import c_char_p, c_double, c_float, c_int, c_int64, c_longlong, c_void_p
from typing import Any, Optional

_lock = threading.Lock()
_cuda: Optional[ctypes.CDLL] = None
_host: Any = None


class NativeLibraryError(RuntimeError):
    """The engine's native code could not be built or loaded."""


class KvLayout(ctypes.Structure):
    """Mirror of ``AxonKvLayout``: where a layer's keys and values lie in its page pool."""

    _fields_ = [
        ("block_table", c_void_p),
        ("table_stride", ctypes.c_int32),
        ("page_size", ctypes.c_int32),
        ("kv_heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("page_stride", c_int64),
        ("entry_offset", c_int64),
        ("v_offset", c_int64),
        ("v_dim", ctypes.c_int32),
        ("planes", ctypes.c_int32),
        ("n_pages", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("fault", c_void_p),
    ]


P = c_void_p
_SIGNATURES = {
    "axon_embed": [P, P, c_int, P, c_int, c_int, c_float, P],
    "axon_rmsnorm": [P, P, P, P, c_int, c_int, c_int, c_float, c_int, P],
    "axon_rmsnorm_fold": [P, P, P, P, c_int, c_int, c_int, c_float, c_int, P, c_int, c_int, P, P],
    "axon_fold_partials": [P, c_int, c_int, P, P, c_int, c_int, c_int, c_int, c_int, P],
    "axon_gemm_plain": [P, c_int, P, c_int, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, P],
    "axon_swiglu": [P, P, c_int, c_int, c_int, P],
    "axon_rope_table": [P, P, P, c_int, c_int, c_float, P],
    "axon_rope_kv_write": [P, P, P, P, P, P, c_int, ctypes.POINTER(KvLayout), c_int, c_int, c_int, c_int, c_int,
                           P, c_int, c_int, P, P],
    "axon_attention_plain": [P, P, c_int, P, P, P, ctypes.POINTER(KvLayout), c_int, c_int, c_float, c_int, P],
    "axon_residual_add": [P, P, c_int, c_longlong, P],
    "axon_convert": [P, c_int, P, c_int, c_longlong, P],
    "axon_argmax": [P, P, c_int, c_int, c_longlong, P],
    "axon_repeat_penalty": [P, P, P, c_int, c_int, c_longlong, c_int, P],
    "axon_argmax_rows": [P, P, P, c_int, c_int, c_longlong, P],
    "axon_gather_rows": [P, P, P, c_int, c_int, c_longlong, P],
    "axon_topk": [P, P, P, P, P, c_int, c_int, c_longlong, P],
    "axon_sample_temperature": [P, P, P, P, P, c_int, c_int, c_longlong, P],
    "axon_gemm_tc": [P, P, P, P, c_int, c_int, c_int, c_int, c_int, P],
    "axon_gemm_tc_status": [],
    "axon_gemm_tc_clear_status": [],
    "axon_gemm_tc_small": [P, P, P, P, c_int, c_int, c_int, c_int, c_int, P, c_longlong, P, c_int, c_int, c_int,
                           ctypes.POINTER(c_int), P],
    "axon_gemm_prefers_swapped": [c_int, c_int, c_int, c_int, c_int],
    "axon_mma_probe": [c_int, c_int, P, P, P],
    "axon_attention_fa": [P, P, P, P, c_int, P, c_int, ctypes.POINTER(KvLayout), c_int, c_float, c_int, c_int,
                          c_int, c_int, P, P, P],
    "axon_attention_fa_decode_fused": [P, P, c_int, c_int, P, P, c_int, P, P, P, c_int, ctypes.POINTER(KvLayout), c_int,
                                       c_float, c_int, c_int, c_int, c_int, P, P, P],
    "axon_attention_tc": [P, P, P, P, c_int, P, c_int, ctypes.POINTER(KvLayout), c_int, c_float, c_int, c_int, P],
    "axon_attention_tc_status": [],
}
_OPTIONAL_SIGNATURES: dict = {}


def register_signature(name: str, argtypes: list, optional: bool = True) -> None:
    """Declare a launcher that a kernel module adds to the library."""
    (_OPTIONAL_SIGNATURES if optional else _SIGNATURES)[name] = argtypes
    if _cuda is not None:
        _declare(_cuda, name, argtypes)


def _declare(lib: ctypes.CDLL, name: str, argtypes: list) -> None:
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = c_int


def cuda() -> ctypes.CDLL:
    """The CUDA library; built for sm_100a on first use."""
    global _cuda
    if _cuda is not None:
        return _cuda
    with _lock:
        if _cuda is not None:
            return _cuda
        from ..csrc import build
        try:
            path = build.build_cuda()
            lib = ctypes.CDLL(path)
        except (build.BuildError, OSError) as e:
            raise NativeLibraryError(
                f"axon_b200's CUDA kernels are not available ({e}); there is no fallback path") from e
        lib.axon_last_error.restype = c_char_p
        lib.axon_last_error.argtypes = []
        lib.axon_topk_max.restype = c_int
        lib.axon_topk_max.argtypes = []
        lib.axon_gemm_tc_force_tile.restype = None
        lib.axon_gemm_modelled_us.argtypes = [c_int, c_int, c_int, c_int, c_int]
        lib.axon_gemm_modelled_us.restype = ctypes.c_double
        lib.axon_gemm_tc_force_tile.argtypes = [c_int, c_int]
        lib.axon_gemm_tc_force_plain_out.restype = None
        lib.axon_gemm_tc_force_plain_out.argtypes = [c_int]
        lib.axon_gemm_tc_test_stuck_wait.restype = None
        lib.axon_gemm_tc_test_stuck_wait.argtypes = [ctypes.c_uint]
        for name, sig in list(_SIGNATURES.items()) + list(_OPTIONAL_SIGNATURES.items()):
            try:
                _declare(lib, name, sig)
            except AttributeError:
                if name in _SIGNATURES:
                    raise NativeLibraryError(f"libaxon_cuda.so lacks {name}") from None
        _cuda = lib
        return lib


def host() -> Any:
    """The host extension module (pages, cache manager, scheduler, sampler)."""
    global _host
    if _host is not None:
        return _host
    with _lock:
        if _host is not None:
            return _host
        from ..csrc import build
        try:
            path = build.build_host()
            spec = importlib.util.spec_from_file_location("axon_host", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
        except (build.BuildError, ImportError, OSError) as e:
            raise NativeLibraryError(f"axon_b200's host library is not available ({e})") from e
        _host = mod
        return mod


class KernelError(RuntimeError):
    """A launcher refused its arguments or the launch failed."""


_launches = 0


def launch_count() -> int:
    """How many kernel launchers of the library have been called so far (each launches
    its kernels on the current stream; benches report the difference over a region)."""
    return _launches


def add_launches(n: int) -> None:
    """Count launches that did not go through a launcher call: a replayed CUDA graph
    launches every kernel that was captured into it."""
    global _launches
    _launches += n


def check(status: int) -> None:
    global _launches
    _launches += 1
    if status != 0:
        msg = cuda().axon_last_error().decode("utf-8", "replace")
        raise KernelError(msg or f"kernel launcher returned {status}")


def current_stream() -> int:
    """The raw handle of PyTorch's current CUDA stream on the current device.  Asked for at
    every launch, so it goes through the one C call PyTorch has for it when that exists
    (``torch.cuda.current_stream()`` costs several microseconds of Python)."""
    import torch
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None:
        return raw(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream
