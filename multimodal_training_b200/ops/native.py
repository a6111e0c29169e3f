"""ctypes binding of the in-tree sm_100a kernel library (``libmmt_b200.so``).

The library exports plain C symbols; tensors cross the boundary as raw device
pointers plus the current CUDA stream.  On a machine with a GPU the library is
mandatory: :func:`lib` raises if it is missing instead of falling back to
PyTorch, so a silent non-native path cannot pass the GPU tests.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_long, c_void_p
from pathlib import Path

import torch

_LIB = None
LIB_PATH = Path(__file__).resolve().parent.parent / "libmmt_b200.so"

# kernel launches issued through this module (bench.py reports the count)
launch_count = 0

_P = c_void_p
_SIGS = {
    "mmt_version": (c_char_p, []),
    "mmt_get_error": (c_int, [_P]),
    "mmt_clear_error": (c_int, []),
    "mmt_error_word_address": (c_void_p, []),
    "mmt_gemm_bf16": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_int, c_int, c_float, c_int, _P]),
    "mmt_rmsnorm_fwd": (c_int, [_P, _P, _P, _P, c_long, c_int, c_float, _P]),
    "mmt_rmsnorm_bwd_parts": (c_int, [c_long]),
    "mmt_rmsnorm_bwd": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_long, c_int, c_int, _P]),
    "mmt_rmsnorm_bwd_add": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_long, c_int, c_int, _P]),
    "mmt_rope": (c_int, [_P, _P, _P, c_long, c_int, c_int, c_long, c_int, _P]),
    "mmt_swiglu_fwd": (c_int, [_P, _P, c_long, c_int, _P]),
    "mmt_swiglu_bwd": (c_int, [_P, _P, _P, c_long, c_int, _P]),
    "mmt_gelu_fwd": (c_int, [_P, _P, c_long, _P]),
    "mmt_gelu_bwd": (c_int, [_P, _P, _P, c_long, _P]),
    "mmt_add": (c_int, [_P, _P, _P, c_long, _P]),
    "mmt_gather_rows": (c_int, [_P, _P, _P, c_long, c_int, c_long, c_long, c_long, c_long, _P]),
    "mmt_scatter_rows": (c_int, [_P, _P, _P, c_long, c_int, c_long, c_long, c_long, c_long, c_int, _P]),
    "mmt_colsum_parts": (c_int, [c_long]),
    "mmt_colsum": (c_int, [_P, _P, _P, c_long, c_int, c_long, c_int, _P]),
    "mmt_ce_stats": (c_int, [_P, _P, _P, _P, _P, c_long, c_int, c_long, c_long, _P]),
    "mmt_ce_grad": (c_int, [_P, _P, _P, _P, _P, c_long, c_int, c_long, c_long, _P]),
    "mmt_adamw": (c_int, [_P, _P, _P, _P, _P, c_long, c_long, c_float, c_float, c_float, c_float, c_float, c_int, _P,
                          _P]),
    "mmt_adamw_bf16": (c_int, [_P, _P, _P, _P, c_long, c_long, c_float, c_float, c_float, c_float, c_float, c_int, _P, _P]),
    "mmt_sumsq": (c_int, [_P, c_long, _P, _P]),
    "mmt_clip_coef": (c_int, [_P, c_float, c_float, _P, _P]),
}


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    """Load (once) and return the kernel library; raises if it is not built."""
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m multimodal_training_b200.csrc.build` "
                "(the GPU path has no PyTorch fallback)")
        _LIB = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGS.items():
            try:
                fn = getattr(_LIB, name)
            except AttributeError:
                continue
            fn.restype = res
            fn.argtypes = args
    return _LIB


def declare(name: str, restype, argtypes) -> None:
    """Register the signature of an entry point defined by another module."""
    _SIGS[name] = (restype, argtypes)
    if _LIB is not None and hasattr(_LIB, name):
        fn = getattr(_LIB, name)
        fn.restype = restype
        fn.argtypes = argtypes


_DEVICE_INDEX = None


def stream() -> int:
    """Raw handle of the current CUDA stream of this process's device.

    ``torch.cuda.current_stream().cuda_stream`` builds a Stream object and resolves the device on every call
    (about 3 us, once per kernel launch); the private raw getter costs well under 0.1 us.  A process drives one
    GPU, so the device index is read once."""
    global _DEVICE_INDEX
    if _DEVICE_INDEX is None:
        _DEVICE_INDEX = torch.cuda.current_device()
    try:
        return torch._C._cuda_getCurrentRawStream(_DEVICE_INDEX)
    except AttributeError:      # a torch build without the raw getter
        return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code}")


# entry points that launch more than one kernel per call
_LAUNCHES = {"mmt_rmsnorm_bwd": 2, "mmt_rmsnorm_bwd_add": 2, "mmt_colsum": 2, "mmt_attn_bwd": 3}


_FN: dict = {}


def call(name: str, *args) -> None:
    """Invoke an int-returning entry point and raise on a non-zero code."""
    global launch_count
    launch_count += _LAUNCHES.get(name, 1)
    fn = _FN.get(name)
    if fn is None:
        fn = _FN[name] = getattr(lib(), name)
    code = fn(*args)
    if code != 0:
        raise RuntimeError(f"{name} failed with code {code}")


def get_error() -> tuple[int, int, int, int]:
    """Synchronise and return the device error word (code, where, block, aux)."""
    buf = (c_int * 4)()
    check(lib().mmt_get_error(buf), "mmt_get_error")
    return tuple(buf)  # type: ignore[return-value]


ERROR_NAMES = {1: "an mbarrier wait ran out", 2: "a wait on a peer's flag ran out",
               3: "an out-of-range access was skipped", 4: "tensor memory could not be allocated"}


def format_error(code: int, where: int, block: int, aux: int) -> str:
    return (f"device-side failure: {ERROR_NAMES.get(code, 'code ' + str(code))} (code={code} site={where} "
            f"block={block} aux={aux}); results of this step are not valid")


def error_word_tensor() -> "torch.Tensor":
    """The device error word as an int32[4] tensor (for an asynchronous copy to pinned host memory)."""
    from ..parallel.symm import tensor_from_ptr
    addr = lib().mmt_error_word_address()
    if not addr:
        raise RuntimeError("the kernel library could not allocate its error word")
    return tensor_from_ptr(addr, (4,), torch.int32, torch.device("cuda", torch.cuda.current_device()))


def raise_on_device_error() -> None:
    code, where, block, aux = get_error()
    if code != 0:
        lib().mmt_clear_error()
        raise RuntimeError(format_error(code, where, block, aux))
