"""ctypes binding of libxma_b200.so (declared in include/xma_b200.h).

The library is the only implementation of the hot path: if it is missing the import of this module
raises, and every wrapper turns a non-zero status into an exception. There is no fallback.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libxma_b200.so")

F32, F16, BF16, I32, I64 = 0, 1, 2, 3, 4
ROW_PAD = 128
W_NK, W_KN = 0, 1
EPI_PLAIN, EPI_SWIGLU, EPI_DSWIGLU, EPI_SWIGLU_PACKED, EPI_DSWIGLU_PACKED = 0, 1, 2, 3, 4
IMPL_AUTO, IMPL_SIMT, IMPL_TC, IMPL_TC_PAIR = 0, 1, 2, 3

DEV_ID_OUT_OF_RANGE, DEV_WAIT_TIMEOUT, DEV_BAD_TILE = 1, 2, 4
ABI_VERSION = 3
TUNE_GU_PREFETCH, TUNE_TMA_PREFETCH, TUNE_TMA_PREFETCH_MASK, TUNE_EPI_WARPS, TUNE_PLAIN_PAIRS, TUNE_DW_DYNAMIC = 0, 1, 2, 3, 4, 5
TUNE_DSWIGLU_STAGED, TUNE_ODD_TAIL = 6, 7

_DTYPE_CODES = {
    torch.float32: F32,
    torch.float16: F16,
    torch.bfloat16: BF16,
    torch.int32: I32,
    torch.int64: I64,
}

# name -> argument types (every function returns int unless listed in _RESTYPES)
_SIGNATURES = {
    "xma_b200_abi_version": [],
    "xma_b200_error_string": [c_int],
    "xma_b200_continuous_count": [c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p],
    "xma_b200_route_topk_softmax": [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                    c_void_p],
    "xma_b200_route_topk_softmax_bwd": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int,
                                        c_void_p, c_void_p],
    "xma_b200_count_sort_scratch_bytes": [c_int64, c_int],
    "xma_b200_tile_capacity": [c_int64, c_int],
    "xma_b200_count_sort": [c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p,
                            c_void_p],
    "xma_b200_count_sort_static_scratch_limit": [],
    "xma_b200_count_sort_static": [c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p],
    "xma_b200_gather_rows": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_int64,
                             c_void_p, c_int64, c_void_p],
    "xma_b200_spread_rows": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int64,
                             c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p],
    "xma_b200_combine_rows": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p,
                              c_int64, c_void_p],
    "xma_b200_combine_bwd": [c_void_p, c_int, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int64, c_int64,
                             c_void_p, c_void_p],
    "xma_b200_grouped_gemm_rows": [c_void_p, c_int64, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_int64,
                                   c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int,
                                   c_int, c_void_p, c_void_p],
    "xma_b200_grouped_gemm_rows_peer": [c_void_p, c_int64, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_int64,
                                        c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int, c_int64,
                                        c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p],
    "xma_b200_grouped_gemm_dw": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int64,
                                 c_int64, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "xma_b200_grouped_gemm_uses_tensor_cores": [c_int, c_int64, c_int64],
    "xma_b200_grouped_gemm_choice": [c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int],
    "xma_b200_tuning_set": [c_int, c_int],
    "xma_b200_swiglu_fwd": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int64, c_int64,
                            c_void_p],
    "xma_b200_swiglu_bwd": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p,
                            c_int64, c_int, c_int64, c_int64, c_void_p],
    "xma_b200_swiglu_packed_fwd": [c_void_p, c_int64, c_void_p, c_int64, c_int, c_int64, c_int64, c_void_p],
    "xma_b200_swiglu_packed_bwd": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int64,
                                   c_int64, c_void_p],
    "xma_b200_rmsnorm_fwd": [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int64,
                             c_void_p, c_int, c_int64, c_int64, c_float, c_float, c_void_p],
    "xma_b200_rmsnorm_bwd_partial_rows": [c_int64],
    "xma_b200_rmsnorm_bwd": [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p,
                             c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_int64, c_int64, c_float, c_float,
                             c_void_p],
    "xma_b200_router_prob_partial_rows": [c_int64],
    "xma_b200_router_prob_sums": [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_int, c_void_p],
    "xma_b200_load_balancing_loss_bwd": [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p],
    "xma_b200_pack_sequence": [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int,
                               c_void_p, c_void_p],
    "xma_b200_unpack_sequence": [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int,
                                 c_void_p, c_void_p],
    "xma_b200_ep_plan": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                         c_void_p, c_int64, c_void_p, c_void_p],
    "xma_b200_ep_dispatch": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                             c_int, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p],
    "xma_b200_ep_dispatch_part": [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                  c_int, c_int, c_int, c_int, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_void_p,
                                  c_void_p],
    "xma_b200_ep_copy_rows": [c_void_p, c_int, c_void_p, c_int64, c_int64, c_void_p, c_void_p],
    "xma_b200_ep_publish": [c_void_p, c_int64, c_void_p, c_void_p],
    "xma_b200_ep_return": [c_void_p, c_int, c_int64, c_void_p, c_int64, c_int64, c_int, c_void_p, c_int64, c_void_p,
                           c_void_p],
    "xma_b200_exchange_alloc": [c_int64, c_void_p],
    "xma_b200_exchange_free": [c_void_p],
    "xma_b200_exchange_handle_bytes": [],
    "xma_b200_exchange_export": [c_void_p, c_void_p],
    "xma_b200_exchange_open": [c_void_p, c_void_p],
    "xma_b200_exchange_close": [c_void_p],
}
_RESTYPES = {
    "xma_b200_error_string": c_char_p,
    "xma_b200_count_sort_scratch_bytes": c_int64,
    "xma_b200_tile_capacity": c_int64,
    "xma_b200_count_sort_static_scratch_limit": c_int64,
}


def _load() -> ctypes.CDLL:
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            f"{_LIB_PATH} is missing: build it with `python accelerated-model-architectures_b200/build.py` "
            "(the CUDA library is the only implementation of this package; there is no fallback)"
        )
    lib = ctypes.CDLL(_LIB_PATH)
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, c_int)
    if lib.xma_b200_abi_version() != ABI_VERSION:
        raise ImportError(
            f"{_LIB_PATH} has ABI version {lib.xma_b200_abi_version()}, this package binds version {ABI_VERSION}: "
            "rebuild it with `python accelerated-model-architectures_b200/build.py --force`"
        )
    return lib


lib = _load()
EXPORTED_SYMBOLS = tuple(_SIGNATURES)


def error_string(code: int) -> str:
    return lib.xma_b200_error_string(int(code)).decode()


def check(rc: int, name: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{name} failed with status {rc}: {error_string(rc)}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODES[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}") from None


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "xma (B200 build) only runs on CUDA tensors; got a tensor on "
                f"{t.device} (there is no CPU implementation in this package)"
            )


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_STATUS_WORDS: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 the kernels OR error bits into (see include/xma_b200.h)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    word = _STATUS_WORDS.get(idx)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _STATUS_WORDS[idx] = word
    return word


def read_and_clear_device_status(device: torch.device | None = None) -> int:
    """Synchronises, returns the accumulated status bits of the device and clears them."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = status_word(device)
    value = int(word.item())
    if value:
        word.zero_()
    return value


def describe_device_status(value: int) -> str:
    names = []
    if value & DEV_ID_OUT_OF_RANGE:
        names.append("expert/bin id or peer row word out of range")
    if value & DEV_WAIT_TIMEOUT:
        names.append("bounded device-side wait expired")
    if value & DEV_BAD_TILE:
        names.append("inconsistent tile table")
    return f"xma_b200 device status {value}: " + ", ".join(names)


def check_device_status(device: torch.device | None = None) -> None:
    """Synchronises `device` (default: the current one) and raises if any kernel of this library flagged an
    asynchronous condition since the last check: an id or row word out of range that was skipped, a
    bounded wait that expired (the kernel left tiles unwritten), an inconsistent tile table. Results
    computed while the word was non-zero are undefined. The kernels never stop a training loop by
    themselves, so call this where a host synchronisation is acceptable (once per optimizer step, say), or set
    XMA_B200_CHECK_STATUS=1 to have `MoE.forward` check after every call."""
    raise_on_device_status(device)


def raise_on_device_status(device: torch.device | None = None) -> None:
    value = read_and_clear_device_status(device)
    if value:
        raise RuntimeError(describe_device_status(value))
