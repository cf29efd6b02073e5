"""The C-ABI library loads on a machine without a GPU and exports every symbol the public header
declares; the host layer rejects what it must without touching a device."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "xma_b200.h")
LIB = os.path.join(ROOT, "accelerated-model-architectures_b200", "xma", "lib", "libxma_b200.so")


def declared_symbols() -> list[str]:
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xma_b200_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "xma_b200_continuous_count" in names and "xma_b200_grouped_gemm_rows" in names
    assert len(names) >= 18


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(LIB)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/xma_b200.h but not exported"
    assert lib.xma_b200_abi_version() == 1


def test_python_binding_covers_header():
    from xma import _lib

    assert sorted(_lib.EXPORTED_SYMBOLS) == declared_symbols()


def test_host_side_argument_errors_need_no_gpu():
    from xma import _lib

    lib = _lib.lib
    assert lib.xma_b200_tile_capacity(1024, 8) == 16
    assert lib.xma_b200_tile_capacity(-1, 8) < 0
    assert lib.xma_b200_count_sort_scratch_bytes(10, 2000) < 0  # more than 1024 experts
    assert lib.xma_b200_count_sort_scratch_bytes(8193, 8) == 256 + 2 * 8 * 8
    # null pointers and bad dtypes are refused before anything is launched
    assert lib.xma_b200_continuous_count(None, _lib.I32, 10, 4, None, None, None) == -1
    assert lib.xma_b200_swiglu_fwd(None, 0, None, 0, None, 0, _lib.BF16, 4, 4, None) == -1
    assert lib.xma_b200_swiglu_fwd(None, 0, None, 0, None, 0, _lib.BF16, 0, 4, None) == 0
    assert "dtype" in _lib.error_string(-2)


def test_kernel_backend_contract():
    import xma
    from xma.accelerator import resolve_kernel_backend

    assert resolve_kernel_backend(None) == xma.KernelBackend.cuda
    assert resolve_kernel_backend(xma.KernelBackend.cuda) == xma.KernelBackend.cuda
    for kb in (xma.KernelBackend.torch, xma.KernelBackend.triton):
        with pytest.raises(ValueError):
            resolve_kernel_backend(kb)


def test_no_cpu_fallback():
    """CPU tensors are refused loudly: the package has no CPU implementation."""
    import xma
    from xma.functional import continuous_count, swiglu
    from xma.layers import MoE, SwiGLU

    with pytest.raises(RuntimeError):
        continuous_count(torch.zeros(8, dtype=torch.int32), 4)
    with pytest.raises(RuntimeError):
        swiglu(torch.zeros(2, 4), torch.zeros(2, 4))
    moe = MoE(4, 2, 16, 16, SwiGLU(), True, False, 0.02)
    with pytest.raises(RuntimeError):
        moe(torch.zeros(3, 16))
    assert continuous_count(torch.zeros(8, dtype=torch.int32), 1).tolist() == [8]


def test_state_dict_layout_matches_reference():
    """Parameter/buffer names and shapes of xma/layers/moe/__init__.py:22-43,122-160."""
    from xma.layers import MoE, SwiGLU

    moe = MoE(4, 2, 16, 24, SwiGLU(), True, False, 0.02)
    shapes = {k: tuple(v.shape) for k, v in moe.state_dict().items()}
    assert shapes == {
        "gate.weight": (4, 16),
        "c_fc.weight": (4, 48, 16),
        "c_fc.N_array": (4,),
        "c_fc.K_array": (4,),
        "c_proj.weight": (4, 16, 24),
        "c_proj.N_array": (4,),
        "c_proj.K_array": (4,),
    }
