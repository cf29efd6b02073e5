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
    assert lib.xma_b200_abi_version() == 3


def test_python_binding_covers_header():
    from xma import _lib

    assert sorted(_lib.EXPORTED_SYMBOLS) == declared_symbols()


def test_host_side_argument_errors_need_no_gpu():
    from xma import _lib

    lib = _lib.lib
    assert lib.xma_b200_tile_capacity(1024, 8) == 16
    assert lib.xma_b200_tile_capacity(-1, 8) < 0
    assert lib.xma_b200_count_sort_scratch_bytes(10, 2000) < 0  # more than 1024 experts
    # 2 tiles of 8192 ids, 1 chunk of the scan: ticket | counts [2][8] u32 | chunk base [8] u32 | status words [8] u64
    assert lib.xma_b200_count_sort_scratch_bytes(8193, 8) == 256 + 2 * 8 * 4 + 8 * 4 + 8 * 8
    # null pointers and bad dtypes are refused before anything is launched
    assert lib.xma_b200_continuous_count(None, _lib.I32, 10, 4, None, None, None) == -1
    assert lib.xma_b200_swiglu_fwd(None, 0, None, 0, None, 0, _lib.BF16, 4, 4, None) == -1
    assert lib.xma_b200_swiglu_fwd(None, 0, None, 0, None, 0, _lib.BF16, 0, 4, None) == 0
    assert "dtype" in _lib.error_string(-2)


def test_later_entry_points_reject_bad_arguments_without_a_gpu():
    """pack / unpack_sequence, fused_residual_add_rmsnorm and the load-balancing loss: shape and pointer errors are
    answered on the host, and an empty problem is a successful no-op."""
    from xma import _lib

    lib = _lib.lib
    NULL, DTYPE, SHAPE = -1, -2, -3
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.cast(buf, ctypes.c_void_p)
    for fn in (lib.xma_b200_pack_sequence, lib.xma_b200_unpack_sequence):
        assert fn(p, p, p, _lib.I32, -1, 4, 8, 16, 1, None, None) == SHAPE
        assert fn(p, p, p, _lib.I32, 0, 4, 8, 16, 1, None, None) == 0       # no sequences
        assert fn(p, p, p, _lib.I32, 2, 4, 8, 0, 1, None, None) == 0        # empty rows
        assert fn(p, p, None, _lib.I32, 2, 4, 8, 16, 1, None, None) == NULL  # no offsets
        assert fn(p, None, p, _lib.I32, 2, 4, 8, 16, 1, None, None) == NULL  # no destination
        assert fn(p, p, p, _lib.F32, 2, 4, 8, 16, 1, None, None) == DTYPE    # offsets must be int32 / int64
    assert lib.xma_b200_pack_sequence(p, None, p, _lib.I32, 2, 4, 0, 16, 1, None, None) == 0  # nothing to write
    # rmsnorm: empty problems, missing tensors, a residual without the output for the updated stream
    f = ctypes.c_float
    assert lib.xma_b200_rmsnorm_fwd(p, 8, None, 0, None, p, 8, None, 0, None, _lib.BF16, 0, 8, f(1e-5), f(1.0), None) == 0
    assert lib.xma_b200_rmsnorm_fwd(None, 8, None, 0, None, p, 8, None, 0, None, _lib.BF16, 4, 8, f(1e-5), f(1.0), None) == NULL
    assert lib.xma_b200_rmsnorm_fwd(p, 8, p, 8, None, p, 8, None, 0, None, _lib.BF16, 4, 8, f(1e-5), f(1.0), None) == NULL
    assert lib.xma_b200_rmsnorm_fwd(p, 8, None, 0, None, p, 8, None, 0, None, _lib.I32, 4, 8, f(1e-5), f(1.0), None) == DTYPE
    assert lib.xma_b200_rmsnorm_bwd(p, 8, None, p, 8, None, 0, None, p, 8, None, 0, p, 0, _lib.BF16, 4, 8, f(1e-5), f(1.0), None) == SHAPE
    assert lib.xma_b200_rmsnorm_bwd_partial_rows(10) == 10 and lib.xma_b200_rmsnorm_bwd_partial_rows(10 ** 9) >= 148
    # load-balancing loss: more than 1024 experts, a row stride shorter than a row, no logits
    assert lib.xma_b200_router_prob_sums(p, _lib.BF16, 8, 4, 2000, ctypes.cast(buf, ctypes.POINTER(f)), 4, None) == SHAPE
    assert lib.xma_b200_router_prob_sums(p, _lib.BF16, 4, 4, 8, ctypes.cast(buf, ctypes.POINTER(f)), 4, None) == SHAPE
    assert lib.xma_b200_load_balancing_loss_bwd(None, _lib.BF16, 8, 4, 8, None, None, None) == NULL
    assert lib.xma_b200_load_balancing_loss_bwd(None, _lib.BF16, 8, 0, 8, None, None, None) == 0


def test_expert_parallel_entry_points_reject_bad_arguments_without_a_gpu():
    from xma._lib import lib

    NULL, DTYPE, SHAPE, LARGE = -1, -2, -3, -8  # status codes of the C ABI
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.cast(buf, ctypes.c_void_p)
    out = ctypes.c_void_p()
    # ep_plan: null tables, experts not divisible by the ranks, rank outside the world
    assert lib.xma_b200_ep_plan(None, 2, 8, 0, p, p, p, p, p, 4, p, 512, None, None) == NULL
    assert lib.xma_b200_ep_plan(p, 3, 8, 0, p, p, p, p, p, 4, p, 512, None, None) == SHAPE
    assert lib.xma_b200_ep_plan(p, 2, 8, 2, p, p, p, p, p, 4, p, 512, None, None) == SHAPE
    # ep_dispatch: nothing to move is fine, null source is not, more rows than an origin word addresses is too large
    args = lambda src, rows: (src, 2, 64, p, p, None, 2, p, 8, 2, 0, rows, 64, p, p, 1 << 20, None, None)
    assert lib.xma_b200_ep_dispatch(*args(None, 0)) == 0
    assert lib.xma_b200_ep_dispatch(*args(None, 16)) == NULL
    assert lib.xma_b200_ep_dispatch(*args(p, (1 << 24) + 1)) == LARGE
    assert lib.xma_b200_ep_dispatch(p, 9, 64, p, p, None, 2, p, 8, 2, 0, 16, 64, p, p, 1 << 20, None, None) == DTYPE
    # ep_copy_rows / ep_return / ep_publish
    assert lib.xma_b200_ep_copy_rows(p, 2, None, 16, 64, p, None) == NULL
    assert lib.xma_b200_ep_copy_rows(p, 2, p, 16, 0, p, None) == SHAPE
    assert lib.xma_b200_ep_return(p, 2, 64, p, 16, 64, 0, p, 128, None, None) == SHAPE
    assert lib.xma_b200_ep_return(p, 2, 64, p, 0, 64, 2, p, 128, None, None) == 0
    assert lib.xma_b200_ep_publish(p, 4, None, None) == NULL
    # a row map is required (and only the plain epilogue allowed) when rows go to other ranks' buffers
    gemm = lambda row_map, epilogue, world=2, cap=512: lib.xma_b200_grouped_gemm_rows_peer(
        p, 64, p, 0, p, 64, None, 0, row_map, p, world, cap, p, p, 2, 4, 64, 64, epilogue, 2, 0, None, None)
    assert gemm(None, 0) == SHAPE
    assert gemm(p, 1) == SHAPE
    # ... and the table's size and the buffers' row count bound what a row-map word may name
    assert gemm(p, 0, world=0) == SHAPE
    assert gemm(p, 0, world=129) == SHAPE
    assert gemm(p, 0, cap=0) == SHAPE
    assert gemm(p, 0, cap=(1 << 24) + 1) == SHAPE
    # host-only queries and switches
    assert lib.xma_b200_grouped_gemm_choice(0, 0, 8, 264, 4096, 4096, 0, 0, 0) == 1  # fp32: CUDA cores
    assert lib.xma_b200_tuning_set(99, 0) == SHAPE
    previous = lib.xma_b200_tuning_set(1, 7)
    assert lib.xma_b200_tuning_set(1, previous) == 7
    # exchange buffers
    assert lib.xma_b200_exchange_alloc(0, ctypes.byref(out)) == SHAPE
    assert lib.xma_b200_exchange_alloc(1024, None) == NULL
    assert lib.xma_b200_exchange_export(None, buf) == NULL
    assert lib.xma_b200_exchange_open(None, ctypes.byref(out)) == NULL
    assert lib.xma_b200_exchange_free(None) == 0 and lib.xma_b200_exchange_close(None) == 0
    assert lib.xma_b200_exchange_handle_bytes() == 64


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


def test_no_cpu_fallback_in_the_later_functions():
    """fused_residual_add_rmsnorm, load_balancing_loss, pack_sequence / unpack_sequence: the reference's argument
    checks apply first, CPU tensors are refused loudly, a backend other than cuda raises ValueError."""
    import xma
    from xma.functional import fused_residual_add_rmsnorm, load_balancing_loss, pack_sequence, unpack_sequence

    x, w = torch.zeros(4, 8), torch.ones(8)
    with pytest.raises(RuntimeError):
        fused_residual_add_rmsnorm(x, None, w, 1e-5)
    with pytest.raises(AssertionError):
        fused_residual_add_rmsnorm(torch.zeros(8), None, w, 1e-5)  # x should be 2D
    with pytest.raises(ValueError):
        fused_residual_add_rmsnorm(x, None, w, 1e-5, kernel_backend=xma.KernelBackend.triton)
    with pytest.raises(RuntimeError):
        load_balancing_loss(torch.zeros(4, 8), 2)
    with pytest.raises(AssertionError):
        load_balancing_loss(torch.zeros(4, 8), 9)  # top-k above the number of experts
    padded, cu = torch.zeros(2, 4, 3), torch.tensor([0, 2, 5], dtype=torch.int32)
    with pytest.raises(RuntimeError):
        pack_sequence([padded], cu, 5)
    with pytest.raises(RuntimeError):
        unpack_sequence([torch.zeros(5, 3)], cu, 2, 4)
    with pytest.raises(AssertionError):
        pack_sequence([padded], cu, 5, "middle")
    with pytest.raises(AssertionError):
        pack_sequence(padded, cu, 5)  # a list or tuple of tensors, as in the reference
    with pytest.raises(AssertionError):
        unpack_sequence([torch.zeros(5, 3)], cu, 3, 4)  # batch_size must match cu_seqlens
    with pytest.raises(ValueError):
        pack_sequence([padded], cu, 5, kernel_backend=xma.KernelBackend.torch)


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
