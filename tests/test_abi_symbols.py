"""The shared library loads on a CPU-only box and exports what the header declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    names = set()
    for h in (ROOT / "include").glob("*.h"):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        names |= set(re.findall(r"\b(mp_[a-z0-9_]+)\s*\(", text))
    return names


@pytest.fixture(scope="module")
def built_lib():
    from mindpipe_b200 import build
    return build.build()


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(str(built_lib))
    syms = declared_symbols()
    assert len(syms) >= 10
    for name in sorted(syms):
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"


def test_ctypes_table_matches_header(built_lib):
    from mindpipe_b200 import _lib
    assert set(_lib.SIGNATURES) == declared_symbols()
    lib = _lib.load()
    assert lib.mp_abi_version() >= 1
    assert lib.mp_status_string(0) == b"ok"
    assert b"workspace" in lib.mp_status_string(-4)


def test_argument_validation_needs_no_gpu(built_lib):
    """Null pointers and bad shapes are rejected before anything touches a device."""
    from mindpipe_b200 import _lib
    lib = _lib.load()
    assert lib.mp_w4a16_quantize(None, 8, 128, 128, None, None, None, None) == -1
    assert lib.mp_act_quant_per_token(None, 4, 64, None, None, None, None) == -1
    assert lib.mp_w4a16_decode_workspace_bytes(16, 4096, 4096) > 0       # partial tiles of the persistent kernels
    assert lib.mp_w4a16_decode_workspace_bytes(32, 4096, 4096) > 0
    assert lib.mp_w4a16_decode_workspace_bytes_ex(16, 4096, 4096, 4) > 0
    assert lib.mp_w4a16_decode_workspace_bytes(128, 4096, 4096) == 0     # decode kernel is M <= 64
    assert lib.mp_w4a16_decode_workspace_bytes(1, 4096, 100) == 0        # K must be a multiple of 128
    assert lib.mp_w4a16_linear_decode_host_many(None, 0, None) == -1
    too_many_rows = (_lib.HostLinear * 1)()
    too_many_rows[0].x_host_f16 = too_many_rows[0].x_stage_f16 = too_many_rows[0].y_stage_f16 = 4096   # never touched
    too_many_rows[0].M, too_many_rows[0].N, too_many_rows[0].K, too_many_rows[0].group = 17, 128, 128, 128
    assert lib.mp_w4a16_linear_decode_host_many(too_many_rows, 1, None) == -2      # host-buffer form: M <= 16
    assert lib.mp_host_buffer_device_alias(None, 0, None) == -1
    assert lib.mp_moe_ep_push_signal(None, None, 2, 1, 256, 128, None, None, 0, None, None, None) == -1
    assert lib.mp_moe_combine_after_peers(None, 2, None, None, None, None, None, 4, 128, 2, None, None, None) == -1
    with pytest.raises(_lib.MindPipeKernelError, match="invalid argument"):
        _lib.check(-1, "probe", M=1)


def test_ops_reject_cpu_tensors():
    import torch
    from mindpipe_b200 import ops
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.act_quant_per_token(torch.zeros(2, 64, dtype=torch.float16))
    with pytest.raises(TypeError):
        ops.act_quant_per_token([1, 2, 3])


def test_decode_kernel_selector_and_its_workspace_rule(built_lib):
    """mp_set_decode_kernel is host state (the default for calls that do not choose): it returns the previous
    choice, rejects unknown kinds, and decides whether a decode call of at most 16 rows wants scratch (the
    partial tiles of the persistent tcgen05 kernels)."""
    from mindpipe_b200 import _lib, ops
    lib = _lib.load()
    MMA_SYNC, UMMA, AUTO = 0, 1, 2
    first = lib.mp_set_decode_kernel(AUTO)
    try:
        assert first in (MMA_SYNC, UMMA, AUTO)
        assert lib.mp_set_decode_kernel(7) == -1                       # invalid argument, choice unchanged
        assert lib.mp_set_decode_kernel(AUTO) == AUTO
        # every kernel choice but the mma.sync ring kernel may cut row blocks between blocks of a persistent
        # grid and then wants the same, shape-independent scratch
        need = lib.mp_w4a16_decode_workspace_bytes(16, 28672, 8192)
        assert need > 0
        for m, n, k in [(16, 22016, 4096), (8, 28672, 8192), (1, 4096, 4096), (16, 8192, 28672)]:
            assert lib.mp_w4a16_decode_workspace_bytes(m, n, k) == need
        assert lib.mp_set_decode_kernel(UMMA) == AUTO
        assert lib.mp_w4a16_decode_workspace_bytes(1, 4096, 4096) == need
        assert lib.mp_set_decode_kernel(MMA_SYNC) == UMMA
        assert lib.mp_w4a16_decode_workspace_bytes(16, 8192, 28672) == 0
        assert ops.set_decode_kernel("auto") == "mma_sync"
        with pytest.raises(ValueError, match="unknown decode kernel"):
            ops.set_decode_kernel("wgmma")
        # the default rule: the tcgen05 kernel for 9..16 tokens on 70B-sized weights with a workspace, else mma.sync
        assert ops.w4a16_decode_kernel_choice(16, 22016, 4096) == "umma"
        assert ops.w4a16_decode_kernel_choice(16, 22016, 4096, have_workspace=False) == "mma_sync"
        assert ops.w4a16_decode_kernel_choice(8, 22016, 4096) == "mma_sync"
        assert ops.w4a16_decode_kernel_choice(16, 4096, 4096) == "mma_sync"
        assert ops.w4a16_decode_kernel_choice(32, 28672, 8192) == "umma"          # 17..64 rows: wide activation tile
        assert ops.w4a16_decode_kernel_choice(32, 4096, 11008) == "mma_sync"
        assert ops.w4a16_decode_kernel_choice(64, 28672, 8192) == "umma"
        assert ops.w4a16_decode_kernel_choice(64, 8192, 8192) == "mma_sync"
        assert ops.w4a16_decode_kernel_choice(64, 28672, 8192, have_workspace=False) == "mma_sync"
        assert lib.mp_w4a16_decode_kernel_choice(65, 4096, 4096, 1) < 0
        assert ops.decode_options() == 0
        assert ops.decode_options(kernel="umma", pdl=True) == 0x2 | 0x10
        assert ops.decode_options(kernel="mma_sync", pdl=False) == 0x1 | 0x20
        with pytest.raises(ValueError):
            ops.decode_options(kernel="wgmma")
        # per-call options are validated before anything touches a device
        assert lib.mp_w4a16_linear_decode_opts(None, None, None, None, None, 1, 8, 128, 128, None, 0, 0x3, None) == -1
        assert lib.mp_w4a16_linear_decode_opts(None, None, None, None, None, 1, 8, 128, 128, None, 0, 0x30, None) == -1
    finally:
        lib.mp_set_decode_kernel(first)
