"""CPU checks of the C-ABI library: it loads, exports every declared symbol, and its
argument checks (which run before any CUDA call) report errors in the reference's form."""
import ctypes

import pytest

from dqmoe_b200 import _lib


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _lib.declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), name
    assert set(declared) == set(_lib.SIGNATURES)
    assert lib.dqmoe_abi_version() == 1


def test_workspace_size_is_host_arithmetic():
    lib = _lib.load()
    small = lib.dqmoe_moe_workspace_bytes(64, 1024, 2048, 8, 2, 1024)
    big = lib.dqmoe_moe_workspace_bytes(4096, 4096, 14336, 8, 2, 1024)
    assert 0 < small < big
    assert small % 256 == 0 and big % 256 == 0
    # n*H + n*I bytes of FP8 rows dominate the block-mode workspace
    assert big >= 8192 * (4096 + 14336)
    assert lib.dqmoe_moe_workspace_bytes(64, 1024, 2048, 8, 2, 7) == 0  # unknown mode
    # tensor/channel modes keep a bf16 copy of the intermediate
    assert lib.dqmoe_moe_workspace_bytes(64, 1024, 2048, 8, 2, 512) > small


def test_argument_errors_have_reference_format():
    lib = _lib.load()
    rc = lib.dqmoe_route_topk(None, 4, 8, 9, 0, None, None, None)  # k > E
    assert rc == 1
    msg = lib.dqmoe_last_error().decode()
    assert msg.startswith("[ASSERT FAILED] route.cu:") and "Condition:" in msg
    with pytest.raises(RuntimeError, match=r"\[ASSERT FAILED\]"):
        _lib.check(rc)
    rc = lib.dqmoe_moe_forward(None, None, None, None, None, None, None, None, None, 0, 4, 64, 64, 2, 1, 3, 1, None)
    assert rc == 1 and "quant_mode_value=3" in lib.dqmoe_last_error().decode()
    # T == 0 returns silently like the reference (csrc/pybind11_register.h:125-126)
    assert lib.dqmoe_moe_forward(None, None, None, None, None, None, None, None, None, 0, 0, 64, 64, 2, 1, 0, 1, None) == 0
    # misaligned workspace pointer
    buf = ctypes.create_string_buffer(1024)
    addr = ctypes.addressof(buf)
    mis = ctypes.c_void_p((addr + 255) // 256 * 256 + 8)
    one = ctypes.c_void_p(addr)
    rc = lib.dqmoe_moe_forward(one, None, one, None, one, None, one, one, mis, 0, 4, 64, 64, 2, 1, 0, 1, None)
    assert rc == 1 and "is not aligned!" in lib.dqmoe_last_error().decode()
