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


def test_plugin_descriptor_host_calls():
    """The plugin-shaped front end: creation checks, workspace arithmetic and serialisation need no GPU."""
    from dqmoe_b200 import plugin
    p = plugin.MoePlugin(8, 2, 1024, 2048, 64, quant_mode=1024, output_type=plugin.DT_HALF)
    f = p.fields
    assert f["number_of_experts"] == 8 and f["quant_mode"] == 1024 and f["output_type"] == plugin.DT_HALF
    lib = _lib.load()
    layer = lib.dqmoe_moe_workspace_bytes(64, 1024, 2048, 8, 2, 1024)
    # HALF output stages the bf16 result [T, k, H] behind the layer's workspace
    assert p.workspace_size(64) == layer + 64 * 2 * 1024 * 2
    assert p.workspace_size(65) == 0 and p.workspace_size(-1) == 0
    direct = plugin.MoePlugin(8, 2, 1024, 2048, 64, quant_mode=1024, output_type=plugin.DT_BF16)
    assert direct.workspace_size(64) == layer
    blob = p.serialize()
    assert len(blob) == 36
    assert plugin.MoePlugin.deserialize(blob).fields == f
    with pytest.raises(RuntimeError, match="expected 36"):
        plugin.MoePlugin.deserialize(blob[:-4])
    # use_bias = 1 and FLOAT operands (with FLOAT output) are accepted
    assert plugin.MoePlugin(8, 2, 1024, 2048, 64, use_bias=1).fields["use_bias"] == 1
    f32 = plugin.MoePlugin(8, 2, 1024, 2048, 64, type=plugin.DT_FLOAT, output_type=plugin.DT_FLOAT, quant_mode=0)
    assert f32.workspace_size(64) == lib.dqmoe_moe_workspace_bytes_f32(64, 1024, 2048, 8, 2)
    for bad in (dict(use_bias=2), dict(type=plugin.DT_FLOAT, quant_mode=0),
                dict(type=plugin.DT_FLOAT, quant_mode=512, output_type=plugin.DT_FLOAT),
                dict(type=plugin.DT_HALF, quant_mode=0, output_type=plugin.DT_BF16),
                dict(type=plugin.DT_HALF, quant_mode=512, output_type=plugin.DT_HALF),
                dict(type=plugin.DT_BF16, quant_mode=512), dict(type=plugin.DT_FP8, quant_mode=0),
                dict(output_type=3)):
        with pytest.raises(RuntimeError, match=r"\[ASSERT FAILED\] plugin.cu"):
            plugin.MoePlugin(8, 2, 1024, 2048, 64, **bad)
    with pytest.raises(RuntimeError, match="expert_hidden_size=1000"):
        plugin.MoePlugin(8, 2, 1000, 2048, 64)
