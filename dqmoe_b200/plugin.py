"""The layer behind the reference's TensorRT-plugin interface (test/trt_test.py:97-150).

`MoePlugin` holds the nine creation fields of the "mixture_of_experts" plugin and offers the
calls a TensorRT plugin class forwards: workspace size, enqueue with the plugin's input
list, serialise / deserialise. It binds the dqmoe_plugin_* entry points of the C ABI; torch
only supplies device memory and the stream.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import _lib

# nvinfer1::DataType codes used by the `type` / `output_type` fields
DT_FLOAT, DT_HALF, DT_FP8, DT_BF16 = 0, 1, 6, 7
_TORCH_OUT = {DT_FLOAT: torch.float32, DT_HALF: torch.float16, DT_BF16: torch.bfloat16}
# input order of the plugin (test/trt_test.py:140-150)
INPUT_NAMES = ("input", "weight1", "weight2", "index", "bias1", "bias2", "actscale", "scale_a", "scale_b")


class Fields(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "number_of_experts", "top_k", "expert_hidden_size", "expert_inter_size", "max_num_tokens", "use_bias",
        "type", "output_type", "quant_mode")]


class MoePlugin:
    def __init__(self, number_of_experts: int, top_k: int, expert_hidden_size: int, expert_inter_size: int,
                 max_num_tokens: int, use_bias: int = 0, type: int = DT_FP8, output_type: int = DT_BF16,
                 quant_mode: int = 512, _handle: Optional[int] = None):
        self._lib = _lib.load()
        self._h = ctypes.c_void_p(_handle)
        if _handle is None:
            f = Fields(number_of_experts, top_k, expert_hidden_size, expert_inter_size, max_num_tokens, use_bias,
                       type, output_type, quant_mode)
            _lib.check(self._lib.dqmoe_plugin_create(ctypes.byref(f), ctypes.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.dqmoe_plugin_destroy(self._h)
            self._h = None

    @property
    def fields(self) -> dict:
        f = Fields()
        _lib.check(self._lib.dqmoe_plugin_get_fields(self._h, ctypes.byref(f)))
        return {n: int(getattr(f, n)) for n, _ in Fields._fields_}

    def workspace_size(self, num_tokens: int) -> int:
        return int(self._lib.dqmoe_plugin_workspace_size(self._h, num_tokens))

    def serialize(self) -> bytes:
        n = int(self._lib.dqmoe_plugin_serialization_size())
        buf = ctypes.create_string_buffer(n)
        _lib.check(self._lib.dqmoe_plugin_serialize(self._h, buf, n))
        return buf.raw

    @classmethod
    def deserialize(cls, blob: bytes) -> "MoePlugin":
        lib = _lib.load()
        h = ctypes.c_void_p(None)
        _lib.check(lib.dqmoe_plugin_deserialize(blob, len(blob), ctypes.byref(h)))
        return cls(0, 0, 0, 0, 0, _handle=h.value)

    def enqueue(self, inputs: Sequence[Optional[torch.Tensor]], workspace: Optional[torch.Tensor] = None,
                output: Optional[torch.Tensor] = None) -> torch.Tensor:
        """inputs in INPUT_NAMES order (None for absent entries); returns [num_tokens, top_k, hidden]."""
        f = self.fields
        x = inputs[0]
        if not x.is_cuda:
            raise RuntimeError("[ASSERT FAILED] plugin.py  Condition: input.is_cuda()  (dqmoe_b200 has no CPU path)")
        T = x.shape[0]
        if workspace is None:
            workspace = torch.empty(max(self.workspace_size(T), 256), dtype=torch.uint8, device=x.device)
        if output is None:
            output = torch.empty((T, f["top_k"], f["expert_hidden_size"]), dtype=_TORCH_OUT[f["output_type"]],
                                 device=x.device)
        ptrs = (ctypes.c_void_p * len(INPUT_NAMES))()
        for i in range(len(INPUT_NAMES)):
            t = inputs[i] if i < len(inputs) else None
            ptrs[i] = None if t is None else t.data_ptr()
        outs = (ctypes.c_void_p * 1)(output.data_ptr())
        with torch.cuda.device(x.device):
            stream = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
            _lib.check(self._lib.dqmoe_plugin_enqueue(self._h, T, ptrs, outs, workspace.data_ptr(), stream))
        return output
