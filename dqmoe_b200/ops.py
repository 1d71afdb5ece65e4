"""Torch-tensor front end of the C ABI: every function takes CUDA tensors,
passes their device pointers to libdqmoe_b200.so on the current torch stream and
returns without synchronising. Torch is used for memory and streams only.

Names follow the reference's operator surface where it has one
(csrc/pybind11_register.h:153-163) and the helper functions of its tests
(test/util.py:18-68) for the quantisers.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib

QUANT_NONE = 0
QUANT_FP8_TENSOR = 256
QUANT_FP8_CHANNEL = 512
QUANT_FP8_BLOCK = 1024
QUANT_FP8_MX = 2048
SCORE_SOFTMAX = 0
SCORE_SIGMOID = 1

FP8 = torch.float8_e4m3fn


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _cuda(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise RuntimeError(f"[ASSERT FAILED] ops.py  Condition: {name}.is_cuda  Info: dqmoe_b200 has no CPU path")
    if not t.is_contiguous():
        raise RuntimeError(f"[ASSERT FAILED] ops.py  Condition: {name}.is_contiguous()")
    return t


def device_status() -> int:
    """Synchronise the current device and return (then clear) the kernels' sticky status word."""
    code = ctypes.c_int(0)
    _lib.check(_lib.load().dqmoe_device_status(ctypes.byref(code)))
    return code.value


# ---------------------------------------------------------------------- layer

def moe_workspace_bytes(T: int, H: int, I: int, E: int, k: int, quant_mode: int) -> int:
    return int(_lib.load().dqmoe_moe_workspace_bytes(T, H, I, E, k, quant_mode))


def _check_scales(a_scale, b_scale, b1_scale, T, H, I, E, quant_mode):
    """Scale tensors must be fp32 CUDA tensors with exactly the element count the mode reads
    (include/dqmoe.h lists the shapes); a short tensor would be read out of bounds by the kernels."""
    g = lambda x: (x + 127) // 128
    want = {QUANT_FP8_TENSOR: (1, E, E), QUANT_FP8_CHANNEL: (T, E * 2 * I, E * H),
            QUANT_FP8_BLOCK: (T * g(H), E * g(2 * I) * g(H), E * g(H) * g(I)),
            QUANT_FP8_MX: (T * H // 32, E * 2 * I * H // 32, E * H * I // 32)}[quant_mode]  # weights' tiled: same size
    dtype = torch.uint8 if quant_mode == QUANT_FP8_MX else torch.float32  # MXFP8 scales are UE8M0 bytes
    for name, t, n in zip(("a_scale", "b_scale", "b1_scale"), (a_scale, b_scale, b1_scale), want):
        if t is None or not t.is_cuda or t.dtype != dtype or not t.is_contiguous() or t.numel() != n:
            got = "None" if t is None else f"{t.dtype} {tuple(t.shape)} on {t.device}"
            raise RuntimeError(f"[ASSERT FAILED] ops.py  Condition: {name} is a contiguous {dtype} CUDA tensor of {n} "
                               f"elements for quant mode {quant_mode}  Info: got {got}")


def _check_bias(bias, E, cols, name):
    if bias is None:
        return
    if not bias.is_cuda or bias.dtype != torch.float32 or not bias.is_contiguous() or tuple(bias.shape) != (E, cols):
        raise RuntimeError(f"[ASSERT FAILED] ops.py  Condition: {name} is a contiguous fp32 CUDA tensor [{E}, {cols}]")


def moe_forward(a, a_scale, b, b_scale, b1, b1_scale, d, m_indices, workspace, quant_mode: int,
                fused: bool = True, bias1: Optional[torch.Tensor] = None,
                bias2: Optional[torch.Tensor] = None) -> None:
    """One MoE layer into d[T, k, H]; see dqmoe_moe_forward (and dqmoe_moe_forward_bias for
    the fp32 expert biases bias1 [E, 2I] / bias2 [E, H]) in include/dqmoe.h."""
    lib = _lib.load()
    T, H = a.shape
    E, I2, _ = b.shape
    I = b1.shape[2]
    k = d.shape[1]
    for name, t in (("a", a), ("b", b), ("b1", b1), ("d", d), ("m_indices", m_indices), ("workspace", workspace)):
        _cuda(t, name)
    quant_mode = int(quant_mode)
    if quant_mode in (QUANT_FP8_TENSOR, QUANT_FP8_CHANNEL, QUANT_FP8_BLOCK, QUANT_FP8_MX):
        _check_scales(a_scale, b_scale, b1_scale, T, H, I, E, quant_mode)
    _check_bias(bias1, E, 2 * I, "bias1")
    _check_bias(bias2, E, H, "bias2")
    with torch.cuda.device(a.device):
        if bias1 is None and bias2 is None:
            _lib.check(lib.dqmoe_moe_forward(
                _p(a), _p(a_scale), _p(b), _p(b_scale), _p(b1), _p(b1_scale), _p(d), _p(m_indices),
                _p(workspace), workspace.numel() * workspace.element_size(), T, H, I, E, k,
                quant_mode, int(bool(fused)), _stream(a.device)))
        else:
            _lib.check(lib.dqmoe_moe_forward_bias(
                _p(a), _p(a_scale), _p(b), _p(b_scale), _p(b1), _p(b1_scale), _p(bias1), _p(bias2), _p(d),
                _p(m_indices), _p(workspace), workspace.numel() * workspace.element_size(), T, H, I, E, k,
                quant_mode, _stream(a.device)))


def moe_forward_f16(a, b, b1, d, m_indices, workspace, bias1=None, bias2=None) -> None:
    """The unquantised layer on fp16 tensors into d[T, k, H] (fp16); see dqmoe_moe_forward_f16."""
    lib = _lib.load()
    for name, t in (("a", a), ("b", b), ("b1", b1), ("d", d), ("m_indices", m_indices), ("workspace", workspace)):
        _cuda(t, name)
    for name, t in (("a", a), ("b", b), ("b1", b1), ("d", d)):
        if t.dtype != torch.float16:
            raise RuntimeError(f"[ASSERT FAILED] ops.py  Condition: {name}.scalar_type() == at::kHalf")
    T, H = a.shape
    E, I, k = b.shape[0], b1.shape[2], d.shape[1]
    _check_bias(bias1, E, 2 * I, "bias1")
    _check_bias(bias2, E, H, "bias2")
    with torch.cuda.device(a.device):
        _lib.check(lib.dqmoe_moe_forward_f16_bias(_p(a), _p(b), _p(b1), _p(bias1), _p(bias2), _p(d), _p(m_indices),
                                                  _p(workspace), workspace.numel() * workspace.element_size(), T, H,
                                                  I, E, k, _stream(a.device)))


def moe_workspace_bytes_f32(T: int, H: int, I: int, E: int, k: int) -> int:
    return int(_lib.load().dqmoe_moe_workspace_bytes_f32(T, H, I, E, k))


def moe_forward_f32(a, b, b1, d, m_indices, workspace, bias1=None, bias2=None) -> None:
    """The unquantised layer on fp32 tensors (TF32 tensor-core products) into d[T, k, H] fp32;
    see dqmoe_moe_forward_f32."""
    lib = _lib.load()
    for name, t in (("a", a), ("b", b), ("b1", b1), ("d", d), ("m_indices", m_indices), ("workspace", workspace)):
        _cuda(t, name)
    for name, t in (("a", a), ("b", b), ("b1", b1), ("d", d)):
        if t.dtype != torch.float32:
            raise RuntimeError(f"[ASSERT FAILED] ops.py  Condition: {name}.scalar_type() == at::kFloat")
    T, H = a.shape
    E, I, k = b.shape[0], b1.shape[2], d.shape[1]
    _check_bias(bias1, E, 2 * I, "bias1")
    _check_bias(bias2, E, H, "bias2")
    with torch.cuda.device(a.device):
        _lib.check(lib.dqmoe_moe_forward_f32(_p(a), _p(b), _p(b1), _p(bias1), _p(bias2), _p(d), _p(m_indices),
                                             _p(workspace), workspace.numel() * workspace.element_size(), T, H, I, E,
                                             k, _stream(a.device)))


def moe_block(x: torch.Tensor, logits: torch.Tensor, b, b_scale, b1, b1_scale, k: int, scoring: str = "softmax",
              quant_mode: int = QUANT_FP8_BLOCK, workspace: Optional[torch.Tensor] = None,
              n_shared: int = 0) -> torch.Tensor:
    """Router -> layer -> weighted combine from bf16 activations x [T, H]; see dqmoe_moe_block.
    quant_mode 0 (bf16 weights) or 256 / 512 / 1024 (e4m3 weights with that mode's scales).

    With n_shared > 0 the last n_shared experts of b / b1 are shared experts that every token
    passes through with weight 1 (dqmoe_moe_block_shared); logits are [T, E - n_shared]."""
    lib = _lib.load()
    for name, t in (("x", x), ("logits", logits), ("b", b), ("b1", b1)):
        _cuda(t, name)
    T, H = x.shape
    E_all, I = b.shape[0], b1.shape[2]
    E = E_all - n_shared
    if n_shared < 0 or E <= 0 or logits.shape[1] != E:
        raise RuntimeError("[ASSERT FAILED] ops.py  Condition: logits is [T, num_experts - n_shared]")
    need = int(lib.dqmoe_moe_block_workspace_bytes(T, H, I, E_all, k + n_shared, int(quant_mode)))
    if workspace is None:
        workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=x.device)
    out = torch.empty((T, H), dtype=torch.bfloat16, device=x.device)
    mode = {"softmax": SCORE_SOFTMAX, "sigmoid": SCORE_SIGMOID}[scoring]
    with torch.cuda.device(x.device):
        _lib.check(lib.dqmoe_moe_block_shared(_p(x), _p(logits), _p(b), _p(b_scale), _p(b1), _p(b1_scale), _p(out),
                                              _p(workspace), workspace.numel(), T, H, I, E, k, n_shared, mode,
                                              int(quant_mode), _stream(x.device)))
    return out


# ---------------------------------------------------------------------- routing

def route_topk(logits: torch.Tensor, k: int, scoring: str = "softmax") -> Tuple[torch.Tensor, torch.Tensor]:
    """(indices int32 [T, k], weights fp32 [T, k]) from fp32 logits [T, E]."""
    _cuda(logits, "logits")
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise RuntimeError("[ASSERT FAILED] ops.py  Condition: logits is fp32 [T, E]")
    T, E = logits.shape
    mode = {"softmax": SCORE_SOFTMAX, "sigmoid": SCORE_SIGMOID}[scoring]
    idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    with torch.cuda.device(logits.device):
        _lib.check(_lib.load().dqmoe_route_topk(_p(logits), T, E, k, mode, _p(idx), _p(w), _stream(logits.device)))
    return idx, w


def route_sort(m_indices: torch.Tensor, E: int):
    """(counts[E], offsets[E+1], dest_to_src[n], src_to_dest[n]) int32 for m_indices [T, k]."""
    _cuda(m_indices, "m_indices")
    if m_indices.dtype != torch.int32:
        raise RuntimeError("[ASSERT FAILED] ops.py  Condition: m_indices.scalar_type() == torch::kInt")
    lib = _lib.load()
    n = m_indices.numel()
    dev = m_indices.device
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    d2s = torch.empty(n, dtype=torch.int32, device=dev)
    s2d = torch.empty(n, dtype=torch.int32, device=dev)
    ws_bytes = int(lib.dqmoe_route_sort_workspace_bytes(n, E))
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.dqmoe_route_sort(_p(m_indices), n, E, _p(counts), _p(offsets), _p(d2s), _p(s2d),
                                        _p(ws), ws_bytes, _stream(dev)))
    return counts, offsets, d2s, s2d


def mtile_prefix(offsets: torch.Tensor) -> torch.Tensor:
    _cuda(offsets, "offsets")
    E = offsets.numel() - 1
    out = torch.empty(E + 1, dtype=torch.int32, device=offsets.device)
    with torch.cuda.device(offsets.device):
        _lib.check(_lib.load().dqmoe_mtile_prefix(_p(offsets), E, _p(out), _stream(offsets.device)))
    return out


def segment_ids(counts: torch.Tensor, values: torch.Tensor, n: int) -> torch.Tensor:
    """out[r] = values[s] for the counts[s] rows of segment s (run-length expansion, int32)."""
    _cuda(counts, "counts")
    _cuda(values, "values")
    out = torch.empty(n, dtype=torch.int32, device=counts.device)
    with torch.cuda.device(counts.device):
        _lib.check(_lib.load().dqmoe_segment_ids(_p(counts), _p(values), counts.numel(), _p(out), n,
                                                 _stream(counts.device)))
    return out


# ---------------------------------------------------------------------- permute / finalize

def moe_permute(a: torch.Tensor, dest_to_src: torch.Tensor, k: int,
                scale: Optional[torch.Tensor] = None):
    """Expert-order gather of rows of a [T, H] (and of a per-row scale matrix [T, C])."""
    _cuda(a, "a")
    _cuda(dest_to_src, "dest_to_src")
    n = dest_to_src.numel()
    H = a.shape[1]
    out = torch.empty((n, H), dtype=a.dtype, device=a.device)
    cols = 0
    out_scale = None
    if scale is not None:
        _cuda(scale, "scale")
        cols = scale.shape[1] if scale.dim() == 2 else 1
        out_scale = torch.empty((n, cols), dtype=torch.float32, device=a.device)
    with torch.cuda.device(a.device):
        _lib.check(_lib.load().dqmoe_permute_rows(_p(a), H * a.element_size(), k, _p(dest_to_src), n, _p(out),
                                                  _p(scale), cols, _p(out_scale), _stream(a.device)))
    return (out, out_scale) if scale is not None else out


def moe_permute_quant_block(x: torch.Tensor, dest_to_src: torch.Tensor, k: int):
    """Gather fused with 1x128 FP8 quantisation of bf16 activations x [T, H]."""
    _cuda(x, "x")
    _cuda(dest_to_src, "dest_to_src")
    assert x.dtype == torch.bfloat16
    n = dest_to_src.numel()
    H = x.shape[1]
    q = torch.empty((n, H), dtype=FP8, device=x.device)
    s = torch.empty((n, (H + 127) // 128), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().dqmoe_permute_quant_block_1x128(_p(x), H, k, _p(dest_to_src), n, _p(q), _p(s),
                                                               _stream(x.device)))
    return q, s


def finalize_scatter(rows: torch.Tensor, dest_to_src: torch.Tensor, d: torch.Tensor) -> None:
    """d.view(n, H)[dest_to_src[r]] = rows[r]."""
    _cuda(rows, "rows")
    _cuda(d, "d")
    n = dest_to_src.numel()
    with torch.cuda.device(rows.device):
        _lib.check(_lib.load().dqmoe_finalize_scatter(_p(rows), rows.shape[1] * rows.element_size(),
                                                      _p(dest_to_src), n, _p(d), _stream(rows.device)))


def finalize_weighted(d: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """out[t] = sum_j weights[t, j] * d[t, j]  (bf16 [T, k, H] -> bf16 [T, H])."""
    _cuda(d, "d")
    _cuda(weights, "weights")
    assert d.dtype == torch.bfloat16 and weights.dtype == torch.float32
    T, k, H = d.shape
    out = torch.empty((T, H), dtype=torch.bfloat16, device=d.device)
    with torch.cuda.device(d.device):
        _lib.check(_lib.load().dqmoe_finalize_weighted(_p(d), _p(weights), _p(out), T, k, H, _stream(d.device)))
    return out


# ---------------------------------------------------------------------- quantisers (test/util.py:18-68)

def per_token_cast_to_fp8(x: torch.Tensor):
    _cuda(x, "x")
    assert x.dim() == 2 and x.dtype == torch.bfloat16
    m, n = x.shape
    q = torch.empty((m, n), dtype=FP8, device=x.device)
    s = torch.empty((m, 1), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().dqmoe_quant_fp8_rowwise(_p(x), m, n, _p(q), _p(s), _stream(x.device)))
    return q, s


def per_channel_cast_to_fp8(x: torch.Tensor):
    _cuda(x, "x")
    assert x.dim() == 3 and x.dtype == torch.bfloat16
    e, m, n = x.shape
    q = torch.empty((e, m, n), dtype=FP8, device=x.device)
    s = torch.empty((e, m, 1), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().dqmoe_quant_fp8_rowwise(_p(x), e * m, n, _p(q), _p(s), _stream(x.device)))
    return q, s


def per_token_block_cast_to_fp8(x: torch.Tensor):
    _cuda(x, "x")
    assert x.dim() == 2 and x.dtype == torch.bfloat16
    m, n = x.shape
    q = torch.empty((m, n), dtype=FP8, device=x.device)
    s = torch.empty((m, (n + 127) // 128), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().dqmoe_quant_fp8_block_1x128(_p(x), m, n, _p(q), _p(s), _stream(x.device)))
    return q, s


def per_block_cast_to_fp8(x: torch.Tensor):
    _cuda(x, "x")
    assert x.dtype == torch.bfloat16
    x3 = x[None] if x.dim() == 2 else x
    e, m, n = x3.shape
    q = torch.empty((e, m, n), dtype=FP8, device=x.device)
    s = torch.empty((e, (m + 127) // 128, (n + 127) // 128), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().dqmoe_quant_fp8_block_128x128(_p(x3), e, m, n, _p(q), _p(s), _stream(x.device)))
    return q, s


def per_tensor_cast_to_fp8(x: torch.Tensor, per_expert: bool = False):
    """One scale for the tensor, or one per leading index when per_expert."""
    _cuda(x, "x")
    assert x.dtype == torch.bfloat16
    e = x.shape[0] if per_expert else 1
    numel_per = x.numel() // e
    q = torch.empty(x.shape, dtype=FP8, device=x.device)
    s = torch.empty(e, dtype=torch.float32, device=x.device)
    scratch = torch.empty(e, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().dqmoe_quant_fp8_tensor(_p(x), e, numel_per, _p(q), _p(s), _p(scratch),
                                                      _stream(x.device)))
    return q, s


def mx_cast_to_fp8(x: torch.Tensor):
    """MXFP8: (e4m3 of x's shape, UE8M0 scale bytes [..., n/32]) for bf16 x [..., n]; see dqmoe_quant_mxfp8."""
    _cuda(x, "x")
    assert x.dtype == torch.bfloat16 and x.shape[-1] % 32 == 0
    n = x.shape[-1]
    rows = x.numel() // n
    q = torch.empty(x.shape, dtype=FP8, device=x.device)
    s = torch.empty((*x.shape[:-1], n // 32), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().dqmoe_quant_mxfp8(_p(x), rows, n, _p(q), _p(s), _stream(x.device)))
    return q, s


def mx_tile_scales(sf: torch.Tensor, cols: int, offsets=None, mtile_pref=None, dest_to_src=None, k: int = 1) -> torch.Tensor:
    """Row-major UE8M0 scale bytes [..., cols/32] -> the tiled layout the MXFP8 grouped GEMM reads (see
    dqmoe_mx_tile_scales). Without offsets the rows form 128-row blocks by their index (weights); with offsets /
    mtile_pref [E+1] they are expert-sorted activation rows; dest_to_src gathers rows of `sf` first."""
    _cuda(sf, "sf")
    assert sf.dtype == torch.uint8 and sf.shape[-1] == cols // 32
    lib = _lib.load()
    rows = dest_to_src.numel() if dest_to_src is not None else sf.numel() // (cols // 32)
    E = offsets.numel() - 1 if offsets is not None else 0
    nbytes = int(lib.dqmoe_mx_tiled_scale_bytes(rows, E, cols))
    out = torch.zeros(max(nbytes, 16), dtype=torch.uint8, device=sf.device)
    with torch.cuda.device(sf.device):
        _lib.check(lib.dqmoe_mx_tile_scales(_p(sf), rows, cols, _p(dest_to_src), k, _p(offsets), _p(mtile_pref), E, _p(out),
                                            _stream(sf.device)))
    return out


def mx_cast_weights_to_fp8(w: torch.Tensor):
    """MXFP8 weights [E, rows, cols] (rows a multiple of 128): (e4m3 bytes, scale bytes in the tiled layout)."""
    q, s = mx_cast_to_fp8(w)
    return q, mx_tile_scales(s, w.shape[-1])


def moe_permute_quant_mx(x: torch.Tensor, dest_to_src: torch.Tensor, k: int, offsets: torch.Tensor,
                         mtile_pref: torch.Tensor):
    """Gather fused with the MXFP8 quantisation of bf16 activations x [T, H]; scales come out tiled."""
    _cuda(x, "x")
    _cuda(dest_to_src, "dest_to_src")
    assert x.dtype == torch.bfloat16
    lib = _lib.load()
    n, H = dest_to_src.numel(), x.shape[1]
    E = offsets.numel() - 1
    q = torch.empty((n, H), dtype=FP8, device=x.device)
    s = torch.zeros(max(int(lib.dqmoe_mx_tiled_scale_bytes(n, E, H)), 16), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(lib.dqmoe_permute_quant_mxfp8(_p(x), H, k, _p(dest_to_src), n, _p(offsets), _p(mtile_pref), E, _p(q),
                                                 _p(s), _stream(x.device)))
    return q, s


def nvfp4_global_scale(x: torch.Tensor) -> torch.Tensor:
    """amax / (448 * 6) of x as a [1] fp32 tensor: the usual NVFP4 global scale (set-up arithmetic in torch)."""
    # tensor / tensor: an IEEE division (a division by a Python scalar may run as a multiplication by 1 / 2688)
    return (x.float().abs().amax().clamp(min=1e-4) / torch.full((), 2688.0, device=x.device)).reshape(1)


def nvfp4_cast(x: torch.Tensor, gscale: torch.Tensor):
    """NVFP4: (packed e2m1 bytes [..., n/2], UE4M3 scale bytes [..., n/16]) for bf16 x [..., n]; gscale holds one
    global scale for all of x, or one per index of x's first dimension (weights [E, rows, n]); see
    dqmoe_quant_nvfp4."""
    _cuda(x, "x")
    _cuda(gscale, "gscale")
    assert x.dtype == torch.bfloat16 and x.shape[-1] % 16 == 0 and gscale.dtype == torch.float32
    n = x.shape[-1]
    rows = x.numel() // n
    groups = gscale.numel()
    assert groups == 1 or groups == x.shape[0]
    q = torch.empty((*x.shape[:-1], n // 2), dtype=torch.uint8, device=x.device)
    s = torch.empty((*x.shape[:-1], n // 16), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().dqmoe_quant_nvfp4(_p(x), rows, n, _p(gscale), max(rows // groups, 1), _p(q), _p(s),
                                                 _stream(x.device)))
    return q, s


def nvfp4_cast_weights(w: torch.Tensor):
    """NVFP4 weights [E, rows, cols] (rows a multiple of 128, cols of 64): (packed bytes, scale bytes in the tiled
    layout of the grouped GEMM, per-expert global scales [E])."""
    g = (w.float().abs().amax(dim=(1, 2)).clamp(min=1e-4) / torch.full((), 2688.0, device=w.device)).contiguous()
    q, s = nvfp4_cast(w, g)
    return q, mx_tile_scales(s, 2 * w.shape[-1]), g


def grouped_gemm_nvfp4(a, a_sf, a_g, w, w_sf, w_g, offsets, mtile_pref, N: int, gated: bool, out, out_sf=None, out_g=None,
                       dest_to_src=None) -> None:
    """The grouped GEMM in the NVFP4 mode; see dqmoe_grouped_gemm_nvfp4. a [n, K/2] packed."""
    n, K = a.shape[0], a.shape[1] * 2
    E = w.shape[0]
    with torch.cuda.device(a.device):
        _lib.check(_lib.load().dqmoe_grouped_gemm_nvfp4(_p(a), _p(a_sf), _p(a_g), _p(w), _p(w_sf), _p(w_g), _p(offsets),
                                                        _p(mtile_pref), n, N, K, E, int(bool(gated)), _p(out), _p(out_sf),
                                                        _p(out_g), _p(dest_to_src), _stream(a.device)))


def moe_forward_nvfp4(a, a_sf, a_g, b, b_sf, b_g, b1, b1_sf, b1_g, act_g, d, m_indices, workspace, bias1=None,
                      bias2=None) -> None:
    """The layer in the NVFP4 mode; see dqmoe_moe_forward_nvfp4. a [T, H/2] packed with row-major scale bytes
    [T, H/16]; weights packed with tiled scale bytes and per-expert global scales (nvfp4_cast_weights)."""
    for name, t in (("a", a), ("b", b), ("b1", b1), ("d", d), ("m_indices", m_indices), ("workspace", workspace)):
        _cuda(t, name)
    T, H = a.shape[0], a.shape[1] * 2
    E, I = b1.shape[0], b1.shape[2] * 2
    k = m_indices.shape[1]
    assert a.dtype == torch.uint8 and b.dtype == torch.uint8 and b1.dtype == torch.uint8 and d.dtype == torch.bfloat16
    assert tuple(b.shape) == (E, 2 * I, H // 2) and tuple(b1.shape) == (E, H, I // 2) and tuple(d.shape) == (T, k, H)
    assert a_sf.dtype == torch.uint8 and tuple(a_sf.shape) == (T, H // 16) and m_indices.dtype == torch.int32
    for g, cnt in ((a_g, 1), (b_g, E), (b1_g, E), (act_g, 1)):
        assert g.dtype == torch.float32 and g.numel() == cnt and g.is_cuda
    _check_bias(bias1, E, 2 * I, "bias1")
    _check_bias(bias2, E, H, "bias2")
    with torch.cuda.device(a.device):
        _lib.check(_lib.load().dqmoe_moe_forward_nvfp4(
            _p(a), _p(a_sf), _p(a_g), _p(b), _p(b_sf), _p(b_g), _p(b1), _p(b1_sf), _p(b1_g), _p(act_g), _p(bias1), _p(bias2),
            _p(d), _p(m_indices), _p(workspace), workspace.numel() * workspace.element_size(), T, H, I, E, k,
            _stream(a.device)))


# ---------------------------------------------------------------------- grouped GEMM

def grouped_gemm_mx(a, a_sf, w, w_sf, offsets, mtile_pref, N: int, gated: bool, out, out_sf=None, dest_to_src=None) -> None:
    """The grouped GEMM in the MXFP8 mode; see dqmoe_grouped_gemm_mx."""
    n, K = a.shape
    E = w.shape[0]
    with torch.cuda.device(a.device):
        _lib.check(_lib.load().dqmoe_grouped_gemm_mx(_p(a), _p(a_sf), _p(w), _p(w_sf), _p(offsets), _p(mtile_pref), n, N, K,
                                                     E, int(bool(gated)), _p(out), _p(out_sf), _p(dest_to_src),
                                                     _stream(a.device)))


def grouped_gemm(a, a_scale, w, w_scale, offsets, mtile_pref, N: int, quant_mode: int, gated: bool,
                 out, out_scale=None, amax=None, dest_to_src=None) -> None:
    """The MoeGemmRunner::runGemm step with fused epilogue; see dqmoe_grouped_gemm."""
    n, K = a.shape
    E = w.shape[0]
    with torch.cuda.device(a.device):
        _lib.check(_lib.load().dqmoe_grouped_gemm(
            _p(a), _p(a_scale), _p(w), _p(w_scale), _p(offsets), _p(mtile_pref), n, N, K, E, int(quant_mode),
            int(bool(gated)), _p(out), _p(out_scale), _p(amax), _p(dest_to_src), _stream(a.device)))


def requant_from_amax(act: torch.Tensor, amax: torch.Tensor, per_row: bool, n_rows_device: Optional[torch.Tensor] = None,
                      out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    """Second pass of the tensor / channel modes. n_rows_device: int32 [1] on the device bounding the rows
    that are processed (dqmoe_requant_from_amax_dev); rows past it keep what `out` held."""
    n, I = act.shape
    if out is None:
        q = torch.empty((n, I), dtype=FP8, device=act.device)
        s = torch.empty(n if per_row else 1, dtype=torch.float32, device=act.device)
    else:
        q, s = out
    with torch.cuda.device(act.device):
        _lib.check(_lib.load().dqmoe_requant_from_amax_dev(_p(act), n, I, _p(amax), int(per_row), _p(q), _p(s),
                                                           _p(n_rows_device), _stream(act.device)))
    return q, s
