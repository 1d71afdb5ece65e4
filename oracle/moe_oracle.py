"""CPU oracle of the MoE-layer hot path. TEST INFRASTRUCTURE ONLY.

A restatement in torch-on-CPU of what the reference computes for this path, used
as the checker by tests/, by __graft_entry__.smoke() and as the timed CPU
baseline of bench.py. Nothing in the shipped package imports it.

What it follows (paths inside the reference project):
  * test/util.py:18-68   the four torch input quantisers
                         (sf = clamp(amax, 1e-4) / 448, q = e4m3(x * (1 / sf)))
  * test/util.py:71-92   the bf16 layer (gate half first, silu(gate) * value)
  * test/util.py:95-158  the FP8-simulating block-wise layer: where values are
                         rounded to bf16 and where the intermediate is re-quantised
  * csrc/moe_kernels.h:452-471, test/util.py:80  the expert sort (stable order)
  * csrc/moe_kernels.h:581-609  the unweighted scatter into d[T, k, H]
The channel-wise and tensor-wise FP8 layers, the router and the weighted combine
have no torch counterpart in the reference; they are written here by analogy
with the block-wise one and are marked "parity unpinned" below.

Pinning: tests/golden/make_golden.py imports the reference's test/util.py and
stores its outputs for seeded inputs; tests/test_oracle_golden.py checks every
function here that has a reference counterpart against those files bit for bit.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np
import torch
import torch.nn.functional as F

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
AMAX_FLOOR = 1e-4
GROUP = 128

QUANT_NONE, QUANT_TENSOR, QUANT_CHANNEL, QUANT_BLOCK = 0, 256, 512, 1024
QUANT_MX = 2048   # MXFP8: e4m3 with one UE8M0 scale per 32 elements (no counterpart in the reference)
QUANT_NVFP4 = 4096  # e2m1 with one UE4M3 scale per 16 elements and an fp32 global scale (the reference's FP4 bit, no code)
MX_GROUP = 32


# ---------------------------------------------------------------------- quantisers

def _scale_and_cast(x_grouped: torch.Tensor, amax: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """The arithmetic shared by every quantiser of test/util.py:18-68.

    amax (fp32, broadcastable to x_grouped) -> sf = max(amax, 1e-4) / 448;
    bytes = e4m3(x * (1 / sf)), the product taken in fp32 (bf16 tensor times fp32 tensor).
    """
    sf = amax.clamp(min=AMAX_FLOOR) / FP8_MAX
    q = (x_grouped * (1.0 / sf)).to(FP8)
    return q, sf


def quant_rowwise(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """One scale per row of the last dimension: per_token_cast_to_fp8 for [m, n]
    (test/util.py:18-23) and per_channel_cast_to_fp8 for [e, m, n] (test/util.py:26-30)."""
    amax = x.abs().float().amax(dim=-1, keepdim=True)
    q, sf = _scale_and_cast(x, amax)
    return q.contiguous(), sf


def quant_block_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """per_token_block_cast_to_fp8 (test/util.py:34-45): 128-wide groups along a row, zero padded."""
    m, n = x.shape
    groups = -(-n // GROUP)
    padded = torch.zeros((m, groups * GROUP), dtype=x.dtype)
    padded[:, :n] = x
    g = padded.view(m, groups, GROUP)
    amax = g.abs().float().amax(dim=2, keepdim=True)
    q, sf = _scale_and_cast(g, amax)
    return q.view(m, groups * GROUP)[:, :n].contiguous(), sf.view(m, groups)


def quant_block_128x128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """per_block_cast_to_fp8 (test/util.py:48-68): one scale per 128x128 block of each matrix."""
    w3 = w[None] if w.dim() == 2 else w
    e, m, n = w3.shape
    bm, bn = -(-m // GROUP), -(-n // GROUP)
    padded = torch.zeros((e, bm * GROUP, bn * GROUP), dtype=w.dtype)
    padded[:, :m, :n] = w3
    g = padded.view(e, bm, GROUP, bn, GROUP)
    amax = g.abs().float().amax(dim=(2, 4), keepdim=True)
    q, sf = _scale_and_cast(g, amax)
    return q.view(e, bm * GROUP, bn * GROUP)[:, :m, :n].contiguous(), sf.view(e, bm, bn)


def quant_tensor(x: torch.Tensor, per_expert: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """One scale for the whole tensor, or one per leading index. Parity unpinned: the
    reference has this mode only inside its CUDA path (csrc/moe_kernels.h:136-221), with
    neither a torch generator nor a test; the formula is that of the other quantisers."""
    if per_expert:
        flat = x.reshape(x.shape[0], -1)
        amax = flat.abs().float().amax(dim=1).view(-1, *([1] * (x.dim() - 1)))
        q, sf = _scale_and_cast(x, amax)
        return q.contiguous(), sf.reshape(-1)
    amax = x.abs().float().amax().view(*([1] * x.dim()))
    q, sf = _scale_and_cast(x, amax)
    return q.contiguous(), sf.reshape(1)


def quant_mx(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """MXFP8 quantiser, parity unpinned (the reference reserves mode bits for block-scaled formats,
    csrc/quantization.h:30-38, but has no code for them). Per 32 consecutive elements of the last dimension:
    s = 2^ceil(log2(max(amax, 1e-4) / 448)), the smallest power of two that brings the group inside the e4m3
    range (the rule of DeepGEMM's UE8M0 path, which the reference's README.md:11 names as its road map);
    bytes = e4m3(x / s); the scale is stored as the biased exponent byte log2(s) + 127."""
    n = x.shape[-1]
    assert n % MX_GROUP == 0
    g = x.float().reshape(*x.shape[:-1], n // MX_GROUP, MX_GROUP)
    s = g.abs().amax(dim=-1, keepdim=True).clamp(min=AMAX_FLOOR) / FP8_MAX
    bits = s.contiguous().view(torch.int32)
    e = (bits >> 23) + ((bits & 0x7FFFFF) != 0).to(torch.int32)   # ceil(log2(s)) + 127
    inv = ((254 - e) << 23).view(torch.float32)                   # 1 / s, exact
    q = (g * inv).to(FP8)
    return q.reshape(x.shape).contiguous(), e.to(torch.uint8).reshape(*x.shape[:-1], n // MX_GROUP)


def dequant_mx(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    n = q.shape[-1]
    scale = (sf.to(torch.int32) << 23).view(torch.float32)        # 2^(byte - 127)
    return (q.float().reshape(*q.shape[:-1], n // MX_GROUP, MX_GROUP) * scale.unsqueeze(-1)).reshape(q.shape)



# ---------------------------------------------------------------------- NVFP4 (parity unpinned)

NVFP4_GROUP = 16
E2M1_MAX = 6.0
_E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
# round-to-nearest-even thresholds between neighbouring codes; a tie goes to the even code
_E2M1_MID = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
_E2M1_TIE_UP = torch.tensor([False, True, False, True, False, True, False])  # tie at mid[i] goes to code i + 1?


def e2m1_codes(v: torch.Tensor) -> torch.Tensor:
    """fp32 -> e2m1 code 0..15 (sign in bit 3), round to nearest even, saturating at 6."""
    mag = v.abs()
    code = torch.zeros(v.shape, dtype=torch.int32)
    for i in range(7):
        up = (mag >= _E2M1_MID[i]) if bool(_E2M1_TIE_UP[i]) else (mag > _E2M1_MID[i])
        code += up.to(torch.int32)
    return code | (torch.signbit(v).to(torch.int32) << 3)


def nvfp4_global_scale(x: torch.Tensor) -> torch.Tensor:
    """The usual global scale of a tensor: amax / (448 * 6), so that the largest block scale is the largest e4m3."""
    return (x.float().abs().amax().clamp(min=AMAX_FLOOR) / (FP8_MAX * E2M1_MAX)).reshape(1)


def quant_nvfp4(x: torch.Tensor, g: torch.Tensor):
    """NVFP4 quantiser, parity unpinned (the reference names the format, csrc/quantization.h:30-33, 81-84, and has
    no code for it). x [..., n] with n a multiple of 16; g: fp32 global scale, one value or one per leading index
    of x (per expert for weights). Per 16 consecutive elements: scale byte = e4m3((amax / 6) / g) saturating at
    448; nibbles = e2m1(x * (1 / (e4m3 * g))), zeros where the scale byte is zero. Returns the packed bytes
    [..., n/2] (element 2i in the low nibble) and the scale bytes [..., n/16] (e4m3 bit patterns, uint8)."""
    n = x.shape[-1]
    assert n % NVFP4_GROUP == 0
    grp = x.float().reshape(*x.shape[:-1], n // NVFP4_GROUP, NVFP4_GROUP)
    gg = g.float().reshape(-1, *([1] * (grp.dim() - 1))) if g.numel() > 1 else g.float().reshape(())
    s = ((grp.abs().amax(dim=-1, keepdim=True) / E2M1_MAX) / gg).clamp(max=FP8_MAX)
    s8 = s.to(FP8)
    d = s8.float() * gg
    inv = torch.where(d > 0, 1.0 / d, torch.zeros_like(d))
    codes = e2m1_codes(grp * inv).reshape(*x.shape[:-1], n // 2, 2)
    packed = (codes[..., 0] | (codes[..., 1] << 4)).to(torch.uint8)
    return packed.contiguous(), s8.view(torch.uint8).reshape(*x.shape[:-1], n // NVFP4_GROUP).contiguous()


def dequant_nvfp4(packed: torch.Tensor, sf: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    p = packed.to(torch.int32)
    codes = torch.stack([p & 15, p >> 4], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    vals = _E2M1_VALUES[(codes & 7).long()] * torch.where((codes & 8) != 0, -1.0, 1.0)
    n = vals.shape[-1]
    scale = sf.view(FP8).float()
    gg = g.float().reshape(-1, *([1] * (vals.dim() - 1))) if g.numel() > 1 else g.float().reshape(())
    return (vals.reshape(*vals.shape[:-1], n // NVFP4_GROUP, NVFP4_GROUP) * scale.unsqueeze(-1)).reshape(vals.shape) * gg


def moe_layer_nvfp4(a_q, a_sf, a_g, b_q, b_sf, b_g, b1_q, b1_sf, b1_g, act_g, m_indices, E: int, bias1=None, bias2=None):
    """The layer in the NVFP4 mode (parity unpinned), same steps as the other quantised modes: dequantise, fp32
    linear, round to bf16, SwiGLU in bf16, re-quantise the intermediate to NVFP4 with the given global scale
    act_g, dequantise, fp32 linear, round to bf16."""
    T, k = m_indices.shape
    H = a_q.shape[1] * 2
    d = torch.zeros((T, k, H), dtype=torch.bfloat16)
    a_f = dequant_nvfp4(a_q, a_sf, a_g)
    for e in range(E):
        tok, slot = torch.where(m_indices == e)
        if tok.numel() == 0:
            continue
        inter = F.linear(a_f[tok], dequant_nvfp4(b_q[e], b_sf[e], b_g[e:e + 1]))
        if bias1 is not None:
            inter = inter + bias1[e].float()
        act = _swiglu_bf16(inter.to(torch.bfloat16))
        q, s = quant_nvfp4(act, act_g)
        out = F.linear(dequant_nvfp4(q, s, act_g), dequant_nvfp4(b1_q[e], b1_sf[e], b1_g[e:e + 1]))
        if bias2 is not None:
            out = out + bias2[e].float()
        d[tok, slot] = out.to(torch.bfloat16)
    return d


# ---------------------------------------------------------------------- routing

def route_topk(logits: torch.Tensor, k: int, scoring: str = "softmax") -> Tuple[torch.Tensor, torch.Tensor]:
    """Parity unpinned (the reference's tests use randn + torch.topk, test/torch_test.py:78-80).
    Rank by logit, value descending then expert id ascending; weights are softmax or sigmoid
    scores of the selected experts normalised to sum 1."""
    x = logits.float()
    order = torch.sort(x, dim=1, descending=True, stable=True).indices[:, :k]
    sel = torch.gather(x, 1, order)
    if scoring == "softmax":
        score = torch.exp(sel - x.amax(dim=1, keepdim=True))
    elif scoring == "sigmoid":
        score = torch.sigmoid(sel)
    else:
        raise ValueError(scoring)
    return order.to(torch.int32), score / score.sum(dim=1, keepdim=True)


def route_sort(m_indices: torch.Tensor, E: int):
    """counts[E], offsets[E+1], dest_to_src[n], src_to_dest[n] for m_indices [T, k].

    Rows of an expert keep ascending source order t*k+j, the order torch.where yields in
    test/util.py:80 (the reference's GetGroupIndex, csrc/moe_kernels.h:452-461, assigns
    slots with atomics and fixes only the per-expert ranges). Ids outside [0, E) are dropped."""
    ids = m_indices.reshape(-1).to(torch.int64).numpy()
    n = ids.shape[0]
    bucket = np.where((ids >= 0) & (ids < E), ids, E)
    order = np.argsort(bucket, kind="stable")
    counts = np.bincount(bucket, minlength=E + 1)
    offsets = np.zeros(E + 1, dtype=np.int64)
    offsets[1:] = np.cumsum(counts[:E])
    kept = int(offsets[E])
    dest_to_src = order.astype(np.int32)
    dest_to_src[kept:] = -1
    src_to_dest = np.full(n, -1, dtype=np.int32)
    src_to_dest[order[:kept]] = np.arange(kept, dtype=np.int32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.int32))
    return t(counts[:E]), t(offsets), t(dest_to_src), t(src_to_dest)


def permute_rows(a: torch.Tensor, dest_to_src: torch.Tensor, k: int) -> torch.Tensor:
    """expandInputRowsGatherKernel (csrc/moe_kernels.h:487-514): out[r] = a[dest_to_src[r] // k]."""
    idx = dest_to_src.to(torch.int64)
    out = torch.zeros((idx.numel(),) + tuple(a.shape[1:]), dtype=a.dtype)
    keep = idx >= 0
    out[keep] = a[(idx[keep] // k)]
    return out


def finalize_weighted(d: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """Parity unpinned (no counterpart; the reference leaves d as [T, k, H]):
    out[t] = sum_j w[t, j] * d[t, j], fp32 accumulation in slot order, bf16 result."""
    acc = torch.zeros((d.shape[0], d.shape[2]), dtype=torch.float32)
    for j in range(d.shape[1]):
        acc = torch.addcmul(acc, d[:, j].float(), weights[:, j:j + 1].float())
    return acc.to(torch.bfloat16)


# ---------------------------------------------------------------------- layers

def _swiglu_bf16(inter: torch.Tensor) -> torch.Tensor:
    gate, value = inter.chunk(2, dim=-1)  # gate rows come first in b (test/util.py:86-87)
    return F.silu(gate) * value


def _linear_bias(x, w, bias):
    """x w^T + bias with the product accumulated and the bias added in fp32, one rounding to x's type."""
    return (F.linear(x.float(), w.float()) + bias.float()).to(x.dtype)


def moe_layer_bf16(a, b, b1, m_indices, E: int, bias1=None, bias2=None) -> torch.Tensor:
    """torch_moe_grouped (test/util.py:71-92): linear, SwiGLU, linear, scatter to [T, k, H], in the operands'
    type (bf16 in the reference's test; fp16 and fp32 operands take the same steps). With expert biases
    bias1 [E, 2I] / bias2 [E, H] (fp32; parity unpinned: the reference never applies its bias arguments)
    each linear adds its expert's bias before rounding."""
    T, k = m_indices.shape
    d = torch.zeros((T, k, a.shape[1]), dtype=a.dtype)
    for e in range(E):
        tok, slot = torch.where(m_indices == e)
        if tok.numel() == 0:
            continue
        inter = F.linear(a[tok], b[e]) if bias1 is None else _linear_bias(a[tok], b[e], bias1[e])
        act = _swiglu_bf16(inter)
        d[tok, slot] = F.linear(act, b1[e]) if bias2 is None else _linear_bias(act, b1[e], bias2[e])
    return d


def _expand(scale: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Blow a [ceil(rows/128), ceil(cols/128)] or [rows, ceil(cols/128)] scale grid up to [rows, cols]."""
    s = scale.repeat_interleave(GROUP, dim=-1)[..., :cols]
    if s.shape[-2] != rows:
        s = s.repeat_interleave(GROUP, dim=-2)[..., :rows, :]
    return s


def moe_layer_fp8(a_q, a_s, b_q, b_s, b1_q, b1_s, m_indices, E: int, quant_mode: int,
                  return_intermediate: bool = False, bias1=None, bias2=None):
    """FP8-simulating layer. Block mode restates fp8_blockwise_torch_moe_grouped
    (test/util.py:95-158): dequantise, fp32 linear, round to bf16, SwiGLU in bf16,
    re-quantise the intermediate, dequantise, fp32 linear, round to bf16. Channel and
    tensor modes apply the same steps with their scale shapes (parity unpinned: the
    reference has no torch model of them), and so does the MXFP8 mode with its 1x32 power-of-two
    scales (parity unpinned: the format is not in the reference). bias1 [E, 2I] / bias2 [E, H] (fp32, parity unpinned)
    are added to the fp32 products before the rounding to bf16."""
    T, k = m_indices.shape
    H = a_q.shape[1]
    I = b1_q.shape[2]
    d = torch.zeros((T, k, H), dtype=torch.bfloat16)
    a_f = a_q.float()
    inter_store = {}

    acts = {}
    for e in range(E):
        tok, slot = torch.where(m_indices == e)
        if tok.numel() == 0:
            continue
        if quant_mode == QUANT_BLOCK:
            dq_a = a_f[tok] * _expand(a_s[tok], tok.numel(), H)
            dq_b = b_q[e].float() * _expand(b_s[e], 2 * I, H)
        elif quant_mode == QUANT_CHANNEL:
            dq_a = a_f[tok] * a_s[tok].view(-1, 1)
            dq_b = b_q[e].float() * b_s[e].view(-1, 1)
        elif quant_mode == QUANT_TENSOR:
            dq_a = a_f[tok] * a_s.view(())
            dq_b = b_q[e].float() * b_s[e]
        elif quant_mode == QUANT_MX:
            dq_a = dequant_mx(a_q[tok], a_s[tok])
            dq_b = dequant_mx(b_q[e], b_s[e])
        else:
            raise ValueError(quant_mode)
        inter = F.linear(dq_a, dq_b)
        if bias1 is not None:
            inter = inter + bias1[e].float()
        acts[e] = (tok, slot, _swiglu_bf16(inter.to(torch.bfloat16)))

    if quant_mode == QUANT_TENSOR:
        # one scale for the whole intermediate (csrc/moe_kernels.h:136-204), torch formula
        amax = max([v[2].abs().float().amax().item() for v in acts.values()] + [0.0])
        # shape [1], not 0-dim: a 0-dim fp32 factor would leave the product below in bf16
        sf_all = torch.tensor([amax], dtype=torch.float32).clamp(min=AMAX_FLOOR) / FP8_MAX

    for e, (tok, slot, act) in acts.items():
        if quant_mode == QUANT_BLOCK:
            q, s = quant_block_1x128(act)
            dq_act = q.float() * _expand(s, act.shape[0], I)
            dq_b1 = b1_q[e].float() * _expand(b1_s[e], H, I)
        elif quant_mode == QUANT_CHANNEL:
            q, s = quant_rowwise(act)
            dq_act = q.float() * s
            dq_b1 = b1_q[e].float() * b1_s[e].view(-1, 1)
        elif quant_mode == QUANT_MX:
            q, s = quant_mx(act)
            dq_act = dequant_mx(q, s)
            dq_b1 = dequant_mx(b1_q[e], b1_s[e])
        else:
            q = (act * (1.0 / sf_all)).to(FP8)
            s = sf_all
            dq_act = q.float() * sf_all
            dq_b1 = b1_q[e].float() * b1_s[e]
        inter_store[e] = (q, s)
        out = F.linear(dq_act, dq_b1)
        if bias2 is not None:
            out = out + bias2[e].float()
        d[tok, slot] = out.to(torch.bfloat16)
    if return_intermediate:
        return d, inter_store
    return d


def moe_block(x, logits, b, b1, k: int, scoring: str, quant_mode: int, quantized=None, n_shared: int = 0) -> torch.Tensor:
    """Router -> layer -> weighted combine, [T, H] -> [T, H] (parity unpinned as a whole).

    With n_shared > 0 the last n_shared experts of b / b1 are shared experts: every token runs
    through them with weight 1, as extra slots after its k routed ones."""
    E = b.shape[0]
    idx, w = route_topk(logits, k, scoring)
    if n_shared:
        T = idx.shape[0]
        extra = torch.arange(E - n_shared, E, dtype=idx.dtype).expand(T, n_shared)
        idx = torch.cat([idx, extra], dim=1)
        w = torch.cat([w, torch.ones(T, n_shared, dtype=w.dtype)], dim=1)
    if quant_mode == QUANT_NONE:
        d = moe_layer_bf16(x, b, b1, idx, E)
    else:
        a_q, a_s, b_q, b_s, b1_q, b1_s = quantized if quantized is not None else quantize_inputs(x, b, b1, quant_mode)
        d = moe_layer_fp8(a_q, a_s, b_q, b_s, b1_q, b1_s, idx, E, quant_mode)
    return finalize_weighted(d, w)


def quantize_inputs(a, b, b1, quant_mode: int):
    """Input quantisation as the reference's generators do it (test/util.py:162-235)."""
    if quant_mode == QUANT_BLOCK:
        return (*quant_block_1x128(a), *quant_block_128x128(b), *quant_block_128x128(b1))
    if quant_mode == QUANT_CHANNEL:
        return (*quant_rowwise(a), *quant_rowwise(b), *quant_rowwise(b1))
    if quant_mode == QUANT_TENSOR:
        return (*quant_tensor(a), *quant_tensor(b, per_expert=True), *quant_tensor(b1, per_expert=True))
    if quant_mode == QUANT_MX:
        return (*quant_mx(a), *quant_mx(b), *quant_mx(b1))
    raise ValueError(quant_mode)


# ---------------------------------------------------------------------- metrics

def cosine(x: torch.Tensor, ref: torch.Tensor) -> float:
    x, ref = x.double().flatten(), ref.double().flatten()
    return float((x @ ref) / (x.norm() * ref.norm()).clamp(min=1e-300))


def max_rel_err(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max |x - ref| / max |ref| (the definition used by every layer-output tolerance here)."""
    return float((x.double() - ref.double()).abs().max() / ref.double().abs().max().clamp(min=1e-300))
