"""Inference-side elementwise / normalisation ops that exist for bf16 AND fp32 activations: post-norm residual
update with a single gain, scalar-gain RMS norm of selected rows, scaled embedding lookup, logit soft-capping, xIELU
and gated SiLU, plus the frequency spectrum of interleaved-pair rotary embeddings (plain or YaRN-blended); for the
sandwich layout (a weighted RMS norm before and after every sublayer): embedding plus learned position vector,
weighted RMS norm of rows, fused out-norm + residual + next in-norm, and the squared ReLU; for the parallel layout (one
layer norm feeds mixer and feed-forward): layer norm of rows and the fused residual update + next layer norm, and the
clamped gate activation.
CUDA tensors run the kernels in csrc/norm/scalar_rmsnorm.cu, csrc/norm/sandwich_norm.cu, csrc/norm/parallel_norm.cu and
csrc/activation/xielu.cu;
CPU tensors run the PyTorch restatement below (CPU tests).  Sums, gains and the residual stream are fp32 in both.

Reference: none — the reference has no model code (reference llmctl/runtime/engine.py:119-140 loads HF models)."""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from . import native

c_void_p, c_int, c_ll, c_float = native.c_void_p, native.c_int, native.c_ll, native.c_float
native.register_signature("llmctl_postnorm_residual", [c_void_p, c_int, c_ll, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p])
native.register_signature("llmctl_scalar_rmsnorm", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p])
native.register_signature("llmctl_embed_scale", [c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int, c_int, c_void_p])
native.register_signature("llmctl_softcap", [c_void_p, c_ll, c_float, c_void_p])
native.register_signature("llmctl_xielu", [c_void_p, c_void_p, c_int, c_ll, c_float, c_float, c_void_p])
native.register_signature("llmctl_gated_silu", [c_void_p, c_ll, c_void_p, c_int, c_int, c_int, c_void_p])
native.register_signature("llmctl_gated_gelu_tanh", [c_void_p, c_ll, c_void_p, c_int, c_int, c_int, c_void_p])
native.register_signature("llmctl_sigmoid_gate", [c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_void_p])
native.register_signature("llmctl_relu_squared", [c_void_p, c_void_p, c_int, c_ll, c_void_p])
native.register_signature("llmctl_embed_positions", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
native.register_signature("llmctl_rmsnorm_rows", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
native.register_signature("llmctl_gated_clamped", [c_void_p, c_ll, c_void_p, c_int, c_int, c_int, c_float, c_float, c_void_p])
native.register_signature("llmctl_layernorm_rows", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                                     c_float, c_void_p])
native.register_signature("llmctl_parallel_residual", [c_void_p, c_int, c_ll, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                                                        c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p])
native.register_signature("llmctl_sandwich_residual", [c_void_p, c_int, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                                        c_int, c_float, c_void_p])


def _is32(t: torch.Tensor) -> int:
    if t.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError(f"activations must be bfloat16 or float32, got {t.dtype}")
    return int(t.dtype == torch.float32)


def rope_frequencies(dims: int, base: float, scaling: Optional[Dict[str, Any]] = None) -> Tuple[torch.Tensor, float]:
    """Per-pair frequencies ``f_i = base^(-2i/dims)`` (fp32, [dims/2]) and the factor applied to cos and sin.
    ``scaling`` = {factor, original, fast, slow} blends towards ``f_i / factor`` between the pairs that make
    ``fast`` and ``slow`` turns over ``original`` positions (YaRN), and raises the cos/sin amplitude to
    ``0.1 ln(factor) + 1``.  ``scaling`` = {factor} alone divides every frequency by ``factor`` (linear position
    interpolation)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    mult = 1.0
    if scaling and "original" not in scaling:
        f = f / float(scaling["factor"])
    elif scaling:
        factor, orig = float(scaling["factor"]), float(scaling["original"])

        def pair_of(turns: float) -> float:
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
        hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp_(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    return f.to(torch.float32), float(mult)


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, mult: float) -> torch.Tensor:
    """CPU restatement of csrc/rope/rope_interleaved.cuh: x [T, ..., 2 * len(freq)] fp32."""
    ang = positions.to(torch.float32).unsqueeze(-1) * freq
    cos, sin = torch.cos(ang) * mult, torch.sin(ang) * mult
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    u, v = x[..., 0::2], x[..., 1::2]
    return torch.stack([u * cos - v * sin, v * cos + u * sin], dim=-1).flatten(-2)


def embed_scale(tokens: torch.Tensor, table: torch.Tensor, scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x = table[tokens] * scale`` -> (fp32 residual stream, the same in the table's type)."""
    T, W = tokens.numel(), table.shape[1]
    if table.is_cuda:
        x = torch.empty(T, W, dtype=torch.float32, device=table.device)
        xa = x if table.dtype == torch.float32 else torch.empty(T, W, dtype=table.dtype, device=table.device)
        native.call("llmctl_embed_scale", tokens.data_ptr(), table.data_ptr(), _is32(table), float(scale), x.data_ptr(),
                    None if xa is x else xa.data_ptr(), T, W, native.stream_ptr())
        return x, xa
    x = table[tokens.reshape(-1)].float() * scale
    return x, (x if table.dtype == torch.float32 else x.to(table.dtype))


def postnorm_residual(y: torch.Tensor, x: torch.Tensor, gain: torch.Tensor, eps: float, act_dtype: torch.dtype) -> torch.Tensor:
    """``x += gain * y / rms(y)`` in place on the fp32 stream ``x``; returns the new stream in ``act_dtype`` (``x``
    itself for fp32).  ``y``: [T, W] bf16 or fp32; ``gain``: one fp32 number on x's device."""
    T, W = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and y.shape == x.shape and y.stride(1) == 1
    if x.is_cuda:
        xa = x if act_dtype == torch.float32 else torch.empty(T, W, dtype=act_dtype, device=x.device)
        native.call("llmctl_postnorm_residual", y.data_ptr(), _is32(y), y.stride(0), x.data_ptr(),
                    None if xa is x else xa.data_ptr(), int(act_dtype == torch.float32), gain.data_ptr(), T, W, float(eps),
                    native.stream_ptr())
        return xa
    yf = y.float()
    x += yf * (gain.float() / torch.sqrt(yf.pow(2).mean(-1, keepdim=True) + eps))
    return x if act_dtype == torch.float32 else x.to(act_dtype)


def scalar_rmsnorm(x: torch.Tensor, rows: Optional[torch.Tensor], gain: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``gain * x[rows] / rms(x[rows])`` of the fp32 stream (all rows when ``rows`` is None) in ``out_dtype``."""
    n = x.shape[0] if rows is None else rows.numel()
    if x.is_cuda:
        out = torch.empty(n, x.shape[1], dtype=out_dtype, device=x.device)
        native.call("llmctl_scalar_rmsnorm", x.data_ptr(), native.ptr(rows), out.data_ptr(), int(out_dtype == torch.float32),
                    gain.data_ptr(), n, x.shape[1], float(eps), native.stream_ptr())
        return out
    xs = x if rows is None else x[rows]
    return (xs * (gain.float() / torch.sqrt(xs.pow(2).mean(-1, keepdim=True) + eps))).to(out_dtype)


def softcap_(logits: torch.Tensor, cap: float) -> torch.Tensor:
    """``cap * tanh(logits / cap)`` in place on fp32 logits."""
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    if logits.is_cuda:
        native.call("llmctl_softcap", logits.data_ptr(), logits.numel(), float(cap), native.stream_ptr())
        return logits
    return logits.copy_(cap * torch.tanh(logits / cap))


def xielu_coefficients(p: torch.Tensor) -> Tuple[float, float]:
    """(a_pos, a_neg) = (softplus(p0), 1/2 + softplus(p1)) in fp32 from the layer's two learned numbers."""
    sp = F.softplus(p.detach().float().cpu())
    return float(sp[0]), float(0.5 + sp[1])


def xielu(z: torch.Tensor, a_pos: float, a_neg: float) -> torch.Tensor:
    """z > 0: a_pos z^2 + z/2;  z <= 0: a_neg (exp(z) - 1 - z) + z/2."""
    if z.is_cuda:
        z = z.contiguous()
        out = torch.empty_like(z)
        native.call("llmctl_xielu", z.data_ptr(), out.data_ptr(), _is32(z), z.numel(), a_pos, a_neg, native.stream_ptr())
        return out
    v = z.float()
    return torch.where(v > 0, a_pos * v * v + 0.5 * v, a_neg * (torch.expm1(v.clamp(max=0.0)) - v) + 0.5 * v).to(z.dtype)


def gated_silu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` of a packed [rows, 2F] activation (gate first), bf16 or fp32."""
    rows, F2 = gate_up.shape
    if gate_up.is_cuda:
        assert gate_up.stride(1) == 1
        out = torch.empty(rows, F2 // 2, dtype=gate_up.dtype, device=gate_up.device)
        native.call("llmctl_gated_silu", gate_up.data_ptr(), gate_up.stride(0), out.data_ptr(), _is32(gate_up), rows, F2 // 2,
                    native.stream_ptr())
        return out
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def gated_gelu_tanh(gate_up: torch.Tensor) -> torch.Tensor:
    """``gelu_tanh(gate) * up`` of a packed [rows, 2F] activation (gate first), bf16 or fp32;
    ``gelu_tanh(g) = g/2 (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3)))``."""
    rows, F2 = gate_up.shape
    if gate_up.is_cuda:
        assert gate_up.stride(1) == 1
        out = torch.empty(rows, F2 // 2, dtype=gate_up.dtype, device=gate_up.device)
        native.call("llmctl_gated_gelu_tanh", gate_up.data_ptr(), gate_up.stride(0), out.data_ptr(), _is32(gate_up), rows, F2 // 2,
                    native.stream_ptr())
        return out
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.gelu(g, approximate="tanh") * u).to(gate_up.dtype)


def sigmoid_gate_(y: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
    """``y *= sigmoid(z)`` in place; y: contiguous [rows, F]; z: [rows, F] pre-activation gates, a view with unit column
    stride of the same type."""
    rows, Fc = y.shape
    assert y.is_contiguous() and z.shape == y.shape and z.stride(1) == 1 and z.dtype == y.dtype
    if y.is_cuda:
        native.call("llmctl_sigmoid_gate", y.data_ptr(), z.data_ptr(), z.stride(0), _is32(y), rows, Fc, native.stream_ptr())
        return y
    return y.copy_((y.float() * torch.sigmoid(z.float())).to(y.dtype))


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    """``max(z, 0)^2``, evaluated in fp32, in z's type."""
    if z.is_cuda:
        z = z.contiguous()
        out = torch.empty_like(z)
        native.call("llmctl_relu_squared", z.data_ptr(), out.data_ptr(), _is32(z), z.numel(), native.stream_ptr())
        return out
    return torch.relu(z.float()).pow(2).to(z.dtype)


def embed_positions(tokens: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, pos_table: torch.Tensor) -> torch.Tensor:
    """``x[t] = table[tokens[t]] + pos_table[positions[t]]`` -> the fp32 residual stream [T, W]."""
    T, W = tokens.numel(), table.shape[1]
    if table.is_cuda:
        x = torch.empty(T, W, dtype=torch.float32, device=table.device)
        native.call("llmctl_embed_positions", tokens.data_ptr(), positions.data_ptr(), table.data_ptr(), pos_table.data_ptr(),
                    _is32(table), x.data_ptr(), T, W, native.stream_ptr())
        return x
    return table[tokens.reshape(-1)].float() + pos_table[positions.reshape(-1).long()].float()


def rmsnorm_rows(x: torch.Tensor, rows: Optional[torch.Tensor], w: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``w * x[rows] / rms(x[rows])`` of the fp32 stream (all rows when ``rows`` is None) in ``out_dtype``; w: fp32 [W]."""
    n = x.shape[0] if rows is None else rows.numel()
    assert x.dtype == torch.float32 and w.dtype == torch.float32
    if x.is_cuda:
        out = torch.empty(n, x.shape[1], dtype=out_dtype, device=x.device)
        native.call("llmctl_rmsnorm_rows", x.data_ptr(), native.ptr(rows), w.data_ptr(), out.data_ptr(), int(out_dtype == torch.float32),
                    n, x.shape[1], float(eps), native.stream_ptr())
        return out
    xs = x if rows is None else x[rows]
    return (xs / torch.sqrt(xs.pow(2).mean(-1, keepdim=True) + eps) * w).to(out_dtype)


def sandwich_residual(y: torch.Tensor, x: torch.Tensor, w_out: torch.Tensor, w_next: Optional[torch.Tensor], eps: float,
                      act_dtype: torch.dtype, want_fp32: bool = False):
    """``x += w_out * y / rms(y)`` in place on the fp32 stream; with ``w_next`` also returns ``w_next * x / rms(x)`` of the
    new stream in ``act_dtype`` (the next sublayer's input) from the same pass.  Weights: fp32 [W].  ``want_fp32``: returns
    (input in ``act_dtype``, the same before rounding in fp32) — a router reads the unrounded one."""
    T, W = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and y.shape == x.shape and y.stride(1) == 1
    if x.is_cuda:
        out = torch.empty(T, W, dtype=act_dtype, device=x.device) if w_next is not None else None
        out32 = None
        if want_fp32 and w_next is not None and act_dtype != torch.float32:
            out32 = torch.empty(T, W, dtype=torch.float32, device=x.device)
        native.call("llmctl_sandwich_residual", y.data_ptr(), _is32(y), y.stride(0), x.data_ptr(), w_out.data_ptr(), native.ptr(w_next),
                    native.ptr(out), int(act_dtype == torch.float32), native.ptr(out32), T, W, float(eps), native.stream_ptr())
        return (out, out if out32 is None else out32) if want_fp32 else out
    yf = y.float()
    x += yf / torch.sqrt(yf.pow(2).mean(-1, keepdim=True) + eps) * w_out
    if w_next is None:
        return (None, None) if want_fp32 else None
    h32 = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w_next
    h = h32.to(act_dtype)
    return (h, h32) if want_fp32 else h


def gated_clamped(gate_up: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """``g sigmoid(alpha g) (u + 1)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)`` of a packed
    [rows, 2F] activation (gate first), bf16 or fp32."""
    rows, F2 = gate_up.shape
    if gate_up.is_cuda:
        assert gate_up.stride(1) == 1
        out = torch.empty(rows, F2 // 2, dtype=gate_up.dtype, device=gate_up.device)
        native.call("llmctl_gated_clamped", gate_up.data_ptr(), gate_up.stride(0), out.data_ptr(), _is32(gate_up), rows, F2 // 2,
                    float(limit), float(alpha), native.stream_ptr())
        return out
    g, u = gate_up.float().chunk(2, dim=-1)
    g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(gate_up.dtype)


def _layernorm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt((x - mu).pow(2).mean(-1, keepdim=True) + eps) * w + b


def layernorm_rows(x: torch.Tensor, rows: Optional[torch.Tensor], w: torch.Tensor, b: torch.Tensor, eps: float,
                   out_dtype: torch.dtype, add: Optional[torch.Tensor] = None, want_fp32: bool = False):
    """Layer norm ``(x - mean) / sqrt(var + eps) * w + b`` of the fp32 stream's rows (all when ``rows`` is None) in
    ``out_dtype``; ``add`` (fp32 [W], only with all rows) is first added to the stream in place.  ``want_fp32``: returns
    (normed in ``out_dtype``, the same before rounding)."""
    n = x.shape[0] if rows is None else rows.numel()
    assert x.dtype == torch.float32 and x.is_contiguous() and w.dtype == torch.float32 and b.dtype == torch.float32
    assert add is None or rows is None
    if x.is_cuda:
        out = torch.empty(n, x.shape[1], dtype=out_dtype, device=x.device)
        out32 = torch.empty(n, x.shape[1], dtype=torch.float32, device=x.device) if want_fp32 and out_dtype != torch.float32 else None
        native.call("llmctl_layernorm_rows", x.data_ptr(), native.ptr(rows), native.ptr(add), w.data_ptr(), b.data_ptr(), out.data_ptr(),
                    int(out_dtype == torch.float32), native.ptr(out32), n, x.shape[1], float(eps), native.stream_ptr())
        return (out, out if out32 is None else out32) if want_fp32 else out
    if add is not None:
        x += add
    h32 = _layernorm(x if rows is None else x[rows], w, b, eps)
    h = h32.to(out_dtype)
    return (h, h32) if want_fp32 else h


def parallel_residual(a: torch.Tensor, f: Optional[torch.Tensor], x: torch.Tensor, mult: float, eps: float, act_dtype: torch.dtype,
                      w_next: Optional[torch.Tensor] = None, b_next: Optional[torch.Tensor] = None,
                      add: Optional[torch.Tensor] = None, want_fp32: bool = False):
    """``x += mult * (a + f)`` in place on the fp32 stream (a: [T, W] mixer output, bf16 or fp32; f: fp32 feed-forward
    output or None), then ``x += add`` if given; with ``w_next`` / ``b_next`` also returns the layer norm of the new
    stream (the next layer's input) from the same pass, as ``layernorm_rows`` does."""
    T, W = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous() and a.shape == x.shape and a.stride(1) == 1
    assert f is None or (f.dtype == torch.float32 and f.is_contiguous() and f.shape == x.shape)
    if x.is_cuda:
        out = torch.empty(T, W, dtype=act_dtype, device=x.device) if w_next is not None else None
        out32 = None
        if want_fp32 and w_next is not None and act_dtype != torch.float32:
            out32 = torch.empty(T, W, dtype=torch.float32, device=x.device)
        native.call("llmctl_parallel_residual", a.data_ptr(), _is32(a), a.stride(0), native.ptr(f), x.data_ptr(), float(mult),
                    native.ptr(add), native.ptr(w_next), native.ptr(b_next), native.ptr(out), int(act_dtype == torch.float32),
                    native.ptr(out32), T, W, float(eps), native.stream_ptr())
        return (out, out if out32 is None else out32) if want_fp32 else out
    x += mult * (a.float() + (f if f is not None else 0.0))
    if add is not None:
        x += add
    if w_next is None:
        return (None, None) if want_fp32 else None
    h32 = _layernorm(x, w_next, b_next, eps)
    h = h32.to(act_dtype)
    return (h, h32) if want_fp32 else h
