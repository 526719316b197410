"""Recurrent sequence mixers over per-sequence state slots — csrc/recurrent/gla.cu, csrc/recurrent/selective_scan.cu.

A ragged batch describes its portions as int32 ``[n, 4] = (first token row, tokens, position of the first token, state
slot)``.  A portion that starts at position 0 starts from a zero state whatever its slot holds (slots are handed out
again without clearing); any other portion continues from its slot; the state after the portion's last token goes
back to the slot.  Slot -1 (padding rows of a fixed-shape batch) keeps no state.

``gla_scan`` / ``gla_output``: gated linear attention, state ``[slots, H, d, e]`` fp32.
``causal_conv_silu`` / ``selective_scan``: the short causal convolution and the selective state-space scan, state
``[slots, C, N]`` fp32 plus the last ``taps - 1`` raw convolution inputs ``[slots, taps - 1, C]`` fp32.
CPU tensors run the PyTorch restatements below (CPU tests); on a GPU a missing kernel raises.

Reference: none — the reference has no model code (reference llmctl/runtime/engine.py:119-140)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import native
from .elementwise import _is32

c_void_p, c_int, c_ll, c_float = native.c_void_p, native.c_int, native.c_ll, native.c_float
native.register_signature("llmctl_gla_scan", [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_void_p, c_int, c_int,
                                               c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p])
native._KERNELS_PER_CALL["llmctl_gla_scan"] = 2
native.register_signature("llmctl_gla_output", [c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p])
native.register_signature("llmctl_causal_conv_silu", [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                       c_int, c_int, c_int, c_void_p])
native.register_signature("llmctl_selective_scan", [c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p, c_ll, c_void_p, c_void_p, c_void_p,
                                                     c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                     c_int, c_int, c_int, c_void_p])


def gla_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, z_bias: Optional[torch.Tensor], portions: torch.Tensor,
             state: torch.Tensor, H: int, d: int, e: int, q_scale: float, tau: float) -> torch.Tensor:
    """q, k: [T, H d]; v: [T, H e]; z: [T, H d] decay logits (all views with unit column stride, one type); z_bias: fp32
    [H d] or None.  ``S <- diag(a) S + k v^T``, ``o = S^T (q_scale q)`` with ``a = sigmoid(z + z_bias)^(1/tau)`` per head.
    Updates ``state`` ([slots, H, d, e] fp32) in place; returns o: fp32 [T, H e]."""
    T = q.shape[0]
    if q.is_cuda:
        assert all(t.stride(1) == 1 and t.dtype == q.dtype for t in (q, k, v, z)) and state.dtype == torch.float32 and state.is_contiguous()
        out = torch.empty(T, H * e, dtype=torch.float32, device=q.device)
        work = torch.empty(T, 3 * H * d, dtype=torch.float32, device=q.device)        # prepared queries, keys, decays
        native.call("llmctl_gla_scan", q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), z.data_ptr(),
                    z.stride(0), native.ptr(z_bias), portions.data_ptr(), portions.shape[0], T, state.data_ptr(), out.data_ptr(),
                    work.data_ptr(), H, d, e, float(q_scale), float(tau), _is32(q), native.stream_ptr())
        return out
    out = torch.zeros(T, H, e, dtype=torch.float32)
    zf = z.float() + (z_bias if z_bias is not None else 0.0)
    a = torch.exp(F.logsigmoid(zf) / tau).view(T, H, d)
    qf, kf, vf = q.float().view(T, H, d) * q_scale, k.float().view(T, H, d), v.float().view(T, H, e)
    for t0, n, pos0, slot in portions.tolist():
        S = state[slot].clone() if (slot >= 0 and pos0 > 0) else torch.zeros(H, d, e)
        for t in range(t0, t0 + n):
            S = a[t][:, :, None] * S + kf[t][:, :, None] * vf[t][:, None, :]
            out[t] = torch.einsum("hde,hd->he", S, qf[t])
        if slot >= 0 and n > 0:
            state[slot] = S
    return out.reshape(T, H * e)


def gla_output(o: torch.Tensor, w: torch.Tensor, gate: torch.Tensor, H: int, e: int, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``o / sqrt(mean(o^2) + eps) * w * silu(gate)`` per (token, head); o: fp32 [T, H e]; w: fp32 [e]; gate: [T, H e]
    pre-activation (unit column stride).  Returns [T, H e] in ``out_dtype``."""
    T = o.shape[0]
    if o.is_cuda:
        assert o.is_contiguous() and gate.stride(1) == 1 and gate.dtype == out_dtype
        out = torch.empty(T, H * e, dtype=out_dtype, device=o.device)
        native.call("llmctl_gla_output", o.data_ptr(), w.data_ptr(), gate.data_ptr(), gate.stride(0), out.data_ptr(), T, H, e, float(eps),
                    int(out_dtype == torch.float32), native.stream_ptr())
        return out
    oh = o.view(T, H, e)
    y = oh / torch.sqrt(oh.pow(2).mean(-1, keepdim=True) + eps) * w
    return (y.reshape(T, H * e) * F.silu(gate.float())).to(out_dtype)


def causal_conv_silu(x: torch.Tensor, w: torch.Tensor, wb: Optional[torch.Tensor], portions: torch.Tensor, seq_rows: torch.Tensor,
                     conv_state: torch.Tensor) -> torch.Tensor:
    """x: [T, C] raw inputs (unit column stride); w: fp32 [C, taps], last column = the current token's; wb: fp32 [C] or
    None; conv_state: fp32 [slots, taps - 1, C], the raw inputs before each portion (read only; ``selective_scan`` stores
    the new ones).  Returns silu(conv) [T, C] in x's type."""
    T, C = x.shape
    taps = w.shape[1]
    if x.is_cuda:
        assert x.stride(1) == 1 and conv_state.is_contiguous()
        out = torch.empty(T, C, dtype=x.dtype, device=x.device)
        native.call("llmctl_causal_conv_silu", x.data_ptr(), x.stride(0), w.data_ptr(), native.ptr(wb), portions.data_ptr(),
                    seq_rows.data_ptr(), conv_state.data_ptr(), out.data_ptr(), T, C, taps, _is32(x), native.stream_ptr())
        return out
    out = torch.zeros(T, C, dtype=torch.float32)
    for t0, n, pos0, slot in portions.tolist():
        before = conv_state[slot] if (slot >= 0 and pos0 > 0) else torch.zeros(taps - 1, C)
        xs = torch.cat([before, x[t0:t0 + n].float()], dim=0)
        acc = torch.zeros(n, C)
        for j in range(taps):
            acc += xs[j:j + n] * w[:, j]
        out[t0:t0 + n] = acc + (wb if wb is not None else 0.0)
    return F.silu(out).to(x.dtype)


def selective_scan(u: torch.Tensor, bc: torch.Tensor, off_b: int, off_c: int, dtp: torch.Tensor, dt_bias: torch.Tensor, A: torch.Tensor,
                   D: torch.Tensor, z: torch.Tensor, x: torch.Tensor, portions: torch.Tensor, state: torch.Tensor,
                   conv_state: torch.Tensor) -> torch.Tensor:
    """u: [T, C] convolved inputs; bc: [T, *] with B at columns off_b.. and C at off_c.. (N each); dtp: [T, C]; dt_bias, D:
    fp32 [C]; A: fp32 [C, N] (negative); z: [T, C] gate pre-activation; x: [T, C] raw convolution inputs (views with unit
    column stride, one type).  ``S <- exp(dt A) S + dt u B``, ``y = (S C + D u) silu(z)``, ``dt = softplus(dtp + dt_bias)``.
    Updates ``state`` ([slots, C, N] fp32) and ``conv_state`` ([slots, taps - 1, C] fp32) in place; returns y [T, C] in u's type."""
    T, C = u.shape
    N = A.shape[1]
    keep = conv_state.shape[1]
    if u.is_cuda:
        assert u.is_contiguous() and all(t.stride(1) == 1 and t.dtype == u.dtype for t in (bc, dtp, z, x))
        assert state.is_contiguous() and conv_state.is_contiguous() and A.is_contiguous()
        out = torch.empty(T, C, dtype=u.dtype, device=u.device)
        native.call("llmctl_selective_scan", u.data_ptr(), bc.data_ptr(), bc.stride(0), off_b, off_c, dtp.data_ptr(), dtp.stride(0),
                    dt_bias.data_ptr(), A.data_ptr(), D.data_ptr(), z.data_ptr(), z.stride(0), x.data_ptr(), x.stride(0),
                    portions.data_ptr(), portions.shape[0], state.data_ptr(), conv_state.data_ptr(), out.data_ptr(), C, N, keep + 1,
                    _is32(u), native.stream_ptr())
        return out
    out = torch.zeros(T, C, dtype=torch.float32)
    uf, Bf, Cf = u.float(), bc[:, off_b:off_b + N].float(), bc[:, off_c:off_c + N].float()
    dt = F.softplus(dtp.float() + dt_bias)
    for t0, n, pos0, slot in portions.tolist():
        S = state[slot].clone() if (slot >= 0 and pos0 > 0) else torch.zeros(C, N)
        for t in range(t0, t0 + n):
            S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * uf[t])[:, None] * Bf[t][None, :]
            out[t] = S @ Cf[t] + D * uf[t]
        if slot >= 0 and n > 0:
            state[slot] = S
            before = conv_state[slot] if pos0 > 0 else torch.zeros(keep, C)
            conv_state[slot] = torch.cat([before, x[t0:t0 + n].float()], dim=0)[-keep:] if keep else conv_state[slot]
    return (out * F.silu(z.float())).to(u.dtype)
