"""Pre-norm with an input convolution over time ("canon" convolution) on an fp32 residual stream — csrc/norm/canon_norm.cu.

All sublayers of a layer read the same normed stream ``n = x / sqrt(mean(x^2) + eps)``, each through its own norm weight
and its own short causal depthwise convolution: ``h = w n``, ``out = h + conv(h)``, ``conv(h)_t = sum_j c[:, j]
h_(t - taps + 1 + j)`` with zeros before position 0.  The last ``taps - 1`` rows of ``n`` of every sequence live in its
state slot (``[slots, taps - 1, W]`` fp32, oldest first), so a prompt may be cut anywhere.

``residual_rms`` is the residual update ``x += a + f`` fused with the statistics of the next norm; ``norm_canon`` forms
the sublayers' inputs from ``x`` and those statistics and then rewrites the state.  CPU tensors run the PyTorch
restatements below (CPU tests); on a GPU a missing kernel raises.

Reference: none — the reference has no model code (reference llmctl/runtime/engine.py:119-140)."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import native
from .elementwise import _is32

c_void_p, c_int, c_ll, c_float = native.c_void_p, native.c_int, native.c_ll, native.c_float
native.register_signature("llmctl_residual_rms", [c_void_p, c_int, c_ll, c_void_p, c_int, c_ll, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p])
native.register_signature("llmctl_norm_canon", [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                 c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
native._KERNELS_PER_CALL["llmctl_norm_canon"] = 2
native.register_signature("llmctl_residual_norm_canon_small", [c_void_p, c_int, c_ll, c_void_p, c_int, c_ll, c_void_p, c_float, c_int, c_void_p,
                                                                c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                                c_int, c_int, c_int, c_void_p])

MAX_TAPS = 8
SMALL_PORTION = 8       # portions of at most this many tokens each can take the single-launch path


def residual_rms(a: Optional[torch.Tensor], f: Optional[torch.Tensor], x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x += a + f`` in place on the fp32 stream (a, f: [T, W] bf16 or fp32 with unit column stride, or None); returns
    ``1 / sqrt(mean(x^2) + eps)`` of the new rows, fp32 [T]."""
    T, W = x.shape
    assert x.dtype == torch.float32 and x.is_contiguous()
    for t in (a, f):
        assert t is None or (t.shape == x.shape and t.stride(1) == 1)
    if x.is_cuda:
        r = torch.empty(T, dtype=torch.float32, device=x.device)
        native.call("llmctl_residual_rms", native.ptr(a), _is32(a) if a is not None else 0, a.stride(0) if a is not None else 0,
                    native.ptr(f), _is32(f) if f is not None else 0, f.stride(0) if f is not None else 0, x.data_ptr(), r.data_ptr(),
                    T, W, float(eps), native.stream_ptr())
        return r
    if a is not None or f is not None:
        x += (a.float() if a is not None else 0.0) + (f.float() if f is not None else 0.0)
    return torch.rsqrt(x.pow(2).mean(-1) + eps)


def norm_canon(x: torch.Tensor, r: torch.Tensor, norm_w: Sequence[torch.Tensor], conv_w: Sequence[torch.Tensor], portions: torch.Tensor,
               seq_rows: torch.Tensor, state: torch.Tensor, out_dtype: torch.dtype) -> List[torch.Tensor]:
    """x: fp32 [T, W]; r: fp32 [T] from ``residual_rms``; norm_w[s]: fp32 [W]; conv_w[s]: fp32 [W, taps] (last column = the
    current token's), one pair per sublayer (one or two); portions: int32 [B, 4] = (first token row, tokens, position of
    the first token, state slot); seq_rows: int32 [T], the portion of every token; state: fp32 [slots, taps - 1, W],
    updated in place.  Returns one [T, W] tensor in ``out_dtype`` per sublayer."""
    T, W = x.shape
    S, taps = len(norm_w), conv_w[0].shape[1]
    assert S in (1, 2) and len(conv_w) == S and 1 <= taps <= MAX_TAPS and state.shape[1:] == (taps - 1, W)
    if x.is_cuda:
        assert x.is_contiguous() and state.is_contiguous() and all(w.is_contiguous() and w.dtype == torch.float32 for w in (*norm_w, *conv_w))
        outs = [torch.empty(T, W, dtype=out_dtype, device=x.device) for _ in range(S)]
        native.call("llmctl_norm_canon", x.data_ptr(), r.data_ptr(), S, norm_w[0].data_ptr(), conv_w[0].data_ptr(), outs[0].data_ptr(),
                    native.ptr(norm_w[1]) if S > 1 else None, native.ptr(conv_w[1]) if S > 1 else None,
                    outs[1].data_ptr() if S > 1 else None, portions.data_ptr(), portions.shape[0], seq_rows.data_ptr(),
                    state.data_ptr() if taps > 1 else None, T, W, taps, int(out_dtype == torch.float32), native.stream_ptr())
        return outs
    n = x * r[:, None]
    keep = taps - 1
    outs = [torch.zeros(T, W, dtype=torch.float32) for _ in range(S)]
    for t0, cnt, pos0, slot in portions.tolist():
        if cnt <= 0:
            continue
        before = state[slot] if (slot >= 0 and pos0 > 0) else torch.zeros(keep, W)
        rows = torch.cat([before, n[t0:t0 + cnt]], dim=0)                    # [keep + cnt, W]
        for s in range(S):
            acc = rows[keep:].clone()
            for j in range(taps):
                acc += rows[j:j + cnt] * conv_w[s][:, j]
            outs[s][t0:t0 + cnt] = acc * norm_w[s]
        if slot >= 0 and keep:
            state[slot] = rows[-keep:]
    return [o.to(out_dtype) for o in outs]


def residual_norm_canon(a: Optional[torch.Tensor], f: Optional[torch.Tensor], x: torch.Tensor, eps: float, norm_w: Sequence[torch.Tensor],
                        conv_w: Sequence[torch.Tensor], portions: torch.Tensor, seq_rows: torch.Tensor, state: torch.Tensor,
                        out_dtype: torch.dtype, small: bool = False) -> List[torch.Tensor]:
    """``residual_rms`` followed by ``norm_canon``: the end of one layer and the start of the next.  ``small``: every portion
    has at most ``SMALL_PORTION`` tokens (a decoding batch) — on a GPU the whole step is then one launch."""
    if small and x.is_cuda:
        T, W = x.shape
        S, taps = len(norm_w), conv_w[0].shape[1]
        assert x.dtype == torch.float32 and x.is_contiguous() and state.is_contiguous() and S in (1, 2) and 1 <= taps <= MAX_TAPS
        for t in (a, f):
            assert t is None or (t.shape == x.shape and t.stride(1) == 1)
        outs = [torch.empty(T, W, dtype=out_dtype, device=x.device) for _ in range(S)]
        native.call("llmctl_residual_norm_canon_small", native.ptr(a), _is32(a) if a is not None else 0, a.stride(0) if a is not None else 0,
                    native.ptr(f), _is32(f) if f is not None else 0, f.stride(0) if f is not None else 0, x.data_ptr(), float(eps), S,
                    norm_w[0].data_ptr(), conv_w[0].data_ptr(), outs[0].data_ptr(), native.ptr(norm_w[1]) if S > 1 else None,
                    native.ptr(conv_w[1]) if S > 1 else None, outs[1].data_ptr() if S > 1 else None, portions.data_ptr(),
                    portions.shape[0], state.data_ptr() if taps > 1 else None, W, taps, int(out_dtype == torch.float32), native.stream_ptr())
        return outs
    r = residual_rms(a, f, x, eps)
    return norm_canon(x, r, norm_w, conv_w, portions, seq_rows, state, out_dtype)
