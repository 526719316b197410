"""Soft-capped sliding-window attention with kept first tokens, a distance bias and a sink over a paged cache —
csrc/attention/softcap_window_attention.cu.

``window_kv_append``: from a packed projection ``[q | k | v | ...]``: fp32 biases, unit-RMS norm of every value head, q in
fp32, ``[k | v]`` into the token's cache row (``[pages, bs, G d + G e]``).
``softcap_window_attention``: for query position i of head h and key position j <= i that is seen (``i - j < window`` or
``j < keep_first``; ``window`` 0 sees everything):

    s = q . k * scale;   cap > 0: s <- cap tanh(s / cap);   s <- s - slopes[h] (i - j)
    p = exp(s) / (sum over seen keys exp(s') + exp(sinks[h]))           (no sink term when ``sinks`` is None)
    o = sum p v, times sigmoid(gate) element by element where a gate is given

CPU tensors run the PyTorch restatements below (CPU tests); on a GPU a missing kernel raises.

Reference: none — the reference has no attention code (reference llmctl/serve/server.py:199-204)."""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import native
from .diff_attention import key_splits
from .elementwise import _is32

c_void_p, c_int, c_ll, c_float = native.c_void_p, native.c_int, native.c_ll, native.c_float
native.register_signature("llmctl_window_kv_append", [c_void_p, c_ll, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                                                       c_void_p, c_int, c_int, c_void_p])
native.register_signature("llmctl_softcap_attention_heads_per_cta", [c_int, c_int, c_int, c_int])
native.register_signature("llmctl_softcap_attention_mma_ok", [c_int, c_int, c_int, c_int, c_int])
native.register_signature("llmctl_softcap_window_attention", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_ll,
                                                               c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
                                                               c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p])
native._KERNELS_PER_CALL["llmctl_softcap_attention_heads_per_cta"] = 0
native._KERNELS_PER_CALL["llmctl_softcap_attention_mma_ok"] = 0

TILE_TOKENS = 16        # widest query tile of the FMA attention kernel
TILE_TOKENS_MMA = 128   # widest query tile of the tensor-core kernel (8 warps x 16 rows)


def distance_slopes(heads: int) -> torch.Tensor:
    """``2^(-8 (h + 1) / heads)`` for head h: the per-head slope of the linear distance bias, fp32 [heads]."""
    h = torch.arange(1, heads + 1, dtype=torch.float64)
    return torch.pow(torch.tensor(2.0, dtype=torch.float64), -8.0 * h / heads).to(torch.float32)


def window_kv_append(proj: torch.Tensor, bias: Optional[torch.Tensor], H: int, G: int, d: int, e: int, value_norm: bool, eps: float,
                     slots: torch.Tensor, cache: torch.Tensor) -> torch.Tensor:
    """proj: [T, >= H d + G d + G e] packed projection (unit column stride); bias: fp32 [H d + G d + G e] or None.
    Returns q: fp32 [T, H d]; writes ``[k | v]`` (values brought to unit RMS per head if ``value_norm``) into ``cache`` at
    ``slots`` (int64, page * bs + offset; negative = skip)."""
    T = proj.shape[0]
    Nq, Nk, Nv = H * d, G * d, G * e
    if proj.is_cuda:
        assert proj.stride(1) == 1 and cache.is_contiguous() and cache.dtype == proj.dtype and cache.shape[-1] == Nk + Nv
        assert bias is None or (bias.dtype == torch.float32 and bias.numel() == Nq + Nk + Nv)
        q = torch.empty(T, Nq, dtype=torch.float32, device=proj.device)
        native.call("llmctl_window_kv_append", proj.data_ptr(), proj.stride(0), native.ptr(bias), H, G, d, e, int(value_norm), float(eps),
                    slots.data_ptr(), q.data_ptr(), cache.data_ptr(), T, _is32(proj), native.stream_ptr())
        return q
    f = proj[:, :Nq + Nk + Nv].float()
    if bias is not None:
        f = f + bias
    v = f[:, Nq + Nk:].reshape(T, G, e)
    if value_norm:
        v = v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    ok = slots >= 0
    cache.view(-1, Nk + Nv)[slots[ok]] = torch.cat([f[:, Nq:Nq + Nk], v.reshape(T, Nv)], dim=-1)[ok].to(cache.dtype)
    return f[:, :Nq].contiguous()


def uses_tensor_cores(dtype: torch.dtype, H: int, G: int, d: int, e: int, tile_tokens: int) -> bool:
    """bf16 caches whose sizes fit the mma.sync kernel (d a multiple of 16, e a multiple of 8 up to 128, shared memory)
    run on it; fp32 and other sizes run the FMA kernel.  Same rule as llmctl_softcap_attention_mma_ok."""
    if dtype != torch.bfloat16 or not native.has_symbol("llmctl_softcap_attention_mma_ok"):
        return False
    if os.environ.get("LLMCTL_SOFTCAP_ATTENTION", "") == "fma":        # ablation switch: the FMA kernel for bf16 too
        return False
    return bool(native.lib().llmctl_softcap_attention_mma_ok(H, G, d, e, tile_tokens))


def tile_width(dtype: torch.dtype, H: int, G: int, d: int, e: int, cuda: bool, decode_only: bool) -> int:
    """Width of the ragged batch's query tiles the attention wants for a batch with prompt portions."""
    return TILE_TOKENS_MMA if cuda and not decode_only and uses_tensor_cores(dtype, H, G, d, e, TILE_TOKENS_MMA) else TILE_TOKENS


def softcap_window_attention(q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, tiles: torch.Tensor, tile_tokens: int,
                             positions: torch.Tensor, gate: Optional[torch.Tensor], slopes: Optional[torch.Tensor],
                             sinks: Optional[torch.Tensor], scale: float, cap: float, window: int, keep_first: int, H: int, G: int,
                             d: int, e: int, block_size: int, out_dtype: torch.dtype, max_context: int = 0, splits: int = 0,
                             tensor_cores: bool = True) -> torch.Tensor:
    """q: fp32 [T, H d]; tiles: int32 [n, 4] = (first token row, tokens <= tile_tokens, block-table row, 0), the tokens of a
    tile being consecutive positions of one sequence; gate: [T, H e] pre-sigmoid (a view with unit column stride) or None;
    slopes, sinks: fp32 [H] or None.  ``tile_tokens``: 1 (every tile is one decoded token), up to 16, or — where
    ``uses_tensor_cores`` — up to 128.  ``max_context`` (longest context in the batch) lets the kernel split the keys when
    tiles are few.  Returns [T, H e] in ``out_dtype``."""
    T = q.shape[0]
    bs = block_size
    if q.is_cuda:
        assert q.dtype == torch.float32 and q.is_contiguous() and cache.is_contiguous() and cache.dtype == out_dtype
        assert gate is None or (gate.stride(1) == 1 and gate.dtype == out_dtype)
        out = torch.empty(T, H * e, dtype=out_dtype, device=q.device)
        n = tiles.shape[0]
        mma = tensor_cores and uses_tensor_cores(cache.dtype, H, G, d, e, tile_tokens)
        assert mma or tile_tokens <= TILE_TOKENS
        hb = int(native.lib().llmctl_softcap_attention_heads_per_cta(H, G, int(tile_tokens), int(mma)))
        if mma and tile_tokens > 1:
            splits = 1                      # prompt tiles fill the tensor-core kernel's CTAs by themselves
        elif not splits:
            seen = min(max_context, window + keep_first) if window > 0 else max_context
            splits = key_splits(n * (H // hb), seen, 8 if mma else 2, 64 if mma else 128)
        part_ml = torch.empty(n * (H // hb) * splits * 64, dtype=torch.float32, device=q.device) if splits > 1 else None
        part_o = torch.empty(n * (H // hb) * splits * 32 * e, dtype=torch.float32, device=q.device) if splits > 1 else None
        native.call("llmctl_softcap_window_attention", q.data_ptr(), cache.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
                    tiles.data_ptr(), n, int(tile_tokens), positions.data_ptr(), native.ptr(gate), gate.stride(0) if gate is not None else 0,
                    native.ptr(slopes), native.ptr(sinks), float(scale), float(cap), int(window), int(keep_first), H, G, d, e, bs,
                    out.data_ptr(), int(splits), native.ptr(part_ml), native.ptr(part_o), _is32(cache), int(mma), native.stream_ptr())
        return out
    out = torch.zeros(T, H, e, dtype=torch.float32)
    flat = cache.view(-1, cache.shape[-1]).float()
    rep = H // G
    qh = q.view(T, H, d)
    for t0, n, seq, _ in tiles.tolist():
        table = block_tables[seq]
        for t in range(t0, t0 + n):
            i = int(positions[t])
            js = [j for j in range(i + 1) if window <= 0 or i - j < window or j < keep_first]
            kv = flat[[int(table[j // bs]) * bs + j % bs for j in js]]
            k = kv[:, :G * d].reshape(-1, G, d).repeat_interleave(rep, dim=1)               # [n, H, d]
            v = kv[:, G * d:].reshape(-1, G, e).repeat_interleave(rep, dim=1)               # [n, H, e]
            s = torch.einsum("hd,nhd->hn", qh[t], k) * scale
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            if slopes is not None:
                s = s - slopes.float()[:, None] * (i - torch.tensor(js, dtype=torch.float32))[None, :]
            if sinks is not None:
                w = torch.softmax(torch.cat([s, sinks.float()[:, None]], dim=-1), -1)[:, :-1]
            else:
                w = torch.softmax(s, -1)
            out[t] = torch.einsum("hn,nhe->he", w, v)
    out = out.reshape(T, H * e)
    if gate is not None:
        out = out * torch.sigmoid(gate.float())
    return out.to(out_dtype)
