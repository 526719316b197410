"""Differential attention over a paged cache — csrc/attention/diff_attention.cu.

Every query head has two query vectors and its key/value head two key vectors; each pair gives a causal softmax map of
its own over the SAME values, and the head's output is ``a1 - lam * a2``, brought to unit RMS, times ``post_scale`` and
an optional per-(token, head) sigmoid gate.  A layer's cache is ``[pages, bs, G*2*d + G*e]``: a token's row holds the
keys of all heads (head by head as [map 1 | map 2]) and then the values.  ``rotary_kv_append`` rotates the first ``rot``
numbers of every query and key vector and appends keys and values to the cache; ``diff_attention`` is the attention.
CPU tensors run the PyTorch restatement below (CPU tests); on a GPU a missing kernel raises.

Reference: none — the reference has no attention code (reference llmctl/serve/server.py:199-204)."""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import native
from .elementwise import _is32, rotate_interleaved

c_void_p, c_int, c_ll, c_float = native.c_void_p, native.c_int, native.c_ll, native.c_float
native.register_signature("llmctl_rotary_kv_append", [c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p,
                                                       c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
native.register_signature("llmctl_diff_attention_heads_per_cta", [c_int, c_int, c_int])
native.register_signature("llmctl_diff_attention", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_ll,
                                                     c_float, c_float, c_float, c_float, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                     c_int, c_void_p, c_void_p, c_int, c_int, c_void_p])
native.register_signature("llmctl_diff_attention_mma_ok", [c_int, c_int, c_int, c_int, c_int])
native._KERNELS_PER_CALL["llmctl_diff_attention_heads_per_cta"] = 0
native._KERNELS_PER_CALL["llmctl_diff_attention_mma_ok"] = 0

TILE_TOKENS = 16        # widest query tile of the FMA attention kernel
TILE_TOKENS_MMA = 128   # widest query tile of the tensor-core kernel (8 warps x 16 rows)


def rotary_kv_append(proj: torch.Tensor, nq: int, nk: int, d: int, nv: int, rot: int, freq: torch.Tensor, mult: float,
                     positions: torch.Tensor, slots: torch.Tensor, cache: torch.Tensor) -> torch.Tensor:
    """proj: [T, >= (nq + nk) d + nv] packed projection (nq query vectors, nk key vectors of d numbers, nv value numbers);
    the first ``rot`` numbers of every query and key vector are rotated as interleaved pairs at the token's position.
    Returns q: fp32 [T, nq d]; writes ``[k | v]`` into ``cache`` ([pages, bs, nk d + nv]) at ``slots`` (int64, page * bs +
    offset; negative = skip)."""
    T = proj.shape[0]
    Nq, Nk = nq * d, nk * d
    if proj.is_cuda:
        assert proj.stride(1) == 1 and cache.is_contiguous() and cache.dtype == proj.dtype and cache.shape[-1] == Nk + nv
        q = torch.empty(T, Nq, dtype=torch.float32, device=proj.device)
        native.call("llmctl_rotary_kv_append", proj.data_ptr(), proj.stride(0), nq, nk, d, nv, rot, native.ptr(freq), float(mult),
                    positions.data_ptr(), slots.data_ptr(), q.data_ptr(), cache.data_ptr(), T, _is32(proj), native.stream_ptr())
        return q
    f = proj.float()
    q = f[:, :Nq].reshape(T, nq, d).clone()
    k = f[:, Nq:Nq + Nk].reshape(T, nk, d).clone()
    if rot:
        q[..., :rot] = rotate_interleaved(q[..., :rot], positions, freq, mult)
        k[..., :rot] = rotate_interleaved(k[..., :rot], positions, freq, mult)
    ok = slots >= 0
    cache.view(-1, Nk + nv)[slots[ok]] = torch.cat([k.reshape(T, Nk), f[:, Nq + Nk:Nq + Nk + nv]], dim=-1)[ok].to(cache.dtype)
    return q.reshape(T, Nq)


def uses_tensor_cores(dtype: torch.dtype, H: int, G: int, d: int, e: int, tile_tokens: int) -> bool:
    """bf16 caches whose sizes fit the mma.sync kernel (d a multiple of 16, e a multiple of 8 up to 128, shared memory)
    run on it; fp32 and other sizes run the FMA kernel.  Same rule as llmctl_diff_attention_mma_ok."""
    if dtype != torch.bfloat16 or not native.has_symbol("llmctl_diff_attention_mma_ok"):
        return False
    if os.environ.get("LLMCTL_DIFF_ATTENTION", "") == "fma":           # ablation switch: the FMA kernel for bf16 too
        return False
    return bool(native.lib().llmctl_diff_attention_mma_ok(H, G, d, e, tile_tokens))


def tile_width(dtype: torch.dtype, H: int, G: int, d: int, e: int, cuda: bool, decode_only: bool) -> int:
    """Width of the ragged batch's query tiles the attention wants for a batch with prompt portions."""
    return TILE_TOKENS_MMA if cuda and not decode_only and uses_tensor_cores(dtype, H, G, d, e, TILE_TOKENS_MMA) else TILE_TOKENS


def heads_per_cta(H: int, G: int, tile_tokens: int) -> int:
    return int(native.lib().llmctl_diff_attention_heads_per_cta(H, G, tile_tokens))


def key_splits(ctas: int, max_context: int, per_sm: int = 2, min_keys: int = 128, sms: int = 148) -> int:
    """Slices to cut every tile's keys into: with few CTAs (a decoding batch) and long contexts the keys are spread
    over about ``per_sm`` CTAs per SM, at least ``min_keys`` keys per slice (the tensor-core kernel's decode CTAs are
    single warps on 32-key tiles: 8 per SM, 64 keys)."""
    return int(max(1, min(per_sm * sms // max(ctas, 1), max_context // min_keys, 64)))


def diff_attention(q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, tiles: torch.Tensor, tile_tokens: int,
                   positions: torch.Tensor, gate: Optional[torch.Tensor], scale: float, lam: float, post_scale: float, eps: float,
                   H: int, G: int, d: int, e: int, block_size: int, out_dtype: torch.dtype, max_context: int = 0,
                   splits: int = 0, tensor_cores: bool = True) -> torch.Tensor:
    """q: fp32 [T, H*2*d] (rotated); tiles: int32 [n, 4] = (first token row, tokens <= tile_tokens, block-table row, 0),
    the tokens of a tile being consecutive positions of one sequence; gate: [T, H] pre-sigmoid (a view with unit column
    stride) or None.  ``tile_tokens``: 1 (every tile is one decoded token), up to 16, or — where ``uses_tensor_cores`` —
    up to 128.  ``tensor_cores`` False forces the FMA kernel.  ``max_context`` (longest context in the batch) lets the
    kernel split the keys when tiles are few.
    Returns [T, H e] in ``out_dtype``."""
    T = q.shape[0]
    bs = block_size
    if q.is_cuda:
        assert q.dtype == torch.float32 and q.is_contiguous() and cache.is_contiguous() and cache.dtype == out_dtype
        assert gate is None or (gate.stride(1) == 1 and gate.dtype == out_dtype)
        out = torch.empty(T, H * e, dtype=out_dtype, device=q.device)
        n = tiles.shape[0]
        mma = tensor_cores and uses_tensor_cores(cache.dtype, H, G, d, e, tile_tokens)
        assert mma or tile_tokens <= TILE_TOKENS
        if mma and tile_tokens > 1:
            hb, splits = 1, 1               # prompt tiles fill the tensor-core kernel's CTAs by themselves
        else:
            hb = heads_per_cta(H, G, tile_tokens)
            if not splits:
                splits = key_splits(n * (H // hb), max_context, 8 if mma else 2, 64 if mma else 128)
        part_ml = torch.empty(n * (H // hb) * splits * 64, dtype=torch.float32, device=q.device) if splits > 1 else None
        part_o = torch.empty(n * (H // hb) * splits * 32 * e, dtype=torch.float32, device=q.device) if splits > 1 else None
        native.call("llmctl_diff_attention", q.data_ptr(), cache.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
                    tiles.data_ptr(), n, int(tile_tokens), positions.data_ptr(), native.ptr(gate), gate.stride(0) if gate is not None else 0,
                    float(scale), float(lam), float(post_scale), float(eps), H, G, d, e, bs, out.data_ptr(), int(splits),
                    native.ptr(part_ml), native.ptr(part_o), _is32(cache), int(mma), native.stream_ptr())
        return out
    out = torch.zeros(T, H, e, dtype=torch.float32)
    flat = cache.view(-1, cache.shape[-1]).float()
    rep = H // G
    qh = q.view(T, H, 2, d)
    for t0, n, seq, _ in tiles.tolist():
        table = block_tables[seq]
        for t in range(t0, t0 + n):
            i = int(positions[t])
            rows = [int(table[j // bs]) * bs + j % bs for j in range(i + 1)]
            kv = flat[rows]
            k = kv[:, :G * 2 * d].reshape(-1, G, 2, d).repeat_interleave(rep, dim=1)        # [n, H, 2, d]
            v = kv[:, G * 2 * d:].reshape(-1, G, e).repeat_interleave(rep, dim=1)           # [n, H, e]
            w = torch.softmax(torch.einsum("hmd,nhmd->hmn", qh[t], k) * scale, -1)
            a = torch.einsum("hmn,nhe->hme", w, v)
            o = a[:, 0] - lam * a[:, 1]
            o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * post_scale
            if gate is not None:
                o = o * torch.sigmoid(gate[t].float())[:, None]
            out[t] = o
    return out.reshape(T, H * e).to(out_dtype)
