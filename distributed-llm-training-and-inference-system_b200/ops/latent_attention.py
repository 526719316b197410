"""Latent (low-rank joint key/value) attention over a paged cache — csrc/attention/latent_attention.cu.

The cache row of a token is ``[c | kr]``: the normed latent (R numbers) and the rotated key part shared by all heads
(dr numbers).  ``latent_kv_write`` norms the query latent, norms + rotates + appends the key/value side;
``latent_attention`` is multi-query attention of absorbed queries against those rows for a ragged batch (portions
of prompts next to single decoded tokens).  CPU tensors run a PyTorch restatement.

Reference: none — the reference has no attention code (reference llmctl/serve/server.py:199-204)."""
from __future__ import annotations

from typing import Optional

import torch

from . import native
from .elementwise import _is32, rotate_interleaved

c_void_p, c_int, c_ll, c_float = native.c_void_p, native.c_int, native.c_ll, native.c_float
native.register_signature("llmctl_latent_kv_write", [c_void_p, c_ll, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                      c_void_p, c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_void_p])
native.register_signature("llmctl_latent_attention", [c_void_p, c_int, c_ll, c_ll, c_void_p, c_ll, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                                       c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_int,
                                                       c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p])
native._KERNELS_PER_CALL["llmctl_latent_attention"] = 1
native.register_signature("llmctl_latent_attention_t5_ok", [c_int, c_int, c_int])
native.register_signature("llmctl_latent_attention_t5_status", [c_int])
native.register_signature("llmctl_latent_attention_t5", [c_void_p, c_int, c_ll, c_ll, c_void_p, c_ll, c_int, c_void_p, c_ll, c_void_p, c_int, c_int,
                                                          c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_int,
                                                          c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
native._KERNELS_PER_CALL["llmctl_latent_attention_t5"] = 2

ROWS_PER_TILE = 16          # query rows (token, head) a CTA owns; tiles are built by the engine with this limit
ROWS_PER_TILE_WIDE = 32     # the tensor-core kernel also takes tiles of 32 rows (half the key traffic per row)
ROWS_PER_TILE_TCGEN05 = 128     # query rows per CTA of the tcgen05 kernel (UMMA M)
TILE_WIDTHS = (ROWS_PER_TILE, ROWS_PER_TILE_WIDE, ROWS_PER_TILE_TCGEN05)


def uses_tensor_cores(dtype: torch.dtype, R: int, dr: int) -> bool:
    """bf16 with these sizes runs the mma.sync kernel (which also takes bf16 absorbed queries); same rule as
    llmctl_latent_attention_uses_tensor_cores."""
    return dtype == torch.bfloat16 and (R + dr) % 16 == 0 and R % 8 == 0 and R <= 512


def uses_tcgen05(dtype: torch.dtype, R: int, dr: int, block_size: int, cuda: bool) -> bool:
    """bf16 on a GPU with latent and rope widths that are whole 128-byte swizzle panels (R and R + dr multiples of 64,
    R + dr <= 576) and pages of whole 32-key tiles: the tcgen05 kernel (csrc/attention/latent_attention_t5.cu)."""
    if not (cuda and dtype == torch.bfloat16 and native.has_symbol("llmctl_latent_attention_t5")):
        return False
    return bool(native.lib().llmctl_latent_attention_t5_ok(int(R), int(dr), int(block_size)))


def tcgen05_status(clear: bool = True) -> int:
    """0 unless a bounded wait of the tcgen05 kernel ran out since the last clearing call (synchronises the device)."""
    return int(native.lib().llmctl_latent_attention_t5_status(int(clear)))


def rows_per_tile(dtype: torch.dtype, R: int, dr: int, cuda: bool, rows_wanted: int = ROWS_PER_TILE_WIDE) -> int:
    """Query rows per attention tile for these sizes: 32 where the tensor-core kernel runs, its shared memory
    ((rows + 64 keys) x (R + dr + 8) bf16 + score and probability tiles) fits and a tile has more than 16 rows to fill
    (``rows_wanted``: the tokens of a prompt portion, or the heads of a decoding token), else 16."""
    wide = ROWS_PER_TILE_WIDE
    smem = (wide + 64) * (R + dr + 8) * 2 + wide * (68 * 4 + 72 * 2 + 16)
    ok = cuda and rows_wanted > ROWS_PER_TILE and uses_tensor_cores(dtype, R, dr) and smem <= 227 * 1024
    return wide if ok else ROWS_PER_TILE


def latent_kv_write(d: torch.Tensor, Q: int, R: int, dr: int, wq: torch.Tensor, wkv: Optional[torch.Tensor],
                    cache: Optional[torch.Tensor], slots: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor,
                    mult: float, eps: float) -> torch.Tensor:
    """d: [T, Q + R + dr] = raw [query latent | key/value latent | key rope part] (R = dr = 0 for a layer without a
    cache of its own).  Returns the normed query latent [T, Q]; writes ``[norm(c) * wkv | rotate(kr)]`` into
    ``cache`` ([blocks, block_size, R + dr]) at ``slots`` (int64 [T], negative = skip)."""
    T = d.shape[0]
    if d.is_cuda:
        assert d.stride(1) == 1
        cq = torch.empty(T, Q, dtype=d.dtype, device=d.device)
        native.call("llmctl_latent_kv_write", d.data_ptr(), d.stride(0), Q, R, dr, wq.data_ptr(), native.ptr(wkv), cq.data_ptr(),
                    native.ptr(cache), slots.data_ptr(), positions.data_ptr(), freq.data_ptr(), float(mult), float(eps), T,
                    _is32(d), native.stream_ptr())
        return cq
    f = d.float()

    def norm(v, w):
        return v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    cq = norm(f[:, :Q], wq).to(d.dtype)
    if R:
        row = torch.cat([norm(f[:, Q:Q + R], wkv), rotate_interleaved(f[:, Q + R:Q + R + dr], positions, freq, mult)], dim=-1)
        ok = slots >= 0
        cache.view(-1, R + dr)[slots[ok]] = row[ok].to(cache.dtype)
    return cq


def latent_attention(ql: torch.Tensor, q: torch.Tensor, dn: int, cache: torch.Tensor, block_tables: torch.Tensor,
                     tiles: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, mult: float, scale: float,
                     heads_per_tile: int, max_context: int, splits: int = 1, tensor_cores: bool = True,
                     rows: int = ROWS_PER_TILE, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """ql: [T, H, R] absorbed queries (any token / head strides; fp32, or bf16 where ``uses_tensor_cores``); q: [T, H * (dn + dr)] raw queries (the rope part of each head is rotated
    here); tiles: int32 [n, 4] = (first token row, tokens, block-table row, 0) with tokens * heads_per_tile <=
    ``rows`` (16, or 32 where ``rows_per_tile`` says so), all tokens of a tile in one sequence with growing positions.  Returns [T, H, R] in q's type:
    softmax(scale * (ql . c + rot(qr) . kr)) c over cache positions 0..position of each token.  ``sinks``: fp32 [H] or None;
    ``exp(sinks[h])`` (not scaled) joins the softmax denominator of head h: a key without a value."""
    T, H, R = ql.shape
    D = cache.shape[-1]
    dr = D - R
    block_size = cache.shape[1]
    if q.is_cuda:
        assert ql.stride(2) == 1 and q.stride(1) == 1 and cache.is_contiguous()
        assert ql.dtype == torch.float32 or (tensor_cores and (uses_tensor_cores(q.dtype, R, dr) or rows == ROWS_PER_TILE_TCGEN05))
        out = torch.empty(T, H, R, dtype=q.dtype, device=q.device)
        splits = max(1, int(splits))
        per = (max_context + splits - 1) // splits
        per = max(64, (per + 63) // 64 * 64)
        partial = torch.empty(T * H * splits * (R + 2), dtype=torch.float32, device=q.device) if splits > 1 else None
        if rows == ROWS_PER_TILE_TCGEN05:
            qfull = torch.empty(T, H, D, dtype=torch.bfloat16, device=q.device)
            native.call("llmctl_latent_attention_t5", ql.data_ptr(), int(ql.dtype == torch.bfloat16), ql.stride(0), ql.stride(1),
                        q.data_ptr(), q.stride(0), dn, cache.data_ptr(), cache.shape[0] * block_size, block_tables.data_ptr(),
                        block_tables.shape[1], block_size, tiles.data_ptr(), tiles.shape[0], T, positions.data_ptr(),
                        freq.data_ptr(), float(mult), float(scale), H, R, dr, heads_per_tile, splits, per, qfull.data_ptr(),
                        out.data_ptr(), native.ptr(partial), native.ptr(sinks), native.stream_ptr())
            return out
        native.call("llmctl_latent_attention", ql.data_ptr(), int(ql.dtype == torch.bfloat16), ql.stride(0), ql.stride(1),
                    q.data_ptr(), q.stride(0), dn, cache.data_ptr(),
                    block_tables.data_ptr(), block_tables.shape[1], block_size, tiles.data_ptr(), tiles.shape[0], T,
                    positions.data_ptr(), freq.data_ptr(), float(mult), float(scale), H, R, dr, heads_per_tile, splits, per,
                    out.data_ptr(), native.ptr(partial), _is32(q), int(tensor_cores), int(rows), native.ptr(sinks), native.stream_ptr())
        return out
    out = torch.zeros(T, H, R, dtype=torch.float32)
    rows = cache.view(-1, D).float()
    qh = q.float().view(T, H, dn + dr)
    for t0, n, seq, _ in tiles.tolist():
        bt = block_tables[seq].long()
        for t in range(t0, t0 + n):
            p = int(positions[t])
            j = torch.arange(p + 1)
            kv = rows[bt[j // block_size] * block_size + j % block_size]          # [p + 1, D]
            qr = rotate_interleaved(qh[t, :, dn:], positions[t:t + 1].expand(H), freq, mult)
            s = (ql[t].float() @ kv[:, :R].t() + qr @ kv[:, R:].t()) * scale
            if sinks is not None:
                s = torch.cat([s, sinks.float()[:, None]], dim=-1)
                out[t] = torch.softmax(s, -1)[:, :-1] @ kv[:, :R]
            else:
                out[t] = torch.softmax(s, -1) @ kv[:, :R]
    return out.to(q.dtype)
