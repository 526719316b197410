"""Ragged batch of one engine step: portions of prompts next to single decoded tokens, over the paged cache.

The host builds the whole description (tokens, positions, cache slots, block tables, attention query tiles, rows
whose logits are wanted) in one pinned int32 staging buffer; one copy takes it to the device.  Models that declare
``ragged = True`` consume it in ``forward_ragged`` (``models/nafazen.py``).

Reference: the reference right-pads a batch and recomputes whole sequences (reference llmctl/serve/server.py:171-204)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence as Seq, Tuple

import numpy as np
import torch

from ..ops.latent_attention import ROWS_PER_TILE, TILE_WIDTHS


@dataclass
class Portion:
    """The next ``len(tokens)`` tokens of one sequence, which already holds ``start`` tokens in the cache; ``want`` lists
    the offsets within ``tokens`` whose logits are asked for.  ``state_slot``: the sequence's slot in the per-sequence
    states of recurrent layers (-1: the model keeps none)."""
    seq_id: int
    tokens: Seq[int]
    start: int
    want: Seq[int]
    block_table: Seq[int]
    state_slot: int = -1


class RaggedBatch:
    """``pad_to = (sequences, block-table columns, context bound)`` fixes the shape of a decode-only batch: missing
    sequences become padding rows (token 0 at position 0, no cache slot, logits ignored), and ``refill`` rewrites the
    same pinned and device buffers for the next step, so that the step can be captured once and replayed as a CUDA
    graph."""

    def __init__(self, portions: List[Portion], block_size: int, device: torch.device, sm_count: int = 148,
                 pad_to: Optional[Tuple[int, int, int]] = None):
        self.block_size, self.device, self._sms, self.pad_to = block_size, device, sm_count, pad_to
        self.decode_only = all(len(p.tokens) == 1 for p in portions)
        # attention query tiles come in the widths the kernels take (16 / 32 / 128 rows); a tile of a decode-only batch
        # is one token with as many of its heads as fit
        self._tile_tokens = tuple(1 if self.decode_only else w for w in TILE_WIDTHS)
        if pad_to is not None:
            assert self.decode_only and len(portions) <= pad_to[0]
            T = B = n_out = pad_to[0]
            ntiles = (T,) * len(TILE_WIDTHS)
            max_blocks, self.max_context = pad_to[1], pad_to[2]
        else:
            T = sum(len(p.tokens) for p in portions)
            B = len(portions)
            assert T > 0
            self.max_context = max(p.start + len(p.tokens) for p in portions)
            max_blocks = max(len(p.block_table) for p in portions)
            n_out = sum(len(p.want) for p in portions)
            ntiles = tuple(sum((len(p.tokens) + w - 1) // w for p in portions) for w in self._tile_tokens)
        # int32 words: tokens(2T) | slots(2T) | out_rows(2 n_out) | positions(T) | block tables(B max_blocks) | tiles(4 n) per width
        # | block-table row of every token(T) | portions(4 B)
        sizes = [2 * T, 2 * T, 2 * n_out, T, B * max_blocks] + [4 * n for n in ntiles] + [T, 4 * B]
        offs = np.concatenate([[0], np.cumsum(sizes)])
        self._host = torch.zeros(int(offs[-1]), dtype=torch.int32, pin_memory=device.type == "cuda")
        a = self._host.numpy()
        self._h = (a[offs[0]:offs[1]].view(np.int64), a[offs[1]:offs[2]].view(np.int64), a[offs[2]:offs[3]].view(np.int64),
                   a[offs[3]:offs[4]], tuple(a[offs[5 + k]:offs[6 + k]].reshape(n, 4) for k, n in enumerate(ntiles)),
                   a[offs[4]:offs[5]].reshape(B, max_blocks), a[offs[5 + len(ntiles)]:offs[6 + len(ntiles)]],
                   a[offs[6 + len(ntiles)]:offs[7 + len(ntiles)]].reshape(B, 4))
        dev = torch.empty_like(self._host, device=device) if device.type == "cuda" else self._host
        self._dev = dev
        self.nbytes = self._host.numel() * 4
        self.num_tokens, self.num_out, self.num_tiles = T, n_out, ntiles[0]
        self.tokens = dev[offs[0]:offs[1]].view(torch.int64)
        self.slots = dev[offs[1]:offs[2]].view(torch.int64)
        self.out_rows = dev[offs[2]:offs[3]].view(torch.int64)
        self.positions = dev[offs[3]:offs[4]]
        self._tiles = {w: dev[offs[5 + k]:offs[6 + k]].view(ntiles[k], 4) for k, w in enumerate(TILE_WIDTHS)}
        self.block_tables = dev[offs[4]:offs[5]].view(B, max_blocks)
        self.seq_rows = dev[offs[5 + len(ntiles)]:offs[6 + len(ntiles)]]       # int32 [T]: row of block_tables per token
        # int32 [B, 4] = (first token row, tokens, position of the first token, state slot) per portion; row b belongs to
        # block_tables[b] and seq_rows == b (recurrent layers walk a portion's tokens from its slot's state)
        self.portions = dev[offs[6 + len(ntiles)]:offs[7 + len(ntiles)]].view(B, 4)
        self.refill(portions)

    def refill(self, portions: List[Portion]) -> None:
        """Write the description of ``portions`` into the (same) buffers and copy it to the device."""
        tokens, slots, out_rows, positions, tiles, tables, seq_rows, prows = self._h
        block_size = self.block_size
        if self.pad_to is not None:
            assert len(portions) <= self.pad_to[0] and all(len(p.tokens) == 1 for p in portions)
            tokens[:] = 0
            slots[:] = -1
            positions[:] = 0
            tables[:] = 0
            seq_rows[:] = np.arange(self.pad_to[0])
            for r in range(self.pad_to[0]):                 # padding rows too: one tile and one (ignored) logits row each
                for tl in tiles:
                    tl[r] = (r, 1, r, 0)
                out_rows[r] = r
                prows[r] = (r, 1, 0, -1)                    # a padding row keeps no state
        t = o = 0
        ti = [0] * len(tiles)
        for b, p in enumerate(portions):
            n = len(p.tokens)
            bt = np.asarray(p.block_table, dtype=np.int64)
            pos = np.arange(p.start, p.start + n)
            assert len(bt) * block_size >= p.start + n, "the sequence owns too few cache blocks for this portion"
            assert len(bt) <= tables.shape[1] and p.start + n <= max(self.max_context, 1)
            tokens[t:t + n] = np.asarray(p.tokens, dtype=np.int64)
            positions[t:t + n] = pos
            slots[t:t + n] = bt[pos // block_size] * block_size + pos % block_size
            tables[b, :len(bt)] = bt
            seq_rows[t:t + n] = b
            prows[b] = (t, n, p.start, p.state_slot)
            if self.pad_to is None:
                for w in p.want:
                    assert 0 <= w < n
                    out_rows[o] = t + w
                    o += 1
                for k, width in enumerate(self._tile_tokens):
                    for s in range(0, n, width):
                        tiles[k][ti[k]] = (t + s, min(width, n - s), b, 0)
                        ti[k] += 1
            t += n
        if self._dev is not self._host:
            self._dev.copy_(self._host, non_blocking=True)

    # ---- attention tiling -----------------------------------------------------------------------------------
    def tiles(self, rows: int = ROWS_PER_TILE) -> torch.Tensor:
        """int32 [n, 4] = (first token row, tokens, block-table row, 0) for kernels whose CTAs own ``rows`` query rows."""
        return self._tiles[rows]

    def heads_per_tile(self, heads: int, rows: int = ROWS_PER_TILE) -> int:
        """A tile holds ``rows`` (token, head) rows: ``rows`` tokens x 1 head in a batch with prompt portions, 1 token x
        up to ``rows`` heads when every sequence decodes."""
        return min(heads, rows) if self.decode_only else 1

    def attention_splits(self, heads: int, rows: int = ROWS_PER_TILE) -> int:
        """Split the keys of long contexts over CTAs when the tiles alone would leave most SMs idle."""
        hpt = self.heads_per_tile(heads, rows)
        ctas = self._tiles[rows].shape[0] * ((heads + hpt - 1) // hpt)
        return int(max(1, min(2 * self._sms // max(ctas, 1), self.max_context // 64)))
