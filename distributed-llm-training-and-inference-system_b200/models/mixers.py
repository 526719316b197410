"""Sequence mixers for ragged, paged inference batches.

``LatentAttention``: attention whose keys and values are linear images of one cached low-rank latent per token plus a
single rotated key part shared by all heads.  Queries go through their own normed latent.  Only ``[c | kr]`` is cached
(``R + dr`` numbers per token and layer instead of ``2 H d``); a layer may also read the cache of an earlier layer
(``kv_from``) and then has no key/value down-projection at all.  Per step:

    d        = h Wd^T                (one packed GEMM: query latent | key/value latent | key rope part)
    cq, cache= norm / rotate / append        (ops.latent_attention.latent_kv_write)
    q        = cq Wuq^T              [T, H, dn + dr]
    ql       = qn Uk_h               [T, H, R]   absorbed queries, fp32
    ol       = attention over the cache rows (ops.latent_attention.latent_attention)   [T, H, R]
    out      = (ol Uv_h^T) Wo^T

Optional parts of ``LatentAttention`` (fields of its spec): ``sink`` — a learned number per head whose exponential joins
the softmax denominator (a key without a value, not scaled); ``out_gate`` — the concatenated heads are multiplied element
by element with the sigmoid of one more projection of the mixer's input (packed into the down-projection GEMM).

``SoftcapWindowAttention``: grouped-query attention without rotation whose scores pass a tanh soft cap and lose a linear
distance bias with one slope per head; a sliding window that also keeps the first tokens of the sequence; a softmax with
one added to the denominator (a sink of score 0); values cached at unit RMS per head; projection biases; a sigmoid output
gate.  Every part is a field of ``SoftcapWindowAttentionSpec``.  Per step:

    p        = h Wp^T                           (one packed GEMM: q | k | v | gate)
    q, cache = bias / value norm / append       (ops.softcap_attention.window_kv_append)
    o        = attention over kept + window keys, gate      (ops.softcap_attention.softcap_window_attention)
    out      = o Wo^T + bo

``PooledWindowAttention``: grouped-query attention over a sliding window of ``window`` tokens plus one pooled key/value
(the mean of the cached keys / values) per block of ``pool`` tokens that lies wholly before the window.  Optional parts,
each a field of ``PooledWindowAttentionSpec``: projection biases, an RMS norm over the whole q and the whole k
projection, rotation of the first ``rot_dims`` numbers of every head (plain or YaRN-blended spectrum), a learned score
temperature per head, mixing of the normalised attention weights across heads by a learned [H, H] matrix, and mixing of
the layer's values with the values the first such layer computed for the same token.  Per step:

    qkv      = h Wqkv^T                         (one packed GEMM)
    q, cache = bias / norm / rotate / value mix / append     (ops.window_attention.window_qkv_write)
    pooled rows of the blocks the step completes             (ops.window_attention.window_pool_update)
    o        = attention over window + pooled rows           (ops.window_attention.pooled_window_attention)
    out      = o Wo^T

``DifferentialAttention``: grouped-query attention in which every head has two score maps (two query vectors against
two key vectors of its key/value head) over the same values; the head's output is ``a1 - lam a2`` brought to unit RMS,
times ``1 - diff`` and, optionally, a sigmoid gate per (token, head).  ``lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff`` is
one number of the layer.  Partial interleaved rotation on every query and key vector.  Per step:

    p        = h Wp^T                           (one packed GEMM: q | k | v | gate logits)
    q, cache = rotate / append                  (ops.diff_attention.rotary_kv_append)
    o        = both maps, difference, norm, gate        (ops.diff_attention.diff_attention)
    out      = o Wo^T

``GatedLinearAttention`` and ``SelectiveScan`` are recurrences: they keep no per-token cache but ONE state per sequence
in a state slot (``serve/ragged.py`` ``RaggedBatch.portions`` names each portion's slot), fp32.

``GatedLinearAttention``: per head ``S <- diag(a) S + k v^T``, ``o = S^T q`` with a decay per key channel
``a = sigmoid(z)^(1/tau)``, ``z`` from a low-rank projection with bias; heads are RMS-normed with one shared weight,
gated by ``silu`` of a projection and projected out.  Per step: one packed GEMM (q | k | v | gate | decay latent), the small
decay GEMM, ``ops.recurrent.gla_scan``, ``ops.recurrent.gla_output``, the output GEMM.

``SelectiveScan`` (Mamba): ``[x | z] = h Win^T``; ``u = silu(causal conv(x))``; ``[dt | B | C] = u Wx^T``;
``dt = softplus(dt Wdt^T + b)``; ``S <- exp(dt A) S + dt u B``, ``y = (S C + D u) silu(z)``; output GEMM.  The state of a
sequence is S and the last ``taps - 1`` inputs of the convolution.

Reference: none — the reference has no model code (reference llmctl/runtime/engine.py:119-140)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import diff_attention as dops
from ..ops import functional as ops
from ..ops import latent_attention as lops
from ..ops import recurrent as rops
from ..ops import softcap_attention as sops
from ..ops import window_attention as wops
from ..ops.elementwise import rope_frequencies, sigmoid_gate_


@dataclass
class LatentAttentionSpec:
    heads: int
    dim: int            # unrotated query/key size per head (dn)
    rot_dim: int        # rotated query/key size per head (dr)
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_scaling: Optional[Dict[str, Any]] = None
    kv_from: Optional[int] = None       # index of the layer whose cache this layer reads
    sink: bool = False                  # a learned number per head joins the softmax denominator
    out_gate: bool = False              # heads * sigmoid(Wg h) before the output projection

    @property
    def cache_width(self) -> int:
        return self.kv_rank + self.rot_dim


class LatentAttention(nn.Module):
    stateful = False

    def __init__(self, width: int, spec: LatentAttentionSpec, eps: float, dtype, device):
        super().__init__()
        s = self.spec = spec
        self.eps = eps
        own = s.kv_from is None
        kw = dict(dtype=dtype, device=device)
        self.n_down = s.q_rank + (s.kv_rank + s.rot_dim if own else 0)
        rows = self.n_down + (s.heads * s.vdim if s.out_gate else 0)
        self.w_down = nn.Parameter(torch.empty(rows, width, **kw))                      # [dq ; dkv ; gate]
        self.sink = nn.Parameter(torch.zeros(s.heads, dtype=torch.float32, device=device)) if s.sink else None
        self.q_norm = nn.Parameter(torch.ones(s.q_rank, **kw))
        self.kv_norm = nn.Parameter(torch.ones(s.kv_rank, **kw)) if own else None
        self.w_uq = nn.Parameter(torch.empty(s.heads * (s.dim + s.rot_dim), s.q_rank, **kw))
        self.w_uk = nn.Parameter(torch.empty(s.heads, s.dim, s.kv_rank, **kw))          # per head [dn, R]
        self.w_uv = nn.Parameter(torch.empty(s.heads, s.vdim, s.kv_rank, **kw))         # per head [dv, R]
        self.w_o = nn.Parameter(torch.empty(width, s.heads * s.vdim, **kw))
        f, self.rot_mult = rope_frequencies(s.rot_dim, s.rot_base, s.rot_scaling)
        self.register_buffer("rot_freq", f.to(device), persistent=False)

    def load(self, get, prefix: str) -> None:
        s = self.spec
        with torch.no_grad():
            parts = [get(prefix + "dq")] + ([get(prefix + "dkv")] if s.kv_from is None else []) + ([get(prefix + "g")] if s.out_gate else [])
            self.w_down.copy_(torch.cat(parts, dim=0))
            if s.sink:
                self.sink.copy_(get(prefix + "sink").float())
            self.q_norm.copy_(get(prefix + "dq.norm"))
            if s.kv_from is None:
                self.kv_norm.copy_(get(prefix + "dkv.norm"))
            self.w_uq.copy_(get(prefix + "uq"))
            self.w_uk.copy_(get(prefix + "uk").view(s.heads, s.dim, s.kv_rank))
            self.w_uv.copy_(get(prefix + "uv").view(s.heads, s.vdim, s.kv_rank))
            self.w_o.copy_(get(prefix + "o"))

    def forward(self, h: torch.Tensor, batch, cache: torch.Tensor) -> torch.Tensor:
        """h: [T, W] in the activation type; ``cache``: this layer's (or its source layer's) [blocks, bs, R + dr]."""
        s = self.spec
        T = h.shape[0]
        own = s.kv_from is None
        d = ops.linear(h, self.w_down)
        cq = lops.latent_kv_write(d, s.q_rank, s.kv_rank if own else 0, s.rot_dim if own else 0, self.q_norm, self.kv_norm,
                                  cache if own else None, batch.slots, batch.positions, self.rot_freq, self.rot_mult, self.eps)
        q = ops.linear(cq, self.w_uq)                                                   # [T, H * (dn + dr)]
        qn = q.view(T, s.heads, s.dim + s.rot_dim)[:, :, :s.dim].transpose(0, 1)        # [H, T, dn], a view
        # absorbed queries ql[t, h] = Uk_h^T qn[t, h]: fp32, except that the tensor-core attention kernel takes them
        # in bf16 (it multiplies in bf16 anyway); the kernel reads the [H, T, R] product through its strides
        if q.is_cuda and q.dtype == torch.bfloat16:
            if lops.uses_tensor_cores(q.dtype, s.kv_rank, s.rot_dim):
                ql = torch.bmm(qn, self.w_uk)
            else:
                ql = torch.bmm(qn, self.w_uk, out_dtype=torch.float32)
        else:
            ql = torch.bmm(qn.float(), self.w_uk.float())
        ql = ql.transpose(0, 1)
        # batches with prompt portions fill the tcgen05 kernel's 128-row tiles; a decoding token has only its heads to
        # offer, and the 16 / 32-row kernel reads the cache once for them
        if not batch.decode_only and lops.uses_tcgen05(q.dtype, s.kv_rank, s.rot_dim, cache.shape[1], q.is_cuda):
            rows = lops.ROWS_PER_TILE_TCGEN05
        else:
            rows = lops.rows_per_tile(q.dtype, s.kv_rank, s.rot_dim, q.is_cuda, s.heads if batch.decode_only else lops.ROWS_PER_TILE_WIDE)
        ol = lops.latent_attention(ql, q, s.dim, cache, batch.block_tables, batch.tiles(rows), batch.positions,
                                   self.rot_freq, self.rot_mult, s.scale, batch.heads_per_tile(s.heads, rows), batch.max_context,
                                   batch.attention_splits(s.heads, rows), rows=rows, sinks=self.sink)
        o = torch.bmm(ol.transpose(0, 1), self.w_uv.transpose(1, 2)).transpose(0, 1).reshape(T, s.heads * s.vdim)
        if s.out_gate:
            o = sigmoid_gate_(o, d[:, self.n_down:])
        return ops.linear(o, self.w_o)

    def cache_shape(self, num_blocks: int, block_size: int) -> Tuple[int, ...]:
        return (num_blocks, block_size, self.spec.cache_width)


@dataclass
class PooledWindowAttentionSpec:
    heads: int
    kv_heads: int
    dim: int            # query/key size per head
    vdim: int           # value size per head
    scale: float
    window: int = 0     # 0: every earlier token is seen, nothing is pooled
    pool: int = 0       # tokens per pooled block
    rot_dims: int = 0   # rotated numbers per head (even, <= dim); 0: no rotation
    rot_base: float = 10000.0
    rot_scaling: Optional[Dict[str, Any]] = None
    bias: bool = True
    qk_norm: bool = True            # RMS norm over the whole q / k projection, per-coordinate weights
    head_temperature: bool = True   # scores of head h are multiplied by a learned number
    talking_heads: bool = True      # normalised weights are mixed across heads by a learned [H, H] matrix
    v_mix: bool = False             # values are blended with those of the first v_mix layer

    @property
    def cache_width(self) -> int:
        return self.kv_heads * (self.dim + self.vdim)

    def rows_per_page(self, block_size: int) -> int:
        return block_size + wops.pooled_rows_per_page(block_size, self.pool if self.window else 0)


class PooledWindowAttention(nn.Module):
    TILE_TOKENS = 16        # tile width of the ragged batch this mixer asks for (serve/ragged.py)

    def __init__(self, width: int, spec: PooledWindowAttentionSpec, eps: float, dtype, device):
        super().__init__()
        s = self.spec = spec
        if s.heads % s.kv_heads or s.rot_dims % 2 or s.rot_dims > s.dim or (s.window and s.pool < 1):
            raise ValueError(f"inconsistent attention sizes: {s}")
        self.eps = eps
        kw = dict(dtype=dtype, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        nq, nk, nv = s.heads * s.dim, s.kv_heads * s.dim, s.kv_heads * s.vdim
        self.w_qkv = nn.Parameter(torch.empty(nq + nk + nv, width, **kw))               # [q ; k ; v]
        self.b_qkv = nn.Parameter(torch.zeros(nq + nk + nv, **kw)) if s.bias else None
        self.q_norm = nn.Parameter(torch.ones(nq, **f32)) if s.qk_norm else None
        self.k_norm = nn.Parameter(torch.ones(nk, **f32)) if s.qk_norm else None
        self.temp = nn.Parameter(torch.ones(s.heads, **f32)) if s.head_temperature else None
        self.talk = nn.Parameter(torch.eye(s.heads, **f32)) if s.talking_heads else None
        self.vmix = nn.Parameter(torch.zeros(1, **f32)) if s.v_mix else None
        self.w_o = nn.Parameter(torch.empty(width, s.heads * s.vdim, **kw))
        if s.rot_dims:
            f, self.rot_mult = rope_frequencies(s.rot_dims, s.rot_base, s.rot_scaling)
        else:
            f, self.rot_mult = torch.zeros(1), 1.0
        self.register_buffer("rot_freq", f.to(device), persistent=False)

    def load(self, get, prefix: str) -> None:
        """Checkpoint names under ``prefix``: q, k, v (+ ``.b`` biases, ``q.norm`` / ``k.norm``), temp, talk, vmix, o."""
        s = self.spec
        with torch.no_grad():
            self.w_qkv.copy_(torch.cat([get(prefix + "q"), get(prefix + "k"), get(prefix + "v")], dim=0))
            if s.bias:
                self.b_qkv.copy_(torch.cat([get(prefix + "q.b"), get(prefix + "k.b"), get(prefix + "v.b")], dim=0))
            if s.qk_norm:
                self.q_norm.copy_(get(prefix + "q.norm").float())
                self.k_norm.copy_(get(prefix + "k.norm").float())
            if s.head_temperature:
                self.temp.copy_(get(prefix + "temp").float())
            if s.talking_heads:
                self.talk.copy_(get(prefix + "talk").float())
            if s.v_mix:
                self.vmix.copy_(get(prefix + "vmix").float().reshape(1))
            self.w_o.copy_(get(prefix + "o"))

    def forward(self, h: torch.Tensor, batch, cache: torch.Tensor, v_first: Optional[torch.Tensor] = None):
        """h: [T, W] in the activation type; ``cache``: this layer's [pages, bs + PS, G (d + e)].  ``v_first``: the values
        of the first v_mix layer for the step's tokens (None in that layer itself, which then returns them).  Returns
        (output [T, W], v_first)."""
        s = self.spec
        T = h.shape[0]
        bs = batch.block_size
        qkv = ops.linear(h, self.w_qkv)
        v_mode = 0
        if s.v_mix:
            v_mode = 2 if v_first is not None else 1
            if v_first is None:
                v_first = torch.empty(T, s.kv_heads * s.vdim, dtype=h.dtype, device=h.device)
        q = wops.window_qkv_write(qkv, self.b_qkv, self.q_norm, self.k_norm, s.heads, s.kv_heads, s.dim, s.vdim, s.rot_dims,
                                  self.rot_freq, self.rot_mult, self.eps, batch.positions, batch.slots, cache, bs,
                                  v_first if v_mode else None, v_mode, self.vmix)
        pool = s.pool if s.window else 0
        wops.window_pool_update(cache, batch.positions, batch.slots, batch.seq_rows, batch.block_tables, bs, pool)
        o = wops.pooled_window_attention(q, cache, batch.block_tables, batch.tiles(self.TILE_TOKENS),
                                         1 if batch.decode_only else self.TILE_TOKENS, batch.positions, self.temp, self.talk,
                                         s.scale, s.heads, s.kv_heads, s.dim, s.vdim, s.window, pool, bs, h.dtype,
                                         max_context=batch.max_context)
        return ops.linear(o, self.w_o), v_first


@dataclass
class SoftcapWindowAttentionSpec:
    heads: int
    kv_heads: int
    dim: int            # query/key size per head
    vdim: int           # value size per head
    scale: float
    softcap: float = 0.0        # scores become softcap * tanh(score / softcap); 0: no cap
    window: int = 0             # position i sees j <= i with i - j < window; 0: every earlier token
    keep_first: int = 0         # ... or j < keep_first
    distance_bias: bool = True  # slope_h (i - j) is taken off the score, slope_h = 2^(-8 (h + 1) / heads)
    sink_one: bool = True       # one is added to the softmax denominator (a sink of score 0 without a value)
    value_norm: bool = True     # every value head is cached at unit RMS (no weight)
    bias: bool = True           # q, k, v and output projections have biases
    out_gate: bool = True       # heads * sigmoid(Wg h) before the output projection

    @property
    def cache_width(self) -> int:
        return self.kv_heads * (self.dim + self.vdim)


class SoftcapWindowAttention(nn.Module):
    stateful = False

    def __init__(self, width: int, spec: SoftcapWindowAttentionSpec, eps: float, dtype, device):
        super().__init__()
        s = self.spec = spec
        if s.heads % s.kv_heads or s.window < 0 or s.keep_first < 0 or s.softcap < 0:
            raise ValueError(f"inconsistent attention sizes: {s}")
        self.eps = eps
        kw = dict(dtype=dtype, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        self.nq, self.nk, self.nv = s.heads * s.dim, s.kv_heads * s.dim, s.kv_heads * s.vdim
        self.n_qkv = self.nq + self.nk + self.nv
        self.w_in = nn.Parameter(torch.empty(self.n_qkv + (s.heads * s.vdim if s.out_gate else 0), width, **kw))     # [q ; k ; v ; gate]
        self.b_in = nn.Parameter(torch.zeros(self.n_qkv, **f32)) if s.bias else None
        self.w_o = nn.Parameter(torch.empty(width, s.heads * s.vdim, **kw))
        self.b_o = nn.Parameter(torch.zeros(width, **f32)) if s.bias else None
        self.register_buffer("slopes", sops.distance_slopes(s.heads).to(device) if s.distance_bias else None, persistent=False)
        self.register_buffer("sinks", torch.zeros(s.heads, **f32) if s.sink_one else None, persistent=False)

    def load(self, get, prefix: str) -> None:
        """Checkpoint names under ``prefix``: q, k, v (+ ``.b`` biases), g, o (+ ``o.b``)."""
        s = self.spec
        with torch.no_grad():
            parts = [get(prefix + "q"), get(prefix + "k"), get(prefix + "v")] + ([get(prefix + "g")] if s.out_gate else [])
            self.w_in.copy_(torch.cat(parts, dim=0))
            self.w_o.copy_(get(prefix + "o"))
            if s.bias:
                self.b_in.copy_(torch.cat([get(prefix + "q.b"), get(prefix + "k.b"), get(prefix + "v.b")], dim=0).float())
                self.b_o.copy_(get(prefix + "o.b").float())

    def cache_shape(self, num_blocks: int, block_size: int) -> Tuple[int, ...]:
        return (num_blocks, block_size, self.spec.cache_width)

    def forward(self, h: torch.Tensor, batch, cache: torch.Tensor) -> torch.Tensor:
        """h: [T, W] in the activation type; ``cache``: this layer's [pages, bs, G (d + e)]."""
        s = self.spec
        p = ops.linear(h, self.w_in)
        q = sops.window_kv_append(p, self.b_in, s.heads, s.kv_heads, s.dim, s.vdim, s.value_norm, self.eps, batch.slots, cache)
        gate = p[:, self.n_qkv:] if s.out_gate else None
        # prompt portions: tiles of 128 tokens on the tensor-core kernel, of 16 on the FMA kernel; decoded tokens: one each
        width = sops.tile_width(cache.dtype, s.heads, s.kv_heads, s.dim, s.vdim, q.is_cuda, batch.decode_only)
        o = sops.softcap_window_attention(q, cache, batch.block_tables, batch.tiles(width), 1 if batch.decode_only else width,
                                          batch.positions, gate, self.slopes, self.sinks, s.scale, s.softcap, s.window, s.keep_first,
                                          s.heads, s.kv_heads, s.dim, s.vdim, batch.block_size, h.dtype, max_context=batch.max_context)
        y = ops.linear(o, self.w_o)
        return y if self.b_o is None else torch.add(y, self.b_o)        # fp32 sum: the residual update takes either type


@dataclass
class DifferentialAttentionSpec:
    heads: int
    kv_heads: int
    dim: int            # size of each of the two query / key vectors of a head
    vdim: int           # value size per head
    scale: float
    diff: float         # the constant in lam; the output is multiplied by 1 - diff
    rot_dims: int = 0   # rotated numbers per query / key vector (even, <= dim); 0: no rotation
    rot_base: float = 10000.0
    rot_scaling: Optional[Dict[str, Any]] = None
    head_gate: bool = True      # sigmoid gate per (token, head) from a projection of the mixer's input

    @property
    def cache_width(self) -> int:
        return self.kv_heads * (2 * self.dim + self.vdim)


class DifferentialAttention(nn.Module):
    TILE_TOKENS = dops.TILE_TOKENS      # tile width of the ragged batch this mixer asks for (serve/ragged.py)
    stateful = False

    def __init__(self, width: int, spec: DifferentialAttentionSpec, eps: float, dtype, device):
        super().__init__()
        s = self.spec = spec
        if s.heads % s.kv_heads or s.rot_dims % 2 or s.rot_dims > s.dim:
            raise ValueError(f"inconsistent attention sizes: {s}")
        self.eps = eps
        kw = dict(dtype=dtype, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        self.nq, self.nk, self.nv = s.heads * 2 * s.dim, s.kv_heads * 2 * s.dim, s.kv_heads * s.vdim
        self.w_in = nn.Parameter(torch.empty(self.nq + self.nk + self.nv + (s.heads if s.head_gate else 0), width, **kw))   # [q ; k ; v ; g]
        self.lam_q = nn.Parameter(torch.zeros(2, s.dim, **f32))
        self.lam_k = nn.Parameter(torch.zeros(2, s.dim, **f32))
        self.w_o = nn.Parameter(torch.empty(width, s.heads * s.vdim, **kw))
        if s.rot_dims:
            f, self.rot_mult = rope_frequencies(s.rot_dims, s.rot_base, s.rot_scaling)
        else:
            f, self.rot_mult = torch.zeros(1), 1.0
        self.register_buffer("rot_freq", f.to(device), persistent=False)
        self._lam: Optional[float] = None

    def load(self, get, prefix: str) -> None:
        """Checkpoint names under ``prefix``: q, k, v, g ([heads, width]), lq1, lk1, lq2, lk2, o."""
        s = self.spec
        with torch.no_grad():
            parts = [get(prefix + "q"), get(prefix + "k"), get(prefix + "v")] + ([get(prefix + "g")] if s.head_gate else [])
            self.w_in.copy_(torch.cat(parts, dim=0))
            self.lam_q.copy_(torch.stack([get(prefix + "lq1").float(), get(prefix + "lq2").float()]))
            self.lam_k.copy_(torch.stack([get(prefix + "lk1").float(), get(prefix + "lk2").float()]))
            self.w_o.copy_(get(prefix + "o"))
        self._lam = None

    @property
    def lam(self) -> float:
        """``exp(lq1 . lk1) - exp(lq2 . lk2) + diff``, evaluated once in fp32."""
        if self._lam is None:
            dots = (self.lam_q.detach().float() * self.lam_k.detach().float()).sum(-1).cpu()
            e = torch.exp(dots)
            self._lam = float(e[0] - e[1] + torch.tensor(self.spec.diff, dtype=torch.float32))
        return self._lam

    def cache_shape(self, num_blocks: int, block_size: int) -> Tuple[int, ...]:
        return (num_blocks, block_size, self.spec.cache_width)

    def forward(self, h: torch.Tensor, batch, cache: torch.Tensor) -> torch.Tensor:
        """h: [T, W] in the activation type; ``cache``: this layer run's [pages, bs, G (2 d + e)]."""
        s = self.spec
        p = ops.linear(h, self.w_in)
        q = dops.rotary_kv_append(p, 2 * s.heads, 2 * s.kv_heads, s.dim, self.nv, s.rot_dims, self.rot_freq, self.rot_mult,
                                  batch.positions, batch.slots, cache)
        gate = p[:, self.nq + self.nk + self.nv:] if s.head_gate else None
        # prompt portions: tiles of 128 tokens on the tensor-core kernel, of 16 on the FMA kernel; decoded tokens: one each
        width = dops.tile_width(cache.dtype, s.heads, s.kv_heads, s.dim, s.vdim, q.is_cuda, batch.decode_only)
        o = dops.diff_attention(q, cache, batch.block_tables, batch.tiles(width), 1 if batch.decode_only else width,
                                batch.positions, gate, s.scale, self.lam, 1.0 - s.diff, self.eps, s.heads, s.kv_heads, s.dim, s.vdim,
                                batch.block_size, h.dtype, max_context=batch.max_context)
        return ops.linear(o, self.w_o)


@dataclass
class GatedLinearAttentionSpec:
    heads: int
    dim: int            # query / key size per head
    vdim: int           # value size per head
    tau: float          # the decay is sigmoid(z)^(1/tau)
    decay_rank: int     # inner size of the low-rank decay projection


class GatedLinearAttention(nn.Module):
    stateful = True

    def __init__(self, width: int, spec: GatedLinearAttentionSpec, eps: float, dtype, device):
        super().__init__()
        s = self.spec = spec
        self.eps = eps
        kw = dict(dtype=dtype, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        self.nk, self.nv = s.heads * s.dim, s.heads * s.vdim
        self.w_in = nn.Parameter(torch.empty(2 * self.nk + 2 * self.nv + s.decay_rank, width, **kw))     # [q ; k ; v ; g ; a1]
        self.w_a2 = nn.Parameter(torch.empty(self.nk, s.decay_rank, **kw))
        self.b_a2 = nn.Parameter(torch.zeros(self.nk, **f32))
        self.norm = nn.Parameter(torch.ones(s.vdim, **f32))
        self.w_o = nn.Parameter(torch.empty(width, self.nv, **kw))

    def load(self, get, prefix: str) -> None:
        """Checkpoint names under ``prefix``: q, k, v, g, a1, a2 (+ ``a2.b``), norm, o."""
        with torch.no_grad():
            self.w_in.copy_(torch.cat([get(prefix + n) for n in ("q", "k", "v", "g", "a1")], dim=0))
            self.w_a2.copy_(get(prefix + "a2"))
            self.b_a2.copy_(get(prefix + "a2.b").float())
            self.norm.copy_(get(prefix + "norm").float())
            self.w_o.copy_(get(prefix + "o"))

    def state_shapes(self) -> Tuple[Tuple[int, ...], ...]:
        s = self.spec
        return ((s.heads, s.dim, s.vdim),)

    def forward(self, h: torch.Tensor, batch, state) -> torch.Tensor:
        """h: [T, W] in the activation type; ``state``: (this layer run's [slots, H, d, e] fp32,)."""
        s = self.spec
        nk, nv = self.nk, self.nv
        p = ops.linear(h, self.w_in)
        z = ops.linear(p[:, 2 * nk + 2 * nv:], self.w_a2)
        o = rops.gla_scan(p[:, :nk], p[:, nk:2 * nk], p[:, 2 * nk:2 * nk + nv], z, self.b_a2, batch.portions, state[0], s.heads, s.dim,
                          s.vdim, s.dim ** -0.5, s.tau)
        y = rops.gla_output(o, self.norm, p[:, 2 * nk + nv:2 * nk + 2 * nv], s.heads, s.vdim, self.eps, h.dtype)
        return ops.linear(y, self.w_o)


@dataclass
class SelectiveScanSpec:
    inner: int          # channels
    state: int          # state numbers per channel (N)
    dt_rank: int
    conv: int           # taps of the causal convolution


class SelectiveScan(nn.Module):
    stateful = True

    def __init__(self, width: int, spec: SelectiveScanSpec, dtype, device):
        super().__init__()
        s = self.spec = spec
        if s.conv < 1:
            raise ValueError("the convolution needs at least one tap")
        kw = dict(dtype=dtype, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        self.w_in = nn.Parameter(torch.empty(2 * s.inner, width, **kw))                 # [x ; z]
        self.conv_w = nn.Parameter(torch.empty(s.inner, s.conv, **f32))
        self.conv_b = nn.Parameter(torch.zeros(s.inner, **f32))
        self.w_x = nn.Parameter(torch.empty(s.dt_rank + 2 * s.state, s.inner, **kw))    # [dt ; B ; C]
        self.w_dt = nn.Parameter(torch.empty(s.inner, s.dt_rank, **kw))
        self.dt_bias = nn.Parameter(torch.zeros(s.inner, **f32))
        self.A = nn.Parameter(-torch.ones(s.inner, s.state, **f32))                    # -exp(A_log), fp32
        self.D = nn.Parameter(torch.ones(s.inner, **f32))
        self.w_o = nn.Parameter(torch.empty(width, s.inner, **kw))

    def load(self, get, prefix: str) -> None:
        """Checkpoint names under ``prefix``: in, conv (+ ``conv.b``), x, dt (+ ``dt.b``), A_log, D, o."""
        with torch.no_grad():
            self.w_in.copy_(get(prefix + "in"))
            self.conv_w.copy_(get(prefix + "conv").float())
            self.conv_b.copy_(get(prefix + "conv.b").float())
            self.w_x.copy_(get(prefix + "x"))
            self.w_dt.copy_(get(prefix + "dt"))
            self.dt_bias.copy_(get(prefix + "dt.b").float())
            self.A.copy_(-torch.exp(get(prefix + "A_log").float()))
            self.D.copy_(get(prefix + "D").float())
            self.w_o.copy_(get(prefix + "o"))

    def state_shapes(self) -> Tuple[Tuple[int, ...], ...]:
        s = self.spec
        return ((s.inner, s.state), (max(s.conv - 1, 0), s.inner))

    def forward(self, h: torch.Tensor, batch, state) -> torch.Tensor:
        """h: [T, W] in the activation type; ``state``: this layer run's ([slots, C, N], [slots, taps - 1, C]) fp32."""
        s = self.spec
        C, R, N = s.inner, s.dt_rank, s.state
        xz = ops.linear(h, self.w_in)
        x, z = xz[:, :C], xz[:, C:]
        u = rops.causal_conv_silu(x, self.conv_w, self.conv_b, batch.portions, batch.seq_rows, state[1])
        bc = ops.linear(u, self.w_x)
        dtp = ops.linear(bc[:, :R], self.w_dt)
        y = rops.selective_scan(u, bc, R, R + N, dtp, self.dt_bias, self.A, self.D, z, x, batch.portions, state[0], state[1])
        return ops.linear(y, self.w_o)
