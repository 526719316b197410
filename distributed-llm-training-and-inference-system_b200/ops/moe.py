"""Mixture-of-experts feed-forward — csrc/moe/moe.cu: routing (sigmoid or softmax scores, top-k, optional
renormalisation, optional choice correction and restriction of the choice to the best groups of experts),
device-side token permutation into per-expert segments, grouped expert GEMMs and the combine, with the routing weight
applied to the expert's input or to its output; trailing router outputs may be identity experts, which return their
input.  The experts' activation is the gated SiLU or the clamped gate.  No host synchronisation on CUDA.  CPU tensors
run a PyTorch restatement.

Reference: none — the reference has no model code."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import native
from .elementwise import _is32, gated_clamped, gated_silu

c_void_p, c_int, c_ll, c_float = native.c_void_p, native.c_int, native.c_ll, native.c_float
native.register_signature("llmctl_moe_route", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
native.register_signature("llmctl_moe_plan", [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
native.register_signature("llmctl_gemm_bf16_grouped", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_void_p, c_void_p,
                                                        c_int, c_void_p])
native.register_signature("llmctl_moe_permute", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                                  c_int, c_int, c_int, c_void_p])
native.register_signature("llmctl_grouped_gemm", [c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p, c_int, c_int,
                                                   c_int, c_void_p])
native.register_signature("llmctl_moe_combine", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                  c_void_p, c_int, c_int, c_void_p])
TILE_ROWS = 64      # row tile of the grouped GEMM (llmctl_moe_tile_rows)
TILE_ROWS_TCGEN05 = 128     # row tile of the tcgen05 GEMM's grouped mode


def uses_tcgen05(act_dtype: torch.dtype, W: int, F: int) -> bool:
    """bf16 expert GEMMs whose rows are TMA-addressable (16-byte row pitch) run on the tcgen05 GEMM's grouped mode."""
    return (act_dtype == torch.bfloat16 and W % 8 == 0 and F % 8 == 0 and native.has_symbol("llmctl_gemm_bf16_grouped"))


def route(x: torch.Tensor, w_router: torch.Tensor, top: int, w_gate: Optional[torch.Tensor] = None, softmax: bool = False,
          renormalise: bool = False, correction: Optional[torch.Tensor] = None, groups: Optional[Tuple[int, int]] = None):
    """x: fp32 [T, W].  ``softmax``: False = sigmoid scores, True = softmax over all experts, 2 = the largest raw logits
    are chosen and the weights are a softmax over the chosen logits only.  ``correction``: fp32 [E] added to the scores
    for the choice only (the weights are the plain scores).  ``groups`` = (count, keep): the experts form ``count`` equal
    groups of neighbours and only those of the ``keep`` groups with the largest best choice score can be chosen.
    Returns (ids int32 [T, top], weights fp32 [T, top], gate fp32 [T] or None, counts int32 [E])."""
    T, W = x.shape
    E = w_router.shape[0]
    n_groups, keep = (int(groups[0]), int(groups[1])) if groups else (1, 1)
    if x.is_cuda:
        ids = torch.empty(T, top, dtype=torch.int32, device=x.device)
        wts = torch.empty(T, top, dtype=torch.float32, device=x.device)
        gate = torch.empty(T, dtype=torch.float32, device=x.device) if w_gate is not None else None
        counts = torch.empty(E, dtype=torch.int32, device=x.device)
        native.call("llmctl_moe_route", x.data_ptr(), w_router.data_ptr(), native.ptr(w_gate), _is32(w_router), T, W, E, top,
                    int(softmax), int(renormalise), native.ptr(correction), n_groups, keep, ids.data_ptr(), wts.data_ptr(),
                    native.ptr(gate), counts.data_ptr(), native.stream_ptr())
        return ids, wts, gate, counts
    z = x @ w_router.float().t()
    s = z if int(softmax) == 2 else torch.softmax(z, -1) if softmax else torch.sigmoid(z)
    c = s if correction is None else s + correction.float()
    if n_groups > 1 and keep < n_groups:
        best = c.view(T, n_groups, E // n_groups).max(-1).values
        kept = torch.zeros(T, n_groups, dtype=torch.bool).scatter_(1, torch.topk(best, keep, dim=-1).indices, True)
        c = c.masked_fill(~kept.repeat_interleave(E // n_groups, dim=1), float("-inf"))
    ids = torch.topk(c, top, dim=-1).indices
    wts = torch.gather(s, 1, ids)
    if int(softmax) == 2:
        wts = torch.softmax(wts, -1)
    elif renormalise:
        wts = wts / (wts.sum(-1, keepdim=True) + 1e-20)
    gate = torch.sigmoid(x @ w_gate.float().reshape(-1)) if w_gate is not None else None
    return ids.to(torch.int32), wts, gate, torch.bincount(ids.reshape(-1), minlength=E).to(torch.int32)


def moe_ffn(x: torch.Tensor, act_dtype: torch.dtype, w_router: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
            top: int, *, scale_input: bool, shared_out: Optional[torch.Tensor] = None, w_shared_gate: Optional[torch.Tensor] = None,
            softmax: bool = False, renormalise: bool = False, correction: Optional[torch.Tensor] = None,
            groups: Optional[Tuple[int, int]] = None, clamp: Optional[Tuple[float, float]] = None) -> torch.Tensor:
    """x: fp32 [T, W] stream; w_gate_up: [E, 2F, W] (gate rows first); w_down: [E, W, F]; ``shared_out``: [T, W] output
    of a shared expert that runs for every token, multiplied by sigmoid(w_shared_gate . x) when that is given.
    Returns fp32 [T, W] = sum over the chosen experts (+ shared).  ``scale_input``: the routing weight multiplies the
    expert's input (expert(w x)); otherwise its output (w expert(x)).  The router may have more rows than there are
    experts with weights: the trailing ones are identity experts (output = weight * x; needs ``scale_input`` False).
    ``correction`` / ``groups``: see ``route``.  ``clamp`` = (limit, alpha): the experts' activation is the clamped gate
    (``elementwise.gated_clamped``) instead of the gated SiLU."""
    T, W = x.shape
    E, F2, _ = w_gate_up.shape
    identity = w_router.shape[0] - E
    assert identity >= 0 and not (identity and scale_input)

    def activate(gu):
        return gated_clamped(gu, clamp[0], clamp[1]) if clamp else gated_silu(gu)
    ids, wts, gate, counts = route(x, w_router, top, w_shared_gate, softmax, renormalise, correction, groups)
    if x.is_cuda:
        is32 = int(act_dtype == torch.float32)
        pairs = T * top
        F_ = F2 // 2
        tc5 = uses_tcgen05(act_dtype, W, F_) and w_gate_up.dtype == torch.bfloat16 and w_gate_up.is_contiguous() and w_down.is_contiguous()
        rows = TILE_ROWS_TCGEN05 if tc5 else TILE_ROWS
        max_tiles = (pairs + rows - 1) // rows + min(E, pairs)      # every expert's segment is padded to whole tiles
        meta = torch.empty(2 * E + 2 + max_tiles, dtype=torch.int32, device=x.device)
        pair_row = torch.empty(pairs, dtype=torch.int32, device=x.device)
        xs = torch.empty(max_tiles * rows, W, dtype=act_dtype, device=x.device)
        st = native.stream_ptr()
        native.call("llmctl_moe_plan", counts.data_ptr(), E, meta.data_ptr(), max_tiles, rows, st)
        native.call("llmctl_moe_permute", x.data_ptr(), W, ids.data_ptr(), wts.data_ptr(), int(scale_input), meta.data_ptr(), E,
                    pair_row.data_ptr(), xs.data_ptr(), is32, T, top, st)
        gu = torch.empty(max_tiles * rows, F2, dtype=act_dtype, device=x.device)
        eo = torch.empty(max_tiles * rows, W, dtype=act_dtype, device=x.device)
        if tc5:
            tile_expert, num_tiles = meta[2 * E + 2:], meta[2 * E:]
            native.call("llmctl_gemm_bf16_grouped", xs.data_ptr(), w_gate_up.data_ptr(), gu.data_ptr(), max_tiles, F2, W, W, F2,
                        tile_expert.data_ptr(), num_tiles.data_ptr(), E, st)
            act = activate(gu)
            native.call("llmctl_gemm_bf16_grouped", act.data_ptr(), w_down.data_ptr(), eo.data_ptr(), max_tiles, W, F_, F_, W,
                        tile_expert.data_ptr(), num_tiles.data_ptr(), E, st)
        else:
            native.call("llmctl_grouped_gemm", xs.data_ptr(), W, w_gate_up.data_ptr(), gu.data_ptr(), F2, F2, W, meta.data_ptr(), E,
                        max_tiles, is32, st)
            act = activate(gu)
            native.call("llmctl_grouped_gemm", act.data_ptr(), F_, w_down.data_ptr(), eo.data_ptr(), W, W, F_, meta.data_ptr(),
                        E, max_tiles, is32, st)
        y = torch.empty(T, W, dtype=torch.float32, device=x.device)
        native.call("llmctl_moe_combine", eo.data_ptr(), W, pair_row.data_ptr(), wts.data_ptr(), top, int(not scale_input),
                    native.ptr(shared_out), native.ptr(gate), x.data_ptr() if identity else None, y.data_ptr(), T, is32, st)
        return y
    y = torch.zeros(T, W, dtype=torch.float32)
    for k in range(top):
        for e in range(E + identity):
            sel = (ids[:, k] == e).nonzero().reshape(-1)
            if sel.numel() == 0:
                continue
            w = wts[sel, k].unsqueeze(-1)
            if e >= E:
                y[sel] += w * x[sel]
                continue
            xin = (x[sel] * w if scale_input else x[sel]).to(act_dtype)
            h = activate(F.linear(xin, w_gate_up[e]))
            o = F.linear(h, w_down[e]).float()
            y[sel] += o if scale_input else w * o
    if shared_out is not None:
        y += shared_out.float() * (gate.unsqueeze(-1) if gate is not None else 1.0)
    return y
