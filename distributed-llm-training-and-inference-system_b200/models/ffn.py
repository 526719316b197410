"""Feed-forward layers for inference batches: two-matrix MLPs with the xIELU or the squared-ReLU activation, a gated
MLP with the tanh form of GELU on the gate, and a
routed mixture of gated experts (sigmoid, softmax or chosen-logit softmax weights) with an optional shared expert.

Reference: none — the reference has no model code (reference llmctl/runtime/engine.py:119-140)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from ..ops import elementwise as eops
from ..ops import functional as ops
from ..ops import moe as mops


class XieluMLP(nn.Module):
    """``Wdown xielu(Wup h)``; the activation's two coefficients are functions of two learned numbers."""

    def __init__(self, width: int, ff: int, dtype, device):
        super().__init__()
        self.up = nn.Parameter(torch.empty(ff, width, dtype=dtype, device=device))
        self.down = nn.Parameter(torch.empty(width, ff, dtype=dtype, device=device))
        self.act = nn.Parameter(torch.zeros(2, dtype=dtype, device=device))
        self._coef = None

    def load(self, get, prefix: str) -> None:
        with torch.no_grad():
            self.up.copy_(get(prefix + "up"))
            self.down.copy_(get(prefix + "down"))
            self.act.copy_(get(prefix + "act"))
        self._coef = None

    def forward(self, h: torch.Tensor, x32: torch.Tensor) -> torch.Tensor:
        if self._coef is None:
            self._coef = eops.xielu_coefficients(self.act)
        return ops.linear(eops.xielu(ops.linear(h, self.up), *self._coef), self.down)


class SquaredReluMLP(nn.Module):
    """``Wdown relu(Wup h)^2``."""

    def __init__(self, width: int, ff: int, dtype, device):
        super().__init__()
        self.up = nn.Parameter(torch.empty(ff, width, dtype=dtype, device=device))
        self.down = nn.Parameter(torch.empty(width, ff, dtype=dtype, device=device))

    def load(self, get, prefix: str) -> None:
        with torch.no_grad():
            self.up.copy_(get(prefix + "up"))
            self.down.copy_(get(prefix + "down"))

    def forward(self, h: torch.Tensor, x32: torch.Tensor) -> torch.Tensor:
        return ops.linear(eops.relu_squared(ops.linear(h, self.up)), self.down)


class GatedGeluMLP(nn.Module):
    """``Wdown (gelu_tanh(Wgate h) * (Wup h))``; gate and up run as one packed GEMM."""

    def __init__(self, width: int, ff: int, dtype, device):
        super().__init__()
        self.gate_up = nn.Parameter(torch.empty(2 * ff, width, dtype=dtype, device=device))       # [gate ; up]
        self.down = nn.Parameter(torch.empty(width, ff, dtype=dtype, device=device))

    def load(self, get, prefix: str) -> None:
        with torch.no_grad():
            self.gate_up.copy_(torch.cat([get(prefix + "gate"), get(prefix + "up")], dim=0))
            self.down.copy_(get(prefix + "down"))

    def forward(self, h: torch.Tensor, x32: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.linear(eops.gated_gelu_tanh(ops.linear(h, self.gate_up)), self.down)


class GatedExpertMoE(nn.Module):
    """``top`` of ``experts`` gated-SiLU experts per token.  Scores are sigmoids of fp32 router logits (or a softmax over
    all experts, ``softmax_scores`` True; or, ``softmax_scores`` 2, the largest logits are chosen and weighted by a
    softmax over the chosen logits only), optionally renormalised over the chosen ones; the score multiplies the expert's input
    (``scale_input``) or its output.  A shared expert of its own size runs for every token, times sigmoid(wg . h)
    when ``shared_gate``.  Optional parts: ``identity`` further router outputs behind the experts stand for identity
    experts (output = input, no weights); ``correction``: a learned vector added to the scores for the choice only;
    ``groups`` = (count, keep): the router outputs form ``count`` equal groups of neighbours and only the ``keep`` groups
    with the largest best choice score can be chosen from; ``clamp`` = (limit, alpha): the experts compute
    ``g sigmoid(alpha g) (u + 1)`` on ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)`` instead of the gated
    SiLU."""

    def __init__(self, width: int, experts: int, top: int, ff: int, shared_ff: Optional[int], dtype, device, *,
                 scale_input: bool = True, softmax_scores: bool = False, renormalise: bool = False, shared_gate: bool = True,
                 identity: int = 0, correction: bool = False, groups: Optional[Tuple[int, int]] = None,
                 clamp: Optional[Tuple[float, float]] = None):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.top, self.scale_input, self.softmax_scores, self.renormalise = top, scale_input, softmax_scores, renormalise
        self.groups, self.clamp = groups, clamp
        if groups and ((experts + identity) % groups[0] or not 1 <= groups[1] <= groups[0] or groups[1] * ((experts + identity) // groups[0]) < top):
            raise ValueError(f"expert groups {groups} do not fit {experts} + {identity} router outputs with {top} choices")
        self.router = nn.Parameter(torch.empty(experts + identity, width, **kw))
        self.correction = nn.Parameter(torch.zeros(experts + identity, dtype=torch.float32, device=device)) if correction else None
        self.gate_up = nn.Parameter(torch.empty(experts, 2 * ff, width, **kw))
        self.down = nn.Parameter(torch.empty(experts, width, ff, **kw))
        self.shared_gate_up = nn.Parameter(torch.empty(2 * shared_ff, width, **kw)) if shared_ff else None
        self.shared_down = nn.Parameter(torch.empty(width, shared_ff, **kw)) if shared_ff else None
        self.shared_gate = nn.Parameter(torch.empty(width, **kw)) if shared_ff and shared_gate else None

    def load(self, get, prefix: str) -> None:
        E = self.gate_up.shape[0]
        with torch.no_grad():
            self.router.copy_(get(prefix + "router"))
            if self.correction is not None:
                try:
                    self.correction.copy_(get(prefix + "correction").float())
                except KeyError:            # a checkpoint without the vector chooses by the plain scores
                    self.correction.zero_()
            for e in range(E):
                self.gate_up[e].copy_(torch.cat([get(f"{prefix}e{e}.gate"), get(f"{prefix}e{e}.up")], dim=0))
                self.down[e].copy_(get(f"{prefix}e{e}.down"))
            if self.shared_gate_up is not None:
                self.shared_gate_up.copy_(torch.cat([get(prefix + "shared.gate"), get(prefix + "shared.up")], dim=0))
                self.shared_down.copy_(get(prefix + "shared.down"))
            if self.shared_gate is not None:
                self.shared_gate.copy_(get(prefix + "shared.sg").reshape(-1))

    def forward(self, h: torch.Tensor, x32: torch.Tensor) -> torch.Tensor:
        """h: the layer's input in the activation type, x32: the same in fp32 (what the router and the experts read).
        Returns fp32 [T, W]."""
        shared = None
        if self.shared_gate_up is not None:
            shared = ops.linear(eops.gated_silu(ops.linear(h, self.shared_gate_up)), self.shared_down)
        return mops.moe_ffn(x32, h.dtype, self.router, self.gate_up, self.down, self.top, scale_input=self.scale_input,
                            shared_out=shared, w_shared_gate=self.shared_gate, softmax=self.softmax_scores,
                            renormalise=self.renormalise, correction=self.correction, groups=self.groups, clamp=self.clamp)
