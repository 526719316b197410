"""Namisun: a decoder-only design that interleaves three kinds of sequence mixers (``models/mixers.py``) — selective
state-space scans, gated linear attention and differential attention — each next to a mixture-of-experts feed-forward
(``models/ffn.py``) in a PARALLEL residual layout with one layer norm per layer:

    h = LN(x);    x <- x + m (mixer(h) + ff(h))          LN(v) = (v - mean) / sqrt(var + eps) * w + b

The residual stream ``x`` is fp32 and starts as ``embed[token]``; the output is ``embed . LN_final(x) * logit_scale`` (tied
embedding).  A contiguous range of layers may be LOOPED: layers ``start .. stop-1`` run ``times`` times in a row with the
same weights before the rest follow; every pass keeps a cache / state of its own, and a learned vector ``step[t]`` joins
the stream right before pass t's first layer.  A "layer run" below is one execution of one layer; caches and states
are per run.

The router of a mixture sees the experts and, behind them, ``identity`` identity experts (output = input): softmax
scores over all of them, a learned correction added for the choice only, choice restricted to the best ``keep`` of
``count`` groups of neighbouring router outputs, weights = chosen scores renormalised.  Experts compute
``g sigmoid(1.702 g) (u + 1)`` on the clamped gate and up projections.  The layer list, every size and every constant come
from the checkpoint's ``config.json``:

    {"architecture": "Namisun", "width", "vocab", "norm": {"eps"}, "residual_mult", "logit_scale",
     "loop": {"start", "stop", "times"}?,
     "layers": [{"type": "mamba1", "mixer": {"inner", "state", "dt_rank", "conv"}, "mlp": ...},
                {"type": "gla", "mixer": {"heads", "dim", "vdim", "tau"}, "mlp": ...},
                {"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "diff",
                                                "rot": {"base", "dims", "scaling": {"factor"}?}?}, "mlp": ...}]}
    mlp: null | {"kind": "moe", "router": {"experts", "top", "identity"?, "groups": {"count", "keep"}?}, "expert": {"ff", "limit"}}

Checkpoint tensors: ``embed``, ``loop.step`` [times, width], ``final.norm`` (+ ``.b``), ``l<i>.norm1`` (+ ``.b``),
``l<i>.mix.*`` (see the mixers' ``load``), ``l<i>.mlp.{router,correction,e<k>.{gate,up,down}}``; linear weights are
[out, in].  The model runs ragged paged batches only (``forward_ragged``); the serving engine owns the caches, the state
slots and their reuse.

Reference: none — the reference serves whatever HF returns (reference llmctl/serve/server.py:127-160)."""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import elementwise as eops
from ..ops import functional as ops
from .ffn import GatedExpertMoE
from .mixers import (DifferentialAttention, DifferentialAttentionSpec, GatedLinearAttention, GatedLinearAttentionSpec, SelectiveScan,
                     SelectiveScanSpec)
from .registry import Architecture, register_architecture

MIXER_TYPES = ("mamba1", "gla", "attention")
EXPERT_GATE_ALPHA = 1.702       # the experts' gate is g * sigmoid(1.702 g)


@dataclass
class NamisunLayer:
    type: str
    mixer: Any                              # the mixer's spec
    mlp: Optional[Dict[str, Any]]


@dataclass
class NamisunConfig:
    name: str = "namisun"
    width: int = 256
    vocab_size: int = 512
    norm_eps: float = 1e-5
    residual_mult: float = 1.0
    logit_scale: float = 1.0
    loop: Optional[Tuple[int, int, int]] = None          # (start, stop, times)
    layers: List[NamisunLayer] = field(default_factory=list)
    max_position_embeddings: int = 1 << 20               # no position table: bounded by the cache pool only
    raw: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: Dict[str, Any], name: str = "namisun") -> "NamisunConfig":
        layers: List[NamisunLayer] = []
        for i, l in enumerate(d["layers"]):
            m = l["mixer"]
            if l["type"] == "mamba1":
                spec: Any = SelectiveScanSpec(inner=int(m["inner"]), state=int(m["state"]), dt_rank=int(m["dt_rank"]), conv=int(m["conv"]))
            elif l["type"] == "gla":
                spec = GatedLinearAttentionSpec(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])),
                                                tau=float(m["tau"]), decay_rank=int(m.get("decay_rank", 0)))
            elif l["type"] == "attention":
                rot = m.get("rot") or {}
                spec = DifferentialAttentionSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                                                 vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]), diff=float(m["diff"]),
                                                 rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)),
                                                 rot_scaling=rot.get("scaling") or None, head_gate=True)
                if spec.heads % spec.kv_heads:
                    raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r} (known: {MIXER_TYPES})")
            mlp = l.get("mlp")
            if mlp is not None and mlp.get("kind") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            layers.append(NamisunLayer(l["type"], spec, mlp))
        loop = None
        lp = d.get("loop")
        if lp and int(lp.get("times", 1)) >= 1 and int(lp["stop"]) > int(lp["start"]):
            loop = (int(lp["start"]), int(lp["stop"]), int(lp.get("times", 1)))
            if not 0 <= loop[0] < loop[1] <= len(layers):
                raise ValueError(f"loop {lp} does not fit {len(layers)} layers")
        return cls(name=name, width=int(d["width"]), vocab_size=int(d["vocab"]), norm_eps=float((d.get("norm") or {}).get("eps", 1e-5)),
                   residual_mult=float(d.get("residual_mult", 1.0)), logit_scale=float(d.get("logit_scale", 1.0)), loop=loop,
                   layers=layers, raw=d)

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    def runs(self) -> List[Tuple[int, Optional[int]]]:
        """The layer runs in order: (layer index, number of the pass this run opens or None)."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        out: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(start)]
        for t in range(times):
            out += [(i, t if i == start else None) for i in range(start, stop)]
        return out + [(i, None) for i in range(stop, n)]

    def num_parameters(self) -> int:
        with torch.device("meta"):
            m = NamisunModel(self, dtype=torch.bfloat16, device="meta")
        return sum(p.numel() for p in m.parameters())


class NamisunBlock(nn.Module):
    def __init__(self, cfg: NamisunConfig, layer: NamisunLayer, dtype, device, decay_rank: Optional[int] = None):
        super().__init__()
        W = cfg.width
        self.norm_w = nn.Parameter(torch.ones(W, dtype=torch.float32, device=device))
        self.norm_b = nn.Parameter(torch.zeros(W, dtype=torch.float32, device=device))
        if layer.type == "mamba1":
            self.mixer: nn.Module = SelectiveScan(W, layer.mixer, dtype, device)
        elif layer.type == "gla":
            self.mixer = GatedLinearAttention(W, layer.mixer, cfg.norm_eps, dtype, device)
        else:
            self.mixer = DifferentialAttention(W, layer.mixer, cfg.norm_eps, dtype, device)
        self.mlp: Optional[GatedExpertMoE] = None
        if layer.mlp is not None:
            r, ex = layer.mlp["router"], layer.mlp["expert"]
            g = r.get("groups")
            self.mlp = GatedExpertMoE(W, int(r["experts"]), int(r["top"]), int(ex["ff"]), None, dtype, device, scale_input=False,
                                      softmax_scores=True, renormalise=True, shared_gate=False, identity=int(r.get("identity", 0)),
                                      correction=True, groups=(int(g["count"]), int(g["keep"])) if g else None,
                                      clamp=(float(ex["limit"]), EXPERT_GATE_ALPHA))


class NamisunModel(nn.Module):
    ragged = True           # runs ragged paged batches through ``forward_ragged`` (serve/engine.py)
    stateful = True         # keeps per-sequence states: the engine hands out state slots with the pages

    def __init__(self, cfg: NamisunConfig, *, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg, self.dtype = cfg, dtype
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.width, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([NamisunBlock(cfg, l, dtype, device) for l in cfg.layers])
        times = cfg.loop[2] if cfg.loop else 0
        self.loop_step = nn.Parameter(torch.zeros(times, cfg.width, dtype=torch.float32, device=device)) if times else None
        self.final_w = nn.Parameter(torch.ones(cfg.width, dtype=torch.float32, device=device))
        self.final_b = nn.Parameter(torch.zeros(cfg.width, dtype=torch.float32, device=device))
        self.runs = cfg.runs()
        self._out_norm: Optional[Tuple[torch.Tensor, torch.Tensor]] = None

    # ---- weights ---------------------------------------------------------------------------------------
    def load_state(self, tensors: Dict[str, torch.Tensor]) -> None:
        """``tensors``: checkpoint names -> tensors (any float type; converted to the model's)."""
        dev = self.embed.device

        def get(name: str) -> torch.Tensor:
            if name not in tensors:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            return tensors[name].to(dev)
        with torch.no_grad():
            self.embed.copy_(get("embed"))
            if self.loop_step is not None:
                self.loop_step.copy_(get("loop.step").float())
            self.final_w.copy_(get("final.norm").float())
            self.final_b.copy_(get("final.norm.b").float())
            for i, blk in enumerate(self.blocks):
                blk.norm_w.copy_(get(f"l{i}.norm1").float())
                blk.norm_b.copy_(get(f"l{i}.norm1.b").float())
                blk.mixer.load(get, f"l{i}.mix.")
                if blk.mlp is not None:
                    blk.mlp.load(get, f"l{i}.mlp.")
        self._out_norm = None

    def init_random(self, seed: int = 0) -> None:
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                leaf = name.rsplit(".", 1)[-1]
                if leaf == "A":
                    p.copy_(-torch.exp(torch.rand(p.shape, generator=g) * 1.5 - 1.0))
                elif leaf == "dt_bias":
                    p.copy_(torch.rand(p.shape, generator=g) * 2.0 - 3.0)
                elif leaf == "b_a2":
                    p.copy_(torch.rand(p.shape, generator=g) * 3.0 + 1.0)
                elif leaf in ("lam_q", "lam_k"):
                    p.copy_(0.3 * torch.randn(p.shape, generator=g))
                elif leaf in ("correction", "norm_b", "final_b", "conv_b"):
                    p.copy_(0.05 * torch.randn(p.shape, generator=g))
                elif leaf == "loop_step":
                    p.copy_(0.2 * torch.randn(p.shape, generator=g))
                elif leaf == "conv_w":
                    p.copy_(torch.randn(p.shape, generator=g) / p.shape[-1] ** 0.5)
                elif p.dim() == 1:
                    p.copy_((1.0 + 0.1 * torch.randn(p.shape, generator=g)).to(p.dtype))
                else:
                    p.copy_((torch.randn(p.shape, generator=g) / p.shape[-1] ** 0.5).to(p.dtype))
        for blk in self.blocks:
            if isinstance(blk.mixer, DifferentialAttention):
                blk.mixer._lam = None
        self._out_norm = None

    # ---- caches and states -----------------------------------------------------------------------------
    def cache_bytes_per_block(self, block_size: int) -> int:
        it = torch.empty((), dtype=self.dtype).element_size()
        return sum(block_size * self.cfg.layers[li].mixer.cache_width for li, _ in self.runs if self.cfg.layers[li].type == "attention") * it

    def allocate_caches(self, num_blocks: int, block_size: int, device, state_slots: int = 1) -> List[Any]:
        """One entry per layer run: the paged ``[pages, block_size, G (2 d + e)]`` key/value cache of an attention run, or
        the tuple of fp32 state tensors ``[state_slots, ...]`` of a recurrent run."""
        out: List[Any] = []
        for li, _ in self.runs:
            mixer = self.blocks[li].mixer
            if mixer.stateful:
                out.append(tuple(torch.zeros(state_slots, *shape, dtype=torch.float32, device=device) for shape in mixer.state_shapes()))
            else:
                out.append(torch.zeros(mixer.cache_shape(num_blocks, block_size), dtype=self.dtype, device=device))
        return out

    # ---- forward ---------------------------------------------------------------------------------------
    def _step_vector(self, run: Tuple[int, Optional[int]]) -> Optional[torch.Tensor]:
        return self.loop_step[run[1]] if run[1] is not None else None

    @torch.no_grad()
    def forward_ragged(self, batch, caches: List[Any], layer_trace: Optional[list] = None) -> torch.Tensor:
        """``batch``: serve.ragged.RaggedBatch.  Returns fp32 logits [len(batch.out_rows), vocab]."""
        cfg, dt, eps, m = self.cfg, self.dtype, self.cfg.norm_eps, self.cfg.residual_mult
        blocks, runs = self.blocks, self.runs
        x, _ = eops.embed_scale(batch.tokens, self.embed, 1.0)
        h = h32 = None
        if runs:
            b0 = blocks[runs[0][0]]
            h, h32 = eops.layernorm_rows(x, None, b0.norm_w, b0.norm_b, eps, dt, add=self._step_vector(runs[0]), want_fp32=True)
        for r, run in enumerate(runs):
            blk = blocks[run[0]]
            a = blk.mixer(h, batch, caches[r])
            f = blk.mlp(h, h32) if blk.mlp is not None else None
            nxt = runs[r + 1] if r + 1 < len(runs) else None
            if nxt is None or layer_trace is not None:
                eops.parallel_residual(a, f, x, m, eps, dt)
                if layer_trace is not None:
                    layer_trace.append(x.clone())
                if nxt is not None:
                    nb = blocks[nxt[0]]
                    h, h32 = eops.layernorm_rows(x, None, nb.norm_w, nb.norm_b, eps, dt, add=self._step_vector(nxt), want_fp32=True)
            else:
                # residual update, the next pass's step vector and the next layer's norm in one pass over the rows
                nb = blocks[nxt[0]]
                h, h32 = eops.parallel_residual(a, f, x, m, eps, dt, nb.norm_w, nb.norm_b, add=self._step_vector(nxt), want_fp32=True)
        if batch.num_out == 0:                  # a step that only fills the caches and states
            return torch.empty(0, cfg.vocab_size, dtype=torch.float32, device=x.device)
        if self._out_norm is None:              # logit_scale folded into the final norm's weight and bias
            self._out_norm = (self.final_w.detach() * cfg.logit_scale, self.final_b.detach() * cfg.logit_scale)
        y = eops.layernorm_rows(x, batch.out_rows, self._out_norm[0], self._out_norm[1], eps, dt)
        if y.is_cuda and dt == torch.bfloat16:
            if ops.kernel_config().gemm == "native" and ops._gemm_ok(y, self.embed) and self.embed.shape[0] % 8 == 0:
                return ops.gemm_raw(y, self.embed, out_dtype=torch.float32)
            return torch.mm(y, self.embed.t(), out_dtype=torch.float32)
        return torch.nn.functional.linear(y.float(), self.embed.float())


def _complete_config(cfg: NamisunConfig, directory) -> None:
    """The inner size of a gated-linear-attention layer's decay projection is not in ``config.json``: it is the first
    extent of the checkpoint's ``l<i>.mix.a1``."""
    missing = [i for i, l in enumerate(cfg.layers) if l.type == "gla" and not l.mixer.decay_rank]
    if not missing:
        return
    from safetensors import safe_open
    with safe_open(str(Path(directory) / "model.safetensors"), framework="pt") as f:
        for i in missing:
            cfg.layers[i].mixer.decay_rank = int(f.get_slice(f"l{i}.mix.a1").get_shape()[0])


def _load_weights(model: NamisunModel, directory) -> None:
    from safetensors.torch import load_file
    model.load_state(load_file(str(Path(directory) / "model.safetensors")))


def build_namisun(cfg: NamisunConfig, *, dtype=torch.bfloat16, device=None, seed: int = 42, **_ignored) -> NamisunModel:
    m = NamisunModel(cfg, dtype=dtype, device=device)
    m.init_random(seed)
    return m


register_architecture(Architecture(name="Namisun", config_from_dict=NamisunConfig.from_dict, config_type=NamisunConfig,
                                   build=build_namisun, load_weights=_load_weights, complete_config=_complete_config))


def example_config(width: int = 48, vocab: int = 80, pattern: str = "MGAG", moe: str = "1101", loop: Optional[Tuple[int, int, int]] = (1, 3, 2),
                   heads: int = 4, kv_heads: int = 2, dim: int = 8, vdim: int = 12, rot_dims: int = 4, rot_factor: Optional[float] = 4.0,
                   diff: float = 0.3, gla_heads: int = 2, gla_dim: int = 8, gla_vdim: int = 10, tau: float = 8.0, decay_rank: int = 4,
                   inner: int = 40, state: int = 6, dt_rank: int = 3, conv: int = 3, experts: int = 6, identity: int = 2, top: int = 2,
                   groups: Optional[Tuple[int, int]] = (4, 2), ff: int = 16, limit: float = 1.5, residual_mult: float = 0.7,
                   logit_scale: float = 0.5) -> Dict[str, Any]:
    """A small configuration dictionary for tests, benchmarks and examples.  ``pattern``: one character per layer for its
    mixer (M selective scan, G gated linear attention, A differential attention); ``moe``: one character per layer, 1 =
    the layer has a mixture-of-experts feed-forward, 0 = none; ``loop`` = (start, stop, times) or None."""
    layers = []
    for i, ch in enumerate(pattern):
        if ch == "M":
            layer: Dict[str, Any] = {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}
        elif ch == "G":
            layer = {"type": "gla", "mixer": {"heads": gla_heads, "dim": gla_dim, "vdim": gla_vdim, "tau": tau, "decay_rank": decay_rank}}
        else:
            rot: Dict[str, Any] = {"base": 10000.0, "dims": rot_dims}
            if rot_factor:
                rot["scaling"] = {"factor": rot_factor}
            layer = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5,
                                                    "diff": diff, "rot": rot if rot_dims else None}}
        mlp: Optional[Dict[str, Any]] = None
        if moe[i % len(moe)] == "1":
            router: Dict[str, Any] = {"experts": experts, "top": top, "identity": identity}
            if groups:
                router["groups"] = {"count": groups[0], "keep": groups[1]}
            mlp = {"kind": "moe", "router": router, "expert": {"ff": ff, "limit": limit}}
        layer["mlp"] = mlp
        layers.append(layer)
    cfg: Dict[str, Any] = {"architecture": "Namisun", "width": width, "vocab": vocab, "norm": {"eps": 1e-5},
                           "residual_mult": residual_mult, "logit_scale": logit_scale, "layers": layers}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg
