"""Tupidra: a decoder-only design whose layers run a sequence mixer and a gated feed-forward IN PARALLEL on the same
residual stream, each behind its own weighted RMS norm and its own short causal convolution over time on the normed input:

    n   = x / sqrt(mean(x^2) + eps)
    h_s = canon_s(w_s n),   canon(h)_t = h_t + sum_j c[:, j] h_(t - taps + 1 + j)         s = 1 (mixer), 2 (feed-forward)
    x  <- x + mixer(h_1) + ff(h_2)

The residual stream ``x`` is fp32 and starts as ``embed[token]``; the output is ``head . (w_final n_final)``.  Three kinds of
mixers (``models/mixers.py``): ``mamba1`` (selective state-space scan), ``attention`` (grouped-query attention with a
tanh soft cap, a linear distance bias, a sliding window that keeps the first tokens, one added to the softmax denominator,
unit-RMS values, projection biases and a sigmoid output gate) and ``latent_attention`` (low-rank key/value latent with a
shared rotated key part, YaRN-blended rotation, a learned sink per head, a sigmoid output gate, optionally reading an
earlier layer's cache).  The feed-forward is ``Wdown (gelu_tanh(Wgate h) * (Wup h))`` (``models/ffn.py``).  Per-sequence
state: the last ``taps - 1`` rows of ``n`` of every layer (shared by both sublayers), the scan's state and its own
convolution inputs; per-token cache: keys and unit-RMS values of attention layers, latent and rotated key part of latent
layers.  The layer list, every size and every constant come from the checkpoint's ``config.json``:

    {"architecture": "Tupidra", "width", "vocab", "norm": {"eps"}, "canon": {"taps"},
     "layers": [{"type": "mamba1", "mixer": {"inner", "state", "dt_rank", "conv"}, "mlp": ...},
                {"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap",
                                                "mask": {"size", "keep_first"}}, "mlp": ...},
                {"type": "latent_attention", "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "kv_from"?,
                                                       "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}?}},
                 "mlp": ...}]}
    mlp: null | {"kind": "dense", "ff"}

Checkpoint tensors: ``embed``, ``head``, ``final.norm``, ``l<i>.norm1|norm2``, ``l<i>.canon1|canon2`` ([width, taps], last
column = the current token's), ``l<i>.mix.*`` (see the mixers' ``load``), ``l<i>.mlp.{gate,up,down}``; linear weights are
[out, in].  The model runs ragged paged batches only (``forward_ragged``); the serving engine owns the caches, the state
slots and their reuse.

Reference: none — the reference serves whatever HF returns (reference llmctl/serve/server.py:127-160)."""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn

from ..ops import canon as cops
from ..ops import elementwise as eops
from ..ops import functional as ops
from .ffn import GatedGeluMLP
from .mixers import (LatentAttention, LatentAttentionSpec, SelectiveScan, SelectiveScanSpec, SoftcapWindowAttention,
                     SoftcapWindowAttentionSpec)
from .registry import Architecture, register_architecture

MIXER_TYPES = ("mamba1", "attention", "latent_attention")


@dataclass
class TupidraLayer:
    type: str
    mixer: Any                              # the mixer's spec
    ff: int                                 # inner size of the feed-forward, 0 = none


@dataclass
class TupidraConfig:
    name: str = "tupidra"
    width: int = 256
    vocab_size: int = 512
    norm_eps: float = 1e-6
    taps: int = 4                           # taps of the input convolutions (1 = none)
    layers: List[TupidraLayer] = field(default_factory=list)
    max_position_embeddings: int = 1 << 20               # no position table: bounded by the cache pool only
    raw: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, d: Dict[str, Any], name: str = "tupidra") -> "TupidraConfig":
        layers: List[TupidraLayer] = []
        for i, l in enumerate(d["layers"]):
            m = l["mixer"]
            if l["type"] == "mamba1":
                spec: Any = SelectiveScanSpec(inner=int(m["inner"]), state=int(m["state"]), dt_rank=int(m["dt_rank"]), conv=int(m["conv"]))
            elif l["type"] == "attention":
                mask = m.get("mask") or {}
                spec = SoftcapWindowAttentionSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                                                  vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]),
                                                  softcap=float(m.get("softcap") or 0.0), window=int(mask.get("size") or 0),
                                                  keep_first=int(mask.get("keep_first") or 0))
                if spec.heads % spec.kv_heads:
                    raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            elif l["type"] == "latent_attention":
                rot = m["rot"]
                if int(rot["dims"]) != int(m["rot_dim"]) or int(m["rot_dim"]) % 2:
                    raise ValueError(f"layer {i}: the rotated part must be rot_dim = rot.dims (even) numbers")
                src = m.get("kv_from")
                spec = LatentAttentionSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                                           kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]), scale=float(m["scale"]),
                                           rot_base=float(rot["base"]), rot_scaling=rot.get("scaling") or None,
                                           kv_from=None if src is None else int(src), sink=True, out_gate=True)
                if src is not None:
                    if not 0 <= int(src) < i or layers[int(src)].type != "latent_attention" or layers[int(src)].mixer.kv_from is not None:
                        raise ValueError(f"layer {i}: kv_from must name an earlier latent-attention layer that has a cache of its own")
                    if layers[int(src)].mixer.cache_width != spec.cache_width:
                        raise ValueError(f"layer {i}: its latent and rope sizes differ from those of layer {src}")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r} (known: {MIXER_TYPES})")
            mlp = l.get("mlp")
            if mlp is not None and mlp.get("kind") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            layers.append(TupidraLayer(l["type"], spec, int(mlp["ff"]) if mlp is not None else 0))
        taps = int((d.get("canon") or {}).get("taps", 1))
        if not 1 <= taps <= cops.MAX_TAPS:
            raise ValueError(f"canon.taps must lie in 1..{cops.MAX_TAPS}")
        return cls(name=name, width=int(d["width"]), vocab_size=int(d["vocab"]), norm_eps=float((d.get("norm") or {}).get("eps", 1e-6)),
                   taps=taps, layers=layers, raw=d)

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    def num_parameters(self) -> int:
        with torch.device("meta"):
            m = TupidraModel(self, dtype=torch.bfloat16, device="meta")
        return sum(p.numel() for p in m.parameters())


class TupidraBlock(nn.Module):
    def __init__(self, cfg: TupidraConfig, layer: TupidraLayer, dtype, device):
        super().__init__()
        W = cfg.width
        f32 = dict(dtype=torch.float32, device=device)
        subs = 2 if layer.ff else 1
        self.norm_w = nn.ParameterList([nn.Parameter(torch.ones(W, **f32)) for _ in range(subs)])
        self.canon_w = nn.ParameterList([nn.Parameter(torch.zeros(W, cfg.taps, **f32)) for _ in range(subs)])
        if layer.type == "mamba1":
            self.mixer: nn.Module = SelectiveScan(W, layer.mixer, dtype, device)
        elif layer.type == "attention":
            self.mixer = SoftcapWindowAttention(W, layer.mixer, cfg.norm_eps, dtype, device)
        else:
            self.mixer = LatentAttention(W, layer.mixer, cfg.norm_eps, dtype, device)
        self.mlp = GatedGeluMLP(W, layer.ff, dtype, device) if layer.ff else None


class TupidraModel(nn.Module):
    ragged = True           # runs ragged paged batches through ``forward_ragged`` (serve/engine.py)
    stateful = True         # keeps per-sequence states: the engine hands out state slots with the pages

    def __init__(self, cfg: TupidraConfig, *, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg, self.dtype = cfg, dtype
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.width, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([TupidraBlock(cfg, l, dtype, device) for l in cfg.layers])
        self.final_w = nn.Parameter(torch.ones(cfg.width, dtype=torch.float32, device=device))
        self.head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.width, dtype=dtype, device=device))

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
            self.head.copy_(get("head"))
            self.final_w.copy_(get("final.norm").float())
            for i, blk in enumerate(self.blocks):
                for s in range(len(blk.norm_w)):
                    blk.norm_w[s].copy_(get(f"l{i}.norm{s + 1}").float())
                    blk.canon_w[s].copy_(get(f"l{i}.canon{s + 1}").float())
                blk.mixer.load(get, f"l{i}.mix.")
                if blk.mlp is not None:
                    blk.mlp.load(get, f"l{i}.mlp.")

    def init_random(self, seed: int = 0) -> None:
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for name, p in self.named_parameters():
                leaf = name.rsplit(".", 1)[-1]
                if leaf == "A":
                    p.copy_(-torch.exp(torch.rand(p.shape, generator=g) * 1.5 - 1.0))
                elif leaf == "dt_bias":
                    p.copy_(torch.rand(p.shape, generator=g) * 2.0 - 3.0)
                elif leaf == "sink":
                    p.copy_(torch.randn(p.shape, generator=g))
                elif leaf in ("conv_b", "b_in", "b_o"):
                    p.copy_(0.05 * torch.randn(p.shape, generator=g))
                elif leaf == "conv_w" or ".canon_w." in name:
                    p.copy_(torch.randn(p.shape, generator=g) / (2.0 * p.shape[-1] ** 0.5))
                elif p.dim() == 1:
                    p.copy_((1.0 + 0.1 * torch.randn(p.shape, generator=g)).to(p.dtype))
                else:
                    p.copy_((torch.randn(p.shape, generator=g) / p.shape[-1] ** 0.5).to(p.dtype))

    # ---- caches and states -----------------------------------------------------------------------------
    def cache_bytes_per_block(self, block_size: int) -> int:
        it = torch.empty((), dtype=self.dtype).element_size()
        own = [l.mixer.cache_width for l in self.cfg.layers
               if l.type == "attention" or (l.type == "latent_attention" and l.mixer.kv_from is None)]
        return sum(own) * block_size * it

    def allocate_caches(self, num_blocks: int, block_size: int, device, state_slots: int = 1) -> List[Any]:
        """One entry per layer: ``(input-convolution state, mixer cache or states)``.  The first is fp32 ``[state_slots,
        taps - 1, width]``; the second the paged cache of an attention layer (a layer that reads another layer's cache gets
        that very tensor) or the tuple of fp32 state tensors ``[state_slots, ...]`` of a scan layer."""
        out: List[Any] = []
        for i, blk in enumerate(self.blocks):
            canon = torch.zeros(state_slots, self.cfg.taps - 1, self.cfg.width, dtype=torch.float32, device=device)
            mixer = blk.mixer
            if mixer.stateful:
                own: Any = tuple(torch.zeros(state_slots, *shape, dtype=torch.float32, device=device) for shape in mixer.state_shapes())
            elif getattr(mixer.spec, "kv_from", None) is not None:
                own = out[mixer.spec.kv_from][1]
            else:
                own = torch.zeros(mixer.cache_shape(num_blocks, block_size), dtype=self.dtype, device=device)
            out.append((canon, own))
        return out

    # ---- forward ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward_ragged(self, batch, caches: List[Any], layer_trace: Optional[list] = None) -> torch.Tensor:
        """``batch``: serve.ragged.RaggedBatch.  Returns fp32 logits [len(batch.out_rows), vocab]."""
        cfg, dt, eps = self.cfg, self.dtype, self.cfg.norm_eps
        x, _ = eops.embed_scale(batch.tokens, self.embed, 1.0)
        small = batch.decode_only               # one token per portion: the layer's glue is a single launch
        a = f = None
        for i, blk in enumerate(self.blocks):
            canon_state, own = caches[i]
            # the previous layer's residual update (x += a + f), this layer's norm statistics and both sublayers' inputs
            hs = cops.residual_norm_canon(a, f, x, eps, list(blk.norm_w), list(blk.canon_w), batch.portions, batch.seq_rows, canon_state, dt, small)
            if layer_trace is not None and i > 0:
                layer_trace.append(x.clone())
            a = blk.mixer(hs[0], batch, own)
            f = blk.mlp(hs[1]) if blk.mlp is not None else None
        if a is not None:
            cops.residual_rms(a, f, x, eps)
            if layer_trace is not None:
                layer_trace.append(x.clone())
        if batch.num_out == 0:                  # a step that only fills the caches and states
            return torch.empty(0, cfg.vocab_size, dtype=torch.float32, device=x.device)
        y = eops.rmsnorm_rows(x, batch.out_rows, self.final_w, eps, dt)
        if y.is_cuda and dt == torch.bfloat16:
            if ops.kernel_config().gemm == "native" and ops._gemm_ok(y, self.head) and self.head.shape[0] % 8 == 0:
                return ops.gemm_raw(y, self.head, out_dtype=torch.float32)
            return torch.mm(y, self.head.t(), out_dtype=torch.float32)
        return torch.nn.functional.linear(y.float(), self.head.float())


def _load_weights(model: TupidraModel, directory) -> None:
    from safetensors.torch import load_file
    model.load_state(load_file(str(Path(directory) / "model.safetensors")))


def build_tupidra(cfg: TupidraConfig, *, dtype=torch.bfloat16, device=None, seed: int = 42, **_ignored) -> TupidraModel:
    m = TupidraModel(cfg, dtype=dtype, device=device)
    m.init_random(seed)
    return m


register_architecture(Architecture(name="Tupidra", config_from_dict=TupidraConfig.from_dict, config_type=TupidraConfig,
                                   build=build_tupidra, load_weights=_load_weights))


def example_config(width: int = 48, vocab: int = 80, pattern: str = "MALc", ff: str = "1101", taps: int = 3, heads: int = 4,
                   kv_heads: int = 2, dim: int = 8, vdim: int = 12, softcap: float = 5.0, window: int = 9, keep_first: int = 2,
                   lat_heads: int = 3, lat_dim: int = 6, rot_dim: int = 4, lat_vdim: int = 10, kv_rank: int = 16, q_rank: int = 12,
                   yarn: bool = True, inner: int = 40, state: int = 6, dt_rank: int = 3, conv: int = 3, ff_size: int = 40) -> Dict[str, Any]:
    """A small configuration dictionary for tests, benchmarks and examples.  ``pattern``: one character per layer for its
    mixer (M selective scan, A soft-capped window attention, L latent attention with a cache of its own, c latent
    attention reading the latest L layer's cache); ``ff``: one character per layer, 1 = the layer has a feed-forward."""
    layers: List[Dict[str, Any]] = []
    last_l = None
    for i, ch in enumerate(pattern):
        if ch == "M":
            layer: Dict[str, Any] = {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}
        elif ch == "A":
            layer = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5,
                                                    "softcap": softcap, "mask": {"size": window, "keep_first": keep_first}}}
        else:
            rot: Dict[str, Any] = {"base": 10000.0, "dims": rot_dim}
            if yarn:
                rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
            mixer = {"heads": lat_heads, "dim": lat_dim, "rot_dim": rot_dim, "vdim": lat_vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                     "scale": (lat_dim + rot_dim) ** -0.5, "rot": rot}
            if ch == "c":
                mixer["kv_from"] = last_l
            else:
                last_l = i
            layer = {"type": "latent_attention", "mixer": mixer}
        layer["mlp"] = {"kind": "dense", "ff": ff_size} if ff[i % len(ff)] == "1" else None
        layers.append(layer)
    return {"architecture": "Tupidra", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "canon": {"taps": taps}, "layers": layers}
