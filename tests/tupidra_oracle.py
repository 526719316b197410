"""A plain, slow restatement of the Tupidra design in float64, for tests: whole sequences, no cache, no state slots, no
batching, one function per mechanism.  It shares no code with the package.

Layer:      x <- x + mixer(canon1(rms(x) w1)) + ff(canon2(rms(x) w2))
canon(h)_t = h_t + sum_j w[:, j] h_(t - taps + 1 + j)                   (zeros before the sequence's start)
Mixers:     selective scan; softcapped window attention (grouped heads, unit-RMS values, distance bias, kept first
            tokens, one added to the softmax denominator, sigmoid output gate); latent attention (normed query and
            key/value latents, one rotated key part for all heads, learned sink in the denominator, output gate,
            optionally reading another layer's latent)."""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

F64 = torch.float64


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def canon(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h: [T, W]; w: [W, taps].  The last tap multiplies the current token."""
    T, taps = h.shape[0], w.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def yarn_spectrum(dims: int, base: float, scaling: Optional[Dict[str, float]]):
    """Frequencies per pair and the amplitude of cos / sin."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_pairs(v: torch.Tensor, pos: int, freqs: List[float], amp: float) -> torch.Tensor:
    """v: [..., 2 len(freqs)]: numbers 2i and 2i + 1 form a pair."""
    out = v.clone()
    for i, f in enumerate(freqs):
        a = pos * f
        c, s = math.cos(a) * amp, math.sin(a) * amp
        u, w = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u * c - w * s
        out[..., 2 * i + 1] = w * c + u * s
    return out


def latent_kv(h: torch.Tensor, P: Dict[str, torch.Tensor], m: Dict[str, Any], eps: float):
    """The cached part of a latent-attention layer: (normed latent [T, R], rotated shared key part [T, dr])."""
    R, dr = m["kv_rank"], m["rot_dim"]
    freqs, amp = yarn_spectrum(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    d = h @ P["dkv"].T
    c = rms(d[:, :R], eps) * P["dkv.norm"]
    kr = torch.stack([rotate_pairs(d[t, R:R + dr], t, freqs, amp) for t in range(h.shape[0])])
    return c, kr


def latent_core(q: torch.Tensor, k: torch.Tensor, kr: torch.Tensor, v: torch.Tensor, sink: torch.Tensor, scale: float,
                freqs: List[float], amp: float) -> torch.Tensor:
    """q: [T, H, dn + dr] (rotated part last, not yet rotated); k: [T, H, dn]; kr: [T, dr] rotated; v: [T, H, dv]."""
    T, H, dn = k.shape
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        for hd in range(H):
            qr = rotate_pairs(q[t, hd, dn:], t, freqs, amp)
            s = (k[:t + 1, hd] @ q[t, hd, :dn] + kr[:t + 1] @ qr) * scale
            mx = max(float(s.max()), float(sink[hd]))
            e = torch.exp(s - mx)
            out[t, hd] = (e[:, None] * v[:t + 1, hd]).sum(0) / (e.sum() + math.exp(float(sink[hd]) - mx))
    return out


def latent_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], m: Dict[str, Any], eps: float, c: torch.Tensor, kr: torch.Tensor):
    T = h.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    freqs, amp = yarn_spectrum(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    cq = rms(h @ P["dq"].T, eps) * P["dq.norm"]
    q = (cq @ P["uq"].T).view(T, H, dn + dr)
    k = (c @ P["uk"].T).view(T, H, dn)
    v = (c @ P["uv"].T).view(T, H, dv)
    gate = torch.sigmoid(h @ P["g"].T).view(T, H, dv)
    out = latent_core(q, k, kr, v, P["sink"], m["scale"], freqs, amp)
    return (out * gate).reshape(T, H * dv) @ P["o"].T


def window_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, cap: float, size: int, keep: int) -> torch.Tensor:
    """q: [T, H, d]; k: [T, G, d]; v: [T, G, e] (already at unit RMS).  Returns [T, H, e].  A configuration without a cap
    or without a window has none (cap / size 0 or None)."""
    T, H = q.shape[0], q.shape[1]
    G, e = k.shape[1], v.shape[2]
    out = torch.zeros(T, H, e, dtype=F64)
    for i in range(T):
        for hd in range(H):
            g = hd // (H // G)
            slope = 2.0 ** (-8.0 * (hd + 1) / H)
            den, acc = 1.0, torch.zeros(e, dtype=F64)
            for j in range(i + 1):
                if not size or i - j < size or j < keep:
                    s = float(q[i, hd] @ k[j, g]) * scale
                    if cap:
                        s = cap * math.tanh(s / cap)
                    s -= slope * (i - j)
                    w = math.exp(s)
                    den += w
                    acc += w * v[j, g]
            out[i, hd] = acc / den
    return out


def window_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], m: Dict[str, Any], eps: float):
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ P["q"].T + P["q.b"]).view(T, H, d)
    k = (h @ P["k"].T + P["k.b"]).view(T, G, d)
    v = rms((h @ P["v"].T + P["v.b"]).view(T, G, e), eps)
    gate = torch.sigmoid(h @ P["g"].T).view(T, H, e)
    mask = m.get("mask") or {}
    out = window_core(q, k, v, m["scale"], m.get("softcap"), mask.get("size"), mask.get("keep_first") or 0)
    return (out * gate).reshape(T, H * e) @ P["o"].T + P["o.b"]


def selective_scan(h: torch.Tensor, P: Dict[str, torch.Tensor], m: Dict[str, Any]):
    T = h.shape[0]
    C, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
    xz = h @ P["in"].T
    x, z = xz[:, :C], xz[:, C:]
    u = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        acc = P["conv.b"].clone()
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                acc = acc + P["conv"][:, j] * x[s]
        u[t] = acc * torch.sigmoid(acc)
    p = u @ P["x"].T
    dt = torch.nn.functional.softplus(p[:, :R] @ P["dt"].T + P["dt.b"])
    Bm, Cm = p[:, R:R + N], p[:, R + N:R + 2 * N]
    A = -torch.exp(P["A_log"])
    S = torch.zeros(C, N, dtype=F64)
    y = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * u[t])[:, None] * Bm[t][None, :]
        y[t] = S @ Cm[t] + P["D"] * u[t]
    return (y * (z * torch.sigmoid(z))) @ P["o"].T


def feed_forward(h: torch.Tensor, P: Dict[str, torch.Tensor]):
    return (gelu_tanh(h @ P["gate"].T) * (h @ P["up"].T)) @ P["down"].T


def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: Dict[str, Any], tensors: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one whole sequence; ``layers_out`` collects the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = tensors["embed"].to(F64)[torch.tensor(tokens)]
    latents: Dict[int, Any] = {}
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        n = rms(x, eps)
        h1 = canon(n * tensors[f"l{i}.norm1"].to(F64), tensors[f"l{i}.canon1"].to(F64))
        P = sub(tensors, f"l{i}.mix.")
        if layer["type"] == "mamba1":
            a = selective_scan(h1, P, m)
        elif layer["type"] == "attention":
            a = window_attention(h1, P, m, eps)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_kv(h1, P, m, eps)
                src = i
            a = latent_attention(h1, P, m, eps, *latents[src])
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            h2 = canon(n * tensors[f"l{i}.norm2"].to(F64), tensors[f"l{i}.canon2"].to(F64))
            a = a + feed_forward(h2, sub(tensors, f"l{i}.mlp."))
        x = x + a
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * tensors["final.norm"].to(F64)) @ tensors["head"].to(F64).T


def random_weights(cfg: Dict[str, Any], seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random checkpoint tensors (float32 values that bfloat16 holds exactly) for a configuration dictionary."""
    g = torch.Generator().manual_seed(seed)
    W, taps = cfg["width"], cfg["canon"]["taps"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s / i ** 0.5).to(torch.bfloat16).float()

    def vec(n, mean=0.0, s=1.0):
        return (mean + s * torch.randn(n, generator=g)).to(torch.bfloat16).float()
    t: Dict[str, torch.Tensor] = {"embed": mat(cfg["vocab"], W, W ** 0.5), "head": mat(cfg["vocab"], W), "final.norm": vec(W, 1.0, 0.1)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        t[p + "norm1"], t[p + "canon1"] = vec(W, 1.0, 0.1), mat(W, taps, 0.8)
        if layer["type"] == "mamba1":
            C, N, R = m["inner"], m["state"], m["dt_rank"]
            t[p + "mix.in"], t[p + "mix.conv"], t[p + "mix.conv.b"] = mat(2 * C, W), mat(C, m["conv"]), vec(C, 0.0, 0.1)
            t[p + "mix.x"], t[p + "mix.dt"], t[p + "mix.dt.b"] = mat(R + 2 * N, C), mat(C, R), vec(C, -2.0, 0.7)
            t[p + "mix.A_log"] = (torch.rand(C, N, generator=g) * 2.0 - 1.5).to(torch.bfloat16).float()
            t[p + "mix.D"], t[p + "mix.o"] = vec(C, 1.0, 0.2), mat(W, C)
        elif layer["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n_, rows in (("q", H * d), ("k", G * d), ("v", G * e)):
                t[p + "mix." + n_], t[p + "mix." + n_ + ".b"] = mat(rows, W, 2.0), vec(rows, 0.0, 0.3)
            t[p + "mix.g"], t[p + "mix.o"], t[p + "mix.o.b"] = mat(H * e, W), mat(W, H * e), vec(W, 0.0, 0.1)
        else:
            H, dn, dr, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"], t[p + "mix.uq"] = mat(Q, W), vec(Q, 1.0, 0.1), mat(H * (dn + dr), Q, 2.0)
            if m.get("kv_from") is None:
                t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = mat(R + dr, W), vec(R, 1.0, 0.1)
            t[p + "mix.uk"], t[p + "mix.uv"], t[p + "mix.sink"] = mat(H * dn, R, 2.0), mat(H * dv, R), vec(H, 0.0, 1.5)
            t[p + "mix.g"], t[p + "mix.o"] = mat(H * dv, W), mat(W, H * dv)
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            t[p + "norm2"], t[p + "canon2"] = vec(W, 1.0, 0.1), mat(W, taps, 0.8)
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(ff, W), mat(ff, W), mat(W, ff)
    return t
