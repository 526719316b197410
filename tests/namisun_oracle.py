"""Plain float64 restatement of the Namisun design: one function per mechanism, whole sequences, no cache, no state
slots, no code shared with the package.  ``forward`` returns the logits of every position and the residual stream after
every layer run.  ``random_weights`` makes a checkpoint-named tensor dictionary for a configuration dictionary."""
import math

import torch

F64 = torch.float64


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def rotate_pairs(x, pos, dims, base, factor):
    """x [T, ..., n]: coordinates (2i, 2i+1), i < dims/2, are turned by pos * base^(-2i/dims) / factor."""
    i = torch.arange(dims // 2, dtype=F64)
    ang = pos.to(F64)[:, None] * (float(base) ** (-2.0 * i / dims) / factor)
    c, s = torch.cos(ang), torch.sin(ang)
    while c.dim() < x.dim():
        c, s = c.unsqueeze(1), s.unsqueeze(1)
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def differential_attention(q, k, v, scale, lam, diff, eps, gate=None):
    """q [T, H, 2, d], k [T, G, 2, d] (already rotated), v [T, G, e], gate [T, H] pre-sigmoid or None -> [T, H, e]."""
    T, H = q.shape[:2]
    G = k.shape[1]
    seen = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        maps = []
        for m in range(2):
            s = (q[:, h, m] @ k[:, g, m].T) * scale
            maps.append(torch.softmax(s.masked_fill(~seen, -math.inf), -1) @ v[:, g])
        out[:, h] = unit_rms(maps[0] - lam * maps[1], eps) * (1.0 - diff)
    if gate is not None:
        out = out * torch.sigmoid(gate)[:, :, None]
    return out


def attention_mixer(h, W, p, m, eps):
    T = h.shape[0]
    H, G, d, e = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q = (h @ W[p + "q"].T).view(T, H, 2, d)
    k = (h @ W[p + "k"].T).view(T, G, 2, d)
    v = (h @ W[p + "v"].T).view(T, G, e)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        pos = torch.arange(T)
        q = rotate_pairs(q, pos, rot["dims"], rot["base"], factor)
        k = rotate_pairs(k, pos, rot["dims"], rot["base"], factor)
    lam = math.exp(float((W[p + "lq1"] * W[p + "lk1"]).sum())) - math.exp(float((W[p + "lq2"] * W[p + "lk2"]).sum())) + m["diff"]
    o = differential_attention(q, k, v, m["scale"], lam, m["diff"], eps, h @ W[p + "g"].T)
    return o.reshape(T, H * e) @ W[p + "o"].T


def gated_linear_recurrence(q, k, v, a):
    """q, k, a [T, H, d], v [T, H, e]: S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=F64)
    o = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = (S * q[t][:, :, None]).sum(1)
    return o


def gla_mixer(h, W, p, m, eps):
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m.get("vdim", m["dim"])
    q = (h @ W[p + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ W[p + "k"].T).view(T, H, d)
    v = (h @ W[p + "v"].T).view(T, H, e)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    a = torch.sigmoid(z).pow(1.0 / m["tau"]).view(T, H, d)
    o = unit_rms(gated_linear_recurrence(q, k, v, a), eps) * W[p + "norm"]
    return (o.reshape(T, H * e) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def causal_conv(x, w, b):
    """x [T, C], w [C, taps] (last column = current token), zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x], 0)
    out = torch.zeros(T, C, dtype=F64)
    for j in range(taps):
        out += pad[j:j + T] * w[:, j]
    return out + b


def selective_recurrence(u, dt, A, B, C, D):
    """u, dt [T, Cn]; A [Cn, N]; B, C [T, N]; D [Cn]."""
    T, Cn = u.shape
    S = torch.zeros(Cn, A.shape[1], dtype=F64)
    y = torch.zeros(T, Cn, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * u[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * u[t]
    return y


def mamba_mixer(h, W, p, m):
    Cn, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ W[p + "in"].T
    x, z = xz[:, :Cn], xz[:, Cn:]
    u = silu(causal_conv(x, W[p + "conv"], W[p + "conv.b"]))
    proj = u @ W[p + "x"].T
    dt = torch.nn.functional.softplus(proj[:, :R] @ W[p + "dt"].T + W[p + "dt.b"])
    y = selective_recurrence(u, dt, -torch.exp(W[p + "A_log"]), proj[:, R:R + N], proj[:, R + N:R + 2 * N], W[p + "D"])
    return (y * silu(z)) @ W[p + "o"].T


def route(h, W, p, r):
    """Returns (ids [T, top], weights [T, top]) over experts + identity experts."""
    T = h.shape[0]
    n = r["experts"] + r.get("identity", 0)
    s = torch.softmax(h @ W[p + "router"].T, -1)
    c = s + W[p + "correction"]
    g = r.get("groups")
    if g:
        size = n // g["count"]
        best = c.view(T, g["count"], size).max(-1).values
        keep = torch.zeros(T, g["count"], dtype=torch.bool).scatter_(1, torch.topk(best, g["keep"], -1).indices, True)
        c = c.masked_fill(~keep[:, :, None].expand(T, g["count"], size).reshape(T, n), -math.inf)
    ids = torch.topk(c, r["top"], -1).indices
    w = torch.gather(s, 1, ids)
    return ids, w / (w.sum(-1, keepdim=True) + 1e-20)


def expert(x, W, p, limit):
    g = torch.clamp(W[p + "gate"] @ x, max=limit)
    u = torch.clamp(W[p + "up"] @ x, -limit, limit)
    return W[p + "down"] @ (g * torch.sigmoid(1.702 * g) * (u + 1.0))


def moe(h, W, p, m):
    ids, w = route(h, W, p, m["router"])
    E = m["router"]["experts"]
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            y[t] += w[t, j] * (h[t] if e >= E else expert(h[t], W, f"{p}e{e}.", m["expert"]["limit"]))
    return y


def layer_runs(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None) for i in range(lp["stop"], n)]


def forward(cfg, W, tokens):
    """-> (logits [T, vocab], [stream after every layer run])."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = W["embed"][torch.as_tensor(tokens)]
    trace = []
    for i, t in layer_runs(cfg):
        if t is not None:
            x = x + W["loop.step"][t]
        l = cfg["layers"][i]
        h = layer_norm(x, W[f"l{i}.norm1"], W[f"l{i}.norm1.b"], eps)
        p = f"l{i}.mix."
        if l["type"] == "gla":
            a = gla_mixer(h, W, p, l["mixer"], eps)
        elif l["type"] == "attention":
            a = attention_mixer(h, W, p, l["mixer"], eps)
        else:
            a = mamba_mixer(h, W, p, l["mixer"])
        f = moe(h, W, f"l{i}.mlp.", l["mlp"]) if l.get("mlp") else 0.0
        x = x + mult * (a + f)
        trace.append(x)
    y = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    return y @ W["embed"].T * cfg.get("logit_scale", 1.0), trace


def greedy(cfg, W, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(cfg, W, toks)[0][-1].argmax()))
    return toks[len(prompt):]


def random_weights(cfg, seed=0, dtype=torch.float32, slow_decay=False):
    """Checkpoint-named tensors.  ``slow_decay``: decays close to 1 in the recurrent layers, so that a token far back
    still weighs in the state."""
    g = torch.Generator().manual_seed(seed)
    Wd = cfg["width"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s / i ** 0.5).to(dtype)

    def vec(n, mean=0.0, s=0.1):
        return (mean + s * torch.randn(n, generator=g)).to(dtype)
    W = {"embed": mat(cfg["vocab"], Wd, Wd ** 0.5), "final.norm": vec(Wd, 1.0), "final.norm.b": vec(Wd)}
    if cfg.get("loop"):
        W["loop.step"] = (0.3 * torch.randn(cfg["loop"]["times"], Wd, generator=g)).to(dtype)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", l["mixer"]
        W[f"l{i}.norm1"], W[f"l{i}.norm1.b"] = vec(Wd, 1.0), vec(Wd)
        if l["type"] == "mamba1":
            Cn, N, R = m["inner"], m["state"], m["dt_rank"]
            W[p + "in"], W[p + "conv"], W[p + "conv.b"] = mat(2 * Cn, Wd), mat(Cn, m["conv"]), vec(Cn)
            W[p + "x"], W[p + "dt"] = mat(R + 2 * N, Cn), mat(Cn, R)
            W[p + "dt.b"] = (torch.rand(Cn, generator=g) * 2.0 - (5.0 if slow_decay else 2.0)).to(dtype)
            W[p + "A_log"] = (torch.rand(Cn, N, generator=g) * 1.5 - (3.0 if slow_decay else 0.5)).to(dtype)
            W[p + "D"], W[p + "o"] = vec(Cn, 1.0), mat(Wd, Cn)
        elif l["type"] == "gla":
            H, d, e, r = m["heads"], m["dim"], m.get("vdim", m["dim"]), m["decay_rank"]
            W[p + "q"], W[p + "k"], W[p + "v"], W[p + "g"] = mat(H * d, Wd, 2.0), mat(H * d, Wd, 2.0), mat(H * e, Wd), mat(H * e, Wd)
            W[p + "a1"], W[p + "a2"] = mat(r, Wd), mat(H * d, r)
            W[p + "a2.b"] = (torch.rand(H * d, generator=g) * 3.0 + (4.0 if slow_decay else 0.0)).to(dtype)
            W[p + "norm"], W[p + "o"] = vec(e, 1.0), mat(Wd, H * e)
        else:
            H, G, d, e = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
            W[p + "q"], W[p + "k"], W[p + "v"] = mat(H * 2 * d, Wd, 2.0), mat(G * 2 * d, Wd, 2.0), mat(G * e, Wd)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                W[p + n] = vec(d, 0.0, 0.4)
            W[p + "g"], W[p + "o"] = mat(H, Wd, 2.0), mat(Wd, H * e)
        if l.get("mlp"):
            p = f"l{i}.mlp."
            r, ff = l["mlp"]["router"], l["mlp"]["expert"]["ff"]
            n = r["experts"] + r.get("identity", 0)
            W[p + "router"] = mat(n, Wd, 3.0)
            W[p + "correction"] = vec(n, 0.0, 0.15)
            for e in range(r["experts"]):
                W[f"{p}e{e}.gate"], W[f"{p}e{e}.up"], W[f"{p}e{e}.down"] = mat(ff, Wd, 2.0), mat(ff, Wd, 2.0), mat(Wd, ff)
    return W
