"""Serving throughput of a ragged-batch design (Nafazen, Teluzen, Namisun, Tupidra) beside the GPT/LLaMA family at equal parameter count:
prefill and decode tokens/s through ``InferenceEngine.generate`` (the scheduler, block manager and step function a
user gets), random weights, a few layer sizes that resemble real models; plus device-timed runs of the design's own
attention and expert kernels against the measured roofline, next to the GPT family's like kernels.
``bench.py --arch-compare nafazen|teluzen|namisun|tupidra`` prints the result as one JSON line.  Tupidra is also set beside
Namisun (the other parallel-layout design with state slots) of equal width and depth, with both designs' like kernels.

Reference: the reference's serving benchmark is ``llmctl bench e2e`` (reference llmctl/cli/commands/bench.py:98-160)."""
from __future__ import annotations

import json
import time
from pathlib import Path
from typing import Any, Dict, List

import torch

SIZES: Dict[str, Dict[str, Any]] = {
    # width, heads, latent sizes, feed-forwards; 4 layers: dense, MoE, dense, MoE (the last one reads layer 1's cache)
    "w2048": dict(width=2048, vocab=32000, heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=768, ff=8192,
                  experts=8, top=2, expert_ff=2048, shared_ff=2048, pattern="aDbMaDcM"),
    "w4096": dict(width=4096, vocab=32000, heads=32, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=1536, ff=14336,
                  experts=16, top=2, expert_ff=1792, shared_ff=3584, pattern="aDbMaDcM"),
}


TELUZEN_SIZES: Dict[str, Dict[str, Any]] = {
    # 4 layers: dense, MoE, dense, MoE; windows of 512 tokens + pooled blocks of 16; layers 1 and 3 mix values with layer 1's
    "w1024": dict(width=1024, vocab=32000, heads=8, kv_heads=2, dim=128, vdim=128, rot_dims=64, window=512, pool=16, ff=4096,
                  experts=8, top=2, expert_ff=1024, shared_ff=1024, pattern="DMDM", v_mix="0101", max_positions=8192),
    "w2048": dict(width=2048, vocab=32000, heads=16, kv_heads=4, dim=128, vdim=128, rot_dims=64, window=512, pool=16, ff=8192,
                  experts=8, top=2, expert_ff=2048, shared_ff=2048, pattern="DMDM", v_mix="0101", max_positions=8192),
}


NAMISUN_SIZES: Dict[str, Dict[str, Any]] = {
    # 6 layers: scan, linear attention, differential attention, twice; a mixture of 6 experts + 2 identity experts in every
    # layer.  No loop here: a looped range adds compute without parameters, and the GPT beside it has equal parameters.
    "w1024": dict(width=1024, vocab=32000, pattern="MGAMGA", moe="1", loop=None, heads=8, kv_heads=2, dim=64, vdim=128, rot_dims=64,
                  rot_factor=8.0, gla_heads=8, gla_dim=64, gla_vdim=128, decay_rank=16, inner=2048, state=16, dt_rank=64, conv=4,
                  experts=6, identity=2, top=2, groups=(4, 2), ff=1024, limit=7.0),
    "w2048": dict(width=2048, vocab=32000, pattern="MGAMGA", moe="1", loop=None, heads=16, kv_heads=4, dim=64, vdim=128, rot_dims=64,
                  rot_factor=8.0, gla_heads=16, gla_dim=64, gla_vdim=128, decay_rank=16, inner=4096, state=16, dt_rank=128, conv=4,
                  experts=6, identity=2, top=2, groups=(4, 2), ff=2048, limit=7.0),
    "w4096": dict(width=4096, vocab=32000, pattern="MGAMGA", moe="1", loop=None, heads=32, kv_heads=8, dim=64, vdim=128, rot_dims=64,
                  rot_factor=8.0, gla_heads=32, gla_dim=64, gla_vdim=128, decay_rank=16, inner=8192, state=16, dt_rank=256, conv=4,
                  experts=6, identity=2, top=2, groups=(4, 2), ff=3072, limit=7.0),
}


TUPIDRA_SIZES: Dict[str, Dict[str, Any]] = {
    # 6 layers: scan, latent attention, soft-capped window attention (window 512 + 8 kept tokens), twice; the second latent
    # layer reads the first one's cache; a gated GELU feed-forward beside every mixer; input convolutions of 4 taps
    "w1024": dict(width=1024, vocab=32000, pattern="MLAMcA", ff="1", taps=4, heads=8, kv_heads=2, dim=128, vdim=128, softcap=30.0,
                  window=512, keep_first=8, lat_heads=8, lat_dim=128, rot_dim=64, lat_vdim=128, kv_rank=512, q_rank=384, inner=2048,
                  state=16, dt_rank=64, conv=4, ff_size=4096),
    "w2048": dict(width=2048, vocab=32000, pattern="MLAMcA", ff="1", taps=4, heads=16, kv_heads=4, dim=128, vdim=128, softcap=30.0,
                  window=512, keep_first=8, lat_heads=16, lat_dim=128, rot_dim=64, lat_vdim=128, kv_rank=512, q_rank=768, inner=4096,
                  state=16, dt_rank=128, conv=4, ff_size=8192),
    "w4096": dict(width=4096, vocab=32000, pattern="MLAMcA", ff="1", taps=4, heads=32, kv_heads=8, dim=128, vdim=128, softcap=30.0,
                  window=512, keep_first=8, lat_heads=32, lat_dim=128, rot_dim=64, lat_vdim=128, kv_rank=512, q_rank=1536, inner=8192,
                  state=16, dt_rank=256, conv=4, ff_size=16384),
}


def _peaks() -> Dict[str, float]:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    except Exception:  # noqa: BLE001
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def _gpt_equal(ncfg, params: int):
    """A GPT configuration of the same width, depth, heads and vocabulary whose feed-forward width is chosen so that
    the parameter counts match."""
    from ..models.config import ModelConfig
    L, W = len(ncfg.layers), ncfg.width
    H = next(l.mixer.heads for l in ncfg.layers if hasattr(l.mixer, "heads"))
    hd = W // H
    fixed = 2 * ncfg.vocab_size * W + L * (4 * W * H * hd + 2 * W) + W
    ffn = max(256, int((params - fixed) / (3 * W * L)) // 128 * 128)
    return ModelConfig(name=f"gpt-equal-{W}", layers=L, hidden=W, ffn=ffn, heads=H, head_dim=hd, vocab_size=ncfg.vocab_size,
                       max_position_embeddings=8192)


def _serve(cfg, prompts: List[List[int]], new_tokens: int, block_size: int) -> Dict[str, float]:
    from .engine import InferenceEngine
    total = sum(len(p) for p in prompts) + len(prompts) * (new_tokens + 1)
    blocks = (total + block_size - 1) // block_size + 2 * len(prompts)
    eng = InferenceEngine(cfg, max_batch_size=len(prompts), max_batch_tokens=max(8192, total), device="cuda", kv_block_size=block_size,
                          num_kv_blocks=blocks)
    passes: List[Dict[str, float]] = []
    for rnd in range(4):                   # the first pass warms up (tensor maps, graphs, allocator); median of the other three
        for k in ("prefill_tokens", "decode_tokens", "prefill_time_s", "decode_time_s", "decode_steps"):
            eng.stats[k] = 0 if "time" not in k else 0.0
        torch.cuda.synchronize()
        eng.generate(prompts, max_tokens=new_tokens if rnd else 4, temperature=0.0)
        torch.cuda.synchronize()
        s = eng.stats
        passes.append({"prefill_tok_s": s["prefill_tokens"] / max(s["prefill_time_s"], 1e-9),
                       "decode_tok_s": s["decode_tokens"] / max(s["decode_time_s"], 1e-9),
                       "decode_ms_per_step": 1e3 * s["decode_time_s"] / max(s["decode_steps"], 1)})
    out = {k: sorted(r[k] for r in passes[1:])[1] for k in passes[0]}
    del eng
    torch.cuda.empty_cache()
    return out


def _time_flushed(fn, iters: int = 5) -> float:
    """Device time of ``fn`` with the L2 flushed (a 256 MB buffer rewritten) before every timed call."""
    junk = torch.empty(64 << 20, dtype=torch.float32, device="cuda")
    for _ in range(2):
        fn()
    total = 0.0
    for _ in range(iters):
        for _ in range(3):              # ~120 us of device work: the host has enqueued fn before the device gets to it
            junk.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters * 1e-3


def _time(fn, iters: int = 10) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e-3


def _kernels(size: Dict[str, Any], peaks: Dict[str, float]) -> Dict[str, Any]:
    """The design's own kernels in isolation (bf16): latent attention as prefill (2 x 2048 tokens) and as decode
    (32 sequences at context 4096, cache larger than L2), and the grouped expert GEMM."""
    from ..ops import latent_attention as L
    from ..ops import moe as M
    from ..ops import native
    from ..ops.elementwise import rope_frequencies
    from .ragged import Portion, RaggedBatch
    dev = torch.device("cuda")
    H, dn, dr, R = size["heads"], size["dim"], size["rot_dim"], size["kv_rank"]
    bs, res = 64, {}
    freq, mult = rope_frequencies(dr, 10000.0, None)
    freq = freq.to(dev)
    for name, nseq, ctx, new in (("prefill", 2, 2048, 2048), ("decode", 32, 4096, 1)):
        per = (ctx + bs - 1) // bs
        cache = torch.randn(nseq * per, bs, R + dr, device=dev).to(torch.bfloat16)
        ps = [Portion(i, [0] * new, ctx - new, [], list(range(i * per, (i + 1) * per))) for i in range(nseq)]
        b = RaggedBatch(ps, bs, dev)
        T = b.num_tokens
        ql = torch.randn(T, H, R, device=dev)
        q = torch.randn(T, H * (dn + dr), device=dev).to(torch.bfloat16)
        rows = L.ROWS_PER_TILE_TCGEN05 if new > 1 and L.uses_tcgen05(q.dtype, R, dr, bs, True) else L.rows_per_tile(q.dtype, R, dr, True, H if new == 1 else 32)                     # the tiling and query type the model path takes
        if L.uses_tensor_cores(q.dtype, R, dr):
            ql = ql.to(torch.bfloat16)
        t = _time(lambda: L.latent_attention(ql, q, dn, cache, b.block_tables, b.tiles(rows), b.positions, freq, mult, 0.07,
                                             b.heads_per_tile(H, rows), b.max_context, b.attention_splits(H, rows), rows=rows), 5)
        keys = nseq * (ctx * new - new * (new - 1) // 2)                 # visible (query, key) pairs per head
        flops = 2.0 * H * keys * (2 * R + dr)
        bytes_ = nseq * ctx * (R + dr) * 2 + T * H * (R * ql.element_size() + R * 2)
        res[f"latent_attention_{name}"] = {"ms": t * 1e3, "tflops": flops / t / 1e12, "gbs": bytes_ / t / 1e9,
                                           "frac_of_bf16_peak": flops / t / 1e12 / peaks["bf16_tflops"],
                                           "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"]}
    W, E, top, F = size["width"], size["experts"], size["top"], size["expert_ff"]
    T = 4096
    x = torch.randn(T, W, device=dev)
    wr = torch.randn(E, W, device=dev).to(torch.bfloat16)
    wgu = (torch.randn(E, 2 * F, W, device=dev) / W ** 0.5).to(torch.bfloat16)
    wd = (torch.randn(E, W, F, device=dev) / F ** 0.5).to(torch.bfloat16)
    t = _time(lambda: M.moe_ffn(x, torch.bfloat16, wr, wgu, wd, top, scale_input=True), 5)
    flops = 2.0 * T * top * 3 * F * W
    res["moe_ffn_4096_tokens"] = {"ms": t * 1e3, "tflops": flops / t / 1e12, "frac_of_bf16_peak": flops / t / 1e12 / peaks["bf16_tflops"]}
    res.update(_gpt_kernels(size, peaks))
    res["native_launches"] = native.launch_count
    return res


def _teluzen_kernels(size: Dict[str, Any], peaks: Dict[str, float]) -> Dict[str, Any]:
    """The design's own kernels in isolation (bf16): projection post-processing + cache append, pooled-window attention
    as prefill (2 x 2048 tokens) and as decode (32 sequences at context 4096, L2 flushed before every call), and the
    mixture-of-experts layer on 4096 tokens."""
    from ..ops import moe as M
    from ..ops import native
    from ..ops import window_attention as WA
    from ..ops.elementwise import rope_frequencies
    from .ragged import Portion, RaggedBatch
    dev = torch.device("cuda")
    H, G, d, e, S, P = size["heads"], size["kv_heads"], size["dim"], size["vdim"], size["window"], size["pool"]
    bs, res = 64, {}
    PS = WA.pooled_rows_per_page(bs, P)
    Wc = G * (d + e)
    freq, mult = rope_frequencies(size["rot_dims"], 10000.0, None)
    freq = freq.to(dev)
    temp, talk = torch.ones(H, device=dev), (torch.eye(H, device=dev) + 0.1 * torch.randn(H, H, device=dev))
    for name, nseq, ctx, new in (("prefill", 2, 2048, 2048), ("decode", 32, 4096, 1)):
        per = (ctx + bs - 1) // bs
        cache = torch.randn(nseq * per, bs + PS, Wc, device=dev).to(torch.bfloat16)
        ps = [Portion(i, [0] * new, ctx - new, [], list(range(i * per, (i + 1) * per))) for i in range(nseq)]
        b = RaggedBatch(ps, bs, dev)
        T = b.num_tokens
        q = torch.randn(T, H * d, device=dev)
        tile_tokens = 1 if new == 1 else 16
        t = _time_flushed(lambda: WA.pooled_window_attention(q, cache, b.block_tables, b.tiles(16), tile_tokens, b.positions, temp, talk,
                                                             0.09, H, G, d, e, S, P, bs, torch.bfloat16, max_context=b.max_context))
        pairs = 0                                   # visible (query, key) pairs per head
        for i in range(ctx - new, ctx):
            pairs += min(i + 1, S) + max(i - S + 1, 0) // P
        pairs *= nseq
        flops = 2.0 * H * pairs * (d + e)
        rows = nseq * (min(ctx, S + new - 1) + max(ctx - S, 0) // P)            # cache rows a step has to read at least once
        bytes_ = rows * Wc * 2 + T * H * (d * 4 + e * 2)
        res[f"window_attention_{name}"] = {"ms": t * 1e3, "tflops": flops / t / 1e12, "gbs": bytes_ / t / 1e9,
                                           "frac_of_bf16_peak": flops / t / 1e12 / peaks["bf16_tflops"],
                                           "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"],
                                           "tensor_cores": WA.uses_tensor_cores(torch.bfloat16, H, G, d, e, tile_tokens)}
        if new > 1:
            qkv = torch.randn(T, (H + G) * d + G * e, device=dev).to(torch.bfloat16)
            bias = torch.zeros((H + G) * d + G * e, device=dev, dtype=torch.bfloat16)
            nw_q, nw_k = torch.ones(H * d, device=dev), torch.ones(G * d, device=dev)
            t = _time_flushed(lambda: WA.window_qkv_write(qkv, bias, nw_q, nw_k, H, G, d, e, size["rot_dims"], freq, mult, 1e-5, b.positions,
                                                          b.slots, cache, bs))
            bytes_ = T * (((H + G) * d + G * e) * 2 + H * d * 4 + Wc * 2)
            res["window_qkv_write_prefill"] = {"ms": t * 1e3, "gbs": bytes_ / t / 1e9, "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"]}
    W, E, top, F = size["width"], size["experts"], size["top"], size["expert_ff"]
    T = 4096
    x = torch.randn(T, W, device=dev)
    wr = torch.randn(E, W, device=dev).to(torch.bfloat16)
    wgu = (torch.randn(E, 2 * F, W, device=dev) / W ** 0.5).to(torch.bfloat16)
    wd = (torch.randn(E, W, F, device=dev) / F ** 0.5).to(torch.bfloat16)
    t = _time(lambda: M.moe_ffn(x, torch.bfloat16, wr, wgu, wd, top, scale_input=False, softmax=2), 5)
    flops = 2.0 * T * top * 3 * F * W
    res["moe_ffn_4096_tokens"] = {"ms": t * 1e3, "tflops": flops / t / 1e12, "frac_of_bf16_peak": flops / t / 1e12 / peaks["bf16_tflops"]}
    res.update(_gpt_kernels(size, peaks))
    res["native_launches"] = native.launch_count
    return res


def _namisun_kernels(size: Dict[str, Any], peaks: Dict[str, float]) -> Dict[str, Any]:
    """The design's own kernels in isolation (bf16, L2 flushed before every call): differential attention, the gated
    linear attention scan and the selective scan as prefill (2 x 2048 tokens) and as decode (32 sequences; context 4096
    for the attention), the rotation + cache append, the fused residual + layer norm, and the mixture-of-experts layer
    on 4096 tokens."""
    from ..ops import diff_attention as DA
    from ..ops import elementwise as E
    from ..ops import moe as M
    from ..ops import native
    from ..ops import recurrent as R
    from ..ops.elementwise import rope_frequencies
    from .ragged import Portion, RaggedBatch
    dev = torch.device("cuda")
    bf = torch.bfloat16
    H, G, d, e = size["heads"], size["kv_heads"], size["dim"], size["vdim"]
    gH, gd, ge = size["gla_heads"], size["gla_dim"], size["gla_vdim"]
    C, N, Rk, taps = size["inner"], size["state"], size["dt_rank"], size["conv"]
    W = size["width"]
    bs, res = 64, {}
    Wc = G * (2 * d + e)
    freq, mult = rope_frequencies(size["rot_dims"], 10000.0, {"factor": size["rot_factor"]})
    freq = freq.to(dev)
    for name, nseq, ctx, new in (("prefill", 2, 2048, 2048), ("decode", 32, 4096, 1)):
        per = (ctx + bs - 1) // bs
        cache = torch.randn(nseq * per, bs, Wc, device=dev).to(bf)
        ps = [Portion(i, [0] * new, ctx - new, [], list(range(i * per, (i + 1) * per)), i) for i in range(nseq)]
        b = RaggedBatch(ps, bs, dev)
        T = b.num_tokens
        q = torch.randn(T, H * 2 * d, device=dev)
        gate = torch.randn(T, H, device=dev).to(bf)
        width = DA.tile_width(bf, H, G, d, e, True, new == 1)               # the tiling the model path takes
        tile_tokens = 1 if new == 1 else width
        t = _time_flushed(lambda: DA.diff_attention(q, cache, b.block_tables, b.tiles(width), tile_tokens, b.positions, gate, d ** -0.5, 0.5, 0.7,
                                                    1e-5, H, G, d, e, bs, bf, max_context=b.max_context))
        pairs = nseq * sum(i + 1 for i in range(ctx - new, ctx))                  # visible (query, key) pairs per head
        flops = 2.0 * H * pairs * (2 * d + 2 * e)                                 # two score maps, two weight x value products
        bytes_ = nseq * ctx * Wc * 2 + T * H * (2 * d * 4 + e * 2)
        res[f"diff_attention_{name}"] = {"ms": t * 1e3, "tflops": flops / t / 1e12, "gbs": bytes_ / t / 1e9,
                                         "frac_of_bf16_peak": flops / t / 1e12 / peaks["bf16_tflops"],
                                         "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"],
                                         "tensor_cores": DA.uses_tensor_cores(bf, H, G, d, e, tile_tokens)}
        if new > 1:
            proj = torch.randn(T, H * 2 * d + Wc + H, device=dev).to(bf)
            t = _time_flushed(lambda: DA.rotary_kv_append(proj, 2 * H, 2 * G, d, G * e, size["rot_dims"], freq, mult, b.positions, b.slots, cache))
            bytes_ = T * ((H * 2 * d + Wc) * 2 + H * 2 * d * 4 + Wc * 2)
            res["rotary_kv_append_prefill"] = {"ms": t * 1e3, "gbs": bytes_ / t / 1e9, "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"]}
        # gated linear attention: the scan reads q, k, v, z and writes fp32 outputs; a decode step moves the whole state twice
        nk, nv = gH * gd, gH * ge
        p = torch.randn(T, 2 * nk + nv, device=dev).to(bf)
        z = torch.randn(T, nk, device=dev).to(bf)
        zb = torch.rand(nk, device=dev) * 4
        state = torch.zeros(nseq, gH, gd, ge, device=dev)
        t = _time_flushed(lambda: R.gla_scan(p[:, :nk], p[:, nk:2 * nk], p[:, 2 * nk:], z, zb, b.portions, state, gH, gd, ge, gd ** -0.5, 16.0))
        bytes_ = T * ((3 * nk + nv) * 2 + nv * 4) + 2 * state.numel() * 4
        flops = 4.0 * T * gH * gd * ge
        res[f"gla_scan_{name}"] = {"ms": t * 1e3, "gbs": bytes_ / t / 1e9, "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"],
                                   "fp32_tflops": flops / t / 1e12}
        # selective scan
        xz = torch.randn(T, 2 * C, device=dev).to(bf)
        u = torch.randn(T, C, device=dev).to(bf)
        bc = torch.randn(T, Rk + 2 * N, device=dev).to(bf)
        dtp = torch.randn(T, C, device=dev).to(bf)
        dtb, A, D = torch.randn(C, device=dev) - 1.0, -torch.exp(torch.randn(C, N, device=dev)), torch.randn(C, device=dev)
        sst, cst = torch.zeros(nseq, C, N, device=dev), torch.zeros(nseq, taps - 1, C, device=dev)
        t = _time_flushed(lambda: R.selective_scan(u, bc, Rk, Rk + N, dtp, dtb, A, D, xz[:, C:], xz[:, :C], b.portions, sst, cst))
        bytes_ = T * (4 * C * 2 + 2 * N * 2) + 2 * sst.numel() * 4
        res[f"selective_scan_{name}"] = {"ms": t * 1e3, "gbs": bytes_ / t / 1e9, "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"],
                                         "exp_per_s_e12": T * C * N / t / 1e12}
        if new > 1:
            cw, cb = torch.randn(C, taps, device=dev), torch.randn(C, device=dev)
            t = _time_flushed(lambda: R.causal_conv_silu(xz[:, :C], cw, cb, b.portions, b.seq_rows, cst))
            bytes_ = T * C * 4
            res["causal_conv_prefill"] = {"ms": t * 1e3, "gbs": bytes_ / t / 1e9, "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"]}
            x = torch.randn(T, W, device=dev)
            a, f = torch.randn(T, W, device=dev).to(bf), torch.randn(T, W, device=dev)
            w1, b1 = torch.ones(W, device=dev), torch.zeros(W, device=dev)
            t = _time_flushed(lambda: E.parallel_residual(a, f, x, 0.5, 1e-5, bf, w1, b1, want_fp32=True))
            bytes_ = T * W * (2 + 4 + 4 + 4 + 2 + 4)
            res["parallel_residual_norm_prefill"] = {"ms": t * 1e3, "gbs": bytes_ / t / 1e9, "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"]}
    E_, ident, top, F = size["experts"], size["identity"], size["top"], size["ff"]
    T = 4096
    x = torch.randn(T, W, device=dev)
    wr = torch.randn(E_ + ident, W, device=dev).to(bf)
    corr = torch.randn(E_ + ident, device=dev) * 0.01
    wgu = (torch.randn(E_, 2 * F, W, device=dev) / W ** 0.5).to(bf)
    wd = (torch.randn(E_, W, F, device=dev) / F ** 0.5).to(bf)
    t = _time(lambda: M.moe_ffn(x, bf, wr, wgu, wd, top, scale_input=False, softmax=True, renormalise=True, correction=corr,
                                groups=size["groups"], clamp=(size["limit"], 1.702)), 5)
    flops = 2.0 * T * top * 3 * F * W * E_ / (E_ + ident)          # about ident / (E + ident) of the choices are identity experts
    res["moe_ffn_4096_tokens"] = {"ms": t * 1e3, "tflops": flops / t / 1e12, "frac_of_bf16_peak": flops / t / 1e12 / peaks["bf16_tflops"]}
    gsize = dict(size, expert_ff=F)
    res.update(_gpt_kernels(gsize, peaks))
    res["native_launches"] = native.launch_count
    return res


def _tupidra_kernels(size: Dict[str, Any], peaks: Dict[str, float]) -> Dict[str, Any]:
    """The design's own kernels in isolation (bf16, L2 flushed before every call), each next to Namisun's like kernel at the
    same token counts: soft-capped window attention against differential attention (prefill 2 x 2048 tokens; decode 32
    sequences at context 4096), bias + value norm + append against rotation + append, residual + statistics and norm +
    input convolution against the fused residual + layer norm, latent attention with sinks (Nafazen's kernels), the gated
    GELU, and the selective scan both designs share."""
    from ..ops import canon as C
    from ..ops import diff_attention as DA
    from ..ops import elementwise as E
    from ..ops import latent_attention as L
    from ..ops import native
    from ..ops import recurrent as R
    from ..ops import softcap_attention as SA
    from ..ops.elementwise import rope_frequencies
    from .ragged import Portion, RaggedBatch
    dev = torch.device("cuda")
    bf = torch.bfloat16
    H, G, d, e = size["heads"], size["kv_heads"], size["dim"], size["vdim"]
    window, keep, cap = size["window"], size["keep_first"], size["softcap"]
    LH, dn, dr, Rk = size["lat_heads"], size["lat_dim"], size["rot_dim"], size["kv_rank"]
    Cn, N, Rdt, taps = size["inner"], size["state"], size["dt_rank"], size["conv"]
    W, ctaps = size["width"], size["taps"]
    bs, res = 64, {}
    Wc = G * (d + e)
    slopes, sinks = SA.distance_slopes(H).to(dev), torch.zeros(H, device=dev)
    freq, mult = rope_frequencies(dr, 10000.0, {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0})
    freq = freq.to(dev)
    # Namisun's differential attention at equal heads and key / value bytes per token: two maps of d / 2
    nd, nWc = d // 2, G * (d + e)
    nfreq, nmult = rope_frequencies(nd, 10000.0, {"factor": 8.0})
    for name, nseq, ctx, new in (("prefill", 2, 2048, 2048), ("decode", 32, 4096, 1)):
        per = (ctx + bs - 1) // bs
        cache = torch.randn(nseq * per, bs, Wc, device=dev).to(bf)
        ps = [Portion(i, [0] * new, ctx - new, [], list(range(i * per, (i + 1) * per)), i) for i in range(nseq)]
        b = RaggedBatch(ps, bs, dev)
        T = b.num_tokens
        q = torch.randn(T, H * d, device=dev)
        gate = torch.randn(T, H * e, device=dev).to(bf)
        width = SA.tile_width(bf, H, G, d, e, True, new == 1)
        tile_tokens = 1 if new == 1 else width
        t = _time_flushed(lambda: SA.softcap_window_attention(q, cache, b.block_tables, b.tiles(width), tile_tokens, b.positions, gate, slopes,
                                                              sinks, d ** -0.5, cap, window, keep, H, G, d, e, bs, bf, max_context=b.max_context))
        seen = lambda i: min(i + 1, window) + max(min(keep, i + 1 - window), 0)
        pairs = nseq * sum(seen(i) for i in range(ctx - new, ctx))                 # visible (query, key) pairs per head
        flops = 2.0 * H * pairs * (d + e)
        read_keys = nseq * (min(ctx, window + keep + (new - 1)))                    # cache rows a step must read
        bytes_ = read_keys * Wc * 2 + T * H * (d * 4 + 2 * e * 2)
        res[f"softcap_window_attention_{name}"] = {"ms": t * 1e3, "tflops": flops / t / 1e12, "gbs": bytes_ / t / 1e9,
                                                   "frac_of_bf16_peak": flops / t / 1e12 / peaks["bf16_tflops"],
                                                   "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"],
                                                   "tensor_cores": SA.uses_tensor_cores(bf, H, G, d, e, tile_tokens)}
        # Namisun: differential attention, full causal context
        nq = torch.randn(T, H * 2 * nd, device=dev)
        ngate = torch.randn(T, H, device=dev).to(bf)
        nwidth = DA.tile_width(bf, H, G, nd, e, True, new == 1)
        ntile = 1 if new == 1 else nwidth
        t = _time_flushed(lambda: DA.diff_attention(nq, cache, b.block_tables, b.tiles(nwidth), ntile, b.positions, ngate, nd ** -0.5, 0.5, 0.7,
                                                    1e-5, H, G, nd, e, bs, bf, max_context=b.max_context))
        npairs = nseq * sum(i + 1 for i in range(ctx - new, ctx))
        nflops = 2.0 * H * npairs * (2 * nd + 2 * e)
        nbytes = nseq * ctx * nWc * 2 + T * H * (2 * nd * 4 + e * 2)
        res[f"namisun_diff_attention_{name}"] = {"ms": t * 1e3, "tflops": nflops / t / 1e12, "gbs": nbytes / t / 1e9,
                                                 "frac_of_bf16_peak": nflops / t / 1e12 / peaks["bf16_tflops"],
                                                 "frac_of_hbm": nbytes / t / 1e9 / peaks["hbm_gbs"]}
        # latent attention with sinks
        lcache = torch.randn(nseq * per, bs, Rk + dr, device=dev).to(bf)
        ql = torch.randn(T, LH, Rk, device=dev)
        lq = torch.randn(T, LH * (dn + dr), device=dev).to(bf)
        rows = L.ROWS_PER_TILE_TCGEN05 if new > 1 and L.uses_tcgen05(bf, Rk, dr, bs, True) else L.rows_per_tile(bf, Rk, dr, True, LH if new == 1 else 32)
        if L.uses_tensor_cores(bf, Rk, dr):
            ql = ql.to(bf)
        lsinks = torch.randn(LH, device=dev)
        for label, sk in (("latent_attention_sinks", lsinks), ("nafazen_latent_attention", None)):
            t = _time_flushed(lambda: L.latent_attention(ql, lq, dn, lcache, b.block_tables, b.tiles(rows), b.positions, freq, mult, 0.07,
                                                         b.heads_per_tile(LH, rows), b.max_context, b.attention_splits(LH, rows), rows=rows, sinks=sk))
            keys = nseq * (ctx * new - new * (new - 1) // 2)
            flops = 2.0 * LH * keys * (2 * Rk + dr)
            bytes_ = nseq * ctx * (Rk + dr) * 2 + T * LH * (Rk * ql.element_size() + Rk * 2)
            res[f"{label}_{name}"] = {"ms": t * 1e3, "tflops": flops / t / 1e12, "gbs": bytes_ / t / 1e9,
                                      "frac_of_bf16_peak": flops / t / 1e12 / peaks["bf16_tflops"], "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"]}
        # selective scan (shared with Namisun)
        xz = torch.randn(T, 2 * Cn, device=dev).to(bf)
        u = torch.randn(T, Cn, device=dev).to(bf)
        bc = torch.randn(T, Rdt + 2 * N, device=dev).to(bf)
        dtp = torch.randn(T, Cn, device=dev).to(bf)
        dtb, A, D = torch.randn(Cn, device=dev) - 1.0, -torch.exp(torch.randn(Cn, N, device=dev)), torch.randn(Cn, device=dev)
        sst, cst = torch.zeros(nseq, Cn, N, device=dev), torch.zeros(nseq, taps - 1, Cn, device=dev)
        t = _time_flushed(lambda: R.selective_scan(u, bc, Rdt, Rdt + N, dtp, dtb, A, D, xz[:, Cn:], xz[:, :Cn], b.portions, sst, cst))
        bytes_ = T * (4 * Cn * 2 + 2 * N * 2) + 2 * sst.numel() * 4
        res[f"selective_scan_{name}"] = {"ms": t * 1e3, "gbs": bytes_ / t / 1e9, "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"]}
        # the layer's glue: residual + statistics, norm + input convolution for both sublayers; Namisun: residual + layer norm
        x = torch.randn(T, W, device=dev)
        a, f = torch.randn(T, W, device=dev).to(bf), torch.randn(T, W, device=dev).to(bf)
        nw = [torch.ones(W, device=dev), torch.ones(W, device=dev)]
        cw = [torch.randn(W, ctaps, device=dev), torch.randn(W, ctaps, device=dev)]
        cstate = torch.zeros(nseq, ctaps - 1, W, device=dev)
        r = C.residual_rms(None, None, x, 1e-6)
        t1 = _time_flushed(lambda: C.residual_rms(a, f, x, 1e-6))
        t2 = _time_flushed(lambda: C.norm_canon(x, r, nw, cw, b.portions, b.seq_rows, cstate, bf))
        bytes_ = T * W * (2 + 2 + 4 + 4) + T * W * (4 + 2 + 2)
        res[f"residual_norm_canon_{name}"] = {"ms": (t1 + t2) * 1e3, "ms_residual": t1 * 1e3, "ms_norm_canon": t2 * 1e3,
                                              "gbs": bytes_ / (t1 + t2) / 1e9, "frac_of_hbm": bytes_ / (t1 + t2) / 1e9 / peaks["hbm_gbs"]}
        if new == 1:        # the model's decode path: one launch for all of it
            t3 = _time_flushed(lambda: C.residual_norm_canon(a, f, x, 1e-6, nw, cw, b.portions, b.seq_rows, cstate, bf, small=True))
            res[f"residual_norm_canon_{name}"].update({"ms_three_launches": (t1 + t2) * 1e3, "ms": t3 * 1e3, "gbs": bytes_ / t3 / 1e9,
                                                       "frac_of_hbm": bytes_ / t3 / 1e9 / peaks["hbm_gbs"]})
        f32, w1, b1 = torch.randn(T, W, device=dev), torch.ones(W, device=dev), torch.zeros(W, device=dev)
        t = _time_flushed(lambda: E.parallel_residual(a, f32, x, 0.5, 1e-5, bf, w1, b1, want_fp32=True))
        bytes_ = T * W * (2 + 4 + 4 + 4 + 2 + 4)
        res[f"namisun_residual_norm_{name}"] = {"ms": t * 1e3, "gbs": bytes_ / t / 1e9, "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"]}
        if new > 1:
            proj = torch.randn(T, H * d + Wc + H * e, device=dev).to(bf)
            bias = torch.randn(H * d + Wc, device=dev)
            t = _time_flushed(lambda: SA.window_kv_append(proj, bias, H, G, d, e, True, 1e-6, b.slots, cache))
            bytes_ = T * ((H * d + Wc) * 2 + H * d * 4 + Wc * 2)
            res["window_kv_append_prefill"] = {"ms": t * 1e3, "gbs": bytes_ / t / 1e9, "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"]}
            nproj = torch.randn(T, H * 2 * nd + nWc + H, device=dev).to(bf)
            t = _time_flushed(lambda: DA.rotary_kv_append(nproj, 2 * H, 2 * G, nd, G * e, nd, nfreq.to(dev), nmult, b.positions, b.slots, cache))
            bytes_ = T * ((H * 2 * nd + nWc) * 2 + H * 2 * nd * 4 + nWc * 2)
            res["namisun_rotary_kv_append_prefill"] = {"ms": t * 1e3, "gbs": bytes_ / t / 1e9, "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"]}
            F = size["ff_size"]
            gu = torch.randn(T, 2 * F, device=dev).to(bf)
            t = _time_flushed(lambda: E.gated_gelu_tanh(gu))
            t_silu = _time_flushed(lambda: E.gated_silu(gu))
            res["gated_gelu_prefill"] = {"ms": t * 1e3, "gbs": T * F * 6 / t / 1e9, "frac_of_hbm": T * F * 6 / t / 1e9 / peaks["hbm_gbs"],
                                         "gated_silu_ms": t_silu * 1e3}
    res.update(_gpt_kernels(dict(size, top=1, expert_ff=size["ff_size"]), peaks))
    res["native_launches"] = native.launch_count
    return res


def _gpt_kernels(size: Dict[str, Any], peaks: Dict[str, float]) -> Dict[str, Any]:
    """The GPT family's like kernels at like sizes: causal flash attention over the same 2 x 2048 tokens, paged decode
    attention over the same 32 contexts of 4096 (head size 128 for both), and the SwiGLU feed-forward's two GEMMs on
    4096 tokens at the width that gives the mixture-of-experts layer's active parameters."""
    from ..ops import functional as ops
    from ..ops import serving as S
    dev = torch.device("cuda")
    H, D, res = size["heads"], 128, {}
    B, n = 2, 2048
    q, k, v = (torch.randn(B, n, H, D, device=dev).to(torch.bfloat16) for _ in range(3))
    t = _time(lambda: ops.attention(q, k, v, causal=True), 5)
    flops = 4.0 * B * H * D * n * (n + 1) / 2
    res["gpt_flash_attention_prefill"] = {"ms": t * 1e3, "tflops": flops / t / 1e12, "frac_of_bf16_peak": flops / t / 1e12 / peaks["bf16_tflops"]}
    nseq, ctx, bs = 32, 4096, 64
    per = ctx // bs
    kc, vc = (torch.randn(nseq * per, bs, H, D, device=dev).to(torch.bfloat16) for _ in range(2))
    tables = torch.arange(nseq * per, dtype=torch.int32, device=dev).view(nseq, per)
    lens = torch.full((nseq,), ctx, dtype=torch.int32, device=dev)
    qd = torch.randn(nseq, H, D, device=dev).to(torch.bfloat16)
    t = _time(lambda: S.paged_attention_decode(qd, kc, vc, tables, lens, ctx), 5)
    bytes_ = 2.0 * nseq * ctx * H * D * 2
    res["gpt_paged_attention_decode"] = {"ms": t * 1e3, "gbs": bytes_ / t / 1e9, "frac_of_hbm": bytes_ / t / 1e9 / peaks["hbm_gbs"]}
    W, T = size["width"], 4096
    F = size["top"] * size["expert_ff"]
    x = torch.randn(T, W, device=dev).to(torch.bfloat16)
    wgu = (torch.randn(2 * F, W, device=dev) / W ** 0.5).to(torch.bfloat16)
    wd = (torch.randn(W, F, device=dev) / F ** 0.5).to(torch.bfloat16)
    t = _time(lambda: ops.linear(ops.swiglu(ops.linear(x, wgu)), wd), 5)
    flops = 2.0 * T * 3 * F * W
    res["gpt_swiglu_ffn_4096_tokens"] = {"ms": t * 1e3, "tflops": flops / t / 1e12, "frac_of_bf16_peak": flops / t / 1e12 / peaks["bf16_tflops"]}
    return res


def run(which: str = "nafazen", sizes: List[str] | None = None, prompt_len: int = 1024, batch: int = 8, new_tokens: int = 64) -> Dict[str, Any]:
    if which == "nafazen":
        from ..models.nafazen import NafazenConfig as Config, example_config
        table, kernels = SIZES, _kernels
    elif which == "teluzen":
        from ..models.teluzen import TeluzenConfig as Config, example_config
        table, kernels = TELUZEN_SIZES, _teluzen_kernels
    elif which == "namisun":
        from ..models.namisun import NamisunConfig as Config, example_config
        table, kernels = NAMISUN_SIZES, _namisun_kernels
    elif which == "tupidra":
        from ..models.tupidra import TupidraConfig as Config, example_config
        table, kernels = TUPIDRA_SIZES, _tupidra_kernels
    else:
        raise ValueError(f"no architecture comparison for {which!r}")
    peaks = _peaks()
    out: Dict[str, Any] = {"metric": "serving_tokens_per_s", "design": which, "dtype": "bf16", "data": "synthetic, random weights",
                           "workload": {"prompts": batch, "prompt_len": prompt_len, "new_tokens": new_tokens}, "peaks": peaks, "sizes": {}}
    g = torch.Generator().manual_seed(0)
    for name in sizes or list(table):
        size = table[name]
        ncfg = Config.from_dict(example_config(**size), name=f"{which}-{name}")
        params = ncfg.num_parameters()
        gcfg = _gpt_equal(ncfg, params)
        prompts = [torch.randint(0, 32000, (prompt_len,), generator=g).tolist() for _ in range(batch)]
        t0 = time.time()
        row = {"params": params, "gpt_params": gcfg.num_parameters(), "gpt_ffn": gcfg.ffn,
               which: _serve(ncfg, prompts, new_tokens, 64), "gpt": _serve(gcfg, prompts, new_tokens, 16),
               "kernels": kernels(size, peaks)}
        if which == "tupidra" and name in NAMISUN_SIZES:          # the closest design: parallel layout, scans, state slots
            from ..models.namisun import NamisunConfig, example_config as namisun_example
            ccfg = NamisunConfig.from_dict(namisun_example(**NAMISUN_SIZES[name]), name=f"namisun-{name}")
            row["namisun_params"] = ccfg.num_parameters()
            row["namisun"] = _serve(ccfg, prompts, new_tokens, 64)
        row["seconds"] = round(time.time() - t0, 1)
        out["sizes"][name] = row
    return out
