"""Namisun's CUDA kernels against the CPU restatements of the same ops and the engine on a GPU against the plain oracle
(``namisun_oracle.py``), in fp32 (tight) and bf16 (rounding-sized)."""
import pytest
import torch

import namisun_oracle as oracle
from test_namisun_cpu import CONFIGS, make_engine, paged, ref_logits, run_cut, small_cfg

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("W", [12, 200, 1000, 5000])
def test_layer_norm_kernels(cuda_device, W):
    from llmctl_b200.ops import elementwise as E
    torch.manual_seed(0)
    x, a, f = torch.randn(9, W) + 2.0, torch.randn(9, W), torch.randn(9, W)
    w, b, add = torch.rand(W) + 0.5, torch.randn(W), torch.randn(W)
    rows = torch.tensor([7, 0, 3])
    for dt in (torch.float32, torch.bfloat16):
        xc, xg = x.clone(), x.clone().to(cuda_device)
        hc, hc32 = E.layernorm_rows(xc, None, w, b, 1e-5, dt, add=add, want_fp32=True)
        hg, hg32 = E.layernorm_rows(xg, None, w.to(cuda_device), b.to(cuda_device), 1e-5, dt, add=add.to(cuda_device), want_fp32=True)
        assert torch.allclose(xg.cpu(), xc, atol=1e-6) and torch.allclose(hg32.cpu(), hc32, atol=2e-5)
        assert hg.dtype == dt and torch.allclose(hg.float().cpu(), hc.float(), atol=2e-5 if dt == torch.float32 else 4e-2)
        sel = E.layernorm_rows(xg, rows.to(cuda_device), w.to(cuda_device), b.to(cuda_device), 1e-5, torch.float32)
        assert torch.allclose(sel.cpu(), E.layernorm_rows(xc, rows, w, b, 1e-5, torch.float32), atol=2e-5)
        ag = a.to(dt).to(cuda_device)
        hc2 = E.parallel_residual(a.to(dt), f, xc, 0.3, 1e-5, torch.float32, w, b, add=add)
        hg2 = E.parallel_residual(ag, f.to(cuda_device), xg, 0.3, 1e-5, torch.float32, w.to(cuda_device), b.to(cuda_device), add=add.to(cuda_device))
        assert torch.allclose(xg.cpu(), xc, atol=1e-5) and torch.allclose(hg2.cpu(), hc2, atol=3e-5)
        assert E.parallel_residual(ag, None, xg, 1.5, 1e-5, dt) is None
        E.parallel_residual(a.to(dt), None, xc, 1.5, 1e-5, dt)
        assert torch.allclose(xg.cpu(), xc, atol=1e-5)


@pytest.mark.parametrize("experts,identity,top,groups,W,Ff", [(6, 2, 2, (4, 2), 16, 24), (4, 4, 3, (2, 1), 40, 8), (3, 0, 1, None, 12, 10),
                                                              (16, 0, 4, (4, 2), 64, 32)])
def test_mixture_kernels(cuda_device, experts, identity, top, groups, W, Ff):
    from llmctl_b200.ops import moe as M
    torch.manual_seed(4)
    T, n = 150, experts + identity
    x = torch.randn(T, W)
    router, corr = torch.randn(n, W) * 2, torch.randn(n) * 0.3 - 0.2
    gu, dn = torch.randn(experts, 2 * Ff, W), torch.randn(experts, W, Ff) / 3
    ic, wc, _, cc = M.route(x, router, top, softmax=True, renormalise=True, correction=corr, groups=groups)
    ig, wg, _, cg = M.route(x.to(cuda_device), router.to(cuda_device), top, softmax=True, renormalise=True, correction=corr.to(cuda_device), groups=groups)
    assert torch.equal(ig.cpu().sort(-1).values, ic.sort(-1).values) and cg.cpu().tolist() == cc.tolist()
    assert torch.allclose(torch.zeros(T, n).scatter_(1, ig.cpu().long(), wg.cpu()), torch.zeros(T, n).scatter_(1, ic.long(), wc), atol=1e-6)
    want = M.moe_ffn(x, torch.float32, router, gu, dn, top, scale_input=False, softmax=True, renormalise=True, correction=corr, groups=groups,
                     clamp=(0.8, 1.702))
    got = M.moe_ffn(x.to(cuda_device), torch.float32, router.to(cuda_device), gu.to(cuda_device), dn.to(cuda_device), top, scale_input=False,
                    softmax=True, renormalise=True, correction=corr.to(cuda_device), groups=groups, clamp=(0.8, 1.702))
    assert torch.allclose(got.cpu(), want, atol=5e-5)
    gotb = M.moe_ffn(x.to(cuda_device), torch.bfloat16, router.to(cuda_device), gu.to(cuda_device).bfloat16(), dn.to(cuda_device).bfloat16(), top,
                     scale_input=False, softmax=True, renormalise=True, correction=corr.to(cuda_device), groups=groups, clamp=(0.8, 1.702))
    assert (gotb.cpu() - want).abs().max() < 0.05 * want.abs().max() + 0.05


@pytest.mark.parametrize("H,G,d,e,n,far,bs", [(4, 2, 8, 12, 45, 3, 16), (2, 2, 6, 5, 133, 15, 16), (3, 1, 4, 7, 64, 0, 64), (6, 3, 10, 34, 19, 8, 8),
                                              (8, 2, 32, 72, 300, 63, 64), (4, 1, 128, 256, 70, 64, 64), (16, 1, 16, 130, 40, 7, 16),
                                              (4, 4, 16, 8, 259, 127, 16), (6, 2, 64, 128, 257, 128, 64), (32, 2, 32, 40, 130, 31, 8), (2, 1, 8, 300, 40, 5, 16)])
def test_differential_attention_kernels(cuda_device, H, G, d, e, n, far, bs):
    """Prompt tiles, single-token tiles with several heads per CTA, and key slices, against the oracle; a far key
    dominates the first map of the last query."""
    from llmctl_b200.ops import diff_attention as DA
    torch.manual_seed(5)
    q, k, v, gate = torch.randn(n, H, 2, d), torch.randn(n, G, 2, d), torch.randn(n, G, e), torch.randn(n, H)
    k[far, :, 0] = 3.0 * q[n - 1, ::H // G, 0]
    lam, diff, scale, eps = 0.55, 0.3, d ** -0.5, 1e-5
    want = oracle.differential_attention(q.double(), k.double(), v.double(), scale, lam, diff, eps, gate.double())
    order = torch.randperm((n + bs - 1) // bs + 2).tolist()
    cache, table = paged(torch.cat([k.reshape(n, -1), v.reshape(n, -1)], -1), order, bs)
    pos = torch.arange(n, dtype=torch.int32, device=cuda_device)
    qg = q.reshape(n, -1).to(cuda_device)
    t16 = torch.tensor([[s, min(16, n - s), 0, 0] for s in range(0, n, 16)], dtype=torch.int32, device=cuda_device)
    t1 = torch.tensor([[s, 1, 0, 0] for s in range(n)], dtype=torch.int32, device=cuda_device)
    t128 = torch.tensor([[s, min(128, n - s), 0, 0] for s in range(0, n, 128)], dtype=torch.int32, device=cuda_device)
    for dt, tol in ((torch.float32, 3e-5), (torch.bfloat16, 6e-2)):
        cg, gg = cache.to(dt).to(cuda_device), gate.to(dt).to(cuda_device)
        cases = [(t16, 16, 1, False), (t1, 1, 1, False), (t16, 16, 3, False), (t1, 1, 4, False), (t1[-3:], 1, 0, False)]
        if DA.uses_tensor_cores(dt, H, G, d, e, 128):
            cases += [(t128, 128, 1, True), (t16, 16, 1, True), (t1, 1, 1, True), (t1, 1, 4, True), (t1[-3:], 1, 0, True)]
        for tiles, width, splits, tc in cases:
            got = DA.diff_attention(qg, cg, table.to(cuda_device), tiles, width, pos, gg, scale, lam, 1.0 - diff, eps, H, G, d, e, bs, dt,
                                    max_context=n, splits=splits, tensor_cores=tc)
            first = int(tiles[0, 0])
            err = (got.float().cpu().view(n, H, e)[first:].double() - want[first:]).abs().max()
            assert err < tol, (dt, width, splits, tc, float(err))
        if dt == torch.bfloat16 and DA.uses_tensor_cores(dt, H, G, d, e, 128):
            # the tensor-core kernel keeps queries and weights as bf16 pairs: it agrees with the fp32 FMA kernel on the
            # same bf16 cache far more closely than bf16 rounding of the output alone would explain away
            a = DA.diff_attention(qg, cg, table.to(cuda_device), t128, 128, pos, gg, scale, lam, 1.0 - diff, eps, H, G, d, e, bs, dt, tensor_cores=True)
            b = DA.diff_attention(qg, cg, table.to(cuda_device), t16, 16, pos, gg, scale, lam, 1.0 - diff, eps, H, G, d, e, bs, dt, tensor_cores=False)
            assert (a.float() - b.float()).abs().max() <= 0.02 and ((a.float() - b.float()).abs() > 1e-6).float().mean() < 0.1


@pytest.mark.parametrize("H,d,e,cuts", [(2, 8, 10, (9, 1, 1, 4)), (1, 3, 1, (2, 2, 2)), (3, 5, 33, (1, 1, 13)), (2, 70, 6, (5, 3)), (2, 130, 64, (40, 2)),
                                        (4, 40, 72, (100, 1, 1))])
def test_gated_linear_attention_kernels(cuda_device, H, d, e, cuts):
    from llmctl_b200.ops import recurrent as R
    torch.manual_seed(6)
    n = sum(cuts)
    q, k, v, z = torch.randn(n, H * d), torch.randn(n, H * d), torch.randn(n, H * e), torch.randn(n, H * d) * 2
    zb, w, gate = torch.rand(H * d) * 4, torch.rand(e) + 0.5, torch.randn(n, H * e)
    a = torch.sigmoid((z + zb).double()).pow(0.25).view(n, H, d)
    want = oracle.gated_linear_recurrence(q.double().view(n, H, d) * d ** -0.5, k.double().view(n, H, d), v.double().view(n, H, e), a)
    wanty = (oracle.unit_rms(want, 1e-5) * w.double()).reshape(n, H * e) * oracle.silu(gate.double())
    state = torch.randn(3, H, d, e, device=cuda_device)
    out, at = [], 0
    for c in cuts:
        sl = slice(at, at + c)
        pt = torch.tensor([[0, c, at, 1]], dtype=torch.int32, device=cuda_device)
        out.append(R.gla_scan(q[sl].to(cuda_device), k[sl].to(cuda_device), v[sl].to(cuda_device), z[sl].to(cuda_device), zb.to(cuda_device), pt,
                              state, H, d, e, d ** -0.5, 4.0))
        at += c
    o = torch.cat(out)
    scale = want.abs().max()
    assert (o.cpu().double().view(n, H, e) - want).abs().max() < 1e-5 * scale + 1e-5
    y = R.gla_output(o, w.to(cuda_device), gate.to(cuda_device), H, e, 1e-5, torch.float32)
    assert torch.allclose(y.cpu().double(), wanty, atol=1e-4)
    yb = R.gla_output(o, w.to(cuda_device), gate.to(cuda_device).bfloat16(), H, e, 1e-5, torch.bfloat16)
    assert (yb.float().cpu().double() - wanty).abs().max() < 0.02 * wanty.abs().max() + 0.02


@pytest.mark.parametrize("C,N,R_,taps,cuts", [(12, 6, 3, 3, (9, 1, 1, 4)), (5, 1, 1, 4, (2, 2, 1, 1, 1)), (40, 17, 2, 2, (1, 1, 13)), (7, 4, 2, 1, (3, 2)),
                                              (160, 20, 12, 4, (200, 1, 1)), (33, 40, 2, 4, (20,)), (64, 70, 4, 3, (9, 3))])
def test_selective_scan_kernels(cuda_device, C, N, R_, taps, cuts):
    from llmctl_b200.ops import recurrent as R
    torch.manual_seed(7)
    n = sum(cuts)
    x, z = torch.randn(n, C), torch.randn(n, C)
    cw, cb = torch.randn(C, taps), torch.randn(C) * 0.1
    A, D, dtb = -torch.exp(torch.randn(C, N) - 1.0), torch.randn(C), torch.randn(C) - 1.0
    u_want = oracle.silu(oracle.causal_conv(x.double(), cw.double(), cb.double()))
    bc, dtp = torch.randn(n, R_ + 2 * N), torch.randn(n, C)
    dt = torch.nn.functional.softplus(dtp.double() + dtb.double())
    want = oracle.selective_recurrence(u_want, dt, A.double(), bc[:, R_:R_ + N].double(), bc[:, R_ + N:].double(), D.double()) * oracle.silu(z.double())
    g = lambda t: t.to(cuda_device)    # noqa: E731
    state, conv_state = torch.randn(2, C, N, device=cuda_device), torch.randn(2, taps - 1, C, device=cuda_device)
    out, at = [], 0
    seq_rows = torch.zeros(n, dtype=torch.int32, device=cuda_device)
    xz = g(torch.cat([x, z], -1))                 # x and z as strided views of one projection, as the mixer passes them
    for c in cuts:
        sl = slice(at, at + c)
        pt = torch.tensor([[0, c, at, 1]], dtype=torch.int32, device=cuda_device)
        u = R.causal_conv_silu(xz[sl, :C], g(cw), g(cb), pt, seq_rows[sl], conv_state)
        assert torch.allclose(u.cpu().double(), u_want[sl], atol=2e-5)
        out.append(R.selective_scan(u, g(bc[sl]), R_, R_ + N, g(dtp[sl]), g(dtb), g(A), g(D), xz[sl, C:], xz[sl, :C], pt, state, conv_state))
        at += c
    assert (torch.cat(out).cpu().double() - want).abs().max() < 1e-5 * want.abs().max() + 2e-5
    if taps > 1:
        assert torch.allclose(conv_state[1].cpu(), torch.cat([torch.zeros(taps - 1, C), x])[-(taps - 1):])


@pytest.mark.parametrize("N", [17, 40])
def test_selective_scan_many_portions(cuda_device, N):
    """Enough portions to fill the GPU: the scan takes its 4-lanes-per-channel layout for any state count; every portion
    against the oracle, each in its own slot."""
    from llmctl_b200.ops import recurrent as R
    torch.manual_seed(9)
    C, R_, taps, nport, n = 320, 3, 3, 30, 5
    T = nport * n
    x, z, u = torch.randn(T, C), torch.randn(T, C), torch.randn(T, C)
    A, D, dtb = -torch.exp(torch.randn(C, N) - 1.0), torch.randn(C), torch.randn(C) - 1.0
    bc, dtp = torch.randn(T, R_ + 2 * N), torch.randn(T, C)
    dt = torch.nn.functional.softplus(dtp.double() + dtb.double())
    g = lambda t: t.to(cuda_device)    # noqa: E731
    state, conv_state = torch.randn(nport, C, N, device=cuda_device), torch.randn(nport, taps - 1, C, device=cuda_device)
    pt = torch.tensor([[i * n, n, 0, nport - 1 - i] for i in range(nport)], dtype=torch.int32, device=cuda_device)
    got = R.selective_scan(g(u), g(bc), R_, R_ + N, g(dtp), g(dtb), g(A), g(D), g(z), g(x), pt, state, conv_state).cpu().double()
    for i in range(nport):
        sl = slice(i * n, (i + 1) * n)
        want = oracle.selective_recurrence(u[sl].double(), dt[sl], A.double(), bc[sl, R_:R_ + N].double(), bc[sl, R_ + N:].double(), D.double())
        want = want * oracle.silu(z[sl].double())
        assert (got[sl] - want).abs().max() < 1e-5 * want.abs().max() + 2e-5, f"portion {i}"
        assert torch.allclose(conv_state[nport - 1 - i].cpu(), x[sl][-(taps - 1):])


# ---- the engine on a GPU ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_engine_fp32_against_oracle(cuda_device, name):
    cfg = small_cfg(**CONFIGS[name])
    w = oracle.random_weights(cfg, seed=11, slow_decay=True)
    torch.manual_seed(12)
    toks = torch.randint(0, cfg["vocab"], (75,)).tolist()
    want, layers = oracle.forward(cfg, w, toks)
    eng = make_engine(cfg, w, device="cuda", blocks=32)
    assert eng.kv.allocate(1, len(toks))
    trace = []
    got = eng.forward_portions([eng.portion(1, toks, 0, list(range(len(toks))))], layer_trace=trace)
    for r, (a, b) in enumerate(zip(trace, layers)):
        assert torch.allclose(a.cpu().double(), b, atol=3e-4), f"layer run {r}"
    assert torch.allclose(got.cpu().float(), want.float(), atol=3e-4)
    for cuts in ([30] + [1] * 45, [2] * 37 + [1], [3, 2, 2, 7, 1, 16, 8, 2, 9, 25], [8] * 9 + [3]):
        e2 = make_engine(cfg, w, device="cuda", blocks=32)
        assert torch.allclose(run_cut(e2, 1, toks, cuts), want.float(), atol=3e-4), f"cuts {cuts}"


def test_engine_bf16_odd_vocabulary_and_mixed_batches(cuda_device):
    """bf16 end to end stays within rounding of the oracle on the same (bf16-rounded) weights; how a prompt is cut and
    what else is in the batch changes the logits by rounding only.  The vocabulary is not a multiple of 8."""
    cfg = small_cfg(vocab=77, width=64, inner=64, ff=32, moe="0000")       # no routers: bf16 noise cannot flip a choice
    w = {k: v.bfloat16().float() for k, v in oracle.random_weights(cfg, seed=13).items()}
    torch.manual_seed(14)
    seqs = {1: torch.randint(0, 77, (61,)).tolist(), 2: torch.randint(0, 77, (9,)).tolist(), 3: torch.randint(0, 77, (30,)).tolist()}
    want = {i: ref_logits(cfg, w, t) for i, t in seqs.items()}
    eng = make_engine(cfg, {k: v.bfloat16() for k, v in w.items()}, dt=torch.bfloat16, device="cuda", blocks=32)
    plan = [[(1, 20), (2, 3)], [(1, 1), (3, 29), (2, 1)], [(2, 5), (1, 40), (3, 1)]]
    at, got = {i: 0 for i in seqs}, {i: [] for i in seqs}
    for step in plan:
        portions = []
        for i, c in step:
            assert eng.kv.allocate(i, at[i] + c)
            portions.append(eng.portion(i, seqs[i][at[i]:at[i] + c], at[i], list(range(c))))
        lg = eng.forward_portions(portions).float().cpu()
        o = 0
        for i, c in step:
            got[i].append(lg[o:o + c])
            o, at[i] = o + c, at[i] + c
    for i in seqs:
        g = torch.cat(got[i])
        rel = (g - want[i]).pow(2).mean().sqrt() / want[i].pow(2).mean().sqrt()
        assert rel < 0.03, f"sequence {i}: {float(rel)}"


def test_slot_reuse_and_graph_replayed_decoding(cuda_device):
    """Greedy generation through scheduler + engine with decode steps replayed as a CUDA graph equals the oracle's; the
    requests outnumber the seats, so pages and state slots are handed out again while the graph's buffers stay put."""
    cfg = small_cfg()
    w = oracle.random_weights(cfg, seed=71, slow_decay=True)
    torch.manual_seed(72)
    prompts = [torch.randint(0, 80, (n,)).tolist() for n in (11, 3, 19, 7, 26)]
    want = [oracle.greedy(cfg, w, p, 12) for p in prompts]
    for graphs in (False, True):
        eng = make_engine(cfg, w, device="cuda", blocks=24, max_batch=2, graphs=graphs)
        assert eng.generate(prompts, max_tokens=12, temperature=0.0) == want, f"graphs={graphs}"
        assert eng.kv.free_state_slots == 2 and eng.kv.free_blocks == 24
