"""Namisun through the framework (op table, ragged batches, block manager with state slots, scheduler, engine) against
the plain oracle in ``namisun_oracle.py``, on small random configurations.  These run on the CPU implementations of the
ops; ``test_namisun_gpu.py`` repeats the kernel-level and end-to-end comparisons on the CUDA kernels."""
import copy
import io
import json

import pytest
import torch

import namisun_oracle as oracle

F32 = 3e-4      # fp32 end to end against float64: rounding only


def make_engine(cfg, weights, dt=torch.float32, device="cpu", blocks=24, bs=8, max_batch=4, graphs=False):
    from llmctl_b200.serve.engine import InferenceEngine
    eng = InferenceEngine(copy.deepcopy(cfg), max_batch_size=max_batch, max_batch_tokens=blocks * bs, device=device,
                          kv_block_size=bs, num_kv_blocks=blocks, dtype=dt, kv_watermark=0.0, cuda_graphs=graphs)
    eng.model.load_state(weights)
    return eng


def small_cfg(**kw):
    from llmctl_b200.models.namisun import example_config
    return example_config(**kw)


def ref_logits(cfg, w, toks):
    return oracle.forward(cfg, w, toks)[0].float()


def run_cut(eng, sid, toks, cuts, want_all=True):
    """Feed ``toks`` in portions of the given sizes; returns logits of every position."""
    out, at = [], 0
    for c in cuts:
        assert eng.kv.allocate(sid, at + c)
        out.append(eng.forward_portions([eng.portion(sid, toks[at:at + c], at, list(range(c)))]))
        at += c
    assert at == len(toks)
    return torch.cat(out).float().cpu()




# ---- mechanisms alone ------------------------------------------------------------------------------------------
def test_layer_norm_and_parallel_residual():
    from llmctl_b200.ops import elementwise as E
    torch.manual_seed(0)
    x, a, f = torch.randn(5, 12) + 3.0, torch.randn(5, 12), torch.randn(5, 12)
    w, b, add = torch.rand(12) + 0.5, torch.randn(12), torch.randn(12)
    want = oracle.layer_norm(x.double(), w.double(), b.double(), 1e-3)
    assert torch.allclose(E.layernorm_rows(x.clone(), None, w, b, 1e-3, torch.float32).double(), want, atol=1e-6)
    assert torch.allclose(E.layernorm_rows(x.clone(), torch.tensor([3, 0]), w, b, 1e-3, torch.float32).double(), want[[3, 0]], atol=1e-6)
    # a per-pass vector joins the stream (in place) before the norm
    x2 = x.clone()
    h, h32 = E.layernorm_rows(x2, None, w, b, 1e-3, torch.bfloat16, add=add, want_fp32=True)
    assert torch.allclose(x2, x + add) and h.dtype == torch.bfloat16 and torch.equal(h, h32.to(torch.bfloat16))
    assert torch.allclose(h32.double(), oracle.layer_norm((x + add).double(), w.double(), b.double(), 1e-3), atol=1e-5)
    # the variance is about the mean: a constant row norms to the bias
    assert torch.allclose(E.layernorm_rows(torch.full((1, 12), 7.0), None, w, b, 1e-3, torch.float32), b.unsqueeze(0), atol=1e-5)
    # x += m (a + f), then the next pass's vector, then the next layer's norm
    x3 = x.clone()
    h = E.parallel_residual(a, f, x3, 0.4, 1e-3, torch.float32, w, b, add=add)
    new = x.double() + 0.4 * (a.double() + f.double()) + add.double()
    assert torch.allclose(x3.double(), new, atol=1e-6) and torch.allclose(h.double(), oracle.layer_norm(new, w.double(), b.double(), 1e-3), atol=1e-5)
    x4 = x.clone()
    assert E.parallel_residual(a.to(torch.bfloat16), None, x4, 2.0, 1e-3, torch.bfloat16) is None
    assert torch.allclose(x4, x + 2.0 * a.to(torch.bfloat16).float(), atol=1e-6)


def test_linear_position_interpolation_spectrum():
    from llmctl_b200.ops.elementwise import rope_frequencies
    f, m = rope_frequencies(6, 250.0, {"factor": 8.0})
    i = torch.arange(3, dtype=torch.float64)
    assert m == 1.0 and torch.allclose(f.double(), 250.0 ** (-2 * i / 6) / 8.0, rtol=1e-6)


def test_clamped_gate_activation():
    from llmctl_b200.ops.elementwise import gated_clamped
    g = torch.tensor([[-5.0, -0.5, 0.3, 0.9, 2.0, 7.0]])
    u = torch.tensor([[0.5, -0.2, 0.0, 0.7, 1.5, -9.0]])
    out = gated_clamped(torch.cat([g, u], -1), 1.0, 1.702)
    gg, uu = g.clamp(max=1.0), u.clamp(-1.0, 1.0)          # the gate is clamped from above only
    assert torch.allclose(out, gg * torch.sigmoid(1.702 * gg) * (uu + 1.0), atol=1e-6)
    assert out[0, 0] < 0 and out[0, 5] == 0.0                # a very negative gate passes; up <= -limit gives 0


@pytest.mark.parametrize("experts,identity,top,groups", [(6, 2, 2, (4, 2)), (8, 0, 3, (2, 1)), (5, 1, 1, None), (4, 4, 4, (2, 1)), (3, 0, 3, None)])
def test_routing_choice_groups_and_weights(experts, identity, top, groups):
    from llmctl_b200.ops import moe as M
    torch.manual_seed(3)
    T, W = 40, 16
    n = experts + identity
    x = torch.randn(T, W)
    r = {"experts": experts, "identity": identity, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    # corrections that are large against the scores, some negative: choice and weight must not be mixed up, and a
    # masked expert must lose against a negative choice score
    Wt = {"router": torch.randn(n, W).double(), "correction": (torch.randn(n) * 0.5 - 0.4).double()}
    ids, wts, _, counts = M.route(x, Wt["router"].float(), top, softmax=True, renormalise=True, correction=Wt["correction"].float(), groups=groups)
    oi, ow = oracle.route(x.double(), {"p.router": Wt["router"], "p.correction": Wt["correction"]}, "p.", r)
    assert torch.equal(ids.long().sort(-1).values, oi.sort(-1).values)
    got = torch.zeros(T, n, dtype=torch.float64).scatter_(1, ids.long(), wts.double())
    want = torch.zeros(T, n, dtype=torch.float64).scatter_(1, oi, ow)
    assert torch.allclose(got, want, atol=1e-6) and torch.allclose(wts.sum(-1), torch.ones(T), atol=1e-5)
    assert counts.tolist() == torch.bincount(oi.reshape(-1), minlength=n).tolist()
    if groups:      # every choice of a token lies in its kept groups
        size = n // groups[0]
        assert all(len({int(e) // size for e in row}) <= groups[1] for row in ids)


@pytest.mark.parametrize("experts,identity,top,groups", [(6, 2, 2, (4, 2)), (4, 4, 3, (2, 1)), (3, 0, 1, None)])
def test_mixture_with_identity_experts(experts, identity, top, groups):
    from llmctl_b200.ops import moe as M
    torch.manual_seed(4)
    T, W, Ff = 30, 12, 10
    n = experts + identity
    x = torch.randn(T, W)
    m = {"router": {"experts": experts, "identity": identity, "top": top}, "expert": {"ff": Ff, "limit": 0.8}}
    if groups:
        m["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    Wt = {"p.router": torch.randn(n, W) * 2, "p.correction": torch.randn(n) * 0.2}
    for e in range(experts):
        Wt[f"p.e{e}.gate"], Wt[f"p.e{e}.up"], Wt[f"p.e{e}.down"] = torch.randn(Ff, W), torch.randn(Ff, W), torch.randn(W, Ff) / 3
    gu = torch.stack([torch.cat([Wt[f"p.e{e}.gate"], Wt[f"p.e{e}.up"]]) for e in range(experts)])
    dn = torch.stack([Wt[f"p.e{e}.down"] for e in range(experts)])
    y = M.moe_ffn(x, torch.float32, Wt["p.router"], gu, dn, top, scale_input=False, softmax=True, renormalise=True,
                  correction=Wt["p.correction"], groups=groups, clamp=(0.8, 1.702))
    want = oracle.moe(x.double(), {k: v.double() for k, v in Wt.items()}, "p.", m)
    assert torch.allclose(y.double(), want, atol=2e-5)


@pytest.mark.parametrize("H,G,d,e,rot", [(4, 2, 8, 12, 4), (3, 3, 6, 6, 6), (6, 1, 4, 10, 0), (2, 2, 10, 3, 2), (1, 1, 2, 1, 2)])
def test_rotation_and_cache_append(H, G, d, e, rot):
    from llmctl_b200.ops import diff_attention as DA
    from llmctl_b200.ops.elementwise import rope_frequencies
    torch.manual_seed(1)
    T, bs = 7, 4
    Nq, Nk, Nv = H * 2 * d, G * 2 * d, G * e
    proj = torch.randn(T, Nq + Nk + Nv + H)
    f, mult = rope_frequencies(rot, 500.0, {"factor": 4.0}) if rot else (torch.zeros(1), 1.0)
    pos = torch.tensor([0, 1, 2, 40, 41, 999, 5], dtype=torch.int32)
    slots = torch.tensor([0, 1, 2, 9, 10, -1, 7])
    cache = torch.zeros(5, bs, Nk + Nv)
    q = DA.rotary_kv_append(proj, 2 * H, 2 * G, d, Nv, rot, f, mult, pos, slots, cache)
    qo, ko = proj[:, :Nq].double().view(T, H, 2, d), proj[:, Nq:Nq + Nk].double().view(T, G, 2, d)
    if rot:
        qo, ko = oracle.rotate_pairs(qo, pos, rot, 500.0, 4.0), oracle.rotate_pairs(ko, pos, rot, 500.0, 4.0)
    assert torch.allclose(q.double(), qo.reshape(T, Nq), atol=2e-5)
    ok = slots >= 0
    flat = cache.view(-1, Nk + Nv)
    assert torch.allclose(flat[slots[ok], :Nk].double(), ko.reshape(T, Nk)[ok], atol=2e-5)
    assert torch.equal(flat[slots[ok], Nk:], proj[ok, Nq + Nk:Nq + Nk + Nv])
    untouched = torch.ones(5 * bs, dtype=torch.bool)
    untouched[slots[ok]] = False
    assert torch.equal(flat[untouched], torch.zeros_like(flat[untouched]))


def paged(cache_rows, order, bs):
    """Scatter consecutive token rows into pages in the given order -> (cache [pages, bs, Wc], block table)."""
    n, Wc = cache_rows.shape
    pages = (n + bs - 1) // bs
    cache = torch.zeros(max(order[:pages]) + 1, bs, Wc, dtype=cache_rows.dtype)
    for j in range(n):
        cache[order[j // bs], j % bs] = cache_rows[j]
    return cache, torch.tensor([order[:pages]], dtype=torch.int32)


@pytest.mark.parametrize("H,G,d,e,n,far", [(4, 2, 8, 12, 45, 3), (2, 2, 6, 5, 33, 15), (3, 1, 4, 7, 64, 0), (6, 3, 10, 34, 19, 8)])
def test_differential_attention_against_oracle(H, G, d, e, n, far):
    """Both maps, shared values, the difference, the unit-RMS norm, the gate; one far key is made to dominate map 1 of
    the last queries, so that dropping it (a page or tile border, a lost block) cannot hide among the other keys."""
    from llmctl_b200.ops import diff_attention as DA
    torch.manual_seed(5)
    bs = 16
    q = torch.randn(n, H, 2, d)
    k = torch.randn(n, G, 2, d)
    v = torch.randn(n, G, e)
    gate = torch.randn(n, H)
    k[far, :, 0] = 3.0 * q[n - 1, ::H // G, 0]            # key `far` lines up with the last query's first map
    lam, diff, scale, eps = 0.55, 0.3, 0.4, 1e-5
    want = oracle.differential_attention(q.double(), k.double(), v.double(), scale, lam, diff, eps, gate.double())
    cache, table = paged(torch.cat([k.reshape(n, -1), v.reshape(n, -1)], -1), [3, 0, 5, 1, 4], bs)
    pos = torch.arange(n, dtype=torch.int32)
    tiles = torch.tensor([[s, min(16, n - s), 0, 0] for s in range(0, n, 16)], dtype=torch.int32)
    got = DA.diff_attention(q.reshape(n, -1), cache, table, tiles, 16, pos, gate, scale, lam, 1.0 - diff, eps, H, G, d, e, bs, torch.float32)
    assert torch.allclose(got.double().view(n, H, e), want, atol=2e-5)
    # without the far key the last row changes visibly: the test would see a dropped key
    k2 = k.clone()
    k2[far] = 0.0
    other = oracle.differential_attention(q.double(), k2.double(), v.double(), scale, lam, diff, eps, gate.double())
    assert (other[n - 1] - want[n - 1]).abs().max() > 1e-2


@pytest.mark.parametrize("H,d,e,cuts", [(2, 8, 10, (9, 1, 1, 4)), (1, 3, 1, (2, 2, 2)), (3, 5, 33, (1, 1, 13)), (2, 70, 6, (5, 3))])
def test_gated_linear_attention_scan_and_state_slots(H, d, e, cuts):
    """Portions of one sequence through a state slot (with garbage in it at the start) equal the whole recurrence."""
    from llmctl_b200.ops import recurrent as R
    torch.manual_seed(6)
    n = sum(cuts)
    q, k, v, z = torch.randn(n, H * d), torch.randn(n, H * d), torch.randn(n, H * e), torch.randn(n, H * d) * 2
    zb = torch.rand(H * d) * 4
    tau = 4.0
    a = torch.sigmoid((z + zb).double()).pow(1 / tau).view(n, H, d)
    want = oracle.gated_linear_recurrence(q.double().view(n, H, d) * d ** -0.5, k.double().view(n, H, d), v.double().view(n, H, e), a)
    state = torch.randn(3, H, d, e)               # slot 1 is used; what it held must not leak in
    keep0, keep2 = state[0].clone(), state[2].clone()
    out, at = [], 0
    for c in cuts:
        sl = slice(at, at + c)
        out.append(R.gla_scan(q[sl], k[sl], v[sl], z[sl], zb, torch.tensor([[0, c, at, 1]], dtype=torch.int32), state, H, d, e, d ** -0.5, tau))
        at += c
    assert torch.allclose(torch.cat(out).double().view(n, H, e), want, atol=2e-5)
    assert torch.equal(state[0], keep0) and torch.equal(state[2], keep2)
    w, gate = torch.rand(e) + 0.5, torch.randn(n, H * e)
    y = R.gla_output(torch.cat(out), w, gate, H, e, 1e-5, torch.float32)
    wanty = (oracle.unit_rms(want, 1e-5) * w.double()).reshape(n, H * e) * oracle.silu(gate.double())
    assert torch.allclose(y.double(), wanty, atol=2e-5)


@pytest.mark.parametrize("C,N,R_,taps,cuts", [(12, 6, 3, 3, (9, 1, 1, 4)), (5, 1, 1, 4, (2, 2, 1, 1, 1)), (40, 17, 2, 2, (1, 1, 13)), (7, 4, 2, 1, (3, 2))])
def test_selective_scan_with_convolution_and_state_slots(C, N, R_, taps, cuts):
    """The convolution reaches back over portion borders through the stored inputs (portions shorter than the taps
    included); conv + scan over portions equal the whole recurrence."""
    from llmctl_b200.ops import recurrent as R
    torch.manual_seed(7)
    n = sum(cuts)
    x, z = torch.randn(n, C), torch.randn(n, C)
    cw, cb = torch.randn(C, taps), torch.randn(C) * 0.1
    A, D, dtb = -torch.exp(torch.randn(C, N)), torch.randn(C), torch.randn(C)
    u_want = oracle.silu(oracle.causal_conv(x.double(), cw.double(), cb.double()))
    bc, dtp = torch.randn(n, R_ + 2 * N), torch.randn(n, C)
    dt = torch.nn.functional.softplus(dtp.double() + dtb.double())
    want = oracle.selective_recurrence(u_want, dt, A.double(), bc[:, R_:R_ + N].double(), bc[:, R_ + N:].double(), D.double()) * oracle.silu(z.double())
    state, conv_state = torch.randn(2, C, N), torch.randn(2, taps - 1, C)
    out, us, at = [], [], 0
    seq_rows = torch.zeros(n, dtype=torch.int32)
    for c in cuts:
        sl = slice(at, at + c)
        pt = torch.tensor([[0, c, at, 1]], dtype=torch.int32)
        u = R.causal_conv_silu(x[sl], cw, cb, pt, seq_rows[sl], conv_state)
        out.append(R.selective_scan(u, bc[sl], R_, R_ + N, dtp[sl], dtb, A, D, z[sl], x[sl], pt, state, conv_state))
        us.append(u)
        at += c
    assert torch.allclose(torch.cat(us).double(), u_want, atol=2e-5)
    assert torch.allclose(torch.cat(out).double(), want, atol=5e-5)
    if taps > 1:
        tail = torch.cat([torch.zeros(taps - 1, C), x])[-(taps - 1):]
        assert torch.allclose(conv_state[1], tail)


def test_two_portions_of_different_sequences_in_one_call():
    from llmctl_b200.ops import recurrent as R
    torch.manual_seed(8)
    H, d, e = 2, 4, 5
    q, k, v, z = (torch.randn(9, H * d) for _ in range(4))
    v = torch.randn(9, H * e)
    state = torch.zeros(4, H, d, e)
    both = R.gla_scan(q, k, v, z, None, torch.tensor([[0, 5, 0, 3], [5, 4, 0, 0]], dtype=torch.int32), state, H, d, e, 1.0, 2.0)
    s2 = torch.zeros(4, H, d, e)
    a = R.gla_scan(q[:5], k[:5], v[:5], z[:5], None, torch.tensor([[0, 5, 0, 1]], dtype=torch.int32), s2, H, d, e, 1.0, 2.0)
    b = R.gla_scan(q[5:], k[5:], v[5:], z[5:], None, torch.tensor([[0, 4, 0, 2]], dtype=torch.int32), s2, H, d, e, 1.0, 2.0)
    assert torch.allclose(both, torch.cat([a, b]), atol=1e-6)
    assert torch.allclose(state[3], s2[1]) and torch.allclose(state[0], s2[2])


# ---- block manager: state slots -----------------------------------------------------------------------------------
def test_state_slots_follow_the_pages():
    from llmctl_b200.serve.native_host import KVBlockManager
    kv = KVBlockManager(8, 4, 0.0, state_slots=2)
    assert kv.allocate(10, 3) and kv.allocate(11, 5)
    a, b = kv.state_slot(10), kv.state_slot(11)
    assert {a, b} == {0, 1} and kv.free_state_slots == 0
    assert not kv.allocate(12, 1) and kv.state_slot(12) == -1 and kv.free_blocks == 5       # pages left, but no slot
    assert kv.allocate(10, 6) and kv.state_slot(10) == a                                     # growing keeps the slot
    kv.free(10)
    assert kv.free_state_slots == 1 and kv.allocate(12, 1) and kv.state_slot(12) == a        # handed out again
    with pytest.raises(RuntimeError):
        kv.fork(11, 13)                                                                      # a state cannot be shared
    plain = KVBlockManager(4, 4, 0.0)
    assert plain.allocate(1, 2) and plain.state_slot(1) == -1


# ---- whole model ---------------------------------------------------------------------------------------------------
CONFIGS = {
    "default": dict(),
    "no-loop-plain": dict(loop=None, pattern="AGM", moe="111", heads=2, kv_heads=2, rot_dims=0, identity=0, groups=None, top=1, residual_mult=1.0,
                          logit_scale=1.0),
    "loop-at-start-3x": dict(loop=(0, 2, 3), pattern="GAM", moe="010", rot_factor=None, rot_dims=8, conv=1, dt_rank=1, state=1),
    "loop-whole-once": dict(loop=(0, 4, 1), pattern="MMAG", moe="0000", kv_heads=1, heads=3, dim=6, vdim=5, gla_heads=1, gla_dim=3, gla_vdim=3),
    "loop-at-end": dict(loop=(2, 4, 2), pattern="AMGA", moe="1111", experts=4, identity=4, top=4, groups=(2, 1), conv=5, inner=24, state=9,
                        decay_rank=1, width=40),
}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_every_layer_run_against_oracle(name):
    cfg = small_cfg(**CONFIGS[name])
    w = oracle.random_weights(cfg, seed=11)
    torch.manual_seed(12)
    toks = torch.randint(0, cfg["vocab"], (37,)).tolist()
    want, layers = oracle.forward(cfg, w, toks)
    eng = make_engine(cfg, w)
    assert eng.kv.allocate(1, len(toks))
    trace = []
    got = eng.forward_portions([eng.portion(1, toks, 0, list(range(len(toks))))], layer_trace=trace)
    assert len(trace) == len(layers) == len(oracle.layer_runs(cfg))
    for r, (a, b) in enumerate(zip(trace, layers)):
        assert torch.allclose(a.double(), b, atol=F32), f"layer run {r}"
    assert torch.allclose(got.float(), want.float(), atol=F32)
    # the fused residual + next-norm path (no trace) gives the same logits
    eng2 = make_engine(cfg, w)
    assert eng2.kv.allocate(1, len(toks))
    assert torch.allclose(eng2.forward_portions([eng2.portion(1, toks, 0, list(range(len(toks))))]).float(), want.float(), atol=F32)


@pytest.mark.parametrize("name", ["default", "loop-at-end", "loop-at-start-3x"])
def test_prefill_then_token_by_token_and_portions_down_to_two(name):
    cfg = small_cfg(**CONFIGS[name])
    w = oracle.random_weights(cfg, seed=21, slow_decay=True)
    torch.manual_seed(22)
    toks = torch.randint(0, cfg["vocab"], (50,)).tolist()
    want = ref_logits(cfg, w, toks)
    for cuts in ([50], [20] + [1] * 30, [1] * 50, [2] * 25, [3, 2, 2, 7, 1, 16, 8, 2, 9], [8, 8, 8, 8, 8, 8, 2], [7, 9, 17, 15, 2]):
        eng = make_engine(cfg, w)
        assert torch.allclose(run_cut(eng, 1, toks, cuts), want, atol=F32), f"cuts {cuts}"


def test_far_tokens_reach_through_state_and_cache():
    """With slow decays the first token still moves the last logits of a long prompt: losing the state or a page on the
    way (portions cut at page borders and inside pages) would show."""
    cfg = small_cfg(pattern="GMA", moe="000", loop=None)
    w = oracle.random_weights(cfg, seed=31, slow_decay=True)
    torch.manual_seed(32)
    toks = torch.randint(0, cfg["vocab"], (90,)).tolist()
    want = ref_logits(cfg, w, toks)
    other = ref_logits(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert (other[-1] - want[-1]).abs().max() > 30 * F32            # the first token matters at the end
    eng = make_engine(cfg, w, blocks=16)
    assert torch.allclose(run_cut(eng, 1, toks, [8, 16, 1, 7, 31, 1, 1, 25]), want, atol=F32)


def test_unequal_requests_in_one_batch_equal_each_alone():
    cfg = small_cfg()
    w = oracle.random_weights(cfg, seed=41)
    torch.manual_seed(42)
    seqs = {1: torch.randint(0, 80, (29,)).tolist(), 2: torch.randint(0, 80, (5,)).tolist(), 3: torch.randint(0, 80, (17,)).tolist(),
            4: torch.randint(0, 80, (1,)).tolist()}
    want = {i: ref_logits(cfg, w, t) for i, t in seqs.items()}
    # step plan: (sequence, tokens) per step; prompts in portions beside single decoded tokens, sequences skip steps
    plan = [[(1, 9), (2, 2), (4, 1)], [(1, 1), (3, 16)], [(2, 1), (1, 12), (3, 1)], [(2, 2), (1, 7)]]
    eng = make_engine(cfg, w, blocks=16)
    at = {i: 0 for i in seqs}
    got = {i: [] for i in seqs}
    for step in plan:
        portions = []
        for i, c in step:
            assert eng.kv.allocate(i, at[i] + c)
            portions.append(eng.portion(i, seqs[i][at[i]:at[i] + c], at[i], list(range(c))))
        lg = eng.forward_portions(portions).float()
        o = 0
        for i, c in step:
            got[i].append(lg[o:o + c])
            o += c
            at[i] += c
    for i in seqs:
        assert at[i] == len(seqs[i]) and torch.allclose(torch.cat(got[i]), want[i], atol=F32), f"sequence {i}"


def test_pages_and_state_slots_are_used_again():
    """A pool that holds two short requests at a time serves six in turn: every page and both state slots are handed out
    several times, and what the earlier owner left in them (slow decays: states far from zero) must not show."""
    cfg = small_cfg()
    w = oracle.random_weights(cfg, seed=51, slow_decay=True)
    torch.manual_seed(52)
    eng = make_engine(cfg, w, blocks=6, bs=8, max_batch=2)
    assert eng.state_slots == 2
    seqs = [torch.randint(0, 80, (int(n),)).tolist() for n in (20, 24, 9, 17, 24, 3)]
    want = [ref_logits(cfg, w, t) for t in seqs]
    used_slots = []
    for a in range(0, 6, 2):
        ids = (a + 1, a + 2)
        for sid in ids:
            assert eng.kv.allocate(sid, len(seqs[sid - 1]))
            used_slots.append(eng.kv.state_slot(sid))
        # first halves together, second halves together
        halves = {sid: len(seqs[sid - 1]) // 2 for sid in ids}
        l1 = eng.forward_portions([eng.portion(sid, seqs[sid - 1][:halves[sid]], 0, list(range(halves[sid]))) for sid in ids]).float()
        l2 = eng.forward_portions([eng.portion(sid, seqs[sid - 1][halves[sid]:], halves[sid], list(range(len(seqs[sid - 1]) - halves[sid])))
                                   for sid in ids]).float()
        o1 = o2 = 0
        for sid in ids:
            n, hlf = len(seqs[sid - 1]), halves[sid]
            got = torch.cat([l1[o1:o1 + hlf], l2[o2:o2 + n - hlf]])
            o1, o2 = o1 + hlf, o2 + n - hlf
            assert torch.allclose(got, want[sid - 1], atol=F32), f"request {sid}"
            eng.kv.free(sid)
    assert sorted(set(used_slots)) == [0, 1] and len(used_slots) == 6


def test_long_decoding_across_pages():
    cfg = small_cfg(pattern="AGM", moe="101", loop=(0, 3, 2))
    w = oracle.random_weights(cfg, seed=61)
    torch.manual_seed(62)
    toks = torch.randint(0, 80, (70,)).tolist()
    eng = make_engine(cfg, w, blocks=10, bs=8)
    assert torch.allclose(run_cut(eng, 1, toks, [6] + [1] * 64), ref_logits(cfg, w, toks), atol=F32)


def test_greedy_generation_through_scheduler_and_engine():
    cfg = small_cfg()
    w = oracle.random_weights(cfg, seed=71)
    torch.manual_seed(72)
    prompts = [torch.randint(0, 80, (n,)).tolist() for n in (11, 3, 19)]
    eng = make_engine(cfg, w, blocks=20, max_batch=2)              # three requests on two seats: the third waits for a slot
    got = eng.generate(prompts, max_tokens=9, temperature=0.0)
    for p, g in zip(prompts, got):
        assert g == oracle.greedy(cfg, w, p, 9)
    assert eng.kv.free_state_slots == 2 and eng.kv.free_blocks == 20


def test_checkpoint_directory_config_reader_and_trace_replay(tmp_path):
    """config.json + model.safetensors in a directory: the registry picks the design, the decay projection's inner size
    comes from the checkpoint, and the trace replayer feeds a mixed schedule through the engine."""
    from safetensors.torch import save_file
    from llmctl_b200.serve import replay
    cfg = small_cfg(decay_rank=5)
    w = oracle.random_weights(cfg, seed=81, dtype=torch.bfloat16)
    for l in cfg["layers"]:
        l["mixer"].pop("decay_rank", None)                          # a checkpoint's config does not carry it
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in w.items()}, str(tmp_path / "model.safetensors"))
    torch.manual_seed(82)
    a, b = torch.randint(0, 80, (21,)).tolist(), torch.randint(0, 80, (12,)).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:9], "want": [8]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[9:11], "want": []}, {"id": "b", "tokens": b[:11], "want": [0, 10]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[11:], "want": [0]}, {"id": "a", "tokens": a[11:], "want": [9]}], "end": ["a", "b"]}]
    out = io.StringIO()
    rc = replay.run(str(tmp_path), "float32", str(tmp_path / "out"), 128, "cpu", stdin=io.StringIO("\n".join(json.dumps(s) for s in steps)), stdout=out)
    assert rc == 0 and out.getvalue().split() == ["done", "0", "done", "1", "done", "2"]
    import numpy as np
    wf = {k: v.float() for k, v in w.items()}
    full_cfg = small_cfg(decay_rank=5)
    la, lb = ref_logits(full_cfg, wf, a), ref_logits(full_cfg, wf, b)
    V = cfg["vocab"]
    got0 = torch.from_numpy(np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").reshape(-1, V))
    got1 = torch.from_numpy(np.fromfile(tmp_path / "out" / "1.f32", dtype="<f4").reshape(-1, V))
    got2 = torch.from_numpy(np.fromfile(tmp_path / "out" / "2.f32", dtype="<f4").reshape(-1, V))
    assert torch.allclose(got0, la[[8]], atol=F32) and torch.allclose(got1, lb[[0, 10]], atol=F32)
    assert torch.allclose(got2, torch.stack([lb[11], la[20]]), atol=F32)
