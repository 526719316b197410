"""Tupidra through the framework (op table, ragged batches, block manager with state slots, scheduler, engine) against the
plain oracle in ``tupidra_oracle.py``, on small random configurations.  These run on the CPU implementations of the ops;
``test_tupidra_gpu.py`` repeats the kernel-level and end-to-end comparisons on the CUDA kernels."""
import copy
import io
import json

import pytest
import torch

import tupidra_oracle as oracle

F32 = 3e-4      # fp32 end to end against float64: rounding only


def make_engine(cfg, weights, dt=torch.float32, device="cpu", blocks=24, bs=8, max_batch=4, graphs=False):
    from llmctl_b200.serve.engine import InferenceEngine
    eng = InferenceEngine(copy.deepcopy(cfg), max_batch_size=max_batch, max_batch_tokens=blocks * bs, device=device,
                          kv_block_size=bs, num_kv_blocks=blocks, dtype=dt, kv_watermark=0.0, cuda_graphs=graphs)
    eng.model.load_state(weights)
    return eng


def small_cfg(**kw):
    from llmctl_b200.models.tupidra import example_config
    return example_config(**kw)


def ref_logits(cfg, w, toks, layers=None):
    return oracle.forward(cfg, w, toks, layers).float()


def run_cut(eng, sid, toks, cuts):
    """Feed ``toks`` in portions of the given sizes; returns logits of every position."""
    out, at = [], 0
    for c in cuts:
        assert eng.kv.allocate(sid, at + c)
        out.append(eng.forward_portions([eng.portion(sid, toks[at:at + c], at, list(range(c)))]))
        at += c
    assert at == len(toks)
    return torch.cat(out).float().cpu()


def paged(n_tokens, bs, device="cpu", start=0, shuffle=True, seed=0):
    """A one-sequence ragged batch over shuffled pages: (batch, table)."""
    from llmctl_b200.serve.ragged import Portion, RaggedBatch
    nb = (start + n_tokens + bs - 1) // bs
    g = torch.Generator().manual_seed(seed)
    table = (torch.randperm(nb + 3, generator=g)[:nb] if shuffle else torch.arange(nb)).tolist()
    p = Portion(1, [0] * n_tokens, start, list(range(n_tokens)), table, 0)
    return RaggedBatch([p], bs, torch.device(device)), table


CONFIGS = {
    "default": dict(),
    "one_kv_head_window_1": dict(pattern="AAM", ff="101", kv_heads=1, window=1, keep_first=0, taps=2, softcap=2.0),
    "own_kv_heads_long_window": dict(pattern="ALA", ff="111", heads=3, kv_heads=3, dim=5, vdim=7, window=500, keep_first=5, taps=1),
    "no_yarn_no_ff": dict(pattern="LcMc", ff="0000", yarn=False, lat_heads=1, lat_dim=3, rot_dim=2, lat_vdim=1, kv_rank=5, q_rank=1, taps=4),
    "scan_edges": dict(pattern="MM", ff="10", inner=7, state=1, dt_rank=1, conv=1, taps=5, width=20),
    "keep_more_than_window": dict(pattern="AL", ff="11", window=3, keep_first=6, heads=6, kv_heads=2, dim=4, vdim=2, rot_dim=8, lat_dim=2),
}


# ---- mechanisms alone ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("taps,cuts", [(4, [9]), (4, [1, 1, 1, 2, 4]), (3, [2, 1, 6]), (1, [4, 5]), (8, [3, 2, 4]), (2, [1] * 9)])
def test_input_convolution_with_state(taps, cuts):
    from llmctl_b200.ops import canon as C
    torch.manual_seed(taps)
    T, W, eps = sum(cuts), 10, 1e-3
    x = torch.randn(T, W) * 2
    nw = [torch.rand(W) + 0.5, torch.rand(W) + 0.5]
    cw = [torch.randn(W, taps), torch.randn(W, taps)]
    n = oracle.rms(x.double(), eps)
    want = [oracle.canon(n * nw[s].double(), cw[s].double()) for s in range(2)]
    state = torch.full((3, taps - 1, W), 7.0)                 # garbage: a portion at position 0 must not read it
    got = [[], []]
    at = 0
    for c in cuts:
        xs = x[at:at + c].clone()
        r = C.residual_rms(None, None, xs, eps)
        portions = torch.tensor([[0, c, at, 2]], dtype=torch.int32)
        hs = C.norm_canon(xs, r, nw, cw, portions, torch.zeros(c, dtype=torch.int32), state, torch.float32)
        for s in range(2):
            got[s].append(hs[s])
        at += c
    for s in range(2):
        assert torch.allclose(torch.cat(got[s]).double(), want[s], atol=1e-5)
    # one sublayer only, two sequences in one call, one of them without a slot
    xs = x.clone()
    r = C.residual_rms(None, None, xs, eps)
    half = T // 2
    portions = torch.tensor([[0, half, 0, 1], [half, T - half, 0, -1]], dtype=torch.int32)
    seq_rows = torch.tensor([0] * half + [1] * (T - half), dtype=torch.int32)
    hs = C.norm_canon(xs, r, nw[:1], cw[:1], portions, seq_rows, state, torch.float32)
    n2 = oracle.rms(x[half:].double(), eps)
    assert len(hs) == 1 and torch.allclose(hs[0][half:].double(), oracle.canon(n2 * nw[0].double(), cw[0].double()), atol=1e-5)


def test_residual_update_and_statistics():
    from llmctl_b200.ops import canon as C
    torch.manual_seed(1)
    x, a, f = torch.randn(6, 14) + 1.0, torch.randn(6, 14), torch.randn(6, 14)
    x1 = x.clone()
    r = C.residual_rms(a.to(torch.bfloat16), f, x1, 1e-2)
    new = x.double() + a.to(torch.bfloat16).double() + f.double()
    assert torch.allclose(x1.double(), new, atol=1e-6)
    assert torch.allclose(r.double(), 1.0 / torch.sqrt(new.pow(2).mean(-1) + 1e-2), atol=1e-6)
    x2 = x.clone()
    C.residual_rms(a, None, x2, 1e-2)
    assert torch.allclose(x2, x + a, atol=1e-6)
    # eps sits inside the root: a zero row norms to zero, not to NaN
    assert torch.isfinite(C.residual_rms(None, None, torch.zeros(1, 14), 1e-6)).all()


def test_gated_gelu_and_sigmoid_gate():
    from llmctl_b200.ops import elementwise as E
    g = torch.tensor([[-6.0, -1.0, -0.1, 0.0, 0.4, 3.0]])
    u = torch.tensor([[0.5, -2.0, 1.0, 3.0, -1.0, 0.25]])
    out = E.gated_gelu_tanh(torch.cat([g, u], -1))
    assert torch.allclose(out.double(), oracle.gelu_tanh(g.double()) * u.double(), atol=1e-6)
    y, z = torch.randn(3, 5), torch.randn(3, 9)
    want = y * torch.sigmoid(z[:, 2:7])
    assert torch.allclose(E.sigmoid_gate_(y, z[:, 2:7]), want, atol=1e-6)


@pytest.mark.parametrize("dims,base,scaling", [(8, 10000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}),
                                               (48, 5e5, {"factor": 16.0, "original": 4096, "fast": 24.0, "slow": 2.0}),
                                               (4, 100.0, {"factor": 2.0, "original": 16, "fast": 1.0, "slow": 1.0}),     # lo == hi: the ramp's floor
                                               (6, 50.0, None)])
def test_rotation_spectrum(dims, base, scaling):
    from llmctl_b200.ops.elementwise import rope_frequencies
    f, m = rope_frequencies(dims, base, scaling)
    wf, wm = oracle.yarn_spectrum(dims, base, scaling)
    assert torch.allclose(f.double(), torch.tensor(wf, dtype=torch.float64), rtol=1e-6) and abs(m - wm) < 1e-7


def _window_case(H, G, d, e, n, bs, window, keep, cap, seed=0, start=0):
    """Random q / k / v for one sequence of n tokens written to a paged cache; returns what the op and the oracle need."""
    from llmctl_b200.ops import softcap_attention as S
    torch.manual_seed(seed)
    q, k, v = torch.randn(n, H, d), torch.randn(n, G, d), torch.randn(n, G, e)
    batch, table = paged(n, bs, seed=seed)
    cache = torch.zeros(len(table) + 3, bs, G * (d + e))
    proj = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), torch.zeros(n, 3)], dim=-1)
    return S, q, k, v, batch, cache, proj


@pytest.mark.parametrize("H,G,d,e,n,bs,window,keep,cap", [(4, 2, 8, 6, 40, 8, 9, 2, 5.0), (3, 1, 5, 7, 33, 16, 1, 0, 0.0), (2, 2, 4, 3, 50, 8, 0, 0, 3.0),
                                                          (6, 3, 3, 2, 27, 4, 4, 7, 20.0), (1, 1, 2, 1, 20, 64, 100, 3, 1.0)])
def test_window_attention_alone(H, G, d, e, n, bs, window, keep, cap):
    S, q, k, v, batch, cache, proj = _window_case(H, G, d, e, n, bs, window, keep, cap, seed=H)
    bias = torch.randn(proj.shape[1] - 3) * 0.3
    qo = S.window_kv_append(proj, bias, H, G, d, e, True, 1e-4, batch.slots, cache)
    nq, nk = H * d, G * d
    qb = q.double() + bias[:nq].view(H, d).double()
    kb = k.double() + bias[nq:nq + nk].view(G, d).double()
    vb = oracle.rms(v.double() + bias[nq + nk:].view(G, e).double(), 1e-4)
    assert torch.allclose(qo.double(), qb.reshape(n, -1), atol=1e-6)
    want = oracle.window_core(qb, kb, vb, 0.4, cap, window, keep)
    gate = torch.randn(n, H * e)
    for width in (1, 16):
        tiles = torch.tensor([[s, min(width, n - s), 0, 0] for s in range(0, n, width)], dtype=torch.int32)
        got = S.softcap_window_attention(qo, cache, batch.block_tables, tiles, width, batch.positions, gate, S.distance_slopes(H),
                                         torch.zeros(H), 0.4, cap, window, keep, H, G, d, e, bs, torch.float32)
        assert torch.allclose(got.double(), (want * torch.sigmoid(gate.double()).view(n, H, e)).reshape(n, -1), atol=2e-6)


@pytest.mark.parametrize("bs,window,keep", [(8, 24, 3), (16, 17, 1), (4, 9, 0)])
def test_window_edges_and_kept_tokens_decide(bs, window, keep):
    """One key is made dominant (its score reaches the cap, all others sit far below): the output is its value exactly
    while it is seen and has nothing of it one position later; a dominant kept token never leaves."""
    from llmctl_b200.ops import softcap_attention as S
    H = G = 1
    d, e, n, cap = 4, 3, 3 * window + 7, 12.0
    for star in ([bs - 1, bs, 2 * bs + 1] + ([0] if keep else [])):
        q = torch.zeros(n, H, d)
        q[:, 0, 0] = 40.0
        k = torch.zeros(n, G, d)
        k[:, 0, 0] = -1.0
        k[star, 0, 0] = 1.0
        v = torch.randn(n, G, e)
        v[star] = torch.tensor([5.0, -3.0, 2.0])
        batch, table = paged(n, bs, seed=star)
        cache = torch.zeros(len(table) + 3, bs, d + e)
        qo = S.window_kv_append(torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], -1), None, H, G, d, e, False, 0.0,
                                batch.slots, cache)
        for width in (1, 16):
            tiles = torch.tensor([[s, min(width, n - s), 0, 0] for s in range(0, n, width)], dtype=torch.int32)
            out = S.softcap_window_attention(qo, cache, batch.block_tables, tiles, width, batch.positions, None, S.distance_slopes(H), torch.zeros(H),
                                             1.0, cap, window, keep, H, G, d, e, bs, torch.float32)
            want = oracle.window_core(q.double(), k.double(), v.double(), 1.0, cap, window, keep)
            assert torch.allclose(out.double(), want.reshape(n, -1), atol=1e-5)
            last_seen = n - 1 if star < keep else star + window - 1
            assert torch.allclose(out[last_seen], v[star, 0], atol=1e-3)                      # e^24 against the rest
            if last_seen + 1 < n:
                assert (out[last_seen + 1] - v[star, 0]).abs().max() > 0.5


@pytest.mark.parametrize("H,dn,dr,dv,R,n,bs,far", [(3, 6, 4, 5, 16, 70, 8, 0), (2, 4, 8, 3, 12, 130, 16, 15), (1, 2, 2, 1, 4, 40, 8, 8),
                                                   (4, 8, 4, 8, 8, 300, 64, 63)])
def test_latent_attention_sink_and_far_key(H, dn, dr, dv, R, n, bs, far):
    """The mixer alone against the oracle; then a far key is made decisive by scaling its latent and the last query."""
    from llmctl_b200.models.mixers import LatentAttention, LatentAttentionSpec
    torch.manual_seed(n)
    W, Q, eps = 20, 6, 1e-5
    scaling = {"factor": 4.0, "original": 32, "fast": 4.0, "slow": 1.0}
    m = {"heads": H, "dim": dn, "rot_dim": dr, "vdim": dv, "kv_rank": R, "q_rank": Q, "scale": 0.3, "rot": {"base": 500.0, "dims": dr, "scaling": scaling}}
    cfg = {"width": W, "vocab": 8, "norm": {"eps": eps}, "canon": {"taps": 1}, "layers": [{"type": "latent_attention", "mixer": m, "mlp": None}]}
    wts = oracle.random_weights(cfg, n)
    P = oracle.sub(wts, "l0.mix.")
    spec = LatentAttentionSpec(heads=H, dim=dn, rot_dim=dr, vdim=dv, kv_rank=R, q_rank=Q, scale=0.3, rot_base=500.0, rot_scaling=scaling,
                               sink=True, out_gate=True)
    mixer = LatentAttention(W, spec, eps, torch.float32, "cpu")
    mixer.load(lambda name: wts[name], "l0.mix.")
    h = torch.randn(n, W)
    h[far] *= 6.0
    batch, table = paged(n, bs, seed=n)
    cache = torch.zeros(len(table) + 3, bs, R + dr)
    got = mixer(h, batch, cache)
    c, kr = oracle.latent_kv(h.double(), P, m, eps)
    want = oracle.latent_attention(h.double(), P, m, eps, c, kr)
    assert torch.allclose(got.double(), want, atol=2e-5)
    # a large sink swallows the weights: the output shrinks towards zero
    P2 = dict(P)
    P2["sink"] = P["sink"] + 30.0
    mixer.sink.data += 30.0
    got2 = mixer(h, batch, torch.zeros_like(cache))
    assert torch.allclose(got2.double(), oracle.latent_attention(h.double(), P2, m, eps, c, kr), atol=2e-5)
    assert float(got2.detach().abs().mean()) < 0.5 * float(got.detach().abs().mean())


@pytest.mark.parametrize("C_,N,R_,taps,cuts", [(10, 4, 3, 3, [12]), (6, 1, 1, 1, [2, 5]), (9, 5, 2, 4, [1, 1, 1, 3, 2, 6])])
def test_selective_scan_mixer_alone(C_, N, R_, taps, cuts):
    from llmctl_b200.models.mixers import SelectiveScan, SelectiveScanSpec
    from llmctl_b200.serve.ragged import Portion, RaggedBatch
    torch.manual_seed(C_)
    W, n = 12, sum(cuts)
    m = {"inner": C_, "state": N, "dt_rank": R_, "conv": taps}
    cfg = {"width": W, "vocab": 8, "norm": {"eps": 1e-5}, "canon": {"taps": 1}, "layers": [{"type": "mamba1", "mixer": m, "mlp": None}]}
    wts = oracle.random_weights(cfg, 1)
    mixer = SelectiveScan(W, SelectiveScanSpec(inner=C_, state=N, dt_rank=R_, conv=taps), torch.float32, "cpu")
    mixer.load(lambda name: wts[name], "l0.mix.")
    h = torch.randn(n, W)
    want = oracle.selective_scan(h.double(), oracle.sub(wts, "l0.mix."), m)
    state = tuple(torch.full((2, *s), 3.0) for s in mixer.state_shapes())       # garbage in the slot
    out, at = [], 0
    for c in cuts:
        b = RaggedBatch([Portion(1, [0] * c, at, [], [0, 1, 2, 3], 1)], 8, torch.device("cpu"))
        out.append(mixer(h[at:at + c], b, state))
        at += c
    assert torch.allclose(torch.cat(out).double(), want, atol=2e-5)


# ---- whole model ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_every_layer(name):
    cfg = small_cfg(**CONFIGS[name])
    w = oracle.random_weights(cfg, 11)
    torch.manual_seed(2)
    toks = torch.randint(0, cfg["vocab"], (29,)).tolist()
    layers = []
    want = ref_logits(cfg, w, toks, layers)
    eng = make_engine(cfg, w)
    assert eng.kv.allocate(1, len(toks))
    trace = []
    got = eng.forward_portions([eng.portion(1, toks, 0, list(range(len(toks))))], layer_trace=trace)
    assert len(trace) == len(cfg["layers"])
    for a, b in zip(trace, layers):
        assert torch.allclose(a.double(), b, atol=F32 * max(1.0, float(b.abs().max())))
    assert torch.allclose(got, want, atol=F32 * max(1.0, float(want.abs().max())))


@pytest.mark.parametrize("name,cuts", [("default", [1] * 26), ("default", [2, 2, 3, 2, 9, 1, 7]), ("keep_more_than_window", [5, 1, 2, 2, 16]),
                                       ("no_yarn_no_ff", [13, 2, 2, 1, 8]), ("scan_edges", [2, 1, 1, 1, 2, 19]),
                                       ("one_kv_head_window_1", [7, 19])])
def test_portions_against_whole_prompt(name, cuts):
    cfg = small_cfg(**CONFIGS[name])
    w = oracle.random_weights(cfg, 5)
    torch.manual_seed(3)
    toks = torch.randint(0, cfg["vocab"], (sum(cuts),)).tolist()
    want = ref_logits(cfg, w, toks)
    got = run_cut(make_engine(cfg, w), 1, toks, cuts)
    assert torch.allclose(got, want, atol=F32 * max(1.0, float(want.abs().max())))


def test_layers_of_one_kind_with_unlike_sizes_and_shared_caches_out_of_order():
    """Two latent layers with caches of their own, two attention layers and two scans, each pair with its own sizes and
    constants; the last two layers read the FIRST and the SECOND latent layer's cache (not the latest one), with their own
    scale and the rotation base of the layer they read.  Portions cut anywhere against the whole-prompt oracle."""
    a = small_cfg(pattern="LLAMcc", ff="111111", taps=3)
    b = small_cfg(pattern="LLAMcc", ff="101101", heads=6, kv_heads=3, dim=4, vdim=6, softcap=3.0, window=5, keep_first=0, inner=24, state=3,
                  dt_rank=5, conv=2, ff_size=24, lat_heads=2, lat_dim=4, rot_dim=6, lat_vdim=8, kv_rank=10, q_rank=7)
    cfg = copy.deepcopy(a)
    cfg["layers"][1], cfg["layers"][5] = copy.deepcopy(b["layers"][1]), copy.deepcopy(b["layers"][5])
    cfg["layers"][4]["mixer"]["kv_from"], cfg["layers"][5]["mixer"]["kv_from"] = 0, 1
    cfg["layers"].insert(3, copy.deepcopy(b["layers"][2]))
    cfg["layers"].insert(5, copy.deepcopy(b["layers"][3]))            # L L A A' M M' c(0) c'(1)
    for i in (1, 7):
        cfg["layers"][i]["mixer"]["rot"]["base"] = 500.0
    cfg["layers"][7]["mixer"]["scale"], cfg["layers"][3]["mixer"]["scale"], cfg["norm"]["eps"] = 0.7, 0.9, 1e-3
    w = oracle.random_weights(cfg, 3)
    torch.manual_seed(8)
    cuts = [7, 2, 20, 1, 1, 3, 16]
    toks = torch.randint(0, cfg["vocab"], (sum(cuts),)).tolist()
    want = ref_logits(cfg, w, toks)
    got = run_cut(make_engine(cfg, w), 1, toks, cuts)
    assert torch.allclose(got, want, atol=F32 * max(1.0, float(want.abs().max())))


def test_unequal_batches_skipped_steps_and_reused_pages_and_slots():
    """Three requests at a time in a pool of 2 state slots' worth ... no: 3 seats, 9 pages of 8 tokens: five requests of
    unequal length, portions of 1-11 tokens beside single tokens, requests that skip steps; pages and slots of finished
    requests go to the next ones.  Every position's logits equal the request's own whole-prompt logits."""
    cfg = small_cfg(pattern="MALcA", ff="11011", window=7, keep_first=2)
    w = oracle.random_weights(cfg, 9)
    torch.manual_seed(4)
    lens = [30, 9, 17, 24, 5]
    prompts = [torch.randint(0, cfg["vocab"], (n,)).tolist() for n in lens]
    want = [ref_logits(cfg, w, p) for p in prompts]
    eng = make_engine(cfg, w, blocks=9, bs=8, max_batch=3)
    pos = [0] * len(prompts)
    got = [[] for _ in prompts]
    waiting, live, step = list(range(len(prompts))), [], 0
    sizes = [3, 1, 11, 2, 1, 1, 5]
    while waiting or live:
        while waiting and len(live) < 3 and eng.kv.allocate(waiting[0] + 1, min(sizes[0], lens[waiting[0]])):
            live.append(waiting.pop(0))
        portions, who = [], []
        for i in list(live):
            if (step + i) % 4 == 3:                     # this request sits the step out
                continue
            c = min(sizes[(step + 2 * i) % len(sizes)], lens[i] - pos[i])
            if not eng.kv.allocate(i + 1, pos[i] + c):
                continue                                # no page free right now: wait for somebody to finish
            portions.append(eng.portion(i + 1, prompts[i][pos[i]:pos[i] + c], pos[i], list(range(c))))
            who.append((i, c))
            pos[i] += c
        if portions:
            lg, o = eng.forward_portions(portions).float(), 0
            for i, c in who:
                got[i].append(lg[o:o + c])
                o += c
        for i in list(live):
            if pos[i] == lens[i]:
                eng.kv.free(i + 1)
                live.remove(i)
        step += 1
        assert step < 500
    for i in range(len(prompts)):
        assert torch.allclose(torch.cat(got[i]), want[i], atol=F32 * max(1.0, float(want[i].abs().max()))), i


def test_first_token_and_long_decoding_across_pages():
    """Slow decays and a kept first token: the first token still moves the last logits of a long decode; decoding runs
    token by token over several pages and windows."""
    cfg = small_cfg(pattern="AM", ff="11", window=6, keep_first=1, taps=2)
    w = oracle.random_weights(cfg, 3)
    w["l1.mix.A_log"] = torch.full_like(w["l1.mix.A_log"], -6.0)
    w["l1.mix.dt.b"] = torch.full_like(w["l1.mix.dt.b"], -4.0)
    torch.manual_seed(8)
    toks = torch.randint(0, cfg["vocab"], (90,)).tolist()
    want = ref_logits(cfg, w, toks)
    got = run_cut(make_engine(cfg, w), 1, toks, [10] + [1] * 80)
    assert torch.allclose(got, want, atol=F32 * max(1.0, float(want.abs().max())))
    other = ref_logits(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert (other[-1] - want[-1]).abs().max() > 100 * F32


def test_greedy_generation_through_scheduler_and_engine():
    cfg = small_cfg(pattern="MAL", ff="111", window=8, keep_first=2)
    w = oracle.random_weights(cfg, 21)
    torch.manual_seed(5)
    prompts = [torch.randint(0, cfg["vocab"], (n,)).tolist() for n in (5, 12, 3, 9, 7)]
    eng = make_engine(cfg, w, blocks=16, bs=8, max_batch=2)             # more requests than seats
    outs = eng.generate(prompts, max_tokens=6, temperature=0.0)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for _ in range(6):
            seq.append(int(ref_logits(cfg, w, seq)[-1].argmax()))
        assert list(o) == seq[len(p):]


def test_config_reader_registry_and_trace_replay(tmp_path):
    from safetensors.torch import save_file
    from llmctl_b200.models.registry import architecture_named
    from llmctl_b200.models.tupidra import TupidraConfig
    from llmctl_b200.serve import replay
    cfg = small_cfg(pattern="MLAc", ff="1110")
    w = oracle.random_weights(cfg, 2)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(torch.bfloat16) if v.dtype.is_floating_point else v for k, v in w.items()}, str(tmp_path / "model.safetensors"))
    arch = architecture_named("Tupidra")
    parsed = arch.config_from_dict(cfg)
    assert isinstance(parsed, TupidraConfig) and [l.type for l in parsed.layers] == ["mamba1", "latent_attention", "attention", "latent_attention"]
    assert parsed.layers[3].mixer.kv_from == 1 and parsed.layers[3].ff == 0 and parsed.taps == cfg["canon"]["taps"]
    bad = copy.deepcopy(cfg)
    bad["layers"][3]["mixer"]["kv_from"] = 2            # not a latent layer
    with pytest.raises(ValueError):
        arch.config_from_dict(bad)
    torch.manual_seed(6)
    a, b = torch.randint(0, cfg["vocab"], (21,)).tolist(), torch.randint(0, cfg["vocab"], (10,)).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:9], "want": [8]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[9:11], "want": []}, {"id": "b", "tokens": b[:7], "want": [0, 6]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[7:], "want": [2]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[11:], "want": [9]}], "end": ["a"]}]
    out = io.StringIO()
    rc = replay.run(str(tmp_path), "float32", str(tmp_path / "out"), 128, device="cpu", stdin=io.StringIO("\n".join(json.dumps(s) for s in steps)),
                    stdout=out)
    assert rc == 0 and out.getvalue().split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    import numpy as np
    la, lb = ref_logits(cfg, w, a), ref_logits(cfg, w, b)
    rd = lambda s: torch.from_numpy(np.fromfile(tmp_path / "out" / f"{s}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
    tol = F32 * max(1.0, float(la.abs().max()))
    assert torch.allclose(rd(0), la[[8]], atol=tol) and torch.allclose(rd(1), lb[[0, 6]], atol=tol)
    assert torch.allclose(rd(2), lb[[9]], atol=tol) and torch.allclose(rd(3), la[[20]], atol=tol)
