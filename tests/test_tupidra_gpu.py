"""Tupidra's CUDA kernels against the CPU restatements of the same ops and the engine on a GPU against the plain oracle
(``tupidra_oracle.py``), in fp32 (tight) and bf16 (rounding-sized)."""
import pytest
import torch

import tupidra_oracle as oracle
from test_tupidra_cpu import CONFIGS, make_engine, paged, ref_logits, run_cut, small_cfg

pytestmark = pytest.mark.gpu


def rel(a, b):
    """Largest row error: rms of the difference (mean taken off) over the rms of the reference row."""
    d = a.double() - b.double()
    d = d - d.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / b.double().pow(2).mean(-1).sqrt().clamp_min(1e-9)).max())


@pytest.mark.parametrize("W,taps,cuts", [(10, 4, [1, 1, 2, 1, 7]), (1000, 3, [40]), (5000, 8, [3, 2, 9]), (256, 1, [5, 5]), (64, 2, [1] * 6)])
def test_input_convolution_kernels(cuda_device, W, taps, cuts):
    from llmctl_b200.ops import canon as C
    torch.manual_seed(W)
    T = sum(cuts)
    x, a, f = torch.randn(T, W) * 2, torch.randn(T, W), torch.randn(T, W)
    nw = [torch.rand(W) + 0.5, torch.rand(W) + 0.5]
    cw = [torch.randn(W, taps), torch.randn(W, taps)]
    dev = cuda_device
    for dt in (torch.float32, torch.bfloat16):
        sc, sg = torch.full((3, taps - 1, W), 5.0), torch.full((3, taps - 1, W), 5.0, device=dev)
        at = 0
        for c in cuts:
            xc, xg = x[at:at + c].clone(), x[at:at + c].clone().to(dev)
            ac, fc = a[at:at + c].to(dt), f[at:at + c]
            rc = C.residual_rms(ac, fc, xc, 1e-5)
            rg = C.residual_rms(ac.to(dev), fc.to(dev), xg, 1e-5)
            assert torch.allclose(xg.cpu(), xc, atol=1e-6) and torch.allclose(rg.cpu(), rc, rtol=1e-5)
            # two sequences in the call: the portion under test (slot 1) and a one-token stranger at position 0 (slot 0)
            portions = torch.tensor([[0, c, at, 1]], dtype=torch.int32)
            rows = torch.zeros(c, dtype=torch.int32)
            hc = C.norm_canon(xc, rc, nw, cw, portions, rows, sc, dt)
            hg = C.norm_canon(xg, rg, [w.to(dev) for w in nw], [w.to(dev) for w in cw], portions.to(dev), rows.to(dev), sg, dt)
            for s in range(2):
                assert hg[s].dtype == dt and torch.allclose(hg[s].float().cpu(), hc[s].float(), atol=1e-4 if dt == torch.float32 else 0.1, rtol=1e-2)
            assert torch.allclose(sg.cpu(), sc, atol=1e-5)
            at += c
        h1 = C.norm_canon(xg, rg, [nw[1].to(dev)], [cw[1].to(dev)], portions.to(dev), rows.to(dev), sg.clone(), torch.float32)
        assert len(h1) == 1


@pytest.mark.parametrize("W,taps", [(10, 4), (1000, 3), (4096, 8), (64, 1), (48, 2)])
def test_single_launch_glue_for_short_portions(cuda_device, W, taps):
    """Decoding batches: residual update, statistics, both inputs and the new state rows in one launch per layer, for three
    sequences side by side (portions of 1-8 tokens, one at position 0 over a slot that holds garbage, one without a slot)."""
    from llmctl_b200.ops import canon as C
    torch.manual_seed(W + taps)
    dev = cuda_device
    nw = [torch.rand(W) + 0.5, torch.rand(W) + 0.5]
    cw = [torch.randn(W, taps), torch.randn(W, taps)]
    for dt in (torch.float32, torch.bfloat16):
        sc = torch.randn(4, taps - 1, W)
        sg = sc.clone().to(dev)
        pos = [5, 0, 9]
        for lens in ([1, 1, 1], [8, 3, 2], [2, 1, 5], [1, 1, 1]):
            T = sum(lens)
            x, a, f = torch.randn(T, W) * 2, torch.randn(T, W).to(dt), torch.randn(T, W).to(dt)
            starts = [0, lens[0], lens[0] + lens[1]]
            portions = torch.tensor([[starts[i], lens[i], pos[i], (2, 0, -1)[i]] for i in range(3)], dtype=torch.int32)
            rows = torch.tensor(sum(([i] * lens[i] for i in range(3)), []), dtype=torch.int32)
            xc, xg = x.clone(), x.clone().to(dev)
            hc = C.residual_norm_canon(a, f, xc, 1e-5, nw, cw, portions, rows, sc, dt)
            hg = C.residual_norm_canon(a.to(dev), f.to(dev), xg, 1e-5, [w.to(dev) for w in nw], [w.to(dev) for w in cw], portions.to(dev),
                                       rows.to(dev), sg, dt, small=True)
            assert torch.allclose(xg.cpu(), xc, atol=1e-6) and torch.allclose(sg.cpu(), sc, atol=1e-5)
            for s in range(2):
                assert hg[s].dtype == dt and torch.allclose(hg[s].float().cpu(), hc[s].float(), atol=1e-4 if dt == torch.float32 else 0.1, rtol=1e-2)
            pos = [pos[i] + lens[i] for i in range(3)]
        h1 = C.residual_norm_canon(None, None, xg, 1e-5, [nw[0].to(dev)], [cw[0].to(dev)], portions.to(dev), rows.to(dev), sg, dt, small=True)
        assert len(h1) == 1


def test_activation_kernels(cuda_device):
    from llmctl_b200.ops import elementwise as E
    torch.manual_seed(0)
    gu = torch.randn(37, 2 * 50) * 3
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 5e-2)):
        want = E.gated_gelu_tanh(gu.to(dt))
        got = E.gated_gelu_tanh(gu.to(dt).to(cuda_device))
        assert torch.allclose(got.float().cpu(), want.float(), atol=tol, rtol=1e-2)
        y, z = torch.randn(9, 20).to(dt), torch.randn(9, 64).to(dt)
        want = E.sigmoid_gate_(y.clone(), z[:, 7:27])
        got = E.sigmoid_gate_(y.clone().to(cuda_device), z.to(cuda_device)[:, 7:27])
        assert torch.allclose(got.float().cpu(), want.float(), atol=tol, rtol=1e-2)


def _attention_case(H, G, d, e, n, bs, start, seed):
    torch.manual_seed(seed)
    q, k, v = torch.randn(n + start, H, d), torch.randn(n + start, G, d), torch.randn(n + start, G, e)
    proj = torch.cat([q.reshape(n + start, -1), k.reshape(n + start, -1), v.reshape(n + start, -1), torch.randn(n + start, H * e)], dim=-1)
    bias = torch.randn(H * d + G * d + G * e) * 0.3
    return proj, bias


@pytest.mark.parametrize("H,G,d,e,n,bs,window,keep,cap", [(4, 2, 8, 6, 45, 16, 9, 2, 5.0), (3, 1, 5, 7, 133, 16, 1, 0, 0.0), (8, 2, 16, 16, 300, 64, 70, 4, 20.0),
                                                          (8, 4, 48, 40, 200, 64, 75, 5, 25.0), (4, 4, 32, 64, 150, 8, 0, 0, 3.0),
                                                          (16, 2, 128, 128, 90, 64, 40, 50, 30.0), (2, 1, 16, 136, 70, 16, 33, 1, 8.0),
                                                          (32, 4, 64, 64, 520, 64, 256, 3, 15.0)])
def test_window_attention_kernels(cuda_device, H, G, d, e, n, bs, window, keep, cap):
    """FMA (fp32, bf16) and tensor-core kernels, prompt tiles and single-token tiles with and without key slices, against the
    CPU restatement over the same paged cache."""
    from llmctl_b200.ops import softcap_attention as S
    dev = cuda_device
    proj, bias = _attention_case(H, G, d, e, n, bs, 0, H * d)
    batch_c, table = paged(n, bs, seed=n)
    batch_g, _ = paged(n, bs, device=dev, seed=n)
    slopes, sinks = S.distance_slopes(H), torch.randn(H)
    nqkv = H * d + G * d + G * e
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        pc = proj.to(dt)
        cc = torch.zeros(len(table) + 3, bs, G * (d + e), dtype=dt)
        cg = torch.zeros_like(cc, device=dev)
        qc = S.window_kv_append(pc, bias, H, G, d, e, True, 1e-5, batch_c.slots, cc)
        qg = S.window_kv_append(pc.to(dev), bias.to(dev), H, G, d, e, True, 1e-5, batch_g.slots, cg)
        assert torch.allclose(qg.cpu(), qc, atol=1e-6) and torch.allclose(cg.float().cpu(), cc.float(), atol=1e-6 if dt == torch.float32 else 2e-2)
        cg.copy_(cc)                    # same cache bits for both from here on
        gate_c = pc[:, nqkv:]
        tiles1 = torch.tensor([[s, 1, 0, 0] for s in range(n)], dtype=torch.int32)
        want = S.softcap_window_attention(qc, cc, batch_c.block_tables, tiles1, 1, batch_c.positions, gate_c, slopes, sinks, 0.2, cap, window,
                                          keep, H, G, d, e, bs, torch.float32).float()
        runs = [(16, False, 0), (1, False, 0), (1, False, 3)]
        if dt == torch.bfloat16 and S.uses_tensor_cores(dt, H, G, d, e, 128):
            runs += [(128, True, 0), (1, True, 0), (1, True, 2), (1, True, 5)]
        for width, tc, splits in runs:
            tiles = torch.tensor([[s, min(width, n - s), 0, 0] for s in range(0, n, width)], dtype=torch.int32).to(dev)
            got = S.softcap_window_attention(qg, cg, batch_g.block_tables, tiles, width, batch_g.positions, pc.to(dev)[:, nqkv:], slopes.to(dev),
                                             sinks.to(dev), 0.2, cap, window, keep, H, G, d, e, bs, dt, max_context=n, splits=splits,
                                             tensor_cores=tc)
            assert (got.float().cpu() - want).abs().max() < tol * max(1.0, float(want.abs().max())), (dt, width, tc, splits)
        # no sink, no slopes, no gate
        want2 = S.softcap_window_attention(qc, cc, batch_c.block_tables, tiles1, 1, batch_c.positions, None, None, None, 0.2, cap, window, keep,
                                           H, G, d, e, bs, torch.float32).float()
        for width in (16, 128 if dt == torch.bfloat16 and S.uses_tensor_cores(dt, H, G, d, e, 128) else 1):
            tiles = torch.tensor([[s, min(width, n - s), 0, 0] for s in range(0, n, width)], dtype=torch.int32).to(dev)
            got = S.softcap_window_attention(qg, cg, batch_g.block_tables, tiles, width, batch_g.positions, None, None, None, 0.2, cap, window,
                                             keep, H, G, d, e, bs, dt, max_context=n)
            assert (got.float().cpu() - want2).abs().max() < tol * max(1.0, float(want2.abs().max())), (dt, width)


@pytest.mark.parametrize("bs,window,keep,d,e", [(64, 76, 5, 16, 8), (16, 40, 1, 32, 16), (8, 33, 0, 16, 24)])
def test_window_edges_decide_on_every_kernel(cuda_device, bs, window, keep, d, e):
    """A dominant key (score at the cap against scores at minus the cap) at page borders, key-tile borders and position 0:
    the output is its value while it is seen and free of it one position later, in prompt tiles and in decoded tokens."""
    from llmctl_b200.ops import softcap_attention as S
    dev = cuda_device
    H, G, cap = 2, 1, 12.0
    n = 3 * window + 2 * bs + 5
    for star in ([bs - 1, bs, 31, 32, 2 * bs + 1] + ([0] if keep else [])):
        q = torch.zeros(n, H, d)
        q[:, :, 0] = 40.0
        k = torch.zeros(n, G, d)
        k[:, 0, 0] = -1.0
        k[star, 0, 0] = 1.0
        torch.manual_seed(star)
        v = torch.randn(n, G, e).to(torch.bfloat16).float()
        v[star, 0, :3] = torch.tensor([5.0, -3.0, 2.0])
        proj = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], -1)
        batch, table = paged(n, bs, device=dev, seed=star)
        want = oracle.window_core(q.double(), k.double(), v.double(), 1.0, cap, window, keep).reshape(n, -1)
        last_seen = n - 1 if star < keep else star + window - 1
        for dt in (torch.float32, torch.bfloat16):
            cache = torch.zeros(len(table) + 3, bs, G * (d + e), dtype=dt, device=dev)
            qo = S.window_kv_append(proj.to(dt).to(dev), None, H, G, d, e, False, 0.0, batch.slots, cache)
            for width, tc, splits in [(16, False, 0), (1, False, 2)] + ([(128, True, 0), (1, True, 0), (1, True, 3)] if dt == torch.bfloat16 else []):
                tiles = torch.tensor([[s, min(width, n - s), 0, 0] for s in range(0, n, width)], dtype=torch.int32).to(dev)
                out = S.softcap_window_attention(qo, cache, batch.block_tables, tiles, width, batch.positions, None, S.distance_slopes(H).to(dev),
                                                 torch.zeros(H, device=dev), 1.0, cap, window, keep, H, G, d, e, bs, dt, max_context=n,
                                                 splits=splits, tensor_cores=tc).float().cpu()
                assert torch.allclose(out.double(), want, atol=1e-4 if dt == torch.float32 else 3e-2), (star, dt, width, tc)
                # head 1 has the small slope (2^-8 a position): the distance bias leaves the dominant key dominant
                assert torch.allclose(out[last_seen, e:e + 3], v[star, 0, :3], atol=3e-2)
                if last_seen + 1 < n:
                    assert (out[last_seen + 1, e:e + 3] - v[star, 0, :3]).abs().max() > 0.5


@pytest.mark.parametrize("H,dn,dr,R,n,bs,far", [(3, 6, 4, 16, 70, 8, 0), (4, 16, 16, 48, 200, 64, 63), (8, 16, 64, 64, 300, 64, 64),
                                                (4, 32, 64, 128, 260, 64, 127), (16, 64, 64, 192, 140, 64, 5)])
def test_latent_attention_sinks_on_every_kernel(cuda_device, H, dn, dr, R, n, bs, far):
    """Absorbed queries against a paged latent cache with a learned sink per head: FMA, mma.sync and tcgen05 kernels, prompt
    tiles and decoded tokens, with and without key slices, against the CPU restatement; one far cache row is made large."""
    from llmctl_b200.ops import latent_attention as L
    from llmctl_b200.ops.elementwise import rope_frequencies
    dev = cuda_device
    torch.manual_seed(n)
    freq, mult = rope_frequencies(dr, 1e4, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0})
    ql = torch.randn(n, H, R) * 0.5
    q = torch.randn(n, H * (dn + dr))
    rows = torch.randn(n, R + dr)
    rows[far] *= 4.0
    sinks = torch.randn(H) * 2
    batch_c, table = paged(n, bs, seed=n)
    batch_g, _ = paged(n, bs, device=dev, seed=n)
    for dt, tol in ((torch.float32, 3e-5), (torch.bfloat16, 3e-2)):
        cc = torch.zeros(len(table) + 3, bs, R + dr, dtype=dt)
        cc.view(-1, R + dr)[batch_c.slots] = rows.to(dt)
        cg = cc.to(dev)
        tiles1 = torch.tensor([[s, 1, 0, 0] for s in range(n)], dtype=torch.int32)
        qc = q.to(dt)
        want = L.latent_attention(ql, qc, dn, cc, batch_c.block_tables, tiles1, batch_c.positions, freq, mult, 0.1, 1, n, sinks=sinks).float()
        none = L.latent_attention(ql, qc, dn, cc, batch_c.block_tables, tiles1, batch_c.positions, freq, mult, 0.1, 1, n).float()
        assert (want - none).abs().max() > 1e-3
        cases = [(16, False, 1), (16, False, 3)]
        if dt == torch.bfloat16 and L.uses_tensor_cores(dt, R, dr):
            cases += [(L.rows_per_tile(dt, R, dr, True), True, 1), (16, True, 2)]
        if L.uses_tcgen05(dt, R, dr, bs, True):
            cases += [(128, True, 1), (128, True, 2)]
        for rows_per, tc, splits in cases:
            for decode in (False, True):
                hpt = min(H, rows_per) if decode else 1
                width = 1 if decode else rows_per
                tiles = torch.tensor([[s, min(width, n - s), 0, 0] for s in range(0, n, width)], dtype=torch.int32).to(dev)
                qlg = ql.to(dev).to(dt) if (tc and dt == torch.bfloat16) else ql.to(dev)
                got = L.latent_attention(qlg, qc.to(dev), dn, cg, batch_g.block_tables, tiles, batch_g.positions, freq.to(dev), mult, 0.1, hpt, n,
                                         splits, tensor_cores=tc, rows=rows_per, sinks=sinks.to(dev)).float().cpu()
                assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max())), (dt, rows_per, tc, splits, decode)
        assert L.tcgen05_status() == 0


GPU_CONFIGS = dict(CONFIGS)
GPU_CONFIGS["tensor_core_sizes"] = dict(width=64, vocab=96, pattern="AMLcA", ff="11011", taps=4, heads=4, kv_heads=2, dim=16, vdim=16, window=40,
                                        keep_first=3, lat_heads=4, lat_dim=16, rot_dim=16, lat_vdim=16, kv_rank=48, q_rank=24, inner=64, state=8,
                                        dt_rank=4, conv=4, ff_size=64)
GPU_CONFIGS["panel_sizes"] = dict(width=128, vocab=131, pattern="LAc", ff="111", taps=2, heads=8, kv_heads=2, dim=32, vdim=64, window=0, keep_first=0,
                                  softcap=0.0, lat_heads=4, lat_dim=32, rot_dim=64, lat_vdim=32, kv_rank=128, q_rank=32, ff_size=128)


@pytest.mark.parametrize("name", sorted(GPU_CONFIGS))
def test_engine_fp32_against_oracle(cuda_device, name):
    cfg = small_cfg(**GPU_CONFIGS[name])
    w = oracle.random_weights(cfg, 11)
    torch.manual_seed(2)
    toks = torch.randint(0, cfg["vocab"], (75,)).tolist()
    layers = []
    want = ref_logits(cfg, w, toks, layers)
    eng = make_engine(cfg, w, device="cuda", blocks=12, bs=16)
    assert eng.kv.allocate(1, len(toks))
    trace = []
    got = eng.forward_portions([eng.portion(1, toks, 0, list(range(len(toks))))], layer_trace=trace).cpu()
    for a, b in zip(trace, layers):
        assert torch.allclose(a.double().cpu(), b, atol=3e-4 * max(1.0, float(b.abs().max())))
    assert rel(got, want) < 1e-4
    eng.kv.free(1)
    assert rel(run_cut(eng, 2, toks, [2, 30, 1, 1, 17, 2, 22]), want) < 1e-4
    eng.kv.free(2)
    assert rel(run_cut(eng, 3, toks[:40], [1] * 40), want[:40]) < 1e-4


@pytest.mark.parametrize("name", ["tensor_core_sizes", "panel_sizes", "default"])
def test_engine_bf16_mixed_batches(cuda_device, name):
    """bf16 serving against the float64 oracle within rounding, and — tighter — against itself: unequal requests in one batch
    with portions down to two tokens next to decoded tokens give what each request gives alone."""
    cfg = small_cfg(**GPU_CONFIGS[name])
    w = oracle.random_weights(cfg, 13)
    torch.manual_seed(7)
    prompts = [torch.randint(0, cfg["vocab"], (n,)).tolist() for n in (150, 37, 5, 260)]
    eng = make_engine(cfg, w, dt=torch.bfloat16, device="cuda", blocks=12, bs=64)
    alone = []
    for i, p in enumerate(prompts):
        alone.append(run_cut(eng, 10 + i, p, [len(p)]))
        eng.kv.free(10 + i)
        assert rel(alone[-1], ref_logits(cfg, w, p)) < 6e-2
    pos, got, k = [0] * 4, [[] for _ in prompts], 0
    chunks = [7, 2, 130, 64, 1, 3]
    while any(pos[i] < len(prompts[i]) for i in range(4)):
        portions, who = [], []
        for i in range(4):
            if pos[i] >= len(prompts[i]) or (k + i) % 5 == 4:
                continue
            c = min(chunks[(k + i) % len(chunks)], len(prompts[i]) - pos[i])
            assert eng.kv.allocate(i + 1, pos[i] + c)
            portions.append(eng.portion(i + 1, prompts[i][pos[i]:pos[i] + c], pos[i], list(range(c))))
            who.append((i, c))
            pos[i] += c
        if portions:
            lg, o = eng.forward_portions(portions).float().cpu(), 0
            for i, c in who:
                got[i].append(lg[o:o + c])
                o += c
        k += 1
    for i in range(4):
        assert rel(torch.cat(got[i]), alone[i]) < 3e-2, i


def test_slot_reuse_and_graph_replayed_decoding(cuda_device):
    """Greedy generation through scheduler + engine with CUDA-graph decode steps: more requests than seats, so seats, slots
    and pages change hands and the batch bucket changes while sequences are mid-way (a graph captured then must not touch
    their states); fp32 so that the tokens can be compared with the oracle's."""
    cfg = small_cfg(pattern="MAL", ff="111", window=8, keep_first=2)
    w = oracle.random_weights(cfg, 21)
    torch.manual_seed(5)
    prompts = [torch.randint(0, cfg["vocab"], (n,)).tolist() for n in (5, 12, 3, 9, 7, 4)]
    eng = make_engine(cfg, w, device="cuda", blocks=16, bs=8, max_batch=3, graphs=True)
    lens = [3, 9, 5, 7, 2, 8]
    want = []
    for p, n in zip(prompts, lens):
        seq = list(p)
        for _ in range(n):
            seq.append(int(ref_logits(cfg, w, seq)[-1].argmax()))
        want.append(seq[len(p):])
    seqs = [eng.add_request(p, max_tokens=n, temperature=0.0) for p, n in zip(prompts, lens)]
    steps = 0
    while any(not s.finished for s in seqs) and eng.has_work():
        eng.step()
        steps += 1
        assert steps < 200
    assert [list(s.generated) for s in seqs] == want
