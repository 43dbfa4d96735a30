"""Optimizer features on the GPU: CUDA-graph capture, AMP GradScaler, state paging, rounding modes.

Model: the reference's capturable / AMP / offload tests (``tests/test_capturable.py``,
``tests/test_amp.py``, ``tests/test_cpu_offload.py`` patterns: an eager oracle stepped with the
same gradients).  Every comparison is against the eager kernels or the fp32 torch statement.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _params(seed=0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    shapes = [("a.weight", (64, 256)), ("b.weight", (128, 64)), ("norm.weight", (256,)), ("bias", (40,))]
    return [(n, (torch.randn(s, generator=g) * 0.05).to(dtype).to(_dev()).requires_grad_()) for n, s in shapes]


def _grads(params, step, scale=1.0):
    g = torch.Generator().manual_seed(100 + step)
    return [(torch.randn(p.shape, generator=g) * 1e-2 * scale).to(p.dtype).to(p.device) for _, p in params]


def test_capturable_cuda_graph_replay_matches_eager():
    from gefen_x_b200 import Gefen

    pa, pb = _params(), _params()
    oa = Gefen(pa, lr=1e-2, weight_decay=0.01)
    ob = Gefen(pb, lr=1e-2, weight_decay=0.01, capturable=True)
    static = [torch.zeros_like(p) for _, p in pb]
    for (_, p), s in zip(pb, static):
        p.grad = s
    # warm-up (eager, on a side stream as graph capture requires): first-step analysis, plans
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    for step in range(3):
        gs = _grads(pa, step)
        for (_, p), g in zip(pa, gs):
            p.grad = g
        oa.step()
        with torch.cuda.stream(side):
            for s, g in zip(static, gs):
                s.copy_(g)
            ob.step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ob.step()
    for step in range(3, 8):
        gs = _grads(pa, step)
        for (_, p), g in zip(pa, gs):
            p.grad = g
        oa.step()
        for s, g in zip(static, gs):
            s.copy_(g)
        graph.replay()
    torch.cuda.synchronize()
    for (n, a), (_, b) in zip(pa, pb):
        # the capturable scalars are fp32 on the device (the eager ones come from host doubles), so
        # a bf16 parameter may round the other way: one ulp (2^-12 at 0.05), state bit-identical
        torch.testing.assert_close(a.float(), b.float(), rtol=0, atol=1e-3, msg=n)
        assert torch.equal(oa.state[a]["m_codebook"], ob.state[b]["m_codebook"]), n
        assert torch.equal(oa.state[a]["m_magnitude"], ob.state[b]["m_magnitude"]), n
    assert float(ob.state[pb[0][1]]["step"]) == 8.0
    assert all(v == 0 for v in ob.kernel_status().values())


def test_grad_scaler_unscales_in_kernel_and_skips_on_overflow():
    from gefen_x_b200 import Gefen

    pa, pb = _params(dtype=torch.float32), _params(dtype=torch.float32)
    oa = Gefen(pa, lr=1e-2)
    ob = Gefen(pb, lr=1e-2)
    scaler = torch.amp.GradScaler("cuda", init_scale=1024.0, growth_interval=1000)
    scaler.scale(torch.ones((), device=_dev()))      # creates the scale tensor, as scaling a loss does
    for step in range(4):
        gs = _grads(pa, step)
        for (_, p), g in zip(pa, gs):
            p.grad = g
        oa.step()
        for (_, p), g in zip(pb, gs):
            p.grad = g * scaler.get_scale()          # what backward of a scaled loss would leave
        scaler.step(ob)
        scaler.update()
    for (n, a), (_, b) in zip(pa, pb):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-6, msg=n)
        assert torch.equal(oa.state[a]["m_codebook"], ob.state[b]["m_codebook"]), n
    # overflow: nothing moves, the scale backs off
    before = [p.detach().clone() for _, p in pb]
    idx = [ob.state[p]["m_codebook"].clone() for _, p in pb]
    for (_, p), g in zip(pb, _grads(pb, 99)):
        p.grad = g * scaler.get_scale()
    pb[0][1].grad[0, 0] = float("inf")
    scale0 = scaler.get_scale()
    scaler.step(ob)
    scaler.update()
    assert scaler.get_scale() < scale0
    for (_, p), b0, i0 in zip(pb, before, idx):
        assert torch.equal(p, b0)
        assert torch.equal(ob.state[p]["m_codebook"], i0)


def test_state_paged_to_host_between_steps_comes_back():
    from gefen_x_b200 import Gefen

    pa, pb = _params(), _params()
    oa = Gefen(pa, lr=1e-2)
    ob = Gefen(pb, lr=1e-2)
    for step in range(5):
        gs = _grads(pa, step)
        for (_, p), g in zip(pa, gs):
            p.grad = g
        for (_, p), g in zip(pb, gs):
            p.grad = g
        oa.step()
        ob.step()
        # an offloading wrapper parks the state on the host after every step
        for _, p in pb:
            st = ob.state[p]
            for k, v in list(st.items()):
                if torch.is_tensor(v):
                    st[k] = v.cpu()
    for (n, a), (_, b) in zip(pa, pb):
        torch.testing.assert_close(a.float(), b.float(), rtol=0, atol=1e-3, msg=n)
        assert torch.equal(oa.state[a]["m_codebook"].cpu(), ob.state[b]["m_codebook"].cpu()), n


def test_stochastic_rounding_is_seeded_by_step_and_stays_close_to_nearest():
    from gefen_x_b200 import Gefen

    def run(stochastic):
        ps = _params()
        opt = Gefen(ps, lr=1e-2, stochastic_round=stochastic)
        for step in range(3):
            for (_, p), g in zip(ps, _grads(ps, step)):
                p.grad = g
            opt.step()
        return ps, opt

    p1, o1 = run(True)
    p2, o2 = run(True)
    pn, on = run(False)
    # the rounding hash is seeded by the step count: two identical runs agree bit for bit
    assert all(torch.equal(o1.state[a]["m_codebook"], o2.state[b]["m_codebook"])
               for (_, a), (_, b) in zip(p1, p2))
    cb = on._gefen_codebook_on(_dev())
    moved = 0
    for (_, a), (_, b) in zip(p1, pn):
        ia, ib = o1.state[a]["m_codebook"].long(), on.state[b]["m_codebook"].long()
        moved += int((ia != ib).sum())
        assert int((ia - ib).abs().max()) <= 16         # nearby codewords (the runs drift apart a little)
        assert (cb[ia] - cb[ib]).abs().mean().item() < 0.02
    assert moved > 0


def test_fast_path_notices_paged_state_and_replaced_parameters_with_stable_gradients():
    """Gradients accumulated in place keep their addresses from step to step, so only the plan
    check stands between a remembered launch plan and state / parameter storage that was replaced
    in the meantime (state parked on the host by an offload wrapper, ``p.data`` re-assigned,
    betas edited): each of these must send the step back through the full path."""
    from gefen_x_b200 import Gefen

    pa, pb = _params(), _params()
    oa = Gefen(pa, lr=1e-2)
    ob = Gefen(pb, lr=1e-2)
    for ps in (pa, pb):
        for _, p in ps:
            p.grad = torch.zeros_like(p)
    for step in range(8):
        gs = _grads(pa, step)
        for ps in (pa, pb):
            for (_, p), g in zip(ps, gs):
                p.grad.copy_(g)                       # in place: the gradient pointers never change
        if step == 5:
            for o in (oa, ob):
                o.param_groups[0]["beta1"] = 0.8
        oa.step()
        ob.step()
        if step >= 2:
            assert oa._fast is not None               # the undisturbed optimizer stays on the fast path
        if step in (2, 3):
            for _, p in pb:                           # park the state on the host, as an offloader does
                st = ob.state[p]
                for k, v in list(st.items()):
                    if torch.is_tensor(v):
                        st[k] = v.cpu()
        if step == 4:
            for _, p in pb:                           # new storage for the parameters, same values
                p.data = p.data.clone()
    for (n, a), (_, b) in zip(pa, pb):
        assert torch.equal(a, b), n
        assert torch.equal(oa.state[a]["m_codebook"], ob.state[b]["m_codebook"].to(_dev())), n
        assert torch.equal(oa.state[a]["m_magnitude"], ob.state[b]["m_magnitude"].to(_dev())), n
    assert all(v == 0 for v in ob.kernel_status().values())


def test_stochastic_rounding_under_cuda_graph_replay_draws_fresh_noise():
    """The rounding seed of a capturable optimizer lives on the device and advances inside the
    captured region: two replays over the same gradient must not repeat the same rounding
    decisions, and a replayed run equals the eager capturable run step by step."""
    from gefen_x_b200 import Gefen

    pa, pb = _params(seed=3), _params(seed=3)
    oa = Gefen(pa, lr=1e-2, stochastic_round=True, capturable=True)     # eager oracle
    ob = Gefen(pb, lr=1e-2, stochastic_round=True, capturable=True)     # graph replays
    for ps in (pa, pb):
        for _, p in ps:
            p.grad = torch.zeros_like(p)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for step in range(3):
            gs = _grads(pa, step)
            for ps, o in ((pa, oa), (pb, ob)):
                for (_, p), g in zip(ps, gs):
                    p.grad.copy_(g)
                o.step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ob.step()
    oa.step()                                         # capture records the step without running it
    graph.replay()
    torch.cuda.synchronize()
    fixed = _grads(pa, 50)
    snaps = []
    for rep in range(2):
        for ps in (pa, pb):
            for (_, p), g in zip(ps, fixed):
                p.grad.copy_(g)
        before = {n: ob.state[p]["m_codebook"].clone() for n, p in pb}
        mags = {n: ob.state[p]["m_magnitude"].clone() for n, p in pb}
        oa.step()
        graph.replay()
        torch.cuda.synchronize()
        snaps.append({n: ob.state[p]["m_codebook"].clone() for n, p in pb})
        for (n, a), (_, b) in zip(pa, pb):
            assert torch.equal(oa.state[a]["m_codebook"], ob.state[b]["m_codebook"]), (rep, n)
        # restore the momentum so that the second replay quantises exactly the same values
        if rep == 0:
            for o, ps in ((oa, pa), (ob, pb)):
                for n, p in ps:
                    o.state[p]["m_codebook"].copy_(before[n])
                    o.state[p]["m_magnitude"].copy_(mags[n])
    differing = sum(int((snaps[0][n] != snaps[1][n]).sum()) for n, _ in pb)
    assert differing > 0, "two replays made identical rounding decisions: the seed is frozen in the graph"


def test_requantise_and_dense_dequantise_kernels():
    """Index remap onto a new codebook and the dense momentum export against their torch statements."""
    from gefen_x_b200 import Gefen
    from gefen_x_b200.ckpt.dcp import dense_momentum
    from gefen_x_b200.ops import quant as Q
    from gefen_x_b200.quant import codebook as C

    dev = _dev()
    g = torch.Generator().manual_seed(4)
    for numel, period in ((1 << 16, 256), (1000 * 24, 24), (4099 * 3, 3)):
        idx = torch.randint(0, 256, (numel,), generator=g, dtype=torch.uint8).to(dev)
        mag = torch.rand(numel // period, generator=g).to(dev)
        cb = torch.sort(torch.rand(256, generator=g) * 2 - 1).values.to(dev)
        for dt in (torch.float32, torch.bfloat16):
            got = Q.dequantize(idx, mag, cb, period, dt)
            want = (cb[idx.long()].view(-1, period) * mag[:, None]).reshape(-1)
            assert torch.allclose(got.float(), want.to(dt).float(), atol=0, rtol=0)
        perm = torch.randperm(256, generator=g).to(torch.uint8)
        want = perm.to(dev)[idx.long()]
        assert torch.equal(Q.remap_indices_(idx.clone(), perm), want)
    # through the optimizer: a refresh re-learns the codebook and remaps in place
    ps = _params()
    opt = Gefen(ps, lr=1e-2, codebook_refresh_every=2)
    for step in range(4):
        for (_, p), gr in zip(ps, _grads(ps, step)):
            p.grad = gr
        before = {n: opt.state[p]["m_codebook"].clone() for n, p in ps} if step == 2 else None
        old_cb = opt._gefen_codebook.clone() if step == 2 else None
        opt.step()
    assert opt._gefen_global_step == 4
    st = opt.state[ps[0][1]]
    dm = dense_momentum(opt._gefen_codebook, st, ps[0][1].shape)
    want = C.dequantize_indices(opt._gefen_codebook.to(dev), st["m_codebook"]) * st["m_magnitude"]
    assert torch.equal(dm.reshape(-1), want.reshape(-1))


def test_deterministic_policy_is_replica_exact():
    """deterministic=True: two replicas stepping the same data agree bit for bit, run after run
    (reference tests/test_deterministic_mode.py: replica hashes)."""
    from gefen_x_b200 import Gefen

    def run():
        g = torch.Generator().manual_seed(0)
        shapes = [("a.weight", (512, 2048)), ("b.weight", (1024, 512)), ("flat", (1 << 20,)), ("bias", (40,))]
        ps = [(n, (torch.randn(s, generator=g) * 0.05).bfloat16().to(_dev()).requires_grad_()) for n, s in shapes]
        opt = Gefen(ps, lr=1e-2, weight_decay=0.01, deterministic=True)
        for step in range(4):
            gg = torch.Generator().manual_seed(100 + step)
            for _, p in ps:
                p.grad = (torch.randn(p.shape, generator=gg) * 1e-2).bfloat16().to(_dev())
            opt.step()
        return ps, opt

    (pa, oa), (pb, ob) = run(), run()
    for (n, a), (_, b) in zip(pa, pb):
        assert torch.equal(a, b), n
        for key in ("m_codebook", "m_magnitude"):
            assert torch.equal(oa.state[a][key], ob.state[b][key]), (n, key)
        vk = "v_row" if "v_row" in oa.state[a] else "vmean"
        assert torch.equal(oa.state[a][vk], ob.state[b][vk]), (n, vk)
    assert oa.state_dict()["gefen_deterministic"] is True


def test_fp8_newton_schulz_on_the_fp8_gemm_tracks_bf16():
    """fp8_ns: e4m3 products through the library's row-scaled fp8 GEMM against the bf16
    iterations on the tcgen05 GEMM (reference tests/test_muon_combined_levers.py: a relative
    difference near 0.11 when fp8 engages, bit-equal results when the size gate turns it off)."""
    from gefen_x_b200.optim import newton_schulz as NS

    g = torch.Generator().manual_seed(7)
    for shape in ((2048, 3072), (3072, 1536)):
        m = torch.randn(shape, generator=g).to(_dev())
        ref = NS.zeropower_via_newtonschulz(m, ns_steps=5).float()
        got = NS.zeropower_via_newtonschulz(m, ns_steps=5, use_fp8=True).float()
        rel = float((got - ref).norm() / ref.norm())
        assert 1e-4 < rel < 0.2, (shape, rel)             # engaged (not bit-equal) and close
        assert float(torch.linalg.matrix_norm(got, ord=2)) < 1.4
    small = torch.randn(512, 1024, generator=g).to(_dev())
    assert torch.equal(NS.zeropower_via_newtonschulz(small, ns_steps=5, use_fp8=True),
                       NS.zeropower_via_newtonschulz(small, ns_steps=5))


def test_e4m3_row_quantisation_kernel_matches_the_torch_statement():
    from gefen_x_b200.ops.quant import quantize_cols_e4m3_t, quantize_rows_e4m3
    from gefen_x_b200.optim.newton_schulz import quantize_rowwise_fp8

    g = torch.Generator().manual_seed(11)
    for rows, cols in ((64, 128), (300, 14336), (33, 2056)):
        wide = (torch.randn(rows, cols + 8, generator=g) * torch.rand(rows, 1, generator=g) * 3).bfloat16().to(_dev())
        x = wide[:, :cols]                                   # row stride != cols
        x[0].zero_()                                         # an all-zero row: scale clamps, q = 0
        q, sc, y = quantize_rows_e4m3(x)
        qr, sr = quantize_rowwise_fp8(x)
        assert y is None and torch.equal(sc, sr)
        assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
        x2 = torch.randn(rows, cols, generator=g).bfloat16().to(_dev())
        q, sc, y = quantize_rows_e4m3(x, x2, 3.4445, -4.775, want_y=True)
        want = (3.4445 * x.float() + -4.775 * x2.float()).bfloat16()
        torch.testing.assert_close(y.float(), want.float(), rtol=1e-2, atol=1e-6)   # fma vs two roundings: 1 ulp
        qr, sr = quantize_rowwise_fp8(y)
        assert torch.equal(sc, sr) and torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
    for rows, cols in ((128, 64), (4096, 1536), (208, 2056), (16, 16)):
        x = (torch.randn(rows, cols + 8, generator=g) * torch.rand(1, cols + 8, generator=g) * 3).bfloat16().to(_dev())
        x = x[:, :cols]
        x[:, 3].zero_()
        qt, st = quantize_cols_e4m3_t(x)
        qr, sr = quantize_rowwise_fp8(x.t().contiguous())
        assert torch.equal(st, sr), (rows, cols)
        assert torch.equal(qt.view(torch.uint8), qr.view(torch.uint8)), (rows, cols)

@pytest.mark.parametrize("kind", ["muon", "hybrid"])
def test_muon_and_hybrid_cuda_graph_replay_match_eager(kind):
    """``GefenMuon`` / ``GefenMuonHybrid`` with ``capturable=True``: a captured step replays with the
    same result as eager steps, the learning rate is a device tensor that is changed in place between
    replays and never read back to the host (reference ``tests/test_capturable.py``,
    ``gefen_muon.py:1243-1300``)."""
    from gefen_x_b200 import GefenMuon, GefenMuonHybrid

    def params():
        g = torch.Generator().manual_seed(1)
        shapes = [("layers.0.q.weight", (128, 256)), ("layers.0.up.weight", (256, 128)),
                  ("layers.1.q.weight", (128, 256))]
        if kind == "hybrid":
            shapes += [("embed_tokens.weight", (64, 128)), ("norm.weight", (128,))]
        return [(n, (torch.randn(s, generator=g) * 0.05).bfloat16().to(_dev()).requires_grad_()) for n, s in shapes]

    def build(ps, lr):
        if kind == "muon":
            return GefenMuon(ps, lr=lr, weight_decay=0.05, capturable=True, normuon=True)
        return GefenMuonHybrid(ps, lr=lr, weight_decay=0.05, capturable=True)

    pa, pb = params(), params()
    lra = torch.tensor(2e-2, device=_dev())
    lrb = torch.tensor(2e-2, device=_dev())
    oa, ob = build(pa, lra), build(pb, lrb)
    for ps in (pa, pb):
        for _, p in ps:
            p.grad = torch.zeros_like(p)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for step in range(2):
            gs = _grads(pa, step)
            for ps, o in ((pa, oa), (pb, ob)):
                for (_, p), g in zip(ps, gs):
                    p.grad.copy_(g)
                o.step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ob.step()
    for step in range(2, 6):
        if step == 4:
            lra.fill_(5e-3)
            lrb.fill_(5e-3)                              # picked up by the replay: the lr is read on the device
        gs = _grads(pa, step)
        for ps in (pa, pb):
            for (_, p), g in zip(ps, gs):
                p.grad.copy_(g)
        oa.step()
        graph.replay()
    torch.cuda.synchronize()
    moved = 0.0
    start = params()
    for (n, a), (_, b), (_, p0) in zip(pa, pb, start):
        torch.testing.assert_close(a.float(), b.float(), rtol=0, atol=2e-3, msg=n)
        moved += (a.float() - p0.float()).abs().max().item()
    assert moved > 1e-2


def test_non_contiguous_parameter_steps_like_its_contiguous_copy():
    """A parameter that is a transposed view (what a non-contiguous local shard looks like to the
    optimizer): the kernels run on a contiguous copy and the result is copied back; trajectory and
    state equal those of a contiguous parameter with the same values (reference ``gefen.py:3703-3732``,
    tests/test_fused_fsdp2_noncontig.py)."""
    from gefen_x_b200 import Gefen

    g = torch.Generator().manual_seed(4)
    base = (torch.randn(256, 128, generator=g) * 0.05).bfloat16().to(_dev())
    pa = base.clone().t().contiguous().requires_grad_()          # [128, 256] contiguous
    pb = base.clone().t().requires_grad_()                       # the same values, strides (1, 128)
    assert not pb.is_contiguous()
    oa, ob = Gefen([("w", pa)], lr=1e-2, weight_decay=0.01), Gefen([("w", pb)], lr=1e-2, weight_decay=0.01)
    for step in range(4):
        gr = (torch.randn(128, 256, generator=torch.Generator().manual_seed(70 + step)) * 1e-2).bfloat16().to(_dev())
        pa.grad = gr.clone()
        pb.grad = gr.t().contiguous().t()                        # a non-contiguous gradient as well
        oa.step()
        ob.step()
    assert not pb.is_contiguous()
    assert torch.equal(pa.detach(), pb.detach())
    assert torch.equal(oa.state[pa]["m_codebook"], ob.state[pb]["m_codebook"])
    torch.testing.assert_close(oa.state[pa]["v_row"], ob.state[pb]["v_row"], rtol=1e-5, atol=0)



@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_streamed_update_kernels_match_the_register_pipelined_ones_bit_for_bit(dtype):
    """Plans of 2-byte tensors with 16-element row alignment run the streamed kernels (rows arrive
    through shared-memory rings filled by bulk async copies), with 16 elements per thread when every
    block period is a multiple of 16 and 8 otherwise.  They keep the per-element arithmetic of the
    register-pipelined kernels, so indices and magnitudes are bit-identical and the second moments
    agree to the order of the atomics.  Shapes: a partial last
    column tile, rows that do not fill the last row step, narrow rows (several rows per step),
    1-D tensors, and more groups than tiles for the smallest plan."""
    from gefen_x_b200 import Gefen
    from gefen_x_b200.ops import update as U

    shapes = [("w0", (96, 2064)), ("w1", (1000, 4096)), ("w2", (2048, 1024)), ("w3", (324, 48)),
              ("w4", (64, 14336)), ("n0", (8192,)), ("n1", (4096,))]
    fixed_periods = {"w0": 16512, "w1": 512000, "w2": 2048, "w3": 1296, "w4": 7168, "n0": 1024, "n1": 512}

    def run(streaming, shp, wide=True):
        U.set_streaming(streaming)
        U.set_wide_chunks(wide)
        try:
            g = torch.Generator().manual_seed(3)
            ps = [(n, (torch.randn(s, generator=g) * 0.05).to(dtype).to(_dev()).requires_grad_()) for n, s in shp]
            opt = Gefen(ps, lr=1e-2, weight_decay=0.01)
            # fixed block periods (the search would pick them from the data): one of each kind of
            # block-to-row relation, all multiples of 16 as the widest kernels need
            opt._predict_period_from_grad_sq = lambda name, p, grad: fixed_periods[name]
            for step in range(4):
                gg = torch.Generator().manual_seed(50 + step)
                for _, p in ps:
                    p.grad = (torch.randn(p.shape, generator=gg) * 1e-2).to(dtype).to(_dev())
                opt.step()
            torch.cuda.synchronize()
            assert all(v == 0 for v in opt.kernel_status().values())
            kinds = sorted({pl.fast for pl in opt._plan_cache._plans.values() if pl.kind == "factored"})
            return ps, opt, kinds
        finally:
            U.set_streaming(True)
            U.set_wide_chunks(False)

    for shp in (shapes, shapes[3:4]):
        pb, ob, kb = run(False, shp)
        # streamed kernels with 16 and with 8 elements per thread against the register-pipelined ones
        for wide, want in ((True, [4]), (False, [3])):
            pa, oa, ka = run(True, shp, wide)
            periods = {n: int(oa.state[a]["automatic_period"]) for n, a in pa}
            assert ka == want and kb == [1], (ka, kb, periods)
            for (n, a), (_, b) in zip(pa, pb):
                # the statistics are summed with atomics in all kernels: a parameter may round the other way
                torch.testing.assert_close(a.float(), b.float(), rtol=0, atol=1e-3, msg=n)
                assert (a != b).float().mean().item() < 1e-3, n
                sa, sb = oa.state[a], ob.state[b]
                assert torch.equal(sa["m_codebook"], sb["m_codebook"]), n
                assert torch.equal(sa["m_magnitude"], sb["m_magnitude"]), n
                for key in ("v_row", "v_col", "vmean"):
                    if key in sa:
                        torch.testing.assert_close(sa[key], sb[key], rtol=2e-5, atol=1e-12, msg=n + key)


def test_pre_launch_hook_tells_heavy_host_preparation_from_a_plan_rebuild():
    """The sharded runtime aligns its ranks with a host barrier only before steps that all ranks
    prepare at length (period search, codebook learning); a step that merely rebuilds a launch plan,
    which can happen on one rank alone, reports ``heavy=False`` so that nobody waits in a barrier the
    others never enter."""
    from gefen_x_b200 import Gefen

    ps = _params()
    opt = Gefen(ps, lr=1e-2)
    calls = []
    opt._pre_launch_hook = lambda heavy: calls.append(bool(heavy))
    for _, p in ps:
        p.grad = torch.zeros_like(p)
    for step in range(6):
        for (_, p), g in zip(ps, _grads(ps, step)):
            p.grad.copy_(g)
        if step == 4:
            for _, p in ps:
                p.data = p.data.clone()            # invalidates the remembered plan: full path, light
        opt.step()
    assert calls[0] is True                        # first step: periods and codebook
    assert calls[1:] and not any(calls[1:])        # later full-path steps only rebuild plans
    assert len(calls) < 6                          # the steady state in between took the fast path
