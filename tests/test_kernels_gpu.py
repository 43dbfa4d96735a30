"""GPU parity tests: every sm_100a kernel against a plain torch fp32 statement of the same op.

Model: reference tests/test_fused_update_v2_full_parity.py (bit patterns for the
quantised momentum, tolerance where reduction order differs),
tests/test_gefen_factored_v.py, tests/test_factored_v_ema_parity.py,
tests/test_find_period_backend.py.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _pair(shape, dtype, seed):
    """Two optimizers (kernel vs decomposed torch) on identical params."""
    from gefen_x_b200 import Gefen

    g = torch.Generator().manual_seed(seed)
    base = (torch.randn(shape, generator=g) * 0.05).to(dtype)
    pa = base.clone().to(_dev()).requires_grad_()
    pb = base.clone().to(_dev()).requires_grad_()
    return pa, pb, g


@pytest.mark.parametrize("shape,dtype", [
    ((256, 512), torch.bfloat16), ((96, 1000), torch.float32), ((64, 24), torch.bfloat16),
    ((300, 328), torch.float16), ((8, 4096), torch.bfloat16), ((33, 7), torch.float32),
])
@pytest.mark.parametrize("factored", [True, False])
def test_update_kernels_match_decomposed(shape, dtype, factored):
    from gefen_x_b200 import Gefen

    pa, pb, g = _pair(shape, dtype, 1)
    kw = dict(lr=1e-2, weight_decay=0.05, factored_v_2d=factored)
    oa = Gefen([("w", pa)], fused=True, **kw)
    ob = Gefen([("w", pb)], fused=False, **kw)
    for step in range(4):
        grad = (torch.randn(shape, generator=g) * 1e-3).to(dtype).to(_dev())
        pa.grad = grad.clone()
        pb.grad = grad.clone()
        if step == 0:
            ob.step()
            # share the first-step analysis so that both sides use one codebook / period
            oa._set_codebook(ob._gefen_codebook.clone())
            oa.state[pa]["automatic_period"] = ob.state[pb]["automatic_period"]
            oa.step()
        else:
            oa.step()
            ob.step()
        sa, sb = oa.state[pa], ob.state[pb]
        assert sa["automatic_period"] == sb["automatic_period"]
        assert torch.equal(sa["m_magnitude"], sb["m_magnitude"]), "magnitudes differ at step %d" % step
        mism = (sa["m_codebook"] != sb["m_codebook"]).float().mean().item()
        assert mism == 0.0, "index mismatch fraction %g at step %d" % (mism, step)
        if factored and len(shape) == 2:
            assert torch.allclose(sa["v_row"], sb["v_row"], rtol=2e-5, atol=1e-12)
            assert torch.allclose(sa["v_col"], sb["v_col"], rtol=2e-5, atol=1e-12)
        else:
            assert torch.allclose(sa["vmean"], sb["vmean"], rtol=2e-5, atol=1e-12)
        tol = 1e-6 if dtype == torch.float32 else 1e-2
        assert torch.allclose(pa.float(), pb.float(), rtol=tol, atol=tol * 0.05)
    torch.cuda.synchronize()
    assert all(v == 0 for v in oa.kernel_status().values())


@pytest.mark.parametrize("shape,period,factored", [
    ((64, 4096), 131072, True),      # two blocks spanning 32 rows each
    ((64, 4096), 131072, False),     # same through the two-phase block path
    ((1 << 20,), 1 << 19, False),    # flat tensor, two long blocks
    ((48, 2048), 1024, True),        # period divides the row
    ((96, 2048), 3072, True),        # vector path, block boundaries fall inside rows (and inside warps)
    ((96, 4096), 6144, True),        # same with two warps per row
    ((100, 24), 40, True),           # scalar path, blocks straddle rows
])
def test_update_kernels_forced_periods(shape, period, factored):
    from gefen_x_b200 import Gefen

    pa, pb, g = _pair(shape, torch.bfloat16, 11)
    kw = dict(lr=1e-2, weight_decay=0.01, factored_v_2d=factored)
    oa = Gefen([("w", pa)], fused=True, **kw)
    ob = Gefen([("w", pb)], fused=False, **kw)
    oa.state[pa]["automatic_period"] = period
    ob.state[pb]["automatic_period"] = period
    for step in range(3):
        grad = (torch.randn(shape, generator=g) * 1e-3).bfloat16().to(_dev())
        pa.grad = grad.clone()
        pb.grad = grad.clone()
        if step == 0:
            ob.step()
            oa._set_codebook(ob._gefen_codebook.clone())
        else:
            ob.step()
        oa.step()
        sa, sb = oa.state[pa], ob.state[pb]
        assert torch.equal(sa["m_magnitude"], sb["m_magnitude"])
        assert torch.equal(sa["m_codebook"], sb["m_codebook"])
        key = "v_row" if (factored and len(shape) == 2) else "vmean"
        assert torch.allclose(sa[key], sb[key], rtol=5e-5, atol=1e-12)
        assert torch.allclose(pa.float(), pb.float(), rtol=1e-2, atol=5e-4)


def test_first_step_analysis_on_gpu_matches_cpu():
    from gefen_x_b200.ops import quant as Q
    from gefen_x_b200.quant import codebook as C
    from gefen_x_b200.quant import partitioning as P

    g = torch.Generator().manual_seed(3)
    x = (torch.randn(96 * 80, generator=g) * 1e-3)
    xd = x.to(_dev())
    for period in (1, 8, 80, 96 * 80 // 2):
        want = C.block_normalised_histogram(x, period)
        got = Q.histogram(xd, period).cpu()
        assert torch.equal(want, got), period
    for dt in (torch.bfloat16, torch.float32):
        xs = x.to(dt)
        divs = P.divisors(xs.numel())
        want = P.block_variance_errors(xs.float().square().double(), divs)
        got = Q.period_errors(xs.to(_dev()), divs, input_is_squared=False)
        for a, b in zip(want, got):
            assert abs(a - b) <= 1e-6 * max(abs(a), 1e-12) + 1e-14
    # end to end: same period on both backends
    p_cpu = P.find_period_by_block_variance(x.square(), print_results=False, backend="cpu",
                                            parameter_shape=(96, 80))
    p_gpu = P.find_period_by_block_variance(xd, print_results=False, backend="cuda_kernel",
                                            parameter_shape=(96, 80), input_is_squared=False)
    assert p_cpu == p_gpu


def test_multi_source_gradient_and_clip_scale():
    """Peer-slice summation (here: 4 local buffers) fused into the update == update on their mean."""
    from gefen_x_b200 import Gefen
    from gefen_x_b200.ops import update as U

    shape = (128, 256)
    g = torch.Generator().manual_seed(5)
    base = (torch.randn(shape, generator=g) * 0.05).bfloat16()
    pa = base.clone().to(_dev())
    pb = base.clone().to(_dev())
    srcs = [(torch.randn(shape, generator=g) * 1e-3).bfloat16().to(_dev()) for _ in range(4)]
    mean = (sum(s.float() for s in srcs) * 0.25).bfloat16()
    coef = torch.tensor([0.5], device=_dev())
    oa = Gefen([("w", pa)], lr=1e-2)
    ob = Gefen([("w", pb)], lr=1e-2)
    peer = U.PeerGrad(ptrs=[s.data_ptr() for s in srcs], shape=shape, dtype=torch.bfloat16,
                      device=_dev(), scale=0.25)
    assert torch.equal(peer.materialize(), mean)
    oa._grad_source = lambda p: peer
    ob._grad_source = lambda p: U.LocalGrad(mean)
    oa._external_grad_scale = coef
    ob._external_grad_scale = coef
    for _ in range(3):
        oa.step()
        ob.step()
    assert torch.equal(oa.state[pa]["m_codebook"], ob.state[pb]["m_codebook"])
    # the column statistics are summed with atomics across CTAs (order not fixed), so the second
    # moment, and with it the parameters, may differ in the last bit between two runs
    torch.testing.assert_close(pa.float(), pb.float(), rtol=1.6e-2, atol=1e-5)
    # partial sums of squares + clip coefficient
    partials = torch.zeros(512, device=_dev())
    out = torch.empty(shape, dtype=torch.bfloat16, device=_dev())
    U.reduce_sources(out, [s.data_ptr() for s in srcs], out.numel(), 0.25, partials,
                     torch.bfloat16, _dev())
    assert torch.equal(out, mean)
    cc = torch.zeros(2, device=_dev())
    U.clip_coef(partials, 1e-3, cc)
    norm = mean.float().square().sum().sqrt().item()
    assert abs(cc[1].item() - norm) < 1e-4 * norm
    assert abs(cc[0].item() - min(1.0, 1e-3 / (norm + 1e-6))) < 1e-5


def test_model_kernels_match_torch():
    from gefen_x_b200.ops import model as M

    g = torch.Generator().manual_seed(7)
    dev = _dev()
    for d, rows in ((2560, 37), (128, 1000), (4096, 16), (64, 5)):
        x = torch.randn(rows, d, generator=g).bfloat16().to(dev)
        w = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16().to(dev)
        dy = torch.randn(rows, d, generator=g).bfloat16().to(dev)
        y, rstd = M.rmsnorm_fwd(x, w, 1e-6)
        ref = M.rmsnorm_ref(x.float(), w.float(), 1e-6)
        assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2)
        dx, dw = M.rmsnorm_bwd(dy, x, w, rstd)
        xr = x.float().requires_grad_()
        wr = w.float().requires_grad_()
        M.rmsnorm_ref(xr, wr, 1e-6).backward(dy.float())
        assert torch.allclose(dx.float(), xr.grad, rtol=3e-2, atol=3e-2)
        assert torch.allclose(dw, wr.grad, rtol=2e-2, atol=5e-2)
        # the residual-path gradient added inside the kernel
        res = torch.randn(rows, d, generator=g).bfloat16().to(dev)
        dx2, dw2 = M.rmsnorm_bwd(dy, x, w, rstd, res=res)
        assert torch.allclose(dx2.float(), xr.grad + res.float(), rtol=3e-2, atol=3e-2)
        assert torch.equal(dw2, dw)
    # rope (both layouts, forward then inverse is the identity up to bf16 rounding)
    B, S, n, hd = 2, 33, 4, 128
    cos, sin = M.rope_tables(S, hd, 1e6, dev)
    for inter in (False, True):
        x = torch.randn(B, S, n, hd, generator=g).to(dev)
        ref = M.rope_ref(x, cos, sin, interleaved=inter)
        got = M.rope_(x.clone(), cos, sin, interleaved=inter)
        assert torch.allclose(got, ref, atol=1e-5)
        back = M.rope_(got.clone(), cos, sin, inverse=True, interleaved=inter)
        assert torch.allclose(back, x, atol=1e-5)
        # strided source / destination (column slices of a fused buffer), bf16, and an odd head size
        for dt, hd2 in ((torch.bfloat16, 128), (torch.float32, 24)):
            c2, s2 = M.rope_tables(S, hd2, 1e6, dev)
            fused = torch.randn(B * S, 3 * n * hd2 + 8, generator=g).to(dt).to(dev)
            src = fused[:, n * hd2:2 * n * hd2]
            out = torch.zeros(B * S, 2 * n * hd2, dtype=dt, device=dev)
            M.rope_into(out[:, n * hd2:], src, c2, s2, S, n, hd2, interleaved=inter)
            want = M.rope_ref(src.reshape(B, S, n, hd2), c2, s2, interleaved=inter).reshape(B * S, n * hd2)
            tol = 2e-2 if dt == torch.bfloat16 else 1e-5
            assert torch.allclose(out[:, n * hd2:].float(), want.float(), atol=tol)
            assert float(out[:, :n * hd2].abs().max()) == 0.0
    # swiglu
    gu = torch.randn(50, 2 * 688, generator=g).bfloat16().to(dev)
    dz = torch.randn(50, 688, generator=g).bfloat16().to(dev)
    gur = gu.float().requires_grad_()
    out_ref = torch.nn.functional.silu(gur[:, :688]) * gur[:, 688:]
    out_ref.backward(dz.float())
    assert torch.allclose(M.swiglu_fwd(gu).float(), out_ref, rtol=2e-2, atol=2e-2)
    assert torch.allclose(M.swiglu_bwd(gu, dz).float(), gur.grad, rtol=3e-2, atol=3e-2)
    # cross-entropy forward + in-place gradient
    for V in (1024, 151936, 1003):
        T = 9
        logits = (torch.randn(T, V, generator=g) * 2).bfloat16().to(dev)
        tgt = torch.randint(0, V, (T,), generator=g).to(dev)
        tgt[3] = -100
        lr = logits.float().requires_grad_()
        loss_ref = torch.nn.functional.cross_entropy(lr, tgt, ignore_index=-100, reduction="none")
        (loss_ref.sum() * 0.125).backward()
        work = logits.clone()
        loss = M.xent_fwd_bwd_(work, tgt, 0.125)
        assert torch.allclose(loss, loss_ref, rtol=1e-3, atol=1e-3)
        assert torch.allclose(work.float(), lr.grad, rtol=2e-2, atol=2e-3)


def test_decoder_kernel_path_matches_torch_path():
    from gefen_x_b200.models.decoder import DecoderLM, get_config

    cfg = get_config("tiny-llama", qk_norm=True)
    ref = DecoderLM(cfg, device=_dev(), dtype=torch.float32, impl="torch", seed=3)
    ker = DecoderLM(cfg, device=_dev(), dtype=torch.bfloat16, impl="kernel", seed=3)
    g = torch.Generator().manual_seed(9)
    tok = torch.randint(0, 1024, (2, 65), generator=g).to(_dev())
    l_ref = ref(tok[:, :-1], tok[:, 1:])
    l_ker = ker(tok[:, :-1], tok[:, 1:])
    l_ref.backward()
    l_ker.backward()
    assert abs(l_ref.item() - l_ker.item()) < 3e-2
    for (n, a), (_, b) in zip(ref.named_parameters(), ker.named_parameters()):
        denom = a.grad.abs().max().item() + 1e-6
        assert (a.grad - b.grad.float()).abs().max().item() / denom < 0.08, n


def test_sharded_trainer_single_gpu_tracks_cpu_fp32():
    from gefen_x_b200.models.decoder import get_config
    from gefen_x_b200.parallel.fsdp import ShardedTrainer

    cfg = get_config("tiny-llama")
    g = torch.Generator().manual_seed(2)
    tok = torch.randint(0, 1024, (4, 129), generator=g)
    cpu = ShardedTrainer(cfg, device="cpu", dtype=torch.float32, lr=6e-4, weight_decay=0.01,
                         clip_grad_norm=1.0, seed=5)
    gpu = ShardedTrainer(cfg, device=_dev(), dtype=torch.bfloat16, lr=6e-4, weight_decay=0.01,
                         clip_grad_norm=1.0, seed=5)
    lc, lg = [], []
    for _ in range(20):
        lc.append(cpu.step(tok[:, :-1], tok[:, 1:]).item())
        lg.append(gpu.step(tok[:, :-1].pin_memory(), tok[:, 1:].pin_memory()).item())
    gpu.check_status()
    assert lg[-1] < lg[0] - 0.5
    assert abs(lc[-1] - lg[-1]) / lc[-1] < 0.12, (lc, lg)   # bf16 vs fp32 after 20 steps
    assert gpu.state_bytes_per_param() < 1.1


@pytest.mark.parametrize("m,n,k,a_t,b_t", [
    (256, 512, 128, False, False), (128, 256, 64, False, False), (300, 264, 200, False, False),
    (2048, 6144, 2560, False, False), (256, 512, 128, False, True), (256, 512, 128, True, False),
    (256, 512, 128, True, True), (1024, 1024, 4096, False, True), (520, 136, 328, True, True),
])
def test_tcgen05_gemm_matches_fp32(m, n, k, a_t, b_t):
    from gefen_x_b200.ops import tcgemm

    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn((k, m) if a_t else (m, k), generator=g).bfloat16().to(_dev())
    b = torch.randn((k, n) if b_t else (n, k), generator=g).bfloat16().to(_dev())
    d = torch.randn(m, n, generator=g).bfloat16().to(_dev())
    af = a.float().t() if a_t else a.float()
    bf = b.float() if b_t else b.float().t()
    ref = af @ bf
    tcgemm.set_pair_kernel(False)          # this test covers the single-CTA kernel
    try:
        out = tcgemm.gemm(a, b, a_t=a_t, b_t=b_t)
        out2 = tcgemm.gemm(a, b, a_t=a_t, b_t=b_t, alpha=0.5, beta=-2.0, d=d)
    finally:
        tcgemm.set_pair_kernel(True)
    torch.cuda.synchronize()
    assert int(tcgemm.status_word(_dev()).item()) == 0
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-2, err
    ref2 = 0.5 * ref - 2.0 * d.float()
    err2 = (out2.float() - ref2).abs().max().item()
    assert err2 <= 2e-2 * ref2.abs().max().item() + 1e-2, err2


@pytest.mark.parametrize("m,n,k,a_t,b_t,bn", [
    (512, 512, 256, False, False, 256), (512, 512, 256, False, False, 128), (256, 256, 64, False, False, 0),
    (1024, 768, 4096, False, False, 0), (300, 264, 200, False, False, 256), (520, 136, 328, True, True, 128),
    (512, 1024, 512, False, True, 256), (512, 1024, 512, True, False, 128), (768, 640, 1024, True, True, 256),
    (4096, 4096, 1024, False, False, 0), (129, 128, 64, False, True, 0), (1024, 768, 8192, True, True, 0),
    (4352, 4352, 512, False, False, 0),
])
def test_pair_gemm_matches_fp32(m, n, k, a_t, b_t, bn):
    """CTA-pair tcgen05 GEMM (cta_group::2) against the fp32 product, all operand layouts, both tile
    widths, ragged edges, and the alpha / beta * D epilogue."""
    from gefen_x_b200.ops import tcgemm

    g = torch.Generator().manual_seed(m + n + k + bn)
    a = torch.randn((k, m) if a_t else (m, k), generator=g).bfloat16().to(_dev())
    b = torch.randn((k, n) if b_t else (n, k), generator=g).bfloat16().to(_dev())
    d = torch.randn(m, n, generator=g).bfloat16().to(_dev())
    af = a.float().t() if a_t else a.float()
    bf = b.float() if b_t else b.float().t()
    ref = af @ bf
    assert tcgemm.pair_eligible(m, n, k)
    tcgemm.set_pair_kernel(True, bn)
    try:
        out = tcgemm.gemm(a, b, a_t=a_t, b_t=b_t)
        out2 = tcgemm.gemm(a, b, a_t=a_t, b_t=b_t, alpha=0.5, beta=-2.0, d=d)
        torch.cuda.synchronize()
    finally:
        tcgemm.set_pair_kernel(True, 0)
    assert int(tcgemm.status_word(_dev()).item()) == 0
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-2, err
    ref2 = 0.5 * ref - 2.0 * d.float()
    err2 = (out2.float() - ref2).abs().max().item()
    assert err2 <= 2e-2 * ref2.abs().max().item() + 1e-2, err2
    # sum of squares of the stored output from the epilogue: accumulates into the slots, and two runs
    # agree bit for bit (every slot has one writer, also for the K-split tail tiles)
    sq, sq2 = torch.zeros(2048, device=_dev()), torch.zeros(2048, device=_dev())
    out3 = tcgemm.gemm(a, b, a_t=a_t, b_t=b_t, sumsq=sq)
    tcgemm.gemm(a, b, a_t=a_t, b_t=b_t, sumsq=sq2)
    want = out3.float().square().sum().item()
    assert abs(sq.sum().item() - want) <= 1e-4 * want, (sq.sum().item(), want)
    assert torch.equal(sq, sq2)
    tcgemm.gemm(a, b, a_t=a_t, b_t=b_t, sumsq=sq)
    assert abs(sq.sum().item() - 2 * want) <= 2e-4 * want
    # the single-CTA kernel gives the same product
    tcgemm.set_pair_kernel(False)
    try:
        out1 = tcgemm.gemm(a, b, a_t=a_t, b_t=b_t)
    finally:
        tcgemm.set_pair_kernel(True, 0)
    assert (out1.float() - out.float()).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("m,f,k,h", [(512, 512, 256, 384), (300, 264, 320, 384), (1024, 1792, 512, 384),
                                     (512, 1024, 2048, 1024)])
def test_pair_gemm_swiglu_epilogues(m, f, k, h):
    """SwiGLU fused into the gate/up projection and its derivative fused into the down_proj input
    gradient, against the fp32 statement and against the unfused kernels."""
    from gefen_x_b200.ops import model as M
    from gefen_x_b200.ops import tcgemm

    g = torch.Generator().manual_seed(m + f + k)
    x = (torch.randn(m, k, generator=g) * 0.5).bfloat16().to(_dev())
    wgu = (torch.randn(2 * f, k, generator=g) * (k ** -0.5)).bfloat16().to(_dev())
    gu, act = tcgemm.gemm_swiglu_fwd(x, wgu)
    torch.cuda.synchronize()
    assert int(tcgemm.status_word(_dev()).item()) == 0
    gu_ref = x.float() @ wgu.float().t()
    assert (gu.float() - gu_ref).abs().max().item() <= 2e-2 * gu_ref.abs().max().item() + 1e-2
    # the activation is computed from the rounded gate / up values, like the separate kernel
    act_unfused = M.swiglu_fwd(gu)
    assert (act.float() - act_unfused.float()).abs().max().item() <= 1e-2 * act_unfused.float().abs().max().item() + 1e-3
    gr, ur = gu.float()[:, :f], gu.float()[:, f:]
    act_ref = torch.nn.functional.silu(gr) * ur
    assert (act.float() - act_ref).abs().max().item() <= 1e-2 * act_ref.abs().max().item() + 1e-3

    dy = (torch.randn(m, h, generator=g) * 0.5).bfloat16().to(_dev())
    wd = (torch.randn(h, f, generator=g) * (h ** -0.5)).bfloat16().to(_dev())
    dgu = tcgemm.gemm_swiglu_bwd(dy, wd, gu)
    torch.cuda.synchronize()
    assert int(tcgemm.status_word(_dev()).item()) == 0
    dact = (dy.float() @ wd.float()).bfloat16()
    dgu_unfused = M.swiglu_bwd(gu, dact)
    scale = dgu_unfused.float().abs().max().item()
    assert (dgu.float() - dgu_unfused.float()).abs().max().item() <= 2e-2 * scale + 1e-3


def test_tcgen05_gemm_batched():
    from gefen_x_b200.ops import tcgemm

    g = torch.Generator().manual_seed(0)
    a = torch.randn(5, 192, 320, generator=g).bfloat16().to(_dev())
    b = torch.randn(5, 136, 320, generator=g).bfloat16().to(_dev())
    out = tcgemm.gemm(a, b)
    ref = torch.bmm(a.float(), b.float().transpose(1, 2))
    torch.cuda.synchronize()
    assert int(tcgemm.status_word(_dev()).item()) == 0
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


@pytest.mark.parametrize("shape,dtype,nesterov", [((256, 512), torch.bfloat16, True),
                                                  ((96, 1000), torch.float32, False),
                                                  ((512, 264), torch.bfloat16, True)])
def test_muon_momentum_emit_kernel_matches_decomposed(shape, dtype, nesterov):
    from gefen_x_b200 import GefenMuon

    pa, pb, g = _pair(shape, dtype, 21)
    oa = GefenMuon([("w", pa)], lr=1e-2, fused=True, nesterov=nesterov)
    ob = GefenMuon([("w", pb)], lr=1e-2, fused=False, nesterov=nesterov)
    for step in range(3):
        grad = (torch.randn(shape, generator=g) * 1e-3).to(dtype).to(_dev())
        pa.grad = grad.clone()
        pb.grad = grad.clone()
        if step == 0:
            ob.step()
            oa._set_codebook(ob._gefen_codebook.clone())
            oa.state[pa]["automatic_period"] = ob.state[pb]["automatic_period"]
        else:
            ob.step()
        oa.step()
        sa, sb = oa.state[pa], ob.state[pb]
        assert torch.equal(sa["m_magnitude"], sb["m_magnitude"])
        assert torch.equal(sa["m_codebook"], sb["m_codebook"])
        # Newton-Schulz in bf16 on two GEMM back ends: compare the applied update loosely
        assert torch.allclose(pa.float(), pb.float(), rtol=2e-2, atol=2e-3)


def test_sharded_trainer_muon_hybrid_single_gpu():
    from gefen_x_b200.models.decoder import get_config
    from gefen_x_b200.parallel.fsdp import ShardedTrainer

    cfg = get_config("tiny-llama", qk_norm=True)
    g = torch.Generator().manual_seed(2)
    tok = torch.randint(0, 1024, (4, 129), generator=g).to(_dev())
    tr = ShardedTrainer(cfg, device=_dev(), dtype=torch.bfloat16, lr=2e-3, weight_decay=0.01,
                        clip_grad_norm=1.0, seed=5, optimizer="muon_hybrid")
    losses = [tr.step(tok[:, :-1], tok[:, 1:]).item() for _ in range(15)]
    tr.check_status()
    assert losses[-1] < losses[0] - 0.5, losses
    assert len(tr.muon.owned) == cfg.n_layers * 7
    assert tr.state_bytes_per_param() < 1.2


@pytest.mark.parametrize("B,S,nq,nkv,hd,flash", [(2, 128, 8, 2, 64, False), (1, 256, 4, 4, 128, False),
                                                 (2, 72, 6, 3, 128, False), (2, 128, 8, 2, 64, True),
                                                 (1, 384, 4, 4, 128, True), (2, 512, 8, 2, 128, True),
                                                 (1, 256, 6, 1, 64, True)])
def test_own_attention_matches_sdpa(B, S, nq, nkv, hd, flash):
    """Own attention (fused tcgen05 forward or GEMM-composed forward; GEMM-composed backward with own
    row kernels) against fp32 SDPA: output and all three gradients."""
    import torch.nn.functional as F

    from gefen_x_b200.ops import attention as A

    dev = _dev()
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, S, nq, hd, generator=g).bfloat16().to(dev)
    k = torch.randn(B, S, nkv, hd, generator=g).bfloat16().to(dev)
    v = torch.randn(B, S, nkv, hd, generator=g).bfloat16().to(dev)
    do = torch.randn(B, S, nq, hd, generator=g).bfloat16().to(dev)
    assert A.supported(q, k)
    assert not flash or A.flash_supported(S, hd)
    out, ctx = A.attention_fwd(q, k, v, flash=flash)
    dq, dk, dv = A.attention_bwd(ctx, do)
    from gefen_x_b200.ops import tcgemm

    assert int(tcgemm.status_word(dev).item()) == 0
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    ref = F.scaled_dot_product_attention(qr.transpose(1, 2), kr.transpose(1, 2), vr.transpose(1, 2),
                                         is_causal=True, enable_gqa=nq != nkv).transpose(1, 2)
    ref.backward(do.float())
    assert torch.allclose(out.float(), ref, atol=3e-2, rtol=3e-2)
    for got, want in ((dq, qr.grad), (dk, kr.grad), (dv, vr.grad)):
        err = (got.float() - want).abs().max().item()
        assert err < 0.06 * max(1.0, want.abs().max().item()), err


def test_decoder_trains_with_gemm_composed_attention():
    from gefen_x_b200.models.decoder import get_config
    from gefen_x_b200.ops import model as M
    from gefen_x_b200.parallel.fsdp import ShardedTrainer

    cfg = get_config("tiny-llama", hidden=256, ffn=512, n_layers=2)
    g = torch.Generator().manual_seed(2)
    tok = torch.randint(0, cfg.vocab_size, (2, 129), generator=g).to(_dev())

    def run(impl):
        M.set_attention_impl(impl)
        try:
            tr = ShardedTrainer(cfg, device=_dev(), dtype=torch.bfloat16, lr=6e-4, clip_grad_norm=1.0, seed=5)
            return [float(tr.step(tok[:, :-1], tok[:, 1:]).item()) for _ in range(8)]
        finally:
            M.set_attention_impl("sdpa")

    a, b = run("sdpa"), run("tcgen05")
    assert b[-1] < b[0] - 0.3
    for x, y in zip(a, b):
        assert abs(x - y) < 0.05 * max(1.0, abs(x)), (a, b)


def test_bounded_wait_runs_out_reports_and_leaves_the_gpu_usable():
    """A wait on a flag that nobody sets gives up after its iteration budget, records kWaitTimeout in the
    status word instead of trapping, and the context stays usable; the trainer turns the status word
    into a host-side error (reference contract: every rank raises, nothing hangs,
    tests/test_precollective_failure_sync.py:215-239)."""
    from gefen_x_b200.models.decoder import get_config
    from gefen_x_b200.ops._ext import ops
    from gefen_x_b200.parallel.fsdp import ShardedTrainer

    dev = _dev()
    flags = torch.zeros(4, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ops().comm_wait(flags, 4, 7, 2000, status)                 # the flags stay at 0: the budget runs out
    torch.cuda.synchronize()
    assert int(status.item()) == 1                             # kWaitTimeout
    x = torch.arange(1024, device=dev, dtype=torch.float32)
    assert float((x * 2).sum().item()) == 1023 * 1024          # later kernels run normally
    status.zero_()
    flags.fill_(7)
    ops().comm_wait(flags, 4, 7, 2000, status)                 # a satisfied wait leaves the status alone
    flags[2] = 9
    ops().comm_wait(flags, 4, 8, 2000, status)                 # one peer behind: times out again
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    tr = ShardedTrainer(get_config("tiny-llama"), device=dev, dtype=torch.bfloat16)
    tr.check_status()                                          # clean
    ops().comm_wait(torch.zeros(1, dtype=torch.int32, device=dev), 1, 5, 1000, tr.status)
    with pytest.raises(RuntimeError, match="bounded wait"):
        tr.check_status()


def test_operators_trace_under_torch_compile():
    """Fake implementations are registered for the kernel operators, so a compiled function may call
    them (no graph break), and a compiled optimizer step gives the eager result."""
    from gefen_x_b200 import Gefen
    from gefen_x_b200.ops._ext import ops

    dev = _dev()
    ops()                                                      # loads the library and registers the fakes
    g = torch.Generator().manual_seed(3)
    x = torch.randn(64, 256, generator=g).bfloat16().to(dev)
    w = (1 + 0.1 * torch.randn(256, generator=g)).bfloat16().to(dev)

    def norm(x, w):
        y = torch.empty_like(x)
        rstd = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
        torch.ops.gefenx.rmsnorm_fwd(x, w, y, rstd, 1e-6)
        return y * 2

    want = norm(x, w)
    got = torch.compile(norm, fullgraph=True)(x, w)
    torch.testing.assert_close(got, want)

    def params():
        gg = torch.Generator().manual_seed(5)
        return [("a.weight", (torch.randn(64, 256, generator=gg) * 0.05).bfloat16().to(dev).requires_grad_()),
                ("b", (torch.randn(512, generator=gg) * 0.05).bfloat16().to(dev).requires_grad_())]

    pa, pb = params(), params()
    oa, ob = Gefen(pa, lr=1e-2), Gefen(pb, lr=1e-2)
    compiled = torch.compile(ob.step, mode="reduce-overhead")
    for step in range(3):
        gg = torch.Generator().manual_seed(40 + step)
        for (_, a), (_, b) in zip(pa, pb):
            gr = (torch.randn(a.shape, generator=gg) * 1e-2).bfloat16().to(dev)
            a.grad, b.grad = gr.clone(), gr.clone()
        oa.step()
        compiled()
    for (n, a), (_, b) in zip(pa, pb):
        assert torch.equal(a, b), n
        assert torch.equal(oa.state[a]["m_codebook"], ob.state[b]["m_codebook"]), n


def test_pair_gemm_dynamic_schedule_matches_static():
    """The dynamic tile schedule (pairs draw units from a device counter through the shared-memory
    ring) computes exactly what the static one does: plain, K-split tail, fused SwiGLU epilogues,
    the gradient-norm sums (same total; placement varies), and the counter is back at zero after
    every launch (launch after launch on the same stream)."""
    from gefen_x_b200.ops import tcgemm

    g = torch.Generator().manual_seed(21)
    dev = _dev()
    shapes = [(4096, 4096, 1024, False, False), (1024, 768, 8192, True, True), (4352, 4352, 512, False, True),
              (300, 264, 200, False, False), (2048, 6144, 2560, False, False)]
    try:
        for m, n, k, a_t, b_t in shapes:
            a = torch.randn((k, m) if a_t else (m, k), generator=g).bfloat16().to(dev)
            b = torch.randn((k, n) if b_t else (n, k), generator=g).bfloat16().to(dev)
            d = torch.randn(m, n, generator=g).bfloat16().to(dev)
            tcgemm.set_dynamic_schedule(False)
            want = tcgemm.gemm(a, b, a_t=a_t, b_t=b_t, alpha=0.5, beta=1.0, d=d)
            sq0 = torch.zeros(2048, device=dev)
            tcgemm.gemm(a, b, a_t=a_t, b_t=b_t, sumsq=sq0)
            tcgemm.set_dynamic_schedule(True)
            for _ in range(3):                                     # repeated launches reuse the counter
                got = tcgemm.gemm(a, b, a_t=a_t, b_t=b_t, alpha=0.5, beta=1.0, d=d)
                assert torch.equal(got, want), (m, n, k)
            sq1 = torch.zeros(2048, device=dev)
            tcgemm.gemm(a, b, a_t=a_t, b_t=b_t, sumsq=sq1)
            assert abs(sq1.sum().item() - sq0.sum().item()) <= 1e-5 * sq0.sum().item()
        x = (torch.randn(1024, 512, generator=g) * 0.5).bfloat16().to(dev)
        wgu = (torch.randn(2 * 1792, 512, generator=g) * 0.05).bfloat16().to(dev)
        dy = (torch.randn(1024, 1024, generator=g) * 0.5).bfloat16().to(dev)
        wd = (torch.randn(1024, 1792, generator=g) * 0.03).bfloat16().to(dev)
        tcgemm.set_dynamic_schedule(False)
        gu0, act0 = tcgemm.gemm_swiglu_fwd(x, wgu)
        dgu0 = tcgemm.gemm_swiglu_bwd(dy, wd, gu0)
        tcgemm.set_dynamic_schedule(True)
        gu1, act1 = tcgemm.gemm_swiglu_fwd(x, wgu)
        dgu1 = tcgemm.gemm_swiglu_bwd(dy, wd, gu1)
        assert torch.equal(gu0, gu1) and torch.equal(act0, act1) and torch.equal(dgu0, dgu1)
        torch.cuda.synchronize()
        assert int(tcgemm.status_word(dev).item()) == 0
    finally:
        tcgemm.set_dynamic_schedule(False)



def test_pair_gemm_e4m3_row_scaled_matches_fp32_statement():
    """The e4m3 variant of the CTA-pair kernel (tcgen05 kind f8f6f4, scales in the epilogue) against the
    fp32 statement of the same quantised values: full and partial tiles, a K that does not fill its last
    128-byte row, a K-split tail wave, and both tile schedules."""
    from gefen_x_b200.ops import tcgemm

    g = torch.Generator().manual_seed(31)
    dev = _dev()
    try:
        for dynamic in (False, True):
            tcgemm.set_dynamic_schedule(dynamic)
            for m, n, k in [(4096, 4096, 1024), (300, 264, 208), (4352, 4352, 512), (2048, 1024, 4096), (129, 128, 128)]:
                a = torch.randn(m, k, generator=g)
                b = torch.randn(n, k, generator=g)
                sa = (a.abs().amax(1, keepdim=True) / 448.0).clamp_(min=1e-12)
                sb = (b.abs().amax(1, keepdim=True) / 448.0).clamp_(min=1e-12)
                aq = (a / sa).to(torch.float8_e4m3fn).to(dev)
                bq = (b / sb).to(torch.float8_e4m3fn).to(dev)
                want = ((aq.float() * sa.to(dev)) @ (bq.float() * sb.to(dev)).t())
                got = tcgemm.gemm_e4m3(aq, sa.to(dev), bq, sb.to(dev))
                assert got.dtype == torch.bfloat16 and got.shape == (m, n)
                err = (got.float() - want).abs().max().item()
                assert err <= 1e-2 * want.abs().max().item() + 1e-3, (m, n, k, dynamic, err)
        torch.cuda.synchronize()
        assert int(tcgemm.status_word(dev).item()) == 0
    finally:
        tcgemm.set_dynamic_schedule(False)


def test_fp8_newton_schulz_own_gemm_tracks_the_library_gemm():
    from gefen_x_b200.optim import newton_schulz as NS

    g = torch.Generator().manual_seed(5)
    x = torch.randn(1024, 2048, generator=g).bfloat16().to(_dev())
    try:
        NS.set_fp8_gemm("tcgen05")
        own = NS.zeropower_via_newtonschulz(x, ns_steps=5, use_fp8=True)
        NS.set_fp8_gemm("library")
        lib = NS.zeropower_via_newtonschulz(x, ns_steps=5, use_fp8=True)
    finally:
        NS.set_fp8_gemm("tcgen05")
    bf = NS.zeropower_via_newtonschulz(x, ns_steps=5, use_fp8=False)
    # same quantised operands, fp32 accumulation in both: the results agree far inside the fp8 error
    assert (own.float() - lib.float()).abs().max().item() <= 2e-2
    assert (own.float() - bf.float()).abs().mean().item() <= 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_muon_epilogue_kernels_match_the_torch_chain(dtype):
    """NorMuon row normalisation, the cautious mask and the parameter update in three launches
    (``csrc/muon_ops.cu``) against the chain of torch ops they replace (``GefenMuon._normuon_normalize``,
    ``cautious_mask_``, the apply), with the products rounded where torch rounds them: vector and
    scalar column counts, each feature alone and together, two steps (the second moment carries)."""
    from gefen_x_b200.ops._ext import ops
    from gefen_x_b200.optim.muon import cautious_mask_

    dev = _dev()
    g = torch.Generator().manual_seed(17)
    beta2, eps, lr_ratio, wdf = 0.95, 1e-8, 3e-3, 0.9997
    for rows, cols in [(512, 1024), (300, 264), (130, 100)]:
        for normuon, cautious in [(True, False), (False, True), (True, True)]:
            p0 = (torch.randn(rows, cols, generator=g) * 0.05).to(dtype).to(dev)
            p_ref, p_ker = p0.clone(), p0.clone()
            v_ref = torch.zeros(rows, 1, dtype=torch.float32, device=dev)
            v_ker = v_ref.clone()
            for step in (1, 2):
                u = (torch.randn(rows, cols, generator=g) * 0.3).to(dtype).to(dev)
                gr = torch.randn(rows, cols, generator=g).to(dtype).to(dev)
                bc = 1 - beta2 ** step
                # the torch chain
                ur = u.clone()
                if normuon:
                    row_norm = torch.linalg.vector_norm(ur, dim=1, keepdim=True, dtype=torch.float32)
                    row_sq = row_norm.square()
                    v_ref.mul_(beta2).add_(row_sq, alpha=(1 - beta2) / cols)
                    denom = (v_ref / bc).sqrt_().add_(eps)
                    frob = row_sq.sum().sqrt_() / torch.linalg.vector_norm(row_norm / denom).clamp(min=1e-38)
                    ur.mul_((frob / denom).to(dtype))
                if cautious:
                    ur = cautious_mask_(ur, gr)
                p_ref.mul_(wdf)
                p_ref.add_(ur, alpha=-lr_ratio)
                # the kernels (update in place, parameter in the same pass)
                uk = u.clone()
                scal = torch.tensor([bc, lr_ratio, wdf], dtype=torch.float32, device=dev)
                ops().muon_epilogue(uk, gr if cautious else None, v_ker if normuon else None, p_ker, scal,
                                    normuon, cautious, beta2, eps)
                tol = 1.6e-2 if dtype == torch.bfloat16 else 1e-5
                torch.testing.assert_close(uk.float(), ur.float(), rtol=tol, atol=1e-6)
                assert (uk != ur).float().mean().item() < (0.02 if dtype == torch.bfloat16 else 1.0)
                torch.testing.assert_close(p_ker.float(), p_ref.float(), rtol=tol, atol=1e-5)
                if normuon:
                    torch.testing.assert_close(v_ker, v_ref, rtol=1e-5, atol=1e-12)


def test_gefen_muon_with_normuon_and_cautious_takes_the_epilogue_kernels():
    """``GefenMuon(normuon=True, cautious=True)`` on CUDA matrices follows the same optimizer on the CPU
    (the torch chain) over several steps."""
    from gefen_x_b200 import GefenMuon

    g = torch.Generator().manual_seed(23)
    w = torch.randn(64, 128, generator=g) * 0.05
    grads = [torch.randn(64, 128, generator=g) * 1e-2 for _ in range(4)]
    outs = []
    for dev in (torch.device("cpu"), _dev()):
        p = w.clone().to(dev).requires_grad_()
        opt = GefenMuon([("w", p)], lr=1e-2, normuon=True, cautious=True)
        for gr in grads:
            p.grad = gr.to(dev)
            opt.step()
        outs.append(p.detach().cpu())
    torch.testing.assert_close(outs[0], outs[1], rtol=0, atol=2e-3)


def test_pair_gemm_symmetric_mode_equals_the_full_product():
    """``symmetric=True`` computes the 256 x 256 tiles on and below the diagonal and mirrors the rest:
    the result is exactly symmetric and equals the full product up to the order of the K-split sums
    (the two launches split different tiles of their tail waves: one bf16 ulp); sizes that are and are
    not multiples of the tile, with and without the addend, both schedules."""
    from gefen_x_b200.ops import tcgemm

    g = torch.Generator().manual_seed(41)
    dev = _dev()
    try:
        for dynamic in (False, True):
            tcgemm.set_dynamic_schedule(dynamic)
            for m, k in [(4096, 1024), (2048, 4096), (2104, 520), (2304, 768), (2048, 128)]:
                x = (torch.randn(m, k, generator=g) * 0.1).bfloat16().to(dev)
                full = tcgemm.gemm(x, x)
                sym = tcgemm.gemm(x, x, symmetric=True)
                assert torch.equal(sym, sym.t()), (m, k)
                torch.testing.assert_close(sym.float(), full.float(), rtol=1.6e-2, atol=1e-3, msg=str((m, k)))
                gm = sym                                                   # an exactly symmetric matrix
                u_full = tcgemm.gemm(gm, gm, alpha=2.0, beta=-4.0, d=gm)
                u_sym = tcgemm.gemm(gm, gm, alpha=2.0, beta=-4.0, d=gm, symmetric=True)
                assert torch.equal(u_sym, u_sym.t()), (m, k)
                torch.testing.assert_close(u_sym.float(), u_full.float(), rtol=1.6e-2, atol=2e-2, msg=str((m, k)))
        torch.cuda.synchronize()
        assert int(tcgemm.status_word(dev).item()) == 0
    finally:
        tcgemm.set_dynamic_schedule(False)
