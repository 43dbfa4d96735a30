"""Loss-curve parity with the reference's own optimizer code, on CPU.

The unmodified reference package (installed under ``baseline/_ref``; skipped when that folder is
absent) and this package train the same small MLP from the same weights on the same batches;
the two loss curves have to stay within 1% of each other at every step.  Both run their
torch (non-fused) statements, the path the CUDA kernels of either side are tested against
(reference ``tests/test_gefen.py`` compares its fused kernels with that statement the same way).
"""
import os
import sys

import pytest
import torch
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "gefen")),
                                reason="the reference package is not installed under baseline/_ref")


def _reference():
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import gefen

    return gefen


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(32, 64), nn.GELU(), nn.Linear(64, 64), nn.GELU(), nn.Linear(64, 8))


def _train(make_opt, steps=150):
    m = _model()
    opt = make_opt(m)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(512, 32, generator=g)
    y = (x @ torch.randn(32, 8, generator=g)).tanh()
    out = []
    for _ in range(steps):
        i = torch.randint(0, 512, (64,), generator=g)
        loss = ((m(x[i]) - y[i]) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        out.append(loss.item())
    return torch.tensor(out, dtype=torch.float64)


def _assert_curves_agree(a, b, tol=0.01):
    assert torch.equal(a[:1], b[:1])                      # same start
    assert a[-20:].mean() < 0.6 * a[0]                    # it did train
    rel = ((a - b).abs() / a.abs()).max().item()
    assert rel < tol, rel


@pytest.mark.parametrize("kw", [dict(), dict(factored_v_2d=False), dict(weight_decay=0.0, betas=(0.8, 0.95))])
def test_gefen_loss_curve_matches_the_reference(kw):
    import gefen_x_b200 as ours

    ref = _reference()
    base = dict(lr=3e-3, weight_decay=0.01, fused=False)
    base.update(kw)
    a = _train(lambda m: ref.Gefen(list(m.named_parameters()), **base))
    b = _train(lambda m: ours.Gefen(list(m.named_parameters()), **base))
    _assert_curves_agree(a, b)


def test_muon_hybrid_loss_curve_matches_the_reference():
    import gefen_x_b200 as ours

    ref = _reference()
    kw = dict(lr=3e-3, weight_decay=0.01, fused=False)
    a = _train(lambda m: ref.GefenMuonHybrid(m, **kw))
    b = _train(lambda m: ours.GefenMuonHybrid(m, **kw))
    _assert_curves_agree(a, b)


def _train_with_handover(first, second, kw, steps=(20, 20)):
    """``first``'s optimizer for some steps, its ``state_dict`` loaded into ``second``'s, more steps."""
    import copy

    m = _model()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(512, 32, generator=g)
    y = (x @ torch.randn(32, 8, generator=g)).tanh()
    out = []

    def run(opt, n):
        for _ in range(n):
            i = torch.randint(0, 512, (64,), generator=g)
            loss = ((m(x[i]) - y[i]) ** 2).mean()
            opt.zero_grad()
            loss.backward()
            opt.step()
            out.append(loss.item())

    opt = first.Gefen(list(m.named_parameters()), lr=3e-3, fused=False, **kw)
    run(opt, steps[0])
    sd = copy.deepcopy(opt.state_dict())
    opt2 = second.Gefen(list(m.named_parameters()), lr=3e-3, fused=False, **kw)
    opt2.load_state_dict(sd)
    run(opt2, steps[1])
    return torch.tensor(out, dtype=torch.float64), sd


@pytest.mark.parametrize("kw", [dict(), dict(factored_v_2d=False)])
def test_native_checkpoints_load_across_the_two_packages(kw):
    """Same top-level keys, same per-parameter state keys, and a checkpoint written by either
    package resumes in the other as it does in its own (reference schema: src/gefen/gefen.py
    ``state_dict`` / ``load_state_dict``)."""
    import gefen_x_b200 as ours

    ref = _reference()
    rr, sd_r = _train_with_handover(ref, ref, kw)
    ro, _ = _train_with_handover(ref, ours, kw)
    oo, sd_o = _train_with_handover(ours, ours, kw)
    orf, _ = _train_with_handover(ours, ref, kw)
    assert set(sd_r) == set(sd_o)
    k = next(iter(sd_r["state"]))
    assert set(sd_r["state"][k]) == set(sd_o["state"][k])
    for name in sd_r["state"][k]:
        a, b = sd_r["state"][k][name], sd_o["state"][k][name]
        if torch.is_tensor(a):
            assert a.dtype == b.dtype and a.shape == b.shape, name
    assert ((rr - ro).abs() / rr).max().item() < 1e-5
    assert ((oo - orf).abs() / oo).max().item() < 1e-5


def test_hybrid_checkpoints_and_group_keys_match_the_reference():
    """GefenMuonHybrid: same sections, same parameter-group keys (a named Newton-Schulz schedule is
    stored resolved, the group's ``eps`` is the normalisation epsilon), and a checkpoint of either
    package resumes in the other."""
    import copy

    import gefen_x_b200 as ours

    ref = _reference()

    def handover(first, second):
        m = _model()
        g = torch.Generator().manual_seed(1)
        x = torch.randn(512, 32, generator=g)
        y = (x @ torch.randn(32, 8, generator=g)).tanh()
        out = []

        def run(opt, n):
            for _ in range(n):
                i = torch.randint(0, 512, (64,), generator=g)
                loss = ((m(x[i]) - y[i]) ** 2).mean()
                opt.zero_grad()
                loss.backward()
                opt.step()
                out.append(loss.item())

        opt = first.GefenMuonHybrid(m, lr=3e-3, fused=False)
        run(opt, 20)
        sd = copy.deepcopy(opt.state_dict())
        opt2 = second.GefenMuonHybrid(m, lr=3e-3, fused=False)
        opt2.load_state_dict(sd)
        run(opt2, 20)
        return torch.tensor(out, dtype=torch.float64), sd

    rr, sd_r = handover(ref, ref)
    ro, _ = handover(ref, ours)
    oo, sd_o = handover(ours, ours)
    orf, _ = handover(ours, ref)
    assert set(sd_r) == set(sd_o)
    for part in ("muon", "backup"):
        assert set(sd_r[part]) == set(sd_o[part]), part
        gr, go = sd_r[part]["param_groups"][0], sd_o[part]["param_groups"][0]
        assert set(gr) == set(go), (part, set(gr) ^ set(go))
        for k in ("ns_steps", "eps", "beta1", "beta2", "momentum", "adjust_lr_fn", "sharded_mode", "fp8_ns"):
            if k in gr:
                assert gr[k] == go[k], (part, k, gr[k], go[k])
    assert ((rr - ro).abs() / rr).max().item() < 1e-3
    assert ((oo - orf).abs() / oo).max().item() < 1e-3
