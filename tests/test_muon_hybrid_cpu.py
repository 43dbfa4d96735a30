"""CPU tests of GefenMuon, GefenMuonHybrid and the parameter split.

Model: reference tests/test_gefen_muon_hybrid.py, tests/test_hybrid_ctor_and_lrcache_cpu.py,
tests/test_hybrid_load_atomicity.py, tests/test_muon_quality_levers.py,
tests/test_zero_incompat_guard_cpu.py.
"""
import copy
import math

import pytest
import torch
import torch.nn as nn

from gefen_x_b200 import Gefen, GefenMuon, GefenMuonHybrid, split_params_for_muon, validate_split
from gefen_x_b200.optim import newton_schulz as NS
from gefen_x_b200.optim.muon import adjust_lr_ratio, cautious_mask_, stable_distributed_owner


class Tiny(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = nn.Embedding(50, 32)
        self.fc1 = nn.Linear(32, 64)
        self.norm = nn.LayerNorm(64)
        self.fc2 = nn.Linear(64, 32, bias=False)
        self.lm_head = nn.Linear(32, 50, bias=False)
        self.lm_head.weight = self.embed.weight           # tied

    def forward(self, x):
        return self.lm_head(self.fc2(self.norm(torch.relu(self.fc1(self.embed(x))))))


def _train(model, opt, steps=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, 50, (8, 12), generator=g)
    y = torch.randint(0, 50, (8, 12), generator=g)
    out = []
    for _ in range(steps):
        loss = nn.functional.cross_entropy(model(x).view(-1, 50), y.view(-1))
        opt.zero_grad()
        loss.backward()
        opt.step()
        out.append(loss.item())
    return out


def test_newton_schulz_orthogonalises():
    torch.manual_seed(0)
    for shape in ((48, 96), (96, 48), (64, 64)):
        g = torch.randn(shape, dtype=torch.float64)
        o = NS.zeropower_via_newtonschulz(g, ns_steps=8)
        s = torch.linalg.svdvals(o.double())
        assert s.max() < 1.35 and s.min() > 0.55, (shape, s.min().item(), s.max().item())
    for name in ("tuned3", "tuned4"):
        sched = NS.resolve_schedule(name, None, 5)
        o = NS.zeropower_via_newtonschulz(torch.randn(32, 80, dtype=torch.float64), sched, len(sched))
        s = torch.linalg.svdvals(o.double())
        assert s.max() < 1.3 and s.min() > 0.3
    with pytest.raises(ValueError):
        NS.resolve_schedule("nope", None, 5)
    mats = [torch.randn(16, 40) for _ in range(3)]
    outs = NS.zeropower_batched(mats, ns_steps=5)
    for m, o in zip(mats, outs):
        single = NS.zeropower_via_newtonschulz(m, ns_steps=5)
        assert torch.allclose(o.float(), single.float(), atol=3e-2)


def test_fp8_newton_schulz_gates_and_numerics(monkeypatch):
    """e4m3 products (CPU statement of the quantised values): close to the bf16 iterations,
    gated by size and 16-element alignment (reference tests/test_gefen_muon.py fp8 cases)."""
    assert NS.fp8_applies((2048, 4096), True) and not NS.fp8_applies((2048, 4096), False)
    assert not NS.fp8_applies((1024, 4096), True)              # below the size gate
    assert not NS.fp8_applies((1544, 4104), True)              # not multiples of 16
    q, sc = NS.quantize_rowwise_fp8(torch.tensor([[1.0, -2.0, 0.5], [0.0, 0.0, 0.0]]))
    assert q.dtype == torch.float8_e4m3fn and float(q[0, 1].float()) == -448.0
    assert torch.allclose(q.float() * sc, torch.tensor([[1.0, -2.0, 0.5], [0.0, 0.0, 0.0]]), rtol=0.07)
    monkeypatch.setattr(NS, "FP8_MIN_DIM", 64)
    g = torch.Generator().manual_seed(3)
    for shape in ((64, 128), (160, 96)):
        m = torch.randn(shape, generator=g)
        ref = NS.zeropower_via_newtonschulz(m, ns_steps=5).float()
        got = NS.zeropower_via_newtonschulz(m, ns_steps=5, use_fp8=True).float()
        assert got.shape == ref.shape
        cos = torch.nn.functional.cosine_similarity(got.reshape(-1), ref.reshape(-1), dim=0)
        assert cos > 0.97, (shape, float(cos))       # e4m3 noise: relative error of 0.1-0.2 at this size
        s = torch.linalg.svdvals(got.double())
        assert s.max() < 1.4 and s.min() > 0.3
    outs = NS.zeropower_batched([torch.randn(64, 128, generator=g) for _ in range(2)], ns_steps=5, use_fp8=True)
    assert len(outs) == 2 and outs[0].shape == (64, 128)
    # through the optimizer: the flag reaches the iterations and training still descends
    calls = []
    real = NS._iterate_fp8
    monkeypatch.setattr(NS, "_iterate_fp8", lambda x, sch: (calls.append(tuple(x.shape)), real(x, sch))[1])
    w = (torch.randn(64, 96, generator=g) * 0.1).requires_grad_()
    opt = GefenMuon([("w", w)], lr=1e-2, fp8_ns=True, fused=False)
    w.grad = torch.randn(64, 96, generator=g)
    opt.step()
    assert calls == [(64, 96)]


def test_lr_ratio_owner_and_cautious():
    assert adjust_lr_ratio(None, (128, 32)) == 2.0
    assert adjust_lr_ratio("original", (32, 128)) == 1.0
    assert abs(adjust_lr_ratio("match_rms_adamw", (64, 256)) - 0.2 * 16) < 1e-12
    assert [stable_distributed_owner(i, 4) for i in range(6)] == [0, 1, 2, 3, 0, 1]
    with pytest.raises(ValueError):
        stable_distributed_owner(0, 0)
    u = torch.tensor([1.0, -1.0, 2.0, -2.0])
    g = torch.tensor([1.0, 1.0, -1.0, -1.0])
    out = cautious_mask_(u.clone(), g)
    assert torch.equal(out, torch.tensor([2.0, 0.0, 0.0, -4.0]))


def test_muon_rejects_non_2d_and_trains():
    with pytest.raises(ValueError, match="2D"):
        GefenMuon([torch.zeros(8, requires_grad=True)], fused=False)
    torch.manual_seed(1)
    lin = nn.Linear(24, 40, bias=False)
    opt = GefenMuon(lin.named_parameters(), lr=2e-2, fused=False, normuon=True, cautious=True)
    x = torch.randn(16, 24)
    y = torch.randn(16, 40)
    losses = []
    for _ in range(12):
        loss = ((lin(x) - y) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]
    st = opt.state[lin.weight]
    assert "vmean" not in st and "v_row" not in st and st["m_codebook"].dtype == torch.uint8
    assert st["normuon_v"].shape == (40, 1) and st["normuon_step"] == 12
    # wrapper that swaps in flat partitions is refused at step time
    opt.param_groups[0]["params"] = [torch.zeros(10, requires_grad=True)]
    with pytest.raises(ValueError, match="DeepSpeed ZeRO"):
        opt.step()


def test_split_and_validation():
    m = Tiny()
    muon, backup = split_params_for_muon(m)
    assert [n for n, _ in muon] == ["fc1.weight", "fc2.weight"]
    assert "embed.weight" in [n for n, _ in backup] and "fc1.bias" in [n for n, _ in backup]
    validate_split(muon, backup, m)
    with pytest.raises(ValueError, match="BOTH"):
        validate_split(muon, backup + [muon[0]])
    with pytest.raises(ValueError, match="neither"):
        validate_split(muon[:1], backup, m)
    with pytest.raises(TypeError):
        validate_split([m.fc1.weight], backup)


@pytest.mark.parametrize("backup_kind", ["gefen", "adamw"])
def test_hybrid_trains_checkpoints_and_loads_atomically(backup_kind):
    torch.manual_seed(2)
    m = Tiny()
    opt = GefenMuonHybrid(m, lr=5e-3, backup_optimizer=backup_kind, fused=False, weight_decay=0.01,
                          no_decay_substrings=("norm", "bias"))
    losses = _train(m, opt, 8)
    assert losses[-1] < losses[0]
    names = [g.get("param_names") for g in opt.param_groups]
    assert len(opt.param_groups) >= 3                      # muon + decay + no-decay
    # the named schedule is stored resolved (three iterations of tuned coefficients), as the reference does
    assert opt.param_groups[0]["ns_steps"] == 3 and len(opt.param_groups[0]["ns_coefficients"]) == 3
    assert "ns_schedule" not in opt.param_groups[0] and opt.param_groups[0]["normuon"] is True
    with pytest.raises(NotImplementedError):
        opt.add_param_group({"params": []})
    # LR schedulers mutate the live group dicts
    for g in opt.param_groups:
        g["lr"] = g["lr"] * 0.5
    assert opt.muon.param_groups[0]["lr"] == 2.5e-3
    sd = opt.state_dict()
    assert set(sd) == {"muon", "backup", "backup_optimizer"} and sd["backup_optimizer"] == backup_kind
    # resume: identical continuation
    torch.manual_seed(2)
    m2 = Tiny()
    m2.load_state_dict(m.state_dict())
    o2 = GefenMuonHybrid(m2, lr=5e-3, backup_optimizer=backup_kind, fused=False, weight_decay=0.01,
                         no_decay_substrings=("norm", "bias"))
    o2.load_state_dict(copy.deepcopy(sd))
    a = _train(m, opt, 3, seed=5)
    b = _train(m2, o2, 3, seed=5)
    assert a == b
    # atomicity: a checkpoint whose backup half is broken leaves the muon half untouched
    before = copy.deepcopy(o2.muon.state_dict()["gefen_global_step"])
    bad = copy.deepcopy(opt.state_dict())
    bad["backup"]["param_groups"] = bad["backup"]["param_groups"][:-1] if len(bad["backup"]["param_groups"]) > 1 \
        else []
    with pytest.raises(Exception):
        o2.load_state_dict(bad)
    assert o2.muon.state_dict()["gefen_global_step"] == before
    wrong = dict(sd, backup_optimizer="adamw" if backup_kind == "gefen" else "gefen")
    with pytest.raises(ValueError, match="backup_optimizer"):
        o2.load_state_dict(wrong)


def test_hybrid_call_forms():
    m = Tiny()
    a = GefenMuonHybrid(m, lr=1e-3, fused=False)
    b = GefenMuonHybrid(list(m.named_parameters()), lr=1e-3, fused=False)
    c = GefenMuonHybrid.from_model(m, lr=1e-3, fused=False)
    muon, backup = split_params_for_muon(m)
    d = GefenMuonHybrid(muon, backup, lr=1e-3, fused=False)
    for o in (a, b, c, d):
        assert len(o.muon.param_groups[0]["params"]) == 2
    with pytest.raises(TypeError):
        GefenMuonHybrid([m.fc1.weight], lr=1e-3, fused=False)
    with pytest.raises(TypeError, match="backup_substrings is only valid"):      # the reference's type and wording
        GefenMuonHybrid(muon, backup, lr=1e-3, fused=False, backup_substrings=("x",))
    assert a.state[m.fc1.weight] is a.muon.state[m.fc1.weight]


def test_tensor_lr_is_read_back_once_per_value_not_once_per_parameter():
    """A tensor learning rate costs one ``Tensor.item()`` (a device-to-host synchronisation on CUDA) per
    value: constant -> no read after the first step; an in-place scheduler update bumps the tensor's
    version and is picked up; the results equal those of the same schedule given as Python floats
    (reference tests/test_lr_item_no_sync.py)."""
    import torch

    from gefen_x_b200 import GefenMuon

    shapes = [(32, 32), (48, 32), (32, 48), (64, 32), (32, 64)]

    def build(lr):
        torch.manual_seed(7)
        ps = [("l%d" % i, (torch.randn(r, c) * 0.02).requires_grad_()) for i, (r, c) in enumerate(shapes)]
        return GefenMuon(ps, lr=lr, ns_steps=2, adjust_lr_fn="match_rms_adamw"), ps

    def grads(ps, gen):
        for _, p in ps:
            p.grad = torch.randn(p.shape, generator=gen) * 1e-3

    orig_item = torch.Tensor.item
    calls = {"n": 0}

    def counting_item(self):
        calls["n"] += 1
        return orig_item(self)

    def run(lr, schedule=None, steps=4, count_from=1):
        opt, ps = build(lr)
        gen = torch.Generator().manual_seed(3)
        counted = 0
        for s in range(steps):
            grads(ps, gen)
            if schedule is not None:
                schedule(opt, s)
            if s >= count_from:
                calls["n"] = 0
                torch.Tensor.item = counting_item
            try:
                opt.step()
            finally:
                torch.Tensor.item = orig_item
            if s >= count_from:
                counted += calls["n"]
        return [p.detach().clone() for _, p in ps], counted

    base, n_float = run(float(torch.tensor(1e-2, dtype=torch.float32)))    # the fp32 value the tensor holds
    const, n_tensor = run(torch.tensor(1e-2))
    assert n_tensor == n_float                                   # no read of a constant tensor after warm-up
    for a, b in zip(base, const):
        assert torch.equal(a, b)

    def decay_tensor(opt, s):
        if s > 0:
            opt.param_groups[0]["lr"].mul_(0.5)                  # in place: bumps the version

    def decay_float(opt, s):
        if s > 0:
            opt.param_groups[0]["lr"] = float(torch.tensor(opt.param_groups[0]["lr"], dtype=torch.float32) * 0.5)

    sched_t, n_sched = run(torch.tensor(1e-2), decay_tensor)
    sched_f, _ = run(float(torch.tensor(1e-2, dtype=torch.float32)), decay_float)
    assert n_sched - n_float == 3                                # one read per new value (steps 1..3)
    for a, b, c in zip(sched_t, sched_f, const):
        assert torch.equal(a, b) and not torch.equal(a, c)
