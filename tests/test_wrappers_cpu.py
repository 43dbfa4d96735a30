"""Optimizer wrappers that rewrite ``param_groups`` (DeepSpeed ZeRO style), uneven and empty shards,
non-finite gradients: all on CPU.

Model: reference ``tests/test_zero_offload_cpu.py`` / ``test_zero_incompat_guard_cpu.py`` (ZeRO is
simulated by swapping ``param_groups[*]["params"]`` for flat fp32 partitions, no DeepSpeed needed)
and the uneven / empty shard cases of ``tests/test_muon_fsdp2_parity.py:47-53``.
"""
import pytest
import torch

from gefen_x_b200 import Gefen, GefenMuon, GefenMuonHybrid


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 8))


def test_plain_gefen_steps_flat_partitions_like_a_zero_wrapper():
    model = _model()
    opt = Gefen(model.named_parameters(), lr=1e-2, fused=False)
    # a ZeRO wrapper replaces the parameters of every group by one flat fp32 partition
    flat = torch.cat([p.detach().reshape(-1).float() for p in model.parameters()]).requires_grad_()
    originals = list(opt.param_groups[0]["params"])
    opt.param_groups[0]["params"] = [flat]
    g = torch.Generator().manual_seed(1)
    before = flat.detach().clone()
    for _ in range(3):
        flat.grad = torch.randn(flat.shape, generator=g) * 1e-2
        opt.step()
    assert not torch.equal(before, flat.detach())
    st = opt.state[flat]
    assert st["m_codebook"].dtype == torch.uint8 and st["m_codebook"].numel() == flat.numel()
    # the state of the parameters the wrapper orphaned does not leak into the checkpoint
    for p in originals:
        opt.state[p]["stale"] = torch.zeros(1)
    sd = opt.state_dict()
    assert len(sd["state"]) == 1 and sd["param_groups"][0]["params"] == [0]
    opt2 = Gefen([("flat", flat.detach().clone().requires_grad_())], lr=1e-2, fused=False)
    opt2.load_state_dict(sd)
    assert opt2._gefen_global_step == 3


def test_muon_family_refuses_flattened_parameters_before_touching_state():
    model = _model()
    mats = [(n, p) for n, p in model.named_parameters() if p.ndim == 2]
    opt = GefenMuon(mats, lr=1e-2, fused=False)
    flat = torch.cat([p.detach().reshape(-1) for _, p in mats]).requires_grad_()
    opt.param_groups[0]["params"] = [flat]
    flat.grad = torch.ones_like(flat)
    with pytest.raises(ValueError, match="1-D parameter"):
        opt.step()
    assert len(opt.state) == 0 or all("step" not in st for st in opt.state.values())
    hyb = GefenMuonHybrid(_model(), lr=1e-2, fused=False)
    assert hyb.muon is not None and hyb.backup is not None


def test_non_finite_gradients_do_not_poison_the_codebook_indices():
    p = (torch.randn(8, 64, generator=torch.Generator().manual_seed(0)) * 0.1).requires_grad_()
    opt = Gefen([("w", p)], lr=1e-2, fused=False, factored_v_2d=False)
    p.grad = torch.randn(8, 64, generator=torch.Generator().manual_seed(1)) * 1e-2
    opt.step()
    p.grad = torch.full((8, 64), float("nan"))
    opt.step()                                         # must not raise; indices stay valid bytes
    idx = opt.state[p]["m_codebook"]
    assert idx.dtype == torch.uint8 and int(idx.max()) <= 255


def test_empty_and_single_element_parameters_are_no_ops_or_period_one():
    a = torch.zeros(0, 4, requires_grad=True)
    b = torch.ones(1, requires_grad=True)
    c = (torch.randn(6, 10, generator=torch.Generator().manual_seed(0))).requires_grad_()
    opt = Gefen([("a", a), ("b", b), ("c", c)], lr=1e-2, fused=False)
    for t in (a, b, c):
        t.grad = torch.ones_like(t) * 1e-2
    opt.step()
    opt.step()
    assert "m_codebook" not in opt.state.get(a, {})
    assert opt.state[b]["automatic_period"] == 1
    assert float(b.detach()) < 1.0
