"""Argument validation, group registration, wrapper guards and checkpoint validation on CPU.

Behaviours the reference pins in ``tests/test_validation_cpu.py``,
``test_epsilon_muon_param_group_cpu.py``, ``test_zero_incompat_guard_cpu.py`` and
``test_native_load_atomicity.py``, restated here against this package.
"""
import copy

import pytest
import torch
import torch.nn as nn

from gefen_x_b200 import Gefen, GefenMuon, GefenMuonHybrid
from gefen_x_b200.optim import newton_schulz as NS

BAD_EPS = [0.0, -1e-8, float("nan"), float("inf"), float("-inf")]


def _mat(rows=8, cols=8):
    return nn.Parameter(torch.randn(rows, cols))


@pytest.mark.parametrize("eps", BAD_EPS)
def test_epsilons_must_be_finite_and_positive(eps):
    with pytest.raises(ValueError, match="eps"):
        Gefen([nn.Parameter(torch.ones(8))], eps=eps, fused=False)
    with pytest.raises(ValueError, match="eps"):
        GefenMuon([_mat()], fused=False, eps=eps)
    with pytest.raises(ValueError, match="normuon_eps"):
        GefenMuon([_mat()], fused=False, normuon_eps=eps)


def test_schedule_rules():
    assert NS.normalize_schedule((3.0, -4.0, 2.0), 5) == [(3.0, -4.0, 2.0)] * 5
    for coeffs, steps in (((), 5), ((3.0, -4.0), 5), ((3.0, -4.0, 2.0), 100), ((3.0, -4.0, 2.0), 0),
                          ([(3.0, -4.0, 2.0, 1.0)], 5), ([(1.0, 1.0, 1.0)] * 100, 5)):
        with pytest.raises(ValueError):
            NS.normalize_schedule(coeffs, steps)
    for steps in (0, -1, 100):
        with pytest.raises(ValueError):
            GefenMuon([("w", _mat())], fused=False, ns_steps=steps)
        with pytest.raises(ValueError):
            GefenMuon([("w", _mat())], fused=False, ns_schedule="standard", ns_steps=steps)
    # an explicit schedule carries its own length: ns_steps is ignored
    for sched in ("tuned3", [(3.0, -4.0, 2.0), (2.5, -3.5, 1.5)]):
        g = GefenMuon([("w", _mat())], fused=False, ns_schedule=sched, ns_steps=0).param_groups[0]
        assert g["ns_steps"] == len(g["ns_coefficients"]) and "ns_schedule" not in g


def test_muon_add_param_group_resolves_options_and_is_atomic():
    first = _mat()
    opt = GefenMuon([("first", first)], weight_decay=0.0, fused=False)
    first.grad = torch.randn_like(first)
    opt.step()
    added = _mat()
    opt.add_param_group({"params": [("added", added)], "lr": 2e-4, "eps": 2e-7, "momentum": 0.8, "nesterov": False,
                         "ns_schedule": "tuned3", "sharded_mode": "approx", "batched_ns": True, "normuon": True,
                         "normuon_beta2": 0.9, "normuon_eps": 1e-6, "cautious": True, "weight_decay": 0.0})
    g = opt.param_groups[-1]
    assert g["param_names"] == ["added"] and g["lr"] == 2e-4 and g["eps"] == 2e-7
    assert g["beta1"] == g["momentum"] == 0.8 and g["beta2"] == 0.0 and g["nesterov"] is False
    assert g["ns_steps"] == 3 and len(g["ns_coefficients"]) == 3 and g["sharded_mode"] == "approx"
    assert g["batched_ns"] is True and g["normuon"] is True and g["normuon_eps"] == 1e-6 and g["cautious"] is True
    first.grad, added.grad = torch.randn_like(first), torch.randn_like(added)
    before = added.detach().clone()
    opt.step()
    assert "step" in opt.state[added] and not torch.equal(added, before)
    n = len(opt.param_groups)
    with pytest.raises(ValueError, match="only supports 2D"):
        opt.add_param_group({"params": [("ok", _mat()), ("bad", nn.Parameter(torch.randn(8)))]})
    for eps in BAD_EPS:
        with pytest.raises(ValueError, match="normuon_eps"):
            opt.add_param_group({"params": [_mat()], "normuon_eps": eps})
    assert len(opt.param_groups) == n


def _hybrid(**kw):
    torch.manual_seed(0)
    muon = [("blocks.0.attn.w", _mat(8, 16)), ("blocks.0.mlp.w", _mat(16, 8))]
    backup = [("embed.weight", _mat(12, 8)), ("norm.weight", nn.Parameter(torch.randn(8)))]
    kw.setdefault("lr", 1e-3)
    kw.setdefault("fused", False)
    return GefenMuonHybrid(muon, backup, **kw)


def _swap_to_flat_partitions(groups):
    flats = []
    for g in groups:
        flat = nn.Parameter(torch.zeros(sum(p.numel() for p in g["params"])))
        flat.grad = torch.full_like(flat, 1e-3)
        g["params"] = [flat]
        flats.append(flat)
    return flats


def test_flat_partition_wrappers_get_an_explaining_error():
    opt = GefenMuon([("a", _mat(8, 16))], lr=1e-3, fused=False)
    for flat in _swap_to_flat_partitions(opt.param_groups):
        flat.grad = None                                    # the guard looks at parameters, not gradients
    with pytest.raises(ValueError, match="DeepSpeed ZeRO") as e:
        opt.step()
    assert "flat partition" in str(e.value) and "plain Gefen" in str(e.value)
    hyb = _hybrid()
    foreign = nn.Parameter(torch.zeros(64))
    with pytest.raises(KeyError, match="DeepSpeed ZeRO"):
        bool(hyb.state[foreign])
    with pytest.raises(KeyError, match="DeepSpeed ZeRO"):
        hyb.state[foreign] = {}
    with pytest.raises(TypeError, match="DeepSpeed ZeRO"):
        hyb.param_groups = [{"params": []}]
    flats = _swap_to_flat_partitions(hyb.param_groups)      # ownership was frozen at construction
    with pytest.raises(KeyError, match="DeepSpeed ZeRO"):
        bool(hyb.state[flats[0]])
    with pytest.raises(ValueError, match="DeepSpeed ZeRO"):
        hyb.step()
    with pytest.raises(ValueError, match="ZeRO stage 3"):
        GefenMuonHybrid([("model.w", nn.Parameter(torch.empty(0))), ("model.norm", nn.Parameter(torch.empty(0)))],
                        lr=1e-3, fused=False)
    ok = GefenMuonHybrid([], [("norm.weight", nn.Parameter(torch.randn(8))), ("slot", nn.Parameter(torch.zeros(0)))],
                         lr=1e-3, fused=False)
    assert ok.muon is None and ok.backup is not None


def test_hybrid_state_is_a_live_dict_view():
    opt = _hybrid()
    assert isinstance(opt.state, dict)
    assert set(opt.state.keys()) == set(opt.muon.state.keys()) | set(opt.backup.state.keys())
    p = opt.backup.param_groups[0]["params"][0]
    base = opt.state[p]
    assert opt.backup.state[p] is base and opt.state.setdefault(p, {"x": 1}) is base
    repl = dict(base, marker=7)
    opt.state.update({p: repl})
    assert opt.backup.state[p] is repl and opt.state.pop(p) is repl and opt.state.pop(p, "absent") == "absent"
    fresh = {"seeded": True}
    assert opt.state.setdefault(p, fresh) is fresh and opt.backup.state[p] is fresh
    del opt.state[p]
    with pytest.raises(KeyError):
        del opt.state[p]
    ghost = nn.Parameter(torch.zeros(3))
    assert ghost not in opt.state and opt.state.get(ghost) is None
    for bad in (lambda: opt.state.update({ghost: {}}), lambda: opt.state.setdefault(ghost, {}),
                lambda: opt.state.pop(ghost)):
        with pytest.raises(KeyError, match="DeepSpeed ZeRO"):
            bad()
    with pytest.raises(NotImplementedError, match="popitem"):
        opt.state.popitem()
    opt.state.clear()
    assert not dict(opt.muon.state) and not dict(opt.backup.state) and not opt.state
    adam = _hybrid(backup_optimizer="adamw")
    q = adam.backup.param_groups[0]["params"][0]
    entry = adam.state[q]                                   # auto-created in the owning child
    entry["flag"] = True
    assert adam.backup.state[q] is entry and adam.backup.param_groups[0]["param_names"]
    assert "backup_optimizer='adamw'" in repr(adam) and "muon_params=2" in repr(adam)


def _trained(kind, seed):
    torch.manual_seed(seed)
    layer = nn.Linear(8, 8, bias=False)
    if kind == "muon":
        opt = GefenMuon(list(layer.named_parameters()), lr=1e-3, fused=False, normuon=True)
    else:
        opt = Gefen(list(layer.named_parameters()), lr=1e-3, fused=False, factored_v_2d=(kind == "factored"))
    layer.weight.grad = torch.randn_like(layer.weight)
    opt.step()
    return layer, opt


def _first(sd):
    return next(iter(sd["state"].values()))


CORRUPTIONS = {
    "period": ("block", lambda sd: _first(sd).__setitem__("automatic_period", 0)),
    "index dtype": ("block", lambda sd: _first(sd).__setitem__("m_codebook", _first(sd)["m_codebook"].float())),
    "negative magnitude": ("block", lambda sd: _first(sd).__setitem__(
        "m_magnitude", torch.full_like(_first(sd)["m_magnitude"], -1.0))),
    "momentum removed": ("block", lambda sd: (_first(sd).pop("m_codebook"), _first(sd).pop("m_magnitude"))),
    "nan second moment": ("block", lambda sd: _first(sd).__setitem__(
        "vmean", torch.full_like(_first(sd)["vmean"], float("nan")))),
    "half a factored moment": ("factored", lambda sd: _first(sd).pop("v_col")),
    "negative normuon": ("muon", lambda sd: _first(sd).__setitem__(
        "normuon_v", torch.full_like(_first(sd)["normuon_v"], -1.0))),
    "vector counter": ("block", lambda sd: _first(sd).__setitem__("step", torch.tensor([1.0, 2.0]))),
    "fractional counter": ("block", lambda sd: _first(sd).__setitem__("step", torch.tensor(1.5))),
    "boolean counter": ("block", lambda sd: _first(sd).__setitem__("step", torch.tensor(True))),
    "negative counter": ("muon", lambda sd: _first(sd).__setitem__("step", torch.tensor(-1.0))),
    # sizes that do not fit the live parameter: the kernels would index them out of bounds
    "index rows": ("block", lambda sd: _first(sd).__setitem__(
        "m_codebook", torch.cat((_first(sd)["m_codebook"], _first(sd)["m_codebook"])))),
    "index period": ("block", lambda sd: _first(sd).__setitem__(
        "m_codebook", _first(sd)["m_codebook"].reshape(-1, 2).contiguous())),
    "magnitude count": ("block", lambda sd: _first(sd).__setitem__("m_magnitude", _first(sd)["m_magnitude"][:-1])),
    "period not a divisor": ("block", lambda sd: _first(sd).__setitem__("automatic_period", 7)),
    "vmean count": ("block", lambda sd: _first(sd).__setitem__(
        "vmean", torch.cat((_first(sd)["vmean"], _first(sd)["vmean"])))),
    "row moment length": ("factored", lambda sd: _first(sd).__setitem__("v_row", _first(sd)["v_row"][:-1])),
    "column moment length": ("factored", lambda sd: _first(sd).__setitem__(
        "v_col", torch.cat((_first(sd)["v_col"], _first(sd)["v_col"])))),
    "normuon rows": ("muon", lambda sd: _first(sd).__setitem__("normuon_v", _first(sd)["normuon_v"][:-1])),
}


@pytest.mark.parametrize("name", sorted(CORRUPTIONS))
def test_malformed_checkpoints_are_rejected_before_anything_changes(name):
    kind, corrupt = CORRUPTIONS[name]
    _, source = _trained(kind, 1)
    layer, target = _trained(kind, 2)
    sd = copy.deepcopy(source.state_dict())
    corrupt(sd)
    weights = layer.weight.detach().clone()
    before = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in target.state[layer.weight].items()}
    step_before, cb_before = target._gefen_global_step, target._gefen_codebook.clone()
    calls = []
    target.register_load_state_dict_pre_hook(lambda o, s: calls.append("pre"))
    target.register_load_state_dict_post_hook(lambda o: calls.append("post"))
    with pytest.raises(ValueError):
        target.load_state_dict(sd)
    assert calls == ["pre"]                                  # the post hook fires only after a commit
    assert torch.equal(layer.weight, weights) and target._gefen_global_step == step_before
    assert torch.equal(target._gefen_codebook, cb_before)
    after = target.state[layer.weight]
    assert set(after) == set(before)
    for k, v in before.items():
        assert torch.equal(after[k], v) if torch.is_tensor(v) else after[k] == v
    target.load_state_dict(source.state_dict())             # a good checkpoint still loads, hooks fire once
    assert calls == ["pre", "pre", "post"]


def test_bad_codebook_is_rejected():
    _, source = _trained("block", 1)
    _, target = _trained("block", 2)
    sd = copy.deepcopy(source.state_dict())
    bad = torch.linspace(-1.0, 1.0, 255)
    sd["gefen_codebook"] = bad
    for g in sd["param_groups"]:
        g["_gefen_checkpoint_metadata"] = dict(g["_gefen_checkpoint_metadata"], codebook=bad)
    with pytest.raises(ValueError, match="codebook"):
        target.load_state_dict(sd)


def test_hybrid_warns_when_muon_keeps_its_native_lr_scale():
    with pytest.warns(UserWarning, match="adjust_lr_fn"):
        _hybrid(adjust_lr_fn=None)
