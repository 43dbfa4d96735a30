"""CPU tests of the Gefen optimizer: the 2-layer Llama config, bit-exact resume,
parameter groups / names, validation, load atomicity and the AMP skip protocol.

Model: reference tests/test_core_correctness_cpu.py, tests/test_cpu_step_checkpoint.py
(bit-exact resume ``:109-144``), tests/test_validation_cpu.py,
tests/test_native_load_atomicity.py, tests/test_amp_grad_scaler.py.
"""
import copy
import io
import warnings

import pytest
import torch
import torch.nn as nn

from gefen_x_b200 import Gefen
from gefen_x_b200.models.decoder import DecoderLM, get_config


def _tiny_model(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(32, 48), nn.ReLU(), nn.Linear(48, 16))


def _train(model, opt, steps, seed=0, start=0):
    g = torch.Generator().manual_seed(seed)
    data = [(torch.randn(8, 32, generator=g), torch.randn(8, 16, generator=g)) for _ in range(64)]
    losses = []
    for i in range(start, start + steps):
        x, y = data[i]
        loss = ((model(x) - y) ** 2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses


def _state_equal(a, b):
    assert a.keys() == b.keys()
    for k in a:
        va, vb = a[k], b[k]
        if torch.is_tensor(va):
            assert torch.equal(va, vb), k
        else:
            assert va == vb, k


def test_config1_two_layer_llama_trains_and_resumes_bit_exact():
    """BASELINE config 1: hidden 256, 4 heads / 2 KV heads, FFN 688, vocab 1024, untied,
    Gefen defaults, lr 6e-4, betas (0.9, 0.999), wd 0.01, batch 4 x seq 128, 20 steps,
    save / load mid-run, bit-exact continuation."""
    cfg = get_config("tiny-llama")

    def make():
        m = DecoderLM(cfg, dtype=torch.float32, impl="torch", seed=7)
        o = Gefen(m.named_parameters(), lr=6e-4, betas=(0.9, 0.999), weight_decay=0.01, fused=False)
        return m, o

    g = torch.Generator().manual_seed(11)
    batches = [torch.randint(0, 1024, (4, 129), generator=g)] * 20   # one batch of 4 x 128, 20 steps

    def run(m, o, lo, hi):
        out = []
        for i in range(lo, hi):
            t = batches[i]
            loss = m(t[:, :-1], t[:, 1:])
            o.zero_grad()
            loss.backward()
            o.step()
            out.append(loss.item())
        return out

    m1, o1 = make()
    full = run(m1, o1, 0, 20)
    assert full[-1] < full[0] - 0.5, full
    n_params = sum(p.numel() for p in m1.parameters())
    assert o1.state_bytes() / n_params < 1.1          # ~1 byte per parameter

    m2, o2 = make()
    first = run(m2, o2, 0, 10)
    buf = io.BytesIO()
    torch.save({"model": m2.state_dict(), "opt": o2.state_dict()}, buf)
    buf.seek(0)
    ck = torch.load(buf, weights_only=False)
    m3, o3 = make()
    m3.load_state_dict(ck["model"])
    o3.load_state_dict(ck["opt"])
    rest = run(m3, o3, 10, 20)
    assert first + rest == full                        # bit-exact losses
    for a, b in zip(m1.parameters(), m3.parameters()):
        assert torch.equal(a, b)
    for pa, pb in zip(o1.param_groups[0]["params"], o3.param_groups[0]["params"]):
        _state_equal(o1.state[pa], o3.state[pb])
    assert torch.equal(o1._gefen_codebook, o3._gefen_codebook)
    assert o1._gefen_global_step == o3._gefen_global_step == 20


def test_state_layout_and_factored_routing():
    m = _tiny_model()
    opt = Gefen(m.named_parameters(), lr=1e-2, fused=False)
    _train(m, opt, 2)
    w = m[0].weight
    st = opt.state[w]
    assert st["name"] == "0.weight"
    P = st["automatic_period"]
    assert st["m_codebook"].dtype == torch.uint8 and st["m_codebook"].shape == (w.numel() // P, P)
    assert st["m_magnitude"].shape == (w.numel() // P, 1) and st["m_magnitude"].dtype == torch.float32
    assert st["v_row"].shape == (48,) and st["v_col"].shape == (32,) and st["factored_step"] == 2
    b = opt.state[m[0].bias]
    assert "vmean" in b and "v_row" not in b and b["vmean_step"] == 2
    assert opt._gefen_codebook.shape == (256,)
    opt2 = Gefen(_tiny_model().named_parameters(), fused=False, factored_v_2d=False)
    m2 = nn.Sequential(*[copy.deepcopy(x) for x in m])
    opt2 = Gefen(m2.named_parameters(), fused=False, factored_v_2d=False)
    _train(m2, opt2, 1)
    assert "vmean" in opt2.state[m2[0].weight]


def test_param_groups_names_and_defaults():
    m = _tiny_model()
    opt = Gefen([
        {"params": [("A.Weight", m[0].weight)], "lr": 3e-3, "weight_decay": 0.1},
        {"params": [m[0].bias, m[2].bias], "betas": (0.8, 0.9)},
        {"params": [m[2].weight], "name": "Head"},
    ], lr=1e-3, fused=False)
    g0, g1, g2 = opt.param_groups
    assert g0["param_names"] == ["a.weight"] and g0["lr"] == 3e-3 and g0["weight_decay"] == 0.1
    assert g0["beta1"] == 0.9 and "betas" not in g0
    assert g1["param_names"] == ["group_1_param_0", "group_1_param_1"]
    assert g1["param_names_synthesized"] == [True, True] and (g1["beta1"], g1["beta2"]) == (0.8, 0.9)
    assert g2["param_names"] == ["head"] and g2["param_names_synthesized"] == [False]
    implicit = Gefen([m[0].weight.detach().clone().requires_grad_()], fused=False)
    assert implicit.param_groups[0]["param_names"] == ["param_0"]
    with pytest.raises(ValueError):
        opt.add_param_group({"params": [m[0].weight]})
    assert len(opt.param_groups) == 3                 # failed add leaves groups untouched


def test_constructor_validation():
    p = [torch.zeros(4, requires_grad=True)]
    with pytest.raises(ValueError):
        Gefen(p, lr=-1.0, fused=False)
    with pytest.raises(ValueError):
        Gefen(p, betas=(1.0, 0.9), fused=False)
    with pytest.raises(ValueError):
        Gefen(p, eps=-1e-8, fused=False)
    with pytest.raises(ValueError):
        Gefen(p, weight_decay=-0.1, fused=False)
    with pytest.raises(ValueError):
        Gefen(p, codebook_refresh_every=-1, fused=False)
    with pytest.raises(ValueError):
        Gefen(p, capturable=True, codebook_refresh_every=5, fused=False)
    with pytest.raises(ValueError):
        Gefen(p, deterministic=True, factored_v_2d=True, stochastic_round=True, fused=False)
    with pytest.raises(TypeError):
        Gefen(p, deterministic=1, fused=False)
    with pytest.raises(ValueError):
        Gefen([], fused=False)
    if not torch.cuda.is_available():
        with warnings.catch_warnings(record=True) as w:
            warnings.simplefilter("always")
            o = Gefen(p)
        assert o.fused is False and any("fused=True" in str(x.message) for x in w)


def test_rejects_sparse_and_mismatched_grads_before_mutation():
    p = torch.zeros(8, 4, requires_grad=True)
    opt = Gefen([p], fused=False)
    p.grad = torch.zeros(8, 4).to_sparse()
    with pytest.raises(RuntimeError, match="sparse"):
        opt.step()
    assert "step" not in opt.state[p] and opt._gefen_codebook is None


def test_state_dict_schema_and_metadata_mirror():
    m = _tiny_model()
    opt = Gefen(m.named_parameters(), lr=1e-2, fused=False)
    _train(m, opt, 3)
    sd = opt.state_dict()
    assert set(sd) >= {"state", "param_groups", "gefen_global_step", "gefen_deterministic", "gefen_codebook"}
    assert sd["gefen_global_step"] == 3 and sd["gefen_deterministic"] is False
    meta = sd["param_groups"][0]["_gefen_checkpoint_metadata"]
    assert meta["format_version"] == 1 and meta["global_step"] == 3
    assert torch.equal(meta["codebook"], sd["gefen_codebook"]) and meta["device_anchor"].dtype == torch.uint8
    for st in sd["state"].values():
        assert not any(k.startswith("_") or k == "stepsize" for k in st)
    # a tool that keeps only the two standard keys still round-trips the codebook
    stripped = {"state": sd["state"], "param_groups": sd["param_groups"]}
    m2 = _tiny_model()
    o2 = Gefen(m2.named_parameters(), lr=1e-2, fused=False)
    o2.load_state_dict(stripped)
    assert torch.equal(o2._gefen_codebook, opt._gefen_codebook) and o2._gefen_global_step == 3
    # loading does not mutate the caller's dict
    assert "_gefen_checkpoint_metadata" in sd["param_groups"][0] and "gefen_codebook" in sd


def test_load_refuses_missing_codebook_and_policy_mismatch_atomically():
    m = _tiny_model()
    opt = Gefen(m.named_parameters(), lr=1e-2, fused=False)
    _train(m, opt, 2)
    sd = opt.state_dict()
    bad = {"state": sd["state"],
           "param_groups": [{k: v for k, v in g.items() if k != "_gefen_checkpoint_metadata"}
                            for g in sd["param_groups"]]}
    m2 = _tiny_model(1)
    o2 = Gefen(m2.named_parameters(), lr=1e-2, fused=False)
    _train(m2, o2, 1)
    before = copy.deepcopy(o2.state_dict())
    with pytest.raises(ValueError, match="no frozen codebook"):
        o2.load_state_dict(bad)
    o3 = Gefen(_tiny_model(2).named_parameters(), fused=False, deterministic=True)
    with pytest.raises(ValueError, match="deterministic"):
        o3.load_state_dict(sd)
    # structurally broken checkpoint: live optimizer untouched
    broken = copy.deepcopy(sd)
    broken["param_groups"][0]["params"] = broken["param_groups"][0]["params"][:-1]
    with pytest.raises(ValueError):
        o2.load_state_dict(broken)
    after = o2.state_dict()
    assert after["gefen_global_step"] == before["gefen_global_step"]
    for k in before["state"]:
        _state_equal(before["state"][k], after["state"][k])


def test_legacy_one_group_per_param_checkpoint_loads():
    m = _tiny_model()
    opt = Gefen(m.named_parameters(), lr=1e-2, fused=False)
    _train(m, opt, 2)
    sd = opt.state_dict()
    g = sd["param_groups"][0]
    legacy = dict(sd)
    legacy["param_groups"] = []
    for i, pid in enumerate(g["params"]):
        one = {k: v for k, v in g.items() if k not in ("params", "param_names", "param_names_synthesized")}
        one.update(params=[pid], name=g["param_names"][i], param_names=[g["param_names"][i]],
                   param_names_synthesized=[False])
        legacy["param_groups"].append(one)
    m2 = _tiny_model()
    o2 = Gefen(m2.named_parameters(), lr=1e-2, fused=False)
    o2.load_state_dict(legacy)
    assert len(o2.param_groups) == 1 and len(o2.param_groups[0]["params"]) == 4
    assert o2._gefen_global_step == 2


def test_amp_overflow_skips_step_without_mutation():
    m = _tiny_model()
    opt = Gefen(m.named_parameters(), lr=1e-2, fused=False)
    _train(m, opt, 1)
    before = [p.detach().clone() for p in m.parameters()]
    step_before = opt._gefen_global_step
    for p in m.parameters():
        p.grad = torch.ones_like(p)
    opt.found_inf = torch.tensor(1.0)
    opt.grad_scale = torch.tensor(1024.0)
    try:
        opt.step()
    finally:
        del opt.found_inf, opt.grad_scale
    for a, b in zip(before, m.parameters()):
        assert torch.equal(a, b)
    assert opt._gefen_global_step == step_before
    # a finite step with a scale divides the gradients (scale 4 on 4x grads == plain step)
    m_a, m_b = _tiny_model(3), _tiny_model(3)
    oa = Gefen(m_a.named_parameters(), lr=1e-2, fused=False)
    ob = Gefen(m_b.named_parameters(), lr=1e-2, fused=False)
    g = torch.Generator().manual_seed(5)
    grads = [torch.randn(p.shape, generator=g) for p in m_a.parameters()]
    for p, gr in zip(m_a.parameters(), grads):
        p.grad = gr.clone()
    for p, gr in zip(m_b.parameters(), grads):
        p.grad = gr * 4.0
    oa.step()
    ob.found_inf = torch.tensor(0.0)
    ob.grad_scale = torch.tensor(4.0)
    ob.step()
    for a, b in zip(m_a.parameters(), m_b.parameters()):
        assert torch.allclose(a, b, atol=1e-7)


def test_codebook_refresh_requantises_and_keeps_training():
    m = _tiny_model()
    opt = Gefen(m.named_parameters(), lr=1e-2, fused=False, codebook_refresh_every=2)
    losses = _train(m, opt, 6)
    assert losses[-1] < losses[0]
    assert opt._gefen_codebook.shape == (256,)


def test_closure_runs_first_and_returns_loss():
    m = _tiny_model()
    opt = Gefen(m.named_parameters(), lr=1e-2, fused=False)
    x, y = torch.randn(4, 32), torch.randn(4, 16)

    def closure():
        opt.zero_grad()
        loss = ((m(x) - y) ** 2).mean()
        loss.backward()
        return loss

    out = opt.step(closure)
    assert out is not None and out.item() > 0 and opt._gefen_global_step == 1


def test_capturable_counters_are_tensors_and_match_eager_on_cpu():
    ma, mb = _tiny_model(4), _tiny_model(4)
    oa = Gefen(ma.named_parameters(), lr=1e-2, fused=False)
    ob = Gefen(mb.named_parameters(), lr=1e-2, fused=False, capturable=True)
    la = _train(ma, oa, 4)
    lb = _train(mb, ob, 4)
    assert torch.is_tensor(ob.state[mb[0].weight]["step"])
    assert float(ob.state[mb[0].weight]["step"]) == 4.0
    assert max(abs(a - b) for a, b in zip(la, lb)) < 1e-5
    sd = ob.state_dict()
    oc = Gefen(_tiny_model(4).named_parameters(), lr=1e-2, fused=False)
    oc.load_state_dict(sd)                           # capturable -> eager: counters become ints
    assert oc.state[oc.param_groups[0]["params"][0]]["step"] == 4
