"""CPU tests of the lr tooling (model: reference tests/test_find_lr.py, tests/test_lr_calibration.py)."""
import torch
import torch.nn as nn

from gefen_x_b200 import Gefen, GefenMuonHybrid
from gefen_x_b200.models.decoder import DecoderLM, get_config
from gefen_x_b200.tools import (calibrate_relative, calibrate_vs_adamw, lr_range_test,
                                measure_update_rms)
from gefen_x_b200.tools.find_lr import distribute_lrs, find_lr, main


def _setup(hybrid=False):
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.Tanh(), nn.Linear(32, 8))
    x, y = torch.randn(32, 16), torch.randn(32, 8)

    def closure():
        loss = ((model(x) - y) ** 2).mean()
        loss.backward()
        return loss.detach()

    opt = GefenMuonHybrid(list(model.named_parameters()), lr=1e-2, fused=False) if hybrid else \
        Gefen(model.named_parameters(), lr=1e-2, fused=False)
    return model, opt, closure


def test_probes_are_non_destructive():
    for hybrid in (False, True):
        model, opt, closure = _setup(hybrid)
        for _ in range(2):
            opt.zero_grad()
            closure()
            opt.step()
        before = [p.detach().clone() for p in model.parameters()]
        stats = measure_update_rms(opt, closure, num_steps=6, warmup=2)
        assert len(stats) == len(opt.param_groups) and all(s.update_rms > 0 for s in stats)
        rel = calibrate_relative(opt, closure, num_steps=6, warmup=2)
        assert abs(rel.multipliers[rel.reference_label] - 1.0) < 1e-9
        vs = calibrate_vs_adamw(opt, closure, num_steps=6, warmup=2)
        assert len(vs) == 4 and all(v.ratio > 0 for v in vs)
        for a, b in zip(before, model.parameters()):
            assert torch.equal(a, b)


def test_range_test_and_find_lr():
    model, opt, closure = _setup()
    res = lr_range_test(opt, closure, start_lr=1e-5, end_lr=10.0, num_iter=40)
    assert 1e-5 <= res.suggested_lr <= 10.0 and len(res.lrs) == len(res.losses)
    cfg = get_config("tiny-llama", n_layers=1, hidden=64, ffn=128, vocab_size=128)
    lm = DecoderLM(cfg, seed=0)
    g = torch.Generator().manual_seed(0)
    blocks = torch.randint(0, 128, (24, 17), generator=g)
    w0 = [p.detach().clone() for p in lm.parameters()]
    r = find_lr(lm, blocks, optimizer="gefen", num_iter=12, bs=4, fused=False, verbose=False)
    assert r.lr > 0 and len(r.curve) > 3
    r2 = find_lr(lm, blocks[4:], optimizer="gefen_muon", method="sweep", eval_blocks=blocks[:4],
                 sweep_lrs=[1e-3, 1e-2], sweep_steps=4, warmup=2, bs=4, fused=False, verbose=False)
    assert r2.lr in (1e-3, 1e-2)
    for a, b in zip(w0, lm.parameters()):
        assert torch.equal(a, b)
    assert distribute_lrs([1, 2, 3], ["a", "b"]) == {"a": [1, 3], "b": [2]}


def test_cli_runs(capsys):
    assert main(["--model", "tiny-llama", "--num-iter", "4", "--num-blocks", "12", "--seq-len", "16",
                 "--bs", "2", "--device", "cpu", "--json"]) == 0
    assert '"lr"' in capsys.readouterr().out


def test_calibration_records_and_runner_helpers_follow_the_reference_tool():
    """Record fields of the AdamW comparison, reference selectors, summaries and the name
    classifier / split of the model runner (reference tools/lr_calibration.py:486-499,
    tools/run_model_calibration.py:40-103)."""
    from gefen_x_b200.tools import run_model_calibration as R

    model, opt, closure = _setup(True)
    vs = calibrate_vs_adamw(opt, closure, betas=(0.9, 0.99), num_steps=6, warmup=2)
    r = vs[0]
    assert {"name", "is_muon", "rows", "cols", "gefen_rms", "adamw_rms", "ratio", "active_ratio",
            "sqrt_max"} <= set(r.__dict__)
    assert any(v.is_muon and v.sqrt_max for v in vs) and any(not v.is_muon and v.sqrt_max is None for v in vs)
    assert all(abs(v.ratio - v.adamw_rms / v.gefen_rms) < 1e-9 for v in vs)
    rel = calibrate_relative(opt, closure, reference="gefen", num_steps=6, warmup=2)
    assert ":adam" in rel.reference_label and "multiplier" in rel.summary()
    assert calibrate_relative(opt, closure, reference="muon", num_steps=6, warmup=2).reference_label.count("muon")
    assert R.classify_param_type("model.layers.0.self_attn.q_proj.weight") == "q_proj"
    assert R.param_type("model.embed_tokens.weight") == "embed" and R.param_type("lm_head.weight") == "lm_head"
    assert R.param_type("model.norm.weight") == "norm" and R.param_type("x.bias") == "bias"
    muon, backup = R.split_params_for_muon(model)
    assert all(p.ndim == 2 for _, p in muon) and len(muon) + len(backup) == len(list(model.parameters()))
    assert len(R.CORPUS) == 8


def test_build_token_stream_packs_local_files(tmp_path):
    import json
    from types import SimpleNamespace

    from gefen_x_b200.tools.find_lr import build_token_stream

    class Tok:
        eos_token_id = 1

        def __call__(self, text, add_special_tokens=False):
            return {"input_ids": [2 + (ord(c) % 50) for c in text]}

    path = tmp_path / "rows.jsonl"
    rows = [{"text": "abcdefgh" * 5}, {"instruction": "sum", "input": "1 2", "output": "3"}, {"other": 1}]
    path.write_text("\n".join(json.dumps(r) for r in rows))
    args = SimpleNamespace(dataset=str(path), split="train", max_rows=0, seq=8, eval_blocks=2)
    train, ev = build_token_stream(Tok(), args)
    assert train.shape[1] == 8 and ev.shape[1] == 8 and ev.shape[0] == 1 and train.dtype == torch.long
    total = 40 + 1 + len("sum\n1 2\n3") + 1
    assert train.shape[0] + ev.shape[0] == total // 8
    assert int((torch.cat([train, ev]) == 1).sum()) >= 1                # the EOS separators survive packing
    args.seq = 64
    try:
        build_token_stream(Tok(), args)
        raise AssertionError("expected a ValueError for too little text")
    except ValueError:
        pass


def _tiny_lm():
    cfg = get_config("tiny-llama", n_layers=1, hidden=64, ffn=128, vocab_size=128)
    return DecoderLM(cfg, seed=0)


def test_parallel_sweep_runs_spawned_workers_and_reports_worker_failures():
    from gefen_x_b200.tools.find_lr import find_lr_parallel_sweep

    g = torch.Generator().manual_seed(0)
    blocks = torch.randint(0, 128, (24, 17), generator=g)
    res = find_lr_parallel_sweep(_tiny_lm, blocks[4:], blocks[:4], optimizer="gefen", sweep_lrs=[1e-3, 1e-2],
                                 devices=["cpu"], sweep_steps=3, warmup=1, bs=4, worker_timeout=300)
    assert res.lr in (1e-3, 1e-2) and len(res.curve) == 2 and res.details["devices"] == ["cpu"]
    try:
        find_lr_parallel_sweep(_tiny_lm, blocks[4:], blocks[:4], optimizer="no-such-optimizer", sweep_lrs=[1e-3],
                               devices=["cpu"], sweep_steps=2, warmup=1, bs=4, worker_timeout=300)
        raise AssertionError("a failing worker must raise in the parent")
    except RuntimeError as e:
        assert "worker on cpu failed" in str(e)
    try:
        find_lr_parallel_sweep("/no/such/checkpoint", ["cpu"])
        raise AssertionError("the model-path form needs a dataset")
    except ValueError as e:
        assert "dataset" in str(e)
