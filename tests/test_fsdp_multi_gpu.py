"""Multi-GPU tests of the sharded runtime: 2 ranks must follow the 1-GPU trajectory.

Ranks are child processes started with torch.distributed.run on one node.  The
reference's multi-rank tests follow the same "single-process oracle on the same
seeded full tensors" pattern (reference tests/test_muon_fsdp2_parity.py:60-70).
"""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _single_gpu_losses(world, clip, optimizer="gefen"):
    from gefen_x_b200.models.decoder import get_config
    from gefen_x_b200.parallel.fsdp import ShardedTrainer

    cfg = get_config("tiny-llama", qk_norm=True, hidden=256, ffn=512, n_layers=3)
    dev = torch.device("cuda", 0)
    tr = ShardedTrainer(cfg, device=dev, dtype=torch.bfloat16, lr=6e-4, weight_decay=0.01,
                        clip_grad_norm=clip, seed=5, optimizer=optimizer)
    g = torch.Generator().manual_seed(2)
    tok = torch.randint(0, cfg.vocab_size, (world * 2, 129), generator=g).to(dev)
    return [float(tr.step(tok[:, :-1], tok[:, 1:]).item()) for _ in range(12)]


@pytest.mark.parametrize("rs_mode,clip,ag", [("stash", "1.0", "plain"), ("fused", "none", "plain"),
                                             ("stash", "1.0", "ag"), ("stash", "1.0", "hybrid"),
                                             ("stash", "1.0", "kgather"), ("stash", "1.0", "nvls"),
                                             ("fused", "1.0", "nvls"), ("fused", "1.0", "plain")])
def test_two_ranks_track_single_gpu(tmp_path, rs_mode, clip, ag):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = tmp_path / "losses.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "_fsdp_worker.py"), str(out), rs_mode, clip, ag]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    if ag == "nvls" and not out.exists() and "multicast" in (proc.stdout + proc.stderr):
        pytest.skip("no NVLS multicast mapping on this system")
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    multi = json.load(open(out))
    ref = _single_gpu_losses(2, None if clip == "none" else float(clip),
                             "muon_hybrid" if ag == "hybrid" else "gefen")
    got = multi["mean_loss"]
    assert multi.get("nvls", False) == (ag == "nvls")
    assert got[-1] < got[0] - 0.5
    for a, b in zip(ref, got):
        assert abs(a - b) < 0.05 * max(1.0, abs(a)), (ref, got)
    assert multi["state_bytes_per_param"] < 1.2


def test_one_optimizer_over_two_devices_matches_single_device():
    """Layer-wise model parallel (parameters of one optimizer on two GPUs): per-device codebook,
    threshold and bucket-table copies; same trajectory as all parameters on one device
    (reference tests/test_codebook_multi_device.py)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from gefen_x_b200 import Gefen

    def params(devs):
        g = torch.Generator().manual_seed(0)
        shapes = [("a.weight", (64, 256)), ("b.weight", (128, 64)), ("norm.weight", (256,)), ("c.weight", (32, 512))]
        return [(n, (torch.randn(s, generator=g) * 0.05).bfloat16().to(devs[i % len(devs)]).requires_grad_())
                for i, (n, s) in enumerate(shapes)]

    d0, d1 = torch.device("cuda", 0), torch.device("cuda", 1)
    pa, pb = params([d0]), params([d0, d1])
    oa, ob = Gefen(pa, lr=1e-2, weight_decay=0.01), Gefen(pb, lr=1e-2, weight_decay=0.01)
    for step in range(4):
        g = torch.Generator().manual_seed(100 + step)
        for (_, a), (_, b) in zip(pa, pb):
            gr = (torch.randn(a.shape, generator=g) * 1e-2).bfloat16()
            a.grad = gr.to(a.device)
            b.grad = gr.to(b.device)
        oa.step()
        ob.step()
    assert {p.device for _, p in pb} == {d0, d1}
    for (n, a), (_, b) in zip(pa, pb):
        assert torch.equal(oa.state[a]["m_codebook"].cpu(), ob.state[b]["m_codebook"].cpu()), n
        torch.testing.assert_close(a.float().cpu(), b.float().cpu(), rtol=0, atol=1e-3, msg=n)
    assert all(v == 0 for v in ob.kernel_status().values())


def _launch(world, script, *args, timeout=600):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    if world == 1:
        cmd = [sys.executable, os.path.join(ROOT, "tests", script)] + [str(a) for a in args]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
               "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
               os.path.join(ROOT, "tests", script)] + [str(a) for a in args]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]


@pytest.mark.parametrize("save_world,load_world", [(2, 1), (1, 2), (4, 2)])
def test_trainer_checkpoint_reshards(tmp_path, save_world, load_world):
    """Resharding checkpoint of the runtime: saved on N ranks, loaded on M; the resumed run continues on
    the saver's loss trajectory (re-quantisation of the momentum on the new shards is the only
    difference), and the rank-local native state dict resumes on the same trajectory (reference
    tests/test_dcp_resharding.py:320-397)."""
    if torch.cuda.device_count() < max(save_world, load_world):
        pytest.skip("needs {} GPUs".format(max(save_world, load_world)))
    _launch(save_world, "_fsdp_ckpt_worker.py", "save", tmp_path)
    saved = json.load(open(tmp_path / "save_w{}.json".format(save_world)))
    assert saved["native_resume_drift"] <= 2e-3, saved
    _launch(load_world, "_fsdp_ckpt_worker.py", "load", tmp_path)
    loaded = json.load(open(tmp_path / "load_w{}.json".format(load_world)))
    assert loaded["step_count"] == 9
    for a, b in zip(saved["continued"], loaded["resumed"]):
        assert abs(a - b) <= 0.02 * abs(a), (saved, loaded)


def test_sharded_optimizer_state_equals_single_gpu_state(tmp_path):
    """Two ranks fed the same batch reduce to exactly the single-GPU gradient, so the sharded optimizer
    state, gathered by rows, must be the single-GPU state: factored row / column moments (the column
    sums cross the shards inside the kernel), weights, and the quantised momentum wherever the two runs
    chose the same block period."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _launch(1, "_fsdp_ckpt_worker.py", "state", tmp_path)
    _launch(2, "_fsdp_ckpt_worker.py", "state", tmp_path)
    one = torch.load(tmp_path / "state_w1.pt")
    two = torch.load(tmp_path / "state_w2.pt")
    cb1, cb2 = one.pop("__codebook__"), two.pop("__codebook__")
    same_codebook = torch.allclose(cb1, cb2, rtol=0, atol=1e-6)
    assert set(one) == set(two) and one
    compared_indices = 0
    for name, a in one.items():
        b = two[name]
        # after one step v = (1 - beta2) * sums of g^2: only the summation order differs.  The token
        # embedding's gradient is a scatter-add of bf16 rows (repeated tokens round differently when the
        # same rows arrive as two halves from two ranks), so it is compared loosely.
        tol = 5e-2 if "embed_tokens" in name else 1e-4
        torch.testing.assert_close(b["v_row"], a["v_row"], rtol=tol, atol=1e-12, msg=name)
        for vc in b["v_col"]:
            torch.testing.assert_close(vc, a["v_col"][0], rtol=tol, atol=1e-12, msg=name)
        torch.testing.assert_close(b["v_col"][0], b["v_col"][1], rtol=0, atol=0, msg=name)   # shards agree exactly
        torch.testing.assert_close(b["w"], a["w"], rtol=0, atol=4e-3, msg=name)
        if same_codebook and all(p == a["period"] for p in b["periods"]):
            compared_indices += 1
            differ = (a["idx"] != b["idx"]).float().mean().item()
            assert differ <= 0.002, (name, differ)
            torch.testing.assert_close(b["dense"], a["dense"], rtol=0, atol=2e-2 * a["dense"].abs().max().item())
    # the quantised momentum is comparable wherever both runs chose the same blocks and codebook
    assert compared_indices > 0 or not same_codebook


@pytest.mark.parametrize("kind", ["gefen", "hybrid"])
def test_optimizers_under_torch_fully_shard(tmp_path, kind):
    """``Gefen`` and ``GefenMuonHybrid`` on the DTensor parameters that torch's ``fully_shard`` creates
    (uneven row shards included): the sharded run tracks the single-GPU run on the same global batch,
    and a state dict taken mid-run (rank-local payloads for plain Gefen) resumes on the same
    trajectory (reference tests/test_gefen_fsdp2_checkpoint.py, tests/test_fused_fsdp2_noncontig.py)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    one, two = tmp_path / "one.json", tmp_path / "two.json"
    _launch(1, "_fsdp2_worker.py", one, kind)
    _launch(2, "_fsdp2_worker.py", two, kind)
    a, b = json.load(open(one)), json.load(open(two))
    assert b["local_shape_of_uneven"] == [[148, 512]]          # 296 rows over 2 ranks
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) <= 0.05 * max(1e-3, abs(x)), (a["losses"], b["losses"])
    for x, y in zip(b["continued"], b["resumed"]):
        assert abs(x - y) <= 0.01 * max(1e-3, abs(x)), (b["continued"], b["resumed"])
