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


_DCP_SHAPES = [("layer.weight", (16, 24)), ("layer.bias", (16,)), ("head.weight", (8, 16))]


def _dcp_worker(rank, world, port, path, saver, loader, q):
    """Train 3 steps with ``saver``'s package on 2 Gloo ranks, save through its DCP wrapper, load
    into ``loader``'s package, step both once more and report the largest parameter difference."""
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    import gefen_x_b200 as ours

    mods = {"ref": _reference(), "ours": ours}
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mesh = init_device_mesh("cpu", (world,))

        def full(seed):
            g = torch.Generator().manual_seed(seed)
            return {n: torch.randn(s, generator=g) * 0.1 for n, s in _DCP_SHAPES}

        def make(mod):
            ps = [(n, distribute_tensor(t.clone(), mesh, [Shard(0)]).requires_grad_(True))
                  for n, t in full(0).items()]
            return ps, mod.Gefen(ps, lr=1e-2, fused=False, factored_v_2d=False)

        def step(ps, opt, k):
            for (n, p), t in zip(ps, full(100 + k).values()):
                p.grad = distribute_tensor(t, mesh, [Shard(0)])
            opt.step()

        S, L = mods[saver], mods[loader]
        ps, opt = make(S)
        for k in range(3):
            step(ps, opt, k)
        sd = S.GefenDCPState(opt).state_dict()
        keys = sorted(sd.keys())
        dcp.save({"optimizer": sd}, storage_writer=S.GefenFileSystemWriter(path), planner=S.GefenSavePlanner())
        dist.barrier()
        ps2, opt2 = make(L)
        for (_, a), (_, b) in zip(ps, ps2):
            b.data.copy_(a.data)
        dcp.load({"optimizer": L.GefenDCPState(opt2)}, checkpoint_id=path)
        step(ps, opt, 3)
        step(ps2, opt2, 3)
        diff = max(float((a.detach().to_local() - b.detach().to_local()).abs().max())
                   for (_, a), (_, b) in zip(ps, ps2))
        q.put((rank, dict(keys=keys, diff=diff)))
    except Exception:  # pragma: no cover - reported to the parent
        import traceback

        q.put((rank, dict(error=traceback.format_exc())))
    finally:
        dist.destroy_process_group()


def _dcp_run(saver, loader):
    import socket
    import tempfile

    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_dcp_worker, args=(r, 2, port, os.path.join(d, "ck"), saver, loader, q))
                 for r in range(2)]
        for pr in procs:
            pr.start()
        res = dict(q.get(timeout=300) for _ in range(2))
        for pr in procs:
            pr.join(timeout=60)
    for r in res:
        assert "error" not in res[r], res[r].get("error")
    return res


def test_dcp_checkpoints_load_across_the_two_packages():
    """A DCP checkpoint (``GefenDCPState`` + writer + planner) saved by either package on 2 Gloo
    ranks loads in the other: same key set, and the step after the load lands where the
    reference's own save -> load lands (the re-blocking at load is common to both)."""
    own = _dcp_run("ref", "ref")
    r2o = _dcp_run("ref", "ours")
    o2r = _dcp_run("ours", "ref")
    assert own[0]["keys"] == r2o[0]["keys"] == o2r[0]["keys"]
    for r in (0, 1):
        assert abs(r2o[r]["diff"] - own[r]["diff"]) < 1e-6, (r, r2o[r]["diff"], own[r]["diff"])
        assert abs(o2r[r]["diff"] - own[r]["diff"]) < 1e-6, (r, o2r[r]["diff"], own[r]["diff"])
        assert own[r]["diff"] < 5e-3


_MUON_SHAPES = [("a.weight", (16, 24)), ("b.weight", (8, 16)), ("c.weight", (24, 8)),
                ("d.weight", (5, 8)), ("e.weight", (1, 8))]          # uneven and empty row shards


def _dmuon_worker(rank, world, port, path, saver, loader, q):
    """``sharded_mode="distributed"`` on 2 Gloo ranks with ``saver``'s package, consolidated
    ``state_dict`` to a file, loaded by ``loader``'s package, one more step on both."""
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    import gefen_x_b200 as ours

    mods = {"ref": _reference(), "ours": ours}
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mesh = init_device_mesh("cpu", (world,))

        def full(seed):
            g = torch.Generator().manual_seed(seed)
            return {n: torch.randn(s, generator=g) * 0.1 for n, s in _MUON_SHAPES}

        def make(mod):
            ps = [(n, distribute_tensor(t.clone(), mesh, [Shard(0)]).requires_grad_(True))
                  for n, t in full(0).items()]
            return ps, mod.GefenMuon(ps, lr=2e-2, fused=False, sharded_mode="distributed")

        def step(ps, opt, k):
            for n, p in ps:
                p.grad = distribute_tensor(full(100 + k)[n], mesh, [Shard(0)])
            opt.step()

        S, L = mods[saver], mods[loader]
        ps, opt = make(S)
        for k in range(3):
            step(ps, opt, k)
        after3 = {n: p.full_tensor().detach().clone() for n, p in ps}
        sd = opt.state_dict()
        if rank == 0:
            torch.save({"sd": sd, "weights": after3}, path)
        dist.barrier()
        blob = torch.load(path, weights_only=False)
        ps2, opt2 = make(L)
        for n, p in ps2:
            p.data.copy_(distribute_tensor(blob["weights"][n], mesh, [Shard(0)]))
        opt2.load_state_dict(blob["sd"])
        step(ps, opt, 3)
        step(ps2, opt2, 3)
        diff = max(float((a.full_tensor().detach() - b.full_tensor().detach()).abs().max())
                   for (_, a), (_, b) in zip(ps, ps2))
        man = sd["gefen_muon_distributed"]
        q.put((rank, dict(diff=diff, after3={n: t.numpy() for n, t in after3.items()},
                          man_keys=sorted(man), entry_keys=sorted(man["groups"][0]["params"][0]),
                          owners=[e["owner"] for e in man["groups"][0]["params"]])))
    except Exception:  # pragma: no cover - reported to the parent
        import traceback

        q.put((rank, dict(error=traceback.format_exc())))
    finally:
        dist.destroy_process_group()


def _spawn2(target, *args):
    import socket
    import tempfile

    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=target, args=(r, 2, port, os.path.join(d, "ck.pt")) + args + (q,))
                 for r in range(2)]
        for pr in procs:
            pr.start()
        res = dict(q.get(timeout=300) for _ in range(2))
        for pr in procs:
            pr.join(timeout=60)
    for r in res:
        assert "error" not in res[r], res[r].get("error")
    return res


def test_distributed_muon_trajectory_and_manifest_match_the_reference():
    """Owner-computed Muon on 2 ranks: the same parameters as the reference package after three
    steps (the CPU statements share their roundings), the same manifest fields and owners, and
    the consolidated checkpoint of either package continues in the other without a difference."""
    import numpy as np

    rr = _spawn2(_dmuon_worker, "ref", "ref")
    oo = _spawn2(_dmuon_worker, "ours", "ours")
    ro = _spawn2(_dmuon_worker, "ref", "ours")
    orf = _spawn2(_dmuon_worker, "ours", "ref")
    for n in rr[0]["after3"]:
        assert np.abs(rr[0]["after3"][n] - oo[0]["after3"][n]).max() < 1e-6, n
    assert rr[0]["man_keys"] == oo[0]["man_keys"] and rr[0]["entry_keys"] == oo[0]["entry_keys"]
    assert rr[0]["owners"] == oo[0]["owners"]
    for res in (rr, oo, ro, orf):
        for r in (0, 1):
            assert res[r]["diff"] < 1e-6, res[r]["diff"]


_PERIOD_SHAPES = [(7,), (64,), (100,), (3, 5), (48, 96), (96, 48), (128, 128), (30, 77), (256,), (2, 3, 4), (1,),
                  (512, 64), (17, 17)]


@pytest.mark.parametrize("kw", [dict(), dict(factored_v_2d=False), dict(codebook_refresh_every=1)])
def test_periods_codebook_and_parameters_match_the_reference_over_shapes(kw):
    """First-step analysis against the reference package: the same block period for every
    shape, a bit-identical learned codebook (also after a refresh), parameters within an ulp."""
    import gefen_x_b200 as ours

    def run(mod):
        g = torch.Generator().manual_seed(0)
        ps = [("p%d.weight" % i, (torch.randn(s, generator=g) * 0.1).requires_grad_())
              for i, s in enumerate(_PERIOD_SHAPES)]
        opt = mod.Gefen(ps, lr=1e-3, fused=False, **kw)
        for _ in range(2):
            for _, p in ps:
                ramp = 1 + torch.arange(p.shape[-1]).float() / p.shape[-1]      # column structure
                p.grad = torch.randn(p.shape, generator=g) * ramp
            opt.step()
        return [opt.state[p]["automatic_period"] for _, p in ps], [p.detach() for _, p in ps], opt

    pa, wa, oa = run(_reference())
    pb, wb, ob = run(ours)
    assert pa == pb
    assert torch.equal(oa.state_dict()["gefen_codebook"], ob.state_dict()["gefen_codebook"])
    for a, b in zip(wa, wb):
        torch.testing.assert_close(a, b, rtol=0, atol=1e-7)


def test_muon_parameter_split_matches_the_reference():
    import importlib

    import gefen_x_b200 as ours

    _reference()
    ref_params = importlib.import_module("gefen.params")

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = nn.Linear(8, 8, bias=False)
            self.norm = nn.LayerNorm(8)
            self.mlp = nn.Linear(8, 16)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed_tokens = nn.Embedding(10, 8)
            self.layers = nn.ModuleList([Block(), Block()])
            self.lm_head = nn.Linear(8, 10, bias=False)
            self.wte = nn.Embedding(4, 8)

    m = Net()

    def names(parts):
        return [sorted(n for n, _ in part) for part in parts]

    assert names(ref_params.split_params_for_muon(m)) == names(ours.split_params_for_muon(m))


def _rank_local_worker(rank, world, port, path, saver, loader, q):
    """Plain Gefen on row shards (rank-local codebooks and blocks): ``state_dict`` of ``saver``'s
    package written by rank 0, loaded on both ranks by ``loader``'s package, one more step."""
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    import gefen_x_b200 as ours

    mods = {"ref": _reference(), "ours": ours}
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mesh = init_device_mesh("cpu", (world,))

        def full(seed, shape):
            return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * 0.1

        def make(mod):
            ps = [("w", distribute_tensor(full(0, (16, 24)), mesh, [Shard(0)]).requires_grad_(True)),
                  ("b", distribute_tensor(full(1, (16,)), mesh, [Shard(0)]).requires_grad_(True))]
            return ps, mod.Gefen(ps, lr=1e-2, fused=False, factored_v_2d=False)

        def step(ps, opt, k):
            for i, (n, p) in enumerate(ps):
                p.grad = distribute_tensor(full(100 + 10 * k + i, tuple(p.shape)), mesh, [Shard(0)])
            opt.step()

        S, L = mods[saver], mods[loader]
        ps, opt = make(S)
        for k in range(3):
            step(ps, opt, k)
        sd = opt.state_dict()
        weights = {n: p.full_tensor().detach().clone() for n, p in ps}
        if rank == 0:
            torch.save({"sd": sd, "weights": weights}, path)
        dist.barrier()
        blob = torch.load(path, weights_only=False)
        ps2, opt2 = make(L)
        for n, p in ps2:
            p.data.copy_(distribute_tensor(blob["weights"][n], mesh, [Shard(0)]))
        opt2.load_state_dict(blob["sd"])
        step(ps, opt, 3)
        step(ps2, opt2, 3)
        diff = max(float((a.full_tensor().detach() - b.full_tensor().detach()).abs().max())
                   for (_, a), (_, b) in zip(ps, ps2))
        meta = sd["param_groups"][0]["_gefen_checkpoint_metadata"]
        first = sd["state"][sd["param_groups"][0]["params"][0]]
        q.put((rank, dict(diff=diff, top=sorted(sd), meta=sorted(meta), version=meta["format_version"],
                          marker=sorted(meta["rank_local_sharded_state"]), carrier=sorted(map(str, first)),
                          signature=meta["rank_local_sharded_state"]["signatures"])))
    except Exception:  # pragma: no cover - reported to the parent
        import traceback

        q.put((rank, dict(error=traceback.format_exc())))
    finally:
        dist.destroy_process_group()


def test_rank_local_dtensor_checkpoints_load_across_the_two_packages():
    """``rank_local_dtensor_v2``: the same outer schema (carrier and member entries, marker,
    metadata version, per-rank signatures) and files of either package restore in the other."""
    rr = _spawn2(_rank_local_worker, "ref", "ref")
    oo = _spawn2(_rank_local_worker, "ours", "ours")
    ro = _spawn2(_rank_local_worker, "ref", "ours")
    orf = _spawn2(_rank_local_worker, "ours", "ref")
    for key in ("top", "meta", "version", "marker", "carrier", "signature"):
        assert rr[0][key] == oo[0][key], key
    for res in (rr, oo, ro, orf):
        for r in (0, 1):
            assert res[r]["diff"] < 1e-6, res[r]["diff"]


def test_public_surface_and_scheduler_hooks_match_the_reference():
    """Every public name, constructor argument and default of the reference exists here; the hybrid
    is a ``torch.optim.Optimizer`` for LR schedulers and dispatches step / state-dict hooks."""
    import inspect

    import gefen_x_b200 as ours

    ref = _reference()
    assert [n for n in ref.__all__ if not hasattr(ours, n)] == []
    for cls in ("Gefen", "GefenMuon", "GefenMuonHybrid", "GefenDCPState"):
        ra = inspect.signature(getattr(ref, cls).__init__).parameters
        oa = inspect.signature(getattr(ours, cls).__init__).parameters
        assert [k for k in ra if k not in oa] == [], cls
        assert [(k, ra[k].default, oa[k].default) for k in ra
                if ra[k].default is not inspect.Parameter.empty and ra[k].default != oa[k].default] == [], cls
        rm = {n for n, _ in inspect.getmembers(getattr(ref, cls), callable) if not n.startswith("_")}
        om = {n for n, _ in inspect.getmembers(getattr(ours, cls), callable) if not n.startswith("_")}
        assert sorted(rm - om) == [], cls
    m = _model()
    opt = ours.GefenMuonHybrid(m, lr=3e-3, fused=False)
    assert isinstance(opt, torch.optim.Optimizer)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: 0.5)
    calls = []
    handle = opt.register_step_post_hook(lambda o, a, k: calls.append("step"))
    opt.register_state_dict_pre_hook(lambda o: calls.append("sd"))
    opt.register_load_state_dict_post_hook(lambda o: calls.append("loaded"))
    m(torch.randn(4, 32)).sum().backward()
    opt.step()
    sched.step()
    assert [g["lr"] for g in opt.param_groups] == [1.5e-3] * len(opt.param_groups)
    assert opt.muon.param_groups[0]["lr"] == 1.5e-3           # the scheduler reached the child
    opt.load_state_dict(opt.state_dict())
    assert calls == ["step", "sd", "loaded"]
    handle.remove()
    opt.step()
    assert calls == ["step", "sd", "loaded"]


class _ShardedNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed_tokens = nn.Embedding(12, 8)
        self.fc1 = nn.Linear(8, 16, bias=True)
        self.fc2 = nn.Linear(16, 8, bias=False)
        self.norm = nn.LayerNorm(8)
        self.lm_head = nn.Linear(8, 12, bias=False)


def _hybrid_sharded_worker(rank, world, port, path, saver, loader, mode, q):
    """GefenMuonHybrid over a model whose parameters are row-sharded DTensors on 2 Gloo ranks."""
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    import gefen_x_b200 as ours

    mods = {"ref": _reference(), "ours": ours}
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mesh = init_device_mesh("cpu", (world,))

        def make(mod):
            torch.manual_seed(0)
            m = _ShardedNet()
            for n, p in list(m.named_parameters()):
                parent, _, leaf = n.rpartition(".")
                setattr(m.get_submodule(parent) if parent else m, leaf,
                        nn.Parameter(distribute_tensor(p.detach().clone(), mesh, [Shard(0)])))
            return m, mod.GefenMuonHybrid(m, lr=1e-2, fused=False, sharded_mode=mode)

        def step(m, opt, k):
            g = torch.Generator().manual_seed(100 + k)
            for _, p in m.named_parameters():
                p.grad = distribute_tensor(torch.randn(p.shape, generator=g) * 0.1, mesh, [Shard(0)])
            opt.step()

        m, opt = make(mods[saver])
        for k in range(3):
            step(m, opt, k)
        after = {n: p.full_tensor().detach().clone() for n, p in m.named_parameters()}
        sd = opt.state_dict()
        if rank == 0:
            torch.save({"sd": sd, "weights": after}, path)
        dist.barrier()
        blob = torch.load(path, weights_only=False)
        m2, opt2 = make(mods[loader])
        for n, p in m2.named_parameters():
            p.data.copy_(distribute_tensor(blob["weights"][n], mesh, [Shard(0)]))
        opt2.load_state_dict(blob["sd"])
        step(m, opt, 3)
        step(m2, opt2, 3)
        diff = max(float((a.full_tensor().detach() - b.full_tensor().detach()).abs().max())
                   for (_, a), (_, b) in zip(m.named_parameters(), m2.named_parameters()))
        q.put((rank, dict(diff=diff, after={n: t.numpy() for n, t in after.items()})))
    except Exception:  # pragma: no cover - reported to the parent
        import traceback

        q.put((rank, dict(error=traceback.format_exc())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["distributed", "approx", "exact"])
def test_hybrid_on_dtensor_shards_matches_the_reference_in_every_sharded_mode(mode):
    """Three steps of the hybrid on row shards give the reference's parameters (to an ulp) in
    every ``sharded_mode``, and its checkpoint (consolidated Muon manifest or rank-local payloads
    for the Muon half, rank-local payloads for the backup half) moves between the packages."""
    import numpy as np

    ro = _spawn2(_hybrid_sharded_worker, "ref", "ours", mode)
    orf = _spawn2(_hybrid_sharded_worker, "ours", "ref", mode)
    for n in ro[0]["after"]:
        assert np.abs(ro[0]["after"][n] - orf[0]["after"][n]).max() < 1e-6, n
    for res in (ro, orf):
        for r in (0, 1):
            assert res[r]["diff"] < 1e-6, res[r]["diff"]


@pytest.mark.parametrize("kw", [dict(deterministic=True), dict(eps=1e-6, betas=(0.95, 0.99)), dict(weight_decay=0.1),
                                dict(codebook_refresh_every=5), dict(lr=torch.tensor(3e-3))],
                         ids=["deterministic", "eps-betas", "decay", "refresh", "tensor-lr"])
def test_gefen_options_follow_the_reference(kw):
    import gefen_x_b200 as ours

    ref = _reference()
    base = dict(lr=3e-3, fused=False)
    base.update(kw)
    a = _train(lambda m: ref.Gefen(list(m.named_parameters()), **base), steps=40)
    b = _train(lambda m: ours.Gefen(list(m.named_parameters()), **base), steps=40)
    assert ((a - b).abs() / a).max().item() < 2e-3


@pytest.mark.parametrize("kw", [dict(nesterov=False), dict(normuon=True), dict(cautious=True),
                                dict(adjust_lr_fn="original"), dict(ns_schedule="tuned4"), dict(batched_ns=True),
                                dict(momentum=0.9, weight_decay=0.05)],
                         ids=["plain-momentum", "normuon", "cautious", "original-lr", "tuned4", "batched", "decay"])
def test_muon_options_follow_the_reference(kw):
    import gefen_x_b200 as ours

    ref = _reference()

    def make(mod):
        return lambda m: mod.GefenMuon([(n, p) for n, p in m.named_parameters() if p.ndim == 2], lr=3e-3,
                                       fused=False, **kw)

    a = _train(make(ref), steps=40)
    b = _train(make(ours), steps=40)
    assert ((a - b).abs() / a).max().item() < 2e-3


def test_gradient_histogram_dump_matches_the_reference(tmp_path):
    """``LIST_STEPS_SAVE_HIST_GRAD`` / ``SAVE_CODEBOOK_PREFIX``: the same file name, dictionary keys
    and counts as the reference package writes."""
    import importlib

    import gefen_x_b200 as ours

    ref = _reference()
    out = {}
    for tag, mod, qname in (("ref", ref, "gefen.quantization"), ("ours", ours, "gefen_x_b200.quant.codebook")):
        qm = importlib.import_module(qname)
        qm.LIST_STEPS_SAVE_HIST_GRAD = [2]
        qm.SAVE_CODEBOOK_PREFIX = str(tmp_path / tag / "cb")
        try:
            _train(lambda m: mod.Gefen(list(m.named_parameters()), lr=3e-3, fused=False), steps=4)
        finally:
            qm.LIST_STEPS_SAVE_HIST_GRAD = None
            qm.SAVE_CODEBOOK_PREFIX = None
        files = sorted(os.listdir(tmp_path / tag))
        assert files == ["cb_grad_hist_step_2.pt"]
        out[tag] = torch.load(tmp_path / tag / files[0])
    a, b = out["ref"], out["ours"]
    assert sorted(a) == sorted(b)
    assert torch.equal(a["hist"], b["hist"]) and a["num_samples"] == b["num_samples"]
    assert torch.equal(a["bin_edges"], b["bin_edges"]) and a["bin_width"] == b["bin_width"]


def test_module_level_functions_and_constants_match_the_reference():
    """Every public constant and function of the reference's modules exists under the same name
    in its counterpart here, and the single-tensor statements give the same numbers."""
    import importlib
    import inspect

    _reference()
    pairs = [("gefen.gefen", "gefen_x_b200.optim.gefen"), ("gefen.partitioning", "gefen_x_b200.quant.partitioning"),
             ("gefen.quantization", "gefen_x_b200.quant.codebook"), ("gefen.gefen_muon", "gefen_x_b200.optim.muon"),
             ("gefen.hybrid", "gefen_x_b200.optim.hybrid"), ("gefen.params", "gefen_x_b200.optim.params"),
             ("gefen.dcp", "gefen_x_b200.ckpt.dcp"), ("gefen.tools.find_lr", "gefen_x_b200.tools.find_lr"),
             ("gefen.tools.lr_calibration", "gefen_x_b200.tools.lr_calibration"),
             ("gefen.tools.run_model_calibration", "gefen_x_b200.tools.run_model_calibration")]
    for rname, oname in pairs:
        rm, om = importlib.import_module(rname), importlib.import_module(oname)
        consts = [n for n, v in vars(rm).items() if n.isupper() and not n.startswith("_")
                  and isinstance(v, (int, float, str, bool, tuple, type(None)))]
        assert [n for n in consts if not hasattr(om, n)] == [], rname
        assert [(n, getattr(rm, n), getattr(om, n)) for n in consts if getattr(rm, n) != getattr(om, n)] == [], rname
        funcs = [n for n, v in vars(rm).items() if not n.startswith("_") and (inspect.isfunction(v) or inspect.isclass(v))
                 and v.__module__ == rm.__name__]
        assert [n for n in funcs if not hasattr(om, n)] == [], rname
    rg, og = importlib.import_module("gefen.gefen"), importlib.import_module("gefen_x_b200.optim.gefen")
    g = torch.Generator().manual_seed(5)
    flat = torch.randn(96, generator=g)
    for op in ("mean", "max"):
        assert torch.equal(rg.automatic_partition_reduce(flat, 8, op), og.automatic_partition_reduce(flat, 8, op))
    cb = torch.sort(torch.cat([torch.tensor([-1.0, 1.0]), torch.rand(254, generator=g) * 2 - 1])).values
    vals = torch.rand(12, 8, generator=g) * 2 - 1
    ia, ib = rg.gefen_nearest_codebook_indices(cb, vals), og.gefen_nearest_codebook_indices(cb, vals)
    assert ia.dtype == ib.dtype == torch.uint8 and torch.equal(ia, ib)
    like = torch.zeros(1, dtype=torch.bfloat16)
    assert torch.equal(rg.gefen_dequantize_unpacked_indices(cb, ia, like), og.gefen_dequantize_unpacked_indices(cb, ib, like))
    va, vb = torch.rand(12, 1, generator=g), None
    vb = va.clone()
    rg.automatic_vmean_update(va, vals, 0.99, use_fused=False)
    og.automatic_vmean_update(vb, vals, 0.99, use_fused=False)
    torch.testing.assert_close(va, vb, rtol=1e-6, atol=0)
    items = [("w", flat, 8, flat)]
    kw = dict(codebook_device=torch.device("cpu"), num_codebooks=256, force_endpoints=True, verbose=False,
              compute_mse_logging=False)
    assert torch.equal(rg.learn_gefen_exact_codebook_from_grad_periods(grad_periods=iter(items), **kw),
                       og.learn_gefen_exact_codebook_from_grad_periods(grad_periods=iter(items), **kw))


def _dcp_reshard_worker(rank, world, port, path, pkg, mode, q):
    """``mode="save"``: 3 steps and a DCP save with ``pkg``; ``mode="load"``: load into ``pkg`` at this
    world size, one more step, report the full parameters."""
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    import gefen_x_b200 as ours

    mod = {"ref": _reference(), "ours": ours}[pkg]
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mesh = init_device_mesh("cpu", (world,))

        def full(seed):
            g = torch.Generator().manual_seed(seed)
            return {n: torch.randn(s, generator=g) * 0.1 for n, s in _DCP_SHAPES}

        ps = [(n, distribute_tensor(t.clone(), mesh, [Shard(0)]).requires_grad_(True)) for n, t in full(0).items()]
        opt = mod.Gefen(ps, lr=1e-2, fused=False, factored_v_2d=False)

        def step(k):
            for (_, p), t in zip(ps, full(100 + k).values()):
                p.grad = distribute_tensor(t, mesh, [Shard(0)])
            opt.step()

        if mode == "save":
            for k in range(3):
                step(k)
            dcp.save({"optimizer": mod.GefenDCPState(opt).state_dict()},
                     storage_writer=mod.GefenFileSystemWriter(path), planner=mod.GefenSavePlanner())
            weights = {n: p.full_tensor().detach().clone() for n, p in ps}      # collective: every rank
            if rank == 0:
                torch.save(weights, path + ".weights")
            dist.barrier()
            q.put((rank, "saved"))
        else:
            weights = torch.load(path + ".weights")
            for n, p in ps:
                p.data.copy_(distribute_tensor(weights[n], mesh, [Shard(0)]))
            dcp.load({"optimizer": mod.GefenDCPState(opt)}, checkpoint_id=path)
            step(3)
            q.put((rank, {n: p.full_tensor().detach().numpy() for n, p in ps}))
    except Exception:  # pragma: no cover - reported to the parent
        import traceback

        q.put((rank, dict(error=traceback.format_exc())))
    finally:
        dist.destroy_process_group()


def _spawn_world(world, target, *args):
    import socket

    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=target, args=(r, world, port) + args + (q,)) for r in range(world)]
    for pr in procs:
        pr.start()
    res = dict(q.get(timeout=300) for _ in range(world))
    for pr in procs:
        pr.join(timeout=60)
    for r in res:
        assert not (isinstance(res[r], dict) and "error" in res[r]), res[r].get("error")
    return res


def test_dcp_resharding_across_packages_matches_the_reference_loader(tmp_path):
    """A 2-rank DCP checkpoint of the reference resharded to 1 and to 4 ranks by this package
    lands where the reference's own loader lands; a checkpoint of this package reshards in the
    reference the same way."""
    import numpy as np

    path = str(tmp_path / "from_ref")
    _spawn_world(2, _dcp_reshard_worker, path, "ref", "save")
    for world in (1, 4):
        a = _spawn_world(world, _dcp_reshard_worker, path, "ref", "load")[0]
        b = _spawn_world(world, _dcp_reshard_worker, path, "ours", "load")[0]
        assert max(float(np.abs(a[n] - b[n]).max()) for n in a) < 1e-6, world
    path = str(tmp_path / "from_ours")
    _spawn_world(2, _dcp_reshard_worker, path, "ours", "save")
    a = _spawn_world(4, _dcp_reshard_worker, path, "ref", "load")[0]
    b = _spawn_world(4, _dcp_reshard_worker, path, "ours", "load")[0]
    assert max(float(np.abs(a[n] - b[n]).max()) for n in a) < 1e-6


@pytest.mark.parametrize("kw", [dict(backup_optimizer="adamw"), dict(backup_1d_period_one=True),
                                dict(backup_2d_period_one=True), dict(no_decay_substrings=("bias",), weight_decay=0.1),
                                dict(muon_lr=1e-3, backup_lr=5e-3), dict(muon_weight_decay=0.2, backup_weight_decay=0.0),
                                dict(backup_substrings=("0.",)),
                                dict(nesterov=False, momentum=0.9, ns_steps=4, ns_schedule=None)],
                         ids=["adamw-backup", "1d-period-one", "2d-period-one", "no-decay", "split-lr", "split-decay",
                              "routing", "plain-quintic"])
def test_hybrid_routing_options_follow_the_reference(kw):
    import gefen_x_b200 as ours

    ref = _reference()
    a = _train(lambda m: ref.GefenMuonHybrid(m, lr=3e-3, fused=False, **kw), steps=40)
    b = _train(lambda m: ours.GefenMuonHybrid(m, lr=3e-3, fused=False, **kw), steps=40)
    assert ((a - b).abs() / a).max().item() < 2e-3


@pytest.mark.parametrize("kw", [dict(force_1d_period_one=True), dict(force_2d_period_one=True),
                                dict(period_one_substrings=("2.",)),
                                dict(factored_v_2d=False, force_2d_period_one=True)],
                         ids=["1d", "2d", "substrings", "unfactored-2d"])
def test_period_one_options_follow_the_reference(kw):
    import gefen_x_b200 as ours

    ref = _reference()
    a = _train(lambda m: ref.Gefen(list(m.named_parameters()), lr=3e-3, fused=False, **kw), steps=40)
    b = _train(lambda m: ours.Gefen(list(m.named_parameters()), lr=3e-3, fused=False, **kw), steps=40)
    assert ((a - b).abs() / a).max().item() < 2e-3


def test_misuse_raises_the_same_exception_types_as_the_reference():
    import gefen_x_b200 as ours

    ref = _reference()

    def p(shape=(4, 8)):
        return torch.randn(shape).requires_grad_()

    def with_grad(m, grad_of):
        w = p()
        opt = m.Gefen([("w", w)], lr=1e-3, fused=False)
        w.grad = grad_of(w)
        opt.step()

    def dup(m):
        w = p()
        m.Gefen([("a", w), ("b", w)], lr=1e-3, fused=False)

    cases = {
        "negative lr": lambda m: m.Gefen([("w", p())], lr=-1.0, fused=False),
        "beta of 1": lambda m: m.Gefen([("w", p())], lr=1e-3, betas=(1.0, 0.9), fused=False),
        "negative eps": lambda m: m.Gefen([("w", p())], lr=1e-3, eps=-1, fused=False),
        "negative decay": lambda m: m.Gefen([("w", p())], lr=1e-3, weight_decay=-1, fused=False),
        "no parameters": lambda m: m.Gefen([], lr=1e-3, fused=False),
        "unnamed parameters": lambda m: m.Gefen([p()], lr=1e-3, fused=False),
        "duplicate parameter": dup,
        "complex parameter": lambda m: m.Gefen([("w", torch.zeros(4, dtype=torch.complex64).requires_grad_())],
                                               lr=1e-3, fused=False),
        "negative refresh": lambda m: m.Gefen([("w", p())], lr=1e-3, fused=False, codebook_refresh_every=-2),
        "muon on a vector": lambda m: m.GefenMuon([("w", p((8,)))], lr=1e-3, fused=False),
        "muon mode": lambda m: m.GefenMuon([("w", p())], lr=1e-3, fused=False, sharded_mode="x"),
        "muon schedule": lambda m: m.GefenMuon([("w", p())], lr=1e-3, fused=False, ns_schedule="zzz"),
        "muon zero iterations": lambda m: m.GefenMuon([("w", p())], lr=1e-3, fused=False, ns_steps=0),
        "muon momentum": lambda m: m.GefenMuon([("w", p())], lr=1e-3, fused=False, momentum=1.5),
        "muon lr rule": lambda m: m.GefenMuon([("w", p())], lr=1e-3, fused=False, adjust_lr_fn="zz"),
        "hybrid backup kind": lambda m: m.GefenMuonHybrid(_model(), lr=1e-3, fused=False, backup_optimizer="sgd"),
        "hybrid add group": lambda m: m.GefenMuonHybrid(_model(), lr=1e-3, fused=False).add_param_group({"params": []}),
        "load of an empty dict": lambda m: m.Gefen([("w", p())], lr=1e-3, fused=False).load_state_dict(
            {"state": {}, "param_groups": []}),
        "nan gradient": lambda m: with_grad(m, lambda w: torch.full_like(w, float("nan"))),
        "sparse gradient": lambda m: with_grad(m, lambda w: torch.zeros_like(w).to_sparse()),
    }
    for name, fn in cases.items():
        kinds = []
        for m in (ref, ours):
            try:
                fn(m)
                kinds.append("ok")
            except Exception as exc:  # noqa: BLE001
                kinds.append(type(exc).__name__)
        assert kinds[0] == kinds[1], (name, kinds)
