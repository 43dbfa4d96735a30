"""Fail-fast agreement among ranks, with every failure injected on the host (Gloo, CPU).

Model: the reference's host-side injection tests for its agreement collectives
(``tests/test_dcp_resharding.py``, ``tests/test_gefen_muon.py`` failure-sync cases;
the collectives themselves at reference ``src/gefen/gefen.py:559-615``).  No GPU is involved.
"""
import os
import socket

import torch
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    from gefen_x_b200 import Gefen
    from gefen_x_b200.parallel import control

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    out = {}
    try:
        # 1. one failing rank is seen by every rank
        out["any_failed"] = control.synchronize_step_failure(rank == 1)
        out["none_failed"] = control.synchronize_step_failure(False)
        # 2. bounds agreement
        lo, hi = control.synchronize_step_control_range((float(rank), 2.0), (float(rank), 2.0))
        out["range"] = (lo, hi)
        # 3. an exception on rank 1 raises on both ranks, before anything else happens
        exc = ValueError("injected on rank 1") if rank == 1 else None
        try:
            control.raise_if_any_rank_failed(exc, what="test step")
            out["raised"] = None
        except ValueError as e:
            out["raised"] = ("own", str(e))
        except RuntimeError as e:
            out["raised"] = ("peer", str(e))
        # 4. a GradScaler overflow on one rank skips the step on every rank, nothing mutated
        mesh = init_device_mesh("cpu", (world,))
        g = torch.Generator().manual_seed(0)
        full = torch.randn(16, 24, generator=g) * 0.1
        p = distribute_tensor(full.clone(), mesh, [Shard(0)]).requires_grad_(True)
        opt = Gefen([("w", p)], lr=1e-2, fused=False, factored_v_2d=False)
        p.grad = distribute_tensor(torch.randn(16, 24, generator=g), mesh, [Shard(0)])
        opt.step()                                   # a clean first step builds the state
        before = p.to_local().clone()
        idx_before = opt.state[p]["m_codebook"].clone()
        step_before = opt._gefen_global_step
        opt.grad_scale = torch.tensor(1024.0)
        opt.found_inf = torch.tensor(1.0 if rank == 1 else 0.0)
        p.grad = distribute_tensor(torch.randn(16, 24, generator=g) * 1024.0, mesh, [Shard(0)])
        opt.step()
        out["skipped"] = (bool(torch.equal(before, p.to_local())),
                          bool(torch.equal(idx_before, opt.state[p]["m_codebook"])),
                          opt._gefen_global_step == step_before)
        # 5. the same gradients without the overflow flag do step, on both ranks
        opt.found_inf = torch.tensor(0.0)
        opt.step()
        out["stepped"] = (not torch.equal(before, p.to_local()), opt._gefen_global_step == step_before + 1)
        q.put((rank, out))
    except Exception as e:  # pragma: no cover - reported to the parent
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))
    finally:
        dist.destroy_process_group()


def test_failure_agreement_and_amp_skip_across_gloo_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    results = dict(q.get(timeout=180) for _ in range(world))
    for pr in procs:
        pr.join(timeout=60)
    for r in range(world):
        assert "error" not in results[r], results[r].get("error")
        o = results[r]
        assert o["any_failed"] is True and o["none_failed"] is False
        assert o["range"] == ((0.0, 2.0), (1.0, 2.0))
        assert o["skipped"] == (True, True, True)
        assert o["stepped"] == (True, True)
    assert results[1]["raised"][0] == "own" and "injected" in results[1]["raised"][1]
    assert results[0]["raised"][0] == "peer" and "another rank failed" in results[0]["raised"][1]


def _leaver(rank, world, port, q):
    """Rank 1 leaves between steps; rank 0 learns it from the store before its next collective."""
    import datetime

    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    store = dist.distributed_c10d._get_default_store()
    t = torch.ones(4)
    dist.all_reduce(t)                      # step 0: everybody is there
    if rank == 1:
        store.set("left/1", "1")            # announce, then leave with nothing in flight
        q.put((rank, "left"))
        dist.destroy_process_group()
        return
    store.wait(["left/1"], datetime.timedelta(seconds=20))
    gone = store.get("left/1") == b"1"
    q.put((rank, "peer gone: skip collective" if gone else "peer alive"))
    dist.destroy_process_group()


def test_rank_leaving_between_steps_is_seen_on_the_host():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaver, args=(r, world, port, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for pr in procs:
        pr.join(timeout=60)
    assert results[1] == "left"
    assert results[0] == "peer gone: skip collective"


def _rank_local_worker(rank, world, port, path, q):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    from gefen_x_b200 import Gefen

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mesh = init_device_mesh("cpu", (world,))

        def full(seed, shape):
            return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * 0.1

        def make():
            ps = [("w", distribute_tensor(full(0, (16, 24)), mesh, [Shard(0)]).requires_grad_(True)),
                  ("b", distribute_tensor(full(1, (16,)), mesh, [Shard(0)]).requires_grad_(True))]
            return ps, Gefen(ps, lr=1e-2, fused=False, factored_v_2d=False)

        def step(ps, opt, k):
            for i, (n, p) in enumerate(ps):
                p.grad = distribute_tensor(full(100 + 10 * k + i, tuple(p.shape)), mesh, [Shard(0)])
            opt.step()

        ps, opt = make()
        for k in range(3):
            step(ps, opt, k)
        sd = opt.state_dict()                                  # collective: carries every rank's payload
        rl = sd["param_groups"][0]["_gefen_checkpoint_metadata"]["rank_local_sharded_state"]
        carrier = sd["state"][sd["param_groups"][0]["params"][0]]
        n_payloads = sum(1 for k in carrier if str(k).startswith("_gefen_rank_local_payload_"))
        weights = {n: p.full_tensor().detach().clone() for n, p in ps}
        if rank == 0:
            torch.save({"sd": sd, "weights": weights}, path)
        dist.barrier()
        blob = torch.load(path, weights_only=False)            # both ranks read the file rank 0 wrote
        ps2, opt2 = make()
        for n, p in ps2:
            p.data.copy_(distribute_tensor(blob["weights"][n], mesh, [Shard(0)]))
        opt2.load_state_dict(blob["sd"])
        same_idx = all(torch.equal(opt.state[a]["m_codebook"], opt2.state[b]["m_codebook"])
                       for (_, a), (_, b) in zip(ps, ps2))
        step(ps, opt, 3)
        step(ps2, opt2, 3)
        same_w = all(torch.equal(a.to_local(), b.to_local()) for (_, a), (_, b) in zip(ps, ps2))
        # a single-process optimizer refuses the rank-local file
        refused = False
        try:
            Gefen([("w", full(0, (16, 24)).requires_grad_(True))], lr=1e-2, fused=False).load_state_dict(blob["sd"])
        except ValueError as e:
            refused = "same" in str(e)
        q.put((rank, dict(fmt=rl["format"], world=rl["world_size"], n_payloads=n_payloads,
                          same_idx=same_idx, same_w=same_w, refused=refused)))
    except Exception:  # pragma: no cover - reported to the parent
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))
    finally:
        dist.destroy_process_group()


def test_rank_local_checkpoint_of_sharded_parameters_round_trips():
    import tempfile

    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        procs = [ctx.Process(target=_rank_local_worker, args=(r, world, port, os.path.join(d, "opt.pt"), q))
                 for r in range(world)]
        for pr in procs:
            pr.start()
        results = dict(q.get(timeout=300) for _ in range(world))
        for pr in procs:
            pr.join(timeout=60)
    for r in range(world):
        assert "error" not in results[r], results[r].get("error")
        o = results[r]
        assert o["fmt"] == "rank_local_dtensor_v2" and o["world"] == 2 and o["n_payloads"] == 2
        assert o["same_idx"] and o["same_w"] and o["refused"]
