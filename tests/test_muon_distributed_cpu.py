"""GefenMuon ``sharded_mode="distributed"`` among Gloo ranks (CPU DTensor meshes standing in for
FSDP2): owners orthogonalise, everyone applies its rows; the consolidated checkpoint written on 2
ranks continues on 2 ranks and in a single process.

Model: reference ``tests/test_muon_fsdp2_parity.py:60-70`` (single-process oracle on the same seeded
full tensors) and the distributed-manifest checks of ``tests/test_gefen_muon.py``.
"""
import os
import socket
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

SHAPES = [("a.weight", (16, 24)), ("b.weight", (8, 16)), ("c.weight", (24, 8)),
          ("d.weight", (5, 8)),      # uneven row shards (3 + 2)
          ("e.weight", (1, 8))]      # rank 1 holds an empty shard


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _full(seed):
    g = torch.Generator().manual_seed(seed)
    return {n: torch.randn(s, generator=g) * 0.1 for n, s in SHAPES}


def _oracle(steps, load=None, start=0):
    from gefen_x_b200 import GefenMuon

    params = [(n, t.clone().requires_grad_(True)) for n, t in _full(0).items()]
    opt = GefenMuon(params, lr=2e-2, fused=False, sharded_mode="exact")
    if load is not None:
        sd, weights = load
        for (n, p) in params:
            p.data.copy_(weights[n])
        opt.load_state_dict(sd)
    for step in range(start, start + steps):
        for (n, p) in params:
            p.grad = _full(100 + step)[n]
        opt.step()
    return {n: p.detach().clone() for n, p in params}, opt


def _worker(rank, world, port, path, q):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    from gefen_x_b200 import GefenMuon

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mesh = init_device_mesh("cpu", (world,))

        def make():
            ps = [(n, distribute_tensor(t.clone(), mesh, [Shard(0)]).requires_grad_(True))
                  for n, t in _full(0).items()]
            return ps, GefenMuon(ps, lr=2e-2, fused=False, sharded_mode="distributed")

        def step(ps, opt, k):
            for n, p in ps:
                p.grad = distribute_tensor(_full(100 + k)[n], mesh, [Shard(0)])
            opt.step()

        ps, opt = make()
        for k in range(3):
            step(ps, opt, k)
        after3 = {n: p.full_tensor().detach().clone() for n, p in ps}
        owned = sorted(n for n, p in ps if "step" in opt.state.get(p, {}))
        sd = opt.state_dict()                       # collective: consolidated on every rank
        man = sd["gefen_muon_distributed"]
        if rank == 0:
            torch.save({"sd": sd, "weights": after3}, path)
        dist.barrier()
        # continue on 2 ranks from the file
        blob = torch.load(path, weights_only=False)
        ps2, opt2 = make()
        for n, p in ps2:
            p.data.copy_(distribute_tensor(blob["weights"][n], mesh, [Shard(0)]))
        opt2.load_state_dict(blob["sd"])
        owned2 = sorted(n for n, p in ps2 if "step" in opt2.state.get(p, {}))
        step(ps2, opt2, 3)
        step(ps, opt, 3)
        cont = {n: p.full_tensor().detach().clone() for n, p in ps}
        cont2 = {n: p.full_tensor().detach().clone() for n, p in ps2}
        q.put((rank, dict(after3={n: t.numpy() for n, t in after3.items()},
                          cont={n: t.numpy() for n, t in cont.items()},
                          cont2={n: t.numpy() for n, t in cont2.items()}, owned=owned, owned2=owned2,
                          consolidated=man["consolidated"], n_state=len(sd["state"]),
                          owners=[e["owner"] for e in man["groups"][0]["params"]])))
    except Exception:  # pragma: no cover - reported to the parent
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))
    finally:
        dist.destroy_process_group()


def test_distributed_muon_matches_exact_and_checkpoint_is_consolidated():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "muon.pt")
        procs = [ctx.Process(target=_worker, args=(r, world, port, path, q)) for r in range(world)]
        for pr in procs:
            pr.start()
        results = dict(q.get(timeout=300) for _ in range(world))
        for pr in procs:
            pr.join(timeout=60)
        for r in range(world):
            assert "error" not in results[r], results[r].get("error")
        blob = torch.load(path, weights_only=False)
    ref3, _ = _oracle(3)
    ref4, _ = _oracle(4)
    r0, r1 = results[0], results[1]
    # ownership: stable index mod world; state only on the owner; both ranks hold the whole checkpoint
    assert r0["owned"] == ["a.weight", "c.weight", "e.weight"] and r1["owned"] == ["b.weight", "d.weight"]
    assert r0["owned2"] == r0["owned"] and r1["owned2"] == r1["owned"]
    assert r0["consolidated"] and r1["consolidated"] and r0["n_state"] == 5 and r1["n_state"] == 5
    assert r0["owners"] == [0, 1, 0, 1, 0]
    for n, _ in SHAPES:
        assert torch.allclose(torch.from_numpy(r0["after3"][n]), ref3[n], atol=2e-5), n
        assert torch.allclose(torch.from_numpy(r0["cont"][n]), ref4[n], atol=2e-5), n
        assert torch.allclose(torch.from_numpy(r0["cont2"][n]), torch.from_numpy(r0["cont"][n]), atol=1e-6), n
    # the same file continues in a single process (exact mode)
    single, _ = _oracle(1, load=(blob["sd"], blob["weights"]), start=3)
    for n, _ in SHAPES:
        assert torch.allclose(single[n], ref4[n], atol=2e-5), n
    # a manifest that contradicts the live optimizer is refused before anything is loaded
    import copy

    from gefen_x_b200 import GefenMuon

    def fresh():
        ps = [(n, t.clone().requires_grad_(True)) for n, t in _full(0).items()]
        return ps, GefenMuon(ps, lr=2e-2, fused=False)

    def tampered(edit):
        sd = copy.deepcopy(blob["sd"])
        edit(sd["gefen_muon_distributed"], sd)
        return sd

    cases = {
        "version": lambda m, sd: m.__setitem__("version", 7),
        "ownership": lambda m, sd: m.__setitem__("ownership", "round_robin"),
        "list": lambda m, sd: m.__setitem__("groups", "nope"),
        "lists": lambda m, sd: m["groups"][0]["params"].pop(),
        "is 'zzz'": lambda m, sd: m["groups"][0]["params"][1].__setitem__("name", "zzz"),
        "shape": lambda m, sd: m["groups"][0]["params"][0].__setitem__("shape", (3, 3)),
        "owner": lambda m, sd: m["groups"][0]["params"][2].__setitem__("owner", 1),
        "momentum is missing": lambda m, sd: sd["state"][0].pop("m_codebook"),
        "state keys": lambda m, sd: m["groups"][0]["params"][0].__setitem__(
            "state_keys", tuple(m["groups"][0]["params"][0]["state_keys"]) + ("ghost",)),
    }
    for needle, edit in cases.items():
        ps, opt = fresh()
        before = {n: p.detach().clone() for n, p in ps}
        with pytest.raises(ValueError, match="refused the distributed checkpoint"):
            opt.load_state_dict(tampered(edit))
        assert all("m_codebook" not in st for st in opt.state.values()), needle
        assert all(torch.equal(p, before[n]) for n, p in ps)
    ps, opt = fresh()
    opt.load_state_dict(copy.deepcopy(blob["sd"]))           # the untouched file still loads



def _presence_worker(rank, world, port, case, q):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import Shard, distribute_tensor

    from gefen_x_b200 import GefenMuon

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mesh = init_device_mesh("cpu", (world,))
        ps = [(n, distribute_tensor(t.clone(), mesh, [Shard(0)]).requires_grad_(True)) for n, t in _full(0).items()]
        opt = GefenMuon(ps, lr=2e-2, fused=False, sharded_mode="distributed")
        for n, p in ps:                                   # one good step: state exists everywhere
            p.grad = distribute_tensor(_full(100)[n], mesh, [Shard(0)])
        opt.step()
        before_p = {n: p.to_local().detach().clone() for n, p in ps}
        before_s = {n: {k: (v.detach().clone() if torch.is_tensor(v) else v) for k, v in opt.state.get(p, {}).items()}
                    for n, p in ps}
        for n, p in ps:
            p.grad = distribute_tensor(_full(101)[n], mesh, [Shard(0)])
        if rank == 1:
            if case == "one_missing":
                ps[1][1].grad = None                      # rank 1 alone lacks the gradient of one matrix
            else:
                for _, p in ps:                           # rank 1 has no gradient at all
                    p.grad = None
        err = None
        try:
            opt.step()
        except RuntimeError as exc:
            err = str(exc)
        unchanged = all(torch.equal(p.to_local(), before_p[n]) for n, p in ps)
        for n, p in ps:
            st = opt.state.get(p, {})
            for k, v in before_s[n].items():
                same = torch.equal(st[k], v) if torch.is_tensor(v) else st[k] == v
                unchanged = unchanged and bool(same)
        q.put((rank, {"err": err, "unchanged": unchanged}))
    except Exception:  # pragma: no cover - reported to the parent
        import traceback

        q.put((rank, {"error": traceback.format_exc()}))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["one_missing", "all_missing"])
def test_ranks_that_disagree_on_gradient_presence_refuse_the_step_together(case):
    """One rank lacks a gradient the other has (or has none at all): every rank raises before any
    gather collective, nobody hangs, and neither parameters nor optimizer state have moved
    (reference tests/test_muon_grad_presence.py)."""
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_presence_worker, args=(r, world, port, case, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=240) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    for r in range(world):
        assert "error" not in got[r], got[r].get("error")
        assert got[r]["err"] is not None and "disagree" in got[r]["err"], got[r]
        assert got[r]["unchanged"], r
