"""Worker: the optimizers under torch's own FSDP2 (``fully_shard``) on WORLD_SIZE GPUs.

argv[1]: output JSON, argv[2]: "gefen" | "hybrid".  A small bf16 MLP stack (one layer with an odd
number of rows, so the row shards are uneven) is wrapped layer by layer with ``fully_shard``; its
DTensor parameters are stepped by ``Gefen`` / ``GefenMuonHybrid``.  Mid-run the optimizer state is
saved (``rank_local_dtensor_v2`` for plain Gefen: a collective ``state_dict()``) into a fresh optimizer,
which must continue on the same trajectory.  Reference call sites: ``src/gefen/tools/find_lr.py:467-474``,
tests ``tests/test_gefen_fsdp2_checkpoint.py``, ``tests/test_fused_fsdp2_noncontig.py``.
"""
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

DIMS = [(256, 512), (512, 37 * 8), (37 * 8, 256), (256, 64)]
GLOBAL_BATCH = 16


def build(dev):
    torch.manual_seed(0)
    layers = []
    for i, (a, b) in enumerate(DIMS):
        layers.append(nn.Linear(a, b, bias=(i == 1)))
        if i + 1 < len(DIMS):
            layers.append(nn.GELU())
    model = nn.Sequential(*layers).to(device=dev, dtype=torch.bfloat16)
    return model


def batch(step, world, rank, dev):
    # the same global batch of 16 rows whatever the world size: a rank takes its slice of it
    g = torch.Generator().manual_seed(900 + step)
    x = torch.randn(GLOBAL_BATCH, 256, generator=g)
    y = torch.randn(GLOBAL_BATCH, 64, generator=g)
    if world > 1:
        per = GLOBAL_BATCH // world
        x, y = x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per]
    return x.to(dev).bfloat16(), y.to(dev).bfloat16()


def make_opt(kind, model):
    from gefen_x_b200 import Gefen, GefenMuonHybrid

    if kind == "hybrid":
        return GefenMuonHybrid(model, lr=2e-3, weight_decay=0.01)
    # block second moment in both runs: sharded (DTensor) matrices always take it, as in the reference
    return Gefen(list(model.named_parameters()), lr=2e-3, weight_decay=0.01, factored_v_2d=False)


def run_step(model, opt, step, world, rank, dev):
    x, y = batch(step, world, rank, dev)
    out = model(x)
    loss = (out.float() - y.float()).square().mean()
    loss.backward()
    opt.step()
    opt.zero_grad(set_to_none=True)
    return float(loss.item())


def main():
    out_path, kind = sys.argv[1], sys.argv[2]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    model = build(dev)
    if world > 1:
        from torch.distributed.fsdp import fully_shard

        for layer in model:
            if isinstance(layer, nn.Linear):
                fully_shard(layer)
        fully_shard(model)
    opt = make_opt(kind, model)
    losses = [run_step(model, opt, s, world, rank, dev) for s in range(6)]
    uneven = [tuple(p.to_local().shape) if hasattr(p, "to_local") else tuple(p.shape)
              for n, p in model.named_parameters() if tuple(p.shape) == (296, 512)]
    # checkpoint round trip into a fresh optimizer on the same (sharded) parameters
    sd = opt.state_dict()
    opt2 = make_opt(kind, model)
    opt2.load_state_dict(sd)
    weights = [p.detach().clone() for p in model.parameters()]
    cont = [run_step(model, opt, s, world, rank, dev) for s in range(6, 8)]
    with torch.no_grad():
        for p, w in zip(model.parameters(), weights):
            p.copy_(w)
    resumed = [run_step(model, opt2, s, world, rank, dev) for s in range(6, 8)]
    t = torch.tensor(losses + cont + resumed, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t)
        t /= world
    if rank == 0:
        n = len(losses)
        vals = t.tolist()
        with open(out_path, "w") as fh:
            json.dump({"losses": vals[:n], "continued": vals[n:n + 2], "resumed": vals[n + 2:],
                       "local_shape_of_uneven": uneven, "world": world,
                       "state_keys": sorted(str(k) for k in sd.keys())}, fh)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
