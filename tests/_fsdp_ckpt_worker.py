"""Worker for the multi-GPU checkpoint / state tests of the sharded runtime (torch.distributed.run).

argv[1]: mode, argv[2]: working directory.
  "save"   train 6 steps on a global batch of 4 sequences, write a resharding checkpoint, check that the
           native rank-local state dict resumes on the same trajectory, and record the next 3 losses
  "load"   fresh trainer (other seed) on WORLD_SIZE ranks, load the checkpoint, run the same 3 steps
  "state"  every rank takes ONE step on the SAME batch (the reduced gradient then equals a single GPU's
           on that batch) and the optimizer state of every matrix is gathered by rows
"""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from gefen_x_b200.models.decoder import get_config  # noqa: E402
from gefen_x_b200.parallel.fsdp import ShardedTrainer  # noqa: E402

GLOBAL_SEQS = int(os.environ.get("GX_GLOBAL_SEQS", "4"))      # sequences of the global batch


def config():
    if os.environ.get("GX_CKPT_MODEL"):                 # e.g. "llama3-8b:2": a preset with this many layers
        name, layers = os.environ["GX_CKPT_MODEL"].split(":")
        return get_config(name, n_layers=int(layers))
    return get_config("tiny-llama", qk_norm=True, hidden=256, ffn=512, n_layers=2)


def batch(step, world, rank, dev, same=False):
    g = torch.Generator().manual_seed(700 + step)
    tok = torch.randint(0, config().vocab_size, (GLOBAL_SEQS, 129), generator=g)
    if same:
        mine = tok[:2]
    else:
        per = GLOBAL_SEQS // world
        mine = tok[rank * per:(rank + 1) * per]
    mine = mine.to(dev)
    return mine[:, :-1], mine[:, 1:]


def mean_over_ranks(values, dev, world):
    t = torch.tensor(values, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t)
    return (t / world).tolist()


def gather_state(tr, dev, world, rank):
    out = {}
    for name, view in tr.named_shards:
        if view.dim() != 2:
            continue
        st = tr.opt.state[view]
        cb = tr.opt._gefen_codebook_on(dev)
        entry = {"period": int(st["automatic_period"]), "rows": int(view.shape[0])}
        dense = (cb[st["m_codebook"].long()] * st["m_magnitude"]).reshape(view.shape).float().cpu()
        parts = {"idx": st["m_codebook"].reshape(view.shape).cpu(), "dense": dense, "v_row": st["v_row"].cpu(),
                 "v_col": st["v_col"].cpu(), "w": view.float().cpu()}
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, (entry["period"], parts))
            entry["periods"] = [g[0] for g in gathered]
            for k in ("idx", "dense", "v_row", "w"):
                entry[k] = torch.cat([g[1][k] for g in gathered], dim=0)
            entry["v_col"] = [g[1]["v_col"] for g in gathered]
        else:
            entry["periods"] = [entry["period"]]
            entry.update({k: parts[k] for k in ("idx", "dense", "v_row", "w")})
            entry["v_col"] = [parts["v_col"]]
        out[name] = entry
    return out


def main():
    mode, work = sys.argv[1], sys.argv[2]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    seed = 5 if mode != "load" else 99
    tr = ShardedTrainer(config(), device=dev, dtype=torch.bfloat16, world=world, rank=rank, lr=6e-4,
                        weight_decay=0.01, clip_grad_norm=1.0, seed=seed, wait_iters=20_000_000)
    ckpt = os.path.join(work, "ckpt")
    result = {}
    if mode == "save":
        for s in range(6):
            tr.step(*batch(s, world, rank, dev))
        tr.save_checkpoint(ckpt)
        native = tr.state_dict()
        cont = [float(tr.step(*batch(s, world, rank, dev)).item()) for s in range(6, 9)]
        tr.load_state_dict(native)
        again = [float(tr.step(*batch(s, world, rank, dev)).item()) for s in range(6, 9)]
        # the kernels accumulate second-moment statistics with atomics, so two GPU runs agree to the last
        # bits only (the CPU test pins the exact resume): report the largest relative difference
        drift = max(abs(a - b) / max(1e-9, abs(a)) for a, b in zip(cont, again))
        result = {"continued": mean_over_ranks(cont, dev, world), "native_resume_drift": drift}
    elif mode == "load":
        tr.step(*batch(50, world, rank, dev))          # the optimizer already holds other state
        tr.load_checkpoint(ckpt)
        resumed = [float(tr.step(*batch(s, world, rank, dev)).item()) for s in range(6, 9)]
        result = {"resumed": mean_over_ranks(resumed, dev, world), "step_count": tr.step_count}
    elif mode == "state":
        tr.step(*batch(0, world, rank, dev, same=True))
        st = gather_state(tr, dev, world, rank)
        st["__codebook__"] = tr.opt._gefen_codebook.float().cpu()
        if rank == 0:
            torch.save(st, os.path.join(work, "state_w{}.pt".format(world)))
    tr.check_status()
    if world > 1:
        drifts = [None] * world
        dist.all_gather_object(drifts, result.get("native_resume_drift", 0.0))
        result["native_resume_drift"] = max(drifts)
    if rank == 0:
        with open(os.path.join(work, "{}_w{}.json".format(mode, world)), "w") as fh:
            json.dump(result, fh)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
