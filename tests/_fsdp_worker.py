"""Worker for the multi-GPU trainer tests (launched with torch.distributed.run).

Trains a small decoder on WORLD_SIZE GPUs through ``ShardedTrainer`` and writes the
per-step losses of every rank (gathered on rank 0) to the JSON file given as argv[1].
argv[2]: rs_mode ("stash" | "fused"), argv[3]: clip ("1.0" or "none"), argv[4]: "ag" turns the
all-gather-fused QKV projection on, "hybrid" trains with the sharded Muon hybrid, "kgather"
gathers the parameters and reduces the gradients with the peer-load kernels instead of the copy engines.
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


def main():
    out_path, rs_mode, clip = sys.argv[1], sys.argv[2], sys.argv[3]
    ag = len(sys.argv) > 4 and sys.argv[4] == "ag"
    hybrid = len(sys.argv) > 4 and sys.argv[4] == "hybrid"
    kgather = len(sys.argv) > 4 and sys.argv[4] == "kgather"
    nvls = len(sys.argv) > 4 and sys.argv[4] == "nvls"
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = get_config("tiny-llama", qk_norm=True, hidden=256, ffn=512, n_layers=3)
    try:
        tr = _build(cfg, dev, world, rank, clip, rs_mode, ag, hybrid, kgather, nvls)
    except RuntimeError as exc:
        if nvls and "multicast" in str(exc):
            dist.barrier()
            dist.destroy_process_group()
            sys.exit(77)                        # no NVLS on this system: the test skips
        raise
    g = torch.Generator().manual_seed(2)
    tok_all = torch.randint(0, cfg.vocab_size, (world * 2, 129), generator=g)
    tok = tok_all[rank * 2:(rank + 1) * 2].to(dev)
    losses = []
    for _ in range(12):
        losses.append(float(tr.step(tok[:, :-1], tok[:, 1:]).item()))
    tr.check_status()
    t = torch.tensor(losses, device=dev, dtype=torch.float64)
    gathered = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(gathered, t)
    if rank == 0:
        mean = torch.stack(gathered).mean(0).tolist()
        with open(out_path, "w") as fh:
            json.dump({"mean_loss": mean, "state_bytes_per_param": tr.state_bytes_per_param(),
                       "nvls": tr.nvls}, fh)
    dist.barrier()
    dist.destroy_process_group()


def _build(cfg, dev, world, rank, clip, rs_mode, ag, hybrid, kgather, nvls):
    return ShardedTrainer(cfg, device=dev, dtype=torch.bfloat16, world=world, rank=rank, lr=6e-4,
                        weight_decay=0.01, clip_grad_norm=None if clip == "none" else float(clip),
                        rs_mode=rs_mode, seed=5, wait_iters=20_000_000, ag_gemm=ag, nvls=True if nvls else False,
                        optimizer="muon_hybrid" if hybrid else "gefen",
                        gather_mode="kernel" if kgather else "ce", reduce_ctas=8 if kgather else 148,
                        reduce_mode="kernel" if kgather else "ce")


if __name__ == "__main__":
    main()
