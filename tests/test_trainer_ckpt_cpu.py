"""Checkpoints of the sharded runtime, single process on CPU: bit-exact native resume and a
``torch.distributed.checkpoint`` round trip through the stand-in protocol (weights in place,
optimizer state dense, factored second moment as row / column vectors).

Model: the reference's resume contracts (``tests/test_cpu_step_checkpoint.py:109-144`` bit-exact native
resume; ``tests/test_dcp_resharding.py:174-246`` DCP round trip); the multi-rank reshard of the
runtime itself runs on GPUs (``tests/test_fsdp_multi_gpu.py``).
"""
import copy

import pytest
import torch

from gefen_x_b200.models.decoder import get_config
from gefen_x_b200.parallel.fsdp import ShardedTrainer


def _trainer(seed=3):
    cfg = get_config("tiny-llama", n_layers=2, vocab_size=256, hidden=64, n_heads=4, n_kv_heads=2, ffn=176)
    return ShardedTrainer(cfg, device="cpu", dtype=torch.float32, lr=3e-3, weight_decay=0.01,
                          clip_grad_norm=1.0, seed=seed)


def _batch(i):
    g = torch.Generator().manual_seed(50 + i)
    t = torch.randint(0, 256, (2, 33), generator=g)
    return t[:, :-1], t[:, 1:]


def test_native_state_dict_resumes_bit_for_bit():
    a = _trainer()
    for i in range(3):
        a.step(*_batch(i))
    saved = copy.deepcopy(a.state_dict())
    tail_a = [a.step(*_batch(i)).item() for i in range(3, 6)]

    b = _trainer(seed=11)                      # different weights: everything must come from the checkpoint
    b.step(*_batch(9))                         # and an optimizer that already has (other) state
    b.load_state_dict(saved)
    assert b.step_count == 3
    tail_b = [b.step(*_batch(i)).item() for i in range(3, 6)]
    assert tail_a == tail_b
    for ga, gb in zip(a.all_groups, b.all_groups):
        assert torch.equal(ga.shard_w, gb.shard_w)

    other = ShardedTrainer(get_config("tiny-llama", n_layers=1, vocab_size=256, hidden=64, n_heads=4,
                                      n_kv_heads=2, ffn=176), device="cpu", dtype=torch.float32)
    with pytest.raises(ValueError, match="n_layers"):
        other.load_state_dict(saved)


def test_resharding_checkpoint_round_trip(tmp_path):
    from gefen_x_b200.ckpt.lazy import LazyShard

    a = _trainer()
    for i in range(4):
        a.step(*_batch(i))
    path = str(tmp_path / "ckpt")
    LazyShard.accounting.reset()
    a.save_checkpoint(path)
    own = a.num_params()
    # dense optimizer state exists one slot at a time while it is written, never all at once
    largest = max(v.numel() for _n, v in a.named_shards)
    assert LazyShard.accounting.peak <= 3 * 4 * largest
    assert LazyShard.accounting.peak < 8 * own / 2

    b = _trainer(seed=11)
    b.load_checkpoint(path)
    assert b.step_count == 4 and b.opt._gefen_global_step == a.opt._gefen_global_step
    for (na, va), (nb, vb) in zip(a.named_shards, b.named_shards):
        assert na == nb and torch.equal(va, vb), na
    cb_a, cb_b = a.opt._gefen_codebook, b.opt._gefen_codebook
    for (_n, pa), (_m, pb) in zip(a.named_shards, b.named_shards):
        sa, sb = a.opt.state[pa], b.opt.state[pb]
        ma = cb_a[sa["m_codebook"].long()] * sa["m_magnitude"]
        mb = cb_b[sb["m_codebook"].long()] * sb["m_magnitude"]
        assert (ma.reshape(-1) - mb.reshape(-1)).abs().max() <= 2e-2 * ma.abs().max() + 1e-12
        if "v_row" in sa:
            assert torch.allclose(sa["v_row"], sb["v_row"]) and torch.allclose(sa["v_col"], sb["v_col"])
            assert int(sa["factored_step"]) == int(sb["factored_step"])
        else:
            assert torch.allclose(sa["vmean"].mean(), sb["vmean"].mean(), rtol=0.05, atol=1e-12)
        assert int(sa["step"]) == int(sb["step"])
    la = [a.step(*_batch(i)).item() for i in range(4, 7)]
    lb = [b.step(*_batch(i)).item() for i in range(4, 7)]
    for x, y in zip(la, lb):
        assert abs(x - y) <= 2e-3 * abs(x), (la, lb)
