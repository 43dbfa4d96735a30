"""CPU tests of the sharded runtime's host-side layout arithmetic (no GPU, no process group)."""
import torch

from gefen_x_b200.models.decoder import get_config, layer_param_specs
from gefen_x_b200.parallel.fsdp import Group, embed_group_shapes


def test_row_shards_partition_every_parameter():
    cfg = get_config("tiny-llama", qk_norm=True)
    shapes = [("l." + n, s) for n, (_, s) in layer_param_specs(cfg).items()]
    for world in (1, 2, 3, 8):
        g = Group("layer", shapes, world)
        full = torch.arange(g.full_numel, dtype=torch.float64)
        rebuilt = torch.full_like(full, -1)
        for r in range(world):
            shard = torch.empty(g.shard_numel[r], dtype=torch.float64)
            for sp in g.specs:
                src, n = g.local_slice(sp, r)
                shard[sp.shard_off[r]:sp.shard_off[r] + n] = full[src:src + n]
            # what the gather kernel does: copy each rank's segments back to their place
            for sp in g.specs:
                dst, n = g.local_slice(sp, r)
                rebuilt[dst:dst + n] = shard[sp.shard_off[r]:sp.shard_off[r] + n]
        assert torch.equal(rebuilt, full)
        assert sum(g.shard_numel) == g.full_numel
        for sp in g.specs:
            assert sum(sp.shard_rows) == sp.rows


def test_embed_group_follows_tying():
    tied = embed_group_shapes(get_config("qwen3-4b"))
    untied = embed_group_shapes(get_config("llama3-8b"))
    assert [n for n, _ in tied] == ["model.embed_tokens.weight", "model.norm.weight"]
    assert [n for n, _ in untied][-1] == "lm_head.weight"


def test_arena_guard_lines_catch_a_write_past_a_buffer():
    import torch

    from gefen_x_b200.parallel.symm import SymmetricArena

    arena = SymmetricArena(1 << 14, torch.device("cpu"))
    a, off_a = arena.alloc(100, torch.float32)
    b, off_b = arena.alloc(33, torch.bfloat16)
    a.fill_(1.0)
    b.fill_(2.0)
    assert arena.check_guards() == []                     # writing inside the buffers is fine
    arena.buf[off_b + 33 * 2 + 14] = 0                    # lands in the guard line behind `b`
    bad = arena.check_guards()
    assert len(bad) == 1 and off_b + 66 <= bad[0] <= off_b + 66 + 16


def test_row_only_matrix_view_keeps_rows_inside_blocks():
    """A long-block 1-D tensor is viewed as a matrix whose row length divides the period."""
    from gefen_x_b200.ops.update import _pick_tcols, _row_only_cols, two_phase_block

    for period in (8388608, 3670016, 524288, 49152, 6144, 4096, 2048, 1000, 24):
        c = _row_only_cols(period)
        assert period % c == 0
        if period > 4096 and period % 8 == 0:
            assert 256 <= c <= 4096 and c % 8 == 0
        else:
            assert c == period
    # short blocks: several whole blocks per row, rows that start on 16-element boundaries
    for period, numel in ((8, 4096), (64, 4096), (24, 4800), (512, 8192)):
        c = _row_only_cols(period, numel)
        assert c % period == 0 and numel % c == 0 and c <= 2048 and c % 16 == 0 and c > period
    assert _row_only_cols(8, 40) == 8 and _row_only_cols(1000, 3000) == 1000
    assert _pick_tcols(512) == 256 and _pick_tcols(48) in (32, 64)
    assert two_phase_block(1 << 20, 4) and not two_phase_block(64, 4) and not two_phase_block(1 << 20, 4096)


def test_trainer_steps_on_cpu_through_the_same_api():
    """The trainer's step (manual layer backward, clip norm, Gefen update) on CPU tensors: the loss of
    a repeated batch falls, the state stays near one byte per parameter, the device-only trace refuses."""
    import pytest
    import torch

    from gefen_x_b200.models.decoder import get_config
    from gefen_x_b200.parallel.fsdp import ShardedTrainer

    cfg = get_config("tiny-llama")
    tr = ShardedTrainer(cfg, device=torch.device("cpu"), dtype=torch.float32, lr=6e-4, weight_decay=0.01,
                        clip_grad_norm=1.0, seed=3)
    tok = torch.randint(0, cfg.vocab_size, (4, 129), generator=torch.Generator().manual_seed(0))
    losses = [float(tr.step(tok[:, :-1], tok[:, 1:])) for _ in range(5)]
    assert losses[-1] < losses[0] - 1.0, losses
    assert tr.state_bytes_per_param() < 1.1
    tr.check_status()
    with pytest.raises(RuntimeError, match="CUDA"):
        tr.traced_step(tok[:, :-1], tok[:, 1:])


def test_context_parallel_hook_is_declared_and_refuses():
    """Sequence parallelism is a declared, unimplemented hook (the reference has none either)."""
    import pytest
    import torch

    from gefen_x_b200.models.decoder import get_config
    from gefen_x_b200.parallel.fsdp import ShardedTrainer

    cfg = get_config("tiny-llama", n_layers=1)
    with pytest.raises(NotImplementedError, match="context_parallel"):
        ShardedTrainer(cfg, device=torch.device("cpu"), dtype=torch.float32, world=1, rank=0, context_parallel=2)

