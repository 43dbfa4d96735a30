"""The exact-resume gate of ``benchmarks/trainer_resume.py`` on CPU: a run stopped at a step, written to
disk and continued in fresh objects ends with the same model, optimizer and scheduler state, bit for
bit, as a run that never stopped (reference ``tests/test_transformers_trainer_resume.py`` over
``benchmarks/trainer_resume/run.py``; its Hugging Face ``Trainer`` needs ``accelerate``, which this
environment lacks, so the loop here is plain torch with the same state-dict contract)."""
import argparse
import copy
import importlib.util
import os

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_spec = importlib.util.spec_from_file_location("trainer_resume", os.path.join(ROOT, "benchmarks", "trainer_resume.py"))
harness = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(harness)


def test_state_digest_is_structural_and_tensor_exact():
    left = {"b": [torch.tensor([1.0, 2.0]), 3], "a": (True, None)}
    reordered = {"a": (True, None), "b": [torch.tensor([1.0, 2.0]), 3]}
    changed = copy.deepcopy(left)
    changed["b"][0][1] = 2.0001
    assert harness.state_digest(left) == harness.state_digest(reordered)
    assert harness.state_digest(left) != harness.state_digest(changed)
    # dtype and shape are part of the digest, not only the bytes
    assert harness.state_digest(torch.zeros(4)) != harness.state_digest(torch.zeros(2, 2))
    assert harness.state_digest(torch.zeros(2, dtype=torch.int32)) != harness.state_digest(torch.zeros(2))


def test_recipe_parser_rejects_unknown_and_duplicate_cells():
    assert harness._recipe_list("gefen,gefen_muon_hybrid") == ("gefen", "gefen_muon_hybrid")
    with pytest.raises(argparse.ArgumentTypeError, match="unknown recipes"):
        harness._recipe_list("gefen,adamw")
    with pytest.raises(argparse.ArgumentTypeError, match="duplicates"):
        harness._recipe_list("gefen,gefen")


def test_fixed_token_dataset_is_reproducible():
    first = harness.FixedTokenDataset(samples=4, seq_len=8, vocab_size=32, seed=9)
    second = harness.FixedTokenDataset(samples=4, seq_len=8, vocab_size=32, seed=9)
    assert torch.equal(first.input_ids, second.input_ids)
    row = first[0]
    assert torch.equal(row["input_ids"], row["labels"])
    assert torch.equal(row["attention_mask"], torch.ones(8, dtype=torch.long))


def test_all_recipes_resume_exactly_on_cpu(tmp_path):
    args = harness.parse_args(["--output-dir", str(tmp_path), "--device", "cpu", "--dtype", "float32", "--no-fused",
                               "--steps", "3", "--split-step", "1", "--warmup-steps", "1", "--batch-size", "1",
                               "--gradient-accumulation-steps", "2", "--seq-len", "16", "--ns-steps", "1"])
    summary = harness.run(args)
    assert summary["passed"] is True
    assert set(summary["recipes"]) == set(harness.RECIPES)
    for result in summary["recipes"].values():
        for key in ("model_sha256", "optimizer_sha256", "scheduler_sha256"):
            assert result["baseline"][key] == result["resumed"][key]
        assert result["baseline"]["losses"] == result["resumed"]["losses"]


def test_split_step_must_lie_inside_the_run(tmp_path):
    args = harness.parse_args(["--output-dir", str(tmp_path), "--steps", "3", "--split-step", "3"])
    with pytest.raises(ValueError, match="split-step"):
        harness.run(args)
