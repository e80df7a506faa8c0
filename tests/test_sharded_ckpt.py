"""Sharded torch_dist store: ranks under TP / EP / DP write their rectangles, and the store reloads bit-exactly as full
Megatron-named tensors, into a single-rank actor, and into another parallel layout — optimizer state included."""
import os
import sys

import pytest
import torch

from dist_utils import run_distributed

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE = ("--model-name {preset} --fp32 --rollout-batch-size 4 --n-samples-per-prompt 2 --rollout-max-response-len 8 "
        "--num-rollout 1 --rm-type even_fraction --lr 1e-3 "
        "--data-source-path miles_b200.rollout.data_source.SyntheticSource --synthetic-prompt-len 6 10")


def _actor(preset, extra, ps_kw):
    from miles_b200.args import parse_args
    from miles_b200.parallel.state import ParallelState
    from miles_b200.train.actor import TrainActor

    args = parse_args((BASE.format(preset=preset) + " " + extra).split())
    ps = ParallelState.build(**ps_kw)
    actor = TrainActor(args, ps)
    actor.init()
    return actor, args


def _fake_step(actor, seed):
    """Deterministic, layout-independent optimizer state: master = param, moments = functions of the master weights."""
    for d in actor.optimizer.domains:
        d.exp_avg.copy_(d.master * 0.5 + 0.25)
        d.exp_avg_sq.copy_(d.master * d.master + 1.0)
    actor.optimizer.step_count = 7 + seed


def _full_ours(preset):
    from miles_b200.models.config import PRESETS
    from miles_b200.models.qwen3 import build_model
    from miles_b200.parallel.state import ParallelState

    m = build_model(PRESETS[preset], ParallelState(), dtype=torch.float32, device="cpu", seed=5)
    return {n: p.detach().clone() for n, p in m.named_parameters()}


def _save_body(rank, world, preset, ps_kw, root, extra=""):
    sys.path.insert(0, ROOT)
    from miles_b200.checkpoint import manager

    actor, args = _actor(preset, f"--save {root} --seed 5 {extra}", ps_kw)
    _fake_step(actor, 0)
    manager.save_from_actor(actor, args, 3)
    if extra:
        # the writer thread works from host copies: training may overwrite parameters and state straight away
        for p in actor.model.parameters():
            p.data.zero_()
        for d in actor.optimizer.domains:
            d.exp_avg.zero_()
        manager.finalize_async_save()
        assert os.path.exists(os.path.join(root, "iter_0000003", ".complete"))


def _load_body(rank, world, preset, ps_kw, root, out):
    sys.path.insert(0, ROOT)
    from miles_b200.checkpoint import manager

    actor, args = _actor(preset, f"--load {root} --seed 11", ps_kw)      # another seed: every value must come from the store
    assert actor.start_rollout_id == 4 and actor.optimizer.step_count == 7
    for d in actor.optimizer.domains:
        lo, hi = d.shard
        mask = torch.zeros(d.numel, dtype=torch.bool)
        for p, o in zip(d.params, d.offsets):
            mask[o:o + p.numel()] = True
        mask = mask[lo:hi]
        want = d.param_buf[lo:hi].float()
        assert torch.equal(d.master[mask], want[mask])
        assert torch.equal(d.exp_avg[mask], (want * 0.5 + 0.25)[mask])
        assert torch.equal(d.exp_avg_sq[mask], (want * want + 1.0)[mask])
    torch.save({n: p.detach().clone() for n, p in actor.named_weights()}, os.path.join(out, f"w{rank}.pt"))


@pytest.mark.parametrize("preset,src,dst", [("tiny", dict(tp=2), dict(tp=1)), ("tiny-moe", dict(ep=2), dict(tp=2, ep=2)),
                                            ("tiny", dict(tp=1), dict(tp=2))])
def test_store_round_trips_across_layouts(tmp_path, preset, src, dst):
    from miles_b200.checkpoint import torch_dist
    from miles_b200.models.config import PRESETS
    from miles_b200.models.convert import megatron_to_ours, shard_for_rank
    from miles_b200.parallel.state import ParallelState

    root, out = str(tmp_path / "ckpt"), str(tmp_path / "out")
    os.makedirs(out)
    run_distributed(_save_body, 2, (preset, src, root))
    d = os.path.join(root, "iter_0000003")
    assert os.path.exists(os.path.join(d, ".metadata")) and os.path.exists(os.path.join(d, "common.pt"))
    assert open(os.path.join(root, "latest_checkpointed_iteration.txt")).read().strip() == "3"
    # (a) read back as full Megatron-named tensors without a process group: equals the full model built from the same seed
    cfg = PRESETS[preset]
    full = megatron_to_ours(torch_dist.load_state(d), cfg)
    want = _full_ours(preset)
    assert set(full) == set(want)
    for n in want:
        assert torch.equal(full[n], want[n]), n
    # the optimizer state sits in model space under Megatron's entry names
    opt = torch_dist.load_state(d, prefix_filter=("rng", "_extra_state"))
    k = "optimizer.state.exp_avg.decoder.layers.0.self_attention.linear_proj.weight"
    assert torch.equal(opt[k], want["layers.0.attn.wo"] * 0.5 + 0.25)
    # (b) reload under another layout
    run_distributed(_load_body, 2, (preset, dst, root, out))
    for r in range(2):
        got = torch.load(os.path.join(out, f"w{r}.pt"))
        ps = ParallelState.build(**dst, rank=r, world_size=2, create_groups=False)
        for n, t in got.items():
            assert torch.equal(t, shard_for_rank(n, want[n], cfg, ps)), (n, r)


def test_async_save_writes_the_staged_state(tmp_path):
    from miles_b200.checkpoint import torch_dist
    from miles_b200.models.config import PRESETS
    from miles_b200.models.convert import megatron_to_ours

    root = str(tmp_path / "ckpt")
    run_distributed(_save_body, 2, ("tiny", dict(tp=2), root, "--async-save"))
    d = os.path.join(root, "iter_0000003")
    full = megatron_to_ours(torch_dist.load_state(d), PRESETS["tiny"])
    want = _full_ours("tiny")
    for n in want:
        assert torch.equal(full[n], want[n]), n
    opt = torch_dist.load_state(d, prefix_filter=("rng", "_extra_state"))
    k = "optimizer.state.exp_avg.decoder.layers.1.mlp.linear_fc2.weight"
    assert torch.equal(opt[k], want["layers.1.mlp.w2"] * 0.5 + 0.25)
    assert open(os.path.join(root, "latest_checkpointed_iteration.txt")).read().strip() == "3"


def test_stacked_layer_entries_are_unstacked(tmp_path):
    """A store that keeps all layers under one entry with a leading layer axis (as Megatron-core may) reads back as
    per-layer names."""
    from miles_b200.checkpoint import torch_dist

    st = {"decoder.layers.self_attention.linear_proj.weight": torch.randn(3, 4, 4),
          "decoder.layers.mlp.experts.experts.linear_fc1.weight": torch.randn(3, 2, 6, 4),
          "embedding.word_embeddings.weight": torch.randn(8, 4)}
    d = torch_dist.save_state(st, str(tmp_path / "s"))
    got = torch_dist.load_state(d)
    assert torch.equal(got["decoder.layers.1.self_attention.linear_proj.weight"], st["decoder.layers.self_attention.linear_proj.weight"][1])
    assert torch.equal(got["decoder.layers.2.mlp.experts.linear_fc1.weight1"],
                       st["decoder.layers.mlp.experts.experts.linear_fc1.weight"][2, 1])
    assert not torch_dist.has_per_layer_names(d)
