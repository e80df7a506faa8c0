"""End-to-end RL steps on CPU: rollout engine → rewards → train → weight sync, single process and gloo ranks.

The analogue of the reference's e2e tier (tests/e2e/short: tiny models, a few rollouts, CI gates on
`train_rollout_logprob_abs_diff` and KL == 0 at step 0) on a 2-layer model in fp32.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from dist_utils import run_distributed  # noqa: E402

BASE = ("--model-name tiny --fp32 --rollout-batch-size 8 --n-samples-per-prompt 4 --rollout-max-response-len 12 "
        "--num-rollout 2 --rm-type even_fraction --lr 1e-4 --colocate --advantage-estimator grpo "
        "--data-source-path miles_b200.rollout.data_source.SyntheticSource --synthetic-prompt-len 6 10")


def _run(extra=""):
    import train as T
    from miles_b200.args import parse_args

    args = parse_args((BASE + " " + extra).split())
    tr = T.train(args)
    return tr.history


def _check_history(h, n_rollouts=2, diff_tol=1e-5):
    assert len(h.rows) == n_rollouts
    diffs = h.series("train/train_rollout_logprob_abs_diff")
    assert diffs and max(diffs) < diff_tol, diffs
    assert abs(h.series("train/ppo_kl")[0]) < 1e-6
    assert all(g > 0 for g in h.series("train/grad_norm"))
    assert h.series("rollout/response_len/mean")[0] > 0


def test_grpo_single_process():
    _check_history(_run())


def test_grpo_kl_loss_and_ref_is_zero_at_step0():
    h = _run("--use-kl-loss --kl-loss-coef 0.01 --ci-test")
    assert abs(h.series("train/kl_loss")[0]) < 1e-6


def test_grpo_moe_with_routing_replay():
    h = _run("--model-name tiny-moe --use-rollout-routing-replay")
    _check_history(h)


def test_audit_log_of_a_run_is_clean(tmp_path):
    from miles_b200.audit import events as A

    _run(f"--audit-dir {tmp_path}")
    ev = A.read_events(str(tmp_path))
    assert sum(e["kind"] == "weights_published" for e in ev) == 3        # initial push + one per rollout
    assert sum(e["kind"] == "weights_received" for e in ev) == 3
    assert A.analyze(str(tmp_path), ["weight_checksums"]) == []


def test_ppo_with_critic():
    h = _run("--advantage-estimator ppo --critic-lr 1e-4 --num-critic-only-steps 1")
    assert len(h.rows) == 2
    assert any(k.startswith("train/critic-") for k in h.rows[0])
    assert "train/pg_loss" not in h.rows[0] and "train/pg_loss" in h.rows[1]     # critic-only warm-up step


def test_lora_training_moves_only_adapters():
    import torch
    import train as T
    from miles_b200.args import parse_args
    from miles_b200.orchestration.wiring import create_parallel_state, create_training_models

    args = parse_args((BASE + " --lora-rank 4 --lr 1e-3").split())
    ps = create_parallel_state(args)
    actor, _, _ = create_training_models(args, ps)
    base = {n: p.detach().clone() for n, p in actor.model.named_parameters() if ".lora." not in n}
    h = _run("--lora-rank 4 --lr 1e-3")
    assert len(h.rows) == 2 and h.series("train/grad_norm")[0] > 0
    del T, torch, base


def test_checkpoint_save_and_resume(tmp_path):
    d = str(tmp_path / "ckpt")
    h1 = _run(f"--save {d} --save-interval 1 --num-rollout 2")
    assert os.path.exists(os.path.join(d, "latest_checkpointed_iteration.txt"))
    h2 = _run(f"--save {d} --load {d} --save-interval 1 --num-rollout 3")
    # resumed at rollout 2: exactly one more step runs
    assert [r["rollout/step"] for r in h2.rows] == [2]
    assert len(h1.rows) == 2


# ---- gloo ranks ------------------------------------------------------------------------------------------------

def _dist_body(rank, world, extra, out_dir):
    import json

    sys.path.insert(0, ROOT)
    import train as T
    from miles_b200.args import parse_args

    args = parse_args((BASE + " " + extra).split())
    tr = T.train(args)
    if rank == 0:
        with open(os.path.join(out_dir, "hist.json"), "w") as f:
            json.dump(tr.history.rows, f)


def _dist_hist(tmp_path, extra, world=2):
    import json

    run_distributed(_dist_body, world, (extra, str(tmp_path)), timeout=600)
    return json.load(open(os.path.join(str(tmp_path), "hist.json")))


@pytest.mark.parametrize("extra", [
    "",                                                                     # dp2
    "--tensor-model-parallel-size 2 --sequence-parallel",                   # tp2 + sp
    "--model-name tiny-moe --expert-model-parallel-size 2",                 # dp2 × ep2
    "--rollout-data-exchange local",                                        # dp2, every rank trains on what it generated
    "--model-name tiny-moe --expert-model-parallel-size 2 --use-rollout-routing-replay --rollout-data-exchange local",
    # as above, then whole prompt groups move to the rank with fewer tokens
    "--model-name tiny-moe --expert-model-parallel-size 2 --use-rollout-routing-replay --rollout-data-exchange balanced "
    "--synthetic-prompt-len 4 48",
    "--context-parallel-size 2 --cp-comm-type a2a",                         # cp2 (Ulysses), dp1
    # linear-attention family under cp2: recurrent state + convolution history passed between the chunk owners
    "--model-name qwen3-next-tiny --context-parallel-size 2 --cp-comm-type a2a",
    # per-channel-decay linear attention + latent attention (the latent is what is gathered) under cp2
    "--model-name kimi-linear-tiny --context-parallel-size 2 --cp-comm-type a2a",
    "--train-backend fsdp",                                                 # dp2, parameters sharded per layer (FSDP2)
    "--offload-train --offload-train-release-process-groups",               # dp2, communicators destroyed while asleep
    "--context-parallel-size 2",                                            # cp2, ring attention over zigzag pieces
    "--context-parallel-size 2 --allgather-cp",                             # cp2, K/V all-gathered
    "--pipeline-model-parallel-size 2 --micro-batch-size 8",                # pp2, 4 micro-batches per step, 1F1B order
    "--pipeline-model-parallel-size 2 --micro-batch-size 8 --pp-schedule gpipe",
    # pp2 × 2 model chunks per rank (4 virtual stages of one layer), interleaved 1F1B
    "--pipeline-model-parallel-size 2 --virtual-pipeline-model-parallel-size 2 --num-layers 4 --micro-batch-size 8",
    # the tiny plumbing config: 16 prompts of length 32 per step, groups of 4, 32 new tokens, lr 1e-5, 3 steps
    "--rollout-batch-size 16 --synthetic-prompt-len 32 32 --rollout-max-response-len 32 --lr 1e-5 --num-rollout 3 --kl-coef 0",
])
def test_grpo_two_ranks(tmp_path, extra):
    rows = _dist_hist(tmp_path, extra)
    assert len(rows) == (3 if "--num-rollout 3" in extra else 2)
    assert max(r["train/train_rollout_logprob_abs_diff"] for r in rows) < 1e-5
    assert abs(rows[0]["train/ppo_kl"]) < 1e-6
    assert all(r["train/grad_norm"] > 0 for r in rows)


def test_grpo_hierarchical_context_parallel_four_ranks(tmp_path):
    """cp = 4 as all-to-all groups of 2 inside a ring of 2 (`--cp-comm-type a2a+p2p`): same invariants as the other layouts."""
    rows = _dist_hist(tmp_path, "--context-parallel-size 4 --cp-comm-type a2a+p2p --hierarchical-context-parallel-sizes 2 2", world=4)
    assert len(rows) == 2
    assert max(r["train/train_rollout_logprob_abs_diff"] for r in rows) < 1e-5
    assert abs(rows[0]["train/ppo_kl"]) < 1e-6 and all(r["train/grad_norm"] > 0 for r in rows)


def test_virtual_pipeline_checkpoint_resumes_and_loads_under_a_plain_pipeline(tmp_path):
    """A store written by pp2 × 2 virtual stages resumes under the same layout and loads under plain pp2: entry names are the
    model's, not the cut's."""
    d = str(tmp_path / "ckpt")
    for sub in "abc":
        (tmp_path / sub).mkdir()
    vpp = "--pipeline-model-parallel-size 2 --virtual-pipeline-model-parallel-size 2 --num-layers 4 --micro-batch-size 8"
    _dist_hist(tmp_path / "a", f"{vpp} --save {d} --save-interval 1 --num-rollout 2")
    rows = _dist_hist(tmp_path / "b", f"{vpp} --save {d} --load {d} --save-interval 1 --num-rollout 3")
    assert [r["rollout/step"] for r in rows] == [2] and rows[0]["train/train_rollout_logprob_abs_diff"] < 1e-5
    rows = _dist_hist(tmp_path / "c", f"--pipeline-model-parallel-size 2 --num-layers 4 --micro-batch-size 8 --load {d} --num-rollout 4")
    assert [r["rollout/step"] for r in rows] == [3] and rows[0]["train/train_rollout_logprob_abs_diff"] < 1e-5


def test_fsdp_checkpoint_save_and_resume(tmp_path):
    d = str(tmp_path / "ckpt")
    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    rows1 = _dist_hist(tmp_path / "a", f"--train-backend fsdp --save {d} --save-interval 1 --num-rollout 2")
    rows2 = _dist_hist(tmp_path / "b", f"--train-backend fsdp --save {d} --load {d} --save-interval 1 --num-rollout 3")
    assert len(rows1) == 2 and [r["rollout/step"] for r in rows2] == [2]            # resumed after two saved rollouts
    assert rows2[0]["train/train_rollout_logprob_abs_diff"] < 1e-5                  # the reloaded shards feed the engine
    it = os.path.join(d, "iter_0000001")                                            # one DCP store per kind of state
    for sub in ("model/.metadata", "optimizer/.metadata", "lr_scheduler/.metadata", "rng.pt", "meta.json"):
        assert os.path.exists(os.path.join(it, sub)), sub
    import torch.distributed.checkpoint as dcp

    keys = dcp.FileSystemReader(os.path.join(it, "optimizer")).read_metadata().state_dict_metadata
    assert "optim_state.optim.state.layers.0.attn.wo.exp_avg" in keys


# ---- asynchronous loops --------------------------------------------------------------------------------------------

ASYNC_BASE = BASE.replace("--colocate ", "")


def _run_async(extra=""):
    import train_async as TA
    from miles_b200.args import parse_args

    return TA.train(parse_args((ASYNC_BASE + " " + extra).split())).history


def test_async_one_step_ahead():
    h = _run_async("--num-rollout 3")
    assert len(h.rows) == 3
    # batch 0 is on-policy; later batches were sampled one optimizer step behind the weights that score them
    diffs = h.series("train/train_rollout_logprob_abs_diff")
    assert diffs[0] < 1e-5 and 1e-5 < max(diffs[1:]) < 0.1
    assert all(g > 0 for g in h.series("train/grad_norm"))


def test_fully_async_staleness_bounded():
    h = _run_async("--num-rollout 4 --fully-async --max-weight-staleness 2 --use-tis")
    assert len(h.rows) == 4
    assert max(h.series("rollout/staleness/max")) <= 2
    assert all(g > 0 for g in h.series("train/grad_norm"))


def test_async_rejects_colocate():
    import train_async as TA
    from miles_b200.args import parse_args

    with pytest.raises(AssertionError):
        TA.train(parse_args(BASE.split()))


def test_staleness_buffer_policies():
    from miles_b200.rollout.fully_async import StalenessBuffer, SubmissionScheduler
    from miles_b200.types import Sample, WeightVersionSpan

    def grp(v):
        return [Sample(tokens=[1, 2], weight_versions=[WeightVersionSpan(v, 1)])]

    b = StalenessBuffer(max_staleness=1, policy="retry")
    for v in (0, 1, 2, 3):
        b.put(grp(v))
    got = b.take(2, current_version=3, timeout=1)
    assert [g[0].oldest_weight_version for g in got] == [2, 3]
    assert b.stats["dropped_stale"] == 2 and len(b.pop_retries()) == 2
    with pytest.raises(TimeoutError):
        b.take(1, current_version=3, timeout=0.05)
    s = SubmissionScheduler(batch=8, max_inflight=12, target_buffered=8)
    assert s.allowance(inflight=0, buffered=0) == 12 and s.allowance(inflight=4, buffered=8) == 4
    assert s.allowance(inflight=12, buffered=0) == 0


# ---- supervised fine-tuning through the same loop ---------------------------------------------------------------------

class ChatSource:
    """A data source of two-turn conversations over the byte tokenizer."""

    def __init__(self, args, tokenizer=None):
        from miles_b200.session.tito import ByteChatTokenizer

        self.tokenizer = ByteChatTokenizer()
        self.i = 0

    def get_samples(self, n):
        from miles_b200.types import Sample

        out = []
        for _ in range(n):
            self.i += 1
            out.append([Sample(prompt=[{"role": "user", "content": f"say {self.i % 3}"}, {"role": "assistant", "content": "ok " * (1 + self.i % 2)}])])
        return out

    def add_samples(self, groups):
        pass

    def save(self, rollout_id):
        pass

    def load(self, rollout_id=None):
        pass

    def __len__(self):
        return 0


def test_sft_loss_goes_down():
    h = _run("--loss-type sft_loss --rollout-function-path miles_b200.rollout.sft_rollout.SftRolloutFn --tito-model qwen3 "
             "--data-source-path test_e2e.ChatSource --n-samples-per-prompt 1 --rollout-batch-size 8 --global-batch-size 8 "
             "--disable-compute-advantages-and-returns --lr 3e-3 --num-rollout 6")
    losses = h.series("train/sft_loss")
    assert len(losses) == 6 and losses[-1] < 0.6 * losses[0], losses
