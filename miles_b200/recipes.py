"""Launch recipes: one function per model / setting that turns a few knobs into the full argument list of a training job.

The reference keeps one script per model (`scripts/run_qwen3_4b.py`, `run_qwen3_30b_a3b.py`, `run_qwen3_235b_a22b.py`,
`run_qwen3_30b_a3b_fsdp.py`, `run_qwen3_0_6b_fsdp.py`, `run_qwen3_dense.py`, `run_qwen3_sft.py`, … — scripts/*.py): each
composes checkpoint / rollout / optimiser / GRPO / parallelism / engine arguments for the hardware at hand and submits the
job.  Here a recipe is a function returning a `Recipe` (argument list + entry point + GPU count); `run.py` at the repository
root prints or runs it:

    python run.py list
    python run.py qwen3-30b-a3b --num-gpus 8 --mode debug_minimal --dry-run
    python run.py qwen3-4b --num-gpus 8 --data /data/dapo-math-17k.jsonl --hf-checkpoint /models/Qwen3-4B -- --lr 2e-6

Modes (the reference's `mode` switch): `normal`; `debug_minimal` — a few short rollouts to see the loop turn;
`debug_one_sample` — one prompt, one sample, for stepping through by hand.  Parallel sizes are chosen for ONE NVSwitch box
of B200s (180 GB each): a dense model up to 8B trains data-parallel, 32B with TP = 8 rollout engines, the 30B-A3B MoE with
expert parallelism over all GPUs, the 235B-A22B MoE with EP = 8 and full recompute.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable


@dataclass
class Recipe:
    name: str
    args: list[str]
    entry: str = "train.py"
    num_gpus: int = 8
    env: dict = field(default_factory=dict)
    notes: str = ""


@dataclass
class Knobs:
    num_gpus: int = 8
    mode: str = "normal"                   # normal | debug_minimal | debug_one_sample
    hf_checkpoint: str | None = None
    data: str | None = None                # prompt jsonl / parquet; synthetic prompts when absent
    eval_data: str | None = None
    save: str | None = None
    mxfp8: bool = False
    true_on_policy: bool = False
    dynamic_sampling: bool = False
    use_kl_loss: bool = False
    wandb_project: str | None = None
    extra: list[str] = field(default_factory=list)


def _s(xs) -> list[str]:
    return [str(x) for x in xs]


def _data(k: Knobs, max_response: int) -> list[str]:
    a = []
    if k.data:
        a += ["--prompt-data", k.data, "--input-key", "prompt", "--label-key", "label", "--apply-chat-template", "--rollout-shuffle",
              "--rm-type", "dapo"]
    else:
        a += ["--data-source-path", "miles_b200.rollout.data_source.SyntheticSource", "--synthetic-prompt-len", 256, 1024,
              "--rm-type", "even_fraction"]
    if k.eval_data:
        a += ["--eval-prompt-data", "eval", k.eval_data, "--eval-interval", 20, "--n-samples-per-eval-prompt", 4,
              "--eval-max-response-len", max_response]
    return a


def _rollout(k: Knobs, prompts: int, samples: int, max_response: int, gbs: int | None = None) -> list[str]:
    if k.mode == "debug_one_sample":
        prompts, samples, max_response = 1, 1, min(max_response, 64)
    elif k.mode == "debug_minimal":
        prompts, samples, max_response = min(prompts, 8), min(samples, 4), min(max_response, 256)
    a = ["--rollout-batch-size", prompts, "--n-samples-per-prompt", samples, "--rollout-max-response-len", max_response,
         "--rollout-temperature", 1.0, "--global-batch-size", gbs if gbs and k.mode == "normal" else prompts * samples,
         "--num-rollout", 3000 if k.mode == "normal" else 2]
    if k.dynamic_sampling and k.mode == "normal":
        a += ["--over-sampling-batch-size", 2 * prompts, "--dynamic-sampling-filter-path",
              "miles_b200.rollout.filter_hub.check_reward_nonzero_std"]
    return a


def _grpo(k: Knobs) -> list[str]:
    a = ["--advantage-estimator", "grpo", "--eps-clip", 0.2, "--eps-clip-high", 0.28, "--entropy-coef", 0.0]
    if k.use_kl_loss:
        a += ["--use-kl-loss", "--kl-loss-coef", 0.0, "--kl-loss-type", "low_var_kl"]
    return a


def _optim(lr: float = 1e-6) -> list[str]:
    return ["--lr", lr, "--lr-decay-style", "constant", "--weight-decay", 0.1, "--adam-beta1", 0.9, "--adam-beta2", 0.98]


def _common(k: Knobs, model: str) -> list[str]:
    a = ["--model-name", model, "--colocate"]
    if k.hf_checkpoint:
        a += ["--hf-checkpoint", k.hf_checkpoint]
    if k.save:
        a += ["--save", k.save, "--save-interval", 20]
    if k.true_on_policy:
        a += ["--true-on-policy-mode"]
    if k.wandb_project:
        a += ["--use-wandb", "--wandb-project", k.wandb_project, "--wandb-group", model]
    return a


def _finish(name: str, k: Knobs, parts: list, entry: str = "train.py", notes: str = "") -> Recipe:
    args = _s(x for p in parts for x in p) + list(k.extra)
    return Recipe(name, args, entry, k.num_gpus, notes=notes)


# ---- dense Qwen3 ---------------------------------------------------------------------------------------------------

def qwen3_dense(k: Knobs, model: str = "qwen3-4B") -> Recipe:
    """Dense Qwen3 (0.6B … 32B): data parallel up to 8B; 32B shards the trainer TP = 4 (+SP) and serves with TP engines."""
    big = model.lower().endswith("32b")
    par = ["--tensor-model-parallel-size", min(4, k.num_gpus), "--sequence-parallel"] if big else []
    perf = ["--use-dynamic-batch-size", "--max-tokens-per-gpu", 16384 if big else 32768, "--recompute-granularity", "full"]
    engine = ["--sglang-mem-fraction-static", 0.6 if big else 0.7]
    return _finish(model.lower(), k, [_common(k, model), _data(k, 8192), _rollout(k, 32, 8, 8192, 256), _grpo(k), _optim(), par, perf, engine],
                   notes="scripts/run_qwen3_4b.py, run_qwen3_dense.py")


def qwen3_4b(k: Knobs) -> Recipe:
    return qwen3_dense(k, "qwen3-4B")


def qwen3_8b(k: Knobs) -> Recipe:
    return qwen3_dense(k, "qwen3-8B")


def qwen3_32b(k: Knobs) -> Recipe:
    return qwen3_dense(k, "qwen3-32B")


def qwen3_0_6b_fsdp(k: Knobs) -> Recipe:
    """The small model on the FSDP backend (parameters sharded per layer, AdamW on the shards)."""
    return _finish("qwen3-0.6b-fsdp", k, [_common(k, "qwen3-0.6B"), ["--train-backend", "fsdp"], _data(k, 4096), _rollout(k, 32, 8, 4096, 256),
                                          _grpo(k), _optim(), ["--use-dynamic-batch-size", "--max-tokens-per-gpu", 32768]],
                   notes="scripts/run_qwen3_0_6b_fsdp.py")


# ---- Qwen3 MoE ---------------------------------------------------------------------------------------------------------

def qwen3_30b_a3b(k: Knobs) -> Recipe:
    """Qwen3-30B-A3B on one box: experts over all GPUs (EP = N), attention data-parallel, routing replay, full recompute,
    32 k-token micro-batches; `--mxfp8` trains and serves the projections in MXFP8."""
    ep = k.num_gpus
    par = ["--expert-model-parallel-size", ep, "--use-rollout-routing-replay"]
    perf = ["--use-dynamic-batch-size", "--max-tokens-per-gpu", 32768, "--recompute-granularity", "full"]
    fp8 = ["--fp8-recipe", "mxfp8"] if k.mxfp8 else []
    return _finish("qwen3-30b-a3b" + ("-mxfp8" if k.mxfp8 else ""), k,
                   [_common(k, "qwen3-30B-A3B"), _data(k, 8192), _rollout(k, 64, 8, 8192, 512), _grpo(k), _optim(), par, perf, fp8,
                    ["--sglang-mem-fraction-static", 0.7]], notes="scripts/run_qwen3_30b_a3b.py:144-176,318-341")


def qwen3_30b_a3b_fsdp(k: Knobs) -> Recipe:
    return _finish("qwen3-30b-a3b-fsdp", k, [_common(k, "qwen3-30B-A3B"), ["--train-backend", "fsdp"], _data(k, 8192), _rollout(k, 32, 8, 8192, 256),
                                             _grpo(k), _optim(), ["--use-dynamic-batch-size", "--max-tokens-per-gpu", 16384,
                                                                  "--recompute-granularity", "full"]],
                   notes="scripts/run_qwen3_30b_a3b_fsdp.py")


def qwen3_235b_a22b(k: Knobs) -> Recipe:
    """Qwen3-235B-A22B: EP = 8 with the optimizer state streamed from NVMe when a directory is given through the extra
    arguments (`-- --optimizer-nvme-dir /nvme/opt`): 235 B parameters × 14 bytes of Adam state do not fit 8 × 180 GB."""
    par = ["--expert-model-parallel-size", k.num_gpus, "--tensor-model-parallel-size", min(4, k.num_gpus), "--sequence-parallel",
           "--use-rollout-routing-replay"]
    perf = ["--use-dynamic-batch-size", "--max-tokens-per-gpu", 8192, "--recompute-granularity", "full", "--offload-train"]
    return _finish("qwen3-235b-a22b", k, [_common(k, "qwen3-235B-A22B"), _data(k, 8192), _rollout(k, 32, 8, 8192, 256), _grpo(k), _optim(),
                                          par, perf, ["--sglang-mem-fraction-static", 0.5]], notes="scripts/run_qwen3_235b_a22b.py")


# ---- other settings ----------------------------------------------------------------------------------------------------

def qwen3_sft(k: Knobs) -> Recipe:
    """Supervised fine-tuning through the same loop: the 'rollout' reads (prompt, answer) pairs, the loss is token NLL."""
    a = [_common(k, "qwen3-4B"), ["--loss-type", "sft_loss", "--rollout-function-path", "miles_b200.rollout.sft_rollout.SftRolloutFn",
                                  "--rollout-batch-size", 128, "--n-samples-per-prompt", 1, "--global-batch-size", 128,
                                  "--num-rollout", 1000 if k.mode == "normal" else 2, "--disable-compute-advantages-and-returns"],
         ["--prompt-data", k.data] if k.data else ["--data-source-path", "miles_b200.rollout.data_source.SyntheticSource"],
         _optim(1e-5), ["--use-dynamic-batch-size", "--max-tokens-per-gpu", 32768]]
    return _finish("qwen3-sft", k, a, notes="scripts/run_qwen3_sft.py")


def qwen3_4b_async(k: Knobs) -> Recipe:
    """One-step-off asynchronous training: generation of step n+1 overlaps the update of step n."""
    r = qwen3_dense(k, "qwen3-4B")
    r.args = [x for x in r.args if x != "--colocate"]
    r.entry, r.name = "train_async.py", "qwen3-4b-async"
    return r


def qwen3_4b_ppo(k: Knobs) -> Recipe:
    r = qwen3_dense(k, "qwen3-4B")
    i = r.args.index("grpo")
    r.args[i] = "ppo"
    r.args += ["--critic-lr", "1e-5", "--num-critic-only-steps", "1", "--kl-coef", "0.0"]
    r.name = "qwen3-4b-ppo"
    return r


RECIPES: dict[str, Callable[[Knobs], Recipe]] = {
    "qwen3-0.6b-fsdp": qwen3_0_6b_fsdp, "qwen3-4b": qwen3_4b, "qwen3-8b": qwen3_8b, "qwen3-32b": qwen3_32b,
    "qwen3-30b-a3b": qwen3_30b_a3b, "qwen3-30b-a3b-fsdp": qwen3_30b_a3b_fsdp, "qwen3-235b-a22b": qwen3_235b_a22b,
    "qwen3-sft": qwen3_sft, "qwen3-4b-async": qwen3_4b_async, "qwen3-4b-ppo": qwen3_4b_ppo,
}


def build(name: str, knobs: Knobs | None = None) -> Recipe:
    if name not in RECIPES:
        raise KeyError(f"unknown recipe {name!r}; known: {sorted(RECIPES)}")
    return RECIPES[name](knobs or Knobs())
