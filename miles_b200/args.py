"""Command-line / YAML configuration.

Flag names are the reference's (miles/utils/arguments.py:141-2788 plus the Megatron model-shape
flags its launch scripts pass, e.g. scripts/models/qwen3-30B-A3B.py:9-45) so existing launch lines
keep working; this is one self-contained argparse parser instead of Megatron's parser extended by
an `extra_args_provider`.  Engine options keep the `--sglang-<name>` spelling and are collected
into `args.engine_kwargs`.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Any

import yaml


def _bool_flag(p, name, default=False, help=""):
    dest = name.lstrip("-").replace("-", "_")
    p.add_argument(name, dest=dest, action="store_true", default=default, help=help)
    if default:
        p.add_argument("--no-" + name.lstrip("-"), dest=dest, action="store_false")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("miles_b200", allow_abbrev=False, conflict_handler="resolve")

    g = p.add_argument_group("cluster")
    g.add_argument("--actor-num-nodes", type=int, default=1)
    g.add_argument("--actor-num-gpus-per-node", type=int, default=8)
    g.add_argument("--critic-num-nodes", type=int, default=None)
    g.add_argument("--critic-num-gpus-per-node", type=int, default=None)
    g.add_argument("--rollout-num-gpus", type=int, default=None)
    g.add_argument("--rollout-num-gpus-per-engine", type=int, default=1)
    g.add_argument("--k8s-selector", type=str, default=None, help="label selector of the engine pods (--worker-provider kubernetes)")
    g.add_argument("--k8s-namespace", type=str, default=None)
    g.add_argument("--k8s-kubectl", type=str, default=None, help="the command that lists pods as JSON (default: kubectl)")
    g.add_argument("--worker-provider", choices=["none", "local", "static", "registration", "kubernetes"], default="none",
                   help="with --rollout-engine http: where engine servers come from. local: launched, watched and restarted "
                        "by this job; static: already running at --rollout-engine-addrs; registration: they announce "
                        "themselves to the hub at --registration-hub-port; none: only a router URL is given (--engine-router-url)")
    g.add_argument("--rollout-num-engines", type=int, default=1, help="engine servers to launch with --worker-provider local")
    g.add_argument("--rollout-engine-addrs", nargs="*", default=None, help="host:port of running engine servers (static provider)")
    g.add_argument("--registration-hub-port", type=int, default=None)
    g.add_argument("--registration-ttl", type=float, default=30.0)
    g.add_argument("--worker-log-dir", type=str, default=None)
    g.add_argument("--num-gpus-per-node", type=int, default=8)
    _bool_flag(g, "--colocate", help="trainer and rollout engine share the same GPUs")
    _bool_flag(g, "--offload-train")
    _bool_flag(g, "--offload-rollout")
    g.add_argument("--offload-train-mode", choices=["vmm", "move"], default="vmm",
                   help="vmm: optimizer state in a CUDA-VMM arena whose pages are released at stable addresses (falls back to "
                        "move where the native runtime or the driver's VMM is missing); move: copy tensors to pinned host memory")
    _bool_flag(g, "--offload", help="shorthand for --offload-train --offload-rollout")
    g.add_argument("--worker-comm-backend", choices=["inproc", "rpc"], default="inproc")

    g = p.add_argument_group("train")
    g.add_argument("--train-backend", choices=["native", "megatron", "fsdp", "torchtitan"], default="native",
                   help="'megatron' selects the TP/PP/EP sharded trainer, 'fsdp' the fully-sharded one; "
                        "both are this package's own implementations")
    g.add_argument("--qkv-format", choices=["thd", "bshd"], default="thd")
    g.add_argument("--megatron-to-hf-mode", choices=["raw", "bridge"], default="raw")
    g.add_argument("--model-name", type=str, default=None, help="preset name or HF config dir")
    g.add_argument("--hf-checkpoint", type=str, default=None)
    g.add_argument("--ref-load", type=str, default=None)
    g.add_argument("--load", type=str, default=None)
    g.add_argument("--save", type=str, default=None)
    g.add_argument("--save-interval", type=int, default=None)
    g.add_argument("--offload-train-release-process-groups", action="store_true",
                   help="with --offload-train: also destroy the trainer's communicators while it sleeps (their device buffers "
                        "are freed) and re-create them on wake-up; only when the rollout engines do not share them "
                        "(--rollout-engine http, or in-process engines with tp = ep = 1)")
    g.add_argument("--export-quant", choices=["none", "fp8", "mxfp8", "nvfp4", "int4"], default="none",
                   help="quantise HF-named tensors on export: --save-hf snapshots and the tensor / broadcast / disk weight sync")
    g.add_argument("--export-quant-ignore", nargs="*", default=None, help="module names (or re:<regex>) kept in high precision")
    g.add_argument("--export-quant-all-linears", action="store_true", help="nvfp4: also the attention and dense-MLP projections (default: routed experts only)")
    g.add_argument("--nvfp4-four-over-six", action="store_true", help="per block, map the maximum to 4 or to 6, whichever quantises with less error")
    g.add_argument("--num-layers-at-start-in-bf16", type=int, default=0)
    g.add_argument("--num-layers-at-end-in-bf16", type=int, default=0)
    g.add_argument("--int4-group-size", type=int, default=32)
    g.add_argument("--int4-asymmetric", action="store_true")
    g.add_argument("--custom-step-runner-path", type=str, default=None,
                   help="module:factory(actor) → an object with forward_only_step / forward_backward_step / zero_grad / apply_step "
                        "(train/step_runner.py) replacing the built-in linear / GPipe / 1F1B schedules")
    g.add_argument("--ckpt-format", choices=["torch_dist", "native"], default="torch_dist",
                   help="torch_dist: one DCP store per iteration with Megatron-named entries and the optimizer state in "
                        "model space, reloadable under any parallel layout; native: one file per rank with that rank's shards")
    g.add_argument("--no-load-rng", action="store_true", help="do not restore the RNG state from a checkpoint")
    _bool_flag(g, "--save-hf")
    g.add_argument("--save-trigger-sentinel", type=str, default=None)
    _bool_flag(g, "--no-save-optim")
    _bool_flag(g, "--no-load-optim")
    _bool_flag(g, "--finetune")
    g.add_argument("--seed", type=int, default=1234)
    g.add_argument("--lr", type=float, default=1e-6)
    g.add_argument("--min-lr", type=float, default=0.0)
    g.add_argument("--lr-decay-style", choices=["constant", "linear", "cosine"], default="constant")
    g.add_argument("--lr-warmup-iters", type=int, default=0)
    g.add_argument("--lr-decay-iters", type=int, default=None)
    g.add_argument("--weight-decay", type=float, default=0.1)
    g.add_argument("--adam-beta1", type=float, default=0.9)
    g.add_argument("--adam-beta2", type=float, default=0.98)
    g.add_argument("--adam-eps", type=float, default=1e-8)
    g.add_argument("--clip-grad", type=float, default=1.0)
    g.add_argument("--optimizer", choices=["adam", "sgd"], default="adam")
    _bool_flag(g, "--optimizer-cpu-offload")
    _bool_flag(g, "--use-precision-aware-optimizer")
    _bool_flag(g, "--bf16", default=True)
    _bool_flag(g, "--fp32", help="train in fp32 (CPU plumbing runs)")
    g.add_argument("--fp8-format", choices=["e4m3", "hybrid"], default=None)
    g.add_argument("--fp8-recipe", choices=["mxfp8", "blockwise", "delayed"], default=None)
    g.add_argument("--fp8-backward", action="store_true",
                   help="with --fp8-recipe mxfp8: dgrad and wgrad of the dense projections in MXFP8 too (operands re-quantised along "
                        "the contraction axis); default: bf16 gradient GEMMs on the unquantised operands")
    g.add_argument("--recompute-granularity", choices=["full", "selective"], default=None)
    g.add_argument("--recompute-method", type=str, default=None)
    g.add_argument("--recompute-num-layers", type=int, default=None)
    _bool_flag(g, "--recompute-loss-function")
    g.add_argument("--attention-backend", type=str, default="flash")
    _bool_flag(g, "--deterministic-mode")
    g.add_argument("--train-iters", type=int, default=None)
    _bool_flag(g, "--disable-fused-comm", help="use NCCL + separate GEMM instead of the fused kernels")

    g = p.add_argument_group("parallel")
    g.add_argument("--tensor-model-parallel-size", type=int, default=1)
    g.add_argument("--pipeline-model-parallel-size", type=int, default=1)
    g.add_argument("--virtual-pipeline-model-parallel-size", type=int, default=None)
    g.add_argument("--pp-schedule", choices=["1f1b", "gpipe"], default="1f1b",
                   help="pipeline order of the micro-batches of an optimizer step")
    g.add_argument("--context-parallel-size", type=int, default=1)
    g.add_argument("--expert-model-parallel-size", type=int, default=1)
    g.add_argument("--expert-tensor-parallel-size", type=int, default=1)
    _bool_flag(g, "--sequence-parallel")
    g.add_argument("--cp-comm-type", choices=["p2p", "a2a", "allgather", "a2a+p2p"], default="p2p")
    g.add_argument("--hierarchical-context-parallel-sizes", type=int, nargs=2, default=None, metavar=("A2A", "P2P"),
                   help="with --cp-comm-type a2a+p2p: size of the inner all-to-all (head-swapping) groups and of the outer ring; "
                        "their product is the context-parallel size")
    _bool_flag(g, "--allgather-cp")
    _bool_flag(g, "--indep-dp")
    g.add_argument("--indep-dp-num-cells", type=int, default=1, help="independent training worlds (cells) averaging gradients")
    g.add_argument("--indep-dp-cell-id", type=int, default=0)
    g.add_argument("--indep-dp-store", default="127.0.0.1:29650", help="host:port of the cross-cell store (cell 0 serves it)")
    g.add_argument("--indep-dp-timeout", type=float, default=30.0, help="seconds before a cross-cell collective gives up")
    g.add_argument("--fsdp-dp-replicate", type=int, default=1)
    _bool_flag(g, "--use-distributed-optimizer", default=True)
    _bool_flag(g, "--overlap-grad-reduce", default=True)
    _bool_flag(g, "--overlap-param-gather", default=True)

    g = p.add_argument_group("model shape (Megatron names)")
    g.add_argument("--num-layers", type=int, default=None)
    g.add_argument("--hidden-size", type=int, default=None)
    g.add_argument("--ffn-hidden-size", type=int, default=None)
    g.add_argument("--num-attention-heads", type=int, default=None)
    _bool_flag(g, "--group-query-attention")
    g.add_argument("--num-query-groups", type=int, default=None)
    g.add_argument("--kv-channels", type=int, default=None)
    _bool_flag(g, "--qk-layernorm")
    _bool_flag(g, "--add-qkv-bias")
    _bool_flag(g, "--disable-bias-linear")
    _bool_flag(g, "--swiglu")
    _bool_flag(g, "--untie-embeddings-and-output-weights")
    g.add_argument("--normalization", type=str, default="RMSNorm")
    g.add_argument("--norm-epsilon", type=float, default=None)
    g.add_argument("--position-embedding-type", type=str, default="rope")
    g.add_argument("--rotary-percent", type=float, default=1.0)
    g.add_argument("--rotary-base", type=float, default=None)
    g.add_argument("--vocab-size", type=int, default=None)
    g.add_argument("--max-position-embeddings", type=int, default=None)
    g.add_argument("--num-experts", type=int, default=None)
    g.add_argument("--moe-router-topk", type=int, default=None)
    g.add_argument("--moe-ffn-hidden-size", type=int, default=None)
    g.add_argument("--moe-layer-freq", type=str, default=None)
    g.add_argument("--moe-router-score-function", type=str, default="softmax")
    g.add_argument("--moe-token-dispatcher-type", type=str, default="alltoall")
    g.add_argument("--moe-router-dtype", type=str, default="fp32")
    g.add_argument("--moe-aux-loss-coeff", type=float, default=0.0)
    g.add_argument("--moe-token-drop-policy", type=str, default="probs")
    _bool_flag(g, "--moe-grouped-gemm")
    _bool_flag(g, "--moe-permute-fusion")

    g = p.add_argument_group("rollout")
    g.add_argument("--rollout-function-path", type=str, default="miles_b200.rollout.inference_rollout.InferenceRolloutFn")
    g.add_argument("--eval-function-path", type=str, default=None)
    g.add_argument("--custom-generate-function-path", type=str, default=None)
    g.add_argument("--rollout-temperature", type=float, default=1.0)
    g.add_argument("--rollout-top-p", type=float, default=1.0)
    g.add_argument("--rollout-top-k", type=int, default=-1)
    g.add_argument("--rollout-max-response-len", type=int, default=1024)
    g.add_argument("--rollout-max-context-len", type=int, default=None)
    g.add_argument("--rollout-max-prompt-len", type=int, default=None)
    g.add_argument("--rollout-stop", type=str, nargs="*", default=None)
    g.add_argument("--rollout-stop-token-ids", type=int, nargs="*", default=None)
    _bool_flag(g, "--rollout-skip-special-tokens")
    g.add_argument("--over-sampling-batch-size", type=int, default=None)
    g.add_argument("--dynamic-sampling-filter-path", type=str, default=None)
    g.add_argument("--buffer-filter-path", type=str, default=None)
    g.add_argument("--rollout-sample-filter-path", type=str, default=None)
    _bool_flag(g, "--partial-rollout")
    g.add_argument("--num-rollout", type=int, default=None)
    g.add_argument("--num-epoch", type=int, default=None)
    g.add_argument("--update-weight-buffer-size", type=int, default=512 * 1024 * 1024)
    g.add_argument("--update-weight-transfer-mode", choices=["auto", "alias", "nvlink", "tensor", "broadcast", "broadcast_packed", "cuda_ipc", "p2p", "disk", "delta"],
                   default="auto")
    g.add_argument("--update-weights-interval", type=int, default=1)
    _bool_flag(g, "--fully-async")
    g.add_argument("--max-weight-staleness", type=int, default=1)
    g.add_argument("--staleness-policy", choices=["drop", "retry", "keep"], default="drop")
    g.add_argument("--fully-async-buffer-groups", type=int, default=None,
                   help="finished prompt groups the producer keeps ready (default: one rollout batch)")
    g.add_argument("--fully-async-take-timeout", type=float, default=None)
    g.add_argument("--rollout-engine", choices=["native", "http", "mock"], default="native")
    g.add_argument("--router-policy", choices=["least_active", "round_robin", "consistent_hashing", "random"], default="least_active")
    _bool_flag(g, "--use-miles-router", default=True)
    _bool_flag(g, "--use-session-server")

    g = p.add_argument_group("data")
    g.add_argument("--prompt-data", type=str, default=None)
    g.add_argument("--input-key", type=str, default="input")
    g.add_argument("--label-key", type=str, default=None)
    g.add_argument("--metadata-key", type=str, default="metadata")
    g.add_argument("--tool-key", type=str, default=None)
    _bool_flag(g, "--apply-chat-template")
    g.add_argument("--apply-chat-template-kwargs", type=json.loads, default=None)
    _bool_flag(g, "--rollout-shuffle")
    g.add_argument("--rollout-seed", type=int, default=42)
    g.add_argument("--rollout-batch-size", type=int, default=None)
    g.add_argument("--n-samples-per-prompt", type=int, default=1)
    g.add_argument("--global-batch-size", type=int, default=None)
    g.add_argument("--num-steps-per-rollout", type=int, default=None)
    g.add_argument("--micro-batch-size", type=int, default=1)
    _bool_flag(g, "--use-dynamic-batch-size")
    g.add_argument("--max-tokens-per-gpu", type=int, default=None)
    _bool_flag(g, "--balance-data")
    g.add_argument("--rollout-pd-prefill-engines", type=int, default=0,
                   help="prefill / decode disaggregation over an HTTP engine fleet: this many of --rollout-num-engines run prompts "
                        "only and hand the KV to the others, which decode")
    g.add_argument("--rollout-data-exchange", choices=["gather", "local", "balanced"], default="gather",
                   help="gather: every rank receives all samples of the step and takes its (balanced) share; local: with one "
                        "engine per data-parallel rank each rank trains on the samples it generated (whole prompt groups "
                        "stay together, nothing but a few metric sums crosses ranks); balanced: local, then the ranks with "
                        "the most tokens hand whole prompt groups to those with the fewest (point to point) until no move "
                        "narrows the spread: every rank waits for the slowest one at each collective of the train step")
    g.add_argument("--log-probs-max-tokens-per-gpu", type=int, default=None)
    g.add_argument("--data-source-path", type=str, default="miles_b200.rollout.data_source.RolloutDataSourceWithBuffer")
    g.add_argument("--synthetic-prompt-len", type=int, nargs=2, default=None, metavar=("MIN", "MAX"),
                   help="prompt length range of miles_b200.rollout.data_source.SyntheticSource")
    g.add_argument("--tokenizer-path", type=str, default=None)

    g = p.add_argument_group("eval")
    g.add_argument("--eval-interval", type=int, default=None)
    g.add_argument("--eval-prompt-data", type=str, nargs="*", default=None)
    g.add_argument("--eval-config", type=str, default=None)
    g.add_argument("--n-samples-per-eval-prompt", type=int, default=1)
    g.add_argument("--eval-temperature", type=float, default=None)
    g.add_argument("--eval-top-p", type=float, default=None)
    g.add_argument("--eval-max-response-len", type=int, default=None)
    _bool_flag(g, "--skip-eval-before-train")

    g = p.add_argument_group("algo")
    g.add_argument("--eps-clip", type=float, default=0.2)
    g.add_argument("--eps-clip-high", type=float, default=None)
    g.add_argument("--eps-clip-c", type=float, default=None)
    g.add_argument("--value-clip", type=float, default=0.2)
    g.add_argument("--kl-coef", type=float, default=0.0)
    g.add_argument("--loss-type", choices=["policy_loss", "value_loss", "sft_loss", "custom_loss", "score_centering"], default="policy_loss")
    g.add_argument("--custom-loss-function-path", type=str, default=None)
    _bool_flag(g, "--use-kl-loss")
    g.add_argument("--kl-loss-coef", type=float, default=0.0)
    g.add_argument("--kl-loss-type", choices=["k1", "k2", "k3", "low_var_kl"], default="k1")
    _bool_flag(g, "--use-unbiased-kl")
    g.add_argument("--advantage-estimator", choices=["grpo", "gspo", "ppo", "reinforce_plus_plus", "reinforce_plus_plus_baseline"], default="grpo")
    _bool_flag(g, "--normalize-advantages")
    _bool_flag(g, "--disable-grpo-std-normalization")
    _bool_flag(g, "--disable-rewards-normalization")
    g.add_argument("--entropy-coef", type=float, default=0.0)
    g.add_argument("--gamma", type=float, default=1.0)
    g.add_argument("--lambd", type=float, default=1.0)
    _bool_flag(g, "--use-tis")
    g.add_argument("--tis-clip", type=float, default=2.0)
    g.add_argument("--tis-clip-low", type=float, default=0.0)
    g.add_argument("--tis-mode", choices=["clip", "icepop"], default="clip")
    g.add_argument("--custom-tis-function-path", type=str, default=None)
    _bool_flag(g, "--get-mismatch-metrics")
    _bool_flag(g, "--use-opsm")
    g.add_argument("--opsm-delta", type=float, default=1e-4)
    _bool_flag(g, "--use-rollout-logprobs")
    _bool_flag(g, "--use-rollout-routing-replay")
    _bool_flag(g, "--use-routing-replay")
    _bool_flag(g, "--calculate-per-token-loss")
    g.add_argument("--log-probs-chunk-size", type=int, default=-1)
    _bool_flag(g, "--skip-actor-forward-only")
    g.add_argument("--opd-kl-coef", type=float, default=0.0)
    g.add_argument("--opd-teacher-url", type=str, default=None)
    g.add_argument("--opd-task-rm-type", type=str, default=None)
    g.add_argument("--multi-turn-env-path", type=str, default=None)
    g.add_argument("--max-turns", type=int, default=8)
    g.add_argument("--max-tokens-per-turn", type=int, default=None)
    g.add_argument("--tools-path", type=str, default=None)
    g.add_argument("--num-critic-only-steps", type=int, default=0)
    g.add_argument("--critic-lr", type=float, default=None)
    g.add_argument("--ref-update-interval", type=int, default=None)
    _bool_flag(g, "--true-on-policy-mode")

    g = p.add_argument_group("reward")
    g.add_argument("--rm-type", type=str, default=None)
    g.add_argument("--rm-url", type=str, default=None)
    g.add_argument("--custom-rm-path", type=str, default=None)
    g.add_argument("--reward-key", type=str, default=None)
    g.add_argument("--eval-reward-key", type=str, default=None)
    _bool_flag(g, "--group-rm")
    g.add_argument("--custom-reward-post-process-path", type=str, default=None)
    g.add_argument("--custom-convert-samples-to-train-data-path", type=str, default=None)

    g = p.add_argument_group("lora")
    g.add_argument("--lora-rank", type=int, default=0)
    g.add_argument("--lora-alpha", type=float, default=16.0)
    g.add_argument("--lora-dropout", type=float, default=0.0)
    g.add_argument("--lora-target-modules", type=str, nargs="*", default=["wqkv", "wo", "w13", "w2"])
    g.add_argument("--lora-num-slots", type=int, default=1)
    g.add_argument("--lora-adapter-path", type=str, default=None)

    g = p.add_argument_group("fault tolerance")
    _bool_flag(g, "--use-fault-tolerance")
    g.add_argument("--ft-components", type=str, nargs="*", default=["train", "rollout"])
    g.add_argument("--rollout-health-check-interval", type=float, default=10.0)
    g.add_argument("--rollout-health-check-timeout", type=float, default=5.0)
    g.add_argument("--rollout-health-check-first-wait", type=float, default=30.0)
    g.add_argument("--ft-failure-threshold", type=int, default=3)
    g.add_argument("--ft-max-retries", type=int, default=30)

    g = p.add_argument_group("tracking")
    _bool_flag(g, "--use-wandb")
    g.add_argument("--wandb-project", type=str, default=None)
    g.add_argument("--wandb-group", type=str, default=None)
    g.add_argument("--wandb-mode", type=str, default=None)
    _bool_flag(g, "--use-tensorboard")
    g.add_argument("--tb-dir", type=str, default=None)
    _bool_flag(g, "--use-mlflow")
    _bool_flag(g, "--use-prometheus")
    g.add_argument("--prometheus-port", type=int, default=9400)
    g.add_argument("--jsonl-metrics-path", type=str, default=None)
    g.add_argument("--event-log-dir", type=str, default=None)
    _bool_flag(g, "--use-dashboard")
    g.add_argument("--dashboard-port", type=int, default=8265)
    g.add_argument("--log-interval", type=int, default=1)

    g = p.add_argument_group("debug")
    _bool_flag(g, "--debug-rollout-only")
    _bool_flag(g, "--debug-train-only")
    g.add_argument("--load-debug-rollout-data", type=str, default=None)
    g.add_argument("--save-debug-rollout-data", type=str, default=None)
    g.add_argument("--dump-details", type=str, default=None,
                   help="directory for everything a post-mortem needs: rollout dumps (rollout_data/{id}.pt), per-rank train data "
                        "(train_data/{id}_{rank}.pt) and, with --use-miles-dashboard, metrics and per-rank phase intervals (dashboard/)")
    g.add_argument("--use-miles-dashboard", action="store_true",
                   help="record metrics and per-rank phase intervals under <dump-details>/dashboard for `python -m miles_b200.dashboard.server "
                        "--dump-details DIR`")
    g.add_argument("--save-debug-train-data", type=str, default=None, help="path pattern ({rollout_id}, {rank}) for per-rank train data")
    _bool_flag(g, "--check-weight-update-equal")
    _bool_flag(g, "--debug-deterministic-collective")
    _bool_flag(g, "--ci-test")
    g.add_argument("--ft-max-attempts", type=int, default=30, help="retries of a failed trainer call under --use-fault-tolerance")
    g.add_argument("--ft-heartbeat-timeout", type=float, default=60.0)
    _bool_flag(g, "--true-on-policy-mode", help="pin every source of train / rollout numeric divergence (see utils/true_on_policy)")
    g.add_argument("--snapshot-dir", type=str, default=None,
                   help="publish a full HF safetensors snapshot of the policy here every --snapshot-interval weight updates")
    g.add_argument("--snapshot-interval", type=int, default=1)
    g.add_argument("--snapshot-keep", type=int, default=2)
    g.add_argument("--optimizer-nvme-dir", type=str, default=None,
                   help="stream fp32 master weights and Adam moments from files in this directory (state larger than HBM + host)")
    g.add_argument("--optimizer-nvme-bucket-numel", type=int, default=64 << 20, help="floats per streamed bucket (three such buffers on the device)")
    g.add_argument("--audit-dir", type=str, default=None,
                   help="write the audit event log here (weight checksums per version; analyse with miles_b200.audit.events)")
    g.add_argument("--ci-save-grad-norm", type=str, default=None)
    g.add_argument("--ci-load-grad-norm", type=str, default=None)
    _bool_flag(g, "--use-pytorch-profiler")
    g.add_argument("--profile-target", type=str, nargs="*", default=["train_overall"])
    g.add_argument("--profile-step-start", type=int, default=10)
    g.add_argument("--profile-step-end", type=int, default=12)
    g.add_argument("--tensorboard-dir", type=str, default=None)
    _bool_flag(g, "--record-memory-history")
    g.add_argument("--memory-snapshot-dir", type=str, default=".")
    g.add_argument("--memory-snapshot-path", type=str, default="snapshot.pickle")
    g.add_argument("--memory-snapshot-num-steps", type=int, default=None)
    g.add_argument("--memory-recorder", choices=["torch"], default="torch")
    _bool_flag(g, "--nvtx", help="NVTX ranges around the trainer's phases")

    g = p.add_argument_group("user functions")
    g.add_argument("--custom-megatron-init-path", type=str, default=None)
    g.add_argument("--custom-model-provider-path", type=str, default=None)
    g.add_argument("--custom-pg-loss-reducer-function-path", type=str, default=None)
    g.add_argument("--custom-rollout-log-function-path", type=str, default=None)
    g.add_argument("--custom-eval-rollout-log-function-path", type=str, default=None)
    g.add_argument("--custom-config-path", type=str, default=None)
    from .args_compat import add_compat_arguments

    add_compat_arguments(p)       # every remaining flag name of the reference's parser
    return p


_ENGINE_PREFIXES = ("--sglang-", "--engine-")


def _split_engine_args(argv: list[str]) -> tuple[list[str], dict[str, Any]]:
    """Pull `--sglang-<name> [value]` / `--engine-<name> [value]` out of argv into a dict."""
    rest, kw = [], {}
    i = 0
    while i < len(argv):
        a = argv[i]
        pref = next((p for p in _ENGINE_PREFIXES if a.startswith(p)), None)
        if pref is None:
            rest.append(a)
            i += 1
            continue
        body = a[len(pref):]
        if "=" in body:
            name, val = body.split("=", 1)
            i += 1
        elif i + 1 < len(argv) and not argv[i + 1].startswith("--"):
            name, val = body, argv[i + 1]
            i += 2
        else:
            name, val = body, True
            i += 1
        if isinstance(val, str):
            for cast in (int, float):
                try:
                    val = cast(val)
                    break
                except ValueError:
                    pass
        kw[name.replace("-", "_")] = val
    return rest, kw


def parse_args(argv: list[str] | None = None, validate: bool = True) -> argparse.Namespace:
    import sys

    argv = list(sys.argv[1:] if argv is None else argv)
    argv, engine_kwargs = _split_engine_args(argv)
    parser = build_parser()
    args = parser.parse_args(argv)
    # `--engine-config` / `--sglang-config FILE`: the YAML serving config ({models: [{name, model_path, server_groups:
    # [{worker_type: regular|prefill|decode, num_gpus, num_gpus_per_engine, overrides}]}]}); the policy model's groups size
    # the HTTP engine fleet, prefill + decode groups run it in prefill / decode roles (`orchestration/wiring.apply_serving_config`)
    args.engine_config = engine_kwargs.pop("config", None)
    args.engine_kwargs = engine_kwargs
    if args.custom_config_path:
        with open(args.custom_config_path) as f:
            for k, v in (yaml.safe_load(f) or {}).items():
                setattr(args, k.replace("-", "_"), v)
    if validate:
        validate_args(args)
    return args


def validate_args(args) -> None:
    """Derived values and cross-flag invariants (reference: `miles_validate_args`, arguments.py:3214-3950)."""
    if args.offload:
        args.offload_train = args.offload_rollout = True
    if args.colocate:
        args.offload_train = args.offload_rollout = True
        if args.rollout_num_gpus is None:
            args.rollout_num_gpus = args.actor_num_nodes * args.actor_num_gpus_per_node
    if args.rollout_num_gpus is None:
        args.rollout_num_gpus = args.actor_num_nodes * args.actor_num_gpus_per_node
    if args.eps_clip_high is None:
        args.eps_clip_high = args.eps_clip
    if args.use_fault_tolerance:
        args.indep_dp = args.indep_dp or "train" in (args.ft_components or [])
    if getattr(args, "enable_witness", False) and not args.audit_dir:
        args.audit_dir = "audit"            # witnesses are events of the audit log
    if getattr(args, "true_on_policy_mode", False):
        from .utils import true_on_policy

        args.true_on_policy_contracts = true_on_policy.apply(args)
    args.rewards_normalization = not args.disable_rewards_normalization
    args.grpo_std_normalization = not args.disable_grpo_std_normalization
    if args.use_rollout_routing_replay:
        args.use_routing_replay = True
    if args.allgather_cp:
        args.cp_comm_type = "allgather"
    if args.fp32:
        args.bf16 = False

    if getattr(args, "dump_details", None):
        d = args.dump_details
        args.save_debug_rollout_data = args.save_debug_rollout_data or os.path.join(d, "rollout_data", "{rollout_id}.pt")
        args.save_debug_train_data = getattr(args, "save_debug_train_data", None) or os.path.join(d, "train_data", "{rollout_id}_{rank}.pt")
        if getattr(args, "use_miles_dashboard", False) and not args.jsonl_metrics_path:
            args.jsonl_metrics_path = os.path.join(d, "dashboard", "metrics.jsonl")
    elif getattr(args, "use_miles_dashboard", False):
        raise ValueError("--use-miles-dashboard needs --dump-details DIR")
    if getattr(args, "use_opd", False):
        if args.opd_type is None:
            raise ValueError("--use-opd needs --opd-type sglang (teacher engines) or megatron (teacher weights in the trainer)")
        if (args.opd_log_prob_top_k or 0) < 0:
            raise ValueError("--opd-log-prob-top-k must be non-negative")
        if (args.opd_log_prob_top_k or 0) > 0 and args.opd_type != "sglang":
            raise ValueError("--opd-log-prob-top-k needs --opd-type sglang")
        if args.opd_type == "sglang":
            from .rollout.opd import parse_teacher_urls

            parse_teacher_urls(args.opd_teacher_urls)          # malformed or duplicate entries fail here, not mid-rollout
            if not (args.opd_teacher_urls or args.opd_teacher_url or getattr(args, "opd_teacher_client", None)):
                raise ValueError("--opd-type sglang needs --opd-teacher-url or --opd-teacher-urls")
            if not getattr(args, "custom_rm_path", None):
                args.custom_rm_path = "miles_b200.rollout.opd.opd_reward"   # scoring rides on the reward hook
        elif args.opd_type == "megatron":
            if not args.opd_teacher_load or not os.path.isdir(args.opd_teacher_load):
                raise ValueError("--opd-type megatron needs --opd-teacher-load pointing at a checkpoint directory")
        if not args.opd_kl_coef:
            args.opd_kl_coef = 1.0
    # four-knob invariant: rollout_batch_size × n_samples = global_batch_size × num_steps_per_rollout
    if args.rollout_batch_size is not None:
        total = args.rollout_batch_size * args.n_samples_per_prompt
        if args.global_batch_size is None and args.num_steps_per_rollout is None:
            args.num_steps_per_rollout = 1
        if args.global_batch_size is None:
            assert total % args.num_steps_per_rollout == 0
            args.global_batch_size = total // args.num_steps_per_rollout
        elif args.num_steps_per_rollout is None:
            assert total % args.global_batch_size == 0, (
                f"rollout_batch_size×n_samples_per_prompt ({total}) must be a multiple of global_batch_size "
                f"({args.global_batch_size})")
            args.num_steps_per_rollout = total // args.global_batch_size
        else:
            assert total == args.global_batch_size * args.num_steps_per_rollout, (
                "rollout_batch_size × n_samples_per_prompt must equal global_batch_size × num_steps_per_rollout")
    if args.over_sampling_batch_size is None:
        args.over_sampling_batch_size = args.rollout_batch_size
    if args.use_dynamic_batch_size:
        assert args.max_tokens_per_gpu is not None, "--use-dynamic-batch-size needs --max-tokens-per-gpu"
    if args.log_probs_max_tokens_per_gpu is None:
        args.log_probs_max_tokens_per_gpu = args.max_tokens_per_gpu
    if args.rollout_max_context_len is None and args.rollout_max_prompt_len is not None:
        args.rollout_max_context_len = args.rollout_max_prompt_len + args.rollout_max_response_len
    if args.advantage_estimator == "ppo" and args.critic_num_nodes is None:
        args.critic_num_nodes = args.actor_num_nodes
        args.critic_num_gpus_per_node = args.actor_num_gpus_per_node
    if args.critic_lr is None:
        args.critic_lr = args.lr
    if args.loss_type == "custom_loss":
        assert args.custom_loss_function_path, "--loss-type custom_loss needs --custom-loss-function-path"
    if args.kl_coef != 0 or args.use_kl_loss:
        args.need_ref = True
    else:
        args.need_ref = False
    if args.sequence_parallel and args.tensor_model_parallel_size == 1:
        args.sequence_parallel = False
    if args.tensor_model_parallel_size > 1:
        args.sequence_parallel = True
    if args.train_backend in ("megatron", "fsdp", "torchtitan"):
        args.train_layout = {"megatron": "tp_pp_ep", "fsdp": "fsdp", "torchtitan": "tp_pp_ep"}[args.train_backend]
    else:
        args.train_layout = "tp_pp_ep"
    if args.debug_rollout_only and args.debug_train_only:
        raise ValueError("--debug-rollout-only and --debug-train-only are exclusive")


def model_config_from_args(args):
    """ModelConfig from --model-name / --hf-checkpoint, overridden by explicit Megatron shape flags."""
    from .models.config import ModelConfig, get_config

    if args.model_name:
        cfg = get_config(args.model_name)
    elif args.hf_checkpoint and os.path.exists(os.path.join(args.hf_checkpoint, "config.json")):
        cfg = ModelConfig.from_hf_config(args.hf_checkpoint)
    else:
        cfg = ModelConfig()
    over = {}
    m = {
        "num_layers": "num_layers", "hidden_size": "hidden_size", "ffn_hidden_size": "ffn_hidden_size",
        "num_attention_heads": "num_heads", "num_query_groups": "num_kv_heads", "kv_channels": "head_dim",
        "norm_epsilon": "rms_eps", "rotary_base": "rope_theta", "vocab_size": "vocab_size",
        "num_experts": "num_experts", "moe_router_topk": "moe_topk", "moe_ffn_hidden_size": "moe_ffn_hidden_size",
        "max_position_embeddings": "max_position",
    }
    for a, c in m.items():
        v = getattr(args, a, None)
        if v is not None:
            over[c] = type(getattr(cfg, c))(v)
    if args.qk_layernorm:
        over["qk_norm"] = True
    if args.add_qkv_bias:
        over["qkv_bias"] = True
    if args.untie_embeddings_and_output_weights:
        over["tie_embeddings"] = False
    if args.num_attention_heads is not None and not args.group_query_attention and args.num_query_groups is None:
        over["num_kv_heads"] = args.num_attention_heads
    return cfg.with_(**over) if over else cfg
