"""Launch helpers: model argument presets, command construction and local execution of training jobs.

Reference: miles/utils/external_utils/command_utils/base_backend.py:67-209 (`ExecuteTrainConfig`,
`U.execute_train(train_args, …)`, `U.convert_checkpoint`), the model scripts under scripts/models/*.py (argument
strings per architecture, e.g. scripts/models/qwen3-30B-A3B.py:9-45) and scripts/run_qwen3_30b_a3b.py (the recipe).
The reference submits a Ray job or a Helm release; a single NVSwitch box needs neither, so the backend here is
`torchrun` on this machine (one process per GPU) — `dry_run=True` returns the command for another scheduler to run.
"""
from __future__ import annotations

import os
import shlex
import subprocess
import sys
from dataclasses import dataclass, field

REPO_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def model_args(name: str) -> list[str]:
    """Megatron-style shape flags of a preset (what the reference keeps in scripts/models/<name>.py)."""
    from ..models.config import PRESETS

    c = PRESETS[name]
    a = ["--num-layers", c.num_layers, "--hidden-size", c.hidden_size, "--ffn-hidden-size", c.ffn_hidden_size,
         "--num-attention-heads", c.num_heads, "--num-query-groups", c.num_kv_heads, "--kv-channels", c.head_dim,
         "--rotary-base", int(c.rope_theta), "--vocab-size", c.vocab_size, "--norm-epsilon", c.rms_eps]
    if c.num_heads != c.num_kv_heads:
        a.append("--group-query-attention")
    if c.qk_norm:
        a.append("--qk-layernorm")
    if c.num_experts:
        a += ["--num-experts", c.num_experts, "--moe-router-topk", c.moe_topk, "--moe-ffn-hidden-size", c.moe_ffn_hidden_size]
    if not c.tie_embeddings:
        a.append("--untie-embeddings-and-output-weights")
    return [str(x) for x in a]


def qwen3_30b_a3b_recipe(num_gpus: int = 8, mxfp8: bool = False) -> list[str]:
    """The reference's B200 recipe (scripts/run_qwen3_30b_a3b.py:152-176,318-341) in this package's flags."""
    tp = min(4, num_gpus)
    ep = min(8 if mxfp8 else 4, num_gpus)
    a = ["--model-name", "qwen3-30B-A3B", "--colocate", "--tensor-model-parallel-size", tp, "--sequence-parallel",
         "--expert-model-parallel-size", ep, "--rollout-batch-size", 32, "--n-samples-per-prompt", 8, "--rollout-max-response-len", 8192,
         "--rollout-temperature", 1.0, "--global-batch-size", 256, "--use-dynamic-batch-size", "--max-tokens-per-gpu", 32768,
         "--recompute-granularity", "full", "--advantage-estimator", "grpo", "--eps-clip", 0.2, "--eps-clip-high", 0.28,
         "--lr", 1e-6, "--weight-decay", 0.1, "--adam-beta2", 0.98, "--sglang-mem-fraction-static", 0.7, "--use-rollout-routing-replay"]
    return [str(x) for x in a]


@dataclass
class ExecuteTrainConfig:
    num_gpus: int = 1
    entry: str = "train.py"                 # train.py | train_async.py | train_multi_policy.py
    master_port: int = 29511
    env: dict = field(default_factory=dict)
    log_file: str | None = None
    dry_run: bool = False
    launcher: str = "torchrun"              # torchrun | workers (ranks as supervised processes of the worker manager)
    num_cells: int = 1                      # workers launcher: independent trainer cells (`--indep-dp`), each its own world
    log_dir: str | None = None              # workers launcher: one log per rank and generation


def build_command(train_args: list[str] | str, cfg: ExecuteTrainConfig) -> list[str]:
    args = shlex.split(train_args) if isinstance(train_args, str) else list(train_args)
    entry = os.path.join(REPO_ROOT, cfg.entry)
    if cfg.num_gpus <= 1:
        return [sys.executable, entry, *args]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={cfg.num_gpus}",
            "--master-addr", "127.0.0.1", "--master-port", str(cfg.master_port), entry, *args]


def trainer_spec(train_args: list[str] | str, cfg: ExecuteTrainConfig, name: str = "trainer"):
    """The trainer as a pool of the worker layer: `num_cells` cells of `num_gpus` ranks, one process per rank, with the
    rendezvous variables of its cell (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT) planned like any other
    pool's.  Every GPU stays visible to every rank (the fused kernels map peers' memory); `{cell}` in the arguments is
    the cell index (e.g. `--indep-dp-cell-id {cell}`).  The reference describes its trainer actors the same way
    (miles/ray/trainer/trainer_spec.py: pools, per-pool environment)."""
    from ..orchestration.worker_spec import CommandWorkerSpec, SchedulingSpec

    args = shlex.split(train_args) if isinstance(train_args, str) else list(train_args)
    return CommandWorkerSpec(name, [sys.executable, os.path.join(REPO_ROOT, cfg.entry), *args],
                             SchedulingSpec(num_cells=cfg.num_cells, workers_per_cell=max(1, cfg.num_gpus), gpus_per_worker=1),
                             env={"CUDA_VISIBLE_DEVICES": "__inherit__", **{k: str(v) for k, v in cfg.env.items()}}, ports=[])


def run_trainer_pool(train_args: list[str] | str, cfg: ExecuteTrainConfig, poll_s: float = 0.2) -> int:
    """Start the trainer pool under the worker manager and wait: 0 when every rank exited 0; the first non-zero exit code
    otherwise, after the remaining ranks were stopped (a rank that died cannot be waited for by its peers' collectives)."""
    import time

    from ..orchestration.workers.manager import WorkerManager

    mgr = WorkerManager(log_dir=cfg.log_dir)
    mgr.launch([trainer_spec(train_args, cfg)], nodes={"local": cfg.num_cells * max(1, cfg.num_gpus)})
    try:
        while True:
            codes = [wk.proc.poll() for c in mgr.cells.values() for wk in c.workers]
            bad = [c for c in codes if c not in (None, 0)]
            if bad:
                return int(bad[0])
            if all(c == 0 for c in codes):
                return 0
            time.sleep(poll_s)
    finally:
        mgr.stop_all()


def execute_train(train_args: list[str] | str, cfg: ExecuteTrainConfig | None = None) -> int | list[str]:
    cfg = cfg or ExecuteTrainConfig()
    if cfg.launcher == "workers":
        if cfg.dry_run:
            from ..orchestration.workers.manager import WorkerManager

            return WorkerManager().launch([trainer_spec(train_args, cfg)], nodes={"local": cfg.num_cells * max(1, cfg.num_gpus)},
                                          dry_run=True)
        return run_trainer_pool(train_args, cfg)
    cmd = build_command(train_args, cfg)
    if cfg.dry_run:
        return cmd
    env = {**os.environ, **{k: str(v) for k, v in cfg.env.items()}}
    out = open(cfg.log_file, "w") if cfg.log_file else None
    try:
        return subprocess.run(cmd, env=env, stdout=out, stderr=subprocess.STDOUT if out else None, cwd=REPO_ROOT).returncode
    finally:
        if out:
            out.close()


def convert_checkpoint(kind: str, **kw) -> int:
    """Run a converter of `miles_b200.tools.convert` (e.g. kind="hf-to-torch-dist", hf=…, out=…)."""
    argv = [kind]
    for k, v in kw.items():
        argv += [f"--{k.replace('_', '-')}", str(v)]
    return subprocess.run([sys.executable, "-m", "miles_b200.tools.convert", *argv], cwd=REPO_ROOT).returncode
