"""Metric fan-out: stdout, JSONL, TensorBoard, W&B, MLflow, Prometheus, in-memory history.

`Tracker.log(metrics, step, step_key)` is the single sink (reference: miles/utils/tracking_utils/
tracking.py:23-56 with one backend class per system, base.py:26-208).  Backends that need packages
absent from the environment disable themselves with one warning instead of failing the run.
"""
from __future__ import annotations

import json
import logging
import os
import time
from typing import Any

log = logging.getLogger("miles_b200")


class _Backend:
    def log(self, metrics: dict, step: int, step_key: str): ...
    def finish(self): ...


class StdoutBackend(_Backend):
    def log(self, metrics, step, step_key):
        body = " ".join(f"{k}={v:.5g}" if isinstance(v, float) else f"{k}={v}" for k, v in sorted(metrics.items()))
        print(f"[{step_key}={step}] {body}", flush=True)


class JsonlBackend(_Backend):
    def __init__(self, path):
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        self.f = open(path, "a")

    def log(self, metrics, step, step_key):
        self.f.write(json.dumps({"ts": time.time(), step_key: step, **metrics}) + "\n")
        self.f.flush()

    def finish(self):
        self.f.close()


class HistoryBackend(_Backend):
    """Keeps everything in memory; CI gates and tests read it (`ci_history` in the reference)."""

    def __init__(self):
        self.rows: list[dict] = []

    def log(self, metrics, step, step_key):
        self.rows.append({step_key: step, **metrics})

    def series(self, key: str) -> list:
        return [r[key] for r in self.rows if key in r]


class TensorboardBackend(_Backend):
    def __init__(self, logdir):
        from torch.utils.tensorboard import SummaryWriter

        self.w = SummaryWriter(logdir)

    def log(self, metrics, step, step_key):
        for k, v in metrics.items():
            if isinstance(v, (int, float)):
                self.w.add_scalar(k, v, step)

    def finish(self):
        self.w.close()


class WandbBackend(_Backend):
    def __init__(self, args):
        import wandb

        self.wandb = wandb
        import os as _os

        if getattr(args, "wandb_key", None):
            _os.environ.setdefault("WANDB_API_KEY", args.wandb_key)
        if getattr(args, "wandb_host", None):
            _os.environ.setdefault("WANDB_BASE_URL", args.wandb_host)
        name = getattr(args, "wandb_run_name", None) or getattr(args, "wandb_group", None)
        if name and getattr(args, "wandb_random_suffix", True):
            import uuid as _uuid

            name = f"{name}-{_uuid.uuid4().hex[:6]}"
        wandb.init(project=args.wandb_project, group=args.wandb_group, mode=args.wandb_mode, config=vars(args), name=name,
                   entity=getattr(args, "wandb_team", None), dir=getattr(args, "wandb_dir", None),
                   id=getattr(args, "wandb_run_id", None), resume="allow" if getattr(args, "wandb_run_id", None) else None)

    def log(self, metrics, step, step_key):
        self.wandb.log({**metrics, step_key: step})

    def finish(self):
        self.wandb.finish()


class MlflowBackend(_Backend):
    def __init__(self, args):
        import mlflow

        self.mlflow = mlflow
        if getattr(args, "mlflow_tracking_uri", None):
            mlflow.set_tracking_uri(args.mlflow_tracking_uri)
        if getattr(args, "mlflow_experiment_name", None):
            mlflow.set_experiment(args.mlflow_experiment_name)
        mlflow.start_run(run_id=getattr(args, "mlflow_run_id", None), run_name=getattr(args, "mlflow_run_name", None))

    def log(self, metrics, step, step_key):
        self.mlflow.log_metrics({k.replace("/", "."): v for k, v in metrics.items() if isinstance(v, (int, float))}, step=step)

    def finish(self):
        self.mlflow.end_run()


class PrometheusBackend(_Backend):
    def __init__(self, port):
        from prometheus_client import Gauge, start_http_server

        self.Gauge = Gauge
        self.gauges: dict[str, Any] = {}
        start_http_server(port)

    def log(self, metrics, step, step_key):
        for k, v in metrics.items():
            if not isinstance(v, (int, float)):
                continue
            name = "miles_" + "".join(c if c.isalnum() else "_" for c in k)
            if name not in self.gauges:
                self.gauges[name] = self.Gauge(name, k)
            self.gauges[name].set(v)


class Tracker:
    def __init__(self, args=None, stdout: bool = True):
        self.backends: list[_Backend] = []
        self.history = HistoryBackend()
        self.backends.append(self.history)
        if stdout:
            self.backends.append(StdoutBackend())
        if args is None:
            return
        self._try(lambda: JsonlBackend(args.jsonl_metrics_path), getattr(args, "jsonl_metrics_path", None))
        self._try(lambda: TensorboardBackend(args.tb_dir or args.tensorboard_dir or "runs"), getattr(args, "use_tensorboard", False))
        self._try(lambda: WandbBackend(args), getattr(args, "use_wandb", False))
        self._try(lambda: MlflowBackend(args), getattr(args, "use_mlflow", False))
        self._try(lambda: PrometheusBackend(args.prometheus_port), getattr(args, "use_prometheus", False))

    def _try(self, make, enabled):
        if not enabled:
            return
        try:
            self.backends.append(make())
        except Exception as e:
            log.warning("tracking backend disabled: %s", e)

    def add_backend(self, backend: _Backend):
        self.backends.append(backend)

    def log(self, metrics: dict, step: int, step_key: str = "rollout/step"):
        clean = {k: (float(v) if hasattr(v, "item") else v) for k, v in metrics.items()}
        for b in self.backends:
            try:
                b.log(clean, step, step_key)
            except Exception as e:  # a broken sink must not stop training
                log.warning("tracking backend %s failed: %s", type(b).__name__, e)

    def finish(self):
        for b in self.backends:
            b.finish()
