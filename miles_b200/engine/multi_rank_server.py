"""One engine server over several GPUs: `torchrun --nproc-per-node N -m miles_b200.engine.multi_rank_server …`.

The reference starts one serving process group per engine when `--rollout-num-gpus-per-engine` > 1 (tensor / expert
parallel SGLang servers behind one HTTP port).  Here every rank runs an `Engine` over the same `ParallelState`:

* MoE models shard the experts over the ranks (`--expert-model-parallel-size N`); each rank serves ITS OWN requests
  (data-parallel attention) and the ranks step in lockstep because every MoE layer is a collective;
* dense models shard the projections (`--tensor-model-parallel-size N`); every rank runs EVERY request (same seeds, same
  tokens) and rank 0's copy is the answer.

Rank 0 owns the HTTP port.  A control loop ties the ranks together: every tick rank 0 broadcasts the commands that arrived
(add request → target rank or all, abort, pause / continue, flush, load weights from a directory, shutdown) over a gloo
group, every rank applies them and takes one engine step, finished requests go back to rank 0 with an object gather.
Nothing here waits on a GPU: a rank that dies ends its peers' next collective through the process-group timeout.
"""
from __future__ import annotations

import argparse
import asyncio
import threading
import time
from typing import Any

import torch
import torch.distributed as dist

try:                                  # at module level: handler annotations are resolved against the module's globals
    from fastapi import Request
except Exception:                     # pragma: no cover - the control loop itself does not need FastAPI
    Request = Any


class ControlLoop:
    """The per-rank side: apply broadcast commands, step, return finished requests."""

    def __init__(self, engine, ps, mode: str, ctrl_group, idle_sleep: float = 0.002):
        self.engine, self.ps, self.mode, self.group, self.idle_sleep = engine, ps, mode, ctrl_group, idle_sleep
        self.rank, self.world = dist.get_rank(ctrl_group), dist.get_world_size(ctrl_group)
        self.inbox: list = []                       # rank 0: commands queued by the HTTP handlers
        self.inbox_lock = threading.Lock()
        self.live: dict[str, Any] = {}              # rid → Request running on this rank
        self.waiters: dict[str, Any] = {}           # rank 0: rid → callback(result dict)
        self.next_target = 0
        self.stop = False
        if engine.lockstep_group is not None:
            import gc

            engine.begin_rollout()                  # collective: peers rendezvous, first-use kernel attributes before any capture
            gc.enable()
            engine.local_done = False               # a server never declares its rollout finished
            engine.global_done = False

    # ---- rank 0 API (any thread) -----------------------------------------------------------------------------
    def submit(self, command: tuple, on_result=None):
        with self.inbox_lock:
            if command[0] == "add" and on_result is not None:
                self.waiters[command[2]] = on_result
            self.inbox.append(command)

    def pick_rank(self) -> int:
        if self.mode == "tp":
            return -1                               # every rank runs it
        self.next_target = (self.next_target + 1) % self.world
        return self.next_target

    # ---- the loop (every rank) ---------------------------------------------------------------------------------
    def _apply(self, cmd: tuple):
        e = self.engine
        kind = cmd[0]
        if kind == "add":
            _, target, rid, body = cmd
            if target in (-1, self.rank):
                self.live[rid] = e.add_request(body["input_ids"], dict(body.get("sampling_params") or {}), body.get("return_logprob", True),
                                               body.get("return_routed_experts", False), rid=rid,
                                               logprob_start_len=body.get("logprob_start_len", -1),
                                               top_logprobs_num=body.get("top_logprobs_num", 0))
        elif kind == "abort":
            e.abort_request(cmd[1])
        elif kind == "pause":
            e.pause_generation(cmd[1] if len(cmd) > 1 else "retract")
        elif kind == "continue":
            e.continue_generation()
        elif kind == "flush":
            e.flush_cache()
        elif kind == "load":
            e.update_weights_from_disk(cmd[1])
            if cmd[2] is not None:
                e.update_weight_version(int(cmd[2]))
        elif kind == "version":
            e.update_weight_version(int(cmd[1]))
        elif kind == "shutdown":
            self.stop = True

    def tick(self) -> bool:
        box = [None]
        if self.rank == 0:
            with self.inbox_lock:
                box[0], self.inbox = self.inbox, []
        dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, 0), group=self.group)
        for cmd in box[0]:
            self._apply(cmd)
        busy = self.engine.step()
        done = []
        for rid, r in list(self.live.items()):
            if r.finished:
                del self.live[rid]
                if self.mode != "tp" or self.rank == 0:
                    done.append((rid, r.to_response(self.engine)))
        gathered = [None] * self.world if self.rank == 0 else None
        dist.gather_object(done, gathered, dst=dist.get_global_rank(self.group, 0), group=self.group)
        if self.rank == 0:
            for part in gathered:
                for rid, out in part:
                    cb = self.waiters.pop(rid, None)
                    if cb is not None:
                        cb(out)
        return busy or bool(box[0])

    def run(self):
        while not self.stop:
            if not self.tick():
                time.sleep(self.idle_sleep)


def build_app(loop: ControlLoop):
    from fastapi import FastAPI
    from fastapi.responses import JSONResponse

    app = FastAPI(title="miles_b200 multi-GPU engine")
    engine = loop.engine
    counter = iter(range(1, 1 << 62))

    @app.post("/generate")
    async def generate(request: Request):
        body = await request.json()
        aio = asyncio.get_running_loop()
        fut = aio.create_future()
        rid = body.get("rid") or f"mr-{next(counter)}"
        loop.submit(("add", loop.pick_rank(), rid, body), lambda out: aio.call_soon_threadsafe(lambda: fut.done() or fut.set_result(out)))
        return JSONResponse(await fut)

    @app.get("/health")
    async def health():
        return {**engine.health(), "ranks": loop.world, "mode": loop.mode}

    @app.post("/abort_request")
    async def abort(request: Request):
        body = await request.json()
        loop.submit(("abort", None if body.get("abort_all") else body.get("rid")))
        return {"success": True}

    @app.post("/pause_generation")
    async def pause(request: Request):
        loop.submit(("pause", "retract"))
        return {"success": True}

    @app.post("/continue_generation")
    async def cont():
        loop.submit(("continue",))
        return {"success": True}

    @app.post("/flush_cache")
    async def flush():
        loop.submit(("flush",))
        return {"success": True}

    @app.post("/update_weights_from_disk")
    async def from_disk(request: Request):
        body = await request.json()
        loop.submit(("load", body["model_path"], body.get("weight_version")))
        return {"success": True}

    @app.post("/update_weight_version")
    async def set_version(request: Request):
        body = await request.json()
        loop.submit(("version", body["weight_version"]))
        return {"success": True}

    @app.get("/get_weight_version")
    async def get_version():
        return {"weight_version": str(engine.weight_version)}

    @app.post("/shutdown")
    async def shutdown():
        loop.submit(("shutdown",))
        return {"success": True}

    return app


def start(engine, ps, mode: str, host: str = "127.0.0.1", port: int = 30000, ctrl_group=None) -> ControlLoop:
    """Every rank calls this; returns after a `shutdown` command.  Rank 0 serves HTTP from a thread next to the loop."""
    ctrl_group = ctrl_group if ctrl_group is not None else dist.new_group(backend="gloo")
    loop = ControlLoop(engine, ps, mode, ctrl_group)
    server = None
    if loop.rank == 0:
        import uvicorn

        server = uvicorn.Server(uvicorn.Config(build_app(loop), host=host, port=port, log_level="warning"))
        threading.Thread(target=server.run, daemon=True, name=f"engine-http-{port}").start()
        while not server.started:
            time.sleep(0.01)
    try:
        loop.run()
    finally:
        if server is not None:
            server.should_exit = True
    return loop


def main():
    from ..models.config import get_config
    from ..parallel.state import ParallelState, init_distributed
    from .engine import Engine

    p = argparse.ArgumentParser()
    p.add_argument("--model-name", default="tiny-moe")
    p.add_argument("--hf-checkpoint", default=None)
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=30000)
    p.add_argument("--mem-fraction-static", type=float, default=0.7)
    p.add_argument("--max-running-requests", type=int, default=256)
    p.add_argument("--tensor-model-parallel-size", type=int, default=None)
    p.add_argument("--expert-model-parallel-size", type=int, default=None)
    a = p.parse_args()
    rank, world, local = init_distributed()
    cfg = get_config(a.hf_checkpoint or a.model_name)
    ep = a.expert_model_parallel_size or (world if cfg.is_moe and not a.tensor_model_parallel_size else 1)
    tp = a.tensor_model_parallel_size or (world if ep == 1 else 1)
    mode = "ep" if ep > 1 else "tp"
    ps = ParallelState.build(tp=tp, ep=ep, sequence_parallel=False)
    dev = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    if dev.type == "cuda" and (tp > 1 or ep > 1):
        from ..parallel.fabric import Fabric

        ps.fused = True
        ps.fabric = Fabric.create(ps)
    engine = Engine(cfg, ps=ps, device=dev, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32,
                    mem_fraction_static=a.mem_fraction_static, max_running_requests=a.max_running_requests, seed=0)
    if a.hf_checkpoint:
        engine.update_weights_from_disk(a.hf_checkpoint)
    start(engine, ps, mode, a.host, a.port)


if __name__ == "__main__":
    main()
