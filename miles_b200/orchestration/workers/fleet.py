"""An engine fleet behind HTTP: engine servers and a router launched, watched and restarted through the worker layer.

`launch_fleet(args, cfg)` starts `--rollout-num-engines` engine servers (one cell each, `--rollout-num-gpus-per-engine`
GPUs) and one router as supervised processes (`--worker-provider local`), or adopts servers that run elsewhere
(`--worker-provider static --rollout-engine-addrs …`, or `registration`: servers announce themselves to the hub at
`--registration-hub-port`).  It returns `RemoteEngine` handles — the engine interface the inference controller and the
weight updater use, spoken over HTTP — and a watcher thread that reconciles cells: a dead launched cell is restarted
under a new generation, re-registered with the router, and comes back with weight version 0, which the controller
treats as stale until the updater has re-sent the weights.

Reference: miles/ray/specs/inference.py:139-424 (engine + router pools, ports, launch flags),
miles/ray/controllers/inference/controller.py:36-267 (cells, reconcile), miles/backends/sglang_utils/sglang_engine.py:37-545.
"""
from __future__ import annotations

import asyncio
import sys
import threading
import time

from ..worker_spec import CommandWorkerSpec, SchedulingSpec
from .manager import WorkerManager
from .provider import CellInfo, CompositeProvider, LocalProcessProvider, StaticWorkerProvider
from .reconcile import LookAgain
from .registration import RegistrationHub


class RemoteEngine:
    """The engine's control surface over HTTP (see `engine/server.py` for the endpoints)."""

    def __init__(self, url: str, name: str = "", generation: int = 0, timeout: float = 600.0):
        self.url, self.name, self.generation, self.timeout = url.rstrip("/"), name or url, generation, timeout

    def _post(self, path: str, body: dict | None = None):
        import requests

        r = requests.post(f"{self.url}/{path}", json=body or {}, timeout=self.timeout)
        r.raise_for_status()
        return r.json() if "json" in r.headers.get("content-type", "") else r.text

    def _get(self, path: str, timeout: float | None = None):
        import requests

        r = requests.get(f"{self.url}/{path}", timeout=timeout or self.timeout)
        r.raise_for_status()
        return r.json() if "json" in r.headers.get("content-type", "") else r.text

    def health(self) -> dict:
        try:
            out = self._get("health", timeout=2.0)
            return out if isinstance(out, dict) else {"status": "ok"}
        except Exception as e:  # unreachable counts as unhealthy
            return {"status": "down", "error": str(e)}

    def pause_generation(self, mode: str = "retract"):
        return self._post("pause_generation", {"mode": mode})

    def continue_generation(self):
        return self._post("continue_generation")

    def flush_cache(self):
        try:
            return self._post("flush_cache")
        except Exception:
            return None                                  # servers without the endpoint flush on weight update

    def update_weights_from_tensor(self, named, weight_version=None, load_format=None):
        """A bucket of HF-named tensors: device tensors go as ONE CUDA-IPC handle (the server maps the trainer's buffer and
        copies device to device), host tensors as bytes."""
        from ...weight_update import cuda_ipc

        named = list(named)
        if named and named[0][1].is_cuda:
            need = sum((t.numel() * t.element_size() + cuda_ipc.ALIGN - 1) // cuda_ipc.ALIGN * cuda_ipc.ALIGN for _, t in named)
            st = getattr(self, "_staging", None)
            if st is None or st.numel() < need:
                self._staging = st = torch_empty_u8(need, named[0][1].device)
        else:
            st = None
        return cuda_ipc.send_bucket(lambda body: self._post("update_weights_from_tensor", body), named,
                                    weight_version=weight_version, staging=st)

    def update_weights_from_disk(self, path: str):
        return self._post("update_weights_from_disk", {"model_path": path})

    def update_weight_version(self, version: int):
        return self._post("update_weight_version", {"weight_version": int(version)})

    def get_weight_version(self) -> int:
        out = self._get("get_weight_version")
        return int(out.get("weight_version", 0)) if isinstance(out, dict) else int(out)

    def release_memory_occupation(self, tags=None):
        return self._post("release_memory_occupation", {"tags": list(tags or [])})

    def resume_memory_occupation(self, tags=None):
        return self._post("resume_memory_occupation", {"tags": list(tags or [])})

    def get_server_info(self) -> dict:
        return self._get("get_server_info")


class Fleet:
    def __init__(self, manager, provider, hub, engines: dict, router_url: str | None, on_restart=None, watch_interval: float = 1.0):
        self.manager, self.provider, self.hub = manager, provider, hub
        self.engines: dict[str, RemoteEngine] = engines            # cell id → handle
        self.router_url = router_url
        self.on_restart = on_restart
        self.watch_interval = watch_interval
        self.events: list[tuple] = []
        self._thread = None
        self._loop = None
        self._stop = None

    # ---- reconcile -----------------------------------------------------------------------------------------------
    async def _reconcile(self, cell_id: str, info: CellInfo | None):
        if info is None or info.pool != "engine":
            return
        eng = self.engines.get(cell_id)
        if eng is None and info.alive:                               # a newly registered external engine
            w = info.workers[0]
            eng = self.engines[cell_id] = RemoteEngine(w.url(), w.name, info.generation)
            self._router("add_worker", eng.url)
            self.events.append(("adopted", cell_id, info.generation))
            return
        if not info.alive and self.manager is not None and cell_id in self.manager.cells:
            self.events.append(("dead", cell_id, info.generation))
            new = await asyncio.get_running_loop().run_in_executor(None, self.manager.restart_cell, cell_id)
            w = new.workers[0]
            await asyncio.get_running_loop().run_in_executor(None, wait_healthy, w.url(), 180.0)
            eng.url, eng.generation = w.url(), new.generation
            self._router("add_worker", eng.url)
            self.events.append(("restarted", cell_id, new.generation))
            if self.on_restart is not None:
                self.on_restart(eng)
            raise LookAgain()                                         # the next poll reconciles the restarted cell

    def _router(self, endpoint: str, url: str):
        if not self.router_url:
            return
        import requests

        try:
            requests.post(f"{self.router_url}/{endpoint}", params={"url": url}, json={"url": url}, timeout=5)
        except Exception:
            pass

    def start_watch(self):
        ready = threading.Event()

        def run():
            self._loop = asyncio.new_event_loop()
            asyncio.set_event_loop(self._loop)

            async def main():
                stop = await self.provider.watch_cells(self._reconcile_quiet, interval=self.watch_interval)
                self._stop = asyncio.Event()
                ready.set()
                await self._stop.wait()
                await stop()

            self._loop.run_until_complete(main())

        self._thread = threading.Thread(target=run, name="fleet-watch", daemon=True)
        self._thread.start()
        ready.wait(30)

    async def _reconcile_quiet(self, cell_id, info):
        try:
            await self._reconcile(cell_id, info)
        except LookAgain:
            raise
        except Exception as e:
            self.events.append(("error", cell_id, str(e)))

    def shutdown(self):
        if self._loop is not None and self._stop is not None:
            self._loop.call_soon_threadsafe(self._stop.set)
            self._thread.join(10)
        if self.manager is not None:
            self.manager.stop_all()


def torch_empty_u8(n: int, device):
    import torch

    return torch.empty(n, dtype=torch.uint8, device=device)


def wait_healthy(url: str, timeout: float = 180.0, alive=None):
    """Poll `url`/health; `alive()` (optional) says whether the process behind it still runs — a worker that died at start-up
    fails the wait at once instead of after the timeout."""
    import requests

    end = time.monotonic() + timeout
    last = None
    while time.monotonic() < end:
        if alive is not None and not alive():
            raise RuntimeError(f"the worker behind {url} exited before it became healthy")
        try:
            if requests.get(f"{url}/health", timeout=2).status_code == 200:
                return
        except Exception as e:
            last = e
        time.sleep(0.25)
    raise TimeoutError(f"{url} did not become healthy in {timeout:.0f}s ({last})")


def engine_spec(args, n: int) -> CommandWorkerSpec:
    ek = dict(getattr(args, "engine_kwargs", {}) or {})
    per = int(getattr(args, "rollout_num_gpus_per_engine", 1) or 1)
    module = "miles_b200.engine.multi_rank_server" if per > 1 else "miles_b200.engine.server"
    cmd = [sys.executable, "-m", module, "--port", "{port}", "--host", "127.0.0.1",
           "--mem-fraction-static", str(ek.get("mem_fraction_static", 0.7)),
           "--max-running-requests", str(ek.get("max_running_requests", 256))]
    if getattr(args, "hf_checkpoint", None):
        cmd += ["--hf-checkpoint", args.hf_checkpoint]
    else:
        cmd += ["--model-name", args.model_name]
    if per > 1:
        # one engine over `per` GPUs: a cell of `per` ranks (rendezvous variables from the planner), rank 0 owns the HTTP port;
        # experts are sharded for MoE models, projections for dense ones (`engine/multi_rank_server.py`)
        cpu = getattr(args, "fp32", False)
        return CommandWorkerSpec("engine", cmd, SchedulingSpec(num_cells=n, workers_per_cell=per, gpus_per_worker=0 if cpu else 1),
                                 env={"CUDA_VISIBLE_DEVICES": "" if cpu else "__inherit__"})
    if getattr(args, "fp32", False):
        cmd += ["--device", "cpu"]
        return CommandWorkerSpec("engine", cmd, SchedulingSpec(num_cells=n, workers_per_cell=1, gpus_per_worker=0))
    # every GPU stays visible to the server and it is told which one is its own: device indices then mean the same in the
    # trainer and in the engine, which is what CUDA-IPC weight buckets rely on
    cmd += ["--device", "cuda:{gpu_ids}"]
    return CommandWorkerSpec("engine", cmd, SchedulingSpec(num_cells=n, workers_per_cell=1, gpus_per_worker=1.0),
                             env={"CUDA_VISIBLE_DEVICES": "__inherit__"})


def router_spec(args) -> CommandWorkerSpec:
    cmd = [sys.executable, "-m", "miles_b200.router.router", "--port", "{port}", "--policy", getattr(args, "router_policy", "least_active")]
    return CommandWorkerSpec("router", cmd, SchedulingSpec(1, 1, 0))


def launch_fleet(args, log_dir: str | None = None, on_restart=None) -> Fleet:
    kind = getattr(args, "worker_provider", "local")
    manager, hub, providers, engines = None, None, [], {}
    router_url = (getattr(args, "engine_kwargs", {}) or {}).get("router_url")
    if kind == "local":
        manager = WorkerManager(log_dir=log_dir)
        specs = [engine_spec(args, int(getattr(args, "rollout_num_engines", 1) or 1))]
        if not router_url:
            specs.append(router_spec(args))
        # colocated: engines share the trainer's GPUs (slot i ↔ rank i); disaggregated: they take the GPUs after the trainer's
        trainer_gpus = 0 if getattr(args, "colocate", False) or getattr(args, "fp32", False) else \
            int(getattr(args, "actor_num_nodes", 1) or 1) * int(getattr(args, "actor_num_gpus_per_node", 1) or 1)
        manager.launch(specs, colocate=True, first_slot=trainer_gpus)
        cells = manager.get_cell_infos()
        for cid, c in cells.items():
            try:
                wait_healthy(c.workers[0].url(), 300.0, alive=lambda cid=cid: manager.cells[cid].alive())
            except Exception as e:
                tail = manager.log_tail(c.workers[0].name, 30)
                manager.stop_all()
                raise RuntimeError(f"{cid} did not start: {e}\n{tail}") from e
            if c.pool == "engine":
                engines[cid] = RemoteEngine(c.workers[0].url(), c.workers[0].name, c.generation)
            elif c.pool == "router":
                router_url = c.workers[0].url()
        providers.append(LocalProcessProvider(manager))
    elif kind == "static":
        addrs = list(getattr(args, "rollout_engine_addrs", None) or [])
        assert addrs, "--worker-provider static needs --rollout-engine-addrs host:port …"
        sp = StaticWorkerProvider("engine", addrs)
        for w in sp.workers:
            wait_healthy(w.url(), 300.0)
            engines[w.cell_id] = RemoteEngine(w.url(), w.name, 0)
        providers.append(sp)
        assert router_url, "--worker-provider static needs --router-url (or one engine address used directly)"
    elif kind == "kubernetes":
        from .kubernetes import KubernetesWorkerProvider

        kp = KubernetesWorkerProvider("engine", getattr(args, "k8s_selector", None) or "app=miles-engine",
                                      namespace=getattr(args, "k8s_namespace", None), kubectl=getattr(args, "k8s_kubectl", None) or "kubectl")
        for cid, c in asyncio.run(kp.list_cells()).items():          # pods are launched by the cluster's own tooling: adopt what runs
            if c.alive and c.pool == "engine":
                wait_healthy(c.workers[0].url(), 300.0)
                engines[cid] = RemoteEngine(c.workers[0].url(), c.workers[0].name, c.generation)
        providers.append(kp)
        assert router_url or engines, "--worker-provider kubernetes found no ready engine pod and no --engine-router-url was given"
    if kind == "registration" or getattr(args, "registration_hub_port", None):
        hub = RegistrationHub(ttl=float(getattr(args, "registration_ttl", 30.0) or 30.0))
        hub.serve(port=int(getattr(args, "registration_hub_port", None) or 30200))
        providers.append(hub)
    fleet = Fleet(manager, CompositeProvider(providers), hub, engines, router_url, on_restart=on_restart)
    for e in engines.values():
        fleet._router("add_worker", e.url)
    fleet.start_watch()
    return fleet
