"""Kubernetes worker provider: cells are pods found by label, read through `kubectl`.

The reference places serving and training workers on a Kubernetes cluster through a provider that lists pods and turns
them into cells (miles/utils/workers/worker_provider/: the K8s flavour next to the Ray and static ones).  This provider
needs no client library: it runs `kubectl get pods -l <selector> -o json` (any command that prints the same JSON will do —
a kubeconfig-aware wrapper, `oc`, a test double) and maps the pod list to `CellInfo`:

  pool        label `miles/pool` (default: the provider's pool name)
  cell        label `miles/cell` (an integer; pods without it are single-worker cells numbered by name order)
  worker      label `miles/worker` (index within the cell, default 0)
  generation  label `miles/generation`, else the pod's restart count
  address     `status.podIP` and the container port named by `port_name` (default "http"), else the first port
  alive       every pod of the cell is `Running` with all containers ready

Launching and deleting pods stays with the cluster's own tooling (a Deployment / StatefulSet / the Helm chart in `charts/`);
the fleet watcher adopts the cells it is shown and routes around the ones that are not alive.
"""
from __future__ import annotations

import asyncio
import json
import shlex

from .provider import BaseWorkerProvider, CellInfo, WorkerInfo, cell_name, worker_name


class KubernetesWorkerProvider(BaseWorkerProvider):
    def __init__(self, pool: str, selector: str, namespace: str | None = None, kubectl: str | list[str] = "kubectl",
                 port_name: str = "http", timeout: float = 20.0):
        self.pool, self.selector, self.namespace, self.port_name, self.timeout = pool, selector, namespace, port_name, timeout
        self.kubectl = shlex.split(kubectl) if isinstance(kubectl, str) else list(kubectl)

    def _command(self) -> list[str]:
        cmd = [*self.kubectl, "get", "pods", "-l", self.selector, "-o", "json"]
        if self.namespace:
            cmd += ["-n", self.namespace]
        return cmd

    async def _pods(self) -> list[dict]:
        proc = await asyncio.create_subprocess_exec(*self._command(), stdout=asyncio.subprocess.PIPE, stderr=asyncio.subprocess.PIPE)
        try:
            out, err = await asyncio.wait_for(proc.communicate(), self.timeout)
        except asyncio.TimeoutError:
            proc.kill()
            raise RuntimeError(f"{' '.join(self._command())} did not answer in {self.timeout:.0f} s")
        if proc.returncode != 0:
            raise RuntimeError(f"{' '.join(self._command())} failed ({proc.returncode}): {err.decode(errors='replace')[-300:]}")
        return list(json.loads(out.decode()).get("items", []))

    def _port(self, pod: dict) -> int | None:
        first = None
        for c in pod.get("spec", {}).get("containers", []):
            for p in c.get("ports", []) or []:
                first = first if first is not None else p.get("containerPort")
                if p.get("name") == self.port_name:
                    return int(p["containerPort"])
        return int(first) if first is not None else None

    @staticmethod
    def _ready(pod: dict) -> bool:
        st = pod.get("status", {})
        cs = st.get("containerStatuses") or []
        return st.get("phase") == "Running" and bool(cs) and all(c.get("ready") for c in cs) \
            and not pod.get("metadata", {}).get("deletionTimestamp")

    async def list_cells(self) -> dict[str, CellInfo]:
        pods = sorted(await self._pods(), key=lambda p: p.get("metadata", {}).get("name", ""))
        cells: dict[str, list] = {}
        auto = 0
        for pod in pods:
            meta, st = pod.get("metadata", {}), pod.get("status", {})
            labels = meta.get("labels", {}) or {}
            pool = labels.get("miles/pool", self.pool)
            if "miles/cell" in labels:
                cell = int(labels["miles/cell"])
            else:
                cell, auto = auto, auto + 1
            index = int(labels.get("miles/worker", 0))
            restarts = sum(int(c.get("restartCount", 0)) for c in st.get("containerStatuses") or [])
            gen = int(labels.get("miles/generation", restarts))
            port = self._port(pod)
            info = WorkerInfo(worker_name(pool, cell, index), pool, cell_name(pool, cell), index, gen, st.get("podIP") or "",
                              (("port", port),) if port is not None else ())
            cells.setdefault(cell_name(pool, cell), []).append((info, self._ready(pod) and bool(st.get("podIP")), pool, gen))
        out = {}
        for cid, ws in cells.items():
            ws.sort(key=lambda t: t[0].index)
            out[cid] = CellInfo(cid, ws[0][2], max(t[3] for t in ws), all(t[1] for t in ws), tuple(t[0] for t in ws))
        return out
