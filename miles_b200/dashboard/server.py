"""Run dashboard: metric collector, GPU sampler, engine scraper, a small store and a web page.

Reference: miles/dashboard/* — a collector actor that receives every `Tracker.log` call, a GPU sampler (NVML), a
scraper of the engines' `/metrics`, a columnar store and a FastAPI server with a static JS front-end.  Here the
collector is a tracking backend (`DashboardBackend`, add it with `Tracker.add_backend`), the store keeps one time
series per metric in memory (optionally mirrored to JSONL), the GPU sampler only *reads* NVML (utilisation, memory,
clocks, power, throttle reasons — it changes no device setting), and the page is a single self-contained HTML file
that polls `/api/series`.

    python -m miles_b200.dashboard.server --jsonl runs/metrics.jsonl --port 8265
"""
from __future__ import annotations

import json
import threading
import time
from collections import defaultdict

from fastapi import FastAPI
from fastapi.responses import HTMLResponse


class SeriesStore:
    def __init__(self, max_points: int = 20000, jsonl: str | None = None):
        self.series: dict[str, list[tuple[float, float]]] = defaultdict(list)
        self.max_points, self.jsonl = max_points, jsonl
        self.lock = threading.Lock()

    def add(self, name: str, x: float, y: float):
        with self.lock:
            s = self.series[name]
            s.append((float(x), float(y)))
            if len(s) > self.max_points:
                del s[: len(s) - self.max_points]

    def add_many(self, metrics: dict, x: float):
        for k, v in metrics.items():
            if isinstance(v, (int, float)):
                self.add(k, x, v)
        if self.jsonl:
            with open(self.jsonl, "a") as f:
                f.write(json.dumps({"x": x, **{k: v for k, v in metrics.items() if isinstance(v, (int, float))}}) + "\n")

    def names(self, prefix: str = "") -> list[str]:
        with self.lock:
            return sorted(n for n in self.series if n.startswith(prefix))

    def get(self, name: str, last: int | None = None) -> list[tuple[float, float]]:
        with self.lock:
            s = self.series.get(name, [])
            return list(s[-last:] if last else s)

    def load_jsonl(self, path: str):
        with open(path) as f:
            for line in f:
                if line.strip():
                    row = json.loads(line)
                    x = row.pop("x", row.pop("rollout/step", 0))
                    for k, v in row.items():
                        if isinstance(v, (int, float)):
                            self.add(k, x, v)


class DashboardBackend:
    """Tracking backend: `Tracker.add_backend(DashboardBackend(store))`."""

    def __init__(self, store: SeriesStore):
        self.store = store

    def log(self, metrics, step, step_key):
        self.store.add_many(metrics, step)

    def finish(self):
        pass


class GpuSampler:
    """Reads NVML every `interval_s` seconds into `gpu{i}/…` series.  Read-only: no clocks, limits or modes are set."""

    FIELDS = ("util", "mem_used_gb", "sm_mhz", "power_w", "throttle_reasons")

    def __init__(self, store: SeriesStore, interval_s: float = 2.0, nvml=None):
        self.store, self.interval_s = store, interval_s
        self.nvml = nvml
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def _nvml(self):
        if self.nvml is None:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
        return self.nvml

    def sample_once(self) -> dict:
        n = self._nvml()
        out, t = {}, time.time()
        for i in range(n.nvmlDeviceGetCount()):
            h = n.nvmlDeviceGetHandleByIndex(i)
            vals = {"util": n.nvmlDeviceGetUtilizationRates(h).gpu, "mem_used_gb": n.nvmlDeviceGetMemoryInfo(h).used / 2 ** 30,
                    "sm_mhz": n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM), "power_w": n.nvmlDeviceGetPowerUsage(h) / 1000.0,
                    "throttle_reasons": n.nvmlDeviceGetCurrentClocksThrottleReasons(h)}
            for k, v in vals.items():
                self.store.add(f"gpu{i}/{k}", t, v)
                out[f"gpu{i}/{k}"] = v
        return out

    def start(self):
        def loop():
            while not self._stop.wait(self.interval_s):
                try:
                    self.sample_once()
                except Exception:
                    return                      # no NVML on this host: the sampler just stops

        self._thread = threading.Thread(target=loop, daemon=True, name="gpu-sampler")
        self._thread.start()

    def stop(self):
        self._stop.set()


def scrape_prometheus(text: str) -> dict[str, float]:
    """Parse an engine's `/metrics` text exposition into {name: value} (labels folded into the name)."""
    out = {}
    for line in text.splitlines():
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        name, _, val = line.rpartition(" ")
        try:
            out[name] = float(val)
        except ValueError:
            continue
    return out


PAGE = """<!doctype html><html><head><meta charset="utf-8"><title>miles_b200</title>
<style>body{font:13px system-ui;margin:16px;background:#111;color:#ddd}canvas{background:#1b1b1b;margin:6px;border-radius:4px}
input{background:#222;color:#ddd;border:1px solid #444;padding:4px;width:320px}.t{display:inline-block;text-align:center}</style></head>
<body><h3>miles_b200 run dashboard</h3><input id="f" placeholder="filter (prefix), e.g. train/ or perf/"><div id="g"></div>
<script>
async function draw(){const p=document.getElementById('f').value;const names=await (await fetch('/api/names?prefix='+encodeURIComponent(p))).json();
const g=document.getElementById('g');g.innerHTML='';for(const n of names.slice(0,48)){const d=await (await fetch('/api/series?name='+encodeURIComponent(n)+'&last=500')).json();
const w=document.createElement('div');w.className='t';const c=document.createElement('canvas');c.width=300;c.height=120;w.appendChild(c);
w.appendChild(document.createElement('br'));w.appendChild(document.createTextNode(n+(d.length?' = '+d[d.length-1][1].toPrecision(5):'')));g.appendChild(w);
if(!d.length)continue;const x=c.getContext('2d');const ys=d.map(e=>e[1]);const lo=Math.min(...ys),hi=Math.max(...ys);x.strokeStyle='#6cf';x.beginPath();
d.forEach((e,i)=>{const X=i/(d.length-1||1)*290+5,Y=110-(hi>lo?(e[1]-lo)/(hi-lo):.5)*100;i?x.lineTo(X,Y):x.moveTo(X,Y)});x.stroke();}}
draw();setInterval(draw,5000);document.getElementById('f').onchange=draw;</script></body></html>"""


def build_app(store: SeriesStore):
    app = FastAPI(title="miles_b200 dashboard")

    @app.get("/", response_class=HTMLResponse)
    async def index():
        return PAGE

    @app.get("/api/names")
    async def names(prefix: str = ""):
        return store.names(prefix)

    @app.get("/api/series")
    async def series(name: str, last: int | None = None):
        return store.get(name, last)

    @app.post("/api/log")
    async def log(body: dict):
        store.add_many(body.get("metrics", {}), body.get("step", time.time()))
        return {"ok": True}

    return app


def main():
    import argparse

    import uvicorn

    p = argparse.ArgumentParser()
    p.add_argument("--jsonl", default=None, help="metrics file written by --jsonl-metrics-path to load at start")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8265)
    p.add_argument("--gpu-interval", type=float, default=2.0)
    a = p.parse_args()
    store = SeriesStore()
    if a.jsonl:
        store.load_jsonl(a.jsonl)
    GpuSampler(store, a.gpu_interval).start()
    uvicorn.run(build_app(store), host=a.host, port=a.port, log_level="warning")


if __name__ == "__main__":
    main()
