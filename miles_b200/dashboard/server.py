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
input,select{background:#222;color:#ddd;border:1px solid #444;padding:4px}.t{display:inline-block;text-align:center}
nav a{margin-right:14px;color:#6cf;cursor:pointer}nav a.on{color:#fff;font-weight:600}table{border-collapse:collapse}
td,th{border-bottom:1px solid #333;padding:3px 8px;text-align:right}.alarm{color:#f66}.warn{color:#fc6}.info{color:#9c9}
.tok{display:inline-block;padding:1px 2px;margin:1px;border-radius:2px;background:#222}.tok.r{background:#234}.tok.m{opacity:.45}</style></head>
<body><h3>miles_b200 run dashboard</h3><nav><a id="n-metrics" class="on">metrics</a><a id="n-timeline">timeline</a><a id="n-advice">advisories</a><a id="n-samples">samples</a></nav>
<div id="metrics"><input id="f" style="width:320px" placeholder="filter (prefix), e.g. train/ or perf/"><div id="g"></div></div>
<div id="timeline" hidden><canvas id="tl" width="1200" height="400"></canvas><pre id="util"></pre></div>
<div id="advice" hidden></div>
<div id="samples" hidden>rollout <select id="rid"></select> <span id="sum"></span><table id="tab"></table><div id="tv"></div></div>
<script>
const J=async u=>(await fetch(u)).json();const $=i=>document.getElementById(i);
for(const t of ['metrics','timeline','advice','samples'])$('n-'+t).onclick=()=>{for(const u of ['metrics','timeline','advice','samples']){$(u).hidden=u!=t;$('n-'+u).className=u==t?'on':''}show[t]()};
const COL={};const color=n=>COL[n]||(COL[n]='hsl('+(Object.keys(COL).length*67%360)+',60%,55%)');
const show={async metrics(){const p=$('f').value;const names=await J('/api/names?prefix='+encodeURIComponent(p));const g=$('g');g.innerHTML='';
for(const n of names.slice(0,48)){const d=await J('/api/series?name='+encodeURIComponent(n)+'&last=500');const w=document.createElement('div');w.className='t';
const c=document.createElement('canvas');c.width=300;c.height=120;w.appendChild(c);w.appendChild(document.createElement('br'));
w.appendChild(document.createTextNode(n+(d.length?' = '+d[d.length-1][1].toPrecision(5):'')));g.appendChild(w);if(!d.length)continue;
const x=c.getContext('2d');const ys=d.map(e=>e[1]);const lo=Math.min(...ys),hi=Math.max(...ys);x.strokeStyle='#6cf';x.beginPath();
d.forEach((e,i)=>{const X=i/(d.length-1||1)*290+5,Y=110-(hi>lo?(e[1]-lo)/(hi-lo):.5)*100;i?x.lineTo(X,Y):x.moveTo(X,Y)});x.stroke();}},
async timeline(){const d=await J('/api/phases');const c=$('tl'),x=c.getContext('2d');x.clearRect(0,0,c.width,c.height);const L=Object.keys(d.lanes);
if(!L.length){x.fillStyle='#888';x.fillText('no phase records (run with --use-miles-dashboard --dump-details DIR)',20,30);return}
c.height=Math.max(120,L.length*26+50);const W=c.width-140,span=Math.max(d.t1-d.t0,1e-9);L.forEach((l,i)=>{x.fillStyle='#aaa';x.fillText(l,4,i*26+22);
for(const r of d.lanes[l]){x.fillStyle=color(r.phase);x.fillRect(130+(r.start-d.t0)/span*W,i*26+8,Math.max(1,(r.end-r.start)/span*W),18)}});
let k=0;for(const n in COL){x.fillStyle=COL[n];x.fillRect(130+k*120,L.length*26+20,10,10);x.fillStyle='#ccc';x.fillText(n,144+k*120,L.length*26+29);k++}
$('util').textContent=JSON.stringify(d.utilisation,null,1)},
async advice(){const a=await J('/api/advisories');$('advice').innerHTML=a.length?a.map(r=>'<p class="'+r.severity+'"><b>['+r.severity+'] '+r.title+'</b><br>'+r.detail+'<br><i>'+r.hint+'</i></p>').join(''):'<p>nothing to report</p>'},
async samples(){const ids=await J('/api/rollouts');const s=$('rid');if(!s.options.length){s.innerHTML=ids.map(i=>'<option>'+i+'</option>').join('');s.onchange=show.samples}
if(!ids.length){$('sum').textContent='no rollout dumps (run with --dump-details DIR)';return}const id=s.value||ids[ids.length-1];const d=await J('/api/rollout/'+id);
$('sum').textContent=JSON.stringify(d.summary);$('tab').innerHTML='<tr><th>group</th><th>sample</th><th>prompt</th><th>response</th><th>reward</th><th>status</th><th>mean logp</th></tr>'+
d.samples.map(r=>'<tr data-g="'+r.group+'" data-s="'+r.sample+'"><td>'+r.group+'</td><td>'+r.sample+'</td><td>'+r.prompt_tokens+'</td><td>'+r.response_tokens+'</td><td>'+r.reward+'</td><td>'+r.status+'</td><td>'+(r.mean_logprob==null?'':r.mean_logprob.toFixed(3))+'</td></tr>').join('');
for(const tr of $('tab').querySelectorAll('tr[data-g]'))tr.onclick=async()=>{const v=await J('/api/sample/'+id+'/'+tr.dataset.g+'/'+tr.dataset.s);
$('tv').innerHTML='<p>reward '+v.reward+' · '+v.status+'</p>'+v.tokens.map(t=>'<span class="tok '+(t.part=='response'?'r':'')+(t.trained===false?' m':'')+'" title="'+t.pos+(t.rollout_log_prob!=null?' logp '+t.rollout_log_prob.toFixed(3):'')+'">'+t.text.replace(/</g,'&lt;')+'</span>').join('')}}};
show.metrics();setInterval(()=>{if(!$('metrics').hidden)show.metrics()},5000);$('f').onchange=show.metrics;</script></body></html>"""


def build_app(store: SeriesStore, dump_dir: str | None = None, tokenizer=None):
    from . import advisory, phases
    from .dump_reader import DumpReader

    app = FastAPI(title="miles_b200 dashboard")
    reader = DumpReader(dump_dir, tokenizer) if dump_dir else None

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

    @app.get("/api/phases")
    async def phase_rows():
        rows = phases.read_phases(dump_dir) if dump_dir else []
        return {"lanes": phases.lanes(rows), "utilisation": phases.utilisation(rows),
                "t0": min((r["start"] for r in rows), default=0.0), "t1": max((r["end"] for r in rows), default=0.0)}

    @app.get("/api/advisories")
    async def advisories(min_gap_s: float = 60.0):
        return advisory.compute_advisories(store, phases.read_phases(dump_dir) if dump_dir else [], min_gap_s)

    @app.get("/api/rollouts")
    async def rollouts():
        return reader.rollout_ids() if reader else []

    @app.get("/api/rollout/{rollout_id}")
    async def rollout(rollout_id: int):
        return {"summary": reader.summary(rollout_id), "samples": reader.samples(rollout_id)}

    @app.get("/api/sample/{rollout_id}/{group}/{sample}")
    async def sample(rollout_id: int, group: int, sample: int):
        return reader.token_view(rollout_id, group, sample)

    return app


def main():
    import argparse

    import uvicorn

    p = argparse.ArgumentParser()
    p.add_argument("--jsonl", default=None, help="metrics file written by --jsonl-metrics-path to load at start")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8265)
    p.add_argument("--gpu-interval", type=float, default=2.0)
    p.add_argument("--dump-details", default=None, help="directory given to the run's --dump-details: phase lanes, rollout dumps, metrics")
    a = p.parse_args()
    store = SeriesStore()
    import os

    if a.dump_details and not a.jsonl and os.path.exists(os.path.join(a.dump_details, "dashboard", "metrics.jsonl")):
        a.jsonl = os.path.join(a.dump_details, "dashboard", "metrics.jsonl")
    if a.jsonl:
        store.load_jsonl(a.jsonl)
    GpuSampler(store, a.gpu_interval).start()
    uvicorn.run(build_app(store, a.dump_details), host=a.host, port=a.port, log_level="warning")


if __name__ == "__main__":
    main()
