"""HTTP surface of the Tinker-style training service (paths follow miles/tinker/server/app.py:58-178).

Training calls are asynchronous in the API: they return `{"request_id": …}` at once and the result is fetched with
`POST /api/v1/retrieve_future`.  One worker task executes the queued operations in arrival order, so calls of all
tenants interleave at batch granularity on the shared base model.
"""
from __future__ import annotations

import asyncio

from fastapi import FastAPI, HTTPException
from fastapi import Request as _Request   # module level: postponed annotations are resolved in module scope

from .service import TinkerService


def build_app(svc: TinkerService):
    app = FastAPI(title="miles_b200 tinker gateway")
    sessions: dict[str, dict] = {}
    exec_lock = asyncio.Lock()

    async def run(fn, *a, **kw) -> dict:
        async with exec_lock:                                   # the base model runs one operation at a time
            fid = await asyncio.get_running_loop().run_in_executor(None, lambda: svc.submit(fn, *a, **kw))
        return {"request_id": fid}

    @app.get("/api/v1/healthz")
    async def healthz():
        return {"status": "ok"}

    @app.api_route("/api/v1/get_server_capabilities", methods=["GET", "POST"])
    async def caps():
        return svc.capabilities()

    @app.post("/api/v1/create_session")
    async def create_session(request: _Request):
        body = await request.json() if await request.body() else {}
        sid = f"sess-{len(sessions)}"
        sessions[sid] = {"tags": body.get("tags", []), "models": []}
        return {"session_id": sid}

    @app.post("/api/v1/session_heartbeat")
    async def heartbeat(request: _Request):
        return {"ok": True}

    @app.post("/api/v1/create_model")
    async def create_model(request: _Request):
        body = await request.json()
        try:
            m = svc.create_model(body.get("model_id"), (body.get("lora_config") or {}).get("rank"), body.get("seed", 0))
        except (RuntimeError, ValueError) as e:
            raise HTTPException(409, str(e))
        if body.get("session_id") in sessions:
            sessions[body["session_id"]]["models"].append(m.model_id)
        return {"model_id": m.model_id, "lora_rank": m.rank}

    @app.post("/api/v1/unload_model")
    async def unload(request: _Request):
        body = await request.json()
        svc.unload_model(body["model_id"])
        return {"unloaded": body["model_id"]}

    @app.post("/api/v1/get_info")
    async def info(request: _Request):
        body = await request.json()
        m = svc.models.get(body["model_id"])
        if m is None:
            raise HTTPException(404, "unknown model")
        return {"model_id": m.model_id, "lora_rank": m.rank, "steps": m.steps, "slot": m.slot}

    @app.post("/api/v1/forward_backward")
    async def forward_backward(request: _Request):
        b = await request.json()
        fb = b.get("forward_backward_input", b)
        return await run(svc.forward_backward, b["model_id"], fb["data"], fb.get("loss_fn", "cross_entropy"), fb.get("loss_fn_config"))

    @app.post("/api/v1/forward")
    async def forward(request: _Request):
        b = await request.json()
        fb = b.get("forward_input", b)
        return await run(svc.forward, b["model_id"], fb["data"], fb.get("loss_fn", "cross_entropy"), fb.get("loss_fn_config"))

    @app.post("/api/v1/optim_step")
    async def optim_step(request: _Request):
        b = await request.json()
        return await run(svc.optim_step, b["model_id"], b.get("adam_params"))

    @app.post("/api/v1/save_weights")
    async def save_weights(request: _Request):
        b = await request.json()
        return await run(svc.save_weights, b["model_id"], b["path"], b.get("export_peft", False))

    @app.post("/api/v1/load_weights")
    async def load_weights(request: _Request):
        b = await request.json()
        return await run(svc.load_weights, b["model_id"], b["path"], b.get("with_optimizer", True))

    @app.post("/api/v1/asample")
    async def asample(request: _Request):
        b = await request.json()
        prompt = b.get("prompt", {})
        tokens = prompt.get("tokens") or [t for ch in prompt.get("chunks", []) for t in ch.get("tokens", [])]
        return await run(svc.sample, b.get("model_id"), tokens, b.get("sampling_params"), b.get("num_samples", 1))

    @app.post("/api/v1/retrieve_future")
    async def retrieve(request: _Request):
        b = await request.json()
        r = svc.retrieve(b["request_id"])
        if r["status"] == "unknown":
            raise HTTPException(404, "unknown request_id")
        if r["status"] == "error":
            return {"type": "RequestFailedResponse", "error": r["error"]}
        return r["result"]

    return app
