"""HTTP front-end of the rollout engine.

Endpoint names and payloads follow the server the reference drives over HTTP
(miles/backends/sglang_utils/sglang_api_client.py:58-460): `/generate`, `/health`, `/health_generate`, `/flush_cache`,
`/pause_generation`, `/continue_generation`, `/abort_request`, `/begin_weight_update`, `/end_weight_update`,
`/update_weights_from_tensor`, `/update_weights_from_disk`, `/update_weight_version`, `/get_weight_version`,
`/release_memory_occupation`, `/resume_memory_occupation`, `/weights_checker`, `/get_server_info`, `/metrics`,
`/start_profile`, `/stop_profile`, `/v1/chat/completions` (needs a tokenizer).

    python -m miles_b200.engine.server --model-name qwen3-0.6B --port 30000 [--hf-checkpoint DIR]
"""
from __future__ import annotations

import argparse
import asyncio
import base64
import hashlib
import io
import threading
import time
from typing import Any

import torch
from fastapi import FastAPI, Request   # module level: postponed annotations are resolved in module scope
from fastapi.responses import JSONResponse, PlainTextResponse


def build_app(engine, tokenizer=None):

    app = FastAPI(title="miles_b200 engine")
    state = {"updating": False, "profile": None, "started": time.time()}
    engine.start_loop()

    async def _wait(req) -> dict:
        loop = asyncio.get_running_loop()
        fut = loop.create_future()

        def done(r):
            loop.call_soon_threadsafe(lambda: fut.done() or fut.set_result(r))

        req.on_done = done
        if req.done.is_set():
            return req.to_response(engine)
        return (await fut).to_response(engine)

    @app.post("/generate")
    async def generate(request: Request):
        body = await request.json()
        ids = body.get("input_ids")
        if ids is None:
            assert tokenizer is not None, "text prompts need a tokenizer"
            ids = tokenizer(body["text"], add_special_tokens=False)["input_ids"]
        batched = bool(ids) and isinstance(ids[0], list)
        batch = ids if batched else [ids]
        sp = body.get("sampling_params") or {}
        sps = sp if isinstance(sp, list) else [sp] * len(batch)
        reqs = [engine.add_request(i, dict(s), body.get("return_logprob", False), body.get("return_routed_experts", False),
                                   rid=(body.get("rid") if not batched else None),
                                   logprob_start_len=body.get("logprob_start_len", -1),
                                   top_logprobs_num=body.get("top_logprobs_num", 0)) for i, s in zip(batch, sps)]
        outs = [await _wait(r) for r in reqs]
        return JSONResponse(outs if batched else outs[0])

    # ---- prefill / decode disaggregation (engine/pd.py): this server as the prefill side or as the decode side ---------
    kv_exports: dict[str, Any] = {}

    @app.post("/prefill")
    async def prefill(request: Request):
        """Run the prompt, sample the first token, keep the KV: the reply carries the usual fields plus `kv` (a CUDA-IPC handle
        of the gathered tensor, or its bytes from a CPU engine) for the decode server; `/release_kv` ends the loan."""
        from ..weight_update import cuda_ipc

        body = await request.json()
        sp = dict(body.get("sampling_params") or {})
        req = engine.add_request(body["input_ids"], {**sp, "max_new_tokens": 1}, body.get("return_logprob", True),
                                 body.get("return_routed_experts", False), rid=body.get("rid"),
                                 logprob_start_len=body.get("logprob_start_len", -1), top_logprobs_num=body.get("top_logprobs_num", 0),
                                 keep_kv=True)
        out = await _wait(req)
        if req.rid in engine.held_kv:
            kv = engine.export_kv(req.rid)
            flat, manifest = cuda_ipc.pack_bucket([("kv", kv)])
            kv_exports[req.rid] = flat                       # alive until /release_kv: the peer maps this buffer
            out["kv"] = cuda_ipc.export_bucket(flat, manifest) if flat.is_cuda else cuda_ipc.serialize_bucket(flat, manifest)
            out["seed"] = req.seed
        return JSONResponse(out)

    @app.post("/release_kv")
    async def release_kv(request: Request):
        body = await request.json()
        kv_exports.pop(body["rid"], None)
        engine.release_kv(body["rid"])
        return {"success": True}

    @app.post("/generate_prefilled")
    async def generate_prefilled(request: Request):
        from ..weight_update import cuda_ipc

        body = await request.json()
        flat, manifest = cuda_ipc.open_bucket(body["kv"], engine.device)
        kv = cuda_ipc.split_bucket(flat, manifest)[0][1]
        routed = body.get("routed_experts")
        if routed is not None:
            from ..types import decode_routed_experts

            n = len(body["input_ids"])
            routed = decode_routed_experts(routed, n + 1, engine.model.num_moe_layers, engine.cfg.moe_topk)
        req = engine.add_prefilled(body["input_ids"], body["first_token"], body["first_logprob"], kv, body.get("sampling_params"),
                                   body.get("return_logprob", True), body.get("return_routed_experts", False), routed=routed,
                                   rid=body.get("rid"), seed=body.get("seed"))
        if flat.is_cuda:
            torch.cuda.current_stream(flat.device).synchronize()       # the copy out of the peer's buffer is complete: it may be released
        del kv, flat
        return JSONResponse(await _wait(req))

    @app.get("/health")
    async def health():
        return engine.health()

    @app.get("/health_generate")
    async def health_generate():
        if engine.paused:
            return engine.health()
        r = engine.add_request([1], {"max_new_tokens": 1, "temperature": 0.0}, False, False)
        await _wait(r)
        return engine.health()

    @app.api_route("/flush_cache", methods=["GET", "POST"])
    async def flush_cache():
        return {"success": engine.flush_cache()}

    @app.post("/pause_generation")
    async def pause(request: Request):
        body = await _json(request)
        engine.pause_generation(body.get("mode", "retract"))
        return {"success": True}

    @app.post("/continue_generation")
    async def cont():
        engine.continue_generation()
        return {"success": True}

    @app.post("/flush_cache")
    async def flush_cache():
        engine.flush_cache()
        return {"success": True}

    @app.post("/abort_request")
    async def abort(request: Request):
        body = await _json(request)
        engine.abort_request(None if body.get("abort_all") else body.get("rid"))
        return {"success": True}

    @app.post("/begin_weight_update")
    async def begin_update():
        state["updating"] = True
        return {"success": True}

    @app.post("/end_weight_update")
    async def end_update():
        state["updating"] = False
        return {"success": True}

    @app.post("/update_weights_from_tensor")
    async def update_from_tensor(request: Request):
        body = await request.json()
        if body.get("ipc_bucket") is not None:
            # one flat bucket: an IPC mapping of the sender's device buffer (or its bytes); copied, then unmapped before
            # the response — the sender reuses the buffer as soon as it has the answer
            from ..weight_update import cuda_ipc

            flat, manifest = cuda_ipc.open_bucket(body["ipc_bucket"], engine.device)
            named = cuda_ipc.split_bucket(flat, manifest)
            engine.update_weights_from_tensor(named, body.get("weight_version"), body.get("load_format"))
            n = len(named)
            if flat.is_cuda:
                torch.cuda.current_stream(flat.device).synchronize()
            del named, flat
            return {"success": True, "num_tensors": n}
        named = []
        for blob in body["serialized_named_tensors"]:
            named += deserialize_named_tensors(blob, engine.device)
        engine.update_weights_from_tensor(named, body.get("weight_version"), body.get("load_format"))
        return {"success": True, "num_tensors": len(named)}

    @app.post("/update_weights_from_disk")
    async def update_from_disk(request: Request):
        body = await request.json()
        engine.update_weights_from_disk(body["model_path"])
        if body.get("weight_version") is not None:
            engine.update_weight_version(int(body["weight_version"]))
        return {"success": True}

    @app.post("/init_weights_update_group")
    async def init_group(request: Request):
        import asyncio

        body = await request.json()
        # the rendezvous blocks until the trainer joins: keep the event loop free meanwhile
        return await asyncio.get_running_loop().run_in_executor(None, lambda: engine.init_weights_update_group(**body))

    @app.post("/update_weights_from_distributed")
    async def update_from_distributed(request: Request):
        import asyncio

        body = await request.json()
        body.pop("selector", None)
        return await asyncio.get_running_loop().run_in_executor(None, lambda: engine.update_weights_from_distributed(**body))

    @app.post("/update_weight_version")
    async def set_version(request: Request):
        body = await request.json()
        engine.update_weight_version(int(body["new_version"] if "new_version" in body else body["weight_version"]))
        return {"success": True}

    @app.get("/get_weight_version")
    async def get_version():
        return {"weight_version": str(engine.get_weight_version())}

    @app.post("/release_memory_occupation")
    async def release(request: Request):
        body = await _json(request)
        engine.pause_generation("retract")
        engine.release_memory_occupation(body.get("tags"))
        return {"success": True}

    @app.post("/resume_memory_occupation")
    async def resume(request: Request):
        body = await _json(request)
        engine.resume_memory_occupation(body.get("tags"))
        return {"success": True}

    @app.post("/weights_checker")
    async def weights_checker(request: Request):
        body = await _json(request)
        sums = weight_checksums(engine.model)
        if body.get("action") == "compare":
            want = body.get("checksums", {})
            bad = [k for k, v in want.items() if sums.get(k) != v]
            return {"success": not bad, "mismatched": bad}
        return {"success": True, "checksums": sums}

    @app.get("/get_server_info")
    async def info():
        return {"model": engine.cfg.name, "stats": engine.stats, "uptime": time.time() - state["started"], **engine.health()}

    @app.get("/metrics")
    async def metrics():
        h = engine.health()
        lines = [f"engine_running_requests {h['running']}", f"engine_waiting_requests {h['waiting']}",
                 f"engine_free_kv_blocks {h['free_blocks']}", f"engine_weight_version {h['weight_version']}"]
        lines += [f"engine_{k}_total {v}" for k, v in engine.stats.items() if isinstance(v, (int, float))]
        return PlainTextResponse("\n".join(lines) + "\n")

    @app.post("/start_profile")
    async def start_profile(request: Request):
        body = await _json(request)
        prof = torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA])
        prof.__enter__()
        state["profile"] = (prof, body.get("output_dir", "."))
        return {"success": True}

    @app.post("/stop_profile")
    async def stop_profile():
        if state["profile"]:
            prof, out = state["profile"]
            prof.__exit__(None, None, None)
            prof.export_chrome_trace(f"{out}/engine_trace_{int(time.time())}.json")
            state["profile"] = None
        return {"success": True}

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        body = await request.json()
        assert tokenizer is not None, "chat completions need a tokenizer"
        ids = tokenizer.apply_chat_template(body["messages"], tools=body.get("tools"), tokenize=True, add_generation_prompt=True)
        sp = {"temperature": body.get("temperature", 1.0), "top_p": body.get("top_p", 1.0),
              "max_new_tokens": body.get("max_tokens") or body.get("max_completion_tokens") or 256}
        out = await _wait(engine.add_request(list(ids), sp, bool(body.get("logprobs")), False))
        fr = out["meta_info"]["finish_reason"] or {}
        return {"id": out["meta_info"]["id"], "object": "chat.completion", "model": body.get("model", engine.cfg.name),
                "choices": [{"index": 0, "message": {"role": "assistant", "content": out["text"]},
                             "finish_reason": "length" if fr.get("type") == "length" else "stop"}],
                "usage": {"prompt_tokens": out["meta_info"]["prompt_tokens"], "completion_tokens": out["meta_info"]["completion_tokens"]},
                "meta_info": out["meta_info"], "output_ids": out["output_ids"]}

    return app


async def _json(request) -> dict:
    try:
        return await request.json()
    except Exception:
        return {}


def weight_checksums(model) -> dict[str, str]:
    out = {}
    for n, p in model.named_parameters():
        out[n] = hashlib.blake2b(p.detach().contiguous().view(torch.uint8).cpu().numpy().tobytes(), digest_size=8).hexdigest()
    return out


def serialize_named_tensors(named: list[tuple[str, torch.Tensor]]) -> str:
    """Wire format of `update_weights_from_tensor` between processes: base64 of a torch-saved dict (CPU tensors)."""
    buf = io.BytesIO()
    torch.save({n: t.detach().cpu() for n, t in named}, buf)
    return base64.b64encode(buf.getvalue()).decode()


def deserialize_named_tensors(blob: str, device) -> list[tuple[str, torch.Tensor]]:
    d = torch.load(io.BytesIO(base64.b64decode(blob)), map_location=device, weights_only=True)
    return list(d.items())


def serve(engine, host="127.0.0.1", port=30000, tokenizer=None, in_thread: bool = False):
    import uvicorn

    app = build_app(engine, tokenizer)
    config = uvicorn.Config(app, host=host, port=port, log_level="warning")
    server = uvicorn.Server(config)
    if in_thread:
        t = threading.Thread(target=server.run, daemon=True, name=f"engine-http-{port}")
        t.start()
        while not server.started:
            time.sleep(0.01)
        return server, t
    server.run()


def main():
    from ..models.config import get_config
    from .engine import Engine

    p = argparse.ArgumentParser()
    p.add_argument("--model-name", default="tiny")
    p.add_argument("--hf-checkpoint", default=None)
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=30000)
    p.add_argument("--mem-fraction-static", type=float, default=0.7)
    p.add_argument("--max-running-requests", type=int, default=256)
    p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--disable-radix-cache", action="store_true", help="do not reuse KV across requests with a common prefix")
    p.add_argument("--chunked-prefill-size", type=int, default=0, help="prefill long prompts in pieces of this many tokens (0: whole)")
    a = p.parse_args()
    cfg = get_config(a.hf_checkpoint or a.model_name)
    dtype = torch.bfloat16 if a.device.startswith("cuda") else torch.float32
    if a.device.startswith("cuda") and torch.device(a.device).index is not None:
        torch.cuda.set_device(torch.device(a.device))      # kernels and allocations of this process default to its own GPU
    eng = Engine(cfg, device=a.device, dtype=dtype, mem_fraction_static=a.mem_fraction_static, max_running_requests=a.max_running_requests,
                 prefix_cache=not a.disable_radix_cache, chunked_prefill_size=a.chunked_prefill_size or None)
    if a.hf_checkpoint:
        eng.update_weights_from_disk(a.hf_checkpoint)
    serve(eng, a.host, a.port)


if __name__ == "__main__":
    main()
