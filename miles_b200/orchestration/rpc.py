"""HTTP RPC between a controller and workers that do not share a process.

Reference: miles/utils/workers/rpc/{client,common,server}/* (`--worker-comm-backend rpc`: workers are served as RPC
endpoints instead of Ray actors; arguments are pickled; methods belong to concurrency groups so that, e.g., a health
probe is answered while `train` is running).

    server = RpcServer(worker_obj, concurrency={"default": 1, "health": 4}, groups={"ping": "health"})
    server.start(port)                          # thread; POST /call {"method", "args", "kwargs"} (pickle, base64)
    proxy = RpcClient("http://127.0.0.1:port")  # proxy.train(…) → remote call, exceptions re-raised locally

Pickle means the two ends must trust each other: this transport is for processes of ONE job on a private network, as
in the reference.
"""
from __future__ import annotations

import base64
import pickle
import threading
import traceback
from concurrent.futures import ThreadPoolExecutor
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any


def _enc(obj) -> bytes:
    return base64.b64encode(pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL))


def _dec(b: bytes):
    return pickle.loads(base64.b64decode(b))


class RemoteError(RuntimeError):
    def __init__(self, kind: str, message: str, remote_traceback: str):
        super().__init__(f"{kind}: {message}\n--- remote traceback ---\n{remote_traceback}")
        self.kind, self.message, self.remote_traceback = kind, message, remote_traceback


class RpcServer:
    def __init__(self, target: Any, concurrency: dict[str, int] | None = None, groups: dict[str, str] | None = None):
        self.target = target
        self.groups = groups or {}
        self.pools = {g: ThreadPoolExecutor(n, thread_name_prefix=f"rpc-{g}") for g, n in (concurrency or {"default": 1}).items()}
        self.pools.setdefault("default", ThreadPoolExecutor(1, thread_name_prefix="rpc-default"))
        self.httpd: ThreadingHTTPServer | None = None
        self.thread: threading.Thread | None = None

    def _dispatch(self, req: dict) -> dict:
        method = req["method"]
        if method.startswith("_") or not hasattr(self.target, method):
            return {"ok": False, "kind": "AttributeError", "message": f"no method {method!r}", "traceback": ""}
        pool = self.pools.get(self.groups.get(method, "default"), self.pools["default"])
        fut = pool.submit(getattr(self.target, method), *req.get("args", ()), **req.get("kwargs", {}))
        try:
            return {"ok": True, "result": fut.result()}
        except BaseException as e:
            return {"ok": False, "kind": type(e).__name__, "message": str(e), "traceback": traceback.format_exc()}

    def start(self, port: int = 0, host: str = "127.0.0.1") -> int:
        server = self

        class Handler(BaseHTTPRequestHandler):
            def do_POST(self):
                n = int(self.headers.get("Content-Length", 0))
                try:
                    out = server._dispatch(_dec(self.rfile.read(n)))
                    body = _enc(out)
                except BaseException as e:        # undecodable request or unpicklable result
                    body = _enc({"ok": False, "kind": type(e).__name__, "message": str(e), "traceback": traceback.format_exc()})
                self.send_response(200)
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def do_GET(self):
                self.send_response(200)
                self.end_headers()
                self.wfile.write(b"ok")

            def log_message(self, *a):
                pass

        self.httpd = ThreadingHTTPServer((host, port), Handler)
        self.thread = threading.Thread(target=self.httpd.serve_forever, daemon=True, name="rpc-server")
        self.thread.start()
        return self.httpd.server_address[1]

    def stop(self):
        if self.httpd is not None:
            self.httpd.shutdown()
            self.httpd.server_close()
        for p in self.pools.values():
            p.shutdown(wait=False)


class RpcClient:
    def __init__(self, url: str, timeout: float = 3600.0):
        self._url, self._timeout = url.rstrip("/"), timeout

    def _call(self, method: str, *args, **kwargs):
        import urllib.request

        req = urllib.request.Request(self._url + "/call", data=_enc({"method": method, "args": args, "kwargs": kwargs}), method="POST")
        with urllib.request.urlopen(req, timeout=self._timeout) as r:
            out = _dec(r.read())
        if out["ok"]:
            return out["result"]
        raise RemoteError(out["kind"], out["message"], out["traceback"])

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        return lambda *a, **kw: self._call(name, *a, **kw)
