"""Session server: an OpenAI-compatible chat endpoint that remembers the exact token trajectory of every session.

Agent frameworks drive rollouts through `POST /sessions/{id}/v1/chat/completions` with growing message lists; the
server maps each call onto token-in-token-out `/generate` calls of the rollout engine and keeps, per session, the ids
the engine consumed and produced, the loss mask (1 for sampled ids, 0 for everything injected by the environment) and
the sampling log-probs.  When the episode ends the trainer pulls the trajectory (`GET /sessions/{id}`) and gets exactly
what the engine saw.  Reference: miles/rollout/session/core.py:195-428 (linear sessions, v1) and session/v2/* (tree
sessions: a request whose messages diverge from the stored conversation forks a branch instead of failing).
"""
from __future__ import annotations

import time
import uuid
from dataclasses import dataclass, field
from typing import Any

from fastapi import FastAPI, HTTPException
from fastapi import Request as _Request   # module level: postponed annotations are resolved in module scope

from .tito import TitoTokenizer


@dataclass
class Session:
    sid: str
    messages: list[dict] = field(default_factory=list)     # conversation the stored ids correspond to
    tokens: list[int] = field(default_factory=list)
    loss_mask: list[int] = field(default_factory=list)     # aligned with tokens[prompt_length:]
    log_probs: list[float] = field(default_factory=list)
    prompt_length: int = 0
    weight_versions: list[list[int]] = field(default_factory=list)
    parent: str | None = None
    created: float = field(default_factory=time.time)
    finished: bool = False
    metadata: dict = field(default_factory=dict)

    def trajectory(self) -> dict:
        return {"session_id": self.sid, "tokens": list(self.tokens), "prompt_length": self.prompt_length,
                "response_length": len(self.tokens) - self.prompt_length, "loss_mask": list(self.loss_mask),
                "rollout_log_probs": list(self.log_probs), "weight_versions": self.weight_versions, "messages": self.messages,
                "parent": self.parent, "metadata": self.metadata}


def _same_prefix(stored: list[dict], incoming: list[dict]) -> bool:
    if len(incoming) < len(stored):
        return False
    return all(a.get("role") == b.get("role") and (a.get("content") or "") == (b.get("content") or "")
               for a, b in zip(stored, incoming))


class SessionManager:
    """Engine-agnostic core (the HTTP layer below is a thin wrapper).  `generate(payload) -> awaitable[dict]` is the
    engine client's `/generate`."""

    def __init__(self, tokenizer, generate, family: str = "auto", tree: bool = True, default_sampling: dict | None = None):
        self.tito = tokenizer if isinstance(tokenizer, TitoTokenizer) else TitoTokenizer(tokenizer, family)
        self.generate = generate
        self.tree = tree
        self.default_sampling = default_sampling or {"temperature": 1.0, "max_new_tokens": 1024}
        self.sessions: dict[str, Session] = {}

    def create(self, sid: str | None = None, metadata: dict | None = None) -> Session:
        sid = sid or uuid.uuid4().hex
        s = Session(sid=sid, metadata=metadata or {})
        self.sessions[sid] = s
        return s

    def get(self, sid: str) -> Session:
        return self.sessions[sid]

    def delete(self, sid: str):
        self.sessions.pop(sid, None)

    def _fork(self, s: Session, keep_messages: int) -> Session:
        """Tree sessions: branch off at the last point both conversations share (a whole number of turns)."""
        child = self.create(metadata=dict(s.metadata))
        child.parent = s.sid
        # replay the shared turns: ids of shared assistant turns are copied verbatim, the rest is re-rendered
        marks = s.metadata.get("_turn_ends", [])
        if keep_messages and keep_messages <= len(marks):
            end = marks[keep_messages - 1]
            child.tokens = s.tokens[:end]
            child.prompt_length = min(s.prompt_length, end)
            n = end - child.prompt_length
            child.loss_mask, child.log_probs = s.loss_mask[:n], s.log_probs[:n]
            child.messages = [dict(m) for m in s.messages[:keep_messages]]
            child.metadata["_turn_ends"] = marks[:keep_messages]
        return child

    async def chat(self, sid: str, messages: list[dict], sampling: dict | None = None, tools: list | None = None) -> dict:
        s = self.sessions[sid]
        if s.messages and not _same_prefix(s.messages, messages):
            if not self.tree:
                raise ValueError("messages diverge from the session's conversation (linear sessions cannot branch)")
            shared = 0
            for a, b in zip(s.messages, messages):
                if a.get("role") != b.get("role") or (a.get("content") or "") != (b.get("content") or ""):
                    break
                shared += 1
            s = self._fork(s, shared)
        new = messages[len(s.messages):]
        marks = s.metadata.setdefault("_turn_ends", [])
        if not s.tokens:
            ids = self.tito.start(messages, tools)
            s.tokens, s.prompt_length = list(ids), len(ids)
        else:
            ids = self.tito.extend(s.messages, new, tools, pretokenized=s.tokens)
            s.tokens += ids
            s.loss_mask += [0] * len(ids)
            s.log_probs += [0.0] * len(ids)
        for _ in new:
            marks.append(len(s.tokens))
        s.messages = [dict(m) for m in messages]
        sp = dict(self.default_sampling)
        sp.update(sampling or {})
        out = await self.generate({"input_ids": list(s.tokens), "sampling_params": sp, "return_logprob": True})
        meta = out["meta_info"]
        pairs = meta.get("output_token_logprobs") or []
        gen = [int(p[1]) for p in pairs]
        s.tokens += gen
        s.loss_mask += [1] * len(gen)
        s.log_probs += [float(p[0]) for p in pairs]
        close = self.tito.close_assistant_turn(gen)
        s.tokens += close
        s.loss_mask += [0] * len(close)
        s.log_probs += [0.0] * len(close)
        for span in meta.get("weight_version_spans") or []:
            s.weight_versions.append(list(span))
        text = out.get("text") or self.tito.decode(self.tito.strip_turn_end(gen))
        s.messages.append({"role": "assistant", "content": text})
        marks.append(len(s.tokens))
        fr = (meta.get("finish_reason") or {}).get("type", "stop")
        return {"id": f"chatcmpl-{uuid.uuid4().hex[:12]}", "object": "chat.completion", "session_id": s.sid, "created": int(time.time()),
                "choices": [{"index": 0, "message": {"role": "assistant", "content": text},
                             "finish_reason": "length" if fr == "length" else "stop"}],
                "usage": {"prompt_tokens": len(s.tokens) - len(gen) - len(close), "completion_tokens": len(gen),
                          "total_tokens": len(s.tokens)}}

    def to_sample(self, sid: str):
        """The finished session as a training `Sample`."""
        from ..types import Sample, Status

        s = self.sessions[sid]
        return Sample(tokens=list(s.tokens), response_length=len(s.tokens) - s.prompt_length, loss_mask=list(s.loss_mask),
                      rollout_log_probs=list(s.log_probs), status=Status.COMPLETED, metadata={"session_id": sid, **s.metadata})


def build_app(manager: SessionManager):
    app = FastAPI(title="miles_b200 session server")

    @app.post("/sessions")
    async def create(request: _Request):
        body = await request.json() if await request.body() else {}
        s = manager.create(body.get("session_id"), body.get("metadata"))
        return {"session_id": s.sid}

    @app.get("/sessions/{sid}")
    async def get(sid: str):
        if sid not in manager.sessions:
            raise HTTPException(404, "unknown session")
        return manager.get(sid).trajectory()

    @app.delete("/sessions/{sid}")
    async def delete(sid: str):
        manager.delete(sid)
        return {"deleted": sid}

    @app.post("/sessions/{sid}/v1/chat/completions")
    async def chat(sid: str, request: _Request):
        body = await request.json()
        if sid not in manager.sessions:
            manager.create(sid)
        sp: dict[str, Any] = {}
        if "max_tokens" in body:
            sp["max_new_tokens"] = body["max_tokens"]
        for k in ("temperature", "top_p", "top_k"):
            if k in body:
                sp[k] = body[k]
        try:
            return await manager.chat(sid, body["messages"], sp, body.get("tools"))
        except ValueError as e:
            raise HTTPException(409, str(e))

    @app.get("/health")
    async def health():
        return {"status": "ok", "sessions": len(manager.sessions)}

    return app


# ---- picking what to train on ---------------------------------------------------------------------------------------

def drop_same_prompt_retries(samples: list) -> list:
    """Default `--session-sample-picker-path`: an agent that retries a call leaves several samples with the same prompt
    ids in one session; only the last attempt of each prompt is trained on (the earlier ones were discarded by the agent).
    The prompt of a multi-turn sample is everything before its last sampled turn."""
    last: dict[tuple, int] = {}
    for i, s in enumerate(samples):
        n = len(s.tokens) - s.response_length
        mask = list(s.loss_mask or [])
        if mask and any(mask):                       # multi-turn: the context ends where the LAST sampled run begins
            j = len(mask) - 1
            while j >= 0 and not mask[j]:
                j -= 1
            while j >= 0 and mask[j]:
                j -= 1
            n += j + 1
        last[tuple(s.tokens[:n])] = i
    keep = set(last.values())
    return [s for i, s in enumerate(samples) if i in keep]


def default_postprocess(samples: list) -> list:
    """Default `--session-sample-postprocessor-path`: samples pass through unchanged."""
    return samples


def session_samples(manager: SessionManager, root_sid: str, args=None) -> list:
    """Training samples of a session tree: every branch is a complete trajectory from the first message on (a fork copies
    the shared turns' ids), so each session of the tree gives one sample; the configured picker then drops what should not
    be trained on and the post-processor has the last word."""
    from ..utils.misc import load_function

    children: dict[str, list[str]] = {}
    for sid, s in manager.sessions.items():
        if s.parent is not None:
            children.setdefault(s.parent, []).append(sid)
    members, stack = [], [root_sid]
    while stack:
        sid = stack.pop()
        members.append(sid)
        stack.extend(children.get(sid, []))
    samples = [manager.to_sample(sid) for sid in sorted(members) if manager.sessions[sid].tokens]
    pick = load_function(getattr(args, "session_sample_picker_path", None) or "miles_b200.session.core.drop_same_prompt_retries")
    post = load_function(getattr(args, "session_sample_postprocessor_path", None) or "miles_b200.session.core.default_postprocess")
    return post(pick(samples))


def start_session_server(args, tokenizer, generate, in_thread: bool = True):
    """Serve sessions on `--session-server-ip` : `--session-server-port` with the `--tito-model` family.  Returns
    (manager, server, thread)."""
    import threading

    import uvicorn

    family = getattr(args, "tito_model", None) or "auto"
    manager = SessionManager(tokenizer, generate, family="auto" if family == "default" else family)
    host = getattr(args, "session_server_ip", None) or "127.0.0.1"
    port = int(getattr(args, "session_server_port", None) or 30300)
    server = uvicorn.Server(uvicorn.Config(build_app(manager), host=host, port=port, log_level="warning"))
    if not in_thread:
        server.run()
        return manager, server, None
    t = threading.Thread(target=server.run, daemon=True, name=f"session-server-{port}")
    t.start()
    while not server.started:
        time.sleep(0.01)
    return manager, server, t
