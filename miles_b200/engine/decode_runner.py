"""Decode-step runner with static buffers and CUDA graphs.

Running requests own a fixed row of a set of static device buffers (last token, position, cache slot, block table,
sampling parameters).  A decode step copies the host mirrors of those buffers to the device (three pinned-memory
copies), replays the CUDA graph captured for the smallest batch bucket that covers the occupied rows, and reads the
sampled ids / log-probs (and routed experts) back with one device→host copy.  Rows of finished requests are padding
(seq_len 0, slot −1: no KV write, attention over zero keys) until the rows are compacted.

The graph contains the whole model forward, the LM head, and the fused sample+log-prob kernel, so a decode step is one
graph launch instead of ~25 launches per layer.

Several steps per host round trip (`steps > 1`): the graph is replayed `steps` times back to back; between replays a few
device-side ops feed the sampled token back (token ← sample, position / length + 1, cache slot from the block table,
random seed + 1) and append the step's outputs to a history buffer.  The host then reads all `steps` tokens of every
row at once and drops what a row produced after its stop token or length limit.  Per-step host work, the lockstep
agreement of expert-parallel ranks and the skew between their hosts are then paid once per `steps` steps.
"""
from __future__ import annotations

import time
import zlib

import numpy as np
import torch

from ..models.qwen3 import ForwardMeta

BUCKETS = [1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512, 768, 1024]


class DecodeRunner:
    def __init__(self, engine, max_rows: int, use_graph: bool):
        self.e = engine
        self.dev = engine.device
        self.use_graph = use_graph
        self.max_rows = max_rows
        self.max_blocks = (engine.max_context_len + engine.block_size - 1) // engine.block_size + 1
        cfg = engine.cfg
        self.n_moe = engine.model.num_moe_layers if cfg.is_moe else 0
        self.topk = cfg.moe_topk
        R, MB = max_rows, self.max_blocks
        # host mirrors (pinned) — int32 pack: tokens | positions | seq_lens | block_table ; int64 pack: slots | seeds
        self.h_i32 = torch.zeros(3 * R + R * MB, dtype=torch.int32).pin_memory()
        self.h_i64 = torch.zeros(2 * R, dtype=torch.int64).pin_memory()
        self.h_f32 = torch.ones(R, dtype=torch.float32).pin_memory()
        self.h_u8 = torch.zeros(R, dtype=torch.uint8).pin_memory()
        self.d_i32 = torch.zeros_like(self.h_i32, device=self.dev)
        self.d_i64 = torch.zeros_like(self.h_i64, device=self.dev)
        self.d_f32 = torch.ones_like(self.h_f32, device=self.dev)
        self.d_u8 = torch.zeros_like(self.h_u8, device=self.dev)
        self.np_i32 = self.h_i32.numpy()
        self.np_i64 = self.h_i64.numpy()
        self.np_f32 = self.h_f32.numpy()
        self.np_u8 = self.h_u8.numpy()
        self.tok_np = self.np_i32[0:R]
        self.pos_np = self.np_i32[R:2 * R]
        self.len_np = self.np_i32[2 * R:3 * R]
        self.bt_np = self.np_i32[3 * R:].reshape(R, MB)
        self.slot_np = self.np_i64[0:R]
        self.seed_np = self.np_i64[R:2 * R]
        self.slot_np[:] = -1
        # outputs
        self.o_tok = torch.zeros(R, dtype=torch.int64, device=self.dev)
        self.o_lp = torch.zeros(R, dtype=torch.float32, device=self.dev)
        self.o_routed = torch.zeros(R, max(self.n_moe, 1), max(self.topk, 1), dtype=torch.int32, device=self.dev)
        self.h_tok = torch.zeros(R, dtype=torch.int64).pin_memory()
        self.h_lp = torch.zeros(R, dtype=torch.float32).pin_memory()
        self.h_routed = torch.zeros(R, max(self.n_moe, 1), max(self.topk, 1), dtype=torch.int32).pin_memory()
        # histories of a multi-step call: [step, row]
        self.max_steps = 32
        self.chunk_steps = 8                  # outputs come back to the host in chunks of this many steps
        self._chunks: list = []               # [(first step not yet on the host after this chunk, event)] of the last call
        self._on_host = 0
        self._events = [torch.cuda.Event() for _ in range(self.max_steps // self.chunk_steps + 1)]
        S = self.max_steps
        self.hist_tok = torch.zeros(S, R, dtype=torch.int64, device=self.dev)
        self.hist_lp = torch.zeros(S, R, dtype=torch.float32, device=self.dev)
        self.hist_routed = torch.zeros(S, R, max(self.n_moe, 1), max(self.topk, 1), dtype=torch.int32, device=self.dev)
        self.hh_tok = torch.zeros(S, R, dtype=torch.int64).pin_memory()
        self.hh_lp = torch.zeros(S, R, dtype=torch.float32).pin_memory()
        self.hh_routed = torch.zeros(S, R, max(self.n_moe, 1), max(self.topk, 1), dtype=torch.int32).pin_memory()
        self.rows: list = [None] * R          # row → Request
        self.free_rows = list(range(R - 1, -1, -1))
        self.high = 0                         # 1 + highest occupied row
        from .. import ops

        self._err = ops._k().C.error_flag(self.d_i32)      # device error flag: raised (71) when a step samples an id outside the vocabulary
        self.last_logits = None               # [B, V] logits of the last eager step (for top-k log-probs read by the host)
        self.graphs: dict[int, tuple] = {}
        self.launches_per_graph: dict[int, int] = {}
        self.pool = None

    # ---- row bookkeeping -------------------------------------------------------------------
    def attach(self, req):
        row = self.free_rows.pop()
        req.row = row
        self.rows[row] = req
        self.bt_np[row, :len(req.blocks)] = req.blocks
        req.bt_len = len(req.blocks)
        self.np_f32[row] = req.sampling.temperature if req.sampling.temperature > 0 else 1.0
        self.np_u8[row] = 1 if req.sampling.temperature <= 0 else 0
        self.high = max(self.high, row + 1)

    def detach(self, req):
        row = getattr(req, "row", None)
        if row is None:
            return
        self.rows[row] = None
        self.len_np[row] = 0
        self.slot_np[row] = -1
        self.free_rows.append(row)
        req.row = None
        while self.high > 0 and self.rows[self.high - 1] is None:
            self.high -= 1

    def compact(self):
        """Move the highest rows into holes so that the occupied rows form a prefix."""
        self.free_rows.sort(reverse=True)
        while self.free_rows and self.free_rows[-1] < self.high - 1:
            hole = self.free_rows[-1]
            src = self.high - 1
            if self.rows[src] is None:
                self.high -= 1
                continue
            req = self.rows[src]
            self.free_rows.pop()
            self.rows[hole], self.rows[src] = req, None
            req.row = hole
            self.bt_np[hole, :req.bt_len] = self.bt_np[src, :req.bt_len]
            self.np_f32[hole], self.np_u8[hole] = self.np_f32[src], self.np_u8[src]
            self.len_np[src] = 0
            self.slot_np[src] = -1
            self.free_rows.append(src)
            self.free_rows.sort(reverse=True)
            while self.high > 0 and self.rows[self.high - 1] is None:
                self.high -= 1

    # ---- one decode step -------------------------------------------------------------------
    def _bucket(self, n: int) -> int:
        for b in BUCKETS:
            if b >= n:
                return min(b, self.max_rows)
        return self.max_rows

    def bucket_needed(self) -> int:
        return self._bucket(max(self.high, 1))

    def _forward(self, B: int, record: bool):
        e = self.e
        uniform = e.lockstep_group is not None      # lockstep ranks run every decode step with the same row count
        if uniform:
            e.ps.moe_uniform_tokens = True
        try:
            self._forward_impl(B, record)
        finally:
            if uniform:
                e.ps.moe_uniform_tokens = False

    def _forward_impl(self, B: int, record: bool):
        e = self.e
        R, MB = self.max_rows, self.max_blocks
        tokens = self.d_i32[0:B]
        meta = ForwardMeta(
            positions=self.d_i32[R:R + B], cu_seqlens=None, max_seqlen=1, kv_cache=e.kv.layers,
            block_table=self.d_i32[3 * R:].view(R, MB)[:B], seq_lens=self.d_i32[2 * R:2 * R + B],
            slot_mapping=self.d_i64[0:B], record_topk=[] if record else None)
        hidden = e.model(tokens, meta)
        hidden = e.ps.sp_gather(hidden)
        logits = e.model.logits(hidden)
        if not torch.cuda.is_current_stream_capturing():
            self.last_logits = logits               # eager steps only (requests that want the k most likely tokens run eagerly)
        from .. import ops

        tok, lp = ops._k().sample_logprob(logits, self.d_f32[:B], self.d_u8[:B], self.d_i64[R:R + B], 0)
        self.o_tok[:B].copy_(tok)
        self.o_lp[:B].copy_(lp)
        if record and meta.record_topk:
            self.o_routed[:B].copy_(torch.stack(meta.record_topk, dim=1))

    def _advance(self, B: int, k: int, record: bool):
        """Device-side hand-over between two replays of one multi-step call (rows with length 0 are padding)."""
        R, MB = self.max_rows, self.max_blocks
        from .. import ops

        C = ops._k().C
        C.decode_advance(self.o_tok[:B], self.o_lp[:B], self.o_routed[:B] if record else None, self.hist_tok[k, :B], self.hist_lp[k, :B],
                         self.hist_routed[k, :B] if record else None, self.d_i32[0:B], self.d_i32[R:R + B], self.d_i32[2 * R:2 * R + B],
                         self.d_i32[3 * R:].view(R, MB)[:B], self.e.block_size, self.d_i64[0:B], self.d_i64[R:R + B],
                         self.e.cfg.vocab_size, self._err)

    def step(self, reqs: list, step_no: int, min_bucket: int = 0, steps: int = 1):
        """Run `steps` decode steps for the attached requests (every request must own cache blocks for `steps` more
        tokens).  Returns (tokens, logprobs, routed | None) as numpy views indexed [row] for one step and [step, row] for
        several."""
        e = self.e
        bs = e.block_size
        if len(self.free_rows) and (self.high - len(reqs)) > max(8, len(reqs) // 4):
            self.compact()
        for r in reqs:
            row = r.row
            n = len(r.input_ids) + len(r.output_ids)
            pos = n - 1
            if len(r.blocks) != r.bt_len:
                self.bt_np[row, r.bt_len:len(r.blocks)] = r.blocks[r.bt_len:]
                r.bt_len = len(r.blocks)
            self.tok_np[row] = r.output_ids[-1] if r.output_ids else r.input_ids[-1]
            self.pos_np[row] = pos
            self.len_np[row] = n
            self.slot_np[row] = r.blocks[pos // bs] * bs + pos % bs
            self.seed_np[row] = (r.seed * 1000003 + n) & 0x7FFFFFFFFFFFFFFF
        B = min(max(self._bucket(max(self.high, 1)), int(min_bucket)), self.max_rows)
        record = self.n_moe > 0 and any(r.return_routed_experts for r in reqs)
        self.d_i32.copy_(self.h_i32, non_blocking=True)
        self.d_i64.copy_(self.h_i64, non_blocking=True)
        self.d_f32.copy_(self.h_f32, non_blocking=True)
        self.d_u8.copy_(self.h_u8, non_blocking=True)
        e.stats["h2d_bytes"] = e.stats.get("h2d_bytes", 0) + self.h_i32.numel() * 4 + self.h_i64.numel() * 8 + 5 * self.max_rows
        key = (B, record)
        steps = max(1, min(int(steps), self.max_steps))
        self._chunks, self._on_host = [], 0
        eager = any(getattr(r, "top_logprobs_num", 0) > 0 for r in reqs)      # their logits are read after the step
        for k in range(steps):
            if self.use_graph and not eager:
                if key not in self.graphs:
                    self._capture(key)
                self.graphs[key].replay()
                from .. import ops

                ops._k().C.count_launches(self.launches_per_graph[key])
            else:
                self._forward(B, record)
            if steps > 1:
                self._advance(B, k, record)
                if (k + 1) % self.chunk_steps == 0 or k + 1 == steps:
                    self._flush_chunk(B, k + 1, record)
        if steps > 1:
            # the copies were queued chunk by chunk behind the replays (`_flush_chunk`): the caller reads step k after
            # `wait_step(k)` and does its bookkeeping for one chunk while the GPU runs the next ones
            return self.hh_tok.numpy(), self.hh_lp.numpy(), (self.hh_routed.numpy() if record else None)
        self.h_tok[:B].copy_(self.o_tok[:B], non_blocking=True)
        self.h_lp[:B].copy_(self.o_lp[:B], non_blocking=True)
        nbytes = 12 * B
        if record:
            self.h_routed[:B].copy_(self.o_routed[:B], non_blocking=True)
            nbytes += self.h_routed[:B].numel() * 4
        e.stats["d2h_bytes"] = e.stats.get("d2h_bytes", 0) + nbytes
        t0 = time.perf_counter()
        torch.cuda.current_stream().synchronize()
        e.stats["decode_wait_s"] = e.stats.get("decode_wait_s", 0.0) + time.perf_counter() - t0   # host idle, GPU busy
        return self.h_tok.numpy(), self.h_lp.numpy(), (self.h_routed.numpy() if record else None)

    def _flush_chunk(self, B: int, end: int, record: bool):
        """Queue the device→host copies of the history rows [start, end) and mark the point with an event."""
        e = self.e
        start = self._chunks[-1][0] if self._chunks else 0
        self.hh_tok[start:end, :B].copy_(self.hist_tok[start:end, :B], non_blocking=True)
        self.hh_lp[start:end, :B].copy_(self.hist_lp[start:end, :B], non_blocking=True)
        nbytes = 12 * B * (end - start)
        if record:
            self.hh_routed[start:end, :B].copy_(self.hist_routed[start:end, :B], non_blocking=True)
            nbytes += self.hh_routed[start:end, :B].numel() * 4
        e.stats["d2h_bytes"] = e.stats.get("d2h_bytes", 0) + nbytes
        ev = self._events[len(self._chunks)]
        ev.record()
        self._chunks.append((end, ev))

    def wait_step(self, k: int):
        """Block until the outputs of step `k` of the last multi-step call are in the host buffers."""
        while self._on_host <= k and self._chunks:
            end, ev = self._chunks.pop(0)
            t0 = time.perf_counter()
            ev.synchronize()
            self.e.stats["decode_wait_s"] = self.e.stats.get("decode_wait_s", 0.0) + time.perf_counter() - t0   # host idle, GPU busy
            self._on_host = end

    @torch.no_grad()
    def warmup(self):
        """One eager decode step on padding rows only (no KV writes): initialises per-kernel attributes before any
        graph capture.  Expert-parallel ranks call this together (every MoE layer is a collective).  Runs without autograd:
        a recorded forward would keep every layer's worst-case-sized dispatch buffers alive until the step ends."""
        if getattr(self, "_warm", False):
            return
        self.d_i32.copy_(self.h_i32)
        self.d_i64.copy_(self.h_i64)
        self._forward(1, self.n_moe > 0)
        torch.cuda.synchronize()
        self._warm = True

    def _capture(self, key):
        from .. import ops

        B, record = key
        if self.e.lockstep_group is None:
            # eager warm-up with the same shapes (initialises per-kernel attributes and the allocator pool); lockstep
            # engines must not run an extra forward here because their peers would not match its collectives
            self._forward(B, record)
            torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        n0 = ops._k().launch_count()
        with torch.cuda.graph(g, pool=self.pool):
            self._forward(B, record)
        self.launches_per_graph[key] = ops._k().launch_count() - n0
        if self.pool is None:
            self.pool = g.pool()
        self.graphs[key] = g

    @torch.no_grad()
    def precapture(self, records=(True,)) -> int:
        """Capture the decode graph of every batch bucket that has none yet (for each routing-record variant asked for), on
        padding rows only.  Serving stacks do this at start-up; here it is a call of its own so that a caller can place the
        cost (≈ a second per graph) where it wants it — e.g. after a warm-up rollout, not inside a measured one.  A capture
        records kernels without running them, so expert-parallel ranks may capture independently."""
        if not self.use_graph:
            return 0
        self.d_i32.copy_(self.h_i32)            # padding state: rows of finished requests have length 0 and no cache slot
        self.d_i64.copy_(self.h_i64)
        n = 0
        for b in BUCKETS:
            if b > self.max_rows:
                break
            for rec in records:
                key = (b, bool(rec) and self.n_moe > 0)
                if key not in self.graphs:
                    self._capture(key)
                    n += 1
        torch.cuda.synchronize()
        return n

    def reset_graphs(self):
        self.graphs.clear()
        self.pool = None
