"""Expert-parallel MoE over the NVLink fabric, with no host synchronisation.

forward   dispatch kernel: every (token, slot) row is stored straight into the owning rank's receive buffer (the row is
          allocated with a remote atomicAdd on that rank's counter) together with {source rank, source pair, expert}
          → flag barrier → counting sort of the received rows by local expert (device-side count) → grouped tcgen05
          GEMMs (gate/up, SwiGLU, down) → return kernel: each output row is stored into the source rank's return buffer
          at its (token, slot) position → flag barrier → weighted sum over the slots.
backward  the same two hops in reverse with the placement remembered from the forward pass (no atomics).

Replaces the reference's Megatron "alltoall" token dispatcher + permute fusion + TE GroupedLinear
(scripts/models/qwen3-30B-A3B.py:35-43).  Because nothing waits on the host, the whole layer can be captured in the
engine's CUDA-graph decode step.
"""
from __future__ import annotations

import torch

from ..ops.cuda_more import experts_backward, experts_forward, moe_max_rows_pad, small_moe_bt
from .fabric import CH_EP, CH_EP2

CAPACITY_FACTOR = 2.0       # receive rows per rank = factor × max_tokens × k (uniform routing gives 1.0)
DEFAULT_MAX_TOKENS = 16384 + 2048


class _Buffers:
    def __init__(self, fab, H: int, k: int, max_tokens: int, ranks: list[int]):
        self.cap = int(CAPACITY_FACTOR * max_tokens * k + 127) // 128 * 128
        self.max_pairs = max_tokens * k
        self.recv_x = fab.alloc(self.cap * H, torch.bfloat16, "moe.recv_x")
        self.recv_meta = fab.alloc(self.cap * 4, torch.int32, "moe.recv_meta")
        self.counter = fab.alloc(64, torch.int32, "moe.counter")
        self.ret = fab.alloc(self.max_pairs * H, torch.bfloat16, "moe.ret")
        self.recv_x_ptrs = fab.peer_ptrs(self.recv_x, ranks)
        self.recv_meta_ptrs = fab.peer_ptrs(self.recv_meta, ranks)
        self.counter_ptrs = fab.peer_ptrs(self.counter, ranks)
        self.ret_ptrs = fab.peer_ptrs(self.ret, ranks)
        self.expert_ids = torch.empty(self.cap, dtype=torch.int32, device=fab.device)
        self.n_recv = torch.zeros(1, dtype=torch.int32, device=fab.device)
        self.pair_ids = torch.arange(self.max_pairs, dtype=torch.int32, device=fab.device)
        self.minus_one = torch.full((), -1, dtype=torch.int32, device=fab.device)
        self.tickets = torch.zeros(2, dtype=torch.int32, device=fab.device)     # last-block tickets of the signalling kernels
        key = (tuple(ranks), "raw")
        if key not in fab._flag_ptrs:
            fab._flag_ptrs[key] = fab.flags.ptrs(ranks)
        self.flag_ptrs = fab._flag_ptrs[key]


def _buffers(fab, H, k, ps, T) -> _Buffers:
    key = ("moe", H, k)
    b = fab._moe.get(key)
    if b is None:
        max_tokens = getattr(fab, "moe_max_tokens", DEFAULT_MAX_TOKENS)
        b = _Buffers(fab, H, k, max_tokens, ps.ep_ranks)
        fab._moe[key] = b
    assert T * k <= b.max_pairs, f"{T} tokens exceed the fabric's MoE buffers (set fabric.moe_max_tokens before first use)"
    return b


import os

# Decode path variant with the cross-rank barriers folded into the kernels on either side of them (8 launches per layer
# instead of 11).  Measured on 2 GPUs it is 4 % SLOWER than the separate one-block barrier kernels (1.63 vs 1.57 ms for 12
# layers at 8 rows per rank: the signalling epilogue and the in-kernel wait lengthen kernels on the critical path by more
# than the three launches they remove), so it is off unless MILES_EP_FOLDED=1.
FOLDED_BARRIERS = os.environ.get("MILES_EP_FOLDED", "0") == "1"


def _decode_path(C, fab, b, x, w13, w2, wf, idx32, sent_row, cap, T, H, k, e_local, ep, me):
    """Inference with the same row count on every rank (the engine's agreed decode bucket): 8 launches per layer —
    dispatch+signal, wait+count+sort, gather, W13, SwiGLU, W2, return+signal, wait+combine."""
    n_pairs = T * k
    dev = x.device
    C.moe_dispatch_signal(x, idx32, k, e_local, me, b.recv_x_ptrs, b.recv_meta_ptrs, b.counter_ptrs, ep, b.cap, sent_row, fab.err,
                          b.flag_ptrs, CH_EP, fab.epochs, b.tickets[0:1])
    bt = small_moe_bt(n_pairs, e_local, w13, w2)
    max_rows = moe_max_rows_pad(cap, e_local, bt)
    seg = torch.empty(e_local + 1, dtype=torch.int32, device=dev)
    tile = torch.empty(max_rows // bt, dtype=torch.int32, device=dev)
    row_src = torch.empty(max_rows, dtype=torch.int32, device=dev)
    C.moe_recv_align(b.recv_meta, b.counter, cap, e_local, seg, tile, row_src, bt, b.flag_ptrs, me, ep, CH_EP, fab.epochs, fab.err)
    x_perm = torch.empty(max_rows, H, dtype=x.dtype, device=dev)
    C.moe_gather(b.recv_x.view(b.cap, H), x_perm, row_src, seg, 1)
    _, y_perm = experts_forward(x_perm, w13, w2, seg, tile, bt)
    C.moe_return_signal(y_perm, row_src, b.recv_meta, seg, b.ret_ptrs, ep, b.flag_ptrs, me, CH_EP2, fab.epochs, b.tickets[1:2])
    out = torch.empty(T, H, dtype=x.dtype, device=dev)
    C.moe_combine_wait(b.ret.view(b.max_pairs, H), wf, sent_row, out, k, b.flag_ptrs, me, ep, CH_EP2, fab.epochs, fab.err)
    return out


class _FusedMoE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w13, w2, topk_w, topk_idx, fab, ps, num_experts, grad_mode=True):
        C = fab.C
        T, H = x.shape
        k = topk_idx.shape[1]
        e_local = num_experts // ps.ep_size
        ep, me = ps.ep_size, ps.ep_rank
        ranks = ps.ep_ranks
        b = _buffers(fab, H, k, ps, T)
        x = x.contiguous()
        idx32 = topk_idx.to(torch.int32).contiguous().view(-1)
        wf = topk_w.float().contiguous()
        n_pairs = T * k
        sent_row = torch.empty(max(n_pairs, 1), dtype=torch.int32, device=x.device)
        if not grad_mode and getattr(ps, "moe_uniform_tokens", False):
            small_cap = min(b.cap, (ep * max(n_pairs, 1) + 127) // 128 * 128)
            if small_cap <= 16384 and FOLDED_BARRIERS:
                return _decode_path(C, fab, b, x, w13, w2, wf, idx32, sent_row, small_cap, T, H, k, e_local, ep, me)
        if n_pairs:
            C.moe_dispatch(x, idx32, k, e_local, me, b.recv_x_ptrs, b.recv_meta_ptrs, b.counter_ptrs, ep, b.cap, sent_row, fab.err)
        fab.barrier(ranks, CH_EP)
        # `needs_input_grad` follows the inputs' requires_grad flags even under no_grad (the engine serves the trainer's
        # parameters): without the caller's grad mode inference would take the 128-row training tiles and clone what
        # backward needs.  (Inside `forward` grad mode is always off, so the wrapper samples it.)
        need_bwd = grad_mode and any(ctx.needs_input_grad[:4])
        # Rows that can arrive here: the buffer capacity in general; ep · T · k when every rank of the group runs this call
        # with the same T (the engine's decode steps agree on one batch bucket).  Everything sized by this bound — the
        # expert-id scan, the tile table, the padded row space — then shrinks from ~300k rows to a few hundred.
        cap = b.cap
        if getattr(ps, "moe_uniform_tokens", False) and not need_bwd:
            cap = min(cap, (ep * max(n_pairs, 1) + 127) // 128 * 128)
        small = cap <= 16384                # one-block scan that also resets the receive counter (no separate memset)
        C.recv_expert_ids(b.recv_meta, b.counter, cap, b.expert_ids[:cap], b.n_recv, small)
        if not small:
            b.counter.zero_()
        # decode-sized calls (about n_pairs rows arrive when the routing is balanced): pad segments to 16/32/64 rows
        bt = 128 if need_bwd else small_moe_bt(n_pairs, e_local, w13, w2)
        max_rows = moe_max_rows_pad(cap, e_local, bt)
        seg, tile, row_src, _ = C.moe_align(b.expert_ids[:cap], e_local, 0, max_rows, b.n_recv, bt)
        x_perm = torch.empty(max_rows, H, dtype=x.dtype, device=x.device)
        C.moe_gather(b.recv_x.view(b.cap, H), x_perm, row_src, seg, 1)
        h1, y_perm = experts_forward(x_perm, w13, w2, seg, tile, bt)
        meta = b.recv_meta.clone() if need_bwd else b.recv_meta   # the shared buffer is overwritten by the next layer
        C.moe_return(y_perm, row_src, b.recv_meta, seg, b.ret_ptrs, ep)
        fab.barrier(ranks, CH_EP2)
        out = torch.empty(T, H, dtype=x.dtype, device=x.device)
        if need_bwd:
            dst_row = torch.where(sent_row >= 0, b.pair_ids[:max(n_pairs, 1)], b.minus_one)
            if T:
                C.moe_combine(b.ret.view(b.max_pairs, H), wf, dst_row, out, k)
        elif T:
            # the return buffer is indexed by pair: `sent_row` only has to say which pairs took part
            C.moe_combine(b.ret.view(b.max_pairs, H), wf, sent_row, out, k, True)
        if need_bwd:
            ret_saved = b.ret.view(b.max_pairs, H)[:max(n_pairs, 1)].clone()
            ctx.save_for_backward(w13, w2, wf, idx32, sent_row, dst_row, seg, tile, row_src, meta, h1, x_perm, ret_saved)
        ctx.fab, ctx.ps, ctx.k, ctx.e_local, ctx.T, ctx.H = fab, ps, k, e_local, T, H
        return out

    @staticmethod
    def backward(ctx, dout):
        w13, w2, wf, idx32, sent_row, dst_row, seg, tile, row_src, meta, h1, x_perm, ret_saved = ctx.saved_tensors
        fab, ps, k, e_local, T, H = ctx.fab, ctx.ps, ctx.k, ctx.e_local, ctx.T, ctx.H
        C = fab.C
        ep, ranks = ps.ep_size, ps.ep_ranks
        b = _buffers(fab, H, k, ps, T)
        dout = dout.contiguous()
        n_pairs = T * k
        dev = dout.device
        # d(return rows) and d(gate weights): row p of the pair-indexed buffer
        dy_pair = torch.empty(max(n_pairs, 1), H, dtype=dout.dtype, device=dev)
        dw_flat = torch.zeros(max(n_pairs, 1), dtype=torch.float32, device=dev)
        seg1 = torch.tensor([0, n_pairs], dtype=torch.int32, device=dev)
        if n_pairs:
            C.moe_combine_bwd(dout, ret_saved, wf.view(-1), dst_row, seg1, dy_pair, dw_flat, k)
            C.moe_scatter_known(dy_pair, True, idx32, sent_row, k, e_local, b.recv_x_ptrs, ep)
        fab.barrier(ranks, CH_EP)
        max_rows = x_perm.shape[0]
        dy_perm = torch.empty(max_rows, H, dtype=dout.dtype, device=dev)
        C.moe_gather(b.recv_x.view(b.cap, H), dy_perm, row_src, seg, 1)
        dx_perm, dw13, dw2 = experts_backward(dy_perm, x_perm, h1, w13, w2, seg, tile)
        C.moe_return(dx_perm, row_src, meta, seg, b.ret_ptrs, ep)
        fab.barrier(ranks, CH_EP2)
        dx = torch.empty(T, H, dtype=dout.dtype, device=dev)
        if T:
            C.moe_combine(b.ret.view(b.max_pairs, H), None, dst_row, dx, k)
        return dx, dw13, dw2, dw_flat[:n_pairs].view(T, k), None, None, None, None, None


def fused_moe(fab, x, w13, w2, topk_w, topk_idx, num_experts, ps):
    return _FusedMoE.apply(x, w13, w2, topk_w, topk_idx, fab, ps, num_experts, torch.is_grad_enabled())
