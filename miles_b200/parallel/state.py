"""Process-group bookkeeping and the parallel linear/MoE/log-prob entry points the model calls.

Rank order is tp → cp → dp → pp (fastest first), the order the reference hands to Megatron
(miles/backends/megatron_utils/initialize.py:72-136, "tp-cp-ep-dp-pp"); the record mirrors
`ParallelState` in miles/backends/training_utils/parallel.py:32-86.  Expert parallelism takes
`ep` consecutive ranks of the tp×cp×dp block of one pipeline stage (expert-TP is 1), the rest of
that block is expert-data-parallel.

The methods at the bottom are what model code calls.  With every size 1 they are plain ops.  With
TP/EP > 1 they route to `miles_b200.parallel.tp` / `.ep`, which run the fused sm_100a
compute+collective kernels on CUDA tensors and `torch.distributed` collectives (gloo) on CPU.
"""
from __future__ import annotations

import contextlib

from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist

from .. import ops


@dataclass
class ParallelState:
    world_size: int = 1
    rank: int = 0
    tp_size: int = 1
    cp_size: int = 1
    dp_size: int = 1
    pp_size: int = 1
    vpp_size: int = 1                 # model chunks per pipeline rank (interleaved schedule)
    ep_size: int = 1
    tp_rank: int = 0
    cp_rank: int = 0
    dp_rank: int = 0
    pp_rank: int = 0
    ep_rank: int = 0
    edp_size: int = 1
    edp_rank: int = 0
    sequence_parallel: bool = False
    cp_comm_type: str = "p2p"          # p2p (ring) | a2a (Ulysses) | allgather | a2a+p2p (hierarchical)
    cp_a2a_size: int = 1               # hierarchical CP: cp rank = p2p index · a2a size + a2a index
    cp_p2p_size: int = 1
    cp_a2a_group: Any = None
    cp_p2p_group: Any = None
    indep_dp_size: int = 1
    indep_dp_rank: int = 0
    # process groups (None when size 1 or not initialised)
    tp_group: Any = None
    cp_group: Any = None
    dp_group: Any = None
    pp_group: Any = None
    pp_fwd_group: Any = None          # interleaved schedule only: activations / gradients on communicators of their own
    pp_bwd_group: Any = None
    ep_group: Any = None
    edp_group: Any = None
    dp_cp_group: Any = None
    tp_dp_cp_group: Any = None
    world_group: Any = None
    gloo_group: Any = None
    # ranks of each group (global ranks), useful for p2p and fabrics
    tp_ranks: list[int] = field(default_factory=lambda: [0])
    ep_ranks: list[int] = field(default_factory=lambda: [0])
    dp_ranks: list[int] = field(default_factory=lambda: [0])
    pp_ranks: list[int] = field(default_factory=lambda: [0])
    cp_ranks: list[int] = field(default_factory=lambda: [0])
    fabric: Any = None                  # miles_b200.parallel.fabric.Fabric when CUDA + world>1
    fused: bool = True                  # False → NCCL + separate GEMM baseline path

    # ---------------------------------------------------------------------------------------
    @staticmethod
    def single() -> "ParallelState":
        return ParallelState()

    @property
    def is_ulysses_cp(self) -> bool:
        return self.cp_size > 1 and self.cp_comm_type == "a2a"

    @property
    def effective_dp(self) -> int:
        return self.dp_size * self.indep_dp_size

    @property
    def dp_cp_size(self) -> int:
        return self.dp_size * self.cp_size

    @property
    def is_pp_first(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_pp_last(self) -> bool:
        return self.pp_rank == self.pp_size - 1

    @staticmethod
    def coords(rank: int, tp: int, cp: int, dp: int, pp: int) -> tuple[int, int, int, int]:
        t = rank % tp
        c = (rank // tp) % cp
        d = (rank // (tp * cp)) % dp
        p = rank // (tp * cp * dp)
        return t, c, d, p

    @staticmethod
    def build(tp: int = 1, cp: int = 1, pp: int = 1, ep: int = 1, *, sequence_parallel: bool | None = None,
              cp_comm_type: str = "p2p", create_groups: bool = True, rank: int | None = None,
              world_size: int | None = None, vpp: int = 1, cp_hierarchy: tuple[int, int] | None = None) -> "ParallelState":
        """Create all groups.  Every rank must call this with identical arguments."""
        if world_size is None:
            world_size = dist.get_world_size() if dist.is_initialized() else 1
        if rank is None:
            rank = dist.get_rank() if dist.is_initialized() else 0
        assert world_size % (tp * cp * pp) == 0, f"world {world_size} not divisible by tp·cp·pp={tp * cp * pp}"
        dp = world_size // (tp * cp * pp)
        block = tp * cp * dp
        assert block % ep == 0, f"ep={ep} must divide tp·cp·dp={block}"
        t, c, d, p = ParallelState.coords(rank, tp, cp, dp, pp)
        ps = ParallelState(world_size=world_size, rank=rank, tp_size=tp, cp_size=cp, dp_size=dp, pp_size=pp,
                           ep_size=ep, tp_rank=t, cp_rank=c, dp_rank=d, pp_rank=p,
                           sequence_parallel=(tp > 1) if sequence_parallel is None else sequence_parallel,
                           cp_comm_type=cp_comm_type)
        ps.vpp_size = max(1, int(vpp or 1)) if pp > 1 else 1
        in_block = rank % block
        ps.ep_rank = in_block % ep
        ps.edp_size = block // ep
        ps.edp_rank = in_block // ep

        def idx(t_, c_, d_, p_):
            return t_ + tp * (c_ + cp * (d_ + dp * p_))

        groups = {
            "tp": [[idx(a, c_, d_, p_) for a in range(tp)] for p_ in range(pp) for d_ in range(dp) for c_ in range(cp)],
            "cp": [[idx(t_, a, d_, p_) for a in range(cp)] for p_ in range(pp) for d_ in range(dp) for t_ in range(tp)],
            "dp": [[idx(t_, c_, a, p_) for a in range(dp)] for p_ in range(pp) for c_ in range(cp) for t_ in range(tp)],
            "pp": [[idx(t_, c_, d_, a) for a in range(pp)] for d_ in range(dp) for c_ in range(cp) for t_ in range(tp)],
            "dp_cp": [[idx(t_, c_, d_, p_) for d_ in range(dp) for c_ in range(cp)] for p_ in range(pp) for t_ in range(tp)],
            "tp_dp_cp": [[p_ * block + i for i in range(block)] for p_ in range(pp)],
            "ep": [[p_ * block + g * ep + i for i in range(ep)] for p_ in range(pp) for g in range(block // ep)],
            "edp": [[p_ * block + g * ep + i for g in range(block // ep)] for p_ in range(pp) for i in range(ep)],
        }
        if cp_comm_type == "a2a+p2p":
            a2a, p2p = cp_hierarchy or (cp, 1)
            assert a2a * p2p == cp, f"hierarchical context parallel sizes {a2a} × {p2p} must multiply to cp = {cp}"
            ps.cp_a2a_size, ps.cp_p2p_size = a2a, p2p
            # inner groups: neighbouring cp ranks swap sequence for heads; outer groups: K/V travel round a ring of p2p members
            groups["cp_a2a"] = [g[o * a2a:(o + 1) * a2a] for g in groups["cp"] for o in range(p2p)]
            groups["cp_p2p"] = [g[i::a2a] for g in groups["cp"] for i in range(a2a)]
        if ps.vpp_size > 1:
            # interleaved schedule: activations and gradients travel on communicators of their own, so that each ordered pair
            # of ranks carries ONE stream per communicator (with two stages the wrap-around gradients share a direction with
            # the activations) and message order alone matches sends to receives
            groups["pp_fwd"] = [list(g) for g in groups["pp"]]
            groups["pp_bwd"] = [list(g) for g in groups["pp"]]
        from .reloadable import REGISTRY

        for name, lists in groups.items():
            for ranks in lists:
                ranks_sorted = list(ranks)
                handle = None
                if create_groups and dist.is_initialized() and len(ranks_sorted) > 1:
                    handle = REGISTRY.new_group(ranks_sorted)      # recorded: `release_groups` / `reload_groups` below
                if rank in ranks_sorted:
                    setattr(ps, f"{name}_group", handle)
                    REGISTRY.bind(ps, f"{name}_group")
                    if name in ("tp", "ep", "dp", "pp", "cp"):
                        setattr(ps, f"{name}_ranks", ranks_sorted)
        if dist.is_initialized():
            ps.world_group = dist.group.WORLD
        return ps

    @staticmethod
    def release_groups() -> int:
        """Destroy every communicator made by `build` (their device buffers go back to the allocator); every rank calls
        this at the same point.  Collectives are unavailable until `reload_groups`."""
        from .reloadable import REGISTRY

        return REGISTRY.destroy_all() if dist.is_initialized() else 0

    @staticmethod
    def reload_groups() -> int:
        from .reloadable import REGISTRY

        return REGISTRY.reload_all() if dist.is_initialized() else 0

    # ---------------------------------------------------------------------------------------
    # entry points used by the model
    # ---------------------------------------------------------------------------------------
    def column_linear(self, x, w, bias=None):
        """y = gather_seq(x) · wᵀ with w sharded along its output rows."""
        if self.tp_size == 1:
            return ops.linear(x, w, bias)
        from . import tp
        return tp.column_parallel_linear(x, w, bias, self)

    def row_linear(self, x, w):
        """y = reduce(x · wᵀ) with w sharded along its input columns; scattered over seq with SP."""
        if self.tp_size == 1:
            return ops.linear(x, w)
        from . import tp
        return tp.row_parallel_linear(x, w, self)

    def defer_allreduce(self, x) -> bool:
        """True where a row-parallel projection may hand on its UNREDUCED partial sums because the next op is the fused
        all-reduce + residual add + RMSNorm kernel over peer memory: tensor-parallel inference (replicated activations,
        no autograd) on CUDA with the NVLink fabric up — the rollout engine's prefill and decode."""
        return (self.tp_size > 1 and not self.sequence_parallel and self.fabric is not None and self.fused and x.is_cuda
                and x.dtype == torch.bfloat16 and not torch.is_grad_enabled())

    def row_linear_partial(self, x, w):
        """This rank's partial sums of a row-parallel projection, marked so that the consumer reduces them."""
        y = ops.linear(x, w)
        y._tp_partial = True
        return y

    def allreduce_add_rmsnorm(self, partial, residual, w, eps):
        """(rmsnorm(Σ_ranks partial + residual)·w, Σ_ranks partial + residual) in the fused peer-memory kernel(s)."""
        return self.fabric.allreduce_add_rmsnorm(partial, residual, w, eps, self)

    def sp_gather(self, x):
        if self.tp_size == 1 or not self.sequence_parallel:
            return x
        from . import tp
        return tp.gather_sequence(x, self)

    @contextlib.contextmanager
    def no_sequence_parallel(self):
        """Run tensor-parallel layers with replicated activations (all-reduce instead of reduce-scatter/all-gather)."""
        # the engine also ignores context parallelism: CP ranks serve disjoint requests like data-parallel ranks
        old, old_cp = self.sequence_parallel, self.cp_size
        self.sequence_parallel, self.cp_size = False, 1
        try:
            yield self
        finally:
            self.sequence_parallel, self.cp_size = old, old_cp

    def sp_scatter(self, x):
        if self.tp_size == 1 or not self.sequence_parallel:
            return x
        from . import tp
        return tp.scatter_sequence(x, self)

    def sp_slice(self, x):
        """Non-differentiable slice of a per-token tensor to this rank's SP chunk."""
        if self.tp_size == 1 or not self.sequence_parallel:
            return x
        n = x.shape[0] // self.tp_size
        return x[self.tp_rank * n:(self.tp_rank + 1) * n]

    def tp_all_gather_last(self, x):
        if self.tp_size == 1:
            return x
        from . import tp
        return tp.all_gather_last_dim(x, self)

    def moe_ffn(self, x, w13, w2, topk_w, topk_idx, num_experts):
        if self.ep_size == 1:
            return ops.moe_ffn(x, w13, w2, topk_w, topk_idx)
        from . import ep
        return ep.expert_parallel_ffn(x, w13, w2, topk_w, topk_idx, num_experts, self)

    def vocab_parallel_logprob(self, hidden, w, targets, temperature, with_entropy, vocab_size):
        if self.tp_size == 1:
            return ops.logprob_entropy(hidden, w, targets, temperature, with_entropy)
        from . import tp
        return tp.vocab_parallel_logprob(hidden, w, targets, temperature, with_entropy, self)


def init_distributed(backend: str | None = None, timeout_s: float = 1800.0) -> tuple[int, int, int]:
    """Join the default process group from torchrun-style env vars. Returns (rank, world, local_rank)."""
    import datetime
    import os

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s))
    elif torch.cuda.is_available():
        torch.cuda.set_device(local)
    return rank, world, local
