"""Ring (zigzag) and all-gather context-parallel attention vs single-rank attention, forward and gradients (gloo ranks)."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from dist_utils import run_distributed  # noqa: E402


def _body(rank, world, comm, cp_size):
    sys.path.insert(0, ROOT)
    from miles_b200.ops import reference as ref
    from miles_b200.parallel import cp_ring
    from miles_b200.parallel.state import ParallelState

    ps = ParallelState.build(cp=cp_size, cp_comm_type=comm, cp_hierarchy=(2, cp_size // 2) if comm == "a2a+p2p" else None)
    torch.manual_seed(0)                                   # same tensors on every rank
    lens = [7, 12, 5]                                      # 24 real tokens + 8 padding tokens
    T, Hq, Hkv, D = 32, 4, 2, 8
    cu = torch.tensor([0, 7, 19, 24], dtype=torch.int32)
    q, k, v = (torch.randn(T, h, D, dtype=torch.float64).float().requires_grad_() for h in (Hq, Hkv, Hkv))
    g = torch.randn(T, Hq, D)
    # single-rank answer over the real tokens (padding rows are not compared)
    o_ref = ref.attention_varlen(q[:24], k[:24], v[:24], cu, True)
    o_ref.backward(g[:24])
    gq, gk, gv = q.grad.clone(), k.grad.clone(), v.grad.clone()
    own = cp_ring.token_index(T, ps)
    assert own.numel() == T // cp_size
    ql, kl, vl = (t.detach()[own].clone().requires_grad_() for t in (q, k, v))
    fn = {"allgather": cp_ring.allgather_attention, "a2a+p2p": cp_ring.hierarchical_attention}.get(comm, cp_ring.ring_attention)
    o = fn(ql, kl, vl, cu, ps)
    real = own < 24
    assert torch.allclose(o[real], o_ref.detach()[own[real]], atol=1e-5), (o[real] - o_ref.detach()[own[real]]).abs().max()
    gl = g[own].clone()
    gl[~real] = 0                                          # padding rows carry no loss
    o.backward(gl)
    assert torch.allclose(ql.grad[real], gq[own[real]], atol=1e-5)
    assert torch.allclose(kl.grad[real], gk[own[real]], atol=1e-5)
    assert torch.allclose(vl.grad[real], gv[own[real]], atol=1e-5)


@pytest.mark.parametrize("comm,world", [("p2p", 2), ("allgather", 2), ("p2p", 4), ("a2a+p2p", 4), ("a2a+p2p", 2)])
def test_cp_attention_matches_single_rank(comm, world):
    run_distributed(_body, world, (comm, world), timeout=300)


def test_zigzag_layout_covers_every_token_once():
    from miles_b200.parallel import cp_ring

    parts = [cp_ring.rank_token_index(32, 4, r, "zigzag") for r in range(4)]
    assert sorted(torch.cat(parts).tolist()) == list(range(32))
    assert parts[0].tolist() == [0, 1, 2, 3, 28, 29, 30, 31]      # first and last piece: balanced causal work
