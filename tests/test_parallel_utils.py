"""Context-parallel helpers, routing-replay manager and metric reduction (CPU; collectives over gloo ranks)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402

from miles_b200.parallel import cp  # noqa: E402
from miles_b200.train import metrics as M  # noqa: E402
from miles_b200.train.replay import ReplayManager  # noqa: E402


def test_zigzag_and_contiguous_slicing_roundtrip():
    x = torch.arange(16)
    assert cp.slice_with_cp(x, 2, 1).tolist() == list(range(8, 16))
    z0, z1 = cp.slice_with_cp(x, 2, 0, "zigzag"), cp.slice_with_cp(x, 2, 1, "zigzag")
    assert z0.tolist() == [0, 1, 2, 3, 12, 13, 14, 15] and z1.tolist() == [4, 5, 6, 7, 8, 9, 10, 11]
    perm = cp.zigzag_to_contiguous_index(16, 2)
    assert torch.equal(torch.cat([z0, z1])[perm], x)


def test_sum_of_sample_mean():
    x = torch.tensor([1.0, 3.0, 10.0, 20.0, 30.0])
    mask = torch.tensor([1.0, 1.0, 1.0, 0.0, 1.0])
    ids = torch.tensor([0, 0, 1, 1, 1])
    assert float(cp.sum_of_sample_mean(x, mask, ids, 2)) == 2.0 + 20.0
    assert float(cp.sum_of_sample_mean(x, mask, ids, 2, denominators=torch.tensor([4.0, 4.0]))) == 1.0 + 10.0


def _cp_body(rank, world):
    import torch.distributed as dist

    from miles_b200.parallel.state import ParallelState

    ps = ParallelState.build(cp=2, cp_comm_type="a2a")
    torch.manual_seed(0)
    T, H, D = 8, 4, 3
    full = torch.randn(T, H, D)
    mine = full[rank * 4:(rank + 1) * 4].clone().requires_grad_()
    heads = cp.seq_to_heads(mine, ps)                                   # [T, H/cp, D]: all tokens, my two heads
    assert torch.equal(heads, full[:, rank * 2:(rank + 1) * 2])
    back = cp.heads_to_seq(heads, ps)
    assert torch.equal(back, mine)
    (back * torch.arange(4.0).view(4, 1, 1)).sum().backward()           # gradient crosses both all-to-alls
    assert torch.equal(mine.grad, torch.arange(4.0).view(4, 1, 1).expand(4, H, D))
    # differentiable assembly of per-token values
    sel = torch.zeros(6, dtype=torch.bool)
    sel[rank * 3:(rank + 1) * 3] = True
    local = (torch.arange(3.0) + 10 * rank).requires_grad_()
    out = cp.gather_from_cp(local, sel, 6, ps)
    assert out.tolist() == [0.0, 1.0, 2.0, 10.0, 11.0, 12.0]
    (out * torch.arange(6.0)).sum().backward()
    assert local.grad.tolist() == [0.0 + 3 * rank, 1.0 + 3 * rank, 2.0 + 3 * rank]
    # metric reduction with a key only one rank has
    sums = {"a": 2.0 * (rank + 1), **({"only0": 5.0} if rank == 0 else {})}
    red = M.reduce_log_dict(sums, 2.0, group=dist.group.WORLD)
    assert abs(red["a"] - (2.0 + 4.0) / 4.0) < 1e-9 and abs(red["only0"] - 2.5) < 1e-9


def test_cp_collectives_two_ranks():
    run_distributed(_cp_body, 2)


def test_replay_manager_stages():
    torch.manual_seed(0)

    def topk(scores, k):
        w, i = scores.topk(k, dim=-1)
        return w / w.sum(-1, keepdim=True), i

    mgr = ReplayManager(normalize=True)
    routed = mgr.wrap(topk)
    s1, s2 = torch.rand(5, 8), torch.rand(5, 8)
    mgr.set_stage("record")
    _, i1 = routed(s1, 2)
    _, i2 = routed(s2, 2)
    rec = mgr.stacked_record()
    assert rec.shape == (5, 2, 2) and torch.equal(rec[:, 0].long(), i1)
    # replay against different scores: indices are the recorded ones, weights come from the new scores
    t1 = torch.rand(5, 8, requires_grad=True)
    rec[3] = -1                                                         # a padding row falls through to live top-k
    mgr.load_packed(rec)
    mgr.set_stage("replay_forward")
    w, idx = routed(t1, 2)
    assert torch.equal(idx[:3], i1[:3]) and torch.equal(idx[3], t1[3].topk(2).indices)
    want = t1.gather(1, idx)
    assert torch.allclose(w, want / want.sum(-1, keepdim=True))
    w.sum().backward()
    assert t1.grad is not None
    routed(torch.rand(5, 8), 2)
    mgr.set_stage("replay_backward")                                    # recomputation replays the same record again
    _, idx_b = routed(t1.detach(), 2)
    assert torch.equal(idx_b[:3], i1[:3])
    mgr.set_stage("fallthrough")
    assert torch.equal(routed(s2, 2)[1], i2)


def test_perf_and_rollout_stats(tmp_path):
    from miles_b200.models.config import PRESETS

    p = M.perf_metrics(PRESETS["qwen3-30B-A3B"], num_tokens=100_000, seq_len_mean=2048, seconds=2.0, n_gpus=8, peak_tflops=2250.0)
    assert p["perf/actor_train_tok_per_s"] == 50_000 and 0 < p["perf/actor_train_mfu"] < 1
    st = M.rollout_data_stats({"response_lengths": [2, 4], "total_lengths": [5, 9], "rewards": [1.0, -1.0], "raw_reward": [1.0, 0.0],
                               "truncated": [0, 1], "loss_masks": [[1, 0], [1, 1, 1, 1]], "weight_versions": [3, 4]})
    assert st["rollout/response_len/mean"] == 3 and st["rollout/truncated_ratio"] == 0.5 and st["rollout/weight_version/min"] == 3.0
    path = str(tmp_path / "gn.json")
    rec = M.GradNormRecorder(path, "record")
    rec.step(0, 1.5)
    rec.step(1, 2.5)
    rep = M.GradNormRecorder(path, "replay")
    rep.step(1, 2.5)
    try:
        rep.step(0, 1.6)
        raise SystemExit("mismatch not detected")
    except AssertionError:
        pass
    M.check_kl_zero_at_step0(torch.zeros(3), torch.zeros(3))


# ---- reloadable process groups ----------------------------------------------------------------------------------------

def _reload_body(rank, world):
    import torch
    import torch.distributed as dist

    from miles_b200.parallel.reloadable import REGISTRY
    from miles_b200.parallel.state import ParallelState

    ps = ParallelState.build(tp=2)                 # world 4: tp groups {0,1},{2,3}; dp groups {0,2},{1,3}

    class Holder:
        pass

    h = Holder()
    h.group = ps.dp_group
    assert REGISTRY.bind(h, "group") and not REGISTRY.bind(h, "missing")
    x = torch.ones(1) * (rank + 1)
    dist.all_reduce(x, group=ps.tp_group)
    assert x.item() == (3 if rank < 2 else 7)
    n = ps.release_groups()
    assert n > 0 and ps.tp_group is None and ps.dp_group is None and h.group is None and REGISTRY.released
    y = torch.ones(1)
    dist.all_reduce(y)                              # the world group stays
    assert y.item() == world
    assert ps.reload_groups() == n and not REGISTRY.released
    assert ps.tp_group is not None and h.group is ps.dp_group
    z = torch.ones(1) * (rank + 1)
    dist.all_reduce(z, group=h.group)
    assert z.item() == (4 if rank % 2 == 0 else 6)
    assert ps.reload_groups() == 0                  # nothing left to re-create


def test_process_groups_release_and_reload():
    from dist_utils import run_distributed

    run_distributed(_reload_body, 4)
