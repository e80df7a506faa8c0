"""Semantics the trainer shares with the reference, each checked against a per-sample python statement written the way
the reference computes it: terminal reward at the last trainable token, removed samples kept with a zero mask, one
reward vote per rollout, equal micro-batch counts on every DP rank, KL estimator details, the weight-transfer mode map.
"""
from types import SimpleNamespace

import pytest
import torch

from miles_b200.train import math_utils as mu
from miles_b200.train.advantages import compute_advantages_and_returns
from miles_b200.train.data import convert_samples_to_train_data, make_micro_batches
from miles_b200.types import Sample

from dist_utils import run_distributed


def _args(**kw):
    base = dict(advantage_estimator="grpo", kl_coef=0.0, gamma=1.0, lambd=1.0, normalize_advantages=False,
                rewards_normalization=True, grpo_std_normalization=True, n_samples_per_prompt=4)
    base.update(kw)
    return SimpleNamespace(**base)


def _scan_returns(tok_r, gamma):
    out = torch.zeros_like(tok_r)
    run = 0.0
    for t in reversed(range(len(tok_r))):
        run = tok_r[t] + gamma * run
        out[t] = run
    return out


def test_terminal_reward_sits_at_last_trainable_token_reinforce_pp():
    # response ends in two masked tokens (tool output): the reward belongs to token 1, not token 3
    lens = [4, 3]
    mask = torch.tensor([1, 1, 0, 0, 1, 0, 1], dtype=torch.float32)
    rewards = torch.tensor([1.0, 2.0])
    args = _args(advantage_estimator="reinforce_plus_plus", gamma=0.5)
    adv, ret = compute_advantages_and_returns(args, rewards=rewards, response_lengths=lens, loss_mask=mask)
    exp = []
    off = 0
    for r, n in zip(rewards.tolist(), lens):
        m = mask[off:off + n]
        tok = torch.zeros(n)
        tok[m.nonzero()[-1]] += r
        exp.append(_scan_returns(tok, 0.5))
        off += n
    exp = torch.cat(exp)
    assert torch.allclose(ret, exp), (ret, exp)
    assert torch.allclose(adv, exp * (mask > 0))
    assert ret[0].item() == pytest.approx(0.5) and ret[1].item() == pytest.approx(1.0)


def test_terminal_reward_reaches_ppo_gae_with_masked_tail():
    lens = [4]
    mask = torch.tensor([1, 1, 0, 0], dtype=torch.float32)
    values = torch.tensor([0.1, 0.2, 0.3, 0.4])
    args = _args(advantage_estimator="ppo", gamma=0.9, lambd=0.8)
    adv, ret = compute_advantages_and_returns(args, rewards=torch.tensor([1.0]), response_lengths=lens, loss_mask=mask,
                                              values=values)
    # per-sample statement: compress to trainable tokens, reward on the last of them, plain GAE scan
    v = values[:2]
    r = torch.tensor([0.0, 1.0])
    a_ref, _ = mu.vanilla_gae(r[None], v[None], 0.9, 0.8)
    assert torch.allclose(adv[:2], a_ref[0], atol=1e-6)
    assert adv[:2].abs().sum() > 0 and torch.all(adv[2:] == 0)
    # a fully masked sample gives zero advantages
    adv0, _ = compute_advantages_and_returns(args, rewards=torch.tensor([1.0]), response_lengths=[3],
                                             loss_mask=torch.zeros(3), values=torch.zeros(3))
    assert torch.all(adv0 == 0)


def _sample(i, g, reward, n_resp=3, rollout_id=None, remove=False):
    s = Sample(group_index=g, index=i, tokens=[5, 6] + [7] * n_resp)
    s.response_length = n_resp
    s.reward = reward
    s.rollout_id = rollout_id
    s.remove_sample = remove
    return s


def test_removed_samples_stay_with_zero_mask_and_count_in_group_stats():
    group = [_sample(0, 0, 1.0), _sample(1, 0, 0.0, remove=True), _sample(2, 0, 0.0), _sample(3, 0, 1.0)]
    data = convert_samples_to_train_data(_args(), [group])
    assert len(data["tokens"]) == 4
    assert data["loss_masks"][1] == [0, 0, 0] and data["loss_masks"][0] == [1, 1, 1]
    raw = torch.tensor([1.0, 0.0, 0.0, 1.0])
    exp = (raw - raw.mean()) / (raw.std() + 1e-6)
    assert torch.allclose(torch.tensor(data["rewards"]), exp, atol=1e-6)
    assert data["rollout_mask_sums"][1] == 0


def test_rewards_normalised_once_per_rollout():
    # rollout 10 was split into two training rows; it votes once in the group statistics
    group = [_sample(0, 0, 1.0, rollout_id=10), _sample(1, 0, 1.0, rollout_id=10), _sample(2, 0, 0.0, rollout_id=11),
             _sample(3, 0, 0.5, rollout_id=12)]
    data = convert_samples_to_train_data(_args(), [group])
    shared = torch.tensor([1.0, 0.0, 0.5])
    n = (shared - shared.mean()) / (shared.std() + 1e-6)
    assert torch.allclose(torch.tensor(data["rewards"]), torch.stack([n[0], n[0], n[1], n[2]]), atol=1e-6)
    bad = [_sample(0, 0, 1.0, rollout_id=10), _sample(1, 0, 0.0, rollout_id=10)]
    with pytest.raises(ValueError, match="share one reward"):
        convert_samples_to_train_data(_args(), [bad])


def _uneven_counts(rank, world):
    import torch.distributed as dist

    args = SimpleNamespace(use_dynamic_batch_size=False, micro_batch_size=1)
    lengths = [10, 20, 30, 40] if rank == 0 else [10, 20, 30]
    parts = make_micro_batches(args, lengths, dp_group=dist.group.WORLD)
    assert len(parts) == 4, (rank, parts)
    assert sorted(i for p in parts for i in p) == list(range(len(lengths)))
    empty = make_micro_batches(args, [] if rank == 1 else [5, 5], dp_group=dist.group.WORLD)
    assert len(empty) == 2 and (rank == 0 or all(p == [] for p in empty))
    dyn = SimpleNamespace(use_dynamic_batch_size=True, max_tokens_per_gpu=32)
    parts = make_micro_batches(dyn, [30, 30, 30] if rank == 0 else [8], dp_group=dist.group.WORLD)
    assert len(parts) == 3


def test_micro_batch_counts_equal_across_uneven_dp_ranks():
    run_distributed(_uneven_counts, world_size=2)


def test_low_var_kl_clamps_after_the_ratio():
    lp = torch.tensor([0.0, -3.0, 2.0])
    base = torch.tensor([-6.0, 3.0, 2.0])
    ratio = torch.tensor([4.0, 4.0, 1.0])
    d = -(lp - base)
    exp = torch.clamp(ratio * (d.exp() - 1 - d), -10, 10)
    got = mu.compute_approx_kl(lp, base, "low_var_kl", ratio)
    assert torch.allclose(got, exp)
    assert got[1].item() == 10.0           # clamped after the multiply


def test_opsm_masks_per_token_on_advantage_sign():
    # one sequence, mean KL above delta; only the tokens with a negative advantage are dropped
    lp = torch.zeros(4)
    old = torch.full((4,), 0.5)
    adv = torch.tensor([1.0, -1.0, -2.0, 3.0])
    mask = torch.ones(4)
    seq_ids = torch.zeros(4, dtype=torch.long)
    keep, frac = mu.compute_opsm_mask(lp, old, adv, mask, seq_ids, 1, delta=0.1)
    assert keep.tolist() == [1.0, 0.0, 0.0, 1.0]
    assert frac.item() == pytest.approx(0.5)
    keep, _ = mu.compute_opsm_mask(lp, old, adv, mask, seq_ids, 1, delta=1.0)
    assert keep.tolist() == [1.0] * 4


def test_unbiased_kl_ratio_carries_gradient():
    from miles_b200.train import losses

    src = open(losses.__file__).read()
    assert "ratio = torch.exp((log_probs - old).clamp(-20, 20))  " in src and ".clamp(-20, 20)).detach()" not in src
    lp = torch.tensor([-1.0, -2.0], requires_grad=True)
    old = torch.tensor([-1.2, -1.5])
    ref = torch.tensor([-0.7, -2.5])
    ratio = torch.exp(lp - old)
    mu.compute_approx_kl(lp, ref, "k3", ratio).sum().backward()
    g_live = lp.grad.clone()
    lp.grad = None
    mu.compute_approx_kl(lp, ref, "k3", ratio.detach()).sum().backward()
    assert not torch.allclose(g_live, lp.grad)


class _FakeEngine:
    def __init__(self, model=None):
        if model is not None:
            self.model = model
        self.paused = False
        self.version = 0
        self.calls = []

    def pause_generation(self, mode="retract"):
        self.paused = True

    def continue_generation(self):
        self.paused = False

    def flush_cache(self):
        return True

    def update_weight_version(self, v):
        self.version = v

    def get_weight_version(self):
        return self.version


def test_every_cli_transfer_mode_maps_to_an_implementation():
    from miles_b200.args import build_parser
    from miles_b200.weight_update.updater import CLI_MODES, WeightUpdater

    parser = build_parser()
    action = next(a for a in parser._actions if a.dest == "update_weight_transfer_mode")
    model = torch.nn.Linear(2, 2)
    actor = SimpleNamespace(model=model, device=torch.device("cpu"), weight_version=3, args=None,
                            ps=SimpleNamespace(tp_size=1, ep_size=1, pp_size=1, tp_rank=0, ep_rank=0, pp_rank=0))
    for choice in action.choices:
        eng = _FakeEngine(model)
        eng.ps = actor.ps
        up = WeightUpdater(SimpleNamespace(update_weight_transfer_mode=choice), actor, [eng])
        assert hasattr(up, f"_send_{up.mode}"), choice
        if choice != "auto":
            assert up.mode == CLI_MODES[choice]
    assert WeightUpdater(SimpleNamespace(update_weight_transfer_mode="broadcast_packed"), actor, [_FakeEngine(model)]).packed
    with pytest.raises(ValueError, match="needs\\s+the engine in this process"):
        WeightUpdater(SimpleNamespace(update_weight_transfer_mode="p2p"), actor, [_FakeEngine()])
    with pytest.raises(ValueError, match="unknown weight transfer mode"):
        WeightUpdater(SimpleNamespace(), actor, [_FakeEngine(model)], mode="carrier_pigeon")


def test_failed_transfer_leaves_engines_running():
    from miles_b200.weight_update.updater import WeightUpdater

    model = torch.nn.Linear(2, 2)
    actor = SimpleNamespace(model=model, device=torch.device("cpu"), weight_version=1, args=None)
    eng = _FakeEngine(model)
    up = WeightUpdater(SimpleNamespace(update_weight_transfer_mode="alias"), actor, [eng])
    up._send_alias = lambda: (_ for _ in ()).throw(RuntimeError("link down"))
    with pytest.raises(RuntimeError, match="link down"):
        up.update_weights()
    assert eng.paused is False and eng.version == 0


def test_custom_step_runner_is_used(tmp_path):
    """--custom-step-runner-path: the trainer's forwards and backwards go through the plugged runner."""
    import sys
    import textwrap

    mod = tmp_path / "my_runner.py"
    mod.write_text(textwrap.dedent("""
        from miles_b200.train.step_runner import LinearStepRunner

        CALLS = {"fwd": 0, "fwd_bwd": 0}

        class Counting(LinearStepRunner):
            def forward_only_step(self, mbs, pack, compute, *, replay=False):
                CALLS["fwd"] += 1
                return super().forward_only_step(mbs, pack, compute, replay=replay)

            def forward_backward_step(self, mbs, pack, score, *, want_ent, replay):
                CALLS["fwd_bwd"] += 1
                return super().forward_backward_step(mbs, pack, score, want_ent=want_ent, replay=replay)

        def build(actor):
            return Counting(actor)
    """))
    sys.path.insert(0, str(tmp_path))
    try:
        from test_e2e import _run

        h = _run("--custom-step-runner-path my_runner.build --num-rollout 1")
        import my_runner

        assert my_runner.CALLS["fwd"] >= 1 and my_runner.CALLS["fwd_bwd"] >= 1 and h.series("train/grad_norm")[0] > 0
    finally:
        sys.path.remove(str(tmp_path))


# ---- virtual pipeline (interleaved schedule): gradients equal the unpartitioned model's --------------------------------

def _vpp_body(rank, world, out_dir):
    import types

    import torch

    from miles_b200.models.config import PRESETS
    from miles_b200.models.qwen3 import ForwardMeta, build_model
    from miles_b200.parallel.state import ParallelState, init_distributed
    from miles_b200.train.data import pack_micro_batch
    from miles_b200.train.step_runner import InterleavedStepRunner

    init_distributed(backend="gloo")
    ps = ParallelState.build(pp=2, vpp=2)
    cfg = PRESETS["tiny"].with_(num_layers=5)              # 5 layers over 4 virtual stages: the first takes two
    model = build_model(cfg, ps, dtype=torch.float32, device="cpu", seed=3)
    assert [c.layer_range for c in model.chunks] == ([(0, 2), (3, 4)] if rank == 0 else [(2, 3), (4, 5)])
    g = torch.Generator().manual_seed(1)
    shard = {"tokens": [torch.randint(3, cfg.vocab_size, (int(n),), generator=g).tolist() for n in (9, 12, 7, 10, 8, 11)],
             "response_lengths": [4, 5, 3, 6, 2, 5]}
    shard["total_lengths"] = [len(t) for t in shard["tokens"]]
    shard["loss_masks"] = [[1] * r for r in shard["response_lengths"]]
    mbs = [[0, 1], [2], [3, 4], [5]]

    class A:
        pass

    a = A()
    a.ps, a.cfg, a.model, a.device = ps, cfg, model, torch.device("cpu")
    a._meta = lambda pb, replay: ForwardMeta(positions=pb.positions, cu_seqlens=pb.cu_seqlens, max_seqlen=pb.max_seqlen)

    def score_hidden(pb, hidden, with_entropy):
        return model.log_probs(hidden[pb.gather_index], pb.targets, 1.0, with_entropy)

    a._score_hidden = score_hidden
    runner = InterleavedStepRunner(a)
    pack = lambda idx: pack_micro_batch(shard, idx, "cpu", pad_multiple=1)
    weights = {0: 1.0, 1: -0.5, 2: 2.0, 3: 0.25}
    key = {id(m): i for i, m in enumerate(mbs)}
    runner.forward_backward_step(mbs, pack, lambda pb, idx, out, ent: out.sum() * weights[key[id(idx)]], want_ent=False, replay=False)
    grads = {n: p.grad.clone() for n, p in model.named_parameters_global() if p.grad is not None}
    lps = runner.forward_only_step(mbs, pack, lambda pb, idx, lp: lp.clone(), replay=False)
    torch.save({"grads": grads, "lps": lps}, f"{out_dir}/r{rank}.pt")


def test_interleaved_virtual_pipeline_matches_the_unpartitioned_model(tmp_path):
    import os
    import sys

    import torch

    sys.path.insert(0, os.path.dirname(__file__))
    from dist_utils import run_distributed

    from miles_b200.models.config import PRESETS
    from miles_b200.models.qwen3 import ForwardMeta, build_model
    from miles_b200.parallel.state import ParallelState
    from miles_b200.train.data import pack_micro_batch

    run_distributed(_vpp_body, 2, (str(tmp_path),), timeout=300)
    cfg = PRESETS["tiny"].with_(num_layers=5)
    model = build_model(cfg, ParallelState.single(), dtype=torch.float32, device="cpu", seed=3)
    g = torch.Generator().manual_seed(1)
    shard = {"tokens": [torch.randint(3, cfg.vocab_size, (int(n),), generator=g).tolist() for n in (9, 12, 7, 10, 8, 11)],
             "response_lengths": [4, 5, 3, 6, 2, 5]}
    shard["total_lengths"] = [len(t) for t in shard["tokens"]]
    shard["loss_masks"] = [[1] * r for r in shard["response_lengths"]]
    mbs, weights = [[0, 1], [2], [3, 4], [5]], [1.0, -0.5, 2.0, 0.25]
    want_lp = []
    for idx, w in zip(mbs, weights):
        pb = pack_micro_batch(shard, idx, "cpu", pad_multiple=1)
        h = model(pb.tokens, ForwardMeta(positions=pb.positions, cu_seqlens=pb.cu_seqlens, max_seqlen=pb.max_seqlen))
        lp, _ = model.log_probs(h[pb.gather_index], pb.targets)
        (lp.sum() * w).backward()
        want_lp.append(lp.detach())
    want = {n: p.grad for n, p in model.named_parameters()}
    got = {}
    outs = [torch.load(f"{tmp_path}/r{r}.pt") for r in range(2)]
    for o in outs:
        assert not (set(o["grads"]) & set(got)), "a parameter lives on one virtual stage only"
        got.update(o["grads"])
    assert set(got) == set(want), (sorted(set(want) - set(got)), sorted(set(got) - set(want)))
    for n in want:
        assert torch.allclose(got[n], want[n], rtol=1e-4, atol=1e-5), n
    for o in outs:                                                   # forward-only: every stage ends with the same record
        for a, b in zip(o["lps"], want_lp):
            assert torch.allclose(a, b, rtol=1e-4, atol=1e-5)
