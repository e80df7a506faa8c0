"""Loss, advantage and math utilities against closed forms and naive loops (CPU).

Mirrors the reference's unit layer (tests/fast/backends/training_utils: GAE vs vanilla loop, PPO clip, KL estimators,
loss scaling invariance to the micro-batch split).
"""
import math
from types import SimpleNamespace

import pytest
import torch

from miles_b200.train import advantages as A
from miles_b200.train import losses as L
from miles_b200.train import math_utils as mu


def _args(**kw):
    base = dict(advantage_estimator="grpo", eps_clip=0.2, eps_clip_high=0.2, eps_clip_c=None, entropy_coef=0.0,
                use_kl_loss=False, kl_loss_coef=0.0, kl_loss_type="k1", kl_coef=0.0, gamma=1.0, lambd=1.0,
                normalize_advantages=False, calculate_per_token_loss=False, use_tis=False, use_opsm=False,
                loss_type="policy_loss", value_clip=0.2, grpo_std_normalization=True, rewards_normalization=True,
                get_mismatch_metrics=False, use_rollout_logprobs=False, custom_loss_function_path=None,
                custom_tis_function_path=None, tis_clip=2.0, tis_clip_low=0.0, opsm_delta=1e-4, opd_kl_coef=0.0)
    base.update(kw)
    return SimpleNamespace(**base)


def _batch(lengths, **kw):
    R = sum(lengths)
    seq_ids = mu.lengths_to_seq_ids(lengths, "cpu")
    return L.LossBatch(response_lengths=lengths, loss_mask=kw.pop("loss_mask", torch.ones(R)), seq_ids=seq_ids, **kw)


@pytest.mark.parametrize("kind", ["k1", "k2", "k3", "low_var_kl"])
def test_kl_estimators(kind):
    torch.manual_seed(0)
    lp, base = -torch.rand(64), -torch.rand(64)
    kl = mu.compute_approx_kl(lp, base, kind)
    d = lp - base
    if kind == "k1":
        want = d
    elif kind == "k2":
        want = d * d / 2
    else:
        want = torch.exp(-d) - 1 + d
        if kind == "low_var_kl":
            want = want.clamp(-10, 10)
    torch.testing.assert_close(kl, want)
    assert mu.compute_approx_kl(lp, lp, kind).abs().max() == 0


def test_policy_loss_clip_and_dual_clip():
    ppo_kl = torch.tensor([0.0, -0.5, 0.5, -2.0])        # log(old/new)
    adv = torch.tensor([1.0, 1.0, -1.0, -1.0])
    loss, clipfrac = mu.compute_policy_loss(ppo_kl, adv, 0.2, 0.2)
    ratio = torch.exp(-ppo_kl)
    want = torch.maximum(-adv * ratio, -adv * ratio.clamp(0.8, 1.2))
    torch.testing.assert_close(loss, want)
    assert clipfrac.shape == loss.shape
    loss_c, _ = mu.compute_policy_loss(ppo_kl, adv, 0.2, 0.2, 3.0)
    # dual clip bounds the loss of negative-advantage tokens by c·|A|
    assert loss_c[3] <= 3.0 + 1e-6 and loss[3] > 3.0


def test_chunked_gae_matches_vanilla():
    torch.manual_seed(1)
    for T in (1, 7, 128, 300):
        r, v = torch.randn(3, T), torch.randn(3, T)
        a1, ret1 = mu.vanilla_gae(r, v, 0.97, 0.9)
        a2, ret2 = mu.chunked_gae(r, v, 0.97, 0.9, chunk=64)
        torch.testing.assert_close(a1, a2, atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(ret1, ret2, atol=1e-4, rtol=1e-4)


def test_masked_gae_skips_masked_tokens():
    lengths = [5, 3]
    mask = torch.tensor([1, 1, 0, 0, 1, 1, 0, 1.0])
    tok_r = torch.zeros(8)
    tok_r[4] = 1.0
    tok_r[7] = -1.0
    values = torch.zeros(8)
    adv, ret = mu.masked_gae(tok_r, values, mask, lengths, 1.0, 1.0)
    # with γ=λ=1 and zero values every unmasked token sees the final reward
    torch.testing.assert_close(adv[mask > 0], torch.tensor([1.0, 1.0, 1.0, -1.0, -1.0]))


def test_grpo_advantages_and_group_norm():
    args = _args()
    rewards = torch.tensor([1.0, 0.0, 1.0, 1.0])
    normed = A.normalize_group_rewards(args, rewards, [2, 2])
    assert abs(normed[0] + normed[1]) < 1e-6
    assert normed[2] == 0 and normed[3] == 0                      # zero std → only centred
    adv, ret = A.compute_advantages_and_returns(args, rewards=normed, response_lengths=[3, 2, 1, 1],
                                                loss_mask=torch.ones(7))
    torch.testing.assert_close(adv[:3], normed[0].expand(3))
    torch.testing.assert_close(adv[3:5], normed[1].expand(2))


def test_reinforce_pp_returns():
    args = _args(advantage_estimator="reinforce_plus_plus", gamma=0.5, kl_coef=0.0)
    adv, ret = A.compute_advantages_and_returns(args, rewards=torch.tensor([8.0]), response_lengths=[4],
                                                loss_mask=torch.ones(4), log_probs=torch.zeros(4), ref_log_probs=torch.zeros(4))
    torch.testing.assert_close(ret, torch.tensor([1.0, 2.0, 4.0, 8.0]))


def test_masked_whiten():
    x = torch.tensor([1.0, 2.0, 3.0, 100.0])
    m = torch.tensor([1.0, 1.0, 1.0, 0.0])
    w = mu.masked_whiten(x, m)
    assert abs(float((w * m).sum())) < 1e-5
    assert abs(float(((w * m) ** 2).sum() / 3) - 1) < 0.6


def test_on_policy_loss_is_minus_mean_advantage():
    args = _args()
    lengths = [4, 2]
    lp = -torch.rand(6)
    adv = torch.tensor([1.0, 1, 1, 1, -2, -2])
    b = _batch(lengths, advantages=adv, old_log_probs=lp.clone(), rollout_log_probs=lp.clone())
    loss, metrics = L.policy_loss_function(args, b, lp.clone().requires_grad_(), None)
    # ratio == 1 → Σ_samples mean_tokens(−A)
    assert math.isclose(float(loss), -(1.0) + 2.0, rel_tol=1e-6)
    assert float(metrics["pg_clipfrac"]) == 0


def test_loss_scaling_invariant_to_microbatch_split():
    """Σ over micro-batches of the scaled loss equals the single-batch value (sample-mean and per-token)."""
    torch.manual_seed(3)
    lengths = [5, 3, 7, 2]
    R = sum(lengths)
    lp = -torch.rand(R)
    old = lp + 0.05 * torch.randn(R)
    adv = torch.randn(R)
    for per_token in (False, True):
        args = _args(calculate_per_token_loss=per_token)
        full = _batch(lengths, advantages=adv, old_log_probs=old)
        ntok = torch.tensor(float(R))
        whole, _, _ = L.loss_function(args, full, lp, None, global_batch_size=4, global_num_tokens=ntok)
        parts = 0.0
        off = 0
        for chunk in ([5, 3], [7, 2]):
            n = sum(chunk)
            sl = slice(off, off + n)
            b = _batch(chunk, advantages=adv[sl], old_log_probs=old[sl])
            s, _, _ = L.loss_function(args, b, lp[sl], None, global_batch_size=4, global_num_tokens=ntok)
            parts = parts + s
            off += n
        torch.testing.assert_close(whole, parts, atol=1e-6, rtol=1e-5)


def test_gspo_uses_sequence_level_ratio():
    args = _args(advantage_estimator="gspo")
    lengths = [3, 3]
    lp = torch.tensor([-1.0, -1.0, -1.0, -2.0, -2.0, -2.0])
    old = torch.tensor([-1.3, -0.7, -1.0, -2.0, -2.0, -2.0])     # token diffs cancel over sequence 0
    b = _batch(lengths, advantages=torch.ones(6), old_log_probs=old)
    loss, metrics = L.policy_loss_function(args, b, lp, None)
    assert float(metrics["pg_clipfrac"]) == 0
    assert math.isclose(float(loss), -2.0, rel_tol=1e-5)


def test_tis_clips_importance_weights():
    args = _args(use_tis=True, tis_clip=2.0, tis_clip_low=0.0)
    lengths = [2]
    lp = torch.tensor([-1.0, -1.0])
    roll = torch.tensor([-3.0, -1.0])                              # first token: weight e² clipped to 2
    b = _batch(lengths, advantages=torch.ones(2), old_log_probs=lp.clone(), rollout_log_probs=roll)
    loss, metrics = L.policy_loss_function(args, b, lp, None)
    assert math.isclose(float(loss), -(2.0 + 1.0) / 2, rel_tol=1e-5)


def test_value_and_sft_loss():
    args = _args(loss_type="value_loss")
    b = _batch([2, 2], returns=torch.tensor([1.0, 1, 0, 0]), old_values=torch.zeros(4))
    v = torch.tensor([0.1, 0.1, 0.0, 0.0])
    loss, m = L.value_loss_function(args, b, v)
    assert float(loss) > 0
    b2 = _batch([2, 2])
    loss2, _ = L.sft_loss_function(_args(loss_type="sft_loss"), b2, torch.tensor([-1.0, -3.0, -2.0, -2.0]))
    assert math.isclose(float(loss2), 2.0 + 2.0, rel_tol=1e-6)


@pytest.mark.parametrize("name", ["cross_entropy", "importance_sampling", "ppo", "cispo", "dro"])
def test_tinker_losses_run(name):
    args = _args()
    lp = (-torch.rand(6)).requires_grad_()
    b = _batch([4, 2], advantages=torch.randn(6), old_log_probs=lp.detach() - 0.01, rollout_log_probs=lp.detach() - 0.01)
    fn = L.get_loss_function(args, name)
    loss, _ = fn(args, b, lp, None)
    loss.backward()
    assert torch.isfinite(lp.grad).all()


def test_entropy_from_logits():
    logits = torch.zeros(3, 8)
    torch.testing.assert_close(mu.compute_entropy_from_logits(logits), torch.full((3,), math.log(8.0)))
