"""Sample plumbing, train-data conversion, balancing, micro-batching and packing (CPU)."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from miles_b200.train import data as D
from miles_b200.types import (Sample, Status, WeightVersionSpan, decode_routed_experts, encode_routed_experts)


def _sample(prompt_len, resp_len, reward, gi=0, idx=0):
    s = Sample(group_index=gi, index=idx, tokens=list(range(1, prompt_len + 1)))
    s.append_response(list(range(100, 100 + resp_len)), [-0.5] * resp_len)
    s.reward = reward
    s.status = Status.COMPLETED
    return s


def test_sample_append_and_meta():
    s = Sample(tokens=[1, 2, 3])
    s.append_response([4, 5], [-0.1, -0.2])
    s.update_from_meta_info({"finish_reason": {"type": "stop"}, "weight_version": 3}, 2)
    s.append_response([9, 9, 9], None, trainable=False)            # tool output
    s.append_response([6], [-0.3])
    s.update_from_meta_info({"finish_reason": {"type": "length"}, "weight_version": 4}, 1)
    assert s.tokens == [1, 2, 3, 4, 5, 9, 9, 9, 6]
    assert s.response_length == 6 and s.prompt_length == 3
    assert s.loss_mask == [1, 1, 0, 0, 0, 1]
    assert s.rollout_log_probs == pytest.approx([-0.1, -0.2, 0, 0, 0, -0.3])
    assert s.status == Status.TRUNCATED
    assert [(w.version, w.num_tokens) for w in s.weight_versions] == [(3, 2), (4, 1)]
    assert s.oldest_weight_version == 3
    r = Sample.from_dict(s.to_dict())
    assert r.tokens == s.tokens and r.status == s.status and r.loss_mask == s.loss_mask
    assert isinstance(r.weight_versions[0], WeightVersionSpan)


def test_routed_experts_codec():
    arr = np.arange(5 * 3 * 2, dtype=np.int32).reshape(5, 3, 2)    # 6 tokens → 5 recorded rows
    back = decode_routed_experts(encode_routed_experts(arr), 6, 3, 2)
    assert np.array_equal(arr, back)


def test_convert_samples_groups_and_rewards():
    args = SimpleNamespace(n_samples_per_prompt=2, advantage_estimator="grpo", grpo_std_normalization=True,
                           rewards_normalization=True, reward_key=None)
    groups = [[_sample(3, 4, 1.0, 0, 0), _sample(3, 2, 0.0, 0, 1)], [_sample(5, 1, 1.0, 1, 2), _sample(5, 3, 1.0, 1, 3)]]
    data = D.convert_samples_to_train_data(args, groups)
    assert data["response_lengths"] == [4, 2, 1, 3]
    assert data["total_lengths"] == [7, 5, 6, 8]
    assert data["raw_reward"] == [1.0, 0.0, 1.0, 1.0]
    r = data["rewards"]
    assert r[0] > 0 > r[1] and abs(r[0] + r[1]) < 1e-5 and r[2] == 0 and r[3] == 0
    assert all(len(m) == n for m, n in zip(data["loss_masks"], data["response_lengths"]))


@pytest.mark.parametrize("equal", [True, False])
def test_karmarkar_karp_balances(equal):
    rng = np.random.default_rng(0)
    lengths = rng.integers(10, 2000, size=64).tolist()
    parts = D.karmarkar_karp(lengths, 4, equal_size=equal)
    assert sorted(i for p in parts for i in p) == list(range(64))
    sums = [sum(lengths[i] for i in p) for p in parts]
    naive = [sum(lengths[r::4]) for r in range(4)]
    assert max(sums) - min(sums) <= max(naive) - min(naive)
    if equal:
        assert {len(p) for p in parts} == {16}


def test_split_by_dp_round_robin_and_balanced():
    data = {"tokens": [[0] * n for n in (8, 2, 6, 4)], "total_lengths": [8, 2, 6, 4], "response_lengths": [1, 1, 1, 1],
            "loss_masks": [[1]] * 4, "rewards": [0.0, 1.0, 2.0, 3.0], "raw_reward": [0.0] * 4, "meta": "shared"}
    shards = D.split_train_data_by_dp(SimpleNamespace(balance_data=False), data, 2)
    assert shards[0]["partition"] == [0, 2] and shards[1]["rewards"] == [1.0, 3.0] and shards[0]["meta"] == "shared"
    shards = D.split_train_data_by_dp(SimpleNamespace(balance_data=True), data, 2)
    assert sorted(sum(s["total_lengths"]) for s in shards) == [10, 10]


def test_micro_batches_fixed_and_dynamic():
    fixed = D.make_micro_batches(SimpleNamespace(use_dynamic_batch_size=False, micro_batch_size=2), [5, 5, 5, 5, 5])
    assert [len(p) for p in fixed] == [2, 2, 1]
    lengths = [900, 100, 500, 500, 300, 700]
    dyn = D.make_micro_batches(SimpleNamespace(use_dynamic_batch_size=True, max_tokens_per_gpu=1000), lengths)
    assert sorted(i for p in dyn for i in p) == list(range(6))
    assert all(sum(lengths[i] for i in p) <= 1000 for p in dyn)
    assert len(dyn) == 3


def test_pack_micro_batch_alignment():
    shard = {"tokens": [[1, 2, 3, 10, 11], [4, 5, 20]], "response_lengths": [2, 1], "loss_masks": [[1, 0], [1]]}
    b = D.pack_micro_batch(shard, [0, 1], "cpu", pad_multiple=16)
    assert b.tokens.numel() == 16 and b.num_real_tokens == 8
    assert b.cu_seqlens.tolist() == [0, 5, 8, 16]
    assert b.positions[:8].tolist() == [0, 1, 2, 3, 4, 0, 1, 2]
    # the hidden state at row r predicts token r+1
    assert b.gather_index.tolist() == [2, 3, 6]
    assert b.targets.tolist() == [10, 11, 20]
    assert b.tokens[b.gather_index + 1].tolist() == b.targets.tolist()
    assert b.loss_mask.tolist() == [1, 0, 1] and b.seq_ids.tolist() == [0, 0, 1]
    assert b.max_seqlen == 8


def test_pack_replay_rows_follow_tokens():
    re0 = np.arange(4 * 2 * 2, dtype=np.int32).reshape(4, 2, 2)        # 5 tokens → 4 recorded rows
    shard = {"tokens": [[1, 2, 3, 10, 11]], "response_lengths": [2], "loss_masks": [[1, 1]], "rollout_routed_experts": [re0]}
    b = D.pack_micro_batch(shard, [0], "cpu", pad_multiple=8, with_replay=True)
    assert b.replay_topk.shape == (8, 2, 2)
    assert torch.equal(b.replay_topk[:4], torch.from_numpy(re0))
    assert (b.replay_topk[4:] == -1).all()


def test_ragged_codec_and_object_store_backends(tmp_path):
    """Samples survive the typed ragged codec bit-exactly (None vs empty kept apart, routed experts with their shape), the
    encoding is no larger than pickled lists (and is built from a handful of buffers instead of an object per token), and the object store round-trips batches through its three backends."""
    import pickle

    import numpy as np

    from miles_b200.types import Sample
    from miles_b200.utils import object_store, ragged_codec

    rng = np.random.default_rng(0)
    groups = []
    for g in range(3):
        grp = []
        for i in range(4):
            n = int(rng.integers(5, 400))
            s = Sample(tokens=rng.integers(0, 150000, n).tolist(), response_length=n // 2, index=g * 4 + i,
                       metadata={"k": g}, reward=float(i))
            s.loss_mask = [1] * (n // 2) if i % 2 else None
            s.rollout_log_probs = (-rng.random(n // 2)).astype(np.float32).tolist() if i != 3 else []
            s.rollout_routed_experts = rng.integers(0, 128, (n - 1, 2, 8)).astype(np.int32) if i == 0 else None
            grp.append(s)
        groups.append(grp)
    enc = ragged_codec.encode_groups(groups)
    back = ragged_codec.decode_groups(pickle.loads(pickle.dumps(enc, protocol=5)), Sample)
    assert [len(g) for g in back] == [4, 4, 4]
    for ga, gb in zip(groups, back):
        for a, b in zip(ga, gb):
            assert a.tokens == b.tokens and a.loss_mask == b.loss_mask and a.index == b.index and a.metadata == b.metadata
            assert (a.rollout_log_probs is None) == (b.rollout_log_probs is None)
            assert a.rollout_log_probs == [] if a.rollout_log_probs == [] else np.allclose(a.rollout_log_probs, b.rollout_log_probs)
            if a.rollout_routed_experts is None:
                assert b.rollout_routed_experts is None
            else:
                assert np.array_equal(a.rollout_routed_experts, b.rollout_routed_experts)
    naive = len(pickle.dumps([[s.to_dict() for s in g] for g in groups]))
    assert len(pickle.dumps(enc, protocol=5)) < naive
    blob = ragged_codec.dumps([s.to_dict() for s in groups[0]], compress=True)
    assert ragged_codec.loads(blob)[1]["tokens"] == groups[0][1].tokens
    batch = {"tokens": [s.tokens for s in groups[0]], "loss_masks": [[1, 0, 1], [], [1], [0]], "rewards": [0.5, 1.0, 0.0, 2.0],
             "rollout_log_probs": [[-0.5, -1.5], [], [-2.0], [-0.25]], "note": "x"}

    class KV:
        def __init__(self):
            self.d = {}

        def set(self, k, v):
            self.d[k] = v

        def get(self, k):
            return self.d[k]

        def delete_key(self, k):
            self.d.pop(k)

    try:
        for conf in ({}, {"directory": str(tmp_path / "store")}, {"store": KV()}):
            object_store.configure(**conf)
            key = object_store.put(batch)
            got = object_store.get(key)
            assert got["tokens"] == batch["tokens"] and got["loss_masks"] == batch["loss_masks"] and got["note"] == "x"
            assert got["rollout_log_probs"] == batch["rollout_log_probs"] and got["rewards"] == batch["rewards"]
            object_store.remove(key)
            with pytest.raises(Exception):
                object_store.get(key)
    finally:
        object_store.configure()
