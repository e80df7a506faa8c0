"""Vision tower + multimodal merge on CPU: patch ordering, attention confined to one image, merge positions, gradients
reaching the tower through the language model."""
import torch

from miles_b200.models.config import PRESETS
from miles_b200.models.qwen3 import ForwardMeta, build_model
from miles_b200.models.vision import VisionConfig, VisionLanguageModel, VisionTower, merge_multimodal, patch_positions


def _tower(out_hidden):
    cfg = VisionConfig(patch_size=2, in_channels=3, hidden_size=32, num_heads=2, num_layers=2, ffn_hidden_size=64,
                       spatial_merge=2, out_hidden_size=out_hidden)
    return cfg, VisionTower(cfg, dtype=torch.float32, device="cpu", seed=0)


def test_patch_positions_keep_merge_windows_contiguous():
    rows, cols, cu = patch_positions(torch.tensor([[1, 4, 6], [2, 2, 2]]), 2)
    assert cu.tolist() == [0, 24, 28, 32]
    # first window of the first image: rows {0,1} × cols {0,1}
    assert rows[:4].tolist() == [0, 0, 1, 1] and cols[:4].tolist() == [0, 1, 0, 1]
    # second window moves along the width
    assert rows[4:8].tolist() == [0, 0, 1, 1] and cols[4:8].tolist() == [2, 3, 2, 3]
    assert sorted(zip(rows[:24].tolist(), cols[:24].tolist())) == [(r, c) for r in range(4) for c in range(6)]


def test_tower_shapes_and_image_isolation():
    cfg, tower = _tower(48)
    grid = torch.tensor([[1, 4, 4], [1, 2, 6]])
    g = torch.Generator().manual_seed(0)
    patches = torch.randn(16 + 12, cfg.patch_dim, generator=g)
    out = tower(patches, grid)
    assert out.shape == (4 + 3, 48) and torch.isfinite(out).all()
    # changing the second image leaves the first image's features untouched (attention never crosses images)
    p2 = patches.clone()
    p2[16:] += 1.0
    out2 = tower(p2, grid)
    assert torch.allclose(out[:4], out2[:4], atol=1e-6) and not torch.allclose(out[4:], out2[4:], atol=1e-3)


def test_merge_and_gradients_through_language_model():
    lm_cfg = PRESETS["tiny"]
    lm = build_model(lm_cfg, dtype=torch.float32, device="cpu", seed=0)
    cfg, tower = _tower(lm_cfg.hidden_size)
    image_id = lm_cfg.vocab_size - 1
    vlm = VisionLanguageModel(lm, tower, image_id)
    tokens = torch.tensor([5, 6, image_id, image_id, image_id, image_id, 7, 8, 9], dtype=torch.int32)
    grid = torch.tensor([[1, 4, 4]])
    patches = torch.randn(16, cfg.patch_dim, generator=torch.Generator().manual_seed(1))
    T = len(tokens)
    meta = ForwardMeta(positions=torch.arange(T, dtype=torch.int32), cu_seqlens=torch.tensor([0, T], dtype=torch.int32), max_seqlen=T)
    # the merge puts feature i at the i-th placeholder
    feats = tower(patches, grid)
    emb = merge_multimodal(torch.zeros(T, lm_cfg.hidden_size), tokens, image_id, feats)
    assert torch.equal(emb[2:6], feats) and emb[:2].abs().sum() == 0 and emb[6:].abs().sum() == 0
    h = vlm(tokens, meta, patches=patches, grid_thw=grid)
    lp, _ = vlm.log_probs(h[:-1], tokens[1:].long())
    lp[5:].sum().backward()                         # text tokens after the image
    assert tower.patch_embed.grad is not None and tower.patch_embed.grad.abs().sum() > 0
    assert tower.merger_fc2.grad.abs().sum() > 0 and lm.embed.grad.abs().sum() > 0
    # without images the wrapper is the language model
    plain = torch.tensor([5, 6, 7, 8], dtype=torch.int32)
    m2 = ForwardMeta(positions=torch.arange(4, dtype=torch.int32), cu_seqlens=torch.tensor([0, 4], dtype=torch.int32), max_seqlen=4)
    assert torch.equal(vlm(plain, m2), lm(plain, m2))


def test_packed_batch_carries_images_in_sample_order():
    from miles_b200.train.data import pack_micro_batch

    lm_cfg = PRESETS["tiny"]
    lm = build_model(lm_cfg, dtype=torch.float32, device="cpu", seed=0)
    cfg, tower = _tower(lm_cfg.hidden_size)
    image_id = lm_cfg.vocab_size - 1
    vlm = VisionLanguageModel(lm, tower, image_id)
    g = torch.Generator().manual_seed(3)
    img_a = {"patches": torch.randn(16, cfg.patch_dim, generator=g), "grid_thw": torch.tensor([[1, 4, 4]])}
    img_b = {"patches": torch.randn(8, cfg.patch_dim, generator=g), "grid_thw": torch.tensor([[1, 2, 4]])}
    shard = {
        "tokens": [[4, image_id, image_id, image_id, image_id, 9, 10, 11], [5, 6, 7, 8], [3, image_id, image_id, 12, 13]],
        "response_lengths": [3, 2, 2],
        "loss_masks": [[1, 1, 1], [1, 1], [1, 1]],
        "multimodal_train_inputs": [img_a, None, img_b],
    }
    pb = pack_micro_batch(shard, [0, 1, 2], "cpu", pad_multiple=1)
    assert pb.mm_inputs["patches"].shape[0] == 24 and pb.mm_inputs["grid_thw"].tolist() == [[1, 4, 4], [1, 2, 4]]
    meta = ForwardMeta(positions=pb.positions, cu_seqlens=pb.cu_seqlens, max_seqlen=pb.max_seqlen)
    h = vlm(pb.tokens, meta, **pb.mm_inputs)
    # the text-only sample in the middle is unaffected by the images around it
    solo = pack_micro_batch(shard, [1], "cpu", pad_multiple=1)
    h_solo = vlm(solo.tokens, ForwardMeta(positions=solo.positions, cu_seqlens=solo.cu_seqlens, max_seqlen=solo.max_seqlen))
    assert solo.mm_inputs is None and torch.allclose(h[8:12], h_solo, atol=1e-5)
    # order: swapping which image goes with which sample changes the first sample's hidden states
    pb2 = pack_micro_batch(dict(shard, multimodal_train_inputs=[img_a, None, {"patches": img_b["patches"] + 1, "grid_thw": img_b["grid_thw"]}]),
                           [0, 1, 2], "cpu", pad_multiple=1)
    h2 = vlm(pb2.tokens, meta, **pb2.mm_inputs)
    assert torch.allclose(h[:8], h2[:8], atol=1e-5) and not torch.allclose(h[12:], h2[12:], atol=1e-4)
