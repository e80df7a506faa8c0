"""Model ⇄ HF ⇄ Megatron conversions, checkpoint formats, LoRA, critic head and weight-sync protocols (CPU)."""
import os
from types import SimpleNamespace

import pytest
import torch

from miles_b200.models import convert
from miles_b200.models.config import PRESETS
from miles_b200.models.qwen3 import ForwardMeta, build_model
from miles_b200.parallel.state import ParallelState


def _model(name="tiny", seed=0, dtype=torch.float32):
    cfg = PRESETS[name]
    return cfg, build_model(cfg, ParallelState.single(), dtype=dtype, device="cpu", seed=seed)


def _fwd(model, T=24, seed=0):
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, model.cfg.vocab_size, (T,), generator=g, dtype=torch.int32)
    meta = ForwardMeta(positions=torch.arange(T, dtype=torch.int32), cu_seqlens=torch.tensor([0, T], dtype=torch.int32), max_seqlen=T)
    return model(toks, meta), meta


@pytest.mark.parametrize("name", ["tiny", "tiny-moe"])
def test_hf_roundtrip_preserves_forward(name):
    cfg, m = _model(name, seed=1)
    hf = {}
    for n, p in m.named_parameters():
        for hn, t in convert.to_hf(n, p.detach(), cfg):
            hf[hn] = t.clone()
    assert "model.embed_tokens.weight" in hf and any("q_proj" in k for k in hf)
    if cfg.num_experts:
        assert any(".mlp.experts.0.gate_proj.weight" in k for k in hf) and any("mlp.gate.weight" in k for k in hf)
    _, m2 = _model(name, seed=2)
    convert.load_named_into_model(m2, hf.items(), cfg, m2.ps)
    a, _ = _fwd(m)
    b, _ = _fwd(m2)
    torch.testing.assert_close(a, b)


def test_megatron_name_and_qkv_roundtrip():
    cfg, m = _model("tiny", seed=3)
    ours = {n: p.detach().clone() for n, p in m.named_parameters()}
    meg = convert.ours_to_megatron(ours, cfg)
    assert "decoder.layers.0.self_attention.linear_qkv.weight" in meg and "embedding.word_embeddings.weight" in meg
    back = convert.megatron_to_ours(meg, cfg)
    assert set(back) == set(ours)
    for k in ours:
        assert torch.equal(back[k], ours[k]), k
    # Megatron interleaves per query group: [g, q_per_group + 2, d, H]
    w = meg["decoder.layers.0.self_attention.linear_qkv.weight"]
    g, qpg, d = cfg.num_kv_heads, cfg.num_heads // cfg.num_kv_heads, cfg.head_dim
    v = w.view(g, qpg + 2, d, cfg.hidden_size)
    q_ours = ours["layers.0.attn.wqkv"][: cfg.q_size].view(g, qpg, d, cfg.hidden_size)
    assert torch.equal(v[:, :qpg], q_ours)


def test_torch_dist_roundtrip(tmp_path):
    from miles_b200.checkpoint import torch_dist

    cfg, m = _model("tiny", seed=4)
    meg = convert.ours_to_megatron({n: p.detach() for n, p in m.named_parameters()}, cfg)
    d = torch_dist.save_state(meg, str(tmp_path / "ckpt"), iteration=7)
    assert torch_dist.is_torch_dist_dir(d)
    back = torch_dist.load_state(str(tmp_path / "ckpt"))
    assert set(back) == set(meg)
    for k in meg:
        assert torch.equal(back[k], meg[k])


def test_hf_safetensors_io(tmp_path):
    from miles_b200.checkpoint import hf_io

    t = {"a.weight": torch.randn(4, 6).bfloat16(), "b": torch.arange(5, dtype=torch.int32), "c": torch.randn(3)}
    p = str(tmp_path / "x.safetensors")
    hf_io.save_safetensors(p, t, {"format": "pt"})
    back = hf_io.load_safetensors(p)
    assert all(torch.equal(back[k], t[k]) and back[k].dtype == t[k].dtype for k in t)
    assert list(hf_io.load_safetensors(p, ["b"])) == ["b"]


def _lora_args(**kw):
    base = dict(lora_rank=4, lora_alpha=8.0, lora_dropout=0.0, lora_target_modules=["wqkv", "wo", "w13", "w2"], lora_num_slots=1,
                lora_adapter_path=None, seed=0)
    base.update(kw)
    return SimpleNamespace(**base)


def test_lora_zero_init_grads_merge_and_export(tmp_path):
    from miles_b200.train import lora

    cfg, m = _model("tiny", seed=5)
    base_out, _ = _fwd(m)
    ads = lora.apply_lora(m, _lora_args())
    assert len(ads) == 4 * cfg.num_layers
    out0, _ = _fwd(m)
    torch.testing.assert_close(out0, base_out)                      # B = 0 → identity
    trainable = [n for n, p in m.named_parameters() if p.requires_grad]
    assert trainable and all(".lora." in n for n in trainable)
    with torch.no_grad():
        for ad in ads:
            ad.b.normal_(0, 0.05)
    out1, _ = _fwd(m)
    assert (out1 - base_out).abs().max() > 1e-4
    out1.float().pow(2).sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for n, p in m.named_parameters() if p.requires_grad)
    # merged weights reproduce the adapter forward with the adapters switched off, and are restored afterwards
    w_before = m.layers[0].attn.wqkv.detach().clone()
    with lora.merged(m):
        saved = {id(mod): mod.lora for _, _, mod in lora._targets(m)}
        for _, _, mod in lora._targets(m):
            mod.lora = None
        out_m, _ = _fwd(m)
        for _, _, mod in lora._targets(m):
            mod.lora = saved[id(mod)]
    torch.testing.assert_close(out_m, out1, atol=1e-5, rtol=1e-4)
    assert torch.equal(m.layers[0].attn.wqkv, w_before)
    # PEFT export: B of q/k/v are the row blocks of the fused B
    d = lora.export_peft(m, str(tmp_path / "peft"))
    from miles_b200.checkpoint import hf_io
    t = hf_io.load_safetensors(os.path.join(d, "adapter_model.safetensors"))
    bq = t["base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight"]
    assert bq.shape == (cfg.q_size, 4)
    torch.testing.assert_close(bq, m.layers[0].attn.lora["wqkv"].b[0][: cfg.q_size].float())
    # own-format save/load
    lora.save_adapter(m, str(tmp_path / "ad"))
    with torch.no_grad():
        for ad in ads:
            ad.b.zero_()
    lora.load_adapter(m, str(tmp_path / "ad"))
    out2, _ = _fwd(m)
    torch.testing.assert_close(out2, out1)


def test_lora_slots_route_tokens_and_slot_optimizer():
    from miles_b200.train import lora

    cfg, m = _model("tiny", seed=6)
    base_out, _ = _fwd(m, T=16)
    ads = lora.apply_lora(m, _lora_args(lora_num_slots=3))
    with torch.no_grad():
        for ad in ads:
            ad.b[1].normal_(0, 0.05)                                # only slot 1 differs from the base model
    T = 16
    toks = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)

    def run(slots):
        meta = ForwardMeta(positions=torch.arange(T, dtype=torch.int32), cu_seqlens=torch.tensor([0, 8, 16], dtype=torch.int32),
                           max_seqlen=8, lora_slots=slots)
        return m(toks, meta)

    s = torch.tensor([0] * 8 + [1] * 8)
    out = run(s)
    torch.testing.assert_close(out[:8], base_out[:8] * 0 + run(torch.zeros(T, dtype=torch.long))[:8])
    assert (out[8:] - run(torch.zeros(T, dtype=torch.long))[8:]).abs().max() > 1e-5
    # per-slot optimizer touches its own slot only
    opt = lora.SlotOptimizer(m)
    out.float().pow(2).sum().backward()
    before = [p.detach().clone() for _, p in opt.params]
    opt.step(slot=1, lr=1e-2)
    for (n, p), b in zip(opt.params, before):
        assert torch.equal(p[0], b[0]) and torch.equal(p[2], b[2])
    assert any(not torch.equal(p[1], b[1]) for (n, p), b in zip(opt.params, before))


def test_value_head_attach():
    from miles_b200.train.critic import attach_value_head

    cfg, m = _model("tiny", seed=7)
    vh = attach_value_head(m, cfg, torch.float32, "cpu")
    h, _ = _fwd(m)
    v = vh(h).squeeze(-1)
    assert v.shape == (h.shape[0],) and v.dtype == torch.float32
    assert any("value_head" in n for n, _ in m.named_parameters())


def test_fused_weight_sync_cpu_path_and_quant():
    from miles_b200.parallel.weight_sync import fused_weight_sync

    cfg, src = _model("tiny", seed=8)
    _, dst = _model("tiny", seed=9)
    actor = SimpleNamespace(model=src, args=SimpleNamespace(update_weight_buffer_size=1 << 16))
    engine = SimpleNamespace(model=dst)
    n = fused_weight_sync(actor, engine)
    assert n == sum(p.numel() * p.element_size() for p in src.parameters())
    for (a, p), (b, q) in zip(src.named_parameters(), dst.named_parameters()):
        assert torch.equal(p, q), a
    fused_weight_sync(actor, engine, quant="mxfp8_qdq")
    w, wq = src.layers[0].attn.wo, dst.layers[0].attn.wo
    assert not torch.equal(w, wq) and (w - wq).abs().max() < 0.07 * w.abs().max()
    assert torch.equal(src.layers[0].ln1, dst.layers[0].ln1)        # norms are on the skip list


def test_nvme_stream_adam_matches_adamw_and_resumes(tmp_path):
    from miles_b200.train.nvme_stream import NvmeStreamAdam

    torch.manual_seed(0)
    n = 10_000
    p0 = torch.randn(n)
    flat = p0.clone()
    ref_p = torch.nn.Parameter(p0.clone())
    ref_opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    opt = NvmeStreamAdam(flat, str(tmp_path), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, bucket_numel=3000)
    grads = [torch.randn(n) for _ in range(4)]
    for g in grads[:2]:
        opt.step(g)
        ref_p.grad = g.clone()
        ref_opt.step()
    torch.testing.assert_close(flat, ref_p.detach(), atol=1e-6, rtol=1e-5)
    assert opt.bytes_read == opt.bytes_written == 2 * 3 * 4 * n          # every state byte read and written once per step
    sd = opt.state_dict()
    opt.close()
    # a new process picks the files up and continues
    opt2 = NvmeStreamAdam(flat, str(tmp_path), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, bucket_numel=4096)
    opt2.load_state_dict(sd)
    for g in grads[2:]:
        opt2.step(g)
        ref_p.grad = g.clone()
        ref_opt.step()
    torch.testing.assert_close(flat, ref_p.detach(), atol=1e-6, rtol=1e-5)
    opt2.close()


def test_packed_nvfp4_and_int4_export_decode_to_the_fake_quant_values(tmp_path):
    """What the exporters pack must decode to exactly what fake-quantised training computes."""
    from miles_b200 import ops
    from miles_b200.ops import reference as R
    from miles_b200.weight_update import quant_export as qe

    g = torch.Generator().manual_seed(0)
    w = (torch.randn(48, 64, generator=g) * torch.rand(48, 1, generator=g) * 3).bfloat16()
    q, sb, s2 = qe.nvfp4_quantize(w)
    assert q.dtype == torch.uint8 and q.shape == (48, 32) and sb.dtype == torch.float8_e4m3fn and sb.shape == (48, 4)
    assert torch.equal(qe.nvfp4_dequantize(q, sb, s2), R.nvfp4_qdq(w))
    # ties and saturation of the e2m1 rounding
    probe = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, 0.0, 0.26])
    assert qe.e2m1_codes(probe).tolist() == [0, 2, 2, 4, 4, 6, 6, 7, 0, 1]
    # four-over-six never loses to the plain rule, and wins on blocks whose values sit between the coarse upper steps
    x = torch.full((1, 16), 4.2)
    x[0, 0] = 5.0
    big = torch.cat([x, torch.full((1, 16), 448.0 * 6)], 0).float()           # second row pins the tensor scale to 1
    plain = qe.nvfp4_dequantize(*qe.nvfp4_quantize(big), dtype=torch.float32)
    fos = qe.nvfp4_dequantize(*qe.nvfp4_quantize(big, four_over_six=True), dtype=torch.float32)
    assert ((fos - big) ** 2).sum() < ((plain - big) ** 2).sum()
    e_plain = ((qe.nvfp4_dequantize(q, sb, s2).float() - w.float()) ** 2).sum()
    e_fos = ((qe.nvfp4_dequantize(*qe.nvfp4_quantize(w, four_over_six=True)).float() - w.float()) ** 2).sum()
    assert e_fos <= e_plain
    # naming, pairing and eligibility
    named = [("model.layers.0.mlp.experts.3.gate_proj.weight", w), ("model.layers.0.mlp.experts.3.up_proj.weight", w * 2),
             ("model.layers.0.mlp.experts.3.down_proj.weight", w), ("model.layers.0.self_attn.q_proj.weight", w),
             ("model.layers.1.mlp.experts.0.down_proj.weight", w), ("model.norm.weight", torch.ones(64))]
    out = dict(qe.export_nvfp4(named, ignore=["model.layers.1.mlp.experts"], num_layers=2))
    gate, up = "model.layers.0.mlp.experts.3.gate_proj", "model.layers.0.mlp.experts.3.up_proj"
    assert out[gate + ".weight"].dtype == torch.uint8 and torch.equal(out[gate + ".weight_scale_2"], out[up + ".weight_scale_2"])
    assert out["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16           # experts only by default
    assert out["model.layers.1.mlp.experts.0.down_proj.weight"].dtype == torch.bfloat16    # ignore rule
    assert torch.equal(qe.nvfp4_dequantize(out[up + ".weight"], out[up + ".weight_scale"], out[up + ".weight_scale_2"]),
                       R.nvfp4_qdq(w * 2, global_amax=(w * 2).float().abs().max()))
    with pytest.raises(ValueError):
        qe.export_nvfp4(named[:1], num_layers=2)                                           # a gate without its up
    assert qe.is_ignored("a.b.c.weight", ["a.b"]) and qe.is_ignored("a.b.weight", ["re:a\\..*"]) and not qe.is_ignored("a.bc.weight", ["a.b"])
    # int4: symmetric and asymmetric, packing order, decode = fake quant
    parts = qe.int4_quantize(w, 32, True)
    assert parts["weight_packed"].dtype == torch.int32 and parts["weight_packed"].shape == (48, 8) and parts["weight_shape"].tolist() == [48, 64]
    want, _ = ops.int4_fake_quant(w, 1, 32, True)
    assert torch.allclose(qe.int4_dequantize(parts).float(), want.float(), atol=1e-2, rtol=1e-2)
    codes = torch.arange(16, dtype=torch.uint8).reshape(1, 16)
    packed = qe.pack_int32(codes)
    assert packed.tolist() == [[0x76543210, 0xFEDCBA98 - (1 << 32)]] and torch.equal(qe.unpack_int32(packed, 16), codes.long())
    asym = qe.int4_quantize(w, 32, False)
    assert asym["weight_zero_point"].shape == (6, 2)                                      # [M/8, K/g]: packed along M
    assert (qe.int4_dequantize(asym).float() - w.float()).abs().max() < (w.float().abs().max() / 7)
    out4 = dict(qe.export_int4([("model.layers.0.self_attn.q_proj.weight", w), ("lm_head.weight", w)], group_size=32))
    assert "model.layers.0.self_attn.q_proj.weight_packed" in out4 and "lm_head.weight" in out4
    assert qe.quant_config("int4")["quantization_config"]["format"] == "pack-quantized"
    assert qe.quant_config("nvfp4")["quantization_config"]["quant_algo"] == "NVFP4"


@pytest.mark.parametrize("mode,preset", [("nvfp4", "tiny-moe"), ("int4", "tiny")])
def test_quantised_disk_sync_reaches_the_engine_as_the_quantised_values(tmp_path, mode, preset):
    """--export-quant through the disk protocol: the engine ends up with decode(quantise(trainer weights))."""
    from test_e2e import BASE
    from miles_b200.args import parse_args
    from miles_b200.engine.engine import Engine
    from miles_b200.models.convert import hf_state_to_ours, to_hf
    from miles_b200.orchestration.wiring import create_parallel_state, create_training_models
    from miles_b200.weight_update import quant_export as qe
    from miles_b200.weight_update.updater import WeightUpdater

    args = parse_args((BASE.replace("--model-name tiny", f"--model-name {preset}") + f" --export-quant {mode} --export-quant-all-linears "
                       f"--update-weight-transfer-mode disk --update-weight-disk-dir {tmp_path}").split())
    ps = create_parallel_state(args)
    actor, _, _ = create_training_models(args, ps)
    eng = Engine(actor.cfg, ps=ps, device="cpu", dtype=torch.float32, num_blocks=8, block_size=16, seed=99)
    WeightUpdater(args, actor, [eng]).update_weights()
    import json

    cfgj = json.load(open(next(os.path.join(r, "config.json") for r, _, f in os.walk(tmp_path) if "config.json" in f)))
    assert cfgj["quantization_config"]["quant_method"] in ("modelopt", "compressed-tensors")
    got = dict(eng.model.named_parameters())
    hf = [x for n, p in actor.model.named_parameters() for x in to_hf(n, p.data, actor.cfg)]
    packed = qe.export_nvfp4(hf, all_linears=True, num_layers=actor.cfg.num_layers) if mode == "nvfp4" else qe.export_int4(hf)
    want = hf_state_to_ours(dict(qe.dequantize_named(packed, torch.float32)), actor.cfg)
    changed = 0
    for n, p in actor.model.named_parameters():
        assert torch.allclose(got[n].data, want[n].float(), atol=1e-6), n
        changed += int(not torch.equal(want[n].float(), p.data.float()))
    assert changed > 0                                                         # something really was quantised


def test_nvme_streamed_optimizer_in_the_trainer_matches_the_resident_one(tmp_path):
    """--optimizer-nvme-dir: the trainer's distributed Adam keeps master weights and moments in files; two GRPO steps give the
    same weights as the resident optimizer, the sharded checkpoint reads the state through the file-backed views."""
    from test_e2e import BASE, _run
    from miles_b200.args import parse_args
    from miles_b200.orchestration.wiring import create_parallel_state, create_training_models

    h_ref = _run("--weight-decay 0.1")
    h_nv = _run(f"--weight-decay 0.1 --optimizer-nvme-dir {tmp_path}/nv --optimizer-nvme-bucket-numel 4096")
    for k in ("train/grad_norm", "train/loss", "rollout/raw_reward"):
        for a, b in zip(h_ref.series(k), h_nv.series(k)):
            assert abs(a - b) <= 1e-5 * max(1.0, abs(a)), (k, a, b)
    assert os.path.exists(os.path.join(tmp_path, "nv", "actor", "dense", "rank0", "exp_avg.bin"))
    args = parse_args((BASE + f" --optimizer-nvme-dir {tmp_path}/nv2 --save {tmp_path}/ck").split())
    actor, _, _ = create_training_models(args, create_parallel_state(args))
    d = actor.optimizer.domains[0]
    assert d.nvme is not None and d.master.device.type == "cpu" and torch.equal(d.master, d.param_buf[d.shard[0]:d.shard[1]].float().cpu())
    d.exp_avg.fill_(0.25)                                   # through the view, into the file
    assert float(torch.from_numpy(d.nvme.maps["exp_avg"][:4].copy()).sum()) == 1.0
    actor.save_model(0)
    from miles_b200.checkpoint import torch_dist

    opt = torch_dist.load_state(os.path.join(tmp_path, "ck", "iter_0000000"), prefix_filter=("rng", "_extra_state"))
    assert float(opt["optimizer.state.exp_avg.decoder.layers.0.self_attention.linear_proj.weight"].mean()) == 0.25
