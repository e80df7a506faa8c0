"""Model families beyond Qwen3: block semantics, training step, HF name round trip (CPU, fp32)."""
import pytest
import torch

from miles_b200.models import bridges as B
from miles_b200.models import families as Fm
from miles_b200.models.qwen3 import ForwardMeta


def _batch(cfg, lens=(5, 9), seed=0):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    tok = torch.randint(0, cfg.vocab_size, (T,), generator=g)
    pos = torch.cat([torch.arange(l) for l in lens]).int()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    return tok, ForwardMeta(positions=pos, cu_seqlens=cu, max_seqlen=max(lens))


@pytest.mark.parametrize("name", sorted(Fm.FAMILY_PRESETS))
def test_family_trains_and_every_parameter_gets_gradient(name):
    cfg = Fm.FAMILY_PRESETS[name]
    m = Fm.build_family_model(cfg, dtype=torch.float32)
    tok, meta = _batch(cfg)
    opt = torch.optim.Adam([p for p in m.parameters() if p.requires_grad], lr=3e-3)
    losses = []
    for _ in range(6):
        h = m(tok, meta)
        lm = -m.log_probs(h, tok)[0].mean()
        loss = lm + sum(m.aux_losses().values(), torch.tensor(0.0))
        opt.zero_grad()
        loss.backward()
        if not losses:
            assert [n for n, p in m.named_parameters() if p.requires_grad and p.grad is None] == []
        opt.step()
        losses.append(float(lm.detach()))
    assert losses[-1] < losses[0]


@pytest.mark.parametrize("name", sorted(Fm.FAMILY_PRESETS))
def test_family_is_causal_and_sequences_are_independent(name):
    cfg = Fm.FAMILY_PRESETS[name]
    m = Fm.build_family_model(cfg, dtype=torch.float32)
    tok, meta = _batch(cfg)
    with torch.no_grad():
        h = m(tok, meta)
        tok2 = tok.clone()
        tok2[3] = (tok2[3] + 1) % cfg.vocab_size          # inside sequence 0
        h2 = m(tok2, meta)
    assert torch.allclose(h[:3], h2[:3], atol=1e-5)        # earlier tokens of the same sequence
    assert not torch.allclose(h[3:5], h2[3:5], atol=1e-5)
    assert torch.allclose(h[5:], h2[5:], atol=1e-5)        # the other sequence


def test_sparse_latent_attention_with_all_keys_equals_dense():
    cfg = Fm.FAMILY_PRESETS["deepseek-tiny"].with_(index_topk=64)
    dense_cfg = cfg.with_(layer_types=("mla", "mla", "mla"))
    tok, meta = _batch(cfg)
    sparse, dense = Fm.build_family_model(cfg, dtype=torch.float32), Fm.build_family_model(dense_cfg, dtype=torch.float32)
    with torch.no_grad():
        assert torch.allclose(sparse(tok, meta), dense(tok, meta), atol=1e-5)
    # with a short key budget the output differs, and training produces the indexer loss
    few = Fm.build_family_model(cfg.with_(index_topk=2), dtype=torch.float32)
    h = few(tok, meta)
    assert not torch.allclose(h, dense(tok, meta), atol=1e-4)
    assert "indexer_kl" in few.aux_losses() and float(few.aux_losses()["indexer_kl"]) >= 0


def test_hyper_connections_at_init_equal_the_plain_residual_stream():
    cfg = Fm.FAMILY_PRESETS["hyper-tiny"]
    tok, meta = _batch(cfg)
    hyper, plain = Fm.build_family_model(cfg, dtype=torch.float32), Fm.build_family_model(cfg.with_(hc_streams=1), dtype=torch.float32)
    with torch.no_grad():
        assert torch.allclose(hyper(tok, meta), plain(tok, meta), atol=2e-3, rtol=1e-3)


def test_delta_rule_matches_its_definition_and_decays():
    torch.manual_seed(0)
    T, H, dk, dv = 6, 2, 4, 3
    q, k, v = torch.randn(T, H, dk), torch.nn.functional.normalize(torch.randn(T, H, dk), dim=-1), torch.randn(T, H, dv)
    beta, cu = torch.ones(T, H), torch.tensor([0, T])
    # β = 1, no decay, a single repeated unit key: the state stores exactly the last value for that key
    k1 = k[:1].expand(T, H, dk)
    o = Fm.delta_rule(k1, k1, v, beta, torch.zeros(T, H), cu)
    assert torch.allclose(o, v, atol=1e-5)
    # strong decay forgets the past: the output only sees the current token's write
    o_forget = Fm.delta_rule(q, k, v, beta, torch.full((T, H), -50.0), cu)
    expect = torch.einsum("thk,thk->th", k, q)[..., None] * v
    assert torch.allclose(o_forget, expect, atol=1e-5)
    # per-channel decay of equal value is the per-head decay
    g = -torch.rand(T, H)
    assert torch.allclose(Fm.delta_rule(q, k, v, beta, g, cu), Fm.delta_rule(q, k, v, beta, g[..., None].expand(T, H, dk), cu), atol=1e-6)


def test_sigmoid_router_bias_changes_selection_not_weights():
    cfg = Fm.FAMILY_PRESETS["glm-moe-tiny"]
    m = Fm.build_family_model(cfg, dtype=torch.float32)
    tok, meta = _batch(cfg)
    rec0, rec1 = [], []
    with torch.no_grad():
        meta.record_topk = rec0
        m(tok, meta)
        moe = m.layers[1].mlp
        loads = torch.bincount(rec0[0].flatten().long(), minlength=cfg.num_experts)
        for _ in range(200):
            m.update_router_bias([loads], rate=0.01)
        assert float(moe.e_bias[loads.argmax()]) < 0 < float(moe.e_bias[loads.argmin()])
        meta.record_topk = rec1
        m(tok, meta)
    loads1 = torch.bincount(rec1[0].flatten().long(), minlength=cfg.num_experts)
    assert loads1.max() <= loads.max() and not torch.equal(rec0[0], rec1[0])


@pytest.mark.parametrize("name", ["deepseek-tiny", "qwen3-next-tiny", "hyper-tiny"])
def test_family_grpo_end_to_end(name):
    """Rollout (engine re-scoring path for blocks without a paged cache) → rewards → train → weight sync, on-policy at step 0."""
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import train as T
    from miles_b200.args import parse_args

    args = parse_args((f"--model-name {name} --fp32 --rollout-batch-size 4 --n-samples-per-prompt 2 --rollout-max-response-len 6 "
                       "--num-rollout 2 --rm-type even_fraction --lr 1e-4 --colocate --advantage-estimator grpo "
                       "--data-source-path miles_b200.rollout.data_source.SyntheticSource --synthetic-prompt-len 4 6").split())
    h = T.train(args).history
    assert len(h.rows) == 2
    assert max(h.series("train/train_rollout_logprob_abs_diff")) < 1e-4
    assert abs(h.series("train/ppo_kl")[0]) < 1e-6
    assert all(g > 0 for g in h.series("train/grad_norm"))


@pytest.mark.parametrize("name", sorted(Fm.FAMILY_PRESETS))
def test_hf_names_round_trip(name):
    cfg = Fm.FAMILY_PRESETS[name]
    m = Fm.build_family_model(cfg, dtype=torch.float32)
    state = B.full_state(m)
    hf = B.state_to_hf(state, cfg)
    assert all(k.startswith(("model.", "lm_head.")) for k in hf)
    back = B.from_hf(hf, cfg)
    assert sorted(back) == sorted(state)
    for k in state:
        assert torch.equal(back[k], state[k]), k
    kinds = set(cfg.layer_types)
    if kinds & {"mla", "dsa"}:
        assert any("kv_a_proj_with_mqa" in k for k in hf)
    if "dsa" in kinds:
        assert any("indexer.weights_proj" in k for k in hf)
    if kinds & {"gdn", "kda"}:
        assert any("linear_attn.in_proj_qkvz" in k for k in hf) and any("linear_attn.conv1d" in k for k in hf)
    if cfg.n_shared_experts:
        assert any("shared_experts.down_proj" in k for k in hf)
    if cfg.attn_output_gate:
        q = next(v for k, v in hf.items() if k.endswith("self_attn.q_proj.weight"))
        assert q.shape[0] == 2 * cfg.q_size


# ---- context parallelism of the recurrent mixer: state and convolution history passed from rank to rank ---------------

def _linear_cp_body(rank, world, per_channel, cu_list):
    import torch

    from miles_b200.models.families import FamilyConfig, LinearAttention
    from miles_b200.models.qwen3 import ForwardMeta, _Init
    from miles_b200.parallel import cp as _cp
    from miles_b200.parallel.state import ParallelState, init_distributed

    init_distributed(backend="gloo")
    ps = ParallelState.build(cp=world, cp_comm_type="a2a")
    cfg = FamilyConfig(name="t", hidden_size=32, linear_heads=2, linear_key_dim=8, linear_value_dim=8, conv_kernel=4)
    torch.manual_seed(0)
    T = cu_list[-1]
    x_full = torch.randn(T, 32)
    g_full = torch.randn(T, 32)
    cu = torch.tensor(cu_list, dtype=torch.int32)

    def build(p):
        m = LinearAttention(cfg, p, torch.float32, "cpu", _Init(7), "l0", per_channel_decay=per_channel)
        with torch.no_grad():
            m.A_log.fill_(0.3)
            m.dt_bias.normal_(0, 0.5, generator=torch.Generator().manual_seed(3))
        return m

    ref = build(ParallelState.single())
    xr = x_full.clone().requires_grad_()
    yr = ref(xr, ForwardMeta(positions=None, cu_seqlens=cu, max_seqlen=T), 0)
    yr.backward(g_full)
    mod = build(ps)
    lo, hi = _cp.chunk_bounds(T, world, rank)
    xl = x_full[lo:hi].clone().requires_grad_()
    yl = mod(xl, ForwardMeta(positions=None, cu_seqlens=cu, max_seqlen=T), 0)
    assert torch.allclose(yl, yr.detach()[lo:hi], atol=1e-5), float((yl - yr.detach()[lo:hi]).abs().max())
    yl.backward(g_full[lo:hi])
    assert torch.allclose(xl.grad, xr.grad[lo:hi], atol=1e-5), float((xl.grad - xr.grad[lo:hi]).abs().max())
    # parameter gradients: the ranks' contributions add up to the single-rank gradient
    import torch.distributed as dist

    for (n, p), (_, q) in zip(mod.named_parameters(), ref.named_parameters()):
        gsum = p.grad.clone()
        dist.all_reduce(gsum)
        assert torch.allclose(gsum, q.grad, atol=2e-5), (n, float((gsum - q.grad).abs().max()))


@pytest.mark.parametrize("world,per_channel,cu", [(2, False, [0, 5, 19, 24]), (2, True, [0, 12, 24]), (3, False, [0, 3, 24]),
                                                   (3, True, [0, 7, 9, 24])])
def test_linear_attention_context_parallel_state_passing(world, per_channel, cu):
    """Chunks of 12 (or 8) tokens: sequences cut by a chunk boundary (one spans all three ranks; one chunk is shorter than
    the convolution's history only together with its neighbour), a boundary that coincides with a sequence start, both decay
    forms — outputs, input gradients and summed parameter gradients equal the single-rank layer's."""
    import os
    import sys

    sys.path.insert(0, os.path.dirname(__file__))
    from dist_utils import run_distributed

    run_distributed(_linear_cp_body, world, (per_channel, cu), timeout=300)


def test_audio_tower_is_per_clip_and_feeds_the_language_model():
    """Clips packed along time: a clip's rows do not depend on its neighbours, row counts follow the stride and the pooling,
    and the features merged at the audio placeholder tokens carry gradients back into the tower."""
    import torch

    from miles_b200.models.audio import AudioConfig, AudioLanguageModel, AudioTower, output_rows
    from miles_b200.models.config import PRESETS
    from miles_b200.models.qwen3 import ForwardMeta, build_model
    from miles_b200.parallel.state import ParallelState

    cfg = AudioConfig(n_mels=16, hidden_size=64, num_layers=2, num_heads=4, ffn_hidden_size=96, pool=2, out_hidden_size=256)
    tower = AudioTower(cfg, dtype=torch.float32, seed=1)
    g = torch.Generator().manual_seed(0)
    frames = torch.tensor([13, 8, 21])
    feats = torch.randn(int(frames.sum()), 16, generator=g)
    rows = output_rows(frames, 2)
    assert rows.tolist() == [4, 2, 6]
    out = tower(feats, frames)
    assert out.shape == (12, 256)
    alone = tower(feats[13:21], frames[1:2])
    assert torch.allclose(out[4:6], alone, atol=1e-5)                              # clip 1 on its own gives the same rows
    lm = build_model(PRESETS["tiny"], ParallelState.single(), dtype=torch.float32, device="cpu", seed=0)
    model = AudioLanguageModel(lm, tower, audio_token_id=7)
    tokens = torch.tensor([3, 7, 7, 7, 7, 9, 11, 7, 7, 12, 7, 7, 7, 7, 7, 7, 5], dtype=torch.int32)
    meta = ForwardMeta(positions=torch.arange(17, dtype=torch.int32), cu_seqlens=torch.tensor([0, 17], dtype=torch.int32), max_seqlen=17)
    h = model(tokens, meta, audio_features=feats, clip_frames=frames)
    assert h.shape == (17, 256)
    h.float().pow(2).sum().backward()
    assert tower.conv1_w.grad is not None and float(tower.conv1_w.grad.abs().sum()) > 0
    plain = model(tokens.clone().fill_(3), meta)                                   # no audio inputs: the language model alone
    assert plain.shape == (17, 256)


def _mla_cp_body(rank, world, cu_list, sparse=False):
    import torch
    import torch.distributed as dist

    from miles_b200.models.families import FamilyConfig, LatentAttention
    from miles_b200.models.qwen3 import ForwardMeta, _Init
    from miles_b200.parallel import cp as _cp
    from miles_b200.parallel.state import ParallelState, init_distributed

    init_distributed(backend="gloo")
    ps = ParallelState.build(cp=world, cp_comm_type="allgather")
    cfg = FamilyConfig(name="t", hidden_size=64, num_heads=4, q_lora_rank=24, kv_lora_rank=16, qk_nope_head_dim=8, qk_rope_head_dim=8,
                       v_head_dim=8, index_heads=2, index_dim=8, index_topk=6)
    torch.manual_seed(0)
    T = cu_list[-1]
    x_full, g_full = torch.randn(T, 64), torch.randn(T, 64)
    cu = torch.tensor(cu_list, dtype=torch.int32)
    pos_full = torch.cat([torch.arange(b - a) for a, b in zip(cu_list[:-1], cu_list[1:])]).to(torch.int32)
    ref = LatentAttention(cfg, ParallelState.single(), torch.float32, "cpu", _Init(5), "l0", sparse=sparse)
    xr = x_full.clone().requires_grad_()
    yr = ref(xr, ForwardMeta(positions=pos_full, cu_seqlens=cu, max_seqlen=T), 0)
    ((yr * g_full).sum() + (ref.last_index_loss if sparse else 0.0)).backward()
    mod = LatentAttention(cfg, ps, torch.float32, "cpu", _Init(5), "l0", sparse=sparse)
    lo, hi = _cp.chunk_bounds(T, world, rank)
    xl = x_full[lo:hi].clone().requires_grad_()
    yl = mod(xl, ForwardMeta(positions=pos_full[lo:hi], cu_seqlens=cu, max_seqlen=T), 0)
    assert torch.allclose(yl, yr.detach()[lo:hi], atol=1e-5), float((yl - yr.detach()[lo:hi]).abs().max())
    ((yl * g_full[lo:hi]).sum() + (mod.last_index_loss if sparse else 0.0)).backward()
    assert torch.allclose(xl.grad, xr.grad[lo:hi], atol=1e-5)
    for (n, p), (_, q) in zip(mod.named_parameters(), ref.named_parameters()):
        gsum = p.grad.clone()
        dist.all_reduce(gsum)
        assert torch.allclose(gsum, q.grad, atol=2e-5), (n, float((gsum - q.grad).abs().max()))


@pytest.mark.parametrize("world,cu,sparse", [(2, [0, 7, 24], False), (3, [0, 10, 11, 24], False), (2, [0, 9, 24], True)])
def test_latent_attention_context_parallel_gathers_the_latent(world, cu, sparse):
    """Latent attention under context parallelism: the compressed KV and the rotary key are gathered (not per-head K/V);
    outputs, input gradients and summed parameter gradients equal the single-rank layer's."""
    import os
    import sys

    sys.path.insert(0, os.path.dirname(__file__))
    from dist_utils import run_distributed

    run_distributed(_mla_cp_body, world, (cu, sparse), timeout=300)
