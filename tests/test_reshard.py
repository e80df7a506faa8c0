"""Weight-sync resharding: rectangles computed on CPU for every pair of layouts, applied with plain indexing, must turn
the shards of one layout into the shards of another bit-exactly; the GPU case runs the one-kernel transfer into peer
buffers (2 GPUs, trainer TP = 2 and EP = 2 into full-weight engines)."""
import itertools

import pytest
import torch

from miles_b200.models.config import PRESETS
from miles_b200.models.qwen3 import build_model
from miles_b200.parallel.reshard import local_2d, plan_copies
from miles_b200.parallel.state import ParallelState


def _ps(tp, tp_rank, ep, ep_rank):
    ps = ParallelState(world_size=max(tp, ep), rank=0, tp_size=tp, tp_rank=tp_rank, ep_size=ep, ep_rank=ep_rank,
                       sequence_parallel=False)
    return ps


def _shards(name, tp, ep):
    cfg = PRESETS[name]
    out = {}
    for t, e in itertools.product(range(tp), range(ep)):
        m = build_model(cfg, _ps(tp, t, ep, e), dtype=torch.float32, device="cpu", seed=3)
        out[(t, e)] = {n: p.detach().clone() for n, p in m.named_parameters()}
    return cfg, out


@pytest.mark.parametrize("name,src,dst", [("tiny", (2, 1), (1, 1)), ("tiny", (1, 1), (2, 1)), ("tiny", (2, 1), (2, 1)),
                                          ("tiny-moe", (1, 2), (1, 1)), ("tiny-moe", (2, 2), (1, 4)), ("tiny-moe", (1, 4), (2, 2))])
def test_rectangles_turn_one_layout_into_another(name, src, dst):
    cfg, S = _shards(name, *src)
    _, D = _shards(name, *dst)
    for (dt, de), want in D.items():
        got = {n: torch.full_like(p, float("nan")) for n, p in want.items()}
        for (st, se), have in S.items():
            for n, p in have.items():
                rects = plan_copies(n, tuple(p.shape), tuple(want[n].shape), cfg, (src[0], st, src[1], se), (dst[0], dt, dst[1], de))
                s2, d2 = p.reshape(local_2d(tuple(p.shape))), got[n].view(local_2d(tuple(want[n].shape)))
                for (sr, sc, dr, dc, nr, ncol) in rects:
                    d2[dr:dr + nr, dc:dc + ncol] = s2[sr:sr + nr, sc:sc + ncol]
        for n in want:
            assert torch.equal(got[n], want[n]), (n, src, dst, (dt, de))


# ---- 2 GPUs: the one-kernel transfer into peer memory ---------------------------------------------------------------

def _case_reshard(rank, world):
    import torch.distributed as dist

    from miles_b200.args import parse_args
    from miles_b200.engine.engine import Engine
    from miles_b200.models.config import ModelConfig
    from miles_b200.parallel.fabric import Fabric
    from miles_b200.train.actor import TrainActor
    from miles_b200.weight_update.updater import WeightUpdater

    for kind in ("tp", "ep"):
        cfg = ModelConfig(name=f"reshard-{kind}", vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                          ffn_hidden_size=512, **({"num_experts": 4, "moe_topk": 2, "moe_ffn_hidden_size": 128} if kind == "ep" else {}))
        ps = ParallelState.build(tp=world if kind == "tp" else 1, ep=world if kind == "ep" else 1, sequence_parallel=False)
        ps.fabric = Fabric.create(ps)
        args = parse_args("--rollout-batch-size 2 --n-samples-per-prompt 2 --num-rollout 1 --lr 1e-5 --colocate".split())
        actor = TrainActor(args, ps, device=f"cuda:{rank}")
        actor.init(cfg)
        # the engine of every rank holds the FULL model (layout tp = ep = 1) in buffers of its own
        eng = Engine(cfg, ps=ParallelState.single(), device=f"cuda:{rank}", num_blocks=8, block_size=64, use_cuda_graph=False, seed=99)
        want = {n: p.detach().clone() for n, p in build_model(cfg, ParallelState.single(), dtype=torch.bfloat16, device=f"cuda:{rank}",
                                                              seed=getattr(args, "seed", 0)).named_parameters()}
        for quant in (None, "mxfp8_qdq"):
            with torch.no_grad():
                for p in eng.model.parameters():
                    p.fill_(7.0)
            up = WeightUpdater(args, actor, [eng], quant=quant)
            assert up.mode == "nvlink"
            info = up.update_weights()
            torch.cuda.synchronize()
            ps.fabric.check()
            assert info["bytes"] > 0
            from miles_b200.ops import reference as ref
            from miles_b200.parallel.weight_sync import _skip_quant

            for n, p in eng.model.named_parameters():
                w = want[n]
                if quant and not _skip_quant(n, w) and w.dtype == torch.bfloat16:
                    q, sc = ref.mxfp8_quant(w.cpu())
                    w = ref.mxfp8_dequant(q, sc).reshape(w.shape).to(torch.bfloat16).to(p.device)
                assert torch.equal(p.data, w), (kind, quant, n, (p.data.float() - w.float()).abs().max().item())
        dist.barrier()


@pytest.mark.gpu
@pytest.mark.multigpu
def test_trainer_shards_land_in_full_engines_bit_exact():
    import test_multigpu as M

    M._run("_case_reshard_proxy", world=2, timeout=240)
