"""Rollout engine on CPU: paged-KV decode equals a full forward, continuous batching, retraction, pause/abort,
weight updates and the HTTP surface."""
import threading
import time

import pytest
import torch

from miles_b200.engine.engine import Engine
from miles_b200.engine.kv_cache import BlockAllocator
from miles_b200.models.config import PRESETS
from miles_b200.models.qwen3 import ForwardMeta


def _engine(name="tiny", **kw):
    kw.setdefault("num_blocks", 64)
    kw.setdefault("block_size", 4)
    return Engine(PRESETS[name], device="cpu", dtype=torch.float32, seed=0, **kw)


def _full_forward_logprobs(engine, ids):
    T = len(ids)
    meta = ForwardMeta(positions=torch.arange(T, dtype=torch.int32), cu_seqlens=torch.tensor([0, T], dtype=torch.int32), max_seqlen=T)
    h = engine.model(torch.tensor(ids, dtype=torch.int32), meta)
    return torch.log_softmax(engine.model.logits(h).float(), -1)


@pytest.mark.parametrize("name", ["tiny", "tiny-moe"])
def test_greedy_decode_matches_full_forward(name):
    eng = _engine(name)
    prompt = [5, 9, 13, 21, 34, 55, 89]
    out = eng.generate(prompt, {"temperature": 0.0, "max_new_tokens": 9})
    ids = out["output_ids"]
    assert len(ids) == 9 and out["meta_info"]["finish_reason"]["type"] == "length"
    lp = _full_forward_logprobs(eng, prompt + ids)
    for i, t in enumerate(ids):
        row = lp[len(prompt) + i - 1]
        assert int(row.argmax()) == t
        assert abs(float(row[t]) - out["meta_info"]["output_token_logprobs"][i][0]) < 1e-4


def test_sampled_logprobs_are_the_models():
    eng = _engine()
    prompt = [3, 4, 5, 6]
    out = eng.generate(prompt, {"temperature": 1.0, "max_new_tokens": 6, "seed": 7})
    ids = out["output_ids"]
    lp = _full_forward_logprobs(eng, prompt + ids)
    for i, (t, (got, tid, _)) in enumerate(zip(ids, out["meta_info"]["output_token_logprobs"])):
        assert tid == t and abs(float(lp[len(prompt) + i - 1, t]) - got) < 1e-4
    again = eng.generate(prompt, {"temperature": 1.0, "max_new_tokens": 6, "seed": 7})
    assert again["output_ids"] == ids                                   # per-request seed → reproducible


def test_continuous_batching_equals_one_by_one():
    eng = _engine()
    prompts = [[7, 8, 9], [11, 12, 13, 14, 15, 16], [20], [30, 31, 32, 33]]
    sp = {"temperature": 0.0, "max_new_tokens": 7}
    solo = [eng.generate(p, sp)["output_ids"] for p in prompts]
    batch = [o["output_ids"] for o in eng.generate(prompts, sp)]
    assert solo == batch
    assert eng._free_blocks() == 64                                     # every block returned (or held by the prefix cache only)


def test_stop_tokens_and_eos():
    eng = _engine()
    free_run = eng.generate([5, 6, 7], {"temperature": 0.0, "max_new_tokens": 8})["output_ids"]
    stop = free_run[3]
    out = eng.generate([5, 6, 7], {"temperature": 0.0, "max_new_tokens": 8, "stop_token_ids": [stop]})
    assert out["output_ids"] == free_run[: free_run.index(stop) + 1]
    assert out["meta_info"]["finish_reason"]["type"] == "stop"


def test_retraction_under_block_pressure_keeps_results():
    sp = {"temperature": 0.0, "max_new_tokens": 12}
    prompts = [[i + 3, i + 4, i + 5, i + 6] for i in range(6)]
    want = [o["output_ids"] for o in _engine(num_blocks=64).generate(prompts, sp)]
    small = _engine(num_blocks=12)                                      # 48 slots for 6 × 16 tokens
    got = [o["output_ids"] for o in small.generate(prompts, sp)]
    assert got == want and small.stats["retractions"] > 0


def test_pause_abort_and_weight_version_spans():
    eng = _engine()
    req = eng.add_request([4, 5, 6], {"temperature": 0.0, "max_new_tokens": 50})
    for _ in range(4):
        eng.step()
    eng.pause_generation("retract")
    assert not eng.running and eng.step() is False
    eng.update_weight_version(3)
    eng.continue_generation()
    for _ in range(3):
        eng.step()
    eng.abort_request(None)
    assert req.done.is_set()
    r = req.to_response(eng)
    assert r["meta_info"]["finish_reason"]["type"] == "abort" and len(r["output_ids"]) > 0
    versions = [v for v, _ in r["meta_info"]["weight_version_spans"]]
    assert versions == sorted(versions) and versions[-1] == 3


def test_routed_experts_returned_for_moe():
    from miles_b200.types import decode_routed_experts

    eng = _engine("tiny-moe")
    cfg = eng.cfg
    out = eng.generate([3, 4, 5, 6, 7], {"temperature": 0.0, "max_new_tokens": 4}, return_routed_experts=True)
    n = 5 + 4
    n_moe = sum(cfg.layer_is_moe(i) for i in range(cfg.num_layers))
    arr = decode_routed_experts(out["meta_info"]["routed_experts"], n, n_moe, cfg.moe_topk)
    assert arr.shape == (n - 1, n_moe, cfg.moe_topk) and arr.max() < cfg.num_experts and arr.min() >= 0


def test_update_weights_from_tensor_changes_outputs():
    a, b = _engine(), Engine(PRESETS["tiny"], device="cpu", dtype=torch.float32, seed=1, num_blocks=64, block_size=4)
    sp = {"temperature": 0.0, "max_new_tokens": 6}
    assert a.generate([9, 8, 7], sp)["output_ids"] != b.generate([9, 8, 7], sp)["output_ids"]
    b.update_weights_from_tensor([(n, p.detach()) for n, p in a.model.named_parameters()], weight_version=5)
    assert a.generate([9, 8, 7], sp)["output_ids"] == b.generate([9, 8, 7], sp)["output_ids"]
    assert b.get_weight_version() == 5


def test_block_allocator_refcounts():
    al = BlockAllocator(8)
    a = al.alloc(3)
    assert al.num_free == 5 and al.alloc(6) is None
    al.share(a)
    al.release(a)
    assert al.num_free == 5
    al.release(a)
    assert al.num_free == 8


def test_http_server_and_router_roundtrip():
    import requests

    from miles_b200.engine.server import serve
    from miles_b200.router.router import Router, serve as serve_router

    eng = _engine()
    srv, _ = serve(eng, port=31731, in_thread=True)
    router = Router()
    router.add_worker("http://127.0.0.1:31731")
    rsrv, _ = serve_router(router, port=31732, in_thread=True)
    try:
        body = {"input_ids": [5, 6, 7], "sampling_params": {"temperature": 0.0, "max_new_tokens": 5}, "return_logprob": True}
        direct = requests.post("http://127.0.0.1:31731/generate", json=body, timeout=60).json()
        routed = requests.post("http://127.0.0.1:31732/generate", json=body, timeout=60).json()
        assert direct["output_ids"] == routed["output_ids"] and len(direct["output_ids"]) == 5
        assert len(routed["meta_info"]["output_token_logprobs"]) == 5
        assert requests.get("http://127.0.0.1:31732/list_workers", timeout=10).json()["urls"] == ["http://127.0.0.1:31731"]
        assert requests.get("http://127.0.0.1:31731/health", timeout=10).status_code == 200
        requests.post("http://127.0.0.1:31731/update_weight_version", json={"weight_version": 9}, timeout=10)
        assert requests.get("http://127.0.0.1:31731/get_weight_version", timeout=10).json()["weight_version"] == "9"
        router.remove_worker("http://127.0.0.1:31731")
        assert requests.post("http://127.0.0.1:31732/generate", json=body, timeout=10).status_code == 503
    finally:
        srv.should_exit = True
        rsrv.should_exit = True
        eng._stop_loop = True
        time.sleep(0.1)


@pytest.mark.parametrize("name,plen", [("tiny", 10), ("tiny", 12), ("tiny-moe", 7)])
def test_samples_of_one_prompt_share_prompt_kv(name, plen):
    """The n samples of a prompt prefill it once: same tokens and log-probs as without sharing under fixed seeds, an
    n-th of the prefill tokens, fewer blocks in use, and the routed experts of the shared prompt reach every sample."""
    prompts = [[5 + i for i in range(plen)]] * 4 + [[40, 41, 42]] * 2 + [[9, 8, 7, 6, 5]]
    sps = [{"temperature": 1.0, "max_new_tokens": 6, "seed": 100 + i} for i in range(len(prompts))]
    res = {}
    for share in (True, False):
        eng = _engine(name, share_prompt_kv=share)
        free0 = eng.allocator.num_free
        reqs = [eng.add_request(p, dict(sp), True, name == "tiny-moe") for p, sp in zip(prompts, sps)]
        eng.step()                                             # the prefill step
        used_after_prefill = free0 - eng.allocator.num_free
        while not all(r.done.is_set() for r in reqs):
            eng.step()
        res[share] = ([r.to_response(eng) for r in reqs], eng.stats["prefill_tokens"], used_after_prefill)
        assert eng._free_blocks() == free0                     # every reference was released (the prefix cache holds the rest)
    (a, tok_a, used_a), (b, tok_b, used_b) = res[True], res[False]
    assert tok_a == plen + 3 + 5 and tok_b == 4 * plen + 2 * 3 + 5
    assert used_a < used_b
    for x, y in zip(a, b):
        assert x["output_ids"] == y["output_ids"]
        for (l1, t1, _), (l2, t2, _) in zip(x["meta_info"]["output_token_logprobs"], y["meta_info"]["output_token_logprobs"]):
            assert t1 == t2 and abs(l1 - l2) < 1e-5
        assert x["meta_info"].get("routed_experts") == y["meta_info"].get("routed_experts")
    assert a[1]["meta_info"]["cached_tokens"] == plen and a[0]["meta_info"]["cached_tokens"] == 0
    # siblings really diverge (different seeds), so the shared blocks were not written by anyone's decode steps
    assert len({tuple(x["output_ids"]) for x in a[:4]}) > 1


# ---- prefix (radix) cache and chunked prefill --------------------------------------------------------------------------

def test_prefix_cache_tree_pins_and_evicts():
    from miles_b200.engine.kv_cache import BlockAllocator
    from miles_b200.engine.prefix_cache import PrefixCache

    al = BlockAllocator(16)
    pc = PrefixCache(al, 4)
    a = al.alloc(3)
    toks = list(range(12))
    mine = pc.insert(toks, a)
    assert [n.block for n in mine] == a and pc.num_nodes == 3
    al.release(a)                                            # the request is gone; the tree keeps the blocks alive
    assert al.num_free == 13 and pc.evictable() == 3
    assert [n.block for n in pc.match(toks + [99])] == a
    assert [n.block for n in pc.match(toks[:8] + [77, 78, 79, 80])] == a[:2]     # diverges in the third block
    assert pc.match(toks, max_blocks=2)[-1].block == a[1]
    got = pc.acquire(toks[:8])                               # a request takes the first two blocks
    assert [n.users for n in got] == [1, 1] and pc.evictable() == 1               # only the unpinned leaf may go
    b = al.alloc(1)
    other = pc.insert(toks[:8] + [50, 51, 52, 53], [a[0], a[1], b[0]])            # a sibling branch below the shared prefix
    assert len(other) == 3 and pc.num_nodes == 4
    assert pc.evict(10) == 2 and pc.num_nodes == 2           # both leaves; the pinned chain stays
    pc.unpin(got)
    al.release([n.block for n in got])
    al.release(b)
    assert pc.evictable() == 2 and pc.evict(1) == 1          # leaf first: the tree never loses an inner node before its children
    assert [n.block for n in pc.match(toks)] == a[:1]
    assert pc.reset() == 1 and al.num_free == 16


def _gen(eng, prompts, sps):
    outs = eng.generate(prompts, sps)
    return [(o["output_ids"], [round(x[0], 5) for x in o["meta_info"]["output_token_logprobs"]], o["meta_info"]["cached_tokens"]) for o in outs]


@pytest.mark.parametrize("name", ["tiny", "tiny-moe"])
def test_prefix_cache_and_chunked_prefill_keep_results(name):
    """Multi-turn style prompts (each extends the previous conversation) through an engine with the prefix cache, and long
    prompts through chunked prefill: same tokens and log-probs as an engine that recomputes everything in one piece."""
    base = [3 + (i * 7) % 50 for i in range(37)]
    turn2 = base + [60, 61, 62, 63, 64]
    turn3 = turn2 + [70, 71] * 9
    sp = {"temperature": 0.0, "max_new_tokens": 5}
    plain = _engine(name, prefix_cache=False)
    want = [_gen(plain, [p], [dict(sp)])[0] for p in (base, turn2, turn3, base)]
    assert all(w[2] == 0 for w in want)
    cached = _engine(name)
    got = [_gen(cached, [p], [dict(sp)])[0] for p in (base, turn2, turn3, base)]
    for w, g in zip(want, got):
        assert w[0] == g[0] and max(abs(x - y) for x, y in zip(w[1], g[1])) < 1e-4
    bs = cached.block_size
    assert [g[2] for g in got] == [0, (len(base) // bs) * bs, (len(turn2) // bs) * bs, ((len(base) - 1) // bs) * bs]
    assert cached.stats["prefix_cache_hit_tokens"] == sum(g[2] for g in got) and cached.stats["extend_tokens"] > 0
    assert cached._free_blocks() == plain._free_blocks()
    # generated tokens are cached too: a prompt that continues the model's own answer hits beyond the old prompt
    cont = base + want[0][0] + [5, 6, 7]
    assert _gen(cached, [cont], [dict(sp)])[0][2] >= ((len(base) + len(want[0][0]) - 1) // bs) * bs - bs
    # a weight update invalidates the cache
    cached.update_weight_version(3)
    assert cached.prefix_cache.num_nodes == 0 and _gen(cached, [turn2], [dict(sp)])[0][2] == 0
    # chunked prefill: pieces of 16 tokens, several requests in flight, mixed with short prompts
    chunked = _engine(name, prefix_cache=False, chunked_prefill_size=16, max_prefill_tokens=24)
    prompts = [turn3, [9, 8, 7], turn2, base[:20]]
    sps = [{"temperature": 1.0, "max_new_tokens": 6, "seed": 11 + i} for i in range(4)]
    w2 = _gen(plain, prompts, [dict(s) for s in sps])
    g2 = _gen(chunked, prompts, [dict(s) for s in sps])
    for w, g in zip(w2, g2):
        assert w[0] == g[0] and max(abs(x - y) for x, y in zip(w[1], g[1])) < 1e-4
    assert chunked.stats["extend_tokens"] > 0 and chunked._free_blocks() == plain._free_blocks()


def test_eviction_under_pressure_keeps_serving():
    """A cache that fills the pool gives blocks back (least recently used first) instead of failing or retracting."""
    eng = _engine("tiny", num_blocks=24)
    sp = {"temperature": 0.0, "max_new_tokens": 4}
    outs = []
    for i in range(12):
        p = [5 + i] * 30 + [40 + i]
        outs.append(eng.generate(p, dict(sp))["output_ids"])
    assert eng.prefix_cache.stats["evicted_blocks"] > 0 and eng.stats["retractions"] == 0
    again = eng.generate([5 + 11] * 30 + [40 + 11], dict(sp))
    assert again["output_ids"] == outs[11] and again["meta_info"]["cached_tokens"] > 0


def test_prefix_cache_unpinned_count_stays_exact():
    """The scheduler reads `evictable()` every step, so it is a counter: it must equal a walk of the tree through inserts,
    pins by two requests with a common prefix, a reset under a live request, and evictions."""
    from miles_b200.engine.prefix_cache import PrefixCache

    class Alloc:
        def __init__(self):
            self.refs = {}

        def share(self, blocks):
            for b in blocks:
                self.refs[b] = self.refs.get(b, 0) + 1

        def release(self, blocks):
            for b in blocks:
                self.refs[b] -= 1

    def walk(c):
        stack, n = list(c.root.children.values()), 0
        while stack:
            x = stack.pop()
            stack.extend(x.children.values())
            n += x.users == 0
        return n

    a = Alloc()
    c = PrefixCache(a, 2)
    t1, t2 = [1, 2, 3, 4, 5, 6], [1, 2, 3, 4, 9, 9]
    n1 = c.insert(t1, [10, 11, 12]); c.pin(n1)
    n2 = c.insert(t2, [20, 21, 22]); c.pin(n2)          # shares two nodes that own request 1's blocks
    assert c.evictable() == walk(c) == 0 and c.num_nodes == 4
    c.unpin(n1)
    assert c.evictable() == walk(c) == 1                 # only request 1's private tail
    assert c.evict(5) == 1 and c.evictable() == walk(c) == 0
    c.reset()
    c.unpin(n2)                                          # the request finishes after the reset
    assert c.evictable() == walk(c) == 0 and c.num_nodes == 0
    n3 = c.insert(t1, [30, 31, 32])
    assert c.evictable() == walk(c) == 3
    assert c.evict(2) == 2 and c.evictable() == walk(c) == 1


def test_output_top_logprobs_contain_the_sampled_token_and_are_sorted():
    """`top_logprobs_num` on a generating request: one entry per generated token with the k most likely tokens under the
    request's temperature; the greedy token is entry 0 and its log-prob equals the reported one."""
    import torch

    from miles_b200.engine.engine import Engine
    from miles_b200.models.config import PRESETS

    eng = Engine(PRESETS["tiny"], device="cpu", dtype=torch.float32, num_blocks=64)
    ids = list(range(5, 25))
    for temp in (0.0, 0.7):
        r = eng.add_request(ids, {"temperature": temp, "max_new_tokens": 6, "seed": 3}, True, top_logprobs_num=4)
        while not r.finished:
            eng.step()
        out = r.to_response(eng)
        tops = out["meta_info"]["output_top_logprobs"]
        assert len(tops) == 6 and all(len(t) == 4 for t in tops)
        for (lp, tok, _), top in zip(out["meta_info"]["output_token_logprobs"], tops):
            assert [x[0] for x in top] == sorted((x[0] for x in top), reverse=True)
            if temp == 0.0:
                assert top[0][1] == tok and abs(top[0][0] - lp) < 1e-4
            hit = [x for x in top if x[1] == tok]
            assert not hit or abs(hit[0][0] - lp) < 1e-4
    plain = eng.generate(ids, {"temperature": 0.0, "max_new_tokens": 3})
    assert "output_top_logprobs" not in plain["meta_info"]


@pytest.mark.parametrize("model", ["tiny", "tiny-moe"])
def test_prefill_decode_disaggregation_matches_one_engine(model):
    """Prompts run on a prefill engine, the KV moves as one tensor, decoding continues on another engine: tokens, log-probs,
    routed experts and finish reasons equal those of a single engine; both engines end with every block free."""
    import asyncio

    import torch

    from miles_b200.engine.engine import Engine
    from miles_b200.engine.pd import PDClient
    from miles_b200.models.config import PRESETS

    cfg = PRESETS[model]
    mk = lambda: Engine(cfg, device="cpu", dtype=torch.float32, num_blocks=96, seed=5)
    ref, P, D = mk(), mk(), mk()
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(3, cfg.vocab_size, (int(n),), generator=g).tolist() for n in (5, 16, 33, 47)]
    sps = [{"temperature": 0.0, "max_new_tokens": m, "stop_token_ids": list(range(0, cfg.vocab_size, 5)) if i == 2 else []}
           for i, m in enumerate((6, 1, 12, 9))]
    want = ref.generate(prompts, [dict(sp) for sp in sps], return_routed_experts=True)
    client = PDClient([P], [D])

    async def run():
        outs = await asyncio.gather(*[client.generate({"input_ids": p, "sampling_params": dict(sp), "return_logprob": True,
                                                       "return_routed_experts": True}) for p, sp in zip(prompts, sps)])
        await client.finish()
        return outs

    got = asyncio.run(run())
    from miles_b200.types import decode_routed_experts
    for w, o, p in zip(want, got, prompts):
        assert o["output_ids"] == w["output_ids"] and o["meta_info"]["finish_reason"]["type"] == w["meta_info"]["finish_reason"]["type"]
        a = [x[0] for x in o["meta_info"]["output_token_logprobs"]]
        b = [x[0] for x in w["meta_info"]["output_token_logprobs"]]
        assert max(abs(x - y) for x, y in zip(a, b)) < 1e-5
        if cfg.is_moe:
            n = len(p) + len(w["output_ids"])
            r1 = decode_routed_experts(w["meta_info"]["routed_experts"], n, ref.model.num_moe_layers, cfg.moe_topk)
            r2 = decode_routed_experts(o["meta_info"]["routed_experts"], n, ref.model.num_moe_layers, cfg.moe_topk)
            assert (r1 == r2).all()
    assert client.stats["requests"] >= 2 and D.stats["received_kv_tokens"] == client.stats["handed_over_tokens"]
    assert D.stats["prefill_tokens"] == 0                                 # the decode engine never ran a prompt
    for e in (P, D):
        assert not e.held_kv and not e.running and e._free_blocks() == e.allocator.num_blocks


def test_prefill_decode_disaggregation_over_http():
    """Two engine servers, one in each role: `/prefill` → `/generate_prefilled` → `/release_kv` give the single-engine answer
    (the KV travels as bytes between CPU engines, as a CUDA-IPC handle between GPU ones)."""
    import asyncio

    from miles_b200.engine.pd import PDHttpClient
    from miles_b200.engine.server import serve

    ref, P, D = _engine("tiny-moe"), _engine("tiny-moe"), _engine("tiny-moe")
    ps, _ = serve(P, port=31741, in_thread=True)
    ds, _ = serve(D, port=31742, in_thread=True)
    try:
        prompt = list(range(7, 40))
        sp = {"temperature": 0.0, "max_new_tokens": 7}
        want = ref.generate(prompt, dict(sp), return_routed_experts=True)
        client = PDHttpClient(["http://127.0.0.1:31741"], ["http://127.0.0.1:31742"])

        async def run():
            out = await client.generate({"input_ids": prompt, "sampling_params": dict(sp), "return_logprob": True,
                                         "return_routed_experts": True})
            await client.finish()
            return out

        got = asyncio.run(run())
        assert got["output_ids"] == want["output_ids"]
        assert got["meta_info"]["routed_experts"] == want["meta_info"]["routed_experts"]
        a, b = ([x[0] for x in o["meta_info"]["output_token_logprobs"]] for o in (got, want))
        assert max(abs(x - y) for x, y in zip(a, b)) < 1e-5
        assert not P.held_kv and D.stats["received_kv_tokens"] == len(prompt) and D.stats["prefill_tokens"] == 0
    finally:
        ps.should_exit = True
        ds.should_exit = True
        P._stop_loop = D._stop_loop = True
        time.sleep(0.1)


def _multi_rank_body(rank, world, mode, port, out_dir):
    import json
    import threading

    import torch

    from miles_b200.engine import multi_rank_server as mrs
    from miles_b200.engine.engine import Engine
    from miles_b200.models.config import PRESETS
    from miles_b200.parallel.state import ParallelState, init_distributed

    init_distributed(backend="gloo")
    cfg = PRESETS["tiny-moe" if mode == "ep" else "tiny"]
    ps = ParallelState.build(tp=world if mode == "tp" else 1, ep=world if mode == "ep" else 1, sequence_parallel=False)
    eng = Engine(cfg, ps=ps, device="cpu", dtype=torch.float32, num_blocks=96, seed=4)

    def client():
        import requests

        url = f"http://127.0.0.1:{port}"
        for _ in range(200):
            try:
                if requests.get(f"{url}/health", timeout=2).status_code == 200:
                    break
            except Exception:
                time.sleep(0.1)
        g = torch.Generator().manual_seed(8)
        prompts = [torch.randint(3, cfg.vocab_size, (int(n),), generator=g).tolist() for n in (6, 19, 11, 25, 9)]
        outs = [None] * len(prompts)

        def one(i):
            outs[i] = requests.post(f"{url}/generate", json={"input_ids": prompts[i], "return_logprob": True,
                                                             "sampling_params": {"temperature": 0.0, "max_new_tokens": 5 + i}}, timeout=120).json()

        ts = [threading.Thread(target=one, args=(i,)) for i in range(len(prompts))]
        [t.start() for t in ts]
        [t.join() for t in ts]
        info = requests.get(f"{url}/health", timeout=10).json()
        requests.post(f"{url}/update_weight_version", json={"weight_version": 3}, timeout=10)
        time.sleep(0.2)
        ver = requests.get(f"{url}/get_weight_version", timeout=10).json()["weight_version"]
        with open(f"{out_dir}/out.json", "w") as f:
            json.dump({"prompts": prompts, "outs": outs, "info": info, "version": ver}, f)
        requests.post(f"{url}/shutdown", timeout=10)

    if rank == 0:
        threading.Thread(target=client, daemon=True).start()
    mrs.start(eng, ps, mode, port=port)


@pytest.mark.parametrize("mode,port", [("ep", 31751), ("tp", 31752)])
def test_multi_rank_engine_server_matches_one_engine(tmp_path, mode, port):
    """Two ranks behind one HTTP port: experts sharded with every rank serving its own requests (`ep`), or projections
    sharded with every rank running every request (`tp`); answers equal a single unsharded engine's."""
    import json
    import os
    import sys

    import torch

    sys.path.insert(0, os.path.dirname(__file__))
    from dist_utils import run_distributed

    from miles_b200.engine.engine import Engine
    from miles_b200.models.config import PRESETS

    run_distributed(_multi_rank_body, 2, (mode, port, str(tmp_path)), timeout=300)
    rec = json.load(open(tmp_path / "out.json"))
    assert rec["info"]["ranks"] == 2 and rec["info"]["mode"] == mode and rec["version"] == "3"
    ref = Engine(PRESETS["tiny-moe" if mode == "ep" else "tiny"], device="cpu", dtype=torch.float32, num_blocks=96, seed=4)
    for i, (p, o) in enumerate(zip(rec["prompts"], rec["outs"])):
        w = ref.generate(p, {"temperature": 0.0, "max_new_tokens": 5 + i})
        assert o["output_ids"] == w["output_ids"], (i, o["output_ids"], w["output_ids"])
        a, b = ([x[0] for x in r["meta_info"]["output_token_logprobs"]] for r in (o, w))
        assert max(abs(x - y) for x, y in zip(a, b)) < 1e-4
