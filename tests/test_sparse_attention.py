"""Sparse attention families: statements vs dense attention (CPU) and the CUDA forward vs the statement (GPU)."""
import math

import pytest
import torch

from miles_b200.ops import sparse_attention as SA


def _dense(q, k, v, mask, scale):
    rep = q.shape[1] // k.shape[1]
    kk, vv = k.float().repeat_interleave(rep, 1), v.float().repeat_interleave(rep, 1)
    s = torch.einsum("thd,shd->ths", q.float(), kk) * scale
    s = s.masked_fill(~mask.unsqueeze(1), float("-inf"))
    return torch.einsum("ths,shd->thd", torch.softmax(s, -1), vv)


def test_full_index_list_equals_dense_causal_attention():
    torch.manual_seed(0)
    T, H, Hk, D = 12, 4, 2, 16
    q, k, v = torch.randn(T, H, D), torch.randn(T, Hk, D), torch.randn(T, Hk, D)
    idx = torch.arange(T).view(1, -1).expand(T, T).clone()
    idx[idx > torch.arange(T).view(-1, 1)] = -1
    out, lse = SA.sparse_attention_ref(q, k, v, idx.int())
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    torch.testing.assert_close(out, _dense(q, k, v, mask, 1 / math.sqrt(D)), atol=1e-5, rtol=1e-5)
    assert lse.shape == (T, H)
    # a sink logit only enlarges the denominator
    out_s, _ = SA.sparse_attention_ref(q, k, v, idx.int(), sink=torch.zeros(H))
    assert (out_s.norm(dim=-1) <= out.norm(dim=-1) + 1e-6).all()


def test_indexer_topk_and_dsa_pipeline():
    torch.manual_seed(1)
    T, Hi, Di, H, D = 10, 2, 8, 2, 16
    qi, ki, w = torch.randn(T, Hi, Di), torch.randn(T, Di), torch.rand(T, Hi)
    seq = torch.tensor([0] * 4 + [1] * 6)
    pos = torch.cat([torch.arange(4), torch.arange(6)])
    logits = SA.lightning_indexer(qi, ki, w, pos, pos, seq, seq)
    want = (torch.relu(torch.einsum("thd,sd->ths", qi, ki)) * w.unsqueeze(-1)).sum(1)
    vis = (seq.view(-1, 1) == seq.view(1, -1)) & (pos.view(1, -1) <= pos.view(-1, 1))
    assert torch.equal(torch.isfinite(logits), vis)
    torch.testing.assert_close(logits[vis], want[vis])
    idx = SA.indexer_topk(logits, 3)
    assert idx.shape == (T, 3) and (idx[0] == torch.tensor([0, -1, -1])).all() and idx[4, 0] == 4
    assert all(vis[t, j] for t in range(T) for j in idx[t].tolist() if j >= 0)
    q, k, v = torch.randn(T, H, D, requires_grad=True), torch.randn(T, 1, D), torch.randn(T, 1, D)
    out, idx2, lg = SA.dsa_attention(q, k, v, qi.requires_grad_(), ki, w, topk=3, q_seq=seq, k_seq=seq, q_pos=pos, k_pos=pos)
    out.sum().backward()
    assert q.grad is not None and out.shape == (T, H, D)
    probs = torch.rand(T, 3)
    loss = SA.indexer_kl_loss(lg, probs, idx2)
    loss.backward()
    assert qi.grad is not None and torch.isfinite(loss)


def test_kpool_and_block_sparse():
    torch.manual_seed(2)
    Tkv, T, D, blk = 37, 5, 8, 4
    k = torch.randn(Tkv, D)
    pk = SA.pooled_keys(k, blk)
    torch.testing.assert_close(pk[0], k[:4].mean(0))
    torch.testing.assert_close(pk[-1], k[36:].mean(0))
    q = torch.randn(T, D)
    tok = SA.kpool_select(q, k, blk, top_blocks=2, tail=3)
    assert tok.shape == (T, 2 * blk + 3)
    q_pos = torch.arange(T) + (Tkv - T)
    for t in range(T):
        row = [j for j in tok[t].tolist() if j >= 0]
        assert max(row) == int(q_pos[t]) and sorted(row[-3:]) == list(range(int(q_pos[t]) - 2, int(q_pos[t]) + 1))
        assert all(j <= q_pos[t] for j in row) and len(set(row)) == len(row)
    # block-sparse with every block listed equals dense causal attention
    H = 2
    qq, kk, vv = torch.randn(T, H, D), torch.randn(Tkv, 1, D), torch.randn(Tkv, 1, D)
    nb = (Tkv + blk - 1) // blk
    out, _ = SA.block_sparse_attention(qq, kk, vv, torch.arange(nb).view(1, -1).expand(T, nb).int(), blk)
    mask = torch.arange(Tkv).view(1, -1) <= q_pos.view(-1, 1)
    torch.testing.assert_close(out, _dense(qq, kk, vv, mask, 1 / math.sqrt(D)), atol=1e-5, rtol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("H,Hk,D,Dv", [(8, 2, 128, 128), (16, 1, 576, 512), (4, 4, 64, 64)])
def test_sparse_attention_cuda_forward(H, Hk, D, Dv):
    torch.manual_seed(3)
    T, Tkv, K = 70, 300, 48
    q = torch.randn(T, H, D, device="cuda").bfloat16()
    k = torch.randn(Tkv, Hk, D, device="cuda").bfloat16()
    v = torch.randn(Tkv, Hk, Dv, device="cuda").bfloat16()
    idx = torch.stack([torch.randperm(Tkv, device="cuda")[:K] for _ in range(T)]).int()
    idx[:, 40:] = -1
    idx[3] = -1                                               # a query with nothing visible
    sink = torch.randn(H, device="cuda")
    for sk in (None, sink):
        with torch.no_grad():
            out, lse = SA.sparse_attention(q, k, v, idx, sink=sk)
        ro, rl = SA.sparse_attention_ref(q.float(), k.float(), v.float(), idx, sink=sk)
        torch.testing.assert_close(out.float(), ro, atol=3e-2, rtol=3e-2)
        fin = torch.isfinite(rl)
        torch.testing.assert_close(lse[fin], rl[fin], atol=2e-3, rtol=2e-3)
        if sk is None:
            assert (out[3] == 0).all() and torch.isinf(lse[3]).all()
