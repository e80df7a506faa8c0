"""1F1B pipeline order on 4 gloo ranks: gradients equal the single-process model, activations alive stay bounded."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from dist_utils import run_distributed  # noqa: E402

H, M = 16, 6
TOKENS = [5, 9, 3, 7, 4, 8]


def _weights():
    g = torch.Generator().manual_seed(1)
    return [torch.randn(H, H, generator=g) * 0.3 for _ in range(4)]


def _inputs():
    g = torch.Generator().manual_seed(2)
    return [torch.randn(t, H, generator=g) for t in TOKENS]


def _body(rank, world):
    sys.path.insert(0, ROOT)
    from miles_b200.parallel.pp import PipeStage
    from miles_b200.parallel.state import ParallelState

    ps = ParallelState.build(pp=world)
    stage = PipeStage(ps, H, torch.float32, torch.device("cpu"))
    w = _weights()[rank].clone().requires_grad_()
    xs = _inputs()
    alive, peak = [0], [0]

    def forward_step(i, hidden_in):
        x = xs[i] if stage.is_first else hidden_in
        h = torch.tanh(x @ w)
        alive[0] += 1
        peak[0] = max(peak[0], alive[0])
        if stage.is_last:
            loss = (h ** 2).sum()
            loss.register_hook(lambda g: alive.__setitem__(0, alive[0] - 1))
            return None, loss
        h.register_hook(lambda g: alive.__setitem__(0, alive[0] - 1))
        return h, None

    stage.run_1f1b(M, lambda i: TOKENS[i], forward_step)
    # reference: the four stages in one process
    ws = [t.clone().requires_grad_() for t in _weights()]
    for x in xs:
        h = x
        for t in ws:
            h = torch.tanh(h @ t)
        (h ** 2).sum().backward()
    assert torch.allclose(w.grad, ws[rank].grad, atol=1e-5), (w.grad - ws[rank].grad).abs().max()
    assert peak[0] <= world - rank, (rank, peak[0])        # 1F1B bound; the all-forward order would reach M = 6 on every stage


def test_1f1b_matches_single_process_and_bounds_live_activations():
    run_distributed(_body, 4, (), timeout=300)
