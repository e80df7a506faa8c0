"""The debug build of the extension (device-side index checks): an index outside its tensor is recorded and the access is
skipped — the kernel neither traps nor touches the address — and the host reads what went wrong.  Runs in a child process
because the choice of build is made when the extension is first imported."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import sys
import torch
from miles_b200.ops import cuda as K
from miles_b200.ops import cuda_more as KM

if not K.DEBUG_KERNELS:          # never hand a bad index to kernels that do not check it
    sys.exit(3)
bf16, dev = torch.bfloat16, "cuda"

# 1. KV-cache write: 4 blocks x 16 slots = 64 slots; slot 71 does not exist
kc = torch.zeros(4, 16, 2, 128, dtype=bf16, device=dev)
vc = torch.zeros_like(kc)
k = torch.ones(3, 2, 128, dtype=bf16, device=dev)
v = torch.full((3, 2, 128), 2.0, dtype=bf16, device=dev)
K.kv_cache_write(k, v, kc, vc, torch.tensor([5, 71, -1], dtype=torch.int64, device=dev))
torch.cuda.synchronize()
rep = K.bounds_report()
assert len(rep) == 1 and rep[0]["unit"] == "elementwise.cu" and rep[0]["code"] == 102, rep
assert rep[0]["index"] == 71 and rep[0]["limit"] == 64 and rep[0]["count"] > 0, rep
flat = kc.view(64, 2, 128)
assert bool((flat[5] == 1).all()) and float(kc.float().sum()) == 2 * 128 and float(vc.float().sum()) == 2 * 2 * 128
assert K.bounds_report() == []                      # the report cleared the record

# 2. MoE gather: 2 tokens x k = 1 -> pairs 0..1; row 2 names pair 100
x = torch.arange(2 * 256, dtype=torch.float32, device=dev).reshape(2, 256).to(bf16)
x_perm = torch.full((4, 256), 7.0, dtype=bf16, device=dev)
K.publish_limit(K.LIMIT_MOE_PAIRS, 2)
K.C.moe_gather(x, x_perm, torch.tensor([1, 0, 100, -1], dtype=torch.int32, device=dev), torch.tensor([0, 4], dtype=torch.int32, device=dev), 1)
torch.cuda.synchronize()
rep = K.bounds_report()
assert len(rep) == 1 and rep[0]["unit"] == "moe.cu" and rep[0]["code"] == 201 and rep[0]["index"] == 100 and rep[0]["limit"] == 2, rep
assert torch.equal(x_perm[0], x[1]) and torch.equal(x_perm[1], x[0]) and float(x_perm[2].float().abs().sum()) == 0.0

# 3. paged decode: the block table of request 1 names block 9 of a 4-block cache
kc = torch.randn(4, 64, 2, 128, device=dev).to(bf16)
vc = torch.randn(4, 64, 2, 128, device=dev).to(bf16)
q = torch.randn(2, 8, 128, device=dev).to(bf16)
bt = torch.tensor([[0, 1], [2, 9]], dtype=torch.int32, device=dev)
sl = torch.tensor([100, 100], dtype=torch.int32, device=dev)
out = KM.paged_attention(q, kc, vc, bt, sl)
torch.cuda.synchronize()
rep = K.bounds_report()
assert len(rep) == 1 and rep[0]["unit"] == "paged_decode.cu" and rep[0]["code"] == 301 and rep[0]["index"] == 9 and rep[0]["limit"] == 4, rep
assert bool(torch.isfinite(out.float()).all())
good = KM.paged_attention(q[:1], kc, vc, bt[:1], sl[:1])
assert torch.allclose(out[0].float(), good[0].float(), atol=1e-2) and K.bounds_report() == []
assert K.check_error_flag() == 0
print("debug-build checks ok")
'''


@pytest.mark.gpu
def test_debug_build_records_bad_indices_and_skips_the_access():
    from miles_b200.ops import build as B

    if not os.path.exists(B.so_path(debug=True)):
        pytest.skip("the debug build of the extension is not in the tree (python -m miles_b200.ops.build --debug)")
    env = {**os.environ, "MILES_DEBUG_KERNELS": "1", "PYTHONPATH": ROOT + os.pathsep + os.environ.get("PYTHONPATH", "")}
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "debug-build checks ok" in r.stdout


def test_normal_build_reports_that_it_has_no_checks():
    """CPU: the build helper's paths, and the rule that the checks are opt-in."""
    from miles_b200.ops import build as B

    assert B.so_path(debug=True).endswith("_build_debug/miles_b200_C_debug.so") and B.so_path(debug=False).endswith("_build/miles_b200_C.so")
    assert not B.debug_requested() or os.environ.get("MILES_DEBUG_KERNELS") == "1"
