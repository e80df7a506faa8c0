import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")
    config.addinivalue_line("markers", "multigpu: needs at least 2 CUDA devices")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_cuda = torch.cuda.is_available()
        n = torch.cuda.device_count() if has_cuda else 0
    except Exception:
        has_cuda, n = False, 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and not has_cuda:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and n < 2:
            item.add_marker(skip_multi)


@pytest.fixture
def tiny_args():
    from miles_b200.args import parse_args

    def make(extra: str = ""):
        base = ("--model-name tiny --fp32 --rollout-batch-size 4 --n-samples-per-prompt 4 --rollout-max-response-len 8 "
                "--num-rollout 1 --rm-type even_fraction --lr 1e-5 --colocate")
        return parse_args((base + " " + extra).split())

    return make
