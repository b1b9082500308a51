import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def nan_filled_allocations(request, monkeypatch):
    """In every GPU test, every floating-point CUDA tensor that is allocated without a value
    (torch.empty, torch.empty_like) starts as NaN, also inside recorded steps, where the fill is
    recorded with them: a row that nothing writes, but that something reads as an operand, then
    shows in the logits whatever the allocator happened to hand out."""
    if "gpu" not in request.keywords:
        yield
        return
    import torch

    empty, empty_like = torch.empty, torch.empty_like

    def poison(t):
        if t.is_cuda and t.is_floating_point() and t.numel():
            t.fill_(float("nan"))
        return t

    monkeypatch.setattr(torch, "empty", lambda *a, **k: poison(empty(*a, **k)))
    monkeypatch.setattr(torch, "empty_like", lambda *a, **k: poison(empty_like(*a, **k)))
    yield
