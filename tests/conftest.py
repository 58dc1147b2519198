"""Shared fixtures.  GPU tests carry ``@pytest.mark.gpu`` and are skipped without a CUDA device."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (Blackwell sm_100a)")
    config.addinivalue_line("markers", "slow: long-running")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def rng():
    g = torch.Generator()
    g.manual_seed(1234)
    return g


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def collect_children(procs, limit_s):
    """Outputs of all children; when one fails or the limit passes the others are stopped instead of waiting for a peer
    that is gone (they are between steps or blocked on the host: no kernel of theirs waits on the device for long, every
    in-kernel wait is bounded)."""
    import time
    t0 = time.monotonic()
    while time.monotonic() - t0 < limit_s:
        codes = [p.poll() for p in procs]
        if all(c is not None for c in codes) or any(c not in (None, 0) for c in codes):
            break
        time.sleep(0.2)
    time.sleep(1.0)
    for p in procs:
        if p.poll() is None:
            p.kill()
    return [p.communicate()[0] for p in procs]
