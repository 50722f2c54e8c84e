"""Shared fixtures.  `-m "not gpu"` runs the oracle pins, host logic and ABI checks on CPU;
`-m gpu` runs the parity tests proper, which call the CUDA library through its C ABI."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def orc():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch


def u16(t):
    """torch bf16 tensor -> numpy uint16 bit pattern."""
    import torch

    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def from_u16(a, device="cuda"):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(device).view(torch.bfloat16)


@pytest.fixture(scope="session")
def layer0(cuda, pkg):
    """One full synthetic layer (257 experts) with the reference-format tensors kept."""
    pkg.load_library()
    from p92moe_b200 import synth

    return synth.make_layer(seed=1234, layer=0, keep_raw=True)


@pytest.fixture(scope="session")
def layer0_host(layer0):
    raw = layer0.raw
    return {
        "packed": raw.packed.cpu().numpy(),
        "scales": raw.scales_linear.cpu().numpy(),
        "alpha": raw.alpha.cpu().numpy(),
        "router": u16(layer0.router_weight),
        "bias": layer0.bias.cpu().numpy(),
    }
