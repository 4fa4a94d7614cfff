"""Test configuration: the `gpu` marker and shared helpers.

`-m "not gpu"` covers the oracle against the golden vectors, the host logic and the exported ABI;
`-m gpu` are the parity tests proper: every one of them calls the kernels through the C ABI.
"""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a B200 (runs the CUDA kernels through the C ABI)")


@pytest.fixture(scope="session")
def cuda():
    """torch with a usable CUDA device; GPU tests fail loudly (not skip) when the kernel library is missing."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from krn_b200.runtime import native

    native.library()  # raises LibraryNotFound if the .so was not built: no silent fallback
    torch.cuda.set_device(0)
    return torch


@pytest.fixture(autouse=True)
def _status_word_clean(request):
    """After every GPU test the device status word must be clean (no bounded wait expired)."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import torch

    if torch.cuda.is_available():
        from krn_b200.runtime import native

        torch.cuda.synchronize()
        assert native.device_status()[0] == 0
