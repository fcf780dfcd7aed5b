import pathlib
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_addoption(parser):
    parser.addoption("--emu", action="store_true", default=False,
                     help="run the tests marked gpu on the host emulation of the CUDA library (tests/emu)")
    parser.addoption("--emu-big", action="store_true", default=False,
                     help="with --emu: also run the full-size shapes (slow: minutes per case)")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    config.addinivalue_line("markers", "needs_cuda_runtime: cannot run on the host emulation (graphs, CUTLASS library)")
    config.addinivalue_line("markers", "big: full-size shapes, too slow for the host emulation")
    if config.getoption("--emu"):
        from tests.emu import torch_shim
        torch_shim.install()


def pytest_collection_modifyitems(config, items):
    # A GPU test on a machine without a GPU must fail loudly, not pass by skipping:
    # the reference's own testing notes warn against green runs that executed nothing.
    # Selection is by marker (-m gpu / -m "not gpu"), so nothing is auto-skipped here.
    # Order: files as collected, except that files named test_zz_* go last.
    items.sort(key=lambda item: 1 if "test_zz_" in item.nodeid else 0)   # stable
    if config.getoption("--emu"):
        skip_rt = pytest.mark.skip(reason="needs a real CUDA runtime; not part of the emulation run")
        skip_big = pytest.mark.skip(reason="full-size shape; not part of the emulation run")
        for item in items:
            if "needs_cuda_runtime" in item.keywords:
                item.add_marker(skip_rt)
            elif "big" in item.keywords and not config.getoption("--emu-big"):
                item.add_marker(skip_big)
