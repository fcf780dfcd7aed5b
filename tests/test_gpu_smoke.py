"""The driver's smoke entry point, run as a test: one small quantize + linear on the device against the oracle."""
import pytest

from tests import _util as U

pytestmark = pytest.mark.gpu


def test_smoke_entry_point(capsys):
    U.require_gpu()
    import __graft_entry__ as entry
    entry.smoke()
    assert "smoke ok" in capsys.readouterr().out
