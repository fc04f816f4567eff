"""The entry point the build driver calls on a GPU box: one small decode step and one conversion against the oracle."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


@pytest.mark.gpu
def test_smoke_entry_point_runs():
    import __graft_entry__ as entry

    entry.smoke()
