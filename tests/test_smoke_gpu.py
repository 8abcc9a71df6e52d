"""The smoke run of the repository's entry module (a few generated tokens and whole-prompt logits of tiny random
models against the plain implementation), kept under test so that it cannot fall behind the engine."""
import os
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_the_smoke_run_passes():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if root not in sys.path:
        sys.path.insert(0, root)
    import __graft_entry__
    __graft_entry__.smoke()
