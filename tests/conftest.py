import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle import tk_oracle
    tk_oracle.lib()
    return tk_oracle


@pytest.fixture(autouse=True)
def _guard_bytes_intact(request):
    """After every GPU test: no kernel wrote past the end of a buffer of any cache or exchange that is
    still open (guard bytes behind the arena, the page table, the split-KV workspace, the step metadata
    and the exchange mailbox).  Stands in for a memory checker on out-of-bounds stores."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    from titan_engine_b200.kv import PagedKVCache
    from titan_engine_b200.dist import PeerExchange
    for c in list(PagedKVCache.live):
        c.check_canaries()
    for x in list(PeerExchange.live or []):
        x.check_canaries()
