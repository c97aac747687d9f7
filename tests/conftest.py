import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


try:
    # the property tests draw the same examples on every run (they were explored with random seeds while they were written):
    # a run of the suite is reproducible, and nothing is written next to the sources
    from hypothesis import settings as _hyp_settings

    _hyp_settings.register_profile("repo", derandomize=True, deadline=None, database=None)
    _hyp_settings.load_profile("repo")
except ImportError:      # the property tests are skipped by their own import when hypothesis is missing
    pass


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")
    config.addinivalue_line("markers", "slow: long-running CPU test")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
