import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle_lib():
    import oracle

    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def tmp_models(tmp_path_factory):
    """Cache of synthetic weight directories keyed by (config, seed)."""
    from espresso_b200.synthetic import write_synthetic_model

    cache = {}

    def get(cfg, seed=1234):
        key = (cfg, seed)
        if key not in cache:
            d = tmp_path_factory.mktemp(cfg.name.replace("/", "_"))
            cache[key] = write_synthetic_model(cfg, str(d), seed=seed)
        return cache[key]

    return get
