import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def orc():
    from oracle_lib import oracle
    return oracle()


@pytest.fixture(scope="session")
def figures():
    """record(name, **numbers): appends one JSON line per measured parity figure to the file named by
    MB_FIGURES_FILE (nothing is written when the variable is unset). The figures quoted in the design notes
    come from such a file."""
    import json
    path = os.environ.get("MB_FIGURES_FILE")

    def record(name, **numbers):
        if path:
            with open(path, "a") as f:
                f.write(json.dumps({"name": name, **{k: float(v) for k, v in numbers.items()}}) + "\n")
    return record
