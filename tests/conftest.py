import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import binding
    return binding.oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own compiled code, or None where its tree was never mounted."""
    from oracle import binding
    ref_root = os.environ.get("MUGEN_REF_ROOT", "/root/reference")
    if binding.reference() is None and os.path.isdir(os.path.join(ref_root, "src")):
        binding.build(ref=True)
        binding._reference = False
    return binding.reference()


@pytest.fixture(scope="session")
def golden():
    import json
    with open(os.path.join(ROOT, "tests", "golden", "mla_golden.json")) as f:
        return json.load(f)
