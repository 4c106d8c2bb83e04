import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


def load_golden(name):
    with np.load(os.path.join(GOLDEN, name)) as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def wuda():
    """The product package with a live GPU; a GPU test must never run without the built
    CUDA library, so a missing library is an error, not a skip."""
    import torch
    assert torch.cuda.is_available(), "a test marked gpu ran without a GPU"
    import wuda_b200
    return wuda_b200


def assert_close_logits(got, ref, valid, rtol=1e-2, atol_frac=1e-4):
    """|got - ref| <= rtol*|ref| + atol on the valid positions, with atol = atol_frac x
    the RMS of the valid reference values (logits are sums with cancellation across
    heads, so a purely relative bound is ill-conditioned next to zero)."""
    g = got[valid].astype(np.float64)
    r = ref[valid].astype(np.float64)
    assert np.all(np.isfinite(g)), "non-finite values on valid positions"
    rms = float(np.sqrt(np.mean(r * r))) if r.size else 0.0
    err = np.abs(g - r)
    bound = rtol * np.abs(r) + atol_frac * rms
    worst = int(np.argmax(err - bound)) if r.size else 0
    assert np.all(err <= bound), "max violation at flat index %d: got %r ref %r (rms %g)" % (
        worst, g[worst], r[worst], rms)
    return float(err.max()) if r.size else 0.0, rms
