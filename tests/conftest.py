import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on a GPU box")


@pytest.fixture(scope="session")
def oracle():
    import oracle as o
    o.build()
    return o


@pytest.fixture(scope="session")
def dev():
    """The device under test.  Fails (never skips) if the CUDA library or the GPU is missing."""
    from dwim_b200 import B200
    d = B200(0)
    yield d
    d.close()


# ---- the error measures the parity tests share ---------------------------------
def max_rel_err(got, want) -> float:
    """max |got - want| / max(|want|, rms(want)): "max relative error" with a
    floor, so that outputs near zero do not make the ratio unbounded."""
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    rms = np.sqrt(np.mean(want * want)) if want.size else 0.0
    den = np.maximum(np.abs(want), max(rms, 1e-30))
    return float(np.max(np.abs(got - want) / den)) if want.size else 0.0


def close(got, want, tol):
    """The reference's single-token check (gpu/tests.rs:132-140)."""
    got, want = np.asarray(got).ravel(), np.asarray(want).ravel()
    assert got.shape == want.shape
    bad = np.abs(got - want) > tol * (1.0 + np.maximum(np.abs(got), np.abs(want)))
    assert not bad.any(), f"element {np.argmax(bad)}: {got[np.argmax(bad)]} vs {want[np.argmax(bad)]}"


def close_batch(got, want, what=""):
    """The reference's batch check (gpu/tests.rs:198-211): rms error within a
    thousandth of the outputs' typical magnitude and a hundredth at worst."""
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    typical = np.sqrt(np.mean(want * want))
    e = np.abs(got - want)
    rms, worst = np.sqrt(np.mean(e * e)), e.max()
    assert rms <= 1e-3 * typical and worst <= 1e-2 * typical, \
        f"{what}: rms {rms:.2e}, worst {worst:.2e}, typical {typical:.2e}"
