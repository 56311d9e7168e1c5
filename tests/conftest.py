import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_sessionstart(session):
    """Built libraries are not in the history: compile the CUDA library and the C oracle when nvcc /
    gcc are there.  The build is incremental (by modification time), so a source edit can never be
    tested against an old binary; a machine without nvcc uses the prebuilt library as it is."""
    import shutil
    from library_b200 import build as lib_build
    if shutil.which(lib_build._nvcc()) or not os.path.exists(lib_build.LIB):
        lib_build.build()
    import oracle
    oracle.lib()


def load_golden():
    """tests/golden/csr_golden.npz -> {case: {field: array}} (made by tests/golden/make_golden.py
    from the reference's own CPU code)."""
    z = np.load(os.path.join(ROOT, "tests", "golden", "csr_golden.npz"))
    out = {}
    for key in z.files:
        case, field = key.split("/")
        out.setdefault(case, {})[field] = z[key]
    for c in out.values():
        for f in ("alpha", "beta"):
            c[f] = float(c[f])
        c["kind"] = str(c["kind"])
        c["cols"] = int(c["cols"])
    return out


@pytest.fixture(scope="session")
def golden():
    return load_golden()


def load_golden_complex():
    """tests/golden/csr_golden_complex.npz: complex mv / mm cases from the reference's alphasparse_{c,z}_mv / _mm
    (same generator script)."""
    z = np.load(os.path.join(ROOT, "tests", "golden", "csr_golden_complex.npz"))
    out = {}
    for key in z.files:
        case, field = key.split("/")
        out.setdefault(case, {})[field] = z[key]
    for c in out.values():
        for f in ("alpha", "beta"):
            c[f] = complex(c[f])
        c["kind"] = str(c["kind"])
        c["cols"] = int(c["cols"])
    return out


def rel_l2(a, b):
    wide = np.complex128 if (np.iscomplexobj(a) or np.iscomplexobj(b)) else np.float64
    a = np.asarray(a, dtype=wide).ravel()
    b = np.asarray(b, dtype=wide).ravel()
    d = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / d) if d > 0 else float(np.linalg.norm(a - b))


def max_rel(a, b):
    """The reference test drivers' own metric: max|a-b| / max|b| (cuda/test/check.cu:145-158)."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    m = np.abs(b).max() if b.size else 0.0
    return float(np.abs(a - b).max() / m) if m > 0 else 0.0


@pytest.fixture(scope="session")
def handle():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from library_b200 import api
    torch.cuda.set_device(0)
    return api.Handle()
