import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


# ---- parity errors, both ways ------------------------------------------------------------------------------------
# Every output comparison records the error graded with the reference's floor (the asserted one) and the pure
# relative error max|y - ref| / |ref| beside it; the table is printed at the end of the run.
_PARITY = {}
_CURRENT = [None]


def record_parity(floored: float, pure: float, label: str | None = None):
    key = label or _CURRENT[0] or "?"
    f0, p0, n = _PARITY.get(key, (0.0, 0.0, 0))
    _PARITY[key] = (max(f0, float(floored)), max(p0, float(pure)), n + 1)


@pytest.fixture(autouse=True)
def _parity_scope(request):
    _CURRENT[0] = request.node.nodeid.split("::", 1)[-1]
    yield
    _CURRENT[0] = None


def pytest_terminal_summary(terminalreporter):
    if not _PARITY:
        return
    tr = terminalreporter
    tr.section("parity: max error per test, floored (asserted, <= 2e-3) | pure relative (reported)")
    for key in sorted(_PARITY):
        f, p, n = _PARITY[key]
        tr.write_line(f"{f:9.3e} | {p:9.3e} | {n:3d} checks | {key}")
    out = os.path.join(ROOT, "gpurun_out")
    try:
        os.makedirs(out, exist_ok=True)
        import json
        with open(os.path.join(out, "parity_errors.json"), "w") as fh:
            json.dump({k: {"floored": v[0], "pure_relative": v[1], "checks": v[2]} for k, v in _PARITY.items()}, fh, indent=1)
    except OSError:
        pass


def has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.fixture(scope="session")
def oracle_c():
    from oracle import ztvm_oracle_c
    ztvm_oracle_c.build()
    return ztvm_oracle_c


@pytest.fixture(scope="session")
def backend():
    """The CUDA backend on cuda:0. Fails (does not skip) when the library cannot start on a GPU box."""
    if not has_gpu():
        pytest.skip("no CUDA device")
    import zero_tvm_b200 as z
    be = z.backend.CudaMatmulBackend(0)
    yield be
    be.close()


class Dev:
    """numpy <-> device helpers for the GPU tests (torch is only the allocator here)."""

    @staticmethod
    def put(a: np.ndarray):
        import torch
        a = np.ascontiguousarray(a)
        if a.dtype == np.uint32:
            return torch.from_numpy(a.view(np.int32)).cuda()
        if a.dtype == np.uint16:
            return torch.from_numpy(a.view(np.int16)).cuda()
        return torch.from_numpy(a).cuda()

    @staticmethod
    def empty(shape, dtype, fill=None):
        import torch
        tdt = {np.float16: torch.float16, np.float32: torch.float32, np.uint8: torch.uint8,
               np.uint32: torch.int32}[dtype]
        t = torch.empty(shape, dtype=tdt, device="cuda")
        if fill is not None:
            t.fill_(fill)
            # the fill runs on torch's stream and the library launches on its own: order them here, or a late fill
            # could overwrite what a kernel has already written
            torch.cuda.synchronize()
        return t

    @staticmethod
    def get(t, dtype=None) -> np.ndarray:
        import torch
        torch.cuda.synchronize()
        a = t.cpu().numpy()
        if dtype is not None and a.dtype != dtype:
            a = a.view(dtype)
        return a


@pytest.fixture(scope="session")
def dev():
    return Dev
