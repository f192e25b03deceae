import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


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
