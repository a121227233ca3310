import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as graft  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    return graft.load_package()


@pytest.fixture(scope="session")
def workloads(pkg):
    return __import__(graft.PACKAGE_NAME + ".workloads", fromlist=["workloads"])


@pytest.fixture(scope="session")
def oracle_module():
    from oracle import oracle
    return oracle


@pytest.fixture(scope="session")
def port(oracle_module):
    return oracle_module.port()


@pytest.fixture(scope="session")
def reference(oracle_module):
    """The compiled reference sampler, or None where it was never built."""
    return oracle_module.reference()


@pytest.fixture(scope="session")
def checker(oracle_module):
    """The strongest oracle available: the compiled reference, else the port."""
    return oracle_module.best()


@pytest.fixture(scope="session")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch


@pytest.fixture(scope="session")
def sampler(pkg, torch_cuda):
    handle = pkg.Sampler(max_rows=8192, max_vocab=1 << 20)
    yield handle
    handle.close()


class Parity:
    """Shared GPU-vs-oracle comparison used by the parity tests."""

    def __init__(self, pkg, torch, sampler, checker, port):
        self.pkg, self.torch, self.sampler, self.checker, self.port = pkg, torch, sampler, checker, port

    def uniforms(self, params, step_offset=0):
        return np.array([self.pkg.philox_uniform(p["seed"], p["row_id"], int(p["step"]) + step_offset) for p in params], dtype=np.float32)

    def device_logits(self, logits):
        torch = self.torch
        if logits.dtype == np.uint16:
            return torch.from_numpy(logits.view(np.int16)).cuda().view(torch.bfloat16)
        return torch.from_numpy(logits).cuda()

    def run(self, logits, params, topk_stride=0, stop_lists=None, host=False):
        if host:
            return self.sampler.sample_batch_host(logits, params, stop_lists=stop_lists, topk_stride=topk_stride)
        out = self.sampler.sample_batch(self.device_logits(logits), params, stop_lists=stop_lists, topk_stride=topk_stride)
        self.torch.cuda.synchronize()
        return {k: (v.cpu().numpy() if v is not None else None) for k, v in out.items()}

    def check(self, logits, params, topk_stride=0, host=False, rtol=1e-5):
        """Token ids, status and RNG use bit-exact against the reference arithmetic;
        probabilities within rtol (the device rounds expf correctly, libm is 1 ulp off
        for ~6e-4 of arguments); everything bit-exact against the port run with the
        device's exp rounding."""
        out = self.run(logits, params, topk_stride=topk_stride, host=host)
        uniforms = self.uniforms(params)
        args = (logits, params["temperature"], params["top_k"], params["top_p"], params["min_p"], uniforms)
        want = self.checker.sample_batch(*args)
        ok_rows = want["status"] == 0
        status_as_code = np.where(out["status"] == 0, 0, 1)
        np.testing.assert_array_equal(status_as_code, want["status"], err_msg="row status class")
        np.testing.assert_array_equal(out["token"], want["token"], err_msg="token ids vs reference arithmetic")
        np.testing.assert_allclose(out["probability"][ok_rows], want["probability"][ok_rows], rtol=rtol, atol=0)
        used = (out["flags"].astype(np.uint32) & self.pkg.ROW_FLAG_USED_UNIFORM) != 0
        np.testing.assert_array_equal(used[ok_rows], want["used_uniform"][ok_rows] != 0, err_msg="uniform consumption")
        self.port.set_exp_mode(1)
        try:
            exact = self.port.sample_batch(*args)
        finally:
            self.port.set_exp_mode(0)
        np.testing.assert_array_equal(out["token"], exact["token"], err_msg="token ids vs device-rounding port")
        np.testing.assert_array_equal(out["probability"][ok_rows].view(np.uint32), exact["probability"][ok_rows].view(np.uint32),
                                      err_msg="probability bits vs device-rounding port")
        if topk_stride:
            for r in range(logits.shape[0]):
                k = int(params["top_k"][r])
                if params["temperature"][r] == 0 or k == 0 or k > self.pkg.TOPK_FAST_MAX or out["status"][r] != 0:
                    continue
                row = logits[r] if logits.dtype == np.float32 else (logits[r].astype(np.uint32) << 16).view(np.float32)
                listed = min(k, topk_stride, row.size)
                np.testing.assert_array_equal(out["topk"][r, :listed], self.checker.topk_order(row, listed), err_msg=f"Top-K index set row {r}")
        return out, want


@pytest.fixture(scope="session")
def parity(pkg, torch_cuda, sampler, checker, port):
    return Parity(pkg, torch_cuda, sampler, checker, port)
