"""CPU tests of the drop-in boundary: the library loads without a GPU and exports
exactly what include/moe_b200_sampler.h declares; host-side helpers behave."""
import ctypes
import re
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "moe_b200_sampler.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    library = pkg.library()
    names = declared_functions()
    assert len(names) >= 18
    for name in names:
        assert hasattr(library, name), f"{name} is declared in the header but not exported"
    assert sorted(pkg.EXPORTED_SYMBOLS) == names


def test_row_params_layout_matches_the_header(pkg):
    assert pkg.ROW_PARAMS_DTYPE.itemsize == 40
    assert [pkg.ROW_PARAMS_DTYPE.fields[n][1] for n in ("temperature", "top_k", "top_p", "min_p", "seed", "row_id", "step")] == [0, 4, 8, 12, 16, 24, 32]
    assert ctypes.sizeof(pkg.RouterOptions) == 40


def test_status_tables_carry_the_reference_messages(pkg):
    assert [pkg.row_status_message(c) for c in range(1, 7)] == [
        "cannot sample empty logits", "temperature must be finite and non-negative", "top_p must be in the range (0, 1]",
        "min_p must be in the range [0, 1]", "sampling requires at least one finite logit", "sampling distribution is invalid"]
    library = pkg.library()
    assert [library.moe_row_status_error_code(c) for c in range(0, 8)] == [0, 1, 1, 1, 1, 1, 1, 5]
    assert pkg.router_status_message(101) == "router logits must be finite"
    assert pkg.router_status_message(103) == "selected router weights have a non-positive sum"
    assert library.moe_router_status_error_code(103) == 3 and library.moe_router_status_error_code(105) == 1


def test_router_option_checks_need_no_gpu(pkg):
    library = pkg.library()
    def check(tokens, **kw):
        base = dict(expert_count=8, top_k=2, score_function=0, normalization=1, routed_scaling_factor=1.0, flags=1, selection_bias=None, explicit_expert_ids=None)
        base.update(kw)
        options = pkg.RouterOptions(*[base[f[0]] for f in pkg.RouterOptions._fields_])
        return library.moe_router_check_options(tokens, ctypes.byref(options))
    assert check(4) == 0
    assert check(0) == 104
    assert check(4, top_k=0) == 105 and check(4, top_k=9) == 105 and check(4, expert_count=0) == 105
    assert check(4, routed_scaling_factor=0.0) == 109 and check(4, routed_scaling_factor=float("nan")) == 109
    assert check(4, expert_count=5000, top_k=2) == 110


def test_host_philox_matches_the_oracle(pkg, port):
    for seed, row, step in [(0, 0, 0), (1, 2, 3), (2 ** 40 + 7, 2 ** 33 + 1, 2 ** 35), (2 ** 64 - 1, 2 ** 64 - 1, 2 ** 64 - 1)]:
        assert pkg.philox_uniform(seed, row, step) == port.philox_uniform(seed, row, step)


def test_sampler_needs_a_gpu_and_has_no_fallback(pkg):
    import torch
    if torch.cuda.is_available():
        return
    try:
        pkg.Sampler(8, 128)
    except pkg.MoeError as error:
        assert error.status == 6          # MOE_STATUS_CUDA_ERROR: no device, no CPU path
    else:
        raise AssertionError("creating a sampler without a GPU must fail")


def test_entry_points_refuse_a_null_handle(pkg):
    """Every call that takes a sampler answers MOE_STATUS_INVALID_ARGUMENT (1) to a null handle instead of
    touching the device: checkable without a GPU."""
    library = pkg.library()
    assert library.moe_speculative_verify_batch(None, None, None, None, pkg.DTYPE_F32, 2, 4, 128, 128, None, None, None, None) == 1
    assert library.moe_speculative_verify(None, None, None, None, pkg.DTYPE_F32, 4, 128, 128, None, None, None, None) == 1
    assert library.moe_sample_batch(None, None, None, pkg.DTYPE_F32, 1, 128, 128, None, 0, None, None, None, None, None, None, None, 0) == 1


def test_shard_ranges(pkg):
    parallel = __import__("ncnn_moe_runtime_b200.parallel", fromlist=["x"])
    for total in (0, 1, 7, 256, 8192, 1048576):
        for world in (1, 2, 3, 4, 8):
            ranges = [parallel.shard_range(total, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == total
            assert all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in ranges]
            assert max(sizes) - min(sizes) <= 1
            vocab_ranges = [parallel.vocab_shard_range(total, world, r) for r in range(world)]
            assert vocab_ranges[0][0] == 0 and vocab_ranges[-1][1] == total
            assert all(vocab_ranges[i][1] == vocab_ranges[i + 1][0] for i in range(world - 1))
            assert all(b % 16 == 0 or b == total for b, _ in vocab_ranges)


def test_shared_memory_opt_in_bookkeeping(tmp_path):
    """tests/cpp/opt_in_test.cpp: host-only logic of csrc/moe_internal.h, compiled with the CUDA headers but run without a GPU."""
    import shutil
    import subprocess
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    compiler = shutil.which("g++")
    include = Path("/usr/local/cuda/include")
    if compiler is None or not (include / "cuda_runtime.h").exists():
        import pytest
        pytest.skip("needs g++ and the CUDA headers")
    target = tmp_path / "opt_in_test"
    subprocess.run([compiler, "-std=c++17", "-O1", f"-I{include}", str(root / "tests" / "cpp" / "opt_in_test.cpp"), "-o", str(target)], check=True)
    result = subprocess.run([str(target)], capture_output=True, text=True, timeout=60)
    assert result.returncode == 0, result.stdout + result.stderr
