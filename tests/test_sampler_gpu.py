"""GPU parity of the batched sampler against the CPU oracle, through the C ABI.

Bar: token ids, Top-K index sets, row status and RNG consumption bit-exact;
probabilities within 1e-5 relative of the reference arithmetic and bit-exact
against the oracle port run with the device's exp rounding.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_reference_unit_vectors(pkg, parity):
    # tests/test_runtime.cpp:4333-4362 of the reference
    cases = [
        (np.array([[1, 2, 3]], dtype=np.float32), dict(temperature=0.0), 2, 0),
        (np.array([[3, np.nan, 3]], dtype=np.float32), dict(temperature=0.0), 0, 0),
        (np.array([[np.nan, np.inf]], dtype=np.float32), dict(temperature=0.0), -1, 5),
        (np.array([[1, 2, 3]], dtype=np.float32), dict(top_k=1), 2, 0),
        (np.array([[1, 2, 3]], dtype=np.float32), dict(top_p=0.0), -1, 3),
    ]
    for logits, options, token, status in cases:
        params = pkg.make_row_params(1, **options)
        out = parity.run(logits, params)
        assert out["token"][0] == token and out["status"][0] == status
        if status == 0:
            assert out["probability"][0] == 1.0


def test_config1_single_row(pkg, workloads, parity):
    logits, params = workloads.config1_row(pkg.ROW_PARAMS_DTYPE, rows=1)
    parity.check(logits, params, topk_stride=50)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_headline_shape_small_batch(pkg, workloads, parity, dtype):
    logits, params = workloads.config1_row(pkg.ROW_PARAMS_DTYPE, rows=32, dtype=dtype, seed=11)
    parity.check(logits, params, topk_stride=50)


def test_config2_greedy_and_temperature(pkg, workloads, parity):
    logits, params = workloads.config2_greedy_temperature(pkg.ROW_PARAMS_DTYPE, rows=24)
    parity.check(logits, params)


def test_config3_mixed_parameters(pkg, workloads, parity):
    logits, params = workloads.config3_mixed(pkg.ROW_PARAMS_DTYPE, rows=48)
    parity.check(logits, params, topk_stride=100)


def test_config4_heavy_tail(pkg, workloads, parity):
    logits, params = workloads.config4_heavy_tail(pkg.ROW_PARAMS_DTYPE, rows=64)
    parity.check(logits, params)


def test_config5a_large_vocab_single_gpu(pkg, workloads, parity):
    logits, params = workloads.config5a_large_vocab(pkg.ROW_PARAMS_DTYPE, rows=4)
    parity.check(logits, params, topk_stride=64)


@pytest.mark.parametrize("vocab", [1, 2, 3, 7, 33, 255, 256, 257, 1023, 1025, 4099, 8191])
def test_ragged_small_vocabularies(pkg, parity, vocab):
    rng = np.random.default_rng(vocab)
    rows = 16
    logits = (3 * rng.standard_normal((rows, vocab))).astype(np.float32)
    logits[rng.random((rows, vocab)) < 0.2] = logits[0, 0]      # many exact duplicates
    params = pkg.make_row_params(rows, temperature=rng.uniform(0.3, 1.5, rows).astype(np.float32),
                                 top_k=rng.choice([0, 1, 2, 5, 50, 2000], rows).astype(np.uint32),
                                 top_p=rng.uniform(0.5, 1.0, rows).astype(np.float32),
                                 min_p=rng.choice([0, 0.05], rows).astype(np.float32), seed=vocab)
    params["temperature"][::5] = 0.0
    parity.check(logits, params, topk_stride=64)
    parity.check(logits, params, topk_stride=64, host=True)


def test_unaligned_rows_and_bf16_tail(pkg, parity, torch_cuda):
    torch = torch_cuda
    rng = np.random.default_rng(5)
    rows, vocab, stride = 6, 5003, 5009       # odd stride: every row has a different 16-byte phase
    block = (3 * rng.standard_normal((rows, stride))).astype(np.float32)
    params = pkg.make_row_params(rows, temperature=0.8, top_k=[0, 10, 40, 0, 1, 300], top_p=0.9, seed=5)
    for dtype in ("f32", "bf16"):
        if dtype == "bf16":
            from_bits = __import__("ncnn_moe_runtime_b200.workloads", fromlist=["x"]).to_bf16_bits(block)
            device = torch.from_numpy(from_bits.view(np.int16)).cuda().view(torch.bfloat16)
            logical = from_bits[:, :vocab].copy()
        else:
            device = torch.from_numpy(block).cuda()
            logical = block[:, :vocab].copy()
        out = parity.sampler.sample_batch(device, params, vocab=vocab, topk_stride=16)
        torch.cuda.synchronize()
        uniforms = parity.uniforms(params)
        want = parity.checker.sample_batch(logical, params["temperature"], params["top_k"], params["top_p"], params["min_p"], uniforms)
        np.testing.assert_array_equal(out["token"].cpu().numpy(), want["token"])


def test_non_finite_logits(pkg, parity):
    rng = np.random.default_rng(9)
    vocab = 3000
    base = (2 * rng.standard_normal(vocab)).astype(np.float32)
    rows = []
    a = base.copy(); a[rng.integers(0, vocab, 500)] = -np.inf; rows.append(a)            # masked logits are legal
    b = np.full(vocab, -np.inf, dtype=np.float32); rows.append(b)                          # nothing finite
    c = base.copy(); c[17] = np.inf; rows.append(c)                                        # +inf at the head is an error
    d = np.full(vocab, -np.inf, dtype=np.float32); d[5] = 1.0; rows.append(d)             # a single finite logit
    logits = np.stack(rows)
    for options in (dict(temperature=0.0), dict(top_k=40, top_p=0.9), dict(top_p=0.95), dict(top_k=5000)):
        params = pkg.make_row_params(len(rows), seed=3, **options)
        parity.check(logits, params, topk_stride=40)


def test_invalid_parameters_per_row(pkg, parity):
    logits = np.tile(np.arange(100, dtype=np.float32), (6, 1))
    params = pkg.make_row_params(6, temperature=[1, -1, np.nan, 1, 1, 1], top_p=[1, 1, 1, 0, 1.5, 1], min_p=[0, 0, 0, 0, 0, -0.1])
    out = parity.run(logits, params)
    assert out["status"].tolist() == [0, 2, 2, 3, 3, 4]
    assert [pkg.row_status_message(s) for s in out["status"][1:]] == [
        "temperature must be finite and non-negative", "temperature must be finite and non-negative",
        "top_p must be in the range (0, 1]", "top_p must be in the range (0, 1]", "min_p must be in the range [0, 1]"]


def test_extreme_temperatures(pkg, parity):
    rng = np.random.default_rng(21)
    logits = (3 * rng.standard_normal((8, 4096))).astype(np.float32)
    params = pkg.make_row_params(8, temperature=[1e-30, 1e-6, 1e-3, 50.0, 1e6, 1e30, 3e38, 0.01], top_k=[0, 0, 10, 0, 20, 0, 0, 0], top_p=0.9, seed=4)
    parity.check(logits, params)


def test_top_p_one_still_truncates(pkg, parity):
    # the cumulative reaches 1.0f before the last candidate; ids beyond are unreachable (session.cpp:119-128)
    rng = np.random.default_rng(33)
    logits = (3 * rng.standard_normal((4, 60000))).astype(np.float32)
    params = pkg.make_row_params(4, temperature=[1.0, 0.7, 1.3, 1.0], top_p=1.0, seed=8)
    parity.check(logits, params)


def test_stop_tokens_and_resident_parameters(pkg, parity, torch_cuda):
    torch = torch_cuda
    rng = np.random.default_rng(2)
    rows, vocab = 8, 3001
    logits = (3 * rng.standard_normal((rows, vocab))).astype(np.float32)
    params = pkg.make_row_params(rows, temperature=0.0)
    greedy = logits.argmax(axis=1)
    stops = [[int(greedy[r]), 7] if r % 2 == 0 else [int((greedy[r] + 1) % vocab)] for r in range(rows)]
    out = parity.run(logits, params, stop_lists=stops)
    flagged = (out["flags"] & pkg.ROW_FLAG_STOP_TOKEN) != 0
    assert flagged.tolist() == [r % 2 == 0 for r in range(rows)]
    # resident parameters + step offset: same uniforms as explicit steps
    params = pkg.make_row_params(rows, temperature=1.0, top_k=50, seed=77)
    device = torch.from_numpy(logits).cuda()
    parity.sampler.sample_batch(device, params)
    for step in (1, 2, 5):
        out = parity.sampler.sample_batch(device, None, step_offset=step)
        torch.cuda.synchronize()
        explicit = params.copy(); explicit["step"] = step
        want = parity.checker.sample_batch(logits, explicit["temperature"], explicit["top_k"], explicit["top_p"], explicit["min_p"], parity.uniforms(explicit))
        np.testing.assert_array_equal(out["token"].cpu().numpy(), want["token"])


def test_adversarial_orderings(pkg, parity):
    vocab = 70000
    ascending = np.arange(vocab, dtype=np.float32) * 1e-3
    constant = np.zeros(vocab, dtype=np.float32)
    plateau = np.concatenate([np.full(vocab // 2, 5.0, dtype=np.float32), np.arange(vocab - vocab // 2, dtype=np.float32) * 1e-4 + 5.0])
    logits = np.stack([ascending, ascending[::-1].copy(), constant, plateau])
    for options in (dict(top_k=50, top_p=0.9), dict(top_k=1024), dict(temperature=0.0), dict(top_p=0.9)):
        params = pkg.make_row_params(4, seed=6, **options)
        parity.check(logits, params, topk_stride=64)


@pytest.mark.parametrize("mixed", [False, True], ids=["topk_only", "with_live_and_greedy_rows"])
def test_overlapped_launches_give_the_same_results(pkg, workloads, parity, torch_cuda, mixed):
    """Programmatic dependent launch: consecutive calls may overlap on the GPU; every call
    must still produce exactly what it produces alone (independent batches, separate outputs).
    With Top-K rows only, one streaming launch follows the other directly; with live rows the
    full-vocabulary kernel runs in between."""
    torch = torch_cuda
    logits, params = workloads.config1_row(pkg.ROW_PARAMS_DTYPE, rows=96, vocab=50021, seed=21)
    if mixed:
        params["top_k"][::7] = 0              # some rows go through the live / exact paths
        params["temperature"][::11] = 0.0     # some greedy rows
    batches = [torch.from_numpy(np.roll(logits, shift, axis=0).copy()).cuda() for shift in range(4)]
    sampler = pkg.Sampler(max_rows=96, max_vocab=50021)
    try:
        alone = []
        sampler.sample_batch(batches[0], params)
        for step, batch in enumerate(batches):
            out = sampler.sample_batch(batch, None, step_offset=step, topk_stride=50)
            torch.cuda.synchronize()
            alone.append({k: v.clone() for k, v in out.items()})
        if mixed:
            for out in alone:   # rows without Top-K (whichever kernel finished them) and greedy rows list nothing
                assert bool((out["topk"][::7] == -1).all()) and bool((out["topk"][::11] == -1).all())
        sampler.set_overlap(True)
        together = []
        for repeat in range(3):
            for step, batch in enumerate(batches):
                together.append((step, sampler.sample_batch(batch, None, step_offset=step, topk_stride=50)))   # no synchronisation in between
        torch.cuda.synchronize()
        for step, out in together:
            for key in ("token", "probability", "flags", "status", "topk"):
                if not torch.equal(out[key], alone[step][key]):
                    bad = torch.nonzero((out[key] != alone[step][key]).reshape(96, -1).any(dim=1)).flatten().tolist()
                    raise AssertionError(f"step {step} {key}: rows {bad[:8]} differ: "
                                         f"{out[key][bad[0]].tolist()} vs alone {alone[step][key][bad[0]].tolist()}; params {params[bad[0]]}")
        # and against the oracle for one of them
        explicit = params.copy()
        explicit["step"] = 2
        shifted = np.roll(logits, 2, axis=0)
        want = parity.checker.sample_batch(shifted, explicit["temperature"], explicit["top_k"], explicit["top_p"], explicit["min_p"], parity.uniforms(explicit))
        np.testing.assert_array_equal(alone[2]["token"].cpu().numpy(), want["token"])
    finally:
        sampler.close()


def _check_kept_lists(pkg, parity, torch, logits, params, kept_stride):
    """kept_count / kept_token / kept_probability against sampling_distribution of the oracle:
    ids exact, probabilities within 1e-5 of the reference arithmetic and bit-exact against
    the port run with the device's exp rounding; the sampled token agrees with the plain call."""
    device_logits = parity.device_logits(logits)
    rows = logits.shape[0]
    sampler = pkg.Sampler(max_rows=rows, max_vocab=logits.shape[1])
    try:
        out = sampler.sample_batch(device_logits, params, kept_stride=kept_stride)
        plain = sampler.sample_batch(device_logits, None)
        torch.cuda.synchronize()
        out = {k: v.cpu().numpy() for k, v in out.items() if v is not None}
        np.testing.assert_array_equal(out["token"], plain["token"].cpu().numpy())
        np.testing.assert_array_equal(out["probability"].view(np.uint32), plain["probability"].cpu().numpy().view(np.uint32))
    finally:
        sampler.close()
    widened = logits if logits.dtype == np.float32 else (logits.astype(np.uint32) << 16).view(np.float32)
    parity.port.set_exp_mode(1)
    try:
        for r in range(rows):
            p = params[r]
            if out["status"][r] != 0:
                assert out["kept_count"][r] == 0
                continue
            if p["temperature"] == 0.0:
                assert out["kept_count"][r] == 1 and out["kept_token"][r, 0] == out["token"][r] and out["kept_probability"][r, 0] == 1.0
                continue
            args = (widened[r], float(p["temperature"]), int(p["top_k"]), float(p["top_p"]), float(p["min_p"]))
            ids, probabilities = parity.checker.distribution(*args)
            count = int(out["kept_count"][r])
            assert count == ids.size, (r, count, ids.size)
            shown = min(count, kept_stride)
            np.testing.assert_array_equal(out["kept_token"][r, :shown], ids[:shown], err_msg=f"row {r}")
            np.testing.assert_allclose(out["kept_probability"][r, :shown], probabilities[:shown], rtol=1e-5, atol=0, err_msg=f"row {r}")
            _, exact = parity.port.distribution(*args)
            np.testing.assert_array_equal(out["kept_probability"][r, :shown].view(np.uint32), exact[:shown].view(np.uint32), err_msg=f"row {r}")
            assert np.all(out["kept_token"][r, shown:] == -1)   # entries past the list stay untouched
    finally:
        parity.port.set_exp_mode(0)


def test_kept_candidate_lists_match_sampling_distribution(pkg, workloads, parity, torch_cuda):
    """moe_sample_batch_ex: the vector sampling_distribution returns (session.cpp:76-136), per row."""
    logits, params = workloads.config3_mixed(pkg.ROW_PARAMS_DTYPE, rows=40, vocab=30011, seed=9)
    params["temperature"][::9] = 0.0      # greedy rows list their token alone
    params["top_p"][3] = 2.0              # a rejected row lists nothing
    _check_kept_lists(pkg, parity, torch_cuda, logits, params, kept_stride=128)


def test_kept_candidate_lists_on_golden_rows(pkg, parity, torch_cuda):
    """The committed reference fixture holds full candidate lists for its first rows."""
    from pathlib import Path
    g = np.load(Path(__file__).parent / "golden" / "sampler_reference.npz")
    rows = g["logits"].shape[0]
    params = np.zeros(rows, dtype=pkg.ROW_PARAMS_DTYPE)
    for name in ("temperature", "top_k", "top_p", "min_p"):
        params[name] = g[name]
    params["seed"], params["row_id"] = 5, np.arange(rows)
    sampler = pkg.Sampler(max_rows=rows, max_vocab=g["logits"].shape[1])
    try:
        out = sampler.sample_batch(torch_cuda.from_numpy(g["logits"]).cuda(), params, kept_stride=g["logits"].shape[1])
        torch_cuda.cuda.synchronize()
        out = {k: v.cpu().numpy() for k, v in out.items() if v is not None}
    finally:
        sampler.close()
    cursor = 0
    checked = 0
    for r, count in enumerate(g["dist_count"]):
        if count < 0:
            assert out["kept_count"][r] == 0 or params["temperature"][r] == 0.0
            continue
        assert out["kept_count"][r] == count
        np.testing.assert_array_equal(out["kept_token"][r, :count], g["dist_ids"][cursor:cursor + count])
        np.testing.assert_allclose(out["kept_probability"][r, :count], g["dist_probability"][cursor:cursor + count], rtol=1e-5, atol=0)
        cursor += count
        checked += 1
    assert checked > 8


def test_kept_candidate_lists_without_top_k(pkg, workloads, parity, torch_cuda):
    """Rows without Top-K: short lists finish in the streaming kernel, long ones in the full-vocabulary kernel."""
    logits, params = workloads.config2_greedy_temperature(pkg.ROW_PARAMS_DTYPE, rows=12, vocab=20011, seed=4)
    params["top_p"][1::2] = np.linspace(0.3, 1.0, params["top_p"][1::2].size)
    _check_kept_lists(pkg, parity, torch_cuda, logits, params, kept_stride=20011)


def test_sampled_tokens_from_device_logits(pkg, workloads, parity, torch_cuda):
    """moe_sample_tokens (LogitsOutputMode::SampledToken): logits stay on the device, one 16-byte record per row
    returns; the records equal what moe_sample_batch writes, and the tokens equal the oracle's."""
    torch = torch_cuda
    logits, params = workloads.config3_mixed(pkg.ROW_PARAMS_DTYPE, rows=40, vocab=30011)
    params["top_p"][5] = 0.0                                      # one rejected row
    device = torch.from_numpy(logits).cuda()
    stops = [[int(t)] for t in np.argmax(logits, axis=1)]          # every row's stop list: its arg-max
    want = parity.sampler.sample_batch(device, params, stop_lists=stops)
    torch.cuda.synchronize()
    records = parity.sampler.sample_tokens(device, params, stop_lists=stops)
    assert records.dtype.itemsize == 16
    np.testing.assert_array_equal(records["token"], want["token"].cpu().numpy())
    np.testing.assert_array_equal(records["probability"].view(np.uint32), want["probability"].cpu().numpy().view(np.uint32))
    np.testing.assert_array_equal(records["flags"], want["flags"].cpu().numpy().view(np.uint32))
    np.testing.assert_array_equal(records["status"], want["status"].cpu().numpy())
    assert records["status"][5] == 3 and records["token"][5] == -1
    uniforms = parity.uniforms(params)
    oracle = parity.checker.sample_batch(logits, params["temperature"], params["top_k"], params["top_p"], params["min_p"], uniforms)
    np.testing.assert_array_equal(records["token"], oracle["token"])
    # resident parameters and a step offset, into page-locked memory
    pinned = torch.empty(40 * 16, dtype=torch.uint8).pin_memory()
    view = pinned.numpy().view(pkg.SAMPLED_ROW_DTYPE)
    parity.sampler.sample_tokens(device, None, step_offset=3, results=view)
    oracle = parity.checker.sample_batch(logits, params["temperature"], params["top_k"], params["top_p"], params["min_p"], parity.uniforms(params, 3))
    np.testing.assert_array_equal(view["token"], oracle["token"])


def test_handles_on_two_devices_in_one_process(pkg, workloads, checker, torch_cuda):
    """Kernels that need more than 48 KiB of shared memory opt in per device; a second handle on another GPU of
    the same process must work like the first."""
    torch = torch_cuda
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    logits, params = workloads.config1_row(pkg.ROW_PARAMS_DTYPE, rows=8, vocab=60000, seed=3)
    params["top_k"][:] = 600                                      # the large-buffer instantiation
    uniforms = np.array([pkg.philox_uniform(p["seed"], p["row_id"], p["step"]) for p in params], dtype=np.float32)
    want = checker.sample_batch(logits, params["temperature"], params["top_k"], params["top_p"], params["min_p"], uniforms)
    for device in (0, 1):
        with torch.cuda.device(device):
            handle = pkg.Sampler(max_rows=8, max_vocab=60000, device=device)
            out = handle.sample_batch(torch.from_numpy(logits).cuda(device), params)
            torch.cuda.synchronize(device)
            np.testing.assert_array_equal(out["token"].cpu().numpy(), want["token"])
            wide = np.random.default_rng(device).standard_normal((4, 2048)).astype(np.float32)
            plan = handle.router_dispatch_host(wide, 4, 2048, 8)
            oracle = checker.expert_dispatch(wide, 4, 2048, 8)
            np.testing.assert_array_equal(plan.route_token[:32], oracle["token"])
            handle.close()


def test_bf16_rows_without_topk_are_replayed_over_value_runs(pkg, workloads, parity):
    """bf16 rows without Top-K skip the sort: their candidates are (value, count) runs of a histogram, and the
    reference's sequential sums are replayed over the runs.  Long runs (few distinct values) put the binade
    crossings and the Top-P / draw stops in the middle of runs."""
    rng = np.random.default_rng(77)
    rows, vocab = 28, 40000
    values = (2.0 * rng.standard_normal((rows, vocab))).astype(np.float32)
    values[4:8] = np.round(values[4:8] * 2) / 2                 # about 40 distinct values: runs of a thousand candidates
    values[8:10] = np.round(values[8:10])                       # about 15 distinct values
    values[10] = 1.25                                           # one value only
    values[11] = np.where(rng.random(vocab) < 0.5, 3.0, 2.5)    # two values
    values[12, rng.integers(0, vocab, 9)] = values[12].max()    # ties at the head
    values[13, rng.integers(0, vocab, 3000)] = -np.inf          # masked logits
    values[14] = -np.abs(values[14]) - 3.0                      # everything negative
    values[15] = values[15] * 8.0                               # a peaked row: one or two candidates kept
    values[16, ::2] = 0.0
    values[16, 1::2] = -0.0                                     # zeros of both signs are one value
    logits = workloads.to_bf16_bits(values)
    params = pkg.make_row_params(rows, temperature=rng.choice([0.5, 1.0, 1.7], rows).astype(np.float32), top_k=0,
                                 top_p=rng.choice([0.3, 0.9, 0.999, 1.0], rows).astype(np.float32),
                                 min_p=rng.choice([0.0, 0.0, 1e-4, 0.02], rows).astype(np.float32), seed=77)
    params["top_k"][20:24] = 5000                               # above the on-chip limit: same path, shortened list
    for step in (0, 1, 2):
        params["step"] = step
        parity.check(logits, params)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_more_rows_than_resident_ctas(pkg, workloads, parity, dtype):
    """With more rows than CTAs that fit the GPU at once, a CTA takes several rows in turn and asks for the next
    row's first bytes while it finishes the current one: every kind of row in every position, invalid rows included."""
    rng = np.random.default_rng(91)
    rows, vocab = 1000, 9000 + (0 if dtype == "f32" else 11)
    values = (3.0 * rng.standard_normal((rows, vocab))).astype(np.float32)
    values[rng.integers(0, rows, 40), rng.integers(0, vocab, 40)] += 9.0
    params = pkg.make_row_params(rows, temperature=rng.choice([0.0, 0.6, 1.0, 1.4], rows).astype(np.float32),
                                 top_k=rng.choice([0, 1, 8, 50, 300, 700], rows).astype(np.uint32),
                                 top_p=rng.uniform(0.4, 1.0, rows).astype(np.float32),
                                 min_p=rng.choice([0.0, 0.03], rows).astype(np.float32), seed=91)
    params["top_p"][::97] = 0.0                                   # rejected rows in between
    logits = values if dtype == "f32" else workloads.to_bf16_bits(values)
    parity.check(logits, params, topk_stride=8)


def test_fp32_rows_without_topk_are_ordered_by_value_buckets_or_by_digits(pkg, parity):
    """fp32 rows without Top-K are put in rank order by value buckets (one scatter, then a look inside
    each bucket); rows whose values pile up in a bucket, span more than fp32 can subtract, or hold one
    value fall back to the byte-digit sort.  Every shape must give the reference's token, bit for bit,
    and more rows than CTAs go through the row queue."""
    rng = np.random.default_rng(404)
    vocab = 40009
    rows = []
    rows.append((3.0 * rng.standard_normal(vocab)).astype(np.float32))                      # spread values: buckets
    piled = (3.0 * rng.standard_normal(vocab)).astype(np.float32)
    piled[rng.choice(vocab, 1500, replace=False)] = np.float32(1.2345)                      # 1500 copies of one value: digits
    rows.append(piled)
    rows.append(np.where(rng.random(vocab) < 0.5, np.float32(2.0), np.float32(-1.0)).astype(np.float32))   # two values
    wide = (3.0 * rng.standard_normal(vocab)).astype(np.float32)
    wide[7], wide[11] = np.float32(3.0e38), np.float32(-3.0e38)                             # span overflows fp32
    rows.append(wide)
    near = np.float32(5.0) + (rng.integers(0, 40, vocab).astype(np.float32) * np.float32(2.0 ** -20))   # forty adjacent values
    rows.append(near.astype(np.float32))
    tiny = np.full(vocab, -np.inf, dtype=np.float32)
    tiny[[3, 30000]] = [0.5, 0.25]                                                           # two finite logits
    rows.append(tiny)
    dense = (0.01 * rng.standard_normal(vocab)).astype(np.float32)                          # everything live, narrow range
    rows.append(dense)
    logits = np.stack(rows * 24)                                                            # 168 rows: more than resident CTAs
    count = logits.shape[0]
    temperatures = np.tile(np.array([1.0, 0.7, 1.5, 0.4], dtype=np.float32), count)[:count]
    top_p = np.tile(np.array([1.0, 0.9, 0.97], dtype=np.float32), count)[:count]
    min_p = np.tile(np.array([0.0, 0.0, 0.001, 0.0, 0.02], dtype=np.float32), count)[:count]
    params = pkg.make_row_params(count, seed=77, temperature=temperatures, top_k=0, top_p=top_p, min_p=min_p)
    params["step"] = np.arange(count) % 5
    parity.check(logits, params)
