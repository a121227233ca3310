"""GPU parity of the speculative-decoding verification step (moe_speculative_verify) against the
CPU oracle (the reference's sampling_distribution / candidate_probability with the accept loop and
the residual draw of src/engine/session.cpp:150-202,776-880 around them).

Bar: accepted count, next token, RNG consumption and status exact; probabilities within 1e-5
relative of the reference arithmetic and bit-exact against the port run with the device's exp rounding.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _uniforms(pkg, seed, row_id, step, count):
    return np.array([pkg.philox_uniform(seed, row_id, step + i) for i in range(count)], dtype=np.float32)


def _case(rng, vocab, draft_count, temperature, top_k, top_p, min_p, closeness, port):
    target = (2.5 * rng.standard_normal((draft_count + 1, vocab))).astype(np.float32)
    draft = (target[:draft_count] + closeness * rng.standard_normal((draft_count, vocab)).astype(np.float32)).astype(np.float32)
    proposed = []
    for j in range(draft_count):   # the draft model samples its own distribution
        if temperature == 0.0:
            proposed.append(int(np.argmax(draft[j])))
        else:
            _, token, _, _, _ = port.sample(draft[j], float(rng.random()), temperature, top_k, top_p, min_p)
            proposed.append(token)
    return target, draft, np.array(proposed, dtype=np.int32)


def _compare(pkg, sampler, torch, parity, target, draft, proposed, options, seed, row_id, step):
    temperature, top_k, top_p, min_p = options
    params = np.zeros(1, dtype=pkg.ROW_PARAMS_DTYPE)
    params["temperature"], params["top_k"], params["top_p"], params["min_p"] = temperature, top_k, top_p, min_p
    params["seed"], params["row_id"], params["step"] = seed, row_id, step
    got = sampler.speculative_verify(torch.from_numpy(target).cuda(), torch.from_numpy(draft).cuda() if proposed.size else None,
                                     torch.from_numpy(proposed).cuda(), params)
    uniforms = _uniforms(pkg, seed, row_id, step, proposed.size + 2)
    want = parity.checker.speculative_verify(target, draft, proposed, uniforms, temperature, top_k, top_p, min_p)
    assert (got["status"] == 0) == (want["status"] == 0), (got, want)
    if want["status"] != 0:
        assert pkg.library().moe_row_status_message(got["status"]).decode() == want["message"]
        return got
    assert got["accepted"] == want["accepted"], (got, want)
    assert got["next_token"] == want["next_token"], (got, want)
    assert got["uniforms_used"] == want["uniforms_used"], (got, want)
    np.testing.assert_allclose(got["accepted_probability"], want["accepted_probability"], rtol=1e-5, atol=0)
    np.testing.assert_allclose(got["next_probability"], want["next_probability"], rtol=1e-5, atol=0)
    parity.port.set_exp_mode(1)
    try:
        exact = parity.port.speculative_verify(target, draft, proposed, uniforms, temperature, top_k, top_p, min_p)
    finally:
        parity.port.set_exp_mode(0)
    if exact["accepted"] == got["accepted"] and exact["next_token"] == got["next_token"]:
        np.testing.assert_array_equal(got["accepted_probability"].view(np.uint32), exact["accepted_probability"].view(np.uint32))
        assert got["next_probability"].view(np.uint32) == exact["next_probability"].view(np.uint32)
    return got


@pytest.mark.parametrize("options", [(1.0, 40, 0.95, 0.0), (0.7, 0, 0.9, 0.02), (1.3, 8, 1.0, 0.0), (1.0, 0, 1.0, 0.0), (0.0, 0, 1.0, 0.0)],
                         ids=["topk40", "nucleus_minp", "hot_topk8", "untruncated", "greedy"])
def test_verification_matches_the_reference_loop(pkg, parity, torch_cuda, options):
    rng = np.random.default_rng([77, int(options[1]), int(options[0] * 10)])
    vocab, draft_count = 6007, 5
    sampler = pkg.Sampler(max_rows=2 * draft_count + 1, max_vocab=vocab)
    accepted_seen = set()
    try:
        for case in range(12):
            closeness = [0.05, 0.4, 1.5][case % 3]   # a good, a fair and a poor draft model
            target, draft, proposed = _case(rng, vocab, draft_count, options[0], options[1], options[2], options[3], closeness, parity.port)
            if options[0] == 0.0 and case % 2:
                proposed[rng.integers(draft_count)] = int(rng.integers(vocab))   # a wrong greedy proposal
            got = _compare(pkg, sampler, torch_cuda, parity, target, draft, proposed, options, seed=11, row_id=case, step=3 * case)
            accepted_seen.add(got["accepted"])
    finally:
        sampler.close()
    assert len(accepted_seen) >= 2    # the cases really exercise both rejection and the bonus token


def test_verification_edge_cases(pkg, parity, torch_cuda):
    rng = np.random.default_rng(5)
    vocab = 2051
    sampler = pkg.Sampler(max_rows=9, max_vocab=vocab)
    try:
        # no proposals: the step is an ordinary sample of the single target row
        target, draft, proposed = _case(rng, vocab, 0, 0.8, 20, 0.9, 0.0, 0.3, parity.port)
        _compare(pkg, sampler, torch_cuda, parity, target, draft, proposed, (0.8, 20, 0.9, 0.0), seed=2, row_id=0, step=5)
        # a proposal outside the draft's kept candidates: the reference's internal error
        target, draft, proposed = _case(rng, vocab, 3, 1.0, 4, 1.0, 0.0, 0.3, parity.port)
        proposed[1] = int(np.argmin(draft[1]))
        got = _compare(pkg, sampler, torch_cuda, parity, target, draft, proposed, (1.0, 4, 1.0, 0.0), seed=2, row_id=1, step=0)
        # identical models: every proposal is accepted with probability 1 unless the uniform is exactly... never rejected
        target, _, _ = _case(rng, vocab, 4, 1.0, 50, 1.0, 0.0, 0.0, parity.port)
        draft = target[:4].copy()
        proposed = np.array([parity.port.sample(draft[j], float(rng.random()), 1.0, 50, 1.0, 0.0)[1] for j in range(4)], dtype=np.int32)
        got = _compare(pkg, sampler, torch_cuda, parity, target, draft, proposed, (1.0, 50, 1.0, 0.0), seed=2, row_id=2, step=9)
        assert got["accepted"] == 4
        # a target row without any finite logit fails at that position, like the reference
        target, draft, proposed = _case(rng, vocab, 2, 1.0, 10, 1.0, 0.0, 0.05, parity.port)
        target[0, :] = -np.inf
        _compare(pkg, sampler, torch_cuda, parity, target, draft, proposed, (1.0, 10, 1.0, 0.0), seed=2, row_id=3, step=0)
    finally:
        sampler.close()


def test_host_buffer_entry_point_gives_the_same_outcome(pkg, parity, torch_cuda):
    """moe_speculative_verify_host (host logits, what a Session holds) against the device-buffer call."""
    rng = np.random.default_rng(12)
    vocab, draft_count = 4099, 3
    sampler = pkg.Sampler(max_rows=2 * draft_count + 1, max_vocab=vocab)
    try:
        for case, options in enumerate([(1.0, 30, 0.9, 0.0), (0.0, 0, 1.0, 0.0), (0.9, 0, 0.8, 0.01)]):
            target, draft, proposed = _case(rng, vocab, draft_count, *options, 0.5, parity.port)
            params = np.zeros(1, dtype=pkg.ROW_PARAMS_DTYPE)
            params["temperature"], params["top_k"], params["top_p"], params["min_p"] = options
            params["seed"], params["row_id"], params["step"] = 4, case, 2
            device = sampler.speculative_verify(torch_cuda.from_numpy(target).cuda(), torch_cuda.from_numpy(draft).cuda(),
                                                torch_cuda.from_numpy(proposed).cuda(), params)
            host = sampler.speculative_verify_host(target, draft, proposed, params)
            for key in ("accepted", "next_token", "uniforms_used", "status"):
                assert host[key] == device[key], (key, host, device)
            assert host["next_probability"].view(np.uint32) == device["next_probability"].view(np.uint32)
            np.testing.assert_array_equal(host["accepted_probability"].view(np.uint32), device["accepted_probability"].view(np.uint32))
    finally:
        sampler.close()


def test_batch_of_sessions_equals_each_session_alone(pkg, parity, torch_cuda):
    """moe_speculative_verify_batch: Sessions with their own options, seeds and steps verified side by side give, each,
    the outcome of the reference loop for that Session (and the bits of the one-Session call)."""
    rng = np.random.default_rng(2025)
    vocab, draft_count = 4099, 4
    options = [(1.0, 40, 0.95, 0.0), (0.7, 0, 0.9, 0.02), (0.0, 0, 1.0, 0.0), (1.3, 8, 1.0, 0.0), (1.0, 0, 1.0, 0.0), (0.9, 64, 0.8, 0.0),
               (1.0, 4, 1.0, 0.0)]
    sessions = len(options)
    targets, drafts, proposals = [], [], []
    for b, option in enumerate(options):
        target, draft, proposed = _case(rng, vocab, draft_count, *option, [0.05, 0.4, 1.5][b % 3], parity.port)
        if b == sessions - 1:
            proposed[0] = int(np.argmin(draft[0]))   # outside the draft's kept candidates: this Session fails, the others do not
        targets.append(target), drafts.append(draft), proposals.append(proposed)
    params = np.zeros(sessions, dtype=pkg.ROW_PARAMS_DTYPE)
    for b, option in enumerate(options):
        params[b]["temperature"], params[b]["top_k"], params[b]["top_p"], params[b]["min_p"] = option
        params[b]["seed"], params[b]["row_id"], params[b]["step"] = 31 + b, 100 + b, 7 * b
    sampler = pkg.Sampler(max_rows=sessions * (2 * draft_count + 1), max_vocab=vocab)
    try:
        records, accepted_probability = sampler.speculative_verify_batch(torch_cuda.from_numpy(np.stack(targets)).cuda(),
                                                                         torch_cuda.from_numpy(np.stack(drafts)).cuda(),
                                                                         torch_cuda.from_numpy(np.stack(proposals)).cuda(), params)
        failures = 0
        for b, option in enumerate(options):
            alone = _compare(pkg, sampler, torch_cuda, parity, targets[b], drafts[b], proposals[b], option, seed=31 + b, row_id=100 + b, step=7 * b)
            for name in ("accepted", "next_token", "uniforms_used", "status"):
                assert records[b][name] == alone[name], (b, name, records[b], alone)
            assert records[b]["next_probability"].view(np.uint32) == np.float32(alone["next_probability"]).view(np.uint32)
            kept = int(records[b]["accepted"])
            np.testing.assert_array_equal(accepted_probability[b, :kept].view(np.uint32), alone["accepted_probability"].view(np.uint32))
            failures += int(alone["status"] != 0)
        assert failures == 1
        # no Sessions: nothing to do; too many for the handle: refused
        assert pkg.library().moe_speculative_verify_batch(sampler._handle, None, None, None, pkg.DTYPE_F32, 0, draft_count, vocab, vocab,
                                                          None, None, None, None) == 0
        with pytest.raises(Exception):
            sampler.speculative_verify_batch(torch_cuda.zeros((sessions + 1, draft_count + 1, vocab), device="cuda"),
                                             torch_cuda.zeros((sessions + 1, draft_count, vocab), device="cuda"),
                                             torch_cuda.zeros((sessions + 1, draft_count), dtype=torch_cuda.int32, device="cuda"),
                                             np.zeros(sessions + 1, dtype=pkg.ROW_PARAMS_DTYPE))
    finally:
        sampler.close()
