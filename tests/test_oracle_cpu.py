"""CPU tests: the oracle port against the reference's golden vectors, its unit
assertions and (where it was built) the compiled reference itself."""
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden"


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_philox_known_answers(port):
    # Random123 known-answer vectors for philox4x32-10
    assert port.philox4x32_10([0, 0, 0, 0], [0, 0]).tolist() == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert port.philox4x32_10([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2).tolist() == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert port.philox4x32_10([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0]).tolist() == \
        [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]
    u = port.philox_uniform(0, 0, 0)
    assert u == (0x6627E8D5 >> 8) * 2.0 ** -24 and 0.0 <= u < 1.0


def test_reference_unit_assertions(port):
    # tests/test_runtime.cpp:4333-4362 of the reference
    assert port.sample(np.array([1, 2, 3.0]), 0.5, temperature=0.0)[:3] == (0, 2, 1.0)
    assert port.sample(np.array([3, np.nan, 3.0]), 0.5, temperature=0.0)[:2] == (0, 0)
    status, _, _, _, message = port.sample(np.array([np.nan, np.inf]), 0.5, temperature=0.0)
    assert status == 1 and message == "sampling requires at least one finite logit"
    assert port.sample(np.array([1, 2, 3.0]), 0.5, top_k=1)[:2] == (0, 2)
    status, _, _, _, message = port.sample(np.array([1, 2, 3.0]), 0.5, top_p=0.0)
    assert status == 1 and message == "top_p must be in the range (0, 1]"
    assert port.sample(np.zeros(0), 0.5)[4] == "cannot sample empty logits"
    assert port.sample(np.ones(3), 0.5, temperature=-1.0)[4] == "temperature must be finite and non-negative"
    assert port.sample(np.ones(3), 0.5, min_p=1.5)[4] == "min_p must be in the range [0, 1]"


def test_reference_dispatcher_assertions(port):
    # tests/test_runtime.cpp:3366-3412: grouping order, ranks, weight renormalisation
    logits = np.array([0, 5, 0, 0, 0, 1, 0, 1, 0, 0, 0, 5, 0, 4, 0, 0, 0, 1, 0, 1, 0, 0, 0, 4], dtype=np.float32)
    plan = port.expert_dispatch(logits, 4, 6, 1)
    assert plan["status"] == 0 and plan["assignment_count"] == 4
    assert plan["batch_expert"].tolist() == [1, 5]
    assert plan["token"].tolist() == [0, 2, 1, 3]
    assert abs(plan["weight"][0] - 1.0) < 1e-6
    weighted = port.expert_dispatch(np.array([2.0, 1.0, 0.0], dtype=np.float32), 1, 3, 2)
    assert weighted["rank"].tolist() == [0, 1] and abs(weighted["weight"].sum() - 1.0) < 1e-6
    bad = port.expert_dispatch(np.array([1.0, 2.0], dtype=np.float32), 1, 3, 2)
    assert bad["status"] == 1
    # :3495-3511 sqrt-softplus with a selection bias that picks the expert but is excluded from the weight
    routed = port.expert_dispatch(np.array([4.0, -4.0, 3.0, 2.0], dtype=np.float32), 1, 4, 2, score_function=2, scaling=1.5,
                                  selection_bias=np.array([0, 100.0, 0, 0], dtype=np.float32))
    assert routed["batch_expert"].tolist() == [0, 1] and abs(routed["weight"].sum() - 1.5) < 1e-5
    explicit = port.expert_dispatch(np.array([4.0, -4.0, 3.0, 2.0], dtype=np.float32), 1, 4, 2, score_function=2, scaling=1.5,
                                    explicit_ids=np.array([3, 2], dtype=np.uint32))
    assert explicit["batch_expert"].tolist() == [2, 3]


def test_port_matches_golden_sampler(port):
    g = np.load(GOLDEN / "sampler_reference.npz")
    out = port.sample_batch(g["logits"], g["temperature"], g["top_k"], g["top_p"], g["min_p"], g["uniforms"], threads=4)
    np.testing.assert_array_equal(out["status"], g["status"])
    np.testing.assert_array_equal(out["token"], g["token"])
    np.testing.assert_array_equal(bits(out["probability"]), bits(g["probability"]))
    np.testing.assert_array_equal(out["used_uniform"], g["used_uniform"])
    cursor = 0
    for r, count in enumerate(g["dist_count"]):
        if count < 0:
            continue
        ids, probabilities = port.distribution(g["logits"][r], float(g["temperature"][r]), int(g["top_k"][r]), float(g["top_p"][r]), float(g["min_p"][r]))
        np.testing.assert_array_equal(ids, g["dist_ids"][cursor:cursor + count])
        np.testing.assert_array_equal(bits(probabilities), bits(g["dist_probability"][cursor:cursor + count]))
        cursor += count
    for r in range(g["rank_order_64"].shape[0]):
        np.testing.assert_array_equal(port.topk_order(g["logits"][r], 64), g["rank_order_64"][r])


def test_port_replays_the_public_session_route(port):
    """Session::sample with its own mt19937_64 == the port fed the same uniforms in order."""
    g = np.load(GOLDEN / "session_route_reference.npz")
    uniforms = g["mt19937_uniforms"]
    cursor = 0
    for r in range(g["logits"].shape[0]):
        temperature, top_k, top_p, min_p = g["options"][r]
        status, token, probability, used, _ = port.sample(g["logits"][r], float(uniforms[cursor]), float(temperature), int(top_k), float(top_p), float(min_p))
        cursor += used
        assert status == g["status"][r] and token == g["token"][r]
        assert np.float32(probability).view(np.uint32) == g["probability"][r].view(np.uint32)
    assert cursor > 4  # the fixture really consumed uniforms


def test_port_matches_golden_router(port):
    g = np.load(GOLDEN / "router_reference.npz")
    for index in range(int(g["case_count"][0])):
        tokens, experts, top_k, score_function, normalization, flags = (int(v) for v in g[f"case{index}_meta"])
        bias = g[f"case{index}_bias"]
        plan = port.expert_dispatch(g[f"case{index}_logits"], tokens, experts, top_k, score_function=score_function, normalization=normalization,
                                    scaling=float(g[f"case{index}_scaling"][0]), selection_bias=bias if bias.size else None, flags=flags)
        for tag in ("dispatch", "into"):   # dispatch_into must equal dispatch (tests/test_runtime.cpp:3446-3492)
            np.testing.assert_array_equal(plan["batch_expert"], g[f"case{index}_{tag}_expert"])
            np.testing.assert_array_equal(plan["batch_offset"], g[f"case{index}_{tag}_offset"])
            np.testing.assert_array_equal(plan["token"], g[f"case{index}_{tag}_token"])
            np.testing.assert_array_equal(plan["rank"], g[f"case{index}_{tag}_rank"])
            np.testing.assert_allclose(plan["weight"], g[f"case{index}_{tag}_weight"], rtol=1e-6, atol=0)
        np.testing.assert_array_equal(bits(plan["weight"]), bits(g[f"case{index}_dispatch_weight"]))


def test_port_against_the_compiled_reference(port, reference):
    if reference is None:
        pytest.skip("oracle/_ref was not built on this machine")
    rng = np.random.default_rng(5)
    for trial in range(30):
        vocab = int(rng.integers(1, 6000))
        logits = (3 * rng.standard_normal(vocab)).astype(np.float32)
        if trial % 3 == 0:
            logits[rng.integers(0, vocab, vocab // 4 + 1)] = logits[0]
        if trial % 5 == 0:
            logits[rng.integers(0, vocab, 3)] = -np.inf
        options = (float(rng.uniform(0.3, 1.5)), int(rng.choice([0, 1, 20, 40, 100])), float(rng.uniform(0.5, 1.0)), float(rng.choice([0, 0.02, 0.1])))
        a, b = reference.distribution(logits, *options), port.distribution(logits, *options)
        np.testing.assert_array_equal(a[0], b[0])
        np.testing.assert_array_equal(bits(a[1]), bits(b[1]))
        u = float(rng.random())
        assert reference.sample(logits, u, *options) == port.sample(logits, u, *options)
    # Session::sample (public API, own RNG) == injected-uniform route of the shim
    uniforms = reference.mt19937_uniforms(4321, 16)
    requests = [((3 * rng.standard_normal(700)).astype(np.float32), dict(temperature=1.0, top_k=int(k), top_p=0.9, min_p=0.0)) for k in (0, 5, 50, 0, 1, 7)]
    results = reference.session_samples(4321, requests)
    cursor = 0
    for (logits, option), result in zip(requests, results):
        status, token, probability, used, _ = port.sample(logits, float(uniforms[cursor]), **option)
        cursor += used
        assert (status, token) == result[:2] and np.float32(probability) == np.float32(result[2])


def test_exp_mode_switch_changes_only_ulps(port):
    rng = np.random.default_rng(8)
    logits = (3 * rng.standard_normal((8, 4000))).astype(np.float32)
    args = (logits, np.full(8, 0.9, np.float32), np.full(8, 40, np.uint32), np.full(8, 0.95, np.float32), np.zeros(8, np.float32), rng.random(8).astype(np.float32))
    a = port.sample_batch(*args)
    port.set_exp_mode(1)
    try:
        b = port.sample_batch(*args)
    finally:
        port.set_exp_mode(0)
    np.testing.assert_array_equal(a["token"], b["token"])
    np.testing.assert_allclose(a["probability"], b["probability"], rtol=1e-6)


def test_bf16_rounding_helper(workloads):
    import torch
    rng = np.random.default_rng(3)
    values = np.concatenate([(4 * rng.standard_normal(5000)).astype(np.float32), np.array([0.0, -0.0, 1.0, np.inf, -np.inf, 3.0e38, 1e-40], np.float32)])
    ours = workloads.to_bf16_bits(values)
    theirs = torch.from_numpy(values).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    np.testing.assert_array_equal(ours, theirs)
    np.testing.assert_array_equal(workloads.bf16_bits_to_float(ours), torch.from_numpy(values).to(torch.bfloat16).to(torch.float32).numpy())


def test_port_matches_golden_speculative_verification(port):
    """The accept loop of speculative decoding (session.cpp:776-880) as executed by the reference,
    and the reference's own sample_residual_distribution (:150-202) driven by std::mt19937_64."""
    g = np.load(GOLDEN / "speculative_reference.npz")
    pinned_residuals = 0
    rejections = 0
    for index in range(int(g["case_count"][0])):
        tag = f"case{index}_"
        temperature, top_k, top_p, min_p = (float(v) for v in g[tag + "options"])
        got = port.speculative_verify(g[tag + "target"], g[tag + "draft"], g[tag + "proposed"], g[tag + "uniforms"], temperature, int(top_k), top_p, min_p)
        accepted, next_token, used = (int(v) for v in g[tag + "accepted"])
        assert got["status"] == 0
        assert (got["accepted"], got["next_token"], got["uniforms_used"]) == (accepted, next_token, used)
        np.testing.assert_array_equal(bits(got["accepted_probability"]), bits(g[tag + "accepted_probability"]))
        assert bits(np.array([got["next_probability"]], np.float32))[0] == bits(g[tag + "next_probability"])[0]
        rejections += accepted < g[tag + "proposed"].size
        # residual: force a rejection of the draft's own best token at position 0, then draw with the
        # uniform the reference's generator produced; equal to the reference function's own result
        status, token, _seed = (int(v) for v in g[tag + "residual"])
        if status != 0:
            continue
        residual_temperature = max(temperature, 0.5)
        target, draft = g[tag + "target"][0], g[tag + "draft"][0]
        proposal = np.array([int(np.argmax(draft))], np.int32)
        uniforms = np.array([np.float32(0.99999994), g[tag + "residual_uniform"][0], 0.5], np.float32)
        forced = port.speculative_verify(np.stack([target, target]), draft[None], proposal, uniforms, residual_temperature, int(top_k), top_p, min_p)
        if forced["status"] == 0 and forced["accepted"] == 0:
            assert forced["next_token"] == token
            assert bits(np.array([forced["next_probability"]], np.float32))[0] == bits(g[tag + "residual_probability"])[0]
            pinned_residuals += 1
    assert rejections >= 4 and pinned_residuals >= 4


def test_port_speculative_matches_compiled_reference(port, oracle_module):
    ref = oracle_module.reference()
    if ref is None:
        pytest.skip("the compiled reference is not present")
    rng = np.random.default_rng(8)
    vocab, count = 900, 3
    for case in range(40):
        temperature = float(rng.choice([0.0, 0.6, 1.0, 1.4]))
        top_k, top_p, min_p = int(rng.choice([0, 6, 60])), float(rng.choice([1.0, 0.9, 0.5])), float(rng.choice([0.0, 0.03]))
        target = (2.5 * rng.standard_normal((count + 1, vocab))).astype(np.float32)
        draft = (target[:count] + rng.choice([0.05, 0.6, 2.0]) * rng.standard_normal((count, vocab))).astype(np.float32)
        proposed = np.array([int(np.argmax(draft[j])) if temperature == 0.0 or rng.random() < 0.3
                             else port.sample(draft[j], float(rng.random()), temperature, top_k, top_p, min_p)[1] for j in range(count)], np.int32)
        uniforms = rng.random(count + 2).astype(np.float32)
        a = port.speculative_verify(target, draft, proposed, uniforms, temperature, top_k, top_p, min_p)
        b = ref.speculative_verify(target, draft, proposed, uniforms, temperature, top_k, top_p, min_p)
        assert (a["status"], a["message"], a["accepted"], a["next_token"], a["uniforms_used"]) == \
               (b["status"], b["message"], b["accepted"], b["next_token"], b["uniforms_used"])
        np.testing.assert_array_equal(bits(a["accepted_probability"]), bits(b["accepted_probability"]))
        assert bits(np.array([a["next_probability"]], np.float32))[0] == bits(np.array([b["next_probability"]], np.float32))[0]


def test_indexer_selection_orders_by_score_then_index(checker):
    # scored_index_precedes (cpu_latent_attention.cpp:257-262): score descending, index ascending on equality
    scores = np.array([1, 3, 3, 2, 5, 3, -0.0, 0.0], dtype=np.float32)
    assert checker.indexer_topk(scores, 4).tolist() == [4, 1, 2, 5]
    assert checker.indexer_topk(scores, 8).tolist() == [4, 1, 2, 5, 3, 0, 6, 7]
    assert checker.indexer_topk(scores, 100).tolist() == [4, 1, 2, 5, 3, 0, 6, 7]
    rng = np.random.default_rng(0)
    values = rng.standard_normal(5000).astype(np.float32)
    want = np.lexsort((np.arange(values.size), -values))[:300]
    np.testing.assert_array_equal(checker.indexer_topk(values, 300), want.astype(np.uint32))
