"""GPU parity of the router (scoring, stable Top-K, weights, grouping) and of the
regroup gather against the CPU oracle, through the C ABI.

Bar: expert ids, route order (expert ascending, token ascending, rank
ascending) and ranks bit-exact; weights within 1e-5 relative of the reference
arithmetic and bit-exact against the oracle port run with the device's exp
rounding."""
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def as_plan(plan, experts):
    offsets = plan.expert_offsets.astype(np.int64)
    counts = np.diff(offsets[:experts + 1])
    total = int(offsets[experts])
    return np.nonzero(counts)[0], offsets, total


def compare(plan, want, experts, exact_weights=None):
    assert plan.status == 0 and want["status"] == 0
    batch_expert, offsets, total = as_plan(plan, experts)
    np.testing.assert_array_equal(batch_expert, want["batch_expert"])
    np.testing.assert_array_equal(offsets[batch_expert], want["batch_offset"][:-1])
    assert total == want["batch_offset"][-1]
    np.testing.assert_array_equal(plan.route_token[:total], want["token"])
    np.testing.assert_array_equal(plan.route_rank[:total], want["rank"])
    np.testing.assert_allclose(plan.route_weight[:total], want["weight"], rtol=1e-5, atol=0)
    if exact_weights is not None:
        np.testing.assert_array_equal(plan.route_weight[:total].view(np.uint32), exact_weights.view(np.uint32))


def both_oracles(checker, port, *args, **kwargs):
    want = checker.expert_dispatch(*args, **kwargs)
    port.set_exp_mode(1)
    try:
        exact = port.expert_dispatch(*args, **kwargs)
    finally:
        port.set_exp_mode(0)
    return want, exact


def test_reference_unit_vectors(sampler, checker, port, pkg):
    # tests/test_runtime.cpp:3366-3412,3446-3492,3495-3539 of the reference
    logits = np.array([0, 5, 0, 0, 0, 1, 0, 1, 0, 0, 0, 5, 0, 4, 0, 0, 0, 1, 0, 1, 0, 0, 0, 4], dtype=np.float32)
    plan = sampler.router_dispatch_host(logits, 4, 6, 1)
    batch_expert, offsets, total = as_plan(plan, 6)
    assert batch_expert.tolist() == [1, 5] and plan.route_token[:total].tolist() == [0, 2, 1, 3]
    assert abs(plan.route_weight[0] - 1.0) < 1e-6
    tied = np.array([0, 0, -1, -1], dtype=np.float32)
    want, exact = both_oracles(checker, port, tied, 1, 4, 2, score_function=1, normalization=0, scaling=2.0, flags=0)
    compare(sampler.router_dispatch_host(tied, 1, 4, 2, score_function=pkg.ROUTER_SIGMOID, normalization=0, scaling=2.0, flags=0), want, 4, exact["weight"])
    wide = np.array([(i % 7) - 3 for i in range(20)], dtype=np.float32)
    for top_k in (16, 17):
        want, exact = both_oracles(checker, port, wide, 1, 20, top_k)
        compare(sampler.router_dispatch_host(wide, 1, 20, top_k), want, 20, exact["weight"])
    duplicate = np.array([0, 1, 2, 3], dtype=np.float32)
    want, exact = both_oracles(checker, port, duplicate, 1, 4, 2, explicit_ids=np.array([1, 1], dtype=np.uint32))
    compare(sampler.router_dispatch_host(duplicate, 1, 4, 2, explicit_ids=np.array([1, 1], dtype=np.uint32)), want, 4, exact["weight"])
    deepseek = np.array([4, -4, 3, 2], dtype=np.float32)
    bias = np.array([0, 100, 0, 0], dtype=np.float32)
    want, exact = both_oracles(checker, port, deepseek, 1, 4, 2, score_function=2, scaling=1.5, selection_bias=bias)
    plan = sampler.router_dispatch_host(deepseek, 1, 4, 2, score_function=pkg.ROUTER_SQRT_SOFTPLUS, scaling=1.5, selection_bias=bias)
    compare(plan, want, 4, exact["weight"])
    assert abs(plan.route_weight[:2].sum() - 1.5) < 1e-5


def test_golden_router_fixture(sampler):
    g = np.load(GOLDEN / "router_reference.npz")
    for index in range(int(g["case_count"][0])):
        tokens, experts, top_k, score_function, normalization, flags = (int(v) for v in g[f"case{index}_meta"])
        bias = g[f"case{index}_bias"]
        plan = sampler.router_dispatch_host(g[f"case{index}_logits"], tokens, experts, top_k, score_function=score_function, normalization=normalization,
                                            scaling=float(g[f"case{index}_scaling"][0]), selection_bias=bias if bias.size else None, flags=flags)
        want = dict(status=0, batch_expert=g[f"case{index}_dispatch_expert"], batch_offset=g[f"case{index}_dispatch_offset"],
                    token=g[f"case{index}_dispatch_token"], rank=g[f"case{index}_dispatch_rank"], weight=g[f"case{index}_dispatch_weight"])
        compare(plan, want, experts)


@pytest.mark.parametrize("score_function", [0, 1, 2])
def test_config5b_router(sampler, workloads, checker, port, score_function, torch_cuda):
    torch = torch_cuda
    tokens, experts, top_k = 4096, 256, 8
    logits, bias = workloads.config5b_router(tokens, experts)
    want, exact = both_oracles(checker, port, logits, tokens, experts, top_k, score_function=score_function, selection_bias=bias)
    compare(sampler.router_dispatch_host(logits, tokens, experts, top_k, score_function=score_function, selection_bias=bias), want, experts, exact["weight"])
    # the device-buffer entry point and the regroup gather
    device_plan = sampler.router_dispatch(torch.from_numpy(logits).cuda(), top_k, score_function=score_function, selection_bias=torch.from_numpy(bias).cuda())
    torch.cuda.synchronize()
    assert int(device_plan.status.item()) == 0
    np.testing.assert_array_equal(device_plan.route_token.cpu().numpy().view(np.uint32), want["token"])
    hidden = torch.randn(tokens, 96, device="cuda")
    gathered = sampler.regroup_gather(hidden, device_plan.route_token)
    torch.cuda.synchronize()
    assert torch.equal(gathered, hidden[device_plan.route_token.long()])
    odd = torch.randn(tokens, 37, device="cuda")
    assert torch.equal(sampler.regroup_gather(odd, device_plan.route_token), odd[device_plan.route_token.long()])


def test_router_shapes_and_ties(sampler, checker, port):
    rng = np.random.default_rng(12)
    for tokens, experts, top_k in ((1, 1, 1), (3, 2, 2), (257, 33, 5), (64, 512, 32), (9, 1000, 64), (5, 20, 20)):
        logits = np.round(rng.standard_normal((tokens, experts)).astype(np.float32) * 2) / 2   # coarse grid: many ties
        bias = np.round(rng.standard_normal(experts).astype(np.float32)) / 4
        for score_function in (0, 1, 2):
            for normalization, flags, scaling in ((1, 1, 1.0), (0, 0, 2.5), (0, 1, 0.5)):
                kwargs = dict(score_function=score_function, normalization=normalization, flags=flags, scaling=scaling, selection_bias=bias)
                want, exact = both_oracles(checker, port, logits, tokens, experts, top_k, **kwargs)
                compare(sampler.router_dispatch_host(logits, tokens, experts, top_k, **kwargs), want, experts, exact["weight"])
    explicit = rng.integers(0, 16, size=(40, 4)).astype(np.uint32)   # hash routes, duplicates allowed
    logits = rng.standard_normal((40, 16)).astype(np.float32)
    want, exact = both_oracles(checker, port, logits, 40, 16, 4, score_function=2, explicit_ids=explicit)
    compare(sampler.router_dispatch_host(logits, 40, 16, 4, score_function=2, explicit_ids=explicit), want, 16, exact["weight"])


def test_wide_routers(sampler, checker, port, pkg):
    """More than 1024 experts or top_k above 16: the k survivors are radix-selected before the rank order is
    established, the select kernel needs more than 48 KiB of shared memory, and the offsets scan walks several chunks."""
    rng = np.random.default_rng(21)
    for tokens, experts, top_k in ((3, 1025, 8), (8, 4096, 8), (5, 2048, 64), (4, 600, 40), (2, 4096, 300)):
        logits = (rng.standard_normal((tokens, experts)) * 2).astype(np.float32)
        logits[:, ::7] = logits[:, 3:4]                      # exact ties across experts
        bias = (0.1 * rng.standard_normal(experts)).astype(np.float32)
        for score_function in (0, 1, 2):
            kwargs = dict(score_function=score_function, selection_bias=bias)
            want, exact = both_oracles(checker, port, logits, tokens, experts, top_k, **kwargs)
            compare(sampler.router_dispatch_host(logits, tokens, experts, top_k, **kwargs), want, experts, exact["weight"])
    assert sampler.router_dispatch_host(np.zeros((1, 4097), dtype=np.float32), 1, 4097, 2).status == 110


def test_cross_session_coalescing(sampler, checker, torch_cuda):
    """src/engine/cpu_executor.cpp:3217-3264 of the reference: every Session of a decode step is dispatched on its
    own (one token each), then the routes that name the same expert are merged into one batch with token_index
    rewritten to the Session's position in the step.  One dispatch of the stacked [sessions x experts] router
    logits yields exactly those batches: same expert sets, and inside an expert the Sessions in ascending order
    with the ranks and weights of their own plans."""
    rng = np.random.default_rng(33)
    sessions, experts, top_k = 48, 64, 6
    logits = rng.standard_normal((sessions, experts)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(experts)).astype(np.float32)
    merged = {}
    for session in range(sessions):
        plan = checker.expert_dispatch(logits[session], 1, experts, top_k, score_function=1, selection_bias=bias)
        for b, expert in enumerate(plan["batch_expert"]):
            for i in range(plan["batch_offset"][b], plan["batch_offset"][b + 1]):
                assert plan["token"][i] == 0
                merged.setdefault(int(expert), []).append((session, int(plan["rank"][i]), np.float32(plan["weight"][i])))
    stacked = sampler.router_dispatch_host(logits, sessions, experts, top_k, score_function=1, selection_bias=bias)
    assert stacked.status == 0
    offsets = stacked.expert_offsets.astype(np.int64)
    assert sorted(merged) == [e for e in range(experts) if offsets[e + 1] > offsets[e]]
    for expert, routes in merged.items():
        rows = slice(offsets[expert], offsets[expert + 1])
        assert stacked.route_token[rows].tolist() == [r[0] for r in routes]      # Session order = the order the executor appends in
        assert stacked.route_rank[rows].tolist() == [r[1] for r in routes]
        np.testing.assert_allclose(stacked.route_weight[rows], np.array([r[2] for r in routes]), rtol=1e-5, atol=0)


def test_regroup_gather_refuses_tokens_outside_the_matrix(sampler, torch_cuda):
    torch = torch_cuda
    hidden = torch.randn(10, 64, device="cuda")
    route_token = torch.tensor([3, 9, 10, 0, 4000000000 - 2**32, 7], dtype=torch.int32, device="cuda")   # 10 and 4e9 are out of range
    assert sampler.regroup_gather_check() is False
    gathered = sampler.regroup_gather(hidden, route_token)
    assert sampler.regroup_gather_check() is True
    assert sampler.regroup_gather_check() is False                      # the mark is cleared by the check
    assert torch.equal(gathered[[0, 1, 3, 5]], hidden[[3, 9, 0, 7]])
    assert torch.count_nonzero(gathered[[2, 4]]).item() == 0            # zero-filled, nothing dereferenced


def test_router_errors(sampler, pkg):
    logits = np.zeros((4, 8), dtype=np.float32)
    assert sampler.router_dispatch_host(logits, 0, 8, 2).status == 104
    assert sampler.router_dispatch_host(logits, 4, 8, 0).status == 105
    assert sampler.router_dispatch_host(logits, 4, 8, 9).status == 105
    assert sampler.router_dispatch_host(logits, 4, 8, 2, scaling=0.0).status == 109
    bad = logits.copy(); bad[2, 3] = np.inf
    plan = sampler.router_dispatch_host(bad, 4, 8, 2)
    assert plan.status == 101 and pkg.router_status_message(plan.status) == "router logits must be finite"
    plan = sampler.router_dispatch_host(logits, 4, 8, 2, explicit_ids=np.array([[0, 1], [2, 9], [1, 1], [0, 0]], dtype=np.uint32))
    assert plan.status == 102
    # sigmoid of a very negative logit underflows to 0: renormalising a zero sum is an InvalidModel error in the reference
    tiny = np.full((2, 4), -200.0, dtype=np.float32)
    plan = sampler.router_dispatch_host(tiny, 2, 4, 2, score_function=pkg.ROUTER_SIGMOID)
    assert plan.status == 103 and pkg.library().moe_router_status_error_code(103) == 3
    # after a failed call the handle still works
    assert sampler.router_dispatch_host(logits, 4, 8, 2).status == 0
