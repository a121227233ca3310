"""moe_router_dispatch_static: the router entry point for hosts that may not
allocate device memory while routing (a memory planner owns the whole GPU, or
the decode loop cannot take an allocation's device-wide synchronisation).

Its scratch is a fixed array inside the library, so the test checks three
things through the C ABI: it returns what moe_router_dispatch returns, twice in
a row with different shapes (the array keeps the previous call's contents, so
stale counters would show up on the second call), it takes no device memory,
and it refuses work that does not fit the fixed array with a readable message.

Collected last on purpose: a failure here must not hide any other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

MAX_ROUTES = 65536
MAX_EXPERTS = 4096


def plan_buffers(pkg, torch, logits, top_k):
    tokens, experts = logits.shape
    routes = tokens * top_k
    device = logits.device
    return pkg.DispatchPlan(torch.empty(experts + 1, dtype=torch.int32, device=device), torch.empty(routes, dtype=torch.int32, device=device),
                            torch.empty(routes, dtype=torch.int32, device=device), torch.empty(routes, dtype=torch.float32, device=device),
                            torch.full((1,), -1, dtype=torch.int32, device=device))


def call_static(pkg, torch, logits, top_k, score_function, bias, normalization=1, scaling=1.0, flags=1, out=None):
    tokens, experts = logits.shape
    device = logits.device
    if out is None:
        out = plan_buffers(pkg, torch, logits, top_k)
    options = pkg.RouterOptions(experts, top_k, score_function, normalization, scaling, flags, bias.data_ptr() if bias is not None else None, None)
    message = C.create_string_buffer(256)
    stream = torch.cuda.current_stream(device).cuda_stream
    code = pkg.library().moe_router_dispatch_static(C.c_void_p(stream), C.c_void_p(logits.data_ptr()), tokens, C.byref(options),
                                                    C.c_void_p(out.expert_offsets.data_ptr()), C.c_void_p(out.route_token.data_ptr()),
                                                    C.c_void_p(out.route_rank.data_ptr()), C.c_void_p(out.route_weight.data_ptr()),
                                                    C.c_void_p(out.status.data_ptr()), message, 256)
    return code, message.value.decode(), out


def test_static_router_matches_the_allocating_entry_point(pkg, workloads, sampler, checker, torch_cuda):
    torch = torch_cuda
    # calls in a row: a large sigmoid case, a smaller softmax case with fewer experts, the widest router the
    # fixed array serves, and a call that fills it to the last route
    cases = [(4096, 256, 8, pkg.ROUTER_SIGMOID, 11), (300, 40, 6, pkg.ROUTER_SOFTMAX, 12), (8, MAX_EXPERTS, 8, pkg.ROUTER_SIGMOID, 13),
             (MAX_ROUTES // 16, 64, 16, pkg.ROUTER_SQRT_SOFTPLUS, 14)]
    for tokens, experts, top_k, score_function, seed in cases:
        logits_host, bias_host = workloads.config5b_router(tokens, experts, seed=seed)
        logits = torch.from_numpy(logits_host).cuda()
        bias = torch.from_numpy(bias_host).cuda()
        want = sampler.router_dispatch(logits, top_k, score_function=score_function, selection_bias=bias)
        torch.cuda.synchronize()
        buffers = plan_buffers(pkg, torch, logits, top_k)   # the caller's outputs exist before the measured call
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        code, message, got = call_static(pkg, torch, logits, top_k, score_function, bias, out=buffers)
        torch.cuda.synchronize()
        assert code == 0, message
        assert torch.cuda.mem_get_info()[0] == free_before      # the call took no device memory
        assert int(got.status.item()) == 0 and int(want.status.item()) == 0
        assert torch.equal(got.expert_offsets, want.expert_offsets)
        assert torch.equal(got.route_token, want.route_token)
        assert torch.equal(got.route_rank, want.route_rank)
        # the same kernels ran on both paths: the weights agree to the bit
        assert torch.equal(got.route_weight.view(torch.int32), want.route_weight.view(torch.int32))
        # ... and with the CPU oracle directly
        oracle = checker.expert_dispatch(logits_host, tokens, experts, top_k, score_function=score_function, selection_bias=bias_host)
        total = int(oracle["batch_offset"][-1])
        assert total == tokens * top_k == int(got.expert_offsets[experts].item())
        np.testing.assert_array_equal(got.route_token.cpu().numpy().view(np.uint32)[:total], oracle["token"])
        np.testing.assert_array_equal(got.route_rank.cpu().numpy().view(np.uint32)[:total], oracle["rank"])
        np.testing.assert_allclose(got.route_weight.cpu().numpy()[:total], oracle["weight"], rtol=1e-5, atol=0)


def test_static_router_reports_data_errors_and_recovers(pkg, torch_cuda):
    torch = torch_cuda
    logits = torch.zeros((4, 8), device="cuda")
    logits[2, 3] = float("inf")
    code, _, out = call_static(pkg, torch, logits, 2, pkg.ROUTER_SOFTMAX, None)
    torch.cuda.synchronize()
    assert code == 0 and int(out.status.item()) == 101            # "router logits must be finite"
    code, _, out = call_static(pkg, torch, torch.zeros((4, 8), device="cuda"), 2, pkg.ROUTER_SOFTMAX, None)
    torch.cuda.synchronize()
    assert code == 0 and int(out.status.item()) == 0              # the error word was reset
    assert out.expert_offsets.cpu().tolist() == [0, 4, 8, 8, 8, 8, 8, 8, 8]


def test_static_router_refuses_what_does_not_fit(pkg, torch_cuda):
    torch = torch_cuda
    tokens = MAX_ROUTES // 8 + 1
    code, message, _ = call_static(pkg, torch, torch.zeros((tokens, 16), device="cuda"), 8, pkg.ROUTER_SOFTMAX, None)
    assert code == 1 and "MOE_ROUTER_STATIC_MAX_ROUTES" in message
    code, message, _ = call_static(pkg, torch, torch.zeros((2, 16), device="cuda"), 17, pkg.ROUTER_SOFTMAX, None)
    assert code == 1 and message == "expert dispatch requires 0 < top_k <= expert_count"
