"""GPU parity of moe_indexer_topk against the CPU oracle's statement of the latent-attention indexer selection
(src/kernels/cpu_latent_attention.cpp:414-423 of the reference: std::partial_sort with scored_index_precedes).

Bar: the selected index lists equal the oracle's, position by position (integer work: bit-exact)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def check(sampler, checker, torch, scores, top_k, count=None):
    rows, stride = scores.shape
    count = stride if count is None else count
    device = torch.from_numpy(scores).cuda()
    indices, values = sampler.indexer_topk(device, top_k, count=count, with_scores=True)
    torch.cuda.synchronize()
    indices = indices.cpu().numpy()
    values = values.cpu().numpy()
    selected = min(top_k, count)
    for r in range(rows):
        want = checker.indexer_topk(scores[r, :count], top_k)
        np.testing.assert_array_equal(indices[r, :selected].view(np.uint32), want, err_msg=f"row {r}")
        np.testing.assert_array_equal(values[r, :selected].view(np.uint32), scores[r, want].view(np.uint32))
        assert np.all(indices[r, selected:] == -1)


def test_reference_shaped_scores(sampler, checker, torch_cuda):
    # the scores of select_compressed_indices are sums of relu(dot) * weight: many exact zeros, a few large values
    rng = np.random.default_rng(41)
    for count, top_k in ((513, 512), (4096, 512), (40000, 2048), (131072, 2048), (9000, 8192)):
        scores = np.maximum(0.0, rng.standard_normal((3, count))).astype(np.float32) * rng.random((3, count)).astype(np.float32)
        check(sampler, checker, torch_cuda, scores, top_k)


def test_ties_small_and_ragged(sampler, checker, torch_cuda):
    rng = np.random.default_rng(42)
    for count, top_k in ((1, 1), (2, 1), (7, 7), (33, 5), (100, 64), (1000, 1), (257, 300), (5000, 4095)):
        scores = (np.round(rng.standard_normal((4, count)) * 2) / 2).astype(np.float32)     # coarse grid: the selection cuts through ties
        scores[0] = 1.0                                                                        # one row all equal: lowest indices win
        scores[1, ::3] = -0.0                                                                  # -0 == +0 in the comparator
        check(sampler, checker, torch_cuda, scores, top_k)
    # a strided view: only the first `count` entries of every row take part
    padded = rng.standard_normal((5, 3000)).astype(np.float32)
    check(sampler, checker, torch_cuda, padded, 128, count=2500)


def test_limits(sampler, pkg, torch_cuda):
    torch = torch_cuda
    scores = torch.zeros((1, 10), device="cuda")
    with pytest.raises(pkg.MoeError):
        sampler.indexer_topk(scores, 0)
    with pytest.raises(pkg.MoeError):
        sampler.indexer_topk(scores, 8193)
    indices = sampler.indexer_topk(scores, 16)          # more than there are entries
    torch.cuda.synchronize()
    assert indices.cpu().numpy()[0].tolist() == list(range(10)) + [-1] * 6
