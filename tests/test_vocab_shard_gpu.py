"""Vocabulary-sharded sampling on ONE GPU: the slices a multi-GPU run would own
are processed one after another by moe_sample_local_candidates, stacked the way
an all-gather would stack them, and finished by moe_sample_merge_candidates.
The result must equal both the unsharded GPU call and the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shards", [2, 4, 8])
def test_config5a_vocab_sharded(pkg, workloads, parity, torch_cuda, shards):
    torch = torch_cuda
    parallel = __import__("ncnn_moe_runtime_b200.parallel", fromlist=["x"])
    logits, params = workloads.config5a_large_vocab(pkg.ROW_PARAMS_DTYPE, rows=6, vocab=1 << 20)
    device = torch.from_numpy(logits).cuda()
    rows, vocab = logits.shape
    top_k = 64
    lists = []
    for rank in range(shards):
        begin, end = parallel.vocab_shard_range(vocab, shards, rank)
        lists.append(parity.sampler.local_candidates(device[:, begin:end], begin, top_k))
    gathered = torch.stack(lists)   # [shards, rows, k], the layout of all_gather_into_tensor
    out = parity.sampler.merge_candidates(gathered, params, top_k, topk_stride=top_k)
    torch.cuda.synchronize()
    whole = parity.sampler.sample_batch(device, params, topk_stride=top_k)
    torch.cuda.synchronize()
    for key in ("token", "probability", "flags", "status", "topk"):
        assert torch.equal(out[key], whole[key]), key
    uniforms = parity.uniforms(params)
    want = parity.checker.sample_batch(logits, params["temperature"], params["top_k"], params["top_p"], params["min_p"], uniforms)
    np.testing.assert_array_equal(out["token"].cpu().numpy(), want["token"])
    np.testing.assert_allclose(out["probability"].cpu().numpy(), want["probability"], rtol=1e-5)
    for r in range(rows):
        np.testing.assert_array_equal(out["topk"][r].cpu().numpy(), parity.checker.topk_order(logits[r], top_k))


def test_ragged_shards_ties_and_short_slices(pkg, parity, torch_cuda):
    torch = torch_cuda
    rng = np.random.default_rng(17)
    rows, vocab, top_k = 5, 1000, 48
    logits = np.round(rng.standard_normal((rows, vocab)).astype(np.float32) * 3) / 3   # ties across shard boundaries
    logits[0, :] = 1.0                                                                     # one constant row
    logits[1, 500:] = -np.inf
    params = pkg.make_row_params(rows, temperature=[1.0, 0.7, 1.2, 0.0, 1.0], top_k=top_k, top_p=[0.9, 1.0, 0.8, 1.0, 0.95], seed=5)
    device = torch.from_numpy(logits).cuda()
    bounds = [0, 13, 14, 400, 970, 1000]   # includes slices shorter than top_k
    lists = [parity.sampler.local_candidates(device[:, b:e].contiguous(), b, top_k) for b, e in zip(bounds[:-1], bounds[1:])]
    out = parity.sampler.merge_candidates(torch.stack(lists), params, top_k, topk_stride=top_k)
    torch.cuda.synchronize()
    uniforms = parity.uniforms(params)
    want = parity.checker.sample_batch(logits, params["temperature"], params["top_k"], params["top_p"], params["min_p"], uniforms)
    np.testing.assert_array_equal(out["token"].cpu().numpy(), want["token"])
    np.testing.assert_array_equal(out["status"].cpu().numpy() != 0, want["status"] != 0)
