"""Generates tests/golden/*.npz from the reference's own code.

Run it where the reference checkout exists (it needs oracle/_ref/libref_oracle.so,
built by `make -C oracle ref`):

    python tests/golden/make_golden.py

Every array in the fixtures was produced by executing the unmodified reference:
Session::sample through the public API (with the Session's own mt19937_64),
sampling_distribution with injected uniforms, std::stable_sort with the
reference comparator, and ExpertDispatcher::dispatch / dispatch_into.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import oracle as oracle_module  # noqa: E402

HERE = Path(__file__).resolve().parent


def sampler_cases(ref):
    rng = np.random.default_rng(20260101)
    logits, temperature, top_k, top_p, min_p, uniforms = [], [], [], [], [], []
    vocab = 1536
    for case in range(96):
        row = (3.0 * rng.standard_normal(vocab)).astype(np.float32)
        kind = case % 8
        if kind == 1:
            row[rng.integers(0, vocab, 200)] = row[3]                      # heavy duplication
        elif kind == 2:
            row[rng.integers(0, vocab, 300)] = -np.inf                     # masked entries
        elif kind == 3:
            row = np.round(row * 4) / 4                                     # coarse grid: many ties
        elif kind == 4:
            row[rng.integers(0, vocab, 8)] += rng.uniform(5, 15, 8).astype(np.float32)
        elif kind == 5:
            row = (row.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)  # bf16-representable values
        elif kind == 6:
            row[:] = -np.inf
            row[rng.integers(0, vocab)] = 0.5                               # a single finite logit
        elif kind == 7:
            row[rng.integers(0, vocab)] = np.inf if case % 16 == 7 else row.max()
        logits.append(row)
        temperature.append([0.0, 0.7, 1.0, 1.3, 0.3, 1.0, 1.0, 0.9][kind] if case % 3 else float(rng.uniform(0.3, 1.5)))
        top_k.append(int(rng.choice([0, 1, 5, 20, 50, 100, 2000])))
        top_p.append(float(rng.choice([1.0, 0.95, 0.9, 0.5, rng.uniform(0.5, 1.0)])))
        min_p.append(float(rng.choice([0.0, 0.0, 0.02, 0.05, 0.1])))
        uniforms.append(float(rng.random()))
    logits = np.stack(logits)
    arrays = dict(logits=logits, temperature=np.array(temperature, np.float32), top_k=np.array(top_k, np.uint32),
                  top_p=np.array(top_p, np.float32), min_p=np.array(min_p, np.float32), uniforms=np.array(uniforms, np.float32))
    out = ref.sample_batch(logits, arrays["temperature"], arrays["top_k"], arrays["top_p"], arrays["min_p"], arrays["uniforms"], threads=1)
    arrays.update(token=out["token"], probability=out["probability"], status=out["status"], used_uniform=out["used_uniform"])
    # full candidate lists (ids and renormalised probabilities) for the first rows with temperature > 0
    ids, probabilities, counts = [], [], []
    for r in range(32):
        if arrays["temperature"][r] == 0:
            counts.append(-1)
            continue
        result = ref.distribution(logits[r], float(arrays["temperature"][r]), int(top_k[r]), float(top_p[r]), float(min_p[r]))
        if isinstance(result[0], int):
            counts.append(-2)
            continue
        counts.append(len(result[0]))
        ids.append(result[0])
        probabilities.append(result[1])
    arrays["dist_count"] = np.array(counts, np.int32)
    arrays["dist_ids"] = np.concatenate(ids) if ids else np.zeros(0, np.int32)
    arrays["dist_probability"] = np.concatenate(probabilities) if probabilities else np.zeros(0, np.float32)
    arrays["rank_order_64"] = np.stack([ref.topk_order(logits[r], 64) for r in range(16)])
    return arrays


def session_route_cases(ref):
    """Session::sample through the reference's public API, its own RNG (seed 1234)."""
    rng = np.random.default_rng(7)
    requests, logits_list, options = [], [], []
    for case in range(24):
        vocab = 512
        row = (2.5 * rng.standard_normal(vocab)).astype(np.float32)
        option = dict(temperature=float(rng.choice([0.0, 0.8, 1.0, 1.2])), top_k=int(rng.choice([0, 1, 10, 40])),
                      top_p=float(rng.choice([1.0, 0.9, 0.7])), min_p=float(rng.choice([0.0, 0.05])))
        requests.append((row, option))
        logits_list.append(row)
        options.append([option["temperature"], option["top_k"], option["top_p"], option["min_p"]])
    results = ref.session_samples(1234, requests)
    return dict(logits=np.stack(logits_list), options=np.array(options, np.float64), status=np.array([r[0] for r in results], np.int32),
                token=np.array([r[1] for r in results], np.int32), probability=np.array([r[2] for r in results], np.float32),
                mt19937_uniforms=ref.mt19937_uniforms(1234, 32), seed=np.array([1234], np.uint64))


def router_cases(ref):
    rng = np.random.default_rng(99)
    out = {}
    index = 0
    for score_function in (0, 1, 2):
        for (tokens, experts, top_k) in ((16, 8, 2), (32, 64, 8), (5, 20, 17), (1, 20, 16)):
            logits = rng.standard_normal((tokens, experts)).astype(np.float32)
            if index % 3 == 0:
                logits = np.round(logits * 2) / 2   # ties
            bias = (0.1 * rng.standard_normal(experts)).astype(np.float32) if index % 2 == 0 else None
            normalization = index % 2
            flags = 1 if index % 4 < 2 else 0
            scaling = [1.0, 1.5, 2.0][index % 3]
            for into in (False, True):
                plan = ref.expert_dispatch(logits, tokens, experts, top_k, score_function=score_function, normalization=normalization, scaling=scaling,
                                           selection_bias=bias, flags=flags, use_dispatch_into=into)
                assert plan["status"] == 0
                tag = f"case{index}_{'into' if into else 'dispatch'}"
                out[tag + "_expert"] = plan["batch_expert"]
                out[tag + "_offset"] = plan["batch_offset"]
                out[tag + "_token"] = plan["token"]
                out[tag + "_rank"] = plan["rank"]
                out[tag + "_weight"] = plan["weight"]
            out[f"case{index}_logits"] = logits
            out[f"case{index}_bias"] = bias if bias is not None else np.zeros(0, np.float32)
            out[f"case{index}_meta"] = np.array([tokens, experts, top_k, score_function, normalization, flags], np.int64)
            out[f"case{index}_scaling"] = np.array([scaling], np.float32)
            index += 1
    out["case_count"] = np.array([index], np.int64)
    return out


def speculative_cases(ref):
    """Verification steps of speculative decoding: the reference's sampling_distribution /
    candidate_probability under the accept loop, and its own sample_residual_distribution
    driven by std::mt19937_64 (the residual draws of the injected-uniform loop are checked
    against it by tests/test_oracle_cpu.py)."""
    rng = np.random.default_rng(20260303)
    vocab, draft_count = 768, 4
    out = {}
    index = 0
    for options in ((1.0, 40, 0.95, 0.0), (0.7, 0, 0.9, 0.02), (1.3, 8, 1.0, 0.0), (1.0, 0, 1.0, 0.0), (0.0, 0, 1.0, 0.0)):
        for closeness in (0.05, 0.5, 1.5):
            temperature, top_k, top_p, min_p = options
            target = (2.5 * rng.standard_normal((draft_count + 1, vocab))).astype(np.float32)
            draft = (target[:draft_count] + closeness * rng.standard_normal((draft_count, vocab)).astype(np.float32)).astype(np.float32)
            proposed = []
            for j in range(draft_count):
                if temperature == 0.0:
                    proposed.append(int(np.argmax(draft[j])) if rng.random() < 0.7 else int(rng.integers(vocab)))
                else:
                    proposed.append(ref.sample(draft[j], float(rng.random()), temperature, top_k, top_p, min_p)[1])
            proposed = np.array(proposed, np.int32)
            uniforms = rng.random(draft_count + 2).astype(np.float32)
            got = ref.speculative_verify(target, draft, proposed, uniforms, temperature, top_k, top_p, min_p)
            assert got["status"] == 0
            tag = f"case{index}_"
            out[tag + "target"], out[tag + "draft"], out[tag + "proposed"], out[tag + "uniforms"] = target, draft, proposed, uniforms
            out[tag + "options"] = np.array(options, np.float64)
            out[tag + "accepted"] = np.array([got["accepted"], got["next_token"], got["uniforms_used"]], np.int64)
            out[tag + "accepted_probability"] = got["accepted_probability"]
            out[tag + "next_probability"] = np.array([got["next_probability"]], np.float32)
            # the reference's residual sampler itself on the first position, with its own generator
            seed = int(rng.integers(1 << 40))
            status, token, probability, _ = ref.residual_with_generator(target[0], draft[0], seed, max(temperature, 0.5), top_k, top_p, min_p)
            out[tag + "residual"] = np.array([status, token, seed], np.int64)
            out[tag + "residual_probability"] = np.array([probability], np.float32)
            out[tag + "residual_uniform"] = ref.mt19937_uniforms(seed, 1)
            index += 1
    out["case_count"] = np.array([index], np.int64)
    return out


def main():
    ref = oracle_module.reference()
    if ref is None:
        raise SystemExit("oracle/_ref/libref_oracle.so is missing: run `make -C oracle ref` where the reference checkout exists")
    np.savez_compressed(HERE / "sampler_reference.npz", **sampler_cases(ref))
    np.savez_compressed(HERE / "session_route_reference.npz", **session_route_cases(ref))
    np.savez_compressed(HERE / "router_reference.npz", **router_cases(ref))
    np.savez_compressed(HERE / "speculative_reference.npz", **speculative_cases(ref))
    for name in ("sampler_reference.npz", "session_route_reference.npz", "router_reference.npz", "speculative_reference.npz"):
        print(name, (HERE / name).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
