"""Seeded synthetic inputs with the shapes, sizes and value distributions of the
five benchmark configurations.  No dataset is involved: the reference has no
benchmark suite for its sampler, so these generators stand in for one.

Every generator returns (logits, params) with logits a numpy array [rows, vocab]
(float32, or uint16 holding bf16 bit patterns) and params an array of
moe_row_params.  The same arrays feed the CUDA path and the CPU oracle.
"""
from __future__ import annotations

import numpy as np


def to_bf16_bits(values: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even (NaN kept quiet)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    rounding = ((bits >> 16) & 1) + np.uint32(0x7FFF)
    rounded = ((bits + rounding) >> 16).astype(np.uint16)
    nan = np.isnan(values)
    if nan.any():
        rounded[nan] = 0x7FC0
    return rounded


def bf16_bits_to_float(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def _params(rows, row_params_dtype, temperature, top_k, top_p, min_p, seed, step=0, row_offset=0):
    params = np.zeros(rows, dtype=row_params_dtype)
    params["temperature"] = temperature
    params["top_k"] = top_k
    params["top_p"] = top_p
    params["min_p"] = min_p
    params["seed"] = seed
    params["row_id"] = np.arange(row_offset, row_offset + rows, dtype=np.uint64)
    params["step"] = step
    return params


def config1_row(row_params_dtype, rows=1, vocab=201088, dtype="f32", seed=0, row_offset=0):
    """3*N(0,1) + 32 boosted indices U(5,15) + 64 forced exact duplicates; T=0.7, k=50, p=0.9, min_p=0.05."""
    rng = np.random.default_rng([seed, 101, row_offset])
    logits = (3.0 * rng.standard_normal((rows, vocab))).astype(np.float32)
    for r in range(rows):
        boosted = rng.choice(vocab, size=min(32, vocab), replace=False)
        logits[r, boosted] += rng.uniform(5.0, 15.0, size=boosted.size).astype(np.float32)
        n_dup = min(64, vocab // 2)
        targets = rng.choice(vocab, size=n_dup, replace=False)
        sources = rng.choice(vocab, size=n_dup, replace=False)
        logits[r, targets] = logits[r, sources]
        # make sure some duplicates sit inside the top-50 region: copy a few top values
        order = np.argsort(-logits[r])[:60]
        picks = rng.choice(order[30:], size=min(6, order.size - 30), replace=False) if order.size > 36 else []
        for p in picks:
            logits[r, rng.integers(0, vocab)] = logits[r, p]
    params = _params(rows, row_params_dtype, 0.7, 50, 0.9, 0.05, seed, row_offset=row_offset)
    if dtype == "bf16":
        return to_bf16_bits(logits), params
    return logits, params


def config2_greedy_temperature(row_params_dtype, rows=256, vocab=129280, seed=1):
    """bf16 2*N(0,1); 10 % of rows get a 4-way tie at the max; rows alternate greedy / T=1 untruncated."""
    rng = np.random.default_rng([seed, 102])
    logits = to_bf16_bits((2.0 * rng.standard_normal((rows, vocab))).astype(np.float32))
    tied = rng.random(rows) < 0.10
    values = bf16_bits_to_float(logits)
    for r in np.nonzero(tied)[0]:
        top = logits[r, np.argmax(values[r])]
        where = rng.choice(vocab, size=min(4, vocab), replace=False)
        logits[r, where] = top
    temperature = np.where(np.arange(rows) % 2 == 0, 0.0, 1.0).astype(np.float32)
    params = _params(rows, row_params_dtype, temperature, 0, 1.0, 0.0, seed)
    return logits, params


def config3_mixed(row_params_dtype, rows=1024, vocab=151936, seed=2):
    """fp32 3*N(0,1) + 16 spikes U(4,12) per row; per-row k, p, min_p, T."""
    rng = np.random.default_rng([seed, 103])
    logits = (3.0 * rng.standard_normal((rows, vocab))).astype(np.float32)
    for r in range(rows):
        spikes = rng.choice(vocab, size=min(16, vocab), replace=False)
        logits[r, spikes] += rng.uniform(4.0, 12.0, size=spikes.size).astype(np.float32)
    top_k = rng.choice(np.array([1, 20, 40, 100, 0], dtype=np.uint32), size=rows)
    top_p = rng.uniform(0.5, 1.0, size=rows).astype(np.float32)
    min_p = rng.choice(np.array([0.0, 0.02, 0.1], dtype=np.float32), size=rows)
    temperature = rng.uniform(0.3, 1.5, size=rows).astype(np.float32)
    params = _params(rows, row_params_dtype, temperature, top_k, top_p, min_p, seed)
    return logits, params


def config4_heavy_tail(row_params_dtype, rows=8192, vocab=201088, seed=3, row_offset=0):
    """bf16 2*Student-t(3); Top-P 0.95 only."""
    rng = np.random.default_rng([seed, 104, row_offset])
    logits = to_bf16_bits((2.0 * rng.standard_t(3.0, size=(rows, vocab))).astype(np.float32))
    params = _params(rows, row_params_dtype, 1.0, 0, 0.95, 0.0, seed, row_offset=row_offset)
    return logits, params


def config5a_large_vocab(row_params_dtype, rows=64, vocab=1048576, seed=4):
    """fp32 3*N(0,1); top_k 64, top_p 0.9."""
    rng = np.random.default_rng([seed, 105])
    logits = (3.0 * rng.standard_normal((rows, vocab))).astype(np.float32)
    params = _params(rows, row_params_dtype, 1.0, 64, 0.9, 0.0, seed)
    return logits, params


def config5b_router(tokens=4096, experts=256, seed=4):
    """router logits N(0,1), per-expert bias N(0,0.1); sigmoid Top-8."""
    rng = np.random.default_rng([seed, 106])
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(experts)).astype(np.float32)
    return logits, bias
