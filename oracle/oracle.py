"""ctypes access to the CPU oracles.  TEST INFRASTRUCTURE ONLY.

Two shared libraries export the same `oracle_*` C functions:

* ``oracle/_ref/libref_oracle.so`` — the reference's own C++ sources compiled in
  place (``make -C oracle ref``); kind ``"reference"``.
* ``oracle/liboracle_port.so`` — this repository's CPU restatement
  (``make -C oracle port``); kind ``"port"``.

Only tests, the smoke check and the CPU-baseline legs of the benchmark may
import this module.  The shipped library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PORT_PATH = HERE / "liboracle_port.so"
REF_PATH = HERE / "_ref" / "libref_oracle.so"

STATUS_NAMES = {0: "Ok", 1: "InvalidArgument", 2: "IoError", 3: "InvalidModel", 4: "UnsupportedModel", 5: "InternalError"}


def build(port: bool = True, ref: bool = True) -> None:
    """Compile the oracles (the reference one only where its checkout exists)."""
    targets = []
    if port:
        targets.append("port")
    if ref:
        targets.append("ref")
    subprocess.run(["make", "-s", "-j8", "-C", str(HERE), *targets], check=True)


def _ptr(array, ctype):
    return array.ctypes.data_as(C.POINTER(ctype))


class Oracle:
    """One loaded oracle library with numpy-friendly wrappers."""

    def __init__(self, path: Path):
        self.path = Path(path)
        self.lib = C.CDLL(str(self.path))
        lib = self.lib
        lib.oracle_kind.restype = C.c_char_p
        self.kind = lib.oracle_kind().decode()
        f32p, i32p, u32p = C.POINTER(C.c_float), C.POINTER(C.c_int32), C.POINTER(C.c_uint32)
        lib.oracle_sampling_distribution.argtypes = [f32p, C.c_size_t, C.c_float, C.c_uint32, C.c_float, C.c_float,
                                                     i32p, f32p, C.c_size_t, C.POINTER(C.c_size_t), C.c_char_p, C.c_size_t]
        lib.oracle_sampling_distribution.restype = C.c_int
        lib.oracle_sample_with_uniform.argtypes = [f32p, C.c_size_t, C.c_float, C.c_uint32, C.c_float, C.c_float, C.c_float,
                                                   i32p, f32p, C.POINTER(C.c_int), C.c_char_p, C.c_size_t]
        lib.oracle_sample_with_uniform.restype = C.c_int
        lib.oracle_topk_order.argtypes = [f32p, C.c_size_t, C.c_size_t, i32p]
        lib.oracle_topk_order.restype = None
        lib.oracle_sample_batch.argtypes = [C.c_void_p, C.c_int, C.c_size_t, C.c_size_t, C.c_size_t, f32p, u32p, f32p, f32p, f32p,
                                            i32p, f32p, i32p, i32p, C.c_int]
        lib.oracle_sample_batch.restype = C.c_int
        lib.oracle_expert_dispatch.argtypes = [C.c_int, f32p, C.c_size_t, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, C.c_int, C.c_float,
                                               f32p, C.c_size_t, u32p, C.c_size_t, C.c_uint32,
                                               u32p, u32p, u32p, u32p, f32p, C.c_size_t,
                                               C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.c_char_p, C.c_size_t]
        lib.oracle_expert_dispatch.restype = C.c_int
        lib.oracle_speculative_verify.argtypes = [f32p, f32p, C.c_size_t, C.c_size_t, i32p, C.c_float, C.c_uint32, C.c_float, C.c_float, f32p,
                                                  u32p, f32p, i32p, f32p, u32p, C.c_char_p, C.c_size_t]
        lib.oracle_speculative_verify.restype = C.c_int
        if self.kind == "port":
            lib.oracle_set_exp_mode.argtypes = [C.c_int]
            lib.oracle_philox4x32_10.argtypes = [u32p, u32p, u32p]
            lib.oracle_philox_uniform.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64]
            lib.oracle_philox_uniform.restype = C.c_float
        else:
            lib.oracle_session_create.argtypes = [C.c_uint64, C.c_char_p, C.c_size_t]
            lib.oracle_session_create.restype = C.c_void_p
            lib.oracle_session_sample.argtypes = [C.c_void_p, f32p, C.c_size_t, C.c_float, C.c_uint32, C.c_float, C.c_float,
                                                  i32p, f32p, C.c_char_p, C.c_size_t]
            lib.oracle_session_sample.restype = C.c_int
            lib.oracle_session_destroy.argtypes = [C.c_void_p]
            lib.oracle_mt19937_uniforms.argtypes = [C.c_uint64, C.c_size_t, f32p]
            lib.oracle_residual_with_generator.argtypes = [f32p, f32p, C.c_size_t, C.c_float, C.c_uint32, C.c_float, C.c_float, C.c_uint64,
                                                           i32p, f32p, C.c_char_p, C.c_size_t]
            lib.oracle_residual_with_generator.restype = C.c_int

    # -- sampler -----------------------------------------------------------
    def set_exp_mode(self, mode: int) -> None:
        """0 = libm expf (reference arithmetic), 1 = fp64 exp rounded to fp32 (device arithmetic)."""
        if self.kind != "port":
            if mode != 0:
                raise ValueError("the reference oracle only has its own libm arithmetic")
            return
        self.lib.oracle_set_exp_mode(mode)

    def distribution(self, logits, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0):
        """Candidate ids and renormalised probabilities, or (status, message)."""
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        ids = np.empty(logits.size, dtype=np.int32)
        probabilities = np.empty(logits.size, dtype=np.float32)
        count = C.c_size_t(0)
        message = C.create_string_buffer(256)
        status = self.lib.oracle_sampling_distribution(_ptr(logits, C.c_float), logits.size, temperature, top_k, top_p, min_p,
                                                       _ptr(ids, C.c_int32), _ptr(probabilities, C.c_float), logits.size,
                                                       C.byref(count), message, 256)
        if status != 0:
            return status, message.value.decode()
        return ids[:count.value].copy(), probabilities[:count.value].copy()

    def sample(self, logits, uniform, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0):
        """-> (status, token, probability, used_uniform, message)"""
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        token = C.c_int32(-1)
        probability = C.c_float(0.0)
        used = C.c_int(0)
        message = C.create_string_buffer(256)
        status = self.lib.oracle_sample_with_uniform(_ptr(logits, C.c_float), logits.size, temperature, top_k, top_p, min_p, uniform,
                                                     C.byref(token), C.byref(probability), C.byref(used), message, 256)
        return status, token.value, probability.value, used.value, message.value.decode()

    def topk_order(self, logits, count):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        count = min(int(count), logits.size)
        ids = np.empty(count, dtype=np.int32)
        self.lib.oracle_topk_order(_ptr(logits, C.c_float), logits.size, count, _ptr(ids, C.c_int32))
        return ids

    def indexer_topk(self, scores, top_k):
        """Latent-attention indexer selection (cpu_latent_attention.cpp:414-423): indices of the top_k scores, score
        descending, index ascending on ties.  The reference's own function is a file-static that cannot be linked
        from outside its translation unit, so both oracles answer this with the port's restatement."""
        lib = port().lib
        lib.oracle_indexer_topk.argtypes = [C.POINTER(C.c_float), C.c_size_t, C.c_size_t, C.POINTER(C.c_uint32)]
        lib.oracle_indexer_topk.restype = None
        scores = np.ascontiguousarray(scores, dtype=np.float32)
        selected = np.empty(min(int(top_k), scores.size), dtype=np.uint32)
        lib.oracle_indexer_topk(_ptr(scores, C.c_float), scores.size, int(top_k), _ptr(selected, C.c_uint32))
        return selected

    def sample_batch(self, logits, temperature, top_k, top_p, min_p, uniforms, threads=None):
        """logits: [rows, vocab] float32, or uint16 holding bf16 bit patterns.

        -> dict(token, probability, status, used_uniform)
        """
        logits = np.ascontiguousarray(logits)
        if logits.dtype == np.float32:
            dtype = 0
        elif logits.dtype == np.uint16:
            dtype = 1
        else:
            raise TypeError("logits must be float32 or uint16 (bf16 bits)")
        rows, vocab = logits.shape
        temperature = np.ascontiguousarray(temperature, dtype=np.float32)
        top_k = np.ascontiguousarray(top_k, dtype=np.uint32)
        top_p = np.ascontiguousarray(top_p, dtype=np.float32)
        min_p = np.ascontiguousarray(min_p, dtype=np.float32)
        uniforms = np.ascontiguousarray(uniforms, dtype=np.float32)
        for array in (temperature, top_k, top_p, min_p, uniforms):
            assert array.shape == (rows,)
        tokens = np.full(rows, -1, dtype=np.int32)
        probabilities = np.zeros(rows, dtype=np.float32)
        statuses = np.zeros(rows, dtype=np.int32)
        used = np.zeros(rows, dtype=np.int32)
        if threads is None:
            threads = os.cpu_count() or 1
        self.lib.oracle_sample_batch(logits.ctypes.data_as(C.c_void_p), dtype, rows, vocab, vocab,
                                     _ptr(temperature, C.c_float), _ptr(top_k, C.c_uint32), _ptr(top_p, C.c_float), _ptr(min_p, C.c_float),
                                     _ptr(uniforms, C.c_float), _ptr(tokens, C.c_int32), _ptr(probabilities, C.c_float),
                                     _ptr(statuses, C.c_int32), _ptr(used, C.c_int32), int(threads))
        return {"token": tokens, "probability": probabilities, "status": statuses, "used_uniform": used}

    # -- philox (port only) --------------------------------------------------
    def philox4x32_10(self, counter, key):
        counter = np.ascontiguousarray(counter, dtype=np.uint32)
        key = np.ascontiguousarray(key, dtype=np.uint32)
        out = np.zeros(4, dtype=np.uint32)
        self.lib.oracle_philox4x32_10(_ptr(counter, C.c_uint32), _ptr(key, C.c_uint32), _ptr(out, C.c_uint32))
        return out

    def philox_uniform(self, seed, row, step):
        return float(self.lib.oracle_philox_uniform(int(seed), int(row), int(step)))

    def philox_uniforms(self, seed, rows, step=0, row_offset=0):
        return np.array([self.philox_uniform(seed, row_offset + r, step) for r in range(rows)], dtype=np.float32)

    # -- reference Session route (reference only) ----------------------------
    def session_samples(self, seed, requests):
        """Run Session::sample for each (logits, options-dict) in order on one Session."""
        message = C.create_string_buffer(256)
        handle = self.lib.oracle_session_create(int(seed), message, 256)
        if not handle:
            raise RuntimeError(message.value.decode())
        results = []
        try:
            for logits, options in requests:
                logits = np.ascontiguousarray(logits, dtype=np.float32)
                token = C.c_int32(-1)
                probability = C.c_float(0.0)
                status = self.lib.oracle_session_sample(handle, _ptr(logits, C.c_float), logits.size,
                                                        options.get("temperature", 1.0), options.get("top_k", 0),
                                                        options.get("top_p", 1.0), options.get("min_p", 0.0),
                                                        C.byref(token), C.byref(probability), message, 256)
                results.append((status, token.value, probability.value, message.value.decode()))
        finally:
            self.lib.oracle_session_destroy(handle)
        return results

    def speculative_verify(self, target_logits, draft_logits, proposed, uniforms, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0):
        """The verification step of speculative decoding (session.cpp:776-880) for one Session.
        target_logits [(n + 1) x vocab], draft_logits [n x vocab], proposed [n], uniforms [>= n + 1] consumed in order.
        -> dict(status, message, accepted, accepted_probability[n], next_token, next_probability, uniforms_used)"""
        target_logits = np.ascontiguousarray(target_logits, dtype=np.float32)
        draft_logits = np.ascontiguousarray(draft_logits, dtype=np.float32).reshape(-1, target_logits.shape[1])
        proposed = np.ascontiguousarray(proposed, dtype=np.int32)
        uniforms = np.ascontiguousarray(uniforms, dtype=np.float32)
        count = proposed.size
        assert target_logits.shape[0] == count + 1 and draft_logits.shape[0] == count and uniforms.size >= count + 1
        accepted = C.c_uint32(0)
        used = C.c_uint32(0)
        token = C.c_int32(-1)
        probability = C.c_float(0.0)
        accepted_probability = np.zeros(max(count, 1), dtype=np.float32)
        message = C.create_string_buffer(256)
        status = self.lib.oracle_speculative_verify(_ptr(target_logits, C.c_float), _ptr(draft_logits, C.c_float), target_logits.shape[1], count,
                                                    _ptr(proposed, C.c_int32), temperature, top_k, top_p, min_p, _ptr(uniforms, C.c_float),
                                                    C.byref(accepted), _ptr(accepted_probability, C.c_float), C.byref(token),
                                                    C.byref(probability), C.byref(used), message, 256)
        return {"status": status, "message": message.value.decode(), "accepted": accepted.value,
                "accepted_probability": accepted_probability[:accepted.value].copy(), "next_token": token.value,
                "next_probability": np.float32(probability.value), "uniforms_used": used.value}

    def residual_with_generator(self, target_logits, draft_logits, seed, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0):
        """Reference only: sample_residual_distribution (session.cpp:150-202) itself with std::mt19937_64(seed)."""
        target_logits = np.ascontiguousarray(target_logits, dtype=np.float32)
        draft_logits = np.ascontiguousarray(draft_logits, dtype=np.float32)
        token = C.c_int32(-1)
        probability = C.c_float(0.0)
        message = C.create_string_buffer(256)
        status = self.lib.oracle_residual_with_generator(_ptr(target_logits, C.c_float), _ptr(draft_logits, C.c_float), target_logits.size,
                                                         temperature, top_k, top_p, min_p, int(seed), C.byref(token), C.byref(probability),
                                                         message, 256)
        return status, token.value, np.float32(probability.value), message.value.decode()

    def mt19937_uniforms(self, seed, count):
        values = np.zeros(count, dtype=np.float32)
        self.lib.oracle_mt19937_uniforms(int(seed), count, _ptr(values, C.c_float))
        return values

    # -- router --------------------------------------------------------------
    def expert_dispatch(self, router_logits, token_count, expert_count, top_k, score_function=0, normalization=1, scaling=1.0,
                        selection_bias=None, explicit_ids=None, flags=1, use_dispatch_into=False):
        """-> dict(status, message, batch_expert, batch_offset, token, rank, weight, assignment_count)"""
        router_logits = np.ascontiguousarray(router_logits, dtype=np.float32).reshape(-1)
        capacity = max(1, int(token_count) * int(top_k))
        batch_expert = np.zeros(max(1, expert_count), dtype=np.uint32)
        batch_offset = np.zeros(max(1, expert_count) + 1, dtype=np.uint32)
        route_token = np.zeros(capacity, dtype=np.uint32)
        route_rank = np.zeros(capacity, dtype=np.uint32)
        route_weight = np.zeros(capacity, dtype=np.float32)
        batch_count = C.c_size_t(0)
        assignment_count = C.c_size_t(0)
        message = C.create_string_buffer(256)
        bias_ptr, bias_count = None, 0
        if selection_bias is not None:
            selection_bias = np.ascontiguousarray(selection_bias, dtype=np.float32)
            bias_ptr, bias_count = _ptr(selection_bias, C.c_float), selection_bias.size
        explicit_ptr, explicit_count = None, 0
        if explicit_ids is not None:
            explicit_ids = np.ascontiguousarray(explicit_ids, dtype=np.uint32).reshape(-1)
            explicit_ptr, explicit_count = _ptr(explicit_ids, C.c_uint32), explicit_ids.size
        status = self.lib.oracle_expert_dispatch(int(bool(use_dispatch_into)), _ptr(router_logits, C.c_float), router_logits.size,
                                                 token_count, expert_count, top_k, score_function, normalization, scaling,
                                                 bias_ptr, bias_count, explicit_ptr, explicit_count, flags,
                                                 _ptr(batch_expert, C.c_uint32), _ptr(batch_offset, C.c_uint32), _ptr(route_token, C.c_uint32),
                                                 _ptr(route_rank, C.c_uint32), _ptr(route_weight, C.c_float), capacity,
                                                 C.byref(batch_count), C.byref(assignment_count), message, 256)
        result = {"status": status, "message": message.value.decode()}
        if status == 0:
            nb = batch_count.value
            total = int(batch_offset[nb])
            result.update(batch_expert=batch_expert[:nb].copy(), batch_offset=batch_offset[:nb + 1].copy(), token=route_token[:total].copy(),
                          rank=route_rank[:total].copy(), weight=route_weight[:total].copy(), assignment_count=assignment_count.value)
        return result


_cache: dict[str, Oracle] = {}


def port() -> Oracle:
    if "port" not in _cache:
        if not PORT_PATH.exists():
            build(port=True, ref=False)
        _cache["port"] = Oracle(PORT_PATH)
    return _cache["port"]


def reference() -> Oracle | None:
    """The compiled reference, or None where it was never built."""
    if "ref" not in _cache:
        if not REF_PATH.exists():
            return None
        _cache["ref"] = Oracle(REF_PATH)
    return _cache["ref"]


def best() -> Oracle:
    """The compiled reference when present, else the port."""
    return reference() or port()
