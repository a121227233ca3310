"""ctypes binding of libmoe_b200_sampler.so (the C ABI in include/moe_b200_sampler.h).

This is a thin harness layer for tests and the benchmark: every call goes
straight to the C entry point of the same name.  There is no fallback: if the
CUDA library has not been built, importing the binding works but `library()`
raises, and every computing call needs a B200.

The directory name is not a Python identifier; load it with
`__graft_entry__.load_package()` (registers it as ``ncnn_moe_runtime_b200``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIBRARY_PATH = HERE / "libmoe_b200_sampler.so"


SPECULATIVE_RESULT_DTYPE = np.dtype([("accepted", np.uint32), ("next_token", np.int32), ("next_probability", np.float32),
                                     ("uniforms_used", np.uint32), ("status", np.int32), ("flags", np.uint32)])
SPECULATIVE_MAX_DRAFT = 16
# numpy view of moe_sampled_row (16 bytes): what moe_sample_tokens returns per row
SAMPLED_ROW_DTYPE = np.dtype([("token", np.int32), ("probability", np.float32), ("flags", np.uint32), ("status", np.int32)])


class SampleOutputs(C.Structure):
    """moe_sample_outputs of include/moe_b200_sampler.h."""
    _fields_ = [("token_id", C.c_void_p), ("probability", C.c_void_p), ("row_flags", C.c_void_p), ("row_status", C.c_void_p),
                ("topk_index", C.c_void_p), ("topk_stride", C.c_uint32), ("kept_token", C.c_void_p), ("kept_probability", C.c_void_p),
                ("kept_count", C.c_void_p), ("kept_stride", C.c_uint32)]

DTYPE_F32 = 0
DTYPE_BF16 = 1
ROW_FLAG_STOP_TOKEN = 1
ROW_FLAG_USED_UNIFORM = 2
TOPK_FAST_MAX = 1024
ROUTER_SOFTMAX, ROUTER_SIGMOID, ROUTER_SQRT_SOFTPLUS = 0, 1, 2
ROUTER_FLAG_NORMALIZE_TOPK = 1

# numpy view of moe_row_params (40 bytes)
ROW_PARAMS_DTYPE = np.dtype([("temperature", np.float32), ("top_k", np.uint32), ("top_p", np.float32), ("min_p", np.float32),
                             ("seed", np.uint64), ("row_id", np.uint64), ("step", np.uint64)], align=True)
assert ROW_PARAMS_DTYPE.itemsize == 40


class RouterOptions(C.Structure):
    _fields_ = [("expert_count", C.c_uint32), ("top_k", C.c_uint32), ("score_function", C.c_int32), ("normalization", C.c_int32),
                ("routed_scaling_factor", C.c_float), ("flags", C.c_uint32), ("selection_bias", C.c_void_p),
                ("explicit_expert_ids", C.c_void_p)]


EXPORTED_SYMBOLS = [
    "moe_sampler_create", "moe_sampler_destroy", "moe_sampler_last_error", "moe_row_status_message", "moe_row_status_error_code",
    "moe_philox_uniform", "moe_host_alloc", "moe_host_free", "moe_sample_batch", "moe_sample_batch_ex", "moe_speculative_verify", "moe_speculative_verify_batch", "moe_speculative_verify_host", "moe_sample_batch_host",
    "moe_sample_local_candidates", "moe_sample_merge_candidates", "moe_router_dispatch", "moe_router_status_message",
    "moe_router_status_error_code", "moe_router_check_options", "moe_router_dispatch_host", "moe_regroup_gather",
    "moe_router_dispatch_static", "moe_sampler_set_overlap", "moe_sample_tokens", "moe_regroup_gather_check",
    "moe_indexer_topk",
]

_library = None


class MoeError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"moe status {status}: {message}")
        self.status = status
        self.message = message


def library() -> C.CDLL:
    """Loads the CUDA library; raises if it has not been built."""
    global _library
    if _library is not None:
        return _library
    if not LIBRARY_PATH.exists():
        raise FileNotFoundError(f"{LIBRARY_PATH} is missing: build it with `python ncnn-moe-runtime_b200/build.py` (there is no CPU fallback)")
    lib = C.CDLL(str(LIBRARY_PATH))
    vp, u32, u64, i32, f32, sz = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32, C.c_float, C.c_size_t
    lib.moe_sampler_create.argtypes = [C.c_int, u32, u32, C.POINTER(vp)]
    lib.moe_sampler_destroy.argtypes = [vp]
    lib.moe_sampler_destroy.restype = None
    lib.moe_sampler_set_overlap.argtypes = [vp, C.c_int]
    lib.moe_sampler_last_error.argtypes = [vp]
    lib.moe_sampler_last_error.restype = C.c_char_p
    lib.moe_row_status_message.argtypes = [C.c_int]
    lib.moe_row_status_message.restype = C.c_char_p
    lib.moe_row_status_error_code.argtypes = [C.c_int]
    lib.moe_philox_uniform.argtypes = [u64, u64, u64]
    lib.moe_philox_uniform.restype = f32
    lib.moe_host_alloc.argtypes = [sz, C.POINTER(vp)]
    lib.moe_host_free.argtypes = [vp]
    lib.moe_host_free.restype = None
    lib.moe_sample_batch.argtypes = [vp, vp, vp, C.c_int, u32, u32, sz, vp, u64, vp, vp, vp, vp, vp, vp, vp, u32]
    lib.moe_sample_batch_ex.argtypes = [vp, vp, vp, C.c_int, u32, u32, sz, vp, u64, vp, vp, C.POINTER(SampleOutputs)]
    lib.moe_speculative_verify.argtypes = [vp, vp, vp, vp, C.c_int, u32, u32, sz, vp, vp, vp, vp]
    lib.moe_speculative_verify_batch.argtypes = [vp, vp, vp, vp, C.c_int, u32, u32, u32, sz, vp, vp, vp, vp]
    lib.moe_speculative_verify_host.argtypes = [vp, vp, vp, C.c_int, u32, u32, sz, vp, vp, vp, vp]
    lib.moe_sample_batch_host.argtypes = [vp, vp, C.c_int, u32, u32, sz, vp, vp, vp, vp, vp, vp, vp, vp, u32]
    lib.moe_sample_local_candidates.argtypes = [vp, vp, vp, C.c_int, u32, u32, sz, u32, u32, vp]
    lib.moe_sample_merge_candidates.argtypes = [vp, vp, vp, u32, u32, u32, vp, u64, vp, vp, vp, vp, vp, u32]
    lib.moe_router_dispatch.argtypes = [vp, vp, vp, u32, C.POINTER(RouterOptions), vp, vp, vp, vp, vp]
    lib.moe_router_dispatch_host.argtypes = [vp, vp, u32, C.POINTER(RouterOptions), vp, vp, vp, vp, vp]
    lib.moe_router_status_message.argtypes = [C.c_int]
    lib.moe_router_status_message.restype = C.c_char_p
    lib.moe_router_status_error_code.argtypes = [C.c_int]
    lib.moe_router_check_options.argtypes = [u32, C.POINTER(RouterOptions)]
    lib.moe_regroup_gather.argtypes = [vp, vp, vp, u32, u32, vp, u32, vp]
    lib.moe_sample_tokens.argtypes = [vp, vp, vp, C.c_int, u32, u32, sz, vp, u64, vp, vp, vp]
    lib.moe_regroup_gather_check.argtypes = [vp, vp, C.POINTER(i32)]
    lib.moe_indexer_topk.argtypes = [vp, vp, vp, u32, u32, sz, u32, vp, vp]
    lib.moe_router_dispatch_static.argtypes = [vp, vp, u32, C.POINTER(RouterOptions), vp, vp, vp, vp, vp, C.c_char_p, sz]
    _library = lib
    return lib


def row_status_message(code: int) -> str:
    return library().moe_row_status_message(int(code)).decode()


def router_status_message(code: int) -> str:
    return library().moe_router_status_message(int(code)).decode()


def philox_uniform(seed: int, row_id: int, step: int) -> float:
    return float(library().moe_philox_uniform(int(seed), int(row_id), int(step)))


def make_row_params(rows: int, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, seed=0, row_id=None, step=0) -> np.ndarray:
    """Array of moe_row_params; every argument is a scalar or a per-row array."""
    params = np.zeros(rows, dtype=ROW_PARAMS_DTYPE)
    params["temperature"] = temperature
    params["top_k"] = top_k
    params["top_p"] = top_p
    params["min_p"] = min_p
    params["seed"] = seed
    params["row_id"] = np.arange(rows, dtype=np.uint64) if row_id is None else row_id
    params["step"] = step
    return params


def stop_lists_to_csr(stop_lists):
    """[[ids of row 0], [ids of row 1], ...] -> (offsets int32[rows+1], tokens int32[])"""
    offsets = np.zeros(len(stop_lists) + 1, dtype=np.int32)
    offsets[1:] = np.cumsum([len(s) for s in stop_lists])
    tokens = np.array([t for s in stop_lists for t in s], dtype=np.int32)
    return offsets, tokens


def _np_ptr(array):
    return None if array is None else C.c_void_p(array.ctypes.data)


def _dev_ptr(tensor):
    return None if tensor is None else C.c_void_p(tensor.data_ptr())


@dataclass
class DispatchPlan:
    """ExpertDispatchPlan as CSR arrays (numpy or torch, matching the call)."""
    expert_offsets: object
    route_token: object
    route_rank: object
    route_weight: object
    status: int


class Sampler:
    """One moe_sampler handle."""

    def __init__(self, max_rows: int, max_vocab: int, device: int = 0):
        self._lib = library()
        handle = C.c_void_p()
        status = self._lib.moe_sampler_create(int(device), int(max_rows), int(max_vocab), C.byref(handle))
        if status != 0:
            raise MoeError(status, "moe_sampler_create failed (needs a compute-capability 10.x CUDA device)")
        self._handle = handle
        self.device = device
        self.max_rows = max_rows
        self.max_vocab = max_vocab

    def set_overlap(self, enable: bool):
        """Let consecutive sample_batch launches on one stream overlap (see moe_sampler_set_overlap)."""
        self._check(self._lib.moe_sampler_set_overlap(self._handle, int(bool(enable))))

    def close(self):
        if getattr(self, "_handle", None):
            self._lib.moe_sampler_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int):
        if status != 0:
            raise MoeError(status, self._lib.moe_sampler_last_error(self._handle).decode())

    # ---- device-resident logits (torch tensors) ---------------------------------
    def sample_batch(self, logits, params=None, step_offset=0, stop_lists=None, topk_stride=0, stream=None, vocab=None, out=None, kept_stride=0):
        """logits: CUDA tensor [rows, row_stride] float32 or bfloat16.  Returns a dict of CUDA tensors.
        kept_stride > 0 also returns every row's kept candidates (kept_count, kept_token, kept_probability)."""
        import torch
        rows, row_stride = logits.shape
        vocab = row_stride if vocab is None else vocab
        dtype = DTYPE_F32 if logits.dtype == torch.float32 else DTYPE_BF16
        if logits.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("logits must be float32 or bfloat16")
        device = logits.device
        if out is None:
            out = {
                "token": torch.empty(rows, dtype=torch.int32, device=device),
                "probability": torch.empty(rows, dtype=torch.float32, device=device),
                "flags": torch.empty(rows, dtype=torch.int32, device=device),
                "status": torch.empty(rows, dtype=torch.int32, device=device),
                "topk": torch.empty((rows, topk_stride), dtype=torch.int32, device=device) if topk_stride else None,
            }
        offsets = tokens = None
        if stop_lists is not None:
            offsets, tokens = stop_lists_to_csr(stop_lists)
        if params is not None:
            params = np.ascontiguousarray(params, dtype=ROW_PARAMS_DTYPE)
            assert params.shape == (rows,)
        stream_handle = torch.cuda.current_stream(device).cuda_stream if stream is None else stream
        if kept_stride:
            if "kept_count" not in out:
                out["kept_count"] = torch.empty(rows, dtype=torch.int32, device=device)
                out["kept_token"] = torch.full((rows, kept_stride), -1, dtype=torch.int32, device=device)
                out["kept_probability"] = torch.zeros((rows, kept_stride), dtype=torch.float32, device=device)
            outputs = SampleOutputs(_dev_ptr(out["token"]), _dev_ptr(out["probability"]), _dev_ptr(out["flags"]), _dev_ptr(out["status"]),
                                    _dev_ptr(out.get("topk")), int(topk_stride), _dev_ptr(out["kept_token"]), _dev_ptr(out["kept_probability"]),
                                    _dev_ptr(out["kept_count"]), int(kept_stride))
            self._check(self._lib.moe_sample_batch_ex(self._handle, C.c_void_p(stream_handle), _dev_ptr(logits), dtype, rows, vocab, logits.stride(0),
                                                      _np_ptr(params), int(step_offset), _np_ptr(offsets), _np_ptr(tokens), C.byref(outputs)))
            return out
        self._check(self._lib.moe_sample_batch(self._handle, C.c_void_p(stream_handle), _dev_ptr(logits), dtype, rows, vocab, logits.stride(0),
                                               _np_ptr(params), int(step_offset), _np_ptr(offsets), _np_ptr(tokens), _dev_ptr(out["token"]),
                                               _dev_ptr(out["probability"]), _dev_ptr(out["flags"]), _dev_ptr(out["status"]),
                                               _dev_ptr(out.get("topk")), int(topk_stride)))
        return out

    def sample_tokens(self, logits, params=None, step_offset=0, stop_lists=None, stream=None, vocab=None, results=None):
        """moe_sample_tokens: CUDA logits in, one 16-byte record per row out on the host (synchronous).
        results: optional numpy array of SAMPLED_ROW_DTYPE (e.g. a view of page-locked memory) to fill."""
        import torch
        rows, row_stride = logits.shape
        vocab = row_stride if vocab is None else vocab
        dtype = DTYPE_F32 if logits.dtype == torch.float32 else DTYPE_BF16
        if results is None:
            results = np.empty(rows, dtype=SAMPLED_ROW_DTYPE)
        offsets = tokens = None
        if stop_lists is not None:
            offsets, tokens = stop_lists_to_csr(stop_lists)
        if params is not None:
            params = np.ascontiguousarray(params, dtype=ROW_PARAMS_DTYPE)
        stream_handle = torch.cuda.current_stream(logits.device).cuda_stream if stream is None else stream
        self._check(self._lib.moe_sample_tokens(self._handle, C.c_void_p(stream_handle), _dev_ptr(logits), dtype, rows, vocab, logits.stride(0),
                                                _np_ptr(params), int(step_offset), _np_ptr(offsets), _np_ptr(tokens), _np_ptr(results)))
        return results

    def speculative_verify(self, target_logits, draft_logits, proposed, params, stream=None, out=None, sync=True):
        """Verification step of speculative decoding for one Session (moe_speculative_verify).
        target_logits: CUDA [draft_count + 1, row_stride]; draft_logits: CUDA [draft_count, row_stride];
        proposed: CUDA int32 [draft_count]; params: one ROW_PARAMS_DTYPE entry.
        Returns dict(accepted, next_token, next_probability, uniforms_used, status, accepted_probability) on the host
        (sync=False: the device tensors, to be passed back as `out`)."""
        import torch
        draft_count = int(proposed.numel())
        rows, row_stride = target_logits.shape
        assert rows == draft_count + 1
        dtype = DTYPE_F32 if target_logits.dtype == torch.float32 else DTYPE_BF16
        device = target_logits.device
        params = np.ascontiguousarray(params, dtype=ROW_PARAMS_DTYPE).reshape(1)
        if out is None:
            out = (torch.zeros(max(draft_count, 1), dtype=torch.float32, device=device),
                   torch.zeros(SPECULATIVE_RESULT_DTYPE.itemsize, dtype=torch.uint8, device=device))
        accepted_probability, result = out
        stream_handle = torch.cuda.current_stream(device).cuda_stream if stream is None else stream
        self._check(self._lib.moe_speculative_verify(self._handle, C.c_void_p(stream_handle), _dev_ptr(target_logits),
                                                     _dev_ptr(draft_logits) if draft_count else None, dtype, draft_count, row_stride,
                                                     target_logits.stride(0), _dev_ptr(proposed) if draft_count else None, _np_ptr(params),
                                                     _dev_ptr(accepted_probability), _dev_ptr(result)))
        if not sync:
            return out   # device tensors (accepted_probability, raw result record); nothing was waited for
        torch.cuda.synchronize(device)
        record = result.cpu().numpy().view(SPECULATIVE_RESULT_DTYPE)[0]
        out = {name: record[name].item() for name in SPECULATIVE_RESULT_DTYPE.names}
        out["next_probability"] = np.float32(record["next_probability"])
        out["accepted_probability"] = accepted_probability.cpu().numpy()[:out["accepted"]]
        return out

    def speculative_verify_batch(self, target_logits, draft_logits, proposed, params, stream=None, out=None, sync=True):
        """moe_speculative_verify_batch: `sessions` Sessions verified in one call.
        target_logits: CUDA [sessions, draft_count + 1, vocab]; draft_logits: CUDA [sessions, draft_count, vocab] (None when
        draft_count is 0); proposed: CUDA int32 [sessions, draft_count]; params: ROW_PARAMS_DTYPE [sessions].
        Returns (records, accepted_probability): a SPECULATIVE_RESULT_DTYPE array [sessions] and float32 [sessions, draft_count]
        on the host (sync=False: the device tensors, to be passed back as `out`)."""
        import torch
        sessions, positions, vocab = target_logits.shape
        draft_count = positions - 1
        assert target_logits.is_contiguous() and (draft_count == 0 or (draft_logits.is_contiguous() and proposed.is_contiguous()))
        assert draft_count == 0 or (tuple(draft_logits.shape) == (sessions, draft_count, vocab) and tuple(proposed.shape) == (sessions, draft_count))
        dtype = DTYPE_F32 if target_logits.dtype == torch.float32 else DTYPE_BF16
        device = target_logits.device
        params = np.ascontiguousarray(params, dtype=ROW_PARAMS_DTYPE).reshape(sessions)
        if out is None:
            out = (torch.zeros(max(sessions * draft_count, 1), dtype=torch.float32, device=device),
                   torch.zeros(max(sessions, 1) * SPECULATIVE_RESULT_DTYPE.itemsize, dtype=torch.uint8, device=device))
        accepted_probability, result = out
        stream_handle = torch.cuda.current_stream(device).cuda_stream if stream is None else stream
        self._check(self._lib.moe_speculative_verify_batch(self._handle, C.c_void_p(stream_handle), _dev_ptr(target_logits),
                                                           _dev_ptr(draft_logits) if draft_count else None, dtype, sessions, draft_count, vocab, vocab,
                                                           _dev_ptr(proposed) if draft_count else None, _np_ptr(params),
                                                           _dev_ptr(accepted_probability), _dev_ptr(result)))
        if not sync:
            return out
        torch.cuda.synchronize(device)
        records = result.cpu().numpy().view(SPECULATIVE_RESULT_DTYPE)[:sessions].copy()
        return records, accepted_probability.cpu().numpy()[:sessions * draft_count].reshape(sessions, draft_count)

    def speculative_verify_host(self, target_logits, draft_logits, proposed, params):
        """moe_speculative_verify_host: numpy float32 logits [draft_count + 1, vocab] / [draft_count, vocab], numpy int32 proposals."""
        target_logits = np.ascontiguousarray(target_logits, dtype=np.float32)
        proposed = np.ascontiguousarray(proposed, dtype=np.int32)
        draft_count = proposed.size
        draft_logits = np.ascontiguousarray(draft_logits, dtype=np.float32).reshape(draft_count, target_logits.shape[1])
        params = np.ascontiguousarray(params, dtype=ROW_PARAMS_DTYPE).reshape(1)
        accepted_probability = np.zeros(max(draft_count, 1), dtype=np.float32)
        record = np.zeros(1, dtype=SPECULATIVE_RESULT_DTYPE)
        self._check(self._lib.moe_speculative_verify_host(self._handle, _np_ptr(target_logits), _np_ptr(draft_logits) if draft_count else None, DTYPE_F32,
                                                          draft_count, target_logits.shape[1], target_logits.shape[1],
                                                          _np_ptr(proposed) if draft_count else None, _np_ptr(params), _np_ptr(accepted_probability),
                                                          _np_ptr(record)))
        out = {name: record[0][name].item() for name in SPECULATIVE_RESULT_DTYPE.names}
        out["next_probability"] = np.float32(record[0]["next_probability"])
        out["accepted_probability"] = accepted_probability[:out["accepted"]]
        return out

    # ---- host buffers (numpy) ----------------------------------------------------
    def sample_batch_host(self, logits, params, stop_lists=None, topk_stride=0):
        """logits: numpy [rows, vocab] float32, or uint16 holding bf16 bit patterns."""
        logits = np.ascontiguousarray(logits)
        rows, vocab = logits.shape
        if logits.dtype == np.float32:
            dtype = DTYPE_F32
        elif logits.dtype == np.uint16:
            dtype = DTYPE_BF16
        else:
            raise TypeError("logits must be float32 or uint16 (bf16 bits)")
        params = np.ascontiguousarray(params, dtype=ROW_PARAMS_DTYPE)
        out = {
            "token": np.empty(rows, dtype=np.int32),
            "probability": np.empty(rows, dtype=np.float32),
            "flags": np.empty(rows, dtype=np.uint32),
            "status": np.empty(rows, dtype=np.int32),
            "topk": np.empty((rows, topk_stride), dtype=np.int32) if topk_stride else None,
        }
        offsets = tokens = None
        if stop_lists is not None:
            offsets, tokens = stop_lists_to_csr(stop_lists)
        self._check(self._lib.moe_sample_batch_host(self._handle, _np_ptr(logits), dtype, rows, vocab, vocab, _np_ptr(params), _np_ptr(offsets),
                                                    _np_ptr(tokens), _np_ptr(out["token"]), _np_ptr(out["probability"]), _np_ptr(out["flags"]),
                                                    _np_ptr(out["status"]), _np_ptr(out["topk"]), int(topk_stride)))
        return out

    def sample_host_raw(self, logits_ptr, dtype, rows, vocab, params, out):
        """Host-buffer call on preallocated buffers (pinned or pageable) — the benchmark's end-to-end path."""
        self._check(self._lib.moe_sample_batch_host(self._handle, C.c_void_p(logits_ptr), dtype, rows, vocab, vocab, _np_ptr(params), None, None,
                                                    _np_ptr(out["token"]), _np_ptr(out["probability"]), _np_ptr(out["flags"]),
                                                    _np_ptr(out["status"]), None, 0))

    # ---- vocabulary-sharded -------------------------------------------------------
    def local_candidates(self, logits, vocab_begin, top_k, stream=None, out=None):
        """moe_sample_local_candidates: [rows, top_k] int64 records of this vocabulary slice (written to `out` when given)."""
        import torch
        rows, row_stride = logits.shape
        dtype = DTYPE_F32 if logits.dtype == torch.float32 else DTYPE_BF16
        candidates = torch.empty((rows, top_k), dtype=torch.int64, device=logits.device) if out is None else out
        stream_handle = torch.cuda.current_stream(logits.device).cuda_stream if stream is None else stream
        self._check(self._lib.moe_sample_local_candidates(self._handle, C.c_void_p(stream_handle), _dev_ptr(logits), dtype, rows, row_stride,
                                                          logits.stride(0), int(vocab_begin), int(top_k), _dev_ptr(candidates)))
        return candidates

    def merge_candidates(self, gathered, params, top_k, step_offset=0, topk_stride=0, stream=None, out=None):
        """gathered: CUDA int64 tensor [shards, rows, top_k]."""
        import torch
        shards, rows, k = gathered.shape
        assert k == top_k
        device = gathered.device
        out = out if out is not None else {
            "token": torch.empty(rows, dtype=torch.int32, device=device),
            "probability": torch.empty(rows, dtype=torch.float32, device=device),
            "flags": torch.empty(rows, dtype=torch.int32, device=device),
            "status": torch.empty(rows, dtype=torch.int32, device=device),
            "topk": torch.empty((rows, topk_stride), dtype=torch.int32, device=device) if topk_stride else None,
        }
        if params is not None:   # None reuses the parameters uploaded by the previous call
            params = np.ascontiguousarray(params, dtype=ROW_PARAMS_DTYPE)
        stream_handle = torch.cuda.current_stream(device).cuda_stream if stream is None else stream
        self._check(self._lib.moe_sample_merge_candidates(self._handle, C.c_void_p(stream_handle), _dev_ptr(gathered), shards, rows, top_k,
                                                          _np_ptr(params), int(step_offset), _dev_ptr(out["token"]), _dev_ptr(out["probability"]),
                                                          _dev_ptr(out["flags"]), _dev_ptr(out["status"]), _dev_ptr(out["topk"]), int(topk_stride)))
        return out

    # ---- router ---------------------------------------------------------------------
    def router_dispatch_host(self, router_logits, token_count, expert_count, top_k, score_function=ROUTER_SOFTMAX, normalization=1,
                             scaling=1.0, selection_bias=None, explicit_ids=None, flags=ROUTER_FLAG_NORMALIZE_TOPK) -> DispatchPlan:
        router_logits = np.ascontiguousarray(router_logits, dtype=np.float32).reshape(-1)
        options = RouterOptions(expert_count, top_k, score_function, normalization, scaling, flags, None, None)
        if selection_bias is not None:
            selection_bias = np.ascontiguousarray(selection_bias, dtype=np.float32)
            options.selection_bias = selection_bias.ctypes.data
        if explicit_ids is not None:
            explicit_ids = np.ascontiguousarray(explicit_ids, dtype=np.uint32).reshape(-1)
            options.explicit_expert_ids = explicit_ids.ctypes.data
        routes = max(1, int(token_count) * int(top_k))
        offsets = np.zeros(max(1, expert_count) + 1, dtype=np.uint32)
        token = np.zeros(routes, dtype=np.uint32)
        rank = np.zeros(routes, dtype=np.uint32)
        weight = np.zeros(routes, dtype=np.float32)
        status = np.zeros(1, dtype=np.int32)
        code = self._lib.moe_router_dispatch_host(self._handle, _np_ptr(router_logits), int(token_count), C.byref(options), _np_ptr(offsets),
                                                  _np_ptr(token), _np_ptr(rank), _np_ptr(weight), _np_ptr(status))
        if code != 0 and status[0] == 0:
            self._check(code)
        return DispatchPlan(offsets, token, rank, weight, int(status[0]))

    def router_dispatch(self, router_logits, top_k, score_function=ROUTER_SOFTMAX, normalization=1, scaling=1.0, selection_bias=None,
                        explicit_ids=None, flags=ROUTER_FLAG_NORMALIZE_TOPK, stream=None, out=None) -> DispatchPlan:
        """router_logits: CUDA float32 tensor [tokens, experts]; bias / explicit ids CUDA tensors."""
        import torch
        token_count, expert_count = router_logits.shape
        device = router_logits.device
        options = RouterOptions(expert_count, top_k, score_function, normalization, scaling, flags,
                                selection_bias.data_ptr() if selection_bias is not None else None,
                                explicit_ids.data_ptr() if explicit_ids is not None else None)
        routes = token_count * top_k
        if out is None:
            out = DispatchPlan(torch.empty(expert_count + 1, dtype=torch.int32, device=device), torch.empty(routes, dtype=torch.int32, device=device),
                               torch.empty(routes, dtype=torch.int32, device=device), torch.empty(routes, dtype=torch.float32, device=device),
                               torch.zeros(1, dtype=torch.int32, device=device))
        stream_handle = torch.cuda.current_stream(device).cuda_stream if stream is None else stream
        self._check(self._lib.moe_router_dispatch(self._handle, C.c_void_p(stream_handle), _dev_ptr(router_logits), token_count, C.byref(options),
                                                  _dev_ptr(out.expert_offsets), _dev_ptr(out.route_token), _dev_ptr(out.route_rank),
                                                  _dev_ptr(out.route_weight), _dev_ptr(out.status)))
        return out

    def regroup_gather(self, hidden, route_token, stream=None):
        import torch
        token_count, columns = hidden.shape
        routes = route_token.numel()
        gathered = torch.empty((routes, columns), dtype=torch.float32, device=hidden.device)
        stream_handle = torch.cuda.current_stream(hidden.device).cuda_stream if stream is None else stream
        self._check(self._lib.moe_regroup_gather(self._handle, C.c_void_p(stream_handle), _dev_ptr(hidden), token_count, columns,
                                                 _dev_ptr(route_token), routes, _dev_ptr(gathered)))
        return gathered

    def indexer_topk(self, scores, top_k, count=None, with_scores=False, stream=None):
        """moe_indexer_topk: scores CUDA float32 [rows, row_stride] -> int32 tensor [rows, top_k] of indices in rank order
        (score descending, index ascending on ties; -1 beyond min(top_k, count)), and their scores when asked."""
        import torch
        rows, row_stride = scores.shape
        count = row_stride if count is None else count
        indices = torch.empty((rows, top_k), dtype=torch.int32, device=scores.device)
        values = torch.empty((rows, top_k), dtype=torch.float32, device=scores.device) if with_scores else None
        stream_handle = torch.cuda.current_stream(scores.device).cuda_stream if stream is None else stream
        self._check(self._lib.moe_indexer_topk(self._handle, C.c_void_p(stream_handle), _dev_ptr(scores), rows, int(count), scores.stride(0), int(top_k),
                                               _dev_ptr(indices), _dev_ptr(values)))
        return (indices, values) if with_scores else indices

    def regroup_gather_check(self, stream=None) -> bool:
        """True when a regroup_gather since the last check met a token index outside the hidden matrix (synchronises)."""
        import torch
        stream_handle = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        flag = C.c_int32(0)
        self._check(self._lib.moe_regroup_gather_check(self._handle, C.c_void_p(stream_handle), C.byref(flag)))
        return flag.value != 0
