"""ctypes binding of libmini_llm_b200.so - the same calls a C/C++ host makes through
include/mlb.h and include/mini_llm_compat.h. There is no Python or CPU implementation of
the decode path behind these classes: if the library is missing they raise."""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import List, Optional, Sequence

import numpy as np

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libmini_llm_b200.so")
MLB_MAX_LAYERS = 128

MLB_OK = 0
MLB_E_INVALID, MLB_E_IO, MLB_E_FORMAT, MLB_E_CUDA, MLB_E_NOMEM = -1, -2, -3, -4, -5
MLB_E_KV_FULL, MLB_E_CONTEXT_FULL, MLB_E_TIMEOUT, MLB_E_UNSUPPORTED = -6, -7, -8, -9
DT_DEFAULT, DT_F32, DT_BF16, DT_FP8 = 0, 1, 2, 3
_DTYPE_NAMES = {"float32": DT_F32, "bfloat16": DT_BF16, "float8_e4m3": DT_FP8}


class MlbError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[mlb status {status}] {message}")
        self.status = status
        self.message = message


class Config(C.Structure):
    _fields_ = [
        ("dim", C.c_int32), ("layers", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("ffn_dim", C.c_int32), ("vocab", C.c_int32), ("max_context", C.c_int32),
        ("ple_dim", C.c_int32), ("qk_norm", C.c_int32), ("query_gating", C.c_int32),
        ("dn_key_dim", C.c_int32), ("dn_value_dim", C.c_int32),
        ("weight_dtype", C.c_int32), ("kv_dtype", C.c_int32), ("layer_types_set", C.c_int32),
        ("rope_theta", C.c_float), ("rms_eps", C.c_float),
        ("layer_types", C.c_uint8 * MLB_MAX_LAYERS),
    ]


class Sampling(C.Structure):
    _fields_ = [("mode", C.c_int32), ("top_k", C.c_int32), ("temperature", C.c_float),
                ("seeds", C.POINTER(C.c_uint64))]


class KernelStat(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("launches", C.c_int32), ("total_ms", C.c_float),
                ("bytes", C.c_uint64), ("flops", C.c_uint64)]


_lib = None


def lib() -> C.CDLL:
    """Loads the shared library; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python -m mini_llm_cuda_b200.build` "
            "(the decode path has no CPU or PyTorch fallback)")
    L = C.CDLL(_LIB_PATH)
    vp, i32p, f32p, u64p = C.c_void_p, C.POINTER(C.c_int32), C.POINTER(C.c_float), C.POINTER(C.c_uint64)
    cfgp, samp = C.POINTER(Config), C.POINTER(Sampling)
    sigs = {
        "mlb_config_init": (None, [cfgp]),
        "mlb_model_load": (C.c_int, [C.c_char_p, C.c_int, cfgp, C.POINTER(vp)]),
        "mlb_model_get_config": (C.c_int, [vp, cfgp]),
        "mlb_model_weight_bytes": (C.c_uint64, [vp]),
        "mlb_model_free": (None, [vp]),
        "mlb_file_inspect": (C.c_int, [C.c_char_p, cfgp, cfgp, u64p]),
        "mlb_session_new": (C.c_int, [vp, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(vp)]),
        "mlb_session_reset": (C.c_int, [vp]),
        "mlb_session_free": (None, [vp]),
        "mlb_prefill": (C.c_int, [vp, i32p, i32p, C.c_int]),
        "mlb_decode_step": (C.c_int, [vp, samp, i32p, i32p]),
        "mlb_decode_n": (C.c_int, [vp, samp, C.c_int, i32p]),
        "mlb_session_set_stop_token": (C.c_int, [vp, C.c_int]),
        "mlb_shard_range": (C.c_int, [C.c_int, C.c_int, C.c_int, i32p, i32p]),
        "mlb_pool_new": (C.c_int, [C.c_char_p, i32p, C.c_int, C.c_int, C.c_int, cfgp, C.POINTER(vp)]),
        "mlb_pool_free": (None, [vp]),
        "mlb_pool_shards": (C.c_int, [vp, i32p, i32p, i32p, C.c_int]),
        "mlb_pool_set_stop_token": (C.c_int, [vp, C.c_int]),
        "mlb_pool_prefill": (C.c_int, [vp, i32p, i32p, C.c_int]),
        "mlb_pool_decode_n": (C.c_int, [vp, samp, C.c_int, i32p]),
        "mlb_session_stopped": (C.c_int, [vp, i32p]),
        "mlb_decode_timed": (C.c_int, [vp, samp, C.c_int, C.c_int, f32p, f32p, i32p]),
        "mlb_profile_decode": (C.c_int, [vp, samp, C.c_int, C.c_int, C.POINTER(KernelStat), C.c_int, C.POINTER(C.c_int)]),
        "mlb_get_logits": (C.c_int, [vp, f32p]),
        "mlb_get_probs_col": (C.c_int, [vp, C.c_int, f32p]),
        "mlb_session_positions": (C.c_int, [vp, i32p]),
        "mlb_session_step_bytes": (C.c_int, [vp, u64p, u64p, u64p, u64p]),
        "mlb_session_launches_per_step": (C.c_int, [vp]),
        "mlb_session_grid_timers": (C.c_int, [vp, C.POINTER(C.c_longlong), C.c_int]),
        "mlb_session_grid_trace": (C.c_int, [vp, C.POINTER(C.c_longlong), C.c_int]),
        "mlb_op_wait_probe": (C.c_int, [C.c_int, C.c_uint32]),
        "mlb_score_tokens": (C.c_int, [vp, C.POINTER(C.c_int32), C.c_int, C.POINTER(C.c_float)]),
        "mlb_kv_alloc_new": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(vp)]),
        "mlb_kv_alloc_ensure": (C.c_int, [vp, C.c_int, C.c_int, C.c_int]),
        "mlb_kv_alloc_table": (C.c_int, [vp, C.c_int, i32p, C.c_int]),
        "mlb_kv_alloc_free_pages": (C.c_int, [vp]),
        "mlb_kv_alloc_release": (None, [vp, C.c_int]),
        "mlb_kv_alloc_free": (None, [vp]),
        "mlb_rope_table": (None, [f32p, C.c_int, C.c_int, C.c_float]),
        "mlb_op_attn_decode": (C.c_int, [vp, vp, C.c_int, vp, C.c_int, C.c_int, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int,
                                         C.c_int, C.c_int, vp]),
        "mlb_op_gemm_bf16": (C.c_int, [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, vp]),
        "mlb_op_attn_decode_static": (C.c_int, [vp, vp, C.c_int, vp, C.c_int, C.c_int, vp, vp, vp, vp, C.c_int, C.c_int,
                                                C.c_int, C.c_int, C.c_int, vp]),
        "mlb_op_attn_decode_static_status": (C.c_int, [vp]),
        "mlb_op_attn_decode_static_capacity": (C.c_size_t, []),
        "mlb_last_error": (C.c_char_p, []),
        "mlb_version": (C.c_char_p, []),
        "mlb_compat_configure": (C.c_int, [cfgp, C.c_int]),
        "mlb_compat_load_model": (C.c_int, [C.c_char_p]),
        "mlb_compat_load_model_path": (C.c_int, [C.c_char_p]),
        "mlb_compat_load_vocab": (C.c_int, [C.c_char_p]),
        "mlb_compat_vocab_lookup": (C.c_int, [C.c_char_p]),
        "mlb_compat_vocab_token": (C.c_char_p, [C.c_int]),
        "mlb_compat_load_story_context": (C.c_int, [C.c_char_p, C.c_int, C.c_int]),
        "mlb_compat_run_inference": (C.c_int, [C.c_int]),
        "mlb_compat_run_inference_loop": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int]),
        "mlb_compat_set_stop_token": (C.c_int, [C.c_char_p, C.c_int]),
        "mlb_compat_set_streaming": (None, [C.c_int]),
        "mlb_compat_max_context": (C.c_int, []),
        "mlb_compat_vocab_size": (C.c_int, []),
        "mlb_compat_tokens": (i32p, []),
        "mlb_compat_set_tokens": (C.c_int, [i32p, C.c_int]),
        "mlb_compat_last_probs": (f32p, []),
        "mlb_compat_last_loop_ms": (C.c_double, []),
        "mlb_compat_shutdown": (None, []),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(L, name)          # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


EXPORTED_SYMBOLS_NOTE = "every symbol of include/mlb.h and the extern \"C\" part of include/mini_llm_compat.h"


def check(status: int) -> int:
    if status < 0:
        raise MlbError(status, lib().mlb_last_error().decode("utf-8", "replace"))
    return status


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def _ptr(a: np.ndarray, ctype):
    return a.ctypes.data_as(C.POINTER(ctype))


def make_override(**kw) -> Config:
    """Config with every field unset except the given ones (dtype fields accept names)."""
    cfg = Config()
    lib().mlb_config_init(C.byref(cfg))
    for k, v in kw.items():
        if v is None:
            continue
        if k in ("weight_dtype", "kv_dtype") and isinstance(v, str):
            v = _DTYPE_NAMES[v]
        if k == "layer_types":
            for i, t in enumerate(v):
                cfg.layer_types[i] = 1 if t in (1, "delta_net") else 0
            cfg.layer_types_set = 1
            continue
        setattr(cfg, k, v)
    return cfg


def rope_table(max_len: int, head_dim: int, base: float) -> np.ndarray:
    out = np.empty((max_len, head_dim), dtype=np.float32)
    lib().mlb_rope_table(_ptr(out, C.c_float), max_len, head_dim, base)
    return out


def inspect_file(path: str, override: Optional[Config] = None):
    cfg = Config()
    n = C.c_uint64(0)
    check(lib().mlb_file_inspect(path.encode(), C.byref(override) if override is not None else None,
                                 C.byref(cfg), C.byref(n)))
    return cfg, int(n.value)


class Model:
    def __init__(self, path: str, device: int = 0, override: Optional[Config] = None):
        self._h = C.c_void_p()
        check(lib().mlb_model_load(path.encode(), device, C.byref(override) if override is not None else None,
                                   C.byref(self._h)))
        self.config = Config()
        check(lib().mlb_model_get_config(self._h, C.byref(self.config)))

    @property
    def weight_bytes(self) -> int:
        return int(lib().mlb_model_weight_bytes(self._h))

    def close(self):
        if self._h:
            lib().mlb_model_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _sampling(s: Optional[dict], batch: int):
    if not s or s.get("mode", "greedy") in (0, "greedy"):
        return None, None
    seeds = s.get("seeds")
    arr = None
    sp = Sampling(mode=1, top_k=int(s["top_k"]), temperature=float(s["temperature"]))
    if seeds is not None:
        arr = np.ascontiguousarray(seeds, dtype=np.uint64)
        assert arr.size == batch
        sp.seeds = _ptr(arr, C.c_uint64)
    return sp, arr


class Session:
    """One batch of independent sequences on one GPU."""

    def __init__(self, model: Model, batch: int, max_context: int = 0, kv_pages: int = 0):
        self.model = model
        self.batch = batch
        self._h = C.c_void_p()
        check(lib().mlb_session_new(model._h, batch, max_context, 16, kv_pages, C.byref(self._h)))

    def reset(self):
        check(lib().mlb_session_reset(self._h))

    def set_stop_token(self, token_id: int):
        """A sequence that picks this id is appended it and takes no further step (-1: none)."""
        check(lib().mlb_session_set_stop_token(self._h, int(token_id)))

    def stopped(self) -> np.ndarray:
        out = np.zeros(self.batch, dtype=np.int32)
        check(lib().mlb_session_stopped(self._h, _ptr(out, C.c_int32)))
        return out

    def prefill(self, prompts: Sequence[Sequence[int]]):
        assert len(prompts) == self.batch
        lens = _i32([len(p) for p in prompts])
        stride = max(1, int(lens.max()) if len(lens) else 1)
        toks = np.zeros((self.batch, stride), dtype=np.int32)
        for b, p in enumerate(prompts):
            toks[b, :len(p)] = p
        check(lib().mlb_prefill(self._h, _ptr(toks, C.c_int32), _ptr(lens, C.c_int32), stride))

    def score(self, tokens: Sequence[int]) -> np.ndarray:
        """Logits [len][V] of every position of one token sequence (teacher-forced forward)."""
        t = _i32(tokens)
        out = np.empty((len(t), self.model.config.vocab), dtype=np.float32)
        check(lib().mlb_score_tokens(self._h, _ptr(t, C.c_int32), len(t), _ptr(out, C.c_float)))
        return out

    def decode_step(self, sampling: Optional[dict] = None, in_tokens=None) -> np.ndarray:
        out = np.empty(self.batch, dtype=np.int32)
        sp, keep = _sampling(sampling, self.batch)
        it = _i32(in_tokens) if in_tokens is not None else None
        check(lib().mlb_decode_step(self._h, C.byref(sp) if sp else None,
                                    _ptr(it, C.c_int32) if it is not None else None, _ptr(out, C.c_int32)))
        return out

    def decode(self, n: int, sampling: Optional[dict] = None) -> np.ndarray:
        out = np.empty((self.batch, n), dtype=np.int32)
        sp, keep = _sampling(sampling, self.batch)
        check(lib().mlb_decode_n(self._h, C.byref(sp) if sp else None, n, _ptr(out, C.c_int32)))
        return out

    def decode_timed(self, n: int, flush_l2: bool, sampling: Optional[dict] = None):
        out = np.empty((self.batch, n), dtype=np.int32)
        ms = np.empty(n, dtype=np.float32)
        sp, keep = _sampling(sampling, self.batch)
        total = C.c_float(0.0)
        check(lib().mlb_decode_timed(self._h, C.byref(sp) if sp else None, n, 1 if flush_l2 else 0,
                                     _ptr(ms, C.c_float), C.byref(total), _ptr(out, C.c_int32)))
        self.last_total_ms = float(total.value)
        return ms, out

    def profile(self, n: int, flush_l2: bool, sampling: Optional[dict] = None) -> List[dict]:
        stats = (KernelStat * 32)()
        cnt = C.c_int(0)
        sp, keep = _sampling(sampling, self.batch)
        check(lib().mlb_profile_decode(self._h, C.byref(sp) if sp else None, n, 1 if flush_l2 else 0,
                                       stats, 32, C.byref(cnt)))
        return [{"name": stats[i].name.decode(), "launches": stats[i].launches, "total_ms": stats[i].total_ms,
                 "bytes": int(stats[i].bytes), "flops": int(stats[i].flops)} for i in range(cnt.value)]

    def logits(self) -> np.ndarray:
        out = np.empty((self.batch, self.model.config.vocab), dtype=np.float32)
        check(lib().mlb_get_logits(self._h, _ptr(out, C.c_float)))
        return out

    def probs_col(self, seq: int = 0) -> np.ndarray:
        out = np.empty(self.model.config.vocab, dtype=np.float32)
        check(lib().mlb_get_probs_col(self._h, seq, _ptr(out, C.c_float)))
        return out

    def positions(self) -> np.ndarray:
        out = np.empty(self.batch, dtype=np.int32)
        check(lib().mlb_session_positions(self._h, _ptr(out, C.c_int32)))
        return out

    def step_bytes(self) -> dict:
        w, k, s, r = C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_uint64()
        check(lib().mlb_session_step_bytes(self._h, C.byref(w), C.byref(k), C.byref(s), C.byref(r)))
        return {"weights": w.value, "kv": k.value, "state": s.value, "rows": r.value,
                "total": w.value + k.value + s.value + r.value}

    def launches_per_step(self) -> int:
        return check(lib().mlb_session_launches_per_step(self._h))

    def grid_trace(self) -> np.ndarray:
        """[CTAs][256] trace events of the last single-kernel step (MLB_GRID_TIMERS=1), else empty."""
        buf = np.zeros(1024 * 256, dtype=np.int64)
        n = check(lib().mlb_session_grid_trace(self._h, _ptr(buf, C.c_longlong), buf.size))
        return buf[:n * 256].reshape(n, 256).copy()

    def grid_timers(self) -> np.ndarray:
        """[CTAs][20] cycle counters of the single-kernel step (MLB_GRID_TIMERS=1), else empty."""
        buf = np.zeros(1024 * 32, dtype=np.int64)
        n = check(lib().mlb_session_grid_timers(self._h, _ptr(buf, C.c_longlong), buf.size))
        return buf[:n * 32].reshape(n, 32).copy()

    def close(self):
        if self._h:
            lib().mlb_session_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Pool:
    """`batch` independent sequences sharded over several GPUs of one box (mlb_pool_*)."""

    def __init__(self, path: str, devices: Sequence[int], batch: int, max_context: int = 0, override: Optional[Config] = None):
        self._h = C.c_void_p()
        self.batch = batch
        dev = _i32(list(devices))
        check(lib().mlb_pool_new(path.encode(), _ptr(dev, C.c_int32), len(dev), batch, max_context,
                                 C.byref(override) if override is not None else None, C.byref(self._h)))

    def shards(self) -> List[tuple]:
        d, b, e = (np.zeros(64, dtype=np.int32) for _ in range(3))
        n = check(lib().mlb_pool_shards(self._h, _ptr(d, C.c_int32), _ptr(b, C.c_int32), _ptr(e, C.c_int32), 64))
        return [(int(d[i]), int(b[i]), int(e[i])) for i in range(n)]

    def set_stop_token(self, token_id: int):
        check(lib().mlb_pool_set_stop_token(self._h, int(token_id)))

    def prefill(self, prompts: Sequence[Sequence[int]]):
        assert len(prompts) == self.batch
        lens = _i32([len(p) for p in prompts])
        stride = max(1, int(lens.max()))
        toks = np.zeros((self.batch, stride), dtype=np.int32)
        for i, p in enumerate(prompts):
            toks[i, :len(p)] = p
        check(lib().mlb_pool_prefill(self._h, _ptr(toks, C.c_int32), _ptr(lens, C.c_int32), stride))

    def decode(self, n: int, sampling: Optional[dict] = None) -> np.ndarray:
        out = np.empty((self.batch, n), dtype=np.int32)
        sp, keep = _sampling(sampling, self.batch)
        check(lib().mlb_pool_decode_n(self._h, C.byref(sp) if sp else None, n, _ptr(out, C.c_int32)))
        return out

    def close(self):
        if self._h:
            lib().mlb_pool_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def shard_range_c(n_items: int, n_shards: int, shard: int) -> tuple:
    b, e = C.c_int32(), C.c_int32()
    check(lib().mlb_shard_range(n_items, n_shards, shard, C.byref(b), C.byref(e)))
    return b.value, e.value


class KvAllocator:
    """Host-only page allocator of the KV cache (needs no GPU)."""

    def __init__(self, num_pages: int, batch: int, max_pages_per_seq: int):
        self._h = C.c_void_p()
        check(lib().mlb_kv_alloc_new(num_pages, batch, max_pages_per_seq, C.byref(self._h)))

    def ensure(self, seq: int, n_positions: int, block: int = 16) -> int:
        return lib().mlb_kv_alloc_ensure(self._h, seq, n_positions, block)

    def table(self, seq: int) -> List[int]:
        buf = np.empty(4096, dtype=np.int32)
        n = check(lib().mlb_kv_alloc_table(self._h, seq, _ptr(buf, C.c_int32), buf.size))
        return buf[:n].tolist()

    def free_pages(self) -> int:
        return check(lib().mlb_kv_alloc_free_pages(self._h))

    def release(self, seq: int):
        lib().mlb_kv_alloc_release(self._h, seq)

    def __del__(self):
        try:
            if self._h:
                lib().mlb_kv_alloc_free(self._h)
        except Exception:
            pass
