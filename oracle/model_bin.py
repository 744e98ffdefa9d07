"""TEST INFRASTRUCTURE - CPU reader for the ``model.bin`` container.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this package; the product never does.

Restates pytorch_verification/load_model_weights.py:135-351 (container parsing
:167-185, per-tensor read :188-220, block walk :322-344) with the positional tensor
order of load_model.cu:411-421 / :442-450, plus the ``config`` / ``ext`` keys and the
``bfloat16`` file dtype that the product's loader accepts. Matrices are returned
row-major ``[out, in]`` exactly as stored (``y = W @ x``); the reference's transposes
(load_model.cu:87-108, load_model_weights.py:229-231) only change memory order, not
the mathematical matrix.
"""
from __future__ import annotations

import json
import struct
from typing import Optional

import numpy as np

BASE_KEYS = (
    "rmsGamma", "queryWeights", "keyWeights", "valueWeights", "outputProjectionWeights",
    "rmsGamma2", "feedForwardWeights1A", "feedForwardWeights1B", "feedForwardWeights2",
)
OPTIONAL_KEYS = ("queryRMSGamma", "keyRMSGamma", "gatedQueryWeights")


def _e4m3_values() -> np.ndarray:
    """Value of each of the 256 e4m3 codes: 1 sign, 4 exponent (bias 7), 3 mantissa bits; no infinities."""
    v = np.zeros(256, dtype=np.float32)
    for c in range(256):
        e, m = (c >> 3) & 15, c & 7
        if e == 15 and m == 7:
            x = np.nan
        elif e == 0:
            x = m * 2.0 ** -9
        else:
            x = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        v[c] = -x if c & 0x80 else x
    return v


_E4M3_VALUES = _e4m3_values()


def _read_tensor(buf: bytes, off: int, meta: dict):
    shape = [int(s) for s in meta["shape"]]
    n = int(np.prod(shape)) if shape else 1
    dt = meta["dtype"]
    if dt == "float32":
        a = np.frombuffer(buf, dtype="<f4", count=n, offset=off).astype(np.float32)
        nb = 4 * n
    elif dt == "float64":
        a = np.frombuffer(buf, dtype="<f8", count=n, offset=off).astype(np.float32)
        nb = 8 * n
    elif dt == "bfloat16":
        bits = np.frombuffer(buf, dtype="<u2", count=n, offset=off).astype(np.uint32) << 16
        a = bits.view(np.float32)
        nb = 2 * n
    elif dt == "float8_e4m3":
        # offline-quantised matrix (no counterpart in the reference's loader): e4m3 codes, then one float32
        # scale per row; value = code * scale[row]
        rows = shape[0]
        codes = np.frombuffer(buf, dtype=np.uint8, count=n, offset=off)
        scale = np.frombuffer(buf, dtype="<f4", count=rows, offset=off + n).astype(np.float32)
        a = (_E4M3_VALUES[codes].reshape(rows, -1) * scale[:, None]).astype(np.float32).reshape(-1)
        nb = n + 4 * rows
    else:
        raise ValueError(f"Unsupported dtype: {dt}")      # load_model.cu:55-57
    if off + nb > len(buf):
        raise ValueError("tensor data runs past the end of the file")   # load_model.cu:69-72
    return a.reshape(shape).copy(), off + nb


def read_model_bin(path: str, override: Optional[dict] = None) -> dict:
    """Returns {"config": {...}, "tokenEmbeddings", "finalRMSNormGamma", "blocks": [..],
    "ext": [ {...} per block ]} with float32 numpy arrays."""
    with open(path, "rb") as f:
        buf = f.read()
    if len(buf) < 8:
        raise ValueError("file too short")
    (hlen,) = struct.unpack("<Q", buf[:8])
    if 8 + hlen > len(buf):
        raise ValueError("Header length exceeds file size")    # load_model.cu:329-333
    header = json.loads(buf[8:8 + hlen].decode("utf-8"))
    off = 8 + hlen
    off += (8 - off % 8) % 8                                   # load_model.cu:341-343
    out = {}
    out["tokenEmbeddings"], off = _read_tensor(buf, off, header["tokenEmbeddings"])
    out["finalRMSNormGamma"], off = _read_tensor(buf, off, header["finalRMSNormGamma"])
    blocks = []
    for bm in header["transformerBlocks"]:
        blk = {}
        for k in BASE_KEYS + OPTIONAL_KEYS:                    # positional order of the C loader
            if k in bm:
                blk[k], off = _read_tensor(buf, off, bm[k])
        blocks.append(blk)
    out["blocks"] = blocks
    ext = [dict() for _ in blocks]
    for e in header.get("ext", []):
        ext[int(e["block"])][e["name"]], off = _read_tensor(buf, off, e)
    out["ext"] = ext
    cfg = dict(header.get("config", {}))
    if override:
        cfg.update(override)
    V, d = out["tokenEmbeddings"].shape
    cfg.setdefault("layer_types", ["attention"] * len(blocks))
    cfg["dim"], cfg["vocab"], cfg["layers"] = int(d), int(V), len(blocks)
    cfg["ffn_dim"] = int(blocks[0]["feedForwardWeights1A"].shape[0]) if blocks else 0
    if "heads" not in cfg or "head_dim" not in cfg:
        raise ValueError("heads/head_dim are not derivable from tensor shapes: "
                         "the file needs a 'config' key or the caller an override")
    cfg.setdefault("kv_heads", cfg["heads"])
    cfg.setdefault("rope_theta", 10000.0)
    cfg.setdefault("rms_eps", 1e-8)
    cfg.setdefault("qk_norm", any("queryRMSGamma" in b for b in blocks))
    cfg.setdefault("query_gating", any("gatedQueryWeights" in b for b in blocks))
    cfg.setdefault("ple_dim", 0)
    cfg.setdefault("dn_key_dim", cfg["head_dim"])
    cfg.setdefault("dn_value_dim", cfg["head_dim"])
    cfg.setdefault("max_context", 1024)
    cfg.setdefault("weight_dtype", "float32")
    cfg.setdefault("kv_dtype", "float32")
    out["config"] = cfg
    return out
