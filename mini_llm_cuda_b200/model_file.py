"""Writer for the ``model.bin`` weight container and seeded synthetic models.

The container is the one mini-llm-cuda's loader reads (load_model.cu:286-481,
pytorch_verification/load_model_weights.py:135-351):

    u64 little-endian header length | UTF-8 JSON header | zero pad to the next
    multiple of 8 | tensors packed back to back, row-major, in a FIXED order

The loader consumes tensors positionally (load_model.cu:411-421, :442-450), so
keys and data are emitted in exactly that order: ``tokenEmbeddings``,
``finalRMSNormGamma``, then per block ``rmsGamma, queryWeights, keyWeights,
valueWeights, outputProjectionWeights, rmsGamma2, feedForwardWeights1A,
feedForwardWeights1B, feedForwardWeights2`` followed by ``queryRMSGamma,
keyRMSGamma`` (QK-norm) and ``gatedQueryWeights`` (query gating) when present.
Block 0 is the LAST layer executed (inference.cu:384-385).

Two top-level keys that the reference does not know are appended after
``transformerBlocks`` so that a plain file stays readable by it:

``config``  heads, kv_heads, head_dim, layer_types (execution order), rope_theta,
            rms_eps, qk_norm, query_gating, ple_dim, dn_key_dim, dn_value_dim,
            max_context, weight_dtype, kv_dtype (no tensor data)
``ext``     list of ``{name, block, shape, dtype}`` for tensors the reference has
            no slot for (per-layer-embedding table/projection, delta-net beta and
            decay gate weights); their data follows the last block, in list order.

Tensor dtypes in the file: ``float32``, ``float64`` (reference) and ``bfloat16``.

``read_model_bin`` is the inverse of the writer, and ``convert_model_bin`` turns a file
written for the reference (fp32 / fp64, dims in its ``network_meta.h``) into one that carries
its own ``config`` and, optionally, bf16 tensors:

    python -m mini_llm_cuda_b200.model_file convert model/in.bin model/out.bin \
        --heads 8 --head-dim 64 --file-dtype bfloat16 --weight-dtype bfloat16 --kv-dtype bfloat16
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, field, asdict
from typing import Dict, List, Optional

import numpy as np

ATTENTION = "attention"
DELTA_NET = "delta_net"

BASE_KEYS = (
    "rmsGamma", "queryWeights", "keyWeights", "valueWeights", "outputProjectionWeights",
    "rmsGamma2", "feedForwardWeights1A", "feedForwardWeights1B", "feedForwardWeights2",
)
QK_NORM_KEYS = ("queryRMSGamma", "keyRMSGamma")
GATING_KEYS = ("gatedQueryWeights",)
EXT_NAMES = ("pleTable", "pleProjection", "betaWeights", "decayWeights")


@dataclass
class ModelSpec:
    """Runtime replacement for the compile-time dims of network_meta.h:3-20."""
    dim: int
    layers: int
    heads: int
    head_dim: int
    ffn_dim: int
    vocab: int
    kv_heads: Optional[int] = None          # None: MHA (== heads)
    max_context: int = 1024
    rope_theta: float = 10000.0             # ropeDenomBase
    rms_eps: float = 1e-8                   # inference.cu:48
    qk_norm: bool = False                   # CONFIG_QK_RMS_NORM
    query_gating: bool = False              # CONFIG_QUERY_GATING
    ple_dim: int = 0                        # per-layer embedding width, 0 = off
    layer_types: List[str] = field(default_factory=list)   # execution order
    dn_key_dim: Optional[int] = None        # delta-net per-head key dim (default head_dim)
    dn_value_dim: Optional[int] = None
    weight_dtype: str = "float32"           # device weight type: float32 | bfloat16 | float8_e4m3
    kv_dtype: str = "float32"               # KV cache type: float32 | bfloat16

    def __post_init__(self):
        if self.kv_heads is None:
            self.kv_heads = self.heads
        if not self.layer_types:
            self.layer_types = [ATTENTION] * self.layers
        if self.dn_key_dim is None:
            self.dn_key_dim = self.head_dim
        if self.dn_value_dim is None:
            self.dn_value_dim = self.head_dim
        assert len(self.layer_types) == self.layers
        assert self.heads % self.kv_heads == 0

    def block_type(self, block: int) -> str:
        """Type of file block ``block``; block b runs at execution index layers-1-b."""
        return self.layer_types[self.layers - 1 - block]

    def config_dict(self) -> dict:
        d = asdict(self)
        return {
            "heads": d["heads"], "kv_heads": d["kv_heads"], "head_dim": d["head_dim"],
            "layer_types": d["layer_types"], "rope_theta": d["rope_theta"],
            "rms_eps": d["rms_eps"], "qk_norm": d["qk_norm"], "query_gating": d["query_gating"],
            "ple_dim": d["ple_dim"], "dn_key_dim": d["dn_key_dim"],
            "dn_value_dim": d["dn_value_dim"], "max_context": d["max_context"],
            "weight_dtype": d["weight_dtype"], "kv_dtype": d["kv_dtype"],
        }


def periodic_layer_types(layers: int, period: int) -> List[str]:
    """Delta-net at execution index i iff i % period == period-1 (period 0: none)."""
    if period <= 0:
        return [ATTENTION] * layers
    return [DELTA_NET if i % period == period - 1 else ATTENTION for i in range(layers)]


def block_shapes(spec: ModelSpec, block: int) -> Dict[str, tuple]:
    """Shapes (row-major ``[out, in]``) of the tensors of one file block."""
    d, F = spec.dim, spec.ffn_dim
    if spec.block_type(block) == ATTENTION:
        q_out = spec.heads * spec.head_dim
        kv_out = spec.kv_heads * spec.head_dim
        v_out = kv_out
        o_in = q_out
    else:
        q_out = spec.heads * spec.dn_key_dim
        kv_out = q_out
        v_out = spec.heads * spec.dn_value_dim
        o_in = v_out
    shapes = {
        "rmsGamma": (d,), "queryWeights": (q_out, d), "keyWeights": (kv_out, d),
        "valueWeights": (v_out, d), "outputProjectionWeights": (d, o_in), "rmsGamma2": (d,),
        "feedForwardWeights1A": (F, d), "feedForwardWeights1B": (F, d),
        "feedForwardWeights2": (d, F),
    }
    if spec.block_type(block) == ATTENTION:
        if spec.qk_norm:
            shapes["queryRMSGamma"] = (q_out,)
            shapes["keyRMSGamma"] = (kv_out,)
        if spec.query_gating:
            shapes["gatedQueryWeights"] = (q_out, d)
    return shapes


def ext_shapes(spec: ModelSpec, block: int) -> Dict[str, tuple]:
    out = {}
    if spec.ple_dim > 0:
        out["pleTable"] = (spec.vocab, spec.ple_dim)
        out["pleProjection"] = (spec.dim, spec.ple_dim)
    if spec.block_type(block) == DELTA_NET:
        out["betaWeights"] = (spec.heads, spec.dim)
        out["decayWeights"] = (spec.heads, spec.dim)
    return out


def synth_weights(spec: ModelSpec, seed: int = 0, std: float = 0.02,
                  random_gains: bool = False) -> dict:
    """Seeded synthetic weights: every matrix ~N(0, std) drawn in file order with
    numpy's PCG64 ``default_rng(seed)``; gains 1 (or 1+N(0,0.1) when ``random_gains``,
    which makes the gain paths visible to a parity test); delta-net gate weights
    ~N(0, 1/dim) so that their pre-activations are ~N(0,1)."""
    rng = np.random.default_rng(seed)

    def mat(shape, s=std):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(s)).astype(np.float32)

    def gain(shape):
        if random_gains:
            return (1.0 + 0.1 * rng.standard_normal(shape, dtype=np.float32)).astype(np.float32)
        return np.ones(shape, dtype=np.float32)

    w = {"tokenEmbeddings": mat((spec.vocab, spec.dim)),
         "finalRMSNormGamma": gain((spec.dim,)), "blocks": [], "ext": []}
    for b in range(spec.layers):
        blk = {}
        for name, shape in block_shapes(spec, b).items():
            blk[name] = gain(shape) if len(shape) == 1 else mat(shape)
        w["blocks"].append(blk)
    for b in range(spec.layers):
        ext = {}
        for name, shape in ext_shapes(spec, b).items():
            if name in ("betaWeights", "decayWeights"):
                ext[name] = mat(shape, s=1.0 / np.sqrt(spec.dim))
            else:
                ext[name] = mat(shape)
        w["ext"].append(ext)
    return w


def _to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def _to_e4m3_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3 codes (1 sign, 4 exponent bits with bias 7, 3 mantissa bits; largest finite value 448),
    round to nearest even, saturating: what __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3) returns."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    ax = np.minimum(np.abs(x).astype(np.float64), 448.0)
    mant, exp = np.frexp(ax)                      # ax = mant * 2^exp, mant in [0.5, 1)
    e = exp - 1                                   # ax = (2 mant) * 2^e
    normal = ax >= 2.0 ** -6
    q_n = np.rint((2.0 * mant - 1.0) * 8.0)       # 0..8, ties to even
    carry = q_n == 8
    e_n = np.where(carry, e + 1, e)
    q_n = np.where(carry, 0, q_n)
    code_n = ((e_n + 7).astype(np.int64) << 3) | q_n.astype(np.int64)
    code_s = np.rint(ax * 512.0).astype(np.int64)     # subnormals step 2^-9; 8 is the smallest normal
    code = np.where(normal, code_n, code_s)
    code = np.minimum(code, 0x7E)
    return (code.astype(np.uint8) | sign).astype(np.uint8)


def _e4m3_values() -> np.ndarray:
    v = np.zeros(256, dtype=np.float32)
    for c in range(256):
        e, m = (c >> 3) & 15, c & 7
        mag = np.nan if (e == 15 and m == 7) else (m * 2.0 ** -9 if e == 0 else (1.0 + m / 8.0) * 2.0 ** (e - 7))
        v[c] = -mag if c & 0x80 else mag
    return v


def quantize_fp8_rows(a: np.ndarray):
    """Per-row e4m3 as the loader's device kernel does it: scale = max|row| / 448 in float32 (1 for an all-zero
    row), code = e4m3(row / scale). Returns (codes uint8 [rows][cols], scales float32 [rows])."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    amax = np.abs(a).max(axis=1)
    scale = np.where(amax > 0, amax / np.float32(448.0), np.float32(1.0)).astype(np.float32)
    return _to_e4m3_bits(a / scale[:, None]), scale


def _encode(a: np.ndarray, dtype: str) -> bytes:
    if dtype == "float8_e4m3":
        codes, scale = quantize_fp8_rows(a)
        return codes.tobytes() + scale.astype("<f4").tobytes()
    if dtype == "float32":
        return np.ascontiguousarray(a, dtype="<f4").tobytes()
    if dtype == "float64":
        return np.ascontiguousarray(a, dtype="<f8").tobytes()
    if dtype == "bfloat16":
        return _to_bf16_bits(a).astype("<u2").tobytes()
    raise ValueError(f"unsupported file dtype {dtype}")


def write_model_bin(path: str, spec: ModelSpec, weights: dict, file_dtype: str = "float32",
                    with_config: bool = True) -> None:
    """Write ``weights`` (as made by :func:`synth_weights`) to ``path``.

    ``with_config=False`` writes only what the reference loader understands (no
    ``config``/``ext`` keys); such a file needs heads/head_dim from the caller at load.
    Gains are always written as float32.
    """
    def meta(a, dt):
        return {"shape": [int(s) for s in a.shape], "dtype": dt}

    def dt_of(a, name=""):
        if a.ndim == 1:
            return "float32"
        if file_dtype == "float8_e4m3" and name in ("pleTable", "pleProjection"):
            return "bfloat16"        # the device keeps the per-layer embedding in bf16 under FP8 weights
        return file_dtype

    header = {}
    chunks = []
    header["tokenEmbeddings"] = meta(weights["tokenEmbeddings"], dt_of(weights["tokenEmbeddings"]))
    chunks.append(_encode(weights["tokenEmbeddings"], dt_of(weights["tokenEmbeddings"])))
    header["finalRMSNormGamma"] = meta(weights["finalRMSNormGamma"], "float32")
    chunks.append(_encode(weights["finalRMSNormGamma"], "float32"))
    blocks = []
    for b, blk in enumerate(weights["blocks"]):
        order = [k for k in BASE_KEYS + QK_NORM_KEYS + GATING_KEYS if k in blk]
        assert set(order) == set(blk.keys()), f"unknown tensor in block {b}"
        bm = {}
        for k in order:
            bm[k] = meta(blk[k], dt_of(blk[k]))
            chunks.append(_encode(blk[k], dt_of(blk[k])))
        blocks.append(bm)
    header["transformerBlocks"] = blocks
    if with_config:
        header["config"] = spec.config_dict()
        ext_list = []
        for b, ext in enumerate(weights.get("ext", [])):
            for name in EXT_NAMES:
                if name in ext:
                    ext_list.append({"name": name, "block": b, **meta(ext[name], dt_of(ext[name], name))})
                    chunks.append(_encode(ext[name], dt_of(ext[name], name)))
        header["ext"] = ext_list
    else:
        assert not any(weights.get("ext", [])), "ext tensors need with_config=True"
    hbytes = json.dumps(header).encode("utf-8")
    pad = (8 - ((8 + len(hbytes)) % 8)) % 8
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hbytes)))
        f.write(hbytes)
        f.write(b"\0" * pad)
        for c in chunks:
            f.write(c)


def _decode(buf: bytes, shape, dtype: str) -> np.ndarray:
    n = int(np.prod(shape)) if len(shape) else 1
    if dtype == "float32":
        a = np.frombuffer(buf, dtype="<f4", count=n).astype(np.float32)
    elif dtype == "float64":
        a = np.frombuffer(buf, dtype="<f8", count=n).astype(np.float32)     # narrowed as load_model.cu:81-85 does
    elif dtype == "bfloat16":
        a = (np.frombuffer(buf, dtype="<u2", count=n).astype(np.uint32) << 16).view(np.float32)
    elif dtype == "float8_e4m3":
        rows = int(shape[0])
        codes = np.frombuffer(buf, dtype=np.uint8, count=n)
        scale = np.frombuffer(buf, dtype="<f4", count=rows, offset=n).astype(np.float32)
        a = (_e4m3_values()[codes].reshape(rows, -1) * scale[:, None]).astype(np.float32).reshape(-1)
    else:
        raise ValueError(f"Unsupported dtype: {dtype}")                      # load_model.cu:55-57
    return a.reshape(shape)


_DT_SIZE = {"float32": 4, "float64": 8, "bfloat16": 2}


def read_model_bin(path: str):
    """Inverse of :func:`write_model_bin`: returns ``(header, weights)`` with ``weights`` in the
    dict layout of :func:`synth_weights` (fp32 arrays; ``ext`` present when the file has it).
    Tensors are consumed positionally in header order, as load_model.cu:411-450 does."""
    with open(path, "rb") as f:
        raw = f.read()
    if len(raw) < 8:
        raise ValueError("file shorter than its header length field")
    (hlen,) = struct.unpack_from("<Q", raw, 0)
    if 8 + hlen > len(raw):
        raise ValueError("header length exceeds the file")
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    off = 8 + hlen
    off += (8 - off % 8) % 8

    def take(meta):
        nonlocal off
        shape = [int(x) for x in meta["shape"]]
        if meta["dtype"] == "float8_e4m3":
            nbytes = int(np.prod(shape)) + 4 * shape[0]
        elif meta["dtype"] in _DT_SIZE:
            nbytes = int(np.prod(shape)) * _DT_SIZE[meta["dtype"]]
        else:
            raise ValueError(f"Unsupported dtype: {meta['dtype']}")
        if off + nbytes > len(raw):
            raise ValueError("tensor data exceeds the file")
        a = _decode(raw[off:off + nbytes], shape, meta["dtype"])
        off += nbytes
        return a

    weights = {"tokenEmbeddings": take(header["tokenEmbeddings"]),
               "finalRMSNormGamma": take(header["finalRMSNormGamma"]), "blocks": []}
    for blk in header["transformerBlocks"]:
        weights["blocks"].append({k: take(m) for k, m in blk.items()})
    if "ext" in header:
        weights["ext"] = [dict() for _ in header["transformerBlocks"]]
        for e in header["ext"]:
            weights["ext"][int(e["block"])][e["name"]] = take(e)
    return header, weights


def convert_model_bin(src: str, dst: str, heads: int = 0, head_dim: int = 0, kv_heads: int = 0,
                      file_dtype: str = "", weight_dtype: str = "", kv_dtype: str = "",
                      rope_theta: float = 10000.0, rms_eps: float = 1e-8, max_context: int = 1024) -> ModelSpec:
    """Rewrite ``src`` as a file that carries its own ``config`` (and bf16 or FP8 tensors if asked: with
    ``weight_dtype="float8_e4m3"`` the matrices are quantised here, once, to the e4m3 codes and per-row scales
    the device would otherwise compute at every load, and the file is a quarter of the float32 one).

    A file that already has ``config`` keeps it (``weight_dtype`` / ``kv_dtype`` can still be
    changed). A file written for the reference has none: ``heads`` and ``head_dim`` must be given
    (the reference keeps them in network_meta.h), ``rope_theta``, ``rms_eps`` and ``max_context``
    default to its values (ropeDenomBase 10000, eps 1e-8 of inference.cu:48); QK-norm and query
    gating are recognised by their tensors. Returns the spec written."""
    header, weights = read_model_bin(src)
    E = weights["tokenEmbeddings"]
    blocks = weights["blocks"]
    if "config" in header:
        c = dict(header["config"])
        spec = ModelSpec(dim=int(E.shape[1]), layers=len(blocks), heads=int(c["heads"]), head_dim=int(c["head_dim"]),
                         ffn_dim=int(blocks[0]["feedForwardWeights1A"].shape[0]), vocab=int(E.shape[0]),
                         kv_heads=int(c.get("kv_heads", c["heads"])), max_context=int(c.get("max_context", max_context)),
                         rope_theta=float(c.get("rope_theta", rope_theta)), rms_eps=float(c.get("rms_eps", rms_eps)),
                         qk_norm=bool(c.get("qk_norm", False)), query_gating=bool(c.get("query_gating", False)),
                         ple_dim=int(c.get("ple_dim", 0)), layer_types=list(c.get("layer_types", [])),
                         dn_key_dim=c.get("dn_key_dim"), dn_value_dim=c.get("dn_value_dim"),
                         weight_dtype=c.get("weight_dtype", "float32"), kv_dtype=c.get("kv_dtype", "float32"))
    else:
        if heads <= 0 or head_dim <= 0:
            raise ValueError("a file without 'config' needs heads and head_dim (network_meta.h of the build that wrote it)")
        spec = ModelSpec(dim=int(E.shape[1]), layers=len(blocks), heads=heads, head_dim=head_dim,
                         ffn_dim=int(blocks[0]["feedForwardWeights1A"].shape[0]), vocab=int(E.shape[0]),
                         kv_heads=kv_heads or heads, max_context=max_context, rope_theta=rope_theta, rms_eps=rms_eps,
                         qk_norm="queryRMSGamma" in blocks[0], query_gating="gatedQueryWeights" in blocks[0])
    if weight_dtype:
        spec.weight_dtype = weight_dtype
    if kv_dtype:
        spec.kv_dtype = kv_dtype
    if not file_dtype:
        file_dtype = "float8_e4m3" if spec.weight_dtype == "float8_e4m3" else "float32"
    write_model_bin(dst, spec, weights, file_dtype=file_dtype, with_config=True)
    return spec


def _main(argv) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="python -m mini_llm_cuda_b200.model_file")
    sub = ap.add_subparsers(dest="cmd", required=True)
    cv = sub.add_parser("convert", help="rewrite a model.bin with an embedded config, optionally as bf16")
    cv.add_argument("src")
    cv.add_argument("dst")
    cv.add_argument("--heads", type=int, default=0)
    cv.add_argument("--head-dim", type=int, default=0)
    cv.add_argument("--kv-heads", type=int, default=0)
    cv.add_argument("--file-dtype", default="", choices=["", "float32", "float64", "bfloat16", "float8_e4m3"],
                    help="tensor type in the file; default: float8_e4m3 codes with per-row scales when --weight-dtype is float8_e4m3, else float32")
    cv.add_argument("--weight-dtype", default="", choices=["", "float32", "bfloat16", "float8_e4m3"])
    cv.add_argument("--kv-dtype", default="", choices=["", "float32", "bfloat16"])
    cv.add_argument("--rope-theta", type=float, default=10000.0)
    cv.add_argument("--rms-eps", type=float, default=1e-8)
    cv.add_argument("--max-context", type=int, default=1024)
    a = ap.parse_args(argv)
    spec = convert_model_bin(a.src, a.dst, a.heads, a.head_dim, a.kv_heads, a.file_dtype, a.weight_dtype, a.kv_dtype,
                             a.rope_theta, a.rms_eps, a.max_context)
    print(json.dumps(spec.config_dict()))
    return 0


# The configurations the decode path is measured and checked on.
def named_spec(name: str) -> ModelSpec:
    if name == "cfg0":      # CPU-runnable tiny model, fp32
        return ModelSpec(dim=256, layers=4, heads=4, head_dim=64, ffn_dim=768, vocab=4096,
                         max_context=256, rms_eps=1e-5, ple_dim=32,
                         layer_types=periodic_layer_types(4, 2))
    if name == "cfg1":      # 1-GPU latency path, bf16
        return ModelSpec(dim=512, layers=8, heads=8, head_dim=64, ffn_dim=1408, vocab=8192,
                         max_context=1024, rms_eps=1e-5, ple_dim=64,
                         layer_types=periodic_layer_types(8, 4),
                         weight_dtype="bfloat16", kv_dtype="bfloat16")
    if name == "cfg1_ref":  # the sub-model the reference can execute: fp32, all attention, MHA
        return ModelSpec(dim=512, layers=8, heads=8, head_dim=64, ffn_dim=1408, vocab=8192,
                         max_context=1024, rms_eps=1e-8, qk_norm=True, query_gating=True)
    if name == "cfg3":      # gated-delta-net stress
        return ModelSpec(dim=1024, layers=12, heads=8, head_dim=128, ffn_dim=2816, vocab=8192,
                         max_context=4224, rms_eps=1e-5, layer_types=periodic_layer_types(12, 1),
                         weight_dtype="bfloat16", kv_dtype="bfloat16")
    if name == "cfg4":      # FP8 larger model with GQA
        return ModelSpec(dim=2048, layers=24, heads=16, kv_heads=4, head_dim=128, ffn_dim=5632,
                         vocab=32000, max_context=4096, rms_eps=1e-5, ple_dim=128,
                         layer_types=periodic_layer_types(24, 4),
                         weight_dtype="float8_e4m3", kv_dtype="bfloat16")
    raise KeyError(name)


if __name__ == "__main__":
    import sys
    sys.exit(_main(sys.argv[1:]))
