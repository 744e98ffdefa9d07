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


def _encode(a: np.ndarray, dtype: str) -> bytes:
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

    def dt_of(a):
        return "float32" if a.ndim == 1 else file_dtype

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
                    ext_list.append({"name": name, "block": b, **meta(ext[name], dt_of(ext[name]))})
                    chunks.append(_encode(ext[name], dt_of(ext[name])))
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
