"""TEST INFRASTRUCTURE - CPU oracle (fp32, PyTorch on host cores) for the decode path.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this package; the product never does.

What is restated from the reference, and where it comes from:

* block / final norm / tied LM head / vocab softmax:
  pytorch_verification/pyTorch_gradient_verification.py:133-319, with the operation
  order of the CUDA forward where the two differ (inference.cu:93-94 divides by
  sqrt(mean+eps) then multiplies by the gain; inference.cu:154 divides the scores
  by sqrtf(headDim); inference.cu:270 computes silu as v/(1+expf(-v)))
* per-head QK RMS norm: inference.cu:52-81, :97-111, :467-474 (gains are dim long)
* sigmoid query gating: inference.cu:241-250, :486-508, :575-579
* RoPE table: inference.cu:364-374 (adjacent pairs, host float math)
* layer order (block N-1 first): inference.cu:384-385
* greedy pick: inference_orchestrator.cu:74-84, :112 (argmax; lowest index on ties)

What has NO counterpart in the reference and is defined here (parity unpinned by the
reference; the CUDA kernels are held to these definitions): per-layer embeddings,
gated delta-net layers, grouped-query attention, bf16 / FP8-e4m3 weight rounding, bf16
KV cache, temperature/top-k sampling with Philox4x32-10.

Pinning: tests/golden/make_reference_golden.py runs the reference's own PyTorch script
unchanged and stores its logits; tests/test_oracle_pin.py holds `full_forward` and
`DecodeOracle` to those vectors.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import numpy as np
import torch

ATTENTION = "attention"
DELTA_NET = "delta_net"
DN_L2_EPS = 1e-6


def _t(a) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))


def round_bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32)


def quantize_fp8_rows(w: torch.Tensor):
    """Per-output-row e4m3: scale = max|row| / 448, code = rne(row / scale)."""
    amax = w.abs().amax(dim=1)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    codes = (w / scale[:, None]).to(torch.float8_e4m3fn)
    return codes.to(torch.float32), scale


_libm = None


def _libm_f32(name):
    """float32 libm entry (powf / cosf / sinf): the reference builds its table with these on
    the host (inference.cu:369-371); numpy's own float32 routines differ by an ulp or two."""
    global _libm
    import ctypes
    import ctypes.util
    if _libm is None:
        _libm = ctypes.CDLL(ctypes.util.find_library("m") or "libm.so.6")
    fn = getattr(_libm, name)
    fn.restype = ctypes.c_float
    fn.argtypes = [ctypes.c_float] * (2 if name == "powf" else 1)
    return fn


def rope_table(max_len: int, head_dim: int, base: float) -> np.ndarray:
    """[max_len, head_dim] interleaved (cos, sin) - inference.cu:364-374 in float32."""
    powf, cosf, sinf = _libm_f32("powf"), _libm_f32("cosf"), _libm_f32("sinf")
    pairs = head_dim // 2
    inv = np.array([powf(float(base), float(np.float32(-2.0) * np.float32(i) / np.float32(head_dim)))
                    for i in range(pairs)], dtype=np.float32)
    pos = np.arange(max_len, dtype=np.float32)[:, None]
    theta = (pos * inv[None, :]).astype(np.float32)
    tab = np.empty((max_len, head_dim), dtype=np.float32)
    flat = theta.ravel()
    tab[:, 0::2] = np.array([cosf(float(t)) for t in flat], dtype=np.float32).reshape(max_len, pairs)
    tab[:, 1::2] = np.array([sinf(float(t)) for t in flat], dtype=np.float32).reshape(max_len, pairs)
    return tab


class OracleWeights:
    """Weights as the device path sees them: rounded/quantised once, then fp32 math."""

    def __init__(self, model: dict, weight_dtype: Optional[str] = None,
                 kv_dtype: Optional[str] = None):
        cfg = dict(model["config"])
        self.cfg = cfg
        self.weight_dtype = weight_dtype or cfg["weight_dtype"]
        self.kv_dtype = kv_dtype or cfg["kv_dtype"]
        self.dim, self.layers = cfg["dim"], cfg["layers"]
        self.heads, self.kv_heads, self.head_dim = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
        self.ffn_dim, self.vocab = cfg["ffn_dim"], cfg["vocab"]
        self.eps = float(cfg["rms_eps"])
        self.qk_norm, self.gating = bool(cfg["qk_norm"]), bool(cfg["query_gating"])
        self.ple_dim = int(cfg["ple_dim"])
        self.dk, self.dv = int(cfg["dn_key_dim"]), int(cfg["dn_value_dim"])
        self.layer_types = list(cfg["layer_types"])
        self.max_context = int(cfg["max_context"])
        self.rope = _t(rope_table(self.max_context, self.head_dim, float(cfg["rope_theta"])))
        self.E = self._mat(model["tokenEmbeddings"])
        self.g_final = _t(model["finalRMSNormGamma"])
        self.blocks = []
        for b, blk in enumerate(model["blocks"]):
            o = {}
            for k, v in blk.items():
                o[k] = _t(v) if v.ndim == 1 else self._mat(v)
            for k, v in model["ext"][b].items():
                # per-layer-embedding tensors stay bf16 under FP8 weights; the delta-net gate
                # rows are part of the fused projection and follow the main weight type
                o[k] = self._mat(v, small=k in ("pleTable", "pleProjection"))
            self.blocks.append(o)

    def _mat(self, a, small: bool = False) -> torch.Tensor:
        w = _t(a)
        if self.weight_dtype == "float32":
            return w
        if self.weight_dtype == "bfloat16" or small:
            return round_bf16(w)
        if self.weight_dtype == "float8_e4m3":
            codes, scale = quantize_fp8_rows(w)
            return codes * scale[:, None]
        raise ValueError(self.weight_dtype)

    def round_kv(self, x: torch.Tensor) -> torch.Tensor:
        return round_bf16(x) if self.kv_dtype == "bfloat16" else x


def _rms(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    r = torch.sqrt((x * x).mean() + eps)
    return (x / r) * g


def _rms_heads(x: torch.Tensor, g: torch.Tensor, heads: int, eps: float) -> torch.Tensor:
    xh = x.view(heads, -1)
    r = torch.sqrt((xh * xh).mean(dim=1, keepdim=True) + eps)
    return ((xh / r).reshape(-1)) * g


def _rope(x: torch.Tensor, row: torch.Tensor, heads: int) -> torch.Tensor:
    xh = x.view(heads, -1, 2)
    cos, sin = row[0::2], row[1::2]
    a, b = xh[:, :, 0], xh[:, :, 1]
    out = torch.stack([cos * a - sin * b, sin * a + cos * b], dim=2)
    return out.reshape(-1)


class SeqState:
    def __init__(self, w: OracleWeights):
        self.pos = 0
        self.K: List[List[torch.Tensor]] = [[] for _ in range(w.layers)]
        self.V: List[List[torch.Tensor]] = [[] for _ in range(w.layers)]
        self.S = [torch.zeros(w.heads, w.dv, w.dk) if t == DELTA_NET else None
                  for t in w.layer_types]


class DecodeOracle:
    """KV-cached single-token step for one sequence at a time."""

    def __init__(self, weights: OracleWeights):
        self.w = weights

    def new_state(self) -> SeqState:
        return SeqState(self.w)

    @torch.no_grad()
    def step(self, st: SeqState, token: int) -> torch.Tensor:
        """Consumes `token` at position st.pos; returns fp32 logits [V] for the next one."""
        w = self.w
        if st.pos >= w.max_context:
            raise IndexError("context full")
        x = w.E[token].clone()
        for i in range(w.layers):
            blk = w.blocks[w.layers - 1 - i]
            if w.ple_dim > 0:
                x = x + blk["pleProjection"] @ blk["pleTable"][token]
            n = _rms(x, blk["rmsGamma"], w.eps)
            if w.layer_types[i] == ATTENTION:
                a = self._attention(st, i, blk, n)
            else:
                a = self._delta_net(st, i, blk, n)
            y = blk["outputProjectionWeights"] @ a + x
            m2 = _rms(y, blk["rmsGamma2"], w.eps)
            u = blk["feedForwardWeights1A"] @ m2
            h = (u / (1.0 + torch.exp(-u))) * (blk["feedForwardWeights1B"] @ m2)
            x = blk["feedForwardWeights2"] @ h + y
        z = _rms(x, w.g_final, w.eps)
        st.pos += 1
        return w.E @ z

    def _attention(self, st, i, blk, n):
        w = self.w
        q = blk["queryWeights"] @ n
        k = blk["keyWeights"] @ n
        v = blk["valueWeights"] @ n
        if w.qk_norm:
            q = _rms_heads(q, blk["queryRMSGamma"], w.heads, w.eps)
            k = _rms_heads(k, blk["keyRMSGamma"], w.kv_heads, w.eps)
        row = w.rope[st.pos]
        q = _rope(q, row, w.heads)
        k = _rope(k, row, w.kv_heads)
        st.K[i].append(w.round_kv(k).view(w.kv_heads, w.head_dim))
        st.V[i].append(w.round_kv(v).view(w.kv_heads, w.head_dim))
        K = torch.stack(st.K[i], dim=1)            # [Hkv, ctx, hd]
        V = torch.stack(st.V[i], dim=1)
        group = w.heads // w.kv_heads
        qh = q.view(w.kv_heads, group, w.head_dim)
        s = torch.einsum("hgd,hcd->hgc", qh, K) / math.sqrt(w.head_dim)
        m = s.amax(dim=2, keepdim=True)
        e = torch.exp(s - m)
        p = e / e.sum(dim=2, keepdim=True)
        a = torch.einsum("hgc,hcd->hgd", p, V).reshape(-1)
        if w.gating:
            c = blk["gatedQueryWeights"] @ n
            a = a * (1.0 / (1.0 + torch.exp(-c)))
        return a

    def _delta_net(self, st, i, blk, n):
        w = self.w
        q = (blk["queryWeights"] @ n).view(w.heads, w.dk)
        k = (blk["keyWeights"] @ n).view(w.heads, w.dk)
        v = (blk["valueWeights"] @ n).view(w.heads, w.dv)
        beta = torch.sigmoid(blk["betaWeights"] @ n)
        alpha = torch.sigmoid(blk["decayWeights"] @ n)
        qn = q / torch.sqrt((q * q).sum(dim=1, keepdim=True) + DN_L2_EPS)
        kn = k / torch.sqrt((k * k).sum(dim=1, keepdim=True) + DN_L2_EPS)
        S = st.S[i] * alpha[:, None, None]
        u = torch.einsum("hvk,hk->hv", S, kn)
        S = S + beta[:, None, None] * torch.einsum("hv,hk->hvk", v - u, kn)
        st.S[i] = S
        return torch.einsum("hvk,hk->hv", S, qn).reshape(-1)


@torch.no_grad()
def full_forward(w: OracleWeights, tokens: Sequence[int]) -> torch.Tensor:
    """The reference's way: one causal forward over ALL positions (runInference(L),
    inference.cu:376-752). Attention-only models. Returns logits [V, L] (column l =
    prediction after token l), the layout of vocabScores_DEVICE."""
    assert all(t == ATTENTION for t in w.layer_types) and w.ple_dim == 0
    L = len(tokens)
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    x = w.E[tok].T.contiguous()                      # [d, L]
    rope = w.rope[:L].T                              # [hd, L]
    cos, sin = rope[0::2], rope[1::2]                # [hd/2, L]
    H, Hkv, hd = w.heads, w.kv_heads, w.head_dim

    def rms_cols(x, g):
        r = torch.sqrt((x * x).mean(dim=0, keepdim=True) + w.eps)
        return (x / r) * g[:, None]

    def rms_heads_cols(x, g, heads):
        xh = x.view(heads, hd, L)
        r = torch.sqrt((xh * xh).mean(dim=1, keepdim=True) + w.eps)
        return (xh / r).reshape(-1, L) * g[:, None]

    def rope_cols(x, heads):
        xp = x.view(heads, hd // 2, 2, L)
        a, b = xp[:, :, 0], xp[:, :, 1]
        return torch.stack([cos * a - sin * b, sin * a + cos * b], dim=2).reshape(-1, L)

    future = torch.tril(torch.ones(L, L), diagonal=-1).bool()   # key row > query col
    for i in range(w.layers):
        blk = w.blocks[w.layers - 1 - i]
        n = rms_cols(x, blk["rmsGamma"])
        q, k, v = blk["queryWeights"] @ n, blk["keyWeights"] @ n, blk["valueWeights"] @ n
        if w.qk_norm:
            q = rms_heads_cols(q, blk["queryRMSGamma"], H)
            k = rms_heads_cols(k, blk["keyRMSGamma"], Hkv)
        q, k = rope_cols(q, H), rope_cols(k, Hkv)
        k, v = w.round_kv(k), w.round_kv(v)
        group = H // Hkv
        kh = k.view(Hkv, hd, L).repeat_interleave(group, dim=0)
        vh = v.view(Hkv, hd, L).repeat_interleave(group, dim=0)
        s = torch.matmul(kh.transpose(1, 2), q.view(H, hd, L)) / math.sqrt(hd)   # [H, key, query]
        s = s.masked_fill(future, float("-inf"))
        p = torch.softmax(s, dim=1)
        a = torch.matmul(vh, p).reshape(H * hd, L)
        if w.gating:
            a = a * (1.0 / (1.0 + torch.exp(-(blk["gatedQueryWeights"] @ n))))
        y = blk["outputProjectionWeights"] @ a + x
        m2 = rms_cols(y, blk["rmsGamma2"])
        u = blk["feedForwardWeights1A"] @ m2
        x = blk["feedForwardWeights2"] @ ((u / (1.0 + torch.exp(-u))) * (blk["feedForwardWeights1B"] @ m2)) + y
    z = rms_cols(x, w.g_final)
    return w.E @ z


# --------------------------------------------------------------------------------------
# Sampling (no counterpart in the reference, which is greedy on the host).
# --------------------------------------------------------------------------------------
_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32_10(counter, key):
    """Philox4x32 with 10 rounds (Salmon et al., SC'11). counter: 4 u32, key: 2 u32."""
    c = [int(v) & 0xFFFFFFFF for v in counter]
    k = [int(v) & 0xFFFFFFFF for v in key]
    for _ in range(10):
        p0, p1 = _M0 * c[0], _M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k = [(k[0] + _W0) & 0xFFFFFFFF, (k[1] + _W1) & 0xFFFFFFFF]
    return c


def philox_uniform(seed: int, position: int) -> float:
    """u in [0,1): key = 64-bit sequence seed, counter = (position of the token being
    drawn, 0, 0, 0); the top 24 bits of the first output word."""
    out = philox4x32_10((position, 0, 0, 0), (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
    return (out[0] >> 8) * (1.0 / 16777216.0)


def greedy(logits) -> int:
    """argmax over logits, lowest index on ties."""
    a = np.asarray(logits, dtype=np.float32)
    return int(np.flatnonzero(a == a.max())[0])


def sample_top_k(logits, temperature: float, top_k: int, seed: int, position: int,
                 return_margin: bool = False):
    """logits/T -> k largest (ties: lowest index) -> softmax over the kept set in fp32
    (sequential sums in descending order) -> inverse CDF with one Philox uniform."""
    a = np.asarray(logits, dtype=np.float32) / np.float32(temperature)
    k = min(int(top_k), a.size)
    order = np.lexsort((np.arange(a.size), -a.astype(np.float64)))[:k]
    vals = a[order]
    e = np.exp((vals - vals[0]).astype(np.float32)).astype(np.float32)
    total = np.float32(0.0)
    cum = np.empty(k, dtype=np.float32)
    for j in range(k):
        total = np.float32(total + e[j])
        cum[j] = total
    u = np.float32(philox_uniform(seed, position))
    target = np.float32(u * total)
    hit = np.flatnonzero(cum > target)
    j = int(hit[0]) if hit.size else k - 1
    if return_margin:
        # distance of the draw from the nearest CDF boundary, relative to the total
        margin = float(np.min(np.abs(cum.astype(np.float64) - float(target))) / float(total))
        return int(order[j]), margin
    return int(order[j])
