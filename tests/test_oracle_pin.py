"""CPU: the oracle against the vectors produced by the reference's own PyTorch script
(tests/golden/make_reference_golden.py), and its internal consistency."""
import os
import sys

import numpy as np
import pytest

from helpers import load_oracle, write_model, logits_error
from mini_llm_cuda_b200.model_file import ModelSpec, named_spec, periodic_layer_types
from oracle.decode_oracle import (OracleWeights, DecodeOracle, full_forward, philox4x32_10, philox_uniform,
                                  sample_top_k, greedy)
from oracle.model_bin import read_model_bin

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_reference_golden import SEED_WEIGHTS, golden_spec, golden_tokens  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_pytorch_logits.npz")


@pytest.fixture(scope="module")
def golden_model(tmp_path_factory):
    d = tmp_path_factory.mktemp("golden")
    path = write_model(d, golden_spec(), seed=SEED_WEIGHTS, random_gains=True)
    return path, np.load(GOLDEN)


def test_golden_inputs_regenerate(golden_model):
    _, g = golden_model
    assert np.array_equal(golden_tokens(), g["tokens"])


def test_full_forward_matches_reference_script(golden_model):
    path, g = golden_model
    w = OracleWeights(read_model_bin(path))
    logits = full_forward(w, g["tokens"]).numpy()
    for i, c in enumerate(g["columns"]):
        assert logits_error(logits[:, c], g["logits_columns"][i]) < 1e-5
    assert np.array_equal(logits.argmax(axis=0), g["argmax"])
    m = logits.max(axis=0)
    lse = m + np.log(np.exp(logits - m).sum(axis=0))
    assert np.abs(lse - g["logsumexp"]).max() < 1e-4


def test_incremental_matches_reference_script(golden_model):
    path, g = golden_model
    orc = load_oracle(path)
    st = orc.new_state()
    cols = list(g["columns"])
    for i, t in enumerate(g["tokens"]):
        lg = orc.step(st, int(t)).numpy()
        assert int(lg.argmax()) == int(g["argmax"][i])
        if i in cols:
            assert logits_error(lg, g["logits_columns"][cols.index(i)]) < 1e-5


def test_incremental_equals_full_with_qknorm_gating_gqa(tmp_path):
    spec = ModelSpec(dim=128, layers=3, heads=4, kv_heads=2, head_dim=64, ffn_dim=256, vocab=300,
                     max_context=64, qk_norm=True, query_gating=True)
    path = write_model(tmp_path, spec, seed=5)
    w = OracleWeights(read_model_bin(path))
    toks = np.random.default_rng(0).integers(0, 300, size=40)
    full = full_forward(w, toks).numpy()
    orc = DecodeOracle(w)
    st = orc.new_state()
    for i, t in enumerate(toks):
        lg = orc.step(st, int(t)).numpy()
        assert logits_error(lg, full[:, i]) < 1e-5


def test_philox_known_answers():
    # Random123 known-answer vectors for philox4x32-10
    assert philox4x32_10((0, 0, 0, 0), (0, 0)) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert philox4x32_10((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert philox4x32_10((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0)) == \
        [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]
    u = [philox_uniform(7, p) for p in range(2000)]
    assert 0.0 <= min(u) and max(u) < 1.0 and abs(np.mean(u) - 0.5) < 0.03


def test_sampler_properties():
    rng = np.random.default_rng(0)
    lg = rng.standard_normal(500).astype(np.float32)
    assert sample_top_k(lg, 1.0, 1, 3, 10) == greedy(lg)          # k=1 is greedy
    top50 = set(np.argsort(-lg, kind="stable")[:50].tolist())
    picks = [sample_top_k(lg, 1.0, 50, 3, p) for p in range(300)]
    assert set(picks) <= top50 and len(set(picks)) > 10
    tied = np.zeros(16, dtype=np.float32)
    assert greedy(tied) == 0                                       # lowest index on ties
    assert set(sample_top_k(tied, 1.0, 4, 1, p) for p in range(200)) <= {0, 1, 2, 3}


def test_delta_net_state_recurrence_closed_form(tmp_path):
    """One delta-net layer against the closed form S_t = a S (I - b k k^T) + b v k^T."""
    import torch
    spec = ModelSpec(dim=64, layers=1, heads=2, head_dim=64, ffn_dim=64, vocab=50, max_context=16,
                     layer_types=periodic_layer_types(1, 1))
    path = write_model(tmp_path, spec, seed=2)
    orc = load_oracle(path)
    st = orc.new_state()
    S_ref = torch.zeros(2, 64, 64)
    for t in [3, 7, 11]:
        w = orc.w
        blk = w.blocks[0]
        x = w.E[t]
        n = (x / torch.sqrt((x * x).mean() + w.eps)) * blk["rmsGamma"]
        k = (blk["keyWeights"] @ n).view(2, 64)
        v = (blk["valueWeights"] @ n).view(2, 64)
        kn = k / torch.sqrt((k * k).sum(1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(blk["betaWeights"] @ n)
        alpha = torch.sigmoid(blk["decayWeights"] @ n)
        eye = torch.eye(64)
        for h in range(2):
            S_ref[h] = alpha[h] * S_ref[h] @ (eye - beta[h] * torch.outer(kn[h], kn[h])) + beta[h] * torch.outer(v[h], kn[h])
        orc.step(st, t)
        assert (st.S[0] - S_ref).abs().max() < 1e-6
