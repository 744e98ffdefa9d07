"""Shared helpers of the parity tests: seeded models on disk, oracle roll-outs, the error
metric."""
import os

import numpy as np

from mini_llm_cuda_b200.model_file import ModelSpec, synth_weights, write_model_bin
from oracle.decode_oracle import DecodeOracle, OracleWeights, greedy, sample_top_k
from oracle.model_bin import read_model_bin

# Tolerances stated by the task: logits within 1e-3 relative for fp32, 2e-2 for bf16 / FP8.
TOL_FP32 = 1e-3
TOL_LOWP = 2e-2


def logits_error(got, want) -> float:
    """Largest |got - want| relative to the largest |want| of the same logit vector.

    A per-element relative error is meaningless for logits that cross zero; normalising by the
    vector's largest magnitude is the strictest scale-free form that stays finite."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    scale = np.abs(want).max(axis=-1, keepdims=True)
    return float((np.abs(got - want) / np.maximum(scale, 1e-30)).max())


def write_model(tmpdir, spec: ModelSpec, seed=0, random_gains=True, file_dtype="float32", name="m.bin",
                with_config=True):
    weights = synth_weights(spec, seed=seed, random_gains=random_gains)
    path = os.path.join(str(tmpdir), name)
    write_model_bin(path, spec, weights, file_dtype=file_dtype, with_config=with_config)
    return path


def load_oracle(path, override=None) -> DecodeOracle:
    return DecodeOracle(OracleWeights(read_model_bin(path, override)))


def random_prompts(vocab, lens, seed=1):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).astype(np.int32).tolist() for n in lens]


def oracle_rollout(oracle: DecodeOracle, prompt, n_new, sampling=None, seed=0):
    """Greedy (or sampled) continuation; returns (tokens [n_new], logits [n_new, V])."""
    st = oracle.new_state()
    logits = None
    for t in prompt:
        logits = oracle.step(st, int(t))
    toks, all_logits = [], []
    for _ in range(n_new):
        lg = logits.numpy()
        all_logits.append(lg)
        if sampling is None:
            nxt = greedy(lg)
        else:
            nxt = sample_top_k(lg, sampling["temperature"], sampling["top_k"], seed, st.pos)
        toks.append(nxt)
        if st.pos >= oracle.w.max_context:
            break
        logits = oracle.step(st, nxt)
    return np.array(toks, dtype=np.int32), np.stack(all_logits)
