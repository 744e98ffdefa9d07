"""GPU parity: the CUDA decode path, called through the C ABI, against the CPU oracle and
against the logits of the reference's own PyTorch script. Integer results (token ids) must be
identical; logits within 1e-3 (fp32) / 2e-2 (bf16, FP8) of the oracle, in the metric of
helpers.logits_error."""
import dataclasses
import os
import sys

import numpy as np
import pytest

from helpers import (TOL_FP32, TOL_LOWP, load_oracle, logits_error, oracle_rollout, random_prompts,
                     write_model)
from mini_llm_cuda_b200.model_file import ModelSpec, named_spec, periodic_layer_types
from oracle.decode_oracle import sample_top_k

pytestmark = pytest.mark.gpu

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_reference_golden import SEED_WEIGHTS, golden_spec  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_pytorch_logits.npz")


@pytest.fixture(scope="module")
def api(built_lib):
    from mini_llm_cuda_b200 import api as _api
    return _api


def small(**kw) -> ModelSpec:
    base = dict(dim=128, layers=3, heads=2, head_dim=64, ffn_dim=256, vocab=512, max_context=128, rms_eps=1e-5)
    base.update(kw)
    return ModelSpec(**base)


SPECS = {
    "attn_fp32": small(),
    "qknorm_gating": small(qk_norm=True, query_gating=True, rms_eps=1e-8),
    "ple": small(ple_dim=32),
    "delta_only": small(layer_types=periodic_layer_types(3, 1)),
    "mixed_ple": small(layers=4, ple_dim=32, layer_types=periodic_layer_types(4, 2)),
    "gqa": small(dim=256, heads=4, kv_heads=2, query_gating=True),
    "gqa8": small(dim=256, heads=8, kv_heads=1, qk_norm=True),
    "hd128": small(dim=256, heads=2, head_dim=128, qk_norm=True),
    "dn128": small(dim=256, heads=2, head_dim=128, layer_types=periodic_layer_types(3, 1)),
    "dn_kv_mixed_dims": small(dim=256, heads=2, head_dim=64, dn_key_dim=128, dn_value_dim=64,
                              layer_types=periodic_layer_types(3, 3)),
    "bf16": small(ple_dim=32, layers=4, layer_types=periodic_layer_types(4, 2), weight_dtype="bfloat16",
                  kv_dtype="bfloat16"),
    "bf16_w_f32_kv": small(weight_dtype="bfloat16", kv_dtype="float32", query_gating=True),
    "bf16_wide_ple": small(dim=1024, heads=16, head_dim=64, ffn_dim=512, layers=2, ple_dim=128,
                           layer_types=periodic_layer_types(2, 2), weight_dtype="bfloat16", kv_dtype="bfloat16"),
    "fp8": small(dim=256, heads=4, kv_heads=2, ple_dim=32, layers=4, layer_types=periodic_layer_types(4, 4),
                 weight_dtype="float8_e4m3", kv_dtype="bfloat16"),
    # widths that end inside a tile: k-blocks of 64 (d = 192 = 3 blocks, ffn 328 = 5.1 blocks, PLE 24), row tiles of
    # 128 (ffn 328, vocabulary 1000, delta-net projection 3 * (2 * 64 + 64) + 6 = 582 rows), QK-norm and gating on
    "odd_bf16": small(dim=192, heads=3, head_dim=64, ffn_dim=328, vocab=1000, ple_dim=24, layers=4, qk_norm=True,
                      query_gating=True, layer_types=periodic_layer_types(4, 2), weight_dtype="bfloat16", kv_dtype="bfloat16"),
    "odd_fp8": small(dim=192, heads=3, head_dim=64, ffn_dim=336, vocab=1000, ple_dim=24, layers=4, qk_norm=True,
                     layer_types=periodic_layer_types(4, 2), weight_dtype="float8_e4m3", kv_dtype="bfloat16"),
}


def tol_of(spec):
    return TOL_FP32 if spec.weight_dtype == "float32" and spec.kv_dtype == "float32" else TOL_LOWP


@pytest.mark.parametrize("path_mode", ["grid", "chain", "chain_thread"])
@pytest.mark.parametrize("name", list(SPECS))
def test_greedy_rollout_matches_oracle(api, tmp_path, monkeypatch, name, path_mode):
    """Batch 1: 20-token prompt, 48 greedy tokens: identical ids, logits within tolerance at
    every step (context crosses three KV pages). Run through the decode paths: the whole-GPU
    single-kernel step, the kernel chain with TMA-streamed GEMVs, the chain with per-thread-load
    GEMVs."""
    monkeypatch.setenv("MLB_DECODE_PATH", "grid" if path_mode == "grid" else "chain")
    monkeypatch.setenv("MLB_GEMV", "thread" if path_mode == "chain_thread" else "auto")
    spec = SPECS[name]
    path = write_model(tmp_path, spec, seed=3)
    oracle = load_oracle(path)
    prompt = random_prompts(spec.vocab, [20], seed=11)[0]
    want_tok, want_logits = oracle_rollout(oracle, prompt, 48)
    model = api.Model(path)
    sess = api.Session(model, 1)
    sess.prefill([prompt])
    got = []
    worst = 0.0
    for i in range(48):
        t = sess.decode_step()
        got.append(int(t[0]))
        worst = max(worst, logits_error(sess.logits()[0], want_logits[i]))
        if got[-1] != want_tok[i]:
            break
    assert worst < tol_of(spec), f"{name}: logits error {worst}"
    assert got == want_tok[:len(got)].tolist() and len(got) == 48
    sess.close()
    model.close()


@pytest.mark.parametrize("name", ["gqa", "qknorm_gating", "bf16", "fp8", "hd128"])
def test_grid_step_long_context_matches_oracle(api, tmp_path, monkeypatch, name):
    """The whole-GPU single-kernel step with a context long enough for several context splits per
    kv head (more than 8 KV pages): 150-token prompt, 40 greedy tokens, sampled tokens afterwards."""
    monkeypatch.setenv("MLB_DECODE_PATH", "grid")
    monkeypatch.setenv("MLB_PREFILL", "step")    # fp32 activations in the prompt too: identical ids are expected
    spec = dataclasses.replace(SPECS[name], max_context=512)
    path = write_model(tmp_path, spec, seed=13)
    oracle = load_oracle(path)
    prompt = random_prompts(spec.vocab, [150], seed=17)[0]
    want_tok, want_logits = oracle_rollout(oracle, prompt, 40)
    model = api.Model(path)
    sess = api.Session(model, 1)
    sess.prefill([prompt])
    assert sess.launches_per_step() == 1
    got = sess.decode(40)[0]
    assert got.tolist() == want_tok.tolist()
    assert logits_error(sess.logits()[0], want_logits[-1]) < tol_of(spec)
    sess.close()
    model.close()


@pytest.mark.parametrize("kv_dtype,prompt_len,pages_per_split", [("bfloat16", 40, 16), ("float32", 40, 16), ("bfloat16", 300, 16),
                                                                  ("bfloat16", 300, 1), ("bfloat16", 200, 2)])
def test_shape_specialised_step_matches_oracle(api, tmp_path, monkeypatch, kv_dtype, prompt_len, pages_per_split):
    """The whole-GPU step with compile-time shapes (the 1-GPU latency configuration's widths: d=512,
    8 heads of 64, ffn 1408, PLE 64, vocab 8192, bf16 weights) on 4 layers, attention and delta-net
    alternating: short and long contexts, few context splits (every CTA combines them) and many (the
    heads' owners combine them)."""
    monkeypatch.setenv("MLB_DECODE_PATH", "lean")
    monkeypatch.setenv("MLB_PREFILL", "step")
    monkeypatch.setenv("MLB_GRID_PAGES_PER_SPLIT", str(pages_per_split))
    spec = ModelSpec(dim=512, layers=4, heads=8, head_dim=64, ffn_dim=1408, vocab=8192, max_context=512, rms_eps=1e-5,
                     ple_dim=64, layer_types=periodic_layer_types(4, 2), weight_dtype="bfloat16", kv_dtype=kv_dtype)
    path = write_model(tmp_path, spec, seed=5)
    oracle = load_oracle(path)
    prompt = random_prompts(spec.vocab, [prompt_len], seed=6)[0]
    want_tok, want_logits = oracle_rollout(oracle, prompt, 24)
    model = api.Model(path)
    sess = api.Session(model, 1)
    sess.prefill([prompt])
    assert sess.launches_per_step() == 1
    got = []
    worst = 0.0
    for i in range(24):
        got.append(int(sess.decode_step()[0]))
        worst = max(worst, logits_error(sess.logits()[0], want_logits[i]))
        if got[-1] != want_tok[i]:
            break
    assert worst < TOL_LOWP, f"logits error {worst}"
    assert got == want_tok[:len(got)].tolist() and len(got) == 24
    sess.close()
    model.close()


@pytest.mark.parametrize("name,batch,path_mode", [("attn_fp32", 3, "chain"),
                                                  ("mixed_ple", 9, "auto"), ("mixed_ple", 7, "chain"),
                                                  ("bf16", 5, "chain"), ("gqa", 17, "auto"),
                                                  ("qknorm_gating", 8, "chain"),
                                                  ("fp8", 4, "chain"), ("mixed_ple", 2, "chain_thread"),
                                                  ("gqa", 4, "chain_thread")])
def test_ragged_batch_matches_oracle(api, tmp_path, monkeypatch, name, batch, path_mode):
    monkeypatch.setenv("MLB_DECODE_PATH", "chain" if path_mode == "chain_thread" else path_mode)
    monkeypatch.setenv("MLB_GEMV", "thread" if path_mode == "chain_thread" else "auto")
    monkeypatch.setenv("MLB_GEMM", "simt")      # fp32 activations: identical ids are expected (the tensor-core path has its own test)
    monkeypatch.setenv("MLB_PREFILL", "step")   # likewise for the prompt (prompt columns have their own test)
    """Ragged prompts (1 .. 37 tokens) in one batch, decode_n in one call: every sequence
    equals its own batch-1 oracle roll-out."""
    spec = SPECS[name]
    path = write_model(tmp_path, spec, seed=4)
    oracle = load_oracle(path)
    lens = [1 + (7 * i) % 37 for i in range(batch)]
    prompts = random_prompts(spec.vocab, lens, seed=5)
    model = api.Model(path)
    sess = api.Session(model, batch)
    sess.prefill(prompts)
    got = sess.decode(24)
    last = sess.logits()
    for b in range(batch):
        want_tok, want_logits = oracle_rollout(oracle, prompts[b], 24)
        assert got[b].tolist() == want_tok.tolist(), f"sequence {b}"
        assert logits_error(last[b], want_logits[-1]) < tol_of(spec)
    assert sess.positions().tolist() == [l - 1 + 24 for l in lens]
    sess.close()
    model.close()


@pytest.mark.parametrize("name,batch,gemm,split", [("bf16", 16, "tc", 0), ("bf16", 40, "tc", 0), ("bf16_w_f32_kv", 24, "tc", 0),
                                                   ("bf16", 5, "auto", 0), ("bf16_w_f32_kv", 9, "auto", 0), ("fp8", 12, "auto", 0),
                                                   ("bf16_wide_ple", 6, "auto", 0), ("bf16", 40, "tc", 8), ("fp8", 12, "auto", 4),
                                                   ("bf16_wide_ple", 6, "auto", 8), ("bf16", 16, "tc", 1), ("odd_bf16", 21, "auto", 0),
                                                   ("odd_bf16", 21, "auto", 4), ("odd_fp8", 37, "auto", 0), ("odd_fp8", 37, "auto", 2)])
def test_tensor_core_batch_path_matches_oracle(api, tmp_path, monkeypatch, name, batch, gemm, split):
    """Batch >= 4 with bf16 weights, or FP8 weights widened to bf16 tile by tile inside the kernel, runs the
    projections as tcgen05 GEMMs on bf16 activations. `split` pins the largest thread-block cluster that may
    share the k-blocks of an output tile (0: the library's choice).
    Teacher-forced on the oracle's tokens: logits within 2e-2 at every step; the device pick equals
    the oracle's wherever the oracle's top-2 margin exceeds that bound."""
    monkeypatch.setenv("MLB_GEMM", gemm)
    if split:
        monkeypatch.setenv("MLB_TC_SPLIT", str(split))
    spec = SPECS[name]
    path = write_model(tmp_path, spec, seed=6)
    oracle = load_oracle(path)
    lens = [1 + (5 * i) % 23 for i in range(batch)]
    prompts = random_prompts(spec.vocab, lens, seed=9)
    steps = 12
    rolls = [oracle_rollout(oracle, prompts[b], steps) for b in range(batch)]
    model = api.Model(path)
    sess = api.Session(model, batch)
    sess.prefill(prompts)
    worst = 0.0
    checked = 0
    for i in range(steps):
        forced = None if i == 0 else [int(rolls[b][0][i - 1]) for b in range(batch)]
        picks = sess.decode_step(in_tokens=forced)
        lg = sess.logits()
        for b in range(batch):
            want = rolls[b][1][i]
            worst = max(worst, logits_error(lg[b], want))
            top2 = np.sort(want)[-2:]
            if (top2[1] - top2[0]) > 2 * TOL_LOWP * np.abs(want).max():
                assert int(picks[b]) == int(rolls[b][0][i]), (i, b)
                checked += 1
    assert worst < TOL_LOWP, worst
    assert checked > batch      # the margin test did not make the check vacuous
    sess.close()
    model.close()


BASELINE_BATCHED = {
    # the batched configuration: the 1-GPU latency model at 256 sequences, temperature 1.0 / top-k 50
    "cfg2": (dict(dim=512, layers=8, heads=8, head_dim=64, ffn_dim=1408, vocab=8192, max_context=128, rms_eps=1e-5, ple_dim=64,
                  layer_types=periodic_layer_types(8, 4), weight_dtype="bfloat16", kv_dtype="bfloat16"), 256, True),
    # the gated-delta-net stress widths (d=1024, 8 heads, key/value dim 128, ffn 2816) at batch 64, 3 of its 12 layers
    "cfg3": (dict(dim=1024, layers=3, heads=8, head_dim=128, ffn_dim=2816, vocab=2048, max_context=128, rms_eps=1e-5,
                  layer_types=periodic_layer_types(3, 1), weight_dtype="bfloat16", kv_dtype="bfloat16"), 64, False),
    # the quantised larger model's widths (d=2048, 16 query / 4 kv heads of 128, ffn 5632, PLE 128, FP8 tiles widened in the GEMM) at batch 64, 2 layers
    "cfg4": (dict(dim=2048, layers=2, heads=16, kv_heads=4, head_dim=128, ffn_dim=5632, vocab=4096, max_context=128, rms_eps=1e-5,
                  ple_dim=128, layer_types=periodic_layer_types(2, 2), weight_dtype="float8_e4m3", kv_dtype="bfloat16"), 64, False),
}


@pytest.mark.parametrize("name", list(BASELINE_BATCHED))
def test_baseline_batched_shapes_match_oracle(api, tmp_path, name):
    """The batched BASELINE configurations at their real batch and widths on the tensor-core step (the tile
    chooser picks other tiles at 64 / 256 sequences than at the small batches of the other tests). A few of
    the sequences are followed by the oracle, teacher-forced on its tokens: logits within 2e-2 at every
    step, greedy picks equal wherever the oracle's margin exceeds that bound; with sampling (the 256-sequence
    configuration) every draw equals the oracle's top-k / Philox draw on the device's own logits."""
    kw, batch, sampled = BASELINE_BATCHED[name]
    spec = ModelSpec(**kw)
    path = write_model(tmp_path, spec, seed=21, random_gains=(name != "cfg4"))
    oracle = load_oracle(path)
    lens = [3 + (11 * i) % 29 for i in range(batch)]
    prompts = random_prompts(spec.vocab, lens, seed=22)
    watch = [0, batch // 3, batch - 1]
    steps = 6
    rolls = {b: oracle_rollout(oracle, prompts[b], steps) for b in watch}
    seeds = [1000 + b for b in range(batch)]
    samp = {"mode": "top_k", "top_k": 50, "temperature": 1.0, "seeds": seeds} if sampled else None
    model = api.Model(path)
    sess = api.Session(model, batch)
    sess.prefill(prompts)
    assert sess.launches_per_step() > 1          # the tensor-core chain, not a batch-1 kernel
    worst, checked, close_calls = 0.0, 0, 0
    prev = None
    for i in range(steps):
        forced = None
        if i > 0:
            forced = [int(rolls[b][0][i - 1]) if b in rolls else int(prev[b]) for b in range(batch)]
        picks = sess.decode_step(samp, in_tokens=forced)
        lg = sess.logits()
        for b in watch:
            want = rolls[b][1][i]
            worst = max(worst, logits_error(lg[b], want))
            if sampled:
                draw, margin = sample_top_k(lg[b], 1.0, 50, seeds[b], lens[b] + i, return_margin=True)
                if int(picks[b]) != draw:
                    assert margin < 1e-5, (i, b, margin)
                    close_calls += 1
                checked += 1
            else:
                top2 = np.sort(want)[-2:]
                if (top2[1] - top2[0]) > 2 * TOL_LOWP * np.abs(want).max():
                    assert int(picks[b]) == int(rolls[b][0][i]), (i, b)
                    checked += 1
        prev = picks
    assert worst < TOL_LOWP, worst
    assert checked >= len(watch) and close_calls <= 1
    sess.close()
    model.close()


@pytest.mark.parametrize("name,lens,decode_path", [("bf16", [131], "chain"), ("bf16", [1, 2, 130, 60, 201, 17], "auto"),
                                                   ("bf16_w_f32_kv", [300, 5, 129], "chain"), ("bf16", [257], "grid"),
                                                   ("fp8", [280, 3, 70], "auto"), ("odd_fp8", [90, 2, 77, 31], "auto"),
                                                   ("odd_bf16", [101, 64], "auto")])
def test_prompt_by_columns_matches_oracle(api, tmp_path, monkeypatch, name, lens, decode_path):
    """The prompt consumed as columns of tensor-core steps (256 per chunk; prompts that end inside a
    chunk, span several, or have a single token), attention and delta-net layers mixed, PLE; FP8
    weights are widened tile by tile inside the GEMMs: the
    decode steps that follow, teacher-forced on the oracle's tokens, give its logits within 2e-2,
    and the positions are those the token loop leaves."""
    monkeypatch.setenv("MLB_PREFILL", "chunk")
    monkeypatch.setenv("MLB_DECODE_PATH", decode_path)
    spec = dataclasses.replace(SPECS[name], max_context=512)
    path = write_model(tmp_path, spec, seed=21)
    oracle = load_oracle(path)
    batch = len(lens)
    prompts = random_prompts(spec.vocab, lens, seed=23)
    steps = 6
    rolls = [oracle_rollout(oracle, prompts[b], steps) for b in range(batch)]
    model = api.Model(path)
    sess = api.Session(model, batch)
    sess.prefill(prompts)
    assert sess.positions().tolist() == [l - 1 for l in lens]
    worst = 0.0
    checked = 0
    for i in range(steps):
        forced = None if i == 0 else [int(rolls[b][0][i - 1]) for b in range(batch)]
        picks = sess.decode_step(in_tokens=forced)
        lg = sess.logits()
        for b in range(batch):
            want = rolls[b][1][i]
            worst = max(worst, logits_error(lg[b], want))
            top2 = np.sort(want)[-2:]
            if (top2[1] - top2[0]) > 2 * TOL_LOWP * np.abs(want).max():
                assert int(picks[b]) == int(rolls[b][0][i]), (i, b)
                checked += 1
    assert worst < TOL_LOWP, worst
    assert checked > 0
    # a second prompt on the same session starts from a clean cache and state
    sess.prefill(prompts)
    sess.decode_step()
    assert max(logits_error(sess.logits()[b], rolls[b][1][0]) for b in range(batch)) < TOL_LOWP
    sess.close()
    model.close()


@pytest.mark.parametrize("name,length", [("bf16", 40), ("bf16", 300), ("bf16_w_f32_kv", 257), ("fp8", 270)])
def test_scoring_forward_matches_oracle(api, tmp_path, name, length):
    """mlb_score_tokens: logits of every position of one sequence (the reference's full forward
    runInference(L)) against the KV-cached oracle fed the same tokens: within 2e-2 at every
    position, identical argmax wherever the oracle's top-2 margin exceeds that bound. One chunk, and
    several chunks with the run of columns continuing across them."""
    spec = dataclasses.replace(SPECS[name], max_context=512)
    path = write_model(tmp_path, spec, seed=31)
    oracle = load_oracle(path)
    tokens = random_prompts(spec.vocab, [length], seed=37)[0]
    st = oracle.new_state()
    want = np.stack([np.asarray(oracle.step(st, int(t))) for t in tokens])
    model = api.Model(path)
    sess = api.Session(model, 2)
    got = sess.score(tokens)
    assert got.shape == want.shape
    worst = max(logits_error(got[i], want[i]) for i in range(length))
    assert worst < TOL_LOWP, worst
    checked = 0
    for i in range(length):
        top2 = np.sort(want[i])[-2:]
        if (top2[1] - top2[0]) > 2 * TOL_LOWP * np.abs(want[i]).max():
            assert int(np.argmax(got[i])) == int(np.argmax(want[i])), i
            checked += 1
    assert checked > length // 4
    # the session is reset: a prompt and a decode step work as on a fresh one
    sess.prefill([tokens[:20], tokens[:7]])
    assert sess.positions().tolist() == [19, 6]
    sess.decode_step()
    sess.close()
    model.close()


@pytest.mark.parametrize("name,step_mode", [("attn_fp32", False), ("mixed_ple", False), ("bf16", True)])
def test_scoring_forward_in_fp32_activations(api, tmp_path, monkeypatch, name, step_mode):
    """mlb_score_tokens on fp32 weights (and, with MLB_SCORE=step, on bf16 weights): the token loop with the
    given ids forced in. Every position within the fp32 bound of the decode path (1e-3), identical argmax -
    the precision the reference's trainer gets from runInference(L)."""
    if step_mode:
        monkeypatch.setenv("MLB_SCORE", "step")
    spec = dataclasses.replace(SPECS[name], max_context=128)
    path = write_model(tmp_path, spec, seed=33)
    oracle = load_oracle(path)
    tokens = random_prompts(spec.vocab, [90], seed=39)[0]
    st = oracle.new_state()
    want = np.stack([np.asarray(oracle.step(st, int(t))) for t in tokens])
    model = api.Model(path)
    sess = api.Session(model, 1)
    got = sess.score(tokens)
    assert got.shape == want.shape
    assert max(logits_error(got[i], want[i]) for i in range(len(tokens))) < TOL_FP32
    assert np.array_equal(got.argmax(axis=1), want.argmax(axis=1))
    sess.prefill([tokens[:20]])                    # the session is reset afterwards
    assert sess.positions().tolist() == [19]
    sess.close()
    model.close()


def test_prompt_by_columns_needs_bf16_weights(api, tmp_path, monkeypatch):
    monkeypatch.setenv("MLB_PREFILL", "chunk")
    spec = SPECS["attn_fp32"]
    path = write_model(tmp_path, spec, seed=2)
    model = api.Model(path)
    sess = api.Session(model, 1)
    with pytest.raises(api.MlbError) as e:
        sess.prefill([random_prompts(spec.vocab, [40], seed=1)[0]])
    assert e.value.status == api.MLB_E_UNSUPPORTED
    sess.close()
    model.close()


def test_reference_script_golden_logits(api, tmp_path):
    """Column L-1 of the reference's [V x L] logits (its PyTorch script, run unchanged) against a
    KV-cached decode of the same 256 tokens: logits within 1e-3, identical argmax at all 256
    positions."""
    g = np.load(GOLDEN)
    spec = golden_spec()
    path = write_model(tmp_path, spec, seed=SEED_WEIGHTS, random_gains=True)
    tokens = g["tokens"].tolist()
    model = api.Model(path)
    sess = api.Session(model, 1)
    sess.prefill([tokens[:1]])
    cols = g["columns"].tolist()
    picks = []
    for i, t in enumerate(tokens):
        out = sess.decode_step(in_tokens=[t])
        picks.append(int(out[0]))
        if i in cols:
            err = logits_error(sess.logits()[0], g["logits_columns"][cols.index(i)])
            assert err < TOL_FP32, f"column {i}: {err}"
    assert picks == g["argmax"].tolist()
    # probabilities of the last column: softmax as the reference's vocab softmax kernels
    probs = sess.probs_col(0)
    lg = g["logits_columns"][cols.index(255)].astype(np.float64)
    want = np.exp(lg - lg.max())
    want /= want.sum()
    assert np.abs(probs - want).max() < 1e-6 and abs(probs.sum() - 1.0) < 1e-4
    # the prompt path (prefill of all 256 tokens at once) reaches the same state
    sess.prefill([tokens])
    out = sess.decode_step()
    assert int(out[0]) == int(g["argmax"][255])
    assert logits_error(sess.logits()[0], g["logits_columns"][cols.index(255)]) < TOL_FP32
    sess.close()
    model.close()


def test_base_file_without_config_needs_override(api, tmp_path):
    """A file in the reference's plain format (no config key): heads/head_dim come from the
    caller, as they come from network_meta.h in the reference."""
    spec = small(qk_norm=True, query_gating=True, rms_eps=1e-8)
    path = write_model(tmp_path, spec, seed=8, with_config=False)
    with pytest.raises(api.MlbError) as e:
        api.Model(path)
    assert e.value.status == api.MLB_E_INVALID
    ov = api.make_override(heads=2, head_dim=64, max_context=128)
    model = api.Model(path, override=ov)
    assert model.config.qk_norm == 1 and model.config.query_gating == 1     # inferred from the keys present
    oracle = load_oracle(path, {"heads": 2, "head_dim": 64, "max_context": 128})
    prompt = random_prompts(spec.vocab, [9], seed=2)[0]
    want_tok, _ = oracle_rollout(oracle, prompt, 16)
    sess = api.Session(model, 1)
    sess.prefill([prompt])
    assert sess.decode(16)[0].tolist() == want_tok.tolist()
    sess.close()
    model.close()


def test_file_dtypes_float64_and_bfloat16(api, tmp_path):
    spec = small()
    prompt = random_prompts(spec.vocab, [6], seed=2)[0]
    p32 = write_model(tmp_path, spec, seed=9, name="f32.bin")
    p64 = write_model(tmp_path, spec, seed=9, file_dtype="float64", name="f64.bin")
    pbf = write_model(tmp_path, spec, seed=9, file_dtype="bfloat16", name="bf.bin")
    outs = {}
    for key, p in (("f32", p32), ("f64", p64), ("bf", pbf)):
        model = api.Model(p)
        sess = api.Session(model, 1)
        sess.prefill([prompt])
        outs[key] = (sess.decode(8)[0].tolist(), sess.logits()[0].copy())
        sess.close()
        model.close()
    assert outs["f32"][0] == outs["f64"][0] and np.array_equal(outs["f32"][1], outs["f64"][1])
    want_tok, want_logits = oracle_rollout(load_oracle(pbf), prompt, 8)
    assert outs["bf"][0] == want_tok.tolist()
    assert logits_error(outs["bf"][1], want_logits[-1]) < TOL_FP32


def test_context_limit_and_errors(api, tmp_path):
    spec = small(max_context=48)
    path = write_model(tmp_path, spec, seed=10)
    model = api.Model(path)
    sess = api.Session(model, 2)
    prompts = random_prompts(spec.vocab, [40, 10], seed=1)
    sess.prefill(prompts)
    out = sess.decode(12)            # sequence 0 has room for 48-39 = 9 more steps
    assert (out[0, :9] >= 0).all() and (out[0, 9:] == -1).all() and (out[1] >= 0).all()
    oracle = load_oracle(path)
    want0, _ = oracle_rollout(oracle, prompts[0], 9)
    want1, _ = oracle_rollout(oracle, prompts[1], 12)
    assert out[0, :9].tolist() == want0.tolist() and out[1].tolist() == want1.tolist()
    with pytest.raises(api.MlbError) as e:
        sess.prefill([list(range(49)), [1]])
    assert e.value.status == api.MLB_E_CONTEXT_FULL
    with pytest.raises(api.MlbError) as e:
        sess.prefill([[spec.vocab], [1]])
    assert e.value.status == api.MLB_E_INVALID
    with pytest.raises(api.MlbError) as e:
        sess.prefill([[], [1]])
    assert e.value.status == api.MLB_E_INVALID
    # a pool too small for the batch: the allocator reports it, nothing is launched
    tiny = api.Session(model, 2, kv_pages=3)
    with pytest.raises(api.MlbError) as e:
        tiny.prefill(random_prompts(spec.vocab, [40, 40], seed=1))
    assert e.value.status == api.MLB_E_KV_FULL
    tiny.close()
    # run to the very end of the context: the last position is usable, then CONTEXT_FULL
    sess.prefill([prompts[1], prompts[1]])
    out = sess.decode(48)
    assert (out[:, :39] >= 0).all() and (out[:, 39:] == -1).all()
    with pytest.raises(api.MlbError) as e:
        sess.decode_step()
    assert e.value.status == api.MLB_E_CONTEXT_FULL
    sess.close()
    model.close()


def test_topk_sampler_matches_oracle_on_device_logits(api, tmp_path):
    """Teacher-forced: at every step the device's draw must equal the oracle's draw from the
    device's own logits (same Philox counter), except where the uniform lands within 1e-5 of a
    CDF boundary."""
    spec = small(vocab=2048)
    path = write_model(tmp_path, spec, seed=12)
    model = api.Model(path)
    batch = 4
    sess = api.Session(model, batch)
    prompts = random_prompts(spec.vocab, [5, 9, 2, 16], seed=3)
    sess.prefill(prompts)
    seeds = [0, 1, 2, 2**40 + 5]
    samp = {"mode": "top_k", "top_k": 50, "temperature": 0.8, "seeds": seeds}
    pos = [len(p) for p in prompts]       # position of the token being drawn
    close_calls = 0
    distinct = set()
    for step in range(40):
        out = sess.decode_step(samp)
        lg = sess.logits()
        for b in range(batch):
            want, margin = sample_top_k(lg[b], 0.8, 50, seeds[b], pos[b] + step, return_margin=True)
            distinct.add(int(out[b]))
            if int(out[b]) != want:
                assert margin < 1e-5, f"step {step} seq {b}: got {out[b]} want {want} margin {margin}"
                close_calls += 1
    assert close_calls <= 2 and len(distinct) > 20
    # k = 1 equals greedy
    sess.prefill(prompts)
    a = sess.decode(8, {"mode": "top_k", "top_k": 1, "temperature": 1.0})
    sess.prefill(prompts)
    b = sess.decode(8)
    assert np.array_equal(a, b)
    sess.close()
    model.close()


def test_sampler_degenerate_ties(api, tmp_path):
    """All-equal logits (zero embedding table): greedy picks id 0, top-k draws stay inside the
    k lowest ids."""
    from mini_llm_cuda_b200.model_file import synth_weights, write_model_bin
    spec = small(vocab=1536)
    w = synth_weights(spec, seed=1)
    w["tokenEmbeddings"][:] = 0.0
    path = os.path.join(str(tmp_path), "z.bin")
    write_model_bin(path, spec, w)
    model = api.Model(path)
    sess = api.Session(model, 1)
    sess.prefill([[3, 4]])
    assert sess.decode(3)[0].tolist() == [0, 0, 0]
    sess.prefill([[3, 4]])
    out = sess.decode(32, {"mode": "top_k", "top_k": 8, "temperature": 1.0, "seeds": [9]})
    assert set(out[0].tolist()) <= set(range(8)) and len(set(out[0].tolist())) > 2
    sess.close()
    model.close()


def test_cfg1_latency_config_bf16(api, tmp_path):
    """The bench configuration (d=512, 8 layers, 2 of them delta-net, PLE 64, V=8192, bf16):
    128-token prompt, 64 greedy tokens."""
    spec = named_spec("cfg1")
    path = write_model(tmp_path, spec, seed=0, random_gains=False)
    oracle = load_oracle(path)
    prompt = random_prompts(spec.vocab, [128], seed=1)[0]
    want_tok, want_logits = oracle_rollout(oracle, prompt, 64)
    model = api.Model(path)
    sess = api.Session(model, 1)
    sess.prefill([prompt])
    got = sess.decode(64)[0]
    assert got.tolist() == want_tok.tolist()
    assert logits_error(sess.logits()[0], want_logits[-1]) < TOL_LOWP
    nbytes = sess.step_bytes()
    assert nbytes["weights"] == model.weight_bytes and nbytes["kv"] > 0 and nbytes["state"] > 0
    ms, _ = sess.decode_timed(4, True)
    assert (ms > 0).all()
    stats = sess.profile(2, False)
    names = {s["name"] for s in stats}
    assert names in ({"lean_decode_step"}, {"grid_decode_step"}) or names >= {"qkv_gemv_norm_rope_kvappend", "attn_flash_decode_paged",
                                                         "deltanet_state_update", "lmhead_gemv_norm_argmax"}
    sess.close()
    model.close()


@pytest.mark.parametrize("path_mode", ["chain", "grid"])
def test_cfg4_dims_fp8_gqa_reduced_depth(api, tmp_path, monkeypatch, path_mode):
    """The quantised larger configuration at its real widths (d=2048, 16 query / 4 kv heads of 128,
    ffn 5632, PLE 128, FP8 e4m3 weights with per-row scales, bf16 KV) with 4 of its 24 layers and
    a 4096-token vocabulary so that the CPU oracle finishes in seconds."""
    monkeypatch.setenv("MLB_DECODE_PATH", path_mode)
    spec = ModelSpec(dim=2048, layers=4, heads=16, kv_heads=4, head_dim=128, ffn_dim=5632, vocab=4096, max_context=256,
                     rms_eps=1e-5, ple_dim=128, layer_types=periodic_layer_types(4, 4), weight_dtype="float8_e4m3",
                     kv_dtype="bfloat16")
    path = write_model(tmp_path, spec, seed=0, random_gains=False)
    oracle = load_oracle(path)
    prompt = random_prompts(spec.vocab, [40], seed=1)[0]
    want_tok, want_logits = oracle_rollout(oracle, prompt, 12)
    model = api.Model(path)
    sess = api.Session(model, 1)
    sess.prefill([prompt])
    got = sess.decode(12)[0]
    assert got.tolist() == want_tok.tolist()
    assert logits_error(sess.logits()[0], want_logits[-1]) < TOL_LOWP
    sess.close()
    model.close()


def test_cfg0_fp32_64_greedy(api, tmp_path):
    """Config 0 (the CPU-runnable case): d=256, 4 layers alternating attention / delta-net,
    PLE 32, V=4096, fp32; 32-token prompt from seed 1, 64 greedy tokens, max context 256."""
    spec = named_spec("cfg0")
    path = write_model(tmp_path, spec, seed=0, random_gains=False)
    oracle = load_oracle(path)
    prompt = random_prompts(spec.vocab, [32], seed=1)[0]
    want_tok, want_logits = oracle_rollout(oracle, prompt, 64)
    model = api.Model(path)
    sess = api.Session(model, 1)
    sess.prefill([prompt])
    got = []
    for i in range(64):
        got.append(int(sess.decode_step()[0]))
        assert logits_error(sess.logits()[0], want_logits[i]) < TOL_FP32
    assert got == want_tok.tolist()
    sess.close()
    model.close()


@pytest.mark.parametrize("weight_dtype,batch", [("float32", 1), ("float32", 2), ("bfloat16", 1), ("bfloat16", 4)])
def test_stop_token_takes_a_sequence_out_of_the_batch(api, tmp_path, weight_dtype, batch):
    """A sequence that picks the session's stop token keeps it and takes no further step; the other sequences
    of the batch are not disturbed. Checked against the same session's free run (and, for fp32, the oracle)
    on the single-kernel step (batch 1), the GEMV chain (batch 2) and the tensor-core step (batch 4)."""
    spec = small(layers=4, layer_types=periodic_layer_types(4, 2), ple_dim=64 if weight_dtype == "bfloat16" else 32,
                 weight_dtype=weight_dtype, kv_dtype="bfloat16" if weight_dtype == "bfloat16" else "float32")
    path = write_model(tmp_path, spec, seed=31)
    prompts = random_prompts(spec.vocab, [9 + 5 * b for b in range(batch)], seed=32)
    n = 24
    model = api.Model(path)
    sess = api.Session(model, batch)
    sess.prefill(prompts)
    free = sess.decode(n)                                  # [batch][n], no stop token
    if weight_dtype == "float32":
        oracle = load_oracle(path)
        for b in range(batch):
            assert free[b].tolist() == oracle_rollout(oracle, prompts[b], n)[0].tolist()
    stop = int(free[batch - 1][7])                         # the last sequence draws it at step 7 (or earlier)
    first = [next((i for i, t in enumerate(free[b].tolist()) if t == stop), None) for b in range(batch)]
    assert first[batch - 1] is not None and first[batch - 1] <= 7
    sess.set_stop_token(stop)
    sess.prefill(prompts)
    assert not sess.stopped().any()
    part = sess.decode(10)                                 # the stop survives a call boundary
    if sess.stopped().all():
        with pytest.raises(api.MlbError):
            sess.decode(n - 10)
        got = np.concatenate([part, np.full((batch, n - 10), -1, dtype=part.dtype)], axis=1)
    else:
        got = np.concatenate([part, sess.decode(n - 10)], axis=1)
    for b in range(batch):
        k = n if first[b] is None else first[b] + 1
        assert got[b][:k].tolist() == free[b][:k].tolist(), b
        assert (got[b][k:] == -1).all(), b
        assert int(sess.stopped()[b]) == (0 if first[b] is None else 1)
        assert int(sess.positions()[b]) == len(prompts[b]) - 1 + k
    live = [b for b in range(batch) if first[b] is None]
    if live:
        nxt = sess.decode_step()                           # the one-token call skips the ended sequences too
        assert all(int(nxt[b]) == -1 for b in range(batch) if b not in live) and all(int(nxt[b]) >= 0 for b in live)
    else:
        with pytest.raises(api.MlbError):
            sess.decode_step()
    # a new prompt starts every sequence again; without a stop token the free run comes back
    sess.set_stop_token(-1)
    sess.prefill(prompts)
    assert np.array_equal(sess.decode(n), free)
    sess.close()
    model.close()


@pytest.mark.parametrize("devices", [[0, 0, 0], [0, 1]])
def test_pool_shards_sequences_over_devices(api, tmp_path, devices):
    """mlb_pool_*: the sequences of one batch served by several (model, session, host thread) triples give the
    ids one session gives for the whole batch, greedy and sampled, and a stop token reaches every shard.
    [0, 0, 0] runs three shards on one GPU (uneven: 7 sequences as 3 + 2 + 2); [0, 1] needs two GPUs."""
    import torch
    if max(devices) >= torch.cuda.device_count():
        pytest.skip("needs %d GPUs" % (max(devices) + 1))
    spec = small(layers=4, layer_types=periodic_layer_types(4, 2), ple_dim=32)
    path = write_model(tmp_path, spec, seed=41)
    batch, n = 7, 12
    prompts = random_prompts(spec.vocab, [5 + 3 * b for b in range(batch)], seed=42)
    model = api.Model(path)
    sess = api.Session(model, batch)
    sess.prefill(prompts)
    want = sess.decode(n)
    samp = {"mode": "top_k", "top_k": 8, "temperature": 0.9}
    sess.prefill(prompts)
    want_s = sess.decode(n, samp)
    sess.close()
    model.close()
    pool = api.Pool(path, devices, batch)
    sh = pool.shards()
    assert [d for d, _, _ in sh] == devices and sh[0][1] == 0 and sh[-1][2] == batch
    assert all(sh[i][2] == sh[i + 1][1] for i in range(len(sh) - 1))
    pool.prefill(prompts)
    assert np.array_equal(pool.decode(n), want)
    pool.prefill(prompts)
    assert np.array_equal(pool.decode(n, samp), want_s)          # default Philox keys are pool-wide sequence indices
    stop = int(want[batch - 1][5])
    pool.set_stop_token(stop)
    pool.prefill(prompts)
    got = pool.decode(n)
    for b in range(batch):
        row = want[b].tolist()
        k = row.index(stop) + 1 if stop in row else n
        assert got[b][:k].tolist() == row[:k] and (got[b][k:] == -1).all()
    pool.close()
    with pytest.raises(api.MlbError) as e:
        api.Pool(os.path.join(str(tmp_path), "missing.bin"), devices, batch)
    assert "device" in str(e.value)


def test_fp8_file_gives_the_weights_the_loader_would_quantise(api, tmp_path):
    """A model stored as e4m3 codes + per-row scales loads to the same device weights as its float32 file
    quantised at load: identical logits, bit for bit, at batch 1 (FP8 GEMV / single-kernel step) and batch 4."""
    spec = small(dim=256, heads=4, kv_heads=2, ple_dim=32, layers=4, layer_types=periodic_layer_types(4, 2),
                 weight_dtype="float8_e4m3", kv_dtype="bfloat16")
    p32 = write_model(tmp_path, spec, seed=51, name="f32.bin")
    p8 = write_model(tmp_path, spec, seed=51, name="fp8.bin", file_dtype="float8_e4m3")
    for batch in (1, 4):
        prompts = random_prompts(spec.vocab, [6 + 4 * b for b in range(batch)], seed=52)
        outs = []
        for path in (p32, p8):
            model = api.Model(path)
            sess = api.Session(model, batch)
            sess.prefill(prompts)
            toks = sess.decode(6)
            outs.append((toks, sess.logits().copy(), model.weight_bytes))
            sess.close()
            model.close()
        assert np.array_equal(outs[0][0], outs[1][0])
        assert np.array_equal(outs[0][1], outs[1][1])
        assert outs[0][2] == outs[1][2]


def test_compat_entry_points(api, tmp_path, capfd):
    """The reference's entry points (loadModel / loadVocab / runInferenceLoop / runInference)
    through their C-linkage twins."""
    import ctypes as C
    import json
    spec = small(qk_norm=True, query_gating=True, rms_eps=1e-8, max_context=64, vocab=600)
    os.makedirs(os.path.join(str(tmp_path), "model"))
    path = write_model(os.path.join(str(tmp_path), "model"), spec, seed=21, name="tiny.bin")
    vocab = [f"w{i}" for i in range(600)]
    vocab[5] = "\n"
    with open(os.path.join(str(tmp_path), "vocab.json"), "w") as f:
        json.dump(vocab, f)
    prompt = random_prompts(600, [30], seed=4)[0]
    with open(os.path.join(str(tmp_path), "stories.json"), "w") as f:
        json.dump([["w1", "w2"], [vocab[t] for t in prompt]], f)
    L = api.lib()
    cwd = os.getcwd()
    os.chdir(str(tmp_path))
    try:
        assert L.mlb_compat_load_model(b"missing") == 0                      # 1 = ok, 0 = failure
        assert L.mlb_compat_load_model(b"tiny") == 1
        assert L.mlb_compat_load_vocab(b"./vocab.json") == 1
        assert L.mlb_compat_vocab_lookup(b"w17") == 17 and L.mlb_compat_vocab_lookup(b"nope") == -1
        assert L.mlb_compat_vocab_token(17) == b"w17" and L.mlb_compat_vocab_token(600) is None
        assert L.mlb_compat_load_story_context(b"./stories.json", 5, 100) == 0
        # 50 % of a 30-token story = 15 context tokens; the loop then runs to max context
        rc = L.mlb_compat_run_inference_loop(b"./stories.json", 1, 50, 1, 0)
        assert rc == 0                                                       # 0 = ok
        toks = np.ctypeslib.as_array(L.mlb_compat_tokens(), shape=(64,)).copy()
        oracle = load_oracle(path)
        want, _ = oracle_rollout(oracle, prompt[:15], 64 - 15)
        assert toks[:15].tolist() == prompt[:15] and toks[15:].tolist() == want.tolist()
        # token-at-a-time form of the same loop (verbose prints the top 10 each step)
        rc = L.mlb_compat_run_inference_loop(b"./stories.json", 1, 50, 1, 1)
        assert rc == 0
        toks2 = np.ctypeslib.as_array(L.mlb_compat_tokens(), shape=(64,)).copy()
        assert np.array_equal(toks, toks2)
        # stop token by vocabulary string, streamed output: the loop ends with that token, printed as it goes
        stop_at = 15 + 9
        assert L.mlb_compat_set_stop_token(b"nope", 0) != 0
        assert L.mlb_compat_set_stop_token(vocab[int(toks[stop_at])].encode(), 0) == 0
        L.mlb_compat_set_streaming(1)
        assert "Generation took" in capfd.readouterr().out
        rc = L.mlb_compat_run_inference_loop(b"./stories.json", 1, 50, 1, 0)
        assert rc == 0
        first = 15 + toks[15:].tolist().index(int(toks[stop_at]))
        toks3 = np.ctypeslib.as_array(L.mlb_compat_tokens(), shape=(64,)).copy()
        assert toks3[:first + 1].tolist() == toks[:first + 1].tolist()
        out = capfd.readouterr().out
        assert f"Generated {first + 1 - 15} new tokens" in out and f"Final sequence length: {first + 1} tokens" in out
        streamed = "".join("[\\n]" if vocab[t] == "\n" else vocab[t] for t in toks[15:first + 1].tolist())
        assert streamed in out.split("Starting text generation")[1].split("Generation took")[0]
        L.mlb_compat_set_stop_token(None, -1)
        L.mlb_compat_set_streaming(0)
        # runInference(L): probabilities of column L-1
        assert L.mlb_compat_run_inference(15) == 0
        probs = np.ctypeslib.as_array(L.mlb_compat_last_probs(), shape=(600,)).copy()
        st = oracle.new_state()
        for t in prompt[:15]:
            lg = oracle.step(st, t).numpy().astype(np.float64)
        want_p = np.exp(lg - lg.max())
        want_p /= want_p.sum()
        assert np.abs(probs - want_p).max() < 1e-6 and int(probs.argmax()) == int(want[0])
    finally:
        os.chdir(cwd)
        L.mlb_compat_shutdown()
