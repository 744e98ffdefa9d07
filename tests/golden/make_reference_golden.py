"""Generates tests/golden/reference_pytorch_logits.npz by running the reference's own
PyTorch verification script UNCHANGED (pytorch_verification/pyTorch_gradient_verification.py,
forward at :133-319) on a seeded synthetic model.

Run where the reference checkout is available:

    python tests/golden/make_reference_golden.py /path/to/mini-llm-cuda

The script is executed with runpy inside a scratch directory that holds
  * model_15_lr_3e6.bin  - the seeded synthetic model (dims hard-coded by the script at
                           :10-17: dim 512, ffn 2048, 4 layers, 8 heads, vocab 10097)
  * vocab.json           - 10097 made-up token strings "t0".."t10096"
  * sample.json          - 256 of those strings drawn with a seeded generator
so nothing of the reference's own data files is read or stored. json.dump is stubbed
while it runs because the script writes ~1 GB of gradient JSON that nobody needs.

Stored: the seed recipe, the token ids, the logits of 6 columns, and for all 256
columns the argmax id and the log-sum-exp of the logits.
"""
import json
import os
import runpy
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from mini_llm_cuda_b200.model_file import ModelSpec, synth_weights, write_model_bin  # noqa: E402

SEED_WEIGHTS = 1234
SEED_TOKENS = 4321
COLUMNS = [0, 1, 31, 127, 200, 255]


def golden_spec() -> ModelSpec:
    return ModelSpec(dim=512, layers=4, heads=8, head_dim=64, ffn_dim=2048, vocab=10097,
                     max_context=256, rms_eps=1e-8)


def golden_tokens() -> np.ndarray:
    return np.random.default_rng(SEED_TOKENS).integers(0, 10097, size=256).astype(np.int32)


def main(ref_root: str) -> None:
    spec = golden_spec()
    weights = synth_weights(spec, seed=SEED_WEIGHTS, random_gains=True)
    tokens = golden_tokens()
    script = os.path.join(ref_root, "pytorch_verification", "pyTorch_gradient_verification.py")
    with tempfile.TemporaryDirectory() as tmp:
        write_model_bin(os.path.join(tmp, "model_15_lr_3e6.bin"), spec, weights, with_config=False)
        vocab = [f"t{i}" for i in range(10097)]
        with open(os.path.join(tmp, "vocab.json"), "w") as f:
            json.dump(vocab, f)
        with open(os.path.join(tmp, "sample.json"), "w") as f:
            json.dump([vocab[t] for t in tokens], f)
        cwd = os.getcwd()
        real_dump = json.dump
        sys.path.insert(0, os.path.join(ref_root, "pytorch_verification"))
        try:
            os.chdir(tmp)
            json.dump = lambda *a, **k: None
            g = runpy.run_path(script, run_name="__main__")
        finally:
            json.dump = real_dump
            os.chdir(cwd)
            sys.path.pop(0)
    logits = g["logits"].detach().numpy().astype(np.float32)        # [V, L]
    assert logits.shape == (10097, 256)
    assert np.array_equal(g["sample_indices"].numpy().astype(np.int32), tokens)
    m = logits.max(axis=0)
    lse = (m + np.log(np.exp(logits - m).sum(axis=0))).astype(np.float32)
    np.savez_compressed(
        os.path.join(HERE, "reference_pytorch_logits.npz"),
        seed_weights=SEED_WEIGHTS, seed_tokens=SEED_TOKENS, tokens=tokens,
        columns=np.array(COLUMNS, dtype=np.int32),
        logits_columns=logits[:, COLUMNS].T.copy(),                   # [6, V]
        argmax=logits.argmax(axis=0).astype(np.int32), logsumexp=lse,
        weights_checksum=np.float64(sum(float(np.abs(b[k]).sum()) for b in weights["blocks"] for k in b)
                                    + float(np.abs(weights["tokenEmbeddings"]).sum())),
    )
    print("wrote reference_pytorch_logits.npz", logits.shape)


if __name__ == "__main__":
    # the reference checkout: first argument, else $MLB_REFERENCE_ROOT, else a `reference` directory beside this repository
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
        "MLB_REFERENCE_ROOT", os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference"))))
