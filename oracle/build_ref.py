"""TEST / BASELINE INFRASTRUCTURE - builds the reference's own CUDA decode path, unmodified.

The reference fixes its dims with #defines (network_meta.h:3-20) and includes that header by
quoted name, so one binary per configuration is compiled from a scratch copy of the reference
sources in which only network_meta.h is regenerated; main.cu (the training driver) is left out
and oracle/ref_driver.cu supplies `main` + `loadStoryContext`. Nothing of the reference is
written into this repository: the scratch copy lives in a temporary directory and only the
binaries land in oracle/_ref/ (git-ignored, carried to the GPU machine as built files).

    python oracle/build_ref.py [reference_root]        (skips quietly if the checkout is absent)
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

META = """#pragma once
#define dim {dim}
#define dimPairs {pairs}
#define attnHeads {heads}
#define headDim {hd}
#define ropeDenomBase 10000
#define ffnDimMultiplier 4
#define ffnDim {ffn}
#define transformers {layers}
#define maxL {maxl}
#define vocabSize {vocab}
#define TRAINING_BATCH_SIZE 8
#define CONFIG_QK_RMS_NORM {qk}
#define CONFIG_QUERY_GATING {gate}
#define ADEAMIX_BETA1 0.9f
#define ADEAMIX_BETA2 0.999f
#define ADEAMIX_BETA3 0.9999f
#define ADEAMIX_ALPHA 5.0f
#define ADEAMIX_WEIGHT_DECAY 0.01f
"""

# name -> dims. maxL = prompt + generated tokens of the run (the reference loop runs to maxL).
CONFIGS = {
    # reference-comparable variant of the 1-GPU latency config: 128-token prompt + 512 tokens
    "cfg1_ref": dict(dim=512, heads=8, hd=64, ffn=1408, layers=8, maxl=640, vocab=8192, qk="true", gate="true"),
    # same without the two optional features (the PyTorch verification script's architecture)
    "cfg1_ref_base": dict(dim=512, heads=8, hd=64, ffn=1408, layers=8, maxl=640, vocab=8192, qk="false", gate="false"),
    # small case for the parity test: 16-token prompt + 48 tokens
    "tiny_ref": dict(dim=128, heads=2, hd=64, ffn=256, layers=3, maxl=64, vocab=512, qk="true", gate="true"),
}


def default_ref_root() -> str:
    """The reference checkout: $MLB_REFERENCE_ROOT, else a `reference` directory beside this repository."""
    env = os.environ.get("MLB_REFERENCE_ROOT")
    if env:
        return env
    return os.path.normpath(os.path.join(HERE, "..", "..", "reference"))


def build(ref_root: str = "", only=None) -> list:
    ref_root = ref_root or default_ref_root()
    if not os.path.isdir(ref_root) or not os.path.exists(os.path.join(ref_root, "inference.cu")):
        print(f"build_ref: no reference checkout at {ref_root}; keeping prebuilt files in {OUT}")
        return []
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(OUT, exist_ok=True)
    built = []
    for name, cfg in CONFIGS.items():
        if only and name not in only:
            continue
        target = os.path.join(OUT, f"ref_decode_{name}")
        srcs_newest = max(os.path.getmtime(os.path.join(HERE, f)) for f in ("ref_driver.cu", "build_ref.py"))
        if os.path.exists(target) and os.path.getmtime(target) > srcs_newest:
            built.append(target)
            continue
        with tempfile.TemporaryDirectory() as tmp:
            for fn in os.listdir(ref_root):
                p = os.path.join(ref_root, fn)
                if fn.endswith((".cu", ".h")) and fn != "main.cu":
                    shutil.copy(p, tmp)
            shutil.copytree(os.path.join(ref_root, "cJSON"), os.path.join(tmp, "cJSON"))
            with open(os.path.join(tmp, "network_meta.h"), "w") as f:
                f.write(META.format(pairs=cfg["dim"] // 2, **cfg))
            shutil.copy(os.path.join(HERE, "ref_driver.cu"), tmp)
            cu = sorted(fn for fn in os.listdir(tmp) if fn.endswith(".cu"))
            cmd = [nvcc, "-O3", "-w", "-gencode", "arch=compute_100a,code=sm_100a", "-o", target] + cu + \
                  ["cJSON/cJSON.c", "-lcublas", "-lcurand"]
            print("build_ref:", name)
            subprocess.check_call(cmd, cwd=tmp)
        built.append(target)
    return built


if __name__ == "__main__":
    build(sys.argv[1] if len(sys.argv) > 1 else "")
