#!/usr/bin/env python
"""Decode-throughput benchmark of the B200 decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A "step" is one decode step (one new token for every sequence of the batch).

N = 1: the 1-GPU latency configuration: d=512, 8 layers (6 softmax-attention, 2 gated
delta-net), 8 heads of 64, SwiGLU 1408, PLE 64, vocab 8192, bf16 weights / KV, fp32 delta-net
state, batch 1, 128-token uniform-random prompt (seed 1), greedy decode, max context 1024,
weights ~N(0,0.02) from seed 0. `value` is tokens/s with the L2 flushed between steps (device
events per step); `value_l2_warm` the same loop back to back, the way a real decode runs (the
60 MB of weights stay L2-resident); `e2e` goes through mlb_decode_step with host buffers every
token. The K-step loop is repeated and the median repeat is reported.

N > 1 (under torchrun, one rank per GPU): the batched configuration, 256 independent sequences of
the same model (256-token prompts, seed = sequence index, temperature 1.0 / top-k 50 Philox
sampling, paged KV) sharded evenly over the ranks with a full weight replica each and no
collective on the token path: total work is fixed, so the line says "scaling": "strong". Rank 0
also runs all 256 sequences alone in the same run (`single_gpu_same_workload`), which is the
baseline of that curve; the batch-1 figures of the replicas are kept under `replicas_batch1`.

Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

PROMPT_LEN = 128
HBM_FALLBACK_GBS = 6650.0      # earlier measurement on this pool, used only without MEASURED_PEAKS.json
REPEATS = 5                    # the K-step timed loop is repeated; the median repeat is reported

# workload name -> (model, batch per GPU at N=1, prompt length, description)
WORKLOADS = {
    "cfg1": ("cfg1", 1, 128, "cfg1: d=512, 8 layers (6 attention + 2 gated delta-net), 8 heads x 64, ffn 1408, PLE 64, "
                             "vocab 8192, bf16 weights+KV, fp32 delta-net state, batch 1 per GPU, 128-token prompt, greedy"),
    "cfg3": ("cfg3", 64, 64, "cfg3: d=1024, 12 gated delta-net layers, 8 heads, dk=dv=128 (fp32 state 128x128 per head), "
                             "ffn 2816, vocab 8192, bf16 weights, batch 64 per GPU, 64-token prompt, greedy"),
    "cfg4": ("cfg4", 1, 512, "cfg4: d=2048, 24 layers (18 GQA attention 16q/4kv x 128 + 6 gated delta-net), ffn 5632, PLE 128, "
                             "vocab 32000, FP8 e4m3 weights with per-row scales, bf16 KV, batch 1 per GPU, 512-token prompt, greedy"),
}
BATCHED_TEXT = ("256 independent sequences of cfg1 (d=512, 8 layers, bf16), 256-token prompts (seed = sequence index), "
                "temperature 1.0 / top-k 50 Philox sampling, paged KV block 16, max context 512")


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return HBM_FALLBACK_GBS, "fallback"


def captured_traffic(kernel: str):
    """DRAM bytes per launch of a kernel from the tracked record of the profiler captures (bytes read +
    written, one launch; the record names the build and the workload each figure was captured on)."""
    p = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if not os.path.exists(p):
        return None
    with open(p) as f:
        rec = json.load(f)
    ent = rec.get("kernels", {}).get(kernel)
    return ent.get("bytes_per_launch") if ent else None


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, enabled: bool = True):
        self.index = index
        self.enabled = enabled
        self.proc = None
        self.lines = []

    def start(self):
        if not self.enabled:
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["not sampled on this rank" if not self.enabled else "nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_model_file(tmp: str, name: str, spec=None):
    from mini_llm_cuda_b200.model_file import named_spec, synth_weights, write_model_bin
    spec = spec or named_spec(name)
    path = os.path.join(tmp, f"{name}.bin")
    write_model_bin(path, spec, synth_weights(spec, seed=0), with_config=True)
    return spec, path


def prompt_for(vocab: int, n: int, seed: int):
    return np.random.default_rng(seed).integers(0, vocab, size=n).astype(np.int32).tolist()


def dist_setup():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def barrier_sync(world, local):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier(device_ids=[local])
    torch.cuda.synchronize(local)


def max_over_ranks(x: float, world, local) -> float:
    if world == 1:
        return x
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=f"cuda:{local}")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def all_ranks(x: float, world, local):
    if world == 1:
        return [x]
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=f"cuda:{local}")
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [float(o.item()) for o in out]


def shared_model_file(name, world, rank, local):
    """One model file per node, written by rank 0 into a directory that it removes at the end."""
    if world == 1:
        tmp = tempfile.mkdtemp(prefix="mlb_bench_")
        spec, path = make_model_file(tmp, name)
        return spec, path, tmp
    import torch.distributed as dist
    from mini_llm_cuda_b200.model_file import named_spec
    box = [None]
    if rank == 0:
        tmp = tempfile.mkdtemp(prefix="mlb_bench_")
        _, path = make_model_file(tmp, name)
        box = [(path, tmp)]
    dist.broadcast_object_list(box, src=0)
    path, tmp = box[0]
    return named_spec(name), path, (tmp if rank == 0 else None)


# ---------------------------------------------------------------------------------------------------
# checks against the oracle, outside the timed regions
# ---------------------------------------------------------------------------------------------------
def check_greedy_tokens(path, sess, prompt, n=8):
    """First n greedy tokens of one sequence against the KV-cached CPU oracle (identical ids)."""
    from oracle.decode_oracle import DecodeOracle, OracleWeights, greedy
    from oracle.model_bin import read_model_bin
    oracle = DecodeOracle(OracleWeights(read_model_bin(path)))
    st = oracle.new_state()
    lg = None
    for t in prompt:
        lg = oracle.step(st, int(t))
    want = []
    for _ in range(n):
        want.append(greedy(lg.numpy()))
        lg = oracle.step(st, want[-1])
    sess.prefill([prompt])
    got = sess.decode(n)[0].tolist()
    return got == want


def check_sampled_tokens(path, sess, prompts, samp, n=8):
    """Sequence 0 of a sampled batch, n steps: every drawn id equals the oracle's top-k / Philox draw on the
    logits the device produced for that step, and those logits are within the low-precision bound of the
    oracle's (teacher-forced on the device's ids)."""
    from oracle.decode_oracle import DecodeOracle, OracleWeights, sample_top_k
    from oracle.model_bin import read_model_bin
    oracle = DecodeOracle(OracleWeights(read_model_bin(path)))
    st = oracle.new_state()
    lg = None
    for t in prompts[0]:
        lg = oracle.step(st, int(t))
    sess.prefill(prompts)
    ok = True
    for _ in range(n):
        tok = int(sess.decode_step(samp)[0])
        dev = sess.logits()[0]
        want = lg.numpy()
        err = float(np.abs(dev - want).max() / max(np.abs(want).max(), 1e-30))
        draw = sample_top_k(dev, samp["temperature"], samp["top_k"], samp["seeds"][0], st.pos)
        ok = ok and err < 2e-2 and draw == tok
        lg = oracle.step(st, tok)
    return ok


def cpu_baseline(path, prompt, n_tokens=64):
    """The CPU oracle (KV-cached fp32 port of the decode step) on the host cores: a bounded sample of the
    same workload."""
    import torch
    from oracle.decode_oracle import DecodeOracle, OracleWeights, greedy
    from oracle.model_bin import read_model_bin
    oracle = DecodeOracle(OracleWeights(read_model_bin(path)))
    st = oracle.new_state()
    lg = None
    for t in prompt:
        lg = oracle.step(st, int(t))
    t0 = time.perf_counter()
    for _ in range(n_tokens):
        nxt = greedy(lg.numpy())
        lg = oracle.step(st, nxt)
    dt = time.perf_counter() - t0
    return {"value": n_tokens / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n_tokens} greedy decode tokens after the {len(prompt)}-token prompt, KV-cached fp32 oracle, "
                      f"same model and prompt ({os.cpu_count()} logical CPUs visible)"}


def cpu_full_recompute(tmp, n_tokens=64):
    """The reference's way on the host cores: a causal forward over the WHOLE prefix for every generated
    token (runInference(L), inference.cu:376-752; the PyTorch restatement is
    pytorch_verification/pyTorch_gradient_verification.py:133-319), on the attention-only fp32 variant of
    the CPU-runnable configuration (d=256, 4 layers, 4 heads x 64, ffn 768, vocab 4096, 32-token prompt)."""
    import torch
    from mini_llm_cuda_b200.model_file import ModelSpec
    from oracle.decode_oracle import OracleWeights, full_forward, greedy
    from oracle.model_bin import read_model_bin
    spec = ModelSpec(dim=256, layers=4, heads=4, head_dim=64, ffn_dim=768, vocab=4096, max_context=256, rms_eps=1e-5)
    _, path = make_model_file(tmp, "cfg0_attention_only", spec)
    w = OracleWeights(read_model_bin(path))
    toks = prompt_for(spec.vocab, 32, 1)
    t0 = time.perf_counter()
    for _ in range(n_tokens):
        logits = full_forward(w, toks)
        toks.append(greedy(logits[:, -1].numpy()))
    dt = time.perf_counter() - t0
    return {"value": n_tokens / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n_tokens} greedy tokens after a 32-token prompt, full-prefix forward per token (the reference's "
                      "loop), d=256 / 4 attention layers / vocab 4096, fp32"}


def run_reference_arm(args, world, rank, local):
    """The reference's own decode loop (unmodified inference.cu + inference_orchestrator.cu built
    by oracle/build_ref.py) on one B200, on the variant of the workload it implements: same dims,
    every layer softmax attention, fp32, QK-norm + query gating, no PLE. It recomputes the whole
    prefix per token and sorts the vocabulary on the host, so its per-token time grows with L."""
    if rank != 0:
        return
    from mini_llm_cuda_b200.model_file import named_spec, synth_weights, write_model_bin
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_decode_cfg1_ref")
    base = {"impl": "reference", "metric": "decode_tokens_per_s", "unit": "tokens/s", "n_gpus": 1,
            "higher_is_better": True, "scaling": "weak", "data": "synthetic", "dtype": "f32"}
    if not os.path.exists(exe):
        print(json.dumps(dict(base, unavailable="oracle/_ref/ref_decode_cfg1_ref was not built (reference checkout absent at build time)")))
        return
    spec = named_spec("cfg1_ref")
    steps = 512          # the binary is compiled for maxL = 128 + 512
    with tempfile.TemporaryDirectory() as tmp:
        os.makedirs(os.path.join(tmp, "model"))
        write_model_bin(os.path.join(tmp, "model", "m.bin"), spec, synth_weights(spec, seed=0), with_config=False)
        np.asarray(prompt_for(spec.vocab, PROMPT_LEN, 1), dtype="<i4").tofile(os.path.join(tmp, "prompt.i32"))
        best = None
        for _ in range(max(1, min(args.warmup, 1)) + 1):     # one warm run (cuBLAS init), one timed
            r = subprocess.run([exe, "m", "prompt.i32", "out", "1"], cwd=tmp, capture_output=True, text=True, timeout=900)
            if r.returncode != 0:
                print(json.dumps(dict(base, unavailable=f"reference binary failed: rc={r.returncode} {r.stderr[-200:]}")))
                return
            line = [ln for ln in r.stdout.splitlines() if ln.startswith("REF_RESULT")][-1]
            kv = dict(p.split("=") for p in line.split()[1:])
            best = float(kv["loop_ms"])
    value = steps / (best / 1000.0)
    out = dict(base, value=value, steps=steps, warmup=1, ms_per_step=best / steps, vs_baseline=None,
               config={"workload": "cfg1_ref: d=512, 8 layers all softmax-attention, 8 heads x 64, ffn 1408, vocab 8192, fp32 "
                                   "(cuBLAS TF32 mode as main.cu:179), QK-norm + query gating, batch 1, 128-token prompt, "
                                   "512 greedy tokens - the variant of the workload the reference implements",
                       "how": "runInferenceLoop of the unmodified reference, its own std::chrono timer"},
               cpu_baseline={"kind": "reference", "cores": 1, "value": value, "unit": "tokens/s",
                             "sample": "whole 512-token loop, reference CUDA on one B200 driven by one host thread"},
               e2e={"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    print(json.dumps(out))


class timed_range:
    """NVTX range around a timed region, so that a profiler can be pointed at the steps of one section
    (ncu --nvtx --nvtx-include "timed_steps_batch256/"); costs nothing without a profiler."""

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        import torch
        torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        import torch
        torch.cuda.nvtx.range_pop()
        return False


def timed_loop(sess, prompts, W, K, flush, world, local, samp=None):
    """REPEATS times: prompt, W warm-up steps, barrier, K device-timed steps, barrier. Returns the median
    over the repeats of the max over ranks of the K steps' time (ms) and the per-step times of that repeat."""
    totals, per_step = [], []
    for _ in range(REPEATS):
        sess.prefill(prompts)
        sess.decode(W, samp)
        barrier_sync(world, local)
        with timed_range(f"timed_steps_batch{sess.batch}"):
            step_ms, _ = sess.decode_timed(K, flush, samp)
        barrier_sync(world, local)
        mine = float(step_ms.sum()) if flush else sess.last_total_ms
        totals.append(max_over_ranks(mine, world, local))
        per_step.append(step_ms)
    order = np.argsort(totals)
    mid = int(order[len(order) // 2])
    return totals[mid], per_step[mid], totals


def e2e_loop(sess, prompts, W, K, world, local):
    """REPEATS times K tokens through mlb_decode_step with host buffers; median repeat, max over ranks."""
    import torch
    secs = []
    for _ in range(REPEATS):
        sess.prefill(prompts)
        tok = sess.decode(W)[:, -1].copy()
        barrier_sync(world, local)
        t0 = time.perf_counter()
        for _ in range(K):
            tok = sess.decode_step(in_tokens=tok)        # the pending id goes in, the picked id comes back
        torch.cuda.synchronize(local)
        secs.append(time.perf_counter() - t0)
    mine = float(np.median(secs))
    return max_over_ranks(mine, world, local), all_ranks(mine, world, local)


def batched_section(api, model, spec, path, lo, hi, W, KB, world, rank, local, hbm_peak, check):
    """Sequences [lo, hi) of the 256-sequence workload on this rank: KB device-timed steps, back to back, and
    the same steps through mlb_decode_step with the ids crossing the bus every step."""
    import torch
    per = hi - lo
    bs = api.Session(model, per, max_context=512)
    prompts = [prompt_for(spec.vocab, 256, lo + i) for i in range(per)]
    samp = {"mode": "top_k", "top_k": 50, "temperature": 1.0, "seeds": [lo + i for i in range(per)]}
    checked = None
    if check:
        checked = check_sampled_tokens(path, bs, prompts, samp)
    bs.prefill(prompts)
    t0 = time.perf_counter()
    bs.prefill(prompts)
    prompt_s = time.perf_counter() - t0
    total_ms, step_ms, _ = timed_loop(bs, prompts, W, KB, False, world, local, samp)
    bb = bs.step_bytes()
    launches = bs.launches_per_step()
    secs = []
    for _ in range(3):
        bs.prefill(prompts)
        tok = bs.decode(W, samp)[:, -1].copy()
        barrier_sync(world, local)
        t0 = time.perf_counter()
        for _ in range(KB):
            tok = bs.decode_step(samp, in_tokens=tok)
        torch.cuda.synchronize(local)
        secs.append(time.perf_counter() - t0)
    e2e_s = max_over_ranks(float(np.median(secs)), world, local)
    bs.close()
    return {"ms_per_step": total_ms / KB, "ms_per_token_p50": float(np.median(step_ms)), "sequences_per_gpu": per, "steps": KB,
            "algorithmic_bytes_per_step_per_gpu": bb["total"], "hbm_frac": bb["total"] / (total_ms / KB * 1e-3) / 1e9 / hbm_peak,
            "launches_per_step": launches, "prompt_tokens_per_s_per_gpu": per * 255 / prompt_s, "tokens_checked": checked,
            "e2e_ms_per_step": e2e_s / KB * 1e3}


def same_config_pairing(api, tmp, local):
    """The variant of the workload the reference implements (fp32, all attention, QK-norm + gating, 128-token
    prompt, 512 greedy tokens) through this library: the like-for-like row beside `--impl reference`."""
    import torch
    spec, path = make_model_file(tmp, "cfg1_ref")
    model = api.Model(path, device=local)
    os.remove(path)
    sess = api.Session(model, 1)
    prompt = prompt_for(spec.vocab, PROMPT_LEN, 1)
    steps = 512
    sess.prefill([prompt])
    sess.decode(4)
    sess.prefill([prompt])
    sess.decode_timed(steps, False)
    dev_ms = sess.last_total_ms
    sess.prefill([prompt])
    tok = sess.decode(1)[:, -1].copy()
    t0 = time.perf_counter()
    for _ in range(steps - 1):
        tok = sess.decode_step(in_tokens=tok)
    torch.cuda.synchronize(local)
    e2e_s = time.perf_counter() - t0
    launches = sess.launches_per_step()
    sess.close()
    model.close()
    return {"workload": "cfg1_ref: d=512, 8 layers all softmax-attention, 8 heads x 64, ffn 1408, vocab 8192, fp32 weights and KV, "
                        "QK-norm + query gating, batch 1, 128-token prompt, 512 greedy tokens (context 128 -> 640)",
            "value": steps / (dev_ms * 1e-3), "e2e": (steps - 1) / e2e_s, "unit": "tokens/s", "steps": steps,
            "ms_per_step": dev_ms / steps, "launches_per_step": launches,
            "how": "device events around 512 back-to-back steps; e2e: mlb_decode_step per token with host buffers"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-batched", action="store_true")
    ap.add_argument("--skip-pairing", action="store_true")
    ap.add_argument("--workload", default="cfg1", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="sequences per GPU (default: the workload's)")
    args = ap.parse_args()
    world, rank, local = dist_setup()
    if args.impl == "reference":
        run_reference_arm(args, world, rank, local)
        return
    W = max(3, args.warmup)
    K = max(1, args.steps)

    from mini_llm_cuda_b200 import api
    api.lib()                                   # raises if the CUDA library is missing
    import torch                                # plumbing: device sync, barrier, max over ranks

    model_name, wl_batch, prompt_len, wl_text = WORKLOADS[args.workload]
    batch = args.batch or wl_batch
    spec, path, tmp = shared_model_file(model_name, world, rank, local)
    try:
        K = min(K, spec.max_context - prompt_len - W)
        prompts = [prompt_for(spec.vocab, prompt_len, 1 + rank * batch + i) for i in range(batch)]
        model = api.Model(path, device=local)
        sess = api.Session(model, batch)
        hbm_peak, peak_kind = measured_peaks()
        # one nvidia-smi child per node is enough (eight of them on one box cost host time)
        clocks = ClockSampler(local, enabled=(local == 0))

        # ---- checks, outside the timed regions ----------------------------------------------------
        tokens_checked = None
        if rank == 0 and not args.skip_cpu and batch == 1:
            tokens_checked = check_greedy_tokens(path, sess, prompts[0])

        # ---- (1) device-timed, L2 flushed between steps --------------------------------------------
        sess.prefill(prompts)                       # first call: builds graphs and, for long prompts, the column set
        t0 = time.perf_counter()
        sess.prefill(prompts)
        prompt_s = time.perf_counter() - t0         # host clock around the call, which returns after the device is done
        clocks.start()
        flushed_ms, step_ms, flushed_all = timed_loop(sess, prompts, W, K, True, world, local)
        # ---- (2) device-timed, back to back (weights stay in L2) -----------------------------------
        warm_ms, warm_step_ms, _ = timed_loop(sess, prompts, W, K, False, world, local)
        # ---- (3) end to end through the C ABI with host buffers every step -------------------------
        e2e_s, e2e_ranks = e2e_loop(sess, prompts, W, K, world, local)
        clock_info = clocks.stop()
        launches = sess.launches_per_step()

        # ---- (4) per-kernel event timing for the roofline (rank 0) ----------------------------------
        sess.prefill(prompts)
        sess.decode(W)
        bytes_now = sess.step_bytes()
        stats = sess.profile(min(K, 64), True)
        stats.sort(key=lambda s: -s["total_ms"])
        top = stats[0]
        ach = (top["bytes"] / top["launches"]) / (top["total_ms"] / top["launches"] * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": top["name"], "achieved": ach, "peak": hbm_peak, "unit": "GB/s",
                    "frac": ach / hbm_peak, "of": peak_kind,
                    "traffic": captured_traffic(top["name"]),
                    "algorithmic_bytes_per_launch": top["bytes"] // top["launches"],
                    "us_per_launch": top["total_ms"] / top["launches"] * 1e3,
                    "share_of_step": top["total_ms"] / sum(s["total_ms"] for s in stats),
                    "l2": "flushed before each step"}
        step_us = flushed_ms / K * 1e3
        step_roofline = {"algorithmic_bytes_per_step": bytes_now["total"], "ideal_us_at_peak": bytes_now["total"] / hbm_peak / 1e3,
                         "frac_l2_flushed": bytes_now["total"] / (step_us * 1e-6) / 1e9 / hbm_peak,
                         "frac_l2_warm": bytes_now["total"] / (warm_ms / K * 1e-3) / 1e9 / hbm_peak}
        kernels = [{"name": s["name"], "launches_per_step": s["launches"] // min(K, 64),
                    "us_per_launch": round(s["total_ms"] / s["launches"] * 1e3, 3),
                    "GBps": round(s["bytes"] / max(s["total_ms"], 1e-9) / 1e6, 1)} for s in stats]

        latency = {
            "value": world * batch * K / (flushed_ms * 1e-3), "ms_per_step": flushed_ms / K,
            "value_l2_warm": world * batch * K / (warm_ms * 1e-3), "ms_per_step_l2_warm": warm_ms / K,
            "ms_per_token_p50": float(np.median(step_ms)), "ms_per_token_p50_l2_warm": float(np.median(warm_step_ms)),
            "repeats_ms_per_step": [round(t / K, 6) for t in flushed_all],
        }
        e2e = {"value": world * batch * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 4 * batch,
               "d2h_bytes_per_step": 4 * batch, "per_rank_ms_per_token": [round(s / K * 1e3, 5) for s in e2e_ranks],
               "how": "mlb_decode_step per token with host buffers: the pending id goes in with the call (a launch argument of the "
                      "single-kernel step, pinned host memory read by the first kernel otherwise), the picked id and the error word "
                      "are written to pinned host memory by the kernel that advances the sequence and the host polls that word"}
        out = {
            "metric": "decode_tokens_per_s", "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "repeats": REPEATS,
            "higher_is_better": True, "vs_baseline": None,
            "dtype": {"bfloat16": "bf16", "float8_e4m3": "fp8", "float32": "f32"}[spec.weight_dtype], "data": "synthetic",
            "gpu_launches": launches * K, "launches_per_step": launches,
            "prompt": {"tokens_per_s": batch * (prompt_len - 1) / prompt_s, "ms": prompt_s * 1e3,
                       "how": "mlb_prefill of the workload's prompts, second call, host clock (outside the timed decode steps)"},
            "roofline": roofline, "step_roofline": step_roofline, "kernels": kernels, "clocks": clock_info,
            "tokens_checked": tokens_checked,
        }
        # ---- scoring forward (teacher-forced full-sequence logits), where the model allows it ------
        if spec.weight_dtype in ("bfloat16", "float8_e4m3"):
            n_score = min(512, spec.max_context)
            stoks = prompt_for(spec.vocab, n_score, 7 + rank)
            sess.score(stoks)
            t0 = time.perf_counter()
            sess.score(stoks)
            score_s = time.perf_counter() - t0
            out["score"] = {"tokens_per_s": n_score / score_s, "ms": score_s * 1e3,
                            "how": f"mlb_score_tokens on {n_score} tokens, second call, host clock, [len][V] fp32 logits copied to the host"}
        sess.close()

        # ---- (5) batched decode: 256 sequences sharded over the GPUs, top-k 50 sampling -------------
        batched = single = None
        if not args.skip_batched and args.workload == "cfg1":
            from mini_llm_cuda_b200.sharding import shard_range
            lo, hi = shard_range(256, world, rank)
            KB = max(1, min(args.steps, 512 - 256 - W - 1))
            batched = batched_section(api, model, spec, path, lo, hi, W, KB, world, rank, local, hbm_peak,
                                      check=(rank == 0 and not args.skip_cpu))
            batched.update({"workload": BATCHED_TEXT + f", {hi - lo} sequences per GPU, {KB} timed steps back to back",
                            "value": 256 / (batched["ms_per_step"] * 1e-3), "unit": "tokens/s", "scaling": "strong",
                            "e2e_value": 256 / (batched["e2e_ms_per_step"] * 1e-3)})
            if world > 1:
                # the baseline of the strong-scaling curve, in the same run: all 256 sequences on rank 0's GPU
                if rank == 0:
                    single = batched_section(api, model, spec, path, 0, 256, W, KB, 1, 0, local, hbm_peak, check=False)
                    single["value"] = 256 / (single["ms_per_step"] * 1e-3)
                barrier_sync(world, local)

        if world == 1:
            out.update({"value": latency["value"], "ms_per_step": latency["ms_per_step"], "scaling": "weak",
                        "config": {"workload": wl_text, "batch_per_gpu": batch, "prompt_len": prompt_len, "max_context": spec.max_context,
                                   "parallelism": "1 GPU, 1 sequence",
                                   "l2": "flushed (192 MiB write) before every timed step; value_l2_warm is the unflushed loop"},
                        "e2e": e2e})
            out.update({k: v for k, v in latency.items() if k not in ("value", "ms_per_step")})
            if batched:
                out["batched"] = batched
        else:
            if batched is None:
                raise SystemExit("the multi-GPU line reports the sharded 256-sequence workload: run without --skip-batched on cfg1")
            out.update({"value": batched["value"], "ms_per_step": batched["ms_per_step"], "scaling": "strong",
                        "config": {"workload": batched["workload"], "global_batch": 256, "prompt_len": 256, "max_context": 512,
                                   "parallelism": f"256 sequences sharded over {world} GPUs ({256 // world} each), a full weight replica per GPU, "
                                                  "no collective on the token path",
                                   "l2": "steps back to back; a step reads more than the L2 holds only from 128 sequences per GPU on (KV)"},
                        "gpu_launches": batched["launches_per_step"] * batched["steps"], "launches_per_step": batched["launches_per_step"],
                        "steps": batched["steps"],
                        "batched": batched, "single_gpu_same_workload": single,
                        "strong_scaling_speedup": (batched["value"] / single["value"]) if single else None,
                        "replicas_batch1": dict(latency, e2e=e2e, workload=wl_text,
                                                parallelism=f"replicas x{world}, one sequence per GPU (weak scaling)"),
                        "tokens_checked": batched.get("tokens_checked"),
                        "e2e": {"value": batched["e2e_value"], "unit": "tokens/s", "h2d_bytes_per_step": 4 * 256, "d2h_bytes_per_step": 4 * 256,
                                "how": "mlb_decode_step per step on every rank: the pending ids are read from pinned host memory by the step's "
                                       "first kernel, the drawn ids are written to pinned host memory by its last one; host clock, max over ranks"}})

        if rank == 0 and world == 1 and not args.skip_cpu:
            out["cpu_baseline"] = cpu_baseline(path, prompts[0], 64 if args.workload == "cfg1" else 8)
            out["cpu_baseline_full_recompute"] = cpu_full_recompute(tmp, 64)
        elif rank == 0:
            out["cpu_baseline"] = None
        model.close()
        if rank == 0 and world == 1 and not args.skip_pairing and args.workload == "cfg1":
            out["same_config_vs_reference"] = same_config_pairing(api, tmp, local)
        if rank == 0:
            print(json.dumps(out))
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.barrier(device_ids=[local])
        if tmp:
            shutil.rmtree(tmp, ignore_errors=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
