#!/usr/bin/env python
"""Decode-throughput benchmark of the B200 decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A "step" is one decode step (one new token for every sequence of the batch). At N = 1 the
workload is the 1-GPU latency configuration: d=512, 8 layers (6 softmax-attention, 2 gated
delta-net), 8 heads of 64, SwiGLU 1408, PLE 64, vocab 8192, bf16 weights / KV, fp32 delta-net
state, batch 1, 128-token uniform-random prompt (seed 1), greedy decode, max context 1024,
weights ~N(0,0.02) from seed 0. With N > 1 every rank decodes its own sequence on a full
weight replica (no collective on the token path), so per-GPU work is fixed: weak scaling.

Rank 0 prints ONE JSON line. `value` is tokens/s with the L2 flushed between steps (device
events per step, max over ranks); `value_l2_warm` is the same loop back to back, the way a
real decode runs, where the 60 MB of weights stay L2-resident; `e2e` goes through
mlb_decode_step with host buffers every token.
"""
from __future__ import annotations

import argparse
import json
import os
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch on the cfg1 batch-1 workload, from the
# ncu --set full capture summarised in profiles/ncu_full_gemv_cfg1_b1.md (None = not captured).
NCU_TRAFFIC_BYTES = {
    "ffn_down_gemv_residual_ple": 1543680,
    "ffn_gateup_gemv_norm_swiglu": 2913792,
    "qkv_gemv_norm_rope_kvappend": 1614592,
    "oproj_gemv_residual": 557312,
    "deltanet_proj_gemv_norm": 1621504,
    "lmhead_gemv_norm_argmax": 8433408,
    # whole-GPU single-kernel step on cfg4 (profiles/ncu_full_grid_decode_cfg4_b1.md)
    "grid_decode_step": 1156106000,
}

# workload name -> (model, batch per GPU at N=1, prompt length, description)
WORKLOADS = {
    "cfg1": ("cfg1", 1, 128, "cfg1: d=512, 8 layers (6 attention + 2 gated delta-net), 8 heads x 64, ffn 1408, PLE 64, "
                             "vocab 8192, bf16 weights+KV, fp32 delta-net state, batch 1 per GPU, 128-token prompt, greedy"),
    "cfg3": ("cfg3", 64, 64, "cfg3: d=1024, 12 gated delta-net layers, 8 heads, dk=dv=128 (fp32 state 128x128 per head), "
                             "ffn 2816, vocab 8192, bf16 weights, batch 64 per GPU, 64-token prompt, greedy"),
    "cfg4": ("cfg4", 1, 512, "cfg4: d=2048, 24 layers (18 GQA attention 16q/4kv x 128 + 6 gated delta-net), ffn 5632, PLE 128, "
                             "vocab 32000, FP8 e4m3 weights with per-row scales, bf16 KV, batch 1 per GPU, 512-token prompt, greedy"),
}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return HBM_FALLBACK_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
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
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
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


def make_model_file(tmp: str, name: str):
    from mini_llm_cuda_b200.model_file import named_spec, synth_weights, write_model_bin
    spec = named_spec(name)
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


def cpu_baseline(spec, path, prompt, n_tokens=64):
    """The CPU oracle (KV-cached fp32 port of the decode step) on the host cores: a bounded
    sample of the same workload. Also times the reference's way - a full forward over the whole
    prefix per token - on the attention-only fp32 variant of the same dims."""
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
        # no reference binary travelled: time the CPU port the reference's way instead
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-batched", action="store_true")
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

    tmp = tempfile.mkdtemp(prefix="mlb_bench_")
    model_name, wl_batch, prompt_len, wl_text = WORKLOADS[args.workload]
    batch = args.batch or wl_batch
    spec, path = make_model_file(tmp, model_name)
    K = min(K, spec.max_context - prompt_len - W)
    prompts = [prompt_for(spec.vocab, prompt_len, 1 + rank * batch + i) for i in range(batch)]
    model = api.Model(path, device=local)
    os.remove(path)                             # the weights are on the device now
    sess = api.Session(model, batch)
    hbm_peak, peak_kind = measured_peaks()

    clocks = ClockSampler(local)
    # ---- (1) device-timed, L2 flushed between steps --------------------------------------
    sess.prefill(prompts)                       # first call: builds graphs and, for long prompts, the column set
    t0 = time.perf_counter()
    sess.prefill(prompts)
    prompt_s = time.perf_counter() - t0         # host clock around the call, which returns after the device is done
    sess.decode(W)
    barrier_sync(world, local)
    clocks.start()
    step_ms, _ = sess.decode_timed(K, True)
    barrier_sync(world, local)
    flushed_ms = max_over_ranks(float(step_ms.sum()), world, local)
    # ---- (2) device-timed, back to back (weights stay in L2) -----------------------------
    sess.prefill(prompts)
    sess.decode(W)
    barrier_sync(world, local)
    warm_step_ms, _ = sess.decode_timed(K, False)
    barrier_sync(world, local)
    warm_ms = max_over_ranks(sess.last_total_ms, world, local)
    # ---- (3) end to end through the C ABI with host buffers every step -------------------
    sess.prefill(prompts)
    tok = sess.decode(W)[:, -1].copy()
    barrier_sync(world, local)
    t0 = time.perf_counter()
    for _ in range(K):
        tok = sess.decode_step(in_tokens=tok)        # H2D of the pending id, D2H of the picked id
    torch.cuda.synchronize(local)
    e2e_s = max_over_ranks(time.perf_counter() - t0, world, local)
    clock_info = clocks.stop()
    launches = sess.launches_per_step()

    # ---- (4) per-kernel event timing for the roofline (rank 0) ----------------------------
    sess.prefill(prompts)
    sess.decode(W)
    bytes_now = sess.step_bytes()
    stats = sess.profile(min(K, 64), True)
    stats.sort(key=lambda s: -s["total_ms"])
    top = stats[0]
    ach = (top["bytes"] / top["launches"]) / (top["total_ms"] / top["launches"] * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": top["name"], "achieved": ach, "peak": hbm_peak, "unit": "GB/s",
                "frac": ach / hbm_peak, "of": peak_kind,
                "traffic": NCU_TRAFFIC_BYTES.get(top["name"]),
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

    out = {
        "metric": "decode_tokens_per_s", "value": world * batch * K / (flushed_ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": flushed_ms / K, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": {"bfloat16": "bf16", "float8_e4m3": "fp8", "float32": "f32"}[spec.weight_dtype], "data": "synthetic",
        "config": {"workload": wl_text,
                   "batch_per_gpu": batch, "prompt_len": prompt_len, "max_context": spec.max_context,
                   "parallelism": f"replicas x{world}, {batch} sequence(s) per GPU, no collective",
                   "l2": "flushed (192 MiB write) before every timed step; value_l2_warm is the unflushed loop"},
        "value_l2_warm": world * batch * K / (warm_ms * 1e-3), "ms_per_step_l2_warm": warm_ms / K,
        "ms_per_token_p50": float(np.median(step_ms)), "ms_per_token_p50_l2_warm": float(np.median(warm_step_ms)),
        "e2e": {"value": world * batch * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 4 * batch,
                "d2h_bytes_per_step": 4 * batch,
                "how": "mlb_decode_step per token with host buffers: the pending id is read from pinned host memory by the step's first kernel, the picked id and the error word are written to pinned host memory by its last one; one graph launch and one stream synchronisation per token"},
        "gpu_launches": launches * K, "launches_per_step": launches,
        "prompt": {"tokens_per_s": batch * (prompt_len - 1) / prompt_s, "ms": prompt_s * 1e3,
                   "how": "mlb_prefill of the workload's prompts, second call, host clock (outside the timed decode steps)"},
        "roofline": roofline, "step_roofline": step_roofline, "kernels": kernels, "clocks": clock_info,
    }
    # ---- scoring forward (teacher-forced full-sequence logits), where the model allows it ----
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

    # ---- (5) batched decode (256 sequences sharded over the GPUs, top-k 50 sampling) ------
    if not args.skip_batched and args.workload == "cfg1":
        from mini_llm_cuda_b200.sharding import shard_range
        lo, hi = shard_range(256, world, rank)
        per = hi - lo
        bs = api.Session(model, per, max_context=512)
        bprompts = [prompt_for(spec.vocab, 256, lo + i) for i in range(per)]
        samp = {"mode": "top_k", "top_k": 50, "temperature": 1.0, "seeds": [lo + i for i in range(per)]}
        bs.prefill(bprompts)
        t0 = time.perf_counter()
        bs.prefill(bprompts)
        bprompt_s = time.perf_counter() - t0
        bs.decode(W, samp)
        barrier_sync(world, local)
        bms, _ = bs.decode_timed(64, False, samp)
        barrier_sync(world, local)
        btot = max_over_ranks(bs.last_total_ms, world, local)
        bb = bs.step_bytes()
        out["batched"] = {"workload": f"256 sequences ({per} per GPU), 256-token prompts (seed = sequence index), "
                                      "temperature 1.0 top-k 50 Philox sampling, paged KV block 16, 64 timed steps",
                          "value": 256 * 64 / (btot * 1e-3), "unit": "tokens/s", "ms_per_step": btot / 64,
                          "algorithmic_bytes_per_step_per_gpu": bb["total"],
                          "hbm_frac": bb["total"] / (btot / 64 * 1e-3) / 1e9 / hbm_peak, "scaling": "strong",
                          "prompt_tokens_per_s_per_gpu": per * 255 / bprompt_s}
        bs.close()

    if rank == 0 and world == 1 and not args.skip_cpu:
        spec2, path2 = make_model_file(tmp, model_name)
        out["cpu_baseline"] = cpu_baseline(spec2, path2, prompts[0], 64 if args.workload == "cfg1" else 8)
    elif rank == 0:
        out["cpu_baseline"] = None
    model.close()
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
