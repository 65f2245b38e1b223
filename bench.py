#!/usr/bin/env python3
"""Decode-throughput benchmark of the KV-cached token loop.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode iteration for every sequence of the batch: choose the
next id of each sequence on the device (temperature / top-p sampler), then run
one KV-cached forward step on those ids. The default workload is the
whole-box configuration the metric is quoted on: the `modern` Llama-style block
(d768, 8 layers, 12 heads, SwiGLU 2048, vocab 16000, 69.0M parameters,
random-init N(0, 0.02)), 256 independent sequences per GPU, 32-id seeded
prompts fed through the batched prompt feed, then decoded to context 256 with
temperature 0.8 / top-p 0.9. With the default K = 224 the timed region is the
complete decode from context 32 to 256. Sequences are sharded across GPUs, one
weight replica per GPU, no collective on the token path; finished ids are
gathered with NCCL after the loop.

Prints ONE JSON line on rank 0. `value` is whole-job decode tokens/s with
inputs resident in HBM (device time of the K steps, max over ranks); `e2e` is
the same count of new ids divided by the wall time of the public generate call
with host buffers (prompt upload, prompt feed, decode, id download). At N=1 the
line also carries the batch-1 configuration (`batch1`), the per-kernel device
times behind the roofline figure (`kernels`), and the reference's CPU path
timed on this machine's host cores (`cpu_baseline`).

`--impl reference` times the reference's own CPU implementation of the same
path (compiled unmodified into oracle/_ref, else the plain-C restatement) on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_LEN = 32
CONTEXT = 256
SAMPLER = dict(temperature=0.8, top_k=0, top_p=0.9, penalty=1.0)
WEIGHT_SEED = 1004
PROMPT_SEED = 2004


def load_package():
    if "grad_cpp_b200" in sys.modules:
        return sys.modules["grad_cpp_b200"]
    pkg_dir = ROOT / "grad.cpp_b200"
    spec = importlib.util.spec_from_file_location("grad_cpp_b200", pkg_dir / "__init__.py",
                                                  submodule_search_locations=[str(pkg_dir)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["grad_cpp_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 0))), "measured"
    return 6650.0, 1400.0, "fallback"


def seq_prompt(global_seq: int, vocab: int, n: int | None = None):
    """Per-sequence stream, so a sequence is the same whichever GPU it lands on."""
    load_package()
    from grad_cpp_b200 import sharding
    return sharding.seq_prompt(PROMPT_SEED, global_seq, vocab, PROMPT_LEN if n is None else n)


def seq_draws(global_seq: int, n: int):
    load_package()
    from grad_cpp_b200 import sharding
    return sharding.seq_draws(PROMPT_SEED, global_seq, n)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        self.t.join(timeout=2)
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- algorithmic bytes

def weight_elems(dm):
    d, f, L, V = dm.d_model, dm.d_ff, dm.layers, dm.vocab
    per_layer = {"norm_qkv_rope": 3 * d * d + 3 * d + 2 * d, "attn_out_proj": d * d + d,
                 "norm_ffn_up": (2 if dm.arch == 1 else 1) * d * f + (0 if dm.arch == 1 else f) + 2 * d,
                 "ffn_down": f * d + (0 if dm.arch == 1 else d)}
    return per_layer, V * d + 2 * d


def algorithmic_bytes_per_step(dm, batch, ctx, w_bytes, ctx_sum=None):
    """Bytes one decode step must move, per kernel class: weights streamed once per launch
    (w_bytes per element), fp32 activations in and out, and the K/V rows of every cached position
    (ctx positions for each of `batch` sequences, or ctx_sum positions in all when contexts differ)."""
    d, f, L, V = dm.d_model, dm.d_ff, dm.layers, dm.vocab
    if ctx_sum is None:
        ctx_sum = batch * ctx
    per_layer, logits_w = weight_elems(dm)
    act = 4
    out = {
        "embed": batch * d * act * 2,
        "norm_qkv_rope": L * (per_layer["norm_qkv_rope"] * w_bytes + batch * d * act * 4),
        "attn_decode": L * (2 * ctx_sum * d * 4 + batch * d * act * 2),
        "attn_out_proj": L * (per_layer["attn_out_proj"] * w_bytes + batch * d * act * 3),
        "norm_ffn_up": L * (per_layer["norm_ffn_up"] * w_bytes + batch * (d + f) * act),
        "ffn_down": L * (per_layer["ffn_down"] * w_bytes + batch * (f + 2 * d) * act),
        "norm_logits": logits_w * w_bytes + batch * (d + V) * act,
        "advance": batch * 8,
        "select": batch * V * act,
    }
    return out


# ----------------------------------------------------------------------------- our arm

HBM_CLASSES = ("norm_qkv_rope", "attn_decode", "attn_out_proj", "norm_ffn_up", "ffn_down", "norm_logits")
KERNEL_NAMES = {"norm_qkv_rope": "norm_rows_kernel + gemm_bf16_tc_kernel<TC_QKV>", "attn_decode": "attn_decode64_pipe_kernel",
                "attn_out_proj": "gemm_bf16_tc_kernel<TC_RESID>", "norm_ffn_up": "norm_rows_kernel + gemm_bf16_tc_kernel<TC_SWIGLU>",
                "ffn_down": "gemm_bf16_tc_kernel<TC_RESID>", "norm_logits": "norm_rows_kernel + gemm_bf16_tc_kernel<TC_LOGITS>",
                "select": "select_kernel", "decode_step_b1": "decode_b1_kernel"}


def pick_steps(K, full):
    """K decode steps spread evenly over the `full` steps of the complete decode (all of them when K >= full)."""
    if K >= full:
        return list(range(full))
    if K == 1:
        return [full // 2]
    idx = sorted({int(round(x)) for x in np.linspace(0, full - 1, K)})
    assert len(idx) == K
    return idx


def run_ours(args):
    import torch
    import torch.distributed as dist

    g = load_package()
    from grad_cpp_b200 import checkpoint as ck
    from grad_cpp_b200 import sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    g.lib()

    dm = ck.PRESETS["modern"]
    B, W = args.batch, args.warmup
    FULL = CONTEXT - PROMPT_LEN            # decode steps of the complete run (context 32 -> 256)
    K = max(1, min(args.steps, FULL))
    timed = pick_steps(K, FULL)
    precision = g.BF16 if args.precision == "bf16" else g.FP32
    tmp = tempfile.mkdtemp(prefix="gradb_bench_")
    path = str(ck.write_synthetic(Path(tmp) / f"modern_{rank}.bin", dm, WEIGHT_SEED))
    model = g.GPTModel.load(path, local, precision)
    stream = torch.cuda.Stream()
    sess = g.BatchSession(model, B, CONTEXT, stream=stream.cuda_stream)
    prompts = [seq_prompt(rank * B + i, dm.vocab) for i in range(B)]
    if args.eval_only:
        _, peak, kind = peaks()
        if rank == 0:
            print(json.dumps({"eval": bench_scoring(sess, dm, B, peak, kind)}))
        sess.close()
        model.close()
        return
    sp = g.Sampling(0, SAMPLER["temperature"], SAMPLER["penalty"], SAMPLER["top_k"], SAMPLER["top_p"])
    draws = np.stack([seq_draws(rank * B + i, FULL + 1) for i in range(B)])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Warm-up: one complete generation (all FULL >= W decode steps; captures the step graph with the timed
    # call's parameters, warms caches and clocks), and the id gather's first use.
    _, warm_ms, _ = sess.generate(prompts, sp, FULL + 1, uniforms=draws, timings=True)
    if world > 1:
        sharding.gather_ids(np.zeros((B, CONTEXT + 1), np.int32), world, device="cuda")
    est_s = float(np.sum(warm_ms[:FULL])) / 1e3
    reps = int(min(16, max(5, np.ceil(1.0 / max(est_s, 1e-3)))))
    if args.reps:
        reps = args.reps

    launches0 = g.lib().gradb_kernel_launches()
    clocks = ClockSampler(local)
    barrier()
    clocks.start()
    rep_dev, rep_wall, rep_full, ids, step_ms, prefill_ms = [], [], [], None, None, 0.0
    for _ in range(reps):
        t0 = time.perf_counter()
        ids, step_ms, prefill_ms = sess.generate(prompts, sp, FULL + 1, uniforms=draws, timings=True)
        all_ids = sharding.gather_ids(sharding.pad_ids(ids, CONTEXT + 1), world, device="cuda")  # one NCCL all_gather
        torch.cuda.synchronize()
        rep_wall.append(time.perf_counter() - t0)
        rep_dev.append(float(np.sum(step_ms[timed])) / 1e3)
        rep_full.append(float(np.sum(step_ms[:FULL])) / 1e3)
        assert all_ids.shape[0] == world * B
    clk = clocks.stop()
    barrier()
    launches = g.lib().gradb_kernel_launches() - launches0
    new_ids = sum(len(s) - PROMPT_LEN for s in ids)
    assert new_ids == B * (FULL + 1), (new_ids, B, FULL)

    med = lambda v: float(statistics.median(v))
    stats = sharding.max_over_ranks([med(rep_dev), med(rep_wall), med(rep_full), min(rep_dev), max(rep_dev),
                                     float(np.median(step_ms[timed]))], world, device="cuda")
    dev_s, wall, full_s, dev_min, dev_max, p50 = stats

    hbm_peak, tensor_peak, peak_kind = peaks()
    w_bytes = 2 if precision == g.BF16 else 4
    spread = (f"the {K} timed steps are spread evenly over the complete decode (contexts "
              f"{PROMPT_LEN + timed[0] + 1}..{PROMPT_LEN + timed[-1] + 1})" if K < FULL
              else "every step of the complete decode is timed")
    line = {
        "metric": "decode tokens/s", "value": world * B * K / dev_s, "unit": "tokens/s", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": dev_s / K * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": ("bf16 (weights and GEMM activation operands bf16, f32 accumulate; f32 residual stream, attention "
                  "and KV cache)") if precision == g.BF16 else "f32 (projections as three TF32 products per term)",
        "data": "synthetic",
        "config": {"workload": f"modern d768 L8 H12 SwiGLU2048 V16000 (69.0M), {B} sequences/GPU, "
                               f"prompt {PROMPT_LEN} ids via batched prompt feed, sampled decode context "
                               f"{PROMPT_LEN}->{CONTEXT} (T 0.8, top-p 0.9); each repetition runs the complete "
                               f"{FULL}-step decode and {spread}; median of {reps} repetitions",
                   "batch_per_gpu": B, "prompt_len": PROMPT_LEN, "context_end": CONTEXT,
                   "timed_step_contexts": [PROMPT_LEN + timed[0] + 1, PROMPT_LEN + timed[-1] + 1],
                   "repetitions": reps, "warmup_steps_run": FULL,
                   "parallelism": f"sequence-sharded replicas x{world}",
                   "l2": "working set (weights + KV of 256 sequences, >1.5 GB) exceeds L2; no flush needed"},
        "p50_ms_per_step": p50,
        "ms_per_step_min_max": [dev_min / K * 1e3, dev_max / K * 1e3],
        "full_decode": {"steps": FULL, "ms_per_step": full_s / FULL * 1e3, "tokens_per_s": world * B * FULL / full_s,
                        "device_s_timed_per_rank": sum(rep_full)},
        "prefill_ms": prefill_ms,
        "e2e": {"value": world * B * (FULL + 1) / wall, "unit": "tokens/s",
                "h2d_bytes_per_step": (B * PROMPT_LEN * 4 + B * (FULL + 1) * 4) / (FULL + 1),
                "d2h_bytes_per_step": (B * (CONTEXT + 2) * 4 + B * 4) / (FULL + 1),
                "wall_s": wall, "new_ids_per_call": world * B * (FULL + 1),
                "includes": "per call of the public generate: prompt upload, prompt feed, complete decode, id "
                            "download" + (", NCCL all_gather of ids" if world > 1 else "") + "; median of the "
                            "repetitions"},
        "gpu_launches": int(launches),
        "clocks": clk,
    }

    if rank == 0 and not args.main_only:
        # Per-kernel device time over the complete decode, from events around every launch.
        sess.set_profiling(True)
        sess.generate(prompts, sp, FULL + 1, uniforms=draws)
        prof = sess.profile()
        sess.set_profiling(False)
        sess.set_profiling(True)
        sess.generate(prompts, sp, 0, uniforms=None)  # the prompt feed alone, to subtract
        feed = sess.profile()
        sess.set_profiling(False)
        alg = {k: 0.0 for k in prof}
        for i in range(FULL):
            for k, v in algorithmic_bytes_per_step(dm, B, PROMPT_LEN + i + 1, w_bytes).items():
                alg[k] += v
        kernels = {}
        total_ms = sum(prof[k][0] - feed.get(k, (0.0, 0))[0] for k in prof)
        for k, (ms_all, n_all) in prof.items():
            ms = ms_all - feed.get(k, (0.0, 0))[0]
            n = n_all - feed.get(k, (0.0, 0))[1]
            if n <= 0:
                continue
            per = alg[k] / n
            kernels[k] = {"decode_ms": round(ms, 3), "decode_launches": n, "share": round(ms / total_ms, 4),
                          "avg_launch_us": round(ms * 1e3 / n, 2),
                          "algorithmic_bytes_per_launch": per,
                          "achieved_gbs": round(alg[k] / (ms / 1e3) / 1e9, 1) if k in HBM_CLASSES else None,
                          "hbm_frac": round(alg[k] / (ms / 1e3) / 1e9 / hbm_peak, 4) if k in HBM_CLASSES else None,
                          "traffic": ncu_traffic(k, per)}
        dom = max((k for k in kernels if k in HBM_CLASSES), key=lambda k: kernels[k]["decode_ms"])
        kd = kernels[dom]
        achieved = alg[dom] / (kd["decode_ms"] / 1e3) / 1e9
        line["kernels"] = kernels
        line["roofline"] = {"kernel": dom, "kernel_name": KERNEL_NAMES.get(dom), "bound": "hbm", "achieved": achieved,
                            "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": peak_kind,
                            "algorithmic_bytes_per_launch": kd["algorithmic_bytes_per_launch"],
                            "avg_launch_us": kd["avg_launch_us"], "launches": kd["decode_launches"],
                            "share_of_step": kd["share"], "traffic": kd["traffic"],
                            "note": "class with the most device time among the HBM-bound classes, over the complete "
                                    "decode (per-launch CUDA events on the session's stream, graphs off)"}
        if "select" in kernels:
            ks = kernels["select"]
            line["select"] = {"kernel": "select_kernel", "bound": "on-chip (shared memory, one CTA per sequence)",
                              "avg_launch_us": ks["avg_launch_us"], "launches": ks["decode_launches"],
                              "ctas_per_launch": B, "share_of_step": ks["share"],
                              "logits_read_gbs": round(alg["select"] / (ks["decode_ms"] / 1e3) / 1e9, 1)}
        step_bytes = sum(sum(algorithmic_bytes_per_step(dm, B, PROMPT_LEN + i + 1, w_bytes).values())
                         for i in range(FULL))
        line["step_roofline"] = {"algorithmic_bytes_per_step_avg": step_bytes / FULL,
                                 "achieved_gbs": step_bytes / full_s / 1e9, "frac": step_bytes / full_s / 1e9 / hbm_peak,
                                 "over": f"the complete {FULL}-step decode"}
        line["eval"] = bench_scoring(sess, dm, B, tensor_peak, peak_kind)
        if world == 1:
            sess.close()
            sess = None
            line["fp32_check"], line["bf16_vs_fp32"] = bench_fp32_check(g, path, local, dm, B, prompts, draws, sp, ids,
                                                                        model, hbm_peak)
            line["batch1"] = bench_batch1(g, ck, local, hbm_peak)
            line["config1"] = bench_config1(g, ck, local, hbm_peak)
            line["config3"] = bench_config3(g, ck, local, hbm_peak)
            line["config5"] = bench_config5(g, ck, local, hbm_peak)
            line["cpu_baseline"] = cpu_reference(K_sample=args.cpu_tokens, n_seq=None, timed_only=True)

    if sess is not None:
        sess.close()
    model.close()
    try:
        os.remove(path)
        os.rmdir(tmp)
    except OSError:
        pass
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def ncu_traffic(kernel_class, algorithmic_bytes_per_launch):
    """DRAM bytes per launch of a kernel class, scaled from a committed ncu capture (traffic grows in
    proportion to the positions read), or None when no capture of that class is on file."""
    p = ROOT / "profiles" / "ncu_traffic.json"
    if not p.exists():
        return None
    rec = json.loads(p.read_text()).get(kernel_class)
    if not rec:
        return None
    return rec["traffic_over_algorithmic"] * algorithmic_bytes_per_launch


def log_softmax64(x):
    x = x.astype(np.float64)
    x = x - x.max(axis=-1, keepdims=True)
    return x - np.log(np.exp(x).sum(axis=-1, keepdims=True))


def common_prefix_frac(a, b, n_prompt):
    na, nb = a[n_prompt:], b[n_prompt:]
    k = min(len(na), len(nb))
    same = na[:k] == nb[:k]
    return (int(np.argmin(same)) if not same.all() else k) / max(k, 1)


def bench_fp32_check(g, path, device, dm, B, prompts, draws, sp, ids_bf16, model_bf16, hbm_peak):
    """The benchmark workload on an fp32 session (projections as three TF32 products per term): speed, and the
    distance of the bf16 run from it: last-prompt-position logits of every sequence, ids under the same draws."""
    FULL = CONTEXT - PROMPT_LEN
    s16 = g.BatchSession(model_bf16, B, CONTEXT)
    lg16 = s16.prefill(prompts)
    s16.close()
    m32 = g.GPTModel.load(path, device, g.FP32)
    s32 = g.BatchSession(m32, B, CONTEXT)
    lg32 = s32.prefill(prompts)
    s32.generate(prompts, sp, FULL + 1, uniforms=draws)  # warm-up
    ids32, step_ms, pre_ms = s32.generate(prompts, sp, FULL + 1, uniforms=draws, timings=True)
    s32.close()
    m32.close()
    dev_s = float(np.sum(step_ms[:FULL])) / 1e3
    nbytes = sum(sum(algorithmic_bytes_per_step(dm, B, PROMPT_LEN + i + 1, 4).values()) for i in range(FULL))
    speed = {"workload": f"the benchmark workload ({B} sequences, sampled, context {PROMPT_LEN}->{CONTEXT}) on an fp32 "
                         "session", "tokens_per_s": B * FULL / dev_s, "ms_per_step": dev_s / FULL * 1e3,
             "p50_ms_per_step": float(np.median(step_ms[:FULL])), "prefill_ms": pre_ms,
             "hbm_frac": nbytes / dev_s / 1e9 / hbm_peak}
    p32, p16 = log_softmax64(lg32), log_softmax64(lg16)
    err = float(np.abs(lg16 - lg32).max() / np.abs(lg32).max())
    figures = {"logits_max_abs_err_over_max_abs": err,
               "mean_kl_fp32_vs_bf16": float((np.exp(p32) * (p32 - p16)).sum(axis=-1).mean()),
               "first_id_agreement": float(np.mean([a[PROMPT_LEN] == b[PROMPT_LEN] for a, b in zip(ids32, ids_bf16)])),
               "mean_common_prefix_of_rollout": float(np.mean([common_prefix_frac(a, b, PROMPT_LEN)
                                                               for a, b in zip(ids32, ids_bf16)])),
               "greedy_agreement_at_prompt_end": float(np.mean(lg32.argmax(axis=1) == lg16.argmax(axis=1))),
               "over": f"{B} sequences: logits after the {PROMPT_LEN}-id prompt; sampled ids under identical draws"}
    return speed, figures


def decode_block(sess, dm, prompts, sp, max_new, wb, hbm_peak, uniforms=None, T=None):
    """Runs one generation twice (warm-up, timed) and reports decode tokens/s, p50 ms per step and the HBM
    fraction of the algorithmic bytes, integrated over the contexts of the steps actually run."""
    sess.generate(prompts, sp, min(max_new, 8), uniforms=None if uniforms is None else uniforms[:, :min(max_new, 8)])
    sess.generate(prompts, sp, max_new, uniforms=uniforms)
    ids, step_ms, pre_ms = sess.generate(prompts, sp, max_new, uniforms=uniforms, timings=True)
    lens = np.array([len(p) for p in prompts])
    emitted = np.array([len(s) for s in ids]) - lens
    n_steps = int(emitted.max()) - 1      # decode forwards; the last id of a sequence needs none
    dev_s = float(np.sum(step_ms[:n_steps])) / 1e3
    tokens = int(np.sum(emitted - 1))
    nbytes = 0.0
    for i in range(n_steps):
        active = emitted - 1 > i
        ctx_sum = int(np.sum(lens[active] + i + 1))
        nbytes += sum(algorithmic_bytes_per_step(dm, int(active.sum()), 0, wb, ctx_sum=ctx_sum).values())
    return {"tokens_per_s": tokens / dev_s, "decode_steps": n_steps, "ms_per_step": dev_s / n_steps * 1e3,
            "p50_ms_per_step": float(np.median(step_ms[:n_steps])), "prefill_ms": pre_ms,
            "hbm_frac": nbytes / dev_s / 1e9 / hbm_peak, "algorithmic_mb_per_step": nbytes / n_steps / 1e6}, ids


def with_model(g, ck, preset, seed, device, precision, fn):
    dm = ck.PRESETS[preset]
    tmp = tempfile.mkdtemp(prefix="gradb_benchc_")
    path = str(ck.write_synthetic(Path(tmp) / f"{preset}.bin", dm, seed))
    try:
        out = {}
        for name, prec in precision:
            model = g.GPTModel.load(path, device, prec)
            try:
                out[name] = fn(model, dm, 2 if prec == g.BF16 else 4)
            finally:
                model.close()
        return out
    finally:
        os.remove(path)
        os.rmdir(tmp)


def bench_config1(g, ck, device, hbm_peak):
    """`small` GPT-2 block, one sequence, fp32: 16-id prompt, greedy to context 96."""
    prompt = np.random.default_rng(2001).integers(0, 5000, 16).astype(np.int32)

    def run(model, dm, wb):
        sess = g.BatchSession(model, 1, 1024)
        out = {}
        for pen in (1.0, 1.2):
            blk, _ = decode_block(sess, dm, [prompt], g.Sampling(1, 1.0, pen, 0, 1.0), 80, wb, hbm_peak)
            out[f"greedy_penalty_{pen}"] = blk
        sess.close()
        return out

    res = with_model(g, ck, "small", 1001, device, (("f32", g.FP32),), run)
    res["workload"] = "small d512 L6 H8 GELU2048 V5000 (21.5M), 1 sequence, 16-id prompt, greedy decode to context 96"
    return res


def bench_config3(g, ck, device, hbm_peak):
    """`medium` GPT-2 block, 64 ragged prompts (8..64 ids), greedy to context 256, fp32 and bf16."""
    rng = np.random.default_rng(2003)
    lens = rng.integers(8, 65, 64)
    prompts = [rng.integers(0, 16000, int(n)).astype(np.int32) for n in lens]
    keep = {}

    def run(model, dm, wb):
        sess = g.BatchSession(model, 64, 256)
        lg = sess.prefill(prompts)
        blk, ids = decode_block(sess, dm, prompts, g.Sampling(1, 1.0, 1.0, 0, 1.0), 256 - 8 + 1, wb, hbm_peak)
        keep[wb] = (lg, ids)
        sess.close()
        return blk

    res = with_model(g, ck, "medium", 1003, device, (("f32", g.FP32), ("bf16", g.BF16)), run)
    (lg32, ids32), (lg16, ids16) = keep[4], keep[2]
    p32, p16 = log_softmax64(lg32), log_softmax64(lg16)
    res["bf16_vs_fp32"] = {
        "logits_max_abs_err_over_max_abs": float(np.abs(lg16 - lg32).max() / np.abs(lg32).max()),
        "mean_kl_fp32_vs_bf16": float((np.exp(p32) * (p32 - p16)).sum(axis=-1).mean()),
        "first_id_greedy_agreement": float(np.mean([a[n] == b[n] for a, b, n in zip(ids32, ids16, lens)])),
        "mean_common_prefix_of_rollout": float(np.mean([common_prefix_frac(a, b, int(n))
                                                        for a, b, n in zip(ids32, ids16, lens)]))}
    res["workload"] = ("medium d768 L8 H12 GELU3072 V16000 (69.8M), 64 sequences, prompt lengths uniform in [8, 64], "
                       "greedy decode until every context holds 256 ids")
    return res


def bench_config5(g, ck, device, hbm_peak):
    """`modern` block with context 2048: 32 sequences, 1024-id prompts through the batched feed, greedy decode of
    1024 ids; the attention class's share and HBM fraction come from a second, per-launch-timed pass."""
    rng = np.random.default_rng(2005)
    prompts = [rng.integers(0, 16000, 1024).astype(np.int32) for _ in range(32)]
    greedy = g.Sampling(1, 1.0, 1.0, 0, 1.0)

    def run(model, dm, wb):
        sess = g.BatchSession(model, 32, 2048)
        blk, _ = decode_block(sess, dm, prompts, greedy, 1024, wb, hbm_peak)
        blk["prefill_tokens_per_s"] = 32 * 1024 / (blk["prefill_ms"] / 1e3)
        flops = 2.0 * 32 * 1024 * (dm.layers * (4 * dm.d_model ** 2 + 3 * dm.d_model * dm.d_ff)
                                   + dm.layers * 2 * dm.d_model * 1025 / 2) + 2.0 * 32 * dm.vocab * dm.d_model
        blk["prefill_tflops"] = flops / (blk["prefill_ms"] / 1e3) / 1e12
        sess.set_profiling(True)
        sess.generate(prompts, greedy, 1024)
        prof = sess.profile()
        sess.set_profiling(False)
        sess.set_profiling(True)
        sess.generate(prompts, greedy, 0)
        feed = sess.profile()
        sess.set_profiling(False)
        ms = prof["attn_decode"][0] - feed["attn_decode"][0]
        n = prof["attn_decode"][1] - feed["attn_decode"][1]
        total = sum(prof[k][0] - feed[k][0] for k in prof)
        nbytes = sum(algorithmic_bytes_per_step(dm, 32, 1024 + i + 1, wb)["attn_decode"] for i in range(1023))
        blk["attn_decode"] = {"share_of_step": ms / total, "avg_launch_us": ms * 1e3 / max(n, 1),
                              "achieved_gbs": nbytes / (ms / 1e3) / 1e9, "hbm_frac": nbytes / (ms / 1e3) / 1e9 / hbm_peak,
                              "contexts": "1025..2047"}
        sess.close()
        return blk

    res = with_model(g, ck, "modern2k", 1005, device, (("bf16", g.BF16), ("f32", g.FP32)), run)
    res["workload"] = ("modern d768 L8 H12 SwiGLU2048 V16000, context 2048, 32 sequences, 1024-id prompts (batched "
                       "feed), greedy decode of 1024 ids")
    return res


def bench_scoring(sess, dm, B, tensor_peak, peak_kind):
    """Teacher-forced scoring (`grad eval`'s shape: windows of 256 ids, losses over batches of 8) of B windows
    on the benchmark session: ids scored per second, device time and wall time with host buffers."""
    S = CONTEXT
    stream = np.random.default_rng(PROMPT_SEED + 7).integers(0, dm.vocab, B * S + 1).astype(np.int32)
    inp = np.stack([stream[i * S:i * S + S] for i in range(B)])
    tgt = np.stack([stream[i * S + 1:i * S + S + 1] for i in range(B)])
    sess.mean_loss(inp[:32], tgt[:32], 8)  # warm-up: allocates the all-row logits buffer
    dev, wall = [], []
    mean = 0.0
    for _ in range(3):
        t0 = time.perf_counter()
        mean, _ = sess.mean_loss(inp, tgt, 8)
        wall.append(time.perf_counter() - t0)
        dev.append(sess.last_score_ms / 1e3)
    ids = B * S
    d, L, V, dff = dm.d_model, dm.layers, dm.vocab, dm.d_ff
    macs = L * (4 * d * d + 3 * d * dff) + V * d                      # projections + logits, per id
    attn = L * 2 * d * (S + 1) / 2                                    # QK and PV over the causal prefix, mean per id
    flops = 2.0 * (macs + attn) * ids
    dsec = statistics.median(dev)
    return {"workload": f"{B} windows x {S} ids, batches of 8, bf16 tensor-core feed + all-position logits + "
                        "log-softmax/NLL on the device",
            "ids_per_s": ids / dsec, "device_ms": dsec * 1e3, "e2e_ids_per_s": ids / statistics.median(wall),
            "mean_loss": mean, "tflops": flops / dsec / 1e12, "tensor_peak_tflops": tensor_peak,
            "tensor_frac": flops / dsec / 1e12 / tensor_peak if tensor_peak else None, "peak_source": peak_kind}


def bench_batch1(g, ck, device, hbm_peak):
    """Single-sequence decode of the same model in fp32: 32-id prompt, greedy and sampled decode to context 256."""
    import torch
    dm = ck.PRESETS["modern"]
    tmp = tempfile.mkdtemp(prefix="gradb_bench1_")
    path = str(ck.write_synthetic(Path(tmp) / "modern.bin", dm, 1002))
    out = {"workload": "modern 69.0M, 1 sequence, 32-id prompt, decode to context 256"}
    prompt = np.random.default_rng(2002).integers(0, dm.vocab, PROMPT_LEN).astype(np.int32)
    n_new = CONTEXT - PROMPT_LEN
    draws = np.random.default_rng(2003).random((1, n_new + 1), dtype=np.float32)
    for prec_name, prec, wb in (("f32", g.FP32, 4), ("bf16w", g.BF16, 2)):
        model = g.GPTModel.load(path, device, prec)
        sess = g.BatchSession(model, 1, CONTEXT)
        for mode, sp in (("greedy", g.Sampling(1, 1.0, 1.0, 0, 1.0)), ("sampled", g.Sampling(0, 0.8, 1.1, 40, 0.9))):
            sess.generate([prompt], sp, 8, uniforms=draws[:, :8])  # warm-up
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ids, step_ms, pre_ms = sess.generate([prompt], sp, n_new + 1, uniforms=draws, timings=True)
            wall = time.perf_counter() - t0
            ms = step_ms[:n_new]
            dev_s = float(ms.sum()) / 1e3
            bytes_total = sum(sum(algorithmic_bytes_per_step(dm, 1, PROMPT_LEN + i + 1, wb).values())
                              for i in range(n_new))
            out[f"{prec_name}_{mode}"] = {
                "tokens_per_s": n_new / dev_s, "p50_ms_per_token": float(np.median(ms)),
                "p99_ms_per_token": float(np.percentile(ms, 99)), "prefill_ms": pre_ms,
                "e2e_tokens_per_s": (n_new + 1) / wall,
                "hbm_frac": bytes_total / dev_s / 1e9 / hbm_peak,
                "algorithmic_mb_per_token": bytes_total / n_new / 1e6}
        sess.close()
        model.close()
    os.remove(path)
    os.rmdir(tmp)
    return out


# ----------------------------------------------------------------------------- CPU arm

def cpu_reference(K_sample, n_seq, timed_only):
    """The reference's CPU decode on this machine's host cores, on a bounded sample of the
    workload: one independent session per host thread (single-threaded BLAS each, which is how
    M=1 products run fastest), 32-id prompt then K_sample sampled ids each."""
    os.environ.setdefault("OPENBLAS_NUM_THREADS", "1")
    os.environ.setdefault("GRADREF_SEED", "12345")
    from oracle import oracle
    g = load_package()
    from grad_cpp_b200 import checkpoint as ck
    dm = ck.PRESETS["modern"]
    cores = os.cpu_count() or 1
    n_seq = n_seq or min(cores, 64)
    tmp = tempfile.mkdtemp(prefix="gradb_cpu_")
    path = str(ck.write_synthetic(Path(tmp) / "modern.bin", dm, WEIGHT_SEED))
    use_ref = oracle.ref_available()
    if use_ref:
        R = oracle.Ref()
        devnull = os.open(os.devnull, os.O_WRONLY)
        saved = os.dup(1)
        os.dup2(devnull, 1)  # the reference prints a line from load()
        try:
            m = R.load(path)
        finally:
            os.dup2(saved, 1)
            os.close(devnull)
            os.close(saved)
    else:
        oracle.build_port()
        R = oracle.Port()
        m = R.load(path)
    feed_s = [0.0] * n_seq
    dec_s = [0.0] * n_seq

    def one(i):
        prompt = seq_prompt(i, dm.vocab)
        draws = seq_draws(i, K_sample)
        s = R.session(m)
        t0 = time.perf_counter()
        lg = None
        for t in prompt:
            _, lg = R.step(s, int(t), dm.vocab)
        t1 = time.perf_counter()
        for j in range(K_sample):
            if use_ref:
                tok, _ = R.sample_from_logits(m, lg, SAMPLER["temperature"], SAMPLER["top_k"], SAMPLER["top_p"])
            else:
                tok = R.sample(lg, SAMPLER["temperature"], SAMPLER["top_k"], SAMPLER["top_p"], float(draws[j]))
            _, lg = R.step(s, tok, dm.vocab)
        t2 = time.perf_counter()
        R.session_free(s)
        feed_s[i], dec_s[i] = t1 - t0, t2 - t1

    t0 = time.perf_counter()
    threads = [threading.Thread(target=one, args=(i,)) for i in range(n_seq)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    R.free(m)
    os.remove(path)
    os.rmdir(tmp)
    dec_wall = max(dec_s)
    res = {"value": n_seq * K_sample / dec_wall, "unit": "tokens/s", "cores": n_seq,
           "kind": "reference" if use_ref else "port",
           "sample": f"{n_seq} of the workload's sequences, one per host thread (single-threaded OpenBLAS each), "
                     f"32-id prompt fed by step() then {K_sample} sampled ids each; decode part timed",
           "host_cpus": cores, "ms_per_token_per_thread": dec_wall / K_sample * 1e3,
           "e2e_tokens_per_s": n_seq * K_sample / wall}
    return res


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    K = min(args.steps, CONTEXT - PROMPT_LEN)
    K_sample = min(K, args.cpu_tokens)
    t0 = time.perf_counter()
    res = cpu_reference(K_sample, None, False)
    line = {"impl": "reference", "metric": "decode tokens/s", "value": res["value"], "unit": "tokens/s",
            "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": K_sample, "warmup": PROMPT_LEN,
            "ms_per_step": res["ms_per_token_per_thread"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "modern d768 L8 H12 SwiGLU2048 V16000 (69.0M), CPU sample: "
                                   + res["sample"] + "; the untimed prompt feed is the warm-up",
                       "prompt_len": PROMPT_LEN},
            "cpu_baseline": res,
            "e2e": {"value": res["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
            "wall_s": time.perf_counter() - t0}
    print(json.dumps(line))


def main():
    global PROMPT_LEN
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=CONTEXT - PROMPT_LEN)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="sequences per GPU")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--cpu-tokens", type=int, default=48, help="decode ids per sequence in the CPU sample")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN,
                    help="ids per prompt (default 32, the benchmark configuration; longer prompts are for profiling)")
    ap.add_argument("--reps", type=int, default=0, help="repetitions of the complete decode (default: enough for 1 s)")
    ap.add_argument("--main-only", action="store_true",
                    help="only the timed workload: no per-kernel pass, batch-1 block or CPU baseline (for profilers)")
    ap.add_argument("--eval-only", action="store_true",
                    help="only the scoring block (256 windows x 256 ids) on one GPU, printed as one JSON line (for "
                         "profilers: the many-row GEMM and the prompt attention kernels)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    PROMPT_LEN = max(1, min(args.prompt_len, CONTEXT - 2))
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
