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


def algorithmic_bytes_per_step(dm, batch, ctx, w_bytes):
    """Bytes one decode step must move, per kernel class: weights streamed once per launch
    (w_bytes per element), fp32 activations in and out, and the K/V rows of every cached position."""
    d, f, L, V = dm.d_model, dm.d_ff, dm.layers, dm.vocab
    per_layer, logits_w = weight_elems(dm)
    act = 4
    out = {
        "embed": batch * d * act * 2,
        "norm_qkv_rope": L * (per_layer["norm_qkv_rope"] * w_bytes + batch * d * act * 4),
        "attn_decode": L * (batch * 2 * ctx * d * 4 + batch * d * act * 2),
        "attn_out_proj": L * (per_layer["attn_out_proj"] * w_bytes + batch * d * act * 3),
        "norm_ffn_up": L * (per_layer["norm_ffn_up"] * w_bytes + batch * (d + f) * act),
        "ffn_down": L * (per_layer["ffn_down"] * w_bytes + batch * (f + 2 * d) * act),
        "norm_logits": logits_w * w_bytes + batch * (d + V) * act,
        "advance": batch * 8,
        "select": batch * V * act,
    }
    return out


# ----------------------------------------------------------------------------- our arm

def run_ours(args):
    import torch
    import torch.distributed as dist

    g = load_package()
    from grad_cpp_b200 import checkpoint as ck

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
    B, K, W = args.batch, args.steps, args.warmup
    K = min(K, CONTEXT - PROMPT_LEN)
    precision = g.BF16 if args.precision == "bf16" else g.FP32
    tmp = tempfile.mkdtemp(prefix="gradb_bench_")
    path = str(ck.write_synthetic(Path(tmp) / f"modern_{rank}.bin", dm, WEIGHT_SEED))
    model = g.GPTModel.load(path, local, precision)
    stream = torch.cuda.Stream()
    sess = g.BatchSession(model, B, CONTEXT, stream=stream.cuda_stream)
    prompts = [seq_prompt(rank * B + i, dm.vocab) for i in range(B)]
    sp = g.Sampling(0, SAMPLER["temperature"], SAMPLER["penalty"], SAMPLER["top_k"], SAMPLER["top_p"])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # warm-up: W decode steps (builds the step graph, warms caches and clocks)
    draws_w = np.stack([seq_draws(rank * B + i, W + 1) for i in range(B)])
    sess.generate(prompts, sp, W + 1, uniforms=draws_w)

    draws = np.stack([seq_draws(rank * B + i, K + 1) for i in range(B)])
    from grad_cpp_b200 import sharding
    if world > 1:  # the id gather's first use (communicator set-up, allocator warm-up) stays out of the timed region
        sharding.gather_ids(np.zeros((B, CONTEXT + 1), np.int32), world, device="cuda")
    launches0 = g.lib().gradb_kernel_launches()
    clocks = ClockSampler(local)
    barrier()
    clocks.start()
    t0 = time.perf_counter()
    ids, step_ms, prefill_ms = sess.generate(prompts, sp, K + 1, uniforms=draws, timings=True)
    all_ids = sharding.gather_ids(sharding.pad_ids(ids, CONTEXT + 1), world, device="cuda")  # one NCCL all_gather
    assert all_ids.shape[0] == world * B
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    clk = clocks.stop()
    barrier()
    launches = g.lib().gradb_kernel_launches() - launches0

    dev_s = float(np.sum(step_ms[:K])) / 1e3
    dev_s, wall = sharding.max_over_ranks([dev_s, wall], world, device="cuda")
    new_ids = sum(len(s) - PROMPT_LEN for s in ids)
    assert new_ids == B * (K + 1), (new_ids, B, K)

    hbm_peak, tensor_peak, peak_kind = peaks()
    w_bytes = 2 if precision == g.BF16 else 4
    line = {
        "metric": "decode tokens/s", "value": world * B * K / dev_s, "unit": "tokens/s", "n_gpus": world,
        "steps": K, "warmup": W, "ms_per_step": dev_s / K * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16 weights, f32 accumulate, f32 KV cache" if precision == g.BF16 else "f32",
        "data": "synthetic",
        "config": {"workload": f"modern d768 L8 H12 SwiGLU2048 V16000 (69.0M), {B} sequences/GPU, "
                               f"prompt {PROMPT_LEN} ids via batched prompt feed, sampled decode context "
                               f"{PROMPT_LEN}->{PROMPT_LEN + K} (T 0.8, top-p 0.9)",
                   "batch_per_gpu": B, "prompt_len": PROMPT_LEN, "context_end": PROMPT_LEN + K,
                   "parallelism": f"sequence-sharded replicas x{world}",
                   "l2": "working set (weights + KV of 256 sequences, >1.5 GB) exceeds L2; no flush needed"},
        "p50_ms_per_step": float(np.median(step_ms[:K])),
        "prefill_ms": prefill_ms,
        "e2e": {"value": world * B * (K + 1) / wall, "unit": "tokens/s",
                "h2d_bytes_per_step": (B * PROMPT_LEN * 4 + B * (K + 1) * 4) / (K + 1),
                "d2h_bytes_per_step": (B * (CONTEXT + 2) * 4 + B * 4) / (K + 1),
                "wall_s": wall, "includes": "prompt upload, prompt feed, decode, id download"
                                            + (", NCCL all_gather of ids" if world > 1 else "")},
        "gpu_launches": int(launches),
        "clocks": clk,
    }

    if rank == 0 and not args.main_only:
        # Per-kernel device time over the same K steps, from events around every launch.
        sess.set_profiling(True)
        sess.generate(prompts, sp, K + 1, uniforms=draws)
        prof = sess.profile()
        sess.set_profiling(False)
        alg = {k: 0.0 for k in prof}
        for i in range(K):
            for k, v in algorithmic_bytes_per_step(dm, B, PROMPT_LEN + i + 1, w_bytes).items():
                alg[k] += v
        kernels = {}
        total_ms = sum(ms for ms, _ in prof.values())
        for k, (ms, n) in prof.items():
            if n == 0:
                continue
            # profile pass covers the prompt feed too; scale bytes to decode launches only for the decode-only classes
            kernels[k] = {"ms_total": round(ms, 3), "launches": n, "share": round(ms / total_ms, 4)}
        # decode-only profile: subtract the prompt-feed pass by profiling it separately
        sess.set_profiling(True)
        sess.generate(prompts, sp, 0, uniforms=None)
        feed = sess.profile()
        sess.set_profiling(False)
        dom, dom_ms = None, -1.0
        for k in kernels:
            ms = prof[k][0] - feed.get(k, (0.0, 0))[0]
            n = prof[k][1] - feed.get(k, (0.0, 0))[1]
            kernels[k].update({"decode_ms": round(ms, 3), "decode_launches": n,
                               "achieved_gbs": round(alg[k] / (ms / 1e3) / 1e9, 1) if ms > 0 else None})
            if ms > dom_ms:
                dom, dom_ms = k, ms
        n_dom = kernels[dom]["decode_launches"]
        achieved = alg[dom] / (dom_ms / 1e3) / 1e9
        line["kernels"] = kernels
        line["roofline"] = {"kernel": dom, "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                            "frac": achieved / hbm_peak, "peak_source": peak_kind,
                            "algorithmic_bytes_per_launch": alg[dom] / n_dom,
                            "avg_launch_us": dom_ms * 1e3 / n_dom,
                            "traffic": ncu_traffic(dom, alg[dom] / n_dom)}
        step_bytes = sum(sum(algorithmic_bytes_per_step(dm, B, PROMPT_LEN + i + 1, w_bytes).values()) for i in range(K))
        line["step_roofline"] = {"algorithmic_bytes_per_step_avg": step_bytes / K,
                                 "achieved_gbs": step_bytes / dev_s / 1e9, "frac": step_bytes / dev_s / 1e9 / hbm_peak}
        line["eval"] = bench_scoring(sess, dm, B, tensor_peak, peak_kind)
        if world == 1:
            line["batch1"] = bench_batch1(g, ck, local, hbm_peak)
            line["cpu_baseline"] = cpu_reference(K_sample=args.cpu_tokens, n_seq=None, timed_only=True)

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
    ap.add_argument("--main-only", action="store_true",
                    help="only the timed workload: no per-kernel pass, batch-1 block or CPU baseline (for profilers)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    PROMPT_LEN = max(1, min(args.prompt_len, CONTEXT - 2))
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
