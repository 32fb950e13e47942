#!/usr/bin/env python
"""Benchmark of the MLA absorbed-attention decode path on B200.

Workload (BASELINE.json configs[2], the one the headline target is quoted on): DeepSeek-V3-shaped
MLA decode — 61 layers, 128 heads, batch 64, context 16384 per sequence, bf16 paged latent cache
(64-token pages, shuffled block tables), one token appended per sequence per step.  One "step" is
one decode step of the whole attention stack: for every layer append(new c_kv/k_rope rows) and
absorbed attention (q absorb -> split-KV attention -> merge -> W_UV), three kernel launches per layer
through mla_step_layers (the append runs in spare blocks of the absorb launch).  Inputs are seeded synthetic
tensors of the model's shapes; with N GPUs the batch of 64 is sharded by sequence (no collective on
the data path), so total work is fixed ("strong" scaling).

  python bench.py [--gpus N] [--steps K] [--warmup W]            # this implementation
  python bench.py --impl reference ...                           # the reference's CPU path

Prints ONE JSON line (rank 0).  Besides the headline keys the line carries sub-objects for the other
configurations of the workload family, each measured in a few seconds on a handful of layers:
  kv_range  one 131072-token sequence cut into `world` page-aligned KV ranges (world = 1 is the control): per layer
            partial softmax states -> ONE all-gather (NCCL) -> merge + W_UV; with its own parity check
  ragged    128 decode rows with log-uniform lengths 256..32768 (1 GPU): step time, planner balance
  v2lite    16 heads, 27 layers, batch 32, ctx 8192, fp16 (1 GPU): whole-step and attention-kernel fractions
  prefill   4 sequences x one 4096-token chunk, causal (1 GPU)
  verify    speculative-decode verify of K+1 = 5 positions per sequence with rollback, batch 64 (1 GPU)
(--no-extras skips them.)
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from mugen_b200 import synth  # noqa: E402

METRIC, UNIT = "mla_decode_tokens_per_s", "tokens/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one attention launch at the default workload, from an ncu capture.
# The figure belongs to one version of the kernel's source: it is reported only while that file still hashes to the
# value below (otherwise `traffic` is null until the capture is repeated).
NCU_TRAFFIC = {"kernel": "tcgen05-pair128", "source": "mugen_b200/csrc/mla_decode_tc5_pair2.cu",
               "source_sha256_16": "b8d4546c35b93d5f", "bytes_per_launch": 1.2647e9}
# The attention kernel is timed live by CUDA events inside the library on every 7th launch of the timed region
# (7 is coprime to 61 layers, so every layer gets sampled over the steps): an event between two kernels stops
# the next one from becoming resident while the previous drains, and bracketing every launch would slow the
# step that `value` reports by about 3 %.
KERNEL_EVENT_STRIDE = 7


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--layers", type=int, default=61)
    p.add_argument("--batch", type=int, default=64)
    p.add_argument("--ctx", type=int, default=16384)
    p.add_argument("--heads", type=int, default=128)
    p.add_argument("--dtype", default="bf16", choices=["bf16", "f16"])
    p.add_argument("--kernel", default="auto", choices=["auto", "mma", "tcgen05", "tcgen05-pair128", "tcgen05-t16"])
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-cpu", action="store_true")
    p.add_argument("--no-extras", action="store_true", help="skip the kv_range / ragged / v2lite / prefill sub-objects")
    p.add_argument("--only", default="", help="run only this sub-benchmark (kv_range, ragged, v2lite, prefill) and print it")
    return p.parse_args()


def workload_name(a) -> str:
    shape = (a.layers, a.heads, a.batch, a.ctx, a.dtype)
    if shape == (61, 128, 64, 16384, "bf16"):
        tag = "deepseek-v3-shaped MLA decode (configs[2])"
    elif shape == (27, 16, 32, 8192, "f16"):
        tag = "deepseek-v2-lite-shaped MLA decode (configs[1])"
    else:
        tag = "MLA decode (not one of BASELINE.json's configs)"
    return (f"{tag}: {a.layers} layers, {a.heads} heads, batch {a.batch}, "
            f"ctx {a.ctx}, {a.dtype} paged latent cache, page 64")


def ncu_traffic(kernel_name: str, a, seqs_on_this_gpu: int):
    """Per-launch DRAM traffic of the attention kernel from the committed ncu capture, scaled by the sequences this
    GPU streams; None when the capture does not describe the kernel source or the workload that just ran."""
    import hashlib
    try:
        with open(os.path.join(ROOT, NCU_TRAFFIC["source"]), "rb") as f:
            h = hashlib.sha256(f.read()).hexdigest()[:16]
    except OSError:
        return None
    if h != NCU_TRAFFIC["source_sha256_16"] or kernel_name != NCU_TRAFFIC["kernel"] or (a.heads, a.ctx) != (128, 16384):
        return None
    return NCU_TRAFFIC["bytes_per_launch"] * seqs_on_this_gpu / 64.0


def algo_bytes_layer_step(lens, H: int, n_new_rows: int | None = None) -> float:
    """Algorithmic bytes of one layer-step: each cache byte once, the appended rows, q in, out, both weights once,
    the block tables (16-bit storage)."""
    B = len(lens) if n_new_rows is None else n_new_rows
    return (sum(lens) * 1152.0 + B * 1152.0 + B * H * (192 + 128) * 2.0 + 2.0 * H * 128 * 512 * 2
            + sum((n + 63) // 64 for n in lens) * 4.0)


def measured_peak_tflops():
    """(burst, sustained) bf16 matmul rate measured on this pool, or the stated fallbacks."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            j = json.load(f)
        return float(j["bf16_tflops"]), float(j.get("bf16_tflops_sustained", 0.0)) or None
    except (OSError, ValueError, KeyError):
        return 1590.0, 1400.0


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's own cpu_mla_attention (oracle/_ref), else the port (oracle/)
# ------------------------------------------------------------------------------------------------
class CpuArm:
    def __init__(self, a):
        from oracle import binding
        self.a = a
        self.ref = binding.reference()
        self.ora = binding.oracle()
        self.kind = "reference" if self.ref is not None else "port"
        self.cores = os.cpu_count() or 1
        rng = np.random.default_rng(42)
        H = a.heads
        # values exact in bf16 and f16 alike: the reference is f16-only
        fix = synth.both_representable
        self.w_uk = synth.to_bits(fix(rng.standard_normal((H * 128, 512), np.float32) * np.float32(0.02)), synth.DT_F16)
        self.w_uv = synth.to_bits(fix(rng.standard_normal((H * 128, 512), np.float32) * np.float32(0.02)), synth.DT_F16)
        self.cache = synth.to_bits(fix(rng.standard_normal((a.ctx, 576), np.float32)), synth.DT_F16)
        self.q1 = synth.to_bits(fix(rng.standard_normal((1, H, 192), np.float32) * np.float32(0.9)), synth.DT_F16)

    def run(self, n_seq: int, threads: int) -> float:
        """Seconds for one layer's attention over n_seq sequences of ctx tokens.  Every sequence reads the SAME
        18.9 MB cache buffer, so the host's caches serve part of it: the arithmetic per call is unchanged, the
        memory side flatters the CPU (stated in `sample`)."""
        a = self.a
        q = np.ascontiguousarray(np.repeat(self.q1, n_seq, axis=0))
        caches = [self.cache] * n_seq
        lens = [a.ctx] * n_seq
        t0 = time.perf_counter()
        if self.ref is not None:
            self.ref.attention_batch(q, caches, lens, self.w_uk, self.w_uv, synth.W_F16, a.heads, threads)
        else:
            self.ora.attention_batch(q, caches, lens, self.w_uk, self.w_uv, synth.W_F16, a.heads, synth.DT_F16, threads)
        return time.perf_counter() - t0

    def plan(self, budget_s: float):
        """(sequences per sample, threads, seconds for one sequence on one thread) so that one
        sample costs about budget_s of wall clock with every core busy."""
        t1 = self.run(1, 1)
        per_thread = max(1, int(budget_s / max(t1, 1e-3)))
        n = max(1, min(self.a.batch, self.cores * per_thread))
        return n, min(self.cores, n), t1

    def tokens_per_s(self, n_seq: int, seconds: float) -> float:
        # one layer was timed; a decode step runs `layers` of them
        return n_seq / (seconds * self.a.layers)


def run_reference_arm(a, rank: int):
    if rank != 0:
        return
    arm = CpuArm(a)
    budget = 150.0 / max(1, a.steps + a.warmup)
    n_seq, threads, _ = arm.plan(budget)
    for _ in range(a.warmup):
        arm.run(n_seq, threads)
    t = 0.0
    for _ in range(a.steps):
        t += arm.run(n_seq, threads)
    per = t / max(1, a.steps)
    v = arm.tokens_per_s(n_seq, per)
    sample = (f"per step: one layer of cpu_mla_attention over {n_seq} sequences (ctx {a.ctx}, {a.heads} heads, f16) "
              f"on {threads} host threads, all sequences reading one shared cache buffer (favours the CPU's caches); "
              f"tokens/s = sequences / (time x {a.layers} layers)")
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": 1e3 * a.batch / v,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": workload_name(a)},
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": arm.kind, "sample": sample},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap,timestamp")

    def __init__(self, device_index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={device_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def mark_begin(self):
        """The timed region starts now (the sampler itself is started earlier: nvidia-smi needs a few hundred
        milliseconds before its first line)."""
        self.t_begin = time.time()

    def stop(self):
        t_end = time.time()
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons, pw = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = [[x.strip() for x in ln.split(",")] for ln in out.strip().splitlines()]
        lines = [f for f in lines if len(f) >= 8]
        t_begin = getattr(self, "t_begin", None)
        if t_begin is not None:                     # keep the samples taken inside the timed region (+- one period)
            import datetime
            inside = []
            for f in lines:
                try:
                    ts = datetime.datetime.strptime(f[7], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                except ValueError:
                    continue
                if t_begin - 0.1 <= ts <= t_end + 0.1:
                    inside.append(f)
            if inside:
                lines = inside
        for f in lines:
            try:
                sm.append(float(f[0])); mx.append(float(f[1])); pw.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def run_ours(a):
    import torch
    import torch.distributed as dist

    from mugen_b200 import capi
    from mugen_b200.mla import MlaContext

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this implementation has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    assert a.batch % world == 0, "batch must divide over the ranks"
    B = a.batch // world                      # sequences owned by this rank
    H, L = a.heads, a.layers
    dt = synth.DT_BF16 if a.dtype == "bf16" else synth.DT_F16
    tdt = torch.bfloat16 if a.dtype == "bf16" else torch.float16
    kernel = {"auto": capi.KERNEL_AUTO, "mma": capi.KERNEL_MMA, "tcgen05": capi.KERNEL_TCGEN05, "tcgen05-pair128": capi.KERNEL_TCGEN05_PAIR128,
              "tcgen05-t16": capi.KERNEL_TCGEN05_T16}[a.kernel]
    total_steps = a.warmup + a.steps + (0 if a.no_e2e else a.warmup + a.steps)
    start_len = a.ctx - 1 - a.warmup          # the first timed step attends exactly ctx rows
    pages_per_seq = (start_len + total_steps + 64 + 63) // 64
    ctx = MlaContext(n_layers=L, n_heads=H, dtype=dt, n_pages=B * pages_per_seq + 8, max_seqs=B,
                     max_seq_len=pages_per_seq * 64, device=local, kernel=kernel,
                     rope_theta=10000.0, rope_scaling_factor=40.0, rope_original_ctx=4096, rms_norm_eps=1e-6)
    ctx.shuffle_free_pages(42 + rank)

    rng = np.random.default_rng(42 + rank)
    wt = synth.W_BF16 if dt == synth.DT_BF16 else synth.W_F16
    w_uk = synth.to_bits(rng.standard_normal((H * 128, 512), np.float32) * np.float32(0.02), dt)
    w_uv = synth.to_bits(rng.standard_normal((H * 128, 512), np.float32) * np.float32(0.02), dt)
    norm = synth.to_bits(np.ones(512, np.float32), dt)
    for l in range(L):
        ctx.set_layer_weights(l, w_uk, w_uv, wt, norm)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(42 + rank)
    seqs = [ctx.seq_create() for _ in range(B)]
    for l in range(L):
        for s in seqs:
            rows = torch.randn((start_len, 576), device="cuda", dtype=torch.float32, generator=gen).to(tdt)
            ctx.write_rows(l, s, 0, rows.view(torch.int16))
    for s in seqs:
        ctx.advance_seq_len(s, start_len)
    q = (torch.randn((L, B, H, 192), device="cuda", dtype=torch.float32, generator=gen) * 0.9).to(tdt).view(torch.int16)
    kv = torch.randn((L, B, 576), device="cuda", dtype=torch.float32, generator=gen).to(tdt).view(torch.int16)
    out = torch.zeros((L, B, H, 128), device="cuda", dtype=torch.int16)
    assert ctx.status() == 0

    def barrier():
        if world > 1:
            dist.barrier()

    def one_step():
        ctx.step_begin(seqs)
        ctx.step_layers(0, L, kv, q, out)      # per layer: append, absorb, split-KV attention, merge + W_UV
        ctx.step_end()

    clocks = ClockSampler(local) if rank == 0 else None
    for _ in range(a.warmup):
        one_step()
    torch.cuda.synchronize()
    lens_sum = 0
    launches0 = ctx.launch_count()
    ctx.profile_enable(KERNEL_EVENT_STRIDE if L >= KERNEL_EVENT_STRIDE else 1)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(); torch.cuda.synchronize()
    if clocks:
        clocks.mark_begin()
    ev0.record()
    for _ in range(a.steps):
        lens_sum += sum(ctx.seq_len(s) + 1 for s in seqs)
        one_step()
    ev1.record()
    torch.cuda.synchronize(); barrier()
    ms = ev0.elapsed_time(ev1)
    ctx.profile_enable(False)
    n_attn, attn_ms = ctx.profile_read()
    launches = ctx.launch_count() - launches0
    clk = clocks.stop() if clocks else None
    assert ctx.status() == 0, "a kernel flagged a fault during the timed region"

    t = torch.tensor([ms, float(launches), float(lens_sum), attn_ms, float(n_attn)], device="cuda", dtype=torch.float64)
    if world > 1:
        tmax = t.clone(); dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone(); dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        ms = float(tmax[0]); launches = int(tsum[1]); lens_total = float(tsum[2])
    else:
        lens_total = float(lens_sum)
    tokens = a.batch * a.steps
    value = tokens / (ms * 1e-3)

    # ---- roofline of the dominant kernel (split-KV attention), this rank's launches
    peak, peak_src = measured_peak_gbs()
    rows_per_launch = lens_sum / max(1, a.steps)                      # cache rows streamed per launch
    algo_bytes = rows_per_launch * 576 * 2 + B * H * 576 * 2 + (rows_per_launch / 64) * 4
    per_launch_s = (attn_ms * 1e-3) / max(1, n_attn)
    achieved = algo_bytes / per_launch_s / 1e9 if per_launch_s > 0 else 0.0
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": ncu_traffic(ctx.kernel_name(), a, B), "kernel": f"split-KV attention ({ctx.kernel_name()})",
                "peak_source": peak_src, "algorithmic_bytes_per_launch": algo_bytes,
                "avg_launch_us": per_launch_s * 1e6, "launches_timed": n_attn}
    # The same launch seen from the tensor side: 2 * (576 + 512) flops per head and cached row. At 128 heads that is
    # 242 flops per cache byte, the machine's own ratio of measured matmul rate to measured copy rate, so the kernel
    # sits at the corner of the roofline and both fractions are reported.
    tf_burst, tf_sust = measured_peak_tflops()
    flops = rows_per_launch * H * 2.0 * (576 + 512)
    tflops = flops / per_launch_s / 1e12 if per_launch_s > 0 else 0.0
    roofline["tensor_side"] = {"achieved": tflops, "unit": "TFLOP/s", "flops_per_launch": flops,
                               "peak_burst": tf_burst, "frac_of_burst": tflops / tf_burst if tf_burst else None,
                               "peak_sustained": tf_sust, "frac_of_sustained": tflops / tf_sust if tf_sust else None,
                               "flops_per_cache_byte": H * 2.0 * (576 + 512) / 1152.0}
    # whole layer-step view of the same thing (all kernels of the step, cache term only)
    latent_gbs = lens_total * 576 * 2 * L / (ms * 1e-3) / 1e9 / world   # per GPU

    # ---- end to end through the host-buffer entry point
    e2e = None
    if not a.no_e2e:
        hq = q.cpu().pin_memory(); hkv = kv.cpu().pin_memory()
        hout = torch.zeros((L, B, H, 128), dtype=torch.int16).pin_memory()

        def host_step():
            ctx.step_begin(seqs)
            for l in range(L):
                ctx.step_layer_host(l, hkv[l], hq[l], hout[l])
            ctx.step_end()
            torch.cuda.current_stream().synchronize()   # the step's result is read on the host

        for _ in range(a.warmup):
            host_step()
        barrier(); torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            host_step()
        e1.record(); torch.cuda.synchronize(); barrier()
        e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3)
        et = torch.tensor([e_ms], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(et, op=dist.ReduceOp.MAX)
        e2e = {"value": tokens / (float(et[0]) * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": int(world * L * (B * 576 * 2 + B * H * 192 * 2)),
               "d2h_bytes_per_step": int(world * L * B * H * 128 * 2),
               "api": "mla_step_begin / mla_step_layer_host (page-locked host buffers, copies on the context's copy streams overlap the layers' kernels) / mla_step_end (returns when the outputs are on the host), stream synchronised every step"}
        assert ctx.status() == 0

    cpu = None
    if rank == 0 and world == 1 and not a.no_cpu:
        arm = CpuArm(a)
        n_seq, threads, _ = arm.plan(15.0)
        sec = arm.run(n_seq, threads)
        cpu = {"value": arm.tokens_per_s(n_seq, sec), "unit": UNIT, "cores": threads, "kind": arm.kind,
               "sample": f"one layer of cpu_mla_attention over {n_seq} sequences (ctx {a.ctx}, {a.heads} heads, f16) that "
                         f"share one cache buffer, {sec:.2f} s on {threads} threads; scaled by {a.layers} layers"}

    kernel_name = ctx.kernel_name()
    ctx.close()
    del q, kv, out
    torch.cuda.empty_cache()

    line = None
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
                "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": a.dtype, "data": "synthetic",
                "config": {"workload": workload_name(a), "sequences_per_gpu": B, "sharding": f"batch over {world} GPU(s)",
                           "kernel": kernel_name,
                           "l2_policy": "inputs larger than L2: every layer-step streams its own >= 150 MB of cache"},
                "latent_kv_gbs_per_gpu": latent_gbs, "latent_kv_frac_of_8tbs": latent_gbs / 8000.0,
                "latent_kv_frac_of_measured_peak": latent_gbs / peak,
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clk}
    if not a.no_extras:
        extras = run_extras(a, world, rank, local, only="")
        if line is not None:
            line.update(extras)
    if line is not None:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# The other configurations of the workload family, a few seconds each (sub-objects of the JSON line)
# ------------------------------------------------------------------------------------------------
ROPE_KW = dict(rope_theta=10000.0, rope_scaling_factor=40.0, rope_original_ctx=4096, rms_norm_eps=1e-6)


def _weights(ctx, L, H, dt, seed):
    rng = np.random.default_rng(seed)
    wt = synth.W_BF16 if dt == synth.DT_BF16 else synth.W_F16
    w_uk = synth.to_bits(rng.standard_normal((H * 128, 512), np.float32) * np.float32(0.02), dt)
    w_uv = synth.to_bits(rng.standard_normal((H * 128, 512), np.float32) * np.float32(0.02), dt)
    norm = synth.to_bits(np.ones(512, np.float32), dt)
    for l in range(L):
        ctx.set_layer_weights(l, w_uk, w_uv, wt, norm)
    return w_uk, w_uv, wt, norm


def _time_steps(torch, fn, warmup, steps):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _decode_case(torch, lens, H, L, dt, tdt, seed, kernel=0, device=0):
    """A context holding len(lens) sequences of the given lengths in every one of L layers, plus step inputs."""
    from mugen_b200.mla import MlaContext
    B = len(lens)
    pages = sum((n + 16 + 63) // 64 + 1 for n in lens)
    ctx = MlaContext(n_layers=L, n_heads=H, dtype=dt, n_pages=pages + 8, max_seqs=B, max_seq_len=max(lens) + 128,
                     device=device, kernel=kernel, **ROPE_KW)
    ctx.shuffle_free_pages(seed)
    _weights(ctx, L, H, dt, seed)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    seqs = [ctx.seq_create() for _ in range(B)]
    for l in range(L):
        for s, n in zip(seqs, lens):
            rows = torch.randn((n, 576), device="cuda", dtype=torch.float32, generator=gen).to(tdt)
            ctx.write_rows(l, s, 0, rows.view(torch.int16))
    for s, n in zip(seqs, lens):
        ctx.advance_seq_len(s, n)
    q = (torch.randn((L, B, H, 192), device="cuda", dtype=torch.float32, generator=gen) * 0.9).to(tdt).view(torch.int16)
    kv = torch.randn((L, B, 576), device="cuda", dtype=torch.float32, generator=gen).to(tdt).view(torch.int16)
    out = torch.zeros((L, B, H, 128), device="cuda", dtype=torch.int16)
    return ctx, seqs, q, kv, out


def _decode_numbers(torch, ctx, seqs, q, kv, out, lens, H, L, peak, warmup=3, steps=5):
    """Whole-step and attention-kernel numbers of plain decode steps over the given context."""
    def step():
        ctx.step_begin(seqs)
        ctx.step_layers(0, L, kv, q, out)
        ctx.step_end()
    ms = _time_steps(torch, step, warmup, steps)
    ctx.profile_enable(1)
    step()
    torch.cuda.synchronize()
    n_attn, attn_ms = ctx.profile_read()
    ctx.profile_enable(False)
    assert ctx.status() == 0
    cur = [n + warmup + steps + 1 for n in lens]                     # lengths attended by the profiled step
    B = len(lens)
    step_bytes = algo_bytes_layer_step(cur, H)
    attn_bytes = sum(cur) * 1152.0 + B * H * 576 * 2 + sum((n + 63) // 64 for n in cur) * 4.0
    attn_us = attn_ms * 1e3 / max(1, n_attn)
    w, lo, hi = ctx.step_balance()
    return {"layers": L, "ms_per_step": ms, "us_per_layer_step": ms * 1e3 / L,
            "tokens_per_s_this_many_layers": B / (ms * 1e-3),
            "layer_step_algorithmic_bytes": step_bytes, "whole_step_frac_of_measured_peak": step_bytes * L / (ms * 1e-3) / 1e9 / peak,
            "attention_kernel": ctx.kernel_name(), "attention_kernel_us": attn_us,
            "attention_kernel_frac_of_measured_peak": attn_bytes / (attn_us * 1e-6) / 1e9 / peak if attn_us > 0 else None,
            "planner": {"workers": w, "min_pages": lo, "max_pages": hi}}


def sub_ragged(torch, peak):
    """BASELINE.json configs[4], decode part: 128 sequences with log-uniform lengths 256..32768 in one step."""
    lens = synth.ragged_lengths(42, 128, 256, 32768)
    H, L = 128, 4
    ctx, seqs, q, kv, out = _decode_case(torch, lens, H, L, synth.DT_BF16, torch.bfloat16, 4242)
    r = _decode_numbers(torch, ctx, seqs, q, kv, out, lens, H, L, peak)
    ctx.close()
    r.update({"workload": "configs[4] decode rows: 128 sequences, lengths log-uniform 256..32768 (seed 42), 128 heads, bf16",
              "tokens_cached": int(sum(lens)), "tokens_per_s_61_layers_scaled": 128 / (r["us_per_layer_step"] * 61e-6)})
    return r


def sub_v2lite(torch, peak):
    """BASELINE.json configs[1]: 16 heads, 27 layers, batch 32, ctx 8192, fp16."""
    H, L, B, S = 16, 27, 32, 8192
    lens = [S - 9] * B
    ctx, seqs, q, kv, out = _decode_case(torch, lens, H, L, synth.DT_F16, torch.float16, 1717)
    r = _decode_numbers(torch, ctx, seqs, q, kv, out, lens, H, L, peak)
    ctx.close()
    r.update({"workload": "deepseek-v2-lite-shaped MLA decode (configs[1]): 27 layers, 16 heads, batch 32, ctx 8192, f16 paged latent cache",
              "tokens_per_s": r.pop("tokens_per_s_this_many_layers")})
    return r


def sub_kv_range(torch, dist, world, rank, local, peak):
    """BASELINE.json configs[3]: ONE sequence of 131072 tokens, 128 heads, bf16, cut into `world` contiguous
    page-aligned KV ranges (world = 1: the control).  Per layer every rank computes the partial softmax state
    (m, l, acc[512]) of its range for the replicated query, ONE all-gather moves the states, every rank merges
    them and applies W_UV.  The tail rank appends the step's new row."""
    from mugen_b200 import sharding
    from mugen_b200.mla import MlaContext
    H, L, S, dt, tdt = 128, 4, 131072, synth.DT_BF16, torch.bfloat16
    S0 = S - 8                                                       # the timed steps attend about S rows
    a_, b_ = sharding.kv_range_slices(S0, world)[rank]
    owner = rank == world - 1
    n_local = b_ - a_
    ctx = MlaContext(n_layers=L, n_heads=H, dtype=dt, n_pages=(n_local + 64) // 64 + 4, max_seqs=1,
                     max_seq_len=n_local + 256, max_position=S + 256, device=local, **ROPE_KW)
    w_uk, w_uv, wt, norm = _weights(ctx, L, H, dt, 99)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2024)                                            # every rank draws the same sequence
    s = ctx.seq_create()
    ctx.seq_set_base(s, a_)
    layer0_rows = None
    for l in range(L):
        rows = torch.randn((S0, 576), device="cuda", dtype=torch.float32, generator=gen).to(tdt).view(torch.int16)
        if n_local:
            ctx.write_rows(l, s, 0, rows[a_:b_].contiguous())
        if l == 0 and rank == 0:
            layer0_rows = rows
        del rows
    ctx.advance_seq_len(s, n_local)
    q = (torch.randn((L, 1, H, 192), device="cuda", dtype=torch.float32, generator=gen) * 0.9).to(tdt).view(torch.int16)
    kv = torch.randn((L, 1, 576), device="cuda", dtype=torch.float32, generator=gen).to(tdt).view(torch.int16)
    out = torch.zeros((L, 1, H, 128), device="cuda", dtype=torch.int16)
    partial = torch.zeros((1, H, sharding.PART), dtype=torch.float32, device="cuda")
    gathered = torch.zeros((world, 1, H, sharding.PART), dtype=torch.float32, device="cuda")
    ag_events = []

    def exchange(timed):
        if world > 1:
            if timed:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            dist.all_gather_into_tensor(gathered.view(-1, H, sharding.PART), partial)
            if timed:
                e1.record()
                ag_events.append((e0, e1))
        else:
            gathered.copy_(partial.view(1, 1, H, sharding.PART))

    def step(timed=False):
        ctx.step_begin([s], [1 if owner else 0])
        for l in range(L):
            ctx.step_layer_partial(l, kv[l] if owner else None, q[l], partial)
            exchange(timed)
            ctx.merge_partials(l, world, 1, gathered, out[l])
        ctx.step_end()

    # ---- parity of the first step: against the unsplit sequence in one context on rank 0, and against the CPU
    step()
    torch.cuda.synchronize()
    parity = None
    if rank == 0:
        whole = MlaContext(n_layers=1, n_heads=H, dtype=dt, n_pages=(S0 + 64) // 64 + 4, max_seqs=1,
                           max_seq_len=S0 + 256, device=local, **ROPE_KW)
        whole.set_layer_weights(0, w_uk, w_uv, wt, norm)
        ws = whole.seq_create()
        whole.write_rows(0, ws, 0, layer0_rows)
        whole.advance_seq_len(ws, S0)
        out_w = torch.zeros((1, H, 128), device="cuda", dtype=torch.int16)
        whole.step_begin([ws])
        whole.step_append(0, kv[0])
        whole.step_attend(0, q[0], out_w)
        whole.step_end()
        torch.cuda.synchronize()
        got = out[0].cpu().numpy().view(np.uint16)[0]
        mx, rl = synth.error_norms(got, out_w.cpu().numpy().view(np.uint16)[0], dt, dt)
        parity = {"vs_unsplit_single_context": {"max_abs": mx, "rel_l2": rl}}
        try:                                                         # the CPU checker on 8 heads (checker only, untimed)
            from oracle import binding
            cache = whole.read_rows(0, ws, 0, S0 + 1)
            h8 = 8
            want = binding.oracle().attention(q[0].cpu().numpy().view(np.uint16)[0, :h8].copy(), cache, S0 + 1,
                                              w_uk[:h8 * 128].copy(), w_uv[:h8 * 128].copy(), wt, h8, dt)
            mx, rl = synth.error_norms(got[:h8], want, dt, dt)
            parity["vs_cpu_checker_heads_0_7"] = {"max_abs": mx, "rel_l2": rl}
        except Exception as e:                                       # the checker library did not travel
            parity["vs_cpu_checker_heads_0_7"] = {"unavailable": str(e)[:120]}
        parity["tolerance"] = {"max_abs": 2e-2, "rel_l2": 5e-3}
        whole.close()
        del layer0_rows
    if world > 1:
        dist.barrier()
    warm, steps = 2, 4
    ms = _time_steps(torch, step, warm, steps)
    step(timed=True)
    torch.cuda.synchronize()
    ag_us = float(np.mean([a.elapsed_time(b) for a, b in ag_events]) * 1e3) if ag_events else 0.0
    assert ctx.status() == 0
    t = torch.tensor([ms, ag_us], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ag_us = float(t[0]), float(t[1])
    ctx.close()
    us_layer = ms * 1e3 / L
    per_gpu_bytes = (S / world) * 1152.0
    return {"workload": f"configs[3]: one sequence, ctx {S}, 128 heads, bf16, KV range split over {world} GPU(s), {L} layers timed",
            "us_per_layer_step": us_layer, "all_gather_us": ag_us,
            "all_gather_bytes_per_gpu": H * sharding.PART * 4,
            "latent_kv_gbs_per_gpu": per_gpu_bytes / (us_layer * 1e-6) / 1e9,
            "latent_kv_frac_of_measured_peak_per_gpu": per_gpu_bytes / (us_layer * 1e-6) / 1e9 / peak,
            "tokens_per_s_61_layers_scaled": 1.0 / (us_layer * 61e-6), "parity": parity,
            "timing": "CUDA events over 4 steps after 2 warm-up steps, max over ranks"}


def sub_prefill(torch, peak):
    """BASELINE.json configs[4], chunk part: 4 sequences, each appending one 4096-token chunk in ONE step, causal
    (token t attends [0, start+t+1)), at start_position 0 and 8192; 128 heads, bf16, one layer timed."""
    from mugen_b200.mla import MlaContext
    H, N, C, dt, tdt = 128, 4096, 4, synth.DT_BF16, torch.bfloat16
    res = {"workload": "configs[4] chunks: 4 sequences x one 4096-token chunk in one step, causal, 128 heads, bf16, 1 layer"}
    for start in (0, 8192):
        R = N * C
        ctx = MlaContext(n_layers=1, n_heads=H, dtype=dt, n_pages=C * ((start + N) // 64 + 2) + 8, max_seqs=C,
                         max_seq_len=start + N + 64, max_rows=R, **ROPE_KW)
        _weights(ctx, 1, H, dt, 7)
        gen = torch.Generator(device="cuda")
        gen.manual_seed(77)
        seqs = [ctx.seq_create() for _ in range(C)]
        if start:
            for sq in seqs:
                rows = torch.randn((start, 576), device="cuda", dtype=torch.float32, generator=gen).to(tdt)
                ctx.write_rows(0, sq, 0, rows.view(torch.int16))
                ctx.advance_seq_len(sq, start)
        q = (torch.randn((1, R, H, 192), device="cuda", dtype=torch.float32, generator=gen) * 0.9).to(tdt).view(torch.int16)
        kv = torch.randn((1, R, 576), device="cuda", dtype=torch.float32, generator=gen).to(tdt).view(torch.int16)
        out = torch.zeros((1, R, H, 128), device="cuda", dtype=torch.int16)

        def step():
            ctx.step_begin(seqs, [N] * C)
            ctx.step_layers(0, 1, kv, q, out)
            ctx.step_end()
            for sq in seqs:                                          # roll the chunk back: the next step appends it again
                ctx.truncate(sq, start)
        ms = _time_steps(torch, step, 1, 3)
        assert ctx.status() == 0
        pairs = C * (N * start + N * (N + 1) // 2)                   # (query token, cached token) pairs
        expand = C * (start + N) * H * 2.0 * 512 * 256                 # latent rows -> per-head keys and values
        res[f"start_{start}"] = {"ms_per_layer_step": ms, "chunk_tokens_per_s_one_layer": R / (ms * 1e-3),
                                 "chunk_tokens_per_s_61_layers_scaled": R / (ms * 1e-3) / 61,
                                 "tflops_expanded_form": (pairs * H * 2.0 * (192 + 128) + expand) / (ms * 1e-3) / 1e12,
                                 "tflops_if_counted_in_absorbed_form": pairs * H * 2.0 * (576 + 512) / (ms * 1e-3) / 1e12,
                                 "path": "append + gather + key/value expansion (tcgen05 GEMM) + causal flash attention (tcgen05), per chunk"}
        ctx.close()
        del q, kv, out
        torch.cuda.empty_cache()
    return res


def sub_verify(torch, peak):
    """The reference's speculative-decode verify pass at scale (uspp_scheduler.cpp:550-580, 222-237): per step every
    sequence verifies K+1 = 5 positions as one small causal chunk, then rolls back to ctx + accepted + 1 rows."""
    H, L, B, S, K1 = 128, 2, 64, 16384, 5
    lens = [S - 64] * B
    ctx, seqs, _, _, _ = _decode_case(torch, lens, H, L, synth.DT_BF16, torch.bfloat16, 515)
    ctx.close()
    from mugen_b200.mla import MlaContext
    pages = sum((n + 64 + 63) // 64 + 1 for n in lens)
    ctx = MlaContext(n_layers=L, n_heads=H, dtype=synth.DT_BF16, n_pages=pages + 8, max_seqs=B, max_seq_len=S + 128,
                     max_rows=B * K1, **ROPE_KW)
    _weights(ctx, L, H, synth.DT_BF16, 515)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(515)
    seqs = [ctx.seq_create() for _ in range(B)]
    for l in range(L):
        for sq, n in zip(seqs, lens):
            rows = torch.randn((n, 576), device="cuda", dtype=torch.float32, generator=gen).to(torch.bfloat16)
            ctx.write_rows(l, sq, 0, rows.view(torch.int16))
    for sq, n in zip(seqs, lens):
        ctx.advance_seq_len(sq, n)
    R = B * K1
    q = (torch.randn((L, R, H, 192), device="cuda", dtype=torch.float32, generator=gen) * 0.9).to(torch.bfloat16).view(torch.int16)
    kv = torch.randn((L, R, 576), device="cuda", dtype=torch.float32, generator=gen).to(torch.bfloat16).view(torch.int16)
    out = torch.zeros((L, R, H, 128), device="cuda", dtype=torch.int16)
    rng = np.random.default_rng(5)
    cur = list(lens)

    def step():
        ctx.step_begin(seqs, [K1] * B)
        ctx.step_layers(0, L, kv, q, out)
        ctx.step_end()
        acc = rng.integers(0, K1, B)
        for b in range(B):
            cur[b] = min(cur[b] + int(acc[b]) + 1, S - K1)
        ctx.rollback(seqs, cur)
    ms = _time_steps(torch, step, 2, 4)
    assert ctx.status() == 0
    ctx.close()
    us_layer = ms * 1e3 / L
    return {"workload": f"speculative verify: batch {B}, ctx ~{S}, K+1 = {K1} positions per sequence per step, rollback to "
                        f"ctx + accepted + 1 after every step, 128 heads, bf16, {L} layers timed",
            "us_per_layer_step": us_layer, "verified_positions_per_s_61_layers_scaled": R / (us_layer * 61e-6),
            "latent_kv_gbs": R * S * 1152.0 / (us_layer * 1e-6) / 1e9,
            "note": "every verified position is a query row that streams its sequence's cache: K+1 times the bytes of a decode step"}


def run_extras(a, world, rank, local, only=""):
    import torch
    import torch.distributed as dist
    peak, _ = measured_peak_gbs()
    res = {}

    def guarded(name, fn):
        try:
            res[name] = fn()
        except Exception as e:                                       # a sub-benchmark never takes the headline down
            res[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.empty_cache()

    if only in ("", "kv_range"):
        guarded("kv_range", lambda: sub_kv_range(torch, dist, world, rank, local, peak))
    if world == 1:
        if only in ("", "ragged"):
            guarded("ragged", lambda: sub_ragged(torch, peak))
        if only in ("", "v2lite"):
            guarded("v2lite", lambda: sub_v2lite(torch, peak))
        if only in ("", "prefill"):
            guarded("prefill", lambda: sub_prefill(torch, peak))
        if only in ("", "verify"):
            guarded("verify", lambda: sub_verify(torch, peak))
    return res


def main():
    a = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != a.gpus and world > 1:
        a.gpus = world
    if a.impl == "reference":
        run_reference_arm(a, int(os.environ.get("RANK", "0")))
    elif a.only:
        import torch
        import torch.distributed as dist
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        res = run_extras(a, world, int(os.environ.get("RANK", "0")), local, only=a.only)
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps(res))
        if world > 1:
            dist.destroy_process_group()
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
