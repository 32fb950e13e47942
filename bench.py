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

Prints ONE JSON line (rank 0).
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
# dram__bytes_read.sum + dram__bytes_write.sum of one attention launch at the default workload
# (profiles/decode_tc5_pair128_kernel_v3shape_b64_ctx16384.md); only meaningful for that workload and kernel
NCU_TRAFFIC_BYTES_PER_LAUNCH = 1.2491e9
NCU_TRAFFIC_KERNEL = "tcgen05-pair128"
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
    p.add_argument("--kernel", default="auto", choices=["auto", "mma", "tcgen05", "tcgen05-pair", "tcgen05-pair128"])
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-cpu", action="store_true")
    return p.parse_args()


def workload_name(a) -> str:
    return (f"deepseek-v3-shaped MLA decode (configs[2]): {a.layers} layers, {a.heads} heads, batch {a.batch}, "
            f"ctx {a.ctx}, {a.dtype} paged latent cache, page 64")


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
        """Seconds for one layer's attention over n_seq sequences of ctx tokens (same cache
        buffer for every sequence: the arithmetic and the memory traffic per call are unchanged)."""
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
              f"on {threads} host threads; tokens/s = sequences / (time x {a.layers} layers)")
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
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={device_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
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
        for ln in out.strip().splitlines():
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
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
    kernel = {"auto": capi.KERNEL_AUTO, "mma": capi.KERNEL_MMA, "tcgen05": capi.KERNEL_TCGEN05, "tcgen05-pair128": capi.KERNEL_TCGEN05_PAIR128}[a.kernel]
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

    for _ in range(a.warmup):
        one_step()
    torch.cuda.synchronize()
    clocks = ClockSampler(local) if rank == 0 else None
    lens_sum = 0
    launches0 = ctx.launch_count()
    ctx.profile_enable(KERNEL_EVENT_STRIDE if L >= KERNEL_EVENT_STRIDE else 1)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(); torch.cuda.synchronize()
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
                "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH * (B / 64.0) if (ctx.kernel_name() == NCU_TRAFFIC_KERNEL and a.heads == 128 and a.ctx == 16384) else None, "kernel": f"split-KV attention ({ctx.kernel_name()})",
                "peak_source": peak_src, "algorithmic_bytes_per_launch": algo_bytes,
                "avg_launch_us": per_launch_s * 1e6, "launches_timed": n_attn}
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
               "sample": f"one layer of cpu_mla_attention over {n_seq} sequences (ctx {a.ctx}, {a.heads} heads, f16), "
                         f"{sec:.2f} s on {threads} threads; scaled by {a.layers} layers"}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
                "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": a.dtype, "data": "synthetic",
                "config": {"workload": workload_name(a), "sequences_per_gpu": B, "sharding": f"batch over {world} GPU(s)",
                           "kernel": ctx.kernel_name(),
                           "l2_policy": "inputs larger than L2: every layer-step streams its own >= 150 MB of cache"},
                "latent_kv_gbs_per_gpu": latent_gbs, "latent_kv_frac_of_8tbs": latent_gbs / 8000.0,
                "latent_kv_frac_of_measured_peak": latent_gbs / peak,
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clk}
        print(json.dumps(line))
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    a = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != a.gpus and world > 1:
        a.gpus = world
    if a.impl == "reference":
        run_reference_arm(a, int(os.environ.get("RANK", "0")))
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
