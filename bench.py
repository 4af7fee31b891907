#!/usr/bin/env python3
"""Whole-cache KV decode benchmark (the per-step bottleneck of a compressed KV cache).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--scaling weak|strong]

Workload: a Qwen2.5-0.5B-shaped cache - 24 layers x 2 KV heads (48 segments), head dim 64,
32,768 tokens, batch 1.  Keys: per-channel 4-bit, groups of 64 tokens, on N(0,1) values plus a
per-channel bias N(0, sigma=2).  Values: TurboQuant 4-bit on N(0,1).  One step appends one
encoded token per segment and decodes the whole cache to bf16.  Data are synthetic (seeded).

Metric: decode GB/s = algorithmic bytes (packed codes + side information read, decoded bf16
written) per step / step time, summed over all GPUs.  With N GPUs the default is weak scaling
(every rank holds and decodes one full cache of its own; no collective on the data path);
``--scaling strong`` splits the 24 layers of one cache over the ranks instead.

Prints ONE JSON line (rank 0).  ``--impl reference`` times the reference's CPU path (the NumPy
port of its specification, under oracle/) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

LAYERS, KV_HEADS, DIM, TOKENS, BITS, GROUP = 24, 2, 64, 32768, 4, 64
SEGMENTS = LAYERS * KV_HEADS
WORKLOAD = "qwen2.5-0.5b-shaped whole-cache step: 24 layers x 2 kv heads x d=64 x 32768 tokens, K per-channel b=4 G=64, V turboQuant b=4, decode to bf16"


def step_bytes(segments: int, tokens: int) -> tuple[int, int]:
    """(bytes read, bytes written) by one whole-cache decode."""
    stride = DIM * BITS // 8
    groups = (tokens + GROUP - 1) // GROUP
    read = segments * (tokens * stride + groups * 2 * DIM * 2) + segments * (tokens * stride + tokens * 4)
    written = 2 * segments * tokens * DIM * 2
    return read, written


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 - 0.05 <= t <= t1 + 0.15 and len(r) >= 9] or [r for _, r in self.rows if len(r) >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[1]) for r in rows)
        reasons = set()
        for r in rows:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][2]), "reasons": sorted(reasons),
                "samples": len(rows), "power_w_max": max(float(r[3]) for r in rows)}


# ------------------------------------------------------------------------------------------ CPU side
_W = {}


def _cpu_init(seed: int):
    """Per worker process: one segment of synthetic compressed cache (K per-channel, V TurboQuant)."""
    import numpy as np
    from oracle import spec_np
    rng = np.random.default_rng(seed)
    K = (rng.standard_normal((TOKENS, DIM)) + rng.normal(0.0, 2.0, (1, DIM))).astype(np.float32)
    V = rng.standard_normal((TOKENS, DIM)).astype(np.float32)
    kc, kr = spec_np.channel_encode(K, BITS, GROUP)
    vc, vn = spec_np.turbo_encode(V.astype(np.float64), BITS)
    _W.update(k_codes=spec_np.pack_codes(kc, BITS), k_ranges=kr, v_codes=spec_np.pack_codes(vc, BITS),
              v_norms=vn.astype(np.float32))


def _cpu_decode_segments(n: int) -> int:
    """Decodes n segments the way the reference's CPU path does: unpack + channel_decode for keys,
    unpack + turbo_decode for values, results rounded to bf16-sized storage is NOT included."""
    from oracle import spec_np
    for _ in range(n):
        kc = spec_np.unpack_codes(_W["k_codes"], TOKENS, DIM, BITS)
        spec_np.channel_decode(kc, _W["k_ranges"], BITS, GROUP)
        vc = spec_np.unpack_codes(_W["v_codes"], TOKENS, DIM, BITS)
        spec_np.turbo_decode(vc, _W["v_norms"], BITS)
    return n


class CpuArm:
    """The reference's CPU path (NumPy port of its specification) over all host cores."""

    def __init__(self):
        import multiprocessing as mp
        avail = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        self.cores = max(1, min(avail, SEGMENTS))       # processes actually used: one segment each at least
        ctx = mp.get_context("spawn")
        self.pool = ctx.Pool(self.cores, initializer=_cpu_init, initargs=(4,))
        self.pool.map(_cpu_decode_segments, [0] * self.cores)          # start every worker

    def seconds_per_segment(self) -> float:
        t = time.perf_counter()
        self.pool.map(_cpu_decode_segments, [1] * self.cores)
        return (time.perf_counter() - t)

    def run(self, segments: int) -> float:
        """Decodes `segments` segments spread over the cores; returns wall seconds."""
        per = [segments // self.cores + (1 if i < segments % self.cores else 0) for i in range(self.cores)]
        t = time.perf_counter()
        self.pool.map(_cpu_decode_segments, per)
        return time.perf_counter() - t

    def close(self):
        self.pool.terminate()


def cpu_baseline_sample(budget_s: float = 15.0) -> dict:
    arm = CpuArm()
    try:
        t_round = arm.seconds_per_segment()                 # wall time of one segment on every core at once
        rounds = max(1, min(SEGMENTS // arm.cores or 1, int(budget_s / max(t_round, 1e-3))))
        segs = rounds * arm.cores
        secs = arm.run(segs)
        rd, wr = step_bytes(segs, TOKENS)
        return {"value": round((rd + wr) / secs / 1e9, 4), "unit": "GB/s", "cores": arm.cores, "kind": "port",
                "sample": f"{segs} of {SEGMENTS} segments (32768 tokens each, K+V) decoded by the NumPy port of "
                          f"pitch_reference.py, one process per core, {secs:.2f} s"}
    finally:
        arm.close()


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    arm = CpuArm()
    try:
        t_round = arm.seconds_per_segment()
        total = args.steps + args.warmup
        # bounded sample per step so that the whole run stays within a few minutes
        rounds = max(1, min(max(SEGMENTS // arm.cores, 1), int(150.0 / total / max(t_round, 1e-3))))
        segs = rounds * arm.cores
        for _ in range(args.warmup):
            arm.run(segs)
        t = 0.0
        for _ in range(args.steps):
            t += arm.run(segs)
        rd, wr = step_bytes(segs, TOKENS)
        value = (rd + wr) * args.steps / t / 1e9
        sample = (f"each step decodes {segs} of {SEGMENTS} segments (32768 tokens each, K per-channel + V turboQuant) "
                  f"with the NumPy port of pitch_reference.py, one process per host core")
        print(json.dumps({
            "impl": "reference", "metric": "kv_cache_decode_throughput", "value": round(value, 4), "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(t / args.steps * 1e3, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sample": sample},
            "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": arm.cores, "kind": "port", "sample": sample},
            "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }))
    finally:
        arm.close()


# ------------------------------------------------------------------------------------------ GPU side
def build_cache(q, segments: int, tokens0: int, capacity: int, seed: int):
    """Synthetic cache: per segment a seeded generator; returns the cache and host copies of the first
    two segments' inputs for the parity gate."""
    import torch
    from pitch_b200 import ChannelQuantConfig, KVCache, QuantConfig
    dev = q.device
    cache = KVCache(segments, DIM, capacity, ChannelQuantConfig(DIM, BITS, GROUP), QuantConfig("turboQuant", DIM, BITS),
                    out_dtype="bfloat16", pitch=q)
    K = torch.empty((segments, tokens0, DIM), dtype=torch.float32, device=dev)
    V = torch.empty((segments, tokens0, DIM), dtype=torch.float32, device=dev)
    for s in range(segments):
        g = torch.Generator(device=dev)
        g.manual_seed(seed + s)
        bias = torch.randn((1, DIM), generator=g, device=dev) * 2.0
        K[s] = torch.randn((tokens0, DIM), generator=g, device=dev) + bias
        V[s] = torch.randn((tokens0, DIM), generator=g, device=dev)
    cache.prefill(K, V)
    sample = (K[:2].cpu().numpy(), V[:2].cpu().numpy())
    del K, V
    return cache, sample


def parity_gate(cache, sample) -> dict:
    """Timing is only reported for a kernel that agrees with the oracles: the first two segments
    are decoded and compared in full (keys bit-exact after bf16 rounding; value codes bit-exact
    against the float32 oracle, decoded values within bf16 rounding of it)."""
    import numpy as np
    import torch
    from oracle import kernel_f32, spec_np
    Ks, Vs = sample
    T = Ks.shape[1]
    ko, vo = cache.decode()
    torch.cuda.synchronize()
    worst = 0.0
    for s in range(Ks.shape[0]):
        kc, kr = spec_np.channel_encode(Ks[s], BITS, GROUP)
        ref = torch.from_numpy(spec_np.channel_decode(kc, kr, BITS, GROUP)).bfloat16()
        if not torch.equal(ko[s, :T].cpu(), ref):
            raise SystemExit("parity gate failed: per-channel keys differ from the specification")
        vc, vn = kernel_f32.encode("turboQuant", Vs[s], BITS)
        if cache.planes[1].codes[s, :T * 32].cpu().numpy().tobytes() != vc.tobytes():
            raise SystemExit("parity gate failed: TurboQuant codes differ from the float32 oracle")
        v32 = kernel_f32.decode("turboQuant", vc, vn, DIM, BITS)
        got = vo[s, :T].cpu().float().numpy()
        rel = float(np.sqrt(((got - v32) ** 2).sum(1) / (v32 ** 2).sum(1)).max())
        worst = max(worst, rel)
        if rel > 5e-3:
            raise SystemExit(f"parity gate failed: decoded values differ by {rel}")
    return {"segments_checked": int(Ks.shape[0]), "tokens_checked": int(T), "keys": "bit-exact",
            "value_codes": "bit-exact", "values_max_rel_l2_vs_f32_oracle_after_bf16": worst}


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    from pitch_b200 import PITCH
    from pitch_b200.shard import gather_int64, shard_segments

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_gpus = world

    if args.scaling == "strong":
        segments = shard_segments(LAYERS, KV_HEADS, n_gpus, rank, by="layer").segments
    else:
        segments = SEGMENTS
    if args.segments:
        segments = args.segments
    total_steps = args.warmup + args.steps
    tokens0 = TOKENS - total_steps                       # the last timed step decodes exactly 32,768 tokens
    if tokens0 < 1:
        raise SystemExit("too many steps for a 32,768-token cache")

    q = PITCH(dev)
    cache, sample = build_cache(q, segments, tokens0, TOKENS, seed=4 + rank * SEGMENTS)
    gate = parity_gate(cache, sample)

    # new tokens for every step, resident on the device (the e2e leg below brings them from the host)
    g = torch.Generator(device=dev)
    g.manual_seed(1000 + rank)
    new_k = torch.randn((total_steps, segments, 1, DIM), generator=g, device=dev)
    new_v = torch.randn((total_steps, segments, 1, DIM), generator=g, device=dev)

    stream = torch.cuda.current_stream(dev)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t_wall0 = time.time()
    for i in range(args.warmup):
        cache.append(new_k[i], new_v[i])
        cache.decode()
    barrier()
    bytes_total = 0
    # The decode launch is timed on its own in every 8th step only: an event between the append and
    # the decode keeps the decode from starting its prologue under the append (programmatic
    # dependent launch), which the other steps are allowed to do.
    sampled = [i for i in range(args.steps) if i % 8 == 0]
    for i in range(args.steps):
        if i == 0:
            ev[0][0].record(stream)
        cache.append(new_k[args.warmup + i], new_v[args.warmup + i])
        if i % 8 == 0:
            ev[i][1].record(stream)
        cache.decode()
        if i % 8 == 0 or i == args.steps - 1:
            ev[i][2].record(stream)
        rd, wr = step_bytes(segments, cache.tokens)
        bytes_total += rd + wr
    barrier()
    assert cache.tokens == TOKENS
    step_ms = ev[0][0].elapsed_time(ev[-1][2]) / args.steps
    decode_ms = sum(ev[i][1].elapsed_time(ev[i][2]) for i in sampled) / len(sampled)
    sums = cache.checksums()

    # ---- end to end through the public API with host buffers: every step the new token comes from
    # pinned host memory and the decoded cache (both output buffers, whole) goes back to pinned host memory
    e2e_ms, e2e_bytes, d2h, e2e_steps = 0.0, 0, 0, 0
    if not args.kernel_only:
        e2e_steps = max(3, min(10, args.steps))
        cache.truncate(TOKENS - GROUP)                      # make room again (a group boundary)
        hk = torch.randn((e2e_steps + 1, segments, 1, DIM)).pin_memory()
        hv = torch.randn((e2e_steps + 1, segments, 1, DIM)).pin_memory()
        host_k = torch.empty((segments, cache.capacity, DIM), dtype=torch.bfloat16).pin_memory()
        host_v = torch.empty((segments, cache.capacity, DIM), dtype=torch.bfloat16).pin_memory()

        def e2e_step(i):
            dk = hk[i].to(dev, non_blocking=True)
            dv = hv[i].to(dev, non_blocking=True)
            cache.append(dk, dv)
            cache.decode()
            host_k.copy_(cache.planes[0].out, non_blocking=True)
            host_v.copy_(cache.planes[1].out, non_blocking=True)
            return cache.tokens

        e2e_step(0)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(1, e2e_steps + 1):
            t = e2e_step(i)
            rd, wr = step_bytes(segments, t)
            e2e_bytes += rd + wr
        e1.record(stream)
        barrier()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps
        d2h = host_k.numel() * 2 + host_v.numel() * 2
    # keep the GPU busy long enough for nvidia-smi (one sample per 100 ms) to see it under load
    t_busy = time.time()
    while not args.kernel_only and time.time() - t_busy < 0.6:
        cache.decode()
        torch.cuda.synchronize(dev)
    clocks = sampler.stop(t_wall0, time.time()) if rank == 0 else None

    # ---- reduce over ranks: slowest rank sets the time
    stats = torch.tensor([step_ms, decode_ms, e2e_ms], dtype=torch.float64, device=dev)
    rank_step_ms = [round(step_ms, 5)]
    if world > 1:
        every = [torch.zeros_like(stats) for _ in range(world)]
        dist.all_gather(every, stats)                       # per-rank step times, reported next to their maximum
        rank_step_ms = [round(float(e[0]), 5) for e in every]
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    step_ms, decode_ms, e2e_ms = (float(x) for x in stats.cpu())
    # verification checksums travel over NCCL (all_gather of four 64-bit words per rank); nothing else does
    all_sums = gather_int64([sums["keys"]["codes"], sums["keys"]["decoded"], sums["values"]["codes"],
                             sums["values"]["decoded"]], device=dev)

    if rank == 0:
        per_rank_bytes = bytes_total / args.steps
        value = per_rank_bytes * n_gpus / (step_ms * 1e-3) / 1e9
        rd, wr = step_bytes(segments, TOKENS)
        achieved = (rd + wr) / (decode_ms * 1e-3) / 1e9
        peak, peak_src = 6546.9, "fallback"
        mp = ROOT / "MEASURED_PEAKS.json"
        if mp.exists():
            peak, peak_src = float(json.loads(mp.read_text())["hbm_gbs"]), "measured"
        else:
            peak = 6650.0
        # dram__bytes_read.sum + dram__bytes_write.sum per launch at full size, from the ncu capture
        # summarised in profiles/cache_decode_kernel_config4.md (part of the output is still dirty in L2
        # when the kernel ends, so it is below the algorithmic bytes); only valid for the full workload
        traffic = 455.6e6 if segments == SEGMENTS else None
        cpu = cpu_baseline_sample() if (n_gpus == 1 and not args.kernel_only) else None
        out = {
            "metric": "kv_cache_decode_throughput", "value": round(value, 2), "unit": "GB/s", "n_gpus": n_gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(step_ms, 5), "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "segments_per_gpu": segments, "out_dtype": "bf16",
                       "l2": "inputs larger than L2 (516 MB touched per step per GPU)" if segments == SEGMENTS else
                             "working set may fit L2 under strong scaling; reported as is",
                       "parallelism": f"{'one cache per gpu' if args.scaling == 'weak' else 'layers sharded'} x{n_gpus}, no data-path collective"},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "traffic": traffic, "peak_source": peak_src,
                         "frac_of_nominal_8000": round(achieved / 8000.0, 4), "kernel": "cache_decode_kernel<bf16,64,4>",
                         "kernel_ms": round(decode_ms, 5), "kernel_launches_timed": len(sampled)},
            "e2e": None if not e2e_steps else {
                "value": round(e2e_bytes / e2e_steps * n_gpus / (e2e_ms * 1e-3) / 1e9, 3), "unit": "GB/s",
                "h2d_bytes_per_step": int(2 * segments * DIM * 4), "d2h_bytes_per_step": int(d2h),
                "ms_per_step": round(e2e_ms, 4), "steps": e2e_steps},
            "rank_ms_per_step": rank_step_ms,
            "gpu_launches": 2 * args.steps,   # per step: one append launch, one whole-cache decode launch
            "clocks": clocks,
            "parity_gate": gate,
            "checksums": all_sums,
        }
        if args.segments:
            out["reduced"] = True
        if cpu is not None:
            out["cpu_baseline"] = cpu
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak")
    ap.add_argument("--segments", type=int, default=0,
                    help="profiling aid: decode only this many segments per GPU (marks the line \"reduced\")")
    ap.add_argument("--kernel-only", action="store_true",
                    help="profiling aid: skip the end-to-end and CPU-baseline legs")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
