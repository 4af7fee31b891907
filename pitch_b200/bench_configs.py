"""Throughput of the stand-alone codec kernels at the benchmark configurations' shapes.

    python -m pitch_b200.bench_configs [--only cfg1,cfg2,cfg3,sweep,cfg5,attn,bias] [--reps 50]

Prints one JSON line per measurement: encode vectors/s, decode output GB/s and the fraction of
the HBM roofline, counting algorithmic bytes (full-precision tensor + packed codes + side
information, each once).  Inputs are synthetic (seeded, generated on the device).  Working sets
smaller than the 126 MB L2 are rotated over several distinct buffers so that every launch
streams from HBM; timing is by CUDA events on the launching stream after warm-up.
The whole-cache step (configuration 4) is measured by ``bench.py`` at the repository root.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from . import ChannelQuantConfig, KVCache, PITCH, QuantConfig

L2_BYTES = 126 << 20


def hbm_peak() -> tuple[float, str]:
    f = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if f.exists():
        return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def time_launches(fn, n_sets: int, reps: int) -> float:
    """Mean seconds per call of fn(i), i cycling over n_sets buffer sets."""
    for i in range(max(3, n_sets)):
        fn(i % n_sets)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        fn(i % n_sets)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / reps


def report(name, what, seconds, units, unit_name, nbytes, extra):
    peak, src = hbm_peak()
    gbs = nbytes / seconds / 1e9
    print(json.dumps({"config": name, "op": what, "us_per_launch": round(seconds * 1e6, 2),
                      f"{unit_name}_per_s": round(units / seconds, 1), "algorithmic_GB_per_s": round(gbs, 1),
                      "frac_of_hbm_peak": round(gbs / peak, 4), "peak": peak, "peak_source": src,
                      "frac_of_nominal_8000": round(gbs / 8000.0, 4), **extra}), flush=True)


def lognormal_vectors(n, d, seed, dev):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    x = torch.randn((n, d), generator=g, device=dev)
    s = torch.exp(0.5 * torch.randn((n, 1), generator=g, device=dev))
    return x * s


def bench_vector(q, name, method, n, d, bits, reps, out_dtype=torch.float32):
    cfg = QuantConfig(method, d, bits)
    dev = q.device
    in_bytes, code_bytes = n * d * 4, n * cfg.code_stride + n * 4
    n_sets = max(1, -(-2 * L2_BYTES // (in_bytes + code_bytes)))
    xs = [lognormal_vectors(n, d, 100 + i, dev) for i in range(n_sets)]
    codes = [torch.empty(n * cfg.code_stride, dtype=torch.uint8, device=dev) for _ in range(n_sets)]
    scales = [torch.empty(n, dtype=torch.float32, device=dev) for _ in range(n_sets)]
    outs = [torch.empty((n, d), dtype=out_dtype, device=dev) for _ in range(n_sets)]
    t = time_launches(lambda i: q.enqueue_encode(xs[i], codes[i], scales[i], n, cfg), n_sets, reps)
    extra = {"method": method, "dim": d, "bits": bits, "count": n, "buffer_sets": n_sets}
    report(name, "encode", t, n, "vectors", in_bytes + code_bytes, extra)
    t = time_launches(lambda i: q.enqueue_decode(codes[i], scales[i], outs[i], n, cfg), n_sets, reps)
    out_bytes = n * d * outs[0].element_size()
    report(name, "decode", t, n, "vectors", out_bytes + code_bytes,
           {**extra, "out_dtype": str(out_dtype).replace("torch.", ""), "decode_output_GB_per_s": round(out_bytes / t / 1e9, 1)})


def bench_channel(q, name, n, d, bits, G, reps):
    cfg = ChannelQuantConfig(d, bits, G)
    dev = q.device
    groups = cfg.group_count(n)
    in_bytes, code_bytes = n * d * 4, n * cfg.code_stride + groups * cfg.range_stride
    n_sets = max(1, -(-2 * L2_BYTES // (in_bytes + code_bytes)))
    xs = []
    for i in range(n_sets):
        g = torch.Generator(device=dev)
        g.manual_seed(200 + i)
        x = torch.randn((n, d), generator=g, device=dev) + 2.0 * torch.randn((1, d), generator=g, device=dev)
        x[:, torch.randperm(d, generator=g, device=dev)[:4]] *= 20.0
        xs.append(x)
    codes = [torch.empty(n * cfg.code_stride, dtype=torch.uint8, device=dev) for _ in range(n_sets)]
    ranges = [torch.empty(groups * 2 * d, dtype=torch.float16, device=dev) for _ in range(n_sets)]
    outs = [torch.empty((n, d), dtype=torch.float32, device=dev) for _ in range(n_sets)]
    extra = {"method": "perChannel", "dim": d, "bits": bits, "group": G, "count": n, "buffer_sets": n_sets}
    t = time_launches(lambda i: q.enqueue_per_channel_encode(xs[i], codes[i], ranges[i], n, cfg), n_sets, reps)
    report(name, "encode", t, n, "tokens", in_bytes + code_bytes, extra)
    t = time_launches(lambda i: q.enqueue_per_channel_decode(codes[i], ranges[i], outs[i], n, cfg), n_sets, reps)
    report(name, "decode", t, n, "tokens", in_bytes + code_bytes,
           {**extra, "out_dtype": "float32", "decode_output_GB_per_s": round(in_bytes / t / 1e9, 1)})


def bench_cfg5(q, bits, reps, segments=80, tokens=131072):
    """One GPU's shard of the Llama-3-70B-shaped cache: 80 of 640 (layer, head) segments."""
    d = 128
    cfg = QuantConfig("turboQuant", d, bits)
    cache = KVCache(segments, d, tokens, cfg, cfg, out_dtype="float16", pitch=q)
    chunk = 8                                           # prefill a few segments at a time (inputs are 64 MB each)
    for s0 in range(0, segments, chunk):
        k = lognormal_vectors(chunk * tokens, d, 500 + s0, q.device).reshape(chunk, tokens, d)
        v = lognormal_vectors(chunk * tokens, d, 900 + s0, q.device).reshape(chunk, tokens, d)
        for pl, x in zip(cache.planes, (k, v)):
            for j in range(chunk):
                q.enqueue_encode(x[j], pl.codes[s0 + j], pl.side[s0 + j], tokens, cfg)
        torch.cuda.synchronize()
        del k, v
    cache.tokens = tokens
    t = time_launches(lambda i: cache.decode(), 1, reps)
    nbytes = cache.stored_bytes() + cache.decoded_bytes()
    report("cfg5-shard", "whole-cache decode", t, 2 * segments * tokens, "vectors", nbytes,
           {"method": "turboQuant", "dim": d, "bits": bits, "segments": segments, "tokens": tokens, "out_dtype": "float16",
            "decode_output_GB_per_s": round(cache.decoded_bytes() / t / 1e9, 1)})


def bench_attention(q, reps, segments=48, tokens=32768, n_queries=7):
    """Single-token attention straight from the compressed cache at configuration 4's shape
    (Qwen2.5-0.5B: 24 layers x 2 KV heads, 7 query heads per KV head), next to what it replaces:
    whole-cache decode followed by attention over the decoded bf16 cache (torch SDPA)."""
    d = 64
    cache = KVCache(segments, d, tokens, ChannelQuantConfig(d, 4, 64), QuantConfig("turboQuant", d, 4),
                    out_dtype="bfloat16", pitch=q)
    g = torch.Generator(device=q.device)
    g.manual_seed(7)
    k = torch.randn((segments, tokens, d), generator=g, device=q.device) + 2.0 * torch.randn((segments, 1, d), generator=g, device=q.device)
    v = lognormal_vectors(segments * tokens, d, 8, q.device).reshape(segments, tokens, d)
    cache.prefill(k, v)
    del k, v
    qs = [torch.randn((segments, n_queries, d), generator=g, device=q.device) for _ in range(4)]
    out = torch.empty_like(qs[0])
    flush = torch.empty(L2_BYTES * 2, dtype=torch.uint8, device=q.device)       # the compressed cache (113 MB) fits L2

    def timed(fn):
        for i in range(3):
            fn(i)
        ts = []
        for i in range(reps):
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn(i)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e-3)
        ts.sort()
        return ts[len(ts) // 2]

    t = timed(lambda i: cache.attend(qs[i % 4], out=out))
    stored = cache.stored_bytes()
    extra = {"dim": d, "segments": segments, "tokens": tokens, "n_queries": n_queries, "l2": "flushed before every launch",
             "tokens_per_s": round(segments * tokens / t, 1)}
    report("cfg4 attention", "attention from the compressed cache", t, segments * tokens, "kv_tokens", stored, extra)

    def two_step(i):
        ko, vo = cache.decode()
        torch.nn.functional.scaled_dot_product_attention(qs[i % 4].to(torch.bfloat16).unsqueeze(0), ko.unsqueeze(0), vo.unsqueeze(0))
    t2 = timed(two_step)
    report("cfg4 attention", "decode, then torch SDPA over the decoded cache", t2, segments * tokens, "kv_tokens",
           stored + 2 * cache.decoded_bytes(), {**extra, "speedup_of_fused": round(t2 / t, 2)})


def bench_key_bias(q, reps, segments=48, tokens=32768):
    """Whole-cache decode with exact key-bias removal (TurboQuant keys and values, d=64, bf16 out):
    the rotated bias is added back to the decoded keys by one extra element-wise launch."""
    d = 64
    cfg = QuantConfig("turboQuant", d, 4)
    dev = q.device
    inv = 10000.0 ** (-torch.arange(0, d, 2, dtype=torch.float64, device=dev) / d)
    ang = torch.arange(tokens, dtype=torch.float64, device=dev)[:, None] * inv[None, :]
    ang = torch.cat([ang, ang], dim=1)
    kb = (torch.randn((segments, d), device=dev) * 4.0, torch.cos(ang).float().contiguous(), torch.sin(ang).float().contiguous())
    for name, bias in (("without key bias", None), ("with key-bias removal", kb)):
        cache = KVCache(segments, d, tokens, cfg, cfg, out_dtype="bfloat16", pitch=q, key_bias=bias)
        for s0 in range(0, segments, 8):
            x = lognormal_vectors(8 * tokens, d, 300 + s0, dev).reshape(8, tokens, d)
            for pl in cache.planes:
                for j in range(8):
                    q.enqueue_encode(x[j], pl.codes[s0 + j], pl.side[s0 + j], tokens, cfg)
            torch.cuda.synchronize()
        cache.tokens = tokens
        t = time_launches(lambda i: cache.decode(), 1, reps)
        nbytes = cache.stored_bytes() + cache.decoded_bytes()
        report("cfg4-shape TurboQuant keys", "whole-cache decode " + name, t, 2 * segments * tokens, "vectors", nbytes,
               {"dim": d, "segments": segments, "tokens": tokens, "out_dtype": "bfloat16",
                "extra_pass_bytes": 0 if bias is None else cache.decoded_bytes()})


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--only", default="cfg1,cfg2,cfg3,sweep")
    ap.add_argument("--reps", type=int, default=50)
    ap.add_argument("--cfg5-segments", type=int, default=80, help="segments of the config 5 shard (80 = one GPU's share of 640)")
    args = ap.parse_args()
    which = set(args.only.split(","))
    q = PITCH()
    if "cfg1" in which:
        bench_vector(q, "cfg1", "turboQuant", 65536, 64, 4, args.reps)
        bench_vector(q, "cfg1 x64 batch", "turboQuant", 65536 * 64, 64, 4, max(5, args.reps // 5))
        bench_vector(q, "cfg1 x64 batch", "turboQuant", 65536 * 64, 64, 4, max(5, args.reps // 5), torch.bfloat16)
    if "cfg2" in which:
        bench_channel(q, "cfg2", 32768, 64, 4, 64, args.reps)
        bench_channel(q, "cfg2 x48 heads", 32768 * 48, 64, 4, 64, max(5, args.reps // 5))
    if "cfg3" in which:
        for bits in (3, 4):
            bench_vector(q, "cfg3", "polarQuant", 1 << 20, 128, bits, max(5, args.reps // 5))
    if "sweep" in which:
        for method in ("turboQuant", "polarQuant"):
            for d in (64, 128, 256, 512, 1024):
                bench_vector(q, "cfg3 sweep", method, (1 << 27) // d, d, 4, max(5, args.reps // 5))
    if "attn" in which:
        bench_attention(q, max(5, args.reps // 5))
    if "bias" in which:
        bench_key_bias(q, max(5, args.reps // 5))
    if "cfg5" in which:
        for bits in (4, 3):
            bench_cfg5(q, bits, max(3, args.reps // 10), segments=args.cfg5_segments)


if __name__ == "__main__":
    main()
