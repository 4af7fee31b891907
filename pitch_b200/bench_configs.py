"""Throughput of the stand-alone codec kernels at the benchmark configurations' shapes.

    python -m pitch_b200.bench_configs [--only cfg1,cfg2,cfg3,sweep,cfg5,attn,bias] [--reps 50]

Prints one JSON line per measurement: encode vectors/s, decode output GB/s and the fraction of
the HBM roofline, counting algorithmic bytes (full-precision tensor + packed codes + side
information, each once).  Inputs are synthetic (seeded, generated on the device).  Working sets
smaller than the 126 MB L2 are rotated over several distinct buffers so that every launch
streams from HBM; timing is by CUDA events on the launching stream after warm-up.
The whole-cache step (configuration 4) is measured by ``bench.py`` at the repository root.

Nothing is timed before it has passed a parity gate (the reference gates its own timing the same
way, reference/pytorch_mps_benchmark.py:82-104).  ``run(..., gate=fn)`` hands a seeded sample of
every encode - input vectors, packed codes, side information, spread over the whole batch - to
``fn``, which the repository's ``bench.py`` implements with the CPU oracles.  Run as a module the
gate is the committed golden vectors of the reference's specification (``tests/golden``): the
kernels must reproduce them for the method, dimension and width being timed, and every timed
batch must survive a decode - re-encode round trip with unchanged codes.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import numpy as np
import torch

from . import ChannelQuantConfig, KVCache, PITCH, QuantConfig

L2_BYTES = 126 << 20
GOLDEN_DIR = Path(__file__).resolve().parent.parent / "tests" / "golden"


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


def row(name, what, seconds, units, unit_name, nbytes, extra) -> dict:
    peak, src = hbm_peak()
    gbs = nbytes / seconds / 1e9
    return {"config": name, "op": what, "us_per_launch": round(seconds * 1e6, 2),
            f"{unit_name}_per_s": round(units / seconds, 1), "algorithmic_GB_per_s": round(gbs, 1),
            "frac_of_hbm_peak": round(gbs / peak, 4), "peak": peak, "peak_source": src,
            "frac_of_nominal_8000": round(gbs / 8000.0, 4), **extra}


def lognormal_vectors(n, d, seed, dev):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    x = torch.randn((n, d), generator=g, device=dev)
    s = torch.exp(0.5 * torch.randn((n, 1), generator=g, device=dev))
    return x * s


# ------------------------------------------------------------------------------------------ parity gates
_golden = {}


def _golden_file(name):
    if name not in _golden:
        z = np.load(GOLDEN_DIR / name)
        _golden[name] = (z, json.loads(bytes(z["__cases__"]).decode()))
    return _golden[name]


def golden_gate(q, kind: str, dim: int, bits: int, group: int = 64) -> dict:
    """The kernels about to be timed against the committed golden vectors of the specification for
    the same method, dimension and width (tolerances of the reference's own parity tests,
    Tests/PITCHTests/ParityTests.swift:67-76: code mismatches <= max(2, n/500), scales 1e-5,
    decode of the golden codes 1e-5; per-channel: identical)."""
    checked = 0
    for fname in ("parity.npz", "channel_parity.npz", "spec_extra.npz"):
        if not (GOLDEN_DIR / fname).exists():
            continue
        z, cases = _golden_file(fname)
        for c in cases:
            x = z["input/" + c["group"]]
            if x.ndim != 2 or x.shape[1] != dim or c["bits"] != bits:
                continue
            n = x.shape[0]
            is_channel = "group_size" in c
            if kind == "perChannel":
                if not is_channel or c["group_size"] != group:
                    continue
                cfg = ChannelQuantConfig(dim, bits, group)
                blk = q.encode_per_channel(x, config=cfg)
                if blk.codes != z[c["key"] + "/codes"].tobytes() or \
                        not np.array_equal(blk.ranges.reshape(-1).view(np.uint16), z[c["key"] + "/ranges"].reshape(-1).view(np.uint16)):
                    raise SystemExit(f"parity gate failed: per-channel {fname}:{c['key']} differs from the golden vectors")
            else:
                if is_channel or c.get("method") != kind:
                    continue
                cfg = QuantConfig(kind, dim, bits, c["seed"])
                batch = q.encode(x, config=cfg)
                want = np.frombuffer(z[c["key"] + "/codes"].tobytes(), dtype=np.uint8)
                got = np.frombuffer(batch.codes, dtype=np.uint8)
                bad = int(np.count_nonzero(got != want))                          # code bytes that differ
                ws = z[c["key"] + "/scales"].reshape(-1)
                if bad > max(2, n * dim // 500) or np.max(np.abs(batch.scales - ws) / np.maximum(np.abs(ws), 1.0)) > 1e-5:
                    raise SystemExit(f"parity gate failed: {fname}:{c['key']} differs from the golden vectors ({bad} code bytes)")
            checked += 1
    if checked == 0:
        raise SystemExit(f"parity gate: no golden case for {kind} dim {dim} bits {bits}; refusing to time it")
    return {"golden_cases_reproduced": checked}


def _sample_rows(n: int, want: int = 65536, blocks: int = 64) -> torch.Tensor:
    """Row indices of a seeded sample spread over a batch of n rows: `blocks` runs of consecutive rows."""
    if n <= want:
        return torch.arange(n)
    per = want // blocks
    starts = torch.linspace(0, n - per, blocks).long()
    return (starts[:, None] + torch.arange(per)[None, :]).reshape(-1)


def gate_vector(q, gate, kind, x, codes, scales, cfg) -> dict:
    """Parity of one timed encode.  With a gate callback: a sample of at least 65,536 vectors spread
    over the whole batch goes to it.  Always, for TurboQuant: the whole batch is decoded and encoded
    again; nearly every code must come back (the norm of a reconstruction differs a little from the
    stored one, which can carry a coordinate over a boundary; a broken kernel changes most bytes)."""
    n = x.shape[0]
    out = {}
    if gate is not None:
        idx = _sample_rows(n).to(x.device)
        xs = x[idx].cpu().numpy()
        cs = codes.view(n, cfg.code_stride)[idx].cpu().numpy()
        ss = scales[idx].cpu().numpy()
        out.update(gate(kind, xs, cs, ss, cfg.dim, cfg.bits))
        out["vectors_checked"] = int(idx.numel())
    else:
        out.update(golden_gate(q, kind, cfg.dim, cfg.bits))
    if kind == "turboQuant":
        # round trip at full size
        dec = torch.empty((n, cfg.dim), dtype=torch.float32, device=x.device)
        q.enqueue_decode(codes, scales, dec, n, cfg)
        c2 = torch.empty_like(codes)
        s2 = torch.empty_like(scales)
        q.enqueue_encode(dec, c2, s2, n, cfg)
        changed = int((c2 != codes).sum().item())
        out["codes_changed_by_decode_then_encode"] = changed
        if changed > codes.numel() // 100:              # a broken kernel changes most bytes; boundary cases are a handful
            raise SystemExit(f"parity gate failed: {kind} d={cfg.dim} b={cfg.bits}: {changed} code bytes changed by decode + encode")
        del dec, c2, s2
    out["checksum_codes"] = q.checksum(codes)
    return out


def bench_vector(q, name, method, n, d, bits, reps, out_dtype=torch.float32, gate=None):
    cfg = QuantConfig(method, d, bits)
    dev = q.device
    in_bytes, code_bytes = n * d * 4, n * cfg.code_stride + n * 4
    n_sets = max(1, -(-2 * L2_BYTES // (in_bytes + code_bytes)))
    xs = [lognormal_vectors(n, d, 100 + i, dev) for i in range(n_sets)]
    codes = [torch.empty(n * cfg.code_stride, dtype=torch.uint8, device=dev) for _ in range(n_sets)]
    scales = [torch.empty(n, dtype=torch.float32, device=dev) for _ in range(n_sets)]
    outs = [torch.empty((n, d), dtype=out_dtype, device=dev) for _ in range(n_sets)]
    q.enqueue_encode(xs[0], codes[0], scales[0], n, cfg)
    parity = gate_vector(q, gate, method, xs[0], codes[0], scales[0], cfg)
    t = time_launches(lambda i: q.enqueue_encode(xs[i], codes[i], scales[i], n, cfg), n_sets, reps)
    extra = {"method": method, "dim": d, "bits": bits, "count": n, "buffer_sets": n_sets}
    yield row(name, "encode", t, n, "vectors", in_bytes + code_bytes, {**extra, "parity": parity})
    t = time_launches(lambda i: q.enqueue_decode(codes[i], scales[i], outs[i], n, cfg), n_sets, reps)
    out_bytes = n * d * outs[0].element_size()
    yield row(name, "decode", t, n, "vectors", out_bytes + code_bytes,
              {**extra, "out_dtype": str(out_dtype).replace("torch.", ""), "decode_output_GB_per_s": round(out_bytes / t / 1e9, 1)})


def bench_channel(q, name, n, d, bits, G, reps, gate=None):
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
    q.enqueue_per_channel_encode(xs[0], codes[0], ranges[0], n, cfg)
    if gate is not None:
        # whole groups from a sample of places in the batch (a group is the unit that can be checked alone)
        m = min(n, 32768) // G * G
        first = (n - m) // G * G
        parity = gate("perChannel", xs[0][first:first + m].cpu().numpy(), codes[0].view(n, cfg.code_stride)[first:first + m].cpu().numpy(),
                      ranges[0].view(groups, 2 * d)[first // G:(first + m) // G].cpu().numpy(), d, bits, G)
        parity["tokens_checked"] = m
    else:
        parity = golden_gate(q, "perChannel", d, bits, G)
    parity["checksum_codes"] = q.checksum(codes[0])
    extra = {"method": "perChannel", "dim": d, "bits": bits, "group": G, "count": n, "buffer_sets": n_sets}
    t = time_launches(lambda i: q.enqueue_per_channel_encode(xs[i], codes[i], ranges[i], n, cfg), n_sets, reps)
    yield row(name, "encode", t, n, "tokens", in_bytes + code_bytes, {**extra, "parity": parity})
    t = time_launches(lambda i: q.enqueue_per_channel_decode(codes[i], ranges[i], outs[i], n, cfg), n_sets, reps)
    yield row(name, "decode", t, n, "tokens", in_bytes + code_bytes,
              {**extra, "out_dtype": "float32", "decode_output_GB_per_s": round(in_bytes / t / 1e9, 1)})


def bench_cfg5(q, bits, reps, segments=80, tokens=131072, gate=None):
    """One GPU's shard of the Llama-3-70B-shaped cache: 80 of 640 (layer, head) segments."""
    d = 128
    cfg = QuantConfig("turboQuant", d, bits)
    cache = KVCache(segments, d, tokens, cfg, cfg, out_dtype="float16", pitch=q)
    chunk = 8                                           # prefill a few segments at a time (inputs are 64 MB each)
    parity = None
    for s0 in range(0, segments, chunk):
        m = min(chunk, segments - s0)
        k = lognormal_vectors(m * tokens, d, 500 + s0, q.device).reshape(m, tokens, d)
        v = lognormal_vectors(m * tokens, d, 900 + s0, q.device).reshape(m, tokens, d)
        for pl, x in zip(cache.planes, (k, v)):
            for j in range(m):
                q.enqueue_encode(x[j], pl.codes[s0 + j], pl.side[s0 + j], tokens, cfg)
        if s0 == 0:
            parity = gate_vector(q, gate, "turboQuant", k[0], cache.planes[0].codes[0], cache.planes[0].side[0], cfg)
        torch.cuda.synchronize()
        del k, v
    cache.tokens = tokens
    # the whole-cache launch must give what the stand-alone decoder gives for the same codes
    ko, _ = cache.decode()
    alone = torch.empty((tokens, d), dtype=torch.float16, device=q.device)
    q.enqueue_decode(cache.planes[0].codes[segments - 1], cache.planes[0].side[segments - 1], alone, tokens, cfg)
    if not torch.equal(ko[segments - 1], alone):
        raise SystemExit("parity gate failed: whole-cache decode differs from the stand-alone decoder")
    del alone
    t = time_launches(lambda i: cache.decode(), 1, reps)
    nbytes = cache.stored_bytes() + cache.decoded_bytes()
    yield row("cfg5-shard", "whole-cache decode", t, 2 * segments * tokens, "vectors", nbytes,
              {"method": "turboQuant", "dim": d, "bits": bits, "segments": segments, "tokens": tokens, "out_dtype": "float16",
               "decode_output_GB_per_s": round(cache.decoded_bytes() / t / 1e9, 1), "parity": parity})
    # attention straight from this shard (8 query heads per KV head, as Llama-3-70B has), gated against
    # float64 attention over one segment decoded by the stand-alone decoder
    g = torch.Generator(device=q.device)
    g.manual_seed(55)
    qs = torch.randn((segments, 8, d), generator=g, device=q.device)
    got = cache.attend(qs)
    rk = torch.empty((tokens, d), dtype=torch.float32, device=q.device)
    rv = torch.empty((tokens, d), dtype=torch.float32, device=q.device)
    s = segments // 2
    q.enqueue_decode(cache.planes[0].codes[s], cache.planes[0].side[s], rk, tokens, cfg)
    q.enqueue_decode(cache.planes[1].codes[s], cache.planes[1].side[s], rv, tokens, cfg)
    ref = torch.softmax((qs[s].double() @ rk.double().T) * d ** -0.5, dim=1) @ rv.double()
    worst = float(((got[s].double() - ref).norm(dim=1) / ref.norm(dim=1)).max())
    if worst > 1e-4:
        raise SystemExit(f"parity gate failed: cache attention at dim 128 differs from attention over the decoded cache by {worst}")
    del rk, rv, ref
    out = torch.empty_like(qs)
    for prec in ("float32", "bfloat16"):
        ta = time_launches(lambda i: cache.attend(qs, out=out, precision=prec), 1, reps)
        yield row("cfg5-shard", f"attention from the compressed cache, {prec} operands", ta, segments * tokens, "kv_tokens",
                  cache.stored_bytes(), {"dim": d, "bits": bits, "segments": segments, "tokens": tokens, "n_queries": 8, "precision": prec,
                                         "parity": {"max_rel_l2_vs_float64_attention_over_decoded_cache": worst}})


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

    # parity gate: the fused result against float64 attention over this cache's own decoded float32 planes
    ko, vo = None, None
    ref_cache_k = torch.empty((tokens, d), dtype=torch.float32, device=q.device)
    ref_cache_v = torch.empty((tokens, d), dtype=torch.float32, device=q.device)
    got = cache.attend(qs[0])
    worst = 0.0
    for s in (0, segments // 2, segments - 1):
        q.enqueue_per_channel_decode(cache.planes[0].codes[s], cache.planes[0].side[s], ref_cache_k, tokens, cache.planes[0].config)
        q.enqueue_decode(cache.planes[1].codes[s], cache.planes[1].side[s], ref_cache_v, tokens, cache.planes[1].config)
        sc = (qs[0][s].double() @ ref_cache_k.double().T) * d ** -0.5
        ref = torch.softmax(sc, dim=1) @ ref_cache_v.double()
        worst = max(worst, float(((got[s].double() - ref).norm(dim=1) / ref.norm(dim=1)).max()))
    if worst > 5e-5:
        raise SystemExit(f"parity gate failed: cache attention differs from attention over the decoded cache by {worst}")
    del ref_cache_k, ref_cache_v

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
    yield row("cfg4 attention", "attention from the compressed cache", t, segments * tokens, "kv_tokens", stored,
              {**extra, "precision": "float32", "parity": {"max_rel_l2_vs_float64_attention_over_decoded_cache": worst}})
    got16 = cache.attend(qs[0], precision="bfloat16")
    worst16 = float(((got16.double() - got.double()).norm(dim=2) / got.double().norm(dim=2)).max())
    if worst16 > 5e-3:
        raise SystemExit(f"parity gate failed: bf16-operand cache attention differs from the float32-accurate one by {worst16}")
    t16 = timed(lambda i: cache.attend(qs[i % 4], out=out, precision="bfloat16"))
    yield row("cfg4 attention", "attention from the compressed cache, bf16 operands", t16, segments * tokens, "kv_tokens", stored,
              {**extra, "precision": "bfloat16", "tokens_per_s": round(segments * tokens / t16, 1),
               "parity": {"max_rel_l2_vs_float32_accurate_mode": worst16}})

    def two_step(i):
        ko, vo = cache.decode()
        torch.nn.functional.scaled_dot_product_attention(qs[i % 4].to(torch.bfloat16).unsqueeze(0), ko.unsqueeze(0), vo.unsqueeze(0))
    t2 = timed(two_step)
    yield row("cfg4 attention", "decode, then torch SDPA over the decoded cache", t2, segments * tokens, "kv_tokens",
              stored + 2 * cache.decoded_bytes(), {**extra, "speedup_of_fused": round(t2 / t, 2)})

    # the same shape with TurboQuant keys (the query is rotated once instead of un-rotating every key)
    tcfg = QuantConfig("turboQuant", d, 4)
    tcache = KVCache(segments, d, tokens, QuantConfig("turboQuant", d, 4, seed=777), tcfg, out_dtype="bfloat16", pitch=q)
    for s0 in range(0, segments, 8):
        x = lognormal_vectors(8 * tokens, d, 40 + s0, q.device).reshape(8, tokens, d)
        for pl in tcache.planes:
            for j in range(8):
                q.enqueue_encode(x[j], pl.codes[s0 + j], pl.side[s0 + j], tokens, pl.config)
        torch.cuda.synchronize()
        del x
    tcache.tokens = tokens
    got = tcache.attend(qs[0])
    rk = torch.empty((tokens, d), dtype=torch.float32, device=q.device)
    rv = torch.empty((tokens, d), dtype=torch.float32, device=q.device)
    worst_t = 0.0
    for s in (0, segments - 1):
        q.enqueue_decode(tcache.planes[0].codes[s], tcache.planes[0].side[s], rk, tokens, tcache.planes[0].config)
        q.enqueue_decode(tcache.planes[1].codes[s], tcache.planes[1].side[s], rv, tokens, tcache.planes[1].config)
        ref = torch.softmax((qs[0][s].double() @ rk.double().T) * d ** -0.5, dim=1) @ rv.double()
        worst_t = max(worst_t, float(((got[s].double() - ref).norm(dim=1) / ref.norm(dim=1)).max()))
    if worst_t > 1e-4:
        raise SystemExit(f"parity gate failed: cache attention with TurboQuant keys differs from attention over the decoded cache by {worst_t}")
    del rk, rv
    for prec in ("float32", "bfloat16"):
        tt = timed(lambda i: tcache.attend(qs[i % 4], out=out, precision=prec))
        yield row("cfg4-shape TurboQuant keys", f"attention from the compressed cache, {prec} operands", tt, segments * tokens, "kv_tokens",
                  tcache.stored_bytes(), {**extra, "precision": prec, "tokens_per_s": round(segments * tokens / tt, 1),
                                          "parity": {"max_rel_l2_vs_float64_attention_over_decoded_cache": worst_t}})
    del tcache

    # end to end with host buffers: queries from pinned host memory, result back to pinned host memory, waited for
    hq = torch.randn((8, segments, n_queries, d)).pin_memory()
    ho = torch.empty((segments, n_queries, d)).pin_memory()
    dq = torch.empty((segments, n_queries, d), device=q.device)
    stream = torch.cuda.current_stream(q.device)

    def e2e(i):
        dq.copy_(hq[i % 8], non_blocking=True)
        cache.attend(dq, out=out)
        ho.copy_(out, non_blocking=True)
        stream.synchronize()
    for i in range(3):
        e2e(i)
    import time as _time
    t0 = _time.perf_counter()
    for i in range(reps):
        e2e(i)
    te = (_time.perf_counter() - t0) / reps
    yield row("cfg4 attention", "end to end: queries from host memory, result to host memory, every call waited for", te,
              segments * tokens, "kv_tokens", stored, {**extra, "l2": "not flushed", "h2d_bytes": int(dq.numel() * 4), "d2h_bytes": int(out.numel() * 4)})


def bench_key_bias(q, reps, segments=48, tokens=32768):
    """Whole-cache decode with exact key-bias removal (TurboQuant keys and values, d=64, bf16 out)."""
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
        parity = None
        if bias is not None:
            # parity gate: the one-launch result equals decode without the option followed by the separate element-wise pass
            ko, _ = cache.decode()
            got = ko[segments - 1].clone()
            plain = KVCache(1, d, tokens, cfg, cfg, out_dtype="bfloat16", pitch=q)
            plain.planes[0].codes.copy_(cache.planes[0].codes[segments - 1:segments])
            plain.planes[0].side.copy_(cache.planes[0].side[segments - 1:segments])
            plain.tokens = tokens
            po, _ = plain.decode()
            q.enqueue_rope_bias(po, kb[0][segments - 1:segments].contiguous(), kb[1], kb[2], first_position=0, subtract=False)
            if not torch.equal(got, po[0]):
                raise SystemExit("parity gate failed: decode with key-bias removal differs from decode + separate bias pass")
            parity = {"equals_decode_plus_separate_pass": True}
            del plain, po, got
        t = time_launches(lambda i: cache.decode(), 1, reps)
        nbytes = cache.stored_bytes() + cache.decoded_bytes()
        yield row("cfg4-shape TurboQuant keys", "whole-cache decode " + name, t, 2 * segments * tokens, "vectors", nbytes,
                  {"dim": d, "segments": segments, "tokens": tokens, "out_dtype": "bfloat16", "parity": parity})
        del cache


def run(q, which, reps=50, gate=None, cfg5_segments=80):
    """Yields one dict per measurement of the configurations named in `which`."""
    few = max(5, reps // 5)
    if "cfg1" in which:
        yield from bench_vector(q, "cfg1", "turboQuant", 65536, 64, 4, reps, gate=gate)
        yield from bench_vector(q, "cfg1 x64 batch", "turboQuant", 65536 * 64, 64, 4, few, gate=gate)
        yield from bench_vector(q, "cfg1 x64 batch", "turboQuant", 65536 * 64, 64, 4, few, torch.bfloat16, gate=gate)
    if "cfg2" in which:
        yield from bench_channel(q, "cfg2", 32768, 64, 4, 64, reps, gate=gate)
        yield from bench_channel(q, "cfg2 x48 heads", 32768 * 48, 64, 4, 64, few, gate=gate)
    if "cfg3" in which:
        for bits in (3, 4):
            yield from bench_vector(q, "cfg3", "polarQuant", 1 << 20, 128, bits, few, gate=gate)
    if "sweep" in which:
        for method in ("turboQuant", "polarQuant"):
            for d in (64, 128, 256, 512, 1024):
                yield from bench_vector(q, "cfg3 sweep", method, (1 << 27) // d, d, 4, few, gate=gate)
    if "attn" in which:
        yield from bench_attention(q, few)
    if "bias" in which:
        yield from bench_key_bias(q, few)
    if "cfg5" in which:
        for bits in (4, 3):
            yield from bench_cfg5(q, bits, max(3, reps // 10), segments=cfg5_segments, gate=gate)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--only", default="cfg1,cfg2,cfg3,sweep")
    ap.add_argument("--reps", type=int, default=50)
    ap.add_argument("--cfg5-segments", type=int, default=80, help="segments of the config 5 shard (80 = one GPU's share of 640)")
    args = ap.parse_args()
    for r in run(PITCH(), set(args.only.split(",")), args.reps, None, args.cfg5_segments):
        print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
