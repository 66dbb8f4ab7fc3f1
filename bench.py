#!/usr/bin/env python
"""Benchmark of the B200 BitNet ternary x int8 linear path: batch-1 greedy decode of a BitNet-b1.58-2B-shaped
ternary decoder (30 blocks, hidden 2560, FFN 6912, 20 query / 5 KV heads x 128, vocab 128256, fp32 tied head).

A step is one decode token.  Weights are synthetic (seeded N(0, 0.02) masters ternarised per matrix by absmean
on the device); the prompt is seeded uniform token ids.  One JSON line is printed by rank 0.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--prompt P] [--layers L] [--vocab V]

N > 1: the 2B shape has 5 KV heads, which no tensor-parallel degree above 1 divides, so every rank runs an
independent replica ("replicas only", weak scaling) and the value is the sum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE = dict(layers=30, hidden=2560, heads=20, kv_heads=5, head_dim=128, inter=6912, vocab=128256, eps=1e-5,
             theta=500000.0, max_seq_len=2048)
METRIC = "decode tok/s (BitNet-2B shape, bs=1); ternary-linear HBM GB/s vs peak"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
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
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def algorithmic_bytes(shape, ctx_len):
    """Bytes one decode token has to move: packed weights once, int8 activations, fp32/fp64 vectors, KV, head."""
    H, I, qd, kvd = shape["hidden"], shape["inter"], shape["heads"] * shape["head_dim"], shape["kv_heads"] * shape["head_dim"]

    def lin(rows, cols):  # packed words + int8 activations + fp32 outputs
        return rows * ((cols + 15) // 16) * 4 + cols + rows * 4

    per_block = lin(qd, H) + 2 * lin(kvd, H) + lin(H, qd) + 2 * lin(I, H) + lin(H, I)
    ternary = shape["layers"] * per_block
    kv = shape["layers"] * 2 * ctx_len * kvd * 4
    head = shape["vocab"] * H * 4 + shape["vocab"] * 4
    return ternary, kv, head


def build_model(ctx, torch, shape, seed):
    from loom_b200 import cabi
    dev = torch.device("cuda", ctx.device)
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    H, I, hd = shape["hidden"], shape["inter"], shape["head_dim"]
    qd, kvd = shape["heads"] * hd, shape["kv_heads"] * hd
    dims = ((qd, H), (kvd, H), (kvd, H), (H, qd), (I, H), (I, H), (H, I))
    dec = cabi.Decoder(ctx, shape["layers"], H, shape["heads"], shape["kv_heads"], hd, I, shape["vocab"], shape["eps"],
                       shape["theta"], cabi.ACT_SILU, shape["max_seq_len"])
    weights = []
    for b in range(shape["layers"]):
        ws = []
        for r, c in dims:
            master = torch.randn(r * c, device=dev, generator=g, dtype=torch.float32) * 0.02
            ws.append(ctx.pack_ternary_f32(master, r, c))
            del master
        dec.set_block(b, ws)
        weights.append(ws)
    emb = torch.randn(shape["vocab"], H, device=dev, generator=g, dtype=torch.float32) * 0.02
    dec.set_embeddings(emb)
    return dec, weights, emb


def gemv_roofline(ctx, torch, weights, shape, reps=20):
    """Average launch duration of the ternary GEMV over every block's gate and down matrix (60 distinct
    matrices of 4.4 MB, more than L2), replayed as one recorded frame; CUDA events on the launching stream."""
    dev = torch.device("cuda", ctx.device)
    H, I = shape["hidden"], shape["inter"]
    xg = torch.randn(1, H, device=dev)
    xd = torch.randn(1, I, device=dev)
    qg, ag = torch.empty(1, H, dtype=torch.int8, device=dev), torch.empty(1, device=dev)
    qd_, ad = torch.empty(1, I, dtype=torch.int8, device=dev), torch.empty(1, device=dev)
    ctx.quantize_activation(1, H, xg, qg, ag)
    ctx.quantize_activation(1, I, xd, qd_, ad)
    og, od = torch.empty(1, I, device=dev), torch.empty(1, H, device=dev)

    def run():
        for ws in weights:
            ctx.ternary_linear(ws[4], 1, qg, ag, og)
            ctx.ternary_linear(ws[6], 1, qd_, ad, od)

    run()
    ctx.sync()
    ctx.graph_begin()
    run()
    gr = ctx.graph_end()
    for _ in range(3):
        ctx.graph_launch(gr)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        ctx.graph_launch(gr)
    e1.record()
    torch.cuda.synchronize()
    launches = reps * 2 * len(weights)
    us = e0.elapsed_time(e1) * 1e3 / launches
    ctx.graph_free(gr)
    bytes_gate = I * ((H + 15) // 16) * 4 + H + I * 4
    bytes_down = H * ((I + 15) // 16) * 4 + I + H * 4
    per_launch = 0.5 * (bytes_gate + bytes_down)
    return {"bytes": per_launch, "us": us, "launches": launches, "gbs": per_launch / us / 1e3}


def linears_roofline(ctx, torch, dec, shape, reps=20):
    """The ternary projections of one decode step as the step runs them (the fused-prologue instantiations: QKV with the
    block norm, O with the inner norm from float64 + residual, gate+up with the block norm + SwiGLU, down with the inner
    norm + residual; every block, so 30 x 17.4 MB of distinct packed weights, far beyond L2), without attention and head,
    replayed as one recorded frame; CUDA events on the launching stream.  Algorithmic bytes = packed words + int8 rows
    + fp32 outputs of the seven matrices of every block."""
    dec.linears_frame()
    ctx.sync()
    ctx.graph_begin()
    dec.linears_frame()
    gr = ctx.graph_end()
    for _ in range(3):
        ctx.graph_launch(gr)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        ctx.graph_launch(gr)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / reps
    ctx.graph_free(gr)
    tern_b, _, _ = algorithmic_bytes(shape, 0)
    # ncu: 2.57 + 1.76 + 8.96 + 4.56 MB read per block for 17.39 MB algorithmic, 0 written
    traffic = 17.85e6 * shape["layers"]
    return {"bytes": tern_b, "us": us, "gbs": tern_b / us / 1e3, "traffic": traffic}


def run_tp_check(dist, local, world):
    """Before a multi-GPU run is timed: the tensor-parallel path on these GPUs against the CPU oracle's unsharded
    decoder (a small sharded decoder; exact int32 all-reduce; row-sharded linear bit-exact; every rank's logits
    bit-identical; greedy tokens equal to the oracle's), once over NCCL inside the recorded frame and once over the
    peer mailboxes.  The oracle is the checker here, nothing of it is timed.  Returns "ok" or "failed: ..."."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    try:
        import datetime

        import tp_gpu_worker
        gloo = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=180))
        problems = []
        for mode in ("graph", "peer"):
            try:
                failures, _ = tp_gpu_worker.run_checks(mode, local, group=gloo)
            except Exception as exc:
                failures = ["%s: %r" % (type(exc).__name__, exc)]
            problems += ["%s: %s" % (mode, f) for f in failures]
        flag = [None] * world
        dist.all_gather_object(flag, problems, group=gloo)
        allp = ["rank %d %s" % (r, p) for r, ps in enumerate(flag) for p in ps]
        return "ok" if not allp else "failed: " + "; ".join(allp)[:600]
    except Exception as exc:
        return "failed: %r" % (exc,)


def bench_config(args, shape, world):
    """The `config` object of the JSON line: a function of the command line only, so that the two arms of a run
    (`--impl ours` and `--impl reference`) print the same object."""
    return {"workload": "BitNet-b1.58-2B-shape ternary decoder, batch-1 greedy decode (configs[2])",
            "layers": shape["layers"], "hidden": shape["hidden"], "vocab": shape["vocab"], "prompt": args.prompt,
            "context_first_timed_step": args.prompt + args.warmup + 1,
            "parallelism": "replicas only" if world > 1 else "single GPU",
            "l2": "every step streams 0.5 GB of packed weights + 1.3 GB fp32 head, far beyond the 126 MB L2"}


def host_decoder(shape, blocks, ctx_len, seed):
    """A `blocks`-deep decoder of the benchmark's widths for the CPU oracle, built on the host only (no GPU, nothing
    of the CUDA library): packed words drawn with the code frequencies that absmean ternarisation gives N(0, sigma)
    masters (P(0) = P(|z| < 0.399) = 0.310, P(+1) = P(-1) = 0.345), per-matrix scale 0.798 * 0.02, seeded N(0, 1) KV rows
    for `ctx_len` positions, seeded N(0, 0.02) tied embedding / head.  The CPU kernels' time does not depend on the values."""
    from oracle import oracle as orc
    s = shape
    rng = np.random.default_rng(seed)
    H, I, hd = s["hidden"], s["inter"], s["head_dim"]
    qd, kvd = s["heads"] * hd, s["kv_heads"] * hd
    dims = ((qd, H), (kvd, H), (kvd, H), (H, qd), (I, H), (I, H), (H, I))
    odec = orc.Decoder(blocks, H, s["heads"], s["kv_heads"], hd, I, s["vocab"], s["eps"], s["theta"], orc.ACT_SILU, s["max_seq_len"])
    shifts = (2 * np.arange(16, dtype=np.uint32)).reshape(1, 1, 16)
    for b in range(blocks):
        words = []
        for r, c in dims:
            assert c % 16 == 0
            u = rng.random((r, c // 16, 16), dtype=np.float32)
            codes = (u >= 0.345).astype(np.uint32) + (u >= 0.655).astype(np.uint32)  # 0 / 1 / 2 = weight -1 / 0 / +1
            words.append(np.bitwise_or.reduce(codes << shifts, axis=2).astype(np.uint32))
        odec.set_block_packed(b, words, [np.float32(0.798 * 0.02)] * 7)
        k = rng.standard_normal((ctx_len, kvd), dtype=np.float32)
        v = rng.standard_normal((ctx_len, kvd), dtype=np.float32)
        odec.set_kv(b, ctx_len, k, v)
    emb = rng.standard_normal((s["vocab"], H), dtype=np.float32) * np.float32(0.02)
    odec.set_embeddings(emb)
    return odec, emb


def cpu_decode_rate(shape, blocks, ctx_len, tokens, threads, seed):
    """Greedy decode tokens/s of the CPU oracle (restatement of the reference's Go path: AVX2 byte-code kernel, rows
    fanned out over `threads` workers, float64 attention and head) on a `blocks`-deep decoder at context `ctx_len`.
    When `blocks` is less than the model's depth the block time is scaled by depth / blocks and the head counted once."""
    from oracle import oracle as orc
    odec, emb = host_decoder(shape, blocks, ctx_len, seed)
    tok = np.array([1], np.int32)
    logits = odec.forward(tok, simd=1, threads=threads)  # builds the byte-code caches: untimed, like the reference's bench
    times = []
    for _ in range(tokens):
        tok[0] = orc.argmax(logits)
        t0 = time.perf_counter()
        logits = odec.forward(tok, simd=1, threads=threads)  # attention single-threaded, as in the reference
        times.append(time.perf_counter() - t0)
    per_token = float(np.mean(times))
    if blocks < shape["layers"]:
        hid = np.zeros(shape["hidden"], np.float32)
        th = []
        for _ in range(3):
            t0 = time.perf_counter()
            orc.lm_head(hid, emb, threads=threads)
            th.append(time.perf_counter() - t0)
        head = float(np.median(th))
        per_token = max(per_token - head, 1e-9) * (shape["layers"] / blocks) + head
    return 1.0 / per_token, tokens


def gemm_mode(args):
    """Config 1 (batched prefill): M tokens through the gate (2560->6912) and down (6912->2560) projections on
    the tcgen05 GEMM, per-token quantization included; eight distinct matrices per shape, CUDA events."""
    import torch

    import loom_b200

    torch.cuda.set_device(0)
    ts = torch.cuda.Stream()
    torch.cuda.set_stream(ts)
    ctx = loom_b200.Context(0, ts.cuda_stream)
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(args.seed)
    M = args.tokens
    res = {}
    for name, rows, cols in (("gate", 6912, 2560), ("down", 2560, 6912)):
        ws = [ctx.pack_ternary_f32(torch.randn(rows * cols, device=dev, generator=g) * 0.02, rows, cols) for _ in range(8)]
        x = torch.randn(M, cols, device=dev, generator=g)
        out = torch.empty(M, rows, device=dev)
        # weights as pre-expanded int8 codes (the default; built untimed on each matrix's first GEMM), then as 2-bit tiles
        # expanded inside the kernel
        for cached in (1, 0):
            ctx.set_option("gemm_cache", cached)
            for i in range(max(args.warmup, 3, 8)):
                ctx.ternary_gemm(ws[i % 8], M, x, out=out)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.steps):
                ctx.ternary_gemm(ws[i % 8], M, x, out=out)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / args.steps
            res[name if cached else name + "_expand_in_kernel"] = {"us": us, "tops": 2.0 * M * rows * cols / us / 1e6}
        ctx.set_option("gemm_cache", 1)
    # config 0 beside it: the same two shapes at M = 1 through the decode GEMV (16 distinct matrices per replay)
    gemv = {}
    for name, rows, cols in (("gate", 6912, 2560), ("down", 2560, 6912)):
        ws = [ctx.pack_ternary_f32(torch.randn(rows * cols, device=dev, generator=g) * 0.02, rows, cols) for _ in range(16)]
        x = torch.randn(1, cols, device=dev, generator=g)
        q, am = torch.empty(1, cols, dtype=torch.int8, device=dev), torch.empty(1, device=dev)
        ctx.quantize_activation(1, cols, x, q, am)
        out1 = torch.empty(1, rows, device=dev)
        for w in ws:
            ctx.ternary_linear(w, 1, q, am, out1)
        ctx.sync()
        ctx.graph_begin()
        for w in ws:
            ctx.ternary_linear(w, 1, q, am, out1)
        gr = ctx.graph_end()
        for _ in range(3):
            ctx.graph_launch(gr)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            ctx.graph_launch(gr)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (20 * len(ws))
        nbytes = rows * ((cols + 15) // 16) * 4 + cols + rows * 4
        gemv[name] = {"us": us, "gbs": nbytes / us / 1e3, "bytes": nbytes}
        ctx.graph_free(gr)
    # CPU baseline on a bounded sample: the oracle's Dense forward (scalar packed path and AVX2 byte-code path, all host
    # threads), one token at a time like the reference, 8 tokens per shape; M tokens cost M times as much
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import oracle as orc
        threads = orc.host_threads()
        rng = np.random.default_rng(args.seed)
        cpu = {"cores": threads}
        for name, rows, cols in (("gate", 6912, 2560), ("down", 2560, 6912)):
            m = orc.Matrix.from_f32((rng.standard_normal(rows * cols) * 0.02).astype(np.float32), rows, cols)
            xs = rng.standard_normal((8, cols)).astype(np.float32)
            for simd in (0, 1):
                orc.dense_forward(m, orc.ACT_LINEAR, xs[:1], simd=simd, threads=threads)  # builds the byte-code cache (simd=1), untimed
                t0 = time.perf_counter()
                orc.dense_forward(m, orc.ACT_LINEAR, xs, simd=simd, threads=threads)
                cpu["%s_%s_us_per_token" % (name, "avx2" if simd else "scalar")] = (time.perf_counter() - t0) / 8 * 1e6
    peak_bf16 = 1610.8
    try:
        peak_bf16 = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        pass
    tops = 0.5 * (res["gate"]["tops"] + res["down"]["tops"])
    peak_i8 = ctx.i8_peak_tops(20000)  # measured on this GPU: back-to-back tcgen05 kind::i8 MMAs, operands in shared memory
    print(json.dumps({"metric": "prefill GEMM TOP/s (M=%d, 2560<->6912 ternary x int8, tcgen05 kind::i8)" % M, "value": tops,
                      "unit": "TOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
                      "ms_per_step": 1e-3 * 0.5 * (res["gate"]["us"] + res["down"]["us"]), "higher_is_better": True,
                      "dtype": "u8 codes x s8 -> s32 (tcgen05), fp64 rescale", "data": "synthetic",
                      "config": {"workload": "configs[1]: batched prefill, M=%d tokens" % M, "detail": res,
                                 "config0_gemv_m1": gemv},
                      "cpu_baseline": None if cpu is None else {
                          "value": 2.0 * 6912 * 2560 / (0.5 * (cpu["gate_avx2_us_per_token"] + cpu["down_avx2_us_per_token"])) / 1e6,
                          "unit": "TOP/s", "cores": cpu["cores"], "kind": "port",
                          "sample": "8 tokens per shape, one at a time like the reference; per-token microseconds in detail",
                          "detail": cpu},
                      "roofline": {"bound": "tensor", "achieved": tops, "peak": peak_i8, "unit": "TOP/s",
                                   "frac": tops / peak_i8, "traffic": None,
                                   "peak_kind": "measured here: tcgen05 kind::i8 micro-peak (M128 N256 K32, no loads)",
                                   "cross_check_2x_bf16_burst": 2 * peak_bf16}}))
    return 0


def sweep_mode(args):
    """Batch sweep of one ternary projection pair (gate: inter x hidden, down: hidden x inter of --shape) at M = 1 ... 256
    tokens: the decode GEMV (eight tokens per weight pass) against the tcgen05 GEMM (quantizer included), with the
    fraction of the HBM roofline (packed weight bytes per pass / time) and of the int8 tensor roofline (2*M*K*N / time)
    for each, and the crossover batch.  Kernel-level stand-in for the decode batch sweeps of configs 3-4."""
    import torch

    import loom_b200

    shape = {"2b": SHAPE, **TP_SHAPES}[args.shape]
    H, I = shape["hidden"], shape["inter"]
    torch.cuda.set_device(0)
    ts = torch.cuda.Stream()
    torch.cuda.set_stream(ts)
    ctx = loom_b200.Context(0, ts.cuda_stream)
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(args.seed)
    peak, peak_kind = measured_peaks()
    peak_bf16 = 1610.8
    try:
        peak_bf16 = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        pass
    peak_i8 = ctx.i8_peak_tops(20000)
    rows_out = []
    for name, rows, cols in (("gate", I, H), ("down", H, I)):
        wbytes = rows * ((cols + 15) // 16) * 4
        nmat = max(2, min(16, int(300e6 // wbytes) + 1))  # distinct matrices beyond the 126 MB L2
        ws = [ctx.pack_ternary_f32(torch.randn(rows * cols, device=dev, generator=g) * 0.02, rows, cols) for _ in range(nmat)]
        for M in (1, 8, 16, 32, 64, 128, 256):
            x = torch.randn(M, cols, device=dev, generator=g)
            q, am = torch.empty(M, cols, dtype=torch.int8, device=dev), torch.empty(M, device=dev)
            out = torch.empty(M, rows, device=dev)

            def gemv():
                ctx.quantize_activation(M, cols, x, q, am)
                for w in ws:
                    ctx.ternary_linear(w, M, q, am, out)

            def gemm():
                for w in ws:
                    ctx.ternary_gemm(w, M, x, out=out)

            res = {}
            for kind, fn in (("gemv", gemv), ("gemm", gemm)):
                fn()  # sizes every scratch buffer
                ctx.sync()
                ctx.graph_begin()  # a recorded frame: the Python launch loop would otherwise be what is timed
                fn()
                gr = ctx.graph_end()
                for _ in range(3):
                    ctx.graph_launch(gr)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.steps):
                    ctx.graph_launch(gr)
                e1.record()
                torch.cuda.synchronize()
                res[kind] = e0.elapsed_time(e1) * 1e3 / (args.steps * nmat)
                ctx.graph_free(gr)
            per_pass = 8 if cols <= 19000 else 5  # tokens one GEMV pass carries (shared-memory bound for very wide rows)
            passes = (M + per_pass - 1) // per_pass
            rows_out.append({"matrix": "%s %dx%d" % (name, rows, cols), "M": M, "gemv_us": res["gemv"], "gemm_us": res["gemm"],
                             "gemv_hbm_frac": passes * wbytes / res["gemv"] / 1e3 / peak,
                             "gemm_tensor_frac": 2.0 * M * rows * cols / res["gemm"] / 1e6 / peak_i8,
                             "gemm_hbm_frac": wbytes / res["gemm"] / 1e3 / peak,
                             "faster": "gemm" if res["gemm"] < res["gemv"] else "gemv"})
        del ws
    cross = {}
    for r in rows_out:
        if r["faster"] == "gemm" and r["matrix"] not in cross:
            cross[r["matrix"]] = r["M"]
    best = max(r["gemv_hbm_frac"] for r in rows_out if r["M"] == 1)
    print(json.dumps({"metric": "ternary projection batch sweep (%s shape): GEMV vs tcgen05 GEMM" % args.shape.upper(), "value": best,
                      "unit": "fraction of measured HBM peak, GEMV at M=1", "n_gpus": 1, "steps": args.steps, "warmup": 3,
                      "higher_is_better": True, "dtype": "int8 x ternary -> int32, fp64 rescale", "data": "synthetic",
                      "config": {"workload": "gate and down projections of the %s shape, M = 1..256 tokens" % args.shape.upper(),
                                 "crossover_M": cross, "peaks": {"hbm_gbs": peak, "int8_tops": peak_i8,
                                                                 "int8_kind": "measured here: tcgen05 kind::i8 micro-peak",
                                                                 "cross_check_2x_bf16_burst": 2 * peak_bf16}},
                      "sweep": rows_out}))
    return 0


TP_SHAPES = {
    "8b": dict(layers=32, hidden=4096, heads=32, kv_heads=8, head_dim=128, inter=14336, vocab=128256, eps=1e-5,
               theta=500000.0, max_seq_len=1024),
    "70b": dict(layers=80, hidden=8192, heads=64, kv_heads=8, head_dim=128, inter=28672, vocab=128256, eps=1e-5,
                theta=500000.0, max_seq_len=1024),
}


def apply_opts(ctx, args):
    """`--opt key=value` (repeatable): context options for A/B runs (`loom_b200_ctx_set_option`)."""
    for kv in getattr(args, "opt", None) or []:
        k, v = kv.split("=")
        ctx.set_option(k, int(v))


def tp_decode_measure(args, torch, dist, rank, world, local, shape_name, layers, steps, warmup, exchange):
    """Builds rank `rank`'s part of a `shape_name`-shaped ternary decoder (column-sharded Q/K/V/gate/up, row-sharded O/down,
    vocabulary-sharded head) on a context of its own, times `steps` device-resident greedy decode steps (CUDA events,
    barrier + synchronize on both sides, max over ranks) and returns the figures.  Each rank ternarises its own slices
    (synthetic weights, so the per-slice absmean scale stands in for the whole-matrix one; timing does not depend on it)."""
    import loom_b200
    from loom_b200 import cabi

    shape = dict(TP_SHAPES[shape_name])
    if layers:
        shape["layers"] = layers
    dev = torch.device("cuda", local)
    tstream = torch.cuda.Stream()
    torch.cuda.set_stream(tstream)
    ctx = loom_b200.Context(local, tstream.cuda_stream)
    apply_opts(ctx, args)
    if world > 1:
        idt = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            idt.copy_(torch.frombuffer(bytearray(cabi.Context.tp_unique_id()), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        torch.cuda.synchronize()
        ctx.tp_init(rank, world, bytes(idt.cpu().numpy().tobytes()))
        if exchange == "peer":  # row-parallel projections exchange through peer mailboxes (CUDA IPC over NVLink)
            mine = torch.frombuffer(bytearray(ctx.tp_peer_handle()), dtype=torch.uint8).to(dev)
            allh = [torch.zeros(64, dtype=torch.uint8, device=dev) for _ in range(world)]
            dist.all_gather(allh, mine)
            torch.cuda.synchronize()
            ctx.tp_attach_peers(b"".join(bytes(t.cpu().numpy().tobytes()) for t in allh))
    H, I, hd = shape["hidden"], shape["inter"], shape["head_dim"]
    qd_l, kvd_l, I_l = shape["heads"] // world * hd, shape["kv_heads"] // world * hd, I // world
    dims = ((qd_l, H), (kvd_l, H), (kvd_l, H), (H, qd_l), (I_l, H), (I_l, H), (H, I_l))
    g = torch.Generator(device=dev)
    g.manual_seed(args.seed + rank)
    dec = cabi.Decoder(ctx, shape["layers"], H, shape["heads"], shape["kv_heads"], hd, I, shape["vocab"], shape["eps"],
                       shape["theta"], cabi.ACT_SILU, shape["max_seq_len"])
    keep = []
    for b in range(shape["layers"]):
        ws = []
        for r, c in dims:
            master = torch.randn(r * c, device=dev, generator=g, dtype=torch.float32) * 0.02
            ws.append(ctx.pack_ternary_f32(master, r, c))
            del master
        dec.set_block(b, ws)
        keep.append(ws)
    ge = torch.Generator(device=dev)
    ge.manual_seed(args.seed)  # the embedding table is replicated: the same on every rank
    emb = torch.randn(shape["vocab"], H, device=dev, generator=ge, dtype=torch.float32) * 0.02
    dec.set_embeddings(emb)
    rng = np.random.default_rng(args.seed)
    n_prompt = min(args.prompt, 64)  # under a tensor-parallel group prompts run eight tokens per pass: keep it short
    prompt = rng.integers(0, shape["vocab"], n_prompt).astype(np.int32)
    warmup = max(warmup, 3)
    assert n_prompt + warmup + steps + 40 <= shape["max_seq_len"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    dec.generate(prompt, warmup)
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    dec.continue_greedy(steps)
    e1.record()
    barrier()
    dev_s = e0.elapsed_time(e1) * 1e-3
    clocks = sampler.stop()
    # end to end: token id in, logits out, host argmax
    logits = dec.forward(np.array([int(prompt[0])], np.int32))
    tok = int(np.argmax(logits))
    e2e_steps = min(steps, 32)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        logits = dec.forward(np.array([tok], np.int32))
        tok = int(np.argmax(logits))
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([dev_s, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_s, e2e_s = float(t[0].item()), float(t[1].item())
    tern_b, kv_b, head_b = algorithmic_bytes(shape, n_prompt + warmup + steps // 2)
    res = {"shape": shape_name, "layers": shape["layers"], "world": world, "exchange": "none" if world == 1 else exchange,
           "tok_per_s": steps / dev_s, "ms_per_step": 1e3 * dev_s / steps, "e2e_tok_per_s": e2e_steps / e2e_s, "e2e_steps": e2e_steps,
           "launches_per_token": dec.launches_per_token(), "prompt": n_prompt, "clocks": clocks,
           "bytes_per_gpu": (tern_b + kv_b + head_b) / world, "vocab": shape["vocab"]}
    ctx.sync()
    dec.close()
    del keep, emb
    barrier()
    ctx.tp_finalize()
    ctx.close()
    return res


def tp_mode(args):
    """Tensor-parallel batch-1 decode of an 8B / 70B-shaped ternary decoder: one process per GPU (torchrun).  Strong
    scaling: the model is fixed and the group grows."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    r = tp_decode_measure(args, torch, dist, rank, world, local, args.shape, args.layers if args.layers != SHAPE["layers"] else 0,
                          args.steps, args.warmup, args.tp_exchange)
    peak, peak_kind = measured_peaks()
    step_s = r["ms_per_step"] * 1e-3
    line = {
        "metric": "decode tok/s (%s-shape ternary decoder, bs=1, tensor parallel)" % args.shape.upper(), "value": r["tok_per_s"],
        "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 x ternary -> int32, fp64 rescale",
        "data": "synthetic",
        "config": {"workload": "Llama-3-%s-shape ternary decoder, batch-1 greedy decode" % args.shape.upper(),
                   "layers": r["layers"], "prompt": r["prompt"], "parallelism": "tp%d" % world, "exchange": r["exchange"],
                   "l2": "every step streams the rank's packed weights and head slice, far beyond the 126 MB L2"},
        "e2e": {"value": r["e2e_tok_per_s"], "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": r["vocab"] * 4,
                "steps": r["e2e_steps"]},
        "gpu_launches": int(args.steps * r["launches_per_token"]), "clocks": r["clocks"],
        "roofline": {"bound": "hbm", "achieved": r["bytes_per_gpu"] / step_s / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": r["bytes_per_gpu"] / step_s / 1e9 / peak, "traffic": None, "peak_kind": peak_kind,
                     "kernel": "whole decode step, per-GPU bytes (packed weights + KV + fp32 head slice) / step time"},
    }
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def batch_measure(args, torch, dist, rank, world, local, shape_name, B, n_prompt, steps, warmup, layers=0):
    """`B` independent sequences on a `shape_name`-shaped decoder: one GPU, or tensor-parallel over the ranks of the (already
    initialised) process group with the peer-memory exchange.  Every sequence is prefilled with a prompt of its own, then all
    advance together.  Returns the figures (device time of `steps` batch steps: CUDA events, barrier + synchronize on both
    sides, max over ranks)."""
    import loom_b200
    from loom_b200 import cabi

    shape = dict({"2b": SHAPE, **TP_SHAPES}[shape_name])
    if layers:
        shape["layers"] = layers
    warmup = max(warmup, 3)
    shape["max_seq_len"] = n_prompt + warmup + steps + 8
    ts = torch.cuda.Stream()
    torch.cuda.set_stream(ts)
    ctx = loom_b200.Context(local, ts.cuda_stream)
    apply_opts(ctx, args)
    dev = torch.device("cuda", local)
    if world > 1:
        idt = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            idt.copy_(torch.frombuffer(bytearray(cabi.Context.tp_unique_id()), dtype=torch.uint8))
        dist.broadcast(idt, 0)
        torch.cuda.synchronize()
        ctx.tp_init(rank, world, bytes(idt.cpu().numpy().tobytes()))
        mine = torch.frombuffer(bytearray(ctx.tp_peer_handle()), dtype=torch.uint8).to(dev)
        allh = [torch.zeros(64, dtype=torch.uint8, device=dev) for _ in range(world)]
        dist.all_gather(allh, mine)
        torch.cuda.synchronize()
        ctx.tp_attach_peers(b"".join(bytes(t.cpu().numpy().tobytes()) for t in allh))
    g = torch.Generator(device=dev)
    g.manual_seed(args.seed + rank)
    H, I, hd = shape["hidden"], shape["inter"], shape["head_dim"]
    qd, kvd, Il = shape["heads"] // world * hd, shape["kv_heads"] // world * hd, I // world
    dims = ((qd, H), (kvd, H), (kvd, H), (H, qd), (Il, H), (Il, H), (H, Il))
    dec = cabi.Decoder(ctx, shape["layers"], H, shape["heads"], shape["kv_heads"], hd, I, shape["vocab"], shape["eps"],
                       shape["theta"], cabi.ACT_SILU, shape["max_seq_len"])
    dec.set_batch(B)
    keep = []
    for b in range(shape["layers"]):
        ws = []
        for r, c in dims:
            master = torch.randn(r * c, device=dev, generator=g, dtype=torch.float32) * 0.02
            ws.append(ctx.pack_ternary_f32(master, r, c))
            del master
        dec.set_block(b, ws)
        keep.append(ws)
    ge = torch.Generator(device=dev)
    ge.manual_seed(args.seed)  # the embedding table is replicated: the same on every rank
    emb = torch.randn(shape["vocab"], H, device=dev, generator=ge, dtype=torch.float32) * 0.02
    dec.set_embeddings(emb)
    rng = np.random.default_rng(args.seed)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    t0 = time.perf_counter()
    for i in range(B):
        dec.select(i)
        dec.forward(rng.integers(0, shape["vocab"], n_prompt).astype(np.int32), want_logits=False)
    ctx.sync()
    prefill_s = time.perf_counter() - t0
    dec.continue_batch(warmup)
    ctx.sync()
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    dec.continue_batch(steps)
    e1.record()
    barrier()
    dev_s = e0.elapsed_time(e1) * 1e-3
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([dev_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_s = float(t[0].item())
    tern_b, kv_b, head_b = algorithmic_bytes(shape, n_prompt + warmup + steps // 2)
    passes = (B + 7) // 8
    # per GPU: weights once per pass of eight, KV of every sequence, head once per head pass of two rows
    moved = (passes * tern_b + B * kv_b + ((B + 1) // 2) * head_b) / world
    res = {"shape": shape_name, "layers": shape["layers"], "world": world, "batch": B, "prompt": n_prompt, "steps": steps,
           "tok_per_s": B * steps / dev_s, "ms_per_step": 1e3 * dev_s / steps, "per_sequence_tok_per_s": steps / dev_s,
           "prefill_seconds_all_sequences": prefill_s, "prefill_tok_per_s": B * n_prompt / prefill_s, "clocks": clocks,
           "bytes_per_gpu_per_step": moved}
    ctx.sync()
    dec.close()
    del keep, emb
    barrier()
    if world > 1:
        ctx.tp_finalize()
    ctx.close()
    return res


def batch_mode(args):
    """Decode with `--batch` independent sequences (configs[3]: 8B shape, batch 16, 2048-token prompts): up to eight
    sequences per pass over every packed matrix and several hidden rows per pass over the LM head.  value = sequences x
    steps / time.  Under torchrun the decoder is tensor-parallel over the ranks (column-sharded Q/K/V/gate/up, row-sharded
    O/down, vocabulary-sharded head whose tail exchanges (maximum, index) pairs; peer-memory exchange) and `scaling` is
    "strong"."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    r = batch_measure(args, torch, dist, rank, world, local, args.shape, args.batch, args.prompt, args.steps, args.warmup,
                      args.layers if args.layers != SHAPE["layers"] else 0)
    peak, peak_kind = measured_peaks()
    step_s = r["ms_per_step"] * 1e-3
    B = r["batch"]
    if rank == 0:
        print(json.dumps({
            "metric": "decode tok/s (%s-shape ternary decoder, %d independent sequences, %s)" % (
                args.shape.upper(), B, "one GPU" if world == 1 else "tensor parallel over %d GPUs" % world),
            "value": r["tok_per_s"], "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None,
            "dtype": "int8 x ternary -> int32, fp64 rescale", "data": "synthetic",
            "config": {"workload": "%s-shape ternary decoder, batch %d greedy decode, %d-token prompts" % (args.shape.upper(), B, args.prompt),
                       "layers": r["layers"], "batch": B, "prompt": args.prompt,
                       "parallelism": "single GPU" if world == 1 else "tp%d, peer-memory exchange" % world},
            "per_sequence_tok_per_s": r["per_sequence_tok_per_s"], "prefill_seconds_all_sequences": r["prefill_seconds_all_sequences"],
            "prefill_tok_per_s": r["prefill_tok_per_s"], "clocks": r["clocks"],
            "roofline": {"bound": "hbm", "achieved": r["bytes_per_gpu_per_step"] / step_s / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": r["bytes_per_gpu_per_step"] / step_s / 1e9 / peak, "traffic": None, "peak_kind": peak_kind,
                         "kernel": "whole batch step, per GPU: packed weights once per pass of eight sequences, KV of every sequence, fp32 head once per head pass"}}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=SHAPE["layers"])
    ap.add_argument("--vocab", type=int, default=SHAPE["vocab"], help="smaller vocabularies are for profiling captures only")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=16, help="batch mode: independent sequences")
    ap.add_argument("--opt", action="append", default=[], help="context option key=value (repeatable), e.g. --opt tp_fused=0")
    ap.add_argument("--mode", default="decode", choices=["decode", "gemm", "tp", "sweep", "batch"],
                    help="gemm: the batched-prefill GEMM microbenchmark; tp: tensor-parallel decode of --shape under torchrun; "
                         "sweep: GEMV vs GEMM over batch sizes for the gate/down projections of --shape")
    ap.add_argument("--shape", default="8b", choices=sorted(TP_SHAPES) + ["2b"])
    ap.add_argument("--tp-exchange", default="peer", choices=["peer", "nccl"],
                    help="tp mode: how the row-parallel projections exchange their partial results")
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--no-tp-section", action="store_true", help="multi-GPU runs: skip the tensor-parallel decode after the replica measurement")
    args = ap.parse_args()
    if args.mode == "gemm":
        return gemm_mode(args)
    if args.mode == "tp":
        return tp_mode(args)
    if args.mode == "batch":
        return batch_mode(args)
    if args.mode == "sweep":
        args.steps = min(args.steps, 20)
        return sweep_mode(args)
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    shape = dict(SHAPE, layers=args.layers, vocab=args.vocab)
    config = bench_config(args, shape, world)
    ctx_first = config["context_first_timed_step"]

    if args.impl == "reference":
        # The reference's own GPU path is WGSL over wgpu (no graphics stack here) and its CPU path is Go (no toolchain
        # here): this arm times the C++ restatement of that CPU path on the host cores.  Nothing of the CUDA library,
        # and no GPU, is touched.  Rank 0 alone works.
        if rank != 0:
            return 0
        from oracle import oracle as orc
        threads = orc.host_threads()
        tokens = max(8, min(args.steps, 16))
        tokps, timed = cpu_decode_rate(shape, shape["layers"], ctx_first, tokens, threads, args.seed)
        line = {"impl": "reference", "metric": METRIC, "value": tokps, "unit": "tok/s", "n_gpus": args.gpus,
                "steps": args.steps, "tokens_timed": timed, "warmup": args.warmup, "ms_per_step": 1e3 / tokps,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "int8 x ternary -> int32, fp64 rescale", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": tokps, "unit": "tok/s", "cores": threads, "kind": "port",
                                 "sample": "all %d blocks at full width + the full fp32 head on the host (C++ restatement of the "
                                           "Go CPU path, AVX2 byte-code kernel, %d threads), %d greedy tokens from context %d; "
                                           "weights and KV rows are synthetic with the benchmark's shapes and code frequencies"
                                           % (shape["layers"], threads, timed, ctx_first)},
                "e2e": {"value": tokps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    import torch
    import torch.distributed as dist

    import loom_b200

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    torch.cuda.set_device(local)
    tp_check = None
    if world > 1:
        # the check below makes ranks leave and re-join NCCL groups inside one process: keep NVLink multicast objects out of it
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        tp_check = run_tp_check(dist, local, world)
    tstream = torch.cuda.Stream()
    torch.cuda.set_stream(tstream)
    ctx = loom_b200.Context(local, tstream.cuda_stream)
    apply_opts(ctx, args)

    dec, weights, emb = build_model(ctx, torch, shape, args.seed)
    rng = np.random.default_rng(args.seed)
    prompt = rng.integers(0, shape["vocab"], args.prompt).astype(np.int32)
    assert args.prompt + args.warmup + 2 * args.steps + 8 <= shape["max_seq_len"], "prompt + steps exceed MaxSeqLen"

    # prefill + warm-up tokens (untimed); the decode frame is recorded during warm-up.  The prompt runs once before the
    # measured prefill so that the prefill figure does not include first-call allocations.
    dec.forward(prompt, want_logits=False)
    ctx.sync()
    _, m0 = dec.generate(prompt, args.warmup)
    prefill_s = m0.prefill_seconds
    ctx_len = args.prompt + args.warmup
    logits = dec.forward(np.array([int(prompt[0])], np.int32))  # one more step through the host path (warm)
    ctx_len += 1
    assert ctx_len == ctx_first
    peak, peak_kind = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timed region: exactly K decode steps, no host round trip ------------------------------
    # K steps can be as short as a few tens of milliseconds, less than one nvidia-smi sample: the region is repeated
    # from the same KV offset (the sequence is cut back to ctx_first positions) until at least 0.5 s have been timed,
    # every repetition bracketed by barrier + synchronize and timed with CUDA events; the median repetition counts.
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    reps, rep_s, total_s = 0, [], 0.0
    while reps < 3 or (total_s < 0.5 and reps < 200):
        dec.set_kv_offset(ctx_first)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        dec.continue_greedy(args.steps)
        e1.record()
        barrier()
        t = e0.elapsed_time(e1) * 1e-3
        if world > 1:
            tt = torch.tensor([t], device="cuda", dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t = float(tt.item())
        rep_s.append(t)
        total_s += t
        reps += 1
    clocks = sampler.stop()
    dev_s = float(np.median(rep_s))
    ctx_mid = ctx_first + args.steps // 2
    ctx_len = ctx_first + args.steps
    value = world * args.steps / dev_s

    # ---- end to end through the host-facing call: token id in (pinned H2D), logits out (D2H), host argmax -------
    dec.set_kv_offset(ctx_first)
    tok = int(np.argmax(logits))
    for _ in range(3):
        logits = dec.forward(np.array([tok], np.int32))
        tok = int(np.argmax(logits))
    e2e_steps = min(args.steps, shape["max_seq_len"] - ctx_first - 4)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        logits = dec.forward(np.array([tok], np.int32))
        tok = int(np.argmax(logits))
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = world * e2e_steps / e2e_s

    tern_b, kv_b, head_b = algorithmic_bytes(shape, ctx_mid)
    step_linears = linears_roofline(ctx, torch, dec, shape)
    c0 = gemv_roofline(ctx, torch, weights, shape)
    launches_per_token = dec.launches_per_token()
    line = {
        "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * dev_s / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x ternary -> int32, fp64 rescale", "data": "synthetic", "config": config,
        "timed_region": {"repetitions": reps, "seconds_each_median": dev_s, "seconds_total": total_s,
                         "note": "every repetition is exactly `steps` decode steps from context_first_timed_step"},
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": shape["vocab"] * 4,
                "steps": e2e_steps},
        "gpu_launches": int(args.steps * launches_per_token),
        "launches_per_token": launches_per_token,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": step_linears["gbs"], "peak": peak, "unit": "GB/s",
                     "frac": step_linears["gbs"] / peak, "traffic": step_linears["traffic"],
                     "traffic_source": "ncu dram__bytes_read+write of the ternary projections of one decoder block inside the "
                                       "decode step, scaled by the number of blocks (writes 0: outputs stay in L2)",
                     "peak_kind": peak_kind,
                     "kernel": "the ternary projections of one decode step as the step runs them (QKV, O, gate+up, down of every "
                               "block with their fused normalise/quantize prologues and epilogues; no attention, no head), "
                               "replayed as one recorded frame",
                     "bytes_per_frame": step_linears["bytes"], "us_per_frame": step_linears["us"],
                     "c0_gemv": {"achieved": c0["gbs"], "frac": c0["gbs"] / peak, "bytes_per_launch": c0["bytes"],
                                 "us_per_launch": c0["us"], "launches_timed": c0["launches"],
                                 "kernel": "configs[0]: int8 row in, gate 6912x2560 and down 2560x6912, batch 1, 60 distinct "
                                           "matrices per replay, independent launches"}},
        "decode_bytes": {"ternary": tern_b, "kv": kv_b, "fp32_head": head_b,
                         "gbs_all": (tern_b + kv_b + head_b) / (dev_s / args.steps) / 1e9,
                         "frac_of_peak": (tern_b + kv_b + head_b) / (dev_s / args.steps) / 1e9 / peak},
        "prefill": {"tokens": args.prompt, "seconds": prefill_s, "tok_per_s": args.prompt / prefill_s},
    }
    if tp_check is not None:
        line["tp_check"] = tp_check
    if world > 1 and world in (2, 4, 8) and not args.no_tp_section:
        # Strong scaling beside the replica headline: the 8B shape (8 KV heads divide by 2, 4 and 8), batch-1 decode over a
        # tensor-parallel group of all ranks with the peer-mailbox exchange.  The replica decoder is released first.
        dec.close()
        del dec, weights, emb
        ctx.close()
        torch.cuda.empty_cache()
        try:
            r = tp_decode_measure(args, torch, dist, rank, world, local, "8b", 0, min(args.steps, 32), args.warmup, "peer")
            line["tp"] = {k: r[k] for k in ("shape", "layers", "world", "exchange", "tok_per_s", "ms_per_step", "e2e_tok_per_s",
                                            "launches_per_token", "prompt")}
            line["tp"]["note"] = ("strong scaling: compare tok_per_s across the N of a scaling run; the one-GPU figure of the same shape "
                                  "comes from `bench.py --mode tp --shape 8b`")
        except Exception as exc:
            line["tp"] = {"error": "%s: %r" % (type(exc).__name__, exc)}
        # configs[3] over the same ranks: 16 independent sequences on the 8B shape (512-token prompts keep the line quick;
        # `bench.py --mode batch --prompt 2048` is the full configuration)
        try:
            rb = batch_measure(args, torch, dist, rank, world, local, "8b", 16, 512, 8, args.warmup)
            line["tp_batch"] = {k: rb[k] for k in ("shape", "layers", "world", "batch", "prompt", "steps", "tok_per_s", "ms_per_step",
                                                   "per_sequence_tok_per_s", "prefill_tok_per_s")}
        except Exception as exc:
            line["tp_batch"] = {"error": "%s: %r" % (type(exc).__name__, exc)}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            from oracle import oracle as orc
            threads = orc.host_threads()
            sample_blocks = 4
            tokps, timed = cpu_decode_rate(shape, min(sample_blocks, shape["layers"]), ctx_first, 4, threads, args.seed)
            line["cpu_baseline"] = {"value": tokps, "unit": "tok/s", "cores": threads, "kind": "port",
                                    "sample": "%d of %d blocks at full width (C++ restatement of the Go CPU path, AVX2 byte-code "
                                              "kernel, %d threads) at context %d + the full fp32 head, %d tokens; block time x%g, "
                                              "head x1.  `--impl reference` runs all blocks" %
                                              (min(sample_blocks, shape["layers"]), shape["layers"], threads, ctx_first, timed,
                                               shape["layers"] / min(sample_blocks, shape["layers"]))}
        except Exception as exc:  # the baseline is reported, never required for the GPU number
            line["cpu_baseline"] = {"value": None, "unit": "tok/s", "cores": 0, "kind": "port", "sample": "failed: %r" % (exc,)}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
