#!/usr/bin/env python
"""Benchmark of the quantized GEMV hot path (BASELINE.json configs[1]: the standalone GEMV sweep).

A step = one pass over the sweep at batch 1: for every K x N shape (2048x2048, 2048x8192, 8192x2048,
2048x49152) and every format (b4, b5, b6, nf4g128): rotate+quantize an fp32 activation vector
(FWHT-64 + int8) and run the GEMV.  One pass streams ~343 MB of distinct weights, more than the
126 MB L2, so every launch reads its weights from HBM.

  value     GB/s of algorithmic bytes (reference file-format weight bytes + activations + outputs)
            with inputs resident in HBM; whole-job aggregate over all ranks (each rank runs its own
            independent sweep: weak scaling, no collective on the data path).
  e2e       same metric through the host-buffer C-ABI calls (pinned host vectors; H2D + kernels + D2H inside the timed
            region): the sixteen independent projections of a pass queued with kronos_cuda_linear_async and waited for
            once; `sync_per_call` is the same pass with the blocking kronos_cuda_linear.
  roofline  GEMV kernels of the sweep timed one by one with CUDA events (aggregate and per case).
  cpu_baseline  the CPU oracle (a C++ port of the reference CPU path) on one pass, all host threads.

`--impl reference` times that CPU port alone (the reference is a Rust crate and cannot be built
here; its GPU path is Apple Metal and unavailable on this box).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(2048, 2048), (2048, 8192), (8192, 2048), (2048, 49152)]   # (K = cols, N = rows)
FORMATS = ["b4", "b5", "b6", "nf4g128"]
WORKLOAD = "gemv_sweep_batch1: K x N in 2048x2048, 2048x8192, 8192x2048, 2048x49152; b4, b5, b6, nf4g128"
SWEEP_CONFIG = {"workload": WORKLOAD, "l2_policy": "inputs larger than L2 (343 MB of distinct weights per step)"}      # the same dict in both arms


GEMV_SOURCES = ("k2t_gemv_core.cuh", "k2t_gemv.cu", "k2t_device.cuh", "k2t_layout.h")


def gemv_source_hash():
    """sha256 over the sources of the GEMV kernel: a profile summary names the hash it was captured with."""
    import hashlib
    h = hashlib.sha256()
    for name in GEMV_SOURCES:
        with open(os.path.join(ROOT, "kronos-2t_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def ncu_traffic(fmt):
    """dram__bytes_read.sum + dram__bytes_write.sum of one 2048x49152 launch, read from the ncu summary under profiles/ - only
    when that summary was captured from the kernel sources as they are now (its `kernel-source-hash:` line); otherwise
    (None, why)."""
    import re
    path = os.path.join(ROOT, "profiles", f"gemv_{fmt}_2048x49152.md")
    if not os.path.exists(path):
        return None, "no ncu summary under profiles/ for this format"
    text = open(path).read()
    m_hash = re.search(r"kernel-source-hash:\s*([0-9a-f]+)", text)
    m_bytes = re.search(r"dram-bytes-per-launch:\s*([0-9]+)", text)
    if not m_hash or not m_bytes:
        return None, "the ncu summary carries no kernel-source-hash / dram-bytes-per-launch lines"
    if m_hash.group(1) != gemv_source_hash():
        return None, "the GEMV sources changed since the ncu capture (hash %s, now %s)" % (m_hash.group(1), gemv_source_hash())
    return int(m_bytes.group(1)), os.path.relpath(path, ROOT)


def fmt_spec(fmt):
    if fmt.startswith("b"):
        return ("bipolar", int(fmt[1]), 1)
    return ("nf", int(fmt[2]), 2 if fmt.endswith("g128") else 1)


def algorithmic_bytes(fmt, cols, rows, n_tok=1):
    """weights in the reference file format + int8 activations with scale and sum + fp32 outputs."""
    from kronos_2t_b200 import synth
    kind, bits, sgc = fmt_spec(fmt)
    return synth.file_bytes(kind, rows, cols, bits, sgc) + n_tok * (cols + 8 * (cols // 64)) + n_tok * 4 * rows


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only queries) every ~2 ms while the
    timed region runs."""

    def __init__(self, index):
        self.index, self.sm, self.reasons, self.max_mhz, self.err = index, [], set(), None, None
        self._stop = threading.Event()
        self.thread = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.index
            if vis:
                try:
                    idx = int(vis.split(",")[self.index])
                except ValueError:
                    idx = self.index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.nv = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # noqa: BLE001
            self.err = f"nvml unavailable: {e}"
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _sample(self):
        nv = self.nv
        self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
        try:
            r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
        except Exception:  # noqa: BLE001
            r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        for name, bit in (("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40),
                          ("sw_power_cap", 0x4), ("hw_power_brake_slowdown", 0x80)):
            if r & bit:
                self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                self._sample()
            except Exception as e:  # noqa: BLE001
                self.err = str(e)
                return
            time.sleep(0.002)

    def stop(self):
        if self.thread:
            self._stop.set()
            self.thread.join(timeout=2)
            if not self.sm:
                try:
                    self._sample()
                except Exception:  # noqa: BLE001
                    pass
        out = {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
               "samples": len(self.sm), "reasons": sorted(self.reasons)}
        if self.err:
            out["note"] = self.err
        return out


def build_sweep_host(seed0):
    """File-format bytes of the 16 sweep matrices (random codes; see kronos_2t_b200.synth)."""
    from kronos_2t_b200 import synth
    mats = []
    for si, (cols, rows) in enumerate(SHAPES):
        for fi, fmt in enumerate(FORMATS):
            kind, bits, sgc = fmt_spec(fmt)
            seed = seed0 + 16 * si + fi
            if kind == "bipolar":
                d0, d1 = synth.random_bipolar_bytes(seed, rows, cols, bits)
            else:
                d0, d1 = synth.random_nf_bytes(seed, rows, cols, bits, sgc)
            mats.append(dict(fmt=fmt, kind=kind, bits=bits, sgc=sgc, rows=rows, cols=cols, d0=d0, d1=d1))
    return mats


def run_reference(args, rank, world):
    """CPU arm: the oracle's stripe-parallel GEMV (C++ port of the reference CPU path), all host threads."""
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np
    import oracle as o
    threads = os.cpu_count() or 1
    mats = build_sweep_host(1000)
    rng = np.random.Generator(np.random.PCG64(7))
    cases = []
    for m in mats:
        x = rng.standard_normal(m["cols"]).astype(np.float32)
        if m["kind"] == "bipolar":
            om = o.nibble4_from_bipolar(o.Bipolar(m["rows"], m["cols"], m["bits"], m["d0"], m["d1"]))
        else:
            om = o.Nf(m["rows"], m["cols"], m["bits"], m["sgc"], _default_cb(m["bits"]), m["d0"], m["d1"])
        cases.append((m, om, x))
    total_bytes = sum(algorithmic_bytes(m["fmt"], m["cols"], m["rows"]) for m in mats)

    def one_pass():
        for m, om, x in cases:
            act = o.act_populate_fwht(x)
            if m["kind"] == "bipolar":
                o.nibble4_gemv(om, act, threads=threads)
            else:
                o.nf_gemv(om, act, threads=threads)

    for _ in range(args.warmup):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one_pass()
    dt = time.perf_counter() - t0
    val = total_bytes * args.steps / dt / 1e9
    sample = f"{args.steps} full passes of the 16-matrix sweep (stripe-parallel, {threads} threads)"
    print(json.dumps({
        "impl": "reference", "metric": "quantized_gemv_hbm_gbs", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x 4..6-bit codes -> int32, fp32 epilogue", "data": "synthetic (random codes)",
        "config": SWEEP_CONFIG,
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def _default_cb(bits):
    from kronos_2t_b200 import synth
    return synth.NF4_DEFAULT if bits == 4 else synth.NF3_DEFAULT


def run_b200(args, rank, world, local_rank):
    import numpy as np
    import torch
    import kronos_2t_b200 as k2

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"            # the version banner goes to stdout, which carries the one JSON line
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    ctx = k2.Context(local_rank)
    stream = torch.cuda.Stream(device=dev)      # a real (non-default) stream: events and kernels share it
    torch.cuda.set_stream(stream)
    assert stream.cuda_stream != 0
    ctx.set_stream(stream.cuda_stream)

    mats = build_sweep_host(1000 + 100 * rank)
    cases = []
    g = torch.Generator(device="cpu").manual_seed(7 + rank)
    for m in mats:
        if m["kind"] == "bipolar":
            dm = ctx.upload_bipolar(m["rows"], m["cols"], m["bits"], m["d0"], m["d1"])
        else:
            dm = ctx.upload_nf(m["rows"], m["cols"], m["bits"], m["sgc"], _default_cb(m["bits"]), m["d0"], m["d1"])
        cols, rows, nc = m["cols"], m["rows"], m["cols"] // 64
        x_host = torch.randn(cols, generator=g, dtype=torch.float32).pin_memory()
        case = dict(m=m, dm=dm, x_host=x_host, out_host=torch.empty(rows, dtype=torch.float32).pin_memory(),
                    x=x_host.to(dev), q=torch.empty(cols, dtype=torch.int8, device=dev),
                    s=torch.empty(nc, dtype=torch.float32, device=dev), sums=torch.empty(nc, dtype=torch.int32, device=dev),
                    out=torch.empty(rows, dtype=torch.float32, device=dev),
                    bytes=algorithmic_bytes(m["fmt"], cols, rows))
        cases.append(case)
    bytes_per_step = sum(c["bytes"] for c in cases)

    for c in cases:
        c["p"] = (c["x"].data_ptr(), c["q"].data_ptr(), c["s"].data_ptr(), c["sums"].data_ptr(), c["out"].data_ptr())

    def step_launches():
        for c in cases:
            px, pq, ps, pm, po = c["p"]
            ctx.fwht_quant_dev(px, 1, c["m"]["cols"], pq, ps, pm)
            ctx.gemv_dev(c["dm"], pq, ps, pm, 1, po)

    def step_e2e():
        # host buffers in, host buffers out: the sixteen projections of a pass are independent, so they are queued with
        # kronos_cuda_linear_async (copy in, rotate + quantize, GEMV, copy out, each) and waited for once
        for c in cases:
            ctx.linear_async_ptr(c["dm"], c["x_host"].data_ptr(), 1, c["out_host"].data_ptr())
        ctx.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    # one step = one CUDA graph (32 kernel nodes): decode loops are launch-bound otherwise
    step_launches()
    torch.cuda.synchronize()
    l0 = ctx.launch_count
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        step_launches()
    launches_per_step = ctx.launch_count - l0
    ctx.set_stream(stream.cuda_stream)

    def step():
        graph.replay()

    def timed(fn, steps, sample_clocks=False):
        sampler = ClockSampler(local_rank) if sample_clocks else None
        barrier()
        if sampler:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop() if sampler else None
        if dist:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, clocks

    for _ in range(max(args.warmup, 3)):
        step()
    ms, clocks = timed(step, args.steps, sample_clocks=True)
    gpu_launches = launches_per_step * args.steps
    value = bytes_per_step * world * args.steps / (ms / 1e3) / 1e9

    def step_e2e_sync():
        for c in cases:
            ctx.linear_ptr(c["dm"], c["x_host"].data_ptr(), 1, c["out_host"].data_ptr())

    for _ in range(3):
        step_e2e()
        step_e2e_sync()
    e2e_steps = min(args.steps, 50)
    ms_e2e, _ = timed(step_e2e, e2e_steps)
    e2e_value = bytes_per_step * world * e2e_steps / (ms_e2e / 1e3) / 1e9
    ms_e2e_sync, _ = timed(step_e2e_sync, e2e_steps)
    e2e_sync_value = bytes_per_step * world * e2e_steps / (ms_e2e_sync / 1e3) / 1e9
    h2d = sum(c["m"]["cols"] * 4 for c in cases)
    d2h = sum(c["m"]["rows"] * 4 for c in cases)

    # roofline: the GEMV kernel of every case timed alone, replayed from a graph over enough distinct
    # HBM copies of the matrix (>= 256 MB) that no launch finds its weights in L2
    peak, peak_kind = peaks()
    kernels = []
    tot_b = tot_us = tot_us_iso = 0.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for c in cases:
        wbytes = c["dm"].file_bytes
        copies = max(3, -(-(256 << 20) // wbytes))
        clones = [c["dm"]] + [c["dm"].clone() for _ in range(copies - 1)]
        px, pq, ps, pm, po = c["p"]
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for r in range(2):
                for m in clones:
                    ctx.gemv_dev(m, pq, ps, pm, 1, po)
        ctx.set_stream(stream.cuda_stream)
        g.replay()
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(3):
            g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (3 * 2 * copies)
        gbs = c["bytes"] / us / 1e3
        # the same launches each behind the rotation kernel of its activation (the position a GEMV has in a decode step:
        # its weight prefetch overlaps a tiny kernel, not the tail of another large GEMV), minus the rotation kernels alone
        def graph_us(with_gemv):
            gg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gg, stream=stream):
                for r in range(2):
                    for m in clones:
                        ctx.fwht_quant_dev(px, 1, c["m"]["cols"], pq, ps, pm)
                        if with_gemv:
                            ctx.gemv_dev(m, pq, ps, pm, 1, po)
            ctx.set_stream(stream.cuda_stream)
            gg.replay()
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(3):
                gg.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e3 / (3 * 2 * copies)
        us_iso = max(graph_us(True) - graph_us(False), 1e-3)
        kernels.append({"case": f"{c['m']['fmt']} {c['m']['cols']}x{c['m']['rows']}", "us": round(us, 2),
                        "GBps": round(gbs, 1), "frac": round(gbs / peak, 3),
                        "us_isolated": round(us_iso, 2), "frac_isolated": round(c["bytes"] / us_iso / 1e3 / peak, 3)})
        tot_b += c["bytes"]; tot_us += us; tot_us_iso += us_iso
        del g
        for m in clones[1:]:
            m.free()
    big = [k for k in kernels if k["case"].endswith("x49152")]
    big_b = sum(c["bytes"] for c in cases if c["m"]["rows"] == 49152)
    big_us = sum(k["us"] for k in big)
    big_us_iso = sum(k["us_isolated"] for k in big)
    # the wide-batch kernel on the same four large matrices: 64 tokens in one launch (tensor cores for the integer dots)
    gemm_tc = []
    for c in cases:
        if c["m"]["rows"] != 49152:
            continue
        cols, rows, nt = c["m"]["cols"], c["m"]["rows"], 64
        x64 = torch.randn(nt, cols, device=dev)
        q64 = torch.empty(nt, cols, dtype=torch.int8, device=dev)
        s64 = torch.empty(nt, cols // 64, dtype=torch.float32, device=dev)
        m64 = torch.empty(nt, cols // 64, dtype=torch.int32, device=dev)
        o64 = torch.empty(nt, rows, dtype=torch.float32, device=dev)
        ctx.fwht_quant_dev(x64.data_ptr(), nt, cols, q64.data_ptr(), s64.data_ptr(), m64.data_ptr())
        for _ in range(2):
            ctx.gemv_dev(c["dm"], q64.data_ptr(), s64.data_ptr(), m64.data_ptr(), nt, o64.data_ptr())
        torch.cuda.synchronize()
        l0 = ctx.launch_count
        e0.record(stream)
        for _ in range(5):
            ctx.gemv_dev(c["dm"], q64.data_ptr(), s64.data_ptr(), m64.data_ptr(), nt, o64.data_ptr())
        e1.record(stream)
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / 5
        tops = 2.0 * rows * cols * nt / us / 1e6
        gemm_tc.append({"case": f"{c['m']['fmt']} {cols}x{rows} x {nt} tokens", "launches_per_call": (ctx.launch_count - l0) // 5, "us": round(us, 1),
                        "int8_TOPs": round(tops, 1), "frac_of_nominal_int8": round(tops / 4500.0, 4),
                        "tok_s_equivalent": round(nt / us * 1e6)})
    achieved = big_b / big_us / 1e3
    traffic, traffic_src = ncu_traffic("b4")
    traffic_per_format = {f: ncu_traffic(f)[0] for f in ("b4", "nf4g128")}
    roofline = {"bound": "hbm", "kernel": "gemv_kernel, the four 2048x49152 launches of a sweep pass (78% of its bytes)",
                "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                "launch_form": "each case timed alone: a CUDA graph of back-to-back launches over distinct HBM copies of the matrix, "
                               "programmatic dependents of one another as in the decode engine (a launch streams its first weight stages "
                               "while the previous one drains); CUDA events around three replays",
                "isolated": {"achieved": big_b / big_us_iso / 1e3, "frac": big_b / big_us_iso / 1e3 / peak,
                             "form": "the same four launches, each behind the rotation kernel of its activation instead of another large GEMV "
                                     "(what a decode step gives it), rotation time subtracted"},
                "traffic": traffic, "traffic_unit": "bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum, b4 2048x49152)",
                "traffic_source": traffic_src, "traffic_per_format": traffic_per_format,
                "all_16_launches": {"achieved": tot_b / tot_us / 1e3, "frac": tot_b / tot_us / 1e3 / peak,
                                    "achieved_isolated": tot_b / tot_us_iso / 1e3, "frac_isolated": tot_b / tot_us_iso / 1e3 / peak},
                "per_launch": kernels,
                "gemm_tc": gemm_tc,
                "gemm_tc_note": "gemm_tc_kernel (k2t_gemm_tc.cu): bound by the fp32 chains and role hand-offs on the CUDA cores, not by the tensor pipe "
                                "(4% active, profiles/gemm_tc_nf4g128_2048x16384_t64.md); int8 dense nominal 4500 TOP/s, no measured int8 peak on this pool"}

    decode = None
    if not args.no_decode:
        decode = decode_tok_s(ctx, stream, timed_region=lambda fn: timed(fn, 1)[0], world=world)

        roofline["decode"] = [_decode_entry("SmolLM2-135M b4", 192, "int8", "reference order", decode["tok_s"] / world, decode["weight_bytes_per_token"],
                                            decode["kv_bytes_at_256"] // 256, peak)]
        if not args.no_decode_models:
            try:
                decode["models"], roof, attn, pre = decode_models(ctx, lambda fn: timed(fn, 1)[0], rank, world, dist)
                roofline["decode"] += roof
                roofline["attention"] = attn
                roofline["prefill"] = pre
            except Exception as exc:      # the headline line must still come out; the failure is reported in it
                decode["models_error"] = f"{type(exc).__name__}: {exc}"
        if not args.no_decode_moe:
            try:
                decode["moe"], roof = decode_moe(ctx, lambda fn: timed(fn, 1)[0], rank, world, dist)
                roofline["decode"] += roof
                from kronos_2t_b200 import synth as _synth
                roofline.setdefault("prefill", []).append(_prefill_entry(
                    "Qwen3-30B-A3B nf3 experts / nf4g128 attention" + ("" if world == 1 else f" ep{world}"), 480, decode["moe"]["prefill_tok_s_480"],
                    _matmul_ops_per_token(_synth.QWEN3_30B_A3B, dict(top_k=8, d_ff=768)), n_gpus=world))
            except Exception as exc:
                decode["moe_error"] = f"{type(exc).__name__}: {exc}"
        if world > 1:
            try:
                roofline["sharded_parity"] = sharded_parity(ctx, rank, world, dist)
            except Exception as exc:
                roofline["sharded_parity"] = {"error": f"{type(exc).__name__}: {exc}"}
        roofline["prefill_note"] = ("prompt batches of 256 tokens: every dense projection is one launch of the tensor-core kernel (tcgen05.mma kind::i8 for the "
                                    "exact chunk dots, fp32 chains on the CUDA cores in the reference's order), attention of the batch side by side; "
                                    "int8_TOPs = 2 x multiply-adds of the projections x tok/s; the MoE experts still run as expert-batched GEMVs")
        roofline["decode_note"] = ("frac = bytes_per_token * tok_s / (n_gpus * peak): weights of one step in the reference's file format + the cached "
                                   "rows the token attends to; n_gpus > 1: the Qwen2-7B shape tensor-parallel (tp) and the Qwen3-30B-A3B shape "
                                   "expert-parallel (ep) over all ranks - strong scaling of ONE token stream")

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline(mats)
        if decode is not None:
            decode["cpu_baseline"] = cpu_decode_baseline()

    if rank == 0:
        print(json.dumps({
            "metric": "quantized_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "step_form": "one CUDA graph of 32 kernels per step", "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x 4..6-bit codes -> int32, fp32 epilogue", "data": "synthetic (random codes)",
            "config": SWEEP_CONFIG, "per_rank": "each rank runs its own sweep (replicas, no collective)",
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "GB/s", "ms_per_step": ms_e2e / e2e_steps, "steps": e2e_steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "form": "16 x kronos_cuda_linear_async + 1 x kronos_cuda_synchronize per step",
                    "sync_per_call": {"value": e2e_sync_value, "unit": "GB/s", "ms_per_step": ms_e2e_sync / e2e_steps,
                                      "form": "16 x kronos_cuda_linear (each call waits for its result)"}},
            "gpu_launches": int(gpu_launches),
            "roofline": roofline, "cpu_baseline": cpu, "decode": decode,
        }))
    for c in cases:
        c["dm"].free()
    ctx.close()
    if dist:
        dist.destroy_process_group()


def run_case(args, local_rank):
    """Single-case loop for profiling: `--case b4:2048x49152 [--tokens 4]` rotates over enough copies of
    one matrix to exceed L2 (>= 256 MB of distinct weights) and times the GEMV launches with CUDA events."""
    import torch
    import kronos_2t_b200 as k2
    from kronos_2t_b200 import synth

    fmt, shape = args.case.split(":")
    cols, rows = (int(v) for v in shape.split("x"))
    kind, bits, sgc = fmt_spec(fmt)
    n_tok = args.tokens
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ctx = k2.Context(local_rank)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    ctx.set_stream(stream.cuda_stream)
    wbytes = synth.file_bytes(kind, rows, cols, bits, sgc)
    copies = max(3, -(-(256 << 20) // wbytes))
    if kind == "bipolar":
        d0, d1 = synth.random_bipolar_bytes(0, rows, cols, bits)
        mats = [ctx.upload_bipolar(rows, cols, bits, d0, d1)]
    else:
        d0, d1 = synth.random_nf_bytes(0, rows, cols, bits, sgc)
        mats = [ctx.upload_nf(rows, cols, bits, sgc, _default_cb(bits), d0, d1)]
    mats += [mats[0].clone() for _ in range(copies - 1)]   # distinct HBM copies: no launch finds its weights in L2
    nc = cols // 64
    x = torch.randn(n_tok, cols, device=dev)
    q = torch.empty(n_tok, cols, dtype=torch.int8, device=dev)
    sc = torch.empty(n_tok, nc, dtype=torch.float32, device=dev)
    sums = torch.empty(n_tok, nc, dtype=torch.int32, device=dev)
    out = torch.empty(n_tok, rows, dtype=torch.float32, device=dev)
    ctx.fwht_quant_dev(x.data_ptr(), n_tok, cols, q.data_ptr(), sc.data_ptr(), sums.data_ptr())

    ptrs = (q.data_ptr(), sc.data_ptr(), sums.data_ptr(), out.data_ptr())

    def launch(i):
        ctx.gemv_dev(mats[i % copies], ptrs[0], ptrs[1], ptrs[2], n_tok, ptrs[3])

    for i in range(args.warmup):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(args.steps):
        launch(args.warmup + i)
    e1.record(stream)
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    # the same launches replayed from a CUDA graph: no host launch cost between kernels
    us_graph = None
    if not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(copies * 4):
                launch(i)
        ctx.set_stream(stream.cuda_stream)
        graph.replay()
        torch.cuda.synchronize()
        reps = max(1, args.steps // 4)
        e0.record(stream)
        for _ in range(reps):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        us_graph = e0.elapsed_time(e1) * 1e3 / (reps * copies * 4)
    ctx.synchronize()
    b = algorithmic_bytes(fmt, cols, rows, n_tok)
    peak, kind_p = peaks()
    best = us_graph if us_graph is not None else us
    print(json.dumps({"case": args.case, "tokens": n_tok, "copies": copies, "us_per_launch_stream": round(us, 2),
                      "us_per_launch_graph": None if us_graph is None else round(us_graph, 2),
                      "algorithmic_bytes": b, "GBps": round(b / best / 1e3, 1), "frac_of_" + kind_p: round(b / best / 1e3 / peak, 3)}))
    for m in mats:
        m.free()
    ctx.close()


DECODE_WORKLOAD = ("SmolLM2-135M-shaped Llama (hidden 576, 30 layers, 9q/3kv heads of 64, MLP 1536, vocab 49152, tied), b4 "
                   "bit-planes with random codes, int8 Hadamard KV, 128-token prompt then 128 greedy steps, batch 1")


def decode_tok_s(ctx, stream, timed_region, world):
    """Whole-token decode through kronos_cuda_engine_*: prompt token by token, then the device-side greedy loop."""
    import numpy as np
    import kronos_2t_b200 as k2
    from kronos_2t_b200 import synth
    spec = synth.random_model(synth.SMOLLM2_135M, "b4", seed=3)
    eng = k2.Engine(ctx, spec)
    prompt = np.random.Generator(np.random.PCG64(11)).integers(0, spec["cfg"]["vocab"], 128).astype(np.uint32)
    l0 = ctx.launch_count
    eng.forward_token_ids(prompt[:-1])
    eng.decode_greedy(int(prompt[-1]), 127, 128)                      # warm-up (graph capture, caches)
    l1 = ctx.launch_count
    ms_prompt = timed_region(lambda: eng.forward_token_ids(prompt[:-1]))
    ms_decode = min(timed_region(lambda: eng.decode_greedy(int(prompt[-1]), 127, 128)) for _ in range(3))
    out = {"workload": DECODE_WORKLOAD, "tok_s": 128 * world / (ms_decode / 1e3), "ms_per_token": ms_decode / 128,
           "prompt_tok_s": 127 * world / (ms_prompt / 1e3), "weight_bytes_per_token": eng.weight_bytes,
           "weight_gbs": eng.weight_bytes * 128 * world / (ms_decode / 1e3) / 1e9, "kv_bytes_at_256": eng.kv_bytes(256),
           "form": "one CUDA graph replay per token (8 kernels per layer + 3), argmax on the device",
           "note": "each rank decodes its own replica; tok_s is the aggregate"}
    eng.close()
    return out


def _prefill(eng, rng, vocab, lo, hi, timed_region=None):
    """Prompt positions [lo, hi) of random token ids (batches of 256 tokens: every projection one tensor-core launch); returns
    tok/s when timed - the second of two identical passes, so that no kernel is loaded inside the timed region."""
    toks = rng.integers(0, vocab, hi - lo).astype("uint32")
    eng.forward_token_ids(toks, pos_start=lo)
    if timed_region is None:
        return None
    ms = timed_region(lambda: eng.forward_token_ids(toks, pos_start=lo))
    return (hi - lo) / (ms / 1e3)


def _matmul_ops_per_token(cfg, moe=None):
    """Integer multiply-adds x 2 of one token's projections (lm_head left out: a prompt computes it for its last token only)."""
    h, hd = cfg["hidden"], cfg["head_dim"]
    attn = (cfg["n_q"] + 2 * cfg["n_kv"]) * hd * h + h * cfg["n_q"] * hd
    ffn = 3 * cfg["inter"] * h if moe is None else moe["top_k"] * 3 * moe["d_ff"] * h
    return 2 * cfg["layers"] * (attn + ffn)


def _prefill_entry(name, tokens, tok_s, ops_per_token, n_gpus=1):
    tops = ops_per_token * tok_s / 1e12
    return {"model": name, "tokens": tokens, "tok_s": round(tok_s, 1), "int8_TOPs": round(tops, 2), "n_gpus": n_gpus,
            "frac_of_nominal_int8": round(tops / (4500.0 * n_gpus), 4)}


def _attention_us(eng, pos, reps=4):
    """us per layer of the attention launches of one greedy step at `pos` (kronos_cuda_engine_profile_step: every kernel alone
    between two events, which adds a few us to each): (attention kernels, qkv_post kernel)."""
    rows = {}
    for line in eng.profile_step(1, pos, reps).splitlines()[1:]:
        f = [x.strip() for x in line.split("|")]
        if len(f) >= 4 and f[3]:
            rows[f[0]] = float(f[3])
    return rows.get("attention"), rows.get("qkv_post")


def _decode_entry(name, ctx_len, kv, mode, tok_s, weight_bytes, kv_bytes_per_pos, peak, n_gpus=1, parallel=None):
    """One roofline.decode record: bytes a token must stream (weights of one step + the cached rows it attends to)."""
    per_token = weight_bytes + kv_bytes_per_pos * ctx_len
    gbs = per_token * tok_s / 1e9
    return {"model": name, "ctx": ctx_len, "kv": kv, "attention": mode, "n_gpus": n_gpus, "parallel": parallel, "tok_s": round(tok_s, 1),
            "bytes_per_token": per_token, "GBps": round(gbs, 1), "frac": round(gbs / (peak * n_gpus), 4)}


def decode_models(ctx, timed_region, rank, world, dist):
    """Whole-token decode of the larger model shapes (random codes; time does not depend on the values).

    One GPU: the SmolLM2-1.7B shape in nf4g128 at contexts 512 and 8192 with the int8 and the NF4 KV cache, and the
    Qwen2-7B shape in the p55454 plane tier at context 4096.  Contexts beyond 512 positions run twice: in the reference's
    summation order (the default: identical results) and with the split-KV kernels (KRONOS_CUDA_ENGINE_SPLIT_KV_ATTENTION).
    2, 4 or 8 GPUs: the Qwen2-7B shape tensor-parallel over all ranks (8 ranks: two per kv head, query heads 4 + 3); the sum
    and gather steps run inside the engine over peer memory."""
    import numpy as np
    import kronos_2t_b200 as k2
    from kronos_2t_b200 import synth
    rng = np.random.Generator(np.random.PCG64(23))
    peak, _ = peaks()
    out, roof, attn, pre = [], [], [], []
    steps = 64
    name17 = "SmolLM2-1.7B-shaped (hidden 2048, 24 layers, 32q/32kv heads of 64, MLP 8192, vocab 49152), nf4g128"
    if world == 1:
        for kv_bits in (8, 4):
            kv = "int8" if kv_bits == 8 else "nf4"
            cfg = dict(synth.SMOLLM2_1_7B, kv_bits=kv_bits)
            eng = k2.Engine(ctx, synth.random_model(cfg, "nf4g128", seed=5, share_layers=True))
            prefill = _prefill(eng, rng, cfg["vocab"], 0, 1024, timed_region)
            pre.append(_prefill_entry(f"SmolLM2-1.7B nf4g128, {kv} KV", 1024, prefill, _matmul_ops_per_token(cfg)))
            res = {"model": name17, "kv": kv, "prefill_tok_s_1024": prefill, "weight_bytes_per_token": eng.weight_bytes,
                   "kv_bytes_per_pos": eng.kv_bytes_per_pos}
            for key, pos in (("ctx_512", 512 - steps), ("ctx_8192", 8192)):
                if pos > 1024:
                    _prefill(eng, rng, cfg["vocab"], 1024, pos)
                eng.decode_greedy(1, pos, 8)                                          # warm-up (graph capture)
                ms = min(timed_region(lambda: eng.decode_greedy(1, pos, steps)) for _ in range(2))
                res[key] = {"tok_s": steps / (ms / 1e3), "ms_per_token": ms / steps, "positions": [pos, pos + steps],
                            "weight_gbs": eng.weight_bytes * steps / (ms / 1e3) / 1e9, "attention": "reference order"}
                roof.append(_decode_entry("SmolLM2-1.7B nf4g128", pos + steps // 2, kv, "reference order", steps / (ms / 1e3), eng.weight_bytes,
                                          eng.kv_bytes_per_pos, peak))
            if kv_bits == 8:
                a_us, q_us = _attention_us(eng, 8192)
                kv_layer = 32 * 8192 * (2 * 64 + 8)
                attn.append({"kernel": "attn_scores_kernel<64> + attn_values_kernel<64> (reference order)", "model": "SmolLM2-1.7B", "ctx": 8192,
                             "kv_bytes_per_layer": kv_layer, "us_per_layer": a_us, "qkv_post_us": q_us, "GBps": round(kv_layer / a_us / 1e3, 1),
                             "frac": round(kv_layer / a_us / 1e3 / peak, 3)})
            eng.close()
            if kv_bits == 8:          # the same context with the split-KV kernels
                eng = k2.Engine(ctx, synth.random_model(dict(cfg, split_kv_attention=True), "nf4g128", seed=5, share_layers=True))
                eng.decode_greedy(1, 8192, 8)
                ms = min(timed_region(lambda: eng.decode_greedy(1, 8192, steps)) for _ in range(2))
                res["ctx_8192_split_kv"] = {"tok_s": steps / (ms / 1e3), "ms_per_token": ms / steps, "positions": [8192, 8192 + steps],
                                            "attention": "split-KV (fp32-rounding agreement)"}
                roof.append(_decode_entry("SmolLM2-1.7B nf4g128", 8192 + steps // 2, kv, "split-KV", steps / (ms / 1e3), eng.weight_bytes, eng.kv_bytes_per_pos, peak))
                a_us, q_us = _attention_us(eng, 8192)
                attn.append({"kernel": "attn_partial_kernel<64> + attn_finish_kernel<64> (split-KV)", "model": "SmolLM2-1.7B", "ctx": 8192,
                             "kv_bytes_per_layer": kv_layer, "us_per_layer": a_us, "qkv_post_us": q_us, "GBps": round(kv_layer / a_us / 1e3, 1),
                             "frac": round(kv_layer / a_us / 1e3 / peak, 3)})
                eng.close()
            out.append(res)
    tp = world if world in (1, 2, 4, 8) else 4
    group, tp_rank = rank // tp, rank % tp
    name7 = ("Qwen2-7B-shaped (hidden 3584, 28 layers, 28q/4kv heads of 128, MLP 18944, vocab 152064, qkv bias, untied), "
             "p55454 planes (qkv 5, o 5, gate_up 4, down 5, head 4)")
    res7 = {"model": name7, "kv": "int8", "tp": tp, "groups": world // tp,
            "exchange": None if tp == 1 else "2 partial-sum exchanges per layer + 1 logits gather per token, one kernel each over peer memory (no NCCL on the data path)",
            "head_split": None if tp <= 4 else "two ranks per kv head (own copy of its cache), query heads 4 + 3"}
    for split in ((False, True) if world == 1 else (False,)):
        cfg = dict(synth.QWEN2_7B, split_kv_attention=split)
        eng = k2.Engine(ctx, synth.random_model(cfg, "b4", seed=7, modes=synth.P55454, qkv_bias=True, untied=True, tp=(tp, tp_rank), share_layers=True))
        if tp > 1:
            handles = [None] * world
            dist.all_gather_object(handles, eng.tp_handle())
            eng.tp_attach(handles[group * tp:(group + 1) * tp])
            dist.barrier()
        if not split:
            res7["prefill_tok_s_1024"] = _prefill(eng, rng, cfg["vocab"], 0, 1024, timed_region) * (world // tp)
            pre.append(_prefill_entry("Qwen2-7B p55454" + ("" if tp == 1 else f" tp{tp}"), 1024, res7["prefill_tok_s_1024"], _matmul_ops_per_token(cfg), n_gpus=world))
        eng.decode_greedy(1, 4096, 8)
        ms = min(timed_region(lambda: eng.decode_greedy(1, 4096, steps)) for _ in range(2))
        groups = world // tp
        wb = eng.weight_bytes
        if dist:
            import torch
            t = torch.tensor([float(wb)], device="cuda", dtype=torch.float64)
            dist.all_reduce(t)
            wb = int(t.item()) // groups
        key = "ctx_4096_split_kv" if split else "ctx_4096"
        res7[key] = {"tok_s": groups * steps / (ms / 1e3), "ms_per_token": ms / steps, "positions": [4096, 4096 + steps],
                     "weight_gbs": groups * wb * steps / (ms / 1e3) / 1e9, "attention": "split-KV (fp32-rounding agreement)" if split else "reference order"}
        res7["weight_bytes_per_token"] = wb
        kv_pos = 2 * 28 * 4 * (128 + 4)
        roof.append(_decode_entry("Qwen2-7B p55454", 4096 + steps // 2, "int8", "split-KV" if split else "reference order", steps / (ms / 1e3), wb,
                                  kv_pos, peak, n_gpus=tp, parallel=None if tp == 1 else f"tp{tp}"))
        if world == 1:
            a_us, q_us = _attention_us(eng, 4096)
            kv_layer = 4 * 4096 * (2 * 128 + 8)
            attn.append({"kernel": ("attn_partial_kernel<128> + attn_finish_kernel<128> (split-KV)" if split else
                                    "attn_scores_kernel<128> + attn_values_kernel<128> (reference order)"), "model": "Qwen2-7B", "ctx": 4096,
                         "kv_bytes_per_layer": kv_layer, "us_per_layer": a_us, "qkv_post_us": q_us, "GBps": round(kv_layer / a_us / 1e3, 1),
                         "frac": round(kv_layer / a_us / 1e3 / peak, 3)})
        eng.close()
    out.append(res7)
    return out, roof, attn, pre


def sharded_parity(ctx, rank, world, dist):
    """The two-GPU parity tests of tests/test_gpu_tp.py inside an N-rank run (N = 2, 4, 8), outside every timed region:
    a small dense model tensor-parallel over all ranks and a small sparse-MoE model expert-parallel over all ranks, each
    compared - logits of a short prompt and a greedy stream - with the CPU emulation that sums the ranks' partial outputs
    in rank order (oracle.TpModel / oracle.EpModel, the checker; rank 0 only).  Returns {tp_parity_ok, ep_parity_ok}."""
    import numpy as np
    import torch
    import kronos_2t_b200 as k2
    from kronos_2t_b200 import synth
    tokens = [5, 17, 300, 42, 7, 199, 63, 250, 11]
    res = {}

    def run(eng):
        handles = [None] * world
        dist.all_gather_object(handles, eng.tp_handle())
        eng.tp_attach(handles)
        dist.barrier()
        logits = eng.forward_token_ids(tokens, want_all=True)
        greedy = eng.decode_greedy(int(np.argmax(logits[-1])), len(tokens), 12)
        dist.barrier()
        return logits, greedy

    def agree(mine):          # every rank holds the same bits
        t = torch.from_numpy(np.ascontiguousarray(mine).view(np.uint8).copy()).cuda()
        ref = t.clone()
        dist.broadcast(ref, 0)
        same = torch.tensor([int(torch.equal(t, ref))], device="cuda")
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        return bool(same.item())

    tp_cfg = dict(hidden=512, layers=2, n_q=8, n_kv=4, head_dim=64, inter=1024, vocab=2048, max_seq=64, eps=1e-5, theta=1e5)
    eng = k2.Engine(ctx, synth.random_model(tp_cfg, "b5", seed=41, qkv_bias=True, tp=(world, rank)))
    logits, greedy = run(eng)
    eng.close()
    ok = agree(logits) and agree(greedy)
    if rank == 0:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import oracle as o
        specs = [synth.random_model(tp_cfg, "b5", seed=41, qkv_bias=True, tp=(world, r)) for r in range(world)]
        table = np.asarray(specs[0]["embed_bf16"], np.uint16).reshape(-1, tp_cfg["hidden"])
        emu = o.TpModel(specs, lambda t: (table[t].astype(np.uint32) << 16).view(np.float32))
        want = np.stack([emu.forward_token(t) for t in tokens])
        nxt, stream = int(np.argmax(want[-1])), []
        for _ in range(12):
            nxt = o.argmax(emu.forward_token(nxt)); stream.append(nxt)
        emu.close()
        ok = ok and np.array_equal(logits, want) and list(greedy) == stream
    res["tp_parity_ok"] = bool(ok)
    ep_cfg = dict(hidden=256, layers=2, n_q=4, n_kv=2, head_dim=64, inter=256, vocab=512, max_seq=64, eps=1e-6, theta=1e6)
    moe = dict(n_experts=16, top_k=4, d_ff=128, bits=3, sgc=1)
    spec = synth.random_model(ep_cfg, "nf4g128", seed=43, untied=True, moe=moe, ep=(world, rank))
    eng = k2.Engine(ctx, spec)
    logits, greedy = run(eng)
    eng.close()
    ok = agree(logits) and agree(greedy)
    if rank == 0:
        import oracle as o
        whole = synth.random_model(ep_cfg, "nf4g128", seed=43, untied=True, moe=moe)
        emu = o.EpModel(whole, world)
        want = np.stack([emu.forward_token(t) for t in tokens])
        nxt, stream = int(np.argmax(want[-1])), []
        for _ in range(12):
            nxt = o.argmax(emu.forward_token(nxt)); stream.append(nxt)
        emu.close()
        ok = ok and np.array_equal(logits, want) and list(greedy) == stream
    res["ep_parity_ok"] = bool(ok)
    flag = torch.tensor([int(res["tp_parity_ok"]), int(res["ep_parity_ok"])], device="cuda")
    dist.broadcast(flag, 0)
    return {"tp_parity_ok": bool(flag[0].item()), "ep_parity_ok": bool(flag[1].item()),
            "what": "logits of a 9-token prompt and 12 greedy tokens, every rank bit-identical to the rank-order CPU emulation (small models, outside the timed regions)"}


def decode_moe(ctx, timed_region, rank, world, dist):
    """Whole-token decode of the Qwen3-30B-A3B shape (48 layers, 128 experts of 768, top-8, nf3 experts, nf4g128 attention;
    random codes), expert-parallel over all ranks: rank r holds the experts e % world == r, the partial weighted sums are
    exchanged inside the norm kernel after every MoE block."""
    import numpy as np
    import kronos_2t_b200 as k2
    from kronos_2t_b200 import synth
    rng = np.random.Generator(np.random.PCG64(29))
    cfg = dict(synth.QWEN3_30B_A3B)
    t0 = time.perf_counter()
    spec = synth.random_model(cfg, "nf4g128", seed=9, untied=True, share_layers=True, ep=(world, rank),
                              moe=dict(n_experts=128, top_k=8, d_ff=768, bits=3, sgc=1))
    eng = k2.Engine(ctx, spec)
    build_s = time.perf_counter() - t0
    if world > 1:
        handles = [None] * world
        dist.all_gather_object(handles, eng.tp_handle())
        eng.tp_attach(handles)
        dist.barrier()
    steps = 32
    prefill = _prefill(eng, rng, cfg["vocab"], 0, 512 - steps, timed_region)
    out = {"model": "Qwen3-30B-A3B-shaped (hidden 2048, 48 layers, 32q/4kv heads of 128, 128 experts of 768, top-8, vocab 151936), "
                    "nf3 experts, nf4g128 attention", "kv": "int8", "ep": world, "build_s": round(build_s, 1),
           "prefill_tok_s_480": prefill, "weight_bytes_per_token": eng.weight_bytes,
           "exchange": None if world == 1 else "1 partial-sum exchange per MoE block inside the norm kernel (peer memory, no NCCL on the data path)"}
    peak, _ = peaks()
    roof = []
    # a token streams the dense tensors + router of every layer and the routed experts; under expert parallelism the ranks
    # hold disjoint experts, so the experts' bytes are divided and the dense part is read by every rank
    for name, pos in (("ctx_512", 512 - steps), ("ctx_6600", 6600)):
        eng.decode_greedy(1, pos, 4)
        ms = min(timed_region(lambda: eng.decode_greedy(1, pos, steps)) for _ in range(2))
        out[name] = {"tok_s": steps / (ms / 1e3), "ms_per_token": ms / steps, "positions": [pos, pos + steps], "attention": "reference order"}
        roof.append(_decode_entry("Qwen3-30B-A3B nf3 experts / nf4g128 attention", pos + steps // 2, "int8", "reference order", steps / (ms / 1e3),
                                  eng.weight_bytes, eng.kv_bytes_per_pos, peak, n_gpus=world, parallel=None if world == 1 else f"ep{world}"))
    out["ctx_6600"]["note"] = "cache rows 480..6599 are zero: kernel time does not depend on the cached values"
    eng.close()
    return out, roof


def run_decode_only(args, local_rank):
    """Small whole-token run for profilers: engine of the chosen shape, 16-token prompt, then N greedy steps starting at
    position --decode-ctx (positions in between stay zero: kernel time does not depend on the cached values)."""
    import numpy as np
    import torch
    import kronos_2t_b200 as k2
    from kronos_2t_b200 import synth
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    ctx = k2.Context(local_rank)
    pos = max(args.decode_ctx, 15)
    if args.decode_model == "1.7b":
        cfg = dict(synth.SMOLLM2_1_7B, kv_bits=args.kv_bits, max_seq=pos + args.decode_only + args.prefill_only + 1)
        spec = synth.random_model(cfg, "nf4g128", seed=5, share_layers=True)
    elif args.decode_model == "moe":
        cfg = dict(synth.QWEN3_30B_A3B, kv_bits=args.kv_bits, max_seq=pos + args.decode_only + args.prefill_only + 1, layers=args.decode_layers or 48)
        spec = synth.random_model(cfg, "nf4g128", seed=9, untied=True, share_layers=True, moe=dict(n_experts=128, top_k=8, d_ff=768, bits=3, sgc=1))
    elif args.decode_model == "7b":
        cfg = dict(synth.QWEN2_7B, kv_bits=args.kv_bits, max_seq=pos + args.decode_only + args.prefill_only + 1)
        spec = synth.random_model(cfg, "b4", seed=7, modes=synth.P55454, qkv_bias=True, untied=True, share_layers=True)
    else:
        cfg = dict(synth.SMOLLM2_135M, kv_bits=args.kv_bits, max_seq=max(512, pos + args.decode_only + args.prefill_only + 1))
        spec = synth.random_model(cfg, "b4", seed=3)
    if args.split_kv:
        spec["cfg"]["split_kv_attention"] = True
    eng = k2.Engine(ctx, spec)
    if args.prefill_only:          # prompt batches alone: N tokens from position --decode-ctx on, twice (the second pass is timed)
        toks = np.random.Generator(np.random.PCG64(11)).integers(0, cfg["vocab"], args.prefill_only).astype(np.uint32)
        start = args.decode_ctx if args.decode_ctx > 15 else 0
        eng.forward_token_ids(toks, pos_start=start)
        torch.cuda.synchronize()
        l0, t0 = ctx.launch_count, time.perf_counter()
        eng.forward_token_ids(toks, pos_start=start)
        dt = time.perf_counter() - t0
        print(json.dumps({"mode": "prefill-only", "model": args.decode_model, "kv_bits": args.kv_bits, "pos_start": start, "tokens": args.prefill_only,
                          "launches": int(ctx.launch_count - l0), "wall_ms": dt * 1e3, "tok_s": args.prefill_only / dt}))
        eng.close()
        ctx.close()
        return
    prompt = np.random.Generator(np.random.PCG64(11)).integers(0, cfg["vocab"], 16).astype(np.uint32)
    l0 = ctx.launch_count
    eng.forward_token_ids(prompt[:-1])
    l1 = ctx.launch_count
    eng.decode_greedy(int(prompt[-1]), pos, 2)          # graph capture and warm-up
    l2 = ctx.launch_count
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    toks = eng.decode_greedy(int(prompt[-1]), pos, args.decode_only)
    dt = time.perf_counter() - t0
    print(json.dumps({"mode": "decode-only", "model": args.decode_model, "kv_bits": args.kv_bits, "pos_start": pos, "steps": args.decode_only,
                      "prompt_launches": int(l1 - l0), "warmup_launches": int(l2 - l1), "decode_launches": int(ctx.launch_count - l2),
                      "wall_ms": dt * 1e3, "ms_per_token": dt * 1e3 / args.decode_only, "last_token": int(toks[-1])}))
    eng.close()
    ctx.close()


def cpu_decode_baseline():
    """The oracle's dense decode step on the same model shape, all host threads: 16 prompt tokens, 16 greedy steps."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np
    import oracle as o
    from kronos_2t_b200 import synth
    spec = synth.random_model(synth.SMOLLM2_135M, "b4", seed=3)
    threads = os.cpu_count() or 1
    m = o.Model(spec)
    prompt = np.random.Generator(np.random.PCG64(11)).integers(0, spec["cfg"]["vocab"], 16)
    logits = None
    for t in prompt:
        logits = m.forward_token(int(t), threads)
    t0 = time.perf_counter()
    n = 0
    while n < 16 or (time.perf_counter() - t0 < 5.0 and n < 256):
        logits = m.forward_token(o.argmax(logits), threads)
        n += 1
    dt = time.perf_counter() - t0
    m.close()
    return {"value": n / dt, "unit": "tok/s", "cores": threads, "kind": "port", "sample": f"{n} greedy steps after a 16-token prompt"}


def cpu_baseline(mats):
    """Oracle (C++ port of the reference CPU path) on one pass of the same sweep, all host threads."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np
    import oracle as o
    threads = os.cpu_count() or 1
    rng = np.random.Generator(np.random.PCG64(7))
    prepared = []
    for m in mats:
        x = rng.standard_normal(m["cols"]).astype(np.float32)
        if m["kind"] == "bipolar":
            om = o.nibble4_from_bipolar(o.Bipolar(m["rows"], m["cols"], m["bits"], m["d0"], m["d1"]))
        else:
            om = o.Nf(m["rows"], m["cols"], m["bits"], m["sgc"], _default_cb(m["bits"]), m["d0"], m["d1"])
        prepared.append((m, om, x))
    passes, t0 = 0, time.perf_counter()
    while passes < 2 or (time.perf_counter() - t0 < 10.0 and passes < 50):
        if passes == 1:
            t0 = time.perf_counter()   # first pass is warm-up
        for m, om, x in prepared:
            act = o.act_populate_fwht(x)
            (o.nibble4_gemv if m["kind"] == "bipolar" else o.nf_gemv)(om, act, threads=threads)
        passes += 1
    dt = time.perf_counter() - t0
    total = sum(algorithmic_bytes(m["fmt"], m["cols"], m["rows"]) for m in mats) * (passes - 1)
    return {"value": total / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{passes - 1} full passes of the 16-matrix sweep after one warm-up pass"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-token decode measurement")
    ap.add_argument("--no-decode-moe", action="store_true", help="skip the sparse-MoE (30B-A3B-shaped) decode measurement")
    ap.add_argument("--no-decode-models", action="store_true", help="skip the 1.7B / 7B-shaped decode measurements")
    ap.add_argument("--decode-only", type=int, default=0, metavar="N",
                    help="profiling mode: only the whole-token engine - a 16-token prompt, then N greedy steps")
    ap.add_argument("--prefill-only", type=int, default=0, metavar="N",
                    help="small run for profilers: a prompt of N tokens from position --decode-ctx on (model: --decode-model), nothing else")
    ap.add_argument("--decode-model", default="135m", choices=["135m", "1.7b", "7b", "moe"], help="--decode-only: model shape")
    ap.add_argument("--decode-layers", type=int, default=0, help="--decode-only, moe: fewer layers than the shape's 48 (profiling)")
    ap.add_argument("--decode-ctx", type=int, default=15, help="--decode-only: position of the first greedy step")
    ap.add_argument("--kv-bits", type=int, default=8, choices=[4, 8], help="--decode-only: KV cache format")
    ap.add_argument("--split-kv", action="store_true", help="--decode-only: split-KV attention beyond 512 positions (the engine's opt-in flag)")
    ap.add_argument("--case", default=None, help="profile one case, e.g. b4:2048x49152 (fmt:KxN)")
    ap.add_argument("--tokens", type=int, default=1, help="tokens per launch in --case mode (1..4)")
    ap.add_argument("--no-graph", action="store_true", help="--case mode: skip the CUDA-graph replay timing")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.decode_only or args.prefill_only:
        run_decode_only(args, local_rank)
    elif args.case:
        run_case(args, local_rank)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_b200(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
