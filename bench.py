#!/usr/bin/env python
"""Benchmark of the one-bit 2:4 sparse GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--size S]

A step is one pass C = A_sparse x B of the square workload a_rows = n = a_cols = S (default 8192,
the size the >= 60 %-of-sparse-peak target is quoted on) with per-row fp16 scale, fp16 tokens, fp32
accumulation and fp16 output. With N > 1 every rank owns one S-row slab of A (a_rows = S * N, weak
scaling, no data-path collective; B replicated). Rank 0 prints ONE JSON line.

  value     dense-equivalent TFLOP/s (2*m*n*k / t), operands resident in HBM, device-timed
  e2e       the same metric through the host-buffer entry point (onebit_matmul_packed_host) with
            tokens in pinned host memory and the result returned to pinned host memory: both copies
            are inside the timed region, pipelined with the GEMM in column panels (weights stay
            resident: packing is an offline step, as in the reference)
  roofline  tensor-core bound; peak = 2 x the measured dense bf16 peak (2:4 sparse MMA rate)
  cpu_baseline  the CPU oracle (a port of the reference's host check) on a bounded row sample

--impl reference times the reference's CPU implementation of the path (the oracle port: the
reference's host GEMM needs its absent CUTLASS submodule) on the host cores, same config.
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

METRIC = "dense-equivalent TFLOP/s, one-bit 2:4 sparse GEMM (square)"


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs: NVML every 2 ms (the timed region
    of a default run is tens of milliseconds), nvidia-smi as the fallback."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    # NVML clocks-event-reason bits
    REASON_BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index, uuid=None):
        self.index, self.samples, self.stop = index, [], threading.Event()     # samples: (mhz, max mhz, reason bits)
        self.handle = self.nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if isinstance(uuid, str) else uuid)
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.nvml = pynvml
        except Exception:
            self.handle = None
        self.thread = threading.Thread(target=self.run, daemon=True)

    def sample_nvml(self):
        n, h = self.nvml, self.handle
        mhz = n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)
        top = n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)
        try:
            bits = n.nvmlDeviceGetCurrentClocksEventReasons(h)
        except Exception:
            bits = n.nvmlDeviceGetCurrentClocksThrottleReasons(h)
        self.samples.append((int(mhz), int(top), int(bits)))

    def sample_smi(self):
        out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                              "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
        parts = [x.strip() for x in out.strip().split(",")]
        if len(parts) >= 6 and parts[0].isdigit() and parts[1].isdigit():
            order = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            bits = sum(dict(self.REASON_BITS)[name] for i, name in enumerate(order) if parts[2 + i].lower().startswith("active"))
            self.samples.append((int(parts[0]), int(parts[1]), bits))

    def run(self):
        while not self.stop.is_set():
            try:
                if self.handle is not None:
                    self.sample_nvml()
                else:
                    self.sample_smi()
            except Exception:
                pass
            self.stop.wait(0.002 if self.handle is not None else 0.02)

    def __enter__(self):
        self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.thread.join(timeout=10)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = sorted(s[0] for s in self.samples)
        bits = 0
        for s in self.samples:
            bits |= s[2]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_min_mhz": mhz[0], "sm_max_mhz": self.samples[0][1],
                "reasons": [name for name, bit in self.REASON_BITS if bits & bit], "samples": len(self.samples),
                "source": "nvml" if self.handle is not None else "nvidia-smi"}


def cpu_sample(size, rows, threads=0):
    """Times the oracle GEMM on `rows` weight rows of the size^3 workload; returns (TFLOP/s, seconds, cores)."""
    import oracle
    from tests import helpers
    rng = np.random.default_rng(3080)
    dense, scale = helpers.make_weights(rng, rows, size)
    B = helpers.make_tokens(rng, size, size)
    canon, signs, _ = oracle.compress(dense)
    bits, meta = oracle.pack_bits(signs), oracle.meta_reorder(canon, oracle.META_CUTLASS)
    # all host cores, whatever OMP_NUM_THREADS a launcher exported (torchrun sets it to 1)
    cores = len(os.sched_getaffinity(0)) if threads == 0 else threads
    t0 = time.perf_counter()
    oracle.gemm(bits, meta, oracle.META_CUTLASS, B, rows, scale=scale, threads=cores)
    dt = time.perf_counter() - t0
    return 2.0 * rows * size * size / dt / 1e12, dt, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 512
    vals = []
    for i in range(args.warmup + args.steps):
        v, dt, cores = cpu_sample(args.size, rows)
        if i >= args.warmup:
            vals.append((v, dt))
    v = float(np.mean([x[0] for x in vals]))
    ms = float(np.mean([x[1] for x in vals])) * 1e3
    sample = f"{rows} of {args.size} weight rows x full k x full n per step (oracle port, OpenMP)"
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"square {args.size}^3 one-bit 2:4 sparse GEMM", "sample": sample},
            "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def decode_extras(ob, lib, _lib, dev):
    """The memory-bound regime of the same path (config 2: 7B-class layers, few tokens): algorithmic
    HBM GB/s of the decode kernel, launched back to back over a pool of distinct packed weights
    larger than L2 so that every call streams its weights from HBM."""
    import torch
    peaks = load_peaks()
    out = []
    for (m, k) in ((4096, 4096), (11008, 4096), (4096, 11008)):
        w = torch.zeros((m, k // 4, 4), dtype=torch.float16, device=dev)
        w[..., 0], w[..., 3] = 1.0, -1.0
        pw = ob.pack_weight(w.reshape(m, k), apply_mask=False, keep_reference=False)
        del w
        weight_bytes = pw.bits_tile.numel() + pw.meta_tile.numel()
        copies = max(2, int(2.2 * 126e6 / weight_bytes))
        pool = [ob.PackedWeight(m, k, pw.bits_tile.clone(), pw.meta_tile.clone(), None) for _ in range(copies)]
        for n in (1, 4, 8, 16):
            B = torch.randn((k, n), device=dev, dtype=torch.float32).to(torch.float16)
            C = torch.empty((m, n), dtype=torch.float16, device=dev)
            for i in range(copies):
                ob.matmul_packed(pool[i], B, out=C, kernel=_lib.KERNEL_DECODE)
            torch.cuda.synchronize()
            # one pass over the pool captured in a CUDA graph: device-side cost without host launch time
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(copies):
                    ob.matmul_packed(pool[i], B, out=C, kernel=_lib.KERNEL_DECODE)
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(4):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (4 * copies)
            del graph
            alg = weight_bytes + 2 * k * n + 2 * m * n
            out.append({"a_rows": m, "a_cols": k, "n": n, "us_per_call": round(us, 3), "algorithmic_bytes": alg,
                        "gbs": round(alg / us / 1e3, 1), "frac_of_measured_hbm": round(alg / us / 1e3 / peaks["hbm_gbs"], 4),
                        "weight_pool_mb": round(copies * weight_bytes / 1e6, 1)})
        del pool
    return {"kernel": "ob_gemm_decode_kernel", "bound": "hbm", "peak_gbs": peaks["hbm_gbs"], "cases": out,
            "note": "CUDA-graph replay of back-to-back calls over a weight pool > 2 x L2 (every call streams its weights "
                    "from HBM; consecutive calls overlap through programmatic dependent launch); a single call moves "
                    "3-9 MB, so kernel launch, DRAM latency and the instruction issue of the sign expansion, not "
                    "bandwidth, set its time"}


def run_ours(args):
    import torch
    import torch.distributed as dist

    import onebitsparsemul_b200 as ob
    from onebitsparsemul_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = _lib.load()
    S = args.size
    m = n = k = S
    dev = torch.device("cuda", local)

    # synthetic, seeded: random valid 2:4 pattern, Bernoulli signs, scale U[0.01,0.1], tokens N(0,1)
    g = torch.Generator(device=dev)
    g.manual_seed(3080 + rank)
    nib = torch.tensor([0x4, 0x8, 0x9, 0xC, 0xD, 0xE], device=dev)[torch.randint(0, 6, (m, k // 4), device=dev, generator=g)]
    sign = (torch.randint(0, 2, (m, k // 4, 2), device=dev, generator=g) * 2 - 1).to(torch.float16)
    w = torch.zeros((m, k // 4, 4), dtype=torch.float16, device=dev)
    w.scatter_(2, (nib & 3).unsqueeze(-1), sign[..., 0:1])
    w.scatter_(2, (nib >> 2).unsqueeze(-1), sign[..., 1:2])
    scale = torch.empty(m, device=dev).uniform_(0.01, 0.1, generator=g).to(torch.float16)
    layer = ob.BinaryLinear_2_4(k, m, out_dtype=torch.float16).to(dev)
    t0 = time.perf_counter()
    layer.pack(w.reshape(m, k), scale=scale)
    torch.cuda.synchronize()
    pack_ms = (time.perf_counter() - t0) * 1e3
    del w, nib, sign
    B = torch.randn((k, n), device=dev, generator=g, dtype=torch.float32).to(torch.float16)
    C = torch.empty((m, n), dtype=torch.float16, device=dev)
    pw = ob.PackedWeight(m, k, layer.bits_tile, layer.meta_tile, layer.scale)

    def step():
        ob.matmul_packed(pw, B, out=C)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    _lib.check(lib.onebit_check_device_status())

    sync_all()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    try:
        gpu_uuid = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)    # NVML may number the GPUs differently
    except Exception:
        gpu_uuid = None
    with ClockSampler(local, gpu_uuid) as clocks:
        ev[0].record()
        for i in range(args.steps):
            step()
            ev[i + 1].record()
        sync_all()
    total_ms = ev[0].elapsed_time(ev[-1])
    kernel_ms = float(np.mean([ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]))
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    _lib.check(lib.onebit_check_device_status())
    flops_step = 2.0 * m * n * k * world
    value = flops_step * args.steps / (total_ms * 1e-3) / 1e12

    # end to end: tokens in pinned host memory, result into pinned host memory, through the library's
    # host-buffer entry point (onebit_matmul_packed_host): H2D of B and D2H of C are inside the timed
    # region, overlapped with the GEMM panel by panel
    Bh = B.cpu().pin_memory()
    Ch = torch.empty((m, n), dtype=torch.float16).pin_memory()

    def e2e_step():
        ob.matmul_packed_host(pw, Bh, Ch)

    for _ in range(2):
        e2e_step()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(2, min(args.steps, 10))
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    sync_all()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = flops_step * e2e_steps / (float(t.item()) * 1e-3) / 1e12

    decode = None
    if rank == 0 and world == 1 and not args.no_decode:
        decode = decode_extras(ob, lib, _lib, dev)

    if rank == 0:
        peaks = load_peaks()
        sparse_peak = 2.0 * peaks["bf16_tflops"]
        achieved = 2.0 * m * n * k / (kernel_ms * 1e-3) / 1e12
        cpu_v, cpu_dt, cores = cpu_sample(S, 2048)
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            # the reference README publishes 67 349.1 GFLOP/s for this size on an RTX 3060 Ti
            "vs_baseline": (value / world / 67.3491) if S == 8192 else None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"square one-bit 2:4 sparse GEMM a_rows={S * world} n={S} a_cols={S} (config 1), "
                                   f"{S}-row slab of A per GPU, fp16 tokens N(0,1), per-row fp16 scale, fp16 out",
                       "l2": "inputs larger than L2 (B and C 2*S*S bytes each)", "pack_ms": pack_ms},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": Bh.numel() * 2, "d2h_bytes_per_step": Ch.numel() * 2,
                    "note": "onebit_matmul_packed_host: tokens from pinned host memory, result to pinned host memory, "
                            "copies overlapped with the GEMM in column panels; weights resident"},
            "gpu_launches": args.steps,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": sparse_peak, "unit": "TFLOP/s",
                         "frac": achieved / sparse_peak,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the committed ncu capture of
                         # this workload (profiles/prefill_kernel_square8192_ncu_full.md); algorithmic bytes are 2.81e8
                         "traffic": 2.518e8 if S == 8192 else None,
                         "peak_note": f"2 x dense bf16 burst peak ({peaks['bf16_tflops']} TFLOP/s, {peaks['source']}): 2:4 sparse MMA rate",
                         "frac_of_dense_peak": achieved / peaks["bf16_tflops"], "kernel": "ob_gemm_prefill2_kernel<2> (CTA pair)",
                         "kernel_ms": kernel_ms},
            "cpu_baseline": {"value": cpu_v, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                             "sample": f"2048 of {S} weight rows x full k x full n ({cpu_dt:.2f} s)"},
            "clocks": clocks.summary(),
        }
        if decode is not None:
            line["decode"] = decode
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_sharded(args):
    """Supplementary: ONE size^3 GEMM row-sharded over the ranks (strong scaling), optional gather of C."""
    import torch
    import torch.distributed as dist

    from onebitsparsemul_b200 import _lib
    from onebitsparsemul_b200.sharded import ShardedBinaryLinear

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    S = args.size
    layer = ShardedBinaryLinear(S, S)
    g = torch.Generator(device=dev)
    g.manual_seed(3080 + rank)
    rows = layer.rows
    nib = torch.tensor([0x4, 0x8, 0x9, 0xC, 0xD, 0xE], device=dev)[torch.randint(0, 6, (rows, S // 4), device=dev, generator=g)]
    sign = (torch.randint(0, 2, (rows, S // 4, 2), device=dev, generator=g) * 2 - 1).to(torch.float16)
    w = torch.zeros((rows, S // 4, 4), dtype=torch.float16, device=dev)
    w.scatter_(2, (nib & 3).unsqueeze(-1), sign[..., 0:1])
    w.scatter_(2, (nib >> 2).unsqueeze(-1), sign[..., 1:2])
    scale = torch.empty(rows, device=dev).uniform_(0.01, 0.1, generator=g).to(torch.float16)
    layer.pack_slab(w.reshape(rows, S), scale, apply_mask=False)
    del w, nib, sign
    g.manual_seed(3080)                      # B is replicated: same on every rank
    B = torch.randn((S, S), device=dev, generator=g, dtype=torch.float32).to(torch.float16)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        out = layer.forward(B, gather=args.gather)
    _lib.check(lib.onebit_check_device_status())
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = layer.forward(B, gather=args.gather)
    e1.record()
    sync_all()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / args.steps
    if rank == 0:
        print(json.dumps({"metric": METRIC, "value": 2.0 * S * S * S / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
                          "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
                          "scaling": "strong", "dtype": "f16", "data": "synthetic",
                          "config": {"workload": f"ONE square GEMM {S}^3 row-sharded over {world} GPU(s), B replicated, "
                                                 f"gather={args.gather}", "rows_per_rank": layer.rows,
                                     "out_shape": list(out.shape), "fused_backend": layer.fused_backend}}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=8192)
    ap.add_argument("--no-decode", action="store_true", help="skip the supplementary decode-regime numbers")
    ap.add_argument("--workload", default="square", choices=["square", "sharded"],
                    help="square: one size^3 GEMM per GPU (weak scaling, the contract's line); sharded: ONE size^3 GEMM "
                         "row-sharded over all ranks (strong scaling, supplementary)")
    ap.add_argument("--gather", default="none", choices=["none", "all", "overlap", "fused", "push"],
                    help="sharded workload only: gather the full C on every rank")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "sharded":
        run_sharded(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
