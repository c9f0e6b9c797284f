#!/usr/bin/env python
"""Benchmark of the one-bit 2:4 sparse GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--size S]

A step is ONE pass C = A_sparse x B of the square workload a_rows = n = a_cols = S (default 25600, the
largest square of the configuration sweep) with per-row fp16 scale, fp16 tokens, fp32 accumulation and
fp16 output. With N > 1 the SAME problem is sharded by rows of A over the N ranks (strong scaling): rank
g packs and owns a contiguous slab of whole 256-row blocks, the tokens B are replicated, every rank
writes its slab of C, and nothing is exchanged while computing. Rank 0 prints ONE JSON line.

  value     dense-equivalent TFLOP/s (2*S^3 / t) of the whole job, operands resident in HBM, device-timed,
            t = max over ranks
  e2e       the same metric through the host-buffer entry point (onebit_matmul_packed_host): every rank
            takes the tokens from pinned host memory and returns its slab of C to pinned host memory, both
            copies inside the timed region, pipelined with the GEMM in column panels (weights stay
            resident: packing is an offline step, as in the reference)
  roofline  tensor-core bound; peak = 2 x the measured dense bf16 peak (2:4 sparse MMA rate), for the
            kernel launch of rank 0
  cpu_baseline  the CPU oracle (a port of the reference's host check) on a bounded row sample
  gather_nccl_ms / gather_fused_ms   (N > 1) the step when every rank wants the full C: GEMM followed by
            an NCCL all-gather, and the GEMM whose epilogue stores into every peer's C over NVLink
  sharded_bit_identical   outside the timed region, on integer tokens: every rank's slab equals the same
            rows of both gathered results, all ranks hold the same gathered C (checksums), and rank 0
            recomputes sampled rows of every slab with the CPU oracle, bit for bit
  square8192   the 8192^3 GEMM on rank 0 alone, device-timed (the burst figure of earlier records)
  decode       (N = 1) the memory-bound regime: few-token calls over weight pools larger than L2

--impl reference times the reference's CPU implementation of the path (the oracle port: the
reference's host GEMM needs its absent CUTLASS submodule) on the host cores, same config, on a bounded
row sample per step.
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
# the reference README's table for an RTX 3060 Ti, dense-equivalent TFLOP/s
PUBLISHED = {512: 14.8383, 1024: 27.4138, 2048: 46.4786, 4096: 52.1011, 8192: 67.3491, 10240: 66.9947, 16384: 70.8347,
             25600: 69.9825}
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel on one GPU, from ncu
# captures of exactly these workloads (bytes)
MEASURED_TRAFFIC = {8192: 2.518e8, 25600: 9.07e9}


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs: NVML every 2 ms, nvidia-smi as
    the fallback."""

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

    def summary(self, ms_per_step=None):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        mhz = sorted(s[0] for s in self.samples)
        bits = 0
        for s in self.samples:
            bits |= s[2]
        out = {"sm_mhz": mhz[len(mhz) // 2], "sm_min_mhz": mhz[0], "sm_max_mhz": self.samples[0][1],
               "reasons": [name for name, bit in self.REASON_BITS if bits & bit], "samples": len(self.samples),
               "source": "nvml" if self.handle is not None else "nvidia-smi"}
        if ms_per_step is not None:
            # time x clock: millions of SM cycles per step at the median clock seen under load
            out["mcycles_per_step"] = round(ms_per_step * 1e-3 * out["sm_mhz"], 1)
        return out


# ---- the CPU arm ---------------------------------------------------------------------------------------------

class CpuSample:
    """The oracle GEMM on `rows` weight rows of the size^3 workload (all of k, all of n)."""

    def __init__(self, size, rows):
        import oracle
        from tests import helpers
        self.oracle, self.size, self.rows = oracle, size, rows
        rng = np.random.default_rng(3080)
        dense, self.scale = helpers.make_weights(rng, rows, size)
        canon, signs, _ = oracle.compress(dense)
        self.bits, self.meta = oracle.pack_bits(signs), oracle.meta_reorder(canon, oracle.META_CUTLASS)
        # N(0,1) tokens: one 512-row block drawn, then repeated down the matrix (the values do not change the
        # oracle's work, and drawing 6.5e8 normals would take longer than the GEMM sample)
        block = rng.standard_normal((min(size, 512), size), dtype=np.float32).astype(np.float16)
        self.B = np.empty((size, size), np.float16)
        for r0 in range(0, size, block.shape[0]):
            r1 = min(size, r0 + block.shape[0])
            self.B[r0:r1] = block[:r1 - r0]
        # all host cores, whatever OMP_NUM_THREADS a launcher exported (torchrun sets it to 1)
        self.cores = len(os.sched_getaffinity(0))

    def step(self):
        t0 = time.perf_counter()
        self.oracle.gemm(self.bits, self.meta, self.oracle.META_CUTLASS, self.B, self.rows, scale=self.scale, threads=self.cores)
        dt = time.perf_counter() - t0
        return 2.0 * self.rows * self.size * self.size / dt / 1e12, dt


def workload_name(size, world):
    return (f"ONE square one-bit 2:4 sparse GEMM a_rows=n=a_cols={size} (configs 1 and 4), rows of A sharded over {world} GPU(s) "
            f"in slabs of whole 256-row blocks, tokens replicated, fp16 tokens N(0,1), per-row fp16 scale, fp16 out")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # Rows per step: whole 64-row groups (metadata shuffle), as many as keep the whole run near 2.5 minutes, at most the
    # ~1e12 flop of the cpu_baseline leg. A call of the oracle costs a fixed ~1.7 s at 25600 (it converts the tokens)
    # plus ~8.4 ms per row; small samples would time the conversion, not the GEMM.
    per_step_s = 150.0 / max(1, args.warmup + args.steps)
    scale = (args.size / 25600.0) ** 2
    rows = int(max(0.0, per_step_s - 1.7 * scale) / (0.0084 * scale)) // 64 * 64
    rows = max(64, min(rows, args.size, max(64, int(1e12 / (2.0 * args.size * args.size)) // 64 * 64)))
    cpu = CpuSample(args.size, rows)
    vals = []
    for i in range(args.warmup + args.steps):
        v, dt = cpu.step()
        if i >= args.warmup:
            vals.append((v, dt))
    v = float(np.mean([x[0] for x in vals]))
    ms = float(np.mean([x[1] for x in vals])) * 1e3
    sample = f"{rows} of {args.size} weight rows x full k x full n per step (oracle port, OpenMP)"
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload_name(args.size, args.gpus), "sample": sample},
            "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": cpu.cores, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit_line(line)


# ---- our arm ---------------------------------------------------------------------------------------------------

def gpu_weights(rows, k, seed, dev):
    """Seeded synthetic slab: uniformly random valid 2:4 pattern, Bernoulli signs, scale U[0.01, 0.1]."""
    import torch
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    nib = torch.tensor([0x4, 0x8, 0x9, 0xC, 0xD, 0xE], device=dev)[torch.randint(0, 6, (rows, k // 4), device=dev, generator=g)]
    sign = (torch.randint(0, 2, (rows, k // 4, 2), device=dev, generator=g) * 2 - 1).to(torch.float16)
    w = torch.zeros((rows, k // 4, 4), dtype=torch.float16, device=dev)
    w.scatter_(2, (nib & 3).unsqueeze(-1), sign[..., 0:1])
    w.scatter_(2, (nib >> 2).unsqueeze(-1), sign[..., 1:2])
    scale = torch.empty(rows, device=dev).uniform_(0.01, 0.1, generator=g).to(torch.float16)
    return w.reshape(rows, k), scale


def timed(fn, steps, sync_all, reduce_max):
    """Mean milliseconds per call of fn over `steps` calls, device-timed, max over ranks."""
    import torch
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    sync_all()
    return reduce_max(e0.elapsed_time(e1)) / steps


def decode_extras(ob, _lib, dev):
    """The memory-bound regime of the same path (config 2: 7B-class layers, few tokens) and two larger weights
    where bandwidth can dominate: algorithmic HBM GB/s of the few-token kernel, replayed from a CUDA graph over a
    pool of distinct packed weights larger than L2, so that every call streams its weights from HBM."""
    import torch
    peaks = load_peaks()
    out = []
    for (m, k) in ((4096, 4096), (11008, 4096), (4096, 11008), (28672, 8192), (25600, 25600)):
        w = torch.zeros((m, k // 4, 4), dtype=torch.float16, device=dev)
        w[..., 0], w[..., 3] = 1.0, -1.0
        pw = ob.pack_weight(w.reshape(m, k), apply_mask=False, keep_reference=False)
        del w
        weight_bytes = pw.bits_tile.numel() + pw.meta_tile.numel()
        copies = max(3, int(2.2 * 126e6 / weight_bytes) + 1)
        pool = [ob.PackedWeight(m, k, pw.bits_tile.clone(), pw.meta_tile.clone(), None) for _ in range(copies)]
        for n in ((1, 4, 8, 16) if m * k < 1e8 else (1, 8, 16)):
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
    return {"kernel": "ob_gemm_fewtok_kernel (tcgen05; ob_gemm_decode_kernel, the mma.sp form, for n <= 8 at 4096 x 4096 and n = 1 at 4096 x 11008)", "bound": "hbm", "peak_gbs": peaks["hbm_gbs"], "cases": out,
            "note": "CUDA-graph replay of back-to-back calls over a weight pool > 2 x L2 (every call streams its weights "
                    "from HBM; consecutive calls overlap through programmatic dependent launch). The three 7B-class "
                    "shapes move 3-9 MB per call, less than a launch and a DRAM round trip cost at HBM speed; the "
                    "44 MB and 123 MB weights show the kernel's streaming rate"}


def decode_loop_extras(ob, dev):
    """The decode regime as a model sees it: a Llama-7B-shaped stack (4 blocks = 28 linear layers, 152 MB of packed
    weights, more than L2) with every nn.Linear swapped for the one-bit layer, one step captured in a CUDA graph
    and replayed per token."""
    import torch
    from onebitsparsemul_b200.decode_loop import LlamaShapedStack, measure_decode
    peaks = load_peaks()
    torch.cuda.empty_cache()
    stack = LlamaShapedStack(blocks=4, hidden=4096, intermediate=11008, device=dev, seed=1)
    replaced = ob.replace_linear_layers(stack)
    out = {"model": "4 Llama-7B-shaped decoder blocks (q/k/v/o 4096x4096, gate/up 11008x4096, down 4096x11008), random weights, "
                    "element-wise glue between the layers", "replaced_layers": replaced, "cases": []}
    for tokens in (1, 8, 16):
        r = measure_decode(stack, 4096, tokens=tokens, steps=30, device=dev)
        r["frac_of_measured_hbm"] = round(r["weight_gbs"] / peaks["hbm_gbs"], 4)
        out["cases"].append({k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()})
    del stack
    # the same blocks with q/k/v and gate/up as one layer each (12288 x 4096, 22016 x 4096): 4 GEMMs per block
    torch.cuda.empty_cache()
    stack = LlamaShapedStack(blocks=4, hidden=4096, intermediate=11008, device=dev, seed=1, fused=True)
    ob.replace_linear_layers(stack)
    out["fused_projections_note"] = ("q/k/v as one 12288 x 4096 layer and gate/up as one 22016 x 4096 layer, 16 GEMMs instead of 28: "
                                     "slower, not faster, with this kernel -- 172 row blocks x 32 k tiles fill 172 of the 296 CTA "
                                     "slots and no K split fits a wave, where two 11008 x 4096 calls run 258 CTAs of 11 tiles each")
    out["fused_projections"] = []
    for tokens in (1, 8):
        r = measure_decode(stack, 4096, tokens=tokens, steps=30, device=dev)
        r["frac_of_measured_hbm"] = round(r["weight_gbs"] / peaks["hbm_gbs"], 4)
        out["fused_projections"].append({k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()})
    del stack
    torch.cuda.empty_cache()
    return out


def context_baselines(dev, sizes):
    """Numbers that put the headline in context, outside the timed region: the reference's own host check GEMM
    (the CUTLASS template its CLI instantiates, one core, 512^3 -- the size of the reference's CPU-runnable
    configuration) and cuBLAS dense fp16 through torch.matmul at the benchmark sizes."""
    import torch
    out = {}
    try:
        from oracle import build_ref
        r = build_ref.run(512, 512, 512)
        if r is not None:
            out["reference_host_gemm_512"] = {"seconds": r[0], "gflops": r[1], "cores": 1, "kind": "reference",
                                              "what": "cutlass::reference::host::Gemm<half, ColumnMajor, half, RowMajor, float, RowMajor, "
                                                      "float, float>, the instantiation of the reference's --reference-check, dense-equivalent "
                                                      "GFLOP/s of 512^3"}
        else:
            out["reference_host_gemm_512"] = "unavailable on this box: oracle/_ref was not built (no CUTLASS copy)"
    except Exception as exc:
        out["reference_host_gemm_512"] = f"failed: {exc}"[:200]
    dense = {}
    for q in sizes:
        try:
            W = torch.randn((q, q), device=dev, dtype=torch.float32).to(torch.float16)
            B = torch.randn((q, q), device=dev, dtype=torch.float32).to(torch.float16)
            C = torch.empty((q, q), device=dev, dtype=torch.float16)
            for _ in range(3):
                torch.matmul(W, B, out=C)
            torch.cuda.synchronize()
            steps = 20 if q <= 8192 else 6
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                torch.matmul(W, B, out=C)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
            dense[str(q)] = {"ms": ms, "tflops": 2.0 * q ** 3 / (ms * 1e-3) / 1e12}
            del W, B, C
        except Exception as exc:
            dense[str(q)] = f"failed: {exc}"[:200]
    out["torch_matmul_dense_fp16"] = dense
    return out


def bit_identity(ob, _lib, oracle, layer, S, world, rank, dev, reduce_minmax):
    """Outside the timed region, integer tokens (every partial sum exact): the sharded job against the oracle
    and the ranks against each other. Returns a dict of booleans on every rank (rank 0's oracle verdict is
    shared with all ranks)."""
    import torch
    g = torch.Generator(device=dev)
    g.manual_seed(4242)
    Bi = torch.randint(-8, 9, (S, S), device=dev, generator=g).to(torch.float16)
    packed = layer.packed
    layer.packed = ob.PackedWeight(packed.m, packed.k, packed.bits_tile, packed.meta_tile, None, stable=True)   # no scale: exact
    res = {}
    try:
        slab = layer.forward(Bi, gather="none").clone()
        full = slab
        if world > 1:
            mine = slice(layer.start, layer.start + layer.rows)
            full = layer.forward(Bi, gather="all")
            res["slab_equals_nccl_gather"] = bool(torch.equal(full[mine], slab))
            fused = layer.forward(Bi, gather="fused")
            torch.cuda.synchronize()
            res["fused_equals_nccl_gather"] = bool(torch.equal(fused, full))
            # every rank holds the same gathered C
            digest = float(full.view(torch.int16).to(torch.float64).mul_(torch.arange(1, S + 1, device=dev, dtype=torch.float64)).sum().item())
            lo, hi = reduce_minmax(digest)
            res["ranks_hold_the_same_c"] = bool(lo == hi)
        # rank 0: sampled rows of EVERY slab against the CPU oracle, bit for bit (fp16 of the exact fp32 sums)
        ok = 1.0
        if rank == 0:
            gs = torch.Generator(device=dev)
            cols = 256
            Bh = Bi[:, :cols].cpu().numpy()
            for p, (start, rows) in enumerate(layer.partition):
                w, _ = gpu_weights(rows, S, 3080 + p, dev)
                gs.manual_seed(99 + p)
                pick = torch.randperm(rows, device=dev, generator=gs)[:128].sort().values
                canon, signs, _ = oracle.compress(w[pick].cpu().numpy())
                del w
                _, want16 = oracle.gemm(oracle.pack_bits(signs), oracle.meta_reorder(canon, 0), 0, Bh, 128)
                got = (full[start + pick] if world > 1 else slab[pick])[:, :cols].cpu().numpy()
                if not (got == want16).all():
                    ok = 0.0
        lo, _ = reduce_minmax(ok if rank == 0 else 1.0)
        res["oracle_sampled_rows_exact"] = bool(lo == 1.0)
    finally:
        layer.packed = packed
    res["all"] = all(res.values())
    return res


def run_ours(args):
    import torch
    import torch.distributed as dist

    import onebitsparsemul_b200 as ob
    import oracle
    from onebitsparsemul_b200 import _lib
    from onebitsparsemul_b200.sharded import ShardedBinaryLinear

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    S = args.size
    warmup = max(args.warmup, 3)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(x):
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_minmax(x):
        lo = torch.tensor([x], device=dev, dtype=torch.float64)
        hi = lo.clone()
        if world > 1:
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        return float(lo.item()), float(hi.item())

    # this rank's slab of the one problem; B is replicated (same seed everywhere)
    layer = ShardedBinaryLinear(S, S)
    rows = layer.rows
    w, scale = gpu_weights(rows, S, 3080 + rank, dev)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    layer.pack_slab(w, scale, apply_mask=False)
    torch.cuda.synchronize()
    pack_ms = (time.perf_counter() - t0) * 1e3
    del w
    g = torch.Generator(device=dev)
    g.manual_seed(3080)
    B = torch.empty((S, S), dtype=torch.float16, device=dev)
    for r0 in range(0, S, 4096):
        r1 = min(S, r0 + 4096)
        B[r0:r1] = torch.randn((r1 - r0, S), device=dev, generator=g, dtype=torch.float32).to(torch.float16)
    C = torch.empty((rows, S), dtype=torch.float16, device=dev)
    pw = layer.packed

    def step():
        ob.matmul_packed(pw, B, out=C)

    for _ in range(warmup):
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
    total_ms = reduce_max(ev[0].elapsed_time(ev[-1]))
    kernel_ms = float(np.mean([ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]))
    _lib.check(lib.onebit_check_device_status())
    flops_step = 2.0 * S * S * S
    value = flops_step * args.steps / (total_ms * 1e-3) / 1e12

    # end to end: tokens in pinned host memory, this rank's slab of the result into pinned host memory, through
    # the library's host-buffer entry point: H2D of B and D2H of C are inside the timed region, overlapped
    # with the GEMM panel by panel
    Bh = torch.empty((S, S), dtype=torch.float16).pin_memory()
    Bh.copy_(B)
    Ch = torch.empty((rows, S), dtype=torch.float16).pin_memory()

    def e2e_step():
        layer.forward_host(Bh, Ch)                 # one rank: onebit_matmul_packed_host; several: 1/world of B per rank + NVLink all-gather

    for _ in range(2):
        e2e_step()
    e2e_steps = max(2, min(args.steps, 5))
    e2e_ms = timed(e2e_step, e2e_steps, sync_all, reduce_max)
    e2e_value = flops_step / (e2e_ms * 1e-3) / 1e12
    h2d = float(Bh.numel() * 2) if (world == 1 or S % world == 0) else float(Bh.numel() * 2) * world   # B crosses PCIe once per node
    d2h_t = torch.tensor([float(Ch.numel() * 2)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(d2h_t)
    d2h = float(d2h_t.item())
    del Bh, Ch

    # the full C on every rank: NCCL all-gather after the GEMM, and the GEMM whose epilogue stores to every peer
    gathers = {}
    if world > 1:
        gsteps = max(2, min(args.steps, 10))
        for mode in ("all", "fused"):
            try:
                for _ in range(2):
                    layer.forward(B, gather=mode)
                gathers[mode] = timed(lambda: layer.forward(B, gather=mode), gsteps, sync_all, reduce_max)
            except Exception as exc:                       # e.g. no peer-mappable memory on this box
                gathers[mode] = f"failed: {type(exc).__name__}: {exc}"[:200]
        _lib.check(lib.onebit_check_device_status())

    identical = bit_identity(ob, _lib, oracle, layer, S, world, rank, dev, reduce_minmax)
    _lib.check(lib.onebit_check_device_status())
    sync_all()

    # the 8192^3 GEMM on rank 0 alone (the burst-clock figure earlier records carry)
    square = None
    if rank == 0 and not args.no_square8192 and S != 8192:
        del B, C
        torch.cuda.empty_cache()
        q = 8192
        w8, s8 = gpu_weights(q, q, 3080, dev)
        pw8 = ob.pack_weight(w8, scale=s8, apply_mask=False, keep_reference=False)
        del w8
        B8 = torch.randn((q, q), device=dev, dtype=torch.float32).to(torch.float16)
        C8 = torch.empty((q, q), dtype=torch.float16, device=dev)
        for _ in range(5):
            ob.matmul_packed(pw8, B8, out=C8)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            ob.matmul_packed(pw8, B8, out=C8)
        e1.record()
        torch.cuda.synchronize()
        ms8 = e0.elapsed_time(e1) / 20
        peaks = load_peaks()
        square = {"ms": ms8, "tflops": 2.0 * q ** 3 / (ms8 * 1e-3) / 1e12, "steps": 20,
                  "frac_of_2x_burst_peak": 2.0 * q ** 3 / (ms8 * 1e-3) / 1e12 / (2 * peaks["bf16_tflops"]),
                  "traffic": MEASURED_TRAFFIC.get(q), "note": "8.4 ms of work: burst clocks"}
        del pw8, B8, C8

    decode = decode_loop = context = None
    if rank == 0 and world == 1 and not args.no_decode:
        decode = decode_extras(ob, _lib, dev)
        decode_loop = decode_loop_extras(ob, dev)
        context = context_baselines(dev, sorted({8192, S}))
    sync_all()

    if rank == 0:
        peaks = load_peaks()
        timed_s = total_ms * 1e-3
        # a kernel timed inside a long step runs at the sustained clocks of a power-capped part
        sustained = timed_s >= 0.1
        dense_peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
        sparse_peak = 2.0 * dense_peak
        achieved = 2.0 * rows * S * S / (kernel_ms * 1e-3) / 1e12
        cpu_rows = max(64, min(S, int(1e12 / (2.0 * S * S)) // 64 * 64))       # about 1e12 flop: some 10 s of host work
        cpu = CpuSample(S, cpu_rows)
        cpu_v, cpu_dt = cpu.step()
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong",
            # the reference README publishes this size on an RTX 3060 Ti; value is the whole job on n_gpus B200s
            "vs_baseline": (value / PUBLISHED[S]) if S in PUBLISHED else None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload_name(S, world), "rows_per_rank": [r for _, r in layer.partition],
                       "l2": "inputs larger than L2 (B and C are 2*S*S bytes)", "pack_ms_rank0": pack_ms},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "ms_per_step": e2e_ms,
                    "note": "ShardedBinaryLinear.forward_host: tokens from pinned host memory, the rank's slab of the result to "
                            "pinned host memory, weights resident. One rank: onebit_matmul_packed_host (copies overlapped with "
                            "the GEMM in column panels). Several ranks: per column panel each rank uploads 1/N of the tokens, an NCCL "
                            "all-gather over NVLink completes the panel, and the panel of the result leaves while the next "
                            "panels travel and multiply. Bytes are summed over the ranks"},
            "gpu_launches": args.steps * world,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": sparse_peak, "unit": "TFLOP/s",
                         "frac": achieved / sparse_peak, "traffic": MEASURED_TRAFFIC.get(S) if world == 1 else None,
                         "peak_note": f"2 x dense bf16 {'sustained' if sustained else 'burst'} peak ({dense_peak} TFLOP/s, "
                                      f"{peaks['source']}): 2:4 sparse MMA rate; the timed region lasts {timed_s:.2f} s",
                         "frac_of_2x_burst": achieved / (2.0 * peaks["bf16_tflops"]),
                         "frac_of_2x_sustained": achieved / (2.0 * peaks["bf16_tflops_sustained"]),
                         "kernel": "ob_gemm_prefill2_kernel<2> (CTA pair), rank 0's launch", "kernel_ms": kernel_ms,
                         "flop_per_launch": 2.0 * rows * S * S},
            "cpu_baseline": {"value": cpu_v, "unit": "TFLOP/s", "cores": cpu.cores, "kind": "port",
                             "sample": f"{cpu_rows} of {S} weight rows x full k x full n ({cpu_dt:.2f} s)"},
            "clocks": clocks.summary(total_ms / args.steps),
            "sharded_bit_identical": identical["all"], "bit_identity_checks": identical,
        }
        if world > 1:
            line["gather_nccl_ms"] = gathers.get("all")
            line["gather_fused_ms"] = gathers.get("fused")
            line["fused_backend"] = layer.fused_backend
        if square is not None:
            line["square8192"] = square
        if decode is not None:
            line["decode"] = decode
        if decode_loop is not None:
            line["decode_loop"] = decode_loop
        if context is not None:
            line["context"] = context
        emit_line(line)
    if world > 1:
        dist.destroy_process_group()


_LINE_OUT = None


def claim_stdout():
    """Keeps the process's standard output for the one JSON line: whatever else writes to file descriptor 1 from here
    on (a library's banner, e.g. NCCL's version line when NCCL_DEBUG is set; a stray print) goes to standard error."""
    global _LINE_OUT
    sys.stdout.flush()
    _LINE_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def emit_line(line):
    out = _LINE_OUT or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", type=int, default=25600, help="a_rows = n = a_cols of the one GEMM (a multiple of 256)")
    ap.add_argument("--no-decode", action="store_true", help="skip the supplementary decode-regime numbers")
    ap.add_argument("--no-square8192", action="store_true", help="skip the supplementary 8192^3 figure")
    args = ap.parse_args()
    claim_stdout()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
