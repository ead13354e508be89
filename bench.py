#!/usr/bin/env python
"""Benchmark of the MLX Q4 decode projection set on B200 (and its CPU reference arm).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one token's pass over one layer's Q4 g64 projections at batch 1,
hidden 4096: fused q/k/v 4096->6144, o_proj 4096->4096, fused gate/up + SiLU
4096->2x12288 (bf16 mid), down 12288->4096 - one operator call per projection,
through the C ABI of libtessl_b200.so. Weights are seeded synthetic banks
(uniform nibbles, bf16 scale ~U(0.002, 0.02), bias = -8*scale + N(0, 0.001)); the
step rotates over several layers' banks so the weight stream never fits L2.

Printed: ONE JSON line. `value` is effective weight bandwidth (algorithmic
weight bytes of the step / device time) with everything resident in HBM;
`e2e` is the same measured by a compiled C++ host over the C ABI
(tessl_b200/csrc/host_step_driver.cpp) with the activations copied from pinned
host memory and the result read back every step (encode-only mode; the
every-call-synchronous figure and the Python-ctypes figures beside it);
`roofline` describes the dominant kernel, `roofline_prefill` the prefill GEMM;
`cpu_baseline` times the CPU oracle on the same workload; `parity` is the GPU
step's result against the CPU arm's on the same banks (layer 0 of the GPU arm
is the CPU arm's layer). `extra` adds the LM head, small-batch, Q8 and prefill
configurations. `clocks` are nvidia-smi samples taken while the timed graph
keeps replaying for half a second after the timed replay (the timed region is
shorter than one sampling period).

With --gpus N > 1 (launched by torchrun, one rank per GPU) the large outputs
(gate/up) are column-sharded over the ranks and the GEMV kernel itself stores
each finished output into every rank's gather buffer over NVLink peer memory
(an NCCL all-gather if peer memory is unavailable); q/k/v, o_proj and down are
small and run replicated (the row-sharded down variant is timed beside it).
`parity_n` says that every rank's gathered results equal the single-GPU
operators' on the unsharded banks bit for bit. Total work is fixed: "strong".
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, QKV, INTER, GROUP = 4096, 6144, 12288, 64
TRAFFIC_RATIO = 1.0014  # ncu dram__bytes_read.sum + write.sum over algorithmic bytes, q4_gemv_mma_kernel at 12288 x 4096
METRIC = "Q4 GEMV effective weight GB/s"


def q4_weight_bytes(rows: int, cols: int, group: int = GROUP) -> int:
    """Algorithmic bytes of a bank: packed nibbles + one bf16 (scale, bias) pair per group."""
    return rows * cols // 2 + rows * (cols // group) * 4


STEP_WEIGHT_BYTES = (q4_weight_bytes(QKV, HIDDEN) + q4_weight_bytes(HIDDEN, HIDDEN)
                     + 2 * q4_weight_bytes(INTER, HIDDEN) + q4_weight_bytes(HIDDEN, INTER))


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs. The GPU is named by
    its UUID (an index would be wrong under CUDA_VISIBLE_DEVICES); `summary()` says so when no sample
    could be taken."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, torch, device: int, enabled: bool = True):
        self.rows, self.proc, self.enabled, self.why = [], None, enabled, ""
        self.gpu = str(device)
        try:
            self.gpu = "GPU-" + str(torch.cuda.get_device_properties(device).uuid)
        except Exception as e:  # noqa: BLE001
            self.why = f"no UUID for device {device} ({type(e).__name__}); sampled by index"

    def __enter__(self):
        if not self.enabled:
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", self.gpu], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError as e:
            self.proc, self.why = None, f"nvidia-smi did not start ({e})"
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])), mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"unavailable": self.why or f"nvidia-smi returned no sample for {self.gpu}", "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "gpu": self.gpu}


# --------------------------------------------------------------- CPU arm ---

CPU_SEED = 0x7E550100  # the layer both arms share: the CPU arm's only layer, the GPU arm's layer 0


def host_threads() -> int:
    """Host cores this process may run on. Stated explicitly to the oracle: a launcher that sets
    OMP_NUM_THREADS=1 for its ranks (torchrun does) would otherwise shrink the CPU arm to one thread."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_step_inputs(seed: int):
    """One layer's banks and activations as numpy arrays (seeded splitmix64)."""
    from tessl_b200 import synth
    shapes = {"qkv": (QKV, HIDDEN), "o": (HIDDEN, HIDDEN), "gate": (INTER, HIDDEN), "up": (INTER, HIDDEN),
              "down": (HIDDEN, INTER)}
    banks = {}
    for i, (name, (r, c)) in enumerate(shapes.items()):
        p, sb = synth.q4_bank(seed + 16 * i, r, c, GROUP)
        banks[name] = (p.view(np.uint8).reshape(-1), sb.reshape(-1), r, c)
    xs = {n: synth.normal_bf16(seed + 1000 + i, HIDDEN) for i, n in enumerate(("x_qkv", "x_o", "x_mlp"))}
    return banks, xs


def cpu_step(banks, xs, threads: int, rows_fraction: float = 1.0):
    """The decode projection set on the CPU oracle (f64-accumulated dequant-matvec).
    `rows_fraction` < 1 runs the leading share of each projection's rows (a bounded sample)."""
    from oracle import api
    from tessl_b200 import synth

    def mv(name, x):
        p, sb, r, c = banks[name]
        rr = max(8, int(r * rows_fraction)) if rows_fraction < 1.0 else r
        return api.q4_dense_gemm(p[: rr * c // 2], sb[: rr * (c // GROUP) * 2], x, 1, rr, c, GROUP, threads)[0], rr

    done = 0
    _, rr = mv("qkv", xs["x_qkv"]); done += q4_weight_bytes(rr, HIDDEN)
    _, rr = mv("o", xs["x_o"]); done += q4_weight_bytes(rr, HIDDEN)
    g, rr = mv("gate", xs["x_mlp"])
    u, _ = mv("up", xs["x_mlp"]); done += 2 * q4_weight_bytes(rr, HIDDEN)
    gd = g.astype(np.float64)
    mid = (gd / (1.0 + np.exp(-gd)) * u).astype(np.float32)
    mid_full = np.zeros(INTER, np.float32)
    mid_full[: mid.size] = mid
    y, rr = mv("down", synth.f32_to_bf16_bits(mid_full)); done += q4_weight_bytes(rr, INTER)
    return y, done


def run_reference_arm(args, rank: int):
    """`--impl reference`: the reference's own algorithm for this path on the host
    cores. The reference is a Metal/Rust crate that cannot be built or run here,
    so this is the CPU oracle port (oracle/tessl_oracle.c) with every host thread."""
    if rank != 0:
        return
    threads = host_threads()
    banks, xs = cpu_step_inputs(CPU_SEED)
    frac = 0.25  # a bounded sample: the leading quarter of every projection's rows
    for _ in range(max(1, args.warmup)):
        cpu_step(banks, xs, threads, frac)
    t0 = time.perf_counter()
    done = 0
    for _ in range(args.steps):
        _, b = cpu_step(banks, xs, threads, frac)
        done += b
    dt = time.perf_counter() - t0
    gbs = done / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f64 accumulate over bf16 x / Q4 weights", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"leading {frac:.0%} of the rows of each projection, {args.steps} steps"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int, layers: int = 4):
    return {
        "workload": "qwen3.5-style decode projection set, Q4 g64, M=1, hidden 4096: qkv 4096->6144, o 4096->4096, "
                    "gate+up+SiLU 4096->2x12288, down 12288->4096",
        "calls_per_step": 4, "weight_bytes_per_step": STEP_WEIGHT_BYTES,
        "l2": f"weights rotate over {layers} layers' banks ({layers * STEP_WEIGHT_BYTES / 1e6:.0f} MB > 126 MB L2), "
              "one layer per step",
        "parallelism": "single GPU" if n_gpus == 1 else
        f"gate/up column-sharded over {n_gpus} GPUs with one all-gather of the bf16 outputs per step over NVLink (see gather); qkv, o, down replicated",
    }


# --------------------------------------------------------------- GPU arm ---

class Layer:
    """One layer's banks on this rank's GPU: every bank unsharded, plus this rank's row slices of the
    banks the workload shards (gate, up; down for the sharded-down variant)."""

    def __init__(self, torch, nn, sharded, seed: int, world: int, rank: int, host_banks=None):
        """`host_banks` (cpu_step_inputs' dict) makes this layer the very banks the CPU arm runs on;
        without it the banks are drawn on the device (same distributions, all 32 bits of every word)."""
        self.keep = []
        gen = torch.Generator(device="cuda")
        gen.manual_seed(seed)
        names = iter(("qkv", "o", "gate", "up", "down"))
        B = nn.GpuBuffer.from_torch

        def bank(rows, cols):
            if host_banks is not None:
                p, sb, r, c = host_banks[next(names)]
                assert (r, c) == (rows, cols)
                packed = torch.from_numpy(p.view(np.int32).reshape(rows, cols // 8)).cuda()
                return packed, torch.from_numpy(sb.view(np.int16).reshape(rows, cols // GROUP, 2)).cuda().view(torch.bfloat16)
            return device_bank(torch, gen, rows, cols)

        def take(rows, cols, shard_it, keep_full):
            packed, sb = bank(rows, cols)
            sh = sharded.make_shard(rows, world if shard_it else 1, rank if shard_it else 0)
            full = None
            if not (shard_it and world > 1) or keep_full:
                self.keep += [packed, sb]
                full = nn.Q4MlxBank(B(packed), B(sb))
            local = full
            if shard_it and world > 1:
                lp, lsb = sharded.slice_bank(packed, sb, sh)
                self.keep += [lp, lsb]
                local = nn.Q4MlxBank(B(lp), B(lsb))
            return full, local, sh

        check = host_banks is not None  # the layer the N-GPU parity check runs on keeps its unsharded banks
        self.qkv, _, _ = take(QKV, HIDDEN, False, True)
        self.o, _, _ = take(HIDDEN, HIDDEN, False, True)
        self.gate_full, self.gate, self.sh_mid = take(INTER, HIDDEN, True, check)
        self.up_full, self.up, _ = take(INTER, HIDDEN, True, check)
        # down (4096 output rows) runs replicated in the timed step; its row slice serves the
        # sharded-down variant that is timed beside it
        self.down, self.down_local, self.sh_down = take(HIDDEN, INTER, True, True)


def device_bank(torch, gen, rows, cols):
    """A bank drawn on the device: every bit of every packed word random, scale ~U(0.002, 0.02),
    bias = -8 * scale + N(0, 0.001)."""
    packed = torch.randint(0, 2**31 - 1, (rows, cols // 8), dtype=torch.int32, device="cuda", generator=gen)
    packed = packed * 2 + torch.randint(0, 2, packed.shape, dtype=torch.int32, device="cuda", generator=gen)
    sc = (torch.rand((rows, cols // GROUP), device="cuda", generator=gen) * 0.018 + 0.002).to(torch.bfloat16)
    bi = (-8.0 * sc.float() + 0.001 * torch.randn(sc.shape, device="cuda", generator=gen)).to(torch.bfloat16)
    return packed, torch.stack([sc, bi], dim=-1).contiguous()


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist

    from tessl_b200 import build as tb
    from tessl_b200 import nn, sharded

    tb.build()
    torch.cuda.set_device(local_rank)
    rt = nn.Runtime(local_rank)
    st = torch.cuda.ExternalStream(rt.stream, device=local_rank)
    peaks = load_peaks()
    n_layers = 4
    # Layer 0 is the CPU arm's layer (same seeds, same generator); the others only have to keep the
    # weight stream out of L2 and are drawn on the device.
    cpu_inputs = cpu_step_inputs(CPU_SEED)
    layers = [Layer(torch, nn, sharded, 0x7E550000 + 97 * i, world, rank, cpu_inputs[0] if i == 0 else None)
              for i in range(n_layers)]
    dev = torch.device("cuda", local_rank)
    acts = {n: torch.from_numpy(v.view(np.int16)).to(dev).view(torch.bfloat16) for n, v in cpu_inputs[1].items()}
    qkv_out = torch.empty(QKV, device=dev)
    o_out = torch.empty(HIDDEN, device=dev)
    # N > 1: gate/up run on this rank's rows and the kernel itself stores every finished output into
    # all ranks' gather buffers over NVLink (tessl_gemv_q4_mlx_gate_up_silu_sharded); NCCL is the
    # fallback if the peer-mapped allocation is unavailable.
    peer = peer_y = None
    if world > 1:
        why = ""
        try:
            peer = sharded.PeerGather(layers[0].sh_mid.local_rows * 2)
            peer_y = sharded.PeerGather(sharded.slice_rows_per_rank(HIDDEN, world) * 4)
            probe = nn.Runtime(local_rank)  # a trial exchange on a runtime of its own: a failure poisons only that one
            try:
                for _ in range(3):
                    peer.run(probe)
            finally:
                probe.close()
        except Exception as e:  # noqa: BLE001
            peer, why = None, f"{type(e).__name__}: {e}"
        agreed = torch.tensor([1 if peer is not None else 0], device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:
            peer = peer_y = None
            if rank == 0:
                print(f"bench: peer-memory gather unavailable ({why or 'on another rank'}); using NCCL", file=sys.stderr)
    if peer is not None:
        mid_local, mid_full = peer.local(torch.bfloat16), peer.full(torch.bfloat16)
    else:
        mid_local = torch.empty(layers[0].sh_mid.local_rows, device=dev, dtype=torch.bfloat16)
        mid_full = torch.empty(INTER, device=dev, dtype=torch.bfloat16) if world > 1 else mid_local
    y = torch.empty(HIDDEN, device=dev)
    B = nn.GpuBuffer.from_torch
    bufs = {k: B(v) for k, v in acts.items()}
    qkv_b, o_b, midl_b, midf_b, y_b = B(qkv_out), B(o_out), B(mid_local), B(mid_full), B(y)
    sq = nn.QuantShape(QKV, HIDDEN, GROUP)
    so = nn.QuantShape(HIDDEN, HIDDEN, GROUP)
    sg = nn.QuantShape(layers[0].sh_mid.local_rows, HIDDEN, GROUP)
    sd = nn.QuantShape(HIDDEN, INTER, GROUP)
    sd_local = nn.QuantShape(layers[0].sh_down.local_rows, INTER, GROUP)
    launches_per_step = 4  # N > 1 with peer memory: still four, the exchange is inside the gate/up kernel

    # The offline repack (B200 staged layout) of the three launches it serves, for the variant timed beside the
    # headline (one GPU): q/k/v, o and gate/up repacked, down (rows of 12288 columns) row-major.
    # Built after the headline has been timed, so that nothing about the headline depends on it.
    staged_banks = None

    def step(i: int, down_sharded: bool = False, staged: bool = False):
        L = layers[i % n_layers]
        if staged:
            S = staged_banks[i % n_layers]
            nn.gemv_q4_mlx_simd(rt, S["qkv"], bufs["x_qkv"], qkv_b, sq, layout=nn.B200_STAGED)
            nn.gemv_q4_mlx_simd(rt, S["o"], bufs["x_o"], o_b, so, layout=nn.B200_STAGED)
            nn.gemv_q4_mlx_gate_up_silu(rt, S["gate"], S["up"], bufs["x_mlp"], midl_b, sg, True, layout=nn.B200_STAGED)
            nn.gemv_q4_mlx_simd(rt, L.down, midf_b, y_b, sd)
            return y
        nn.gemv_q4_mlx_simd(rt, L.qkv, bufs["x_qkv"], qkv_b, sq)
        nn.gemv_q4_mlx_simd(rt, L.o, bufs["x_o"], o_b, so)
        if peer is not None:
            peer.gate_up_silu(rt, L.gate, L.up, bufs["x_mlp"], sg, True)
        else:
            nn.gemv_q4_mlx_gate_up_silu(rt, L.gate, L.up, bufs["x_mlp"], midl_b, sg, True)
            if world > 1:
                with torch.cuda.stream(st):
                    sharded.all_gather_rows(mid_local, L.sh_mid, out=mid_full)
        if down_sharded and peer_y is not None:
            # K = 12288 is outside the exchanging kernel's widths: the library runs the slice's GEMV and then
            # the stand-alone exchange (two launches)
            peer_y.gemv(rt, L.down_local, midf_b, sd_local)
            return peer_y.full(torch.float32)
        nn.gemv_q4_mlx_simd(rt, L.down, midf_b, y_b, sd)
        return y

    def barrier():
        rt.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    rt.set_encode_only(True)
    for i in range(max(args.warmup, 3)):
        step(i)
        if peer_y is not None:
            step(i, True)
    barrier()

    def timed_graph(down_sharded: bool, sample_clocks: bool, staged: bool = False):
        # Launch-bound inner loop: one CUDA graph holds all K steps (kernels and, on the NCCL
        # fallback, the all-gathers, captured on the runtime's stream).
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            for i in range(args.steps):
                step(i, down_sharded, staged)
        with torch.cuda.stream(st):
            graph.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(torch, local_rank, enabled=sample_clocks) as clocks:
            barrier()
            # The profiler range lets `ncu --profile-from-start off` list exactly the launches of the headline's
            # timed region (the variants timed beside it open none).
            if sample_clocks:
                torch.cuda.profiler.start()
            with torch.cuda.stream(st):
                e0.record(st)
                graph.replay()
                e1.record(st)
            barrier()
            if sample_clocks:
                torch.cuda.profiler.stop()
            ms = e0.elapsed_time(e1)
            if world > 1:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            if sample_clocks:
                # The timed region lasts a few milliseconds, less than one sampling period of nvidia-smi: the
                # same graph keeps replaying (untimed, the same count on every rank) for about half a second
                # so that the clock samples are taken under this very load.
                with torch.cuda.stream(st):
                    for _ in range(min(5000, int(500.0 / max(ms, 1e-3)) + 1)):
                        graph.replay()
                barrier()
        return ms / args.steps, clocks.summary()

    ms_per_step, clocks = timed_graph(False, True)
    value = STEP_WEIGHT_BYTES / (ms_per_step * 1e-3) / 1e9
    variants = None
    if peer_y is not None:
        ms_sharded_down, _ = timed_graph(True, False)
        variants = {"down replicated (the timed step)": round(ms_per_step * 1e3, 3),
                    "down row-sharded + exchange of its f32 outputs": round(ms_sharded_down * 1e3, 3), "unit": "us per step"}

    staged_variant = None
    if world == 1:
        rt.set_encode_only(False)
        sgu = nn.QuantShape(INTER, HIDDEN, GROUP)
        staged_banks = [{"qkv": nn.q4_mlx_repack_staged(rt, L.qkv, sq), "o": nn.q4_mlx_repack_staged(rt, L.o, so),
                         "gate": nn.q4_mlx_repack_staged(rt, L.gate, sgu), "up": nn.q4_mlx_repack_staged(rt, L.up, sgu)}
                        for L in layers]
        rt.set_encode_only(True)
        for i in range(max(args.warmup, 3)):
            step(i, False, True)
        barrier()
        ms_staged, _ = timed_graph(False, False, True)
        staged_variant = {"ms_per_step": round(ms_staged, 5), "value": round(STEP_WEIGHT_BYTES / (ms_staged * 1e-3) / 1e9, 1),
                          "unit": "GB/s", "frac_of_measured_hbm": round(STEP_WEIGHT_BYTES / (ms_staged * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                          "what": "the same step with the q/k/v, o, gate and up banks repacked offline into the B200 staged "
                                  "layout (tessl_q4_mlx_repack_staged: two bulk copies per stage, +0.7 % bytes); down row-major; "
                                  "results bit-identical to the headline step's (checked below)"}

    # ---- parity, outside the timed region ----
    rt.set_encode_only(False)
    if staged_banks is not None:
        y_rm = step(0).clone()
        y_st = step(0, False, True).clone()
        if not torch.equal(y_rm.view(torch.int32), y_st.view(torch.int32)):
            raise SystemExit("bench: the step on staged banks differs from the step on row-major banks")
        staged_variant["parity_vs_row_major"] = "bit-exact"
    parity = check_parity(torch, dist, nn, rt, layers[0], cpu_inputs, step, bufs, mid_full, world, rank,
                          peer_y is not None, dev)
    rt.set_encode_only(True)

    # ---- per-projection device times (one graph per projection, same rotation) ----
    per_kernel = {}
    if world == 1:
        def time_graph(fn, iters):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for i in range(iters):
                    fn(i)
            best = 1e30
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(st):
                for rep in range(6):
                    a.record(st)
                    g.replay()
                    b.record(st)
                    b.synchronize()
                    if rep:
                        best = min(best, a.elapsed_time(b) / iters)
            return best * 1e3  # us per launch

        iters = max(16, min(args.steps, 200))
        gate_f32 = torch.empty(INTER, device=dev)
        gate_f32_b = B(gate_f32)
        shapes = {
            "qkv 6144x4096": (lambda i: nn.gemv_q4_mlx_simd(rt, layers[i % n_layers].qkv, bufs["x_qkv"], qkv_b, sq),
                              q4_weight_bytes(QKV, HIDDEN)),
            "o 4096x4096": (lambda i: nn.gemv_q4_mlx_simd(rt, layers[i % n_layers].o, bufs["x_o"], o_b, so),
                            q4_weight_bytes(HIDDEN, HIDDEN)),
            "gate_up_silu 2x12288x4096": (lambda i: nn.gemv_q4_mlx_gate_up_silu(
                rt, layers[i % n_layers].gate, layers[i % n_layers].up, bufs["x_mlp"], midl_b, sg, True),
                2 * q4_weight_bytes(INTER, HIDDEN)),
            "down 4096x12288": (lambda i: nn.gemv_q4_mlx_simd(rt, layers[i % n_layers].down, midf_b, y_b, sd),
                                q4_weight_bytes(HIDDEN, INTER)),
            "gemv 12288x4096 (target shape)": (lambda i: nn.gemv_q4_mlx_simd(
                rt, layers[i % n_layers].gate, bufs["x_mlp"], gate_f32_b, nn.QuantShape(INTER, HIDDEN, GROUP)),
                q4_weight_bytes(INTER, HIDDEN)),
        }
        for name, (fn, nbytes) in shapes.items():
            us = time_graph(fn, iters)
            per_kernel[name] = {"us": round(us, 3), "weight_gbs": round(nbytes / us / 1e3, 1),
                                "frac_of_measured_hbm": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 4)}
        SB = lambda i: staged_banks[i % n_layers]
        staged_shapes = {
            "qkv 6144x4096": (lambda i: nn.gemv_q4_mlx_simd(rt, SB(i)["qkv"], bufs["x_qkv"], qkv_b, sq, layout=nn.B200_STAGED),
                              q4_weight_bytes(QKV, HIDDEN)),
            "o 4096x4096": (lambda i: nn.gemv_q4_mlx_simd(rt, SB(i)["o"], bufs["x_o"], o_b, so, layout=nn.B200_STAGED),
                            q4_weight_bytes(HIDDEN, HIDDEN)),
            "gate_up_silu 2x12288x4096": (lambda i: nn.gemv_q4_mlx_gate_up_silu(
                rt, SB(i)["gate"], SB(i)["up"], bufs["x_mlp"], midl_b, sg, True, layout=nn.B200_STAGED),
                2 * q4_weight_bytes(INTER, HIDDEN)),
            "gemv 12288x4096 (target shape)": (lambda i: nn.gemv_q4_mlx_simd(
                rt, SB(i)["gate"], bufs["x_mlp"], gate_f32_b, nn.QuantShape(INTER, HIDDEN, GROUP), layout=nn.B200_STAGED),
                q4_weight_bytes(INTER, HIDDEN)),
        }
        staged_variant["per_kernel"] = {}
        for name, (fn, nbytes) in staged_shapes.items():
            us = time_graph(fn, iters)
            staged_variant["per_kernel"][name] = {"us": round(us, 3), "weight_gbs": round(nbytes / us / 1e3, 1),
                                                  "frac_of_measured_hbm": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 4)}
    rt.set_encode_only(False)
    return dict(torch=torch, dist=dist, nn=nn, rt=rt, st=st, layers=layers, acts=acts, step=step, ms_per_step=ms_per_step,
                value=value, clocks=clocks, per_kernel=per_kernel, peaks=peaks, dev=dev,
                launches_per_step=launches_per_step, n_layers=n_layers, parity=parity, variants=variants,
                staged_variant=staged_variant,
                y=y, bufs=bufs, cpu_inputs=cpu_inputs,
                gather="peer memory, stores issued by the GEMV kernel (tessl_gemv_q4_mlx_gate_up_silu_sharded)"
                if peer is not None else "nccl")


def check_parity(torch, dist, nn, rt, L0, cpu_inputs, step, bufs, mid_full, world, rank, has_sharded_down, dev):
    """Layer 0, outside the timed region. (1) The GPU step's y against the CPU arm's y on the same banks and
    activations, within the stated tolerance (1e-2 relative + 2e-3 absolute after bf16 rounding of both).
    (2) N > 1: on every rank the gathered gate/up output and y, in both down variants, against the single-GPU
    operators on the unsharded banks, bit for bit (a row's summation order does not depend on the slice)."""
    from tessl_b200 import synth
    B = nn.GpuBuffer.from_torch
    y_gpu = step(0).clone()
    mid_gpu = mid_full.clone()
    y_cpu, _ = cpu_step(cpu_inputs[0], cpu_inputs[1], host_threads(), 1.0)
    rnd = lambda a: synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(np.asarray(a, np.float32))).astype(np.float64)
    g, w = rnd(y_gpu.cpu().numpy()), rnd(y_cpu)
    err = np.abs(g - w)
    bad = int(np.count_nonzero(err > 2e-3 + 1e-2 * np.abs(w)))
    out = {"gpu_vs_cpu_y": "ok" if bad == 0 else f"{bad} of {w.size} outputs outside 1e-2 rel + 2e-3 abs",
           "max_abs_err": float(err.max()), "layer": "layer 0: the CPU arm's banks and activations (tessl_b200/synth.py seeds)"}
    if bad:
        raise SystemExit(f"bench: the GPU step disagrees with the CPU arm: {out}")
    if world > 1:
        mid_ref = torch.empty(INTER, device=dev, dtype=torch.bfloat16)
        y_ref = torch.empty(HIDDEN, device=dev)
        nn.gemv_q4_mlx_gate_up_silu(rt, L0.gate_full, L0.up_full, bufs["x_mlp"], B(mid_ref), nn.QuantShape(INTER, HIDDEN, GROUP), True)
        nn.gemv_q4_mlx_simd(rt, L0.down, B(mid_ref), B(y_ref), nn.QuantShape(HIDDEN, INTER, GROUP))
        same = bool(torch.equal(mid_gpu.view(torch.int16)[:INTER], mid_ref.view(torch.int16))) and \
            bool(torch.equal(y_gpu.view(torch.int32), y_ref.view(torch.int32)))
        if has_sharded_down:
            y2 = step(0, True).clone()
            same = same and bool(torch.equal(y2.view(torch.int32)[:HIDDEN], y_ref.view(torch.int32)))
        t = torch.tensor([1 if same else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        out["parity_n"] = "ok" if int(t.item()) == 1 else "MISMATCH"
        out["parity_n_what"] = ("gathered gate/up output and y" + (" (down replicated and down sharded)" if has_sharded_down else "")
                                + f" on each of {world} ranks == single-GPU operators on the unsharded banks, bit for bit")
        if out["parity_n"] != "ok":
            raise SystemExit(f"bench: rank {rank}: sharded results differ from the single-GPU operators")
    return out


def measure_sharded_lm_head(ctx, args, world, rank):
    """N > 1 only: the LM head (151936 x 4096, Q4 g64) at M = 1 and M = 8, rows sharded over the ranks; every
    rank streams its slice; at M = 1 the GEMV kernel itself stores the bf16 logits into all ranks' gather
    buffers, at M = 8 the stand-alone exchange follows the small-batch GEMM (NCCL all-gather on the fallback).
    Device time of the slowest rank, whole-job weight bytes per second. The launches rotate over enough
    different slices that the stream exceeds L2 at every N; the first slice's gathered logits are compared on
    every rank, bit for bit, with the single-GPU operator on the unsharded bank (a mismatch ends the run)."""
    torch, dist, nn, rt, st = ctx["torch"], ctx["dist"], ctx["nn"], ctx["rt"], ctx["st"]
    from tessl_b200 import sharded
    rows, cols = 151936, HIDDEN
    sh = sharded.make_shard(rows, world, rank)
    per = sharded.slice_rows_per_rank(rows, world)
    slice_bytes = q4_weight_bytes(per, cols)
    nslices = max(2, -(-int(1.3 * 126e6) // slice_bytes))  # the rotation holds > 1.3 x L2
    B = nn.GpuBuffer.from_torch
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0x7E55AA)  # the same on every rank: each draws the whole bank and keeps its rows
    banks, keep, full0 = [], [], None
    for i in range(nslices):
        packed, sb = device_bank(torch, gen, rows, cols)
        lp, lsb = sharded.slice_bank(packed, sb, sh)
        keep += [lp, lsb]
        banks.append(nn.Q4MlxBank(B(lp), B(lsb)))
        if i == 0:
            keep += [packed, sb]
            full0 = nn.Q4MlxBank(B(packed), B(sb))
        del packed, sb
    x1 = ctx["bufs"]["x_mlp"]
    use_peer = ctx.get("gather", "nccl") != "nccl"
    shape = nn.QuantShape(sh.local_rows, cols, GROUP)
    nbytes = q4_weight_bytes(rows, cols)
    out = {}
    for m in (1, 8):
        # m = 1: the exchanging GEMV (one launch). m = 8: the small-batch GEMM on the slice, its [8, rows / N] bf16
        # block written into this rank's part of the gather buffer, then the stand-alone exchange (two launches).
        peer = None
        if use_peer:
            try:
                peer = sharded.PeerGather(-(-per * m * 2 // 16) * 16)
            except Exception:  # noqa: BLE001
                peer = None
            agreed = torch.tensor([1 if peer is not None else 0], device=ctx["dev"])
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)  # all ranks take the same exchange
            if int(agreed.item()) == 0:
                peer = None
        if m == 1:
            x, xb = None, x1
        else:
            xgen = torch.Generator(device="cuda")
            xgen.manual_seed(0x7E55AB)
            x = torch.randn(m * cols, device=ctx["dev"], generator=xgen).to(torch.bfloat16)
            xb = B(x)
        if peer is not None:
            y_full = peer.full(torch.bfloat16)
            slot = peer.bytes_per_rank // 2
            yl_b = B(peer.local(torch.bfloat16))
        else:
            y_local = torch.zeros(per * m, device=ctx["dev"], dtype=torch.bfloat16)
            y_full = torch.empty(per * m * world, device=ctx["dev"], dtype=torch.bfloat16)
            yl_b = B(y_local)
            slot = per * m
        # many calls per replay: the ranks leave the barrier before a replay tens of microseconds apart, and the
        # first call of a replay waits for the last rank to arrive
        iters = (16 if m == 1 else 8) * nslices

        def call(i):
            bank = banks[i % nslices]
            if m == 1 and peer is not None:
                peer.gemv(rt, bank, xb, shape, y_as_bf16=True)
                return
            if m == 1:
                nn.gemv_q4_mlx_simd(rt, bank, xb, yl_b, shape, y_as_bf16=True)
            else:
                nn.gemm_q4_mlx(rt, bank, xb, yl_b, shape, m, y_as_bf16=True)
            if peer is not None:
                peer.run(rt)
            else:
                with torch.cuda.stream(st):
                    dist.all_gather_into_tensor(y_full, y_local)

        # parity first: slice 0 against the unsharded bank
        call(0)
        rt.synchronize()
        torch.cuda.synchronize()
        want = torch.empty(m * rows, device=ctx["dev"], dtype=torch.bfloat16)
        if m == 1:
            nn.gemv_q4_mlx_simd(rt, full0, xb, B(want), nn.QuantShape(rows, cols, GROUP), y_as_bf16=True)
        else:
            nn.gemm_q4_mlx(rt, full0, xb, B(want), nn.QuantShape(rows, cols, GROUP), m, y_as_bf16=True)
        # rank r's block is [m, its rows]: the gathered result is the single-GPU [m, rows] cut by columns
        got = torch.cat([y_full.view(world, slot)[r, : m * lr].view(m, lr)
                         for r in range(world) for lr in [sharded.make_shard(rows, world, r).local_rows]], dim=1)
        t = torch.tensor([1 if torch.equal(got.reshape(-1).view(torch.int16), want.view(torch.int16)) else 0],
                         device=ctx["dev"])
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        if int(t.item()) != 1:
            raise SystemExit(f"bench: rank {rank}: sharded LM-head logits (m = {m}) differ from the single-GPU operator")
        del want

        rt.set_encode_only(True)
        for i in range(3):
            call(i)
        rt.synchronize()
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for i in range(iters):
                call(i)
        best = 1e30
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for rep in range(4):
            dist.barrier()
            with torch.cuda.stream(st):
                a.record(st)
                g.replay()
                b.record(st)
            b.synchronize()
            if rep:
                best = min(best, a.elapsed_time(b) / iters)
        rt.set_encode_only(False)
        t = torch.tensor([best], device=ctx["dev"])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item()) * 1e3
        if m == 1:
            how = "one launch per call: GEMV on this rank's row slice" + (
                ", its reducer warps storing the bf16 logits into every rank's gather buffer over NVLink, one flag "
                "exchange at the end" if peer is not None else " + one NCCL all-gather of the bf16 logits")
        else:
            how = "two launches per call: the small-batch GEMM on this rank's row slice, then " + (
                "the stand-alone peer-memory exchange of its [8, rows / N] bf16 block" if peer is not None
                else "one NCCL all-gather of its [8, rows / N] bf16 block")
        out[f"lm_head 151936x4096 m={m} sharded over {world} GPUs"] = {
            "us": round(us, 2), "weight_gbs": round(nbytes / us / 1e3, 1), "rows_per_gpu": int(sh.local_rows),
            "slices_in_rotation": nslices, "rotation_mb_per_gpu": round(nslices * slice_bytes / 1e6, 1),
            "parity_n": "ok", "how": how + "; all calls in one CUDA graph"}
        del g, peer, y_full
        torch.cuda.empty_cache()
    return out, "ok"


def measure_e2e_python(ctx, args):
    """The step through the C ABI from Python (ctypes): activations copied from pinned host memory each
    step, the down projection's output read back each step. Timed in encode-only mode and with every
    call synchronous. What an interpreter adds to the compiled host's figure."""
    torch, nn, rt = ctx["torch"], ctx["nn"], ctx["rt"]
    host_x = {k: v.view(torch.int16).cpu().pin_memory() for k, v in ctx["acts"].items()}
    y = ctx["y"]
    host_y_t = torch.empty(y.numel(), dtype=torch.float32).pin_memory()
    host_y = host_y_t.numpy()  # pinned: the read-back is a plain DMA
    yb = nn.GpuBuffer(y.data_ptr(), y.numel() * 4, owner=y, rt=rt)
    xin = {k: nn.GpuBuffer(v.data_ptr(), v.numel() * 2, owner=v, rt=rt) for k, v in ctx["acts"].items()}
    h2d = sum(v.numel() * 2 for v in host_x.values())
    d2h = host_y.nbytes
    steps = max(10, min(args.steps, 100))

    host_np = {k: v.numpy() for k, v in host_x.items()}  # views of the pinned tensors

    def one(i):
        for k, v in host_np.items():
            xin[k].write(v)
        ctx["step"](i)
        yb.read(np.float32, host_y.size, out=host_y)

    def timed():
        for i in range(3):
            one(i)
        rt.synchronize()
        t0 = time.perf_counter()
        for i in range(steps):
            one(i)
        rt.synchronize()
        return (time.perf_counter() - t0) / steps

    dt_sync = timed()  # the C ABI's default: every call returns with the runtime idle
    # The mode a decode loop uses (the reference's C ABI has the same switch, src/capi.rs:305-332 of the
    # reference project): writes and operators are only encoded on the stream, the read of the result waits.
    rt.set_encode_only(True)
    try:
        dt = timed()
    finally:
        rt.set_encode_only(False)
    return {"value": STEP_WEIGHT_BYTES / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": dt * 1e3, "steps": steps,
            "how": "per step: 3 host->device writes from pinned memory, 4 C-ABI operator calls, 1 device->host read of "
                   "the result; writes and operators encoded without waiting (encode-only mode), the read waits",
            "value_every_call_synchronous": STEP_WEIGHT_BYTES / dt_sync / 1e9, "ms_per_step_synchronous": dt_sync * 1e3}


def measure_e2e(ctx, args, device: int):
    """End to end at one GPU: the compiled host (tessl_b200/csrc/host_step_driver.cpp, C++ over the public
    header, built by tessl_b200/build.py) runs the same step with pinned host buffers; its figure is the one
    reported, the Python-ctypes figure sits beside it. The driver builds its banks from the same seeds as
    layer 0 here, and its first result is compared with this process's GPU result."""
    import tempfile

    from tessl_b200 import build as tb
    py = measure_e2e_python(ctx, args)
    steps = max(10, min(args.steps, 1000))
    with tempfile.TemporaryDirectory(prefix="tessl_e2e_") as tmp:
        y_path = os.path.join(tmp, "y.f32")
        cmd = [str(tb.STEP_DRIVER), "--steps", str(steps), "--warmup", str(max(args.warmup, 3)), "--layers", str(ctx["n_layers"]),
               "--seed", hex(CPU_SEED), "--device", str(device), "--y-out", y_path]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
            if r.returncode != 0:
                raise RuntimeError(r.stderr.strip()[-400:] or f"exit code {r.returncode}")
            d = json.loads(r.stdout.strip().splitlines()[-1])
            y_drv = np.fromfile(y_path, dtype=np.float32)
        except Exception as e:  # noqa: BLE001
            py["host"] = "python ctypes"
            py["compiled_host"] = {"unavailable": f"{type(e).__name__}: {e}"}
            return py
    ctx["rt"].set_encode_only(False)
    y_py = ctx["step"](0).cpu().numpy()
    same = bool(np.array_equal(y_drv.view(np.uint32), y_py.view(np.uint32)))
    diff = float(np.abs(y_drv.astype(np.float64) - y_py.astype(np.float64)).max())
    if not same and diff > 2e-3:
        raise SystemExit(f"bench: the compiled host's step disagrees with this process's (max |diff| {diff})")
    return {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": d["h2d_bytes_per_step"],
            "d2h_bytes_per_step": d["d2h_bytes_per_step"], "ms_per_step": d["ms_per_step"], "steps": d["steps"],
            "host": "compiled C++ over include/tessl_b200.h (tessl_b200/csrc/host_step_driver.cpp), host clock around the steps",
            "how": "per step: 3 host->device writes from pinned memory, 4 C-ABI operator calls, 1 device->host read of "
                   "the result; writes and operators encoded without waiting (encode-only mode), the read waits",
            "value_every_call_synchronous": d["value_every_call_synchronous"],
            "ms_per_step_synchronous": d["ms_per_step_synchronous"],
            "first_result_vs_this_process": "bit-exact" if same else f"max |diff| {diff:.3g}",
            "python_ctypes": {k: py[k] for k in ("value", "ms_per_step", "value_every_call_synchronous",
                                                 "ms_per_step_synchronous", "steps")}}


def measure_extra(ctx, args):
    """Other configurations of the path, each timed on the device with CUDA events
    (single GPU): LM head, small-batch GEMM, MLX Q8 GEMV, and the Q4 prefill GEMM."""
    torch, nn, rt, st, dev, peaks = ctx["torch"], ctx["nn"], ctx["rt"], ctx["st"], ctx["dev"], ctx["peaks"]
    B = nn.GpuBuffer.from_torch
    out = {}
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0xC0FFEE)

    def rand_bank(rows, cols):
        packed, sb = device_bank(torch, gen, rows, cols)
        return (packed, sb), nn.Q4MlxBank(B(packed), B(sb))

    def timed(fn, nrot, iters):
        rt.set_encode_only(True)
        for i in range(nrot):
            fn(i)
        rt.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for i in range(iters):
                fn(i % nrot)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = 1e30
        with torch.cuda.stream(st):
            for rep in range(5):
                a.record(st)
                g.replay()
                b.record(st)
                b.synchronize()
                if rep:
                    best = min(best, a.elapsed_time(b) / iters)
        rt.set_encode_only(False)
        return best * 1e3

    # LM head 151936 x 4096, M = 1 and 8 (two banks = 700 MB > L2)
    vocab = 151936
    keep, lm = zip(*[rand_bank(vocab, HIDDEN) for _ in range(2)])
    wb = q4_weight_bytes(vocab, HIDDEN)
    for m in (1, 8):
        x = torch.randn(m * HIDDEN, device=dev, generator=gen).to(torch.bfloat16)
        y = torch.empty(m * vocab, device=dev)
        shape = nn.QuantShape(vocab, HIDDEN, GROUP)
        if m == 1:
            us = timed(lambda i: nn.gemv_q4_mlx_simd(rt, lm[i], B(x), B(y), shape), 2, 8)
        else:
            us = timed(lambda i: nn.gemm_q4_mlx(rt, lm[i], B(x), B(y), shape, m), 2, 4)
        out[f"lm_head 151936x4096 m={m}"] = {"us": round(us, 2), "weight_gbs": round(wb / us / 1e3, 1),
                                            "frac_of_measured_hbm": round(wb / us / 1e3 / peaks["hbm_gbs"], 4)}
    del keep, lm
    torch.cuda.empty_cache()

    # MLX Q8 GEMV 14336 x 4096, M in {1, 4, 8} (six banks = 374 MB > L2)
    n8 = 14336
    codes = [torch.randint(0, 2**31 - 1, (n8, HIDDEN // 4), dtype=torch.int32, device=dev, generator=gen) for _ in range(6)]
    sc = (torch.rand((n8, HIDDEN // GROUP), device=dev, generator=gen) * 0.0045 + 0.0005).to(torch.bfloat16)
    sb8 = torch.stack([sc, (-128.0 * sc.float()).to(torch.bfloat16)], dim=-1).contiguous()
    wb8 = n8 * HIDDEN + n8 * (HIDDEN // GROUP) * 4
    for m in (1, 4, 8):
        x = torch.randn(m * HIDDEN, device=dev, generator=gen).to(torch.bfloat16)
        y = torch.empty(m * n8, device=dev)
        us = timed(lambda i: nn.gemm_q8_mlx(rt, B(codes[i]), B(sb8), B(x), B(y), nn.QuantShape(n8, HIDDEN, GROUP), m),
                   6, 24)
        out[f"q8_mlx 14336x4096 m={m}"] = {"us": round(us, 2), "weight_gbs": round(wb8 / us / 1e3, 1),
                                          "frac_of_measured_hbm": round(wb8 / us / 1e3 / peaks["hbm_gbs"], 4)}
    del codes
    torch.cuda.empty_cache()

    # Q4 prefill GEMM: X [2048, 4096] x W [12288, 4096]^T, f32 out
    M, N, K = 2048, INTER, HIDDEN
    try:
        keep, banks = zip(*[rand_bank(N, K) for _ in range(2)])
        X = torch.randn(M * K, device=dev, generator=gen).to(torch.bfloat16)
        Y = torch.empty(M * N, device=dev)
        us = timed(lambda i: nn.gemm_q4_mlx_tensorops(rt, banks[i], B(X), B(Y), nn.QuantShape(N, K, GROUP), M), 2, 6)
        tf = 2.0 * M * N * K / us / 1e6
        out["prefill_gemm 2048x12288x4096"] = {"us": round(us, 1), "tflops": round(tf, 1),
                                                "frac_of_measured_bf16_burst": round(tf / peaks["bf16_tflops"], 4),
                                                "frac_of_measured_bf16_sustained": round(tf / peaks["bf16_tflops_sustained"], 4)}
    except nn.TesslError as e:
        out["prefill_gemm 2048x12288x4096"] = {"error": str(e)}
    return out


def cpu_baseline(args, ctx_inputs=None):
    """The CPU oracle on full steps of the same workload, all host threads, for about ten seconds."""
    threads = host_threads()
    banks, xs = ctx_inputs if ctx_inputs is not None else cpu_step_inputs(CPU_SEED)
    cpu_step(banks, xs, threads, 0.1)
    t0 = time.perf_counter()
    done, steps = 0, 0
    while time.perf_counter() - t0 < 10.0 and steps < 400:
        _, b = cpu_step(banks, xs, threads, 1.0)
        done += b
        steps += 1
    dt = time.perf_counter() - t0
    # the scalar path on one core, on a bounded sample (the leading quarter of every projection's rows)
    t1 = time.perf_counter()
    done1, steps1 = 0, 0
    while time.perf_counter() - t1 < 3.0 and steps1 < 50:
        _, b = cpu_step(banks, xs, 1, 0.25)
        done1 += b
        steps1 += 1
    dt1 = time.perf_counter() - t1
    return {"value": done / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{steps} full steps (all rows of the four projections), f64-accumulated dequant-matvec in "
                      "C/OpenMP (oracle/tessl_oracle.c)", "seconds": round(dt, 2),
            "one_core": {"value": done1 / dt1 / 1e9, "unit": "GB/s", "cores": 1,
                         "sample": f"{steps1} steps over the leading 25% of each projection's rows"}}


def run_case(spec: str):
    """`--case gemv:N,K[,banks[,iters]]` or `--case prefill:M,N,K[,iters]`: a few plain
    launches of one operator on seeded banks, for capturing one kernel under ncu."""
    import torch

    from tessl_b200 import nn
    kind, _, rest = spec.partition(":")
    a = [int(v) for v in rest.split(",")]
    rt = nn.Runtime()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    B = nn.GpuBuffer.from_torch

    def bank(rows, cols):
        packed, sb = device_bank(torch, gen, rows, cols)
        return (packed, sb), nn.Q4MlxBank(B(packed), B(sb))

    if kind == "gemv":
        n, k = a[0], a[1]
        nb, iters = (a[2] if len(a) > 2 else 8), (a[3] if len(a) > 3 else 12)
        keep, banks = zip(*[bank(n, k) for _ in range(nb)])
        x = torch.randn(k, device="cuda", generator=gen).to(torch.bfloat16)
        y = torch.empty(n, device="cuda")
        for i in range(iters):
            nn.gemv_q4_mlx_simd(rt, banks[i % nb], B(x), B(y), nn.QuantShape(n, k, GROUP))
    elif kind == "prefill":
        m, n, k = a[0], a[1], a[2]
        iters = a[3] if len(a) > 3 else 3
        keep, bk = bank(n, k)
        x = torch.randn(m * k, device="cuda", generator=gen).to(torch.bfloat16)
        y = torch.empty(m * n, device="cuda")
        for i in range(iters):
            nn.gemm_q4_mlx_tensorops(rt, bk, B(x), B(y), nn.QuantShape(n, k, GROUP), m)
    else:
        raise SystemExit(f"unknown case {spec!r}")
    rt.synchronize()
    print(json.dumps({"case": spec, "y0": float(y[0])}))
    rt.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the other configurations (faster)")
    ap.add_argument("--case", default=None, help="run a few launches of one operator and exit (for ncu captures)")
    args = ap.parse_args()
    if args.case:
        run_case(args.case)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.steps > 40:
            args.steps = 40  # each step is ~0.1-0.5 s of CPU work; keep the arm to a few minutes
        run_reference_arm(args, rank)
        return
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import torch
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = run_ours(args, rank, world, local_rank)
    peaks = ctx["peaks"]
    line = {
        "metric": METRIC, "value": round(ctx["value"], 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ctx["ms_per_step"], 5), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32 accumulate over bf16 x / Q4 weights", "data": "synthetic",
        "config": workload_config(world, ctx["n_layers"]),
        "gpu_launches": ctx["launches_per_step"] * args.steps, "gather": ctx.get("gather") if world > 1 else None,
        "clocks": ctx["clocks"], "parity": ctx["parity"],
        "frac_of_measured_hbm": round(ctx["value"] / (peaks["hbm_gbs"] * world), 4),
        "frac_of_nominal_8tbs": round(ctx["value"] / (8000.0 * world), 4),
    }
    if world == 1:
        pk = ctx["per_kernel"]
        # Dominant kernel: the tensor-core GEMV, which serves all four launches of a step.
        dom = ["qkv 6144x4096", "o 4096x4096", "gate_up_silu 2x12288x4096", "down 4096x12288"]
        dom_bytes = STEP_WEIGHT_BYTES
        dom_us = sum(pk[k]["us"] for k in dom)
        achieved = dom_bytes / dom_us / 1e3
        line["roofline"] = {
            "bound": "hbm", "kernel": "q4_gemv_mma_kernel", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
            "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peaks["source"],
            "how": "algorithmic weight bytes of the step's four launches / the sum of their average launch durations, each "
                   "measured with CUDA events over a graph of that launch alone rotating over the layers' banks",
            # ncu: dram__bytes_read+write of one 12288x4096 launch against its algorithmic bytes
            # (profiles/q4_gemv_mma_12288x4096.md); scaled by bytes to the mean launch of the step.
            "traffic": round(dom_bytes / 4 * TRAFFIC_RATIO), "algorithmic_bytes_per_launch": dom_bytes // 4,
            "traffic_source": f"one ncu capture of a 12288x4096 launch (DRAM bytes / algorithmic bytes = {TRAFFIC_RATIO}), scaled "
                              "by bytes to the mean of the step's four launches",
            "launches_per_step": 4,
        }
        line["per_kernel"] = pk
        line["offline_repack"] = ctx["staged_variant"]
        line["e2e"] = measure_e2e(ctx, args, local_rank)
        if not args.no_extra:
            line["extra"] = measure_extra(ctx, args)
            pf = line["extra"].get("prefill_gemm 2048x12288x4096", {})
            if "tflops" in pf:
                # second roofline object: the prefill GEMM (tensor bound), timed alone, so against the burst peak
                line["roofline_prefill"] = {
                    "bound": "tensor", "kernel": "q4_prefill_gemm_pair_kernel<256>", "achieved": pf["tflops"],
                    "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": round(pf["tflops"] / peaks["bf16_tflops"], 4),
                    "peak_source": peaks["source"] + " (burst: the kernel is timed alone)", "traffic": None,
                    "flops_per_launch": 2 * 2048 * INTER * HIDDEN, "workload": "X[2048, 4096] bf16 x W[12288, 4096]^T Q4 g64, f32 out",
                }
        line["cpu_baseline"] = cpu_baseline(args, ctx["cpu_inputs"])
    else:
        line["parity_n"] = ctx["parity"].get("parity_n")
        if ctx["variants"]:
            line["down_variants"] = ctx["variants"]
        # The headline figure is complete here. The two secondary measurements below and the closing
        # barrier involve further collectives; if one of them stalls or fails on some rank, the line is
        # still printed once (with the reason in place of the missing figure) and every rank leaves
        # without waiting for the others.
        emit = threading.Lock()
        printed = [False]

        def print_line():
            with emit:
                if rank == 0 and not printed[0]:
                    print(json.dumps(line), flush=True)
                printed[0] = True

        def leave(reason: str):
            if not printed[0]:
                line.setdefault("extra", {})["incomplete"] = reason
            print_line()
            sys.stdout.flush()
            os._exit(0)

        watchdog = threading.Timer(120.0, leave, args=("secondary measurements did not finish within 120 s",))
        watchdog.daemon = True
        watchdog.start()
        try:
            # every rank copies its activations in and reads its result out; the slowest rank's time counts
            e2e = measure_e2e_python(ctx, args)
            e2e["host"] = "python ctypes (the compiled host drives one GPU)"
            torch = ctx["torch"]
            t = torch.tensor([e2e["ms_per_step"], e2e["ms_per_step_synchronous"]], device=ctx["dev"], dtype=torch.float64)
            ctx["dist"].all_reduce(t, op=ctx["dist"].ReduceOp.MAX)
            e2e["ms_per_step"], e2e["ms_per_step_synchronous"] = float(t[0].item()), float(t[1].item())
            e2e["value"] = STEP_WEIGHT_BYTES / (e2e["ms_per_step"] * 1e-3) / 1e9
            e2e["value_every_call_synchronous"] = STEP_WEIGHT_BYTES / (e2e["ms_per_step_synchronous"] * 1e-3) / 1e9
            e2e["how"] += f"; on each of the {world} ranks, slowest rank's time"
            line["e2e"] = e2e
            sharded_head, head_parity = measure_sharded_lm_head(ctx, args, world, rank)
            line["extra"] = sharded_head
            if head_parity != "ok":
                line["parity_n"] = head_parity
        except Exception as e:  # noqa: BLE001
            leave(f"{type(e).__name__}: {e}")
        print_line()
        ctx["dist"].barrier()
        watchdog.cancel()
        ctx["dist"].destroy_process_group()
        return
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
