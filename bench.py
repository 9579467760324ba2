"""Benchmark of the GGUF quantised-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (``config.workload``): the decode configuration the headline metric is quoted on --
Q4_K GEMVs of one decoder MLP, gate and up ``[18944 x 3584]`` and down ``[3584 x 18944]``, at batch
1, 4 and 16, bf16 activations ~ N(0,1), fp32 outputs.  One *step* is those nine GEMVs over one set
of weights.  Weights rotate over a ring of sets larger than three times the L2 cache, so every
launch streams its weights from HBM.  Data is synthetic (seeded, with the stated distributions).

``value``  = raw quantised weight bytes of a step / device time, inputs resident in HBM (CUDA
             events around exactly K steps, barrier + synchronise on both sides, max over ranks).
``e2e``    = the same metric through the host-buffer API: activations start in pinned host memory
             and outputs end there, every step (weights stay resident, as model parameters do).
``roofline`` is for the dominant kernel (the pipelined GEMV): algorithmic weight bytes of a launch
             / its average duration in the timed region, against the measured HBM copy bandwidth.
``prefill`` reports the tcgen05 GEMM (Q4_K / Q6_K, N=12288, K=4096, M in {256, 512, 2048}).
``cpu_baseline`` times the multi-threaded C port of the reference arithmetic on the host cores on a
             bounded sample.  ``--impl reference`` runs only that port, as the reference arm.

With N > 1 (torchrun, one process per GPU) every weight is column-sharded along N over the ranks
and each projection's output is all-gathered over NCCL; total work is fixed (strong scaling).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = (("gate", 18944, 3584), ("up", 18944, 3584), ("down", 3584, 18944))
BATCHES = (1, 4, 16)
FORMAT = "q4_k"
PREFILL = (("q4_k", 12288, 4096), ("q6_k", 12288, 4096))
PREFILL_M = (256, 512, 2048)
L2_BYTES = 126 * 1024 * 1024
METRIC = "q4k_gemv_weight_gbps"
UNIT = "GB/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def is_grouped(args, world: int) -> bool:
    """Gate and up go out as one grouped launch (they share their activations)."""
    return not args.separate_gate_up and (world == 1 or args.gather in ("fused", "fused-barrier"))


def workload_config(world: int, gather: str = "fused", grouped: bool = False):
    return {
        "workload": "q4_k decode GEMV: gate/up 18944x3584 + down 3584x18944, batch 1/4/16 (9 GEMVs per step)",
        "launches": ("gate and up share their activations and run as one grouped launch (6 GEMV launches per step)"
                     if grouped else "one launch per GEMV"),
        "format": FORMAT, "batches": list(BATCHES), "activations": "bf16", "output": "fp32",
        "l2": "weights rotate over a ring of sets > 3x L2; every launch streams from HBM",
        "parallelism": f"N-sharded x{world}" + ("" if world == 1 else (
            " + peer stores in the GEMV epilogue over NVLink, signal/wait between ranks inside the same launches"
            if gather == "fused" else
            " + peer stores in the GEMV epilogue over NVLink and one barrier kernel after gate+up and after down"
            if gather == "fused-barrier" else " + NCCL all-gather (gate+up together, then down)")),
    }


def reference_config(cores: int):
    gpu = workload_config(1)
    return {"workload": gpu["workload"], "format": gpu["format"], "batches": gpu["batches"],
            "activations": "bf16 values widened to fp32", "output": "fp32",
            "launches": "nine GEMV calls per step, one after another",
            "l2": "one resident set of weights (115 MB, larger than the host caches)",
            "parallelism": f"OpenMP over weight rows, {cores} host threads, rank 0 only"}


# ---------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the C port of the reference arithmetic on the host cores
# ---------------------------------------------------------------------------------------------

def cpu_port_gemv_rate(seconds: float, batches=BATCHES):
    """Weight GB/s of the oracle's multi-threaded C GEMV on gate+up+down at every batch of
    ``batches`` (the same nine GEMVs as a GPU step when ``batches`` is the full set)."""
    from oracle import c_oracle
    from oracle import gguf_oracle as oracle

    c_oracle.use_all_cores()  # process launchers export OMP_NUM_THREADS=1; the baseline uses every host core
    cases = []
    for i, (_, n, k) in enumerate(SHAPES):
        raw = oracle.make_weights(FORMAT, n, k, seed=100 + i)
        for batch in batches:
            x = oracle.make_activations(batch, k, seed=200 + i + 10 * batch, dtype="bf16")
            cases.append((raw, x, n, k))
    step_bytes = sum(c[0].size for c in cases)

    def step():
        for raw, x, n, k in cases:
            c_oracle.gemv(x, raw, FORMAT, n, k)

    step()
    times = []
    t_end = time.perf_counter() + seconds
    while time.perf_counter() < t_end or len(times) < 2:
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return step_bytes / med / 1e9, c_oracle.threads(), len(times), med, step


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import c_oracle

    rate, cores, _, _, step = cpu_port_gemv_rate(0.0)
    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    elapsed = time.perf_counter() - t0
    step_bytes = 3 * 38191104 * len(BATCHES)
    value = step_bytes * args.steps / elapsed / 1e9
    sample = "the full step (nine Q4_K GEMVs: gate, up, down at batch 1, 4, 16) per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        # the same workload as the GPU arm; the other keys describe how this arm runs it
        "data": "synthetic", "config": reference_config(c_oracle.threads()),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": c_oracle.threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's own kernels for this path live in an external package and its CPU "
                "provider cannot build here; this arm times the C port of its stated arithmetic",
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        try:
            with open(self.path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) >= 7 and parts[0].isdigit():
                        rows.append(parts)
            os.remove(self.path)
        except Exception:
            pass
        if rows:
            clocks = [int(r[0]) for r in rows]
            busy = [c for c in clocks if c > 0.5 * max(clocks)] or clocks
            out["sm_mhz"] = statistics.median(busy)
            out["sm_max_mhz"] = int(rows[0][1])
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            out["reasons"] = [n for i, n in enumerate(names) if any(r[3 + i] == "Active" for r in rows)]
            out["samples"] = len(rows)
        return out


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def run_gpu(args):
    import torch
    import torch.distributed as dist

    import tensor_b200 as tb
    from tensor_b200 import synth
    from tensor_b200.peer import PeerArena
    from tensor_b200.projection import FusedGatherGroup, GatherGroup, QuantLinear, QuantLinearPair

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.gpus > 1 and world == 1:
        raise SystemExit("launch multi-GPU runs with torch.distributed.run, one process per GPU")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # the version banner would share stdout with the JSON line
        dist.init_process_group("nccl", device_id=device)
    peaks = measured_peaks()
    fmt = tb.get_format(FORMAT)

    # ---- weights: ring of sets, each rank holding its rows; same seeds on every rank ----
    step_bytes_total = sum(fmt.weight_bytes(n, k) for _, n, k in SHAPES) * len(BATCHES)
    set_bytes_local = sum(fmt.weight_bytes(n // world, k) for _, n, k in SHAPES)
    ring = max(2, -(-3 * L2_BYTES // set_bytes_local) + 1)
    weights = []
    for slot in range(ring):
        row = []
        for j, (_, n, k) in enumerate(SHAPES):
            # distinct seed per (slot, projection, rank): every rank owns different rows
            row.append(synth.make_weights(fmt, n // world, k, seed=1000 * slot + 10 * j + rank, device=device))
        weights.append(row)
    acts = {b: [synth.make_activations(b, k, seed=7 * b + j, device=device) for j, (_, _, k) in enumerate(SHAPES)]
            for b in BATCHES}
    lins = {b: [QuantLinear(weights[0][j], fmt, n, k, b, rank=rank, world=world, variant="auto")
                for j, (_, n, k) in enumerate(SHAPES)] for b in BATCHES}
    grouped = is_grouped(args, world)  # gate + up as one launch
    launches_per_step = len(BATCHES) * (len(SHAPES) - 1 if grouped else len(SHAPES))
    barriers_per_step = 2 * len(BATCHES) if world > 1 and args.gather == "fused-barrier" else 0
    # batches above 1 run a small activation-conversion kernel ahead of each GEMV
    barriers_per_step += sum(launches_per_step // len(BATCHES) for b in BATCHES if b > 1)
    if world > 1 and args.gather == "fused":
        barriers_per_step += len(BATCHES)  # the wait kernel that closes each batch
    # gate and up are needed together (one collective for both); down follows
    if args.gather in ("fused", "fused-barrier"):
        # the GEMVs store their columns into every rank's output; one barrier kernel per group
        out_bytes = sum(b * n * 4 + 256 for b in BATCHES for _, n, _ in SHAPES)
        arena = PeerArena(out_bytes + (1 << 16), device, rank, world)
        fold = args.gather == "fused"  # ordering inside the GEMV launches; else one barrier kernel per group
        share = not args.separate_gate_up  # gate and up read the same activations: one grouped launch
        groups = {b: [FusedGatherGroup(lins[b][0:2], arena, fold, shared_input=share),
                      FusedGatherGroup(lins[b][2:3], arena, fold)] for b in BATCHES}
    else:
        groups = {b: [GatherGroup(lins[b][0:2]), GatherGroup(lins[b][2:3])] for b in BATCHES}

    # one GPU: gate and up read the same activations and go out as ONE launch over both weights
    pairs = None
    if world == 1 and not args.separate_gate_up:
        pairs = {b: QuantLinearPair(weights[0][0], SHAPES[0][1], weights[0][1], SHAPES[1][1], fmt, SHAPES[0][2], b)
                 for b in BATCHES}

    def step(slot, batches=BATCHES):
        for b in batches:
            if pairs is not None:
                pairs[b].forward(acts[b][0], raw1=weights[slot][0], raw2=weights[slot][1])
            else:
                groups[b][0].forward(acts[b][0:2], raws=weights[slot][0:2])
            groups[b][1].forward(acts[b][2:3], raws=weights[slot][2:3])
            if world > 1 and args.gather == "fused":
                groups[b][1].wait()  # the peers' columns of the last projection have landed

    # ---- CUDA graphs: one per ring slot (launch-bound otherwise: a GEMV is a few microseconds) ----
    stream = torch.cuda.Stream(device)
    graphs = {}

    def capture(batches):
        out = []
        with torch.cuda.stream(stream):
            step(0, batches)
            stream.synchronize()
            for slot in range(ring):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    step(slot, batches)
                out.append(g)
        return out

    use_graphs = not args.no_graphs
    if use_graphs:
        try:
            graphs["all"] = capture(BATCHES)
        except Exception as exc:  # pragma: no cover - e.g. a collective that cannot be captured
            use_graphs = False
            if rank == 0:
                print(f"[bench] CUDA graph capture failed ({exc}); timing eager launches", file=sys.stderr)

    def run_steps(count, key="all", batches=BATCHES, offset=0):
        with torch.cuda.stream(stream):
            for i in range(count):
                if use_graphs:
                    graphs[key][(offset + i) % ring].replay()
                else:
                    step((offset + i) % ring, batches)

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(count, key="all", batches=BATCHES):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
        run_steps(count, key, batches)
        with torch.cuda.stream(stream):
            e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # warm-up (also brings the clocks up), then the timed region with clock sampling
    run_steps(max(args.warmup, 3))
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms = timed(args.steps)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / args.steps
    value = step_bytes_total / (ms_per_step * 1e-3) / 1e9

    # ---- per-batch breakdown (outside the headline region) ----
    cases = []
    for b in BATCHES:
        if use_graphs:
            graphs[b] = capture((b,))
        reps = max(20, args.steps)
        run_steps(5, b, (b,))
        t = timed(reps, b, (b,)) / reps
        bytes_b = step_bytes_total // len(BATCHES)
        cases.append({"batch": b, "us_per_3_gemv": t * 1e3, "gbps": bytes_b / (t * 1e-3) / 1e9})

    # ---- roofline of the dominant kernel: the pipelined GEMV ----
    launch_bytes_local = set_bytes_local * len(BATCHES) / launches_per_step  # weight bytes of an average launch
    avg_launch_s = ms_per_step * 1e-3 / launches_per_step
    achieved = launch_bytes_local / avg_launch_s / 1e9
    best = max(cases, key=lambda c: c["gbps"])
    roofline = {
        "bound": "hbm", "kernel": "gemv_mma_kernel (bulk-copy ring + mma.sync)",
        "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
        "peak_source": peaks["source"], "traffic": None,
        "algorithmic_bytes_per_launch": launch_bytes_local,
        "note": f"average over the {launches_per_step} GEMV launches of a step (batch 1/4/16"
                + (", gate and up grouped into one launch" if grouped else "")
                + "), gaps between launches included; "
                f"best batch ({best['batch']}) reaches {best['gbps'] / world:.0f} GB/s per GPU",
    }
    if world == 1:
        # dram__bytes_read.sum + dram__bytes_write.sum from the committed ncu capture of one 38,191,104-byte
        # launch (profiles/gemv_q4k_batch1_18944x3584.md: 38,245,120 B, i.e. no re-reads), scaled to the
        # weight bytes of an average launch of this run (traffic is proportional to the rows streamed)
        roofline["traffic"] = round(launch_bytes_local * 38245120 / 38191104)

    # ---- end to end: host buffers in, host buffers out, every step ----
    # device tensors that travel: with the grouped launch gate and up share one activation buffer
    # and one [m, 2N] output
    live_acts = {b: ([acts[b][0], acts[b][2]] if pairs is not None else list(acts[b])) for b in BATCHES}
    live_outs = {b: ([pairs[b].out, lins[b][2].out] if pairs is not None else [l.out for l in lins[b]])
                 for b in BATCHES}
    x_host = {b: [a.cpu().pin_memory() for a in live_acts[b]] for b in BATCHES}
    y_host = {b: [torch.empty(tuple(o.shape), dtype=torch.float32).pin_memory() for o in live_outs[b]] for b in BATCHES}
    h2d = sum(t.numel() * t.element_size() for b in BATCHES for t in x_host[b])
    d2h = sum(t.numel() * 4 for b in BATCHES for t in y_host[b])

    # Every step copies every activation in from pinned host memory and every output back out.  The
    # copies ride on two side streams and are ordered by events per batch: the largest batch runs
    # first, so its outputs travel while the smaller batches compute, and the inputs of the next
    # step's batch b go in as soon as this step's batch b has been computed.  Buffers are single:
    # the compute of batch b waits until its previous outputs have left and its inputs have arrived.
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    order = sorted(BATCHES, reverse=True)
    ev_in = {b: torch.cuda.Event() for b in BATCHES}
    ev_out = {b: torch.cuda.Event() for b in BATCHES}
    ev_done = {b: torch.cuda.Event() for b in BATCHES}

    def copy_in(b):
        with torch.cuda.stream(s_in):
            for dst, src in zip(live_acts[b], x_host[b]):
                dst.copy_(src, non_blocking=True)
            ev_in[b].record(s_in)

    def e2e_step(i):
        for b in order:
            stream.wait_event(ev_in[b])
            stream.wait_event(ev_out[b])
            with torch.cuda.stream(stream):
                if use_graphs:
                    graphs[b][i % ring].replay()
                else:
                    step(i % ring, (b,))
                ev_done[b].record(stream)
            s_out.wait_event(ev_done[b])
            with torch.cuda.stream(s_out):
                for dst, src in zip(y_host[b], live_outs[b]):
                    dst.copy_(src, non_blocking=True)
                ev_out[b].record(s_out)
            s_in.wait_event(ev_done[b])
            copy_in(b)  # the next step's inputs of this batch

    def e2e_drain():
        for st in (stream, s_in, s_out):
            st.synchronize()

    torch.cuda.synchronize(device)
    for b in BATCHES:
        ev_out[b].record(s_out)
        copy_in(b)
    for i in range(3):
        e2e_step(i)
    e2e_drain()
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    e2e_drain()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": step_bytes_total * args.steps / e2e_s / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "note": "activations from pinned host memory and outputs back to it every step, on copy streams "
                   "ordered by events per batch (largest batch first); weights resident"}

    # ---- prefill GEMM (single GPU numbers; N-sharded when world > 1) ----
    prefill = []
    if rank == 0 or world > 1:
        for name, n, k in PREFILL:
            n_local = n // world
            copies = max(2, -(-2 * L2_BYTES // tb.weight_bytes(name, n_local, k)))
            ws = [synth.make_weights(name, n_local, k, seed=50 + c + rank, device=device) for c in range(copies)]
            for m in PREFILL_M:
                x = synth.make_activations(m, k, seed=60 + m, device=device)
                out = torch.empty((m, n_local), dtype=torch.float32, device=device)
                kern = tb.gguf(m, n_local, k, name, op="gemm")
                for c in range(3):
                    kern.launch(x, ws[c % copies], out)
                torch.cuda.synchronize(device)
                reps = 20
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for c in range(reps):
                    kern.launch(x, ws[c % copies], out)
                e1.record()
                torch.cuda.synchronize(device)
                us = e0.elapsed_time(e1) / reps * 1e3
                tf = 2.0 * m * n_local * k / (us * 1e-6) / 1e12
                prefill.append({"format": name, "m": m, "n": n_local, "k": k, "us": us, "tflops": tf,
                                "frac_of_bf16_peak": tf / peaks["bf16_tflops"]})
            del ws

    status = tb.device_status()
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16 mma / f32 accumulate", "data": "synthetic",
        "config": workload_config(world, args.gather, grouped), "clocks": clocks, "e2e": e2e,
        "gpu_launches": (launches_per_step + barriers_per_step) * args.steps, "roofline": roofline, "cases": cases,
        "prefill": prefill, "cuda_graphs": use_graphs, "device_status": status,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rate, cores, n_steps, med, _ = cpu_port_gemv_rate(10.0)
        line["cpu_baseline"] = {
            "value": rate, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"the same nine GEMVs as a GPU step, {n_steps} passes, median {med * 1e3:.1f} ms per pass"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # Every collective of this run has completed on every rank (the last one returned a value to
        # the host).  Tearing the NCCL communicator down while CUDA graphs that captured its kernels
        # are alive was seen to block, so drop the graphs first and leave without the teardown.
        graphs.clear()
        torch.cuda.synchronize(device)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="native", choices=("native", "reference"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--separate-gate-up", action="store_true",
                    help="one GPU: launch gate and up as two GEMVs instead of one grouped launch")
    ap.add_argument("--no-graphs", action="store_true",
                    help="launch every kernel eagerly (for per-kernel profiling; the numbers then include "
                         "the host's launch overhead)")
    ap.add_argument("--gather", default="fused", choices=("fused", "fused-barrier", "nccl"),
                    help="multi-GPU: peer stores and signal/wait inside the GEMV launches; the same stores with a "
                         "barrier kernel per group; or NCCL all-gather")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
