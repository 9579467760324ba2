"""Benchmark of the GGUF quantised-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python bench.py --single gemv:q4_k:1:18944:3584        # one kernel, one shape, plain launches

Workload (``config.workload``): the decode configuration the headline metric is quoted on --
Q4_K GEMVs of one decoder MLP, gate and up ``[18944 x 3584]`` and down ``[3584 x 18944]``, at batch
1, 4 and 16, bf16 activations ~ N(0,1), fp32 outputs.  One *step* is those nine GEMVs over one set
of weights, issued as one list (six launches: gate and up share their activations).  Weights rotate over a ring of sets larger than three times the L2 cache, so every
launch streams its weights from HBM.  Data is synthetic (seeded, with the stated distributions).

``value``  = raw quantised weight bytes of a step / device time, inputs resident in HBM (CUDA
             events around exactly K steps, barrier + synchronise on both sides, max over ranks).
``e2e``    = the same metric through the host-buffer API: activations start in pinned host memory
             and the results end there, every step (weights stay resident, as model parameters do).
``roofline`` is for the dominant kernel (the pipelined GEMV): algorithmic weight bytes of a launch
             / its average duration in the timed region, against the measured HBM copy bandwidth.
``cases``  per-batch and per-kernel rows: the three batches of the step, the first configuration of
             the benchmark definition (Q8_0 4096 x 4096, fp16) and a Q6_K down projection.
``prefill`` reports the tcgen05 GEMM (Q4_K / Q6_K, N=12288, K=4096, M in {256, 512, 2048}) beside the
             ceiling without decoding: a dense bf16 GEMM on weights dequantised ahead of time.
``decode_step`` is the 36-layer decoder configuration (252 projections per step, batch 1 and 16).
``prefill_70b`` is the 70B-class prefill sweep at M = 4096 (on more than one GPU the fp32 outputs of
             a rank's columns are all-gathered with NCCL in chunks of rows that overlap the next chunk's GEMM).
``cpu_baseline`` times the multi-threaded C port of the reference arithmetic on the host cores on a
             bounded sample.  ``--impl reference`` runs only that port, as the reference arm.

With N > 1 (torchrun, one process per GPU) every weight is column-sharded along N over the ranks;
total work is fixed (strong scaling).  Decode GEMVs store their columns straight into every rank's
output over NVLink (peer-mapped memory) with the cross-GPU ordering folded into the launches: the
first launch of a list waits for the peers' previous signal, the last one signals.
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
# the 36-layer decoder of the benchmark definition: (name, rows N, depth K, format, which activations it reads)
LAYER = (("q", 4096, 4096, "q4_k", 0), ("k", 1024, 4096, "q4_k", 0), ("v", 1024, 4096, "q4_k", 0),
         ("o", 4096, 4096, "q4_k", 1), ("gate", 12288, 4096, "q4_k", 2), ("up", 12288, 4096, "q4_k", 2),
         ("down", 4096, 12288, "q6_k", 3))
# the same layer as the runtime holds it: q, k, v rows concatenated into one weight and gate, up into another when the
# model is loaded (GGUF rows are independent of each other), so a layer is four launches
LAYER_FUSED = (("qkv", 6144, 4096, "q4_k", 0), ("o", 4096, 4096, "q4_k", 1), ("gate_up", 24576, 4096, "q4_k", 2),
               ("down", 4096, 12288, "q6_k", 3))
LAYERS = 36
BIG_PREFILL = (("gate_up", "q4_k", 28672, 8192), ("down", "q6_k", 8192, 28672))
BIG_PREFILL_M = 4096
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


def workload_config(world: int):
    return {
        "workload": "q4_k decode GEMV: gate/up 18944x3584 + down 3584x18944, batch 1/4/16 (9 GEMVs per step)",
        "launches": "gate and up share their activations and run as one grouped launch (6 GEMV launches per step, behind one "
                    "launch that converts the batch-4 and batch-16 activations)",
        "format": FORMAT, "batches": list(BATCHES), "activations": "bf16", "output": "fp32",
        "l2": "weights rotate over a ring of sets > 3x L2; every launch streams from HBM",
        "parallelism": f"N-sharded x{world}" + ("" if world == 1 else
            " + peer stores in the GEMV epilogue over NVLink, signal/wait between ranks inside the same launches "
            "(the nine projections of a step go out as one list: one wait and one signal per step)"),
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
    from tensor_b200 import ops, synth
    from tensor_b200.peer import PeerArena
    from tensor_b200.projection import ShardedGemvList

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
        # NCCL prints its version banner on stdout while the communicator is set up; stdout carries
        # the JSON line alone, so the banner goes to stderr
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=device)
            dist.barrier()
            torch.cuda.synchronize(device)
        finally:
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    peaks = measured_peaks()
    fmt = tb.get_format(FORMAT)
    stream = torch.cuda.Stream(device)
    arena = PeerArena(64 << 20, device, rank, world) if world > 1 else None
    pads = arena.pad_ptrs() if world > 1 else None

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def max_over_ranks(value: float) -> float:
        if world == 1:
            return value
        t = torch.tensor([value], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_replays(graphs, count, after=None):
        """Device time of ``count`` replays cycling over ``graphs`` (max over ranks), in ms."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for i in range(count):
                graphs[i % len(graphs)].replay()
            if after is not None:
                after()
            e1.record(stream)
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    # ---- headline: weights as a ring of sets, each rank holding its rows; same seeds on every rank ----
    step_bytes_total = sum(fmt.weight_bytes(n, k) for _, n, k in SHAPES) * len(BATCHES)
    set_bytes_local = sum(fmt.weight_bytes(n // world, k) for _, n, k in SHAPES)
    ring = max(2, -(-3 * L2_BYTES // set_bytes_local) + 1)
    ring += ring % 2  # even: the two output copies of the N-sharded lists alternate from slot to slot
    weights = [[synth.make_weights(fmt, n // world, k, seed=1000 * slot + 10 * j + rank, device=device)
                for j, (_, n, k) in enumerate(SHAPES)] for slot in range(ring)]
    # the activations of a step are views of ONE device buffer, so that they arrive from the host in one copy;
    # the buffer exists twice and the weight sets of the ring alternate between the copies (the ring is even),
    # so the next step's activations can arrive while this step computes
    acts_src = {b: [synth.make_activations(b, k, seed=7 * b + j, device=device) for j, (_, _, k) in enumerate(SHAPES)]
                for b in BATCHES}
    x_elems = sum(acts_src[b][j].numel() for b in BATCHES for j in (0, 2))
    x_both = [torch.empty(x_elems, dtype=torch.bfloat16, device=device) for _ in range(2)]
    acts_both = []
    for x_buf in x_both:
        views, taken = {}, 0
        for b in BATCHES:
            views[b] = [None, None, None]
            for j in (0, 2):  # gate and up read the same activations
                t = acts_src[b][j]
                views[b][j] = x_buf[taken:taken + t.numel()].view_as(t)
                views[b][j].copy_(t)
                taken += t.numel()
            views[b][1] = views[b][0]
        acts_both.append(views)
    acts, x_all = acts_both[0], x_both[0]
    del acts_src
    # gate and up read the same activations: neighbours in the list, one grouped launch
    lists = {b: ShardedGemvList([(acts[b][0], weights[0][0], fmt, SHAPES[0][1], SHAPES[0][2]),
                                 (acts[b][0], weights[0][1], fmt, SHAPES[1][1], SHAPES[1][2]),
                                 (acts[b][2], weights[0][2], fmt, SHAPES[2][1], SHAPES[2][2])],
                                arena, rank, world) for b in BATCHES}
    # The three batches of a step are independent of one another: the step issues all nine projections as ONE
    # list, so an N-sharded step waits for its peers once and signals them once (the per-batch lists above
    # serve the per-batch rows).
    step_list = ShardedGemvList([(acts[b][0 if j < 2 else 2], weights[0][j], fmt, SHAPES[j][1], SHAPES[j][2])
                                 for b in BATCHES for j in range(3)], arena, rank, world)
    launches_per_step = 2 * len(BATCHES)
    prepare_per_step = 1 if any(b > 1 for b in BATCHES) else 0  # ONE launch converts the batched activations of a list

    def step(slot, batches=BATCHES):
        if tuple(batches) == tuple(BATCHES):
            for i, b in enumerate(BATCHES):
                for j in range(3):
                    step_list.rebind(3 * i + j, x=acts_both[slot % 2][b][0 if j < 2 else 2], w=weights[slot][j])
            flat = step_list.forward()
            return {b: flat[3 * i:3 * i + 3] for i, b in enumerate(BATCHES)}
        outs = {}
        for b in batches:
            for j in range(3):
                lists[b].rebind(j, w=weights[slot][j])
            outs[b] = lists[b].forward()
        return outs

    def final_wait():
        if world > 1:
            ops.peer_sync(pads, rank, device, ops.PEER_WAIT)  # the peers' stores of the last launches have landed

    def capture(batches):
        graphs, outs = [], []
        with torch.cuda.stream(stream):
            step(0, batches)
            step(1, batches)
            stream.synchronize()
            for slot in range(ring):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    outs.append(step(slot, batches))
                graphs.append(g)
        return graphs, outs

    graphs, graph_outs = capture(BATCHES)

    # warm-up (also brings the clocks up), then the timed region with clock sampling
    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            graphs[i % ring].replay()
        final_wait()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms = timed_replays(graphs, args.steps, after=final_wait)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / args.steps
    value = step_bytes_total / (ms_per_step * 1e-3) / 1e9

    # ---- N-sharded outputs: identical on every rank, and this rank's columns equal a local launch ----
    sharded_ok = None
    if world > 1:
        ok = True
        with torch.cuda.stream(stream):
            graphs[0].replay()
            final_wait()
        barrier()
        for b in BATCHES:
            local = ShardedGemvList([(acts[b][0], weights[0][0], fmt, SHAPES[0][1] // world, SHAPES[0][2]),
                                     (acts[b][0], weights[0][1], fmt, SHAPES[1][1] // world, SHAPES[1][2]),
                                     (acts[b][2], weights[0][2], fmt, SHAPES[2][1] // world, SHAPES[2][2])])
            mine = local.forward()
            torch.cuda.synchronize(device)
            for j, (_, n, _) in enumerate(SHAPES):
                got = graph_outs[0][b][j]
                n_local = n // world
                ok &= bool(torch.equal(got[:, rank * n_local:(rank + 1) * n_local], mine[j]))
                ref = got.clone()
                dist.broadcast(ref, src=0)
                ok &= bool(torch.equal(ref, got))
        flag = torch.tensor([1 if ok else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        sharded_ok = bool(flag.item())

    # ---- per-batch rows (medians over several timed runs, outside the headline region) ----
    cases = []
    batch_graphs = {}
    for b in BATCHES:
        batch_graphs[b], _ = capture((b,))
        reps = max(40, args.steps)
        with torch.cuda.stream(stream):
            for i in range(6):
                batch_graphs[b][i % ring].replay()
        samples = [timed_replays(batch_graphs[b], reps, after=final_wait) / reps for _ in range(5)]
        t = statistics.median(samples)
        bytes_b = step_bytes_total // len(BATCHES)
        cases.append({"case": f"gate+up+down q4_k, batch {b}", "batch": b, "us": t * 1e3,
                      "gbps": bytes_b / (t * 1e-3) / 1e9,
                      "frac_of_hbm_peak": bytes_b / world / (t * 1e-3) / 1e9 / peaks["hbm_gbs"], "samples": len(samples)})

    # ---- roofline of the dominant kernel: the pipelined GEMV ----
    launch_bytes_local = set_bytes_local * len(BATCHES) / launches_per_step  # weight bytes of an average launch
    avg_launch_s = ms_per_step * 1e-3 / launches_per_step
    achieved = launch_bytes_local / avg_launch_s / 1e9
    best = max(cases, key=lambda c: c["gbps"])
    roofline = {
        "bound": "hbm", "kernel": "gemv_mma_kernel (bulk-copy ring + mma.sync)",
        "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
        "peak_source": peaks["source"],
        # dram__bytes_read.sum + dram__bytes_write.sum of one captured 38,191,104-byte launch
        # (profiles/gemv_q4k_batch1_18944x3584.md: 38,245,120 B, i.e. no re-reads), scaled to the weight
        # bytes of an average launch of this run (traffic is proportional to the rows streamed)
        "traffic": round(launch_bytes_local * 38265344 / 38191104),
        "algorithmic_bytes_per_launch": launch_bytes_local,
        "note": f"average over the {launches_per_step} GEMV launches of a step (batch 1/4/16, gate and up grouped "
                f"into one launch), gaps between launches included; best batch ({best['batch']}) reaches "
                f"{best['gbps'] / world:.0f} GB/s per GPU",
    }

    # ---- single-kernel rows: the first configuration of the definition and a Q6_K down projection ----
    def single_case(label, name, n, k, m, x_dtype, copies):
        f = tb.get_format(name)
        ws = [synth.make_weights(f, n, k, seed=300 + c, device=device) for c in range(copies)]
        x = synth.make_activations(m, k, seed=301, device=device, dtype=x_dtype)
        lst = ShardedGemvList([(x, ws[0], f, n, k)])
        with torch.cuda.stream(stream):
            lst.forward()
            stream.synchronize()
            g = torch.cuda.CUDAGraph()  # one graph over all the weight copies: launches back to back, as in a step
            with torch.cuda.graph(g, stream=stream):
                for c in range(copies):
                    lst.rebind(0, w=ws[c])
                    lst.forward()
        reps = 10
        samples = [timed_replays([g], reps) / (reps * copies) for _ in range(5)]
        t = statistics.median(samples)
        nbytes = f.weight_bytes(n, k)
        return {"case": label, "batch": m, "us": t * 1e3, "gbps": nbytes / (t * 1e-3) / 1e9,
                "frac_of_hbm_peak": nbytes / (t * 1e-3) / 1e9 / peaks["hbm_gbs"], "samples": len(samples)}

    if world == 1:
        cases.append(single_case("q8_0 4096x4096 fp16 (first configuration; gemv_dp4a_kernel)", "q8_0", 4096, 4096, 1, torch.float16, 24))
        cases.append(single_case("q6_k down 4096x12288 bf16 (gemv_dp4a_kernel)", "q6_k", 4096, 12288, 1, torch.bfloat16, 12))
        for b in BATCHES:
            cases.append(single_case(f"q4_k gate 18944x3584 alone, batch {b}", "q4_k", 18944, 3584, b, torch.bfloat16, 11))

    # ---- end to end: host buffers in, host buffers out, every step ----
    # one GPU: the whole result comes back; N-sharded: every rank reads back the columns it computed (its window
    # of each gathered output), so the host-side result is the concatenation of the ranks' buffers and the
    # read-back uses every GPU's own PCIe link instead of rank 0's alone
    def window(t):
        n_local = t.shape[1] // world
        return t[:, rank * n_local:(rank + 1) * n_local]

    x_host = x_all.cpu().pin_memory()
    y_elems = sum(window(o).numel() for b in BATCHES for o in graph_outs[0][b])
    y_stage = torch.empty(y_elems, dtype=torch.float32, device=device)  # a step's results, gathered for one copy out
    y_host = torch.empty(y_elems, dtype=torch.float32).pin_memory()
    h2d = x_host.numel() * x_host.element_size()
    d2h = y_elems * 4 * world  # all ranks together

    # Every step copies every activation in from pinned host memory (on every rank: activations are
    # replicated) and every result back out, on two side streams ordered by events.
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

    # The outputs and the activations exist in two copies that alternate from step to step, so a whole step goes
    # out as ONE graph launch, its results travel to the host while the next step computes into the other copy,
    # and the next step's activations arrive meanwhile.
    step_in = [torch.cuda.Event(), torch.cuda.Event()]
    step_done = [torch.cuda.Event(), torch.cuda.Event()]
    step_out = [torch.cuda.Event(), torch.cuda.Event()]

    def copy_in(par):
        with torch.cuda.stream(s_in):
            x_both[par].copy_(x_host, non_blocking=True)
            step_in[par].record(s_in)

    def e2e_step(i):
        par = i & 1                          # the ring is even: graph i % ring reads activation copy i & 1
        stream.wait_event(step_in[par])      # this step's inputs have arrived
        stream.wait_event(step_out[par])     # the output copy this step overwrites has been read out
        with torch.cuda.stream(stream):
            graphs[i % ring].replay()
            step_done[par].record(stream)
        # the next step's inputs, into the copy the previous step has finished reading
        s_in.wait_event(step_done[par ^ 1])
        copy_in(par ^ 1)
        # a rank's own columns are written by its own kernels: they are complete when its step is
        s_out.wait_event(step_done[par])
        with torch.cuda.stream(s_out):
            if world == 1:
                torch.cat([o.reshape(-1) for b in BATCHES for o in graph_outs[i % ring][b]], out=y_stage)
            else:
                gather[par].replay()
            y_host.copy_(y_stage, non_blocking=True)
            step_out[par].record(s_out)

    def e2e_drain():
        with torch.cuda.stream(stream):
            final_wait()
        for st in (stream, s_in, s_out):
            st.synchronize()

    # A step's results -> one contiguous staging buffer.  One GPU: the outputs are whole tensors and one
    # concatenation kernel gathers all nine (measured: nine separate copy kernels on the side stream cost the
    # GEMV chain 50 us per step).  N-sharded: this rank's window of an output is a strided view; one
    # concatenation per batch (three kernels) as one graph launch per output copy.
    torch.cuda.synchronize(device)
    gather = []
    if world > 1:
        for par in range(2):
            jobs, taken = [], 0
            for b in BATCHES:
                srcs = [window(o) for o in graph_outs[par][b]]
                cols = sum(t.shape[1] for t in srcs)
                jobs.append((srcs, y_stage[taken:taken + b * cols].view(b, cols)))
                taken += b * cols
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s_out):
                for srcs, dst in jobs:
                    torch.cat(srcs, dim=1, out=dst)
            gather.append(g)
        torch.cuda.synchronize(device)
    for ev in step_out:
        ev.record(s_out)
    step_done[1].record(stream)
    copy_in(0)
    for i in range(4):
        e2e_step(i)
    e2e_drain()
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    e2e_drain()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e = {"value": step_bytes_total * args.steps / e2e_s / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "note": "activations from pinned host memory on every rank and the results back to it, every step, on copy "
                   "streams ordered by events: one graph launch per step, the next step's activations arriving in a "
                   "second buffer meanwhile, its results (N-sharded: the columns each rank "
                   "computed; d2h bytes are the sum over ranks) read back while the next step computes into the other "
                   "copy of the outputs; weights resident"}

    # free the weight ring before the next parts
    del weights, graphs, batch_graphs, graph_outs
    torch.cuda.empty_cache()

    # ---- prefill GEMM beside its ceiling without decoding (dense bf16 GEMM on pre-dequantised weights) ----
    prefill = []
    for name, n, k in PREFILL:
        n_local = n // world
        copies = max(2, -(-2 * L2_BYTES // tb.weight_bytes(name, n_local, k)))
        ws = [synth.make_weights(name, n_local, k, seed=50 + c + rank, device=device) for c in range(copies)]
        dense = [tb.dequantize(w, name, n_local, k).to(torch.bfloat16) for w in ws]
        for m in PREFILL_M:
            x = synth.make_activations(m, k, seed=60 + m, device=device)
            out = torch.empty((m, n_local), dtype=torch.float32, device=device)
            kern = tb.gguf(m, n_local, k, name, op="gemm")
            reps = 20

            def run_ours():
                for c in range(reps):
                    kern.launch(x, ws[c % copies], out)

            def run_dense():
                for c in range(reps):
                    torch.matmul(x, dense[c % copies].t())

            row = {"format": name, "m": m, "n": n_local, "k": k}
            for key, fn in (("us", run_ours), ("ceiling_us", run_dense)):
                fn()
                torch.cuda.synchronize(device)
                samples = []
                for _ in range(3):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    fn()
                    e1.record()
                    torch.cuda.synchronize(device)
                    samples.append(e0.elapsed_time(e1) / reps * 1e3)
                row[key] = statistics.median(samples)
            row["tflops"] = 2.0 * m * n_local * k / (row["us"] * 1e-6) / 1e12
            row["frac_of_bf16_peak"] = row["tflops"] / peaks["bf16_tflops"]
            row["ceiling_tflops"] = 2.0 * m * n_local * k / (row["ceiling_us"] * 1e-6) / 1e12
            row["ceiling"] = "torch.matmul, bf16 operands and output, weights dequantised ahead of time (library GEMM, no decode)"
            prefill.append(row)
        del ws, dense
    torch.cuda.empty_cache()

    # ---- the 36-layer decode step: 252 projections per step as four launches per layer, two calls per layer ----
    decode_step = []
    if not args.skip_decode_step:
        layer_bytes = sum(tb.weight_bytes(f, n, k) for _, n, k, f, _ in LAYER)
        assert layer_bytes == sum(tb.weight_bytes(f, n, k) for _, n, k, f, _ in LAYER_FUSED)
        layer_w = [[synth.make_weights(f, n // world, k, seed=5000 + 10 * layer + j + 100 * rank, device=device)
                    for j, (_, n, k, f, _) in enumerate(LAYER_FUSED)] for layer in range(LAYERS)]
        step_arena = PeerArena(48 << 20, device, rank, world) if world > 1 else None
        step_pads = step_arena.pad_ptrs() if world > 1 else None
        for b in (1, 16):
            xs = {g: synth.make_activations(b, k, seed=40 + g, device=device)
                  for g, k in ((0, 4096), (1, 4096), (2, 4096), (3, 12288))}
            # the q4_k weights of a layer in one list, the q6_k down projection in its own
            q4 = ShardedGemvList([(xs[g], layer_w[0][j], f, n, k) for j, (_, n, k, f, g) in enumerate(LAYER_FUSED) if f == "q4_k"],
                                 step_arena, rank, world)
            q6 = ShardedGemvList([(xs[3], layer_w[0][3], "q6_k", LAYER_FUSED[3][1], LAYER_FUSED[3][2])], step_arena, rank, world)

            def whole_step():
                for layer in range(LAYERS):
                    for j in range(3):
                        q4.rebind(j, w=layer_w[layer][j])
                    q4.forward()
                    q6.rebind(0, w=layer_w[layer][3])
                    q6.forward()

            def step_wait():
                if world > 1:
                    ops.peer_sync(step_pads, rank, device, ops.PEER_WAIT)

            with torch.cuda.stream(stream):
                whole_step()
                stream.synchronize()
                gs = []
                for _ in range(2):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        whole_step()
                    gs.append(g)
                for i in range(2):
                    gs[i].replay()
                step_wait()
            reps = 6
            samples = [timed_replays(gs, reps, after=step_wait) / reps for _ in range(3)]
            t_ms = statistics.median(samples)
            # end to end: the step's input activations from pinned host memory on every rank, the last
            # projection's result back to the host on rank 0
            x_in = xs[0].cpu().pin_memory()
            y_out = torch.empty((b, LAYER[6][1]), dtype=torch.float32).pin_memory()
            last_out = q6.outputs(q6._copy)[0]  # an even number of calls per step: every step ends on the same copy
            barrier()
            t0 = time.perf_counter()
            with torch.cuda.stream(stream):
                for i in range(reps):
                    xs[0].copy_(x_in, non_blocking=True)
                    gs[i % 2].replay()
                    step_wait()
                    if rank == 0:
                        y_out.copy_(last_out, non_blocking=True)
                stream.synchronize()
            e2e_ms = max_over_ranks(time.perf_counter() - t0) / reps * 1e3
            total = layer_bytes * LAYERS
            decode_step.append({
                "batch": b, "layers": LAYERS, "projections": 7 * LAYERS, "weight_bytes": total,
                "ms": t_ms, "gbps": total / (t_ms * 1e-3) / 1e9,
                "frac_of_hbm_peak": total / world / (t_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                "e2e_ms": e2e_ms, "e2e_gbps": total / (e2e_ms * 1e-3) / 1e9,
                "launches_per_layer": 4,
                "note": "q/k/v, o, gate/up in Q4_K (gemv_mma_kernel), down in Q6_K (batch 1: gemv_dp4a_kernel, batch 16: "
                        "gemv_tc_kernel); the rows of q, k, v live in one 6144-row weight and those of "
                        "gate, up in one 24576-row weight (concatenated at load time), so a layer is four GEMV launches; "
                        "projections only (no attention or glue); 121.5 MB of distinct weights per layer, so every launch "
                        "streams from HBM"})
            del q4, q6, gs
        del layer_w
        torch.cuda.empty_cache()

    # ---- the 70B-class prefill sweep at M = 4096 ----
    big_prefill = []
    if not args.skip_big_prefill:
        m = BIG_PREFILL_M
        side = torch.cuda.Stream(device)
        compute = (torch.cuda.Stream(device), torch.cuda.Stream(device))
        for label, name, n, k in BIG_PREFILL:
            n_local = n // world
            w = synth.make_weights(name, n_local, k, seed=900 + rank, device=device)
            x = synth.make_activations(m, k, seed=901, device=device)
            out_local = torch.empty((m, n_local), dtype=torch.float32, device=device)
            kern = tb.gguf(m, n_local, k, name, op="gemm")
            flops = 2.0 * m * n * k
            chunks = 4 if world > 1 else 1
            mc = m // chunks
            kerns = tb.gguf(mc, n_local, k, name, op="gemm")
            gathered = out_full = None
            if world > 1:
                gathered = torch.empty((chunks, world, mc, n_local), dtype=torch.float32, device=device)
                out_full = torch.empty((m, n), dtype=torch.float32, device=device)
            events = [torch.cuda.Event() for _ in range(chunks)]

            def kernel_only():
                kern.launch(x, w, out_local)

            def with_gather():
                # The GEMM runs in chunks of rows that alternate between two compute streams, so two
                # chunks share the SMs at any time (a chunk alone would leave most of them idle where a
                # rank has few weight tiles); chunk i's all-gather and its rearrangement into row-major
                # [M, N] run on a side stream while the chunks after it compute.
                cur = torch.cuda.current_stream(device)
                for st in (compute[0], compute[1], side):
                    st.wait_stream(cur)
                for c in range(chunks):
                    st = compute[c & 1]
                    with torch.cuda.stream(st):
                        kerns.launch(x[c * mc:(c + 1) * mc], w, out_local[c * mc:(c + 1) * mc])
                        events[c].record(st)
                    side.wait_event(events[c])
                    with torch.cuda.stream(side):
                        dist.all_gather_into_tensor(gathered[c].view(world * mc, n_local), out_local[c * mc:(c + 1) * mc])
                        out_full[c * mc:(c + 1) * mc].view(mc, world, n_local).copy_(gathered[c].permute(1, 0, 2))
                for st in (compute[0], compute[1], side):
                    cur.wait_stream(st)

            row = {"projection": label, "format": name, "m": m, "n": n, "k": k, "n_local": n_local}
            for key, fn in (("kernel_us", kernel_only), ("gathered_us", with_gather)):
                if key == "gathered_us" and world == 1:
                    continue
                for _ in range(2):
                    fn()
                barrier()
                samples = []
                for _ in range(3):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(3):
                        fn()
                    e1.record()
                    barrier()
                    samples.append(max_over_ranks(e0.elapsed_time(e1)) / 3 * 1e3)
                row[key] = statistics.median(samples)
            row["kernel_tflops"] = flops / (row["kernel_us"] * 1e-6) / 1e12
            row["kernel_frac_of_bf16_peak"] = row["kernel_tflops"] / world / peaks["bf16_tflops_sustained"]
            row["peak"] = "sustained bf16 (a kernel of a millisecond runs under the power cap)"
            if world > 1:
                row["gathered_tflops"] = flops / (row["gathered_us"] * 1e-6) / 1e12
                recv = (world - 1) * m * n_local * 4
                row["gather_bytes_received_per_gpu"] = recv
                row["gather_floor_us_at_770GBs"] = recv / 770e9 * 1e6
                row["note"] = ("N-sharded; the GEMM runs in 4 chunks of rows on two alternating streams, each chunk's fp32 output "
                               "is all-gathered with NCCL on a side stream and rearranged to row-major [M, N]; the floor is the "
                               "bytes a GPU must receive over NVLink")
            big_prefill.append(row)
            del w, x, out_local, gathered, out_full
        torch.cuda.empty_cache()

    status = tb.device_status()
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16 mma / f32 accumulate", "data": "synthetic",
        "config": workload_config(world), "clocks": clocks, "e2e": e2e,
        "gpu_launches": (launches_per_step + prepare_per_step) * args.steps + (1 if world > 1 else 0),
        "roofline": roofline, "cases": cases, "prefill": prefill, "decode_step": decode_step,
        "prefill_70b": big_prefill, "cuda_graphs": True, "device_status": status,
    }
    if sharded_ok is not None:
        line["sharded_outputs_ok"] = sharded_ok
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rate, cores, n_steps, med, _ = cpu_port_gemv_rate(10.0)
        line["cpu_baseline"] = {
            "value": rate, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"the same nine GEMVs as a GPU step, {n_steps} passes, median {med * 1e3:.1f} ms per pass"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    failed = sharded_ok is False or status != 0
    if world > 1:
        # Every collective of this run has completed on every rank (the last one returned a value to
        # the host).  Tearing the NCCL communicator down while CUDA graphs that captured its kernels
        # are alive was seen to block, so leave without the teardown.
        torch.cuda.synchronize(device)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(1 if failed else 0)
    if failed:
        raise SystemExit(1)


def run_single(args):
    """One kernel at one shape, launched plainly over enough distinct weight copies to exceed the L2: the
    launch sequence to time a shape outside the step, and small enough to hand to a profiler."""
    import torch

    import tensor_b200 as tb
    from tensor_b200 import synth

    parts = args.single.split(":")
    if len(parts) not in (5, 6) or parts[0] not in ("gemv", "gemm"):
        raise SystemExit("--single takes gemv|gemm:FORMAT:M:N:K[:VARIANT]")
    op, name, (m, n, k) = parts[0], parts[1], (int(v) for v in parts[2:5])
    variant = parts[5] if len(parts) == 6 else "auto"
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    fmt = tb.get_format(name)
    nbytes = fmt.weight_bytes(n, k)
    copies = max(2, min(16, -(-(L2_BYTES * 3 // 2) // nbytes)))
    weights = [synth.make_weights(fmt, n, k, seed=500 + c, device=device) for c in range(copies)]
    x_dtype = torch.float16 if args.single_dtype == "float16" else torch.bfloat16
    x = synth.make_activations(m, k, seed=501, device=device, dtype=x_dtype)
    out = torch.empty(m, n, device=device)
    kernel = tb.gguf(m, n, k, fmt, op=op, variant=variant, x_dtype=args.single_dtype)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for w in weights[:2]:
        kernel.launch(x, w, out)
    torch.cuda.synchronize(device)
    start.record()
    for _ in range(args.single_rounds):
        for w in weights:
            kernel.launch(x, w, out)
    stop.record()
    torch.cuda.synchronize(device)
    us = start.elapsed_time(stop) * 1e3 / (args.single_rounds * copies)
    line = {"single": args.single, "x_dtype": args.single_dtype, "us_per_launch": us, "weight_copies": copies,
            "launches": 2 + args.single_rounds * copies, "device_status": tb.device_status()}
    if op == "gemv":
        line["weight_gbps"] = nbytes / us / 1e3
    else:
        line["tflops"] = 2.0 * m * n * k / us / 1e6
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="native", choices=("native", "reference"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-decode-step", action="store_true", help="leave the 36-layer decode step out")
    ap.add_argument("--skip-big-prefill", action="store_true", help="leave the 70B-class prefill sweep out")
    ap.add_argument("--single", default=None, metavar="OP:FORMAT:M:N:K[:VARIANT]",
                    help="time one kernel at one shape with plain launches (e.g. gemv:q4_k:1:18944:3584) and exit")
    ap.add_argument("--single-dtype", default="bfloat16", choices=("bfloat16", "float16"))
    ap.add_argument("--single-rounds", type=int, default=1, help="passes over the weight copies of --single")
    args = ap.parse_args()
    if args.single:
        run_single(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
