#!/usr/bin/env python
"""Benchmark of the attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One step = one pass of the hot path (esp_attn_forward: attention kernel + combine) over one
batch of seeded synthetic input with the shapes of the benchmark configuration. The default
workload is the batched paged decode (32 sequences per GPU, context ~ U[512, 32768],
H32/Hkv4/HD128 bf16, 16-token pages scattered by a seeded page table); the metric is the
HBM bandwidth the pass achieves = algorithmic K/V bytes / time. With N > 1 (torchrun, one
process per GPU) every rank runs its own batch: the path shards by sequence, there is no
collective on the data path ("scaling": "weak"). The split-KV workload (c5) is the one path
with an exchange step: ranks all-gather their partial records (NCCL) and combine locally.

`--impl reference` times the CPU restatement of the reference's kernels (oracle/) on the
host cores instead; the reference itself is Metal-only and cannot run on this box.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode_attn_hbm_bandwidth"
UNIT = "GB/s"

# per workload: query rows per tile, and what the roofline counts
TILE_ROWS = {"c1": 8, "c2": 8, "c3": 128, "c4": 16, "c5": 8}


def attention_flops(w) -> float:
    """Algorithmic flops of one pass: 2 flop per MAC, Q.K^T and P.V, over the visible (row, key)
    pairs (cached keys + causal / ancestor batch keys)."""
    pairs = 0
    for i, t in enumerate(w.trees):
        P, M = int(t["P"]), int(t["M"])
        if w.anc_mask is not None and (w.flags & 2):
            base = int(t["base"])
            vis = sum(bin(int(w.anc_mask[base + r])).count("1") for r in range(M))
        else:
            vis = M * (M + 1) // 2
        pairs += M * P + vis
    return 4.0 * pairs * w.H * w.HD


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            measured_peaks.sustained_tflops = float(d.get("bf16_tflops_sustained", 0.0)) or None
            return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
        except Exception:
            pass
    return 6650.0, 1590.0, "fallback"


measured_peaks.sustained_tflops = None


def build_workload(name: str, rank: int, small: bool = False, world: int = 1):
    from espetero_b200 import shard, workloads as wl
    seed_shift = 1000 * rank
    if name == "c1":
        return wl.config_c1(0xE5B201 + seed_shift)
    if name == "c2":
        n, hi = (4, 4096) if small else (32, 32768)
        if world == 1:
            return wl.config_c2(0xE5B202, n_seqs=n, hi=hi)
        # The box serves world x 32 sequences: every rank's draw of the configuration, spread over
        # the GPUs by total context length (longest first onto the least loaded GPU), as a
        # scheduler that batches by KV footprint would. Whole sequences move; nothing is exchanged.
        lens = np.concatenate([wl.c2_context_lengths(0xE5B202 + 1000 * r, n, 512, hi) for r in range(world)])
        mine = shard.lpt_partition(lens, world)[rank]
        return wl.config_c2(0xE5B202 + seed_shift, lens=lens[mine])
    if name == "c4":
        return wl.config_c4(0xE5B204 + seed_shift, n_seqs=2 if small else 16, prefix=512 if small else 4096)
    if name == "c5":
        return wl.config_c5(0xE5B205 + seed_shift, ctx=8192 if small else 131072)
    if name == "c3":
        return wl.config_c3(0xE5B203 + seed_shift, n_seqs=1 if small else 4, rows=2048 if small else 8192)
    raise SystemExit(f"unknown workload {name}")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region (read-only query)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                       "-i", str(self.gpu)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.p is None:
            return out
        time.sleep(0.15)
        self.p.terminate()  # the exact process started above
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm))
        try:
            os.unlink(self.f.name)
        except OSError:
            pass
        return out


def cpu_sample_workload(name: str):
    """A bounded sample of the workload for the CPU arm (about 10-30 s of host work)."""
    from espetero_b200 import workloads as wl
    if name == "c2":
        return wl.config_c2(0xE5B202, n_seqs=32, hi=32768), "the full batch: 32 sequences, context ~ U[512, 32768]"
    if name == "c1":
        return wl.config_c1(), "full"
    if name == "c4":
        return wl.config_c4(), "full"
    if name == "c5":
        return wl.config_c5(), "full"
    return wl.config_c3(n_seqs=1, rows=1024), "1 sequence x 1024 rows"


_CPU_CASES = {}


def time_cpu(name: str, repeats: int = 1):
    """Time the multithreaded fp32 restatement of the reference kernels (oracle/) on the host.
    The workload and its plan are built once per process; only the kernels are timed."""
    import oracle
    if name not in _CPU_CASES:
        w, sample = cpu_sample_workload(name)
        _CPU_CASES[name] = (w, sample, oracle.plan_tiles(w.trees, w.Hkv, split=512))
    w, sample, (tiles, jobs, nparts) = _CPU_CASES[name]
    threads = oracle.hw_threads()
    single = all(int(t["M"]) == 1 for t in w.trees)
    fn = oracle.decode_gqa_f32 if single else oracle.flash_f32
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        O, lse, parts = fn(w, tiles, 8, nparts, threads)
        if len(jobs):
            oracle.combine_f32(w, parts, jobs, O, lse, 8, threads)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return w.kv_bytes_read() / best / 1e9, threads, sample, best


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # the CPU arm runs on rank 0 alone
    steps = max(1, args.steps)
    vals = []
    for _ in range(min(args.warmup, 1)):
        time_cpu(args.workload)
    t_all = 0.0
    for _ in range(steps):
        v, threads, sample, dt = time_cpu(args.workload)
        vals.append(v)
        t_all += dt
    value = float(np.mean(vals))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * t_all / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": _CPU_CASES[args.workload][0].name, "note": "CPU restatement of the reference's Metal kernels (oracle/), fp32, std::thread"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# DRAM bytes (read + write) of one launch of the dominant kernel on each bench workload, from the
# ncu captures summarised under profiles/ (decode_gqa_c2_batched_decode.md, decode_gqa_c5_long_fp8_decode.md,
# flash_umma_c4_tree_verify.md, flash_umma_pair_c3_causal_prefill.md). A capture cannot run inside a
# timed run, so the figure is carried here; it holds for the default sizes of the workload only.
# The prefill workload was captured on a smaller case only and is tensor-bound: no figure.
NCU_TRAFFIC_BYTES = {"c2": 1.12084e9 + 12.20e6, "c5": 537.83e6 + 4.29e6, "c4": 136.96e6 + 4.32e6}


L2_BYTES = 126e6


class LayerCycle:
    """Keeps the keys of a pass out of L2 between timed steps the way a model does: the pool holds
    one region per attention layer and consecutive passes read consecutive layers. A workload whose
    K/V bytes are below 2 x L2 gets as many layer regions (copies of its pool) as make the cycle
    at least 4 x L2 long, and step i reads region i mod n; nothing is flushed and nothing else runs
    between the timed steps. Larger workloads evict themselves with one region."""

    def __init__(self, op, dp, w):
        self.op, self.dp, self.w = op, dp, w
        nbytes = max(1, w.kv_bytes_read())
        self.n = 1 if nbytes >= 2 * L2_BYTES else min(64, int(-(-4 * L2_BYTES // nbytes)))
        self.region = dp.replicate_layers(self.n)
        self.i = 0

    def args(self, n_jobs=None):
        a = self.op.make_args(self.dp)
        if n_jobs is not None:
            a.n_jobs = n_jobs
        return a

    def next(self, a):
        a.p.kv_base = self.w.kv_base + (self.i % self.n) * self.region
        self.i += 1
        return a

    def describe(self):
        if self.n == 1:
            return "inputs larger than L2"
        return (f"{self.n} layer regions of the pool read in turn ({self.n * self.w.kv_bytes_read() / 1e6:.0f} MB per cycle, "
                f"L2 is 126 MB): a pass reads keys last touched {self.n - 1} passes ago; no flush kernels")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--small", action="store_true", help="reduced sizes (profiling captures)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"], help="split-KV record exchange at N > 1 (c5)")
    ap.add_argument("--fuse", type=int, default=-1, help="option fuse_combine of the library (0 off, 1 small passes, 2 always); -1: its default")
    ap.add_argument("--groups", type=int, default=0, help="CTA target of the planner (default 8 waves of 2 CTAs per SM)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    import torch.distributed as dist
    from espetero_b200 import capi, host, workloads as wl

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU implementation")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    W = max(3, args.warmup)

    from espetero_b200 import shard
    tile_rows = TILE_ROWS[args.workload]
    split_kv = args.workload == "c5" and world > 1
    groups = args.groups or {"c4": 148, "c5": 148 * 2}.get(args.workload, 148 * 2 * 8)
    xch = None
    if not split_kv:
        w = build_workload(args.workload, rank, args.small, world)
        op = host.AttnOp.for_workload(w, tile_rows, local)
        if args.fuse >= 0:
            op.set_option("fuse_combine", args.fuse)
        plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, groups, tile_rows)
        dp = op.upload(w, plan)
        layers = LayerCycle(op, dp, w)
        a_full = layers.args()
        a_attn = layers.args(n_jobs=0)  # attention kernel alone (no combine), for the per-kernel roofline figure
        step = lambda: op.forward(dp, layers.next(a_full))
        step_attn = lambda: op.forward(dp, layers.next(a_attn))
        sharding = "sequences per rank, no collective" + (
            "; the box's batch spread by total context length (LPT)" if world > 1 and args.workload == "c2" else "")
        scaling = "weak"
    else:
        # One long sequence, keys split over the ranks on page boundaries: records for the local
        # keys -> one reduced record per rank -> NCCL all-gather -> every rank merges the world's
        # records in rank order. Total work is fixed: strong scaling.
        ctx_all = 8192 if args.small else 131072
        lo, hi = shard.split_kv_range(ctx_all, world, 16)[rank]
        w = wl.config_c5(0xE5B205 + 1000 * rank, ctx=hi - lo)
        op = host.AttnOp.for_workload(w, tile_rows, local)
        base_plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, args.groups or 148 * 2, tile_rows)
        tiles, red_jobs, n_parts = shard.local_decode_plan(base_plan.tiles, is_last_rank=(rank == world - 1))
        plan = host.Plan(tiles, np.zeros(0, dtype=wl.COMBINE_DT), n_parts, tile_rows)
        dp = op.upload(w, plan)
        for t in (dp.Q, dp.Kb, dp.Vb):  # the query row is replicated: every rank uses rank 0's
            dist.broadcast(t.view(torch.uint8), src=0)  # NCCL has no 16-bit integer type
        layers = LayerCycle(op, dp, w)
        a_attn = layers.args()
        a_full = a_attn
        red_dev = host._dev(red_jobs, dev)
        merge_dev = host._dev(shard.world_merge_jobs(1, world), dev)
        rec_local = torch.zeros(op.parts_floats(1), dtype=torch.float32, device=dev)
        rec_world = torch.zeros(world * op.parts_floats(1), dtype=torch.float32, device=dev)

        # Preferred: one kernel per rank reduces, stores the record into every rank's buffer over
        # NVLink peer mappings and merges (esp_attn_exchange_parts). If the peer mappings cannot be
        # set up on this box (all ranks decide together), the records go through an NCCL all-gather.
        if args.exchange == "p2p":
            try:
                xch = host.PeerExchange(op, n_jobs=1, rows_max=1)
                ok = 1
            except Exception as e:  # noqa: BLE001 - reported below, then the NCCL path is used
                print(f"[rank {rank}] peer exchange unavailable: {e}", file=sys.stderr, flush=True)
                ok = 0
            flag = torch.tensor([ok], dtype=torch.int32, device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 0:
                xch = None

        if xch is not None:
            def step():
                xch.next_epoch()
                op.forward(dp, layers.next(a_attn))
                op.exchange_parts(dp, dp.parts, red_dev, len(red_jobs), xch, parts_max=n_parts)
            sharding = "KV range per rank; one kernel per rank merges, exchanges records over NVLink peer stores and finishes"
        else:
            def step():
                op.forward(dp, layers.next(a_attn))
                op.reduce_parts(dp, dp.parts, red_dev, len(red_jobs), rec_local, 0)
                dist.all_gather_into_tensor(rec_world, rec_local)
                op.combine(dp, rec_world, merge_dev, 1)
            sharding = "KV range per rank; reduced records all-gathered (NCCL), merged on every rank"
        step_attn = lambda: op.forward(dp, layers.next(a_attn))
        scaling = "strong"
    bytes_step = w.kv_bytes_read()
    stream = torch.cuda.current_stream(dev)
    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, n, tail=None):
        """Seconds for n calls of fn: CUDA events on the launching stream, barrier + synchronize on both sides.
        tail() runs before the closing event (it makes the launching stream wait for work on other streams)."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n):
            fn()
        if tail is not None:
            tail()
        e1.record(stream)
        barrier()
        return e0.elapsed_time(e1) / 1e3

    # ---- device-resident throughput (value)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(W):
        step()
    op.check_status()
    n0 = op.launch_count
    t_total = timed(step, args.steps)
    launches = op.launch_count - n0
    # ---- attention kernel alone (roofline of the dominant kernel)
    for _ in range(3):
        step_attn()
    t_attn = timed(step_attn, args.steps) / args.steps
    # nvidia-smi samples every 100 ms: keep the same kernels running (untimed) until it has seen the
    # GPU under this load for about half a second, on every rank alike
    # (a fixed number of steps derived from rank 0's timing, so that ranks which exchange records
    # inside a step all run the same count)
    hold = torch.tensor([min(20000, int(0.6 / max(t_total / args.steps, 1e-6)) + 1)], dtype=torch.int64, device=dev)
    if world > 1:
        dist.broadcast(hold, src=0)
    for _ in range(int(hold.item())):
        step()
    torch.cuda.synchronize(dev)
    clocks = sampler.stop() if rank == 0 else None
    op.check_status()

    # ---- end to end through the C ABI from host buffers: the step's inputs (Q, Kb, Vb and the
    # plan tables) come from pinned host memory, the result goes back; the KV pool is device state.
    arena = host.StepArena(dp)
    a_e2e = arena.patch(op.make_args(dp))
    h_out = torch.empty_like(dp.O, device="cpu").pin_memory()
    h2d = arena.nbytes
    d2h = h_out.numel() * h_out.element_size()

    if split_kv:
        a_attn.Q, a_attn.Kb, a_attn.Vb = a_e2e.Q, a_e2e.Kb, a_e2e.Vb  # the step reads its inputs from the arena
        a_attn.tiles, a_attn.trees, a_attn.blocks = a_e2e.tiles, a_e2e.trees, a_e2e.blocks

    e2e_tail = None
    # Passes of a few microseconds are bound by the host's calls, not by the GPU: pipelining them over
    # three streams only adds calls, so they keep the plain sequence on one stream.
    sequential = split_kv or t_total / args.steps < 25e-6
    if sequential:
        def step_e2e():
            arena.upload()
            if split_kv:
                step()
            else:
                op.forward(dp, layers.next(a_e2e))
            h_out.copy_(dp.O, non_blocking=True)
        e2e_note = "Q/Kb/Vb + plan tables in one arena copied from pinned host memory, O back to the host; the KV pool is resident device state"
    else:
        # Every step copies its own inputs up and its own result down; the steps are pipelined over two
        # sets of buffers and three streams, so the copies of step i + 1 cross PCIe while step i computes
        # (an engine prepares the next batch while the GPU is busy). The closing event waits for the last
        # result to be on the host.
        arenas = [arena, host.StepArena(dp)]
        outs = [dp.O, torch.zeros_like(dp.O)]
        lses = [dp.lse, torch.zeros_like(dp.lse)]
        h_outs = [h_out, torch.empty_like(h_out).pin_memory()]
        a_bufs = []
        for k in range(2):
            ak = arenas[k].patch(op.make_args(dp))
            ak.O, ak.lse = outs[k].data_ptr(), lses[k].data_ptr()
            a_bufs.append(ak)
        copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        ready = [torch.cuda.Event() for _ in range(2)]
        done = [torch.cuda.Event() for _ in range(2)]
        fetched = [torch.cuda.Event() for _ in range(2)]
        turn = [0]

        def step_e2e():
            k = turn[0] & 1
            turn[0] += 1
            copy_in.wait_event(done[k])          # the kernels of step i - 2 have read this arena
            with torch.cuda.stream(copy_in):
                arenas[k].upload()
                ready[k].record(copy_in)
            stream.wait_event(ready[k])
            stream.wait_event(fetched[k])        # the result of step i - 2 has left this O buffer
            op.forward(dp, layers.next(a_bufs[k]))
            done[k].record(stream)
            copy_out.wait_event(done[k])
            with torch.cuda.stream(copy_out):
                h_outs[k].copy_(outs[k], non_blocking=True)
                fetched[k].record(copy_out)

        def e2e_tail():
            for ev in fetched:
                stream.wait_event(ev)
        e2e_note = ("Q/Kb/Vb + plan tables in one arena copied from pinned host memory, O back to the host, every step; two buffer sets, "
                    "copies of step i+1 overlap the kernels of step i; the KV pool is resident device state")
    for _ in range(3):
        step_e2e()
    t_e2e = timed(step_e2e, args.steps, e2e_tail)

    # ---- aggregate over ranks: max time, summed bytes
    tt = torch.tensor([t_total, t_attn, t_e2e], dtype=torch.float64, device=dev)
    bb = torch.tensor([float(bytes_step)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dist.all_reduce(bb, op=dist.ReduceOp.SUM)
    t_total, t_attn_max, t_e2e = [float(x) for x in tt.cpu()]
    bytes_all = float(bb.cpu()[0])

    if rank == 0:
        hbm_peak, tf_peak, which = measured_peaks()
        value = bytes_all * args.steps / t_total / 1e9
        achieved = bytes_step / t_attn / 1e9
        flops = attention_flops(w)
        traffic = NCU_TRAFFIC_BYTES.get(args.workload) if not (args.small or split_kv) else None
        tensor = {"tflops": flops / t_attn / 1e12, "peak_tflops": tf_peak, "frac": flops / t_attn / 1e12 / tf_peak,
                  "flops_per_step": flops}
        if measured_peaks.sustained_tflops:  # the denominator for a kernel timed inside a long, power-capped run
            tensor["peak_tflops_sustained"] = measured_peaks.sustained_tflops
            tensor["frac_of_sustained"] = tensor["tflops"] / measured_peaks.sustained_tflops
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": W,
            "ms_per_step": 1e3 * t_total / args.steps, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "bf16" if w.kv_dtype != wl.E4M3 else "e4m3->f16", "data": "synthetic",
            "config": {"workload": w.name, "sequences_per_gpu": len(w.trees), "H": w.H, "Hkv": w.Hkv, "HD": w.HD, "page": w.bt,
                       "kv_bytes_per_gpu": bytes_step, "tiles": len(plan.tiles), "parts": plan.n_parts, "kernel": op.last_kernel,
                       "l2": layers.describe(),
                       "sharding": sharding},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "traffic": traffic, "peak_source": which, "kernel": op.last_kernel, "ms_per_launch": 1e3 * t_attn},
            "e2e": {"value": bytes_all * args.steps / t_e2e / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": e2e_note},
            "gpu_launches": int(launches), "clocks": clocks, "tensor": tensor,
        }
        if args.workload == "c3":  # the prefill configuration is bound by the tensor cores, not by HBM
            line["metric"], line["unit"] = "prefill_attn_tflops", "TFLOP/s"
            line["value"] = flops * world * args.steps / t_total / 1e12
            line["roofline"] = {"bound": "tensor", "achieved": tensor["tflops"], "peak": tf_peak, "unit": "TFLOP/s",
                                "frac": tensor["frac"], "traffic": traffic, "peak_source": which, "kernel": op.last_kernel,
                                "ms_per_launch": 1e3 * t_attn}
            line["e2e"]["value"] = flops * world * args.steps / t_e2e / 1e12
            line["e2e"]["unit"] = "TFLOP/s"
        if world == 1 and not args.no_cpu:
            v, threads, sample, dt = time_cpu(args.workload)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample, "seconds": dt}
        print(json.dumps(line), flush=True)
    if xch is not None:
        xch.close()
    op.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
