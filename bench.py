#!/usr/bin/env python
"""Benchmark of the attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One step = one pass of the hot path (esp_attn_forward: attention kernel + merge of the split-K
records) over one batch of seeded synthetic input with the shapes of the benchmark configuration.
The default workload is the batched paged decode (32 sequences per GPU, context ~ U[512, 32768],
H32/Hkv4/HD128 bf16, 16-token pages scattered by a seeded page table); the metric is the HBM
bandwidth the pass achieves = algorithmic K/V bytes / time. With N > 1 (torchrun, one process per
GPU) every rank runs its own batch: the path shards by sequence, there is no collective on the data
path ("scaling": "weak"). The default run at N > 1 also times, and reports inside the same JSON
line, the two strong-scaling cases: the one 32-sequence batch spread over the N GPUs by context
length ("c2_strong") and the long-context decode with its keys split over the GPUs by range
("split_kv"). That last one is the only path with an exchange step: one kernel per rank reduces its
records, stores the result into every rank's buffer over NVLink peer mappings and finishes the
merge (esp_attn_exchange_parts); `--exchange nccl` gathers the reduced records with a library
all-gather instead, which is also the fallback when peer mappings cannot be set up.

At N = 1 the pass's output is also compared with the float64 oracle after the timed region
("parity" in the line; `--no-check` skips it).

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
    win = w.extra.get("window") if isinstance(getattr(w, "extra", None), dict) else None
    if win and win["window"] > 0:  # causal rows at positions P + r behind P cached keys, `window` positions visible
        for t in w.trees:
            P, M = int(t["P"]), int(t["M"])
            pairs += int(np.minimum(P + np.arange(M) + 1, win["window"]).sum())
        return 4.0 * pairs * w.H * w.HD
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


def build_workload(name: str, rank: int, small: bool = False, world: int = 1, kv: str = "", window: int = 0, hd: int = 128):
    from espetero_b200 import shard, workloads as wl
    seed_shift = 1000 * rank
    if name == "c1":
        return wl.config_c1(0xE5B201 + seed_shift)
    if name == "c2":
        n, hi = (4, 4096) if small else (32, 32768)
        if world == 1:
            return wl.config_c2(0xE5B202, n_seqs=n, hi=hi, hd=hd, kv_dtype=wl.E4M3 if kv == "e4m3" else None)
        # The box serves world x 32 sequences: every rank's draw of the configuration, spread over
        # the GPUs by total context length (longest first onto the least loaded GPU), as a
        # scheduler that batches by KV footprint would. Whole sequences move; nothing is exchanged.
        lens = np.concatenate([wl.c2_context_lengths(0xE5B202 + 1000 * r, n, 512, hi) for r in range(world)])
        mine = shard.lpt_partition(lens, world)[rank]
        return wl.config_c2(0xE5B202 + seed_shift, lens=lens[mine])
    if name == "c4":
        return wl.config_c4(0xE5B204 + seed_shift, n_seqs=2 if small else 16, prefix=512 if small else 4096,
                            kv_dtype=wl.E4M3 if kv == "e4m3" else None, hd=hd)
    if name == "c5":
        return wl.config_c5(0xE5B205 + seed_shift, ctx=8192 if small else 131072)
    if name == "c3":
        n, rows = (1, 2048) if small else (4, 8192)
        if window > 0:  # the same prefill through a sliding-window layer (not one of the five configurations)
            H, Hkv = 8192 // hd, 1024 // hd
            return wl.make_window_pass("c3_causal_prefill_window" + (f"_hd{hd}" if hd != 128 else ""), 0xE5B203 + seed_shift, [(0, rows)] * n,
                                       H, Hkv, hd, 16, wl.BF16, window, scale=hd ** -0.5)
        return wl.config_c3(0xE5B203 + seed_shift, n_seqs=n, rows=rows, hd=hd)
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


CPU_SAMPLE_HD = 128  # --hd: the CPU arm times the same head dim


def cpu_sample_workload(name: str):
    """A bounded sample of the workload for the CPU arm (about 10-30 s of host work)."""
    from espetero_b200 import workloads as wl
    hd = CPU_SAMPLE_HD
    if name == "c2":
        return wl.config_c2(0xE5B202, n_seqs=32, hi=32768, hd=hd), "the full batch: 32 sequences, context ~ U[512, 32768]"
    if name == "c1":
        return wl.config_c1(), "full"
    if name == "c4":
        return wl.config_c4(hd=hd), "full"
    if name == "c5":
        return wl.config_c5(), "full"
    return wl.config_c3(n_seqs=1, rows=4096, hd=hd), "1 sequence x 4096 rows (a 16th of the pass's flops)"


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
    if name == "c3":  # the prefill configuration is counted in flops (its cached keys are none)
        return attention_flops(w) / best / 1e12, threads, sample, best
    return w.kv_bytes_read() / best / 1e9, threads, sample, best


def l2_note(w) -> str:
    """How the keys of a pass are kept out of L2 between timed steps (see LayerCycle)."""
    n = layer_regions(w)
    if n == 1:
        return "inputs larger than L2"
    return (f"{n} layer regions of the pool read in turn ({n * w.kv_bytes_read() / 1e6:.0f} MB per cycle, "
            f"L2 is 126 MB): a pass reads keys last touched {n - 1} passes ago; no flush kernels")


def workload_config(w):
    """The `config` object of a JSON line: what the workload is, identical on the GPU arm and on the
    reference arm (what each arm ran it with is reported beside it, in `plan` / `cpu_baseline`)."""
    return {"workload": w.name, "sequences_per_gpu": len(w.trees), "H": w.H, "Hkv": w.Hkv, "HD": w.HD, "page": w.bt,
            "kv_bytes_per_gpu": w.kv_bytes_read(), "l2": l2_note(w)}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # the CPU arm runs on rank 0 alone
    steps = max(1, args.steps)
    W = max(0, args.warmup)
    vals = []
    for _ in range(W):
        time_cpu(args.workload)
    t_all = 0.0
    for _ in range(steps):
        v, threads, sample, dt = time_cpu(args.workload)
        vals.append(v)
        t_all += dt
    value = float(np.mean(vals))
    w = _CPU_CASES[args.workload][0]
    METRIC, UNIT = ("prefill_attn_tflops", "TFLOP/s") if args.workload == "c3" else (globals()["METRIC"], globals()["UNIT"])
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": W, "ms_per_step": 1e3 * t_all / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if w.kv_elem_bytes == 2 else "e4m3->f16", "data": "synthetic",
        "config": workload_config(w),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                         "what": "CPU restatement of the reference's Metal kernels (oracle/), fp32, std::thread, rank 0's host cores"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# DRAM bytes (read + write) of one launch of the dominant kernel on each bench workload, from one ncu
# capture per workload (a capture cannot run inside a timed run, so the figure is carried here; it holds
# for the default sizes of the workload only). The prefill workload was captured on a smaller case
# only and is tensor-bound: no figure.
NCU_TRAFFIC_BYTES = {"c2": 1.12084e9 + 12.20e6, "c5": 537.83e6 + 4.29e6, "c4": 136.96e6 + 4.32e6}


L2_BYTES = 126e6


def layer_regions(w) -> int:
    """Layer regions the pool of a workload is given: one if its K/V bytes evict themselves from L2
    (>= 2 x L2), else as many copies as make one cycle at least 4 x L2 long."""
    nbytes = max(1, w.kv_bytes_read())
    return 1 if nbytes >= 2 * L2_BYTES else min(64, int(-(-4 * L2_BYTES // nbytes)))


class LayerCycle:
    """Keeps the keys of a pass out of L2 between timed steps the way a model does: the pool holds
    one region per attention layer and consecutive passes read consecutive layers. A workload whose
    K/V bytes are below 2 x L2 gets as many layer regions (copies of its pool) as make the cycle
    at least 4 x L2 long, and step i reads region i mod n; nothing is flushed and nothing else runs
    between the timed steps. Larger workloads evict themselves with one region."""

    def __init__(self, op, dp, w):
        self.op, self.dp, self.w = op, dp, w
        self.n = layer_regions(w)
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
        return l2_note(self.w)


def default_groups(name: str) -> int:
    """CTA target of the planner per workload: one wave for the short passes, 8 waves of 2 CTAs per SM otherwise."""
    return {"c4": 148, "c5": 148 * 2}.get(name, 148 * 2 * 8)


def bench_plan(name: str, w, groups: int = 0):
    """The plan the bench runs a workload with (the full-size parity tests use the same one)."""
    from espetero_b200 import capi, host
    tile_rows = TILE_ROWS[name]
    win = w.extra.get("window") if isinstance(getattr(w, "extra", None), dict) else None
    if win and win["window"] > 0:  # the generic planner's window branch, with tcgen05-sized tiles
        return host.plan_window(w.trees, groups=w.Hkv, split=512, rows=tile_rows, window=win["window"], pos=win["pos"])
    return host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, groups or default_groups(name), tile_rows)


def parity_rows(name: str, w):
    """Rows compared with the float64 oracle: all of them, except for the prefill workload, whose
    full float64 result is ~1e13 flop: there the first and last 16 rows of every sequence plus 256
    seeded rows, all heads."""
    if name != "c3":
        return None
    rows = set()
    for t in w.trees:
        b, M = int(t["base"]), int(t["M"])
        rows.update(range(b, b + min(16, M)))
        rows.update(range(b + max(0, M - 16), b + M))
    rng = np.random.default_rng(0xC3)
    rows.update(int(r) for r in rng.integers(0, w.n_rows, size=256))
    return np.array(sorted(rows), dtype=np.int32)


def parity_report(name: str, w, O_bits, lse):
    """max |O - float64 oracle| over the checked rows, and how it sits against the stated tolerance
    (2e-3; 1e-2 over an E4M3 pool) plus half an ulp of the 16-bit output and, for rows with a handful
    of keys, the bound on rounding P to 16 bits before P.V (u * sum_j p_j |v_j|)."""
    import oracle
    from espetero_b200 import workloads as wl
    rows = parity_rows(name, w)
    ref, lse_ref, ref_abs = oracle.attention_f64(w, rows=rows, with_abs=True)
    got = wl.from_bits16(O_bits if rows is None else O_bits[rows], w.q_dtype).astype(np.float64)
    got_lse = lse if rows is None else lse[rows]
    tol = 1e-2 if w.kv_dtype == wl.E4M3 else 2e-3
    mant = 10 if w.q_dtype == wl.F16 else 7
    half_ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(ref), 2.0 ** -14))) - mant - 1)
    u_p = 2.0 ** -12 if (w.q_dtype == wl.F16 or w.kv_dtype == wl.E4M3) else 2.0 ** -9
    err = np.abs(got - ref)
    allow = tol + half_ulp + u_p * ref_abs
    fin = np.isfinite(lse_ref)
    lse_err = float(np.abs(got_lse[fin] - lse_ref[fin]).max()) if fin.any() else 0.0
    return {"max_abs_err": float(err.max()), "tol": tol, "rows_checked": int(len(ref)), "elements": int(err.size),
            "beyond_plain_tol": int((err > tol).sum()), "beyond_allowance": int((err > allow).sum()),
            "allowance": "tol + half an ulp of the 16-bit output + 2^-9 (bf16; 2^-12 fp16) x sum_j p_j|v_j| for rounding P",
            "lse_max_abs_err": lse_err, "ok": bool((err <= allow).all() and lse_err < 2e-3),
            "oracle": "float64 direct softmax on the stored values (oracle/)"}


class Bench:
    """Process-wide state of one bench run (one rank)."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU implementation")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.stream = torch.cuda.current_stream(self.dev)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.dev)

    def timed(self, fn, n, tail=None, solo=False):
        """Seconds for n calls of fn: CUDA events on the launching stream, barrier + synchronize on both sides.
        tail() runs before the closing event (it makes the launching stream wait for work on other streams).
        solo: this rank measures alone (no barrier with the others)."""
        torch = self.torch
        sync = (lambda: torch.cuda.synchronize(self.dev)) if solo else self.barrier
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(self.stream)
        for _ in range(n):
            fn()
        if tail is not None:
            tail()
        e1.record(self.stream)
        sync()
        return e0.elapsed_time(e1) / 1e3

    def reduce_max_sum(self, times, total):
        """max over ranks of each time, sum over ranks of `total`."""
        torch = self.torch
        tt = torch.tensor(list(times), dtype=torch.float64, device=self.dev)
        bb = torch.tensor([float(total)], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(tt, op=self.dist.ReduceOp.MAX)
            self.dist.all_reduce(bb, op=self.dist.ReduceOp.SUM)
        return [float(x) for x in tt.cpu()], float(bb.cpu()[0])


class Run:
    """One workload set up on this rank: step() = the whole pass, step_attn() = the attention kernel alone."""
    xch = None
    split_kv = False


def setup_sequences(B: Bench, name: str, w, scaling: str, sharding: str) -> Run:
    """Sequences are whole units of work: this rank's batch, its own pool and plan, no exchange."""
    from espetero_b200 import host
    args = B.args
    r = Run()
    r.name, r.w, r.scaling, r.sharding = name, w, scaling, sharding
    r.op = host.AttnOp.for_workload(w, TILE_ROWS[name], B.local)
    if args.fuse >= 0:
        r.op.set_option("fuse_combine", args.fuse)
    for kv in args.opt:
        r.op.set_option(kv.split("=")[0], int(kv.split("=")[1]))
    r.plan = bench_plan(name, w, args.groups)
    r.dp = r.op.upload(w, r.plan)
    r.layers = LayerCycle(r.op, r.dp, w)
    r.a_full = r.layers.args()
    r.a_attn = r.layers.args(n_jobs=0)  # attention kernel alone (records only, no merge), for the per-kernel roofline figure
    r.step = lambda: r.op.forward(r.dp, r.layers.next(r.a_full))
    r.step_attn = lambda: r.op.forward(r.dp, r.layers.next(r.a_attn))
    return r


def setup_split_kv(B: Bench, small: bool) -> Run:
    """One long sequence, keys split over the ranks on page boundaries: records for the local keys ->
    one kernel per rank reduces them, stores the reduced record into every rank's buffer over NVLink
    peer mappings and merges the world's records in rank order (or: reduce -> NCCL all-gather ->
    merge). Total work is fixed: strong scaling."""
    from espetero_b200 import capi, host, shard, workloads as wl
    torch, dist, args = B.torch, B.dist, B.args
    rank, world, dev = B.rank, B.world, B.dev
    r = Run()
    r.name, r.split_kv, r.scaling = "c5", True, "strong"
    ctx_all = 8192 if small else 131072
    lo, hi = shard.split_kv_range(ctx_all, world, 16)[rank]
    if args.ctx > 0 and world == 1:
        lo, hi = 0, args.ctx
    w = r.w = wl.config_c5(0xE5B205 + 1000 * rank, ctx=hi - lo)
    op = r.op = host.AttnOp.for_workload(w, TILE_ROWS["c5"], B.local)
    for kv in args.opt:
        op.set_option(kv.split("=")[0], int(kv.split("=")[1]))
    base_plan = host.plan_tiles(w.trees, w.Hkv, capi.ESP_PLAN_B200, 1 << 20, 32, args.groups or 148 * 2, TILE_ROWS["c5"])
    tiles, red_jobs, n_parts = shard.local_decode_plan(base_plan.tiles, is_last_rank=(rank == world - 1))
    r.plan = host.Plan(tiles, np.zeros(0, dtype=wl.COMBINE_DT), n_parts, TILE_ROWS["c5"])
    dp = r.dp = op.upload(w, r.plan)
    if world > 1:
        for t in (dp.Q, dp.Kb, dp.Vb):  # the query row is replicated: every rank uses rank 0's
            dist.broadcast(t.view(torch.uint8), src=0)  # NCCL has no 16-bit integer type
    layers = r.layers = LayerCycle(op, dp, w)
    r.a_attn = layers.args()
    r.a_full = r.a_attn
    red_dev = host._dev(red_jobs, dev)
    merge_dev = host._dev(shard.world_merge_jobs(1, world), dev)
    rec_local = torch.zeros(op.parts_floats(1), dtype=torch.float32, device=dev)
    rec_world = torch.zeros(world * op.parts_floats(1), dtype=torch.float32, device=dev)
    xch = None
    if world == 1:
        xch = host.PeerExchange.emulated(op, n_jobs=1, rows_max=1, world=1)
    elif args.exchange == "p2p":
        try:
            xch = host.PeerExchange(op, n_jobs=1, rows_max=1)
            ok = 1
        except Exception as e:  # noqa: BLE001 - reported below, then the NCCL path is used
            print(f"[rank {rank}] peer exchange unavailable: {e}", file=sys.stderr, flush=True)
            ok = 0
        flag = torch.tensor([ok], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)  # all ranks decide together
        if int(flag.item()) == 0:
            xch = None
    r.xch = xch
    if xch is not None:
        # one call per rank and step (esp_attn_forward_exchange): the records-only pass, then ONE kernel that folds the
        # rank's records, stores the result into every rank's buffer over NVLink peer mappings, waits for the peers'
        # and writes the row. (With the library option fuse_exchange = 1 all of it happens inside the decode kernel, in
        # one launch; that measured slower - 64.0 against 57.3 us per step on two GPUs - and is off by default.)
        a_x = layers.args()
        a_x.jobs, a_x.jobs_host, a_x.n_jobs = red_dev.data_ptr(), red_jobs.ctypes.data, len(red_jobs)
        r.keep = (red_jobs, red_dev)

        def step():
            xch.next_epoch()
            op.forward_exchange(dp, layers.next(a_x), xch, rank=rank)
        r.a_full = a_x
        r.sharding = "KV range per rank; records-only pass, then one kernel per rank folds them, exchanges records over NVLink peer stores and finishes"
    else:
        def step():
            op.forward(dp, layers.next(r.a_attn))
            op.reduce_parts(dp, dp.parts, red_dev, len(red_jobs), rec_local, 0)
            dist.all_gather_into_tensor(rec_world, rec_local)
            op.combine(dp, rec_world, merge_dev, 1)
        r.sharding = "KV range per rank; reduced records all-gathered (NCCL), merged on every rank"
    r.step = step
    r.step_attn = lambda: op.forward(dp, layers.next(r.a_attn))
    return r


def time_run(B: Bench, r: Run, steps: int, W: int, solo: bool = False):
    """(seconds per step of the whole pass, of the attention kernel alone, launches per step)."""
    for _ in range(W):
        r.step()
    r.op.check_status()
    n0 = r.op.launch_count
    t_total = B.timed(r.step, steps, solo=solo)
    launches = r.op.launch_count - n0
    if launches == steps and int(getattr(r.a_full, "n_jobs", 1)) == 0:
        # the step IS the attention kernel (one launch, no records to merge): its timed region is the kernel's
        return t_total / steps, t_total / steps, launches
    for _ in range(3):
        r.step_attn()
    t_attn = B.timed(r.step_attn, steps, solo=solo) / steps
    return t_total / steps, t_attn, launches


def time_e2e(B: Bench, r: Run, steps: int, t_step: float):
    """End to end through the C ABI from host buffers: the step's inputs (Q, Kb, Vb and the plan
    tables) come from pinned host memory, the result goes back; the KV pool is device state."""
    from espetero_b200 import host
    torch = B.torch
    op, dp, layers, stream, dev = r.op, r.dp, r.layers, B.stream, B.dev
    arena = host.StepArena(dp)
    a_e2e = arena.patch(op.make_args(dp))
    h_out = torch.empty_like(dp.O, device="cpu").pin_memory()
    h2d = arena.nbytes
    d2h = h_out.numel() * h_out.element_size()
    if r.split_kv:
        for a in (r.a_attn, r.a_full):  # the step reads its inputs from the arena
            a.Q, a.Kb, a.Vb, a.tiles, a.trees, a.blocks = a_e2e.Q, a_e2e.Kb, a_e2e.Vb, a_e2e.tiles, a_e2e.trees, a_e2e.blocks
    e2e_tail = None
    # Passes of a few microseconds are bound by the host's calls, not by the GPU: pipelining them over
    # three streams only adds calls, so they keep the plain sequence on one stream.
    if r.split_kv or t_step < 25e-6:
        def step_e2e():
            arena.upload()
            if r.split_kv:
                r.step()
            else:
                op.forward(dp, layers.next(a_e2e))
            h_out.copy_(dp.O, non_blocking=True)
        note = "Q/Kb/Vb + plan tables in one arena copied from pinned host memory, O back to the host; the KV pool is resident device state"
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
        note = ("Q/Kb/Vb + plan tables in one arena copied from pinned host memory, O back to the host, every step; two buffer sets, "
                "copies of step i+1 overlap the kernels of step i; the KV pool is resident device state")
    for _ in range(3):
        step_e2e()
    return B.timed(step_e2e, steps, e2e_tail) / steps, h2d, d2h, note


def close_run(r: Run):
    if r.xch is not None:
        r.xch.close()
    r.op.close()


def strong_scaling_legs(B: Bench, steps: int):
    """At N > 1: the two fixed-total-work cases, each with the one-GPU time measured by rank 0 alone in
    the same run (the other ranks wait), so that the line carries its own efficiency."""
    from espetero_b200 import shard, workloads as wl
    torch = B.torch
    out = {}
    # ---- the one 32-sequence batch of the configuration, spread over the GPUs by context length
    lens = wl.c2_context_lengths(0xE5B202, 32, 512, 32768)
    mine = shard.lpt_partition(lens, B.world)[B.rank]
    w = wl.config_c2(0xE5B202 + 1000 * B.rank, lens=lens[mine] if len(mine) else lens[:1])
    r = setup_sequences(B, "c2", w, "strong", "the 32 sequences spread by total context length (LPT), no collective")
    t_step, t_attn, _ = time_run(B, r, steps, 3)
    (t_step, t_attn), bytes_all = B.reduce_max_sum([t_step, t_attn], w.kv_bytes_read() if len(mine) else 0)
    close_run(r)
    t1 = 0.0
    if B.rank == 0:
        w1 = wl.config_c2(0xE5B202)
        r1 = setup_sequences(B, "c2", w1, "strong", "one GPU")
        t1, _, _ = time_run(B, r1, steps, 3, solo=True)
        close_run(r1)
    B.barrier()
    if B.rank == 0:
        out["c2_strong"] = {"workload": "c2_batched_decode: ONE batch of 32 sequences over all GPUs", "scaling": "strong",
                            "sequences_per_gpu": len(mine), "value": bytes_all / t_step / 1e9, "unit": UNIT,
                            "us_per_step": 1e6 * t_step, "us_attention_kernel": 1e6 * t_attn, "us_per_step_one_gpu": 1e6 * t1,
                            "speedup_vs_n1": t1 / t_step, "efficiency_vs_n1": t1 / t_step / B.world}
    # ---- one 131072-token sequence, keys split over the GPUs by range
    r = setup_split_kv(B, small=False)
    t_step, t_attn, launches = time_run(B, r, steps, 3)
    (t_step, t_attn), bytes_all = B.reduce_max_sum([t_step, t_attn], r.w.kv_bytes_read())
    route = "p2p" if r.xch is not None else "nccl"
    close_run(r)
    t1 = 0.0
    if B.rank == 0:
        w1 = wl.config_c5()
        r1 = setup_sequences(B, "c5", w1, "strong", "one GPU")
        t1, _, _ = time_run(B, r1, steps, 3, solo=True)
        close_run(r1)
    B.barrier()
    if B.rank == 0:
        out["split_kv"] = {"workload": "c5_long_fp8_decode: one 131072-token sequence, keys split over the GPUs by range",
                           "scaling": "strong", "exchange": route, "value": bytes_all / t_step / 1e9, "unit": UNIT,
                           "us_per_step": 1e6 * t_step, "us_attention_kernel": 1e6 * t_attn,
                           "us_exchange": 1e6 * (t_step - t_attn), "launches_per_step": launches // max(1, steps),
                           "us_per_step_one_gpu": 1e6 * t1, "speedup_vs_n1": t1 / t_step, "efficiency_vs_n1": t1 / t_step / B.world}
    return out


PREP_LAYOUTS = {
    # name: H, Hkv, HD, rot_half, gate interleaved with the query heads, default rows
    "plain128": (64, 8, 128, 64, False, 32768),   # the causal-prefill shape (C3) with full rotary
    "gated256": (32, 8, 256, 32, True, 8192),     # the layout of kernels/40_attention.metal:23-102
}


def run_prep(args):
    """--workload prep: esp_attn_prep alone (the step right before the attention pass; not part of the headline
    metric). Per row the kernel reads (H + 2 Hkv) * HD floats of the fused projection and writes as many 16-bit
    elements: HBM-bound. One JSON line per layout."""
    import torch
    from espetero_b200 import capi, host, workloads as wl
    hbm_peak, _, which = measured_peaks()
    for layout in (sorted(PREP_LAYOUTS) if args.layout == "all" else [args.layout]):
        H, Hkv, HD, rot_half, gated, rows = PREP_LAYOUTS[layout]
        rows = args.rows or rows
        q_stride = 2 * HD if gated else HD
        k_off = H * q_stride
        v_off = k_off + Hkv * HD
        ld = v_off + Hkv * HD
        op = host.AttnOp(H, Hkv, HD, 16, wl.BF16, wl.BF16, 1.0)
        try:
            dev = op.device
            X = torch.randn(rows, ld, device=dev)
            qn, kn = torch.ones(HD, device=dev), torch.ones(HD, device=dev)
            pos = torch.randint(0, 100000, (rows, 4), dtype=torch.int32, device=dev)
            inv = torch.tensor((1e6 ** (-np.arange(rot_half) / rot_half)).astype(np.float32), device=dev)
            sel = torch.zeros(rot_half, dtype=torch.int32, device=dev)
            Q = torch.zeros(rows, H * HD, dtype=torch.int16, device=dev)
            Kb = torch.zeros(rows, Hkv * HD, dtype=torch.int16, device=dev)
            Vb = torch.zeros_like(Kb)
            pp = capi.PrepParams(H, Hkv, ld, 0, q_stride, k_off, v_off, H * HD, Hkv * HD, rot_half, 1e-6, 1.0, 16, 0, 0)
            for _ in range(max(3, args.warmup)):
                op.attn_prep(X, qn, kn, pos, inv, sel, Q, Kb, Vb, pp)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(dev)
            e0.record()
            for _ in range(args.steps):
                op.attn_prep(X, qn, kn, pos, inv, sel, Q, Kb, Vb, pp)
            e1.record()
            torch.cuda.synchronize(dev)
            ms = e0.elapsed_time(e1) / args.steps
            nbytes = rows * (H + 2 * Hkv) * HD * (4 + 2)
            print(json.dumps({"metric": "attn_prep_hbm_bandwidth", "value": nbytes / ms / 1e6, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
                              "ms_per_step": ms, "config": {"workload": "attn_prep", "layout": layout, "rows": rows, "H": H, "Hkv": Hkv, "HD": HD,
                                                            "l2": "inputs larger than L2" if nbytes > 2 * L2_BYTES else "inputs fit L2"},
                              "roofline": {"bound": "hbm", "achieved": nbytes / ms / 1e6, "peak": hbm_peak, "unit": "GB/s", "frac": nbytes / ms / 1e6 / hbm_peak,
                                           "peak_source": which, "kernel": "attn_prep", "ms_per_launch": ms, "algorithmic_bytes": nbytes}}), flush=True)
        finally:
            op.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5", "prep"])
    ap.add_argument("--layout", default="all", choices=["all"] + sorted(PREP_LAYOUTS), help="--workload prep: which projection layout")
    ap.add_argument("--rows", type=int, default=0, help="--workload prep: rows (0: the layout's default)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--small", action="store_true", help="reduced sizes (profiling captures)")
    ap.add_argument("--kv", default="", choices=["", "e4m3"], help="c2 / c4 only: the pass over an FP8 E4M3 pool instead of bf16")
    ap.add_argument("--window", type=int, default=0, help="c3 only: the prefill through a sliding-window layer of this many positions")
    ap.add_argument("--hd", type=int, default=128, choices=[64, 128, 256, 512], help="c2 / c3 / c4 only: the pass with another head dim of the reference's kernels (256: flash_attention's own)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison with the float64 oracle after the timed region")
    ap.add_argument("--no-strong", action="store_true", help="at N > 1: skip the two strong-scaling legs (c2_strong, split_kv)")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"], help="split-KV record exchange at N > 1 (c5)")
    ap.add_argument("--fuse", type=int, default=-1, help="option fuse_combine of the library (0 off, 1 small passes, 2 always); -1: its default")
    ap.add_argument("--ctx", type=int, default=0, help="c5 on one GPU: run the split-KV step of ONE rank holding this many keys (records-only pass + "
                    "exchange with itself): the latency chain of a rank at N GPUs without the NVLink hop, for tuning")
    ap.add_argument("--opt", action="append", default=[], metavar="NAME=VALUE", help="set a library option (esp_attn_set_option) on the pass's context")
    ap.add_argument("--groups", type=int, default=0, help="CTA target of the planner (default 8 waves of 2 CTAs per SM)")
    args = ap.parse_args()
    if args.hd != 128 and args.workload not in ("c2", "c3", "c4"):
        raise SystemExit("--hd applies to c2 (one GPU), c3 and c4")
    global CPU_SAMPLE_HD
    CPU_SAMPLE_HD = args.hd
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.workload == "prep":
        return run_prep(args)

    B = Bench(args)
    torch, dist = B.torch, B.dist
    from espetero_b200 import workloads as wl
    rank, world, dev = B.rank, B.world, B.dev
    W = max(3, args.warmup)

    if args.workload == "c5" and (world > 1 or args.ctx > 0):
        r = setup_split_kv(B, args.small)
    else:
        w = build_workload(args.workload, rank, args.small, world, args.kv, args.window, args.hd)
        sharding = "sequences per rank, no collective" + (
            "; the box's batch spread by total context length (LPT)" if world > 1 and args.workload == "c2" else "")
        r = setup_sequences(B, args.workload, w, "weak", sharding)
    w, op, plan = r.w, r.op, r.plan
    bytes_step = w.kv_bytes_read()

    # ---- device-resident throughput (value) and the attention kernel alone (roofline of the dominant kernel)
    sampler = ClockSampler(B.local)
    if rank == 0:
        sampler.start()
    t_step, t_attn, launches = time_run(B, r, args.steps, W)
    # nvidia-smi samples every 100 ms: keep the same kernels running (untimed) until it has seen the
    # GPU under this load for about half a second, on every rank alike
    # (a fixed number of steps derived from rank 0's timing, so that ranks which exchange records
    # inside a step all run the same count)
    hold = torch.tensor([min(20000, int(0.6 / max(t_step, 1e-6)) + 1)], dtype=torch.int64, device=dev)
    if world > 1:
        dist.broadcast(hold, src=0)
    for _ in range(int(hold.item())):
        r.step()
    torch.cuda.synchronize(dev)
    clocks = sampler.stop() if rank == 0 else None
    op.check_status()

    t_e2e, h2d, d2h, e2e_note = time_e2e(B, r, args.steps, t_step)

    # ---- parity of exactly this pass (plan, options, sizes) with the float64 oracle, off the timed region
    parity = None
    if world == 1 and not args.no_check and not r.split_kv:
        r.dp.O.zero_()
        r.dp.lse.zero_()
        a = r.layers.args()
        a.p.kv_base = w.kv_base  # the first layer region holds the workload's own pool
        op.forward(r.dp, a)
        op.check_status()
        torch.cuda.synchronize(dev)
        parity = parity_report(args.workload, w, r.dp.O.cpu().numpy().view(np.uint16), r.dp.lse.cpu().numpy())

    # ---- aggregate over ranks: max time, summed bytes
    (t_step, t_attn_max, t_e2e), bytes_all = B.reduce_max_sum([t_step, t_attn, t_e2e], bytes_step)
    kernel_name = op.last_kernel
    scaling, sharding, split_kv = r.scaling, r.sharding, r.split_kv
    close_run(r)

    extra = {}
    if world > 1 and args.workload == "c2" and not (args.no_strong or args.small):
        extra = strong_scaling_legs(B, min(args.steps, 50))

    if rank == 0:
        hbm_peak, tf_peak, which = measured_peaks()
        value = bytes_all / t_step / 1e9
        achieved = bytes_step / t_attn / 1e9
        flops = attention_flops(w)
        traffic = NCU_TRAFFIC_BYTES.get(args.workload) if not (args.small or split_kv or args.kv or args.window or args.hd != 128) else None
        tensor = {"tflops": flops / t_attn / 1e12, "peak_tflops": tf_peak, "frac": flops / t_attn / 1e12 / tf_peak,
                  "flops_per_step": flops}
        if measured_peaks.sustained_tflops:  # the denominator for a kernel timed inside a long, power-capped run
            tensor["peak_tflops_sustained"] = measured_peaks.sustained_tflops
            tensor["frac_of_sustained"] = tensor["tflops"] / measured_peaks.sustained_tflops
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": W,
            "ms_per_step": 1e3 * t_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "bf16" if w.kv_dtype != wl.E4M3 else "e4m3->f16", "data": "synthetic",
            "config": workload_config(w),
            "plan": {"planner": "esp_attn_plan_window (rows 128)" if args.window else "ESP_PLAN_B200", "tiles": len(plan.tiles),
                     "parts": plan.n_parts, "kernel": kernel_name,
                     "sharding": sharding},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "traffic": traffic, "peak_source": which, "kernel": kernel_name, "ms_per_launch": 1e3 * t_attn,
                         "launch": "the attention kernel alone: the same plan launched without its combine jobs (records only)",
                         "step_frac": bytes_step / t_step / 1e9 / hbm_peak if world == 1 else bytes_all / world / t_step / 1e9 / hbm_peak,
                         "step": "the whole pass (attention kernel + merge of the split-K records), as in `value`"},
            "e2e": {"value": bytes_all / t_e2e / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": e2e_note},
            "gpu_launches": int(launches), "clocks": clocks, "tensor": tensor,
        }
        if args.workload == "c3":  # the prefill configuration is bound by the tensor cores, not by HBM
            line["metric"], line["unit"] = "prefill_attn_tflops", "TFLOP/s"
            line["value"] = flops * world / t_step / 1e12
            sm = (clocks or {}).get("sm_mhz")
            line["roofline"] = {"bound": "tensor", "achieved": tensor["tflops"], "peak": tf_peak, "unit": "TFLOP/s",
                                "frac": tensor["frac"], "traffic": traffic, "peak_source": which, "kernel": kernel_name,
                                "ms_per_launch": 1e3 * t_attn, "step_frac": flops / t_step / 1e12 / tf_peak,
                                "ms_x_sm_mhz": (1e3 * t_attn * sm) if sm else None}
            line["e2e"]["value"] = flops * world / t_e2e / 1e12
            line["e2e"]["unit"] = "TFLOP/s"
        if parity is not None:
            line["parity"] = parity
        line.update(extra)
        if world == 1 and not args.no_cpu and not args.ctx:
            v, threads, sample, dt = time_cpu(args.workload)
            line["cpu_baseline"] = {"value": v, "unit": line["unit"], "cores": threads, "kind": "port", "sample": sample, "seconds": dt}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
