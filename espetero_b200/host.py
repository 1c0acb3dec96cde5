"""Host-side driver of the C ABI for tests, the smoke check and bench.py.

Plays the role run_forest plays in the reference (src/model/impl/forest.h:2646-2716 builds
the plan, :2855-2947 dispatches attention / combine / kv_save): it owns the device buffers
(torch tensors are used only as device memory and for streams), builds the plan through
esp_attn_plan and calls esp_attn_forward. All arithmetic happens inside
libespetero_attn.so; if the library is missing, importing capi raises.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import capi
from .workloads import COMBINE_DT, E4M3, KVSAVE_DT, TILE_DT, TREE_DT, Workload


@dataclass
class Plan:
    tiles: np.ndarray    # TILE_DT (host)
    jobs: np.ndarray     # COMBINE_DT (host)
    n_parts: int
    tile_rows: int


def plan_tiles(trees: np.ndarray, Hkv: int, mode: int = capi.ESP_PLAN_REFERENCE, split: int = 512, min_chunk: int = 32,
               groups: int = 256, tile_rows: int = 8, max_parts: int = 64) -> Plan:
    """esp_attn_plan: the integer planner (pure host; needs no GPU)."""
    lib = capi.load()
    trees = np.ascontiguousarray(trees, dtype=TREE_DT)
    opts = capi.PlanOpts(mode, split, min_chunk, groups, tile_rows, max_parts)
    nt, nj, np_ = C.c_int32(), C.c_int32(), C.c_int32()
    tp = trees.ctypes.data_as(C.POINTER(capi.Tree))
    capi.check(lib.esp_attn_plan(tp, len(trees), Hkv, C.byref(opts), None, 0, None, 0, C.byref(nt), C.byref(nj), C.byref(np_)))
    tiles = np.zeros(max(1, nt.value), dtype=TILE_DT)
    jobs = np.zeros(max(1, nj.value), dtype=COMBINE_DT)
    capi.check(lib.esp_attn_plan(tp, len(trees), Hkv, C.byref(opts), tiles.ctypes.data_as(C.POINTER(capi.Tile)), len(tiles),
                                 jobs.ctypes.data_as(C.POINTER(capi.Combine)), len(jobs), C.byref(nt), C.byref(nj), C.byref(np_)))
    return Plan(tiles[:nt.value], jobs[:nj.value], np_.value, tile_rows)


def plan_window(trees: np.ndarray, groups: int, split: int = 512, rows: int = 8, window: int = 0, pos=None) -> Plan:
    """esp_attn_plan_window: the generic planner with its sliding-window branch (gemma.h:77-116)."""
    lib = capi.load()
    trees = np.ascontiguousarray(trees, dtype=TREE_DT)
    pos = None if pos is None else np.ascontiguousarray(pos, dtype=np.int32)
    pp = None if pos is None else C.c_void_p(pos.ctypes.data)
    nt, nj, np_, pr = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
    tp = trees.ctypes.data_as(C.POINTER(capi.Tree))
    capi.check(lib.esp_attn_plan_window(tp, len(trees), groups, split, rows, window, pp, None, 0, None, 0, C.byref(nt), C.byref(nj),
                                        C.byref(np_), C.byref(pr)))
    tiles = np.zeros(max(1, nt.value), dtype=TILE_DT)
    jobs = np.zeros(max(1, nj.value), dtype=COMBINE_DT)
    capi.check(lib.esp_attn_plan_window(tp, len(trees), groups, split, rows, window, pp, tiles.ctypes.data_as(C.POINTER(capi.Tile)),
                                        len(tiles), jobs.ctypes.data_as(C.POINTER(capi.Combine)), len(jobs), C.byref(nt), C.byref(nj),
                                        C.byref(np_), C.byref(pr)))
    return Plan(tiles[:nt.value], jobs[:nj.value], np_.value, pr.value)


def _dev(arr: np.ndarray | None, device, pin: bool = False):
    if arr is None:
        return None
    a = np.ascontiguousarray(arr)
    if a.dtype.fields is not None:  # structured records travel as raw int32
        a = a.view(np.int32)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    if a.dtype == np.uint64:
        a = a.view(np.int64)
    t = torch.from_numpy(a)
    return t.to(device)


def _ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


class DevicePass:
    """Device copies of one Workload plus output buffers."""

    def __init__(self, w: Workload, device):
        self.w = w
        self.device = device
        self.Q, self.Kb, self.Vb = _dev(w.Q, device), _dev(w.Kb, device), _dev(w.Vb, device)
        self.kv = _dev(w.kv, device)
        self.kv_scales = _dev(w.kv_scales, device)
        self.blocks = _dev(w.blocks, device)
        self.desc = _dev(w.desc, device)
        self.anc_mask = _dev(w.anc_mask, device)
        self.X = _dev(w.X, device)
        self.trees = _dev(w.trees, device)
        self.win = w.extra.get("window") if isinstance(getattr(w, "extra", None), dict) else None
        self.pos = _dev(self.win["pos"], device) if self.win else None
        self.O = torch.zeros((w.n_rows, w.q_ld), dtype=torch.int16, device=device)
        self.lse = torch.zeros((w.n_rows, w.H), dtype=torch.float32, device=device)
        self.tiles = self.jobs = self.parts = None
        self.plan: Plan | None = None

    def replicate_layers(self, n_layers: int) -> int:
        """Lay the pool out as n_layers equal layer regions (the reference's pool holds one region
        per attention layer, src/model/impl/forest.h:1336-1377), each a copy of the workload's
        pool; layer r's pass uses kv_base = w.kv_base + r * (returned elements per region)."""
        region = self.kv.numel()
        if n_layers > 1:
            self.kv = self.kv.reshape(1, -1).repeat(n_layers, 1).reshape(-1)
        return region

    def set_plan(self, plan: Plan, parts_floats: int):
        self.plan = plan
        self.tiles = _dev(plan.tiles, self.device) if len(plan.tiles) else None
        self.jobs = _dev(plan.jobs, self.device) if len(plan.jobs) else None
        self.parts = torch.zeros(max(4, parts_floats), dtype=torch.float32, device=self.device)


class StepArena:
    """The per-step inputs of a pass (Q, Kb, Vb, tiles, trees, block table) laid out in ONE device
    buffer with a pinned host mirror, as the reference keeps its per-pass tables in one arena
    (PassMeta, src/model/impl/forest.h:1678-1735): a step then needs one host-to-device copy."""

    def __init__(self, dp: DevicePass):
        parts = [("Q", dp.Q), ("Kb", dp.Kb), ("Vb", dp.Vb), ("tiles", dp.tiles), ("trees", dp.trees), ("blocks", dp.blocks)]
        self.offsets, off = {}, 0
        for name, t in parts:
            if t is None:
                continue
            self.offsets[name] = (off, t.numel() * t.element_size())
            off = (off + t.numel() * t.element_size() + 255) // 256 * 256
        self.nbytes = off
        self.dev = torch.empty(off, dtype=torch.uint8, device=dp.device)
        self.host = torch.empty(off, dtype=torch.uint8).pin_memory()
        for name, t in parts:
            if t is None:
                continue
            o, n = self.offsets[name]
            self.host[o:o + n] = t.contiguous().view(-1).view(torch.uint8).cpu()
        self.dev.copy_(self.host)

    def ptr(self, name: str):
        return self.dev.data_ptr() + self.offsets[name][0] if name in self.offsets else None

    def upload(self):
        self.dev.copy_(self.host, non_blocking=True)

    def patch(self, args: capi.Args) -> capi.Args:
        """Point the step inputs of `args` into the arena."""
        for name in ("Q", "Kb", "Vb", "tiles", "trees", "blocks"):
            if name in self.offsets:
                setattr(args, name, self.ptr(name))
        return args


class AttnOp:
    """One esp_attn_ctx. Not thread-safe, like the reference's NativeModel (src/model/api.h:4-6)."""

    def __init__(self, H, Hkv, HD, bt, q_dtype, kv_dtype, scale, flags=0, tile_rows=8, device=0):
        self.lib = capi.load()
        if not torch.cuda.is_available():
            raise RuntimeError("AttnOp needs a CUDA device: the attention path has no CPU implementation")
        self.device = torch.device("cuda", device)
        self.shape = capi.Shape(H, Hkv, HD, bt, q_dtype, kv_dtype, tile_rows, flags, scale)
        self.ctx = C.c_void_p()
        capi.check(self.lib.esp_attn_create(C.byref(self.ctx), device, C.byref(self.shape)))
        self.tile_rows = tile_rows

    @classmethod
    def for_workload(cls, w: Workload, tile_rows: int = 8, device: int = 0) -> "AttnOp":
        return cls(w.H, w.Hkv, w.HD, w.bt, w.q_dtype, w.kv_dtype, w.scale, w.flags, tile_rows, device)

    def close(self):
        if self.ctx:
            self.lib.esp_attn_destroy(self.ctx)
            self.ctx = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_option(self, name: str, value: int):
        capi.check(self.lib.esp_attn_set_option(self.ctx, name.encode(), value))

    def get_option(self, name: str) -> int:
        v = C.c_int()
        capi.check(self.lib.esp_attn_get_option(self.ctx, name.encode(), C.byref(v)))
        return v.value

    def parts_floats(self, n_parts: int) -> int:
        return int(self.lib.esp_attn_parts_floats(C.byref(self.shape), n_parts))

    def upload(self, w: Workload, plan: Plan | None = None) -> DevicePass:
        dp = DevicePass(w, self.device)
        if w.kv_dtype == E4M3 and bool((w.trees["M"] > 1).any()):
            # multi-row passes over an E4M3 pool: scratch for the widened blocks (tensor-core kernels)
            n = int(self.lib.esp_attn_dequant_scratch_bytes(C.byref(self.shape), len(w.blocks)))
            dp.scratch = torch.empty(max(n, 128), dtype=torch.uint8, device=self.device)
        if plan is not None:
            dp.set_plan(plan, self.parts_floats(plan.n_parts))
        return dp

    def params(self, w: Workload) -> capi.Params:
        return capi.Params(w.H, w.Hkv, w.q_ld, w.kv_ld, w.g_ld, w.bt, w.kv_base)

    def make_args(self, dp: DevicePass) -> capi.Args:
        w, plan = dp.w, dp.plan
        a = capi.Args()
        a.Q, a.Kb, a.Vb, a.kv = _ptr(dp.Q), _ptr(dp.Kb), _ptr(dp.Vb), _ptr(dp.kv)
        a.kv_scales, a.blocks, a.desc, a.anc_mask, a.X = _ptr(dp.kv_scales), _ptr(dp.blocks), _ptr(dp.desc), _ptr(dp.anc_mask), _ptr(dp.X)
        a.O, a.lse, a.parts = _ptr(dp.O), _ptr(dp.lse), _ptr(dp.parts)
        a.tiles, a.trees, a.jobs = _ptr(dp.tiles), _ptr(dp.trees), _ptr(dp.jobs)
        a.tiles_host = plan.tiles.ctypes.data if len(plan.tiles) else None
        a.trees_host = w.trees.ctypes.data
        a.jobs_host = plan.jobs.ctypes.data if len(plan.jobs) else None
        a.n_tiles, a.n_trees, a.n_jobs, a.n_rows = len(plan.tiles), len(w.trees), len(plan.jobs), w.n_rows
        a.n_blocks, a.n_block_entries, a.n_parts = w.n_blocks, len(w.blocks), plan.n_parts
        if getattr(dp, "scratch", None) is not None:
            a.dequant_scratch, a.dequant_scratch_bytes = dp.scratch.data_ptr(), dp.scratch.numel()
        if dp.win:
            a.pos, a.window, a.ring, a.bidi = _ptr(dp.pos), dp.win["window"], dp.win["ring"], dp.win["bidi"]
            dp.pos_host = np.ascontiguousarray(dp.win["pos"], dtype=np.int32)   # kept alive with the pass
            a.pos_host = dp.pos_host.ctypes.data
        a.p = self.params(w)
        return a

    def forward(self, dp: DevicePass, args: capi.Args | None = None, stream: int | None = None):
        """esp_attn_forward on torch's current stream (or the given cudaStream_t)."""
        if args is None:
            args = self.make_args(dp)
        s = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        capi.check(self.lib.esp_attn_forward(self.ctx, C.c_void_p(s), C.byref(args)))

    def combine(self, dp: DevicePass, parts, jobs_dev, n_jobs: int, stream: int | None = None):
        s = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        p = self.params(dp.w)
        capi.check(self.lib.esp_attn_combine_parts(self.ctx, C.c_void_p(s), _ptr(parts), _ptr(dp.X), _ptr(dp.O), _ptr(dp.lse),
                                                   C.byref(p), _ptr(jobs_dev), n_jobs))

    def reduce_parts(self, dp: DevicePass, parts, jobs_dev, n_jobs: int, parts_out, out_part0: int = 0, stream: int | None = None):
        """esp_attn_reduce_parts: job j's records -> one unnormalised record out_part0 + j of parts_out."""
        s = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        p = self.params(dp.w)
        capi.check(self.lib.esp_attn_reduce_parts(self.ctx, C.c_void_p(s), _ptr(parts), C.byref(p), _ptr(jobs_dev), n_jobs,
                                                  _ptr(parts_out), out_part0))

    def exchange_parts(self, dp: DevicePass, parts, jobs_dev, n_jobs: int, xch: "PeerExchange", rank: int | None = None,
                       phases: int = 3, rows_max: int = 1, parts_max: int = 64, wait_ms: int = 0, stream: int | None = None):
        """esp_attn_exchange_parts: merge the local records, push the result to every rank's exchange
        buffer over peer memory, wait for the peers' and finish O / lse: one kernel. Advances the
        exchange's epoch when the launch includes the publishing phase of the last (or only) local rank."""
        s = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        p = self.params(dp.w)
        x = xch.descriptor(xch.rank if rank is None else rank, phases, wait_ms)
        capi.check(self.lib.esp_attn_exchange_parts(self.ctx, C.c_void_p(s), _ptr(parts), _ptr(dp.X), _ptr(dp.O), _ptr(dp.lse),
                                                    C.byref(p), _ptr(jobs_dev), n_jobs, rows_max, parts_max, C.byref(x)))

    def forward_exchange(self, dp: DevicePass, args: capi.Args, xch: "PeerExchange", rank: int | None = None, phases: int = 3,
                         wait_ms: int = 0, stream: int | None = None):
        """esp_attn_forward_exchange: a rank's split-KV step in one launch (args carry the records-only plan
        and its reduce job)."""
        s = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        x = xch.descriptor(xch.rank if rank is None else rank, phases, wait_ms)
        capi.check(self.lib.esp_attn_forward_exchange(self.ctx, C.c_void_p(s), C.byref(args), C.byref(x)))

    def attn_prep(self, X, qn_w, kn_w, pos, inv_freq, rope_sel, Q, Kb, Vb, pp: "capi.PrepParams", ktab=None, kv=None,
                  kv_scales=None, stream: int | None = None):
        """esp_attn_prep on device tensors: RMSNorm + rotary + cast of the fused projection X into Q / Kb / Vb
        (and, with ktab, into the paged pool)."""
        s = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        capi.check(self.lib.esp_attn_prep(self.ctx, C.c_void_p(s), _ptr(X), _ptr(qn_w), _ptr(kn_w), _ptr(pos), _ptr(inv_freq),
                                          _ptr(rope_sel), _ptr(Q), _ptr(Kb), _ptr(Vb), _ptr(ktab), _ptr(kv), _ptr(kv_scales),
                                          X.shape[0], C.byref(pp)))

    def kv_save(self, dp: DevicePass, entries: np.ndarray, stream: int | None = None):
        s = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        e = _dev(np.ascontiguousarray(entries, dtype=KVSAVE_DT), self.device)
        p = self.params(dp.w)
        capi.check(self.lib.esp_kv_save(self.ctx, C.c_void_p(s), _ptr(dp.Kb), _ptr(dp.Vb), _ptr(dp.kv), _ptr(dp.kv_scales), _ptr(e),
                                        len(entries), C.byref(p)))
        return e  # keep alive until the stream has run

    def kv_copy_blocks(self, dp: DevicePass, pairs: np.ndarray, region_elems: int, n_layers: int, stream: int | None = None):
        s = torch.cuda.current_stream(self.device).cuda_stream if stream is None else stream
        pr = _dev(np.ascontiguousarray(pairs, dtype=np.int32), self.device)
        p = self.params(dp.w)
        capi.check(self.lib.esp_kv_copy_blocks(self.ctx, C.c_void_p(s), _ptr(dp.kv), _ptr(pr), len(pairs), C.byref(p), region_elems,
                                               n_layers))
        return pr

    def check_status(self):
        s = torch.cuda.current_stream(self.device).cuda_stream
        capi.check(self.lib.esp_attn_check_status(self.ctx, C.c_void_p(s)))

    @property
    def last_kernel(self) -> str:
        return self.lib.esp_attn_last_kernel(self.ctx).decode()

    @property
    def launch_count(self) -> int:
        return int(self.lib.esp_attn_launch_count(self.ctx))


def run_pass(w: Workload, mode: int = capi.ESP_PLAN_REFERENCE, tile_rows: int = 8, split: int = 512, min_chunk: int = 32,
             groups: int = 256, options: dict | None = None, force_parts: bool = False, device: int = 0):
    """Plan + upload + forward + download for one workload; returns (O bits, lse, parts, plan, kernel name).
    force_parts: turn every unsplit tile into a one-record split so that the fp32 records can be inspected."""
    op = AttnOp.for_workload(w, tile_rows, device)
    try:
        for k, v in (options or {}).items():
            op.set_option(k, v)
        plan = plan_tiles(w.trees, w.Hkv, mode, split, min_chunk, groups, tile_rows)
        if force_parts:
            plan = force_partial_records(plan, w.trees)
        dp = op.upload(w, plan)
        op.forward(dp)
        op.check_status()
        torch.cuda.synchronize(op.device)
        O = dp.O.cpu().numpy().view(np.uint16)
        return O, dp.lse.cpu().numpy(), dp.parts.cpu().numpy(), plan, op.last_kernel
    finally:
        op.close()


def force_partial_records(plan: Plan, trees: np.ndarray) -> Plan:
    """Give every unsplit tile its own record and a one-record combine job (the kernels then write
    fp32 [O | m | l] for it and the combine kernel produces the output)."""
    tiles = plan.tiles.copy()
    jobs = list(plan.jobs)
    n_parts = plan.n_parts
    for t in tiles:
        if t["part"] < 0:
            t["part"] = n_parts
            tr = trees[int(t["tree"])]
            jobs.append((int(t["r0"]), min(plan.tile_rows, int(tr["base"]) + int(tr["M"]) - int(t["r0"])), n_parts, 1))
            n_parts += 1
    return Plan(tiles, np.array(jobs, dtype=COMBINE_DT) if jobs else np.zeros(0, dtype=COMBINE_DT), n_parts, plan.tile_rows)


class PeerExchange:
    """The exchange buffers of esp_attn_exchange_parts: this rank's buffer (esp_p2p_alloc) and the
    peers' mapped into this process (esp_p2p_open), handles carried by torch.distributed.

    PeerExchange(op, n_jobs, group=...) is the multi-process form (one process per GPU).
    PeerExchange.emulated(op, n_jobs, world) keeps `world` buffers on ONE GPU in one process, for
    tests that run the ranks' phases one after another.
    The caller bumps `epoch` (next_epoch()) once per exchange, on every rank alike."""

    def __init__(self, op: AttnOp, n_jobs: int, rows_max: int = 1, group=None):
        import torch.distributed as dist
        self.lib, self.op = op.lib, op
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.epoch = 0
        self._own, self._opened, self._desc = [], [], {}
        rec, handle = self._alloc(self._size(op, n_jobs, self.world))
        mine = torch.tensor(list(handle), dtype=torch.uint8, device=op.device)
        every = torch.empty(self.world * mine.numel(), dtype=torch.uint8, device=op.device)
        dist.all_gather_into_tensor(every, mine, group=group)
        every = bytes(every.cpu().numpy().tobytes())
        self.records = [rec if q == self.rank else self._open(every[q * 64:(q + 1) * 64]) for q in range(self.world)]
        dist.barrier(group)  # every rank has mapped every buffer before anyone writes

    @classmethod
    def emulated(cls, op: AttnOp, n_jobs: int, rows_max: int, world: int):
        self = cls.__new__(cls)
        self.lib, self.op, self.rank, self.world, self.epoch = op.lib, op, 0, world, 0
        self._own, self._opened, self._desc = [], [], {}
        nbytes = cls._size(op, n_jobs, world)
        self.sets = [self._alloc(nbytes)[0] for _ in range(world)]
        self.records = None
        return self

    @staticmethod
    def _size(op, n_jobs, world):
        n = op.lib.esp_attn_exchange_bytes(C.byref(op.shape), n_jobs, world)
        if n == 0:
            raise ValueError("exchange size: bad n_jobs / world")
        return n

    def _alloc(self, nbytes):
        ptr, h = C.c_void_p(), C.create_string_buffer(64)
        capi.check(self.lib.esp_p2p_alloc(C.byref(ptr), nbytes, h))
        self._own.append(ptr.value)
        return ptr.value, h.raw

    def _open(self, handle: bytes):
        ptr = C.c_void_p()
        capi.check(self.lib.esp_p2p_open(C.c_char_p(handle), C.byref(ptr)))
        self._opened.append(ptr.value)
        return ptr.value

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def descriptor(self, rank: int, phases: int = 3, wait_ms: int = 0) -> capi.Exchange:
        x = self._desc.get((rank, phases, wait_ms))
        if x is None:  # only the epoch changes between calls
            x = self._desc[(rank, phases, wait_ms)] = capi.Exchange()
            x.rank, x.world, x.phases, x.wait_ms = rank, self.world, phases, wait_ms
            for q in range(self.world):  # emulated ranks: rank q's own buffer is set q; all are local
                x.records[q] = self.sets[q] if self.records is None else self.records[q]
        x.epoch = self.epoch
        return x

    def close(self):
        torch.cuda.synchronize(self.op.device)
        for p in self._opened:
            capi.check(self.lib.esp_p2p_close(C.c_void_p(p)))
        for p in self._own:
            capi.check(self.lib.esp_p2p_free(C.c_void_p(p)))
        self._opened, self._own = [], []
