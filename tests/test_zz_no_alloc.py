"""esp_attn_decode_static: the decode entry point for hosts that may not allocate device
memory while serving (everything pre-sized at start-up, or an allocator that owns the GPU).
Its split-K records live in an array built into the library instead of a caller buffer.

The check: through the C ABI, on the same inputs and plan, its output and LSE must equal
those of esp_attn_forward (same kernels, so the comparison is bit for bit; the stated
tolerance of the suite, 2e-3, is asserted as well) - on two calls in a row, the second over
different inputs, because the array keeps the first call's records. Collected last so that
a failure here cannot hide any other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from espetero_b200 import capi, host, workloads as wl

pytestmark = pytest.mark.gpu


def _both(w, seed_note):
    """Run esp_attn_forward and esp_attn_decode_static on workload w; return both results."""
    lib = capi.load()
    op = host.AttnOp.for_workload(w)
    try:
        plan = host.plan_tiles(w.trees, w.Hkv)           # reference planner: splits every context
        assert plan.n_parts > 0, "the case must use split-K records"
        dp = op.upload(w, plan)
        args = op.make_args(dp)
        op.forward(dp, args)
        torch.cuda.synchronize()
        want_O, want_lse = dp.O.cpu().numpy().copy(), dp.lse.cpu().numpy().copy()
        dp.O.zero_()
        dp.lse.zero_()
        args.parts = None                                 # no caller buffer for the records
        args.n_parts = 0
        stream = torch.cuda.current_stream().cuda_stream
        # One call first (on a device's first call the library looks up its array's address), then the
        # measured one: free device memory as the driver reports it (cudaMemGetInfo sees every
        # allocation of the process, the library's own included; torch's counter would only see torch's).
        capi.check(lib.esp_attn_decode_static(C.byref(op.shape), C.c_void_p(stream), C.byref(args)))
        torch.cuda.synchronize()
        dp.O.zero_()
        dp.lse.zero_()
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        capi.check(lib.esp_attn_decode_static(C.byref(op.shape), C.c_void_p(stream), C.byref(args)))
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        capi.check(lib.esp_attn_decode_static_status(C.c_void_p(stream)))   # no bounded wait ran out
        return want_O, want_lse, dp.O.cpu().numpy(), dp.lse.cpu().numpy()
    finally:
        op.close()


def test_static_records_match_regular_entry_point_twice():
    cases = [
        wl.make_pass("noalloc_a", 9001, [(1024, 1), (300, 1), (4096, 1)], 32, 4, 128, 16, wl.BF16),
        wl.make_pass("noalloc_b", 9002, [(2500, 1), (64, 1)], 32, 8, 256, 16, wl.BF16, wl.E4M3),
    ]
    for i, w in enumerate(cases):
        want_O, want_lse, got_O, got_lse = _both(w, i)
        assert np.array_equal(got_O, want_O), f"call {i}: outputs differ"
        a = wl.from_bits16(got_O.view(np.uint16), w.q_dtype)
        b = wl.from_bits16(want_O.view(np.uint16), w.q_dtype)
        assert np.abs(a - b).max() <= 2e-3
        assert np.abs(got_lse - want_lse).max() <= 2e-3


def test_static_records_capacity_and_shape_limits():
    lib = capi.load()
    w = wl.make_pass("noalloc_big", 9003, [(2048, 1)] * 8, 32, 4, 128, 16, wl.BF16)
    op = host.AttnOp.for_workload(w)
    try:
        plan = host.plan_tiles(w.trees, w.Hkv, split=32, groups=1 << 14)   # 64 records per sequence
        need = (plan.n_parts) * w.Hkv * 8 * w.G * (w.HD + 2)
        assert need > (4 << 20)
        dp = op.upload(w, plan)
        args = op.make_args(dp)
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.esp_attn_decode_static(C.byref(op.shape), C.c_void_p(stream), C.byref(args))
        assert rc == capi.ESP_ERR_CAPACITY and b"esp_attn_forward" in lib.esp_attn_last_error()
    finally:
        op.close()
    # multi-row trees are not decode work
    w2 = wl.make_pass("noalloc_rows", 9004, [(128, 4)], 8, 2, 128, 16, wl.BF16)
    op = host.AttnOp.for_workload(w2)
    try:
        plan = host.plan_tiles(w2.trees, w2.Hkv)
        dp = op.upload(w2, plan)
        args = op.make_args(dp)
        rc = lib.esp_attn_decode_static(C.byref(op.shape), C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(args))
        assert rc == capi.ESP_ERR_UNSUPPORTED
    finally:
        op.close()


def test_static_records_refuse_jobs_beyond_the_array():
    """A combine job that names records past the built-in array, a job list without its host copy and
    a tree whose block list runs past the table are refused before anything is launched."""
    lib = capi.load()
    w = wl.make_pass("noalloc_jobs", 9005, [(1024, 1), (512, 1)], 32, 4, 128, 16, wl.BF16)
    op = host.AttnOp.for_workload(w)
    try:
        plan = host.plan_tiles(w.trees, w.Hkv)
        assert len(plan.jobs) > 0
        dp = op.upload(w, plan)
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        rec = w.Hkv * 8 * w.G * (w.HD + 2)
        # (i) a job whose records end past the array
        args = op.make_args(dp)
        jobs = (capi.Combine * len(plan.jobs)).from_buffer_copy(C.string_at(args.jobs_host, C.sizeof(capi.Combine) * len(plan.jobs)))
        jobs[0].part0 = (4 << 20) // rec - 1
        jobs[0].nparts = 4
        args.jobs_host = C.cast(jobs, C.c_void_p)
        assert lib.esp_attn_decode_static(C.byref(op.shape), stream, C.byref(args)) == capi.ESP_ERR_CAPACITY
        # (ii) jobs without the host copy: the bound cannot be proved
        args = op.make_args(dp)
        args.jobs_host = None
        assert lib.esp_attn_decode_static(C.byref(op.shape), stream, C.byref(args)) == capi.ESP_ERR_INVALID
        assert b"jobs_host" in lib.esp_attn_last_error()
        # (iii) a block table shorter than the trees need
        args = op.make_args(dp)
        args.n_block_entries = 3
        assert lib.esp_attn_decode_static(C.byref(op.shape), stream, C.byref(args)) == capi.ESP_ERR_INVALID
        # the well-formed call still runs afterwards
        args = op.make_args(dp)
        capi.check(lib.esp_attn_decode_static(C.byref(op.shape), stream, C.byref(args)))
        torch.cuda.synchronize()
    finally:
        op.close()
