"""The C-ABI library: loads without a GPU, exports every function include/espetero_attn.h
declares, keeps the record layouts of the reference (kernels/40_attention.metal:124-150,
:804-809, :868-873), and refuses to run without a device instead of falling back."""
import ctypes as C
import os
import re

import pytest
import torch

from espetero_b200 import capi

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "espetero_attn.h")


def _declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(esp_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    lib = capi.load()
    names = _declared_functions()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
        assert n in capi.PROTOTYPES, f"{n} has no ctypes prototype"
    assert lib.esp_attn_abi_version() == 4


def test_record_layouts():
    assert C.sizeof(capi.Params) == 32 and capi.Params.kv_base.offset == 24
    assert C.sizeof(capi.Tree) == 16 and C.sizeof(capi.Tile) == 32
    assert C.sizeof(capi.Combine) == 16 and C.sizeof(capi.KVSaveEntry) == 16
    assert capi.Tile.part.offset == 16 and capi.Tile.last.offset == 20


def test_parts_floats():
    lib = capi.load()
    s = capi.Shape(32, 8, 256, 16, capi.ESP_BF16, capi.ESP_E4M3, 8, 0, 0.0625)
    # records * Hkv * 8 rows * G * (HD + 2), src/model/impl/forest.h:2716
    assert lib.esp_attn_parts_floats(C.byref(s), 32) == 32 * 8 * 8 * 4 * 258


def test_create_rejects_bad_shapes_and_missing_device():
    lib = capi.load()
    ctx = C.c_void_p()
    bad = capi.Shape(30, 8, 128, 16, capi.ESP_BF16, capi.ESP_BF16, 8, 0, 0.1)
    assert lib.esp_attn_create(C.byref(ctx), 0, C.byref(bad)) == capi.ESP_ERR_INVALID
    assert b"multiple of Hkv" in lib.esp_attn_last_error()
    bad = capi.Shape(32, 8, 96, 16, capi.ESP_BF16, capi.ESP_BF16, 8, 0, 0.1)
    assert lib.esp_attn_create(C.byref(ctx), 0, C.byref(bad)) == capi.ESP_ERR_UNSUPPORTED
    bad = capi.Shape(32, 8, 128, 16, capi.ESP_BF16, capi.ESP_F16, 8, 0, 0.1)
    assert lib.esp_attn_create(C.byref(ctx), 0, C.byref(bad)) == capi.ESP_ERR_UNSUPPORTED
    if not torch.cuda.is_available():
        ok = capi.Shape(32, 8, 128, 16, capi.ESP_BF16, capi.ESP_BF16, 8, 0, 0.1)
        rc = lib.esp_attn_create(C.byref(ctx), 0, C.byref(ok))
        assert rc == capi.ESP_ERR_NO_DEVICE and b"no CPU path" in lib.esp_attn_last_error()
        assert not ctx.value


def test_host_op_refuses_to_run_on_cpu():
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from espetero_b200 import host
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        host.AttnOp(8, 2, 128, 16, capi.ESP_F16, capi.ESP_F16, 0.1)


def test_ctypes_structs_have_the_headers_layout(tmp_path):
    """sizeof of every struct the header declares, as gcc sees it, against the ctypes mirrors (a field
    missing from a mirror would otherwise be accepted silently as a Python attribute)."""
    import ctypes as C
    import subprocess
    pairs = {"esp_attn_params": capi.Params, "esp_attn_tree": capi.Tree, "esp_attn_tile": capi.Tile, "esp_attn_combine": capi.Combine,
             "esp_kv_save_entry": capi.KVSaveEntry, "esp_attn_shape": capi.Shape, "esp_plan_opts": capi.PlanOpts,
             "esp_attn_args": capi.Args, "esp_attn_exchange": capi.Exchange, "esp_attn_prep_params": capi.PrepParams,
             "esp_tree_spec": capi.TreeSpec}
    src = tmp_path / "sizes.c"
    body = "".join(f'  printf("{n} %zu\\n", sizeof({n}));\n' for n in pairs)
    src.write_text(f'#include <stdio.h>\n#include "espetero_attn.h"\nint main(void) {{\n{body}  return 0;\n}}\n')
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c99", "-I", os.path.dirname(HEADER), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    sizes = dict(line.split() for line in out.strip().splitlines())
    for name, mirror in pairs.items():
        assert int(sizes[name]) == C.sizeof(mirror), name
