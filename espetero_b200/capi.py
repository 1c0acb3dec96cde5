"""ctypes binding of the C ABI declared in include/espetero_attn.h.

This module only loads the shared library and declares prototypes; it holds no
arithmetic. If the library has not been built (espetero_b200/lib/libespetero_attn.so)
loading raises: there is no CPU or PyTorch fallback for any entry point.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# ESPETERO_ATTN_LIB selects another build of the same library (A/B timing of two builds).
LIB_PATH = os.environ.get("ESPETERO_ATTN_LIB") or os.path.join(_HERE, "lib", "libespetero_attn.so")

ESP_OK = 0
ESP_ERR_INVALID, ESP_ERR_UNSUPPORTED, ESP_ERR_CUDA, ESP_ERR_CAPACITY, ESP_ERR_INJECTED, ESP_ERR_NO_DEVICE = -1, -2, -3, -4, -5, -6
ESP_F16, ESP_BF16, ESP_E4M3 = 0, 1, 2
ESP_ATTN_FLAG_GATE, ESP_ATTN_FLAG_ANC_MASK = 1, 2
ESP_PLAN_REFERENCE, ESP_PLAN_G4, ESP_PLAN_B200 = 0, 1, 2


class Params(C.Structure):
    _fields_ = [("H", C.c_int32), ("Hkv", C.c_int32), ("q_ld", C.c_int32), ("kv_ld", C.c_int32), ("g_ld", C.c_int32),
                ("bt", C.c_int32), ("kv_base", C.c_uint64)]


class Tree(C.Structure):
    _fields_ = [("base", C.c_int32), ("P", C.c_int32), ("table", C.c_int32), ("M", C.c_int32)]


class Tile(C.Structure):
    _fields_ = [("tree", C.c_int32), ("r0", C.c_int32), ("k0", C.c_int32), ("k1", C.c_int32), ("part", C.c_int32),
                ("last", C.c_int32), ("pad0", C.c_int32), ("pad1", C.c_int32)]


class Combine(C.Structure):
    _fields_ = [("r0", C.c_int32), ("rows", C.c_int32), ("part0", C.c_int32), ("nparts", C.c_int32)]


class KVSaveEntry(C.Structure):
    _fields_ = [("src_row", C.c_int32), ("block", C.c_int32), ("pos", C.c_int32), ("pad", C.c_int32)]


class Shape(C.Structure):
    _fields_ = [("H", C.c_int32), ("Hkv", C.c_int32), ("HD", C.c_int32), ("bt", C.c_int32), ("q_dtype", C.c_int32),
                ("kv_dtype", C.c_int32), ("tile_rows", C.c_int32), ("flags", C.c_int32), ("scale", C.c_float),
                ("reserved", C.c_int32 * 3)]


class PlanOpts(C.Structure):
    _fields_ = [("mode", C.c_int32), ("split", C.c_int32), ("min_chunk", C.c_int32), ("groups", C.c_int32),
                ("tile_rows", C.c_int32), ("max_parts", C.c_int32), ("reserved", C.c_int32 * 2)]


class TreeSpec(C.Structure):
    _fields_ = [("root", C.POINTER(C.c_int32)), ("root_len", C.c_int32), ("n_leaves", C.c_int32),
                ("root_pos", C.POINTER(C.c_int32)), ("leaf_offsets", C.POINTER(C.c_int32)), ("leaf_tokens", C.POINTER(C.c_int32)),
                ("noncausal", C.c_int32), ("score_root", C.c_int32)]


class Args(C.Structure):
    _fields_ = [("Q", C.c_void_p), ("Kb", C.c_void_p), ("Vb", C.c_void_p), ("kv", C.c_void_p), ("kv_scales", C.c_void_p),
                ("blocks", C.c_void_p), ("desc", C.c_void_p), ("anc_mask", C.c_void_p), ("X", C.c_void_p), ("O", C.c_void_p),
                ("lse", C.c_void_p), ("parts", C.c_void_p), ("tiles", C.c_void_p), ("trees", C.c_void_p), ("jobs", C.c_void_p),
                ("tiles_host", C.c_void_p), ("trees_host", C.c_void_p), ("jobs_host", C.c_void_p),
                ("n_tiles", C.c_int32), ("n_trees", C.c_int32), ("n_jobs", C.c_int32), ("n_rows", C.c_int32),
                ("n_blocks", C.c_int32), ("n_block_entries", C.c_int32), ("n_parts", C.c_int32), ("reserved", C.c_int32),
                ("p", Params), ("pos", C.c_void_p), ("window", C.c_int32), ("ring", C.c_int32), ("bidi", C.c_int32),
                ("reserved2", C.c_int32), ("dequant_scratch", C.c_void_p), ("dequant_scratch_bytes", C.c_uint64),
                ("qsa_tlist", C.c_void_p), ("qsa_tcount", C.c_void_p), ("qsa_rinfo", C.c_void_p), ("qsa_sel", C.c_void_p),
                ("qsa_nbw", C.c_int32), ("qsa_n_lists", C.c_int32), ("pos_host", C.c_void_p)]


class PrepParams(C.Structure):
    _fields_ = [("H", C.c_int32), ("Hkv", C.c_int32), ("ld", C.c_int32), ("q_off", C.c_int32), ("q_stride", C.c_int32),
                ("k_off", C.c_int32), ("v_off", C.c_int32), ("q_ld", C.c_int32), ("kv_ld", C.c_int32), ("rot_half", C.c_int32),
                ("eps", C.c_float), ("qscale", C.c_float), ("bt", C.c_int32), ("reserved", C.c_int32), ("kv_base", C.c_uint64)]


class ProfileEntry(C.Structure):
    _fields_ = [("kernel", C.c_char * 32), ("launches", C.c_uint32), ("gpu_ms", C.c_float)]


class Exchange(C.Structure):
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("phases", C.c_int32), ("wait_ms", C.c_int32), ("epoch", C.c_uint64),
                ("records", C.c_void_p * 8)]


assert C.sizeof(Params) == 32 and C.sizeof(Tree) == 16 and C.sizeof(Tile) == 32 and C.sizeof(Combine) == 16
assert C.sizeof(KVSaveEntry) == 16

# name -> (restype, argtypes); every symbol the header declares.
PROTOTYPES = {
    "esp_attn_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.POINTER(Shape)]),
    "esp_attn_destroy": (C.c_int, [C.c_void_p]),
    "esp_attn_last_error": (C.c_char_p, []),
    "esp_attn_abi_version": (C.c_int, []),
    "esp_attn_set_option": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int]),
    "esp_attn_get_option": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_int)]),
    "esp_attn_plan_window": (C.c_int, [C.POINTER(Tree), C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                       C.POINTER(Tile), C.c_int32, C.POINTER(Combine), C.c_int32, C.POINTER(C.c_int32),
                                       C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "esp_attn_plan": (C.c_int, [C.POINTER(Tree), C.c_int32, C.c_int32, C.POINTER(PlanOpts), C.POINTER(Tile), C.c_int32,
                                C.POINTER(Combine), C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "esp_attn_parts_floats": (C.c_size_t, [C.POINTER(Shape), C.c_int32]),
    "esp_attn_dequant_scratch_bytes": (C.c_size_t, [C.POINTER(Shape), C.c_int32]),
    "esp_attn_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(Args)]),
    "esp_attn_combine_parts": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.POINTER(Params), C.c_void_p, C.c_int32]),
    "esp_attn_reduce_parts": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(Params), C.c_void_p, C.c_int32, C.c_void_p,
                                        C.c_int32]),
    "esp_attn_exchange_bytes": (C.c_size_t, [C.POINTER(Shape), C.c_int32, C.c_int32]),
    "esp_attn_exchange_parts": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(Params),
                                          C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.POINTER(Exchange)]),
    "esp_shard_lpt": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "esp_attn_split_kv_ranges": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "esp_attn_plan_split_kv": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.POINTER(C.c_int32),
                                         C.POINTER(C.c_int32)]),
    "esp_attn_world_merge_jobs": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.POINTER(C.c_int32)]),
    "esp_attn_forward_exchange": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(Args), C.POINTER(Exchange)]),
    "esp_p2p_alloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t, C.c_char_p]),
    "esp_p2p_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "esp_p2p_close": (C.c_int, [C.c_void_p]),
    "esp_p2p_free": (C.c_int, [C.c_void_p]),
    "esp_kv_slot_save": (C.c_int, [C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                   C.c_uint64, C.c_uint64, C.c_void_p, C.c_int32, C.c_uint64]),
    "esp_kv_slot_load": (C.c_int, [C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(C.c_int32),
                                   C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.c_uint64, C.c_uint64,
                                   C.c_void_p, C.c_int32, C.c_uint64]),
    "esp_attn_prep": (C.c_int, [C.c_void_p] * 14 + [C.c_int32, C.POINTER(PrepParams)]),
    "esp_kv_save": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                              C.POINTER(Params)]),
    "esp_kv_copy_blocks": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(Params), C.c_uint64,
                                     C.c_int32]),
    "esp_kv_pool_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int32, C.c_int32]),
    "esp_kv_pool_destroy": (C.c_int, [C.c_void_p]),
    "esp_kv_free_count": (C.c_int32, [C.c_void_p]),
    "esp_kv_refcount": (C.c_int32, [C.c_void_p, C.c_int32]),
    "esp_kv_alloc": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32)]),
    "esp_kv_retain": (C.c_int, [C.c_void_p, C.c_int32]),
    "esp_kv_release": (C.c_int, [C.c_void_p, C.c_int32]),
    "esp_kv_target_blocks": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                       C.c_int32, C.POINTER(C.c_int32), C.c_void_p, C.c_int32, C.POINTER(C.c_int32)]),
    "esp_kv_target_new_blocks": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "esp_kv_save_entries": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "esp_kv_row_table": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "esp_forest_tree_rows": (C.c_int, [C.POINTER(TreeSpec), C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "esp_forest_anc_masks": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "esp_attn_decode_static": (C.c_int, [C.POINTER(Shape), C.c_void_p, C.POINTER(Args)]),
    "esp_attn_decode_static_status": (C.c_int, [C.c_void_p]),
    "esp_qsa_plan": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32,
                               C.c_void_p, C.c_int32, C.c_void_p]),
    "esp_attn_plan_qsa": (C.c_int, [C.POINTER(Tree), C.c_int32, C.c_int32, C.POINTER(PlanOpts), C.c_void_p, C.POINTER(Tile), C.c_int32,
                                    C.POINTER(Combine), C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "esp_qsa_select": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32]),
    "esp_qsa_tiles": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32]),
    "esp_attn_finite_check": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64, C.c_int32, C.c_float, C.c_void_p]),
    "esp_attn_set_trace": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32]),
    "esp_attn_stamp": (C.c_int, [C.c_void_p, C.c_void_p]),
    "esp_attn_last_kernel": (C.c_char_p, [C.c_void_p]),
    "esp_attn_check_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "esp_attn_set_profile": (C.c_int, [C.c_void_p, C.c_int]),
    "esp_attn_get_profile": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.POINTER(C.c_int32)]),
    "esp_attn_launch_count": (C.c_uint64, [C.c_void_p]),
}

_lib = None


class EspError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[esp {code}] {message}")
        self.code = code


def load() -> C.CDLL:
    """Load the library once; raise if it was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `make -C espetero_b200/csrc` "
                               "(or __graft_entry__.build()); there is no fallback path")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != ESP_OK:
        raise EspError(rc, load().esp_attn_last_error().decode())
