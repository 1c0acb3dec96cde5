"""Seeded synthetic inputs for the attention path (numpy only, host memory).

The reference publishes no dataset for this path; its own kernel check builds a shuffled
page table and an N(0,1) fp16 pool (tools/qsa_check.mm:105-132). These generators do the
same with the shapes and distributions of the five benchmark configurations: values
~ N(0,1) rounded to the storage type, physical block order a seeded permutation of the
pool, context lengths / tree parents / FP8 scales drawn from the same seeded stream.

Everything is returned in storage form: fp16 / bf16 as uint16 bit patterns, E4M3 as uint8
codes, so that the oracle, the CPU baseline and the CUDA kernels see identical bytes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
import numpy as np

F16, BF16, E4M3 = 0, 1, 2
FLAG_GATE, FLAG_ANC_MASK = 1, 2

TREE_DT = np.dtype([("base", "<i4"), ("P", "<i4"), ("table", "<i4"), ("M", "<i4")])
TILE_DT = np.dtype([("tree", "<i4"), ("r0", "<i4"), ("k0", "<i4"), ("k1", "<i4"), ("part", "<i4"), ("last", "<i4"),
                    ("pad0", "<i4"), ("pad1", "<i4")])
COMBINE_DT = np.dtype([("r0", "<i4"), ("rows", "<i4"), ("part0", "<i4"), ("nparts", "<i4")])
KVSAVE_DT = np.dtype([("src_row", "<i4"), ("block", "<i4"), ("pos", "<i4"), ("pad", "<i4")])


# ----------------------------------------------------------------------------- codecs
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (r >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def f16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return b.view(np.float16).astype(np.float32)


def to_bits16(x: np.ndarray, dtype: int) -> np.ndarray:
    return f32_to_f16_bits(x) if dtype == F16 else f32_to_bf16_bits(x)


def from_bits16(b: np.ndarray, dtype: int) -> np.ndarray:
    return f16_bits_to_f32(b) if dtype == F16 else bf16_bits_to_f32(b)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> e4m3fn codes: round to nearest even, subnormal step 2^-9 below 2^-6,
    saturating at +-448, no infinities (the grid of kernels/80_dsv4.metal:22-33)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x), np.float32(448.0))
    m, e = np.frexp(a)  # a = m * 2^e, m in [0.5, 1)
    step = np.where(a < 2.0 ** -6, np.float32(2.0 ** -9), np.ldexp(np.float32(1.0), e - 4)).astype(np.float32)
    q = np.rint(a / step) * step  # rint = nearest even
    m2, e2 = np.frexp(q)
    sub = q < 2.0 ** -6
    code_sub = np.rint(q * 512.0).astype(np.int32)
    code_norm = ((e2 - 1 + 7) << 3) | (np.rint(m2 * 16.0).astype(np.int32) - 8)
    code = np.where(sub, code_sub, code_norm)
    code = np.where(q == 0, 0, code)
    sign = np.where(np.signbit(x), 0x80, 0)
    return (code | sign).astype(np.uint8)


def e4m3_decode(c: np.ndarray) -> np.ndarray:
    c = c.astype(np.int32)
    e, m = (c >> 3) & 0xF, c & 7
    v = np.where(e == 0, np.ldexp(m.astype(np.float32), -9), np.ldexp((8 + m).astype(np.float32), e - 10))
    v = np.where((e == 15) & (m == 7), np.float32(np.nan), v)
    return np.where(c & 0x80, -v, v).astype(np.float32)


# ----------------------------------------------------------------------------- workload
@dataclass
class Workload:
    """One attention pass in host memory, in the layout of the reference's bindings
    (src/model/impl/forest.h:2902-2913)."""
    name: str
    H: int
    Hkv: int
    HD: int
    bt: int
    q_dtype: int
    kv_dtype: int
    scale: float
    flags: int
    n_rows: int
    n_blocks: int
    Q: np.ndarray            # [rows, q_ld] uint16
    Kb: np.ndarray           # [rows, kv_ld] uint16
    Vb: np.ndarray
    kv: np.ndarray           # flat pool, uint16 or uint8
    kv_scales: np.ndarray | None  # [n_blocks, 2, Hkv] float32
    blocks: np.ndarray       # int32
    desc: np.ndarray         # [rows, 4] int32
    anc_mask: np.ndarray | None   # [rows] uint64
    X: np.ndarray | None     # [rows, g_ld] float32
    trees: np.ndarray        # TREE_DT
    kv_base: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def G(self) -> int:
        return self.H // self.Hkv

    @property
    def q_ld(self) -> int:
        return self.H * self.HD

    @property
    def kv_ld(self) -> int:
        return self.Hkv * self.HD

    @property
    def g_ld(self) -> int:
        return 2 * self.H * self.HD

    @property
    def kv_elem_bytes(self) -> int:
        return 1 if self.kv_dtype == E4M3 else 2

    def kv_bytes_read(self) -> int:
        """Algorithmic K+V bytes one pass must read: cached keys of every tree, all kv heads
        (+ FP8 scales); batch keys are not counted."""
        pages = sum((int(t["P"]) + self.bt - 1) // self.bt for t in self.trees)
        keys = int(self.trees["P"].sum())
        b = keys * 2 * self.kv_ld * self.kv_elem_bytes
        if self.kv_dtype == E4M3:
            b += pages * 2 * self.Hkv * 4
        return b


def _normal_bits(rng: np.random.Generator, shape, dtype: int) -> np.ndarray:
    n = int(np.prod(shape))
    out = np.empty(n, dtype=np.uint16)
    step = 1 << 24
    for i in range(0, n, step):
        out[i:i + step] = to_bits16(rng.standard_normal(min(step, n - i), dtype=np.float32), dtype)
    return out.reshape(shape)


def _fill_pool(rng, n_blocks, bt, kv_ld, Hkv, HD, kv_dtype, q_dtype):
    """Pool of n_blocks blocks [K: bt x kv_ld][V: bt x kv_ld]; every block is filled (spare
    blocks too, so that a wrong block id reads plausible numbers, not zeros)."""
    n = n_blocks * 2 * bt * kv_ld
    if kv_dtype != E4M3:
        return _normal_bits(rng, (n,), kv_dtype), None
    # scale per (block, K|V, kv head), log-uniform in [2^-4, 2^2]; code = e4m3(x / s)
    scales = np.exp2(rng.uniform(-4.0, 2.0, size=(n_blocks, 2, Hkv))).astype(np.float32)
    kv = np.empty(n, dtype=np.uint8)
    view = kv.reshape(n_blocks, 2, bt, Hkv, HD)
    chunk = max(1, (1 << 24) // (2 * bt * kv_ld))
    for b0 in range(0, n_blocks, chunk):
        b1 = min(n_blocks, b0 + chunk)
        x = rng.standard_normal((b1 - b0, 2, bt, Hkv, HD), dtype=np.float32)
        view[b0:b1] = e4m3_encode(x / scales[b0:b1, :, None, :, None])
    return kv, scales


def make_pass(name: str, seed: int, trees_PM, H: int, Hkv: int, HD: int, bt: int, q_dtype: int, kv_dtype: int | None = None,
              scale: float | None = None, gate: bool = False, mask: str = "causal", spare_blocks: int = 3,
              parents: list | None = None) -> Workload:
    """Build one pass. trees_PM = [(P, M), ...]. mask: "causal" (desc = (0,0,0,0): each row sees
    batch keys 0..itself), "tree" (ancestor bit mask from `parents` or seeded random parents:
    node i's parent uniform over 0..i-1, node sees its ancestor chain and itself), or
    "forest" (desc with a root of ceil(M/2) rows and one leaf segment: rows of the leaf see
    the whole root and their own segment up to themselves)."""
    rng = np.random.default_rng(seed)
    kv_dtype = q_dtype if kv_dtype is None else kv_dtype
    scale = float(1.0 / np.sqrt(HD)) if scale is None else scale
    q_ld, kv_ld = H * HD, Hkv * HD
    n_rows = sum(M for _, M in trees_PM)
    pages = [(P + bt - 1) // bt for P, _ in trees_PM]
    n_blocks = sum(pages) + spare_blocks
    perm = rng.permutation(n_blocks).astype(np.int32)
    trees = np.zeros(len(trees_PM), dtype=TREE_DT)
    blocks = np.empty(max(1, sum(pages)), dtype=np.int32)
    base = tab = 0
    for i, (P, M) in enumerate(trees_PM):
        trees[i] = (base, P, tab, M)
        blocks[tab:tab + pages[i]] = perm[tab:tab + pages[i]]
        base += M
        tab += pages[i]
    Q = _normal_bits(rng, (n_rows, q_ld), q_dtype)
    Kb = _normal_bits(rng, (n_rows, kv_ld), q_dtype)
    Vb = _normal_bits(rng, (n_rows, kv_ld), q_dtype)
    kv, scales = _fill_pool(rng, n_blocks, bt, kv_ld, Hkv, HD, kv_dtype, q_dtype)
    desc = np.zeros((n_rows, 4), dtype=np.int32)
    anc = None
    flags = FLAG_GATE if gate else 0
    extra = {}
    if mask == "tree":
        anc = np.zeros(n_rows, dtype=np.uint64)
        all_parents = []
        for i, (P, M) in enumerate(trees_PM):
            par = [-1] + [int(rng.integers(0, j)) for j in range(1, M)] if parents is None else list(parents[i])
            all_parents.append(par)
            for j in range(M):
                bits, k = 0, j
                while k >= 0:
                    bits |= 1 << k
                    k = par[k]
                anc[int(trees[i]["base"]) + j] = bits
        flags |= FLAG_ANC_MASK
        extra["parents"] = all_parents
    elif mask == "forest":
        for i, (P, M) in enumerate(trees_PM):
            root = (M + 1) // 2
            b0 = int(trees[i]["base"])
            for j in range(M):
                desc[b0 + j] = (0, 0, 0, 0) if j < root else (root, 0, root, 0)
    X = rng.standard_normal((n_rows, 2 * q_ld), dtype=np.float32) if gate else None
    return Workload(name, H, Hkv, HD, bt, q_dtype, kv_dtype, scale, flags, n_rows, n_blocks, Q, Kb, Vb, kv, scales, blocks, desc,
                    anc, X, trees, 0, extra)


def make_window_pass(name: str, seed: int, trees_PM, H: int, Hkv: int, HD: int, bt: int, q_dtype: int, window: int,
                     ring: int = 0, images=None, scale: float = 1.0, kv_dtype: int | None = None) -> Workload:
    """A pass of a sliding-window layer of the generic kernel (kernels/80_gemma.metal:123-142): causal
    rows at positions P, P + 1, ... behind P cached keys, keys `window` or more positions back masked.
    ring > 0: a tree's cached keys live in its own ring of `ring` blocks (key j in block
    table + (j / bt) % ring), no page table. images = {tree: (first row, end row)}: those rows carry
    desc.w = end and, with bidi, see the whole image. The parameters travel in extra["window"]."""
    n_trees = len(trees_PM)
    w = make_pass(name, seed, trees_PM, H, Hkv, HD, bt, q_dtype, kv_dtype, scale=scale, spare_blocks=3 + n_trees * max(ring, 0))
    pos = np.zeros((w.n_rows, 4), dtype=np.int32)
    for i, (P, M) in enumerate(trees_PM):
        b0 = int(w.trees[i]["base"])
        pos[b0:b0 + M, 0] = P + np.arange(M)
        pos[b0:b0 + M, 1:3] = pos[b0:b0 + M, 0:1]
        if ring > 0:
            w.trees[i]["table"] = i * ring
        if images and i in images:
            a, b = images[i]
            w.desc[b0 + a:b0 + b, 3] = b
    w.extra["window"] = {"pos": pos, "window": int(window), "ring": int(ring), "bidi": 1 if images else 0}
    return w


# ----------------------------------------------------------------------------- the five configurations
def config_c1(seed: int = 0xE5B201) -> Workload:
    """Single-sequence paged decode: 1 query token, H8/Hkv2/HD128 fp16, 1024 cached tokens, 16-token pages."""
    return make_pass("c1_single_decode", seed, [(1024, 1)], 8, 2, 128, 16, F16)


def c2_context_lengths(seed: int = 0xE5B202, n_seqs: int = 32, lo: int = 512, hi: int = 32768) -> np.ndarray:
    """The context lengths config_c2 draws for `seed`."""
    return np.random.default_rng(seed ^ 0x5EED).integers(lo, hi + 1, size=n_seqs)


def config_c2(seed: int = 0xE5B202, n_seqs: int = 32, lo: int = 512, hi: int = 32768, lens=None, hd: int = 128,
              kv_dtype: int | None = None) -> Workload:
    """Batched paged decode: 32 sequences, context ~ U[512, 32768], H32/Hkv4/HD128 bf16, 16-token pages.
    `lens` overrides the drawn lengths (a rank's share of a batch partitioned over several GPUs). hd / kv_dtype: the same
    batch with another head dim of the reference's kernels or over an E4M3 pool (not one of the five configurations)."""
    lens = c2_context_lengths(seed, n_seqs, lo, hi) if lens is None else np.asarray(lens)
    name = "c2_batched_decode" + (f"_hd{hd}" if hd != 128 else "") + ("_e4m3" if kv_dtype == E4M3 else "")
    w = make_pass(name, seed, [(int(p), 1) for p in lens], 32, 4, hd, 16, BF16, kv_dtype=kv_dtype)
    w.extra["ctx_lens"] = lens
    return w


def config_c3(seed: int = 0xE5B203, n_seqs: int = 4, rows: int = 8192, hd: int = 128) -> Workload:
    """Causal prefill: 4 sequences of 8192 tokens, no cached prefix, H64/Hkv8/HD128 bf16. hd = 64 / 256 / 512: the
    same pass with another head dim of the reference's kernels (8192 / hd heads: as many flops; not one of the five configurations)."""
    if hd != 128:  # the same Q width and flops: 8192 / hd heads
        return make_pass(f"c3_causal_prefill_hd{hd}", seed, [(0, rows)] * n_seqs, 8192 // hd, 1024 // hd, hd, 16, BF16,
                         spare_blocks=n_seqs * ((rows + 15) // 16))
    return make_pass("c3_causal_prefill", seed, [(0, rows)] * n_seqs, 64, 8, 128, 16, BF16, spare_blocks=n_seqs * ((rows + 15) // 16))


def config_c4(seed: int = 0xE5B204, n_seqs: int = 16, prefix: int = 4096, nodes: int = 16, kv_dtype: int | None = None,
              hd: int = 128) -> Workload:
    """Forest tree-verify: 16 sequences, 4096-token prefix + 16-node draft tree (random parents). kv_dtype = E4M3: the
    same pass over an FP8 pool (not one of the five configurations: the tcgen05 kernel's own dequantisation).
    hd = 256: the same pass with the reference kernels' own head dim (twice the key bytes; not one of the five either)."""
    name = "c4_tree_verify" if kv_dtype in (None, BF16) else "c4_tree_verify_e4m3"
    if hd != 128:
        name += f"_hd{hd}"
    return make_pass(name, seed, [(prefix, nodes)] * n_seqs, 32, 4, hd, 16, BF16, kv_dtype=kv_dtype, mask="tree")


def config_c5(seed: int = 0xE5B205, ctx: int = 131072, lo: int = 0, hi: int | None = None) -> Workload:
    """Long-context split-KV decode: 1 sequence of 131072 tokens, H32/Hkv8/HD256, E4M3 KV with one fp32
    scale per (page, K|V, kv head) log-uniform in [2^-4, 2^2] (K and V tables drawn independently)."""
    return make_pass("c5_long_fp8_decode", seed, [(ctx, 1)], 32, 8, 256, 16, BF16, kv_dtype=E4M3)


CONFIGS = {"c1": config_c1, "c2": config_c2, "c3": config_c3, "c4": config_c4, "c5": config_c5}
