// C-ABI entry points of the attention path: context, options, host-side validation,
// kernel selection and launches. Mirrors the attention() / kv_save() / kv_cow_copy()
// dispatch code of the reference (src/model/impl/forest.h:2855-2947, :1438-1449).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "host_util.h"
#include "launch.h"

using esp::fail;

struct esp_attn_ctx {
  int device = 0;
  esp_attn_shape shape{};
  int G = 1;
  int tile_rows = 8;
  // options (NativeModel::set_option analogue)
  int opt_attn_gqa = 1;
  int opt_attn_umma = 1;
  int opt_validate = 1;
  int opt_umma_kernel = 0;  // 0: choose by the pass, 1: flash_umma (HBM streaming), 2: flash_umma_pair (L2-resident keys), 3: flash_umma_duo (two query tiles per CTA)
  // host-side fault injection: every Nth pass of 64 rows or more fails before launch
  // (ESPETERO_FAIL_PASS of the reference, forest.h:2521-2531)
  int fail_every = 0;
  uint64_t pass_count = 0;
  uint64_t launches = 0;
  const char* last_kernel = "";
  int* d_status = nullptr;
  unsigned long long* trace = nullptr;  // caller-owned device buffer (esp_attn_set_trace)
  int32_t trace_blocks = 0;
  int opt_fuse_combine = 1;  // small tcgen05 passes merge their split-K records in the attention kernel (last CTA of a job)
  bool finite_armed = false;  // a pass has been checked since the record was last read
  int opt_check_finite = 0;  // scan O for NaN / Inf after every pass (ESPETERO_CHECK_FINITE of the reference)
  int opt_trace_ctas = 0;  // per-CTA stamps behind the block events (the buffer must hold 8 * n_blocks + 2 + 4 * this)
  // driver entry point for tensor maps, resolved without linking libcuda
  void* encode_tiled = nullptr;
  // cached pool tensor map
  CUtensorMap pool_map{};
  const void* map_kv = nullptr;
  uint64_t map_base = 0;
  int32_t map_blocks = 0, map_bt = 0, map_ld = 0;
  // tensor maps of the tcgen05 kernel: pool pages, Kb rows, Vb rows (64 dims x 16 rows per load)
  CUtensorMap upool_map{}, kb_map{}, vb_map{};
  const void* umap_kv = nullptr;
  const void* umap_kb = nullptr;
  const void* umap_vb = nullptr;
  uint64_t umap_base = 0;
  int32_t umap_blocks = 0, umap_rows = 0, umap_ld = 0;
  // Re-planning of reference-shaped multi-row passes (8-row tiles) for the tensor-core kernels: the new
  // tiles and jobs are built on the host and travel through a small ring of pinned staging slots into
  // device slots of the context (see replan_pass).
  int opt_replan = 1;
  int opt_fp8_direct = 1;  // E4M3 pools: passes over mostly cached keys read the codes inside flash_umma (no widening pre-pass)
  int opt_stable_cache = 0;  // see KernelArgs::stable_cache
  int opt_pair_merge = 1;  // flash_umma: passes whose jobs all have two records merge them inside a cluster pair (distributed shared memory)
  int opt_fuse_exchange = 0;  // esp_attn_forward_exchange: 1 = merge and exchange inside the decode kernel (one launch); 0 = two kernels (measured faster)
  uint8_t* replan_dev = nullptr;
  uint8_t* replan_host = nullptr;
  cudaEvent_t replan_done[4] = {nullptr, nullptr, nullptr, nullptr};
  bool replan_used[4] = {false, false, false, false};
  int replan_next = 0;
  std::vector<esp_attn_tile> rp_tiles;
  std::vector<esp_attn_combine> rp_jobs;
  // Per-dispatch GPU time (esp_attn_set_profile; the reference's set_profile, src/model/model.mm:1041-1054): an event
  // pair around every launch while profiling is on, summed per kernel name when the profile is read.
  bool profiling = false;
  struct ProfSpan {
    const char* kernel;
    cudaEvent_t t0, t1;
  };
  std::vector<ProfSpan> prof_pending;
  std::vector<cudaEvent_t> prof_free;
  struct ProfSum {
    const char* kernel;
    uint32_t launches;
    double ms;
  };
  std::vector<ProfSum> prof_sums;
};

namespace {
// Brackets the launches made while it lives with an event pair on `stream` (profiling on), else does nothing.
struct ProfScope {
  esp_attn_ctx* c;
  cudaStream_t stream;
  const char* kernel;
  cudaEvent_t t0 = nullptr, t1 = nullptr;
  static cudaEvent_t take(esp_attn_ctx* c) {
    if (!c->prof_free.empty()) {
      cudaEvent_t e = c->prof_free.back();
      c->prof_free.pop_back();
      return e;
    }
    cudaEvent_t e = nullptr;
    return cudaEventCreate(&e) == cudaSuccess ? e : nullptr;
  }
  ProfScope(esp_attn_ctx* ctx, cudaStream_t s, const char* k) : c(ctx), stream(s), kernel(k) {
    if (!c->profiling) return;
    t0 = take(c), t1 = take(c);
    if (t0 && t1) cudaEventRecord(t0, stream);
  }
  ~ProfScope() {
    if (!c->profiling || !t0 || !t1) return;
    cudaEventRecord(t1, stream);
    c->prof_pending.push_back({kernel, t0, t1});
  }
};
}  // namespace

namespace {

// The context's device allocation: the status word, then (64 ints further) the arrival counters
// of fused merges.
constexpr size_t kStatusBytes = sizeof(int) * (64 + esp::kFixupCounters);
constexpr int kFiniteRecAt = 16;  // ints 16..19 of the status header: the finite-check record of the last pass

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int cuda_fail(cudaError_t e, const char* what) {
  return fail(ESP_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

int elem_bytes(int dt) { return dt == ESP_E4M3 ? 1 : 2; }

int check_shape(const esp_attn_shape& s) {
  if (s.H <= 0 || s.Hkv <= 0 || s.H % s.Hkv != 0) return fail(ESP_ERR_INVALID, "shape: H=%d must be a positive multiple of Hkv=%d", s.H, s.Hkv);
  if (s.HD != 64 && s.HD != 128 && s.HD != 256 && s.HD != 512) return fail(ESP_ERR_UNSUPPORTED, "shape: head dim %d (64, 128, 256 or 512)", s.HD);
  if (s.bt <= 0) return fail(ESP_ERR_INVALID, "shape: bt=%d", s.bt);
  if (s.q_dtype != ESP_F16 && s.q_dtype != ESP_BF16) return fail(ESP_ERR_UNSUPPORTED, "shape: q_dtype %d (fp16 or bf16)", s.q_dtype);
  if (s.kv_dtype != s.q_dtype && s.kv_dtype != ESP_E4M3)
    return fail(ESP_ERR_UNSUPPORTED, "shape: kv_dtype %d must equal q_dtype or be E4M3", s.kv_dtype);
  if (s.tile_rows != 0 && s.tile_rows != 8 && s.tile_rows != 16 && s.tile_rows != 32 && s.tile_rows != 64 && s.tile_rows != 128)
    return fail(ESP_ERR_UNSUPPORTED, "shape: tile_rows %d (8, 16, 32, 64 or 128)", s.tile_rows);
  if (!(s.scale > 0.0f)) return fail(ESP_ERR_INVALID, "shape: scale must be positive");
  return ESP_OK;
}

int check_params(const esp_attn_ctx* c, const esp_attn_params& p) {
  const esp_attn_shape& s = c->shape;
  if (p.H != s.H || p.Hkv != s.Hkv || p.bt != s.bt) return fail(ESP_ERR_INVALID, "params: H/Hkv/bt (%d/%d/%d) differ from the context's (%d/%d/%d)", p.H, p.Hkv, p.bt, s.H, s.Hkv, s.bt);
  if (p.q_ld < s.H * s.HD || p.q_ld % 8) return fail(ESP_ERR_INVALID, "params: q_ld=%d (>= H*HD, multiple of 8)", p.q_ld);
  if (p.kv_ld < s.Hkv * s.HD || p.kv_ld % 16) return fail(ESP_ERR_INVALID, "params: kv_ld=%d (>= Hkv*HD, multiple of 16)", p.kv_ld);
  if (p.kv_base % 16) return fail(ESP_ERR_INVALID, "params: kv_base must be a multiple of 16 elements");
  if ((s.flags & ESP_ATTN_FLAG_GATE) && (p.g_ld < s.H * 2 * s.HD || p.g_ld % 4)) return fail(ESP_ERR_INVALID, "params: g_ld=%d (>= 2*H*HD, multiple of 4)", p.g_ld);
  return ESP_OK;
}

bool windowed_lists(const esp_attn_args& a) { return a.qsa_tlist != nullptr; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// The checks run_forest makes before it encodes a pass (forest.h:2136-2280), on the host
// mirrors of the plan. Nothing is launched when one fails. `deep` = also walk the mirrors
// (the "validate" option of a context).
int esp::validate_pass(const esp_attn_shape& s, int TR, bool deep, const esp_attn_args& a) {
  if (a.n_tiles < 0 || a.n_trees < 0 || a.n_jobs < 0 || a.n_rows < 0) return fail(ESP_ERR_INVALID, "forward: negative count");
  if (a.n_tiles == 0) return ESP_OK;
  if (!a.Q || !a.Kb || !a.Vb || !a.O || !a.tiles || !a.trees) return fail(ESP_ERR_INVALID, "forward: null Q/Kb/Vb/O/tiles/trees");
  if (!aligned16(a.Q) || !aligned16(a.Kb) || !aligned16(a.Vb) || !aligned16(a.O) || !aligned16(a.kv) || !aligned16(a.parts))
    return fail(ESP_ERR_INVALID, "forward: data pointers must be 16-byte aligned");
  if (s.kv_dtype == ESP_E4M3 && !a.kv_scales) return fail(ESP_ERR_INVALID, "forward: E4M3 pool needs kv_scales");
  if ((s.flags & ESP_ATTN_FLAG_GATE) && !a.X) return fail(ESP_ERR_INVALID, "forward: gate flag set but X is null");
  if ((s.flags & ESP_ATTN_FLAG_ANC_MASK) ? !a.anc_mask : !a.desc) return fail(ESP_ERR_INVALID, "forward: the row mask (desc or anc_mask) is null");
  if (a.n_jobs > 0 && (!a.jobs || !a.parts)) return fail(ESP_ERR_INVALID, "forward: combine jobs need jobs and parts");
  if (a.window < 0 || a.ring < 0) return fail(ESP_ERR_INVALID, "forward: window=%d ring=%d", a.window, a.ring);
  if (a.window > 0 && !a.pos) return fail(ESP_ERR_INVALID, "forward: a sliding window needs the rows' positions (pos)");
  if (a.bidi && (s.flags & ESP_ATTN_FLAG_ANC_MASK)) return fail(ESP_ERR_UNSUPPORTED, "forward: bidi uses desc.w and cannot be combined with ancestor masks");
  if (a.qsa_tlist) {
    if (!a.qsa_tcount || !a.qsa_rinfo || !a.qsa_sel || a.qsa_nbw <= 0 || a.qsa_n_lists <= 0)
      return fail(ESP_ERR_INVALID, "forward: sparse attention needs tlist, tcount, rinfo, sel, nbw and the list count together");
    if (s.flags & ESP_ATTN_FLAG_ANC_MASK) return fail(ESP_ERR_UNSUPPORTED, "forward: sparse attention reads the rows' desc records, not ancestor masks");
    if (a.window > 0 || a.ring > 0 || a.bidi) return fail(ESP_ERR_UNSUPPORTED, "forward: sparse attention and sliding-window layers do not combine");
  }
  if (!deep || !a.trees_host || !a.tiles_host) return ESP_OK;
  bool any_cached = false;
  for (int i = 0; i < a.n_trees; ++i) {
    const esp_attn_tree& t = a.trees_host[i];
    if (t.base < 0 || t.M < 0 || t.P < 0 || t.table < 0) return fail(ESP_ERR_INVALID, "tree %d: negative field", i);
    if (int64_t(t.base) + t.M > a.n_rows) return fail(ESP_ERR_INVALID, "tree %d: rows [%d, %d) beyond the pass's %d rows", i, t.base, t.base + t.M, a.n_rows);
    if (t.P > 0) {
      any_cached = true;
      if (a.ring > 0) {
        if (int64_t(t.table) + a.ring > a.n_blocks) return fail(ESP_ERR_INVALID, "tree %d: ring [%d, +%d) beyond the %d blocks of the region", i, t.table, a.ring, a.n_blocks);
      } else if (int64_t(t.table) + (t.P + s.bt - 1) / s.bt > a.n_block_entries) {
        return fail(ESP_ERR_INVALID, "tree %d: block list [%d, +%d) beyond the %d entries of blocks", i, t.table, (t.P + s.bt - 1) / s.bt, a.n_block_entries);
      }
    }
    if ((s.flags & ESP_ATTN_FLAG_ANC_MASK) && t.M > 64) return fail(ESP_ERR_UNSUPPORTED, "tree %d: %d rows with a 64-bit ancestor mask", i, t.M);
  }
  if (any_cached && (!a.kv || (!a.blocks && a.ring <= 0) || a.n_blocks <= 0)) return fail(ESP_ERR_INVALID, "forward: cached keys but no pool / block table");
  for (int i = 0; i < a.n_tiles; ++i) {
    const esp_attn_tile& t = a.tiles_host[i];
    if (t.tree < 0 || t.tree >= a.n_trees) return fail(ESP_ERR_INVALID, "tile %d: tree %d of %d", i, t.tree, a.n_trees);
    const esp_attn_tree& tr = a.trees_host[t.tree];
    if (t.r0 < tr.base || t.r0 >= tr.base + tr.M) return fail(ESP_ERR_INVALID, "tile %d: first row %d outside its tree [%d, %d)", i, t.r0, tr.base, tr.base + tr.M);
    if (a.qsa_tlist && t.pad0 != 0) {  // Qwen sparse attention: k0 / k1 are entries of union list pad1 (the last part is open-ended)
      if (t.k0 < 0 || t.k0 > t.k1) return fail(ESP_ERR_INVALID, "tile %d: list entries [%d, %d)", i, t.k0, t.k1);
      if (t.pad1 < 0 || t.pad1 >= a.qsa_n_lists) return fail(ESP_ERR_INVALID, "tile %d: union list %d of %d", i, t.pad1, a.qsa_n_lists);
    } else if (t.k0 < 0 || t.k0 > t.k1 || t.k1 > tr.P) {
      return fail(ESP_ERR_INVALID, "tile %d: key range [%d, %d) outside [0, %d]", i, t.k0, t.k1, tr.P);
    }
    if (t.part >= a.n_parts) return fail(ESP_ERR_INVALID, "tile %d: record %d of %d", i, t.part, a.n_parts);
    if (t.part >= 0 && !a.parts) return fail(ESP_ERR_INVALID, "tile %d: writes a record but parts is null", i);
  }
  if (a.jobs_host)
    for (int i = 0; i < a.n_jobs; ++i) {
      const esp_attn_combine& j = a.jobs_host[i];
      if (j.rows < 0 || j.rows > TR || j.r0 < 0 || int64_t(j.r0) + j.rows > a.n_rows) return fail(ESP_ERR_INVALID, "job %d: rows [%d, +%d)", i, j.r0, j.rows);
      if (j.part0 < 0 || j.nparts < 0 || int64_t(j.part0) + j.nparts > a.n_parts) return fail(ESP_ERR_INVALID, "job %d: records [%d, +%d) of %d", i, j.part0, j.nparts, a.n_parts);
    }
  return ESP_OK;
}

namespace {

int validate(const esp_attn_ctx* c, const esp_attn_args& a) { return esp::validate_pass(c->shape, c->tile_rows, c->opt_validate != 0, a); }

// Tensor map of one layer region of the pool, as the decode kernel reads it:
// [128-byte line][rows][lines per row], box [line, 16 rows, lines of one head].
int pool_tensor_map(esp_attn_ctx* c, const esp_attn_args& a) {
  const esp_attn_shape& s = c->shape;
  if (c->map_kv == a.kv && c->map_base == a.p.kv_base && c->map_blocks == a.n_blocks && c->map_bt == a.p.bt && c->map_ld == a.p.kv_ld)
    return ESP_OK;
  const int esz = elem_bytes(s.kv_dtype);
  const cuuint64_t line_elems = 128 / esz;
  const cuuint64_t gdim[3] = {line_elems, cuuint64_t(a.n_blocks) * 2 * cuuint64_t(a.p.bt), cuuint64_t(a.p.kv_ld) * esz / 128};
  const cuuint64_t gstride[2] = {cuuint64_t(a.p.kv_ld) * esz, 128};
  const cuuint32_t box[3] = {cuuint32_t(line_elems), cuuint32_t(esp::kDecodeKeyBlock), cuuint32_t(s.HD * esz / 128)};
  const cuuint32_t estr[3] = {1, 1, 1};
  void* base = const_cast<uint8_t*>(static_cast<const uint8_t*>(a.kv)) + a.p.kv_base * esz;
  const CUresult r = reinterpret_cast<EncodeTiledFn>(c->encode_tiled)(
      &c->pool_map, esz == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, base, gdim, gstride, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    c->map_kv = nullptr;
    return fail(ESP_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
  }
  c->map_kv = a.kv, c->map_base = a.p.kv_base, c->map_blocks = a.n_blocks, c->map_bt = a.p.bt, c->map_ld = a.p.kv_ld;
  return ESP_OK;
}

// One 3-D map [64 elements][rows][kv_ld / 64] over 16-bit rows of width kv_ld, box = 64 x 16 x 1.
int rows_tensor_map(esp_attn_ctx* c, CUtensorMap* out, const void* base, uint64_t rows, int32_t kv_ld) {
  const cuuint64_t gdim[3] = {64, rows, cuuint64_t(kv_ld) / 64};
  const cuuint64_t gstride[2] = {cuuint64_t(kv_ld) * 2, 128};
  const cuuint32_t box[3] = {64, 16, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = reinterpret_cast<EncodeTiledFn>(c->encode_tiled)(
      out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ESP_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
  return ESP_OK;
}

int umma_tensor_maps(esp_attn_ctx* c, const esp_attn_args& a) {
  const bool have_pool = a.kv != nullptr && a.n_blocks > 0;
  if (c->umap_kb != a.Kb || c->umap_vb != a.Vb || c->umap_rows != a.n_rows || c->umap_ld != a.p.kv_ld) {
    c->umap_kb = c->umap_vb = nullptr;
    if (int rc = rows_tensor_map(c, &c->kb_map, a.Kb, uint64_t(a.n_rows), a.p.kv_ld)) return rc;
    if (int rc = rows_tensor_map(c, &c->vb_map, a.Vb, uint64_t(a.n_rows), a.p.kv_ld)) return rc;
    c->umap_kb = a.Kb, c->umap_vb = a.Vb, c->umap_rows = a.n_rows, c->umap_ld = a.p.kv_ld;
    c->umap_kv = nullptr;
  }
  if (!have_pool) {
    c->upool_map = c->kb_map;  // never dereferenced: no tile has cached keys
    c->umap_kv = nullptr;
    return ESP_OK;
  }
  if (c->umap_kv != a.kv || c->umap_base != a.p.kv_base || c->umap_blocks != a.n_blocks) {
    c->umap_kv = nullptr;
    const uint8_t* base = static_cast<const uint8_t*>(a.kv) + a.p.kv_base * 2;
    if (int rc = rows_tensor_map(c, &c->upool_map, base, uint64_t(a.n_blocks) * 2 * uint64_t(a.p.bt), a.p.kv_ld)) return rc;
    c->umap_kv = a.kv, c->umap_base = a.p.kv_base, c->umap_blocks = a.n_blocks;
  }
  return ESP_OK;
}

constexpr int kReplanSlots = 4;
constexpr int kReplanTiles = 8192, kReplanJobs = 8192;
constexpr size_t kReplanSlotBytes = size_t(kReplanTiles) * sizeof(esp_attn_tile) + size_t(kReplanJobs) * sizeof(esp_attn_combine);

// Does the plan compute plain full attention for every row of every tree - each 8-row group of each
// tree covered once, over the whole cached range [0, P) (in one tile, or in split tiles that tile the
// range in order and are all merged by one job of this pass), batch keys scanned by the tile that
// ends at P? That is what the reference's planners emit (plan_tiles, src/model/impl/forest.h:1378-1433);
// such a pass may be re-planned freely: only O and lse are its results.
// With `windowed` (a sliding-window layer whose positions the caller mirrors in pos_host) the same for what the
// generic planner emits (g4_plan_tiles, src/model/impl/gemma.h:77-116): the cached range of a row group starts at
// the first key its earliest row can still see, and pad0 carries the first batch key worth scanning.
bool full_attention_plan(const esp_attn_args& a, int TR, bool windowed = false) {
  if (!a.tiles_host || !a.trees_host || (a.n_jobs > 0 && !a.jobs_host)) return false;
  if (windowed && (!a.pos_host || a.window <= 0)) return false;
  int ti = 0, ji = 0;
  for (int t = 0; t < a.n_trees; ++t) {
    const esp_attn_tree& tr = a.trees_host[t];
    for (int r = 0; r < tr.M; r += TR) {
      if (ti >= a.n_tiles) return false;
      const esp_attn_tile& first = a.tiles_host[ti];
      int32_t k_first = 0, b_first = 0;
      if (windowed) {
        int32_t lowest = INT32_MAX;
        for (int i = r; i < std::min(tr.M, r + TR); ++i) lowest = std::min(lowest, a.pos_host[4 * size_t(tr.base + i)]);
        const int64_t start = int64_t(lowest) - a.window + 1;
        k_first = int32_t(std::clamp<int64_t>(start, 0, tr.P));
        b_first = int32_t(std::max<int64_t>(0, start - tr.P));
      }
      if (first.tree != t || first.r0 != tr.base + r || first.pad0 != b_first || first.k0 != k_first) return false;
      if (first.part < 0) {
        if (first.k1 != tr.P || !first.last) return false;
        ++ti;
        continue;
      }
      if (ji >= a.n_jobs) return false;
      const esp_attn_combine& job = a.jobs_host[ji++];
      if (job.r0 != tr.base + r || job.rows != std::min(TR, tr.M - r) || job.part0 != first.part || job.nparts < 1) return false;
      int k = k_first;
      for (int s2 = 0; s2 < job.nparts; ++s2, ++ti) {
        if (ti >= a.n_tiles) return false;
        const esp_attn_tile& x = a.tiles_host[ti];
        if (x.tree != t || x.r0 != tr.base + r || x.part != job.part0 + s2 || x.k0 != k || x.k1 <= x.k0 || x.pad0 != b_first) return false;
        if ((x.last != 0) != (x.k1 == tr.P)) return false;
        k = x.k1;
      }
      if (k != tr.P) return false;
    }
  }
  return ti == a.n_tiles && ji == a.n_jobs;
}

int* option_slot(esp_attn_ctx* c, const char* name) {
  if (!std::strcmp(name, "attn_gqa")) return &c->opt_attn_gqa;
  if (!std::strcmp(name, "attn_umma")) return &c->opt_attn_umma;
  if (!std::strcmp(name, "validate")) return &c->opt_validate;
  if (!std::strcmp(name, "umma_kernel")) return &c->opt_umma_kernel;
  if (!std::strcmp(name, "trace_ctas")) return &c->opt_trace_ctas;
  if (!std::strcmp(name, "fuse_combine")) return &c->opt_fuse_combine;
  if (!std::strcmp(name, "fail_pass")) return &c->fail_every;
  if (!std::strcmp(name, "check_finite")) return &c->opt_check_finite;
  if (!std::strcmp(name, "replan")) return &c->opt_replan;
  if (!std::strcmp(name, "fuse_exchange")) return &c->opt_fuse_exchange;
  if (!std::strcmp(name, "pair_merge")) return &c->opt_pair_merge;
  if (!std::strcmp(name, "stable_cache")) return &c->opt_stable_cache;
  if (!std::strcmp(name, "fp8_direct")) return &c->opt_fp8_direct;
  return nullptr;
}

}  // namespace

static int combine_impl(esp_attn_ctx* c, void* stream, const float* parts, const float* X, void* O, float* lse,
                        const esp_attn_params* p, const esp_attn_combine* jobs, int32_t n_jobs, int rows_max, int parts_max,
                        float* out_parts = nullptr, int32_t out_part0 = 0, const esp_attn_combine* jobs_host = nullptr,
                        int tile_rows = 0);

extern "C" {

const char* esp_attn_last_error(void) { return esp::last_error_buffer(); }
int esp_attn_abi_version(void) { return ESP_ATTN_ABI_VERSION; }

int esp_attn_create(esp_attn_ctx** out, int device, const esp_attn_shape* shape) {
  if (!out || !shape) return fail(ESP_ERR_INVALID, "esp_attn_create: null argument");
  *out = nullptr;
  if (int rc = check_shape(*shape)) return rc;
  int n_dev = 0;
  cudaError_t e = cudaGetDeviceCount(&n_dev);
  if (e != cudaSuccess || n_dev <= 0) return fail(ESP_ERR_NO_DEVICE, "esp_attn_create: no CUDA device (%s); this library has no CPU path", cudaGetErrorString(e));
  if (device < 0 || device >= n_dev) return fail(ESP_ERR_INVALID, "esp_attn_create: device %d of %d", device, n_dev);
  cudaDeviceProp prop{};
  if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return cuda_fail(e, "cudaGetDeviceProperties");
  if (prop.major != 10) return fail(ESP_ERR_NO_DEVICE, "esp_attn_create: device %d is sm_%d%d; the kernels are built for sm_100a only", device, prop.major, prop.minor);
  if ((e = cudaSetDevice(device)) != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  auto* c = new esp_attn_ctx;
  c->device = device;
  c->shape = *shape;
  c->G = shape->H / shape->Hkv;
  c->tile_rows = shape->tile_rows > 0 ? shape->tile_rows : 8;
  c->shape.tile_rows = c->tile_rows;
  if (const char* env = std::getenv("ESPETERO_FAIL_PASS")) c->fail_every = std::atoi(env);
  if (const char* env = std::getenv("ESPETERO_CHECK_FINITE")) c->opt_check_finite = (*env && std::strcmp(env, "0") && std::strcmp(env, "off")) ? 1 : 0;
  cudaDriverEntryPointQueryResult qres{};
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &c->encode_tiled, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !c->encode_tiled) {
    delete c;
    return fail(ESP_ERR_CUDA, "esp_attn_create: cuTensorMapEncodeTiled not available from the driver");
  }
  if ((e = esp::decode_gqa_setup()) != cudaSuccess) {
    delete c;
    return cuda_fail(e, "decode kernel setup");
  }
  if ((e = esp::flash_umma_setup()) != cudaSuccess || (e = esp::flash_umma_pair_setup()) != cudaSuccess ||
      (e = esp::flash_umma_duo_setup()) != cudaSuccess) {
    delete c;
    return cuda_fail(e, "tcgen05 kernel setup");
  }
  if ((e = cudaMalloc(reinterpret_cast<void**>(&c->d_status), kStatusBytes)) != cudaSuccess) {
    delete c;
    return cuda_fail(e, "cudaMalloc(status word)");
  }
  if ((e = cudaMemset(c->d_status, 0, kStatusBytes)) != cudaSuccess) {
    cudaFree(c->d_status);
    delete c;
    return cuda_fail(e, "cudaMemset(status word)");
  }
  // slots for re-planned passes (1.5 MB on the device, as much pinned on the host)
  e = cudaMalloc(reinterpret_cast<void**>(&c->replan_dev), kReplanSlots * kReplanSlotBytes);
  if (e == cudaSuccess) e = cudaMallocHost(reinterpret_cast<void**>(&c->replan_host), kReplanSlots * kReplanSlotBytes);
  for (int i = 0; e == cudaSuccess && i < kReplanSlots; ++i) e = cudaEventCreateWithFlags(&c->replan_done[i], cudaEventDisableTiming);
  if (e != cudaSuccess) {
    esp_attn_destroy(c);
    return cuda_fail(e, "esp_attn_create: plan staging slots");
  }
  *out = c;
  return ESP_OK;
}

int esp_attn_destroy(esp_attn_ctx* c) {
  if (!c) return ESP_OK;
  cudaSetDevice(c->device);
  for (int i = 0; i < kReplanSlots; ++i)
    if (c->replan_done[i]) cudaEventDestroy(c->replan_done[i]);
  for (auto& sp : c->prof_pending) cudaEventDestroy(sp.t0), cudaEventDestroy(sp.t1);
  for (cudaEvent_t e : c->prof_free) cudaEventDestroy(e);
  if (c->replan_dev) cudaFree(c->replan_dev);
  if (c->replan_host) cudaFreeHost(c->replan_host);
  if (c->d_status) cudaFree(c->d_status);
  delete c;
  return ESP_OK;
}

int esp_attn_set_option(esp_attn_ctx* c, const char* name, int value) {
  if (!c || !name) return fail(ESP_ERR_INVALID, "esp_attn_set_option: null argument");
  // attn_vec (src/model/impl/model.h:590): the reference's alternative decode schedule, off there by
  // default; it is not rebuilt here - the one decode kernel serves every single-row pass.
  if (!std::strcmp(name, "attn_vec"))
    return value == 0 ? ESP_OK : fail(ESP_ERR_UNSUPPORTED, "esp_attn_set_option: attn_vec is not built; single-row trees always take the attn_gqa kernel");
  int* slot = option_slot(c, name);
  if (!slot) return fail(ESP_ERR_INVALID, "esp_attn_set_option: unknown option '%s'", name);
  *slot = value;
  return ESP_OK;
}

int esp_attn_get_option(const esp_attn_ctx* c, const char* name, int* value) {
  if (!c || !name || !value) return fail(ESP_ERR_INVALID, "esp_attn_get_option: null argument");
  int* slot = option_slot(const_cast<esp_attn_ctx*>(c), name);
  if (!slot) return fail(ESP_ERR_INVALID, "esp_attn_get_option: unknown option '%s'", name);
  *value = *slot;
  return ESP_OK;
}

int esp_attn_set_trace(esp_attn_ctx* c, void* device_buffer, int32_t n_blocks) {
  if (!c || n_blocks < 0) return fail(ESP_ERR_INVALID, "esp_attn_set_trace: bad argument");
  c->trace = n_blocks > 0 ? static_cast<unsigned long long*>(device_buffer) : nullptr;
  c->trace_blocks = c->trace ? n_blocks : 0;
  return ESP_OK;
}

const char* esp_attn_last_kernel(const esp_attn_ctx* c) { return c ? c->last_kernel : ""; }
uint64_t esp_attn_launch_count(const esp_attn_ctx* c) { return c ? c->launches : 0; }

// Reads the device status word (a kernel whose bounded wait ran out leaves a code there)
// and clears it. Synchronises the stream: meant for tests and post-mortems, not the hot path.
int esp_attn_check_status(esp_attn_ctx* c, void* stream) {
  if (!c) return fail(ESP_ERR_INVALID, "esp_attn_check_status: null context");
  int hdr[kFiniteRecAt + 4] = {0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(hdr, c->d_status, sizeof(hdr), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return cuda_fail(e, "reading the status word");
  const int st = hdr[0];
  if (st == 0 && c->finite_armed && uint32_t(hdr[kFiniteRecAt]) != 0) {
    // the record of the last checked pass (site "attn_out" of the reference's detector)
    const uint32_t hits = uint32_t(hdr[kFiniteRecAt]), idx = uint32_t(hdr[kFiniteRecAt + 1]), cols = uint32_t(c->shape.H * c->shape.HD);
    float val;
    std::memcpy(&val, &hdr[kFiniteRecAt + 3], 4);
    cudaMemsetAsync(c->d_status + kFiniteRecAt, 0, 4 * sizeof(int), s);
    return fail(ESP_ERR_CUDA, "attn_out: %u non-finite elements, first at row %u, column %u (value %g)", hits, idx / cols, idx % cols, double(val));
  }
  if (st != 0) {
    cudaMemsetAsync(c->d_status, 0, kStatusBytes, s);  // the arrival counters too: a kernel that gave up may have left some behind
    return fail(ESP_ERR_CUDA, "a kernel gave up a bounded wait (status %d: %s)", st,
                st == esp::kStatusTmaTimeout ? "TMA load never completed" : st == esp::kStatusMmaTimeout ? "MMA never completed"
               : st == esp::kStatusPeerTimeout ? "a peer GPU never published its records" : "bad block id");
  }
  return ESP_OK;
}

// A reference-shaped multi-row pass (tiles of 8 rows, forest.h:1378-1433) would have to run on the
// CUDA-core kernel: the tcgen05 kernels want 128 (row, head) pairs per CTA. When the plan is plain full
// attention (full_attention_plan) only O and lse are results of the pass, so the pass is planned again
// here for the tensor-core kernels - 128-row tiles for passes over their own rows (prefill), tiles of
// 128 / G rows with the G heads of a kv head for passes over a cached prefix (verify) - and the new
// tiles and jobs replace the caller's for this call. Records go to the caller's `parts` in the new
// tiles' layout (the split is chosen so that they fit). Returns false when the pass stays as it is.
static bool stage_plan(esp_attn_ctx* c, esp_attn_args& a, int& TR, int new_TR, int32_t nt, int32_t nj, cudaStream_t stream, int* rc);

// A sliding-window pass planned the reference's way (8-row tiles, g4_plan_tiles) planned again with 128-row tiles for
// the tcgen05 kernel: the generic planner with a group count that leaves it no budget to split (its tiles then take
// the caller's height), on the caller's host mirror of the positions.
static bool replan_window_pass(esp_attn_ctx* c, esp_attn_args& a, int& TR, cudaStream_t stream, int* rc) {
  *rc = ESP_OK;
  const int new_TR = 128;
  int32_t nt = 0, nj = 0, np = 0, rows = 0;
  c->rp_tiles.resize(kReplanTiles), c->rp_jobs.resize(kReplanJobs);
  const int prc = esp_attn_plan_window(a.trees_host, a.n_trees, 256, 0, new_TR, a.window, a.pos_host, c->rp_tiles.data(), kReplanTiles,
                                       c->rp_jobs.data(), kReplanJobs, &nt, &nj, &np, &rows);
  if (prc != ESP_OK || rows != new_TR || nj != 0 || np != 0) return false;
  return stage_plan(c, a, TR, new_TR, nt, nj, stream, rc);
}

static bool replan_pass(esp_attn_ctx* c, esp_attn_args& a, int& TR, cudaStream_t stream, int* rc) {
  *rc = ESP_OK;
  const esp_attn_shape& s = c->shape;
  int64_t cached = 0, batch = 0;
  for (int i = 0; i < a.n_trees; ++i) cached += int64_t(a.trees_host[i].P) * a.trees_host[i].M, batch += int64_t(a.trees_host[i].M) * a.trees_host[i].M / 2;
  const bool stream_hbm = s.HD == 128 && cached > 2 * batch;
  int hpc = 1;
  if (stream_hbm)
    for (int h = 8; h >= 1; h >>= 1)
      if (h <= c->G && c->G % h == 0) {
        hpc = h;
        break;
      }
  const int new_TR = 128 / hpc;
  if (!esp::flash_umma_supports(s.HD, c->G, new_TR, s.bt, s.q_dtype, s.kv_dtype)) return false;
  esp_plan_opts o{};
  o.mode = ESP_PLAN_B200, o.min_chunk = 32, o.tile_rows = new_TR, o.max_parts = 64;
  o.groups = stream_hbm ? 148 : 148 * 2 * 8;
  o.split = (a.parts && a.n_parts > 0) ? (1 << 20) : 0;
  int32_t nt = 0, nj = 0, np = 0;
  c->rp_tiles.resize(kReplanTiles), c->rp_jobs.resize(kReplanJobs);
  for (int attempt = 0; attempt < 2; ++attempt) {
    const int prc = esp_attn_plan(a.trees_host, a.n_trees, s.Hkv, &o, c->rp_tiles.data(), kReplanTiles, c->rp_jobs.data(), kReplanJobs, &nt, &nj, &np);
    if (prc != ESP_OK) return false;  // more tiles than the slots hold: the pass stays on the general kernel
    // the records must fit the caller's buffer: n_parts records of 8 rows there, np records of new_TR rows here
    if (int64_t(np) * new_TR <= int64_t(a.n_parts) * TR) break;
    if (attempt == 1) return false;
    o.split = 0;
  }
  return stage_plan(c, a, TR, new_TR, nt, nj, stream, rc);
}

// The new tiles and jobs (in rp_tiles / rp_jobs) through a staging slot into device memory; `a` and TR become the
// pass as it runs.
static bool stage_plan(esp_attn_ctx* c, esp_attn_args& a, int& TR, int new_TR, int32_t nt, int32_t nj, cudaStream_t stream, int* rc) {
  // a free staging slot (its previous pass has run)
  const int slot = c->replan_next;
  c->replan_next = (slot + 1) % kReplanSlots;
  if (c->replan_used[slot]) {
    const cudaError_t e = cudaEventSynchronize(c->replan_done[slot]);
    if (e != cudaSuccess) {
      *rc = cuda_fail(e, "waiting for a plan staging slot");
      return false;
    }
  }
  uint8_t* h = c->replan_host + size_t(slot) * kReplanSlotBytes;
  uint8_t* d = c->replan_dev + size_t(slot) * kReplanSlotBytes;
  const size_t tiles_bytes = size_t(nt) * sizeof(esp_attn_tile), jobs_at = size_t(kReplanTiles) * sizeof(esp_attn_tile);
  std::memcpy(h, c->rp_tiles.data(), tiles_bytes);
  std::memcpy(h + jobs_at, c->rp_jobs.data(), size_t(nj) * sizeof(esp_attn_combine));
  cudaError_t e = cudaMemcpyAsync(d, h, tiles_bytes, cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess && nj > 0) e = cudaMemcpyAsync(d + jobs_at, h + jobs_at, size_t(nj) * sizeof(esp_attn_combine), cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) {
    *rc = cuda_fail(e, "uploading the re-planned tiles");
    return false;
  }
  c->replan_used[slot] = true;
  a.tiles = reinterpret_cast<const esp_attn_tile*>(d), a.tiles_host = c->rp_tiles.data(), a.n_tiles = nt;
  a.jobs = nj > 0 ? reinterpret_cast<const esp_attn_combine*>(d + jobs_at) : nullptr, a.jobs_host = nj > 0 ? c->rp_jobs.data() : nullptr, a.n_jobs = nj;
  a.n_parts = int32_t(int64_t(a.n_parts) * TR / new_TR);
  TR = new_TR;
  *rc = slot + 1;  // the caller records the slot's event once the pass is enqueued
  return true;
}

}  // extern "C"

// xch != NULL: the pass is one rank's share of a sequence split over several GPUs and ends with the peer
// exchange inside the decode kernel. *fused_out tells whether that happened; if not, nothing was launched
// for the exchange and the caller takes the two-kernel route.
static int forward_impl(esp_attn_ctx* c, void* stream_v, const esp_attn_args* ap, const esp_attn_exchange* xch, bool* fused_out) {
  if (!c || !ap) return fail(ESP_ERR_INVALID, "esp_attn_forward: null argument");
  esp_attn_args a = *ap;  // the pass as it runs: re-planning may replace tiles and jobs
  const esp_attn_shape& s = c->shape;
  if (int rc = check_params(c, a.p)) return rc;
  if (int rc = validate(c, a)) return rc;
  ++c->pass_count;
  if (c->fail_every > 0 && a.n_rows >= 64 && c->pass_count % uint64_t(c->fail_every) == 0)
    return fail(ESP_ERR_INJECTED, "attention pass failed: injected (ESPETERO_FAIL_PASS)");
  if (a.n_tiles == 0) return ESP_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  int TR = c->tile_rows;

  // the generic kernel's layer options (80_gemma.metal) and the sparse-attention lists (45_qsa.metal) live on the general kernel
  const bool windowed = a.window > 0 || a.ring > 0 || a.bidi != 0 || a.qsa_tlist != nullptr;

  // Kernel choice, as forest.h:2864-2868: single-row trees with G <= 8 take the decode kernel.
  bool single = c->G <= 8 && a.trees_host != nullptr && a.tiles_host != nullptr;
  for (int i = 0; single && i < a.n_trees; ++i) single = a.trees_host[i].M == 1;
  bool decode = single && !windowed_lists(a) && c->opt_attn_gqa && esp::decode_gqa_supports(s.HD, c->G, s.bt, s.q_dtype, s.kv_dtype) && a.kv != nullptr && a.n_blocks > 0 &&
                (size_t(a.p.kv_ld) * elem_bytes(s.kv_dtype)) % 128 == 0 && (a.p.kv_base * elem_bytes(s.kv_dtype)) % 128 == 0;
  // (a tile may start at any key: sliding-window plans begin at the row's first visible key)

  // Multi-row tiles: the tcgen05 kernel when the shape fits it (128 (row, head) pairs per CTA).
  // Over an E4M3 pool they need the caller's scratch: the blocks of the pass are widened to the
  // 16-bit type first (one more pass over the keys, still far faster than the CUDA-core kernel).
  const bool fp8_pool = s.kv_dtype == ESP_E4M3;
  const size_t widened_pool_bytes = size_t(std::max(a.n_block_entries, 0)) * 2 * size_t(a.p.bt) * size_t(a.p.kv_ld) * 2;
  const bool widen = fp8_pool && a.dequant_scratch != nullptr && a.n_block_entries > 0 && a.kv != nullptr && a.blocks != nullptr &&
                     a.dequant_scratch_bytes >= widened_pool_bytes + ((size_t(a.n_block_entries) * 4 + 127) / 128) * 128 &&
                     (reinterpret_cast<uintptr_t>(a.dequant_scratch) & 127) == 0 && a.p.kv_ld % 8 == 0 && a.p.kv_base % 8 == 0;
  // Where the tiles' keys come from: cached keys are streamed from HBM, the pass's own rows sit in L2.
  int64_t keys_cached = 0, keys_batch = 0;
  if (a.tiles_host && a.trees_host)
    for (int i = 0; i < a.n_tiles; ++i) {
      const esp_attn_tile& t = a.tiles_host[i];
      keys_cached += t.k1 - t.k0;
      if (t.last) keys_batch += a.trees_host[t.tree].M;
    }
  // E4M3 pools under passes over mostly cached keys (verify, chunked prefill over a long prefix): flash_umma reads the
  // codes itself. Other passes over such pools widen the blocks they touch into the caller's scratch first.
  // (128-dim heads: flash_umma; 256-dim heads: flash_umma_pair, whatever "umma_kernel" says - they have no other kernel.
  // Passes over mostly their own rows take this route only when the caller gave no scratch to widen into: the converter
  // warps fetch batch keys with plain loads, slower than the 16-bit kernels' TMA but far ahead of the CUDA-core kernel.)
  const bool fp8_direct = fp8_pool && c->opt_fp8_direct && (s.HD == 128 || s.HD == 256) && a.kv != nullptr && a.kv_scales != nullptr &&
                          a.n_blocks > 0 && a.trees_host != nullptr && a.p.kv_ld % 128 == 0 && a.p.kv_base % 16 == 0 &&
                          (s.HD == 256 || c->opt_umma_kernel <= 1) && keys_cached > 0 && (keys_cached > 2 * keys_batch || !widen);
  // A pass that reads no cached key (a prefill from position 0) never touches the pool: its E4M3 type is beside the point.
  const bool pool_unused = fp8_pool && a.tiles_host != nullptr && a.trees_host != nullptr && keys_cached == 0;
  // Reference-shaped sliding-window plans (8-row tiles) are planned again for the tensor cores when the caller mirrors
  // the positions on the host.
  int replan_slot = -1;
  if (windowed && TR == 8 && c->opt_replan && !single && !decode && a.window > 0 && a.pos_host && a.qsa_tlist == nullptr && (!fp8_pool || pool_unused) &&
      c->opt_attn_umma && a.p.kv_ld % 64 == 0 && a.p.kv_base % 64 == 0 &&
      ((c->opt_umma_kernel != 1 && c->opt_umma_kernel != 2 && esp::flash_umma_duo_supports(s.HD, c->G, 128, s.bt, s.q_dtype, pool_unused ? s.q_dtype : s.kv_dtype)) ||
       (s.HD == 256 && esp::flash_umma_supports(s.HD, c->G, 128, s.bt, s.q_dtype, pool_unused ? s.q_dtype : s.kv_dtype))) &&
      full_attention_plan(a, TR, true)) {
    int rrc = ESP_OK;
    if (replan_window_pass(c, a, TR, stream, &rrc)) replan_slot = rrc - 1;
    else if (rrc != ESP_OK) return rrc;
  }
  // Sliding-window layers (window masks, ring addressing, image rows; not sparse lists) with 128-dim heads over a
  // 16-bit pool have their own instantiation of the two-tile tcgen05 kernel, for plans with tcgen05-sized tiles
  // (esp_attn_plan_window with rows = 128 gives them to passes of 256 row groups or more).
  // 256-dim heads (the sliding layers of kernels/80_gemma.metal) have theirs in flash_umma_pair.
  const bool win_tc = windowed && a.qsa_tlist == nullptr && (!fp8_pool || pool_unused) &&
                      ((c->opt_umma_kernel != 1 && c->opt_umma_kernel != 2 && esp::flash_umma_duo_supports(s.HD, c->G, TR, s.bt, s.q_dtype, pool_unused ? s.q_dtype : s.kv_dtype)) ||
                       (s.HD == 256 && esp::flash_umma_supports(s.HD, c->G, TR, s.bt, s.q_dtype, pool_unused ? s.q_dtype : s.kv_dtype)));
  const bool umma_ok = !decode && (!windowed || win_tc) && c->opt_attn_umma && a.tiles_host != nullptr &&
                       (!fp8_pool || widen || fp8_direct || pool_unused) && a.p.kv_ld % 64 == 0 && (fp8_pool || a.p.kv_base % 64 == 0);
  // Reference-shaped plans (8-row tiles) of plain full-attention passes are planned again for the tensor cores.
  if (umma_ok && TR == 8 && c->opt_replan && !single && full_attention_plan(a, TR)) {
    int rrc = ESP_OK;
    if (replan_pass(c, a, TR, stream, &rrc)) replan_slot = rrc - 1;
    else if (rrc != ESP_OK) return rrc;
  }
  bool umma = umma_ok && esp::flash_umma_supports(s.HD, c->G, TR, s.bt, s.q_dtype, fp8_pool ? s.q_dtype : s.kv_dtype);
  // (sliding-window tiles start at any key: their kernel loads from the page boundary below and masks)
  for (int i = 0; umma && !win_tc && i < a.n_tiles; ++i) umma = a.tiles_host[i].k0 % esp::kDecodeKeyBlock == 0;

  esp::KernelArgs k{};
  k.Q = a.Q, k.Kb = a.Kb, k.Vb = a.Vb, k.kv = a.kv, k.kv_scales = a.kv_scales, k.blocks = a.blocks;
  k.desc = (s.flags & ESP_ATTN_FLAG_ANC_MASK) ? nullptr : a.desc;
  k.anc_mask = (s.flags & ESP_ATTN_FLAG_ANC_MASK) ? a.anc_mask : nullptr;
  k.X = (s.flags & ESP_ATTN_FLAG_GATE) ? a.X : nullptr;
  k.O = a.O, k.lse = a.lse, k.parts = a.parts, k.tiles = a.tiles, k.trees = a.trees, k.status = c->d_status, k.counters = c->d_status + 64;
  k.trace = c->trace, k.trace_blocks = c->trace_blocks, k.trace_ctas = c->trace ? c->opt_trace_ctas : 0;
  k.p = a.p, k.HD = s.HD, k.G = c->G, k.tile_rows = TR, k.n_tiles = a.n_tiles;
  k.q_dtype = s.q_dtype, k.kv_dtype = s.kv_dtype, k.n_blocks = a.n_blocks, k.scale = s.scale;
  k.n_trees = a.n_trees, k.n_block_entries = a.n_block_entries;
  k.pos = a.pos, k.window = a.window, k.ring = a.ring, k.bidi = a.bidi;
  k.pair_merge = c->opt_pair_merge;
  k.stable_cache = c->opt_stable_cache;
  k.qsa_tlist = a.qsa_tlist, k.qsa_tcount = a.qsa_tcount, k.qsa_rinfo = a.qsa_rinfo, k.qsa_sel = a.qsa_sel;
  k.qsa_nbw = a.qsa_nbw, k.qsa_n_lists = a.qsa_n_lists;

  esp_attn_args widened = a;  // the pass as the tcgen05 kernels see it when the pool was widened
  if (umma && fp8_direct) {
    widened.kv = nullptr;  // no 16-bit map of the pool: the kernel takes the byte map the decode kernel uses
  } else if (umma && pool_unused) {
    widened.kv = nullptr, widened.kv_scales = nullptr;  // no map of the pool at all: no tile has cached keys
    k.kv = nullptr, k.kv_scales = nullptr, k.kv_dtype = s.q_dtype;
  } else if (umma && fp8_pool) {
    int32_t* identity = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(a.dequant_scratch) + widened_pool_bytes);
    ProfScope prof(c, stream, "kv_dequant");
    const cudaError_t de = esp::launch_kv_dequant(a.kv, a.kv_scales, a.blocks, a.n_block_entries, a.dequant_scratch, identity, a.p, s.HD,
                                                  a.n_blocks, s.q_dtype, stream, &c->launches);
    if (de != cudaSuccess) return cuda_fail(de, "kv_dequant");
    widened.kv = a.dequant_scratch, widened.blocks = identity, widened.kv_scales = nullptr;
    widened.n_blocks = a.n_block_entries, widened.p.kv_base = 0;
    k.kv = widened.kv, k.blocks = widened.blocks, k.kv_scales = nullptr, k.kv_dtype = s.q_dtype;
    k.n_blocks = widened.n_blocks, k.p.kv_base = 0;
  }

  cudaError_t e;
  bool merged = false;  // the attention kernel merged the split-K records itself: no combine launch
  {
  ProfScope prof(c, stream, decode ? "decode_gqa" : (umma ? "flash_umma*" : "flash_general"));
  if (decode) {
    if (int rc = pool_tensor_map(c, a)) return rc;
    c->last_kernel = "decode_gqa";
    // Plans whose split tiles name their jobs (ESP_PLAN_B200) can be merged inside the kernel; whether
    // that pays depends on the pass (decode_fuse_small: small passes and passes with many jobs).
    k.jobs = a.jobs;
    // (option 2 merges in the kernel whatever the size; the records of a kv head's G heads must be a
    // multiple of 16 bytes for the bulk copies: G even)
    k.fuse = c->opt_fuse_combine && (c->opt_fuse_combine == 2 || esp::decode_fuse_small(a.n_tiles, s.Hkv, a.n_jobs, s.HD == 64 || (fp8_pool && s.HD == 128))) && c->G % 2 == 0 &&
             a.n_jobs > 0 && a.jobs && esp::plan_fusable(a.tiles_host, a.n_tiles, a.jobs_host, a.n_jobs, s.Hkv);
    merged = k.fuse != 0;
    if (xch) {
      // the exchange rides on the fused merge of ONE job (one row group: a single long sequence)
      if (!(c->G % 2 == 0 && a.n_jobs == 1 && a.jobs && esp::plan_fusable(a.tiles_host, a.n_tiles, a.jobs_host, a.n_jobs, s.Hkv))) {
        *fused_out = false;
        return ESP_OK;
      }
      k.fuse = 1, merged = true;
      k.x_world = xch->world, k.x_rank = xch->rank, k.x_phases = xch->phases, k.x_tag = uint32_t(xch->epoch);
      k.x_wait_ms = xch->wait_ms ? uint32_t(xch->wait_ms) : 2000u;
      const size_t rank_words = size_t(s.Hkv) * TR * c->G * (s.HD + 2);
      k.x_epoch_off = (xch->epoch & 1) * uint64_t(xch->world) * rank_words;
      for (int q = 0; q < xch->world; ++q) k.x_records[q] = static_cast<uint2*>(xch->records[q]);
    }
    e = esp::launch_decode_gqa(k, c->pool_map, stream, &c->launches);
    if (xch) {
      if (e == cudaErrorCooperativeLaunchTooLarge) {  // the grid would not be resident at once: two-kernel route
        (void)cudaGetLastError();
        *fused_out = false;
        return ESP_OK;
      }
      *fused_out = e == cudaSuccess;
    }
  } else if (umma) {
    if (int rc = umma_tensor_maps(c, widened)) return rc;
    // Which of the two tcgen05 kernels: by where the tiles' keys come from (cached keys are streamed
    // from HBM, the pass's own rows sit in L2), unless the "umma_kernel" option forces one.
    // 256-dim heads run on flash_umma_pair only (one CTA per SM there: its tiles take the whole SM).
    const bool stream_hbm = !win_tc && s.HD == 128 && ((fp8_direct && umma) || c->opt_umma_kernel == 1 || (c->opt_umma_kernel == 0 && keys_cached > 2 * keys_batch));
    if (fp8_direct)
      if (int rc = pool_tensor_map(c, a)) return rc;
    // Passes whose keys are mostly their own rows (prefill) are compute-bound: two query tiles per CTA where the
    // heads allow it (128-dim heads, 2 * (128 / tile_rows) heads within one kv head), else two CTAs per SM.
    const bool duo = !stream_hbm && (c->opt_umma_kernel == 3 || c->opt_umma_kernel == 0) &&
                     esp::flash_umma_duo_supports(s.HD, c->G, TR, s.bt, s.q_dtype, fp8_pool ? s.q_dtype : s.kv_dtype);
    if (duo) {
      c->last_kernel = "flash_umma_duo";
      e = esp::launch_flash_umma_duo(k, c->upool_map, c->kb_map, c->vb_map, stream, &c->launches);
    } else if (stream_hbm) {
      c->last_kernel = "flash_umma";
      e = esp::launch_flash_umma(k, fp8_direct ? c->pool_map : c->upool_map, c->kb_map, c->vb_map, a.tiles_host, a.trees_host, a.n_trees,
                                 c->opt_fuse_combine ? a.jobs_host : nullptr, a.n_jobs, &merged, stream, &c->launches);
    } else {
      c->last_kernel = "flash_umma_pair";
      // 256-dim verify passes (tiles of 128 / G rows x G heads, one wave of CTAs): split tiles that name their jobs
      // merge their records inside the kernel - no second launch, and no pass of the combine kernel over 1 KB records.
      k.jobs = a.jobs;
      k.fuse = s.HD == 256 && c->opt_fuse_combine && 128 / TR == c->G && a.n_jobs > 0 && a.jobs &&
               (c->opt_fuse_combine == 2 || int64_t(a.n_tiles) * s.Hkv <= 148) &&
               esp::plan_fusable(a.tiles_host, a.n_tiles, a.jobs_host, a.n_jobs, s.Hkv);
      merged = k.fuse != 0;
      e = esp::launch_flash_umma_pair(k, fp8_direct ? c->pool_map : c->upool_map, c->kb_map, c->vb_map, fp8_direct, stream, &c->launches);
    }
  } else {
    c->last_kernel = "flash_general";
    e = esp::launch_flash_general(k, stream, &c->launches);
  }
  prof.kernel = c->last_kernel;
  }
  if (e != cudaSuccess) return cuda_fail(e, c->last_kernel);
  if (a.n_jobs > 0 && !merged) {
    int rows_max = TR, parts_max = 64;
    if (a.jobs_host) {
      rows_max = 1, parts_max = 1;
      for (int i = 0; i < a.n_jobs; ++i) {
        rows_max = a.jobs_host[i].rows > rows_max ? a.jobs_host[i].rows : rows_max;
        parts_max = a.jobs_host[i].nparts > parts_max ? a.jobs_host[i].nparts : parts_max;
      }
    }
    ProfScope prof(c, stream, "attention_combine");
    if (int rc = combine_impl(c, stream_v, a.parts, a.X, a.O, a.lse, &a.p, a.jobs, a.n_jobs, rows_max, parts_max, nullptr, 0, a.jobs_host, TR)) return rc;
  }
  if (replan_slot >= 0) cudaEventRecord(c->replan_done[replan_slot], stream);  // the slot's tiles and jobs have been read
  if (c->opt_check_finite && a.n_rows > 0) {
    const cudaError_t fe = esp::launch_finite_check(a.O, uint32_t(a.n_rows), uint32_t(s.H * s.HD), uint64_t(a.p.q_ld),
                                                    s.q_dtype == ESP_F16 ? ESP_FINITE_F16 : ESP_FINITE_BF16, 0x7F800000u,
                                                    reinterpret_cast<uint32_t*>(c->d_status + kFiniteRecAt), stream, &c->launches);
    if (fe != cudaSuccess) return cuda_fail(fe, "finite_check");
    c->finite_armed = true;
  }
  return ESP_OK;
}

extern "C" {

int esp_attn_forward(esp_attn_ctx* c, void* stream, const esp_attn_args* args) { return forward_impl(c, stream, args, nullptr, nullptr); }

int esp_attn_forward_exchange(esp_attn_ctx* c, void* stream, const esp_attn_args* ap, const esp_attn_exchange* xp) {
  if (!c || !ap || !xp) return fail(ESP_ERR_INVALID, "esp_attn_forward_exchange: null argument");
  const esp_attn_exchange& x = *xp;
  if (x.world < 1 || x.world > ESP_ATTN_MAX_PEERS || x.rank < 0 || x.rank >= x.world)
    return fail(ESP_ERR_INVALID, "esp_attn_forward_exchange: rank %d of world %d", x.rank, x.world);
  if (x.phases < 1 || x.phases > 3 || x.wait_ms < 0 || uint32_t(x.epoch) == 0)
    return fail(ESP_ERR_INVALID, "esp_attn_forward_exchange: phases %d, wait_ms %d, epoch %llu", x.phases, x.wait_ms, (unsigned long long)x.epoch);
  for (int q = 0; q < x.world; ++q)
    if (!x.records[q] || (reinterpret_cast<uintptr_t>(x.records[q]) & 7))
      return fail(ESP_ERR_INVALID, "esp_attn_forward_exchange: exchange buffer of rank %d is null or not 8-byte aligned", q);
  if (ap->n_jobs < 1 || !ap->jobs || !ap->jobs_host) return fail(ESP_ERR_INVALID, "esp_attn_forward_exchange: the rank's reduce jobs (device and host copies) are required");
  int parts_max = 1;
  for (int i = 0; i < ap->n_jobs; ++i) parts_max = std::max(parts_max, ap->jobs_host[i].nparts);
  if (x.phases == 2)  // only the second half: the records were published by an earlier launch
    return esp_attn_exchange_parts(c, stream, ap->parts, ap->X, ap->O, ap->lse, &ap->p, ap->jobs, ap->n_jobs, 1, parts_max, xp);
  bool fused = false;
  if (c->opt_fuse_exchange) {
    if (int rc = forward_impl(c, stream, ap, xp, &fused)) return rc;
    if (fused) return ESP_OK;
  }
  // two kernels: the records, then merge + exchange + merge
  esp_attn_args rec = *ap;
  rec.n_jobs = 0, rec.jobs = nullptr, rec.jobs_host = nullptr;
  if (int rc = forward_impl(c, stream, &rec, nullptr, nullptr)) return rc;
  return esp_attn_exchange_parts(c, stream, ap->parts, ap->X, ap->O, ap->lse, &ap->p, ap->jobs, ap->n_jobs, 1, parts_max, xp);
}

int esp_attn_set_profile(esp_attn_ctx* c, int on) {
  if (!c) return fail(ESP_ERR_INVALID, "esp_attn_set_profile: null context");
  for (auto& sp : c->prof_pending) c->prof_free.push_back(sp.t0), c->prof_free.push_back(sp.t1);
  c->prof_pending.clear();
  c->prof_sums.clear();
  c->profiling = on != 0;
  return ESP_OK;
}

int esp_attn_get_profile(esp_attn_ctx* c, esp_attn_profile_entry* out, int32_t cap, int32_t* n) {
  if (!c || !n) return fail(ESP_ERR_INVALID, "esp_attn_get_profile: null argument");
  for (auto& sp : c->prof_pending) {
    cudaError_t e = cudaEventSynchronize(sp.t1);
    float ms = 0.0f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, sp.t0, sp.t1);
    c->prof_free.push_back(sp.t0), c->prof_free.push_back(sp.t1);
    if (e != cudaSuccess) {
      c->prof_pending.clear();
      return cuda_fail(e, "esp_attn_get_profile");
    }
    bool found = false;
    for (auto& s : c->prof_sums)
      if (!std::strcmp(s.kernel, sp.kernel)) {
        ++s.launches, s.ms += ms, found = true;
        break;
      }
    if (!found) c->prof_sums.push_back({sp.kernel, 1u, double(ms)});
  }
  c->prof_pending.clear();
  *n = int32_t(c->prof_sums.size());
  for (int32_t i = 0; out && i < cap && i < *n; ++i) {
    std::snprintf(out[i].kernel, sizeof(out[i].kernel), "%s", c->prof_sums[size_t(i)].kernel);
    out[i].launches = c->prof_sums[size_t(i)].launches;
    out[i].gpu_ms = float(c->prof_sums[size_t(i)].ms);
  }
  if (out && *n > cap) return fail(ESP_ERR_CAPACITY, "esp_attn_get_profile: %d kernels, room for %d", *n, cap);
  return ESP_OK;
}

int esp_qsa_select(void* stream, const float* scores, const int32_t* srows, const int32_t* rinfo, uint32_t* sel, int32_t n_sparse, int32_t nbmax,
                   int32_t nbw) {
  if (n_sparse <= 0) return ESP_OK;
  if (!scores || !srows || !rinfo || !sel || nbmax <= 0 || nbw < (nbmax + 31) / 32) return fail(ESP_ERR_INVALID, "esp_qsa_select: null pointer, or nbw < ceil(nbmax / 32)");
  const cudaError_t e = esp::launch_qsa_select(scores, srows, rinfo, sel, n_sparse, nbmax, nbw, static_cast<cudaStream_t>(stream), nullptr);
  if (e != cudaSuccess) return cuda_fail(e, "qsa_select");
  return ESP_OK;
}

int esp_qsa_tiles(void* stream, const uint32_t* sel, const esp_attn_tree* trees, const int32_t* rinfo, const esp_qsa_tile* qtiles, int32_t n_qtiles,
                  uint32_t* tlist, uint32_t* tcount, int32_t nbmax, int32_t nbw) {
  if (n_qtiles <= 0) return ESP_OK;
  if (!sel || !trees || !rinfo || !qtiles || !tlist || !tcount || nbmax <= 0 || nbw <= 0) return fail(ESP_ERR_INVALID, "esp_qsa_tiles: null pointer or bad size");
  const cudaError_t e = esp::launch_qsa_tiles(sel, trees, rinfo, qtiles, n_qtiles, tlist, tcount, nbmax, nbw, static_cast<cudaStream_t>(stream), nullptr);
  if (e != cudaSuccess) return cuda_fail(e, "qsa_tiles");
  return ESP_OK;
}

int esp_attn_finite_check(void* stream, const void* x, uint32_t rows, uint32_t cols, uint64_t ld, int32_t dtype, float threshold,
                          esp_finite_rec* rec) {
  if (!x || !rec || ld < cols) return fail(ESP_ERR_INVALID, "esp_attn_finite_check: null pointer or ld < cols");
  if (dtype != ESP_FINITE_F32 && dtype != ESP_FINITE_F16 && dtype != ESP_FINITE_BF16) return fail(ESP_ERR_INVALID, "esp_attn_finite_check: dtype %d", dtype);
  if (uint64_t(rows) * cols >= 0xFFFFFFFFull) return fail(ESP_ERR_UNSUPPORTED, "esp_attn_finite_check: more than 2^32 - 1 elements");
  if (rows == 0 || cols == 0) return ESP_OK;
  uint32_t thr_bits;
  std::memcpy(&thr_bits, &threshold, 4);
  thr_bits &= 0x7FFFFFFFu;
  if (thr_bits > 0x7F800000u) thr_bits = 0x7F800000u;  // a NaN threshold: only NaN and Inf offend
  const cudaError_t e = esp::launch_finite_check(x, rows, cols, ld, dtype, thr_bits, reinterpret_cast<uint32_t*>(rec), static_cast<cudaStream_t>(stream), nullptr);
  if (e != cudaSuccess) return cuda_fail(e, "finite_check");
  return ESP_OK;
}

int esp_attn_combine_parts(esp_attn_ctx* c, void* stream, const float* parts, const float* X, void* O, float* lse,
                           const esp_attn_params* p, const esp_attn_combine* jobs, int32_t n_jobs) {
  if (!c) return fail(ESP_ERR_INVALID, "esp_attn_combine_parts: null argument");
  return combine_impl(c, stream, parts, X, O, lse, p, jobs, n_jobs, c->tile_rows, 64);
}

int esp_attn_reduce_parts(esp_attn_ctx* c, void* stream, const float* parts, const esp_attn_params* p, const esp_attn_combine* jobs,
                          int32_t n_jobs, float* parts_out, int32_t out_part0) {
  if (!c || !parts_out || out_part0 < 0) return fail(ESP_ERR_INVALID, "esp_attn_reduce_parts: null or negative argument");
  return combine_impl(c, stream, parts, nullptr, nullptr, nullptr, p, jobs, n_jobs, c->tile_rows, 64, parts_out, out_part0);
}

size_t esp_attn_dequant_scratch_bytes(const esp_attn_shape* s, int32_t n_block_entries) {
  if (!s || n_block_entries <= 0 || s->bt <= 0 || s->Hkv <= 0) return 0;
  // the widened blocks (16-bit, K rows + V rows each) and an identity block table behind them, 128-byte granules
  const size_t pool = size_t(n_block_entries) * 2 * size_t(s->bt) * size_t(s->Hkv) * size_t(s->HD) * 2;
  return pool + ((size_t(n_block_entries) * 4 + 127) / 128) * 128;
}

size_t esp_attn_exchange_bytes(const esp_attn_shape* s, int32_t n_jobs, int32_t world) {
  if (!s || n_jobs <= 0 || world <= 0 || s->Hkv <= 0 || s->H <= 0) return 0;
  const int TR = s->tile_rows > 0 ? s->tile_rows : 8;
  // two epochs x world ranks x records, 8 bytes per record element
  return size_t(2) * size_t(world) * size_t(n_jobs) * size_t(s->Hkv) * size_t(TR) * size_t(s->H / s->Hkv) * size_t(s->HD + 2) * 8;
}

int esp_attn_exchange_parts(esp_attn_ctx* c, void* stream, const float* parts, const float* X, void* O, float* lse,
                            const esp_attn_params* p, const esp_attn_combine* jobs, int32_t n_jobs, int32_t rows_max,
                            int32_t parts_max, const esp_attn_exchange* xp) {
  if (!c || !p || !xp) return fail(ESP_ERR_INVALID, "esp_attn_exchange_parts: null argument");
  if (n_jobs <= 0) return ESP_OK;
  const esp_attn_exchange& x = *xp;
  if (x.world < 1 || x.world > ESP_ATTN_MAX_PEERS || x.rank < 0 || x.rank >= x.world)
    return fail(ESP_ERR_INVALID, "esp_attn_exchange_parts: rank %d of world %d", x.rank, x.world);
  if (x.phases < 1 || x.phases > 3 || x.wait_ms < 0 || uint32_t(x.epoch) == 0)
    return fail(ESP_ERR_INVALID, "esp_attn_exchange_parts: phases %d, wait_ms %d, epoch %llu", x.phases, x.wait_ms,
                (unsigned long long)x.epoch);
  for (int q = 0; q < x.world; ++q)
    if (!x.records[q] || (reinterpret_cast<uintptr_t>(x.records[q]) & 7))
      return fail(ESP_ERR_INVALID, "esp_attn_exchange_parts: exchange buffer of rank %d is null or not 8-byte aligned", q);
  if (!parts || !jobs || ((x.phases & 2) && !O)) return fail(ESP_ERR_INVALID, "esp_attn_exchange_parts: null parts / O / jobs");
  if (int rc = check_params(c, *p)) return rc;
  const esp_attn_shape& s = c->shape;
  if ((s.flags & ESP_ATTN_FLAG_GATE) && !X) return fail(ESP_ERR_INVALID, "esp_attn_exchange_parts: gate flag set but X is null");
  esp::ExchangeArgs k{};
  k.c.parts = parts, k.c.X = (s.flags & ESP_ATTN_FLAG_GATE) ? X : nullptr, k.c.O = O, k.c.lse = lse, k.c.jobs = jobs, k.c.p = *p;
  k.c.HD = s.HD, k.c.G = c->G, k.c.tile_rows = c->tile_rows, k.c.n_jobs = n_jobs, k.c.q_dtype = s.q_dtype;
  k.c.rows_max = rows_max < 1 ? 1 : (rows_max > c->tile_rows ? c->tile_rows : rows_max);
  k.c.n_slices = esp::combine_slices(s.HD, parts_max < 1 ? 1 : parts_max);
  k.rank = x.rank, k.world = x.world, k.phases = x.phases, k.wait_ms = x.wait_ms ? uint32_t(x.wait_ms) : 2000u, k.epoch = x.epoch;
  for (int q = 0; q < x.world; ++q) k.records[q] = static_cast<uint2*>(x.records[q]);
  k.status = c->d_status;
  k.trace = c->trace_blocks >= 1 ? c->trace : nullptr;
  // Every CTA may wait for its peers: the grid has to be resident at once (2 CTAs of 256 threads per SM at least).
  if (esp::exchange_grid_ctas(k.c) > 296)
    return fail(ESP_ERR_UNSUPPORTED, "esp_attn_exchange_parts: %lld CTAs cannot be resident at once; gather the records with a collective and call esp_attn_combine_parts",
                (long long)esp::exchange_grid_ctas(k.c));
  cudaError_t e;
  {
    ProfScope prof(c, static_cast<cudaStream_t>(stream), "exchange_parts");
    e = esp::launch_exchange(k, static_cast<cudaStream_t>(stream), &c->launches);
  }
  if (e != cudaSuccess) return cuda_fail(e, "exchange_parts");
  return ESP_OK;
}

int esp_p2p_alloc(void** ptr, size_t bytes, unsigned char handle[ESP_P2P_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == ESP_P2P_HANDLE_BYTES, "IPC handle size");
  if (!ptr || !handle || bytes == 0) return fail(ESP_ERR_INVALID, "esp_p2p_alloc: null argument or zero size");
  *ptr = nullptr;
  void* d = nullptr;
  cudaError_t e = cudaMalloc(&d, bytes);
  if (e != cudaSuccess) return cuda_fail(e, "esp_p2p_alloc: cudaMalloc");
  if ((e = cudaMemset(d, 0, bytes)) == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t hd;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&hd, d);
  if (e != cudaSuccess) {
    cudaFree(d);
    return cuda_fail(e, "esp_p2p_alloc: zero fill / cudaIpcGetMemHandle");
  }
  memcpy(handle, &hd, sizeof(hd));
  *ptr = d;
  return ESP_OK;
}

int esp_p2p_open(const unsigned char handle[ESP_P2P_HANDLE_BYTES], void** ptr) {
  if (!ptr || !handle) return fail(ESP_ERR_INVALID, "esp_p2p_open: null argument");
  cudaIpcMemHandle_t hd;
  memcpy(&hd, handle, sizeof(hd));
  *ptr = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(ptr, hd, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail(e, "esp_p2p_open: cudaIpcOpenMemHandle");
  return ESP_OK;
}

int esp_p2p_close(void* ptr) {
  if (!ptr) return ESP_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) return cuda_fail(e, "esp_p2p_close: cudaIpcCloseMemHandle");
  return ESP_OK;
}

int esp_p2p_free(void* ptr) {
  if (!ptr) return ESP_OK;
  const cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return cuda_fail(e, "esp_p2p_free: cudaFree");
  return ESP_OK;
}

}  // extern "C"

static int combine_impl(esp_attn_ctx* c, void* stream, const float* parts, const float* X, void* O, float* lse,
                        const esp_attn_params* p, const esp_attn_combine* jobs, int32_t n_jobs, int rows_max, int parts_max,
                        float* out_parts, int32_t out_part0, const esp_attn_combine* jobs_host, int tile_rows) {
  if (!c || !p) return fail(ESP_ERR_INVALID, "esp_attn_combine_parts: null argument");
  if (n_jobs <= 0) return ESP_OK;
  if (!parts || (!O && !out_parts) || !jobs) return fail(ESP_ERR_INVALID, "esp_attn_combine_parts: null parts / O / jobs");
  if (int rc = check_params(c, *p)) return rc;
  const esp_attn_shape& s = c->shape;
  if ((s.flags & ESP_ATTN_FLAG_GATE) && !X) return fail(ESP_ERR_INVALID, "esp_attn_combine_parts: gate flag set but X is null");
  esp::CombineArgs k{};
  k.parts = parts, k.X = (s.flags & ESP_ATTN_FLAG_GATE) ? X : nullptr, k.O = O, k.lse = lse, k.jobs = jobs, k.p = *p;
  const int TR = tile_rows > 0 ? tile_rows : c->tile_rows;  // a re-planned pass merges records of its own tile height
  k.HD = s.HD, k.G = c->G, k.tile_rows = TR, k.n_jobs = n_jobs, k.q_dtype = s.q_dtype;
  k.rows_max = rows_max < 1 ? 1 : (rows_max > TR ? TR : rows_max);
  k.n_slices = esp::combine_slices(s.HD, parts_max);
  k.out_parts = out_parts, k.out_part0 = out_part0;
  if (jobs_host && n_jobs <= esp::kInlineJobsMax) {
    k.n_inline = n_jobs;
    for (int i = 0; i < n_jobs; ++i) k.inline_jobs[i] = jobs_host[i];
  }
  const cudaError_t e = esp::launch_combine(k, static_cast<cudaStream_t>(stream), &c->launches);
  if (e != cudaSuccess) return cuda_fail(e, "attention_combine");
  return ESP_OK;
}

extern "C" {

int esp_attn_prep(esp_attn_ctx* c, void* stream, const float* X, const float* q_norm_w, const float* k_norm_w, const int32_t* pos,
                  const float* inv_freq, const int32_t* rope_sel, void* Q, void* Kb, void* Vb, const int32_t* ktab, void* kv,
                  const float* kv_scales, int32_t rows, const esp_attn_prep_params* pp) {
  if (!c || !pp) return fail(ESP_ERR_INVALID, "esp_attn_prep: null argument");
  if (rows <= 0) return ESP_OK;
  const esp_attn_shape& s = c->shape;
  const esp_attn_prep_params& p = *pp;
  if (!esp::attn_prep_supports(s.HD)) return fail(ESP_ERR_UNSUPPORTED, "esp_attn_prep: head dim %d (128 or 256)", s.HD);
  if (!X || !q_norm_w || !k_norm_w || !pos || !inv_freq || !rope_sel || !Q || !Kb || !Vb)
    return fail(ESP_ERR_INVALID, "esp_attn_prep: null input / output pointer");
  if (p.H != s.H || p.Hkv != s.Hkv) return fail(ESP_ERR_INVALID, "esp_attn_prep: H=%d Hkv=%d do not match the context", p.H, p.Hkv);
  const int npt = s.HD / 32;
  if (p.rot_half < npt || p.rot_half > s.HD / 2 || (p.rot_half & (p.rot_half - 1)))
    return fail(ESP_ERR_INVALID, "esp_attn_prep: rot_half=%d (a power of two in [%d, %d])", p.rot_half, npt, s.HD / 2);
  if (p.ld % 4 || p.q_off % 4 || p.q_stride % 4 || p.k_off % 4 || p.v_off % 4 || p.q_stride < s.HD || p.q_off < 0 || p.k_off < 0 || p.v_off < 0)
    return fail(ESP_ERR_INVALID, "esp_attn_prep: X columns must be multiples of 4 floats (ld=%d q_off=%d q_stride=%d k_off=%d v_off=%d)", p.ld,
                p.q_off, p.q_stride, p.k_off, p.v_off);
  const int64_t need = std::max<int64_t>({int64_t(p.q_off) + int64_t(s.H - 1) * p.q_stride + s.HD, int64_t(p.k_off) + int64_t(s.Hkv) * s.HD,
                                          int64_t(p.v_off) + int64_t(s.Hkv) * s.HD});
  if (p.ld < need) return fail(ESP_ERR_INVALID, "esp_attn_prep: ld=%d but the heads reach column %lld", p.ld, (long long)need);
  if (p.q_ld < s.H * s.HD || p.kv_ld < s.Hkv * s.HD || p.q_ld % 8 || p.kv_ld % 8)
    return fail(ESP_ERR_INVALID, "esp_attn_prep: q_ld=%d kv_ld=%d", p.q_ld, p.kv_ld);
  if (!(p.eps >= 0.0f) || !(p.qscale > 0.0f)) return fail(ESP_ERR_INVALID, "esp_attn_prep: eps / qscale");
  const bool fp8 = s.kv_dtype == ESP_E4M3;
  if (ktab) {
    if (!kv || p.bt <= 0) return fail(ESP_ERR_INVALID, "esp_attn_prep: ktab given but no pool / bt");
    if (fp8 && !kv_scales) return fail(ESP_ERR_INVALID, "esp_attn_prep: E4M3 pool needs kv_scales");
    if (p.kv_base % 8) return fail(ESP_ERR_INVALID, "esp_attn_prep: kv_base must be a multiple of 8 elements");
  }
  // Heads per warp: as many as keep about four CTAs per SM in the grid (the rotation's sines and
  // cosines are formed once per warp), between 1 (decode: few rows) and 16.
  const int heads = s.H + s.Hkv;
  const int64_t want_ctas = 148 * 4;
  const int q4 = (heads + 3) / 4;  // heads per warp if one CTA took the whole row
  const int cap = int(std::clamp<int64_t>(int64_t(rows) * q4 / want_ctas, 1, 16));
  const int per_row = (q4 + cap - 1) / cap;   // CTAs per row
  const int hpw = (q4 + per_row - 1) / per_row;  // spread evenly over them
  esp::PrepArgs a{X, q_norm_w, k_norm_w, pos, inv_freq, rope_sel, Q, Kb, Vb, ktab, kv, kv_scales, rows, hpw, p};
  const cudaError_t e = esp::launch_attn_prep(a, s.HD, s.q_dtype, fp8 && ktab, static_cast<cudaStream_t>(stream), &c->launches);
  if (e != cudaSuccess) return cuda_fail(e, "attn_prep");
  return ESP_OK;
}

int esp_kv_save(esp_attn_ctx* c, void* stream, const void* Kb, const void* Vb, void* kv, const float* kv_scales,
                const esp_kv_save_entry* entries, int32_t n, const esp_attn_params* p) {
  if (!c || !p) return fail(ESP_ERR_INVALID, "esp_kv_save: null argument");
  if (n <= 0) return ESP_OK;
  if (!Kb || !Vb || !kv || !entries) return fail(ESP_ERR_INVALID, "esp_kv_save: null Kb / Vb / kv / entries");
  if (int rc = check_params(c, *p)) return rc;
  if (c->shape.kv_dtype == ESP_E4M3 && !kv_scales) return fail(ESP_ERR_INVALID, "esp_kv_save: E4M3 pool needs kv_scales");
  const cudaError_t e = esp::launch_kv_save(Kb, Vb, kv, kv_scales, entries, n, *p, c->shape.HD, c->shape.q_dtype, c->shape.kv_dtype,
                                            static_cast<cudaStream_t>(stream), &c->launches);
  if (e != cudaSuccess) return cuda_fail(e, "kv_save");
  return ESP_OK;
}

int esp_kv_copy_blocks(esp_attn_ctx* c, void* stream, void* kv, const int32_t* pairs, int32_t n_pairs, const esp_attn_params* p,
                       uint64_t region_elems, int32_t n_layers) {
  if (!c || !p) return fail(ESP_ERR_INVALID, "esp_kv_copy_blocks: null argument");
  if (n_pairs <= 0 || n_layers <= 0) return ESP_OK;
  if (!kv || !pairs) return fail(ESP_ERR_INVALID, "esp_kv_copy_blocks: null kv / pairs");
  if (n_pairs > 65535 || n_layers > 65535) return fail(ESP_ERR_UNSUPPORTED, "esp_kv_copy_blocks: at most 65535 pairs and layers per call");
  if (int rc = check_params(c, *p)) return rc;
  const int esz = elem_bytes(c->shape.kv_dtype);
  if ((region_elems * esz) % 16) return fail(ESP_ERR_INVALID, "esp_kv_copy_blocks: region size must be a multiple of 16 bytes");
  const cudaError_t e = esp::launch_kv_copy_blocks(kv, pairs, n_pairs, *p, region_elems, n_layers, esz, static_cast<cudaStream_t>(stream), &c->launches);
  if (e != cudaSuccess) return cuda_fail(e, "kv_copy_blocks");
  return ESP_OK;
}

}  // extern "C"
