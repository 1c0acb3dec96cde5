// TEST INFRASTRUCTURE: C entry points over the reference's OWN integer host code and per-thread
// kernels, compiled from the reference tree where it lies (see extract_ref.py, which cuts the
// definitions into oracle/_ref/*.inc; nothing of them is stored in this repository). Only tests/
// load the resulting oracle/_ref/libplan_ref.so; the product library never does.
//
// What this file adds around the reference's text is only what that text expects to find:
// fail() (src/model/impl/common.h:48 throws std::runtime_error), a Model that holds the KV pool, a
// host buffer with ensure<T>(), the pool's initial free list (cut from make_pools), and - for the
// three Metal kernels that are written one thread at a time - the handful of Metal types and
// address-space words they use. The functions themselves are the reference's, unmodified.
#include <algorithm>
#include <array>
#include <climits>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace espetero::native {

[[noreturn]] inline void fail(const std::string& msg) { throw std::runtime_error(msg); }
constexpr int kMaxDraft = 16;

#include "_ref/ref_types.inc"

struct VisionCfg {
  int merge = 1;
};
struct Vision {
  VisionCfg c;
};
struct Config {
  int idx_heads = 4, idx_kv = 1, idx_hd = 128;  // the indexer's geometry (kernels/45_qsa.metal:33-34)
};
struct Model {
  KVPool kv;
  Vision vis;
  Config cfg;
  bool qsa = true;
#include "_ref/ref_model_kv.inc"
};
struct HostBuf {
  std::vector<unsigned char> bytes;
  template <class T>
  T* ensure(Model&, size_t n) {
    bytes.assign(n * sizeof(T), 0);
    return reinterpret_cast<T*>(bytes.data());
  }
};
struct PassMeta {};

#include "_ref/ref_tree_plan.inc"

struct Forest {
  Model& m;
  PassMeta& meta;
  explicit Forest(Model& model, PassMeta& pm) : m(model), meta(pm) {}
#include "_ref/ref_target_blocks.inc"
};

#include "_ref/ref_funcs.inc"

// qsa_plan keeps its tables in a pass arena of GPU-visible buffers: plain host memory here
struct Buf {
  std::vector<unsigned char>* bytes = nullptr;
};
inline void* ptr(const Buf& b) { return b.bytes->data(); }
struct PassArena {
  std::vector<std::vector<unsigned char>*> owned;
  Buf alloc(Model&, size_t n) {
    owned.push_back(new std::vector<unsigned char>(n));
    return Buf{owned.back()};
  }
  ~PassArena() {
    for (auto* v : owned) delete v;
  }
};
#include "_ref/ref_qsa_plan.inc"

inline void pool_init(Model& m, int n_blocks, int bt) {
  KVPool& K = m.kv;
  K.bt = bt;
  K.n_blocks = n_blocks;
#include "_ref/ref_pool_init.inc"
}

// run_forest's leaf hosting (the loop is cut from the middle of the function: these are its locals)
inline int leaf_hosting(TreePlan& T, const TreeSpec& b, int& leaf_rows) {
  const bool cands = false;
  int max_leaf = 0;
#include "_ref/ref_leaf_hosting.inc"
  return max_leaf;
}

struct RowsCfg {
  int V = 1 << 30;
  bool gemma = false;
};
// run_forest's row records over a list of planned trees (its locals again)
inline void row_records(Model& m, const RowsCfg& c, std::vector<TreePlan>& trees, int32_t* tok, int32_t* pos, int32_t* csrc, int32_t* rslot,
                        int32_t* desc, int32_t* last, int32_t* cid, int32_t* cown) {
#include "_ref/ref_rows.inc"
}

// run_forest's block tables: read tables, target lists, copy-on-write pairs and save records
inline void block_tables(Model& m, std::vector<TreePlan>& trees, std::vector<int32_t>& table, std::vector<std::pair<int, int>>& cow,
                         std::vector<KVSaveRec>& kv_saves, std::vector<KVSaveRec>& mtp_saves) {
  PassMeta meta;
  Forest F(m, meta);
  const int bt = m.kv.bt;
#include "_ref/ref_block_tables.inc"
}

}  // namespace espetero::native

// ---------------------------------------------------------------- Metal words for the per-thread kernels
namespace msl {
using uint = unsigned int;
using ulong = unsigned long long;
using uchar = unsigned char;
using ushort = unsigned short;
using half = _Float16;
struct half2 {
  half x, y;
};
struct half4 {
  half x, y, z, w;
};
struct float4 {
  float x, y, z, w;
  float4() = default;
  explicit float4(float v) : x(v), y(v), z(v), w(v) {}
  float4(float a, float b, float c, float d) : x(a), y(b), z(c), w(d) {}
};
inline float4 operator*(float s, const float4& v) { return {s * v.x, s * v.y, s * v.z, s * v.w}; }
inline float4 operator*(const float4& v, float s) { return {v.x * s, v.y * s, v.z * s, v.w * s}; }
inline float4 operator+(float s, const float4& v) { return {s + v.x, s + v.y, s + v.z, s + v.w}; }
inline float4 operator/(const float4& a, const float4& b) { return {a.x / b.x, a.y / b.y, a.z / b.z, a.w / b.w}; }
inline float4 operator-(const float4& v) { return {-v.x, -v.y, -v.z, -v.w}; }
inline float4& operator+=(float4& a, const float4& b) {
  a.x += b.x, a.y += b.y, a.z += b.z, a.w += b.w;
  return a;
}
inline float4 exp(const float4& v) { return {std::exp(v.x), std::exp(v.y), std::exp(v.z), std::exp(v.w)}; }
inline float exp(float v) { return std::exp(v); }
inline float max(float a, float b) { return a > b ? a : b; }  // a NaN-free comparison is all the kernels need
inline float min(float a, float b) { return a < b ? a : b; }
inline float fabs(float v) { return std::fabs(v); }
inline float rint(float v) { return std::nearbyint(v); }  // round half to even, as Metal's rint
inline float copysign(float a, float b) { return std::copysign(a, b); }
inline half4 to_half4(const float4& v) { return {half(v.x), half(v.y), half(v.z), half(v.w)}; }
struct half4_ctor {  // half4(o) in the kernel text
  half4 v;
  half4_ctor(const float4& f) : v(to_half4(f)) {}
  operator half4() const { return v; }
};
struct uint2 {
  uint x, y;
};
struct uint3 {
  uint x, y, z;
};
struct uint4 {
  uint x, y, z, w;
};
struct int2 {
  int x, y;
};
template <class To, class From>
inline To as_type(const From& f) {
  static_assert(sizeof(To) == sizeof(From), "as_type: same size");
  To t;
  std::memcpy(&t, &f, sizeof(To));
  return t;
}
#define device
#define constant const
#define kernel inline
#define UNROLL
#define half4(x) (msl::half4)msl::half4_ctor(x)
#include "_ref/ref_e4m3.inc"
#include "_ref/ref_kernels.inc"
#undef half4
#undef UNROLL
#undef kernel
#undef constant
#undef device
}  // namespace msl

using namespace espetero::native;

namespace {
thread_local std::string g_error;
template <class F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return -1;
  }
}
}  // namespace

extern "C" {

const char* ref_last_error(void) { return g_error.c_str(); }

// plan_tiles (src/model/impl/forest.h:1378-1433). qt_flat: per tree, per 8-row group, the sparse list id
// (-1: dense) - the reference's `qt` argument flattened; NULL = nullptr.
int ref_plan_tiles(const AttnTreeRec* trees, int n_trees, int Hkv, int split, int groups, int min_chunk, const int32_t* qt_flat,
                   AttnTileRec* tiles, int tiles_cap, AttnCombineRec* jobs, int jobs_cap, int* n_tiles, int* n_jobs, int* n_parts) {
  return guarded([&] {
    AttnPlan A;
    A.trees.assign(trees, trees + n_trees);
    std::vector<std::vector<int>> qt;
    if (qt_flat) {
      size_t at = 0;
      for (int t = 0; t < n_trees; ++t) {
        const size_t n = size_t((trees[t].M + 7) / 8);
        qt.emplace_back(qt_flat + at, qt_flat + at + n);
        at += n;
      }
    }
    plan_tiles(A, Hkv, split, qt_flat ? &qt : nullptr, groups, min_chunk);
    *n_tiles = int(A.tiles.size()), *n_jobs = int(A.combine.size()), *n_parts = A.parts;
    if (tiles) std::copy_n(A.tiles.begin(), std::min<size_t>(A.tiles.size(), size_t(tiles_cap)), tiles);
    if (jobs) std::copy_n(A.combine.begin(), std::min<size_t>(A.combine.size(), size_t(jobs_cap)), jobs);
  });
}

// g4_plan_tiles (src/model/impl/gemma.h:77-116)
int ref_g4_plan_tiles(const AttnTreeRec* trees, int n_trees, int groups, int split, int window, const int32_t* pos, int rows, G4TileRec* tiles,
                      int tiles_cap, AttnCombineRec* jobs, int jobs_cap, int* n_tiles, int* n_jobs, int* n_parts, int* plan_rows) {
  return guarded([&] {
    G4Plan A;
    A.trees.assign(trees, trees + n_trees);
    g4_plan_tiles(A, groups, split, window, pos, rows);
    *n_tiles = int(A.tiles.size()), *n_jobs = int(A.combine.size()), *n_parts = A.parts, *plan_rows = A.rows;
    if (tiles) std::copy_n(A.tiles.begin(), std::min<size_t>(A.tiles.size(), size_t(tiles_cap)), tiles);
    if (jobs) std::copy_n(A.combine.begin(), std::min<size_t>(A.combine.size(), size_t(jobs_cap)), jobs);
  });
}

// KVPool + kv_alloc / kv_retain / kv_release (src/model/impl/model.h:387-411, :722-737; initial free list forest.h:59-61)
void* ref_model_create(int n_blocks, int bt) {
  auto* m = new Model;
  pool_init(*m, n_blocks, bt);
  return m;
}
void ref_model_destroy(void* m) { delete static_cast<Model*>(m); }
int ref_kv_free(void* m) { return int(static_cast<Model*>(m)->kv.free_list.size()); }
int ref_kv_refcount(void* m, int b) { return static_cast<Model*>(m)->kv.ref[size_t(b)]; }
int ref_kv_alloc(void* m, int* block) {
  return guarded([&] { *block = static_cast<Model*>(m)->kv_alloc(); });
}
void ref_kv_retain(void* m, int b) { static_cast<Model*>(m)->kv_retain(b); }
void ref_kv_release(void* m, int b) { static_cast<Model*>(m)->kv_release(b); }

// Forest::target_blocks and target_new_blocks (forest.h:1785-1829)
int ref_target_blocks(void* mv, const int32_t* parent, int n_parent, int P, int w0, int end, int in_place, int32_t* out, int out_cap, int* n_out,
                      int32_t* cow_pairs, int cow_cap, int* n_cow) {
  return guarded([&] {
    Model& m = *static_cast<Model*>(mv);
    PassMeta meta;
    Forest F(m, meta);
    std::vector<int> pb(parent, parent + n_parent);
    std::vector<std::pair<int, int>> cow;
    const std::vector<int> got = F.target_blocks(pb, P, w0, end, cow, in_place != 0);
    *n_out = int(got.size()), *n_cow = int(cow.size());
    for (size_t i = 0; i < got.size() && int(i) < out_cap; ++i) out[i] = got[i];
    for (size_t i = 0; i < cow.size() && int(i) < cow_cap; ++i) cow_pairs[2 * i] = cow[i].first, cow_pairs[2 * i + 1] = cow[i].second;
  });
}
int ref_target_new_blocks(void* mv, const int32_t* parent, int n_parent, int P, int w0, int end, int in_place) {
  Slot s;
  if (parent) s.blocks.assign(parent, parent + n_parent);
  return target_new_blocks(*static_cast<Model*>(mv), parent ? &s : nullptr, P, w0, end, in_place != 0);
}

// kv_row_table (forest.h:1739-1749)
int ref_kv_row_table(const KVSaveRec* saves, int n, int rows, int32_t* table) {
  return guarded([&] {
    Model m;
    HostBuf hb;
    kv_row_table(m, hb, std::vector<KVSaveRec>(saves, saves + n), rows);
    std::memcpy(table, hb.bytes.data(), size_t(std::max(rows, 1)) * 16);
  });
}

// One tree through run_forest's leaf hosting (forest.h:2196-2220) and row records (:2378-2450).
// readout_rows holds n_leaves + 1 entries (the last is written only with score_root).
int ref_tree_rows(const int32_t* root, int root_len, const int32_t* root_pos, int n_leaves, const int32_t* leaf_offsets, const int32_t* leaf_tokens,
                  int noncausal, int score_root, int base, int pnext, int32_t* host, int32_t* off, int32_t* tok, int32_t* pos4, int32_t* desc4,
                  int32_t* readout_rows, int* n_rows, int* next_root) {
  return guarded([&] {
    TreeSpec b;
    b.root = root, b.root_len = root_len, b.root_pos = root_pos, b.n_leaves = n_leaves, b.leaf_offsets = leaf_offsets, b.leaf_tokens = leaf_tokens;
    b.noncausal = noncausal != 0, b.score_root = score_root != 0;
    Slot parent;
    parent.next_pos = pnext;
    std::vector<TreePlan> trees(1);
    TreePlan& T = trees[0];
    T.spec = &b, T.parent = &parent;
    T.Tr = b.root_len, T.save_len = T.Tr, T.NL = b.n_leaves, T.N = T.NL + (b.score_root ? 1 : 0);
    int leaf_rows = 0;
    if (T.NL > 0) leaf_hosting(T, b, leaf_rows);
    T.M = T.Tr + leaf_rows, T.base = base, T.readout_base = 0, T.cand_base = 0;
    const size_t rows = size_t(base + T.M);
    std::vector<int32_t> tk(rows + 1), ps(4 * rows + 4), cs(3 * rows + 3), rs(rows + 1), ds(4 * rows + 4), last(size_t(T.N) + 1, -1), cid(1), cown(1);
    Model m;
    RowsCfg c;
    row_records(m, c, trees, tk.data(), ps.data(), cs.data(), rs.data(), ds.data(), last.data(), cid.data(), cown.data());
    for (int i = 0; i < T.NL; ++i) host[i] = T.host[size_t(i)], off[i] = T.off[size_t(i)];
    for (int r = 0; r < T.M; ++r) {
      tok[r] = tk[size_t(base + r)];
      for (int k = 0; k < 4; ++k) pos4[4 * r + k] = ps[4 * size_t(base + r) + k], desc4[4 * r + k] = ds[4 * size_t(base + r) + k];
    }
    for (int i = 0; i < T.N; ++i) readout_rows[i] = last[size_t(i)];
    *n_rows = T.M, *next_root = T.next_root;
  });
}

// run_forest's block tables for a list of in-place / forked targets (forest.h:2483-2520): tree i continues a
// parent list of n_parent[i] blocks covering P[i] keys and saves save_len[i] rows from row base[i]; dst_same[i]:
// the target is the parent itself (in-place append). Returns the read table, the targets' lists, the
// copy-on-write pairs and the save records, in the reference's order.
int ref_block_tables(void* mv, int n_trees, const int32_t* parent_blocks, const int32_t* n_parent, const int32_t* P, const int32_t* base,
                     const int32_t* save_len, const int32_t* dst_same, int32_t* table, int table_cap, int* n_table, int32_t* dst_blocks,
                     int dst_cap, int32_t* n_dst, int32_t* cow_pairs, int cow_cap, int* n_cow, KVSaveRec* saves, int saves_cap, int* n_saves) {
  return guarded([&] {
    Model& m = *static_cast<Model*>(mv);
    std::vector<Slot> parents{size_t(n_trees)}, dsts{size_t(n_trees)};
    std::vector<TreePlan> trees(static_cast<size_t>(n_trees));
    size_t at = 0;
    for (int i = 0; i < n_trees; ++i) {
      parents[size_t(i)].blocks.assign(parent_blocks + at, parent_blocks + at + n_parent[i]);
      at += size_t(n_parent[i]);
      TreePlan& T = trees[size_t(i)];
      T.parent = &parents[size_t(i)];
      T.dst = dst_same[i] ? T.parent : &dsts[size_t(i)];
      T.P = P[i], T.base = base[i], T.save_len = save_len[i], T.Tr = save_len[i];
    }
    std::vector<int32_t> tab;
    std::vector<std::pair<int, int>> cow;
    std::vector<KVSaveRec> kv_saves, mtp_saves;
    block_tables(m, trees, tab, cow, kv_saves, mtp_saves);
    *n_table = int(tab.size()), *n_cow = int(cow.size()), *n_saves = int(kv_saves.size());
    for (size_t i = 0; i < tab.size() && int(i) < table_cap; ++i) table[i] = tab[i];
    for (size_t i = 0; i < cow.size() && int(i) < cow_cap; ++i) cow_pairs[2 * i] = cow[i].first, cow_pairs[2 * i + 1] = cow[i].second;
    for (size_t i = 0; i < kv_saves.size() && int(i) < saves_cap; ++i) saves[i] = kv_saves[i];
    size_t d = 0;
    for (int i = 0; i < n_trees; ++i) {
      n_dst[i] = int(trees[size_t(i)].dst_blocks.size());
      for (int b : trees[size_t(i)].dst_blocks)
        if (int(d) < dst_cap) dst_blocks[d++] = b;
    }
  });
}

// qsa_plan (forest.h:1489-1543): per row (s, nb, sparse row or -1, tree), the sparse rows, the 8-row tiles that hold
// sparse rows and, per tree and 8-row group, its tile or -1 (flattened). counts = {M, n_sparse, nbmax, nbb, ncb, n_tiles}.
int ref_qsa_plan(const AttnTreeRec* trees, int n_trees, const int32_t* desc, int sparse, int32_t* rows4, int32_t* srows, int32_t* qtiles4,
                 int32_t* qt_flat, int32_t* counts) {
  return guarded([&] {
    Model m;
    PassArena arena;
    QsaSet q;
    qsa_plan(m, arena, q, std::vector<AttnTreeRec>(trees, trees + n_trees), desc, sparse != 0);
    counts[0] = q.M, counts[1] = q.n_sparse, counts[2] = q.nbmax, counts[3] = q.nbb, counts[4] = q.ncb, counts[5] = int(q.tiles.size());
    std::memcpy(rows4, ptr(q.rows), size_t(q.M) * 16);
    if (q.n_sparse) std::memcpy(srows, ptr(q.srows), size_t(q.n_sparse) * 4);
    if (!q.tiles.empty()) std::memcpy(qtiles4, q.tiles.data(), q.tiles.size() * 16);
    size_t at = 0;
    for (const auto& v : q.qt_of)
      for (int x : v) qt_flat[at++] = x;
  });
}

// ds4_round_e4m3 / ds4_e4m3x2 (kernels/80_dsv4.metal:22-33, :58-60)
float ref_round_e4m3(float v) { return msl::ds4_round_e4m3(v); }
// the two decoded values (times 2^-8, as the kernel leaves them) of the codes in bits 0-15 of w
void ref_e4m3x2(unsigned w, float* lo, float* hi) {
  const msl::half2 h = msl::ds4_e4m3x2(w);
  *lo = float(h.x), *hi = float(h.y);
}

// attention_combine (kernels/40_attention.metal:811-864), one call per grid: every (d4, h, job * 8 + r) thread in turn.
// O: fp16 bits. The kernel is written for 256-dim heads and gated output.
void ref_attention_combine(const float* parts, const float* X, uint16_t* O, const msl::AttnParams* p, const msl::AttnCombine* jobs, int n_jobs) {
  for (unsigned z = 0; z < unsigned(n_jobs) * 8; ++z)
    for (unsigned h = 0; h < unsigned(p->H); ++h)
      for (unsigned x = 0; x < 64; ++x) msl::attention_combine(parts, X, reinterpret_cast<msl::half*>(O), *p, jobs, msl::uint3{x, h, z});
}
// kv_save (:875-889) and kv_copy_blocks (:894-905), every thread of their grids in turn
void ref_kv_save(const uint16_t* Kb, const uint16_t* Vb, uint16_t* kv, const msl::KVSave* entries, int n, const msl::AttnParams* p) {
  for (unsigned y = 0; y < unsigned(n); ++y)
    for (unsigned x = 0; x < unsigned(p->kv_ld + 7) / 8; ++x)
      msl::kv_save(reinterpret_cast<const msl::half*>(Kb), reinterpret_cast<const msl::half*>(Vb), reinterpret_cast<msl::half*>(kv), entries, *p, msl::uint2{x, y});
}
void ref_kv_copy_blocks(uint16_t* kv, const int32_t* pairs, int n_pairs, const msl::AttnParams* p, unsigned long long region_halves, int n_layers) {
  const unsigned nx = unsigned((2ull * unsigned(p->bt) * unsigned(p->kv_ld) + 7) / 8);
  for (unsigned z = 0; z < unsigned(n_layers); ++z)
    for (unsigned y = 0; y < unsigned(n_pairs); ++y)
      for (unsigned x = 0; x < nx; ++x)
        msl::kv_copy_blocks(reinterpret_cast<msl::half*>(kv), reinterpret_cast<const msl::int2*>(pairs), *p, region_halves, msl::uint3{x, y, z});
}

}  // extern "C"
