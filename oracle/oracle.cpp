// TEST INFRASTRUCTURE - not part of the product library.
//
// CPU restatement of the attention path of JarJarFran/espetero, used only as the
// checker in tests/, in the smoke check and as the timed CPU baseline of bench.py.
// The product (espetero_b200/csrc) never links, loads or calls anything here.
//
// PARITY UNPINNED: the reference holds no golden vector, known-answer test or
// fixture for this path (its only numerical check of these kernels,
// tools/qsa_check.mm:296-331, needs Metal), and its Metal kernels cannot run on
// Linux. What pins this file instead: (1) the float64 direct-softmax oracle below
// follows the semantics stated at kernels/40_attention.metal:104-120; (2) the fp32
// restatements of the reference kernels must agree with (1); (3) the integer
// planners are checked against hand-derived cases from the reference's comments.
//
// Contents (reference file:line each part follows):
//   orc_attention_f64   semantics of kernels/40_attention.metal:104-120, :246-247, :281-283, :334-342
//   orc_flash_f32       flash_attention, kernels/40_attention.metal:156-343 (generic HD: 80_gemma.metal:157-342)
//   orc_decode_gqa_f32  attn_decode_gqa, kernels/40_attention.metal:598-781
//   orc_combine_f32     attention_combine, kernels/40_attention.metal:811-864
//   orc_kv_save / orc_kv_copy_blocks  kernels/40_attention.metal:875-905
//   orc_plan_tiles      plan_tiles, src/model/impl/forest.h:1378-1433
//   orc_g4_plan_tiles   g4_plan_tiles (no window), src/model/impl/gemma.h:77-116
//   orc_round_e4m3 / orc_e4m3_*  ds4_round_e4m3, ds4_e4m3x2, kernels/80_dsv4.metal:22-33, :58-60
#if defined(__linux__)
#include <sched.h>
#endif
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace {

// ------------------------------------------------------------------ storage types
enum { ORC_F16 = 0, ORC_BF16 = 1, ORC_E4M3 = 2 };

inline float f16_to_f32(uint16_t h) {
  const uint32_t s = uint32_t(h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, out;
  if (e == 0) {
    if (m == 0) {
      out = s;
    } else {
      int sh = 0;
      while (!(m & 0x400u)) m <<= 1, ++sh;
      out = s | uint32_t(127 - 15 - sh + 1) << 23 | (m & 0x3FFu) << 13;
    }
  } else if (e == 31) {
    out = s | 0x7F800000u | m << 13;
  } else {
    out = s | (e + 112) << 23 | m << 13;
  }
  float f;
  std::memcpy(&f, &out, 4);
  return f;
}

// round-to-nearest-even float -> fp16 bits
inline uint16_t f32_to_f16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint16_t s = uint16_t((x >> 16) & 0x8000u);
  const uint32_t a = x & 0x7FFFFFFFu;
  if (a >= 0x7F800000u) return uint16_t(s | 0x7C00u | ((a > 0x7F800000u) ? 0x200u : 0));
  if (a >= 0x477FF000u) return uint16_t(s | 0x7C00u);  // rounds to inf (>= 65520)
  if (a < 0x33000001u) return s;                       // below half the smallest subnormal
  const int e = int(a >> 23) - 127;
  uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
  int shift;
  uint32_t base;
  if (e < -14) {
    shift = 13 + (-14 - e);
    base = 0;
  } else {
    shift = 13;
    base = uint32_t(e + 15) << 10;
    m &= 0x7FFFFFu;
  }
  uint32_t q = m >> shift;
  const uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1))) ++q;
  return uint16_t(s | (base + q));
}

inline float bf16_to_f32(uint16_t h) {
  const uint32_t x = uint32_t(h) << 16;
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}

inline uint16_t f32_to_bf16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return uint16_t((x >> 16) | 0x40u);
  x += 0x7FFFu + ((x >> 16) & 1u);
  return uint16_t(x >> 16);
}

// e4m3fn code -> value: 1 sign, 4 exponent (bias 7), 3 mantissa, no infinities.
inline float e4m3_to_f32(uint8_t c) {
  const int e = (c >> 3) & 0xF, m = c & 7;
  float v;
  if (e == 0) v = std::ldexp(float(m), -9);
  else if (e == 15 && m == 7) v = std::numeric_limits<float>::quiet_NaN();
  else v = std::ldexp(float(8 + m), e - 10);
  return (c & 0x80) ? -v : v;
}

// Round to the e4m3fn grid: nearest-even, subnormal step 2^-9 below 2^-6,
// saturating at 448 (kernels/80_dsv4.metal:22-33).
inline float round_e4m3(float v) {
  const float a = std::min(std::fabs(v), 448.0f);
  float q;
  if (a < 0.015625f) {
    q = std::nearbyint(a * 512.0f) * (1.0f / 512.0f);
  } else {
    int ex;
    std::frexp(a, &ex);  // a = f * 2^ex, f in [0.5, 1)
    const float step = std::ldexp(1.0f, ex - 1 - 3);
    q = std::nearbyint(a / step) * step;
  }
  return std::copysign(q, v);
}

inline uint8_t f32_to_e4m3(float v) {
  const float q = round_e4m3(v);
  const uint8_t s = std::signbit(q) ? 0x80 : 0;
  const float a = std::fabs(q);
  if (a == 0.0f) return s;
  if (a < 0.015625f) return uint8_t(s | uint8_t(std::lrint(a * 512.0f)));
  int ex;
  const float f = std::frexp(a, &ex);            // a = f 2^ex
  const int e = ex - 1 + 7;                       // biased
  const int m = int(std::lrint(f * 16.0f)) - 8;   // 1.mmm
  return uint8_t(s | (e << 3) | m);
}

inline float load16(const void* p, size_t i, int dt) {
  const uint16_t h = static_cast<const uint16_t*>(p)[i];
  return dt == ORC_F16 ? f16_to_f32(h) : bf16_to_f32(h);
}
inline uint16_t store16(float f, int dt) { return dt == ORC_F16 ? f32_to_f16(f) : f32_to_bf16(f); }
inline float round16(float f, int dt) { return dt == ORC_F16 ? f16_to_f32(f32_to_f16(f)) : bf16_to_f32(f32_to_bf16(f)); }

// ------------------------------------------------------------------ records
struct Params {
  int32_t H, Hkv, q_ld, kv_ld, g_ld, bt;
  uint64_t kv_base;
};
struct Tree {
  int32_t base, P, table, M;
};
struct Tile {
  int32_t tree, r0, k0, k1, part, last, pad0, pad1;
};
struct Combine {
  int32_t r0, rows, part0, nparts;
};
struct KVSave {
  int32_t src_row, block, pos, pad;
};
static_assert(sizeof(Params) == 32 && sizeof(Tree) == 16 && sizeof(Tile) == 32 && sizeof(Combine) == 16 && sizeof(KVSave) == 16,
              "record layout");

struct Problem {
  const void* Q;
  const void* Kb;
  const void* Vb;
  const void* kv;
  const float* kv_scales;  // [n_blocks][2][Hkv] or null
  const int32_t* blocks;
  const int32_t* desc;       // int4 per row or null
  const uint64_t* anc_mask;  // per row or null (wins over desc)
  const float* X;            // gate source or null
  const Tree* trees;
  int32_t n_trees;
  int32_t HD;
  int32_t q_dtype;
  int32_t kv_dtype;
  int32_t tile_rows;
  float scale;
  Params p;
  // Sliding-window layers of the generic kernel (kernels/80_gemma.metal:123-142): pos = int4 per row
  // (x = position), window > 0 masks keys `window` or more positions behind the query, ring > 0
  // reads cached key j from block table + (j / bt) % ring instead of the page table, bidi lets the
  // rows of an image see the image's later rows (desc.w = end of the row's image, 0 outside).
  const int32_t* pos;
  int32_t window, ring, bidi, pad;
};

struct KeyRef {  // one visible key of a row
  bool cached;
  int32_t j;
};

inline bool batch_visible(const Problem& pb, int row, int rr, int j) {
  if (pb.anc_mask) return j < 64 && ((pb.anc_mask[row] >> j) & 1ull);
  const int32_t* d = pb.desc + 4 * size_t(row);
  return (j < d[2]) || (j >= d[0] && (j <= rr || (pb.bidi && j < d[3])));  // 80_gemma.metal:284
}

// The window test of 80_gemma.metal:285: a key at position kpos is visible from a query at qpos
// iff qpos - kpos < window (cached key j sits at position j, a batch key at its row's position).
inline bool in_window(const Problem& pb, const Tree& t, int row, bool cached, int j) {
  if (pb.window <= 0) return true;
  const int qpos = pb.pos[4 * size_t(row)];
  const int kpos = cached ? j : pb.pos[4 * size_t(t.base + j)];
  return qpos - kpos < pb.window;
}

// One K (which 0) or V (1) row of a key, as raw codes (float) plus its scale: cached
// key j of the tree from the paged pool (kernels/40_attention.metal:246-247), or batch
// key j from Kb / Vb.
inline void load_key_row(const Problem& pb, const Tree& t, bool cached, int j, int which, int kvh, float* out, float* scale) {
  const Params& p = pb.p;
  const int HD = pb.HD;
  *scale = 1.0f;
  if (!cached) {
    const uint16_t* src = static_cast<const uint16_t*>(which ? pb.Vb : pb.Kb) + size_t(t.base + j) * p.kv_ld + size_t(kvh) * HD;
    if (pb.q_dtype == ORC_F16) for (int d = 0; d < HD; ++d) out[d] = f16_to_f32(src[d]);
    else for (int d = 0; d < HD; ++d) out[d] = bf16_to_f32(src[d]);
    return;
  }
  const uint64_t b = pb.ring > 0 ? uint64_t(t.table + (j / p.bt) % pb.ring) : uint64_t(pb.blocks[t.table + j / p.bt]);  // 80_gemma.metal:250
  const uint64_t off = p.kv_base + (b * 2 + uint64_t(which)) * uint64_t(p.bt) * p.kv_ld + uint64_t(j % p.bt) * p.kv_ld + uint64_t(kvh) * HD;
  if (pb.kv_dtype == ORC_E4M3) {
    *scale = pb.kv_scales[(b * 2 + which) * p.Hkv + kvh];
    const uint8_t* src = static_cast<const uint8_t*>(pb.kv) + off;
    for (int d = 0; d < HD; ++d) out[d] = e4m3_to_f32(src[d]);
  } else {
    const uint16_t* src = static_cast<const uint16_t*>(pb.kv) + off;
    if (pb.kv_dtype == ORC_F16) for (int d = 0; d < HD; ++d) out[d] = f16_to_f32(src[d]);
    else for (int d = 0; d < HD; ++d) out[d] = bf16_to_f32(src[d]);
  }
}

template <class F>
void parallel_for(int64_t n, int threads, F f) {
  if (threads <= 1 || n <= 1) {
    for (int64_t i = 0; i < n; ++i) f(i);
    return;
  }
  std::atomic<int64_t> next{0};
  std::vector<std::thread> pool;
  const int nt = int(std::min<int64_t>(threads, n));
  for (int t = 0; t < nt; ++t)
    pool.emplace_back([&] {
      for (;;) {
        const int64_t i = next.fetch_add(1);
        if (i >= n) break;
        f(i);
      }
    });
  for (auto& th : pool) th.join();
}

int tree_of_row(const Problem& pb, int row) {
  for (int t = 0; t < pb.n_trees; ++t)
    if (row >= pb.trees[t].base && row < pb.trees[t].base + pb.trees[t].M) return t;
  return -1;
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ codecs
float orc_round_e4m3(float v) { return round_e4m3(v); }
uint8_t orc_e4m3_encode(float v) { return f32_to_e4m3(v); }
float orc_e4m3_decode(uint8_t c) { return e4m3_to_f32(c); }
uint16_t orc_f16_encode(float v) { return f32_to_f16(v); }
float orc_f16_decode(uint16_t h) { return f16_to_f32(h); }
uint16_t orc_bf16_encode(float v) { return f32_to_bf16(v); }
float orc_bf16_decode(uint16_t h) { return bf16_to_f32(h); }
void orc_e4m3_encode_n(const float* v, uint8_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = f32_to_e4m3(v[i]);
}

// ------------------------------------------------------------------ float64 oracle
// Direct (not online) softmax in double over the visible keys of each listed row
// and every head. rows == null: all rows of all trees. O64: [n_eval][H*HD],
// lse64: [n_eval][H] (natural log of the sum of exp(scale q.k)); a row with no
// visible key gives O = 0, lse = -inf. Oabs64 (optional, same shape as O64) receives
// sum_j softmax_j |v_j|, the bound on what rounding P to 16 bits before P.V (as the
// reference kernels do, kernels/40_attention.metal:297) can change. Work unit = (row, kv
// head): each key's K and V rows are decoded once and shared by the G heads of the group.
int orc_attention_f64(const Problem* pbp, const int32_t* rows, int32_t n_rows, double* O64, double* lse64, double* Oabs64,
                      int threads) {
  const Problem& pb = *pbp;
  const Params& p = pb.p;
  const int HD = pb.HD, G = p.H / p.Hkv;
  std::vector<int32_t> all;
  if (!rows) {
    for (int t = 0; t < pb.n_trees; ++t)
      for (int r = 0; r < pb.trees[t].M; ++r) all.push_back(pb.trees[t].base + r);
    rows = all.data();
    n_rows = int32_t(all.size());
  }
  std::atomic<int> bad{0};
  parallel_for(int64_t(n_rows) * p.Hkv, threads, [&](int64_t idx) {
    const int ri = int(idx / p.Hkv), kvh = int(idx % p.Hkv);
    const int row = rows[ri];
    const int ti = tree_of_row(pb, row);
    if (ti < 0) {
      bad = 1;
      return;
    }
    const Tree& t = pb.trees[ti];
    const int rr = row - t.base;
    std::vector<double> q(size_t(G) * HD);
    for (int g = 0; g < G; ++g)
      for (int d = 0; d < HD; ++d)
        q[size_t(g) * HD + d] = double(load16(pb.Q, size_t(row) * p.q_ld + size_t(kvh * G + g) * HD + d, pb.q_dtype));
    std::vector<KeyRef> keys;
    keys.reserve(size_t(t.P) + t.M);
    for (int j = 0; j < t.P; ++j)
      if (in_window(pb, t, row, true, j)) keys.push_back({true, j});
    for (int j = 0; j < t.M; ++j)
      if (batch_visible(pb, row, rr, j) && in_window(pb, t, row, false, j)) keys.push_back({false, j});
    const size_t nk = keys.size();
    std::vector<double> s(size_t(G) * nk);
    std::vector<double> mx(G, -std::numeric_limits<double>::infinity());
    std::vector<float> rowbuf(HD);
    for (size_t k = 0; k < nk; ++k) {
      float sc;
      load_key_row(pb, t, keys[k].cached, keys[k].j, 0, kvh, rowbuf.data(), &sc);
      for (int g = 0; g < G; ++g) {
        double acc = 0;
        const double* qg = q.data() + size_t(g) * HD;
        for (int d = 0; d < HD; ++d) acc += qg[d] * (double(rowbuf[d]) * double(sc));
        acc *= double(pb.scale);
        s[size_t(g) * nk + k] = acc;
        mx[g] = std::max(mx[g], acc);
      }
    }
    std::vector<double> out(size_t(G) * HD, 0.0), outabs(size_t(G) * HD, 0.0), l(G, 0.0);
    for (size_t k = 0; k < nk; ++k) {
      float sc;
      load_key_row(pb, t, keys[k].cached, keys[k].j, 1, kvh, rowbuf.data(), &sc);
      for (int g = 0; g < G; ++g) {
        const double w = std::exp(s[size_t(g) * nk + k] - mx[g]);
        l[g] += w;
        double* og = out.data() + size_t(g) * HD;
        double* oa = outabs.data() + size_t(g) * HD;
        for (int d = 0; d < HD; ++d) {
          const double v = double(rowbuf[d]) * double(sc);
          og[d] += w * v;
          oa[d] += w * std::fabs(v);
        }
      }
    }
    for (int g = 0; g < G; ++g) {
      const int h = kvh * G + g;
      double* dst = O64 + (size_t(ri) * p.H + h) * HD;
      for (int d = 0; d < HD; ++d) {
        double o = nk ? out[size_t(g) * HD + d] / l[g] : 0.0;
        double oa = nk ? outabs[size_t(g) * HD + d] / l[g] : 0.0;
        if (pb.X) {
          const double gate = 1.0 / (1.0 + std::exp(-double(pb.X[size_t(row) * p.g_ld + size_t(h) * 2 * HD + HD + d])));
          o *= gate;
          oa *= gate;
        }
        dst[d] = o;
        if (Oabs64) Oabs64[(size_t(ri) * p.H + h) * HD + d] = oa;
      }
      if (lse64) lse64[size_t(ri) * p.H + h] = nk ? mx[g] + std::log(l[g]) : -std::numeric_limits<double>::infinity();
    }
  });
  return bad ? -1 : 0;
}

// ------------------------------------------------------------------ flash_attention restated (fp32)
// One work unit = (tile, kv head): tile_rows query rows x G heads, 16-key blocks,
// online softmax with the -inf guards, P rounded to the 16-bit type before P.V,
// scores as one fp32 partial sum per 128 dims added in order
// (kernels/40_attention.metal:224-319). Writes the partial record when part >= 0,
// else the gated, normalised output (:321-342). With an E4M3 pool the K scale
// multiplies the score and the V scale multiplies p before it is rounded.
int orc_flash_f32(const Problem* pbp, const Tile* tiles, int32_t n_tiles, void* O, float* lse, float* parts, int threads) {
  const Problem& pb = *pbp;
  const Params& p = pb.p;
  const int HD = pb.HD, G = p.H / p.Hkv, TR = pb.tile_rows, BK = 16;
  const int pdt = pb.q_dtype;  // P takes the 16-bit type of the pass
  parallel_for(int64_t(n_tiles) * p.Hkv, threads, [&](int64_t idx) {
    const Tile& tile = tiles[idx / p.Hkv];
    const int kvh = int(idx % p.Hkv);
    const Tree& t = pb.trees[tile.tree];
    const int end = t.base + t.M;
    const int rows_live = std::min(TR, end - tile.r0);
    const int r_last = tile.r0 + rows_live - 1 - t.base;
    int anc_max = 0, seg_min = 1 << 30;
    if (pb.anc_mask) {
      anc_max = t.M, seg_min = 0;
    } else {
      for (int r = tile.r0; r <= t.base + r_last; ++r) {
        anc_max = std::max(anc_max, pb.desc[4 * size_t(r) + 2]);
        seg_min = std::min(seg_min, pb.desc[4 * size_t(r) + 0]);
      }
    }
    const int k_last = pb.anc_mask ? t.M - 1 : std::max(r_last, anc_max - 1);
    const int n_slot_blocks = (tile.k1 - tile.k0 + BK - 1) / BK;
    const int n_batch_blocks = tile.last ? (k_last + 1 + BK - 1) / BK : 0;
    const int NQ = rows_live * G;  // (row, head) pairs of the unit
    std::vector<float> kt(size_t(BK) * HD), vt(size_t(BK) * HD);
    float ks[16], vs[16];
    std::vector<float> q(size_t(NQ) * HD), acc(size_t(NQ) * HD, 0.0f), m_run(NQ, -INFINITY), l_run(NQ, 0.0f);
    for (int fm = 0; fm < rows_live; ++fm)
      for (int hg = 0; hg < G; ++hg)
        for (int d = 0; d < HD; ++d)
          q[(size_t(fm) * G + hg) * HD + d] =
              load16(pb.Q, size_t(tile.r0 + fm) * p.q_ld + size_t(kvh * G + hg) * HD + d, pb.q_dtype);
    for (int blk = 0; blk < n_slot_blocks + n_batch_blocks; ++blk) {
      const bool in_slot = blk < n_slot_blocks;
      const int j0 = in_slot ? tile.k0 + blk * BK : (blk - n_slot_blocks) * BK;
      const int j_end = in_slot ? tile.k1 : k_last + 1;
      if (!in_slot) {
        const bool anc_vis = j0 < anc_max;
        const bool own_vis = (j0 + BK - 1 >= seg_min) && (j0 <= r_last);
        if (!anc_vis && !own_vis) continue;
      }
      for (int kc = 0; kc < BK; ++kc) {
        const int j = j0 + kc;
        ks[kc] = vs[kc] = 1.0f;
        if (j < j_end) {
          load_key_row(pb, t, in_slot, j, 0, kvh, &kt[size_t(kc) * HD], &ks[kc]);
          load_key_row(pb, t, in_slot, j, 1, kvh, &vt[size_t(kc) * HD], &vs[kc]);
        } else {
          std::fill(&kt[size_t(kc) * HD], &kt[size_t(kc) * HD] + HD, 0.0f);  // zero-filled tail keys (:241-253)
          std::fill(&vt[size_t(kc) * HD], &vt[size_t(kc) * HD] + HD, 0.0f);
        }
      }
      for (int qi = 0; qi < NQ; ++qi) {
        const int fm = qi / G;
        const int row = tile.r0 + fm, rr = row - t.base;
        const float* qv = &q[size_t(qi) * HD];
        float sv[16];
        for (int kc = 0; kc < BK; ++kc) {
          const int j = j0 + kc;
          const float* kr = &kt[size_t(kc) * HD];
          float s = 0.0f;
          for (int d0 = 0; d0 < HD; d0 += 128) {
            float part = 0.0f;
            const int d1 = std::min(HD, d0 + 128);
            for (int d = d0; d < d1; ++d) part += qv[d] * kr[d];
            s = d0 == 0 ? part : s + part;
          }
          s = s * ks[kc] * pb.scale;
          bool vis = j < j_end;
          if (!in_slot) vis = vis && batch_visible(pb, row, rr, j);
          sv[kc] = vis ? s : -INFINITY;
        }
        float mx = -INFINITY;
        for (int kc = 0; kc < BK; ++kc) mx = std::max(mx, sv[kc]);
        const float m_new = std::max(m_run[qi], mx);
        const float corr = (m_new == -INFINITY) ? 1.0f : std::exp(m_run[qi] - m_new);
        float ps = 0.0f, pr[16];
        for (int kc = 0; kc < BK; ++kc) {
          const float pv = (m_new == -INFINITY) ? 0.0f : std::exp(sv[kc] - m_new);
          ps += pv;
          pr[kc] = round16(pv * vs[kc], pdt);
        }
        l_run[qi] = l_run[qi] * corr + ps;
        m_run[qi] = m_new;
        float* a = &acc[size_t(qi) * HD];
        for (int d = 0; d < HD; ++d) a[d] *= corr;
        for (int kc = 0; kc < BK; ++kc) {
          if (pr[kc] == 0.0f) continue;
          const float* vr = &vt[size_t(kc) * HD];
          for (int d = 0; d < HD; ++d) a[d] += pr[kc] * vr[d];
        }
      }
    }
    for (int qi = 0; qi < NQ; ++qi) {
      const int fm = qi / G, hg = qi % G, h = kvh * G + hg, row = tile.r0 + fm;
      const float* a = &acc[size_t(qi) * HD];
      if (tile.part >= 0) {
        float* rec = parts + ((size_t(tile.part) * p.Hkv + kvh) * TR * G + size_t(fm) * G + hg) * (HD + 2);
        for (int d = 0; d < HD; ++d) rec[d] = a[d];
        rec[HD] = m_run[qi];
        rec[HD + 1] = l_run[qi];
        continue;
      }
      const float inv_l = l_run[qi] > 0.0f ? 1.0f / l_run[qi] : 0.0f;
      for (int d = 0; d < HD; ++d) {
        float o = a[d] * inv_l;
        if (pb.X) o = o / (1.0f + std::exp(-pb.X[size_t(row) * p.g_ld + size_t(h) * 2 * HD + HD + d]));
        static_cast<uint16_t*>(O)[size_t(row) * p.q_ld + size_t(h) * HD + d] = store16(o, pb.q_dtype);
      }
      if (lse) lse[size_t(row) * p.H + h] = l_run[qi] > 0.0f ? m_run[qi] + std::log(l_run[qi]) : -INFINITY;
    }
  });
  return 0;
}

// ------------------------------------------------------------------ attn_decode_gqa restated (fp32)
// Single-row trees. Two key slices take 8-key blocks alternately, each block's
// score = (sum of the 128-dim partials) * scale in fp32, softmax without the -inf
// guards on live keys, half(p) into P.V; the slices merge as
// kernels/40_attention.metal:736-757.
int orc_decode_gqa_f32(const Problem* pbp, const Tile* tiles, int32_t n_tiles, void* O, float* lse, float* parts, int threads) {
  const Problem& pb = *pbp;
  const Params& p = pb.p;
  const int HD = pb.HD, G = p.H / p.Hkv, TR = pb.tile_rows, KP = 2;
  const int pdt = pb.q_dtype;
  parallel_for(int64_t(n_tiles) * p.Hkv, threads, [&](int64_t idx) {
    const Tile& tile = tiles[idx / p.Hkv];
    const int kvh = int(idx % p.Hkv);
    const Tree& t = pb.trees[tile.tree];
    const int row = tile.r0;
    const int n_slot = tile.k1 - tile.k0;
    const int n_keys = n_slot + (tile.last ? 1 : 0);
    // scratch of the worker thread, reused by every unit it takes (no allocation in the work loop)
    static thread_local std::vector<float> q, kt, vt, acc, m_s, l_s, out;
    q.resize(size_t(G) * HD), kt.resize(size_t(8) * HD), vt.resize(size_t(8) * HD), out.resize(size_t(HD));
    acc.assign(size_t(KP) * G * HD, 0.0f), m_s.assign(size_t(KP) * G, -INFINITY), l_s.assign(size_t(KP) * G, 0.0f);
    for (int hg = 0; hg < G; ++hg)
      for (int d = 0; d < HD; ++d)
        q[size_t(hg) * HD + d] = load16(pb.Q, size_t(row) * p.q_ld + size_t(kvh * G + hg) * HD + d, pb.q_dtype);
    for (int pr = 0; pr < KP; ++pr)
      for (int j0 = 8 * pr; j0 < n_keys; j0 += 8 * KP) {
        float ks[8], vs[8];
        for (int kc = 0; kc < 8; ++kc) {
          const int j = j0 + kc;
          ks[kc] = vs[kc] = 1.0f;
          if (j >= n_keys) {
            std::fill(&vt[size_t(kc) * HD], &vt[size_t(kc) * HD] + HD, 0.0f);
            continue;
          }
          const bool cached = j < n_slot;
          load_key_row(pb, t, cached, cached ? tile.k0 + j : 0, 0, kvh, &kt[size_t(kc) * HD], &ks[kc]);
          load_key_row(pb, t, cached, cached ? tile.k0 + j : 0, 1, kvh, &vt[size_t(kc) * HD], &vs[kc]);
        }
        for (int hg = 0; hg < G; ++hg) {
          const float* qv = &q[size_t(hg) * HD];
          float sv[8];
          for (int kc = 0; kc < 8; ++kc) {
            if (j0 + kc >= n_keys) {
              sv[kc] = -INFINITY;
              continue;
            }
            const float* kr = &kt[size_t(kc) * HD];
            float s = 0.0f;
            for (int d0 = 0; d0 < HD; d0 += 128) {
              float part = 0.0f;
              const int d1 = std::min(HD, d0 + 128);
              for (int d = d0; d < d1; ++d) part += qv[d] * kr[d];
              s = d0 == 0 ? part : s + part;
            }
            sv[kc] = s * ks[kc] * pb.scale;
          }
          float& m_run = m_s[size_t(pr) * G + hg];
          float& l_run = l_s[size_t(pr) * G + hg];
          float mx = -INFINITY;
          for (int kc = 0; kc < 8; ++kc) mx = std::max(mx, sv[kc]);
          const float m_new = std::max(m_run, mx);  // finite: key j0 is live
          const float corr = std::exp(m_run - m_new);
          float ps = 0.0f, ph[8];
          for (int kc = 0; kc < 8; ++kc) {
            const float pv = std::exp(sv[kc] - m_new);
            ps += pv;
            ph[kc] = round16(pv * vs[kc], pdt);
          }
          l_run = l_run * corr + ps;
          m_run = m_new;
          float* a = &acc[(size_t(pr) * G + hg) * HD];
          for (int d = 0; d < HD; ++d) a[d] *= corr;
          for (int kc = 0; kc < 8; ++kc) {
            if (ph[kc] == 0.0f) continue;
            const float* vr = &vt[size_t(kc) * HD];
            for (int d = 0; d < HD; ++d) a[d] += ph[kc] * vr[d];
          }
        }
      }
    for (int hg = 0; hg < G; ++hg) {
      const int h = kvh * G + hg;
      float M = m_s[hg];
      for (int s = 1; s < KP; ++s) M = std::max(M, m_s[size_t(s) * G + hg]);
      const float w0 = (m_s[hg] == -INFINITY) ? 0.0f : std::exp(m_s[hg] - M);
      float l = l_s[hg] * w0;
      for (int d = 0; d < HD; ++d) out[d] = acc[size_t(hg) * HD + d] * w0;
      for (int s = 1; s < KP; ++s) {
        const float ms = m_s[size_t(s) * G + hg];
        const float w = (ms == -INFINITY) ? 0.0f : std::exp(ms - M);
        l += w * l_s[size_t(s) * G + hg];
        for (int d = 0; d < HD; ++d) out[d] = std::fma(w, acc[(size_t(s) * G + hg) * HD + d], out[d]);
      }
      if (tile.part >= 0) {
        float* rec = parts + ((size_t(tile.part) * p.Hkv + kvh) * TR * G + hg) * (HD + 2);
        for (int d = 0; d < HD; ++d) rec[d] = out[d];
        rec[HD] = M;
        rec[HD + 1] = l;
        continue;
      }
      const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;
      for (int d = 0; d < HD; ++d) {
        float o = out[d] * inv_l;
        if (pb.X) o = o / (1.0f + std::exp(-pb.X[size_t(row) * p.g_ld + size_t(h) * 2 * HD + HD + d]));
        static_cast<uint16_t*>(O)[size_t(row) * p.q_ld + size_t(h) * HD + d] = store16(o, pb.q_dtype);
      }
      if (lse) lse[size_t(row) * p.H + h] = l > 0.0f ? M + std::log(l) : -INFINITY;
    }
  });
  return 0;
}

// ------------------------------------------------------------------ attention_combine restated (fp32)
// kernels/40_attention.metal:811-864: M = max m_s; records summed in split order;
// -inf records weigh 0; O = acc / L * sigmoid(g).
int orc_combine_f32(const float* parts, const float* X, void* O, float* lse, const Params* pp, int32_t HD, int32_t q_dtype,
                    int32_t tile_rows, const Combine* jobs, int32_t n_jobs, int threads) {
  const Params& p = *pp;
  const int G = p.H / p.Hkv, TR = tile_rows;
  const size_t stride = size_t(p.Hkv) * TR * G * (HD + 2);
  parallel_for(int64_t(n_jobs), threads, [&](int64_t ji) {
    const Combine& job = jobs[ji];
    for (int r = 0; r < job.rows; ++r)
      for (int h = 0; h < p.H; ++h) {
        const int kvh = h / G, hg = h % G;
        const float* rec0 = parts + ((size_t(job.part0) * p.Hkv + kvh) * TR * G + size_t(r) * G + hg) * (HD + 2);
        float M = -INFINITY;
        for (int s = 0; s < job.nparts; ++s) M = std::max(M, rec0[s * stride + HD]);
        float L = 0.0f;
        std::vector<float> acc(HD, 0.0f);
        for (int s = 0; s < job.nparts; ++s) {
          const float* rec = rec0 + s * stride;
          const float w = (rec[HD] == -INFINITY) ? 0.0f : std::exp(rec[HD] - M);
          L += w * rec[HD + 1];
          for (int d = 0; d < HD; ++d) acc[d] += w * rec[d];
        }
        const int row = job.r0 + r;
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;
        for (int d = 0; d < HD; ++d) {
          float o = acc[d] * inv;
          if (X) o = o / (1.0f + std::exp(-X[size_t(row) * p.g_ld + size_t(h) * 2 * HD + HD + d]));
          static_cast<uint16_t*>(O)[size_t(row) * p.q_ld + size_t(h) * HD + d] = store16(o, q_dtype);
        }
        if (lse) lse[size_t(row) * p.H + h] = L > 0.0f ? M + std::log(L) : -INFINITY;
      }
  });
  return 0;
}

// ------------------------------------------------------------------ KV writes
// kv_save (kernels/40_attention.metal:875-889). elem_bytes = 2 for 16-bit pools.
// E4M3 pools (extension): the row is divided by the destination block's scale and
// rounded to e4m3.
int orc_kv_save(const void* Kb, const void* Vb, void* kv, const float* kv_scales, const KVSave* entries, int32_t n,
                const Params* pp, int32_t HD, int32_t q_dtype, int32_t kv_dtype) {
  const Params& p = *pp;
  const uint64_t blk = uint64_t(p.bt) * p.kv_ld;
  for (int i = 0; i < n; ++i) {
    const KVSave& e = entries[i];
    const uint64_t src = uint64_t(e.src_row) * p.kv_ld;
    const uint64_t dst = p.kv_base + uint64_t(e.block) * 2 * blk + uint64_t(e.pos) * p.kv_ld;
    if (kv_dtype != ORC_E4M3) {
      std::memcpy(static_cast<uint16_t*>(kv) + dst, static_cast<const uint16_t*>(Kb) + src, size_t(p.kv_ld) * 2);
      std::memcpy(static_cast<uint16_t*>(kv) + dst + blk, static_cast<const uint16_t*>(Vb) + src, size_t(p.kv_ld) * 2);
    } else {
      for (int c = 0; c < p.kv_ld; ++c) {
        const int kvh = c / HD;
        const float sk = kv_scales[(uint64_t(e.block) * 2 + 0) * p.Hkv + kvh];
        const float sv = kv_scales[(uint64_t(e.block) * 2 + 1) * p.Hkv + kvh];
        static_cast<uint8_t*>(kv)[dst + c] = f32_to_e4m3(load16(Kb, src + c, q_dtype) / sk);
        static_cast<uint8_t*>(kv)[dst + blk + c] = f32_to_e4m3(load16(Vb, src + c, q_dtype) / sv);
      }
    }
  }
  return 0;
}

// attn_prep (kernels/40_attention.metal:23-102; generic head dim kernels/82_qwen3_omni.metal:40-88),
// restated per (row, head) in double: RMSNorm over the head, rotary embedding of the pairs
// (d, d + rot_half) at angle pos[sel[d]] * inv_freq[d] (the product in fp32, as the kernels form it),
// queries times qscale. Q64 / K64 / V64 hold the unrounded results, row-major with strides q_ld / kv_ld;
// rounding to the 16-bit output type is the caller's.
struct PrepParams {
  int32_t H, Hkv, ld, q_off, q_stride, k_off, v_off, q_ld, kv_ld, rot_half;
  float eps, qscale;
  int32_t bt, reserved;
  uint64_t kv_base;
};
int orc_attn_prep_f64(const float* X, const float* qn_w, const float* kn_w, const int32_t* pos, const float* inv_freq,
                      const int32_t* sel, double* Q64, double* K64, double* V64, int32_t rows, int32_t HD, const PrepParams* pp) {
  const PrepParams& p = *pp;
  std::vector<double> x(HD);
  for (int64_t row = 0; row < rows; ++row) {
    for (int head = 0; head < p.H + p.Hkv; ++head) {
      const bool is_q = head < p.H;
      const int h = is_q ? head : head - p.H;
      const float* src = X + row * p.ld + (is_q ? p.q_off + int64_t(h) * p.q_stride : p.k_off + int64_t(h) * HD);
      const float* nw = is_q ? qn_w : kn_w;
      double ss = 0.0;
      for (int d = 0; d < HD; ++d) ss += double(src[d]) * double(src[d]);
      const double inv = 1.0 / std::sqrt(ss / double(HD) + double(p.eps));
      for (int d = 0; d < HD; ++d) x[d] = double(src[d]) * inv * double(nw[d]);
      for (int d = 0; d < p.rot_half; ++d) {
        const int sl = sel[d];
        const float position = float(sl == 0 ? pos[4 * row] : (sl == 1 ? pos[4 * row + 1] : pos[4 * row + 2]));
        const float ang = position * inv_freq[d];
        const double c = std::cos(double(ang)), sn = std::sin(double(ang));
        const double lo = x[d], hi = x[d + p.rot_half];
        x[d] = lo * c - hi * sn;
        x[d + p.rot_half] = hi * c + lo * sn;
      }
      double* out = is_q ? Q64 + row * p.q_ld + int64_t(h) * HD : K64 + row * p.kv_ld + int64_t(h) * HD;
      const double scale = is_q ? double(p.qscale) : 1.0;
      for (int d = 0; d < HD; ++d) out[d] = x[d] * scale;
      if (!is_q) {
        const float* v = X + row * p.ld + p.v_off + int64_t(h) * HD;
        for (int d = 0; d < HD; ++d) V64[row * p.kv_ld + int64_t(h) * HD + d] = double(v[d]);
      }
    }
  }
  return 0;
}

// kv_copy_blocks (kernels/40_attention.metal:894-905).
int orc_kv_copy_blocks(void* kv, const int32_t* pairs, int32_t n_pairs, const Params* pp, uint64_t region_elems,
                       int32_t n_layers, int32_t elem_bytes) {
  const Params& p = *pp;
  const uint64_t blk2 = 2 * uint64_t(p.bt) * p.kv_ld;
  for (int l = 0; l < n_layers; ++l)
    for (int i = 0; i < n_pairs; ++i) {
      uint8_t* base = static_cast<uint8_t*>(kv) + uint64_t(l) * region_elems * elem_bytes;
      std::memmove(base + uint64_t(pairs[2 * i + 1]) * blk2 * elem_bytes, base + uint64_t(pairs[2 * i]) * blk2 * elem_bytes,
                   blk2 * elem_bytes);
    }
  return 0;
}

// ------------------------------------------------------------------ planners
// plan_tiles (src/model/impl/forest.h:1378-1433) without the sparse-attention
// branch. Returns the counts through n_tiles / n_jobs / n_parts; arrays may be
// null to size them.
int orc_plan_tiles(const Tree* trees, int32_t n_trees, int32_t Hkv, int32_t split, int32_t groups, int32_t min_chunk,
                   int32_t tile_rows, Tile* tiles, Combine* jobs, int32_t* n_tiles, int32_t* n_jobs, int32_t* n_parts) {
  const int TR = tile_rows;
  int total = 0;
  for (int i = 0; i < n_trees; ++i) total += (trees[i].M + TR - 1) / TR;
  const int budget = std::max(1, groups / std::max(1, Hkv * total));
  int nt = 0, nj = 0, np = 0;
  for (int ti = 0; ti < n_trees; ++ti) {
    const Tree& t = trees[ti];
    int ns = 1;
    if (split > 0 && budget > 1 && t.P >= 64) {
      const int chunk = std::max(std::max(32, min_chunk), std::min(split, ((t.P + budget - 1) / budget + 31) / 32 * 32));
      ns = std::min({(t.P + chunk - 1) / chunk, budget, 64});
    }
    for (int r = 0; r < t.M; r += TR) {
      if (ns == 1) {
        if (tiles) tiles[nt] = Tile{ti, t.base + r, 0, t.P, -1, 1, 0, 0};
        ++nt;
        continue;
      }
      const int per = (t.P + ns - 1) / ns;
      const int step = (per + 31) / 32 * 32;
      const int part0 = np;
      int used = 0;
      for (int k = 0; k < t.P; k += step, ++used) {
        const int k1 = std::min(t.P, k + step);
        if (tiles) tiles[nt] = Tile{ti, t.base + r, k, k1, np, k1 >= t.P ? 1 : 0, 0, 0};
        ++nt;
        ++np;
      }
      if (jobs) jobs[nj] = Combine{t.base + r, std::min(TR, t.M - r), part0, used};
      ++nj;
    }
  }
  *n_tiles = nt;
  *n_jobs = nj;
  *n_parts = np;
  return 0;
}

// g4_plan_tiles with window = 0 (src/model/impl/gemma.h:77-116): min_chunk fixed
// at 32, tiles of `rows` rows only when nothing is split (budget == 1), else 8.
// g4_plan_tiles (src/model/impl/gemma.h:77-116) with its window branch: a sliding tile starts at the
// first key any of its rows can see (k0) and records the first batch key to scan (b0, in pad0).
int orc_g4_plan_tiles(const Tree* trees, int32_t n_trees, int32_t groups, int32_t split, int32_t rows, int32_t window,
                      const int32_t* pos, Tile* tiles, Combine* jobs, int32_t* n_tiles, int32_t* n_jobs, int32_t* n_parts,
                      int32_t* plan_rows) {
  int total = 0;
  for (int i = 0; i < n_trees; ++i) total += (trees[i].M + 7) / 8;
  const int budget = std::max(1, 256 / std::max(1, groups * total));
  const int TR = budget == 1 ? rows : 8;
  int nt = 0, nj = 0, np = 0;
  for (int ti = 0; ti < n_trees; ++ti) {
    const Tree& t = trees[ti];
    for (int r = 0; r < t.M; r += TR) {
      int k0 = 0, b0 = 0;
      if (window > 0) {
        int minpos = std::numeric_limits<int32_t>::max();
        for (int i = r; i < std::min(t.M, r + TR); ++i) minpos = std::min(minpos, pos[4 * (t.base + i)]);
        k0 = std::clamp(minpos - window + 1, 0, t.P);
        b0 = std::max(0, minpos - window + 1 - t.P);
      }
      const int span = t.P - k0;
      int ns = 1;
      if (split > 0 && budget > 1 && span >= 64) {
        const int chunk = std::max(32, std::min(split, ((span + budget - 1) / budget + 31) / 32 * 32));
        ns = std::min({(span + chunk - 1) / chunk, budget, 64});
      }
      if (ns == 1) {
        if (tiles) tiles[nt] = Tile{ti, t.base + r, k0, t.P, -1, 1, b0, 0};
        ++nt;
        continue;
      }
      const int per = (span + ns - 1) / ns;
      const int step = (per + 31) / 32 * 32;
      const int part0 = np;
      int used = 0;
      for (int k = k0; k < t.P; k += step, ++used) {
        const int k1 = std::min(t.P, k + step);
        if (tiles) tiles[nt] = Tile{ti, t.base + r, k, k1, np, k1 >= t.P ? 1 : 0, b0, 0};
        ++nt;
        ++np;
      }
      if (jobs) jobs[nj] = Combine{t.base + r, std::min(8, t.M - r), part0, used};
      ++nj;
    }
  }
  *n_tiles = nt;
  *n_jobs = nj;
  *n_parts = np;
  *plan_rows = TR;
  return 0;
}

// Host threads this process may run on: the affinity mask (a container's share of the box), not the
// machine's core count.
int orc_hw_threads(void) {
#if defined(__linux__)
  cpu_set_t set;
  CPU_ZERO(&set);
  if (sched_getaffinity(0, sizeof(set), &set) == 0 && CPU_COUNT(&set) > 0) return CPU_COUNT(&set);
#endif
  return int(std::max(1u, std::thread::hardware_concurrency()));
}

}  // extern "C"
