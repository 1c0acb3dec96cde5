// Integer tile planner of the attention pass (host only).
//
// ESP_PLAN_REFERENCE reproduces plan_tiles of the reference bit for bit
// (src/model/impl/forest.h:1378-1433, without its sparse-attention branch),
// ESP_PLAN_G4 reproduces g4_plan_tiles with no window (src/model/impl/gemma.h:77-116),
// ESP_PLAN_B200 emits the same records with one chunk size for the whole pass, chosen so
// that (kv head, tile) CTAs of near-equal length fill `groups` CTA slots.
#include <algorithm>
#include <climits>
#include <cstdint>

#include "../../include/espetero_attn.h"
#include "host_util.h"

namespace {

struct Emitter {
  esp_attn_tile* tiles;
  int32_t tiles_cap;
  esp_attn_combine* jobs;
  int32_t jobs_cap;
  bool tag_jobs = false;  // ESP_PLAN_B200: a split tile carries 1 + the index of its combine job in pad1
  int32_t nt = 0, nj = 0, np = 0;
  void tile(const esp_attn_tile& t) {
    if (tiles && nt < tiles_cap) tiles[nt] = t;
    ++nt;
  }
  void job(const esp_attn_combine& j) {
    if (jobs && nj < jobs_cap) jobs[nj] = j;
    ++nj;
  }
  // One row group [r, r + rows) of tree ti over its cached keys, cut into `ns` near-equal
  // ranges whose boundaries are multiples of 32 keys (forest.h:1414-1429).
  void group(int32_t ti, const esp_attn_tree& t, int32_t r, int32_t rows_in_job, int32_t ns) {
    if (ns <= 1) {
      tile({ti, t.base + r, 0, t.P, -1, 1, 0, 0});
      return;
    }
    const int32_t per = (t.P + ns - 1) / ns;
    const int32_t step = (per + 31) / 32 * 32;
    const int32_t part0 = np;
    int32_t used = 0;
    for (int32_t k = 0; k < t.P; k += step, ++used) {
      const int32_t k1 = std::min(t.P, k + step);
      tile({ti, t.base + r, k, k1, np++, k1 >= t.P ? 1 : 0, 0, tag_jobs ? nj + 1 : 0});
    }
    job({t.base + r, rows_in_job, part0, used});
  }
};

inline int32_t ceil_div(int64_t a, int64_t b) { return int32_t((a + b - 1) / b); }

}  // namespace

static int plan_impl(const esp_attn_tree* trees, int32_t n_trees, int32_t Hkv, const esp_plan_opts* opts, const int32_t* qt,
                     esp_attn_tile* tiles, int32_t tiles_cap, esp_attn_combine* jobs, int32_t jobs_cap,
                     int32_t* n_tiles, int32_t* n_jobs, int32_t* n_parts);

extern "C" int esp_attn_plan(const esp_attn_tree* trees, int32_t n_trees, int32_t Hkv, const esp_plan_opts* opts,
                             esp_attn_tile* tiles, int32_t tiles_cap, esp_attn_combine* jobs, int32_t jobs_cap,
                             int32_t* n_tiles, int32_t* n_jobs, int32_t* n_parts) {
  return plan_impl(trees, n_trees, Hkv, opts, nullptr, tiles, tiles_cap, jobs, jobs_cap, n_tiles, n_jobs, n_parts);
}

// plan_tiles with its sparse-attention branch (forest.h:1392-1412): qt = per tree, per 8-row group, the union list of the
// group or -1 (flattened).
extern "C" int esp_attn_plan_qsa(const esp_attn_tree* trees, int32_t n_trees, int32_t Hkv, const esp_plan_opts* opts, const int32_t* qt,
                                 esp_attn_tile* tiles, int32_t tiles_cap, esp_attn_combine* jobs, int32_t jobs_cap, int32_t* n_tiles,
                                 int32_t* n_jobs, int32_t* n_parts) {
  if (qt && opts && (opts->mode != ESP_PLAN_REFERENCE || (opts->tile_rows != 0 && opts->tile_rows != 8)))
    return esp::fail(ESP_ERR_UNSUPPORTED, "esp_attn_plan_qsa: sparse groups are planned by the reference planner with 8-row tiles");
  return plan_impl(trees, n_trees, Hkv, opts, qt, tiles, tiles_cap, jobs, jobs_cap, n_tiles, n_jobs, n_parts);
}

static int plan_impl(const esp_attn_tree* trees, int32_t n_trees, int32_t Hkv, const esp_plan_opts* opts, const int32_t* qt,
                     esp_attn_tile* tiles, int32_t tiles_cap, esp_attn_combine* jobs, int32_t jobs_cap,
                     int32_t* n_tiles, int32_t* n_jobs, int32_t* n_parts) {
  if (!opts || (!trees && n_trees > 0) || n_trees < 0 || Hkv <= 0 || !n_tiles || !n_jobs || !n_parts)
    return esp::fail(ESP_ERR_INVALID, "esp_attn_plan: null or negative argument");
  const int32_t mode = opts->mode;
  if (mode != ESP_PLAN_REFERENCE && mode != ESP_PLAN_G4 && mode != ESP_PLAN_B200)
    return esp::fail(ESP_ERR_INVALID, "esp_attn_plan: unknown mode %d", mode);
  for (int32_t i = 0; i < n_trees; ++i)
    if (trees[i].P < 0 || trees[i].M < 0 || trees[i].base < 0)
      return esp::fail(ESP_ERR_INVALID, "esp_attn_plan: tree %d has a negative field", i);
  const int32_t groups = opts->groups > 0 ? opts->groups : 256;
  const int32_t split = opts->split;
  const int32_t max_parts = opts->max_parts > 0 ? opts->max_parts : 64;
  int32_t TR = opts->tile_rows > 0 ? opts->tile_rows : 8;
  Emitter E{tiles, tiles ? tiles_cap : 0, jobs, jobs ? jobs_cap : 0};

  if (mode == ESP_PLAN_REFERENCE || mode == ESP_PLAN_G4) {
    const int32_t min_chunk = mode == ESP_PLAN_G4 ? 32 : opts->min_chunk;
    // Both reference planners count 8-row groups for the budget; the G4 planner widens its
    // tiles to `tile_rows` only when nothing is split (gemma.h:84).
    const int32_t count_rows = mode == ESP_PLAN_G4 ? 8 : TR;
    int64_t total = 0;
    for (int32_t i = 0; i < n_trees; ++i) total += (trees[i].M + count_rows - 1) / count_rows;
    const int32_t budget = int32_t(std::max<int64_t>(1, groups / std::max<int64_t>(1, int64_t(Hkv) * total)));
    if (mode == ESP_PLAN_G4 && budget != 1) TR = 8;
    size_t qt_at = 0;
    for (int32_t ti = 0; ti < n_trees; ++ti) {
      const esp_attn_tree& t = trees[ti];
      int32_t ns = 1;
      if (split > 0 && budget > 1 && t.P >= 64) {
        const int32_t chunk = std::max(std::max(32, min_chunk), std::min(split, (ceil_div(t.P, budget) + 31) / 32 * 32));
        ns = std::min({ceil_div(t.P, chunk), budget, 64});
      }
      for (int32_t r = 0; r < t.M; r += TR) {
        const int32_t q = qt ? qt[qt_at + r / 8] : -1;
        if (q < 0) {
          E.group(ti, t, r, std::min(mode == ESP_PLAN_G4 ? 8 : TR, t.M - r), ns);
          continue;
        }
        // A group with rows past the dense range reads the entries of union list q (4 keys each; its length is known
        // only on the device: splits assume 513 entries for one row and 128 more per further row, the last part is open).
        const int32_t rows = std::min(8, t.M - r);
        const int32_t est = 516 + 128 * (rows - 1);
        int32_t nq = 1;
        if (split > 0 && budget > 1) {
          const int32_t chunk = std::max(16, std::min(split / 4, (ceil_div(est, budget) + 3) / 4 * 4));
          nq = std::min({ceil_div(est, chunk), budget, 64});
        }
        if (nq == 1) {
          E.tile({ti, t.base + r, 0, 1 << 30, -1, 1, 1, q});
          continue;
        }
        const int32_t step = (ceil_div(est, nq) + 3) / 4 * 4;
        const int32_t part0 = E.np;
        for (int32_t k = 0; k < nq; ++k) {
          const bool lastp = k + 1 == nq;
          E.tile({ti, t.base + r, k * step, lastp ? (1 << 30) : (k + 1) * step, E.np++, lastp ? 1 : 0, 1, q});
        }
        E.job({t.base + r, rows, part0, nq});
      }
      if (qt) qt_at += (t.M + 7) / 8;
    }
  } else {
    E.tag_jobs = true;
    // One chunk size for the pass: total (row group x key) work spread over the CTA slots.
    int64_t work = 0, n_groups = 0;
    for (int32_t i = 0; i < n_trees; ++i) {
      const int64_t rg = (trees[i].M + TR - 1) / TR;
      n_groups += rg;
      work += rg * trees[i].P;
    }
    const int64_t slots = std::max<int64_t>(1, groups / Hkv);
    int32_t chunk = 0;  // 0: no splitting
    if (split > 0 && n_groups < slots) {
      const int64_t want = (ceil_div(work, slots) + 31) / 32 * 32;
      chunk = int32_t(std::clamp<int64_t>(want, std::max(32, opts->min_chunk), std::max(32, split)));
      // One wave: grow the chunk until the tiles fit the slots (a few tiles over the slot count
      // would cost a whole second wave).
      const auto tiles_at = [&](int32_t c) {
        int64_t n = 0;
        for (int32_t i = 0; i < n_trees; ++i) {
          const int64_t rg = (trees[i].M + TR - 1) / TR;
          n += rg * (trees[i].P >= 64 ? std::min<int64_t>(ceil_div(trees[i].P, c), max_parts) : 1);
        }
        return n;
      };
      while (chunk < std::max(32, split) && tiles_at(chunk) > slots) chunk += 32;
    }
    for (int32_t ti = 0; ti < n_trees; ++ti) {
      const esp_attn_tree& t = trees[ti];
      int32_t ns = 1;
      if (chunk > 0 && t.P >= 64) ns = std::min(ceil_div(t.P, chunk), max_parts);
      for (int32_t r = 0; r < t.M; r += TR) E.group(ti, t, r, std::min(TR, t.M - r), ns);
    }
  }
  *n_tiles = E.nt;
  *n_jobs = E.nj;
  *n_parts = E.np;
  if ((tiles && E.nt > tiles_cap) || (jobs && E.nj > jobs_cap))
    return esp::fail(ESP_ERR_CAPACITY, "esp_attn_plan: needs %d tiles and %d jobs", E.nt, E.nj);
  return ESP_OK;
}

// The generic planner with its window branch (src/model/impl/gemma.h:77-116). Budget and tile height
// as in ESP_PLAN_G4; per row group the cached range starts at the first key a row of the group can
// see, and the first batch key worth scanning travels in pad0.
extern "C" int esp_attn_plan_window(const esp_attn_tree* trees, int32_t n_trees, int32_t groups, int32_t split, int32_t rows,
                                    int32_t window, const int32_t* pos, esp_attn_tile* tiles, int32_t tiles_cap,
                                    esp_attn_combine* jobs, int32_t jobs_cap, int32_t* n_tiles, int32_t* n_jobs, int32_t* n_parts,
                                    int32_t* plan_rows) {
  if ((!trees && n_trees > 0) || n_trees < 0 || groups <= 0 || rows <= 0 || window < 0 || !n_tiles || !n_jobs || !n_parts || !plan_rows)
    return esp::fail(ESP_ERR_INVALID, "esp_attn_plan_window: null or negative argument");
  if (window > 0 && !pos) return esp::fail(ESP_ERR_INVALID, "esp_attn_plan_window: a window needs the rows' positions");
  for (int32_t i = 0; i < n_trees; ++i)
    if (trees[i].P < 0 || trees[i].M < 0 || trees[i].base < 0)
      return esp::fail(ESP_ERR_INVALID, "esp_attn_plan_window: tree %d has a negative field", i);
  int64_t row_groups = 0;
  for (int32_t i = 0; i < n_trees; ++i) row_groups += (trees[i].M + 7) / 8;
  const int32_t budget = int32_t(std::max<int64_t>(1, 256 / std::max<int64_t>(1, int64_t(groups) * row_groups)));
  const int32_t TR = budget == 1 ? rows : 8;
  int32_t nt = 0, nj = 0, np = 0;
  auto put_tile = [&](const esp_attn_tile& t) {
    if (tiles && nt < tiles_cap) tiles[nt] = t;
    ++nt;
  };
  for (int32_t ti = 0; ti < n_trees; ++ti) {
    const esp_attn_tree& t = trees[ti];
    for (int32_t r = 0; r < t.M; r += TR) {
      int32_t first_key = 0, first_batch = 0;
      if (window > 0) {
        int32_t lowest = INT32_MAX;  // the earliest query position of the group decides what is still visible
        for (int32_t i = r; i < std::min(t.M, r + TR); ++i) lowest = std::min(lowest, pos[4 * size_t(t.base + i)]);
        const int64_t start = int64_t(lowest) - window + 1;
        first_key = int32_t(std::clamp<int64_t>(start, 0, t.P));
        first_batch = int32_t(std::max<int64_t>(0, start - t.P));
      }
      const int32_t span = t.P - first_key;
      int32_t pieces = 1;
      if (split > 0 && budget > 1 && span >= 64) {
        const int32_t chunk = std::max(32, std::min(split, (ceil_div(span, budget) + 31) / 32 * 32));
        pieces = std::min({ceil_div(span, chunk), budget, 64});
      }
      if (pieces == 1) {
        put_tile({ti, t.base + r, first_key, t.P, -1, 1, first_batch, 0});
        continue;
      }
      const int32_t step = (ceil_div(span, pieces) + 31) / 32 * 32;
      const int32_t part0 = np;
      int32_t used = 0;
      for (int32_t k = first_key; k < t.P; k += step, ++used) {
        const int32_t k1 = std::min(t.P, k + step);
        put_tile({ti, t.base + r, k, k1, np++, k1 >= t.P ? 1 : 0, first_batch, 0});
      }
      if (jobs && nj < jobs_cap) jobs[nj] = {t.base + r, std::min(8, t.M - r), part0, used};
      ++nj;
    }
  }
  *n_tiles = nt, *n_jobs = nj, *n_parts = np, *plan_rows = TR;
  if ((tiles && nt > tiles_cap) || (jobs && nj > jobs_cap))
    return esp::fail(ESP_ERR_CAPACITY, "esp_attn_plan_window: needs %d tiles and %d jobs", nt, nj);
  return ESP_OK;
}

extern "C" size_t esp_attn_parts_floats(const esp_attn_shape* s, int32_t n_parts) {
  if (!s || s->Hkv <= 0 || n_parts <= 0) return 0;
  const int32_t TR = s->tile_rows > 0 ? s->tile_rows : 8;
  return size_t(n_parts) * size_t(s->Hkv) * size_t(TR) * size_t(s->H / s->Hkv) * size_t(s->HD + 2);
}
