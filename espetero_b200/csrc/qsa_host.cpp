// Qwen sparse attention, host side (no GPU needed): the per-row records, sparse rows and 8-row tiles of a pass.
// Reference: qsa_plan, src/model/impl/forest.h:1489-1543. Per row its sequence index s (the tree's cached keys, then
// the row's path: the root rows, then its own segment) and nb = (s + 1) / 4 complete blocks of 4 tokens; a row is
// sparse once nb > 512 (the top-k budget). Tiles are the 8-row groups of the attention plan that hold a sparse row.
#include <algorithm>
#include <cstdint>
#include <vector>

#include "../../include/espetero_attn.h"
#include "host_util.h"

extern "C" int esp_qsa_plan(const esp_attn_tree* trees, int32_t n_trees, const int32_t* desc, int32_t sparse, int32_t* rinfo, int32_t rows_cap,
                            int32_t* srows, int32_t srows_cap, esp_qsa_tile* qtiles, int32_t qtiles_cap, int32_t* qt_of, int32_t qt_cap,
                            esp_qsa_counts* counts) {
  if ((!trees && n_trees > 0) || n_trees < 0 || !counts) return esp::fail(ESP_ERR_INVALID, "esp_qsa_plan: null or negative argument");
  esp_qsa_counts c{};
  int64_t n_groups_all = 0;
  for (int32_t i = 0; i < n_trees; ++i) {
    if (trees[i].base < 0 || trees[i].M < 0 || trees[i].P < 0) return esp::fail(ESP_ERR_INVALID, "esp_qsa_plan: tree %d has a negative field", i);
    c.M = std::max(c.M, trees[i].base + trees[i].M);
    n_groups_all += (trees[i].M + 7) / 8;
  }
  const bool rows_fit = rinfo && rows_cap >= c.M, groups_fit = qt_of && qt_cap >= n_groups_all;
  if (rows_fit) std::fill(rinfo, rinfo + size_t(c.M) * 4, 0);
  std::vector<int32_t> tile_of;  // of the current tree's 8-row groups
  int64_t qt_at = 0;
  for (int32_t ti = 0; ti < n_trees; ++ti) {
    const esp_attn_tree& T = trees[ti];
    tile_of.assign(size_t((T.M + 7) / 8), -1);
    for (int32_t rr = 0; rr < T.M; ++rr) {
      const int32_t r = T.base + rr;
      const int32_t sidx = T.P + (desc ? desc[4 * size_t(r) + 2] + (rr - desc[4 * size_t(r)]) : rr);
      const int32_t nb = (sidx + 1) / 4;
      const bool sp = sparse != 0 && nb > ESP_QSA_TOPK;
      if (rows_fit) {
        int32_t* ri = rinfo + 4 * size_t(r);
        ri[0] = sidx, ri[1] = nb, ri[2] = sp ? c.n_sparse : -1, ri[3] = ti;
      }
      if (!sp) continue;
      if (srows && c.n_sparse < srows_cap) srows[c.n_sparse] = r;
      ++c.n_sparse;
      c.nbmax = std::max(c.nbmax, nb);
      c.nbb = std::max(c.nbb, nb - T.P / 4);
      c.ncb = std::max(c.ncb, T.P / 4);
      int32_t& g = tile_of[size_t(rr / 8)];
      if (g < 0) {  // the group's tile is created by its first sparse row
        g = c.n_tiles;
        if (qtiles && c.n_tiles < qtiles_cap) qtiles[c.n_tiles] = esp_qsa_tile{ti, T.base + rr / 8 * 8, std::min(8, T.M - rr / 8 * 8), 0};
        ++c.n_tiles;
      }
    }
    if (groups_fit) std::copy(tile_of.begin(), tile_of.end(), qt_of + qt_at);
    qt_at += int64_t(tile_of.size());
  }
  *counts = c;
  if ((rinfo && !rows_fit) || (qt_of && !groups_fit) || (srows && c.n_sparse > srows_cap) || (qtiles && c.n_tiles > qtiles_cap))
    return esp::fail(ESP_ERR_CAPACITY, "esp_qsa_plan: needs %d rows, %d sparse rows, %d tiles, %lld groups", c.M, c.n_sparse, c.n_tiles, (long long)qt_at);
  return ESP_OK;
}
