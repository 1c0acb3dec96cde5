// Host-side integer logic around the attention op: the refcounted KV block pool, the block
// lists of a pass's targets (shared prefix, new blocks, copy-on-write pairs), the kv_save
// entries and per-row pool table, and the per-row tree metadata (leaf hosting, positions,
// the `desc` mask records) that the kernels consume.
//
// Reference: KVPool / kv_alloc / kv_retain / kv_release (src/model/impl/model.h:387-411,
// :722-737; pool set-up forest.h:51-62), Forest::target_blocks and target_new_blocks
// (src/model/impl/forest.h:1785-1829), the save entries (forest.h:2488-2499), kv_row_table
// (forest.h:1739-1749), leaf hosting (forest.h:2201-2220) and the row records
// (forest.h:2374-2442). Everything here is integer work and must match bit for bit.
#include <algorithm>
#include <cstring>
#include <vector>

#include "../../include/espetero_attn.h"
#include "host_util.h"

using esp::fail;

struct esp_kv_pool {
  int32_t bt = 0;
  int32_t n_blocks = 0;
  std::vector<int32_t> ref;
  std::vector<int32_t> free_list;
};

extern "C" {

int esp_kv_pool_create(esp_kv_pool** out, int32_t n_blocks, int32_t bt) {
  if (!out || n_blocks <= 0 || bt <= 0) return fail(ESP_ERR_INVALID, "esp_kv_pool_create: n_blocks=%d bt=%d", n_blocks, bt);
  auto* p = new esp_kv_pool;
  p->bt = bt;
  p->n_blocks = n_blocks;
  p->ref.assign(size_t(n_blocks), 0);
  p->free_list.reserve(size_t(n_blocks));
  for (int32_t b = n_blocks - 1; b >= 0; --b) p->free_list.push_back(b);  // block 0 is handed out first
  *out = p;
  return ESP_OK;
}

int esp_kv_pool_destroy(esp_kv_pool* p) {
  delete p;
  return ESP_OK;
}

int32_t esp_kv_free_count(const esp_kv_pool* p) { return p ? int32_t(p->free_list.size()) : 0; }

int32_t esp_kv_refcount(const esp_kv_pool* p, int32_t block) {
  return (p && block >= 0 && block < p->n_blocks) ? p->ref[size_t(block)] : -1;
}

int esp_kv_alloc(esp_kv_pool* p, int32_t* block) {
  if (!p || !block) return fail(ESP_ERR_INVALID, "esp_kv_alloc: null argument");
  if (p->free_list.empty()) return fail(ESP_ERR_CAPACITY, "KV cache full (raise kv_bytes or lower concurrency)");
  const int32_t b = p->free_list.back();
  p->free_list.pop_back();
  p->ref[size_t(b)] = 1;
  *block = b;
  return ESP_OK;
}

int esp_kv_retain(esp_kv_pool* p, int32_t block) {
  if (!p || block < 0 || block >= p->n_blocks || p->ref[size_t(block)] <= 0)
    return fail(ESP_ERR_INVALID, "esp_kv_retain: block %d is not live", block);
  ++p->ref[size_t(block)];
  return ESP_OK;
}

int esp_kv_release(esp_kv_pool* p, int32_t block) {
  if (!p || block < 0 || block >= p->n_blocks || p->ref[size_t(block)] <= 0)
    return fail(ESP_ERR_INVALID, "esp_kv_release: block %d is not live", block);
  if (--p->ref[size_t(block)] == 0) p->free_list.push_back(block);
  return ESP_OK;
}

int32_t esp_kv_target_new_blocks(const esp_kv_pool* p, const int32_t* parent_blocks, int32_t n_parent, int32_t P, int32_t w0,
                                 int32_t end, int32_t in_place) {
  if (!p) return 0;
  const int32_t bt = p->bt, first = w0 / bt;
  int32_t n = (end + bt - 1) / bt - first;
  const bool keeps_partial = n > 0 && in_place && parent_blocks && first < n_parent && first * bt < P &&
                             p->ref[size_t(parent_blocks[first])] == 1;
  if (keeps_partial) --n;
  return std::max(n, 0);
}

int esp_kv_target_blocks(esp_kv_pool* p, const int32_t* parent_blocks, int32_t n_parent, int32_t P, int32_t w0, int32_t end,
                         int32_t in_place, int32_t* out_blocks, int32_t out_cap, int32_t* n_out, int32_t* cow_pairs,
                         int32_t cow_cap, int32_t* n_cow) {
  if (!p || !n_out || !n_cow || (n_parent > 0 && !parent_blocks) || P < 0 || w0 < 0 || end < 0)
    return fail(ESP_ERR_INVALID, "esp_kv_target_blocks: bad argument");
  const int32_t bt = p->bt;
  const int32_t shared = std::min(w0 / bt, n_parent);  // blocks entirely below w0
  const int32_t total = shared + std::max((end + bt - 1) / bt - w0 / bt, 0);
  if (total > out_cap || !out_blocks) {
    *n_out = total;
    *n_cow = total - shared;
    return fail(ESP_ERR_CAPACITY, "esp_kv_target_blocks: the list needs %d entries", total);
  }
  // Count what has to be allocated before touching the pool, so that a full cache leaves it unchanged.
  int32_t fresh = 0;
  for (int32_t i = w0 / bt; i < (end + bt - 1) / bt; ++i) {
    const bool from_parent = i < n_parent && i * bt < P;
    if (!(from_parent && in_place && p->ref[size_t(parent_blocks[i])] == 1)) ++fresh;
  }
  if (fresh > int32_t(p->free_list.size())) return fail(ESP_ERR_CAPACITY, "KV cache full (raise kv_bytes or lower concurrency)");
  int32_t no = 0, nc = 0;
  for (int32_t i = 0; i < shared; ++i) {
    out_blocks[no++] = parent_blocks[i];
    ++p->ref[size_t(parent_blocks[i])];
  }
  for (int32_t i = w0 / bt; i < (end + bt - 1) / bt; ++i) {
    // Every parent position below P is valid: a block that also holds some of them is either
    // kept (an in-place append that owns it alone) or copied into the new block first.
    const bool from_parent = i < n_parent && i * bt < P;
    if (from_parent && in_place && p->ref[size_t(parent_blocks[i])] == 1) {
      out_blocks[no++] = parent_blocks[i];
      ++p->ref[size_t(parent_blocks[i])];
      continue;
    }
    int32_t nb = -1;
    esp_kv_alloc(p, &nb);
    if (from_parent) {
      if (cow_pairs && nc < cow_cap) cow_pairs[2 * nc] = parent_blocks[i], cow_pairs[2 * nc + 1] = nb;
      ++nc;
    }
    out_blocks[no++] = nb;
  }
  *n_out = no;
  *n_cow = nc;
  if (nc > cow_cap && cow_pairs) return fail(ESP_ERR_CAPACITY, "esp_kv_target_blocks: %d copy-on-write pairs", nc);
  return ESP_OK;
}

int esp_kv_save_entries(const int32_t* blocks, int32_t n_blocks_list, int32_t bt, int32_t P, int32_t base_row, int32_t n_rows,
                        esp_kv_save_entry* out) {
  if (n_rows <= 0) return ESP_OK;
  if (!blocks || !out || bt <= 0 || P < 0) return fail(ESP_ERR_INVALID, "esp_kv_save_entries: bad argument");
  if ((P + n_rows + bt - 1) / bt > n_blocks_list) return fail(ESP_ERR_INVALID, "esp_kv_save_entries: block list too short for %d positions", P + n_rows);
  for (int32_t i = 0; i < n_rows; ++i) {
    const int32_t pos = P + i;
    out[i] = esp_kv_save_entry{base_row + i, blocks[pos / bt], pos % bt, 0};
  }
  return ESP_OK;
}

int esp_kv_row_table(const esp_kv_save_entry* entries, int32_t n, int32_t rows, int32_t* table) {
  if (!table || rows < 0 || (n > 0 && !entries)) return fail(ESP_ERR_INVALID, "esp_kv_row_table: bad argument");
  std::fill(table, table + size_t(std::max(rows, 1)) * 4, -1);
  for (int32_t i = 0; i < n; ++i) {
    const esp_kv_save_entry& e = entries[i];
    if (e.src_row < 0 || e.src_row >= rows) return fail(ESP_ERR_INVALID, "esp_kv_row_table: entry %d names row %d of %d", i, e.src_row, rows);
    int32_t* t = table + size_t(e.src_row) * 4;
    const int slot = t[0] < 0 ? 0 : 2;
    if (slot == 2 && t[2] >= 0) return fail(ESP_ERR_INVALID, "a row saved into more than two slots");
    t[slot] = e.block;
    t[slot + 1] = e.pos;
  }
  return ESP_OK;
}

int esp_forest_tree_rows(const esp_tree_spec* spec, int32_t base, int32_t pnext, int32_t* host, int32_t* off, int32_t* tok,
                         int32_t* pos4, int32_t* desc4, int32_t* readout_rows, int32_t rows_cap, int32_t* n_rows,
                         int32_t* next_root) {
  if (!spec || !n_rows) return fail(ESP_ERR_INVALID, "esp_forest_tree_rows: null argument");
  const esp_tree_spec& b = *spec;
  const int32_t Tr = b.root_len, NL = b.n_leaves;
  if (Tr <= 0 || !b.root) return fail(ESP_ERR_INVALID, "a tree needs a root");
  if (NL > 0 && (!b.leaf_offsets || !b.leaf_tokens || !host || !off)) return fail(ESP_ERR_INVALID, "esp_forest_tree_rows: leaves without arrays");
  if (b.noncausal && NL > 0) return fail(ESP_ERR_INVALID, "a noncausal root stands on its own");
  const auto len_of = [&](int32_t i) { return b.leaf_offsets[i + 1] - b.leaf_offsets[i]; };
  for (int32_t i = 0; i < NL; ++i)
    if (len_of(i) <= 0) return fail(ESP_ERR_INVALID, "every leaf needs a token");
  // A leaf whose tokens are a prefix of another leaf is read from that leaf's rows: the host is
  // the longest such leaf, the lowest index among equals.
  int32_t leaf_rows = 0;
  for (int32_t i = 0; i < NL; ++i) {
    int32_t h = i;
    const int32_t* ti = b.leaf_tokens + b.leaf_offsets[i];
    for (int32_t j = 0; j < NL; ++j) {
      if (j == i) continue;
      const int32_t lj = len_of(j), li = len_of(i), lh = len_of(h);
      if (lj < li || (lj == li && j > i)) continue;         // not a host candidate for i
      if (lj < lh || (lj == lh && j >= h)) continue;        // not better than the current host
      if (std::equal(ti, ti + li, b.leaf_tokens + b.leaf_offsets[j])) h = j;
    }
    host[i] = h;
  }
  for (int32_t i = 0; i < NL; ++i) {
    off[i] = 0;
    if (host[i] == i) {
      off[i] = leaf_rows;
      leaf_rows += len_of(i);
    }
  }
  const int32_t M = Tr + leaf_rows;
  *n_rows = M;
  if (M > rows_cap || !pos4 || !desc4) return fail(ESP_ERR_CAPACITY, "esp_forest_tree_rows: the tree has %d rows", M);
  int32_t pmax = pnext - 1;
  for (int32_t j = 0; j < Tr; ++j) {
    int32_t pt = pnext + j, ph = pt, pw = pt;
    if (b.root_pos) pt = b.root_pos[3 * j], ph = b.root_pos[3 * j + 1], pw = b.root_pos[3 * j + 2];
    int32_t* ps = pos4 + 4 * size_t(j);
    ps[0] = pt, ps[1] = ph, ps[2] = pw, ps[3] = 0;
    pmax = std::max(pmax, std::max(pt, std::max(ph, pw)));
    int32_t* d = desc4 + 4 * size_t(j);
    d[0] = 0, d[1] = 0, d[2] = b.noncausal ? Tr : 0, d[3] = 0;  // a noncausal root row sees the whole root
    if (tok) tok[j] = b.root[j];
  }
  const int32_t nr = pmax + 1;
  if (next_root) *next_root = nr;
  int32_t n_read = 0;
  for (int32_t i = 0; i < NL; ++i) {
    const int32_t h = host[i], start = Tr + off[h], len = len_of(i);
    if (readout_rows) readout_rows[n_read] = base + start + len - 1;
    ++n_read;
    if (h != i) continue;
    for (int32_t j = 0; j < len; ++j) {
      const int32_t r = start + j;
      int32_t* ps = pos4 + 4 * size_t(r);
      ps[0] = ps[1] = ps[2] = nr + j, ps[3] = 0;
      int32_t* d = desc4 + 4 * size_t(r);
      d[0] = start, d[1] = 0, d[2] = Tr, d[3] = 0;  // sees the whole root and its own segment up to itself
      if (tok) tok[r] = b.leaf_tokens[b.leaf_offsets[i] + j];
    }
  }
  if (readout_rows && (b.score_root || NL == 0)) readout_rows[n_read] = base + Tr - 1;  // the root's readout comes last
  return ESP_OK;
}

int esp_forest_anc_masks(const int32_t* parents, int32_t n, uint64_t* masks) {
  if (n < 0 || n > 64 || (n > 0 && (!parents || !masks))) return fail(ESP_ERR_INVALID, "esp_forest_anc_masks: 0..64 nodes");
  for (int32_t i = 0; i < n; ++i) {
    if (parents[i] >= i || parents[i] < -1) return fail(ESP_ERR_INVALID, "node %d: parent %d must precede it", i, parents[i]);
    masks[i] = (uint64_t(1) << i) | (parents[i] >= 0 ? masks[parents[i]] : 0);
  }
  return ESP_OK;
}

}  // extern "C"
