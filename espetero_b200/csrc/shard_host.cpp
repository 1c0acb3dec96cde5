// Integer planning of the multi-GPU layer (host only; no counterpart in the reference, which
// runs on one GPU). Sequences are independent units and go to ranks whole; one very long sequence
// is cut by key range on page boundaries, every rank writes partial records for its keys in the
// reference's record format (kernels/40_attention.metal:321-332) and the ranks' reduced records
// are merged in rank order, so that all ranks end with identical bits.
#include <algorithm>
#include <cstdint>
#include <map>
#include <numeric>
#include <utility>
#include <vector>

#include "../../include/espetero_attn.h"
#include "host_util.h"

extern "C" {

// Longest-processing-time greedy: sequences sorted by length (longest first, ties by index), each
// onto the rank with the smallest total so far (ties: lowest rank).
int esp_shard_lpt(const int64_t* lengths, int32_t n, int32_t world, int32_t* rank_of) {
  if (n < 0 || world <= 0 || (n > 0 && (!lengths || !rank_of))) return esp::fail(ESP_ERR_INVALID, "esp_shard_lpt: null or negative argument");
  std::vector<int32_t> order(size_t(n), 0);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return lengths[a] > lengths[b]; });
  std::vector<int64_t> load(size_t(world), 0);
  for (int32_t i : order) {
    const int32_t r = int32_t(std::min_element(load.begin(), load.end()) - load.begin());
    rank_of[i] = r;
    load[size_t(r)] += lengths[i];
  }
  return ESP_OK;
}

// Key range [lo[r], hi[r]) of each rank: the sequence's pages spread as evenly as possible, cuts on
// page boundaries (a page never straddles two GPUs).
int esp_attn_split_kv_ranges(int32_t P, int32_t world, int32_t bt, int32_t* lo, int32_t* hi) {
  if (P < 0 || world <= 0 || bt <= 0 || !lo || !hi) return esp::fail(ESP_ERR_INVALID, "esp_attn_split_kv_ranges: bad argument");
  const int64_t pages = (int64_t(P) + bt - 1) / bt;
  for (int32_t r = 0; r < world; ++r) {
    lo[r] = int32_t(std::min<int64_t>(P, pages * r / world * bt));
    hi[r] = int32_t(std::min<int64_t>(P, pages * (r + 1) / world * bt));
  }
  return ESP_OK;
}

// A rank's plan over its local keys as "records only": every tile writes a partial record (an unsplit
// tile gets a fresh one), only the rank holding the end of the sequence keeps `last` (the row's own key
// counts once), and one reduce job per row group covers the rank's records of that group; every tile
// names that job in pad1 (1 + its index), which lets esp_attn_forward_exchange merge and exchange inside
// the attention kernel (esp_attn_forward ignores the tags of a pass without jobs). tiles are rewritten
// in place.
int esp_attn_plan_split_kv(esp_attn_tile* tiles, int32_t n_tiles, int32_t is_last_rank, esp_attn_combine* jobs, int32_t jobs_cap,
                           int32_t* n_jobs, int32_t* n_parts) {
  if (n_tiles < 0 || (n_tiles > 0 && !tiles) || !n_jobs || !n_parts) return esp::fail(ESP_ERR_INVALID, "esp_attn_plan_split_kv: null or negative argument");
  int32_t np = 0;
  for (int32_t i = 0; i < n_tiles; ++i) np = std::max(np, tiles[i].part + 1);
  std::map<std::pair<int32_t, int32_t>, std::vector<int32_t>> groups;  // (tree, first row) -> records
  for (int32_t i = 0; i < n_tiles; ++i) {
    esp_attn_tile& t = tiles[i];
    if (t.part < 0) t.part = np++;
    if (!is_last_rank) t.last = 0;
    t.pad1 = 0;
    groups[{t.tree, t.r0}].push_back(t.part);
  }
  int32_t nj = 0;
  {
    std::map<std::pair<int32_t, int32_t>, int32_t> job_of;
    for (auto& kv : groups) job_of[kv.first] = int32_t(job_of.size());
    for (int32_t i = 0; i < n_tiles; ++i) tiles[i].pad1 = 1 + job_of[{tiles[i].tree, tiles[i].r0}];
  }
  for (auto& [key, parts] : groups) {
    std::sort(parts.begin(), parts.end());
    for (size_t k = 1; k < parts.size(); ++k)
      if (parts[k] != parts[0] + int32_t(k))
        return esp::fail(ESP_ERR_INVALID, "esp_attn_plan_split_kv: the records of row group (tree %d, row %d) are not consecutive", key.first, key.second);
    if (jobs && nj < jobs_cap) jobs[nj] = {key.second, 1, parts[0], int32_t(parts.size())};
    ++nj;
  }
  *n_jobs = nj, *n_parts = np;
  if (jobs && nj > jobs_cap) return esp::fail(ESP_ERR_CAPACITY, "esp_attn_plan_split_kv: needs %d jobs", nj);
  return ESP_OK;
}

// The final merge over the ranks' reduced records, gathered rank-major (rank r's record of row group g
// is record r * n_groups + g): with one row group, one job over records 0 .. world - 1 in rank order.
int esp_attn_world_merge_jobs(int32_t n_groups, int32_t world, int32_t rows, esp_attn_combine* jobs, int32_t jobs_cap, int32_t* n_jobs) {
  if (n_groups != 1) return esp::fail(ESP_ERR_UNSUPPORTED, "esp_attn_world_merge_jobs: split-KV sharding serves one row group (a single long sequence), got %d", n_groups);
  if (world <= 0 || rows <= 0 || !n_jobs) return esp::fail(ESP_ERR_INVALID, "esp_attn_world_merge_jobs: bad argument");
  *n_jobs = 1;
  if (jobs && jobs_cap >= 1) jobs[0] = {0, rows, 0, world};
  else if (jobs) return esp::fail(ESP_ERR_CAPACITY, "esp_attn_world_merge_jobs: needs 1 job");
  return ESP_OK;
}

}  // extern "C"
