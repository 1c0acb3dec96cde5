// Internal interface between the C-ABI layer (abi.cpp) and the kernel translation
// units. Not installed; the public surface is include/espetero_attn.h.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "../../include/espetero_attn.h"

namespace esp {

// Values a kernel may leave in the context's device status word when a bounded wait runs out.
enum : int { kStatusOk = 0, kStatusTmaTimeout = 1, kStatusMmaTimeout = 2, kStatusBadBlock = 3, kStatusPeerTimeout = 4 };

// What every attention kernel receives: the bindings of the reference dispatch
// (src/model/impl/forest.h:2902-2913) plus the shape constants.
struct KernelArgs {
  const void* Q;
  const void* Kb;
  const void* Vb;
  const void* kv;
  const float* kv_scales;
  const int32_t* blocks;
  const int32_t* desc;
  const uint64_t* anc_mask;
  const float* X;
  void* O;
  float* lse;
  float* parts;
  const esp_attn_tile* tiles;
  const esp_attn_tree* trees;
  int* status;  // device status word of the context
  int* counters;  // kFixupCounters zeroed ints of the context (arrival counters of fused merges), or NULL
  const esp_attn_combine* jobs;  // device copy of the combine jobs (decode kernel, fused merge)
  int32_t fuse;                  // 1: tiles carry their job in pad1 and the last CTA of a job merges (flash_umma: 2 = the two tiles
                                 // of every job run as a cluster pair and merge through distributed shared memory)
  int32_t pair_merge;            // flash_umma: allow the cluster-pair merge (context option "pair_merge")
  int32_t stable_cache;          // the caller's promise (context option "stable_cache"): the kernel before this pass on the
                                 // stream writes neither the block table nor the cached keys [0, P) of any tree (nor their
                                 // scales), so flash_umma may fetch them before that kernel has completed
  unsigned long long* trace;  // optional: CTA (0, 0) writes %globaltimer stamps here (8 events per key block)
  int32_t trace_blocks;       // key blocks the trace buffer holds
  int32_t trace_ctas;         // CTAs whose 4 stamps (start, first scores, loop end, exit) follow at 8 * trace_blocks + 2
  esp_attn_params p;
  int32_t HD;
  int32_t G;
  int32_t tile_rows;
  int32_t n_tiles;
  int32_t q_dtype;
  int32_t kv_dtype;
  int32_t n_blocks;
  int32_t n_trees;          // bounds for the speculative reads ahead of the dependency wait
  int32_t n_block_entries;
  float scale;
  // sliding-window layers (kernels/80_gemma.metal:123-142)
  const int32_t* pos;  // int4 per row, x = position (needed when window > 0)
  int32_t window;      // > 0: keys `window` or more positions behind the query are masked
  int32_t ring;        // > 0: cached key j lives in block table + (j / bt) % ring (no page table)
  int32_t bidi;        // rows of an image also see the image's later rows (desc.w)
  // Qwen sparse attention (general kernel): lists, their lengths, per-row records and selection bitmaps; NULL otherwise
  const uint32_t* qsa_tlist;
  const uint32_t* qsa_tcount;
  const int32_t* qsa_rinfo;
  const uint32_t* qsa_sel;
  int32_t qsa_nbw, qsa_n_lists;
  // Peer exchange at the end of the decode kernel's fused merge (one sequence's keys split over several GPUs);
  // x_world = 0: none. Buffers hold 8-byte words {value, tag}, laid out [epoch parity][rank][record slot].
  int32_t x_world, x_rank, x_phases;  // phases: 1 publish, 2 wait for the world's records and finish the row, 3 both
  uint32_t x_tag, x_wait_ms;
  unsigned long long x_epoch_off;     // words from a buffer's start to this epoch's half
  uint2* x_records[ESP_ATTN_MAX_PEERS];
};

// Small plans travel in the kernel's parameter space (constant bank), one 64-byte line per tile
// holding everything a CTA needs to request its first keys: the tile, its tree, the page-table
// pointer and the page size (G and tile_rows ride in the tile's two unused words). A CTA then
// opens its timeline with one constant-cache miss and one page-table load instead of a chain of
// parameter-line misses and two dependent global loads.
constexpr int kInlinePlanMax = 48;
constexpr int kFixupCounters = 4096;  // ints behind the status word of a context
constexpr int kFixupPerJob = 9;       // decode kernel: per (job, kv head) one ticket of the job and up to 8 of its record groups
struct alignas(64) TileStart {
  esp_attn_tile tile;  // pad1 = first record of the tile's merge job (fused merge)
  esp_attn_tree tree;
  const int32_t* blocks;
  uint16_t bt;
  uint8_t G;
  uint8_t tile_rows;
  uint16_t valid;      // tile index + 1; 0: the record is not in use
  uint8_t fix_parts;   // > 0: records of the tile's merge job; the CTA that finishes last merges them
  uint8_t fix_job;     // index of that job (selects the arrival counter)
};
struct alignas(64) InlinePlan {
  TileStart start[kInlinePlanMax];
};
static_assert(sizeof(TileStart) == 64, "one constant-cache line per tile");

constexpr int kInlineJobsMax = 8;  // one 128-byte constant line: more lines cost a miss per job and SM, which measured slower than the global load
struct CombineArgs {
  const float* parts;
  const float* X;
  void* O;
  float* lse;
  const esp_attn_combine* jobs;
  esp_attn_params p;
  int32_t HD;
  int32_t G;
  int32_t tile_rows;
  int32_t n_jobs;
  int32_t q_dtype;
  int32_t rows_max;  // most rows of any job (<= tile_rows): the grid covers only these
  int32_t n_slices;  // record slices per head: a power of two, 32 <= (HD / 4) * n_slices <= 256
  float* out_parts;  // reduce mode: job j's merged record goes to record out_part0 + j here; else NULL
  int32_t out_part0;
  int32_t n_inline;  // > 0: the jobs also travel in the parameters (no dependent load before the records)
  esp_attn_combine inline_jobs[kInlineJobsMax];
};

// The peer exchange kernel: a merge whose result goes through every rank's exchange buffer.
struct ExchangeArgs {
  CombineArgs c;  // parts, X, O, lse, jobs, shape; out_parts unused
  int32_t rank;
  int32_t world;
  int32_t phases;
  uint32_t wait_ms;
  unsigned long long epoch;
  uint2* records[ESP_ATTN_MAX_PEERS];  // exchange buffers: 8-byte words {value, tag}
  int* status;
  unsigned long long* trace;  // optional: CTA (0, 0) stores %globaltimer at 5 points (esp_attn_set_trace buffer, slots 0-4)
};

// Whether a pass can merge its split-K records inside the attention kernel: every tile that
// writes a record names its job in pad1 (1 + index), lies inside that job's record range and row
// group, every job's records are all written by this pass, and (job, kv head) pairs fit the counters.
inline bool plan_fusable(const esp_attn_tile* tiles, int32_t n_tiles, const esp_attn_combine* jobs, int32_t n_jobs, int32_t Hkv) {
  if (!tiles || !jobs || n_jobs <= 0 || int64_t(n_jobs) * Hkv * kFixupPerJob > kFixupCounters) return false;
  // Records of a job are consecutive and, in a planner's output, written by consecutive tiles in
  // record order: check exactly that (anything else takes the two-kernel route).
  int64_t records = 0, claimed = 0;
  for (int32_t j = 0; j < n_jobs; ++j) {
    if (jobs[j].nparts < 1) return false;
    records += jobs[j].nparts;
  }
  int32_t prev_job = 0, prev_part = -1;
  for (int32_t i = 0; i < n_tiles; ++i) {
    const esp_attn_tile& t = tiles[i];
    if (t.part < 0) continue;
    if (t.pad1 < 1 || t.pad1 > n_jobs) return false;
    const esp_attn_combine& jb = jobs[t.pad1 - 1];
    if (t.part < jb.part0 || t.part >= jb.part0 + jb.nparts || t.r0 != jb.r0) return false;
    if (t.pad1 == prev_job ? t.part != prev_part + 1 : t.part != jb.part0) return false;
    prev_job = t.pad1, prev_part = t.part;
    ++claimed;
  }
  return claimed == records;
}

// Decode passes for which the in-kernel merge pays: small ones (at most one CTA per SM of a B200:
// launch latencies dominate), and passes with many jobs, whose merges happen while other CTAs still
// stream (measured on the batched decode: -1.8 us per step). A pass with a few long jobs that all end
// together (one 131072-token sequence: 8 merges of 37 records) is faster with the combine kernel's
// parallelism (+7 us when merged in the kernel).
// (Instances with 4 KB key blocks - 64-dim heads, 128-dim E4M3 pools: four CTAs per SM - keep the combine kernel for
// the many-job case too: 97.2 against 100.7 us and 114.3 against 119.2 us on the 32-sequence batch.)
inline bool decode_fuse_small(int32_t n_tiles, int32_t Hkv, int32_t n_jobs, bool light_blocks = false) {
  return int64_t(n_tiles) * Hkv <= 148 || (!light_blocks && int64_t(n_jobs) * Hkv >= 32);
}

// Record slices per head for the combine kernel: a slice folds up to eight records per round trip
// to L2, so eight records per slice at most where the CTA allows it; at least one warp per head, at
// most one CTA (256 threads) per head.
inline int32_t combine_slices(int32_t HD, int32_t parts_max) {
  const int tpd = HD / 4, max_nsl = 256 / tpd;
  int nsl = 1;
  while (nsl < max_nsl && (nsl * 8 < parts_max || tpd * nsl < 32)) nsl *= 2;
  return nsl;
}

// attn_prep (kernels/40_attention.metal:23-102): bindings of the reference dispatch (forest.h:2951-2977).
struct PrepArgs {
  const float* X;
  const float* qn_w;
  const float* kn_w;
  const int32_t* pos;       // int4 per row
  const float* inv_freq;
  const int32_t* rope_sel;
  void* Q;
  void* Kb;
  void* Vb;
  const int32_t* ktab;      // int4 per row, or NULL
  void* kv;
  const float* kv_scales;
  int32_t rows;
  int32_t heads_per_warp;   // a warp forms its row's rotation once and reuses it for this many heads
  esp_attn_prep_params p;
};

// Host-side checks of a pass before anything is launched (the checks run_forest makes,
// src/model/impl/forest.h:2136-2280): pointers, alignment, and - with `deep` - every tree, tile and
// combine job of the host mirrors against the row, block-table and record counts of `a`.
// Returns ESP_OK or a negative esp_status with the message set.
int validate_pass(const esp_attn_shape& s, int tile_rows, bool deep, const esp_attn_args& a);

// Launch with programmatic stream serialization: the grid may be scheduled while the previous
// kernel of the stream drains; the kernel orders itself with griddepcontrol.wait.
template <typename... Params, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<Args&&>(args)...);
  return e == cudaSuccess ? cudaGetLastError() : e;
}

// Each launcher enqueues on `stream`, returns cudaGetLastError() of the launch and
// adds the number of kernels it launched to *launches.
cudaError_t launch_flash_general(const KernelArgs& a, cudaStream_t stream, uint64_t* launches);
cudaError_t launch_decode_gqa(const KernelArgs& a, const CUtensorMap& pool_map, cudaStream_t stream, uint64_t* launches);
cudaError_t launch_combine(const CombineArgs& a, cudaStream_t stream, uint64_t* launches);
bool attn_prep_supports(int32_t HD);
cudaError_t launch_attn_prep(const PrepArgs& a, int32_t HD, int32_t q_dtype, bool fp8_pool, cudaStream_t stream, uint64_t* launches);
cudaError_t launch_exchange(const ExchangeArgs& x, cudaStream_t stream, uint64_t* launches);
int64_t exchange_grid_ctas(const CombineArgs& a);
cudaError_t launch_kv_save(const void* Kb, const void* Vb, void* kv, const float* kv_scales, const esp_kv_save_entry* entries,
                           int32_t n, const esp_attn_params& p, int32_t HD, int32_t q_dtype, int32_t kv_dtype,
                           cudaStream_t stream, uint64_t* launches);
// Widens the E4M3 blocks named by blocks[0 .. n_entries) of a layer region to the 16-bit type
// (code * scale) into a compact pool: entry e becomes block e of `out`; `identity` receives 0 .. n_entries-1.
cudaError_t launch_kv_dequant(const void* kv, const float* kv_scales, const int32_t* blocks, int32_t n_entries, void* out,
                              int32_t* identity, const esp_attn_params& p, int32_t HD, int32_t n_blocks, int32_t q_dtype,
                              cudaStream_t stream, uint64_t* launches);
cudaError_t launch_kv_copy_blocks(void* kv, const int32_t* pairs, int32_t n_pairs, const esp_attn_params& p,
                                  uint64_t region_elems, int32_t n_layers, int32_t elem_bytes, cudaStream_t stream,
                                  uint64_t* launches);

cudaError_t launch_qsa_select(const float* scores, const int32_t* srows, const int32_t* rinfo, uint32_t* sel, int32_t n_sparse, int32_t nbmax,
                              int32_t nbw, cudaStream_t stream, uint64_t* launches);
cudaError_t launch_qsa_tiles(const uint32_t* sel, const esp_attn_tree* trees, const int32_t* rinfo, const esp_qsa_tile* qtiles, int32_t n_qtiles,
                             uint32_t* tlist, uint32_t* tcount, int32_t nbmax, int32_t nbw, cudaStream_t stream, uint64_t* launches);

// finite_check over rows x cols elements (row stride ld, in elements) into the 4-word record `rec`.
cudaError_t launch_finite_check(const void* x, uint32_t rows, uint32_t cols, uint64_t ld, int dtype, uint32_t thr_bits, uint32_t* rec,
                                cudaStream_t stream, uint64_t* launches);

// Two tcgen05 kernels with the same contract: flash_umma streams a long cached prefix from HBM
// (one CTA per SM, 128-key blocks, deep K/V rings); flash_umma_pair is for passes whose keys are
// mostly their own rows and sit in L2 (two CTAs per SM, 64-key blocks, short rings).
cudaError_t launch_flash_umma(const KernelArgs& a, const CUtensorMap& pool_map, const CUtensorMap& kb_map, const CUtensorMap& vb_map,
                              const esp_attn_tile* tiles_host, const esp_attn_tree* trees_host, int32_t n_trees,
                              const esp_attn_combine* jobs_host, int32_t n_jobs, bool* merged, cudaStream_t stream,
                              uint64_t* launches);
// e4m3_direct: 256-dim heads over an E4M3 pool read directly; pool_map is then the pool's byte map (the decode kernel's).
cudaError_t launch_flash_umma_pair(const KernelArgs& a, const CUtensorMap& pool_map, const CUtensorMap& kb_map,
                                   const CUtensorMap& vb_map, bool e4m3_direct, cudaStream_t stream, uint64_t* launches);
cudaError_t flash_umma_pair_setup();
// flash_umma_duo: one CTA per SM, two 128-lane query tiles (two head groups of one kv head) against the same 128-key
// blocks; for compute-bound passes (prefill). HD 128 only; a CTA's 2 * (128 / tile_rows) heads must share a kv head.
cudaError_t launch_flash_umma_duo(const KernelArgs& a, const CUtensorMap& pool_map, const CUtensorMap& kb_map,
                                  const CUtensorMap& vb_map, cudaStream_t stream, uint64_t* launches);
cudaError_t flash_umma_duo_setup();
bool flash_umma_duo_supports(int32_t HD, int32_t G, int32_t tile_rows, int32_t bt, int32_t q_dtype, int32_t kv_dtype);
// Shapes the tcgen05 kernels cover: HD 128 (both kernels) or 256 (flash_umma_pair), 16-bit pool of the
// pass's type, tiles of 16..128 rows whose 128 / tile_rows heads belong to one kv head.
bool flash_umma_supports(int32_t HD, int32_t G, int32_t tile_rows, int32_t bt, int32_t q_dtype, int32_t kv_dtype);
cudaError_t flash_umma_setup();

// Shapes the decode kernel covers (the ABI layer falls back to the general kernel otherwise).
bool decode_gqa_supports(int32_t HD, int32_t G, int32_t bt, int32_t q_dtype, int32_t kv_dtype);
// One-time per-device setup (raises dynamic shared memory limits).
cudaError_t decode_gqa_setup();

// Geometry of the pool tensor map the decode kernel expects: a 3-D view
// [bytes of one 128-byte line][rows = n_blocks * 2 * bt][lines per row] of one layer region,
// box = [128 B, 16 rows, lines of one head], 128-byte swizzle.
constexpr int kDecodeKeyBlock = 16;

}  // namespace esp
