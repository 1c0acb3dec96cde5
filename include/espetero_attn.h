/*
 * espetero_attn.h - C ABI of the B200 attention path.
 *
 * Drop-in for the attention step of the reference's forest pass: the dispatch
 * lambda `attention(plan, ...)` and its neighbours `kv_save` / `kv_cow_copy`
 * in src/model/impl/forest.h:2855-2947 and :1438-1449, the integer planner
 * `plan_tiles` (forest.h:1378-1433; generic-head-dim twin `g4_plan_tiles`,
 * src/model/impl/gemma.h:77-116) and the kernels of kernels/40_attention.metal
 * (flash_attention :156, attn_decode_gqa :598, attention_combine :811, kv_save
 * :875, kv_copy_blocks :894) with their generic-HD instantiations
 * (kernels/80_gemma.metal:157-342, kernels/82_qwen3_omni.metal:97-106).
 *
 * Conventions
 *  - every function returns 0 on success and a negative esp_status otherwise;
 *    esp_attn_last_error() gives the message of the calling thread's last
 *    failure. No exception crosses this boundary.
 *  - one context per GPU; a context is not thread-safe (the reference has one
 *    scheduler thread, src/model/api.h:4-6).
 *  - the caller owns every buffer. Unless a function says otherwise, nothing
 *    here allocates device memory, and all device work is enqueued on the
 *    caller's stream without a host synchronisation.
 *  - pointers named *_host are host memory, all other data pointers are device
 *    memory of the context's GPU.
 *  - metadata buffers (tiles, trees, blocks, desc, jobs) must stay unchanged
 *    while a pass that reads them is in flight (docs/design.md:237-243).
 */
#ifndef ESPETERO_ATTN_H
#define ESPETERO_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ESP_ATTN_ABI_VERSION 4

/* ---------------------------------------------------------------- status */
typedef enum esp_status {
  ESP_OK = 0,
  ESP_ERR_INVALID = -1,      /* bad argument (validation failed; nothing was launched) */
  ESP_ERR_UNSUPPORTED = -2,  /* shape / dtype outside what the kernels cover */
  ESP_ERR_CUDA = -3,         /* a CUDA runtime or driver call failed */
  ESP_ERR_CAPACITY = -4,     /* an output array of the caller is too small */
  ESP_ERR_INJECTED = -5,     /* host-side fault injection (ESPETERO_FAIL_PASS) */
  ESP_ERR_NO_DEVICE = -6     /* no usable sm_100 device */
} esp_status;

/* -------------------------------------------------------------- records */
/* Bit-identical to the kernel-side records of the reference
 * (kernels/40_attention.metal:124-150, :804-809, :868-873; host mirrors
 * forest.h:1308-1319, :1342-1345). */

typedef struct esp_attn_params {
  int32_t H;        /* query heads */
  int32_t Hkv;      /* KV head groups of the grid */
  int32_t q_ld;     /* Q / O row stride in elements (H * HD) */
  int32_t kv_ld;    /* K / V row width in elements (Hkv * HD), batch rows and pool */
  int32_t g_ld;     /* row stride of the fused projection X (gate source), in floats */
  int32_t bt;       /* tokens per KV block */
  uint64_t kv_base; /* element offset of this layer's region in the KV pool */
} esp_attn_params;

typedef struct esp_attn_tree {
  int32_t base;  /* absolute first row of the tree in this pass */
  int32_t P;     /* cached keys */
  int32_t table; /* first entry of its block list in `blocks` */
  int32_t M;     /* rows of the tree in this pass */
} esp_attn_tree;

typedef struct esp_attn_tile {
  int32_t tree;
  int32_t r0;   /* absolute first query row */
  int32_t k0;   /* cached key range [k0, k1) */
  int32_t k1;
  int32_t part; /* -1: write O; else index of the partial record */
  int32_t last; /* also scan the batch keys */
  int32_t pad0; /* first batch key to scan in the reference's sliding-window plans (gemma.h:89-94); 0 otherwise */
  int32_t pad1; /* 0 (unused in the reference), or 1 + index of the combine job that merges this tile's
                   record: set by the ESP_PLAN_B200 planner; when every split tile of a pass carries
                   it, small passes merge the records inside the attention kernel (the CTA that
                   finishes a job last does it, in record order) and launch no combine kernel */
} esp_attn_tile;

typedef struct esp_attn_combine {
  int32_t r0;     /* absolute first row */
  int32_t rows;   /* rows of the group (<= tile_rows) */
  int32_t part0;  /* first record */
  int32_t nparts; /* records, merged in this order */
} esp_attn_combine;

typedef struct esp_kv_save_entry {
  int32_t src_row;
  int32_t block;
  int32_t pos;
  int32_t pad;
} esp_kv_save_entry;

/* ---------------------------------------------------------------- shape */
typedef enum esp_dtype {
  ESP_F16 = 0,
  ESP_BF16 = 1,
  ESP_E4M3 = 2 /* KV pool only: e4m3fn codes + one fp32 scale per (block, K|V, kv head) */
} esp_dtype;

enum {
  ESP_ATTN_FLAG_GATE = 1,    /* O *= sigmoid(gate), gate = X[row*g_ld + h*2*HD + HD + d] (40_attention.metal:334-342) */
  ESP_ATTN_FLAG_ANC_MASK = 2 /* batch-key visibility from a 64-bit ancestor mask per row instead of `desc` */
};

typedef struct esp_attn_shape {
  int32_t H;        /* query heads */
  int32_t Hkv;      /* KV heads; G = H / Hkv in {1,2,4,8} for the decode kernel */
  int32_t HD;       /* head dim: 64 (16-bit pools), 128, 256 or 512 on the decode kernel; 64, 128, 256 or 512 on the tcgen05 kernels */
  int32_t bt;       /* tokens per KV block (any value; multiples of 16 take the fast paths) */
  int32_t q_dtype;  /* ESP_F16 | ESP_BF16: Q, Kb, Vb, O */
  int32_t kv_dtype; /* pool type: same as q_dtype, or ESP_E4M3 */
  int32_t tile_rows;/* query rows per tile: 8 (reference), 16, 32, 64 or 128 */
  int32_t flags;
  float scale;      /* softmax(scale * q.k); the reference folds 1/sqrt(HD) here (40_attention.metal:199, :692) */
  int32_t reserved[3];
} esp_attn_shape;

typedef struct esp_attn_ctx esp_attn_ctx;

/* Create / destroy a context on `device`. Creation resolves the driver entry
 * point used to build tensor maps and raises the kernels' shared-memory limits;
 * it allocates one small device block (the status word and 4096 arrival counters of the in-kernel
 * merge, 16.6 KB) and the staging slots of re-planned passes (1.5 MB on the device, as much pinned on
 * the host), all freed by destroy. */
int esp_attn_create(esp_attn_ctx** out, int device, const esp_attn_shape* shape);
int esp_attn_destroy(esp_attn_ctx* ctx);
const char* esp_attn_last_error(void);
int esp_attn_abi_version(void);

/* Runtime options, as NativeModel::set_option(name, int) (src/model/model.mm:936-1004).
 * Names: "attn_gqa" (1: single-row trees take the decode kernel; default 1),
 * "attn_umma" (1: multi-row tiles take the tcgen05 kernel when the shape allows;
 * default 1), "replan" (1: a context with tile_rows 8 plans plain full-attention passes again for the
 * tcgen05 kernels instead of running their 8-row tiles on the CUDA-core kernel - see esp_attn_forward;
 * default 1), "umma_kernel" (which tcgen05 kernel: 0 by the pass, 1 flash_umma - cached keys
 * streamed from HBM, 2 flash_umma_pair - keys of the pass itself, two CTAs per SM, 3 flash_umma_duo - keys of the
 * pass itself, two query tiles per CTA, where the heads allow it, else as 2; default 0), "fuse_combine"
 * (passes whose split tiles name their combine job in pad1 can merge their records inside the
 * attention kernel and launch no combine kernel: 0 never, 1 where it measured faster - small passes
 * and decode passes with many jobs -, 2 whenever possible; default 1), "trace_ctas" (see
 * esp_attn_set_trace), "validate" (1: check host mirrors before launching; default 1), "fail_pass"
 * (N > 0: every Nth pass of 64 rows or more fails with ESP_ERR_INJECTED before anything
 * is launched; initialised from the ESPETERO_FAIL_PASS environment variable, the
 * reference's host-side fault injection, forest.h:2521-2531), "check_finite" (1: scan every pass's
 * output for NaN / Inf, see esp_attn_finite_check; initialised from ESPETERO_CHECK_FINITE; default 0),
 * "fuse_exchange" (see esp_attn_forward_exchange; default 0), "stable_cache" (1: the caller promises that the kernel
 * enqueued before a pass on its stream writes neither the block table nor the cached keys [0, P) of any tree of the
 * pass, nor their E4M3 scales - in the reference's layer the kernel before attention is attn_prep, which writes this
 * pass's rows only; the verify kernel then starts fetching cached key blocks while that kernel still drains
 * (programmatic dependent launch); Q, Kb, Vb and the mask records are waited for as ever; default 0), "fp8_direct" (1: multi-row passes over an E4M3 pool
 * with 128- or 256-dim heads and mostly cached keys dequantise inside the tcgen05 kernel instead of widening the pool into
 * dequant_scratch first; default 1),
 * "attn_vec" (the reference's alternative decode schedule, src/model/impl/model.h:590, off there by
 * default and not built here: 0 is accepted, anything else answers ESP_ERR_UNSUPPORTED). */
int esp_attn_set_option(esp_attn_ctx* ctx, const char* name, int value);
int esp_attn_get_option(const esp_attn_ctx* ctx, const char* name, int* value);

/* -------------------------------------------------------------- planner */
typedef enum esp_plan_mode {
  ESP_PLAN_REFERENCE = 0, /* plan_tiles, forest.h:1378-1433: bit-for-bit */
  ESP_PLAN_G4 = 1,        /* g4_plan_tiles without a window, gemma.h:77-116 */
  ESP_PLAN_B200 = 2       /* same records; chunks sized so that the CTAs fill `groups` slots evenly */
} esp_plan_mode;

typedef struct esp_plan_opts {
  int32_t mode;      /* esp_plan_mode */
  int32_t split;     /* attn_split: most keys of a split tile (reference default 512); 0 = never split */
  int32_t min_chunk; /* attn_min_chunk: fewest keys of a split tile (reference default 32) */
  int32_t groups;    /* CTA target (reference: 256); ESP_PLAN_B200: e.g. 2 * 148 */
  int32_t tile_rows; /* query rows per tile (reference: 8) */
  int32_t max_parts; /* most parts per row group (reference: 64) */
  int32_t reserved[2];
} esp_plan_opts;

/* g4_plan_tiles (src/model/impl/gemma.h:77-116) bit for bit, window branch included: a sliding tile
 * starts at the first cached key any of its rows can see (k0 = min position - window + 1, clamped) and
 * carries the first batch key to scan in pad0. `groups` = kv heads x split groups of the grid, `rows` =
 * rows per tile when nothing is split (8 otherwise), pos = int4 per row. plan_rows receives the tile
 * height the plan was made for. Same capacity protocol as esp_attn_plan. */
int esp_attn_plan_window(const esp_attn_tree* trees, int32_t n_trees, int32_t groups, int32_t split, int32_t rows,
                         int32_t window, const int32_t* pos, esp_attn_tile* tiles, int32_t tiles_cap, esp_attn_combine* jobs,
                         int32_t jobs_cap, int32_t* n_tiles, int32_t* n_jobs, int32_t* n_parts, int32_t* plan_rows);

/* Pure host function. Writes up to tiles_cap tiles and jobs_cap combine jobs and
 * always reports the counts needed (ESP_ERR_CAPACITY if an array was too small;
 * pass NULL arrays to size them). n_parts = partial records the pass needs; the
 * caller sizes `parts` as n_parts * Hkv * tile_rows * G * (HD + 2) floats
 * (forest.h:2716). */
int esp_attn_plan(const esp_attn_tree* trees_host, int32_t n_trees, int32_t Hkv, const esp_plan_opts* opts,
                  esp_attn_tile* tiles_host, int32_t tiles_cap, esp_attn_combine* jobs_host, int32_t jobs_cap,
                  int32_t* n_tiles, int32_t* n_jobs, int32_t* n_parts);

/* Floats the caller must provide in `parts` for n_parts records. */
size_t esp_attn_parts_floats(const esp_attn_shape* shape, int32_t n_parts);

/* -------------------------------------------------------------- forward */
/* The twelve bindings of the reference's attention dispatch
 * (forest.h:2902-2913) plus what the extensions need. */
typedef struct esp_attn_args {
  const void* Q;           /* [rows][q_ld] q_dtype */
  const void* Kb;          /* [rows][kv_ld] q_dtype: this pass's keys */
  const void* Vb;          /* [rows][kv_ld] q_dtype */
  const void* kv;          /* pool; block = [K: bt x kv_ld][V: bt x kv_ld] (forest.h:51-57) */
  const float* kv_scales;  /* ESP_E4M3 only: [n_blocks][2][Hkv] (K row, then V row), this layer's table */
  const int32_t* blocks;   /* flattened block lists */
  const int32_t* desc;     /* int4 per row: (seg_start, 0, anc_len, img_end), relative to the tree's first row */
  const uint64_t* anc_mask;/* ESP_ATTN_FLAG_ANC_MASK: bit j = batch key j of the tree is visible to the row */
  const float* X;          /* gate source, or NULL without ESP_ATTN_FLAG_GATE */
  void* O;                 /* [rows][q_ld] q_dtype */
  float* lse;              /* optional [rows][H]: m + ln(l) of rows written unsplit or combined; NULL to skip */
  float* parts;            /* partial records [O(HD) | m | l] fp32 */
  const esp_attn_tile* tiles;
  const esp_attn_tree* trees;
  const esp_attn_combine* jobs;
  /* host mirrors (the plan the caller built): needed to pick the kernel as
   * forest.h:2864-2868 does and to validate before launching */
  const esp_attn_tile* tiles_host;
  const esp_attn_tree* trees_host;
  const esp_attn_combine* jobs_host;
  int32_t n_tiles;
  int32_t n_trees;
  int32_t n_jobs;
  int32_t n_rows;          /* rows of Q / Kb / Vb / O / desc */
  int32_t n_blocks;        /* blocks of this layer's pool region */
  int32_t n_block_entries; /* entries of `blocks` */
  int32_t n_parts;         /* records `parts` can hold */
  int32_t reserved;
  esp_attn_params p;
  /* Sliding-window layers of the generic attention kernel (kernels/80_gemma.metal:123-142; host
   * src/model/impl/gemma.h:77-116). All zero / NULL for ordinary layers. */
  const int32_t* pos;      /* int4 per row, x = the row's position; needed when window > 0 */
  int32_t window;          /* > 0: a key `window` or more positions behind the query is masked (cached key j
                              is at position j, a batch key at its row's position). Single-row trees rely on
                              the plan instead, as the reference's decode kernel does: its tile starts at the
                              row's first visible key (esp_attn_plan_window). */
  int32_t ring;            /* > 0: cached key j of a tree lives in block tree.table + (j / bt) % ring of the
                              layer region - the slot's ring of a sliding layer - and `blocks` is not read */
  int32_t bidi;            /* 1: rows of an image also see the image's later rows (desc.w = end of the row's
                              image, 0 outside images) */
  int32_t reserved2;
  /* Multi-row passes over an ESP_E4M3 pool (verify / prefill over FP8 keys). 128- or 256-dim heads, keys mostly cached
   * (more than twice the pass's own rows): the tcgen05 kernel reads the codes itself and needs nothing here
   * (option "fp8_direct", default 1); a pass without cached keys never reads the pool and needs nothing either.
   * Other such passes (mostly their own rows behind a short prefix; 64-dim heads) use this optional scratch: with it the pass first widens
   * the blocks of `blocks` to the 16-bit type (code * scale, rounded once) into the scratch and runs the
   * tensor-core kernels on that copy; without it (NULL) 128- and 256-dim passes still read the codes themselves,
   * the rest run on the general kernel.
   * Size: esp_attn_dequant_scratch_bytes. Contents need not survive the call. */
  void* dequant_scratch;
  uint64_t dequant_scratch_bytes;
  /* Qwen sparse attention (flash_attention_qsa, kernels/45_qsa.metal:452-690; the extra bindings 12-16 of its
   * dispatch, src/model/impl/forest.h:1646-1656). NULL / 0 for ordinary passes. With them, a tile whose pad0 is 1
   * reads the cached keys of a union list instead of a key range: k0 / k1 are entries of list pad1 (an entry = one
   * block of 4 keys with an 8-bit row mask), and a sparse row counts a batch key only if the key's block is selected
   * for it or lies in its tail. Tiles with pad0 = 0 are dense as ever. Such passes run on the general kernel. */
  const uint32_t* qsa_tlist;  /* [tiles][ESP_QSA_LMAX] entries (block << 8) | row mask, ascending (esp_qsa_tiles) */
  const uint32_t* qsa_tcount; /* [tiles] entries of each list */
  const int32_t* qsa_rinfo;   /* int4 per pass row: sequence index s, nb = (s + 1) / 4, sparse row or -1, tree (esp_qsa_plan) */
  const uint32_t* qsa_sel;    /* [sparse rows][qsa_nbw] selection bitmaps (esp_qsa_select) */
  int32_t qsa_nbw;            /* bitmap words per sparse row */
  int32_t qsa_n_lists;        /* lists in qsa_tlist (bounds tile.pad1) */
  /* Optional host mirror of `pos` (int4 per row, as the engine builds it before the upload, forest.h:2374-2450).
   * With it a context with tile_rows 8 can plan a sliding-window pass again for the tcgen05 kernel, as it does for
   * plain passes (see esp_attn_forward); without it such plans run on the general kernel as given. */
  const int32_t* pos_host;
} esp_attn_args;

/* Bytes of dequant_scratch for a pass whose block table has n_block_entries entries (pool rows of
 * kv_ld = Hkv * HD elements; wider rows need n_block_entries * 4 * bt * kv_ld + 4 * n_block_entries
 * rounded up to 128). */
size_t esp_attn_dequant_scratch_bytes(const esp_attn_shape* shape, int32_t n_block_entries);

/* Attention over the plan's tiles, then the combine jobs: the reference's
 * attention() lambda. stream is a cudaStream_t.
 * Contexts with tile_rows 8 (the reference's tile height, forest.h:1378-1433): the tensor-core kernels
 * need 128 (row, head) pairs per CTA, which 8-row tiles do not give. When a multi-row pass's plan is
 * plain full attention - every 8-row group of every tree covered once over [0, P), split tiles merged
 * by the pass's own jobs: what plan_tiles emits - only O and lse are its results, and the pass is
 * planned again inside this call for those kernels (tiles of 128 rows, or of 128 / G rows x G heads
 * over a cached prefix); the new tiles travel through pinned staging slots the context owns. The
 * caller's tiles / jobs are only read; `parts` is then scratch in the new tiles' layout and its
 * contents after the call are unspecified. The plans of the generic planner's window branch
 * (g4_plan_tiles, gemma.h:77-116: ranges that start at a row group's first visible key, pad0 = first
 * batch key) are treated the same way when args->pos_host mirrors the rows' positions. Any other plan
 * (records without jobs, window plans without that mirror, sparse plans, hand-made tilings) runs as
 * given. Option "replan" = 0 switches this off. */
int esp_attn_forward(esp_attn_ctx* ctx, void* stream, const esp_attn_args* args);

/* Only the merge step (attention_combine): used after records of other GPUs
 * have been gathered next to the local ones (split-KV over several GPUs). */
int esp_attn_combine_parts(esp_attn_ctx* ctx, void* stream, const float* parts, const float* X, void* O, float* lse,
                           const esp_attn_params* p, const esp_attn_combine* jobs, int32_t n_jobs);

/* First level of a two-level merge (no counterpart in the reference, which has one GPU): job j's
 * records are merged into ONE still unnormalised record [O | M | L], written as record
 * out_part0 + j of parts_out (same layout as `parts`). A GPU that holds only part of a
 * sequence's keys reduces its local records this way, the ranks exchange the reduced records
 * (33 KB per row for H32 / HD256) and esp_attn_combine_parts finishes the merge. */
int esp_attn_reduce_parts(esp_attn_ctx* ctx, void* stream, const float* parts, const esp_attn_params* p,
                          const esp_attn_combine* jobs, int32_t n_jobs, float* parts_out, int32_t out_part0);

/* ---- Split-KV over the GPUs of one box: reduce, exchange over peer memory and merge in ONE kernel.
 * No counterpart in the reference (one GPU). Every rank holds the keys of one range of a long
 * sequence and has written partial records for them (esp_attn_forward with records-only tiles).
 * esp_attn_exchange_parts then, in one launch per rank:
 *   1. merges the rank's records of each job into one unnormalised record [O | M | L];
 *   2. stores that record into slot `rank` of EVERY rank's exchange buffer through peer mappings
 *      (NVLink) as 8-byte words {value, tag = epoch}: each word tells by itself whether it has
 *      arrived, so there is no fence and no separate flag between the data and its consumer;
 *   3. reads the `world` records from its own buffer, polling (bounded) until every word carries
 *      the tag, merges them in rank order: all ranks produce identical bits, O and lse are final.
 * The buffers come from esp_p2p_alloc on each rank (zero-filled) and are opened on the others with
 * esp_p2p_open (the caller carries the 64-byte handles between processes). `epoch` must be the
 * same on all ranks for a call and larger by one for the next call on the same buffers (its low
 * 32 bits are the tag; 0 is never used); the buffers hold two epochs, so a rank may run at most
 * one call ahead of the slowest.
 * The grid must fit on the GPU at once (jobs * rows * head groups <= 296 CTAs), else
 * ESP_ERR_UNSUPPORTED: gather with a library collective and call esp_attn_combine_parts.
 * If a peer never delivers, the kernel gives up after wait_ms, writes nothing to O and
 * esp_attn_check_status reports it; the context stays usable. */
#define ESP_ATTN_MAX_PEERS 8
typedef struct esp_attn_exchange {
  int32_t rank;
  int32_t world;     /* 1 .. ESP_ATTN_MAX_PEERS */
  int32_t phases;    /* 3: the whole exchange in one launch. 1: steps 1-2 only, 2: step 3 only (lets a
                        test run several emulated ranks one after another on one GPU) */
  int32_t wait_ms;   /* bound of the wait in step 3; 0 = 2000 */
  uint64_t epoch;    /* >= 1 */
  void* records[ESP_ATTN_MAX_PEERS];    /* rank q's exchange buffer as mapped in this process (own included) */
} esp_attn_exchange;

/* Bytes of one rank's exchange buffer for a context's shape. */
size_t esp_attn_exchange_bytes(const esp_attn_shape* shape, int32_t n_jobs, int32_t world);

/* rows_max: most rows of any job (1 for decode). jobs are device-resident, as for esp_attn_combine_parts;
 * parts_max: most records of any job (sizes the merge's parallelism; 64 if unknown). */
int esp_attn_exchange_parts(esp_attn_ctx* ctx, void* stream, const float* parts, const float* X, void* O, float* lse,
                            const esp_attn_params* p, const esp_attn_combine* jobs, int32_t n_jobs, int32_t rows_max,
                            int32_t parts_max, const esp_attn_exchange* x);

/* ---- Planning of the multi-GPU layer (pure host functions; no counterpart in the reference).
 * esp_shard_lpt: sequences -> ranks by longest-processing-time greedy on their context lengths
 * (longest first, ties by index, onto the least loaded rank, ties to the lowest): rank_of[i] = rank of
 * sequence i. Whole sequences move; nothing is exchanged on the data path.
 * esp_attn_split_kv_ranges: key range [lo[r], hi[r]) of each rank for one sequence of P keys, cut on
 * page boundaries with the pages spread as evenly as possible.
 * esp_attn_plan_split_kv: turns a rank's plan over its local keys (esp_attn_plan) into the
 * records-only plan esp_attn_exchange_parts / esp_attn_reduce_parts expect: every tile writes a
 * record, only the last rank keeps `last`, job tags are cleared, and one reduce job per row group
 * names the rank's records and is named by its tiles in pad1 (tiles rewritten in place; jobs_cap
 * protocol as esp_attn_plan).
 * esp_attn_world_merge_jobs: the job that merges the ranks' reduced records, gathered rank-major. */
int esp_shard_lpt(const int64_t* lengths, int32_t n, int32_t world, int32_t* rank_of);
int esp_attn_split_kv_ranges(int32_t P, int32_t world, int32_t bt, int32_t* lo, int32_t* hi);
int esp_attn_plan_split_kv(esp_attn_tile* tiles, int32_t n_tiles, int32_t is_last_rank, esp_attn_combine* jobs, int32_t jobs_cap,
                           int32_t* n_jobs, int32_t* n_parts);
int esp_attn_world_merge_jobs(int32_t n_groups, int32_t world, int32_t rows, esp_attn_combine* jobs, int32_t jobs_cap,
                              int32_t* n_jobs);

/* The whole split-KV step of a rank in one call: args carry the rank's records-only plan (tiles tagged by
 * esp_attn_plan_split_kv) and its reduce job (jobs / jobs_host, n_jobs = 1). By default the call runs the
 * records-only pass and then esp_attn_exchange_parts (two launches). With the context option
 * "fuse_exchange" = 1 everything happens inside the decode kernel, in ONE launch: its CTAs fold the rank's
 * records in two short levels as they finish (no CTA waits for another of its GPU); the CTA that completes
 * a kv head's record stores it into every rank's exchange buffer over peer mappings, waits (bounded by
 * wait_ms) for the other ranks' records of the same heads, folds them in rank order and writes O / lse. The
 * waiting CTAs need the whole grid resident at once; a pass whose grid is larger, or that the decode
 * kernel does not take, falls back to the two launches. The one-launch form measured slower (64.0 against
 * 57.3 us per step for a 131072-key E4M3 sequence over two GPUs: its chain of fence, ticket and bulk copy
 * per level costs more than a kernel boundary), which is why it is off by default. Same buffers, epochs,
 * bits-on-every-rank guarantee and failure behaviour as esp_attn_exchange_parts either way. phases = 1
 * publishes without waiting, phases = 2 runs only the second half (both for tests that emulate several
 * ranks on one GPU). */
int esp_attn_forward_exchange(esp_attn_ctx* ctx, void* stream, const esp_attn_args* args, const esp_attn_exchange* x);

/* Device memory another process of the same box can map: cudaMalloc + zero fill + an IPC handle
 * (64 bytes, opaque). esp_p2p_open maps a peer's allocation into this process (peer access is
 * enabled on first use); esp_p2p_close unmaps it; esp_p2p_free releases an own allocation. */
#define ESP_P2P_HANDLE_BYTES 64
int esp_p2p_alloc(void** ptr, size_t bytes, unsigned char handle[ESP_P2P_HANDLE_BYTES]);
int esp_p2p_open(const unsigned char handle[ESP_P2P_HANDLE_BYTES], void** ptr);
int esp_p2p_close(void* ptr);
int esp_p2p_free(void* ptr);

/* ---- Checkpoint files of a sequence's KV blocks in the reference's layout (slot_save / slot_load,
 * src/model/model.mm:604-740): a 120-byte header (magic 0x554b5043, version 4) and the blocks
 * layer-major - for every layer the blocks of the sequence's list in order, block_bytes each (K rows, then
 * V rows). The sections of other subsystems (linear-layer state, MTP rows, n-gram state, index blocks,
 * rings) are written with zero counts; esp_kv_slot_load refuses files that carry them
 * (ESP_ERR_UNSUPPORTED) and, like the reference, files whose geometry or size does not match
 * (ESP_ERR_INVALID). region_bytes = bytes between the layer regions of the pool; a block's bytes sit at
 * layer * region_bytes + block * block_bytes. Both calls allocate staging buffers (up to 64 MB on the
 * device and pinned on the host), synchronise the stream, and free them before they return.
 * Load takes ceil(len / bt) blocks from `pool` (ESP_ERR_CAPACITY "KV cache full" if it has fewer,
 * leaving it unchanged) and reports them in blocks_out.
 * ESP_E4M3 pools (an extension; the reference has no FP8 KV cache): pass the scale table of layer 0
 * in kv_scales ([n_blocks][2][Hkv] fp32 per layer, the layers' tables scales_region_floats apart) and
 * Hkv. The file then carries, behind the blocks, the 2 * Hkv scales of every block of the list for
 * every layer, and says so in the header word the reference leaves at zero (`pad` = scale bytes per
 * block and layer); load restores them into the rows of the blocks it allocated, so the sequence
 * decodes with its own scales whatever used those blocks before. With kv_scales == NULL (16-bit
 * pools) the file is the reference's, byte for byte; a file written with scales is refused by a pool
 * without them and the other way round (ESP_ERR_INVALID). */
typedef struct esp_kv_pool esp_kv_pool;
int esp_kv_slot_save(const char* path, void* stream, const void* kv, const int32_t* blocks_host, int32_t len, int32_t next_pos,
                     int32_t bt, int32_t n_layers, uint64_t region_bytes, uint64_t block_bytes, const float* kv_scales,
                     int32_t Hkv, uint64_t scales_region_floats);
int esp_kv_slot_load(const char* path, void* stream, void* kv, esp_kv_pool* pool, int32_t* blocks_out, int32_t blocks_cap,
                     int32_t* n_blocks, int32_t* len, int32_t* next_pos, int32_t bt, int32_t n_layers, uint64_t region_bytes,
                     uint64_t block_bytes, float* kv_scales, int32_t Hkv, uint64_t scales_region_floats);

/* ---- attn_prep: the step right before the attention pass (kernels/40_attention.metal:23-102, host
 * dispatch src/model/impl/forest.h:2951-2977; generic head dim q3m_attn_prep,
 * kernels/82_qwen3_omni.metal:40-88). Per (row, head) of the fused projection X (fp32):
 * RMSNorm over the head (x * rsqrt(mean x^2 + eps) * weight), rotary embedding of the pairs
 * (d, d + rot_half) for d < rot_half at angle pos[sel[d]] * inv_freq[d] (M-RoPE: pos is an int4 per
 * row - temporal, height, width, unused - and sel[d] in {0, 1, 2} picks the component), queries times
 * qscale, cast to the context's q_dtype into Q / Kb; values are cast into Vb unchanged. With `ktab`
 * (int4 per row: block, pos, block2, pos2; -1 = none) the row's K / V are also written into the paged
 * pool (kv_save folded in; E4M3 pools quantise the rounded 16-bit value with the block's scale, exactly
 * as esp_kv_save would).
 * Layouts: the 256-dim reference kernel reads query head h at X + h * 2 * HD (the gate follows each
 * head: q_stride = 2 * HD), rotates 64 dims (rot_half = 32) and leaves the scale to the attention
 * kernel (qscale = 1); the generic kernel has q_stride = HD, rot_half = HD / 2 and folds the scale. */
typedef struct esp_attn_prep_params {
  int32_t H;
  int32_t Hkv;
  int32_t ld;       /* row stride of X in floats */
  int32_t q_off;    /* column of query head 0 */
  int32_t q_stride; /* floats between consecutive query heads: HD, or 2 * HD with interleaved gates */
  int32_t k_off;    /* column of key head 0 (heads HD apart) */
  int32_t v_off;    /* column of value head 0 (heads HD apart) */
  int32_t q_ld;     /* Q row stride in elements */
  int32_t kv_ld;    /* Kb / Vb row stride and pool row width in elements */
  int32_t rot_half; /* frequencies: dims [0, 2 * rot_half) rotate, the rest pass through; a power of two, <= HD / 2 */
  float eps;
  float qscale;
  int32_t bt;       /* tokens per KV block (ktab) */
  int32_t reserved;
  uint64_t kv_base; /* element offset of the layer's region in the pool (ktab) */
} esp_attn_prep_params;

int esp_attn_prep(esp_attn_ctx* ctx, void* stream, const float* X, const float* q_norm_w, const float* k_norm_w,
                  const int32_t* pos, const float* inv_freq, const int32_t* rope_sel, void* Q, void* Kb, void* Vb,
                  const int32_t* ktab, void* kv, const float* kv_scales, int32_t rows, const esp_attn_prep_params* p);

/* kv_save (40_attention.metal:875-889; forest.h:2935-2947). With an ESP_E4M3
 * pool the rows are quantised with the destination block's scale from kv_scales. */
int esp_kv_save(esp_attn_ctx* ctx, void* stream, const void* Kb, const void* Vb, void* kv, const float* kv_scales,
                const esp_kv_save_entry* entries, int32_t n_entries, const esp_attn_params* p);

/* kv_copy_blocks (40_attention.metal:894-905; forest.h:1438-1449): pairs =
 * (src block, dst block) int32 x 2, copied in each of n_layers regions
 * region_elems apart. */
int esp_kv_copy_blocks(esp_attn_ctx* ctx, void* stream, void* kv, const int32_t* pairs, int32_t n_pairs,
                       const esp_attn_params* p, uint64_t region_elems, int32_t n_layers);

/* ------------------------------------------------- KV blocks and row metadata (host) */
/* Pure host functions (no GPU needed): the integer bookkeeping run_forest does before it
 * encodes a pass. */

/* Refcounted block pool: KVPool::ref / free_list with kv_alloc / kv_retain / kv_release
 * (src/model/impl/model.h:387-411, :722-737; set-up forest.h:51-62: block 0 is handed out
 * first). esp_kv_alloc fails with ESP_ERR_CAPACITY ("KV cache full") when no block is free. */
/* esp_kv_pool: declared above, with the checkpoint functions. */
int esp_kv_pool_create(esp_kv_pool** out, int32_t n_blocks, int32_t bt);
int esp_kv_pool_destroy(esp_kv_pool* pool);
int32_t esp_kv_free_count(const esp_kv_pool* pool);
int32_t esp_kv_refcount(const esp_kv_pool* pool, int32_t block);
int esp_kv_alloc(esp_kv_pool* pool, int32_t* block);
int esp_kv_retain(esp_kv_pool* pool, int32_t block);
int esp_kv_release(esp_kv_pool* pool, int32_t block);

/* Forest::target_blocks (forest.h:1785-1811): the block list of a target that continues a
 * parent list covering [0, P) and writes positions [w0, end). Blocks entirely below w0 are
 * shared (retained), the rest are new; a new block that replaces a parent block holding
 * positions below P is reported as a copy-on-write pair (src, dst); an in-place append keeps
 * a partial block it owns alone. If the pool cannot supply every new block the call fails
 * with ESP_ERR_CAPACITY and leaves the pool unchanged (the reference releases them through
 * its PassGuard, forest.h:2468-2482). With out_blocks == NULL only the counts are reported. */
int esp_kv_target_blocks(esp_kv_pool* pool, const int32_t* parent_blocks, int32_t n_parent, int32_t P, int32_t w0, int32_t end,
                         int32_t in_place, int32_t* out_blocks, int32_t out_cap, int32_t* n_out, int32_t* cow_pairs,
                         int32_t cow_cap, int32_t* n_cow);
/* target_new_blocks (forest.h:1819-1829): how many blocks the call above would allocate. */
int32_t esp_kv_target_new_blocks(const esp_kv_pool* pool, const int32_t* parent_blocks, int32_t n_parent, int32_t P, int32_t w0,
                                 int32_t end, int32_t in_place);
/* The kv_save records of rows [base_row, base_row + n_rows) written at positions P, P + 1, ...
 * of a block list (add_saves, forest.h:2488-2499). */
int esp_kv_save_entries(const int32_t* blocks, int32_t n_blocks_list, int32_t bt, int32_t P, int32_t base_row, int32_t n_rows,
                        esp_kv_save_entry* out);
/* kv_row_table (forest.h:1739-1749): per row the (block, pos) x 2 its K/V go to, -1 = none;
 * table holds max(rows, 1) * 4 ints. A row saved into more than two slots is an error. */
int esp_kv_row_table(const esp_kv_save_entry* entries, int32_t n, int32_t rows, int32_t* table);

/* One tree of a pass, as far as attention is concerned (TreeSpec, src/model/api.h:105-176). */
typedef struct esp_tree_spec {
  const int32_t* root;         /* root_len tokens */
  int32_t root_len;
  int32_t n_leaves;
  const int32_t* root_pos;     /* [root_len][3] M-RoPE positions, or NULL */
  const int32_t* leaf_offsets; /* n_leaves + 1 */
  const int32_t* leaf_tokens;
  int32_t noncausal;           /* root rows see the whole root (no leaves allowed) */
  int32_t score_root;          /* one more readout at the root's last row */
} esp_tree_spec;

/* Rows of one tree (forest.h:2201-2220 leaf hosting, :2374-2442 records): host[i] = the leaf
 * whose rows leaf i is read from (a leaf that is a prefix of another is not given rows),
 * off[i] = first leaf row of a hosting leaf relative to the end of the root; per row tok,
 * pos (int4: t, h, w, 0; the root continues at pnext, leaf rows at next_root + j) and desc
 * (int4: seg_start, 0, anc_len, 0 relative to the tree's first row); readout_rows = the
 * absolute last row of every leaf, then the root's when score_root or there are no leaves.
 * base = absolute first row of the tree. */
int esp_forest_tree_rows(const esp_tree_spec* spec, int32_t base, int32_t pnext, int32_t* host, int32_t* off, int32_t* tok,
                         int32_t* pos4, int32_t* desc4, int32_t* readout_rows, int32_t rows_cap, int32_t* n_rows,
                         int32_t* next_root);
/* Ancestor masks of a general draft tree (node i's parent < i, -1 for a root): bit j of
 * masks[i] = node j is node i or one of its ancestors. The input of ESP_ATTN_FLAG_ANC_MASK. */
int esp_forest_anc_masks(const int32_t* parents, int32_t n, uint64_t* masks);

/* Decode attention for callers that cannot allocate device memory when they run it: an
 * engine that gave the whole GPU to one arena at start-up, a plugin inside a process whose
 * allocator owns the device, a serving loop that forbids cudaMalloc / cudaFree (and the
 * device-wide synchronisation cudaFree implies) after warm-up. It has no counterpart in
 * the reference, whose passes always draw `parts` from a growable arena
 * (meta.parts.ensure, src/model/impl/forest.h:2716).
 *
 * Same computation and results as esp_attn_forward for single-row trees (decode kernel,
 * then the combine jobs), but it needs no context and no `parts` buffer: the split-K
 * records go to an array of ESP_ATTN_STATIC_PARTS_FLOATS floats (16 MiB) that is part of
 * the library's device image - every GPU that loads the library holds it until the
 * process exits. args->parts and args->n_parts are ignored; inputs, outputs and the plan
 * (device and host copies) are passed as for esp_attn_forward. Limits and rules:
 *  - a pass whose records need more than the array holds (the largest record a tile writes or a
 *    combine job reads, + 1, times Hkv * tile_rows * G * (HD + 2) floats) is refused with
 *    ESP_ERR_CAPACITY; shapes the decode kernel does not cover and multi-row trees are refused
 *    with ESP_ERR_UNSUPPORTED; a plan that fails the host checks of esp_attn_forward (trees, tiles
 *    and jobs against the row, block-table and record counts; the host copies tiles_host,
 *    trees_host and - with combine jobs - jobs_host are required) with ESP_ERR_INVALID. Nothing
 *    is launched in any of these cases. A tile may start at any key.
 *  - the call allocates nothing: no cudaMalloc / cudaFree, no allocating library routine.
 *  - the first call on each device (with that device current) looks up the array's device
 *    address and raises the kernels' shared-memory limit; make that call before any stream
 *    capture begins. Host threads that race to make it are serialised by a lock.
 *  - all calls on a GPU share the one array, which keeps the previous call's records:
 *    nothing in it needs clearing (each call overwrites every record it later reads), but
 *    two calls that overlap on the GPU (different streams, or different threads) race on
 *    it - serialise them on one stream.
 *  - failures on the device: the kernels' waits are bounded; one that runs out leaves a code in a
 *    status word next to the array and the pass's output is not valid.
 *    esp_attn_decode_static_status(stream) reads and clears that word for the current device
 *    (ESP_OK, or ESP_ERR_CUDA with the reason); it synchronises the stream and allocates nothing,
 *    so call it at a checkpoint, not per pass. */
#define ESP_ATTN_STATIC_PARTS_FLOATS (4u << 20)
int esp_attn_decode_static(const esp_attn_shape* shape, void* stream, const esp_attn_args* args);
int esp_attn_decode_static_status(void* stream);

/* ---- Qwen sparse attention (kernels/45_qsa.metal; host src/model/impl/forest.h:1462-1676): a query row at
 * sequence index s sees s + 1 tokens; once its nb = (s + 1) / 4 complete blocks of 4 tokens exceed 512 it attends
 * only the 512 blocks its indexer scores highest plus its tail (the tokens past 4 nb). This library takes the
 * indexer's scores as an input (computing them - qsa_prep, qsa_pool, qsa_score_* - is the model's projection work)
 * and provides everything from there: the per-row records and tiles (esp_qsa_plan = qsa_plan, forest.h:1489-1543),
 * the planner branch for such tiles (esp_attn_plan_qsa = plan_tiles with `qt`, forest.h:1392-1412), the top-512
 * selection (esp_qsa_select = qsa_select: radix select on the fp32 bit patterns, ties to the lowest blocks), the
 * tiles' union lists (esp_qsa_tiles = qsa_tiles) and the attention over them (esp_attn_forward with the qsa_*
 * arguments = flash_attention_qsa). All integer results are bit-identical to the reference's. */
#define ESP_QSA_TOPK 512
#define ESP_QSA_LMAX 4112 /* union entries per 8-row tile (QSA_LMAX) */
typedef struct esp_qsa_tile {
  int32_t tree;
  int32_t r0;   /* absolute first row */
  int32_t rows; /* <= 8 */
  int32_t pad;
} esp_qsa_tile;
typedef struct esp_qsa_counts {
  int32_t M;        /* pass rows covered by the trees */
  int32_t n_sparse; /* rows with nb > 512 */
  int32_t nbmax;    /* largest nb of a sparse row: row stride of `scores` */
  int32_t nbb;      /* most blocks of a sparse row that end in pass rows */
  int32_t ncb;      /* most cached blocks (P / 4) of a tree with sparse rows */
  int32_t n_tiles;  /* 8-row tiles that hold sparse rows */
} esp_qsa_counts;
/* qsa_plan (pure host). desc: int4 per row (segment start, 0, root rows, 0) or NULL for chains; sparse = 0: records
 * only (no row is sparse). Outputs: rinfo int4 per row [0, M); srows (the pass row of each sparse row); qtiles; qt_of:
 * per tree, per 8-row group, its tile or -1, flattened (the `qt` of esp_attn_plan_qsa). Arrays may be NULL to size
 * them: counts is always filled; ESP_ERR_CAPACITY if a given array is too small. */
int esp_qsa_plan(const esp_attn_tree* trees, int32_t n_trees, const int32_t* desc, int32_t sparse, int32_t* rinfo, int32_t rows_cap,
                 int32_t* srows, int32_t srows_cap, esp_qsa_tile* qtiles, int32_t qtiles_cap, int32_t* qt_of, int32_t qt_cap,
                 esp_qsa_counts* counts);
/* plan_tiles with its sparse branch (forest.h:1378-1433): opts->mode must be ESP_PLAN_REFERENCE and tile_rows 8; qt as
 * esp_qsa_plan's qt_of (NULL: exactly esp_attn_plan). A group with qt >= 0 gets tiles over entries of list qt (pad0 = 1,
 * pad1 = qt; the last part open-ended: the list's length is known only on the device). */
int esp_attn_plan_qsa(const esp_attn_tree* trees_host, int32_t n_trees, int32_t Hkv, const esp_plan_opts* opts, const int32_t* qt,
                      esp_attn_tile* tiles_host, int32_t tiles_cap, esp_attn_combine* jobs_host, int32_t jobs_cap, int32_t* n_tiles,
                      int32_t* n_jobs, int32_t* n_parts);
/* qsa_select: scores [n_sparse][nbmax] fp32 >= 0 -> sel [n_sparse][nbw] bitmaps (nbw = (nbmax + 31) / 32). One launch. */
int esp_qsa_select(void* stream, const float* scores, const int32_t* srows, const int32_t* rinfo, uint32_t* sel, int32_t n_sparse,
                   int32_t nbmax, int32_t nbw);
/* qsa_tiles: per tile the cached blocks any of its rows reads -> tlist [n_qtiles][ESP_QSA_LMAX], tcount [n_qtiles]. One launch. */
int esp_qsa_tiles(void* stream, const uint32_t* sel, const esp_attn_tree* trees, const int32_t* rinfo, const esp_qsa_tile* qtiles,
                  int32_t n_qtiles, uint32_t* tlist, uint32_t* tcount, int32_t nbmax, int32_t nbw);

/* ---- NaN / Inf / outlier detector, for debugging: the reference's finite_check
 * (src/model/impl/finite_check.h:4-18, kernels/05_finite_check.metal; the attention output is its site
 * "attn_out", src/model/impl/forest.h:4019-4047). Scans rows x cols elements of x (row stride ld, in
 * elements) and fills the caller's device record: hits = offending elements, idx = the smallest
 * offending index (row * cols + col; 0xFFFFFFFF if none), done = blocks finished, val = that element's
 * value as fp32 bits. An element offends when its |x| bits are >= those of `threshold` (NaN and Inf
 * always; pass INFINITY for only those). Two small launches on the stream; nothing is allocated.
 * With the context option "check_finite" = 1 esp_attn_forward runs this check over the pass's O rows
 * into a record of the context and esp_attn_check_status reports the first offender (ESP_ERR_CUDA,
 * "attn_out: ..."); off by default: nothing is launched and the bits are the same. */
typedef struct esp_finite_rec {
  uint32_t hits;
  uint32_t idx;
  uint32_t done;
  uint32_t val;
} esp_finite_rec;
enum { ESP_FINITE_F32 = 0, ESP_FINITE_F16 = 1, ESP_FINITE_BF16 = 2 };
int esp_attn_finite_check(void* stream, const void* x, uint32_t rows, uint32_t cols, uint64_t ld, int32_t dtype, float threshold,
                          esp_finite_rec* rec_device);

/* Name of the attention kernel the last esp_attn_forward on this context
 * launched ("decode_gqa", "flash_umma", "flash_umma_pair", "flash_umma_duo", "flash_general"), for tests and traces. */
const char* esp_attn_last_kernel(const esp_attn_ctx* ctx);

/* Reads and clears the context's device status word: a kernel whose bounded wait ran
 * out (a TMA load or an MMA that never completed) leaves a code there instead of
 * spinning. Synchronises the stream: for tests and post-mortems, not the hot path. */
int esp_attn_check_status(esp_attn_ctx* ctx, void* stream);

/* Timeline of one CTA, for tuning (the reference's counterpart is set_profile,
 * src/model/model.mm:1041-1054, which times whole dispatches): with a caller-owned device
 * buffer of (n_blocks + 1) * 8 uint64 set, CTA (0, 0) of the tcgen05 kernel stores
 * %globaltimer nanoseconds per key block b at [8 * b + e]: e = 0 scores ready (softmax side),
 * 1 scores in registers, 2 P handed over, 3 P seen by the MMA thread, 4 V tile seen,
 * 5 MMAs of the block issued, 6 K tile requested, 7 V tile requested; slot 8 * n_blocks holds
 * the CTA's start and slot 8 * n_blocks + 1 its end. n_blocks = 0 switches tracing off.
 * flash_umma over an E4M3 pool: 6 / 7 = the block's K / V tile converted. flash_umma_duo (two query tiles):
 * 0 / 1 / 2 = tile 0's scores ready, row maxima known, P handed over; 3 / 4 = P of tile 0 / tile 1 seen by the MMA
 * thread; 5 as above; 6 / 7 = tile 1's scores ready, P handed over; the table's last row (b = n_blocks - 1) holds
 * phases of the CTA instead: 0 plan read, 1 set-up done, 2 last P handed over, 3 rows written.
 * With the option "trace_ctas" = N (> 0) the flash_umma kernel also stores four stamps for each of
 * its first N CTAs (linear CTA index c) at [8 * n_blocks + 2 + 4 * c + e]: e = 0 start, 1 first
 * scores seen, 2 last block handed over, 3 exit; the buffer must then hold
 * 8 * n_blocks + 2 + 4 * N values. flash_umma_pair stores at the same place: e = 0 start, 1 last block's
 * O complete, 2 records published (passes that merge inside the kernel), 3 exit. */
int esp_attn_set_trace(esp_attn_ctx* ctx, void* device_buffer, int32_t n_blocks);
/* Enqueue a one-thread kernel that stores %globaltimer (the trace's clock) into *device_slot:
 * before and after a pass it brackets the pass in the trace's time base. */
int esp_attn_stamp(void* stream, uint64_t* device_slot);

/* Per-dispatch GPU time, as NativeModel::set_profile / profile_json (src/model/model.mm:1041-1054: every dispatch timed
 * on its own, summed per kernel). esp_attn_set_profile(ctx, 1) clears the sums and makes every later launch of the
 * context's entry points carry a CUDA event pair; esp_attn_get_profile waits for the pairs recorded so far and reports,
 * per kernel name, its launches and summed milliseconds (n = kernels; ESP_ERR_CAPACITY if cap is too small). Timing
 * events keep consecutive kernels from overlapping (programmatic dependent launch), so a profiled pass is slower
 * than an unprofiled one: a tool for shares, like the reference's. Off by default: nothing is recorded. */
typedef struct esp_attn_profile_entry {
  char kernel[32];
  uint32_t launches;
  float gpu_ms;
} esp_attn_profile_entry;
int esp_attn_set_profile(esp_attn_ctx* ctx, int on);
int esp_attn_get_profile(esp_attn_ctx* ctx, esp_attn_profile_entry* out, int32_t cap, int32_t* n);

/* Kernel launches enqueued by this context since creation. */
uint64_t esp_attn_launch_count(const esp_attn_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* ESPETERO_ATTN_H */
