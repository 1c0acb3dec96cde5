// Forest attention for 128-row tiles on the 5th-generation tensor cores (sm_100a):
// causal prefill, the batched tree-verify pass and any other multi-row tile.
//
// Computes what flash_attention computes (kernels/40_attention.metal:156-343 of the
// reference; generic head dim kernels/80_gemma.metal:157-342): the tile's rows attend to the
// cached key range [k0, k1) of the paged pool and, when tile.last, to the visible batch keys
// of their tree (two-level `desc` mask or a 64-bit ancestor mask per row), writing either
// the partial record [O | m | l] or the gated, normalised output (and its LSE).
//
// B200 structure. One CTA per SM = 128 (query row, head) pairs = the 128 lanes of tensor
// memory: tile_rows rows x (128 / tile_rows) heads of one kv head (16 nodes x 8 heads for a
// verify tile, 128 rows x 1 head for prefill). Keys are processed 128 at a time:
//   S[128 x 128]  = Q . K^T      8 tcgen05.mma (N = 128, K = 16), A = Q tile and B = K tile from
//                                shared memory (K-major, 128-byte swizzle), D in tensor memory
//   softmax        two warpgroups, one per 64-key half of the block; thread (i, half) owns row
//                  i of its half: tcgen05.ld of 64 scores, mask, online max / sum in the exp2
//                  domain (no shuffles), P as bf16 / fp16 pairs back into tensor memory over
//                  the scores it has read (tcgen05.st)
//   O_h[128 x HD] += P_h . V_h    4 tcgen05.mma per half with A = P from tensor memory, B = the
//                                half's 64 V rows from shared memory (MN-major); every half
//                                has its own accumulator and its own (m, l), merged at the end
// Two S buffers let Q.K^T of block b + 1 run while the softmax works on block b. O stays in
// tensor memory for the whole tile and is rescaled only when a row's maximum has grown by more
// than 2^8 since its reference value (warp-uniform decision), so the common step has no
// accumulator traffic. K and V tiles go through 3-deep rings filled by TMA, one bulk tensor
// load per (16-key page, 64-dim half), rows found through the page table for cached keys and
// directly in Kb / Vb for batch keys: up to ~190 KB in flight per SM, enough to stream the
// pool at HBM speed. Warps: 0-3 softmax half A, 4-7 softmax half B, 8 MMA issue (one thread;
// owns tensor memory), 9 K producer, 10 V producer; they hand tiles to one another through
// mbarriers only (TMA complete_tx, tcgen05.commit, a 256-arrival barrier for P). The producers
// start before the Q tile is staged. Blocks that need no mask (all but the diagonal, the tail
// and tree blocks) take a path with no per-key predicate.
// Every wait is bounded: after a timeout the CTA records a status code, stops waiting,
// finishes its loop, frees its tensor memory and returns.
//
// E4M3 pools (template flag F8; the reference dequantises in its attention kernels too,
// kernels/80_dsv4.metal:22-33 for the codec): the pages arrive by TMA as raw codes (2 KB per page and
// kv head: half the bytes of a 16-bit pool) into rings of two 16 KB tiles; six converter warps (three
// for K, three for V, each taking every third page) turn them into fp16 tiles - code x the page's scale for
// the kv head, which the producer fetched while it waited for the slot - in the 128-byte-swizzled
// layout the MMAs read, and the whole pass computes in fp16 (Q is converted when it is staged, P is
// fp16; accumulation and the records stay fp32). One producer warp serves both rings (lanes 0-7 K,
// 8-15 V); with 16 warps the kernel runs in 128 registers per thread. Batch keys (the pass's own rows) are few in
// the passes this variant is for: the converter warps fetch them from Kb / Vb themselves.
#include "umma.cuh"
#include "../launch.h"

namespace esp {
namespace {

constexpr int BM = 128;  // (row, head) pairs per CTA
constexpr int BN = 128;  // keys per block
constexpr int BH = 64;   // keys per softmax half
constexpr int HD = 128;  // head dim of this kernel
constexpr int Q_BYTES = BM * HD * 2;        // [2 halves of 64 dims][128 rows][128 B]
constexpr int KV_TILE = BN * HD * 2;        // [2 halves of 64 dims][128 rows][128 B]
constexpr int HALF_T = 128 * 128;           // bytes between the 64-dim halves of a tile
constexpr int KS = 3, VS = 3;               // K and V ring depths
constexpr int KS8 = 2, RS8 = 2;             // E4M3 pools: converted tiles per ring, raw tiles per ring
constexpr int RAW_TILE = BN * HD;           // 128 keys x 128 codes
constexpr int TILES_BYTES = Q_BYTES + (KS + VS) * KV_TILE;
static_assert(Q_BYTES + 2 * KS8 * KV_TILE + 2 * RS8 * RAW_TILE == TILES_BYTES, "both layouts fill the same window");
constexpr int SMEM_BYTES = TILES_BYTES + 384;  // + mbarriers and bookkeeping; no static shared memory
constexpr uint32_t TMEM_COLS = 512;
// Two S buffers of 128 fp32 columns (the P of a half is written over the first 32 columns of that
// half's scores as 16-bit pairs), then one O accumulator of 128 fp32 columns per half.
constexpr uint32_t COL_S = 0, COL_O = 256;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

constexpr int kSoftmaxThreads = 2 * BM;     // warps 0-3: half A (keys 0-63 of a block), 4-7: half B
constexpr int kHintBlocks = 3;               // key blocks per CTA hinted into L2 ahead of the dependency wait (64 KB each; 8 measured slower)
constexpr int kMmaWarp = 8;                 // MMA issue (one thread), owns tensor memory
constexpr int kTmaWarpK = 9;                // TMA producer of K tiles (lanes 0-7, one 16-key page each)
constexpr int kTmaWarpV = 10;               // TMA producer of V tiles
constexpr int kThreads = 11 * 32;
constexpr int kCvtWarp0 = 10, kCvtWarps = 6;   // E4M3 pools: warp 9 produces both rings, warps 10-15 convert (even: K, odd: V)
constexpr int kThreadsF8 = (kCvtWarp0 + kCvtWarps) * 32;
constexpr int kCvtLanes = kCvtWarps / 2 * 32;  // converter lanes per tile
constexpr int kPages = BN / 16;             // TMA pages per tile

// The n lowest bits set (n <= 0: none, n >= 64: all).
__device__ __forceinline__ uint64_t low_bits64(int n) { return n <= 0 ? 0ull : (n >= 64 ? ~0ull : ((1ull << n) - 1ull)); }

struct PageRef {  // where one 16-key page of a key block comes from
  int raw;        // block id as loaded from the page table (pool), or first row (Kb / Vb)
  int off;        // row inside the block (pool)
  int kind;       // -1: nothing to load, 0: paged pool, 1: Kb / Vb
};

// Barriers and bookkeeping live behind the tiles in dynamic shared memory: with no static shared
// memory the dynamic window starts on a 1024-byte boundary (checked at run time), which the
// swizzled tiles need.
struct Shared {
  uint64_t k_full[KS], k_empty[KS], v_full[VS], v_empty[VS], s_full[2], p_full[2], pv_done, o_full, meta_ready;
  uint64_t raw_full[2][RS8], raw_empty[2][RS8];  // E4M3 pools: [K / V][slot]
  float scl[2][RS8][kPages];                     // ... the scale of each page in a raw slot
  uint32_t tmem_slot;
  int red[4];  // anc_max, seg_min, anc_min, seg_max
  volatile int dead;
};
static_assert(sizeof(Shared) <= 384, "bookkeeping must fit behind the tiles");

__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// Thread-block cluster: rank of this CTA, a barrier over every thread of the cluster (release / acquire), the
// address of a shared-memory location in another CTA of the cluster, and a 16-byte store to it.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map_shared(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f4(uint32_t addr, const float4& v) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

template <int QDT, bool F8>
__global__ void __launch_bounds__(F8 ? kThreadsF8 : kThreads, 1)
    flash_umma_kernel(const __grid_constant__ CUtensorMap pool_map, const __grid_constant__ CUtensorMap kb_map,
                      const __grid_constant__ CUtensorMap vb_map, const __grid_constant__ InlinePlan plan, const KernelArgs a) {
  using QE = Elem16<QDT>;                      // Q and O in memory
  constexpr int CDT = F8 ? ESP_F16 : QDT;      // what the MMAs compute in
  using PE = Elem16<CDT>;
  constexpr int KSx = F8 ? KS8 : KS, VSx = F8 ? KS8 : VS;
  extern __shared__ __align__(1024) uint8_t smem[];
  // full: TMA -> MMA; empty: MMA -> TMA (tcgen05.commit); s_full[i]: S buffer i written;
  // p_full[i]: both halves of P in buffer i written (256 arrivals); pv_done: P.V of a block
  // complete; o_full: last P.V done; meta_ready: the mask bounds of the tile are known
  Shared& sh = *reinterpret_cast<Shared*>(smem + TILES_BYTES);
  uint64_t* k_full = sh.k_full;
  uint64_t* k_empty = sh.k_empty;
  uint64_t* v_full = sh.v_full;
  uint64_t* v_empty = sh.v_empty;
  uint64_t* s_full = sh.s_full;
  uint64_t* p_full = sh.p_full;
  uint64_t& pv_done = sh.pv_done;
  uint64_t& o_full = sh.o_full;
  uint64_t& meta_ready = sh.meta_ready;
  uint32_t& tmem_slot = sh.tmem_slot;
  int* red = sh.red;
  volatile int& dead = sh.dead;
  if ((smem_u32(smem) & 1023u) != 0) {  // never expected; the tiles' swizzle would be wrong
    if (threadIdx.x == 0) atomicExch(a.status, kStatusBadBlock);
    return;
  }
  uint8_t* q_sm = smem;
  uint8_t* k_sm = smem + Q_BYTES;                  // KSx tiles
  uint8_t* v_sm = smem + Q_BYTES + KSx * KV_TILE;  // VSx tiles
  uint8_t* raw_sm = v_sm + VSx * KV_TILE;          // E4M3 pools: RS8 raw K tiles, then RS8 raw V tiles

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const esp_attn_params& p = a.p;
  const int tile_i = int(gridDim.x) - 1 - int(blockIdx.x);  // long (late) tiles first
  const TileStart& ts = plan.start[min(tile_i, kInlinePlanMax - 1)];
  const bool inl = ts.valid == tile_i + 1;  // small plan: everything for the first loads sits in one parameter line
  // The caller's promise (option "stable_cache"): the kernel before this pass writes neither the block table nor the
  // cached keys. With the plan in the parameters the producers then start fetching the cached key blocks while that
  // kernel still drains; the batch keys, Q and the mask records wait for it as ever.
  const bool early = inl && a.stable_cache != 0;
  esp_attn_tile tile;
  esp_attn_tree tree;
  if (inl) {
    tile = ts.tile;
    tree = ts.tree;
  } else {
    pdl_wait();  // the plan is read from device memory: no head start
    tile = a.tiles[tile_i];
    tree = a.trees[tile.tree];
  }
  const int32_t* page_table = inl ? ts.blocks : a.blocks;
  const int bt = inl ? int(ts.bt) : p.bt;
  const int G = inl ? int(ts.G) : a.G, TR = inl ? int(ts.tile_rows) : a.tile_rows, HPC = BM / TR;
  const int fix_parts = inl ? int(ts.fix_parts) : 0;  // > 0: the last CTA of this tile's merge job finishes the rows
  // Pair mode (a.fuse == 2): the two tiles of every job run as one thread-block cluster of two CTAs on neighbouring
  // SMs; the second CTA hands its record to the first through distributed shared memory and the first finishes the
  // rows - no record in global memory, no fence, no ticket. Uniform over the grid.
  const bool pair_mode = a.fuse == 2 && fix_parts == 2 && tile.part >= 0 && HPC == G;
  const int kvh = (int(blockIdx.y) * HPC) / G;
  const int end = tree.base + tree.M;
  const int rows_live = min(TR, end - tile.r0);
  const bool use_anc = a.anc_mask != nullptr;
  const bool desc_mask = tile.last && !use_anc;

  // per softmax thread: its (row, head) and its half of every key block
  const int srow = tid & (BM - 1), half = (tid >> 7) & 1;
  const int fm = srow / HPC, hh = srow % HPC;
  const int head = int(blockIdx.y) * HPC + hh;
  const bool is_softmax = tid < kSoftmaxThreads;
  const bool row_ok = is_softmax && fm < rows_live;
  const int row = row_ok ? tile.r0 + fm : end - 1;
  const int rr = row - tree.base;

  // ---- set-up, step 1: barriers, then everybody may start
  if (tid == 0) {
    for (int s = 0; s < KS; ++s) {
      mbar_init(&k_full[s], F8 ? kCvtLanes : kPages);  // E4M3 pools: the lanes of the tile's converter warps
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < VS; ++s) {
      mbar_init(&v_full[s], F8 ? kCvtLanes : kPages);
      mbar_init(&v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i)
      for (int s = 0; s < RS8; ++s) {
        mbar_init(&sh.raw_full[i][s], kPages);
        mbar_init(&sh.raw_empty[i][s], kCvtLanes);
      }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], kSoftmaxThreads);
    }
    mbar_init(&pv_done, 1);
    mbar_init(&o_full, 1);
    mbar_init(&meta_ready, 1);
    mbar_fence_init();
    red[0] = 0, red[1] = 1 << 30, red[2] = 1 << 30, red[3] = 0;
    dead = 0;
  }
  __syncthreads();

  auto wait_bar = [&](uint64_t* bar, uint32_t parity, int code) {
    if (mbar_try_wait(bar, parity)) return;  // the common case costs one shared-memory round trip
    if (dead) return;
    if (!mbar_wait(bar, parity)) {
      dead = 1;
      atomicExch(a.status, code);
    }
  };
  const bool tracing = a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
  auto stamp = [&](int b, int ev) {
    if (tracing && b < a.trace_blocks) a.trace[8 * b + ev] = global_timer_ns();
  };
  if (tracing && tid == 0) a.trace[8 * a.trace_blocks] = global_timer_ns();
  // Optional per-CTA stamps (start, first scores seen, last block handed over, exit) behind CTA 0's events.
  const int cta_lin = blockIdx.y * gridDim.x + blockIdx.x;
  const bool cta_tracing = a.trace != nullptr && cta_lin < a.trace_ctas;
  auto cta_stamp = [&](int ev) {
    if (cta_tracing) a.trace[8 * a.trace_blocks + 2 + 4 * cta_lin + ev] = global_timer_ns();
  };
  if (tid == 0) cta_stamp(0);

  // Block list: cached 128-key blocks first, then the batch blocks some row of the tile can see
  // (the latter depend on the rows' mask records: see `meta` below).
  const int nbc = (tile.k1 - tile.k0 + BN - 1) / BN;
  const int r_first = tile.r0 - tree.base, r_last = r_first + rows_live - 1;
  struct Meta {
    int k_last, a_hi, b_lo, nbb, anc_min, seg_max;
  };
  auto make_meta = [&]() {
    Meta m{-1, 0, 0, 0, 0, 0};
    if (!tile.last) return m;
    if (use_anc) {
      m.k_last = min(tree.M, 64) - 1;
      m.a_hi = (m.k_last + BN) / BN;
      m.nbb = m.a_hi;
      return m;
    }
    const int anc_max = red[0], seg_min = red[1];
    m.anc_min = red[2], m.seg_max = red[3];
    m.k_last = min(tree.M - 1, max(r_last, anc_max - 1));
    const int n_all = (m.k_last + BN) / BN;
    m.a_hi = min((anc_max + BN - 1) / BN, n_all);  // blocks below the ancestor range
    m.b_lo = max(m.a_hi, seg_min / BN);            // blocks of the rows' own segments
    const int b_hi = min(r_last / BN, n_all - 1);
    m.nbb = m.a_hi + max(0, b_hi - m.b_lo + 1);
    return m;
  };
  auto batch_j0 = [&](const Meta& m, int i) { return BN * (i < m.a_hi ? i : m.b_lo + (i - m.a_hi)); };

  if (F8 && warp == kTmaWarpK) {
    // ================= E4M3 pools: one producer warp for both raw rings (lanes 0-7 the K pages of a block, lanes 8-15
    // its V pages); batch blocks are left to the converter warps.
    if (lane == 0) tma_prefetch_desc(&pool_map);
    const int is_v = (lane >> 3) & 1, pg = lane & 7;
    uint64_t* full = sh.raw_full[is_v];
    uint64_t* empty = sh.raw_empty[is_v];
    uint8_t* ring = raw_sm + is_v * RS8 * RAW_TILE;
    int stage = 0;
    uint32_t par = 1;  // the first use of a slot finds it empty
    auto load_group = [&](int g) {
      const int b = 4 * g + (lane >> 3);
      const int j = tile.k0 + BN * b + 16 * (lane & 7);
      return (b < nbc && j < tile.k1) ? page_table[tree.table + j / bt] : -1;
    };
    if (!early) pdl_wait();
    int g_cur = load_group(0), g_nxt = load_group(1);
    for (int b = 0; b < nbc; ++b) {
      if (b && (b & 3) == 0) {
        g_cur = g_nxt;
        g_nxt = load_group((b >> 2) + 1);
      }
      const int raw = __shfl_sync(0xffffffffu, g_cur, ((b & 3) << 3) | pg);
      if (lane < 2 * kPages) {
        const bool ok = raw >= 0 && raw < a.n_blocks;
        float sc = 0.0f;  // the page's scale for this kv head: on its way while the lane waits for the slot
        if (ok) sc = a.kv_scales[(size_t(raw) * 2 + is_v) * p.Hkv + kvh];
        wait_bar(&empty[stage], par, kStatusMmaTimeout);
        if (!ok) {
          mbar_arrive(&full[stage]);
        } else {
          sh.scl[is_v][stage][pg] = sc;
          const int y = (raw * 2 + is_v) * bt + (tile.k0 + BN * b + 16 * pg) % bt;
          mbar_arrive_expect_tx(&full[stage], 2048);
          tma_load_3d(ring + stage * RAW_TILE + pg * 2048, &pool_map, &full[stage], 0, y, kvh);
        }
        if (++stage == RS8) stage = 0, par ^= 1;
      }
    }
  } else if (F8 && warp >= kCvtWarp0) {
    // ================= E4M3 pools: converter warps. Warps 10, 12, 14 turn raw K tiles into fp16 K tiles, 11, 13, 15 do
    // V (spread over the four schedulers: the conversion instruction runs on the exp2 unit's pipe); a warp takes
    // every third 16-key page of a block. A row's 128 codes are 8 chunks of 16 in the raw tile's 128-byte line and
    // become 16 chunks of 8 halves in the two 64-dim halves of the 16-bit tile.
    const int is_v = (warp - kCvtWarp0) & 1, wi = (warp - kCvtWarp0) >> 1;
    uint64_t* full = is_v ? v_full : k_full;
    uint64_t* empty = is_v ? v_empty : k_empty;
    uint8_t* ring = is_v ? v_sm : k_sm;
    const uint8_t* raw_ring = raw_sm + is_v * RS8 * RAW_TILE;
    if (!early) pdl_wait();
    if (desc_mask) wait_bar(&meta_ready, 0, kStatusMmaTimeout);  // (arrives after the softmax warps' own dependency wait)
    const Meta m = make_meta();
    const int nb = nbc + m.nbb;
    int rst = 0, cst = 0;
    uint32_t rpar = 0, cpar = 1;  // the first use of a converted slot finds it empty
    for (int b = 0; b < nb; ++b) {
      const bool cached = b < nbc;
      const int j0 = cached ? tile.k0 + BN * b : batch_j0(m, b - nbc);
      const int n_valid = cached ? min(BN, tile.k1 - j0) : min(BN, m.k_last + 1 - j0);
      if (cached) wait_bar(&sh.raw_full[is_v][rst], rpar, kStatusTmaTimeout);
      else if (early && b == nbc) pdl_wait();  // the batch keys are what the kernel before this pass has written
      wait_bar(&empty[cst], cpar, kStatusMmaTimeout);
      uint8_t* dst = ring + cst * KV_TILE;
      // a warp takes whole 16-key pages: lane l converts half of row (l % 16) of the page - 4 of its 8 raw chunks
#pragma unroll 1
      for (int pg = wi; pg < kPages; pg += kCvtWarps / 2) {
        const int r = 16 * pg + (lane & 15), cg = lane >> 4;
        uint8_t* drow = dst + r * 128 + cg * HALF_T;  // codes 64 cg .. 64 cg + 63 = the dims of half cg
        if (r >= n_valid) {
          // rows past the range: zeros (stale bytes could be NaN patterns, and 0 x NaN must not happen)
#pragma unroll
          for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(drow + ((c ^ (r & 7)) << 4)) = make_uint4(0, 0, 0, 0);
        } else if (cached) {
          const uint8_t* srow = raw_ring + rst * RAW_TILE + r * 128;
          const __half2 sc2 = __float2half2_rn(sh.scl[is_v][rst][pg]);
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const int c = 4 * cg + cc;  // the row's raw chunk: codes 16 c .. 16 c + 15
            const uint4 v = *reinterpret_cast<const uint4*>(srow + ((c ^ (r & 7)) << 4));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t h[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t lo = e4m3x2_to_f16x2(uint16_t(w[i] & 0xFFFFu)), hi = e4m3x2_to_f16x2(uint16_t(w[i] >> 16));
              __half2 a2 = __hmul2(*reinterpret_cast<__half2*>(&lo), sc2), b2 = __hmul2(*reinterpret_cast<__half2*>(&hi), sc2);
              h[2 * i] = *reinterpret_cast<uint32_t*>(&a2), h[2 * i + 1] = *reinterpret_cast<uint32_t*>(&b2);
            }
            // ... = the 16-byte chunks 2 cc and 2 cc + 1 of the half's 128-byte line
            *reinterpret_cast<uint4*>(drow + (((2 * cc) ^ (r & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<uint4*>(drow + (((2 * cc + 1) ^ (r & 7)) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
          }
        } else {
          // a batch key: the pass's own row, in the Q type
          const uint4* src = reinterpret_cast<const uint4*>(static_cast<const typename QE::T*>(is_v ? a.Vb : a.Kb) +
                                                            size_t(tree.base + j0 + r) * p.kv_ld + size_t(kvh) * HD) + 8 * cg;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint4 v = src[c];
            if constexpr (QDT == ESP_BF16) {
              uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 f = QE::unpack2(w[i]);
                w[i] = PE::pack2(f.x, f.y);
              }
            }
            *reinterpret_cast<uint4*>(drow + ((c ^ (r & 7)) << 4)) = v;
          }
        }
      }
      fence_proxy_async_smem();
      if (cached) {
        mbar_arrive(&sh.raw_empty[is_v][rst]);
        if (++rst == RS8) rst = 0, rpar ^= 1;
      }
      mbar_arrive(&full[cst]);
      if (lane == 0 && wi == 0) stamp(b, is_v ? 7 : 6);  // timeline: the block's K / V tile converted
      if (++cst == KS8) cst = 0, cpar ^= 1;
    }
  } else if (!F8 && (warp == kTmaWarpK || warp == kTmaWarpV)) {
    // ================= TMA producers: warp 9 fills the K ring, warp 10 the V ring, each on its own
    // schedule (a K tile is free as soon as its Q.K^T is done, a V tile only after its P.V);
    // lane w loads the w-th 16-key page of every block. They start right after the barriers
    // exist: the cached blocks do not depend on the Q tile or on the mask records.
    if (warp == kTmaWarpK && lane == 0) {
      tma_prefetch_desc(&pool_map);
      tma_prefetch_desc(&kb_map);
      tma_prefetch_desc(&vb_map);
    }
    {
      const bool is_v = warp == kTmaWarpV;
      const int depth = is_v ? VS : KS;
      uint64_t* full = is_v ? v_full : k_full;
      uint64_t* empty = is_v ? v_empty : k_empty;
      uint8_t* ring = is_v ? v_sm : k_sm;
      const CUtensorMap* batch_map = is_v ? &vb_map : &kb_map;
      int stage = 0;
      uint32_t par = 1;  // the first use of a slot finds it empty
      auto issue = [&](const PageRef& r, int b) {  // lanes 0 .. kPages-1: one 16-key page each
        uint8_t* dst = ring + stage * KV_TILE + lane * 2048;
        wait_bar(&empty[stage], par, kStatusMmaTimeout);
        if (r.kind < 0) {
          mbar_arrive(&full[stage]);
        } else {
          const int y = r.kind ? r.raw : (r.raw * 2 + (is_v ? 1 : 0)) * bt + r.off;
          const CUtensorMap* m = r.kind ? batch_map : &pool_map;
          mbar_arrive_expect_tx(&full[stage], 4096);
          tma_load_3d(dst, m, &full[stage], 0, y, kvh * 2);
          tma_load_3d(dst + HALF_T, m, &full[stage], 0, y, kvh * 2 + 1);
        }
        if (lane == 0) stamp(b, is_v ? 7 : 6);
        if (++stage == depth) stage = 0, par ^= 1;
      };
      // Page-table entries are fetched by the whole warp, four key blocks per load (lane l holds
      // the entry of block 4 g + l / 8, page l % 8), two groups ahead of their use: at the start
      // one round trip to memory lets the first blocks go out back to back, and later the
      // load's latency never meets the issue loop.
      auto load_group = [&](int g) {
        const int b = 4 * g + (lane >> 3);
        const int j = tile.k0 + BN * b + 16 * (lane & 7);
        return (b < nbc && j < tile.k1) ? page_table[tree.table + j / bt] : -1;
      };
      // While the previous kernel of the stream drains (programmatic dependent launch), warm L2
      // with what the first key blocks need: the page-table lines and the tiles themselves. These
      // are hints through L2 only; the real loads below come after the wait, so a page table or a
      // pool the previous kernel was still writing costs nothing but a wasted hint.
      if (inl && nbc > 0) {
#pragma unroll 1
        for (int b = lane >> 3; b < min(nbc, kHintBlocks); b += 4) {
          const int j = tile.k0 + BN * b + 16 * (lane & 7);
          if (j >= tile.k1) break;
          const int raw = ld_cg_s32(page_table + tree.table + j / bt);
          if (raw >= 0 && raw < a.n_blocks) {
            const int y = (raw * 2 + (is_v ? 1 : 0)) * bt + j % bt;
            tma_prefetch_3d(&pool_map, 0, y, kvh * 2);
            tma_prefetch_3d(&pool_map, 0, y, kvh * 2 + 1);
          }
        }
      }
      if (!early) pdl_wait();  // everything above used only parameters, shared memory and hints
      int g_cur = load_group(0), g_nxt = load_group(1);
      for (int b = 0; b < nbc; ++b) {
        if (b && (b & 3) == 0) {
          g_cur = g_nxt;
          g_nxt = load_group((b >> 2) + 1);
        }
        const int raw = __shfl_sync(0xffffffffu, g_cur, ((b & 3) << 3) | (lane & 7));
        if (lane < kPages) {
          const PageRef r{raw, (tile.k0 + BN * b + 16 * lane) % bt, raw >= 0 ? 0 : -1};
          issue(r, b);
        }
      }
      if (early) pdl_wait();  // the batch keys are what the kernel before this pass has written
      if (tile.last && lane < kPages) {
        if (desc_mask) wait_bar(&meta_ready, 0, kStatusMmaTimeout);
        const Meta m = make_meta();
        for (int i = 0; i < m.nbb; ++i) {
          const int j = batch_j0(m, i) + 16 * lane;
          PageRef r{tree.base + j, 0, j <= m.k_last ? 1 : -1};
          issue(r, nbc + i);
        }
      }
    }
  } else {
    // ---- set-up, step 2 (softmax and MMA warps): tensor memory, Q tile, mask bounds
    if (warp == kMmaWarp) {
      tmem_alloc(&tmem_slot, TMEM_COLS);
      tmem_relinquish();
    }
    if (is_softmax && inl)  // hint: this thread's half of its Q row (128 bytes)
      prefetch_l2(static_cast<const typename QE::T*>(a.Q) + size_t(row) * p.q_ld + size_t(head) * HD + half * 64);
    pdl_wait();  // Q, the mask records and, later, O / the records belong to the stream's order
    int4 d = make_int4(0, 0, 0, 0);
    uint64_t am = 0;
    if (is_softmax) {
      // this thread's half of its Q row into the K-major swizzled tile
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const typename QE::T*>(a.Q) + size_t(row) * p.q_ld + size_t(head) * HD) + half * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint4 v = src[i];
        if constexpr (F8 && QDT == ESP_BF16) {  // the pass computes in fp16
          uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 f = QE::unpack2(w[k]);
            w[k] = PE::pack2(f.x, f.y);
          }
        }
        *reinterpret_cast<uint4*>(q_sm + half * HALF_T + srow * 128 + ((i ^ (srow & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      if (tile.last) {
        if (use_anc) am = a.anc_mask[row];
        else d = reinterpret_cast<const int4*>(a.desc)[row];
      }
      if (desc_mask && half == 0) {
        int v0 = d.z, v1 = d.x, v2 = d.z, v3 = d.x;
#pragma unroll
        for (int o = 16; o; o >>= 1) {
          v0 = max(v0, __shfl_xor_sync(0xffffffffu, v0, o));
          v1 = min(v1, __shfl_xor_sync(0xffffffffu, v1, o));
          v2 = min(v2, __shfl_xor_sync(0xffffffffu, v2, o));
          v3 = max(v3, __shfl_xor_sync(0xffffffffu, v3, o));
        }
        if (lane == 0) {
          atomicMax(&red[0], v0);
          atomicMin(&red[1], v1);
          atomicMin(&red[2], v2);
          atomicMax(&red[3], v3);
        }
      }
    }
    tc_fence_before_sync();
    named_barrier(1, kSoftmaxThreads + 32);  // softmax warps + the MMA warp
    tc_fence_after_sync();
    if (tid == 0 && desc_mask) mbar_arrive(&meta_ready);  // the producers may plan the batch blocks
    const Meta meta = make_meta();
    const int nb = nbc + meta.nbb;
    const uint32_t tmem = tmem_slot;

    if (warp == kMmaWarp) {
      // ================= MMA issuer (one thread)
      if (lane == 0 && nb > 0) {
        constexpr uint32_t idesc_qk = umma_idesc<CDT>(BM, BN, 0, 0);
        constexpr uint32_t idesc_pv = umma_idesc<CDT>(BM, HD, 0, 1);
        // Descriptors are built once: inside the loop a descriptor is the base plus a constant in
        // its address field (one thread issues everything, so every integer op here is latency).
        const uint64_t q_desc = umma_smem_desc(smem_u32(q_sm), 16, 1024);
        const uint64_t k_desc = umma_smem_desc(smem_u32(k_sm), 16, 1024);
        const uint64_t v_desc = umma_smem_desc(smem_u32(v_sm), HALF_T, 1024);
        int kst = 0, vst = 0;
        uint32_t kpar = 0, vpar = 0;
        auto issue_qk = [&](int b) {
          wait_bar(&k_full[kst], kpar, kStatusTmaTimeout);
          tc_fence_after_sync();
          const uint64_t kd = k_desc + uint64_t(kst * (KV_TILE >> 4));
          const uint32_t td = tmem + COL_S + (b & 1) * BN;
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint64_t off = uint64_t(((ks >> 2) * HALF_T + (ks & 3) * 32) >> 4);
            umma_ss(td, q_desc + off, kd + off, idesc_qk, ks > 0);
          }
          umma_commit(&k_empty[kst]);  // the K slot may be refilled once these MMAs are done
          umma_commit(&s_full[b & 1]);
          if (++kst == KSx) kst = 0, kpar ^= 1;
        };
        // S of block b + 1 is computed while the softmax warps work on block b (two S buffers);
        // MMAs run in issue order, so Q.K^T of block b + 2 overwrites buffer b & 1 only after
        // P.V of block b has read P from it.
        issue_qk(0);
        if (nb > 1) issue_qk(1);
        for (int b = 0; b < nb; ++b) {
          const int sb = b & 1;
          wait_bar(&p_full[sb], (b >> 1) & 1, kStatusMmaTimeout);  // both halves of P_b are in tensor memory
          stamp(b, 3);
          wait_bar(&v_full[vst], vpar, kStatusTmaTimeout);
          stamp(b, 4);
          tc_fence_after_sync();
          const uint64_t vd = v_desc + uint64_t(vst * (KV_TILE >> 4));
          const uint32_t tp = tmem + COL_S + sb * BN;
          const uint32_t acc = b > 0 ? 1u : 0u;
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int ks = 0; ks < BH / 16; ++ks)
              umma_ts(tmem + COL_O + h * HD, tp + h * BH + ks * 8, vd + uint64_t(((h * BH + ks * 16) * 128) >> 4), idesc_pv,
                      ks > 0 ? 1u : acc);
          umma_commit(&v_empty[vst]);
          umma_commit(&pv_done);
          if (++vst == VSx) vst = 0, vpar ^= 1;
          if (b + 2 < nb) issue_qk(b + 2);
          if (b + 1 == nb) umma_commit(&o_full);
          stamp(b, 5);
        }
      }
    } else {
      // ================= softmax: thread (i, half) owns row i of its half of S and of O_half
      const uint32_t t_lane = tmem + (uint32_t((warp & 3) * 32) << 16);  // this warp's quarter of the lanes
      const uint32_t t_o = t_lane + COL_O + half * HD;
      const float sl2 = a.scale * kLog2e;
      float m_ref = -INFINITY, l_run = 0.0f;  // m_ref in exp2 units of the scaled score
      int vst = 0;
      uint32_t vpar = 0;

      for (int b = 0; b < nb; ++b) {
        const int sb = b & 1;
        const bool cached = b < nbc;
        const int j0 = cached ? tile.k0 + BN * b : batch_j0(meta, b - nbc);
        const int n_valid = cached ? min(BN, tile.k1 - j0) : min(BN, meta.k_last + 1 - j0);
        bool need_mask = n_valid < BN;
        if (!cached) {
          if (use_anc) need_mask = true;
          else need_mask = need_mask || !((j0 + BN - 1 < meta.anc_min) || (j0 >= meta.seg_max && j0 + BN - 1 <= r_first));
        }
        wait_bar(&s_full[sb], (b >> 1) & 1, kStatusMmaTimeout);
        if (tid == 0) stamp(b, 0);
        if (tid == 0 && b == 0) cta_stamp(1);
        tc_fence_after_sync();
        const uint32_t t_s = t_lane + COL_S + sb * BN + half * BH;
        uint32_t sr[2][32];
        tmem_ld32(t_s, sr[0]);
        tmem_ld32(t_s + 32, sr[1]);
        tmem_wait_ld();
        if (tid == 0) stamp(b, 1);
        float mx = -INFINITY;
        if (need_mask) {
          // diagonal, tail and tree blocks: the visibility of this thread's 64 columns as one bit
          // mask (a few integer operations), then one select per score
          const int c0 = half * BH;
          uint64_t vm = low_bits64(n_valid - c0);
          if (!cached) {
            if (use_anc) {
              vm &= half == 0 ? am : 0ull;  // one block, j0 = 0
            } else {
              const int jb = j0 + c0;  // batch key of the half's first column
              vm &= low_bits64(d.z - jb) | (low_bits64(rr - jb + 1) & ~low_bits64(d.x - jb));  // j < d.z || d.x <= j <= rr
            }
          }
          const uint32_t vw[2] = {uint32_t(vm), uint32_t(vm >> 32)};
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const float sc = ((vw[h] >> c) & 1u) ? __uint_as_float(sr[h][c]) : -INFINITY;
              sr[h][c] = __float_as_uint(sc);
              mx = fmaxf(mx, sc);
            }
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int c = 0; c < 32; c += 2) mx = fmaxf(mx, fmaxf(__uint_as_float(sr[h][c]), __uint_as_float(sr[h][c + 1])));
        }
        mx *= sl2;  // scale > 0: the maximum commutes with the scaling
        // lazy rescale: keep the old reference maximum unless this block exceeds it by 2^8
        float factor = 1.0f;
        const bool grow = mx > m_ref + kRescaleThreshold;  // also the first finite maximum (m_ref = -inf)
        if (grow) {
          factor = fast_exp2(m_ref - mx);  // 0 when nothing was seen before
          m_ref = mx;
          l_run *= factor;
        }
        const float neg_m = m_ref == -INFINITY ? 0.0f : -m_ref;
        float ps0 = 0.0f, ps1 = 0.0f;
        uint32_t pk[32];
        // P is rounded to the pass's 16-bit type before P.V (the reference rounds it to fp16, 40_attention.metal:297;
        // a bf16 pass cannot do that: the MMA takes its A and B operands in one 16-bit format only - fp16 P
        // against bf16 V raised "illegal instruction" when it was tried).
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(sr[c >> 4][(2 * c) & 31]), sl2, neg_m));
          const float p1 = fast_exp2(fmaf(__uint_as_float(sr[c >> 4][(2 * c + 1) & 31]), sl2, neg_m));
          ps0 += p0;
          ps1 += p1;
          pk[c] = PE::pack2(p0, p1);
        }
        l_run += ps0 + ps1;
        tmem_st32(t_s, pk);  // over the scores this thread has already read
        if (b > 0) {
          wait_bar(&pv_done, (b - 1) & 1, kStatusMmaTimeout);  // the accumulators hold blocks 0 .. b-1 and are idle
          tc_fence_after_sync();
        }
        if (b > 0 && __any_sync(0xffffffffu, grow)) {
          // O_half of this warp's rows *= factor (1 for rows whose reference did not move)
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(t_o + 32 * c, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            tmem_st32(t_o + 32 * c, o);
          }
        }
        tmem_wait_st();
        if (!F8 && n_valid < BN) {  // (E4M3 pools: the converter warps write zeros there)
          // tail block: V rows past the range are stale or foreign bytes; 0 * NaN must not happen
          wait_bar(&v_full[vst], vpar, kStatusTmaTimeout);
          const int n = (BN - n_valid) * 16;  // 16-byte chunks: 2 dim halves x 8 per row
          for (int i = tid; i < n; i += kSoftmaxThreads) {
            const int r = n_valid + i / 16, c = i % 16;
            *reinterpret_cast<uint4*>(v_sm + vst * KV_TILE + (c >> 3) * HALF_T + r * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
        }
        if (++vst == VSx) vst = 0, vpar ^= 1;
        tc_fence_before_sync();
        mbar_arrive(&p_full[sb]);
        if (tid == 0) stamp(b, 2);
      }

      // ---- epilogue: merge the two halves of every row, then write
      if (tid == 0) cta_stamp(2);
      pdl_launch_dependents();  // the next grid of the stream (the combine) may be scheduled
      if (nb > 0) {
        wait_bar(&o_full, 0, kStatusMmaTimeout);
        tc_fence_after_sync();
      }
      // The rings are idle now (every tile was consumed by an MMA that has completed): their
      // memory stages the halves' (m, l) and, for contiguous records, the records themselves.
      float2* xch = reinterpret_cast<float2*>(k_sm);
      float* stage = reinterpret_cast<float*>(k_sm + 4096);
      xch[half * BM + srow] = make_float2(m_ref, l_run);
      named_barrier(2, kSoftmaxThreads);
      const float2 oth = xch[(half ^ 1) * BM + srow];
      const float M = fmaxf(m_ref, oth.x);
      const float w_self = m_ref == -INFINITY ? 0.0f : fast_exp2(m_ref - M);
      const float w_oth = oth.x == -INFINITY ? 0.0f : fast_exp2(oth.x - M);
      const float l_tot = w_self * l_run + w_oth * oth.y;
      const float wA = half == 0 ? w_self : w_oth, wB = half == 0 ? w_oth : w_self;
      const float inv_l = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
      const int hg = head % G;
      const bool to_rec = tile.part >= 0;
      const bool staged = to_rec && HPC == G;  // the CTA's 128 records are one contiguous range
      float* rec0 = to_rec ? a.parts + (size_t(tile.part) * p.Hkv + kvh) * TR * G * (HD + 2) : nullptr;
      float* rec = to_rec ? rec0 + (size_t(fm) * G + hg) * (HD + 2) : nullptr;
      typename QE::T* op = static_cast<typename QE::T*>(a.O) + size_t(row) * p.q_ld + size_t(head) * HD;
      const float* gp = a.X ? a.X + size_t(row) * p.g_ld + size_t(head) * 2 * HD + HD : nullptr;
      // this thread finishes dims [64 * half, 64 * half + 64) of its row
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        const int d0 = BH * half + 32 * c;
        float v[32];
        if (nb > 0) {
          uint32_t oa[32], ob[32];
          tmem_ld32(t_lane + COL_O + d0, oa);
          tmem_ld32(t_lane + COL_O + HD + d0, ob);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = wA * __uint_as_float(oa[i]) + wB * __uint_as_float(ob[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.0f;
        }
        if (staged) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) *reinterpret_cast<float2*>(stage + srow * (HD + 2) + d0 + i) = make_float2(v[i], v[i + 1]);
        } else if (to_rec) {
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) *reinterpret_cast<float2*>(rec + d0 + i) = make_float2(v[i], v[i + 1]);
          }
        } else if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            float o[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              o[k] = v[i + k] * inv_l;
              if (gp) o[k] *= sigmoid_gate(gp[d0 + i + k]);
            }
            uint4 w;
            w.x = QE::pack2(o[0], o[1]), w.y = QE::pack2(o[2], o[3]), w.z = QE::pack2(o[4], o[5]), w.w = QE::pack2(o[6], o[7]);
            *reinterpret_cast<uint4*>(op + d0 + i) = w;
          }
        }
      }
      if (half == 0) {
        if (staged) {
          stage[srow * (HD + 2) + HD] = M * kLn2;  // -inf stays -inf
          stage[srow * (HD + 2) + HD + 1] = l_tot;
        } else if (to_rec) {
          if (row_ok) rec[HD] = M * kLn2, rec[HD + 1] = l_tot;
        } else if (row_ok && a.lse) {
          a.lse[size_t(row) * p.H + head] = l_tot > 0.0f ? M * kLn2 + __logf(l_tot) : -INFINITY;
        }
      }
      if (staged && pair_mode) {
        // Both CTAs of the pair have staged their record in their own (idle) K ring. Barrier 1: both are past their
        // last MMA, so the first CTA's rings may be written. The second CTA copies its record into the first one's
        // `other` area over distributed shared memory; barrier 2 makes it visible; the first CTA folds the two records
        // in record order and writes the rows.
        named_barrier(2, kSoftmaxThreads);
        cluster_sync_all();
        float* other = stage + BM * (HD + 2);
        const uint32_t me = cluster_ctarank();
        if (me != 0) {
          const uint32_t dst = cluster_map_shared(other, 0);
          const float4* src = reinterpret_cast<const float4*>(stage);
          for (int i = tid; i < BM * (HD + 2) / 4; i += kSoftmaxThreads) st_cluster_f4(dst + 16u * uint32_t(i), src[i]);
        }
        cluster_sync_all();
        if (me == 0) {
          float Mx = -INFINITY, L = 0.0f;
          float acc[BH];
#pragma unroll
          for (int i = 0; i < BH; ++i) acc[i] = 0.0f;
#pragma unroll 1
          for (int s2 = 0; s2 < 2; ++s2) {
            const float* rp = ((tile.pad1 + s2 == tile.part) ? stage : other) + srow * (HD + 2);
            const float m_s = rp[HD];
            if (m_s == -INFINITY) continue;  // an empty record adds nothing
            if (m_s > Mx) {                    // rescale what has been summed so far
              const float f = __expf(Mx - m_s);  // 0 for the first record
              L *= f;
#pragma unroll
              for (int i = 0; i < BH; ++i) acc[i] *= f;
              Mx = m_s;
            }
            const float w = __expf(m_s - Mx);
            L += w * rp[HD + 1];
#pragma unroll
            for (int i = 0; i < BH; i += 2) {
              const float2 o2 = *reinterpret_cast<const float2*>(rp + BH * half + i);
              acc[i] += w * o2.x, acc[i + 1] += w * o2.y;
            }
          }
          if (row_ok) {
            const float inv = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
            for (int i = 0; i < BH; i += 8) {
              float o[8];
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                o[k] = acc[i + k] * inv;
                if (gp) o[k] *= sigmoid_gate(gp[BH * half + i + k]);
              }
              uint4 w4;
              w4.x = QE::pack2(o[0], o[1]), w4.y = QE::pack2(o[2], o[3]), w4.z = QE::pack2(o[4], o[5]), w4.w = QE::pack2(o[6], o[7]);
              *reinterpret_cast<uint4*>(op + BH * half + i) = w4;
            }
            if (half == 0 && a.lse) a.lse[size_t(row) * p.H + head] = L > 0.0f ? Mx + __logf(L) : -INFINITY;
          }
        }
      } else if (staged) {
        // 128 records x (HD + 2) floats, contiguous and 16-byte aligned in `parts`: coalesced copy
        named_barrier(2, kSoftmaxThreads);
        const float4* src = reinterpret_cast<const float4*>(stage);
        float4* dst = reinterpret_cast<float4*>(rec0);
        for (int i = tid; i < BM * (HD + 2) / 4; i += kSoftmaxThreads) dst[i] = src[i];
        if (fix_parts > 0) {
          // Fused merge (what attention_combine does, kernels/40_attention.metal:811-864): every CTA
          // of the job publishes its records and takes a ticket; whoever draws the last ticket
          // merges all records in record order, so the result does not depend on who that is.
          // Nobody waits for anybody.
          __threadfence();
          named_barrier(2, kSoftmaxThreads);
          int* ticket = a.counters + int(ts.fix_job) * int(gridDim.y) + int(blockIdx.y);
          if (tid == 0) {
            const int prev = atomicAdd(ticket, 1);
            red[0] = prev;
            if (prev == fix_parts - 1) *ticket = 0;  // ready for the next pass on this stream
          }
          named_barrier(2, kSoftmaxThreads);
          if (red[0] == fix_parts - 1) {
            __threadfence();
            // Records of the other CTAs come in through shared memory, one bulk copy each (a
            // thread reading its own 520-byte row straight from L2 would fetch every sector four
            // times); this CTA's own record is still in `stage`. The merge runs over the records
            // in record order with a running maximum, so it needs no pass of its own for M.
            float* other = stage + BM * (HD + 2);
            constexpr uint32_t kRecBytes = BM * (HD + 2) * 4;
            uint32_t xpar = nb > 0 ? 1 : 0;  // o_full has completed one phase if the tile had key blocks
            float Mx = -INFINITY, L = 0.0f;
            float acc[BH];
#pragma unroll
            for (int i = 0; i < BH; ++i) acc[i] = 0.0f;
#pragma unroll 1
            for (int s2 = 0; s2 < fix_parts; ++s2) {
              const float* src = stage;
              if (tile.pad1 + s2 != tile.part) {
                named_barrier(2, kSoftmaxThreads);  // the previous record in `other` has been consumed
                if (tid == 0) {
                  asm volatile("fence.proxy.async;" ::: "memory");  // the records were written through the generic proxy
                  mbar_arrive_expect_tx(&o_full, kRecBytes);
                  bulk_load(other, a.parts + (size_t(tile.pad1 + s2) * p.Hkv + kvh) * TR * G * (HD + 2), kRecBytes, &o_full);
                }
                wait_bar(&o_full, xpar, kStatusTmaTimeout);
                xpar ^= 1;
                src = other;
              }
              const float* rp = src + srow * (HD + 2);
              const float m_s = rp[HD];
              if (m_s == -INFINITY) continue;  // an empty record adds nothing
              if (m_s > Mx) {                    // rescale what has been summed so far
                const float f = __expf(Mx - m_s);  // 0 for the first record
                L *= f;
#pragma unroll
                for (int i = 0; i < BH; ++i) acc[i] *= f;
                Mx = m_s;
              }
              const float w = __expf(m_s - Mx);
              L += w * rp[HD + 1];
#pragma unroll
              for (int i = 0; i < BH; i += 2) {
                const float2 o2 = *reinterpret_cast<const float2*>(rp + BH * half + i);
                acc[i] += w * o2.x, acc[i + 1] += w * o2.y;
              }
            }
            if (row_ok) {
              const float inv = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
              for (int i = 0; i < BH; i += 8) {
                float o[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                  o[k] = acc[i + k] * inv;
                  if (gp) o[k] *= sigmoid_gate(gp[BH * half + i + k]);
                }
                uint4 w4;
                w4.x = QE::pack2(o[0], o[1]), w4.y = QE::pack2(o[2], o[3]), w4.z = QE::pack2(o[4], o[5]), w4.w = QE::pack2(o[6], o[7]);
                *reinterpret_cast<uint4*>(op + BH * half + i) = w4;
              }
              if (half == 0 && a.lse) a.lse[size_t(row) * p.H + head] = L > 0.0f ? Mx + __logf(L) : -INFINITY;
            }
          }
        }
      }
    }
  }
  if (pair_mode && !is_softmax) {  // the softmax warps pass the same two barriers inside their epilogue
    __syncwarp();
    cluster_sync_all();
    cluster_sync_all();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tracing && tid == 0) a.trace[8 * a.trace_blocks + 1] = global_timer_ns();
  if (tid == 0) cta_stamp(3);
  if (warp == kMmaWarp) tmem_dealloc(sh.tmem_slot, TMEM_COLS);
}

}  // namespace

bool flash_umma_supports(int32_t HDim, int32_t G, int32_t tile_rows, int32_t bt, int32_t q_dtype, int32_t kv_dtype) {
  if ((HDim != 64 && HDim != 128 && HDim != 256 && HDim != 512) || q_dtype != kv_dtype) return false;  // 64, 256, 512: flash_umma_pair only
  if (tile_rows != 16 && tile_rows != 32 && tile_rows != 64 && tile_rows != 128) return false;
  const int hpc = BM / tile_rows;
  if (hpc > G || G % hpc != 0) return false;
  return bt > 0 && bt % 16 == 0;
}

cudaError_t flash_umma_setup() {
  cudaError_t e = cudaFuncSetAttribute(flash_umma_kernel<ESP_F16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_umma_kernel<ESP_BF16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_umma_kernel<ESP_F16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_umma_kernel<ESP_BF16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  return e;
}

cudaError_t launch_flash_umma(const KernelArgs& a, const CUtensorMap& pool_map, const CUtensorMap& kb_map, const CUtensorMap& vb_map,
                              const esp_attn_tile* tiles_host, const esp_attn_tree* trees_host, int32_t n_trees,
                              const esp_attn_combine* jobs_host, int32_t n_jobs, bool* merged, cudaStream_t stream,
                              uint64_t* launches) {
  *merged = false;
  if (a.n_tiles <= 0) return cudaSuccess;
  InlinePlan plan;
  for (int i = 0; i < kInlinePlanMax; ++i) plan.start[i].valid = 0;
  bool inl = tiles_host && trees_host && a.n_tiles <= kInlinePlanMax && a.p.bt <= 0xffff && a.G <= 0xff;
  for (int i = 0; inl && i < a.n_tiles; ++i) {
    const int t = tiles_host[i].tree;
    if (t < 0 || t >= n_trees) {  // unvalidated plan: leave it to the device copies
      inl = false;
      break;
    }
    TileStart& ts = plan.start[i];
    ts.tile = tiles_host[i];
    ts.tile.pad0 = ts.tile.pad1 = 0;
    ts.tree = trees_host[t];
    ts.blocks = a.blocks, ts.bt = uint16_t(a.p.bt), ts.G = uint8_t(a.G), ts.tile_rows = uint8_t(a.tile_rows);
    ts.valid = uint16_t(i + 1), ts.fix_parts = 0, ts.fix_job = 0;
  }
  if (!inl)
    for (int i = 0; i < kInlinePlanMax; ++i) plan.start[i].valid = 0;
  // Fused merge: possible when the plan is inline, every CTA's records are one contiguous range
  // (its heads are the whole group of a kv head), every job has a counter and every split tile
  // belongs to exactly one job.
  const int grid_y = a.p.H / (BM / a.tile_rows);
  bool fuse = inl && jobs_host && n_jobs > 0 && a.counters && BM / a.tile_rows == a.G && n_jobs <= kInlinePlanMax &&
              int64_t(n_jobs) * grid_y <= kFixupCounters;
  if (fuse) {
    int covered = 0;
    for (int j = 0; fuse && j < n_jobs; ++j) {
      const esp_attn_combine& job = jobs_host[j];
      if (job.nparts < 1 || job.nparts > 255) fuse = false;
      int found = 0;
      for (int i = 0; fuse && i < a.n_tiles; ++i) {
        const esp_attn_tile& t = tiles_host[i];
        if (t.part < job.part0 || t.part >= job.part0 + job.nparts) continue;
        if (t.r0 != job.r0 || plan.start[i].fix_parts) fuse = false;  // a record of another row group, or claimed twice
        plan.start[i].fix_parts = uint8_t(job.nparts), plan.start[i].fix_job = uint8_t(j), plan.start[i].tile.pad1 = job.part0;
        ++found;
      }
      if (found != job.nparts) fuse = false;  // some record of the job is not written by this pass
      covered += found;
    }
    if (!fuse)
      for (int i = 0; i < a.n_tiles; ++i) plan.start[i].fix_parts = 0;
    (void)covered;
  }
  *merged = fuse;
  const int hpc = BM / a.tile_rows;
  const bool f8 = a.kv_dtype == ESP_E4M3;  // pool_map is then the byte map of the pool (16-row boxes of 128-byte lines)
  const dim3 grid(unsigned(a.n_tiles), unsigned(a.p.H / hpc)), block(f8 ? kThreadsF8 : kThreads);
  // Pair mode: every job has exactly two records, written by the tiles 2 j and 2 j + 1 (the kernel walks the tiles
  // from the last one down: cluster ranks 0 and 1 are the tiles 2 j + 1 and 2 j).
  bool pairs = fuse && a.pair_merge && a.n_tiles % 2 == 0;
  for (int i = 0; pairs && i < a.n_tiles; i += 2)
    pairs = plan.start[i].fix_parts == 2 && plan.start[i + 1].fix_parts == 2 && plan.start[i].fix_job == plan.start[i + 1].fix_job;
  KernelArgs k = a;
  k.fuse = pairs ? 2 : (fuse ? 1 : 0);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = SMEM_BYTES, cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  if (pairs) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2, attr[1].val.clusterDim.y = 1, attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  cudaError_t e;
  if (f8)
    e = a.q_dtype == ESP_F16 ? cudaLaunchKernelEx(&cfg, flash_umma_kernel<ESP_F16, true>, pool_map, kb_map, vb_map, plan, k)
                             : cudaLaunchKernelEx(&cfg, flash_umma_kernel<ESP_BF16, true>, pool_map, kb_map, vb_map, plan, k);
  else
    e = a.q_dtype == ESP_F16 ? cudaLaunchKernelEx(&cfg, flash_umma_kernel<ESP_F16, false>, pool_map, kb_map, vb_map, plan, k)
                             : cudaLaunchKernelEx(&cfg, flash_umma_kernel<ESP_BF16, false>, pool_map, kb_map, vb_map, plan, k);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e == cudaSuccess) ++*launches;
  return e;
}

}  // namespace esp
