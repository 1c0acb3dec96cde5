// Forest attention for 128-row tiles on the 5th-generation tensor cores (sm_100a), variant for
// passes whose keys are mostly the pass's own rows (causal prefill): two CTAs per SM, 64-key
// blocks, short K/V rings (the keys sit in L2). flash_umma.cu holds the variant that streams a
// long cached prefix from HBM (one CTA per SM, 128-key blocks, deep rings); both compute the same.
// 256-dim heads (every pass with them runs here) take the whole SM for one CTA: the Q tile sits in tensor
// memory as the A operand of Q.K^T, the rings hold 4 K + 3 V tiles, and one-wave verify passes merge their
// split-K records inside the kernel. Over an E4M3 pool (F8 instantiation) the producers fetch the raw pages,
// converter warps write the fp16 tiles (code x page scale) and the pass computes in fp16. 512-dim heads: a tile runs
// as two CTAs, each with the whole scores and one 256-dim half of V and O.
//
// Computes what flash_attention computes (kernels/40_attention.metal:156-343 of the
// reference; generic head dim kernels/80_gemma.metal:157-342): the tile's rows attend to the
// cached key range [k0, k1) of the paged pool and, when tile.last, to the visible batch keys
// of their tree (two-level `desc` mask or a 64-bit ancestor mask per row), writing either
// the partial record [O | m | l] or the gated, normalised output (and its LSE).
//
// B200 structure. One CTA = 128 (query row, head) pairs = the 128 lanes of tensor memory:
// tile_rows rows x (128 / tile_rows) heads of one kv head (16 nodes x 8 heads for a verify
// tile, 128 rows x 1 head for prefill). Keys are processed 64 at a time:
//   S[128 x 64]   = Q . K^T      tcgen05.mma, A = Q tile and B = K tile from shared memory
//                                (K-major, 128-byte swizzle), D in tensor memory (fp32)
//   softmax        thread i owns row i: tcgen05.ld of its 64 scores, mask, online max / sum
//                  in the exp2 domain (no shuffles), P as bf16 / fp16 pairs back into tensor
//                  memory with tcgen05.st
//   O[128 x HD]  += P . V         tcgen05.mma with A = P from tensor memory, B = V tile from
//                                shared memory (MN-major), accumulating in tensor memory
// O stays in tensor memory for the whole tile and is rescaled only when a row's maximum has
// grown by more than 2^8 since its reference value (warp-uniform decision), so the common
// step has no accumulator traffic at all. K and V tiles are double-buffered and arrive by
// TMA: one bulk tensor load per (16-key page, 64-dim half), rows found through the page table
// for cached keys and directly in Kb / Vb for batch keys. The CTA is warp-specialised: warps
// 0-3 do the softmax (one thread per row), warp 4 issues every MMA from one thread and owns
// the tensor memory, warp 5 is the TMA producer; they hand tiles to one another through
// mbarriers only (TMA complete_tx, tcgen05.commit, and a 128-arrival barrier for P). Blocks
// that need no mask (all but the diagonal, the tail and tree blocks) take a path with no
// per-key predicate. Two CTAs share an SM (97 KB of shared memory and 256 tensor-memory
// columns each) so that one CTA's softmax overlaps the other's MMAs.
// Every wait is bounded: after a timeout the CTA records a status code, stops waiting,
// finishes its loop, frees its tensor memory and returns.
#include <climits>

#include "umma.cuh"
#include "../launch.h"

namespace esp {
namespace {

constexpr int BM = 128;  // (row, head) pairs per CTA
constexpr int BN = 64;   // keys per block
// The head dim is a template parameter (128: two CTAs per SM; 256: the whole SM for one CTA). Tiles
// are stored as HD / 64 chunks of 64 dims, each [rows][128 B] with the 128-byte swizzle.
// 256-dim heads keep the Q tile in tensor memory (A operand of Q.K^T from there): its 64 KB of shared memory
// go to the K / V rings instead, and Q.K^T reads only the K tile through the shared-memory port.
constexpr bool q_in_tmem(int hd) { return hd == 256; }
constexpr int q_bytes(int hd) { return q_in_tmem(hd) ? 0 : BM * hd * 2; }
constexpr int kv_tile(int hd) { return BN * hd * 2; }
// 512-dim heads (the global layers of kernels/80_gemma.metal, gemma.h:119-147): O alone would fill tensor memory, so a
// CTA computes one 256-dim half of the output (blockIdx.z) from the whole 512-dim scores: Q (128 KB, shared memory),
// one K tile (64 KB) and one V half tile (32 KB) fill the SM; the two halves of a tile compute the same S, m and l.
constexpr int v_dims(int hd) { return hd == 512 ? 256 : hd; }
constexpr int HALF_Q = BM * 128;            // bytes between the 64-dim chunks of the Q tile
constexpr int HALF_KV = BN * 128;           // ... of a K / V tile
// Ring depths come in two flavours: (3, 2) lets two CTAs share an SM (passes whose keys sit in L2:
// prefill), (6, 6) takes the whole SM for one CTA and keeps ~160 KB of K/V in flight (passes
// that stream their keys from HBM: verify over a long cached prefix).
constexpr int kMaxStages = 6;
constexpr int tiles_bytes(int hd, int ks, int vs) { return q_bytes(hd) + ks * kv_tile(hd) + vs * kv_tile(v_dims(hd)); }
constexpr int smem_bytes(int hd, int ks, int vs) { return tiles_bytes(hd, ks, vs) + 384; }  // + mbarriers; no static shared memory
// Two S buffers of 64 fp32 columns (P of a block is written over the first 32 columns of its own
// S buffer as 16-bit pairs, once the thread holds its scores in registers), O: HD fp32 columns
// (allocations are powers of two: 256 columns for 128-dim heads, 512 for 256-dim heads).
constexpr uint32_t tmem_cols(int hd) { return hd <= 128 ? 256u : 512u; }  // (512-dim heads: 128 + 256 columns of 512)
constexpr uint32_t COL_S = 0, COL_O = 128;
constexpr uint32_t COL_Q = 384;             // 256-dim heads: the Q tile as 16-bit pairs, 128 columns behind O
constexpr float kRescaleThreshold = 8.0f;   // log2 units

__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// The n lowest bits set (n <= 0: none, n >= 64: all).
__device__ __forceinline__ uint64_t low_bits64(int n) { return n <= 0 ? 0ull : (n >= 64 ? ~0ull : ((1ull << n) - 1ull)); }

struct PageRef {  // where one 16-key page of a key block comes from
  int raw;        // block id as loaded from the page table (pool), or first row (Kb / Vb)
  int off;        // row inside the block (pool)
  int kind;       // -1: nothing to load, 0: paged pool, 1: Kb / Vb
};

// E4M3 pools (F8 instantiation, 256-dim heads): the producers bring the pool's raw pages (16 keys x 256 codes of one
// kv head: the byte map the decode kernel uses) into rings of two 16 KB tiles behind the 16-bit rings; four converter
// warps turn them into the fp16 tiles the MMAs read (code x page scale), and the pass computes in fp16.
constexpr int kRawStages = 2;
constexpr int kCvtWarp0 = 7, kCvtWarps = 4;  // warps 7, 9: K tiles; 8, 10: V tiles
constexpr int kCvtLanes = kCvtWarps / 2 * 32;
constexpr int raw_tile(int hd) { return BN * hd; }
constexpr int smem_bytes_f8(int hd, int ks, int vs) { return tiles_bytes(hd, ks, vs) + 2 * kRawStages * raw_tile(hd) + 384 + 128; }
struct SharedF8 {
  uint64_t raw_full[2][kRawStages], raw_empty[2][kRawStages];
  float scl[2][kRawStages][4];  // scale of each raw page of a slot
};
static_assert(sizeof(SharedF8) <= 128, "E4M3 bookkeeping must fit behind the other");

// Sliding-window layers (WIN instantiation, 256-dim heads; kernels/80_gemma.metal:123-142, :250, :284-285): the K producer
// leaves the positions of a batch block's keys in one of kPosSlots slots for the softmax warps' window masks. With a K
// ring of 3 the producer is at most 4 blocks ahead of the block the softmax warps work on.
constexpr int kPosSlots = 8;
struct SharedWin {
  uint64_t kpos_full[kPosSlots];
  int kpos_min[kPosSlots];
  int kpos[kPosSlots][BN];
};
constexpr int smem_bytes_win(int hd, int ks, int vs) { return tiles_bytes(hd, ks, vs) + 384 + 128 + int(sizeof(SharedWin)); }

constexpr int kSoftmaxThreads = BM;          // warps 0-3: one thread per (row, head) pair
constexpr int kMmaWarp = 4;                  // warp 4: MMA issue (one thread), owns tensor memory
constexpr int kTmaWarpK = 5;                 // warp 5: TMA producer of K tiles (lanes 0-3, one 16-key page each)
constexpr int kTmaWarpV = 6;                 // warp 6: TMA producer of V tiles
constexpr int kThreads = 7 * 32;
constexpr int kThreadsF8 = (kCvtWarp0 + kCvtWarps) * 32;

// Barriers and bookkeeping live behind the tiles in dynamic shared memory: with no static shared
// memory the dynamic window starts on a 1024-byte boundary (checked at run time), which the
// swizzled tiles need, and two CTAs of 112.4 KB fit one SM.
struct Shared {
  uint64_t k_full[kMaxStages], k_empty[kMaxStages], v_full[kMaxStages], v_empty[kMaxStages], s_full[2], p_full[2], pv_done, o_full, q_full, fix_bar;
  uint32_t tmem_slot;
  int red[6];  // anc_max, seg_min, anc_min, seg_max; sliding-window layers: the latest row position, the furthest image end
  volatile int dead;
};
static_assert(sizeof(Shared) <= 384, "bookkeeping must fit behind the tiles");

template <int QDT, int HD, int KS, int VS, bool F8 = false, bool WIN = false>
__global__ void __launch_bounds__(F8 ? kThreadsF8 : kThreads, (!F8 && !WIN && smem_bytes(HD, KS, VS) <= 114 * 1024) ? 2 : 1)
    flash_umma_pair_kernel(const __grid_constant__ CUtensorMap pool_map, const __grid_constant__ CUtensorMap kb_map,
                      const __grid_constant__ CUtensorMap vb_map, const KernelArgs a) {
  using QE = Elem16<QDT>;
  constexpr int CDT = F8 ? ESP_F16 : QDT;  // type of the MMA operands (E4M3 pools: fp16, exact for the codes)
  using PE = Elem16<CDT>;
  static_assert(!F8 || q_in_tmem(HD), "the E4M3 instantiation is for 256-dim heads");
  static_assert(!WIN || (q_in_tmem(HD) && !F8 && KS <= 3), "the sliding-window instantiation is for 256-dim heads over 16-bit pools");
  extern __shared__ __align__(1024) uint8_t smem[];
  // full: TMA -> MMA; empty: MMA -> TMA (tcgen05.commit); s_full[i]: S buffer i written;
  // p_full[i]: P in buffer i written (128 arrivals); pv_done: P.V of a block complete;
  // o_full: last P.V done
  constexpr int HV = v_dims(HD);  // dims of the V tiles and of O in this CTA
  constexpr int NCH = HD / 64;    // 64-dim chunks of a Q / K row
  constexpr int NCHV = HV / 64;   // ... of a V row's part
  constexpr int Q_BYTES = q_bytes(HD), KV_TILE = kv_tile(HD), V_TILE = kv_tile(HV);
  static_assert(HD != 512 || (!F8 && !WIN && KS == 1), "512-dim heads: the plain instantiation only, one K tile");
  // 512-dim heads have room for one K tile only, so the next block's K can be requested only when Q.K^T of this one
  // has read it. The tile is handed over in four parts of two 64-dim chunks, each with its own barriers: a part is
  // requested again as soon as its eight MMAs are done, and the next Q.K^T starts on the parts that have arrived.
  constexpr int KSUB = HD == 512 ? 4 : 1;
  const int vh = HD == 512 ? int(blockIdx.z) : 0;  // which half of the output dims
  const int ho = vh * HV;
  constexpr uint32_t TMEM_COLS = tmem_cols(HD);
  constexpr int TILES_BYTES = tiles_bytes(HD, KS, VS);
  constexpr int RAW_TILE = raw_tile(HD);
  constexpr int RAW_BYTES = F8 ? 2 * kRawStages * RAW_TILE : 0;
  uint8_t* raw_sm = smem + TILES_BYTES;  // F8: K slots, then V slots
  Shared& sh = *reinterpret_cast<Shared*>(smem + TILES_BYTES + RAW_BYTES);
  SharedF8& sh8 = *reinterpret_cast<SharedF8*>(smem + TILES_BYTES + RAW_BYTES + 384);
  SharedWin& shw = *reinterpret_cast<SharedWin*>(smem + TILES_BYTES + RAW_BYTES + 384 + 128);  // WIN only
  uint64_t* k_full = sh.k_full;
  uint64_t* k_empty = sh.k_empty;
  uint64_t* v_full = sh.v_full;
  uint64_t* v_empty = sh.v_empty;
  uint64_t* s_full = sh.s_full;
  uint64_t* p_full = sh.p_full;
  uint64_t& pv_done = sh.pv_done;
  uint64_t& o_full = sh.o_full;
  uint32_t& tmem_slot = sh.tmem_slot;
  int* red = sh.red;
  volatile int& dead = sh.dead;
  if ((smem_u32(smem) & 1023u) != 0) {  // never expected; the tiles' swizzle would be wrong
    if (threadIdx.x == 0) atomicExch(a.status, kStatusBadBlock);
    return;
  }
  uint8_t* q_sm = smem;
  uint8_t* k_sm = smem + Q_BYTES;                 // KS stages, KV_TILE apart
  uint8_t* v_sm = smem + Q_BYTES + KS * KV_TILE;  // VS stages, V_TILE apart

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_wait();  // (256-dim heads are launched with programmatic stream serialization: the launch itself hides behind the previous kernel)
  const esp_attn_params& p = a.p;
  const int G = a.G, TR = a.tile_rows, HPC = BM / TR;
  const esp_attn_tile tile = a.tiles[a.n_tiles - 1 - int(blockIdx.x)];  // long (late) tiles first
  const esp_attn_tree tree = a.trees[tile.tree];
  const int kvh = (int(blockIdx.y) * HPC) / G;
  const int end = tree.base + tree.M;
  const int rows_live = min(TR, end - tile.r0);
  const bool use_anc = a.anc_mask != nullptr;

  // per softmax thread: its (row, head)
  const int fm = (tid & (BM - 1)) / HPC, hh = (tid & (BM - 1)) % HPC;
  const int head = int(blockIdx.y) * HPC + hh;
  const bool row_ok = tid < BM && fm < rows_live;
  const int row = (tid < BM && fm < rows_live) ? tile.r0 + fm : end - 1;
  const int rr = row - tree.base;

  // ---- set-up
  if (tid == 0) {
    for (int s = 0; s < KS * KSUB; ++s) {
      mbar_init(&k_full[s], F8 ? kCvtLanes : 4);  // E4M3 pools: the lanes of the tile's converter warps
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < VS; ++s) {
      mbar_init(&v_full[s], F8 ? kCvtLanes : 4);
      mbar_init(&v_empty[s], 1);
    }
    if constexpr (F8) {
      for (int t = 0; t < 2; ++t)
        for (int s = 0; s < kRawStages; ++s) {
          mbar_init(&sh8.raw_full[t][s], 4);
          mbar_init(&sh8.raw_empty[t][s], kCvtLanes);
        }
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], kSoftmaxThreads);
    }
    mbar_init(&pv_done, 1);
    mbar_init(&o_full, 1);
    mbar_init(&sh.q_full, kSoftmaxThreads);
    mbar_init(&sh.fix_bar, 1);
    if constexpr (WIN)
      for (int i = 0; i < kPosSlots; ++i) mbar_init(&shw.kpos_full[i], 1);
    mbar_fence_init();
    red[0] = 0, red[1] = 1 << 30, red[2] = 1 << 30, red[3] = 0, red[4] = INT_MIN, red[5] = 0;
    dead = 0;
  }
  if (warp == kMmaWarp) {
    tmem_alloc(&tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == kTmaWarpK && lane == 0) {
    tma_prefetch_desc(&pool_map);
    tma_prefetch_desc(&kb_map);
    tma_prefetch_desc(&vb_map);
  }
  int4 d = make_int4(0, 0, 0, 0);
  uint64_t am = 0;
  // Sliding-window layers: a key `window` or more positions behind the query is masked; ring: a sequence's blocks sit
  // in place (no page table); bidi: image rows see their whole image (desc.w = its end).
  const bool windowed = WIN && a.window > 0;
  const bool bidi = WIN && a.bidi != 0 && !use_anc;
  int qpos = 0;
  constexpr bool QT = q_in_tmem(HD);
  uint4 qreg[QT ? HD / 8 : 1];  // Q in tensor memory: the row waits in registers until the allocation is known
  if (tid < BM) {
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const typename QE::T*>(a.Q) + size_t(row) * p.q_ld + size_t(head) * HD);
    if constexpr (QT) {
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) qreg[i] = __ldg(src + i);
    } else {
      // Q row of this thread into the K-major swizzled tile
#pragma unroll
      for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i)
          *reinterpret_cast<uint4*>(q_sm + c * HALF_Q + tid * 128 + ((i ^ (tid & 7)) << 4)) = src[c * 8 + i];
      fence_proxy_async_smem();
    }
    if (tile.last) {
      if (use_anc) am = a.anc_mask[row];
      else d = reinterpret_cast<const int4*>(a.desc)[row];
    }
    if (windowed) {  // the row's position; the latest one of the tile bounds every row's window from above
      qpos = a.pos[4 * size_t(row)];
      int latest = qpos;
#pragma unroll
      for (int o = 16; o; o >>= 1) latest = max(latest, __shfl_xor_sync(0xffffffffu, latest, o));
      if (lane == 0) atomicMax(&red[4], latest);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if constexpr (QT) {
    // Lane i of tensor memory holds row i: column c = dims (2c, 2c + 1), the layout an A operand from tensor
    // memory has (the same as P). The MMA thread learns of it through q_full (128 arrivals).
    if (tid < BM) {
      const uint32_t t_q = tmem_slot + (uint32_t(warp * 32) << 16) + COL_Q;
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        uint32_t w[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          w[4 * i] = qreg[8 * c + i].x, w[4 * i + 1] = qreg[8 * c + i].y;
          w[4 * i + 2] = qreg[8 * c + i].z, w[4 * i + 3] = qreg[8 * c + i].w;
        }
        if constexpr (F8 && QDT != CDT) {  // a bf16 pass over an E4M3 pool computes in fp16
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float2 f = QE::unpack2(w[i]);
            w[i] = PE::pack2(f.x, f.y);
          }
        }
        tmem_st32(t_q + 32 * c, w);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&sh.q_full);
    }
  }
  if ((tile.last && !use_anc) || windowed) {
    if (tid < BM && tile.last && !use_anc) {
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
      if (bidi) {
        int w_end = d.w;
#pragma unroll
        for (int o = 16; o; o >>= 1) w_end = max(w_end, __shfl_xor_sync(0xffffffffu, w_end, o));
        if (lane == 0) atomicMax(&red[5], w_end);
      }
    }
    __syncthreads();
  }
  const uint32_t tmem = tmem_slot;

  // ---- block list: cached 64-key blocks, then the batch blocks some row of the tile can see
  const int r_first = tile.r0 - tree.base, r_last = r_first + rows_live - 1;
  const int anc_max = red[0], seg_min = red[1], anc_min = red[2], seg_max = red[3];
  int k_last = -1, a_lo = 0, a_hi = 0, b_lo = 0, nbb = 0;
  const int lo_max = windowed ? red[4] - a.window + 1 : INT_MIN;  // the latest row's first visible position
  if (tile.last) {
    if (use_anc) {
      k_last = min(tree.M, 64) - 1;
      a_hi = (k_last + BN) / BN;
      nbb = a_hi;
    } else {
      const int reach = max(r_last, red[5] - 1);  // (image rows also see the later rows of their image)
      k_last = min(tree.M - 1, max(reach, anc_max - 1));
      const int n_all = (k_last + BN) / BN;
      a_hi = min((anc_max + BN - 1) / BN, n_all);                 // blocks below the ancestor range
      b_lo = max(a_hi, seg_min / BN);                             // blocks of the rows' own segments
      const int b_hi = min(reach / BN, n_all - 1);
      if (windowed) {  // batch blocks below the first batch key worth scanning (tile.pad0) are left out
        const int f = max(0, tile.pad0) / BN;
        a_lo = min(a_hi, f);
        b_lo = max(b_lo, f);
      }
      nbb = (a_hi - a_lo) + max(0, b_hi - b_lo + 1);
    }
  }
  // A sliding-window tile starts at the first cached key one of its rows can see, at any alignment: pages are loaded
  // from the 16-key boundary below it (the keys in between are behind every row's window).
  const int k0a = WIN ? (tile.k0 & ~15) : tile.k0;
  const int nbc = (tile.k1 - k0a + BN - 1) / BN;
  const int nb = nbc + nbb;
  auto batch_j0 = [&](int i) { return BN * (i < a_hi - a_lo ? a_lo + i : b_lo + (i - (a_hi - a_lo))); };
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
  // Per-CTA stamps (option "trace_ctas"): start, loop done (O complete), records published or rows written, exit.
  const int cta_lin = blockIdx.y * gridDim.x + blockIdx.x;
  const bool cta_tracing = a.trace != nullptr && cta_lin < a.trace_ctas;
  auto cta_stamp = [&](int ev) {
    if (cta_tracing) a.trace[8 * a.trace_blocks + 2 + 4 * cta_lin + ev] = global_timer_ns();
  };
  if (tid == 0) cta_stamp(0);

  if (F8 && (warp == kTmaWarpK || warp == kTmaWarpV)) {
    // ================= E4M3 pools: warp 5 fills the raw K ring, warp 6 the raw V ring; lane w loads the w-th 16-key
    // page of every cached block (one load: 16 rows x 2 lines of 128 codes) and leaves the page's scale beside it.
    // Batch blocks (the pass's own rows, in the Q type) are fetched by the converter warps.
    if (lane < 4 && nbc > 0) {
      const int is_v = warp == kTmaWarpV ? 1 : 0;
      uint64_t* full = sh8.raw_full[is_v];
      uint64_t* empty = sh8.raw_empty[is_v];
      uint8_t* ring = raw_sm + is_v * kRawStages * RAW_TILE;
      auto page_of = [&](int b) {
        const int j = tile.k0 + BN * b + 16 * lane;
        return (b < nbc && j < tile.k1) ? a.blocks[tree.table + j / p.bt] : -1;
      };
      int cur = page_of(0), nxt = page_of(1), nx2 = page_of(2);
      int stage = 0;
      uint32_t par = 1;  // the first use of a slot finds it empty
      for (int b = 0; b < nbc; ++b) {
        const bool ok = cur >= 0 && cur < a.n_blocks;
        float sc = 0.0f;  // on its way while the lane waits for the slot
        if (ok) sc = a.kv_scales[(size_t(cur) * 2 + is_v) * p.Hkv + kvh];
        wait_bar(&empty[stage], par, kStatusMmaTimeout);
        if (!ok) {
          if (cur >= a.n_blocks) atomicExch(a.status, kStatusBadBlock);
          sh8.scl[is_v][stage][lane] = 0.0f;
          mbar_arrive(&full[stage]);
        } else {
          sh8.scl[is_v][stage][lane] = sc;
          const int y = (cur * 2 + is_v) * p.bt + (tile.k0 + BN * b + 16 * lane) % p.bt;
          mbar_arrive_expect_tx(&full[stage], 16 * HD);
          tma_load_3d(ring + stage * RAW_TILE + lane * 16 * HD, &pool_map, &full[stage], 0, y, kvh * (HD / 128));
        }
        if (lane == 0) stamp(b, is_v ? 7 : 6);
        cur = nxt;
        nxt = nx2;
        nx2 = page_of(b + 3);
        if (++stage == kRawStages) stage = 0, par ^= 1;
      }
    }
  } else if (F8 && warp >= kCvtWarp0) {
    // ================= E4M3 pools: converter warps. Warps 7, 9 turn raw K tiles into fp16 K tiles, 8, 10 do V (spread
    // over the schedulers: the conversion instruction runs on the exp2 unit's pipe); a warp takes every second 16-key
    // page of a block, lane l one of the two 128-code lines (l / 16) of row l % 16: 8 raw chunks of 16 codes become
    // 16 chunks of 8 halves in two 64-dim chunks of the 16-bit tile.
    const int is_v = (warp - kCvtWarp0) & 1, wi = (warp - kCvtWarp0) >> 1;
    uint64_t* full = is_v ? v_full : k_full;
    uint64_t* empty = is_v ? v_empty : k_empty;
    uint8_t* ring = is_v ? v_sm : k_sm;
    const int depth = is_v ? VS : KS;
    const uint8_t* raw_ring = raw_sm + is_v * kRawStages * RAW_TILE;
    int rst = 0, cst = 0;
    uint32_t rpar = 0, cpar = 1;  // the first use of a converted slot finds it empty
    for (int b = 0; b < nb; ++b) {
      const bool cached = b < nbc;
      const int j0 = cached ? tile.k0 + BN * b : batch_j0(b - nbc);
      const int n_valid = cached ? min(BN, tile.k1 - j0) : min(BN, k_last + 1 - j0);
      if (cached) wait_bar(&sh8.raw_full[is_v][rst], rpar, kStatusTmaTimeout);
      wait_bar(&empty[cst], cpar, kStatusMmaTimeout);
      uint8_t* dst = ring + cst * KV_TILE;
#pragma unroll 1
      for (int pg = wi; pg < 4; pg += kCvtWarps / 2) {
        const int rl = lane & 15, r = 16 * pg + rl, cg = lane >> 4;
        uint8_t* drow = dst + (2 * cg) * HALF_KV + r * 128;  // dims 128 cg .. 128 cg + 127 = chunks 2 cg and 2 cg + 1
        if (r >= n_valid) {
          // rows past the range: zeros (stale bytes could be NaN patterns, and 0 x NaN must not happen)
#pragma unroll
          for (int c = 0; c < 16; ++c) *reinterpret_cast<uint4*>(drow + (c >> 3) * HALF_KV + (((c & 7) ^ (r & 7)) << 4)) = make_uint4(0, 0, 0, 0);
        } else if (cached) {
          const uint8_t* srow = raw_ring + rst * RAW_TILE + pg * 16 * HD + cg * 2048 + rl * 128;
          const __half2 sc2 = __float2half2_rn(sh8.scl[is_v][rst][pg]);
#pragma unroll
          for (int c = 0; c < 8; ++c) {  // the line's raw chunk c: codes 16 c .. 16 c + 15
            const uint4 v = *reinterpret_cast<const uint4*>(srow + ((c ^ (rl & 7)) << 4));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t h[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t lo = e4m3x2_to_f16x2(uint16_t(w[i] & 0xFFFFu)), hi = e4m3x2_to_f16x2(uint16_t(w[i] >> 16));
              __half2 a2 = __hmul2(*reinterpret_cast<__half2*>(&lo), sc2), b2 = __hmul2(*reinterpret_cast<__half2*>(&hi), sc2);
              h[2 * i] = *reinterpret_cast<uint32_t*>(&a2), h[2 * i + 1] = *reinterpret_cast<uint32_t*>(&b2);
            }
            uint8_t* dch = drow + (c >> 2) * HALF_KV;  // 64-dim chunk 2 cg + c / 4; pieces 2 (c % 4) and 2 (c % 4) + 1 of its line
            *reinterpret_cast<uint4*>(dch + (((2 * (c & 3)) ^ (r & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
            *reinterpret_cast<uint4*>(dch + (((2 * (c & 3) + 1) ^ (r & 7)) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
          }
        } else {
          // a batch key: the pass's own row, in the Q type
          const uint4* src = reinterpret_cast<const uint4*>(static_cast<const typename QE::T*>(is_v ? a.Vb : a.Kb) +
                                                            size_t(tree.base + j0 + r) * p.kv_ld + size_t(kvh) * HD) + 16 * cg;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            uint4 v = src[c];
            if constexpr (QDT != CDT) {
              uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 f = QE::unpack2(w[i]);
                w[i] = PE::pack2(f.x, f.y);
              }
            }
            *reinterpret_cast<uint4*>(drow + (c >> 3) * HALF_KV + (((c & 7) ^ (r & 7)) << 4)) = v;
          }
        }
      }
      fence_proxy_async_smem();
      if (cached) {
        mbar_arrive(&sh8.raw_empty[is_v][rst]);
        if (++rst == kRawStages) rst = 0, rpar ^= 1;
      }
      mbar_arrive(&full[cst]);
      if (++cst == depth) cst = 0, cpar ^= 1;
    }
  } else if (!F8 && (warp == kTmaWarpK || warp == kTmaWarpV)) {
    // ================= TMA producers: warp 5 fills the K ring, warp 6 the V ring, each on its own
    // schedule (a K tile is free as soon as its Q.K^T is done, a V tile only after its P.V);
    // lane w loads the w-th 16-key page of every block.
    // (Sliding-window layers: the whole K producer warp walks the blocks - after the four page lanes have issued a batch
    // block, all lanes leave the positions of its 64 keys, and the earliest of them, for the softmax warps.)
    const bool pos_lanes = WIN && windowed && warp == kTmaWarpK;
    if ((lane < 4 || pos_lanes) && nb > 0) {
      const bool is_v = warp == kTmaWarpV;
      const int depth = is_v ? VS : KS;
      uint64_t* full = is_v ? v_full : k_full;
      uint64_t* empty = is_v ? v_empty : k_empty;
      uint8_t* ring = is_v ? v_sm : k_sm;
      const CUtensorMap* batch_map = is_v ? &vb_map : &kb_map;
      // The page-table entry is only loaded here; the row arithmetic happens when the page is
      // issued, so the load's latency stays off the critical path.
      auto page_of = [&](int b) {
        PageRef r{0, 0, -1};
        if (b >= nb || lane >= 4) return r;
        if (b < nbc) {
          const int j = k0a + BN * b + 16 * lane;
          if (j < tile.k1) {
            // ring layers (kernels/80_gemma.metal:429) keep a sequence's blocks in place: no page table
            r.raw = (WIN && a.ring > 0) ? tree.table + (j / p.bt) % a.ring : a.blocks[tree.table + j / p.bt];
            r.off = j % p.bt;
            r.kind = 0;
          }
        } else {
          const int j = batch_j0(b - nbc) + 16 * lane;
          if (j <= k_last) {
            r.raw = tree.base + j;
            r.kind = 1;
          }
        }
        return r;
      };
      PageRef cur = page_of(0), nxt = page_of(1), nx2 = page_of(2);
      int stage = 0;
      uint32_t par = 1;  // the first use of a stage finds it empty
      for (int b = 0; b < nb; ++b) {
        if (lane < 4) {
          const int nch = is_v ? NCHV : NCH, c0 = is_v ? vh * NCHV : 0;  // (512-dim heads: this CTA's half of the V row)
          uint8_t* dst = ring + stage * (is_v ? V_TILE : KV_TILE) + lane * 2048;
          if (KSUB > 1 && !is_v) {
            // the one K tile of a 512-dim pass, part by part (barriers 0 .. KSUB-1, the same phase for a block)
            constexpr int CPP = NCH / KSUB;  // chunks per part
#pragma unroll
            for (int u = 0; u < KSUB; ++u) {
              wait_bar(&empty[u], par, kStatusMmaTimeout);
              if (cur.kind < 0) {
                mbar_arrive(&full[u]);
              } else {
                const int y = cur.kind ? cur.raw : (cur.raw * 2) * p.bt + cur.off;
                const CUtensorMap* m = cur.kind ? batch_map : &pool_map;
                mbar_arrive_expect_tx(&full[u], 2048 * CPP);
#pragma unroll
                for (int c = u * CPP; c < (u + 1) * CPP; ++c) tma_load_3d(dst + c * HALF_KV, m, &full[u], 0, y, kvh * NCH + c);
              }
            }
          } else {
          wait_bar(&empty[stage], par, kStatusMmaTimeout);
          if (cur.kind < 0) {
            mbar_arrive(&full[stage]);
          } else {
            const int y = cur.kind ? cur.raw : (cur.raw * 2 + (is_v ? 1 : 0)) * p.bt + cur.off;
            const CUtensorMap* m = cur.kind ? batch_map : &pool_map;
            mbar_arrive_expect_tx(&full[stage], 2048 * nch);
#pragma unroll
            for (int c = 0; c < NCH; ++c)
              if (c < nch) tma_load_3d(dst + c * HALF_KV, m, &full[stage], 0, y, kvh * NCH + c0 + c);
          }
          }
          if (lane == 0) stamp(b, is_v ? 7 : 6);
          cur = nxt;
          nxt = nx2;
          nx2 = page_of(b + 3);
          if (++stage == depth) stage = 0, par ^= 1;
        }
        if constexpr (WIN) {
          if (pos_lanes) {
            __syncwarp();  // the page lanes have their slot: the softmax warps are at most KS + 1 blocks behind
            if (b >= nbc) {
              const int slot = (b - nbc) % kPosSlots, jb = batch_j0(b - nbc);
              int lowest = INT_MAX;
#pragma unroll
              for (int q = 0; q < BN / 32; ++q) {
                const int j = jb + lane + 32 * q;
                const int kp = j <= k_last ? a.pos[4 * size_t(tree.base + j)] : INT_MAX;
                shw.kpos[slot][lane + 32 * q] = kp;
                lowest = min(lowest, kp);
              }
#pragma unroll
              for (int o = 16; o; o >>= 1) lowest = min(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
              if (lane == 0) shw.kpos_min[slot] = lowest;
              __syncwarp();
              if (lane == 0) mbar_arrive(&shw.kpos_full[slot]);
            }
          }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA issuer (one thread)
    if (lane == 0 && nb > 0) {
      constexpr uint32_t idesc_qk = umma_idesc<CDT>(BM, BN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc<CDT>(BM, HV, 0, 1);
      // Descriptors are built once: inside the loop a descriptor is the base plus a constant in
      // its address field (one thread issues everything, so every integer op here is latency).
      const uint64_t q_desc = umma_smem_desc(smem_u32(q_sm), 16, 1024);
      const uint64_t k_desc = umma_smem_desc(smem_u32(k_sm), 16, 1024);
      const uint64_t v_desc = umma_smem_desc(smem_u32(v_sm), HALF_KV, 1024);
      auto issue_qk = [&](int b) {
        const int stage = b & 1;               // S buffer
        const int kst = b % KS;                // K ring slot
        const uint64_t kd = k_desc + uint64_t(kst * (KV_TILE >> 4));
        const uint32_t td = tmem + COL_S + stage * BN;
        constexpr int SPP = HD / 16 / KSUB;    // MMAs per part of the K tile (all of them but for 512-dim heads)
#pragma unroll
        for (int u = 0; u < KSUB; ++u) {
          uint64_t* kf = KSUB > 1 ? &k_full[u] : &k_full[kst];
          wait_bar(kf, KSUB > 1 ? uint32_t(b & 1) : uint32_t((b / KS) & 1), kStatusTmaTimeout);
          tc_fence_after_sync();
#pragma unroll
          for (int ks = u * SPP; ks < (u + 1) * SPP; ++ks) {
            const uint64_t db = kd + uint64_t(((ks >> 2) * HALF_KV + (ks & 3) * 32) >> 4);
            if constexpr (QT) {
              umma_ts(td, tmem + COL_Q + ks * 8, db, idesc_qk, ks > 0);
            } else {
              const uint64_t da = q_desc + uint64_t(((ks >> 2) * HALF_Q + (ks & 3) * 32) >> 4);
              umma_ss(td, da, db, idesc_qk, ks > 0);
            }
          }
          umma_commit(KSUB > 1 ? &k_empty[u] : &k_empty[kst]);  // the K slot (part) may be refilled once these MMAs are done
        }
        umma_commit(&s_full[stage]);
      };
      // S of block b + 1 is computed while the softmax warps work on block b (two S buffers);
      // MMAs run in issue order, so Q.K^T of block b + 2 overwrites buffer b & 1 only after
      // P.V of block b has read P from it.
      if constexpr (QT) {
        wait_bar(&sh.q_full, 0, kStatusMmaTimeout);  // the Q tile is in tensor memory
        tc_fence_after_sync();
      }
      issue_qk(0);
      if (nb > 1) issue_qk(1);
      for (int b = 0; b < nb; ++b) {
        const int stage = b & 1;   // S / P buffer
        const int vst = b % VS;    // V ring slot
        wait_bar(&p_full[stage], (b >> 1) & 1, kStatusMmaTimeout);  // P_b is in tensor memory
        stamp(b, 3);
        wait_bar(&v_full[vst], (b / VS) & 1, kStatusTmaTimeout);
        stamp(b, 4);
        tc_fence_after_sync();
        const uint64_t vd = v_desc + uint64_t(vst * (V_TILE >> 4));
        const uint32_t tp = tmem + COL_S + stage * BN;
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks)
          umma_ts(tmem + COL_O, tp + ks * 8, vd + uint64_t((ks * 2048) >> 4), idesc_pv, (b > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&v_empty[vst]);
        umma_commit(&pv_done);
        if (b + 2 < nb) issue_qk(b + 2);
        if (b + 1 == nb) umma_commit(&o_full);
        stamp(b, 5);
      }
    }
  } else {
    // ================= softmax: thread i owns row i of S and O (TMEM lane i)
    const uint32_t t_lane = tmem + (uint32_t(warp * 32) << 16);
    const float sl2 = a.scale * kLog2e;
    float m_ref = -INFINITY, l_run = 0.0f;  // m_ref in exp2 units of the scaled score

    for (int b = 0; b < nb; ++b) {
      const int stage = b & 1;
      const bool cached = b < nbc;
      const int j0 = cached ? k0a + BN * b : batch_j0(b - nbc);
      const int n_valid = cached ? min(BN, tile.k1 - j0) : min(BN, k_last + 1 - j0);
      bool need_mask = n_valid < BN;
      if (!cached) {
        if (use_anc) need_mask = true;
        else need_mask = need_mask || !((j0 + BN - 1 < anc_min) || (j0 >= seg_max && j0 + BN - 1 <= r_first));
      }
      // Sliding-window layers: a cached key sits at position j, so a block needs the window's lower edge when the latest
      // row's first visible position lies beyond its first key; a batch key sits at its row's position, which the K
      // producer left in shared memory with the block's earliest one.
      bool win_keys = false;
      const int wslot = (b - nbc) % kPosSlots;
      if (windowed) {
        if (cached) {
          need_mask = need_mask || j0 < lo_max;
        } else {
          wait_bar(&shw.kpos_full[wslot], uint32_t((b - nbc) / kPosSlots) & 1u, kStatusTmaTimeout);
          win_keys = shw.kpos_min[wslot] < lo_max;
          need_mask = need_mask || win_keys;
        }
      }
      wait_bar(&s_full[stage], (b >> 1) & 1, kStatusMmaTimeout);
      if (tid == 0) stamp(b, 0);
      tc_fence_after_sync();
      const uint32_t t_s = t_lane + COL_S + stage * BN;
      uint32_t sr[2][32];
      tmem_ld32(t_s, sr[0]);
      tmem_ld32(t_s + 32, sr[1]);
      tmem_wait_ld();
      if (tid == 0) stamp(b, 1);
      float mx = -INFINITY;
      if (need_mask) {
        // diagonal, tail and tree blocks: the visibility of this row's 64 columns as one bit mask
        // (a few integer operations), then one select per score
        uint64_t vm = low_bits64(n_valid);
        if (!cached) {
          if (use_anc) {
            vm &= am >> (j0 & 63);  // one block, j0 = 0
          } else {
            const int own_end = bidi ? max(rr + 1, d.w) : rr + 1;  // an image row's segment reaches the image's end
            vm &= low_bits64(d.z - j0) | (low_bits64(own_end - j0) & ~low_bits64(d.x - j0));  // j < d.z || d.x <= j < own_end
          }
          if (win_keys) {
            uint64_t wm = 0;
            for (int c = 0; c < 64; ++c) wm |= uint64_t(qpos - shw.kpos[wslot][c] < a.window) << c;
            vm &= wm;
          }
        } else if (windowed) {
          vm &= ~low_bits64(qpos - a.window + 1 - j0);  // j >= the row's first visible position
        }
        const uint32_t vw[2] = {uint32_t(vm), uint32_t(vm >> 32)};
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const float s = ((vw[h] >> c) & 1u) ? __uint_as_float(sr[h][c]) : -INFINITY;
            sr[h][c] = __float_as_uint(s);
            mx = fmaxf(mx, s);
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
        wait_bar(&pv_done, (b - 1) & 1, kStatusMmaTimeout);  // O holds blocks 0 .. b-1 and is idle
        tc_fence_after_sync();
      }
      if (b > 0 && __any_sync(0xffffffffu, grow)) {
        // O of this warp's rows *= factor (1 for rows whose reference did not move)
#pragma unroll 1
        for (int c = 0; c < HV / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(t_lane + COL_O + 32 * c, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
          tmem_st32(t_lane + COL_O + 32 * c, o);
        }
      }
      tmem_wait_st();
      if (!F8 && n_valid < BN) {  // (E4M3 pools: the converter warps write zeros there)
        // tail block: V rows past the range are stale or foreign bytes; 0 * NaN must not happen
        const int vst = b % VS;
        wait_bar(&v_full[vst], (b / VS) & 1, kStatusTmaTimeout);
        const int n = (BN - n_valid) * 8 * NCHV;  // 16-byte pieces: NCHV chunks x 8 per row
        for (int i = tid; i < n; i += BM) {
          const int r = n_valid + i / (8 * NCHV), c = i % (8 * NCHV);
          *reinterpret_cast<uint4*>(v_sm + vst * V_TILE + (c >> 3) * HALF_KV + r * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
      }
      tc_fence_before_sync();
      mbar_arrive(&p_full[stage]);
      if (tid == 0) stamp(b, 2);
    }

    // ---- epilogue
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the combine grid may be scheduled
    if (nb > 0) {
      wait_bar(&o_full, 0, kStatusMmaTimeout);
      tc_fence_after_sync();
    }
    if (tid == 0) cta_stamp(1);
    const int hg = head % G;
    float* rec = nullptr;
    typename QE::T* op = nullptr;
    const float* gp = nullptr;
    if (tile.part >= 0) rec = a.parts + ((size_t(tile.part) * p.Hkv + kvh) * TR * G + size_t(fm) * G + hg) * (HD + 2);
    else {
      op = static_cast<typename QE::T*>(a.O) + size_t(row) * p.q_ld + size_t(head) * HD;
      if (a.X) gp = a.X + size_t(row) * p.g_ld + size_t(head) * 2 * HD + HD;
    }
    const float inv_l = l_run > 0.0f ? 1.0f / l_run : 0.0f;
    // ---- merge inside the kernel (what attention_combine does, kernels/40_attention.metal:811-864): tiles of 128 / G
    // rows x G heads, whose 128 records are one contiguous range of `parts`. Every CTA stages its records in the idle
    // tile memory, writes them with coalesced stores and draws a ticket of its (job, kv head); whoever draws the last
    // one folds the job's records in record order - each brought back by one bulk copy, summed in tensor memory with
    // weights e^(m_s - M) - and writes the rows. Nobody waits for anybody; the result does not depend on who came last.
    // (256-dim heads only: 128-dim verify passes run on flash_umma, which has its own merge.)
    bool merged_here = false;
    if (QT && a.fuse != 0 && rec != nullptr && HPC == G) {
      named_barrier(2, kSoftmaxThreads);
      if (tid == 0) red[0] = dead;
      named_barrier(2, kSoftmaxThreads);
      merged_here = red[0] == 0;  // after a timed-out wait loads may still be in flight into the tile memory: plain route
    }
    if (QT && merged_here) {
      constexpr int RW = HD + 2;                       // floats per record
      constexpr uint32_t kRecBytes = BM * RW * 4;      // the CTA's records
      float* stage = reinterpret_cast<float*>(smem);   // every issued load was consumed by an MMA that has completed
      float* rec0 = a.parts + (size_t(tile.part) * p.Hkv + kvh) * TR * G * RW;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        if (nb > 0) {  // tensor-memory loads are warp-wide: every lane takes part, rows past the tree store zeros
          tmem_ld32(t_lane + COL_O + 32 * c, o);
          tmem_wait_ld();
        }
        if (nb <= 0 || !row_ok) {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) *reinterpret_cast<float2*>(stage + tid * RW + 32 * c + i) = make_float2(__uint_as_float(o[i]), __uint_as_float(o[i + 1]));
      }
      *reinterpret_cast<float2*>(stage + tid * RW + HD) = row_ok ? make_float2(m_ref * kLn2, l_run) : make_float2(-INFINITY, 0.0f);
      named_barrier(2, kSoftmaxThreads);
      {
        const float4* src = reinterpret_cast<const float4*>(stage);
        float4* dst = reinterpret_cast<float4*>(rec0);
#pragma unroll 8
        for (int i = tid; i < BM * RW / 4; i += kSoftmaxThreads) dst[i] = src[i];
      }
      const esp_attn_combine job = a.jobs[tile.pad1 - 1];
      int* ticket = a.counters + (size_t(tile.pad1 - 1) * p.Hkv + kvh) * kFixupPerJob;
      __threadfence();
      named_barrier(2, kSoftmaxThreads);
      if (tid == 0) {
        const int prev = atomicAdd(ticket, 1);
        if (prev == job.nparts - 1) *ticket = 0;  // ready for the next pass on this stream
        red[0] = prev;
      }
      named_barrier(2, kSoftmaxThreads);
      if (tid == 0) cta_stamp(2);
      if (red[0] == job.nparts - 1) {
        __threadfence();
        // weights: M and L over the job's records of this (row, head)
        const float* recs = a.parts + (size_t(job.part0) * p.Hkv + kvh) * TR * G * RW;
        const size_t part_stride = size_t(p.Hkv) * TR * G * RW;
        // The sum is built in the tensor-memory columns of S and Q (idle now), so this CTA's own O stays where it is and
        // is folded from there when its turn comes; only the other records travel (one bulk copy each into `stage`,
        // the next one requested as soon as the last was consumed).
        auto acc_col = [&](int c) { return c < 4 ? COL_S + 32u * uint32_t(c) : COL_Q + 32u * uint32_t(c - 4); };
        const int own = tile.part - job.part0;
        auto request = [&](int s2) {  // thread 0
          asm volatile("fence.proxy.async;" ::: "memory");  // the records were written through the generic proxy
          mbar_arrive_expect_tx(&sh.fix_bar, kRecBytes);
          bulk_load(stage, recs + size_t(s2) * part_stride, kRecBytes, &sh.fix_bar);
        };
        auto next_other = [&](int s2) { return s2 == own ? s2 + 1 : s2; };
        named_barrier(2, kSoftmaxThreads);  // everybody has copied its share of `stage` to the records
        if (tid == 0 && next_other(0) < job.nparts) request(next_other(0));
        float M = -INFINITY, L = 0.0f;
#pragma unroll 1
        for (int s2 = 0; s2 < job.nparts; ++s2) M = fmaxf(M, __ldcg(recs + size_t(s2) * part_stride + tid * RW + HD));
#pragma unroll 1
        for (int s2 = 0; s2 < job.nparts; ++s2) {
          const float2 ml = __ldcg(reinterpret_cast<const float2*>(recs + size_t(s2) * part_stride + tid * RW + HD));
          if (ml.x != -INFINITY) L = fmaf(__expf(ml.x - M), ml.y, L);
        }
        bool alive = true;
        uint32_t par = 0;
        if (job.nparts == 2) {
          // The common case (a prefix cut in two): one sweep over the dims with both records at hand - this CTA's O in
          // tensor memory, the other one in `stage` - summed in record order like the general loop below, and written.
          if (!mbar_wait(&sh.fix_bar, par)) {
            dead = 1;
            atomicExch(a.status, kStatusTmaTimeout);
          }
          named_barrier(2, kSoftmaxThreads);
          if (!dead) {
            const float m_own = row_ok ? m_ref * kLn2 : -INFINITY, m_oth = stage[tid * RW + HD];
            const float w_own = m_own == -INFINITY ? 0.0f : __expf(m_own - M), w_oth = m_oth == -INFINITY ? 0.0f : __expf(m_oth - M);
            const float w0 = own == 0 ? w_own : w_oth, w1 = own == 0 ? w_oth : w_own;
            const float inv_L = L > 0.0f ? 1.0f / L : 0.0f;
            typename QE::T* orow = static_cast<typename QE::T*>(a.O) + size_t(row) * p.q_ld + size_t(head) * HD;
            const float* gate = a.X ? a.X + size_t(row) * p.g_ld + size_t(head) * 2 * HD + HD : nullptr;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
              uint32_t v[32];
              if (nb > 0) {
                tmem_ld32(t_lane + COL_O + 32 * c, v);
                tmem_wait_ld();
              }
              if (row_ok) {
                float o[32];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  const float2 x = *reinterpret_cast<const float2*>(stage + tid * RW + 32 * c + i);
                  const float a0 = own == 0 ? __uint_as_float(v[i]) : x.x, b0 = own == 0 ? x.x : __uint_as_float(v[i]);
                  const float a1 = own == 0 ? __uint_as_float(v[i + 1]) : x.y, b1 = own == 0 ? x.y : __uint_as_float(v[i + 1]);
                  float s0 = w0 != 0.0f ? w0 * a0 : 0.0f, s1 = w0 != 0.0f ? w0 * a1 : 0.0f;
                  if (w1 != 0.0f) s0 = fmaf(w1, b0, s0), s1 = fmaf(w1, b1, s1);
                  o[i] = s0 * inv_L, o[i + 1] = s1 * inv_L;
                }
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                  if (gate) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) o[i + k] *= sigmoid_gate(gate[32 * c + i + k]);
                  }
                  uint4 w4;
                  w4.x = QE::pack2(o[i], o[i + 1]), w4.y = QE::pack2(o[i + 2], o[i + 3]);
                  w4.z = QE::pack2(o[i + 4], o[i + 5]), w4.w = QE::pack2(o[i + 6], o[i + 7]);
                  *reinterpret_cast<uint4*>(orow + 32 * c + i) = w4;
                }
              }
              __syncwarp();
            }
            if (row_ok && a.lse) a.lse[size_t(row) * p.H + head] = L > 0.0f ? M + __logf(L) : -INFINITY;
          }
          alive = false;  // done (or given up): the general loop and its write-out are skipped
        }
#pragma unroll 1
        for (int s2 = 0; alive && s2 < job.nparts; ++s2) {
          const bool mine = s2 == own;
          float m_s;
          if (mine) {
            m_s = row_ok ? m_ref * kLn2 : -INFINITY;
          } else {
            if (!mbar_wait(&sh.fix_bar, par)) {
              dead = 1;
              atomicExch(a.status, kStatusTmaTimeout);
            }
            par ^= 1;
            named_barrier(2, kSoftmaxThreads);
            if (dead) {  // one verdict for all: the rows are left alone, the status word says why
              alive = false;
              break;
            }
            m_s = stage[tid * RW + HD];
          }
          const float w = m_s == -INFINITY ? 0.0f : __expf(m_s - M);
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32], v[32];
            if (s2 > 0) tmem_ld32(t_lane + acc_col(c), o);
            if (mine && nb > 0) tmem_ld32(t_lane + COL_O + 32 * c, v);
            if (s2 > 0 || (mine && nb > 0)) tmem_wait_ld();
            if (s2 == 0) {
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = 0;
            }
            if (!mine) {
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float2 x = *reinterpret_cast<const float2*>(stage + tid * RW + 32 * c + i);
                v[i] = __float_as_uint(x.x), v[i + 1] = __float_as_uint(x.y);
              }
            }
            if (w != 0.0f) {  // (a record that weighs nothing may hold anything)
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(fmaf(w, __uint_as_float(v[i]), __uint_as_float(o[i])));
            }
            __syncwarp();
            tmem_st32(t_lane + acc_col(c), o);
          }
          tmem_wait_st();
          if (!mine) {
            named_barrier(2, kSoftmaxThreads);  // the record in `stage` has been consumed
            if (tid == 0 && next_other(s2 + 1) < job.nparts) request(next_other(s2 + 1));
          }
        }
        if (alive) {  // (warp-wide tensor-memory loads again: only the stores depend on the row)
          const float inv_L = L > 0.0f ? 1.0f / L : 0.0f;
          typename QE::T* orow = static_cast<typename QE::T*>(a.O) + size_t(row) * p.q_ld + size_t(head) * HD;
          const float* gate = a.X ? a.X + size_t(row) * p.g_ld + size_t(head) * 2 * HD + HD : nullptr;
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(t_lane + acc_col(c), o);
            tmem_wait_ld();
            if (row_ok) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                float v[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                  v[k] = __uint_as_float(o[i + k]) * inv_L;
                  if (gate) v[k] *= sigmoid_gate(gate[32 * c + i + k]);
                }
                uint4 w4;
                w4.x = QE::pack2(v[0], v[1]), w4.y = QE::pack2(v[2], v[3]), w4.z = QE::pack2(v[4], v[5]), w4.w = QE::pack2(v[6], v[7]);
                *reinterpret_cast<uint4*>(orow + 32 * c + i) = w4;
              }
            }
            __syncwarp();
          }
          if (row_ok && a.lse) a.lse[size_t(row) * p.H + head] = L > 0.0f ? M + __logf(L) : -INFINITY;
        }
      }
    }
#pragma unroll 1
    for (int c = 0; c < (merged_here ? 0 : HV / 32); ++c) {
      uint32_t o[32];
      if (nb > 0) {
        tmem_ld32(t_lane + COL_O + 32 * c, o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0;
      }
      if (!row_ok) continue;
      if (rec) {
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          *reinterpret_cast<float2*>(rec + ho + 32 * c + i) = make_float2(__uint_as_float(o[i]), __uint_as_float(o[i + 1]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          float v[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            v[k] = __uint_as_float(o[i + k]) * inv_l;
            if (gp) v[k] *= sigmoid_gate(gp[ho + 32 * c + i + k]);
          }
          uint4 w;
          w.x = QE::pack2(v[0], v[1]), w.y = QE::pack2(v[2], v[3]), w.z = QE::pack2(v[4], v[5]), w.w = QE::pack2(v[6], v[7]);
          *reinterpret_cast<uint4*>(op + ho + 32 * c + i) = w;
        }
      }
    }
    if (row_ok && !merged_here && vh == 0) {  // (512-dim heads: both halves hold the same m and l; the first one writes them)
      if (rec) {
        rec[HD] = m_ref * kLn2;  // -inf stays -inf
        rec[HD + 1] = l_run;
      } else if (a.lse) {
        a.lse[size_t(row) * p.H + head] = l_run > 0.0f ? m_ref * kLn2 + __logf(l_run) : -INFINITY;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tracing && tid == 0) a.trace[8 * a.trace_blocks + 1] = global_timer_ns();
  if (tid == 0) cta_stamp(3);
  if (warp == kMmaWarp) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace

template <int QDT, int HD, int KS, int VS>
cudaError_t setup_variant() {
  return cudaFuncSetAttribute(flash_umma_pair_kernel<QDT, HD, KS, VS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(HD, KS, VS));
}

cudaError_t flash_umma_pair_setup() {
  cudaError_t e = setup_variant<ESP_F16, 128, 3, 2>();
  if (e == cudaSuccess) e = setup_variant<ESP_BF16, 128, 3, 2>();
  if (e == cudaSuccess) e = setup_variant<ESP_F16, 64, 3, 2>();
  if (e == cudaSuccess) e = setup_variant<ESP_BF16, 64, 3, 2>();
  if (e == cudaSuccess) e = setup_variant<ESP_F16, 512, 1, 1>();
  if (e == cudaSuccess) e = setup_variant<ESP_BF16, 512, 1, 1>();
  if (e == cudaSuccess) e = setup_variant<ESP_F16, 256, 4, 3>();
  if (e == cudaSuccess) e = setup_variant<ESP_BF16, 256, 4, 3>();
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(flash_umma_pair_kernel<ESP_F16, 256, 2, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes_f8(256, 2, 2));
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(flash_umma_pair_kernel<ESP_BF16, 256, 2, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes_f8(256, 2, 2));
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(flash_umma_pair_kernel<ESP_F16, 256, 3, 3, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes_win(256, 3, 3));
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(flash_umma_pair_kernel<ESP_BF16, 256, 3, 3, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes_win(256, 3, 3));
  return e;
}

// 128-dim heads: rings of 3 K and 2 V tiles, two CTAs per SM. 256-dim heads (the head dim of
// kernels/40_attention.metal's flash_attention): the Q tile in tensor memory (128 columns behind two S buffers
// and O: all 512), rings of 4 K + 3 V tiles of 32 KB (224 KB: the SM's shared memory), one CTA per SM.
cudaError_t launch_flash_umma_pair(const KernelArgs& a, const CUtensorMap& pool_map, const CUtensorMap& kb_map,
                                   const CUtensorMap& vb_map, bool e4m3_direct, cudaStream_t stream, uint64_t* launches) {
  if (a.n_tiles <= 0) return cudaSuccess;
  const int hpc = BM / a.tile_rows;
  const dim3 grid(unsigned(a.n_tiles), unsigned(a.p.H / hpc)), block(kThreads);
  const bool f16 = a.q_dtype == ESP_F16;
  if (e4m3_direct) {  // 256-dim heads over an E4M3 pool: pool_map is the pool's byte map (16 rows x 2 lines per page and kv head)
    if (a.HD != 256 || a.kv_dtype != ESP_E4M3 || a.kv_scales == nullptr) return cudaErrorInvalidValue;
    constexpr int smem = smem_bytes_f8(256, 2, 2);
    cudaError_t e = f16 ? launch_pdl(flash_umma_pair_kernel<ESP_F16, 256, 2, 2, true>, grid, dim3(kThreadsF8), smem, stream, pool_map, kb_map, vb_map, a)
                        : launch_pdl(flash_umma_pair_kernel<ESP_BF16, 256, 2, 2, true>, grid, dim3(kThreadsF8), smem, stream, pool_map, kb_map, vb_map, a);
    if (e == cudaSuccess) ++*launches;
    return e;
  }
  if (a.window > 0 || a.ring > 0 || a.bidi != 0) {  // sliding-window layers: their own instantiation (256-dim heads, 16-bit pools)
    if (a.HD != 256 || a.kv_dtype == ESP_E4M3) return cudaErrorInvalidValue;
    constexpr int smem = smem_bytes_win(256, 3, 3);
    cudaError_t e = f16 ? launch_pdl(flash_umma_pair_kernel<ESP_F16, 256, 3, 3, false, true>, grid, block, smem, stream, pool_map, kb_map, vb_map, a)
                        : launch_pdl(flash_umma_pair_kernel<ESP_BF16, 256, 3, 3, false, true>, grid, block, smem, stream, pool_map, kb_map, vb_map, a);
    if (e == cudaSuccess) ++*launches;
    return e;
  }
  if (a.HD == 512) {  // one CTA per (tile, head group, half of the output dims)
    const dim3 grid2(grid.x, grid.y, 2);
    constexpr int smem = smem_bytes(512, 1, 1);
    if (f16) flash_umma_pair_kernel<ESP_F16, 512, 1, 1><<<grid2, block, smem, stream>>>(pool_map, kb_map, vb_map, a);
    else flash_umma_pair_kernel<ESP_BF16, 512, 1, 1><<<grid2, block, smem, stream>>>(pool_map, kb_map, vb_map, a);
  } else if (a.HD == 128) {
    constexpr int smem = smem_bytes(128, 3, 2);
    if (f16) flash_umma_pair_kernel<ESP_F16, 128, 3, 2><<<grid, block, smem, stream>>>(pool_map, kb_map, vb_map, a);
    else flash_umma_pair_kernel<ESP_BF16, 128, 3, 2><<<grid, block, smem, stream>>>(pool_map, kb_map, vb_map, a);
  } else if (a.HD == 64) {  // kernels/90_lfm2.metal:160-161: one 64-dim chunk per row, 56 KB per CTA
    constexpr int smem = smem_bytes(64, 3, 2);
    if (f16) flash_umma_pair_kernel<ESP_F16, 64, 3, 2><<<grid, block, smem, stream>>>(pool_map, kb_map, vb_map, a);
    else flash_umma_pair_kernel<ESP_BF16, 64, 3, 2><<<grid, block, smem, stream>>>(pool_map, kb_map, vb_map, a);
  } else {
    constexpr int smem = smem_bytes(256, 4, 3);
    cudaError_t e = f16 ? launch_pdl(flash_umma_pair_kernel<ESP_F16, 256, 4, 3>, grid, block, smem, stream, pool_map, kb_map, vb_map, a)
                        : launch_pdl(flash_umma_pair_kernel<ESP_BF16, 256, 4, 3>, grid, block, smem, stream, pool_map, kb_map, vb_map, a);
    if (e == cudaSuccess) ++*launches;
    return e;
  }
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) ++*launches;
  return e;
}

}  // namespace esp
