// Forest attention on the 5th-generation tensor cores (sm_100a), variant for compute-bound passes
// (causal prefill): one CTA per SM works on TWO 128-lane query tiles against the same key blocks.
// flash_umma.cu streams a long cached prefix from HBM, flash_umma_pair.cu puts two independent CTAs
// on an SM; all three compute the same.
//
// Computes what flash_attention computes (kernels/40_attention.metal:156-343 of the reference):
// the tile's rows attend to the cached key range [k0, k1) of the paged pool and, when tile.last,
// to the visible batch keys of their tree (two-level `desc` mask or a 64-bit ancestor mask per
// row), writing either the partial record [O | m | l] or the gated, normalised output (and LSE).
//
// B200 structure. A CTA covers tile_rows rows x 2 * (128 / tile_rows) heads of one kv head: two
// query tiles of 128 (row, head) pairs = 2 x 128 lanes of tensor memory (prefill: the same 128
// rows for two heads of a group, so both tiles see the same keys under the same mask). Keys are
// processed 128 at a time, one K and one V tile in shared memory serving both query tiles:
//   S_t[128 x 128] = Q_t . K^T   8 tcgen05.mma (N = 128, K = 16) per query tile, operands from shared
//                                memory (K-major, 128-byte swizzle), D in tensor memory. An N = 128
//                                instruction reads 4 KB of A and 4 KB of B for 64 cycles of math: the
//                                shared-memory port keeps up, which it does not with 64-key blocks.
//   softmax        one warpgroup per query tile, thread i owns row i of its tile: its 128 scores in
//                  registers, the row maximum, then P (exp2 domain, two scores per fp32x2
//                  instruction; 16-bit pairs written over the scores with tcgen05.st), handed over
//                  in two halves of 64 keys. (Taking part of the exponentials from a cubic on the
//                  FMA pipe, to relieve the exp2 unit, measured slower: 5.4 ms with a quarter and
//                  6.2 ms with half of them against 4.2 ms for the full prefill pass.)
//   O_t[128 x HD] += P_t . V     8 tcgen05.mma with A = P_t from tensor memory, B = V (MN-major)
// Tensor memory: S_0, S_1, O_0, O_1 of 128 fp32 columns each = all 512 columns. The MMA thread issues
// P_0.V, Q_0.K^T(next), P_1.V, Q_1.K^T(next): while one warpgroup runs its softmax the tensor pipe
// works for the other tile, so the two warpgroups settle half a period apart and the exp2 unit,
// which has as many cycles of work per key block as the tensor pipe, is fed by one of them at any
// time. O stays in tensor memory for the whole tile and is rescaled only when a row's maximum has
// grown by more than 2^8 (warp-uniform decision); S_t of the next block is only written once every
// earlier MMA has completed, so the owner of tile t may touch O_t as soon as it sees S_t.
// Warps: 0-3 softmax of tile 0, 4-7 softmax of tile 1, 8 MMA issue (one thread; owns tensor memory),
// 9 K producer, 10 V producer (TMA, one bulk tensor load per 16-key page and 64-dim half), 11 idle
// (it completes the third warpgroup, which hands most of its registers to the softmax warpgroups).
// They hand tiles to one another through mbarriers only. Every wait is bounded: after a timeout the CTA
// records a status code, stops waiting, finishes its loop, frees its tensor memory and returns.
#include <climits>
#include <cstddef>

#include "umma.cuh"
#include "../launch.h"

namespace esp {
namespace {

constexpr int BM = 128;  // (row, head) pairs per query tile
constexpr int NQ = 2;    // query tiles per CTA
constexpr int BN = 128;  // keys per block
constexpr int HD = 128;  // head dim of this kernel
constexpr int Q_BYTES = BM * HD * 2;        // one query tile: [2 halves of 64 dims][128 rows][128 B]
constexpr int KV_TILE = BN * HD * 2;        // [2 halves of 64 dims][128 rows][128 B]
constexpr int HALF_T = 128 * 128;           // bytes between the 64-dim halves of a tile
constexpr int KS = 2, VS = 2;               // K and V ring depths (the keys of a prefill sit in L2)
constexpr int TILES_BYTES = NQ * Q_BYTES + (KS + VS) * KV_TILE;
constexpr int SMEM_BYTES = TILES_BYTES + 256;  // + mbarriers and bookkeeping; no static shared memory
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_S = 0, COL_O = 256;  // S_t at COL_S + 128 t (P_t over its first 64 columns), O_t at COL_O + 128 t
constexpr float kRescaleThreshold = 8.0f;   // log2 units

constexpr int kSoftmaxThreads = NQ * BM;
constexpr int kMmaWarp = 8;
constexpr int kTmaWarpK = 9;
constexpr int kTmaWarpV = 10;
constexpr int kThreads = 12 * 32;            // warps 8-11 form the third warpgroup; warp 11 only gives up its registers
constexpr int kPages = BN / 16;             // TMA pages per tile
constexpr int kPosSlots = 4;                // batch blocks whose key positions are kept (two in the K ring, two in the softmax)
// Registers move from the third warpgroup (MMA issue, TMA producers) to the softmax warpgroups once the kernel runs
// (setmaxnreg): a softmax thread holds its 128 scores at once. 128 x 96 + 256 x 192 <= 64 K registers.
constexpr int kRegsAux = 96, kRegsSoftmax = 192;

__device__ __forceinline__ uint64_t low_bits64(int n) { return n <= 0 ? 0ull : (n >= 64 ? ~0ull : ((1ull << n) - 1ull)); }

struct PageRef {  // where one 16-key page of a key block comes from
  int raw;        // block id as loaded from the page table (pool), or first row (Kb / Vb)
  int off;        // row inside the block (pool)
  int kind;       // -1: nothing to load, 0: paged pool, 1: Kb / Vb
};

struct Shared {
  uint64_t k_full[KS], k_empty[KS], v_full[VS], v_empty[VS], s_full[NQ], p_full[NQ][2], o_full;
  uint32_t tmem_slot;
  int red[6];  // anc_max, seg_min, anc_min, seg_max; sliding-window layers: latest query position, furthest image end
  volatile int dead;
  // sliding-window layers only (the launch reserves this part for them alone): the positions of a batch block's keys
  uint64_t kpos_full[kPosSlots];
  int kpos_min[kPosSlots];
  int kpos[kPosSlots][BN];
};
static_assert(offsetof(Shared, kpos_full) <= 256, "bookkeeping must fit behind the tiles");
constexpr int SMEM_BYTES_WIN = TILES_BYTES + int((sizeof(Shared) + 127) / 128 * 128);

__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// 32 lanes x 32 bit, 16 consecutive columns (the P of 32 keys as 16-bit pairs).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
      "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
      : "memory");
}
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// tcgen05.wait::ld that also names the registers of an earlier asynchronous load as operands: no use of them can be
// scheduled above the wait.
__device__ __forceinline__ void tmem_wait_ld_of(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
                 "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                 "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

template <int QDT, bool WIN>
__global__ void __launch_bounds__(kThreads, 1)
    flash_umma_duo_kernel(const __grid_constant__ CUtensorMap pool_map, const __grid_constant__ CUtensorMap kb_map,
                          const __grid_constant__ CUtensorMap vb_map, const KernelArgs a) {
  using QE = Elem16<QDT>;
  extern __shared__ __align__(1024) uint8_t smem[];
  // full: TMA -> MMA; empty: MMA -> TMA (tcgen05.commit); s_full[t]: S_t written; p_full[t]: P_t written
  // (128 arrivals); o_full: last P.V done
  Shared& sh = *reinterpret_cast<Shared*>(smem + TILES_BYTES);
  uint64_t* k_full = sh.k_full;
  uint64_t* k_empty = sh.k_empty;
  uint64_t* v_full = sh.v_full;
  uint64_t* v_empty = sh.v_empty;
  uint64_t* s_full = sh.s_full;
  uint64_t (*p_full)[2] = sh.p_full;
  uint64_t& o_full = sh.o_full;
  int* red = sh.red;
  volatile int& dead = sh.dead;
  if ((smem_u32(smem) & 1023u) != 0) {  // never expected; the tiles' swizzle would be wrong
    if (threadIdx.x == 0) atomicExch(a.status, kStatusBadBlock);
    return;
  }
  uint8_t* q_sm = smem;                                // NQ tiles
  uint8_t* k_sm = smem + NQ * Q_BYTES;                 // KS tiles
  uint8_t* v_sm = smem + NQ * Q_BYTES + KS * KV_TILE;  // VS tiles

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const esp_attn_params& p = a.p;
  pdl_wait();  // the plan, Q and the mask records belong to the stream's order
  const int tile_i = int(gridDim.x) - 1 - int(blockIdx.x);  // long (late) tiles first
  const esp_attn_tile tile = a.tiles[tile_i];
  const esp_attn_tree tree = a.trees[tile.tree];
  const int bt = p.bt, G = a.G, TR = a.tile_rows, HPC = BM / TR;
  const int kvh = (int(blockIdx.y) * NQ * HPC) / G;
  const int end = tree.base + tree.M;
  const int rows_live = min(TR, end - tile.r0);
  const bool use_anc = a.anc_mask != nullptr;
  const bool desc_mask = tile.last && !use_anc;

  // per softmax thread: its query tile and its (row, head)
  const int qt = (tid >> 7) & 1, srow = tid & (BM - 1);
  const int fm = srow / HPC, hh = srow % HPC;
  const int head = (int(blockIdx.y) * NQ + qt) * HPC + hh;
  const bool is_softmax = tid < kSoftmaxThreads;
  const bool row_ok = is_softmax && fm < rows_live;
  const int row = row_ok ? tile.r0 + fm : end - 1;
  const int rr = row - tree.base;

  if (tid == 0) {
    for (int s = 0; s < KS; ++s) {
      mbar_init(&k_full[s], kPages);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < VS; ++s) {
      mbar_init(&v_full[s], kPages);
      mbar_init(&v_empty[s], 1);
    }
    for (int i = 0; i < NQ; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i][0], BM);
      mbar_init(&p_full[i][1], BM);
    }
    mbar_init(&o_full, 1);
    mbar_fence_init();
    red[0] = 0, red[1] = 1 << 30, red[2] = 1 << 30, red[3] = 0, red[4] = INT_MIN, red[5] = 0;
    if constexpr (WIN)
      for (int i = 0; i < kPosSlots; ++i) mbar_init(&sh.kpos_full[i], 1);
    dead = 0;
  }
  __syncthreads();

  auto wait_bar = [&](uint64_t* bar, uint32_t parity, int code) {
    if (mbar_try_wait(bar, parity)) return;
    if (dead) return;
    if (!mbar_wait(bar, parity)) {
      dead = 1;
      atomicExch(a.status, code);
    }
  };

  // Optional timeline of CTA (0, 0) (esp_attn_set_trace): per key block, 0 / 1 / 2 = tile 0's scores ready, row maxima
  // known, P handed over; 3 / 4 = P of tile 0 / tile 1 seen by the MMA thread; 5 = the block's MMAs issued; 6 / 7 = tile
  // 1's scores ready, P handed over.
  const bool tracing = a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
  auto stamp = [&](int b, int ev) {
    if (tracing && b < a.trace_blocks) a.trace[8 * b + ev] = global_timer_ns();
  };
  if (tracing && tid == 0) a.trace[8 * a.trace_blocks] = global_timer_ns();
  // phases of the CTA in the last row of the block table: 0 = plan read, barriers set, 1 = Q staged and set-up barrier
  // passed, 2 = last P handed over, 3 = rows written
  auto phase = [&](int ev) {
    if (tracing && tid == 0 && a.trace_blocks > 0) a.trace[8 * (a.trace_blocks - 1) + ev] = global_timer_ns();
  };
  phase(0);

  // Block list: cached 128-key blocks first, then the batch blocks some row of the tile can see.
  // Sliding-window layers (kernels/80_gemma.metal:123-142, :284-285; planner src/model/impl/gemma.h:77-116): a key
  // `window` or more positions behind the query is masked. Their tiles start at the first cached key a row can see,
  // at any alignment: pages are loaded from the 16-key boundary below it (the keys in between are behind every
  // row's window), and batch blocks below the first batch key worth scanning (tile.pad0) are left out.
  const bool windowed = WIN && a.window > 0;
  const bool bidi = WIN && a.bidi != 0 && a.anc_mask == nullptr;  // image rows see their whole image (desc.w = its end)
  const int k0a = WIN ? (tile.k0 & ~15) : tile.k0;
  const int nbc = (tile.k1 - k0a + BN - 1) / BN;
  const int r_first = tile.r0 - tree.base, r_last = r_first + rows_live - 1;
  struct Meta {
    int k_last, a_lo, a_hi, b_lo, nbb, anc_min, seg_max, lo_max;
  };
  auto make_meta_from = [&](int anc_max, int seg_min, int anc_min, int seg_max, int latest, int img_end) {
    Meta m{-1, 0, 0, 0, 0, 0, 0, INT_MIN};
    if (windowed) m.lo_max = latest - a.window + 1;  // the latest row's first visible position
    if (!tile.last) return m;
    if (use_anc) {
      m.k_last = min(tree.M, 64) - 1;
      m.a_hi = (m.k_last + BN) / BN;
      m.nbb = m.a_hi;
      return m;
    }
    m.anc_min = anc_min, m.seg_max = seg_max;
    // (image rows of a bidirectional layer also see the later rows of their image, up to desc.w: img_end is the
    // furthest such end among the tile's rows, 0 otherwise)
    const int reach = max(r_last, img_end - 1);
    m.k_last = min(tree.M - 1, max(reach, anc_max - 1));
    const int n_all = (m.k_last + BN) / BN;
    m.a_hi = min((anc_max + BN - 1) / BN, n_all);  // blocks below the ancestor range
    m.b_lo = max(m.a_hi, seg_min / BN);            // blocks of the rows' own segments
    const int b_hi = min(reach / BN, n_all - 1);
    if (windowed) {
      const int f = max(0, tile.pad0) / BN;
      m.a_lo = min(m.a_hi, f);
      m.b_lo = max(m.b_lo, f);
    }
    m.nbb = (m.a_hi - m.a_lo) + max(0, b_hi - m.b_lo + 1);
    return m;
  };
  auto make_meta = [&]() { return make_meta_from(red[0], red[1], red[2], red[3], red[4], red[5]); };  // after the set-up barrier
  // The same bounds straight from the rows' records, by one warp: the TMA producers do not wait for the softmax
  // warps' set-up to know which batch blocks to fetch.
  auto warp_meta = [&]() {
    int v0 = 0, v1 = 1 << 30, v2 = 1 << 30, v3 = 0, q = INT_MIN, w_end = 0;
    for (int r = lane; r < rows_live; r += 32) {
      if (desc_mask) {
        const int4 d = reinterpret_cast<const int4*>(a.desc)[tile.r0 + r];
        v0 = max(v0, d.z), v1 = min(v1, d.x), v2 = min(v2, d.z), v3 = max(v3, d.x);
        if (bidi) w_end = max(w_end, d.w);
      }
      if (windowed) q = max(q, a.pos[4 * size_t(tile.r0 + r)]);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      v0 = max(v0, __shfl_xor_sync(0xffffffffu, v0, o));
      v1 = min(v1, __shfl_xor_sync(0xffffffffu, v1, o));
      v2 = min(v2, __shfl_xor_sync(0xffffffffu, v2, o));
      v3 = max(v3, __shfl_xor_sync(0xffffffffu, v3, o));
      q = max(q, __shfl_xor_sync(0xffffffffu, q, o));
      w_end = max(w_end, __shfl_xor_sync(0xffffffffu, w_end, o));
    }
    return make_meta_from(v0, v1, v2, v3, q, w_end);
  };
  auto batch_j0 = [&](const Meta& m, int i) { return BN * (i < m.a_hi - m.a_lo ? m.a_lo + i : m.b_lo + (i - (m.a_hi - m.a_lo))); };

  if (warp >= kMmaWarp) {
  setmaxnreg_dec<kRegsAux>();  // the whole third warpgroup, warp 11 included
  if (warp == kTmaWarpK || warp == kTmaWarpV) {
    // ================= TMA producers: warp 9 fills the K ring, warp 10 the V ring; lane w loads the
    // w-th 16-key page of every block.
    if (warp == kTmaWarpK && lane == 0) {
      tma_prefetch_desc(&pool_map);
      tma_prefetch_desc(&kb_map);
      tma_prefetch_desc(&vb_map);
    }
    const bool is_v = warp == kTmaWarpV;
    const int depth = is_v ? VS : KS;
    uint64_t* full = is_v ? v_full : k_full;
    uint64_t* empty = is_v ? v_empty : k_empty;
    uint8_t* ring = is_v ? v_sm : k_sm;
    const CUtensorMap* batch_map = is_v ? &vb_map : &kb_map;
    int stage = 0;
    uint32_t par = 1;  // the first use of a slot finds it empty
    auto issue = [&](const PageRef& r) {  // lanes 0 .. kPages-1: one 16-key page each
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
      if (++stage == depth) stage = 0, par ^= 1;
    };
    // Page-table entries: four key blocks per load (lane l holds the entry of block 4 g + l / 8,
    // page l % 8), two groups ahead of their use.
    auto load_group = [&](int g) {
      const int b = 4 * g + (lane >> 3);
      const int j = k0a + BN * b + 16 * (lane & 7);
      if (!(b < nbc && j < tile.k1)) return -1;
      if (WIN && a.ring > 0) return tree.table + (j / bt) % a.ring;  // a sliding layer's blocks: the slot's ring, no page table
      return a.blocks[tree.table + j / bt];
    };
    int g_cur = load_group(0), g_nxt = load_group(1);
    for (int b = 0; b < nbc; ++b) {
      if (b && (b & 3) == 0) {
        g_cur = g_nxt;
        g_nxt = load_group((b >> 2) + 1);
      }
      const int raw = __shfl_sync(0xffffffffu, g_cur, ((b & 3) << 3) | (lane & 7));
      if (lane < kPages) {
        const PageRef r{raw, (k0a + BN * b + 16 * lane) % bt, raw >= 0 ? 0 : -1};
        issue(r);
      }
    }
    if (tile.last) {
      const Meta m = warp_meta();
      for (int i = 0; i < m.nbb; ++i) {
        const int jb = batch_j0(m, i);
        if (lane < kPages) {
          const int j = jb + 16 * lane;
          PageRef r{tree.base + j, 0, j <= m.k_last ? 1 : -1};
          issue(r);
        }
        if (windowed && !is_v) {
          // the positions of the block's keys, and the earliest of them, for the softmax warps' window masks
          const int slot = i % kPosSlots;
          int lowest = INT_MAX;
#pragma unroll
          for (int q = 0; q < BN / 32; ++q) {
            const int j = jb + lane + 32 * q;
            const int kp = j <= m.k_last ? a.pos[4 * size_t(tree.base + j)] : INT_MAX;
            sh.kpos[slot][lane + 32 * q] = kp;
            lowest = min(lowest, kp);
          }
#pragma unroll
          for (int o = 16; o; o >>= 1) lowest = min(lowest, __shfl_xor_sync(0xffffffffu, lowest, o));
          if (lane == 0) sh.kpos_min[slot] = lowest;
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh.kpos_full[slot]);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA issuer (one thread); the warp owns the tensor memory
    tmem_alloc(&sh.tmem_slot, TMEM_COLS);
    tmem_relinquish();
    tc_fence_before_sync();
    named_barrier(1, kSoftmaxThreads + 32);  // softmax warps + the MMA warp
    tc_fence_after_sync();
    const Meta meta = make_meta();
    const int nb = nbc + meta.nbb;
    const uint32_t tmem = sh.tmem_slot;
    {
      if (lane == 0 && nb > 0) {
        constexpr uint32_t idesc_qk = umma_idesc<QDT>(BM, BN, 0, 0);
        constexpr uint32_t idesc_pv = umma_idesc<QDT>(BM, HD, 0, 1);
        const uint64_t q_desc = umma_smem_desc(smem_u32(q_sm), 16, 1024);
        const uint64_t k_desc = umma_smem_desc(smem_u32(k_sm), 16, 1024);
        const uint64_t v_desc = umma_smem_desc(smem_u32(v_sm), HALF_T, 1024);
        int kst = 0, vst = 0;
        uint32_t kpar = 0, vpar = 0;
        // S_t = Q_t . K^T of the block in K slot kst; the slot is released after tile 1's.
        auto issue_qk = [&](int t) {
          if (t == 0) {
            wait_bar(&k_full[kst], kpar, kStatusTmaTimeout);
            tc_fence_after_sync();
          }
          const uint64_t qd = q_desc + uint64_t((t * Q_BYTES) >> 4);
          const uint64_t kd = k_desc + uint64_t(kst * (KV_TILE >> 4));
          const uint32_t td = tmem + COL_S + t * BN;
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint64_t off = uint64_t(((ks >> 2) * HALF_T + (ks & 3) * 32) >> 4);
            umma_ss(td, qd + off, kd + off, idesc_qk, ks > 0);
          }
          umma_commit(&s_full[t]);
          if (t == NQ - 1) {
            umma_commit(&k_empty[kst]);
            if (++kst == KS) kst = 0, kpar ^= 1;
          }
        };
        issue_qk(0);
        issue_qk(1);
        for (int b = 0; b < nb; ++b) {
#pragma unroll
          for (int t = 0; t < NQ; ++t) {
            const uint64_t vd = v_desc + uint64_t(vst * (KV_TILE >> 4));
            const uint32_t tp = tmem + COL_S + t * BN;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              wait_bar(&p_full[t][h], b & 1, kStatusMmaTimeout);  // P_t of the block's keys [64 h, 64 h + 64) is in tensor memory
              if (h == 0) stamp(b, 3 + t);
              if (t == 0 && h == 0) wait_bar(&v_full[vst], vpar, kStatusTmaTimeout);
              tc_fence_after_sync();
#pragma unroll
              for (int ks = 4 * h; ks < 4 * h + 4; ++ks)
                umma_ts(tmem + COL_O + t * HD, tp + ks * 8, vd + uint64_t((ks * 16 * 128) >> 4), idesc_pv, (b > 0 || ks > 0) ? 1u : 0u);
            }
            if (t == NQ - 1) {
              umma_commit(&v_empty[vst]);
              if (++vst == VS) vst = 0, vpar ^= 1;
            }
            // Q_t . K^T of the next block writes over P_t: issued after the P_t . V that reads it.
            if (b + 1 < nb) issue_qk(t);
          }
          if (b + 1 == nb) umma_commit(&o_full);
          stamp(b, 5);
        }
      }
    }
  }
  } else {
    // ================= softmax: thread i of warpgroup t owns row i of S_t and of O_t
    setmaxnreg_inc<kRegsSoftmax>();
    // set-up: the two Q tiles, mask bounds
    int4 d = make_int4(0, 0, 0, 0);
    uint64_t am = 0;
    int qpos = 0;  // sliding-window layers: the row's position
    {
      // this thread's Q row into its tile (K-major, 128-byte swizzle)
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const typename QE::T*>(a.Q) + size_t(row) * p.q_ld + size_t(head) * HD);
      uint8_t* qd = q_sm + qt * Q_BYTES + srow * 128;
#pragma unroll
      for (int i = 0; i < 16; ++i)
        *reinterpret_cast<uint4*>(qd + (i >> 3) * HALF_T + (((i & 7) ^ (srow & 7)) << 4)) = src[i];
      fence_proxy_async_smem();
      if (tile.last) {
        if (use_anc) am = a.anc_mask[row];
        else d = reinterpret_cast<const int4*>(a.desc)[row];
      }
      if (windowed) {
        qpos = a.pos[4 * size_t(row)];
        int latest = qpos;
#pragma unroll
        for (int o = 16; o; o >>= 1) latest = max(latest, __shfl_xor_sync(0xffffffffu, latest, o));
        if (lane == 0 && qt == 0) atomicMax(&red[4], latest);
      }
      if (desc_mask && qt == 0) {  // both query tiles hold the same rows
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
    }
    tc_fence_before_sync();
    named_barrier(1, kSoftmaxThreads + 32);  // softmax warps + the MMA warp
    tc_fence_after_sync();
    phase(1);
    const Meta meta = make_meta();
    const int nb = nbc + meta.nbb;
    const uint32_t tmem = sh.tmem_slot;
    {
      const uint32_t t_lane = tmem + (uint32_t((warp & 3) * 32) << 16);  // this warp's quarter of the lanes
      const uint32_t t_s = t_lane + COL_S + qt * BN;
      const uint32_t t_o = t_lane + COL_O + qt * HD;
      const float sl2 = a.scale * kLog2e;
      float m_ref = -INFINITY, l_run = 0.0f;  // m_ref in exp2 units of the scaled score
      int vst = 0;
      uint32_t vpar = 0;

      for (int b = 0; b < nb; ++b) {
        const bool cached = b < nbc;
        const int j0 = cached ? k0a + BN * b : batch_j0(meta, b - nbc);
        const int n_valid = cached ? min(BN, tile.k1 - j0) : min(BN, meta.k_last + 1 - j0);
        bool need_mask = n_valid < BN;
        if (!cached) {
          if (use_anc) need_mask = true;
          else need_mask = need_mask || !((j0 + BN - 1 < meta.anc_min) || (j0 >= meta.seg_max && j0 + BN - 1 <= r_first));
        }
        // Sliding-window layers: a cached key sits at position j, so a block needs the window's lower edge when the
        // latest row's first visible position lies beyond its first key; a batch key sits at its row's position, which
        // the K producer left in shared memory with the block's earliest one.
        bool win_keys = false;
        const int wslot = (b - nbc) % kPosSlots;
        if (windowed) {
          if (cached) {
            need_mask = need_mask || j0 < meta.lo_max;
          } else {
            wait_bar(&sh.kpos_full[wslot], uint32_t((b - nbc) / kPosSlots) & 1u, kStatusTmaTimeout);
            win_keys = sh.kpos_min[wslot] < meta.lo_max;
            need_mask = need_mask || win_keys;
          }
        }
        // visibility of this row's 128 columns, 32 per word (only read when need_mask)
        uint32_t vw[4] = {~0u, ~0u, ~0u, ~0u};
        if (need_mask) {
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int c0 = hf * 64;
            uint64_t vm = low_bits64(n_valid - c0);
            if (!cached) {
              if (use_anc) {
                vm &= hf == 0 ? am : 0ull;  // one block, j0 = 0
              } else {
                const int jb = j0 + c0;  // batch key of the half's first column
                const int own_end = bidi ? max(rr + 1, d.w) : rr + 1;  // an image row's segment reaches the image's end
                vm &= low_bits64(d.z - jb) | (low_bits64(own_end - jb) & ~low_bits64(d.x - jb));  // j < d.z || d.x <= j < own_end
              }
              if (win_keys) {
                uint64_t wm = 0;
                for (int c = 0; c < 64; ++c) wm |= uint64_t(qpos - sh.kpos[wslot][c0 + c] < a.window) << c;
                vm &= wm;
              }
            } else if (windowed) {
              vm &= ~low_bits64(qpos - a.window + 1 - (j0 + c0));  // j >= the row's first visible position
            }
            vw[2 * hf] = uint32_t(vm), vw[2 * hf + 1] = uint32_t(vm >> 32);
          }
        }
        auto chunk_max = [&](uint32_t (&s)[32], uint32_t w) {
          float m0 = -INFINITY, m1 = -INFINITY;
          if (need_mask) {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const float sc = ((w >> c) & 1u) ? __uint_as_float(s[c]) : -INFINITY;
              s[c] = __float_as_uint(sc);
              m0 = fmaxf(m0, sc);
            }
          } else {
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
              m0 = fmax3(m0, __uint_as_float(s[c]), __uint_as_float(s[c + 1]));
              m1 = fmax3(m1, __uint_as_float(s[c + 2]), __uint_as_float(s[c + 3]));
            }
          }
          return fmaxf(m0, m1);
        };

        wait_bar(&s_full[qt], b & 1, kStatusMmaTimeout);
        if (srow == 0) stamp(b, qt ? 6 : 0);
        tc_fence_after_sync();
        // the row's 128 scores, all in registers
        uint32_t s0[32], s1[32], s2[32], s3[32];
        tmem_ld32(t_s, s0);
        tmem_ld32(t_s + 32, s1);
        tmem_ld32(t_s + 64, s2);
        tmem_ld32(t_s + 96, s3);
        tmem_wait_ld_of(s0);
        tmem_wait_ld_of(s1);
        float mx = fmaxf(chunk_max(s0, vw[0]), chunk_max(s1, vw[1]));
        tmem_wait_ld_of(s2);
        tmem_wait_ld_of(s3);
        mx = fmaxf(mx, fmaxf(chunk_max(s2, vw[2]), chunk_max(s3, vw[3])));
        mx *= sl2;  // scale > 0: the maximum commutes with the scaling
        if (tid == 0) stamp(b, 1);
        // lazy rescale: keep the old reference maximum unless this block exceeds it by 2^8
        float factor = 1.0f;
        const bool grow = mx > m_ref + kRescaleThreshold;  // also the first finite maximum (m_ref = -inf)
        if (grow) {
          factor = fast_exp2(m_ref - mx);  // 0 when nothing was seen before
          m_ref = mx;
          l_run *= factor;
        }
        const float neg_m = m_ref == -INFINITY ? 0.0f : -m_ref;
        // S_t of this block was written after every earlier MMA had completed: O_t is idle and holds blocks 0 .. b-1.
        if (b > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(t_o + 32 * c, o);
            tmem_wait_ld_of(o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            tmem_st32(t_o + 32 * c, o);
          }
        }
        if (n_valid < BN) {
          // tail block: V rows past the range are stale or foreign bytes; 0 * NaN must not happen. Warpgroup 0 clears
          // them before it hands over P_0; P_1 . V is issued after P_0 . V.
          if (qt == 0) {
            wait_bar(&v_full[vst], vpar, kStatusTmaTimeout);
            const int n = (BN - n_valid) * 16;  // 16-byte chunks: 2 dim halves x 8 per row
            for (int i = srow; i < n; i += BM) {
              const int r = n_valid + i / 16, c = i % 16;
              *reinterpret_cast<uint4*>(v_sm + vst * KV_TILE + (c >> 3) * HALF_T + r * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
          }
        }
        // P is rounded to the pass's 16-bit type before P.V (the reference rounds it to fp16, 40_attention.metal:297; the
        // MMA takes A and B in one 16-bit format only). Scaling and the row sum work on two scores per instruction.
        const uint64_t sl2x2 = f32x2_pack(sl2, sl2), neg_mx2 = f32x2_pack(neg_m, neg_m);
        uint64_t psum0 = f32x2_pack(0.0f, 0.0f), psum1 = psum0;
        auto chunk_p = [&](const uint32_t (&s)[32], uint32_t (&pk)[16]) {
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const uint64_t x2 = f32x2_fma(f32x2_pack(__uint_as_float(s[2 * c]), __uint_as_float(s[2 * c + 1])), sl2x2, neg_mx2);
            float x0, x1;
            f32x2_unpack(x2, x0, x1);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            if (c & 1) psum1 = f32x2_add(psum1, f32x2_pack(p0, p1));
            else psum0 = f32x2_add(psum0, f32x2_pack(p0, p1));
            pk[c] = QE::pack2(p0, p1);
          }
        };
        // P goes back over the scores (all of them are in registers) and is handed to the MMA thread in two halves of
        // 64 keys: the first four P.V instructions run while the second half is still being computed.
        {
          uint32_t pa[16], pb[16];
          chunk_p(s0, pa);
          tmem_st16(t_s, pa);
          chunk_p(s1, pb);
          tmem_st16(t_s + 16, pb);
          chunk_p(s2, pa);
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(&p_full[qt][0]);
          tmem_st16(t_s + 32, pa);
          chunk_p(s3, pb);
          tmem_st16(t_s + 48, pb);
          tmem_wait_st();
        }
        {
          float a0, a1;
          f32x2_unpack(f32x2_add(psum0, psum1), a0, a1);
          l_run += a0 + a1;
        }
        if (++vst == VS) vst = 0, vpar ^= 1;
        tc_fence_before_sync();
        mbar_arrive(&p_full[qt][1]);
        if (srow == 0) stamp(b, qt ? 7 : 2);
      }

      // ---- epilogue: every thread finishes its row
      phase(2);
      pdl_launch_dependents();
      if (nb > 0) {
        wait_bar(&o_full, 0, kStatusMmaTimeout);
        tc_fence_after_sync();
      }
      const float inv_l = l_run > 0.0f ? 1.0f / l_run : 0.0f;
      const int hg = head % G;
      const bool to_rec = tile.part >= 0;
      float* rec = to_rec ? a.parts + (size_t(tile.part) * p.Hkv + kvh) * TR * G * (HD + 2) + (size_t(fm) * G + hg) * (HD + 2) : nullptr;
      const float* gp = a.X ? a.X + size_t(row) * p.g_ld + size_t(head) * 2 * HD + HD : nullptr;
      typename QE::T* op = static_cast<typename QE::T*>(a.O) + size_t(row) * p.q_ld + size_t(head) * HD;
      // (Staging the rows in the idle K ring and writing them out two whole rows per instruction measured slower than
      // these per-thread 16-byte stores: 6.8 us against 4.8 us of epilogue.)
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        const int d0 = 32 * c;
        float v[32];
        if (nb > 0) {
          uint32_t o[32];
          tmem_ld32(t_o + d0, o);
          tmem_wait_ld_of(o);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(o[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.0f;
        }
        if (!row_ok) continue;
        if (to_rec) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) *reinterpret_cast<float2*>(rec + d0 + i) = make_float2(v[i], v[i + 1]);
        } else {
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
      if (row_ok) {
        if (to_rec) {
          rec[HD] = m_ref * kLn2;  // -inf stays -inf
          rec[HD + 1] = l_run;
        } else if (a.lse) {
          a.lse[size_t(row) * p.H + head] = l_run > 0.0f ? m_ref * kLn2 + __logf(l_run) : -INFINITY;
        }
      }
    }
  }
  phase(3);
  tc_fence_before_sync();
  __syncthreads();
  if (tracing && tid == 0) a.trace[8 * a.trace_blocks + 1] = global_timer_ns();
  if (warp == kMmaWarp) tmem_dealloc(sh.tmem_slot, TMEM_COLS);
}

}  // namespace

// Two query tiles of 128 / tile_rows heads each must belong to one kv head.
bool flash_umma_duo_supports(int32_t HDim, int32_t G, int32_t tile_rows, int32_t bt, int32_t q_dtype, int32_t kv_dtype) {
  if (HDim != HD || q_dtype != kv_dtype) return false;
  if (tile_rows != 16 && tile_rows != 32 && tile_rows != 64 && tile_rows != 128) return false;
  const int hpc2 = NQ * BM / tile_rows;
  if (hpc2 > G || G % hpc2 != 0) return false;
  return bt > 0 && bt % 16 == 0;
}

cudaError_t flash_umma_duo_setup() {
  cudaError_t e = cudaFuncSetAttribute(flash_umma_duo_kernel<ESP_F16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_umma_duo_kernel<ESP_BF16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_umma_duo_kernel<ESP_F16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_WIN);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(flash_umma_duo_kernel<ESP_BF16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_WIN);
  return e;
}

cudaError_t launch_flash_umma_duo(const KernelArgs& a, const CUtensorMap& pool_map, const CUtensorMap& kb_map,
                                  const CUtensorMap& vb_map, cudaStream_t stream, uint64_t* launches) {
  if (a.n_tiles <= 0) return cudaSuccess;
  const int hpc2 = NQ * BM / a.tile_rows;
  const bool win = a.window > 0 || a.ring > 0 || a.bidi != 0;  // sliding-window layers: their own instantiation, the rest pays nothing
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(a.n_tiles), unsigned(a.p.H / hpc2)), cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = win ? SMEM_BYTES_WIN : SMEM_BYTES, cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  cudaError_t e;
  if (win)
    e = a.q_dtype == ESP_F16 ? cudaLaunchKernelEx(&cfg, flash_umma_duo_kernel<ESP_F16, true>, pool_map, kb_map, vb_map, a)
                             : cudaLaunchKernelEx(&cfg, flash_umma_duo_kernel<ESP_BF16, true>, pool_map, kb_map, vb_map, a);
  else
    e = a.q_dtype == ESP_F16 ? cudaLaunchKernelEx(&cfg, flash_umma_duo_kernel<ESP_F16, false>, pool_map, kb_map, vb_map, a)
                             : cudaLaunchKernelEx(&cfg, flash_umma_duo_kernel<ESP_BF16, false>, pool_map, kb_map, vb_map, a);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e == cudaSuccess) ++*launches;
  return e;
}

}  // namespace esp
