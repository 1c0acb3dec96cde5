// Paged-KV GQA decode attention for single-row trees (sm_100a).
//
// Replaces attn_decode_gqa of the reference (kernels/40_attention.metal:598-781; the
// generic-head-dim twin g4_attention_dec, kernels/80_gemma.metal:371-550): one CTA per
// (kv head, tile), tile = cached key range [k0, k1) of a tree with one row, plus the row's
// own batch key when tile.last; output = flash_attention's partial record when
// tile.part >= 0, else the gated, normalised row (and its LSE).
//
// B200 structure (bandwidth-bound: every K/V byte is read once from HBM):
//  - the pool region is one 3-D TMA tensor [128-byte line][row][lines per row]; a 16-key
//    block of one kv head (K tile + V tile, 16 rows x HD) is fetched by two bulk tensor
//    loads with the hardware 128-byte swizzle, rows found through the page table;
//  - every warp runs its own ring of STAGES tiles with one mbarrier per slot and takes
//    the tile's 16-key blocks round-robin, so there is no CTA-wide barrier in the loop;
//  - scores are computed transposed, S^T[16 keys x 8 heads] = K . Q^T with mma.sync
//    m16n8k16 (the G <= 8 query heads of the kv head are the N = 8 columns, so no MMA row
//    is padding), online softmax in the exp2 domain with warp shuffles over the key lanes,
//    P^T goes back in as the B operand through movmatrix, O^T[HD x 8 heads] += V^T . P^T
//    with V fragments from ldmatrix.trans;
//  - E4M3 pools: codes are widened to fp16 in registers (exact), the K scale of the page
//    multiplies the score, the V scale multiplies p before it is rounded to fp16;
//  - the warps' (m, l, O) are merged through shared memory, then the row's own key is
//    folded in on CUDA cores, then the record / output is written.
// All waits are bounded: a TMA that never lands sets the context's status word and the
// warp leaves its loop.
#include "common.cuh"
#include "../launch.h"

namespace esp {
namespace {

template <int HD_, int KVDT_, int QDT_, int NW_, int STAGES_>
struct DecodeCfg {
  static constexpr int HD = HD_, KVDT = KVDT_, QDT = QDT_, NW = NW_, STAGES = STAGES_;
  static constexpr bool FP8 = KVDT == ESP_E4M3;
  static constexpr int CDT = FP8 ? ESP_F16 : KVDT;  // MMA operand type
  static constexpr int ESZ = FP8 ? 1 : 2;
  static constexpr int ROW_BYTES = HD * ESZ;         // one key of one kv head
  static constexpr int NCH = ROW_BYTES / 128;        // 128-byte lines per row
  static constexpr int TILE_BYTES = 16 * ROW_BYTES;  // K or V tile of a 16-key block
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int WARP_BYTES = STAGES * STAGE_BYTES;
  static constexpr int OLD = HD + 4;                 // row stride of the merge scratch
  static constexpr int SCRATCH_BYTES = (8 * OLD + 16) * 4;
  static constexpr int SMEM_BYTES = NW * WARP_BYTES + 1024;
  static constexpr int NMT = HD / 16;                // m-tiles of O^T
  static_assert(SCRATCH_BYTES <= WARP_BYTES, "merge scratch must fit in a warp's ring");
  static_assert(ROW_BYTES % 128 == 0, "row must be whole 128-byte lines");
};

// Byte offset of (key row r, byte b of the head's row) in a K or V tile:
// [line][16 rows][128 B], each 16 x 128 B group swizzled by TMA.
__device__ __forceinline__ uint32_t tile_off(uint32_t r, uint32_t b) { return (b >> 7) * 2048u + swz128(r, b & 127u); }

template <class C>
__global__ void __launch_bounds__(C::NW * 32, (C::SMEM_BYTES <= 56 * 1024) ? 4 : (C::SMEM_BYTES <= 110 * 1024) ? 2 : 1)
    decode_gqa_kernel(const __grid_constant__ CUtensorMap pool_map, const KernelArgs a) {
  constexpr int HD = C::HD, NW = C::NW, STAGES = C::STAGES, NMT = C::NMT, OLD = C::OLD;
  using QE = Elem16<C::QDT>;
  using CE = Elem16<C::CDT>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[NW][STAGES];
  __shared__ int fix_info[4];  // fused merge: first record and record count of the tile's job, the ticket drawn
  __shared__ int gave_up;      // a warp's bounded wait ran out: the CTA writes an empty result and leaves its rings alone
  __shared__ uint64_t fix_bar;  // fused merge: completion of the records' bulk copies

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const esp_attn_params& p = a.p;
  const int kvh = blockIdx.x % p.Hkv;
  // Launched with programmatic serialization: while the previous kernel of the stream drains,
  // warm L2 with what this CTA reads first - its plan records, page-table entries and each warp's
  // first key blocks. Hints and L1-bypassing reads only, every index checked: stale or
  // half-written metadata can cost a wasted hint, never a result.
  if (lane < STAGES - 1 && a.n_trees > 0 && a.n_block_entries > 0 && a.blocks != nullptr) {
    const int4* tp = reinterpret_cast<const int4*>(a.tiles + blockIdx.x / p.Hkv);
    const int4 t0 = __ldcg(tp);  // tree, r0, k0, k1
    if (t0.x >= 0 && t0.x < a.n_trees && p.bt > 0) {
      const int4 tr = __ldcg(reinterpret_cast<const int4*>(a.trees + t0.x));  // base, P, table, M
      const int j0 = (t0.z & ~15) + 16 * (warp + lane * NW);
      const long long idx = (long long)tr.z + j0 / p.bt;
      if (a.ring == 0 && t0.z >= 0 && j0 < t0.w && tr.z >= 0 && idx < a.n_block_entries) {
        const int b = __ldcg(a.blocks + idx);
        if (b >= 0 && b < a.n_blocks) {
          const int y = b * 2 * p.bt + j0 % p.bt;
          tma_prefetch_3d(&pool_map, 0, y, kvh * C::NCH);
          tma_prefetch_3d(&pool_map, 0, y + p.bt, kvh * C::NCH);
        }
      }
    }
  }
  pdl_wait();
  const esp_attn_tile tile = a.tiles[blockIdx.x / p.Hkv];
  const esp_attn_tree tree = a.trees[tile.tree];
  const int G = a.G;
  const int row = tile.r0;
  const float sl2 = a.scale * kLog2e;

  uint8_t* wsm = smem + size_t(warp) * C::WARP_BYTES;
  const bool fused = a.fuse && tile.part >= 0;
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&pool_map);
    gave_up = 0;
    mbar_init(&fix_bar, 1);  // made visible by the fence and barrier below
    if (fused) {  // needed only at the very end: the load's latency hides behind the whole stream
      const esp_attn_combine jb = a.jobs[tile.pad1 - 1];
      fix_info[0] = jb.part0, fix_info[1] = jb.nparts;
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(&full_bar[warp][s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  // ---- Q fragments (B operand: k = dim, n = head g), kept in registers for the whole tile
  uint32_t qf[HD / 16][2];
  {
    const int hq = min(g, G - 1);
    const typename QE::T* qrow = static_cast<const typename QE::T*>(a.Q) + size_t(row) * p.q_ld + size_t(kvh * G + hq) * HD;
    if constexpr (!C::FP8) {
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        qf[ks][0] = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t);
        qf[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 8 + 2 * t);
      }
    } else {
      // K fragments of an E4M3 tile hold dims 4t..4t+3 of each 16-dim group: MMA column pairs
      // (2t, 2t+1) and (2t+8, 2t+9) stand for dims (4t, 4t+1) and (4t+2, 4t+3).
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const uint2 w = *reinterpret_cast<const uint2*>(qrow + 16 * ks + 4 * t);
        const float2 f0 = QE::unpack2(w.x), f1 = QE::unpack2(w.y);
        qf[ks][0] = CE::pack2(f0.x, f0.y);
        qf[ks][1] = CE::pack2(f1.x, f1.y);
      }
    }
  }

  // ---- this warp's 16-key blocks: warp, warp + NW, ... of the tile's cached range
  // A tile may start at any key (a sliding-window plan begins at the row's first visible key): the
  // 16-key blocks are cut from the 16-aligned key below it, and the first block masks what lies
  // before k0 the way the last one masks what lies past k1.
  const int kbase = tile.k0 & ~15;
  const int nblk = tile.k1 > tile.k0 ? (tile.k1 - kbase + 15) >> 4 : 0;
  const int n_it = nblk > warp ? (nblk - warp + NW - 1) / NW : 0;

  // Lane L of a window keeps the metadata of iteration win + L (page-table lookups are
  // done 32 at a time, off the critical path of a single block).
  int iss_win = -32, iss_y = 0;
  int use_win = -32;
  float use_ks = 1.0f, use_vs = 1.0f;
  auto block_of_it = [&](int it, int& j0) {
    j0 = kbase + 16 * (warp + it * NW);
    // ring layers (kernels/80_gemma.metal:429) keep a sequence's blocks in place: no page table
    return a.ring > 0 ? tree.table + (j0 / p.bt) % a.ring : a.blocks[tree.table + j0 / p.bt];
  };
  auto issue = [&](int it) {
    if (it - iss_win >= 32) {
      iss_win = it;
      const int mine = it + lane;
      if (mine < n_it) {
        int j0;
        const int b = block_of_it(mine, j0);
        iss_y = b * 2 * p.bt + j0 % p.bt;
      }
    }
    const int y = __shfl_sync(0xffffffffu, iss_y, it - iss_win);
    if (lane == 0) {
      const int slot = it % STAGES;
      uint8_t* dst = wsm + slot * C::STAGE_BYTES;
      mbar_arrive_expect_tx(&full_bar[warp][slot], C::STAGE_BYTES);
      tma_load_3d(dst, &pool_map, &full_bar[warp][slot], 0, y, kvh * C::NCH);
      tma_load_3d(dst + C::TILE_BYTES, &pool_map, &full_bar[warp][slot], 0, y + p.bt, kvh * C::NCH);
    }
  };

  float o[NMT][4];
#pragma unroll
  for (int i = 0; i < NMT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;  // heads 2t, 2t+1 (l: this lane's keys only)

  const int mi = lane >> 3, rj = lane & 7;
  const uint32_t key_k = rj + 8 * (mi & 1), sel_k = mi >> 1;  // K: ldmatrix
  const uint32_t key_v = rj + 8 * (mi >> 1), sel_v = mi & 1;  // V: ldmatrix.trans

  for (int s = 0; s < STAGES - 1 && s < n_it; ++s) issue(s);

  for (int it = 0; it < n_it; ++it) {
    if (it + STAGES - 1 < n_it) issue(it + STAGES - 1);
    const int slot = it % STAGES;
    float kscale = 1.0f, vscale = 1.0f;
    if constexpr (C::FP8) {
      if (it - use_win >= 32) {
        use_win = it;
        const int mine = it + lane;
        if (mine < n_it) {
          int j0;
          const int b = block_of_it(mine, j0);
          use_ks = a.kv_scales[size_t(b * 2) * p.Hkv + kvh];
          use_vs = a.kv_scales[size_t(b * 2 + 1) * p.Hkv + kvh];
        }
      }
      kscale = __shfl_sync(0xffffffffu, use_ks, it - use_win);
      vscale = __shfl_sync(0xffffffffu, use_vs, it - use_win);
    }
    // One verdict for the whole warp (each lane reads its own timer: without the vote lanes could
    // disagree at the limit and the warp-wide shuffles / MMAs below would run with lanes missing).
    if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[warp][slot], (it / STAGES) & 1))) {
      if (lane == 0) {
        atomicExch(a.status, kStatusTmaTimeout);
        gave_up = 1;
      }
      break;
    }
    const uint8_t* kt = wsm + slot * C::STAGE_BYTES;
    uint8_t* vt = wsm + slot * C::STAGE_BYTES + C::TILE_BYTES;
    const int jb = kbase + 16 * (warp + it * NW);  // first key of this block
    const int n_valid = min(16, tile.k1 - jb);
    const int n_skip = tile.k0 - jb;               // > 0 only in the tile's first block
    if (n_valid < 16) {
      // Tail block: rows past the range hold other keys (or stale bytes); V must be zero
      // there (0 * NaN), K is masked by selection below.
      const int n = (16 - n_valid) * C::NCH * 8;
      for (int i = lane; i < n; i += 32) {
        const int r = n_valid + i / (C::NCH * 8), rem = i % (C::NCH * 8);
        *reinterpret_cast<uint4*>(vt + (rem >> 3) * 2048 + r * 128 + (rem & 7) * 16) = make_uint4(0, 0, 0, 0);
      }
      fence_proxy_async_smem();
      __syncwarp();
    }
    const uint32_t kt_u = smem_u32(kt), vt_u = smem_u32(vt);

    // ---- S^T = K . Q^T (two accumulators to shorten the dependent chain)
    float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
    if constexpr (!C::FP8) {
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t af[4];
        ldmatrix_x4(af, kt_u + (ks >> 2) * 2048 + key_k * 128 + (((((ks & 3) << 1) + sel_k) ^ (key_k & 7)) << 4));
        if (ks & 1) mma_16816<C::CDT>(sb, af, qf[ks][0], qf[ks][1]);
        else mma_16816<C::CDT>(sa, af, qf[ks][0], qf[ks][1]);
      }
    } else {
#pragma unroll
      for (int kk = 0; kk < HD / 32; ++kk) {
        uint32_t r[4];
        ldmatrix_x4(r, kt_u + (kk >> 2) * 2048 + key_k * 128 + (((((kk & 3) << 1) + sel_k) ^ (key_k & 7)) << 4));
        uint32_t a0[4] = {e4m3x2_to_f16x2(uint16_t(r[0] & 0xFFFFu)), e4m3x2_to_f16x2(uint16_t(r[1] & 0xFFFFu)),
                          e4m3x2_to_f16x2(uint16_t(r[0] >> 16)), e4m3x2_to_f16x2(uint16_t(r[1] >> 16))};
        uint32_t a1[4] = {e4m3x2_to_f16x2(uint16_t(r[2] & 0xFFFFu)), e4m3x2_to_f16x2(uint16_t(r[3] & 0xFFFFu)),
                          e4m3x2_to_f16x2(uint16_t(r[2] >> 16)), e4m3x2_to_f16x2(uint16_t(r[3] >> 16))};
        mma_16816<C::CDT>(sa, a0, qf[2 * kk][0], qf[2 * kk][1]);
        mma_16816<C::CDT>(sb, a1, qf[2 * kk + 1][0], qf[2 * kk + 1][1]);
      }
    }
    // lane: s[0] = (key g, head 2t), s[1] = (key g, head 2t+1), s[2], s[3] = key g + 8
    const float sc = sl2 * kscale;
    float s0 = (sa[0] + sb[0]) * sc, s1 = (sa[1] + sb[1]) * sc, s2 = (sa[2] + sb[2]) * sc, s3 = (sa[3] + sb[3]) * sc;
    if (g >= n_valid || g < n_skip) s0 = s1 = -INFINITY;
    if (g + 8 >= n_valid || g + 8 < n_skip) s2 = s3 = -INFINITY;

    // ---- online softmax per head over the 16 keys (key lanes: xor 4, 8, 16)
    float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
#pragma unroll
    for (int off = 4; off <= 16; off <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);  // finite: key 0 of the block is live
    const float c0 = fast_exp2(m0 - mn0), c1 = fast_exp2(m1 - mn1);
    const float p0 = fast_exp2(s0 - mn0), p1 = fast_exp2(s1 - mn1), p2 = fast_exp2(s2 - mn0), p3 = fast_exp2(s3 - mn1);
    l0 = l0 * c0 + (p0 + p2);
    l1 = l1 * c1 + (p1 + p3);
    m0 = mn0;
    m1 = mn1;
    // P^T as the B operand (k = key, n = head): transpose the two 8 x 8 halves
    const uint32_t pb0 = movmatrix_trans(CE::pack2(p0 * vscale, p1 * vscale));
    const uint32_t pb1 = movmatrix_trans(CE::pack2(p2 * vscale, p3 * vscale));

    // ---- O^T = O^T * corr + V^T . P^T
    if constexpr (!C::FP8) {
#pragma unroll
      for (int i = 0; i < NMT; ++i) {
        uint32_t af[4];
        ldmatrix_x4_trans(af, vt_u + (i >> 2) * 2048 + key_v * 128 + (((((i & 3) << 1) + sel_v) ^ (key_v & 7)) << 4));
        o[i][0] *= c0, o[i][1] *= c1, o[i][2] *= c0, o[i][3] *= c1;
        mma_16816<C::CDT>(o[i], af, pb0, pb1);
      }
    } else {
      // Per 32 dims: this lane reads dims 32u + 4g .. + 3 of keys 2t, 2t+1, 2t+8, 2t+9 and
      // pairs them by key: m-tile 2u has rows g <-> dim 32u+4g, g+8 <-> 32u+4g+1, m-tile
      // 2u+1 has rows g <-> 32u+4g+2, g+8 <-> 32u+4g+3.
#pragma unroll
      for (int u = 0; u < HD / 32; ++u) {
        const uint32_t bcol = uint32_t(32 * u + 4 * g);
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t key = uint32_t(2 * t + (q & 1) + 8 * (q >> 1));
          w[q] = *reinterpret_cast<const uint32_t*>(vt + tile_off(key, bcol));
        }
        const uint32_t alo = e4m3x2_to_f16x2(uint16_t(w[0] & 0xFFFFu)), ahi = e4m3x2_to_f16x2(uint16_t(w[0] >> 16));
        const uint32_t blo = e4m3x2_to_f16x2(uint16_t(w[1] & 0xFFFFu)), bhi = e4m3x2_to_f16x2(uint16_t(w[1] >> 16));
        const uint32_t clo = e4m3x2_to_f16x2(uint16_t(w[2] & 0xFFFFu)), chi = e4m3x2_to_f16x2(uint16_t(w[2] >> 16));
        const uint32_t dlo = e4m3x2_to_f16x2(uint16_t(w[3] & 0xFFFFu)), dhi = e4m3x2_to_f16x2(uint16_t(w[3] >> 16));
        const uint32_t fa[4] = {__byte_perm(alo, blo, 0x5410), __byte_perm(alo, blo, 0x7632), __byte_perm(clo, dlo, 0x5410),
                                __byte_perm(clo, dlo, 0x7632)};
        const uint32_t fb[4] = {__byte_perm(ahi, bhi, 0x5410), __byte_perm(ahi, bhi, 0x7632), __byte_perm(chi, dhi, 0x5410),
                                __byte_perm(chi, dhi, 0x7632)};
        o[2 * u][0] *= c0, o[2 * u][1] *= c1, o[2 * u][2] *= c0, o[2 * u][3] *= c1;
        mma_16816<C::CDT>(o[2 * u], fa, pb0, pb1);
        o[2 * u + 1][0] *= c0, o[2 * u + 1][1] *= c1, o[2 * u + 1][2] *= c0, o[2 * u + 1][3] *= c1;
        mma_16816<C::CDT>(o[2 * u + 1], fb, pb0, pb1);
      }
    }
    __syncwarp();  // every lane is done with the slot before lane 0 refills it
  }

  // The streaming part is over: let a dependent grid (the combine kernel) be scheduled while
  // this one merges and drains; it still waits for this grid's completion before it reads.
  pdl_launch_dependents();

  // ---- merge the warps through shared memory (their rings are idle now)
#pragma unroll
  for (int off = 4; off <= 16; off <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, off);
    l1 += __shfl_xor_sync(0xffffffffu, l1, off);
  }
  __syncthreads();
  if (gave_up) {
    // A load never landed (the status word says so): loads may still be in flight into the rings, so
    // they are not reused as scratch. The CTA writes an empty record (m = -inf, l = 0: it weighs
    // nothing in a merge) or a zero row, and takes no part in a fused merge.
    for (int hg = warp; hg < G; hg += NW) {
      const int h = kvh * G + hg;
      if (tile.part >= 0) {
        float* rec = a.parts + ((size_t(tile.part) * p.Hkv + kvh) * a.tile_rows * G + hg) * (HD + 2);
        for (int i = lane; i < HD; i += 32) rec[i] = 0.0f;
        if (lane == 0) rec[HD] = -INFINITY, rec[HD + 1] = 0.0f;
      } else {
        typename QE::T* op = static_cast<typename QE::T*>(a.O) + size_t(row) * p.q_ld + size_t(h) * HD;
        for (int i = lane; i < HD; i += 32) op[i] = QE::from_f32(0.0f);
        if (a.lse && lane == 0) a.lse[size_t(row) * p.H + h] = -INFINITY;
      }
    }
    return;
  }
  {
    float* osm = reinterpret_cast<float*>(wsm);
    float* msm = osm + 8 * OLD;
#pragma unroll
    for (int i = 0; i < NMT; ++i) {
      int d_lo, d_hi;
      if constexpr (!C::FP8) {
        d_lo = 16 * i + g, d_hi = 16 * i + 8 + g;
      } else {
        d_lo = 32 * (i >> 1) + 4 * g + 2 * (i & 1), d_hi = d_lo + 1;
      }
      osm[(2 * t) * OLD + d_lo] = o[i][0];
      osm[(2 * t + 1) * OLD + d_lo] = o[i][1];
      osm[(2 * t) * OLD + d_hi] = o[i][2];
      osm[(2 * t + 1) * OLD + d_hi] = o[i][3];
    }
    if (g == 0) {
      msm[2 * t] = m0, msm[2 * t + 1] = m1;
      msm[8 + 2 * t] = l0, msm[8 + 2 * t + 1] = l1;
    }
  }
  __syncthreads();

  constexpr int DPL = HD / 32;
  for (int hg = warp; hg < G; hg += NW) {
    const int h = kvh * G + hg;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, reinterpret_cast<const float*>(smem + size_t(w) * C::WARP_BYTES)[8 * OLD + hg]);
    float l = 0.0f, acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float* ow = reinterpret_cast<const float*>(smem + size_t(w) * C::WARP_BYTES);
      const float mw = ow[8 * OLD + hg];
      const float wg = (mw == -INFINITY) ? 0.0f : fast_exp2(mw - M);
      l = fmaf(wg, ow[8 * OLD + 8 + hg], l);
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[i] = fmaf(wg, ow[hg * OLD + lane + 32 * i], acc[i]);
    }
    if (tile.last) {
      // the row's own key and value (batch row tree.base), kernels/40_attention.metal:647-657
      const typename QE::T* qrow = static_cast<const typename QE::T*>(a.Q) + size_t(row) * p.q_ld + size_t(h) * HD;
      const typename QE::T* krow = static_cast<const typename QE::T*>(a.Kb) + size_t(tree.base) * p.kv_ld + size_t(kvh) * HD;
      const typename QE::T* vrow = static_cast<const typename QE::T*>(a.Vb) + size_t(tree.base) * p.kv_ld + size_t(kvh) * HD;
      float dot = 0.0f;
#pragma unroll
      for (int i = 0; i < DPL; ++i) dot = fmaf(QE::to_f32(qrow[lane + 32 * i]), QE::to_f32(krow[lane + 32 * i]), dot);
#pragma unroll
      for (int off = 16; off; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
      const float s = dot * sl2;
      const float M2 = fmaxf(M, s);
      const float c = (M == -INFINITY) ? 0.0f : fast_exp2(M - M2);
      const float pw = fast_exp2(s - M2);
      l = l * c + pw;
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[i] = fmaf(pw, QE::to_f32(vrow[lane + 32 * i]), acc[i] * c);
      M = M2;
    }
    if (tile.part >= 0) {
      float* rec = a.parts + ((size_t(tile.part) * p.Hkv + kvh) * a.tile_rows * G + hg) * (HD + 2);
#pragma unroll
      for (int i = 0; i < DPL; ++i) rec[lane + 32 * i] = acc[i];
      if (lane == 0) {
        rec[HD] = M * kLn2;
        rec[HD + 1] = l;
      }
    } else {
      const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;
      typename QE::T* op = static_cast<typename QE::T*>(a.O) + size_t(row) * p.q_ld + size_t(h) * HD;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        float v = acc[i] * inv_l;
        if (a.X) v *= sigmoid_gate(a.X[size_t(row) * p.g_ld + size_t(h) * 2 * HD + HD + lane + 32 * i]);
        op[lane + 32 * i] = QE::from_f32(v);
      }
      if (a.lse && lane == 0) a.lse[size_t(row) * p.H + h] = l > 0.0f ? M * kLn2 + __logf(l) : -INFINITY;
    }
  }

  // ---- fused merge (what attention_combine does, kernels/40_attention.metal:811-864), in two levels.
  // The records of a job are cut into at most 8 groups of consecutive records. Every CTA publishes
  // its record and draws a ticket of its group; the CTA that draws a group's last ticket folds the
  // group's records of its kv head in record order into one unnormalised record, stores it over the
  // group's first slot and draws a ticket of the job; whoever draws the job's last ticket folds the
  // group records in group order and finishes the row. Groups that end early are folded while other
  // CTAs still stream, so the tail holds two short folds instead of one long one. Nobody waits for
  // anybody on this GPU, and the result does not depend on which CTAs came last.
  // With a peer exchange (a.x_world > 0: one sequence's keys split over several GPUs) the finished
  // record is not the row yet: it goes into slot `rank` of every rank's exchange buffer as 8-byte
  // words {value, tag} through peer mappings (plain stores over NVLink), and the same CTA then reads
  // the world's records of its heads from its own buffer - polling each word, bounded by a timer,
  // until it carries the call's tag -, folds them in rank order and writes the row. It waits only for
  // the same kv head's CTA on the OTHER GPUs; the host launches this mode only when the whole grid is
  // resident at once, so a waiting CTA never keeps another one off an SM.
  if (fused) {
    const int part0 = fix_info[0], n = fix_info[1];
    const int S = n > 8 ? (n + 7) / 8 : n;  // records per group
    const int n_groups = (n + S - 1) / S;
    const int grp = (tile.part - part0) / S, gsize = min(S, n - grp * S);
    int* tickets = a.counters + (size_t(tile.pad1 - 1) * p.Hkv + kvh) * kFixupPerJob;
    auto last_of = [&](int* ticket, int count) {  // CTA-uniform: did this CTA draw the last of `count` tickets?
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) {
        const int prev = atomicAdd(ticket, 1);
        if (prev == count - 1) *ticket = 0;  // ready for the next pass on this stream
        fix_info[2] = prev;
      }
      __syncthreads();
      const bool last = fix_info[2] == count - 1;
      if (last) __threadfence();
      return last;
    };
    if (!last_of(tickets + 1 + grp, gsize)) return;

    // Records come into shared memory by bulk copies (the rings are idle): the G records of a part are
    // contiguous, as many parts per round as fit. Then every thread folds its 4-dim items over the
    // parts in order with a running maximum.
    const size_t part_stride = size_t(p.Hkv) * a.tile_rows * G * (HD + 2);
    const uint32_t rec_bytes = uint32_t(G) * (HD + 2) * 4;
    float* const kvh_base = a.parts + size_t(kvh) * a.tile_rows * G * (HD + 2);  // record 0 of this kv head
    float* stage = reinterpret_cast<float*>(smem);
    constexpr int MAXI = (8 * HD / 4 + NW * 32 - 1) / (NW * 32);  // items per thread at most: G * HD / 4 items (G <= 8) over the CTA's threads
    const int n_items = G * HD / 4;
    float st_m[MAXI], st_l[MAXI];
    float4 st_acc[MAXI];
    uint32_t par = 0;
    bool alive = true;
    // folds records first, first + step, ... (count of them) into the state
    auto fold = [&](int first, int count, int step) {
#pragma unroll
      for (int k = 0; k < MAXI; ++k) st_m[k] = -INFINITY, st_l[k] = 0.0f, st_acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      const int per_round = max(1, min(count, int((NW * C::WARP_BYTES) / rec_bytes)));
      for (int s0 = 0; s0 < count; s0 += per_round) {
        const int cnt = min(per_round, count - s0);
        __syncthreads();  // the previous round's records have been consumed
        if (threadIdx.x == 0) {
          asm volatile("fence.proxy.async;" ::: "memory");  // the records were written through the generic proxy
          mbar_arrive_expect_tx(&fix_bar, uint32_t(cnt) * rec_bytes);
          for (int s2 = 0; s2 < cnt; ++s2)
            bulk_load(reinterpret_cast<uint8_t*>(stage) + size_t(s2) * rec_bytes, kvh_base + size_t(first + (s0 + s2) * step) * part_stride, rec_bytes, &fix_bar);
        }
        if (!__syncthreads_and(mbar_wait(&fix_bar, par))) {  // one verdict for the CTA: nobody is left behind at a barrier
          if (threadIdx.x == 0) atomicExch(a.status, kStatusTmaTimeout);
          alive = false;
          return;
        }
        par ^= 1;
#pragma unroll
        for (int k = 0; k < MAXI; ++k) {
          const int item = threadIdx.x + k * (NW * 32);
          if (item >= n_items) break;
          const int hg = item / (HD / 4), c4 = item % (HD / 4);
          const float* rec = stage + size_t(hg) * (HD + 2);
          for (int s2 = 0; s2 < cnt; ++s2, rec += size_t(G) * (HD + 2)) {
            const float m_s = rec[HD];
            if (m_s == -INFINITY) continue;          // an empty record adds nothing
            if (m_s > st_m[k]) {                      // rescale what has been summed so far (factor 0 the first time)
              const float f = __expf(st_m[k] - m_s);
              st_l[k] *= f, st_acc[k].x *= f, st_acc[k].y *= f, st_acc[k].z *= f, st_acc[k].w *= f;
              st_m[k] = m_s;
            }
            const float w = __expf(m_s - st_m[k]);
            const float2 o01 = *reinterpret_cast<const float2*>(rec + 4 * c4), o23 = *reinterpret_cast<const float2*>(rec + 4 * c4 + 2);
            st_l[k] = fmaf(w, rec[HD + 1], st_l[k]);
            st_acc[k].x = fmaf(w, o01.x, st_acc[k].x), st_acc[k].y = fmaf(w, o01.y, st_acc[k].y);
            st_acc[k].z = fmaf(w, o23.x, st_acc[k].z), st_acc[k].w = fmaf(w, o23.y, st_acc[k].w);
          }
        }
      }
    };
    fold(part0 + grp * S, gsize, 1);
    if (!alive) return;
    if (n_groups > 1) {
      // the group's record, unnormalised, over the group's first slot (its own records are spent)
      float* gout = kvh_base + size_t(part0 + grp * S) * part_stride;
      __syncthreads();  // every thread is done reading the staged records of the previous iteration
#pragma unroll
      for (int k = 0; k < MAXI; ++k) {
        const int item = threadIdx.x + k * (NW * 32);
        if (item >= n_items) break;
        const int hg = item / (HD / 4), c4 = item % (HD / 4);
        float* rec = gout + size_t(hg) * (HD + 2);
        *reinterpret_cast<float2*>(rec + 4 * c4) = make_float2(st_acc[k].x, st_acc[k].y);
        *reinterpret_cast<float2*>(rec + 4 * c4 + 2) = make_float2(st_acc[k].z, st_acc[k].w);
        if (c4 == 0) *reinterpret_cast<float2*>(rec + HD) = make_float2(st_m[k], st_l[k]);
      }
      if (!last_of(tickets, n_groups)) return;
      fold(part0, n_groups, S);
      if (!alive) return;
    }

    if (a.x_world > 0) {
      // ---- peer exchange: publish, then fold the world's records in rank order
      const size_t rank_words = part_stride;  // one job: a rank's records in a buffer = one record slot of every (kv head, row, head)
      const size_t kvh_off = size_t(kvh) * a.tile_rows * G * (HD + 2);
      if (a.x_phases & 1) {
#pragma unroll
        for (int k = 0; k < MAXI; ++k) {
          const int item = threadIdx.x + k * (NW * 32);
          if (item >= n_items) break;
          const int hg = item / (HD / 4), c4 = item % (HD / 4);
          const size_t off = a.x_epoch_off + size_t(a.x_rank) * rank_words + kvh_off + size_t(hg) * (HD + 2);
          for (int q = 0; q < a.x_world; ++q) {
            uint2* dst = a.x_records[q] + off;
            st_word(dst + 4 * c4, st_acc[k].x, a.x_tag), st_word(dst + 4 * c4 + 1, st_acc[k].y, a.x_tag);
            st_word(dst + 4 * c4 + 2, st_acc[k].z, a.x_tag), st_word(dst + 4 * c4 + 3, st_acc[k].w, a.x_tag);
            if (c4 == 0) st_word(dst + HD, st_m[k], a.x_tag), st_word(dst + HD + 1, st_l[k], a.x_tag);
          }
        }
      }
      if (!(a.x_phases & 2)) return;
      bool ok = true;
      const uint64_t t0 = global_timer_ns();
      const uint64_t limit = uint64_t(a.x_wait_ms) * 1000000ull;
#pragma unroll
      for (int k = 0; k < MAXI; ++k) {
        const int item = threadIdx.x + k * (NW * 32);
        if (item >= n_items) break;
        const int hg = item / (HD / 4), c4 = item % (HD / 4);
        const uint2* rec0 = a.x_records[a.x_rank] + a.x_epoch_off + kvh_off + size_t(hg) * (HD + 2);
        st_m[k] = -INFINITY, st_l[k] = 0.0f, st_acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; ok && q < a.x_world; ++q) {
          const uint2* rec = rec0 + size_t(q) * rank_words;
          uint2 w[6];
          for (;;) {
#pragma unroll
            for (int i = 0; i < 4; ++i) w[i] = ld_word(rec + 4 * c4 + i);
            w[4] = ld_word(rec + HD), w[5] = ld_word(rec + HD + 1);
            bool all = true;
#pragma unroll
            for (int i = 0; i < 6; ++i) all = all && w[i].y == a.x_tag;
            if (all) break;
            if (global_timer_ns() - t0 > limit) {
              ok = false;
              break;
            }
            __nanosleep(32);
          }
          if (!ok) break;
          const float m_q = __uint_as_float(w[4].x);
          if (m_q == -INFINITY) continue;
          if (m_q > st_m[k]) {
            const float f = __expf(st_m[k] - m_q);
            st_l[k] *= f, st_acc[k].x *= f, st_acc[k].y *= f, st_acc[k].z *= f, st_acc[k].w *= f;
            st_m[k] = m_q;
          }
          const float wq = __expf(m_q - st_m[k]);
          st_l[k] += wq * __uint_as_float(w[5].x);
          st_acc[k].x += wq * __uint_as_float(w[0].x), st_acc[k].y += wq * __uint_as_float(w[1].x);
          st_acc[k].z += wq * __uint_as_float(w[2].x), st_acc[k].w += wq * __uint_as_float(w[3].x);
        }
      }
      // Nobody writes O unless every thread of the CTA has all its words.
      if (!__syncthreads_and(ok)) {
        if (threadIdx.x == 0) atomicCAS(a.status, kStatusOk, kStatusPeerTimeout);
        return;
      }
    }

#pragma unroll
    for (int k = 0; k < MAXI; ++k) {
      const int item = threadIdx.x + k * (NW * 32);
      if (item >= n_items) break;
      const int hg = item / (HD / 4), c4 = item % (HD / 4), h = kvh * G + hg;
      const float inv_l = st_l[k] > 0.0f ? 1.0f / st_l[k] : 0.0f;
      float v[4] = {st_acc[k].x * inv_l, st_acc[k].y * inv_l, st_acc[k].z * inv_l, st_acc[k].w * inv_l};
      if (a.X) {
        const float4 gt = *reinterpret_cast<const float4*>(a.X + size_t(row) * p.g_ld + size_t(h) * 2 * HD + HD + 4 * c4);
        v[0] *= sigmoid_gate(gt.x), v[1] *= sigmoid_gate(gt.y), v[2] *= sigmoid_gate(gt.z), v[3] *= sigmoid_gate(gt.w);
      }
      *reinterpret_cast<uint2*>(static_cast<typename QE::T*>(a.O) + size_t(row) * p.q_ld + size_t(h) * HD + 4 * c4) =
          make_uint2(QE::pack2(v[0], v[1]), QE::pack2(v[2], v[3]));
      if (a.lse && c4 == 0) a.lse[size_t(row) * p.H + h] = st_l[k] > 0.0f ? st_m[k] + __logf(st_l[k]) : -INFINITY;
    }
  }
}

template <class C>
cudaError_t setup_one() {
  return cudaFuncSetAttribute(decode_gqa_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
}
template <class C>
cudaError_t launch_one(const KernelArgs& a, const CUtensorMap& m, cudaStream_t stream) {
  if (a.x_world > 0 && (a.x_phases & 2)) {
    // CTAs of this launch wait for CTAs of other GPUs: every CTA of the grid must hold an SM slot at once.
    int per_sm = 0, dev = 0, sms = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_gqa_kernel<C>, C::NW * 32, C::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    if (int64_t(a.n_tiles) * a.p.Hkv > int64_t(per_sm) * sms) return cudaErrorCooperativeLaunchTooLarge;
  }
  return launch_pdl(decode_gqa_kernel<C>, dim3(unsigned(a.n_tiles) * unsigned(a.p.Hkv)), dim3(C::NW * 32), C::SMEM_BYTES, stream, m, a);
}

// Instantiations: (HD, pool type, Q type, warps, stages). Rings are sized for two CTAs per
// SM (<= 110 KB each) so that one CTA's ramp-up and merge overlap the other's streaming. Instances whose
// 16-key blocks are 4 KB (128-dim E4M3, 64-dim) do as much work per block for half the bytes: three-slot rings
// (49 KB per CTA) and a 128-register cap put four CTAs on an SM - measured 0.79 -> 0.85 and 0.86 -> 0.96 of
// the copy peak on the 32-sequence batch against deeper rings with two or three CTAs.
using D128H = DecodeCfg<128, ESP_F16, ESP_F16, 4, 3>;
using D128B = DecodeCfg<128, ESP_BF16, ESP_BF16, 4, 3>;
using D256H = DecodeCfg<256, ESP_F16, ESP_F16, 4, 3>;
using D256B = DecodeCfg<256, ESP_BF16, ESP_BF16, 4, 3>;
using D128EH = DecodeCfg<128, ESP_E4M3, ESP_F16, 4, 3>;
using D128EB = DecodeCfg<128, ESP_E4M3, ESP_BF16, 4, 3>;
using D256EH = DecodeCfg<256, ESP_E4M3, ESP_F16, 4, 3>;
using D256EB = DecodeCfg<256, ESP_E4M3, ESP_BF16, 4, 3>;
// 512-dim heads (the global layers of kernels/80_gemma.metal, HD = 512 instantiations): a 16-key block is
// 32 KB of 16-bit keys and values, so three warps with two blocks each fill the SM's shared memory (one CTA
// per SM, 192 KB in flight); E4M3 blocks are half that and two CTAs fit.
using D512H = DecodeCfg<512, ESP_F16, ESP_F16, 3, 2>;
using D512B = DecodeCfg<512, ESP_BF16, ESP_BF16, 3, 2>;
using D512EH = DecodeCfg<512, ESP_E4M3, ESP_F16, 3, 2>;
using D512EB = DecodeCfg<512, ESP_E4M3, ESP_BF16, 3, 2>;
// 64-dim heads (kernels/90_lfm2.metal:160-161), 16-bit pools. A row of an E4M3 pool would be half a 128-byte
// line: the general kernel keeps those.
using D64H = DecodeCfg<64, ESP_F16, ESP_F16, 4, 3>;
using D64B = DecodeCfg<64, ESP_BF16, ESP_BF16, 4, 3>;

}  // namespace

bool decode_gqa_supports(int32_t HD, int32_t G, int32_t bt, int32_t q_dtype, int32_t kv_dtype) {
  if (HD != 64 && HD != 128 && HD != 256 && HD != 512) return false;
  if (HD == 64 && kv_dtype == ESP_E4M3) return false;
  if (G < 1 || G > 8) return false;
  if (bt <= 0 || bt % 16 != 0) return false;
  if (q_dtype != ESP_F16 && q_dtype != ESP_BF16) return false;
  return kv_dtype == q_dtype || kv_dtype == ESP_E4M3;
}

cudaError_t decode_gqa_setup() {
  cudaError_t e;
  if ((e = setup_one<D128H>()) != cudaSuccess) return e;
  if ((e = setup_one<D128B>()) != cudaSuccess) return e;
  if ((e = setup_one<D256H>()) != cudaSuccess) return e;
  if ((e = setup_one<D256B>()) != cudaSuccess) return e;
  if ((e = setup_one<D128EH>()) != cudaSuccess) return e;
  if ((e = setup_one<D128EB>()) != cudaSuccess) return e;
  if ((e = setup_one<D256EH>()) != cudaSuccess) return e;
  if ((e = setup_one<D256EB>()) != cudaSuccess) return e;
  if ((e = setup_one<D512H>()) != cudaSuccess) return e;
  if ((e = setup_one<D512B>()) != cudaSuccess) return e;
  if ((e = setup_one<D512EH>()) != cudaSuccess) return e;
  if ((e = setup_one<D512EB>()) != cudaSuccess) return e;
  if ((e = setup_one<D64H>()) != cudaSuccess) return e;
  return setup_one<D64B>();
}

cudaError_t launch_decode_gqa(const KernelArgs& a, const CUtensorMap& m, cudaStream_t stream, uint64_t* launches) {
  if (a.n_tiles <= 0) return cudaSuccess;
  cudaError_t e = cudaErrorInvalidValue;
  const bool f16 = a.q_dtype == ESP_F16;
  if (a.kv_dtype == ESP_E4M3) {
    if (a.HD == 128) e = f16 ? launch_one<D128EH>(a, m, stream) : launch_one<D128EB>(a, m, stream);
    else if (a.HD == 256) e = f16 ? launch_one<D256EH>(a, m, stream) : launch_one<D256EB>(a, m, stream);
    else if (a.HD == 512) e = f16 ? launch_one<D512EH>(a, m, stream) : launch_one<D512EB>(a, m, stream);
  } else {
    if (a.HD == 128) e = f16 ? launch_one<D128H>(a, m, stream) : launch_one<D128B>(a, m, stream);
    else if (a.HD == 256) e = f16 ? launch_one<D256H>(a, m, stream) : launch_one<D256B>(a, m, stream);
    else if (a.HD == 512) e = f16 ? launch_one<D512H>(a, m, stream) : launch_one<D512B>(a, m, stream);
    else if (a.HD == 64) e = f16 ? launch_one<D64H>(a, m, stream) : launch_one<D64B>(a, m, stream);
  }
  if (e == cudaSuccess) ++*launches;
  return e;
}

}  // namespace esp
