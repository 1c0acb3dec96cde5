// Forest attention for 128-row tiles on the 5th-generation tensor cores (sm_100a):
// causal prefill, the batched tree-verify pass and any other multi-row tile.
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
// for cached keys and directly in Kb / Vb for batch keys. MMAs are issued by one thread and
// tracked with tcgen05.commit -> mbarrier; two CTAs share an SM (97 KB of shared memory and
// 256 tensor-memory columns each) so that one CTA's softmax overlaps the other's MMAs.
// Every wait is bounded: after a timeout the CTA records a status code, stops waiting,
// finishes its loop, frees its tensor memory and returns.
#include "umma.cuh"
#include "../launch.h"

namespace esp {
namespace {

constexpr int BM = 128;  // (row, head) pairs per CTA
constexpr int BN = 64;   // keys per block
constexpr int HD = 128;  // head dim of this kernel
constexpr int Q_BYTES = BM * HD * 2;        // [2 halves of 64 dims][128 rows][128 B]
constexpr int KV_TILE = BN * HD * 2;        // [2 halves][64 rows][128 B]
constexpr int HALF_Q = BM * 128;            // bytes between the 64-dim halves of the Q tile
constexpr int HALF_KV = BN * 128;           // ... of a K / V tile
constexpr int SMEM_BYTES = Q_BYTES + 4 * KV_TILE + 1024;
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t COL_S = 0, COL_P = 64, COL_O = 96;  // S: 64 fp32, P: 32 (64 x 16 bit), O: 128 fp32
constexpr float kRescaleThreshold = 8.0f;   // log2 units

struct PageRef {  // where one 16-key page of a key block comes from
  int raw;        // block id as loaded from the page table (pool), or first row (Kb / Vb)
  int off;        // row inside the block (pool)
  int kind;       // -1: nothing to load, 0: paged pool, 1: Kb / Vb
};

template <int QDT>
__global__ void __launch_bounds__(BM, 2)
    flash_umma_kernel(const __grid_constant__ CUtensorMap pool_map, const __grid_constant__ CUtensorMap kb_map,
                      const __grid_constant__ CUtensorMap vb_map, const KernelArgs a) {
  using QE = Elem16<QDT>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_k[2], bar_v[2], bar_s, bar_o;
  __shared__ uint32_t tmem_slot;
  __shared__ int red[6];  // anc_max, seg_min, anc_min, seg_max
  __shared__ volatile int dead;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_sm = smem;
  uint8_t* k_sm[2] = {smem + Q_BYTES, smem + Q_BYTES + KV_TILE};
  uint8_t* v_sm[2] = {smem + Q_BYTES + 2 * KV_TILE, smem + Q_BYTES + 3 * KV_TILE};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const esp_attn_params& p = a.p;
  const int G = a.G, TR = a.tile_rows, HPC = BM / TR;
  const esp_attn_tile tile = a.tiles[a.n_tiles - 1 - int(blockIdx.x)];  // long (late) tiles first
  const esp_attn_tree tree = a.trees[tile.tree];
  const int fm = tid / HPC, hh = tid % HPC;
  const int head = int(blockIdx.y) * HPC + hh;
  const int kvh = (int(blockIdx.y) * HPC) / G;
  const int end = tree.base + tree.M;
  const int rows_live = min(TR, end - tile.r0);
  const bool row_ok = fm < rows_live;
  const int row = row_ok ? tile.r0 + fm : end - 1;
  const int rr = row - tree.base;
  const float sl2 = a.scale * kLog2e;

  // ---- set-up: barriers, tensor memory, Q tile, mask bounds
  if (tid == 0) {
    tma_prefetch_desc(&pool_map);
    tma_prefetch_desc(&kb_map);
    tma_prefetch_desc(&vb_map);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_k[s], 4);  // one arrival per page-issuing warp
      mbar_init(&bar_v[s], 4);
    }
    mbar_init(&bar_s, 1);
    mbar_init(&bar_o, 1);
    mbar_fence_init();
    red[0] = 0, red[1] = 1 << 30, red[2] = 1 << 30, red[3] = 0;
    dead = 0;
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  {
    // Q row of this thread into the K-major swizzled tile
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const typename QE::T*>(a.Q) + size_t(row) * p.q_ld + size_t(head) * HD);
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int i = 0; i < 8; ++i)
        *reinterpret_cast<uint4*>(q_sm + c * HALF_Q + tid * 128 + ((i ^ (tid & 7)) << 4)) = src[c * 8 + i];
    fence_proxy_async_smem();
  }
  int4 d = make_int4(0, 0, 0, 0);
  uint64_t am = 0;
  const bool use_anc = a.anc_mask != nullptr;
  if (tile.last) {
    if (use_anc) am = a.anc_mask[row];
    else d = reinterpret_cast<const int4*>(a.desc)[row];
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (tile.last && !use_anc) {
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
    __syncthreads();
  }
  const uint32_t tmem = tmem_slot;
  const uint32_t t_lane = tmem + (uint32_t(warp * 32) << 16);  // this warp's quarter of the lanes

  // ---- block list: cached 64-key blocks, then the batch blocks some row of the tile can see
  const int r_first = tile.r0 - tree.base, r_last = r_first + rows_live - 1;
  const int anc_max = red[0], seg_min = red[1], anc_min = red[2], seg_max = red[3];
  int k_last = -1, a_hi = 0, b_lo = 0, nbb = 0;
  if (tile.last) {
    if (use_anc) {
      k_last = min(tree.M, 64) - 1;
      a_hi = (k_last + BN) / BN;
      nbb = a_hi;
    } else {
      k_last = min(tree.M - 1, max(r_last, anc_max - 1));
      const int n_all = (k_last + BN) / BN;
      a_hi = min((anc_max + BN - 1) / BN, n_all);                 // blocks below the ancestor range
      b_lo = max(a_hi, seg_min / BN);                             // blocks of the rows' own segments
      const int b_hi = min(r_last / BN, n_all - 1);
      nbb = a_hi + max(0, b_hi - b_lo + 1);
    }
  }
  const int nbc = (tile.k1 - tile.k0 + BN - 1) / BN;
  const int nb = nbc + nbb;
  auto batch_j0 = [&](int i) { return BN * (i < a_hi ? i : b_lo + (i - a_hi)); };

  // Page reference of warp `warp`'s 16-key page of block b (lane 0 of each warp issues it).
  // The page-table entry is only loaded here; the row arithmetic happens when the page is
  // issued, one or two iterations later, so the load's latency is off the critical path.
  auto page_of = [&](int b) {
    PageRef r{0, 0, -1};
    if (b >= nb) return r;
    if (b < nbc) {
      const int j = tile.k0 + BN * b + 16 * warp;
      if (j < tile.k1) {
        r.raw = a.blocks[tree.table + j / p.bt];
        r.off = j % p.bt;
        r.kind = 0;
      }
    } else {
      const int j = batch_j0(b - nbc) + 16 * warp;
      if (j <= k_last) {
        r.raw = tree.base + j;
        r.kind = 1;
      }
    }
    return r;
  };
  auto wait_bar = [&](uint64_t* bar, uint32_t parity, int code) {
    if (dead) return;
    if (!mbar_wait(bar, parity)) {
      dead = 1;
      atomicExch(a.status, code);
    }
  };
  auto issue_k = [&](const PageRef& r, int stage) {
    if (r.kind < 0) {
      mbar_arrive(&bar_k[stage]);
      return;
    }
    uint8_t* dst = k_sm[stage] + warp * 2048;
    const int y = r.kind ? r.raw : r.raw * 2 * p.bt + r.off;
    mbar_arrive_expect_tx(&bar_k[stage], 4096);
    tma_load_3d(dst, r.kind ? &kb_map : &pool_map, &bar_k[stage], 0, y, kvh * 2);
    tma_load_3d(dst + HALF_KV, r.kind ? &kb_map : &pool_map, &bar_k[stage], 0, y, kvh * 2 + 1);
  };
  auto issue_v = [&](const PageRef& r, int stage) {
    if (r.kind < 0) {
      mbar_arrive(&bar_v[stage]);
      return;
    }
    uint8_t* dst = v_sm[stage] + warp * 2048;
    const int y = r.kind ? r.raw : (r.raw * 2 + 1) * p.bt + r.off;
    mbar_arrive_expect_tx(&bar_v[stage], 4096);
    tma_load_3d(dst, r.kind ? &vb_map : &pool_map, &bar_v[stage], 0, y, kvh * 2);
    tma_load_3d(dst + HALF_KV, r.kind ? &vb_map : &pool_map, &bar_v[stage], 0, y, kvh * 2 + 1);
  };

  // prologue: K of blocks 0 and 1, V of block 0
  PageRef pg1{0, 0, -1}, pg2{0, 0, -1}, pg3{0, 0, -1};  // pages of blocks b+1, b+2, b+3 (lane 0 of each warp)
  if (lane == 0 && nb > 0) {
    const PageRef pg0 = page_of(0);
    pg1 = page_of(1);
    pg2 = page_of(2);
    pg3 = page_of(3);
    issue_k(pg0, 0);
    issue_v(pg0, 0);
    if (nb > 1) issue_k(pg1, 1);
  }

  constexpr uint32_t idesc_qk = umma_idesc<QDT>(BM, BN, 0, 0);
  constexpr uint32_t idesc_pv = umma_idesc<QDT>(BM, HD, 0, 1);
  float m_ref = -INFINITY, l_run = 0.0f;

  for (int b = 0; b < nb; ++b) {
    const int stage = b & 1;
    const bool cached = b < nbc;
    const int j0 = cached ? tile.k0 + BN * b : batch_j0(b - nbc);
    const int n_valid = cached ? min(BN, tile.k1 - j0) : min(BN, k_last + 1 - j0);

    // ---- S = Q . K^T
    if (tid == 0) {
      wait_bar(&bar_k[stage], (b >> 1) & 1, kStatusTmaTimeout);
      tc_fence_after_sync();
      const uint32_t qa = smem_u32(q_sm), ka = smem_u32(k_sm[stage]);
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const uint64_t da = umma_smem_desc(qa + (ks >> 2) * HALF_Q + (ks & 3) * 32, 16, 1024);
        const uint64_t db = umma_smem_desc(ka + (ks >> 2) * HALF_KV + (ks & 3) * 32, 16, 1024);
        umma_ss(tmem + COL_S, da, db, idesc_qk, ks > 0);
      }
      umma_commit(&bar_s);
    }
    wait_bar(&bar_s, b & 1, kStatusMmaTimeout);
    tc_fence_after_sync();
    // S_b is complete, and so is every earlier MMA: K[stage] and V[stage ^ 1] are free.
    if (lane == 0) {
      if (b + 2 < nb) issue_k(pg2, stage);
      if (b + 1 < nb) issue_v(pg1, stage ^ 1);
      pg1 = pg2;
      pg2 = pg3;
      pg3 = page_of(b + 4);  // its page-table load stays in flight until it is issued
    }
    __syncwarp();

    // ---- this thread's 64 scores
    uint32_t sr[2][32];
    tmem_ld32(t_lane + COL_S, sr[0]);
    tmem_ld32(t_lane + COL_S + 32, sr[1]);
    tmem_wait_ld();
    // does any (row, key) of the block need the tree mask?
    bool need_mask = false;
    if (!cached) {
      if (use_anc) need_mask = true;
      else need_mask = !((j0 + BN - 1 < anc_min) || (j0 >= seg_max && j0 + BN - 1 <= r_first));
    }
    float mx = -INFINITY;
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int col = 32 * h + c;
        float s = __uint_as_float(sr[h][c]) * sl2;
        bool vis = col < n_valid;
        if (need_mask) {
          const int j = j0 + col;
          vis = vis && (use_anc ? ((am >> (j & 63)) & 1ull) != 0 : ((j < d.z) || (j >= d.x && j <= rr)));
        }
        s = vis ? s : -INFINITY;
        sr[h][c] = __float_as_uint(s);
        mx = fmaxf(mx, s);
      }
    // lazy rescale: keep the old reference maximum unless this block exceeds it by 2^8
    float factor = 1.0f;
    const bool grow = mx > m_ref + kRescaleThreshold || (m_ref == -INFINITY && mx > -INFINITY);
    if (grow) {
      factor = fast_exp2(m_ref - mx);  // 0 when nothing was seen before
      m_ref = mx;
      l_run *= factor;
    }
    const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
    float ps = 0.0f;
    uint32_t pk[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      const float p0 = fast_exp2(__uint_as_float(sr[c >> 4][(2 * c) & 31]) - m_use);
      const float p1 = fast_exp2(__uint_as_float(sr[c >> 4][(2 * c + 1) & 31]) - m_use);
      ps += p0 + p1;
      pk[c] = QE::pack2(p0, p1);
    }
    l_run += ps;
    tmem_st32(t_lane + COL_P, pk);
    if (b > 0 && __any_sync(0xffffffffu, grow)) {
      // O of this warp's rows *= factor (1 for rows whose reference did not move)
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(t_lane + COL_O + 32 * c, o);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
        tmem_st32(t_lane + COL_O + 32 * c, o);
      }
    }
    tmem_wait_st();
    if (n_valid < BN) {
      // tail block: V rows past the range are stale or foreign bytes; 0 * NaN must not happen
      wait_bar(&bar_v[stage], (b >> 1) & 1, kStatusTmaTimeout);
      const int n = (BN - n_valid) * 16;  // 16-byte chunks: 2 halves x 8 per row
      for (int i = tid; i < n; i += BM) {
        const int r = n_valid + i / 16, c = i % 16;
        *reinterpret_cast<uint4*>(v_sm[stage] + (c >> 3) * HALF_KV + r * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
      }
      fence_proxy_async_smem();
    }
    tc_fence_before_sync();
    __syncthreads();

    // ---- O += P . V
    if (tid == 0) {
      tc_fence_after_sync();
      wait_bar(&bar_v[stage], (b >> 1) & 1, kStatusTmaTimeout);
      const uint32_t va = smem_u32(v_sm[stage]);
#pragma unroll
      for (int ks = 0; ks < BN / 16; ++ks) {
        const uint64_t db = umma_smem_desc(va + ks * 2048, HALF_KV, 1024);
        umma_ts(tmem + COL_O, tmem + COL_P + ks * 8, db, idesc_pv, (b > 0 || ks > 0) ? 1u : 0u);
      }
      if (b == nb - 1) umma_commit(&bar_o);
    }
  }

  // ---- epilogue
  if (nb > 0) {
    wait_bar(&bar_o, 0, kStatusMmaTimeout);
    tc_fence_after_sync();
  }
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
#pragma unroll 1
  for (int c = 0; c < HD / 32; ++c) {
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
        *reinterpret_cast<float2*>(rec + 32 * c + i) = make_float2(__uint_as_float(o[i]), __uint_as_float(o[i + 1]));
    } else {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          v[k] = __uint_as_float(o[i + k]) * inv_l;
          if (gp) v[k] *= sigmoid_gate(gp[32 * c + i + k]);
        }
        uint4 w;
        w.x = QE::pack2(v[0], v[1]), w.y = QE::pack2(v[2], v[3]), w.z = QE::pack2(v[4], v[5]), w.w = QE::pack2(v[6], v[7]);
        *reinterpret_cast<uint4*>(op + 32 * c + i) = w;
      }
    }
  }
  if (row_ok) {
    if (rec) {
      rec[HD] = m_ref * kLn2;  // -inf stays -inf
      rec[HD + 1] = l_run;
    } else if (a.lse) {
      a.lse[size_t(row) * p.H + head] = l_run > 0.0f ? m_ref * kLn2 + __logf(l_run) : -INFINITY;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace

bool flash_umma_supports(int32_t HDim, int32_t G, int32_t tile_rows, int32_t bt, int32_t q_dtype, int32_t kv_dtype) {
  if (HDim != HD || q_dtype != kv_dtype) return false;
  if (tile_rows != 16 && tile_rows != 32 && tile_rows != 64 && tile_rows != 128) return false;
  const int hpc = BM / tile_rows;
  if (hpc > G || G % hpc != 0) return false;
  return bt > 0 && bt % 16 == 0;
}

cudaError_t flash_umma_setup() {
  cudaError_t e = cudaFuncSetAttribute(flash_umma_kernel<ESP_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(flash_umma_kernel<ESP_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
}

cudaError_t launch_flash_umma(const KernelArgs& a, const CUtensorMap& pool_map, const CUtensorMap& kb_map, const CUtensorMap& vb_map,
                              cudaStream_t stream, uint64_t* launches) {
  if (a.n_tiles <= 0) return cudaSuccess;
  const int hpc = BM / a.tile_rows;
  const dim3 grid(unsigned(a.n_tiles), unsigned(a.p.H / hpc)), block(BM);
  if (a.q_dtype == ESP_F16) flash_umma_kernel<ESP_F16><<<grid, block, SMEM_BYTES, stream>>>(pool_map, kb_map, vb_map, a);
  else flash_umma_kernel<ESP_BF16><<<grid, block, SMEM_BYTES, stream>>>(pool_map, kb_map, vb_map, a);
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) ++*launches;
  return e;
}

}  // namespace esp
