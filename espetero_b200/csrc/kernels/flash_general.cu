// General forest attention: any tile shape, any block size, any mask, every dtype.
//
// Computes what flash_attention computes (kernels/40_attention.metal:156-343 of the
// reference; generic head dim: kernels/80_gemma.metal:157-342): per (kv head, tile) the
// tile's rows x G heads attend to the cached key range [k0, k1) of the paged pool and,
// when tile.last, to the visible batch keys of their tree. It is the kernel the dispatcher
// falls back to when the tensor-core kernels do not cover a shape (odd block sizes,
// tile key ranges that do not start on a 16-key boundary), and the second, independent
// GPU implementation the tests cross-check the fast kernels against.
//
// With the Qwen sparse-attention arguments (KernelArgs::qsa_*) it is also flash_attention_qsa
// (kernels/45_qsa.metal:452-690): a tile with pad0 = 1 reads the cached keys of its union list - entries
// [k0, k1) of list pad1, each one block of 4 keys with an 8-bit row mask - and a sparse row counts a batch key
// only if the key's block is selected for it or lies in its tail.
//
// One warp owns one (row, head) pair at a time: 32 keys per step, lane = key for the
// scores (K rows read straight from the pool, 16 bytes per load), warp-shuffle online
// softmax in the exp2 domain, lane = slice of HD / 32 dims for P.V.
#include "common.cuh"
#include "../launch.h"

namespace esp {
namespace {

constexpr int kWarps = 4;

template <int QDT>
__device__ __forceinline__ void dot16(const uint4& v, const float* q, float& acc) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = Elem16<QDT>::unpack2(w[i]);
    acc = fmaf(q[2 * i], f.x, acc);
    acc = fmaf(q[2 * i + 1], f.y, acc);
  }
}

__device__ __forceinline__ void dot_e4m3(const uint4& v, const float* q, float& acc) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lo_u = e4m3x2_to_f16x2(uint16_t(w[i] & 0xFFFFu));
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&lo_u));
    const uint32_t hi_u = e4m3x2_to_f16x2(uint16_t(w[i] >> 16));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&hi_u));
    acc = fmaf(q[4 * i], lo.x, acc);
    acc = fmaf(q[4 * i + 1], lo.y, acc);
    acc = fmaf(q[4 * i + 2], hi.x, acc);
    acc = fmaf(q[4 * i + 3], hi.y, acc);
  }
}

template <int HD, int QDT, int KVDT>
__global__ void __launch_bounds__(kWarps * 32) flash_general_kernel(const KernelArgs a) {
  constexpr int DPL = HD / 32;  // dims per lane in P.V
  using Q16 = Elem16<QDT>;
  __shared__ float qs[kWarps][HD];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const esp_attn_params& p = a.p;
  const int kvh = blockIdx.x % p.Hkv;
  const esp_attn_tile tile = a.tiles[blockIdx.x / p.Hkv];
  const esp_attn_tree tree = a.trees[tile.tree];
  const int G = a.G, TR = a.tile_rows;
  const int end = tree.base + tree.M;
  const int rows_live = min(TR, end - tile.r0);
  const size_t blk_elems = size_t(p.bt) * p.kv_ld;
  const float sl2 = a.scale * kLog2e;

  for (int pair = warp; pair < rows_live * G; pair += kWarps) {
    const int fm = pair / G, hg = pair % G;
    const int row = tile.r0 + fm, rr = row - tree.base, h = kvh * G + hg;
    __syncwarp();
    for (int d = lane; d < HD; d += 32)
      qs[warp][d] = Q16::to_f32(static_cast<const typename Q16::T*>(a.Q)[size_t(row) * p.q_ld + size_t(h) * HD + d]);
    __syncwarp();
    const float* q = qs[warp];

    // Sliding-window layers (kernels/80_gemma.metal:123-142, :284-285): a key `window` or more
    // positions behind the query is masked; cached key j sits at position j, a batch key at its row's.
    const int qpos = a.window > 0 ? a.pos[4 * size_t(row)] : 0;
    // Block of cached key j (ring layers keep a sequence's blocks in place: table + (j / bt) % ring).
    // The table's contents live on the device and no host check sees them: an id outside the region is
    // recorded in the status word and the key is skipped instead of read.
    auto block_of = [&](int j, bool& ok) {
      const int b = a.ring > 0 ? tree.table + (j / p.bt) % a.ring : a.blocks[tree.table + j / p.bt];
      ok = b >= 0 && b < a.n_blocks;
      if (!ok) atomicExch(a.status, kStatusBadBlock);
      return size_t(ok ? b : 0);
    };
    float m_run = -INFINITY, l_run = 0.0f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.0f;

    // One 32-key step. `s` is this lane's scaled score in the exp2 domain (or -inf),
    // vrow(jj, scale&) gives the address of key jj's V row for this kv head.
    auto softmax_pv = [&](float s, auto&& vrow) {
      float mx = s;
#pragma unroll
      for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m_run, mx);
      if (m_new == -INFINITY) return;  // nothing visible yet
      const float corr = fast_exp2(m_run - m_new);
      const float pv = fast_exp2(s - m_new);
      float ps = pv;
#pragma unroll
      for (int o = 16; o; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      l_run = l_run * corr + ps;
      m_run = m_new;
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[i] *= corr;
      for (int jj = 0; jj < 32; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, pv, jj);
        if (pj == 0.0f) continue;  // warp-uniform
        vrow(jj, pj);
      }
    };

    // ---- cached keys: of the tile's union list (Qwen sparse attention), else [k0, k1)
    const bool sparse_tile = a.qsa_tlist != nullptr && tile.pad0 != 0;
    int4 ri = make_int4(0, 0, -1, 0);
    if (a.qsa_rinfo) ri = reinterpret_cast<const int4*>(a.qsa_rinfo)[row];
    const bool row_sparse = sparse_tile && ri.z >= 0;
    if (sparse_tile) {
      // 8 entries = 32 keys per step: lane -> entry lane / 4, key lane % 4 of its block
      const bool list_ok = tile.pad1 >= 0 && tile.pad1 < a.qsa_n_lists;
      const uint32_t* tl = a.qsa_tlist + size_t(list_ok ? tile.pad1 : 0) * ESP_QSA_LMAX;
      const int e_end = list_ok ? min(min(tile.k1, int(min(a.qsa_tcount[tile.pad1], uint32_t(ESP_QSA_LMAX)))), ESP_QSA_LMAX) : 0;
      for (int e0 = tile.k0; e0 < e_end; e0 += 8) {
        const int e = e0 + (lane >> 2);
        const uint32_t ent = e < e_end ? tl[e] : 0xFFFFFFFFu;
        const int j = int(ent >> 8) * 4 + (lane & 3);
        float s = -INFINITY;
        bool b_ok = false;
        const bool vis = ent != 0xFFFFFFFFu && j < tree.P && ((ent >> uint32_t(fm)) & 1u);
        const size_t b = vis ? block_of(j, b_ok) : 0;
        if (b_ok) {
          const size_t off = p.kv_base + (b * 2) * blk_elems + size_t(j % p.bt) * p.kv_ld + size_t(kvh) * HD;
          float dot = 0.0f;
          if constexpr (KVDT == ESP_E4M3) {
            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(a.kv) + off);
#pragma unroll 4
            for (int c = 0; c < HD / 16; ++c) dot_e4m3(src[c], q + 16 * c, dot);
            dot *= a.kv_scales[(b * 2) * p.Hkv + kvh];
          } else {
            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.kv) + off);
#pragma unroll 4
            for (int c = 0; c < HD / 8; ++c) dot16<KVDT>(src[c], q + 8 * c, dot);
          }
          s = dot * sl2;
        }
        softmax_pv(s, [&](int jj, float pj) {
          const uint32_t ent_j = __shfl_sync(0xffffffffu, ent, jj & ~3);  // (every lane of an entry holds it)
          const int jk = int(ent_j >> 8) * 4 + (jj & 3);
          bool v_ok;
          const size_t bv = block_of(jk, v_ok);  // valid: its score was finite
          const size_t off = p.kv_base + (bv * 2 + 1) * blk_elems + size_t(jk % p.bt) * p.kv_ld + size_t(kvh) * HD + lane * DPL;
          if constexpr (KVDT == ESP_E4M3) {
            const float w = pj * a.kv_scales[(bv * 2 + 1) * p.Hkv + kvh];
            const uint8_t* src = static_cast<const uint8_t*>(a.kv) + off;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[i] = fmaf(w, e4m3_to_f32(src[i]), acc[i]);
          } else {
            const typename Elem16<KVDT>::T* src = static_cast<const typename Elem16<KVDT>::T*>(a.kv) + off;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[i] = fmaf(pj, Elem16<KVDT>::to_f32(src[i]), acc[i]);
          }
        });
      }
    } else
    for (int j0 = tile.k0; j0 < tile.k1; j0 += 32) {
      const int j = j0 + lane;
      float s = -INFINITY;
      bool b_ok = false;
      const size_t b = (j < tile.k1 && (a.window <= 0 || qpos - j < a.window)) ? block_of(j, b_ok) : 0;
      if (b_ok) {
        const size_t off = p.kv_base + (b * 2) * blk_elems + size_t(j % p.bt) * p.kv_ld + size_t(kvh) * HD;
        float dot = 0.0f;
        if constexpr (KVDT == ESP_E4M3) {
          const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(a.kv) + off);
#pragma unroll 4
          for (int c = 0; c < HD / 16; ++c) dot_e4m3(src[c], q + 16 * c, dot);
          dot *= a.kv_scales[(b * 2) * p.Hkv + kvh];
        } else {
          const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.kv) + off);
#pragma unroll 4
          for (int c = 0; c < HD / 8; ++c) dot16<KVDT>(src[c], q + 8 * c, dot);
        }
        s = dot * sl2;
      }
      softmax_pv(s, [&](int jj, float pj) {
        const int jk = j0 + jj;
        bool v_ok;
        const size_t b = block_of(jk, v_ok);  // valid: its score was finite
        const size_t off = p.kv_base + (b * 2 + 1) * blk_elems + size_t(jk % p.bt) * p.kv_ld + size_t(kvh) * HD + lane * DPL;
        if constexpr (KVDT == ESP_E4M3) {
          const float w = pj * a.kv_scales[(b * 2 + 1) * p.Hkv + kvh];
          const uint8_t* src = static_cast<const uint8_t*>(a.kv) + off;
#pragma unroll
          for (int i = 0; i < DPL; ++i) acc[i] = fmaf(w, e4m3_to_f32(src[i]), acc[i]);
        } else {
          const typename Elem16<KVDT>::T* src = static_cast<const typename Elem16<KVDT>::T*>(a.kv) + off;
#pragma unroll
          for (int i = 0; i < DPL; ++i) acc[i] = fmaf(pj, Elem16<KVDT>::to_f32(src[i]), acc[i]);
        }
      });
    }

    // ---- batch keys of the tree (tree mask)
    if (tile.last) {
      int4 d = make_int4(0, 0, 0, 0);
      uint64_t am = 0;
      int k_last;
      if (a.anc_mask) {
        am = a.anc_mask[row];
        k_last = min(tree.M, 64) - 1;
      } else {
        d = reinterpret_cast<const int4*>(a.desc)[row];
        k_last = min(tree.M - 1, max(rr, d.z - 1));
        if (a.bidi) k_last = min(tree.M - 1, max(k_last, d.w - 1));  // an image's rows see the whole image
      }
      for (int j0 = 0; j0 <= k_last; j0 += 32) {
        const int j = j0 + lane;
        bool vis = j <= k_last;
        if (a.anc_mask) vis = vis && ((am >> j) & 1ull);
        else vis = vis && ((j < d.z) || (j >= d.x && (j <= rr || (a.bidi && j < d.w))));
        if (a.window > 0 && vis) vis = qpos - a.pos[4 * size_t(tree.base + j)] < a.window;
        if (vis && row_sparse) {
          // the key's sequence index on this row's path, its block: in the tail (past 4 nb) or selected
          const int sj = tree.P + (j < d.z ? j : d.z + (j - d.x));
          const int bj = sj >> 2;
          vis = sj >= 4 * ri.y || ((a.qsa_sel[size_t(ri.z) * a.qsa_nbw + (bj >> 5)] >> uint32_t(bj & 31)) & 1u);
        }
        float s = -INFINITY;
        if (vis) {
          const uint4* src =
              reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.Kb) + size_t(tree.base + j) * p.kv_ld + size_t(kvh) * HD);
          float dot = 0.0f;
#pragma unroll 4
          for (int c = 0; c < HD / 8; ++c) dot16<QDT>(src[c], q + 8 * c, dot);
          s = dot * sl2;
        }
        softmax_pv(s, [&](int jj, float pj) {
          const typename Q16::T* src =
              static_cast<const typename Q16::T*>(a.Vb) + size_t(tree.base + j0 + jj) * p.kv_ld + size_t(kvh) * HD + lane * DPL;
#pragma unroll
          for (int i = 0; i < DPL; ++i) acc[i] = fmaf(pj, Q16::to_f32(src[i]), acc[i]);
        });
      }
    }

    // ---- epilogue: partial record or the gated, normalised output
    if (tile.part >= 0) {
      float* rec = a.parts + ((size_t(tile.part) * p.Hkv + kvh) * TR * G + size_t(fm) * G + hg) * (HD + 2);
#pragma unroll
      for (int i = 0; i < DPL; ++i) rec[lane * DPL + i] = acc[i];
      if (lane == 0) {
        rec[HD] = m_run * kLn2;  // -inf stays -inf
        rec[HD + 1] = l_run;
      }
    } else {
      const float inv_l = l_run > 0.0f ? 1.0f / l_run : 0.0f;
      typename Q16::T* op = static_cast<typename Q16::T*>(a.O) + size_t(row) * p.q_ld + size_t(h) * HD + lane * DPL;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        float o = acc[i] * inv_l;
        if (a.X) o *= sigmoid_gate(a.X[size_t(row) * p.g_ld + size_t(h) * 2 * HD + HD + lane * DPL + i]);
        op[i] = Q16::from_f32(o);
      }
      if (a.lse && lane == 0) a.lse[size_t(row) * p.H + h] = l_run > 0.0f ? m_run * kLn2 + __logf(l_run) : -INFINITY;
    }
  }
}

template <int HD, int QDT>
cudaError_t launch_typed(const KernelArgs& a, cudaStream_t stream) {
  const dim3 grid(unsigned(a.n_tiles) * unsigned(a.p.Hkv)), block(kWarps * 32);
  if (a.kv_dtype == ESP_E4M3) flash_general_kernel<HD, QDT, ESP_E4M3><<<grid, block, 0, stream>>>(a);
  else flash_general_kernel<HD, QDT, QDT><<<grid, block, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_flash_general(const KernelArgs& a, cudaStream_t stream, uint64_t* launches) {
  if (a.n_tiles <= 0) return cudaSuccess;
  cudaError_t e = cudaErrorInvalidValue;
  if (a.HD == 128) e = a.q_dtype == ESP_F16 ? launch_typed<128, ESP_F16>(a, stream) : launch_typed<128, ESP_BF16>(a, stream);
  else if (a.HD == 256) e = a.q_dtype == ESP_F16 ? launch_typed<256, ESP_F16>(a, stream) : launch_typed<256, ESP_BF16>(a, stream);
  else if (a.HD == 64) e = a.q_dtype == ESP_F16 ? launch_typed<64, ESP_F16>(a, stream) : launch_typed<64, ESP_BF16>(a, stream);
  else if (a.HD == 512) e = a.q_dtype == ESP_F16 ? launch_typed<512, ESP_F16>(a, stream) : launch_typed<512, ESP_BF16>(a, stream);
  if (e == cudaSuccess) ++*launches;
  return e;
}

}  // namespace esp
