// attn_prep for sm_100a: the step that feeds the attention pass.
//
// Reference: kernels/40_attention.metal:23-102 (256-dim heads, gate interleaved with the query
// heads, 64 rotated dims, K / V of saved rows written into the paged pool in the same kernel) and
// its generic twin q3m_attn_prep, kernels/82_qwen3_omni.metal:40-88 (full rotary, scale folded into
// the queries). One warp per (row, head); heads [0, H) are queries, [H, H + Hkv) a key head together
// with its value head. A lane owns HD / 32 consecutive dims, so the rotary partner (d +- rot_half)
// lives in lane ^ (rot_half / (HD / 32)): one shuffle per element.
//
// HBM-bound: per row it reads (H + 2 Hkv) * HD floats of X and writes as many 16-bit elements
// (plus the pool rows): 16-byte loads and 8- or 16-byte stores, every byte touched once.
#include "common.cuh"
#include "../launch.h"

namespace esp {
namespace {

constexpr int kPrepWarps = 4;

template <int HD, int QDT, bool FP8_POOL>
__global__ void __launch_bounds__(kPrepWarps * 32, HD == 128 ? 10 : 8) attn_prep_kernel(const PrepArgs a) {
  using QE = Elem16<QDT>;
  constexpr int NPT = HD / 32;
  const esp_attn_prep_params& p = a.p;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t row = blockIdx.x;
  const int head_first = (blockIdx.y * kPrepWarps + warp) * a.heads_per_warp;
  const int head_end = min(head_first + a.heads_per_warp, p.H + p.Hkv);
  pdl_wait();  // X is the previous kernel's output

  // The rotation depends on the row and the frequency only, not on the head or on which half of a
  // pair a dim is: the CTA forms the rot_half sines and cosines of its row once (sincosf of a large
  // angle costs far more than the rest of a head's arithmetic) and every lane picks its own.
  __shared__ float cs_s[128], sn_s[128];
  for (int f = threadIdx.x; f < p.rot_half; f += kPrepWarps * 32) {
    const int4 pr = reinterpret_cast<const int4*>(a.pos)[row];
    const int sl = a.rope_sel[f];
    const float position = float(sl == 0 ? pr.x : (sl == 1 ? pr.y : pr.z));
    sincosf(position * a.inv_freq[f], &sn_s[f], &cs_s[f]);
  }
  __syncthreads();
  if (head_first >= head_end) return;
  const int partner_xor = p.rot_half / NPT;     // lanes apart
  const bool rotates = lane < 2 * partner_xor;  // this lane's dims lie below 2 * rot_half
  const bool low = lane < partner_xor;
  float cs[NPT], sn[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    cs[i] = 1.0f, sn[i] = 0.0f;
    if (rotates) {
      const int f = (lane * NPT + i) & (p.rot_half - 1);
      cs[i] = cs_s[f];
      sn[i] = low ? -sn_s[f] : sn_s[f];  // x' = x c - partner s below rot_half, x c + partner s above
    }
  }

  // The elements of the next PF heads are requested before this head's arithmetic starts: about
  // 2 KB in flight per warp hide the memory latency at the occupancy the registers allow.
  constexpr int PF = NPT == 4 ? 4 : 1;
  auto src_of = [&](int head) {
    const bool q = head < p.H;
    const int hh = q ? head : head - p.H;
    return a.X + row * p.ld + (q ? p.q_off + size_t(hh) * p.q_stride : p.k_off + size_t(hh) * HD) + lane * NPT;
  };
  float4 nxt[PF][NPT / 4];
#pragma unroll
  for (int k = 0; k < PF; ++k)
    if (head_first + k < head_end) {
#pragma unroll
      for (int i = 0; i < NPT / 4; ++i) nxt[k][i] = reinterpret_cast<const float4*>(src_of(head_first + k))[i];
    }

  // The norm weights are the same for every query head (and for every key head): in registers, once.
  float wq[NPT], wk[NPT];
#pragma unroll
  for (int i = 0; i < NPT; i += 4) {
    const float4 a4 = *reinterpret_cast<const float4*>(a.qn_w + lane * NPT + i);
    const float4 b4 = *reinterpret_cast<const float4*>(a.kn_w + lane * NPT + i);
    wq[i] = a4.x, wq[i + 1] = a4.y, wq[i + 2] = a4.z, wq[i + 3] = a4.w;
    wk[i] = b4.x, wk[i + 1] = b4.y, wk[i + 2] = b4.z, wk[i + 3] = b4.w;
  }

  for (int head = head_first; head < head_end; ++head) {
  const bool is_q = head < p.H;
  const int h = is_q ? head : head - p.H;

  float x[NPT], wv[NPT];
#pragma unroll
  for (int i = 0; i < NPT; i += 4) {
    const float4 v = nxt[0][i / 4];
    x[i] = v.x, x[i + 1] = v.y, x[i + 2] = v.z, x[i + 3] = v.w;
  }
#pragma unroll
  for (int i = 0; i < NPT; ++i) wv[i] = is_q ? wq[i] : wk[i];
#pragma unroll
  for (int k = 0; k + 1 < PF; ++k) {
#pragma unroll
    for (int i = 0; i < NPT / 4; ++i) nxt[k][i] = nxt[k + 1][i];
  }
  if (head + PF < head_end) {
#pragma unroll
    for (int i = 0; i < NPT / 4; ++i) nxt[PF - 1][i] = reinterpret_cast<const float4*>(src_of(head + PF))[i];
  }
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < NPT; ++i) ss = fmaf(x[i], x[i], ss);
#pragma unroll
  for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = rsqrtf(fmaf(ss, 1.0f / float(HD), p.eps));  // the reference's rsqrt (40_attention.metal:64)
#pragma unroll
  for (int i = 0; i < NPT; ++i) x[i] = x[i] * inv * wv[i];

  // Rotary embedding: dims [0, 2 * rot_half) in pairs (d, d + rot_half).
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const float partner = __shfl_xor_sync(0xffffffffu, x[i], partner_xor);
    x[i] = x[i] * cs[i] + partner * sn[i];  // lanes that do not rotate hold c = 1, s = 0
  }

  uint32_t packed[NPT / 2];
  if (is_q) {
#pragma unroll
    for (int i = 0; i < NPT; i += 2) packed[i / 2] = QE::pack2(x[i] * p.qscale, x[i + 1] * p.qscale);
    typename QE::T* q = static_cast<typename QE::T*>(a.Q) + row * p.q_ld + size_t(h) * HD + lane * NPT;
    if constexpr (NPT == 4) *reinterpret_cast<uint2*>(q) = make_uint2(packed[0], packed[1]);
    else *reinterpret_cast<uint4*>(q) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    continue;
  }

  // key head: K as computed, V as it is
  uint32_t vpacked[NPT / 2];
  const float* vsrc = a.X + row * p.ld + p.v_off + size_t(h) * HD + lane * NPT;
#pragma unroll
  for (int i = 0; i < NPT; i += 4) {
    const float4 v = *reinterpret_cast<const float4*>(vsrc + i);
    vpacked[i / 2] = QE::pack2(v.x, v.y);
    vpacked[i / 2 + 1] = QE::pack2(v.z, v.w);
  }
#pragma unroll
  for (int i = 0; i < NPT; i += 2) packed[i / 2] = QE::pack2(x[i], x[i + 1]);
  const size_t col = size_t(h) * HD + lane * NPT;
  typename QE::T* ko = static_cast<typename QE::T*>(a.Kb) + row * p.kv_ld + col;
  typename QE::T* vo = static_cast<typename QE::T*>(a.Vb) + row * p.kv_ld + col;
  if constexpr (NPT == 4) {
    *reinterpret_cast<uint2*>(ko) = make_uint2(packed[0], packed[1]);
    *reinterpret_cast<uint2*>(vo) = make_uint2(vpacked[0], vpacked[1]);
  } else {
    *reinterpret_cast<uint4*>(ko) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    *reinterpret_cast<uint4*>(vo) = make_uint4(vpacked[0], vpacked[1], vpacked[2], vpacked[3]);
  }

  // kv_save folded in: the same (rounded) values into the row's pool entries; a row saved into two
  // slots has two.
  if (a.ktab) {
    const int4 t = reinterpret_cast<const int4*>(a.ktab)[row];
    const size_t blk = size_t(p.bt) * p.kv_ld;
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      const int b = w ? t.z : t.x, ps = w ? t.w : t.y;
      if (b < 0) continue;
      const size_t dst = p.kv_base + size_t(b) * 2 * blk + size_t(ps) * p.kv_ld + col;
      if constexpr (!FP8_POOL) {
        typename QE::T* dk = static_cast<typename QE::T*>(a.kv) + dst;
        if constexpr (NPT == 4) {
          *reinterpret_cast<uint2*>(dk) = make_uint2(packed[0], packed[1]);
          *reinterpret_cast<uint2*>(dk + blk) = make_uint2(vpacked[0], vpacked[1]);
        } else {
          *reinterpret_cast<uint4*>(dk) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          *reinterpret_cast<uint4*>(dk + blk) = make_uint4(vpacked[0], vpacked[1], vpacked[2], vpacked[3]);
        }
      } else {
        // E4M3 pool: the rounded 16-bit value divided by the block's scale (division, as
        // esp_kv_save does, so that prep + save and prep with ktab give the same codes)
        const float sk = a.kv_scales[(size_t(b) * 2) * p.Hkv + h], sv = a.kv_scales[(size_t(b) * 2 + 1) * p.Hkv + h];
        uint8_t ck[NPT], cv[NPT];
#pragma unroll
        for (int i = 0; i < NPT / 2; ++i) {
          const float2 kf = QE::unpack2(packed[i]), vf = QE::unpack2(vpacked[i]);
          ck[2 * i] = f32_to_e4m3(__fdiv_rn(kf.x, sk)), ck[2 * i + 1] = f32_to_e4m3(__fdiv_rn(kf.y, sk));
          cv[2 * i] = f32_to_e4m3(__fdiv_rn(vf.x, sv)), cv[2 * i + 1] = f32_to_e4m3(__fdiv_rn(vf.y, sv));
        }
        uint8_t* dk = static_cast<uint8_t*>(a.kv) + dst;
        if constexpr (NPT == 4) {
          *reinterpret_cast<uint32_t*>(dk) = *reinterpret_cast<const uint32_t*>(ck);
          *reinterpret_cast<uint32_t*>(dk + blk) = *reinterpret_cast<const uint32_t*>(cv);
        } else {
          *reinterpret_cast<uint2*>(dk) = *reinterpret_cast<const uint2*>(ck);
          *reinterpret_cast<uint2*>(dk + blk) = *reinterpret_cast<const uint2*>(cv);
        }
      }
    }
  }
  }  // heads of this warp
}

template <int HD, int QDT>
cudaError_t launch_hd(const PrepArgs& a, bool fp8, dim3 grid, cudaStream_t stream) {
  return fp8 ? launch_pdl(attn_prep_kernel<HD, QDT, true>, grid, dim3(kPrepWarps * 32), 0, stream, a)
             : launch_pdl(attn_prep_kernel<HD, QDT, false>, grid, dim3(kPrepWarps * 32), 0, stream, a);
}

}  // namespace

bool attn_prep_supports(int32_t HD) { return HD == 128 || HD == 256; }

cudaError_t launch_attn_prep(const PrepArgs& a, int32_t HD, int32_t q_dtype, bool fp8_pool, cudaStream_t stream, uint64_t* launches) {
  if (a.rows <= 0) return cudaSuccess;
  const int per_cta = kPrepWarps * a.heads_per_warp;
  const dim3 grid(unsigned(a.rows), unsigned((a.p.H + a.p.Hkv + per_cta - 1) / per_cta));
  cudaError_t e;
  if (HD == 128) e = q_dtype == ESP_F16 ? launch_hd<128, ESP_F16>(a, fp8_pool, grid, stream) : launch_hd<128, ESP_BF16>(a, fp8_pool, grid, stream);
  else e = q_dtype == ESP_F16 ? launch_hd<256, ESP_F16>(a, fp8_pool, grid, stream) : launch_hd<256, ESP_BF16>(a, fp8_pool, grid, stream);
  if (e == cudaSuccess) ++*launches;
  return e;
}

}  // namespace esp
