// TEST INFRASTRUCTURE: C entry points that run the reference's cooperative attention kernels - attn_prep,
// flash_attention<G>, attn_decode_gqa<G> of kernels/40_attention.metal, cut from the reference tree by
// extract_ref.py - on the CPU through the SIMT emulator of ref_simt.h, one threadgroup after the other
// over the kernels' own grids (src/model/impl/forest.h:2897-2921, :2951-2977). Part of
// oracle/_ref/libplan_ref.so; only tests/ load it. These kernels are the 256-dim, fp16, gated originals.
#include "ref_simt.h"

#include <type_traits>

namespace ref_kernels {
using namespace metal_emu;
using uint = metal_emu::uint;  // (the C library declares names of its own for these four)
using ulong = metal_emu::ulong;
using ushort = metal_emu::ushort;
using uchar = metal_emu::uchar;
#define device
#define constant const
#define kernel inline
#define UNROLL
#include "_ref/ref_kernels_simt.inc"
#undef UNROLL
#undef kernel
#undef constant
#undef device
}  // namespace ref_kernels

using namespace ref_kernels;
using metal_emu::half;
using metal_emu::int4;
using metal_emu::uint2;

namespace {

struct AttnArgs {
  const uint16_t *Q, *Kb, *Vb, *kv;
  const int32_t* blocks;
  const int32_t* desc;
  const float* X;
  uint16_t* O;
  const AttnParams* p;
  const AttnTile* tiles;
  const AttnTree* trees;
  float* parts;
};

template <int G>
void flash_group(const AttnArgs& a, unsigned gx, unsigned gy) {
  simt::run_threadgroup(64 * G, [&](unsigned tid) {
    flash_attention<G, 1>(reinterpret_cast<const half*>(a.Q), reinterpret_cast<const half*>(a.Kb), reinterpret_cast<const half*>(a.Vb),
                          reinterpret_cast<const half*>(a.kv), a.blocks, reinterpret_cast<const int4*>(a.desc), a.X, reinterpret_cast<half*>(a.O), *a.p,
                          a.tiles, a.trees, a.parts, uint2(gx, gy), tid, tid / 32, tid % 32);
  });
}
template <int G>
void decode_group(const AttnArgs& a, unsigned gx, unsigned gy) {
  simt::run_threadgroup(128, [&](unsigned tid) {
    attn_decode_gqa<G>(reinterpret_cast<const half*>(a.Q), reinterpret_cast<const half*>(a.Kb), reinterpret_cast<const half*>(a.Vb),
                       reinterpret_cast<const half*>(a.kv), a.blocks, reinterpret_cast<const int4*>(a.desc), a.X, reinterpret_cast<half*>(a.O), *a.p, a.tiles,
                       a.trees, a.parts, uint2(gx, gy), tid / 32, tid % 32);
  });
}

}  // namespace

extern "C" {

// flash_attention<G> (kernels/40_attention.metal:156-343) over grid (Hkv, n_tiles), 64 * G threads per threadgroup.
// which: 0 flash_attention, 1 attn_decode_gqa (:598-781; grid (Hkv, n_tiles), 128 threads). Returns -1 for a G the
// reference does not instantiate (1, 2, 3, 4, 6, 8).
int ref_attention(int which, int G, const uint16_t* Q, const uint16_t* Kb, const uint16_t* Vb, const uint16_t* kv, const int32_t* blocks,
                  const int32_t* desc, const float* X, uint16_t* O, const AttnParams* p, const AttnTile* tiles, int n_tiles, const AttnTree* trees,
                  float* parts) {
  const AttnArgs a{Q, Kb, Vb, kv, blocks, desc, X, O, p, tiles, trees, parts};
  for (unsigned y = 0; y < unsigned(n_tiles); ++y)
    for (unsigned x = 0; x < unsigned(p->Hkv); ++x) {
      if (which == 0) {
        switch (G) {
          case 1: flash_group<1>(a, x, y); break;
          case 2: flash_group<2>(a, x, y); break;
          case 3: flash_group<3>(a, x, y); break;
          case 4: flash_group<4>(a, x, y); break;
          case 6: flash_group<6>(a, x, y); break;
          case 8: flash_group<8>(a, x, y); break;
          default: return -1;
        }
      } else {
        switch (G) {
          case 1: decode_group<1>(a, x, y); break;
          case 2: decode_group<2>(a, x, y); break;
          case 3: decode_group<3>(a, x, y); break;
          case 4: decode_group<4>(a, x, y); break;
          case 6: decode_group<6>(a, x, y); break;
          case 8: decode_group<8>(a, x, y); break;
          default: return -1;
        }
      }
    }
  return 0;
}

// attn_prep (kernels/40_attention.metal:23-102) over grid ((H + Hkv + 3) / 4, rows), 128 threads (forest.h:2976).
void ref_attn_prep(const float* X, const float* qn_w, const float* kn_w, const int32_t* pos, const float* inv_freq, uint16_t* Q, uint16_t* Kb,
                   uint16_t* Vb, const AttnPrepParams* p, const int32_t* rope_sel, const int32_t* ktab, uint16_t* kv, int rows) {
  for (unsigned y = 0; y < unsigned(rows); ++y)
    for (unsigned x = 0; x < unsigned(p->H + p->Hkv + 3) / 4; ++x)
      simt::run_threadgroup(128, [&](unsigned tid) {
        attn_prep(X, qn_w, kn_w, reinterpret_cast<const int4*>(pos), inv_freq, reinterpret_cast<half*>(Q), reinterpret_cast<half*>(Kb),
                  reinterpret_cast<half*>(Vb), *p, rope_sel, reinterpret_cast<const int4*>(ktab), reinterpret_cast<half*>(kv), uint2(x, y), tid / 32,
                  tid % 32);
      });
}


// ---- Qwen sparse attention (kernels/45_qsa.metal:281-690; host dispatch src/model/impl/forest.h:1586-1644)
// qsa_select: one threadgroup of 1024 threads per sparse row; qsa_tiles: one of 256 per tile.
void ref_qsa_select(const float* scores, const int32_t* srows, const int32_t* rinfo, uint32_t* sel, const QsaParams* p, int n_sparse) {
  for (unsigned g = 0; g < unsigned(n_sparse); ++g)
    simt::run_threadgroup(1024, [&](unsigned tid) { qsa_select(scores, srows, reinterpret_cast<const int4*>(rinfo), sel, *p, g, tid, tid / 32, tid % 32); });
}
void ref_qsa_tiles(const uint32_t* sel, const AttnTree* trees, const int32_t* rinfo, const QsaTile* qtiles, int n_qtiles, uint32_t* tlist, uint32_t* tcount,
                   const QsaParams* p) {
  for (unsigned g = 0; g < unsigned(n_qtiles); ++g)
    simt::run_threadgroup(256, [&](unsigned tid) { qsa_tiles(sel, trees, reinterpret_cast<const int4*>(rinfo), qtiles, tlist, tcount, *p, g, tid, tid / 32, tid % 32); });
}
// flash_attention_qsa<G> over grid (Hkv, n_tiles), 64 * G threads per threadgroup.
int ref_attention_qsa(int G, const uint16_t* Q, const uint16_t* Kb, const uint16_t* Vb, const uint16_t* kv, const int32_t* blocks, const int32_t* desc,
                      const float* X, uint16_t* O, const AttnParams* p, const AttnTile* tiles, int n_tiles, const AttnTree* trees, float* parts,
                      const uint32_t* tlist, const uint32_t* tcount, const int32_t* rinfo, const uint32_t* sel, const QsaParams* qp) {
  auto group = [&](auto g_tag, unsigned gx, unsigned gy) {
    constexpr int GG = decltype(g_tag)::value;
    simt::run_threadgroup(64 * GG, [&](unsigned tid) {
      flash_attention_qsa<GG, 1>(reinterpret_cast<const half*>(Q), reinterpret_cast<const half*>(Kb), reinterpret_cast<const half*>(Vb),
                                 reinterpret_cast<const half*>(kv), blocks, reinterpret_cast<const int4*>(desc), X, reinterpret_cast<half*>(O), *p, tiles,
                                 trees, parts, tlist, tcount, reinterpret_cast<const int4*>(rinfo), sel, *qp, uint2(gx, gy), tid, tid / 32, tid % 32);
    });
  };
  for (unsigned y = 0; y < unsigned(n_tiles); ++y)
    for (unsigned x = 0; x < unsigned(p->Hkv); ++x) switch (G) {
        case 1: group(std::integral_constant<int, 1>{}, x, y); break;
        case 2: group(std::integral_constant<int, 2>{}, x, y); break;
        case 4: group(std::integral_constant<int, 4>{}, x, y); break;
        case 6: group(std::integral_constant<int, 6>{}, x, y); break;
        case 8: group(std::integral_constant<int, 8>{}, x, y); break;
        default: return -1;
      }
  return 0;
}

}  // extern "C"
