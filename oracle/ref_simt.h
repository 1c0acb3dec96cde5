// TEST INFRASTRUCTURE: a small SIMT emulator and the Metal vocabulary the reference's attention kernels
// use, so that their source - cut from the reference tree by extract_ref.py, attributes removed, nothing
// else changed - compiles as C++ and runs on the CPU. Every GPU thread is a fiber (ucontext) of one OS
// thread; a threadgroup runs to completion before the next one starts. threadgroup_barrier, simd_shuffle_xor,
// simd_sum and simdgroup_multiply_accumulate are rendezvous points: a fiber that reaches one deposits its
// operand and yields until all fibers of the scope have arrived.
//
// What the emulation fixes that Metal leaves to the hardware: an 8x8 simdgroup matrix keeps element
// (row, column) in lane / slot of thread_elements() the way the kernels themselves assume (row = (lane / 4 & 4)
// + (lane / 2) % 4, columns (lane / 4 & 2) * 2 + (lane % 2) * 2 + {0, 1}: the `fm` / `fn` of
// kernels/40_attention.metal:184-185); a matrix product sums its 8 terms in index order in fp32 (the
// hardware's order is not documented; fp16 products are exact in fp32, so only the order of seven additions
// is a choice); exp / rsqrt / sin / cos are libm's single-precision functions (Metal's fast-math variants
// differ in the last bits). Results are therefore the reference kernels' up to fp32 rounding noise.
#pragma once

#include <ucontext.h>

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <vector>

namespace simt {

constexpr int kSimd = 32;
constexpr size_t kStackBytes = 64 * 1024;  // per fiber; the largest threadgroup (qsa_select) has 1024

struct Fiber {
  ucontext_t ctx;
  char* stack = nullptr;
  bool done = true;
  unsigned tid = 0;
};

// One threadgroup in flight on this OS thread.
struct Group {
  std::vector<Fiber> fibers;
  ucontext_t scheduler;
  int current = -1;
  int live = 0;                    // fibers that have not returned
  // threadgroup barrier
  int bar_count = 0;
  unsigned bar_gen = 0;
  // per-simdgroup rendezvous: arrival count, generation, two operand buffers (alternating by generation)
  struct Simd {
    int count = 0, live = 0;
    unsigned gen = 0;
    float slot[2][kSimd][4];
  };
  std::vector<Simd> simds;
  std::function<void(unsigned tid)> body;
};

inline thread_local Group* g_group = nullptr;

inline void yield() {
  Group& g = *g_group;
  swapcontext(&g.fibers[size_t(g.current)].ctx, &g.scheduler);
}

inline void fiber_entry() {
  Group& g = *g_group;
  Fiber& f = g.fibers[size_t(g.current)];
  g.body(f.tid);
  f.done = true;
  --g.live;
  --g.simds[f.tid / kSimd].live;
  // a fiber that leaves may complete a rendezvous the others are waiting at
  swapcontext(&f.ctx, &g.scheduler);
}

// Runs `body(tid)` for tid in [0, n_threads) as one threadgroup.
inline void run_threadgroup(unsigned n_threads, std::function<void(unsigned)> body) {
  static thread_local Group g;
  static thread_local std::vector<char*> stacks;
  g_group = &g;
  g.body = std::move(body);
  g.fibers.resize(n_threads);
  while (stacks.size() < n_threads) stacks.push_back(static_cast<char*>(std::malloc(kStackBytes)));
  g.simds.assign((n_threads + kSimd - 1) / kSimd, Group::Simd());
  g.bar_count = 0, g.live = int(n_threads);
  for (unsigned t = 0; t < n_threads; ++t) {
    Fiber& f = g.fibers[t];
    f.stack = stacks[t], f.done = false, f.tid = t;
    getcontext(&f.ctx);
    f.ctx.uc_stack.ss_sp = f.stack, f.ctx.uc_stack.ss_size = kStackBytes, f.ctx.uc_link = nullptr;
    makecontext(&f.ctx, fiber_entry, 0);
    ++g.simds[t / kSimd].live;
  }
  while (g.live > 0) {
    for (unsigned t = 0; t < n_threads; ++t) {
      if (g.fibers[t].done) continue;
      g.current = int(t);
      swapcontext(&g.scheduler, &g.fibers[t].ctx);
    }
  }
  g_group = nullptr;
}

inline unsigned this_tid() { return g_group->fibers[size_t(g_group->current)].tid; }

inline void barrier_threadgroup() {
  Group& g = *g_group;
  const unsigned gen = g.bar_gen;
  if (++g.bar_count >= g.live) {
    g.bar_count = 0;
    ++g.bar_gen;
    return;
  }
  while (g.bar_gen == gen) {
    if (g.bar_count >= g.live) {  // the missing fibers have returned meanwhile
      g.bar_count = 0;
      ++g.bar_gen;
      return;
    }
    yield();
  }
}

// Rendezvous of a simdgroup: deposits `n` floats, returns the buffer holding every lane's deposit.
inline const float (*exchange(const float* mine, int n))[4] {
  Group& g = *g_group;
  const unsigned tid = this_tid();
  Group::Simd& s = g.simds[tid / kSimd];
  const unsigned gen = s.gen;
  float(*buf)[4] = s.slot[gen & 1];
  for (int i = 0; i < n; ++i) buf[tid % kSimd][i] = mine[i];
  if (++s.count >= s.live) {
    s.count = 0;
    ++s.gen;
    return buf;
  }
  while (s.gen == gen) {
    if (s.count >= s.live) {
      s.count = 0;
      ++s.gen;
      break;
    }
    yield();
  }
  return buf;
}

}  // namespace simt

// ---------------------------------------------------------------- Metal vocabulary
namespace metal_emu {

using uint = unsigned int;
using ulong = unsigned long long;
using ushort = unsigned short;
using uchar = unsigned char;
using half = _Float16;

template <class T, int N>
struct vec;
template <class T>
struct vec<T, 2> {
  T x, y;
  vec() = default;
  vec(T a, T b) : x(a), y(b) {}
  explicit vec(T s) : x(s), y(s) {}
  template <class U>
  explicit vec(const vec<U, 2>& o) : x(T(o.x)), y(T(o.y)) {}
  T& operator[](int i) { return (&x)[i]; }
  const T& operator[](int i) const { return (&x)[i]; }
};
template <class T>
struct vec<T, 3> {
  T x, y, z;
  vec() = default;
  vec(T a, T b, T c) : x(a), y(b), z(c) {}
};
template <class T>
struct vec<T, 4> {
  T x, y, z, w;
  vec() = default;
  vec(T a, T b, T c, T d) : x(a), y(b), z(c), w(d) {}
  explicit vec(T s) : x(s), y(s), z(s), w(s) {}
  template <class U>
  explicit vec(const vec<U, 4>& o) : x(T(o.x)), y(T(o.y)), z(T(o.z)), w(T(o.w)) {}
  T& operator[](int i) { return (&x)[i]; }
  const T& operator[](int i) const { return (&x)[i]; }
};
using half2 = vec<half, 2>;
using half4 = vec<half, 4>;
using float2 = vec<float, 2>;
using float4 = vec<float, 4>;
using int2 = vec<int, 2>;
using int4 = vec<int, 4>;
using uint2 = vec<uint, 2>;
using uint3 = vec<uint, 3>;
using uint4 = vec<uint, 4>;

inline half2 operator*(const half2& a, half s) { return half2(half(a.x * s), half(a.y * s)); }
inline float4 operator*(const float4& v, float s) { return {v.x * s, v.y * s, v.z * s, v.w * s}; }
inline float4 operator*(float s, const float4& v) { return {s * v.x, s * v.y, s * v.z, s * v.w}; }
inline float4 operator+(float s, const float4& v) { return {s + v.x, s + v.y, s + v.z, s + v.w}; }
inline float4 operator/(const float4& a, const float4& b) { return {a.x / b.x, a.y / b.y, a.z / b.z, a.w / b.w}; }
inline float4 operator-(const float4& v) { return {-v.x, -v.y, -v.z, -v.w}; }
inline float4& operator+=(float4& a, const float4& b) {
  a.x += b.x, a.y += b.y, a.z += b.z, a.w += b.w;
  return a;
}
inline float4 exp(const float4& v) { return {std::exp(v.x), std::exp(v.y), std::exp(v.z), std::exp(v.w)}; }
inline float exp(float v) { return std::exp(v); }
inline float rsqrt(float v) { return 1.0f / std::sqrt(v); }
inline float fma(float a, float b, float c) { return std::fma(a, b, c); }
inline float fabs(float v) { return std::fabs(v); }
inline float rint(float v) { return std::nearbyint(v); }
inline float copysign(float a, float b) { return std::copysign(a, b); }
namespace precise {
inline float cos(float v) { return std::cos(v); }
inline float sin(float v) { return std::sin(v); }
}  // namespace precise
template <class T>
inline T min(T a, T b) { return b < a ? b : a; }
template <class T>
inline T max(T a, T b) { return a < b ? b : a; }
inline int min(int a, short b) { return b < a ? int(b) : a; }
inline int min(short a, int b) { return b < a ? b : int(a); }

template <class To, class From>
inline To as_type(const From& f) {
  static_assert(sizeof(To) == sizeof(From), "as_type: same size");
  To t;
  std::memcpy(&t, &f, sizeof(To));
  return t;
}

enum class mem_flags { mem_none, mem_device, mem_threadgroup };
inline void threadgroup_barrier(mem_flags) { simt::barrier_threadgroup(); }

inline float simd_shuffle_xor(float v, ushort mask) {
  const float(*all)[4] = simt::exchange(&v, 1);
  return all[(simt::this_tid() % simt::kSimd) ^ mask][0];
}
inline float simd_sum(float v) {
  const float(*all)[4] = simt::exchange(&v, 1);
  float s = 0.0f;
  for (int l = 0; l < simt::kSimd; ++l) s += all[l][0];  // lane order (the hardware's reduction tree is not documented)
  return s;
}

inline uint simd_prefix_inclusive_sum(uint v) {
  const float f = as_type<float>(v);  // the exchange carries 32-bit patterns
  const float(*all)[4] = simt::exchange(&f, 1);
  uint s = 0;
  for (unsigned l = 0; l <= simt::this_tid() % simt::kSimd; ++l) s += as_type<uint>(all[l][0]);
  return s;
}
inline uint simd_prefix_exclusive_sum(uint v) { return simd_prefix_inclusive_sum(v) - v; }
inline uint popcount(uint v) { return uint(__builtin_popcount(v)); }
inline uint ctz(uint v) { return uint(__builtin_ctz(v)); }
template <class T>
inline T clamp(T v, T lo, T hi) { return v < lo ? lo : (hi < v ? hi : v); }

// threadgroup atomics: the fibers of a group run one at a time, so plain memory is atomic enough
struct atomic_uint {
  uint v;
};
enum memory_order { memory_order_relaxed };
inline void atomic_store_explicit(atomic_uint* a, uint v, memory_order) { a->v = v; }
inline uint atomic_load_explicit(const atomic_uint* a, memory_order) { return a->v; }
inline uint atomic_fetch_add_explicit(atomic_uint* a, uint v, memory_order) {
  const uint old = a->v;
  a->v += v;
  return old;
}

// 8 x 8 matrix spread over the 32 lanes, two elements per lane.
template <class T, int R, int C>
struct simdgroup_matrix {
  static_assert(R == 8 && C == 8, "8 x 8 only");
  T e[2];
  T* thread_elements() { return e; }
  const T* thread_elements() const { return e; }
};
template <class T, int R, int C>
inline simdgroup_matrix<T, R, C> make_filled_simdgroup_matrix(T v) {
  simdgroup_matrix<T, R, C> m;
  m.e[0] = m.e[1] = v;
  return m;
}
inline int lane_row(int lane) { return ((lane / 4) & 4) + ((lane / 2) % 4); }
inline int lane_col(int lane) { return ((lane / 4) & 2) * 2 + (lane % 2) * 2; }
struct LaneOf {
  int lane[8][8], slot[8][8];
  LaneOf() {
    for (int l = 0; l < 32; ++l)
      for (int e = 0; e < 2; ++e) lane[lane_row(l)][lane_col(l) + e] = l, slot[lane_row(l)][lane_col(l) + e] = e;
  }
};
inline const LaneOf& lane_of() {
  static const LaneOf t;
  return t;
}
// D = A * B + C: products exact in fp32 (fp16 operands), the 8 terms of an element added in index order onto C.
template <class TA, class TB>
inline void simdgroup_multiply_accumulate(simdgroup_matrix<float, 8, 8>& D, const simdgroup_matrix<TA, 8, 8>& A,
                                          const simdgroup_matrix<TB, 8, 8>& B, const simdgroup_matrix<float, 8, 8>& Cm) {
  const float mine[4] = {float(A.e[0]), float(A.e[1]), float(B.e[0]), float(B.e[1])};
  const float(*all)[4] = simt::exchange(mine, 4);
  const LaneOf& t = lane_of();
  const int lane = int(simt::this_tid() % simt::kSimd), r = lane_row(lane), c0 = lane_col(lane);
  float out[2];
  for (int e = 0; e < 2; ++e) {
    float acc = Cm.e[e];
    for (int k = 0; k < 8; ++k) acc += all[t.lane[r][k]][t.slot[r][k]] * all[t.lane[k][c0 + e]][2 + t.slot[k][c0 + e]];
    out[e] = acc;
  }
  D.e[0] = out[0], D.e[1] = out[1];
}

}  // namespace metal_emu
