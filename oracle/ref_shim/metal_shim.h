// Test infrastructure only: a small stand-in for <metal_stdlib> so that two of the reference's
// compute shaders (src/shaders/attn/attention/attention.metal and
// src/shaders/attn/qk_rope_kv/qk_rope_kv.metal, with the headers they include) compile UNMODIFIED as
// C++ and run on the CPU, one threadgroup at a time.  Address-space qualifiers become nothing,
// `threadgroup` arrays inside a kernel become statics shared by the lanes, the lanes of a threadgroup
// are cooperative fibers (ucontext) that meet at threadgroup_barrier / simd_sum.  Nothing of the
// product links this.
#pragma once
#include <ucontext.h>

#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>

typedef unsigned int uint;
typedef unsigned short ushort;
typedef unsigned char uchar;
typedef unsigned long ulong;
typedef _Float16 half;

#define device
#define constant
#define thread
#define threadgroup
#define kernel
#define is_function_constant_defined(x) false

struct uint2 {
  uint x, y;
};
struct uint3 {
  uint x, y, z;
};
struct float4 {
  float x, y, z, w;
  float4() = default;
  float4(float a, float b, float c, float d) : x(a), y(b), z(c), w(d) {}
};
struct char4 {
  signed char x, y, z, w;
};
struct half4 {
  half x, y, z, w;
  half4() = default;
  explicit half4(const float4& f) : x(half(f.x)), y(half(f.y)), z(half(f.z)), w(half(f.w)) {}
  half4 operator*(half s) const {
    half4 r;
    r.x = x * s; r.y = y * s; r.z = z * s; r.w = w * s;
    return r;
  }
};

namespace simt {
// lanes of the threadgroup that is running
constexpr int MAX_LANES = 64;
struct State {
  ucontext_t sched;
  ucontext_t lane[MAX_LANES];
  bool done[MAX_LANES];
  int n = 0, cur = 0, live = 0, arrived = 0;
  unsigned gen = 0;
  float slots[MAX_LANES];
  void (*body)(int) = nullptr;
};
State& state();
void yield();
void barrier();
float simd_sum(float v);
// runs body(lane) for lane in [0, n) as fibers until all have returned
void run_threadgroup(int n, void (*body)(int));
}  // namespace simt

namespace metal {
using std::atomic_compare_exchange_weak_explicit;
using std::atomic_store_explicit;
using std::memory_order_relaxed;
typedef std::atomic<unsigned int> atomic_uint;
enum class mem_flags { mem_none, mem_device, mem_threadgroup };
inline void threadgroup_barrier(mem_flags) { simt::barrier(); }
inline float simd_sum(float v) { return simt::simd_sum(v); }
template <class T, class U>
inline T as_type(U u) {
  static_assert(sizeof(T) == sizeof(U), "as_type needs equal sizes");
  T t;
  std::memcpy(&t, &u, sizeof(T));
  return t;
}
inline float min(float a, float b) { return std::fmin(a, b); }
inline float max(float a, float b) { return std::fmax(a, b); }
inline uint min(uint a, uint b) { return a < b ? a : b; }
inline uint max(uint a, uint b) { return a > b ? a : b; }
inline float clamp(float x, float lo, float hi) { return std::fmin(std::fmax(x, lo), hi); }
inline float exp(float x) { return std::exp(x); }
inline float pow(float a, float b) { return std::pow(a, b); }
inline float cos(float x) { return std::cos(x); }
inline float sin(float x) { return std::sin(x); }
inline float fabs(float x) { return std::fabs(x); }
inline float rint(float x) { return std::nearbyint(x); }
inline float rsqrt(float x) { return 1.0f / std::sqrt(x); }
inline bool isnan(float x) { return std::isnan(x); }
inline bool isinf(float x) { return std::isinf(x); }
}  // namespace metal
