// Cooperative-fiber threadgroup for the CPU build of the reference's shaders (test infrastructure).
#include "metal_shim.h"

namespace simt {

static State g_state;
State& state() { return g_state; }

void yield() {
  State& s = g_state;
  swapcontext(&s.lane[s.cur], &s.sched);
}

void barrier() {
  State& s = g_state;
  const unsigned g = s.gen;
  if (++s.arrived == s.live) {
    s.arrived = 0;
    ++s.gen;
    return;
  }
  while (s.gen == g) yield();
}

// every lane of the threadgroup calls this together (uniform control flow in both shaders)
float simd_sum(float v) {
  State& s = g_state;
  const int lane = s.cur;
  s.slots[lane] = v;
  barrier();
  const int base = lane / 32 * 32;
  float acc = 0.f;
  for (int i = 0; i < 32 && base + i < s.n; ++i) acc += s.slots[base + i];
  barrier();
  return acc;
}

static void trampoline(int lane) {
  State& s = g_state;
  s.body(lane);
  s.done[lane] = true;
  --s.live;
  // lanes that wait at a barrier must not wait for a lane that has left
  if (s.live > 0 && s.arrived == s.live) {
    s.arrived = 0;
    ++s.gen;
  }
}

void run_threadgroup(int n, void (*body)(int)) {
  State& s = g_state;
  constexpr size_t STACK = 256 * 1024;
  static char* stacks = nullptr;
  if (!stacks) stacks = static_cast<char*>(std::malloc(STACK * MAX_LANES));
  s.n = n;
  s.live = n;
  s.arrived = 0;
  s.body = body;
  for (int i = 0; i < n; ++i) {
    s.done[i] = false;
    getcontext(&s.lane[i]);
    s.lane[i].uc_stack.ss_sp = stacks + STACK * i;
    s.lane[i].uc_stack.ss_size = STACK;
    s.lane[i].uc_link = &s.sched;   // a lane that returns comes back to the scheduler
    makecontext(&s.lane[i], reinterpret_cast<void (*)()>(trampoline), 1, i);
  }
  while (s.live > 0) {
    for (int i = 0; i < n; ++i) {
      if (s.done[i]) continue;
      s.cur = i;
      swapcontext(&s.sched, &s.lane[i]);
    }
  }
}

}  // namespace simt
