// The device header library compiled by a plain C++17 compiler: tile arithmetic, address
// translation, context decoding and the bounded wait, checked with ordinary assertions.
// Built and run by tests/test_cpu_device_headers.py; exits 0 when every check holds and prints the
// failed expression otherwise.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <chrono>
#include <set>
#include <thread>
#include <utility>
#include <vector>

#include "iris/iris.cuh"

namespace iris {
uint64_t now_ns() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
void backoff(unsigned ns) {
  if (ns >= 1000) std::this_thread::sleep_for(std::chrono::nanoseconds(ns));
  else std::this_thread::yield();
}
}  // namespace iris

using namespace iris;

static int failures = 0;
#define CHECK(expr)                                                   \
  do {                                                                \
    if (!(expr)) {                                                    \
      ++failures;                                                     \
      printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #expr);        \
    }                                                                 \
  } while (0)

static void tile_views() {
  float data[6 * 10];
  for (int i = 0; i < 60; ++i) data[i] = (float)i;
  TensorView<float> v = make_tensor_view(data, 6, 10, 10);
  TileView t{1, 2, 4, 3};
  CHECK(t.row0() == 4 && t.col0() == 6);
  CHECK(*v.at(2, 3) == 23.0f);
  CHECK(v.tile_ptr(t) == data + 46);
  CHECK(v.tile_ptr_from_indices(1, 2, 4, 3) == v.tile_ptr(t));
  CHECK(v.number_of_tiles(4, 3) == 2 * 4);
  CHECK(v.number_of_tiles(6, 10) == 1 && v.number_of_tiles(1, 1) == 60);
  CHECK(v.in_bounds(5, 9) && !v.in_bounds(6, 0) && !v.in_bounds(0, 10));
  TensorView<float> o = v.offset(2, 4);
  CHECK(o.M == 4 && o.N == 6 && *o.at(0, 0) == 24.0f && o.stride_m == 10);
  // column-major window through the strides
  TensorView<float> cm = make_tensor_view(data, 10, 6, 1, 10);
  CHECK(*cm.at(3, 2) == 23.0f);
  AllReduceConfig cfg{3, nullptr};
  CHECK(cfg.variant_code == 3);
}

static void tile_order() {
  // the swizzled order visits every tile exactly once, walks group_size_m rows before it moves
  // one column on, and the chiplet remap is the identity
  const int shapes[][3] = {{1, 1, 1}, {4, 4, 1}, {4, 4, 4}, {7, 5, 3}, {16, 3, 8}, {5, 9, 6}, {3, 3, 16}};
  for (auto& s : shapes) {
    const int pm = s[0], pn = s[1], g = s[2];
    std::set<std::pair<int, int>> seen;
    for (int id = 0; id < pm * pn; ++id) {
      int m = -1, n = -1;
      compute_tile_indices(id, pm, pn, g, m, n);
      CHECK(m >= 0 && m < pm && n >= 0 && n < pn);
      seen.insert({m, n});
      CHECK(chiplet_transform_chunked(id, pm * pn, 8, 2) == id);
    }
    CHECK((int)seen.size() == pm * pn);
    int m0, n0, m1, n1;
    compute_tile_indices(0, pm, pn, g, m0, n0);
    CHECK(m0 == 0 && n0 == 0);
    if (pm > 1 && g > 1) {
      compute_tile_indices(1, pm, pn, g, m1, n1);
      CHECK(m1 == 1 && n1 == 0);      // down the group first
    }
    if (g == 1 && pn > 1) {
      compute_tile_indices(1, pm, pn, g, m1, n1);
      CHECK(m1 == 0 && n1 == 1);      // group of one row: plain row-major
    }
  }
}

static void translation() {
  // three "ranks": three windows of one buffer
  static int32_t heap[3][64];
  int64_t words[2 + 3 + 17];
  memset(words, 0, sizeof(words));
  words[0] = 1;
  words[1] = 3;
  for (int r = 0; r < 3; ++r) words[2 + r] = (int64_t)(uintptr_t)heap[r];
  DeviceContext ctx = DeviceContext::initialize(words);
  CHECK(ctx.rank == 1 && ctx.world == 3 && ctx.trace.enabled == 0);
  CHECK(ctx.bases[0] == (uint64_t)(uintptr_t)heap[0] && ctx.bases[2] == (uint64_t)(uintptr_t)heap[2]);
  int32_t* mine = &heap[1][10];
  CHECK(ctx.remote(mine, 0) == &heap[0][10] && ctx.remote(mine, 2) == &heap[2][10] && ctx.remote(mine, 1) == mine);
  CHECK(ctx.translate(&heap[2][5], 2, 0) == &heap[0][5]);
  CHECK(translate(mine, 1, 2, ctx.bases) == &heap[2][10]);
  ctx.heap_size = sizeof(heap[0]);
  CHECK(ctx.in_heap(&heap[1][63], 1) && !ctx.in_heap(&heap[1][63] + 1, 1) && !ctx.in_heap(&heap[0][0], 1));
  // tracing words are decoded only when asked for
  words[2 + 3] = 1;
  words[2 + 3 + 1] = 128;
  CHECK(DeviceContext::initialize(words).trace.enabled == 0);
  DeviceContext traced = DeviceContext::initialize(words, true);
  CHECK(traced.trace.enabled == 1 && traced.trace.max_events == 128);

  // the functional API: same argument order as the reference (load: to_rank, from_rank; the rest: from, to)
  for (int r = 0; r < 3; ++r)
    for (int i = 0; i < 64; ++i) heap[r][i] = 100 * r + i;
  CHECK(load(mine, 1, 2, ctx.bases) == 210);
  store(mine, 7, 1, 0, ctx.bases);
  CHECK(heap[0][10] == 7 && heap[1][10] == 110);
  get(&heap[1][3], &heap[1][4], 2, 1, ctx.bases);     // remote read of rank 2 into my memory
  CHECK(heap[1][4] == 203);
  put(&heap[1][5], &heap[1][6], 1, 2, ctx.bases);     // my value into rank 2
  CHECK(heap[2][6] == 105);
  copy(&heap[1][20], &heap[1][21], 0, 2, 1, ctx.bases);   // rank 0 -> rank 2, called from rank 1
  CHECK(heap[2][21] == 20);
  store(mine, 9, 1, 0, ctx.bases, false);             // predicate off: nothing happens
  CHECK(heap[0][10] == 7);
  CHECK(load(mine, 1, 2, ctx.bases, false) == 0);     // masked load returns the default
  Ctx c(ctx);
  c.store(mine, 55, 2);
  CHECK(heap[2][10] == 55 && c.load(mine, 2) == 55);
  CHECK((atomic_add<Sem::acq_rel, Scope::sys>(mine, 5, 1, 2, ctx.bases)) == 55 && heap[2][10] == 60);
  CHECK((atomic_cas<Sem::acq_rel, Scope::sys>(mine, 60, 1, 1, 2, ctx.bases)) == 60 && heap[2][10] == 1);
  CHECK((atomic_cas<Sem::acq_rel, Scope::sys>(mine, 60, 2, 1, 2, ctx.bases)) == 1 && heap[2][10] == 1);
  CHECK((atomic_xchg<Sem::release, Scope::sys>(mine, 3, 1, 2, ctx.bases)) == 1 && heap[2][10] == 3);
  CHECK((atomic_max<Sem::relaxed, Scope::gpu>(mine, 9, 1, 2, ctx.bases)) == 3 && heap[2][10] == 9);
  CHECK((atomic_min<Sem::relaxed, Scope::cta>(mine, 4, 1, 2, ctx.bases)) == 9 && heap[2][10] == 4);
  CHECK((atomic_or<Sem::acquire, Scope::sys>(mine, 3, 1, 2, ctx.bases)) == 4 && heap[2][10] == 7);
  CHECK((atomic_and<Sem::acquire, Scope::sys>(mine, 5, 1, 2, ctx.bases)) == 7 && heap[2][10] == 5);
  CHECK((atomic_xor<Sem::acquire, Scope::sys>(mine, 1, 1, 2, ctx.bases)) == 5 && heap[2][10] == 4);
  CHECK((atomic_sub<Sem::acq_rel, Scope::sys>(mine, 4, 1, 2, ctx.bases)) == 4 && heap[2][10] == 0);
}

static void bounded_waits() {
  int32_t flag = 0, status = 0;
  DeviceContext ctx;
  memset(&ctx, 0, sizeof(ctx));
  ctx.world = 1;
  ctx.status = &status;
  ctx.timeout_ns = 20ull * 1000 * 1000;                 // 20 ms
  const uint64_t t0 = now_ns();
  CHECK(!wait_flag_ge(ctx, &flag, 1));                  // nothing sets the flag: gives up, records why
  const uint64_t waited = now_ns() - t0;
  CHECK(waited >= 15ull * 1000 * 1000 && waited < 2000ull * 1000 * 1000);
  CHECK(status == kTimeoutFlag);
  ctx.fail(kTimeoutBarrier);
  CHECK(status == kTimeoutFlag);                        // the first failure is kept
  status = 0;
  flag = 3;
  CHECK(wait_flag_ge(ctx, &flag, 3) && wait_flag_ge(ctx, &flag, 1) && status == 0);
  CHECK(!wait_flag_ge_limit(&flag, 4, 5ull * 1000 * 1000) && status == 0);   // the plain form records nothing
  // a flag set by another thread ends the wait early
  flag = 0;
  ctx.timeout_ns = 5000ull * 1000 * 1000;
  std::thread setter([&] {
    std::this_thread::sleep_for(std::chrono::milliseconds(10));
    st_release_sys(&flag, 1);
  });
  const uint64_t t1 = now_ns();
  CHECK(wait_flag_ge(ctx, &flag, 1));
  CHECK(now_ns() - t1 < 2000ull * 1000 * 1000);
  setter.join();
  // a barrier round between two "ranks" (two windows of one array), driven from one thread
  static SyncBlock blocks[2];
  memset(blocks, 0, sizeof(blocks));
  DeviceContext r0 = ctx, r1 = ctx;
  r0.world = r1.world = 2;
  r0.rank = 0;
  r1.rank = 1;
  r0.bases[0] = r1.bases[0] = (uint64_t)(uintptr_t)&blocks[0];
  r0.bases[1] = r1.bases[1] = (uint64_t)(uintptr_t)&blocks[1];
  r0.timeout_ns = r1.timeout_ns = 20ull * 1000 * 1000;
  status = 0;
  barrier_signal(r0, &blocks[0]);                       // rank 0 arrives: its slot in rank 1's block counts up
  CHECK(blocks[1].slots[0] == 1 && blocks[0].slots[1] == 0);
  CHECK(barrier_wait(r1, &blocks[1], 1) && status == 0);   // rank 1 sees rank 0
  CHECK(!barrier_wait(r0, &blocks[0], 1) && status == kTimeoutBarrier);   // rank 1 never signalled: bounded, recorded
  status = 0;
  barrier_signal(r1, &blocks[1]);
  CHECK(barrier_wait(r0, &blocks[0], 1) && status == 0);
}

// Object API in a debug build: accesses outside the heap or to a rank that does not exist are
// skipped and recorded; in a regular build the same calls are plain accesses (so they are only made
// here when the macro is set).
static void debug_bounds() {
  static int32_t heap[2][32];
  static int32_t outside[4];
  int32_t status = 0;
  DeviceContext ctx;
  memset(&ctx, 0, sizeof(ctx));
  ctx.rank = 0;
  ctx.world = 2;
  ctx.heap_size = sizeof(heap[0]);
  ctx.status = &status;
  ctx.bases[0] = (uint64_t)(uintptr_t)heap[0];
  ctx.bases[1] = (uint64_t)(uintptr_t)heap[1];
  Ctx c(ctx);
  c.store(&heap[0][3], 11, 1);
  CHECK(heap[1][3] == 11 && status == 0);               // a proper access is unaffected
  CHECK(c.ok(&heap[0][31], 1));
#if defined(IRIS_DEBUG)
  outside[0] = 5;
  c.store(outside, 99, 1);                              // not a heap pointer: skipped, recorded
  CHECK(outside[0] == 5 && status == kBadTranslate);
  status = 0;
  c.store(&heap[0][3], 12, 2);                          // rank 2 does not exist
  CHECK(heap[1][3] == 11 && status == kBadTranslate);
  status = 0;
  CHECK(c.load(&heap[0][3], -1, true, 77) == 77 && status == kBadTranslate);   // masked out: the default comes back
  status = 0;
  CHECK((c.atomic_add<Sem::relaxed, Scope::sys>(&heap[0][32], 1, 1)) == 0 && status == kBadTranslate);   // one past the end
  status = 0;
  CHECK((c.atomic_cas<Sem::relaxed, Scope::sys>(outside, 5, 6, 1)) == 5 && outside[0] == 5 && status == kBadTranslate);
  status = 0;
  c.put(&heap[0][1], outside, 1);
  c.get(outside, &heap[0][1], 1);
  c.copy(&heap[0][1], outside, 0, 1);
  CHECK(outside[0] == 5 && status == kBadTranslate);
  printf("debug bounds checks active\n");
#else
  CHECK(c.ok(outside, 7));                              // the regular build tests nothing
#endif
}

int main() {
  debug_bounds();
  tile_views();
  tile_order();
  translation();
  bounded_waits();
  if (failures) {
    printf("%d check(s) failed\n", failures);
    return 1;
  }
  printf("all host header checks passed\n");
  return 0;
}
