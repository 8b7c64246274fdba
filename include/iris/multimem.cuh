// NVLS (NVLink SHARP) access to the multicast mapping of the symmetric heap: one instruction that
// the NVSwitch fans out to (st / red) or reduces from (ld_reduce) every rank's copy of the same
// heap offset. Addresses are DeviceContext::mc(ptr). This is a switch-side operation issued by an
// ordinary SM instruction; it has nothing to do with cluster-multicast TMA loads.
#pragma once
#include "common.cuh"
#if defined(__CUDACC__)
namespace iris {
namespace multimem {

struct alignas(16) V4 { uint32_t x, y, z, w; };

// Broadcast store of 16 bytes to the same offset on every rank.
IRIS_D void st_v4(void* mc_ptr, V4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_ptr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
IRIS_D void st_u32(void* mc_ptr, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(mc_ptr), "r"(v) : "memory");
}
// Sum of the 8 bf16 (packed) at this offset over all ranks, fp32 accumulation in the switch.
IRIS_D V4 ld_reduce_bf16x8(const void* mc_ptr) {
  V4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}
IRIS_D V4 ld_reduce_f16x8(const void* mc_ptr) {
  V4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}
IRIS_D V4 ld_reduce_f32x4(const void* mc_ptr) {
  V4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return v;
}
// Add 1 to an int32 flag on every rank with release semantics (publishes earlier stores).
IRIS_D void red_release_add_u32(void* mc_ptr, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_ptr), "r"(v) : "memory");
}
IRIS_D void red_add_bf16x8(void* mc_ptr, V4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_ptr), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

IRIS_D void red_add_f16x8(void* mc_ptr, V4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_ptr), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

}  // namespace multimem
}  // namespace iris
#endif
