// Remote memory access on a symmetric heap: load / store / copy / get / put and the atomics,
// each a translation (context.cuh) followed by one ordinary memory instruction on the peer's
// mapping. Over NVLink 5 the peer mapping is plain global memory for the SM, so these compile to
// ld/st/atom.global with the requested semantics, scope and cache operator.
//
// Same names and argument order as the reference's functional API (iris/mem/triton/ops.py:16-685):
//   load(ptr, to_rank, from_rank, bases)           -- note (to, from), every other op is (from, to)
//   store(ptr, value, from_rank, to_rank, bases)
//   copy(src, dst, from_rank, to_rank, cur_rank, bases)
//   get(from_ptr, to_ptr, from_rank, to_rank, bases)   remote load  -> local store
//   put(from_ptr, to_ptr, from_rank, to_rank, bases)   local load   -> remote store
//   atomic_{add,sub,and,or,xor,min,max,xchg}(ptr, val, from_rank, to_rank, bases), atomic_cas(ptr, cmp, val, ...)
// Masks of the reference are a trailing `bool pred` (a masked-off lane does nothing and a load
// returns `other`). Triton's pointer blocks become per-thread elements; the *_block helpers move a
// contiguous range cooperatively with 16-byte vectors.
#pragma once
#include "common.cuh"
#include "context.cuh"

namespace iris {

namespace detail {
template <int N> struct Bits;
template <> struct Bits<1> { using type = uint8_t; };
template <> struct Bits<2> { using type = uint16_t; };
template <> struct Bits<4> { using type = uint32_t; };
template <> struct Bits<8> { using type = uint64_t; };
struct alignas(16) U128 { uint32_t x, y, z, w; };
template <> struct Bits<16> { using type = U128; };

template <class To, class From>
IRIS_HD To bit_cast(const From& f) {
  static_assert(sizeof(To) == sizeof(From), "size mismatch");
  To t;
  __builtin_memcpy(&t, &f, sizeof(To));
  return t;
}

#if defined(__CUDACC__)
// ---- raw loads ------------------------------------------------------------------------------
#define IRIS_LD_BODY(SUFFIX, ...)                                                                       \
  if constexpr (V) asm volatile("ld.volatile.global" SUFFIX : __VA_ARGS__ : "l"(p) : "memory");              \
  else if constexpr (C == CacheOp::ca) asm volatile("ld.global.ca" SUFFIX : __VA_ARGS__ : "l"(p) : "memory"); \
  else if constexpr (C == CacheOp::cg) asm volatile("ld.global.cg" SUFFIX : __VA_ARGS__ : "l"(p) : "memory"); \
  else if constexpr (C == CacheOp::cs) asm volatile("ld.global.cs" SUFFIX : __VA_ARGS__ : "l"(p) : "memory"); \
  else if constexpr (C == CacheOp::cv) asm volatile("ld.global.cv" SUFFIX : __VA_ARGS__ : "l"(p) : "memory"); \
  else asm volatile("ld.global" SUFFIX : __VA_ARGS__ : "l"(p) : "memory");

template <CacheOp C, bool V> IRIS_D uint8_t ld_raw(const uint8_t* p) {
  uint32_t v; IRIS_LD_BODY(".u8 %0, [%1];", "=r"(v)) return (uint8_t)v;
}
template <CacheOp C, bool V> IRIS_D uint16_t ld_raw(const uint16_t* p) {
  uint16_t v; IRIS_LD_BODY(".u16 %0, [%1];", "=h"(v)) return v;
}
template <CacheOp C, bool V> IRIS_D uint32_t ld_raw(const uint32_t* p) {
  uint32_t v; IRIS_LD_BODY(".u32 %0, [%1];", "=r"(v)) return v;
}
template <CacheOp C, bool V> IRIS_D uint64_t ld_raw(const uint64_t* p) {
  uint64_t v; IRIS_LD_BODY(".u64 %0, [%1];", "=l"(v)) return v;
}
template <CacheOp C, bool V> IRIS_D U128 ld_raw(const U128* p) {
  U128 v;
  if constexpr (V) {  // no 128-bit volatile form: two 64-bit volatile loads
    uint64_t a = ld_raw<C, true>((const uint64_t*)p), b = ld_raw<C, true>((const uint64_t*)p + 1);
    v.x = (uint32_t)a; v.y = (uint32_t)(a >> 32); v.z = (uint32_t)b; v.w = (uint32_t)(b >> 32);
  } else {
    IRIS_LD_BODY(".v4.u32 {%0, %1, %2, %3}, [%4];", "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w))
  }
  return v;
}
#undef IRIS_LD_BODY

// ---- raw stores -----------------------------------------------------------------------------
#define IRIS_ST_BODY(SUFFIX, ...)                                                                    \
  if constexpr (C == CacheOp::wb) asm volatile("st.global.wb" SUFFIX ::"l"(p), __VA_ARGS__ : "memory"); \
  else if constexpr (C == CacheOp::cg) asm volatile("st.global.cg" SUFFIX ::"l"(p), __VA_ARGS__ : "memory"); \
  else if constexpr (C == CacheOp::cs) asm volatile("st.global.cs" SUFFIX ::"l"(p), __VA_ARGS__ : "memory"); \
  else if constexpr (C == CacheOp::wt) asm volatile("st.global.wt" SUFFIX ::"l"(p), __VA_ARGS__ : "memory"); \
  else asm volatile("st.global" SUFFIX ::"l"(p), __VA_ARGS__ : "memory");

template <CacheOp C> IRIS_D void st_raw(uint8_t* p, uint8_t v) { uint32_t w = v; IRIS_ST_BODY(".u8 [%0], %1;", "r"(w)) }
template <CacheOp C> IRIS_D void st_raw(uint16_t* p, uint16_t v) { IRIS_ST_BODY(".u16 [%0], %1;", "h"(v)) }
template <CacheOp C> IRIS_D void st_raw(uint32_t* p, uint32_t v) { IRIS_ST_BODY(".u32 [%0], %1;", "r"(v)) }
template <CacheOp C> IRIS_D void st_raw(uint64_t* p, uint64_t v) { IRIS_ST_BODY(".u64 [%0], %1;", "l"(v)) }
template <CacheOp C> IRIS_D void st_raw(U128* p, U128 v) {
  IRIS_ST_BODY(".v4.u32 [%0], {%1, %2, %3, %4};", "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w))
}
#undef IRIS_ST_BODY

// ---- atomics: 4 semantics x 3 scopes, one PTX string each -------------------------------------
#define IRIS_ATOM_ONE(SEM, SCOPE, OPTY, OUT, ...) \
  asm volatile("atom" SEM SCOPE ".global" OPTY : OUT : __VA_ARGS__ : "memory");
#define IRIS_ATOM_SCOPES(SEM, OPTY, OUT, ...)                                         \
  if constexpr (P == Scope::cta) { IRIS_ATOM_ONE(SEM, ".cta", OPTY, OUT, __VA_ARGS__) } \
  else if constexpr (P == Scope::gpu) { IRIS_ATOM_ONE(SEM, ".gpu", OPTY, OUT, __VA_ARGS__) } \
  else { IRIS_ATOM_ONE(SEM, ".sys", OPTY, OUT, __VA_ARGS__) }
#define IRIS_ATOM(OPTY, OUT, ...)                                                           \
  if constexpr (S == Sem::relaxed) { IRIS_ATOM_SCOPES(".relaxed", OPTY, OUT, __VA_ARGS__) }   \
  else if constexpr (S == Sem::acquire) { IRIS_ATOM_SCOPES(".acquire", OPTY, OUT, __VA_ARGS__) } \
  else if constexpr (S == Sem::release) { IRIS_ATOM_SCOPES(".release", OPTY, OUT, __VA_ARGS__) } \
  else { IRIS_ATOM_SCOPES(".acq_rel", OPTY, OUT, __VA_ARGS__) }

#define IRIS_DEF_ATOM(NAME, T, PTXOP, CONSTR)                              \
  template <Sem S, Scope P> IRIS_D T NAME(T* p, T v) {                     \
    T old;                                                                 \
    IRIS_ATOM(PTXOP " %0, [%1], %2;", "=" CONSTR(old), "l"(p), CONSTR(v))   \
    return old;                                                            \
  }
IRIS_DEF_ATOM(atom_add, int32_t, ".add.s32", "r")
IRIS_DEF_ATOM(atom_add, uint32_t, ".add.u32", "r")
IRIS_DEF_ATOM(atom_add, uint64_t, ".add.u64", "l")
IRIS_DEF_ATOM(atom_add, float, ".add.f32", "f")
IRIS_DEF_ATOM(atom_add, double, ".add.f64", "d")
IRIS_DEF_ATOM(atom_and, uint32_t, ".and.b32", "r")
IRIS_DEF_ATOM(atom_and, uint64_t, ".and.b64", "l")
IRIS_DEF_ATOM(atom_or, uint32_t, ".or.b32", "r")
IRIS_DEF_ATOM(atom_or, uint64_t, ".or.b64", "l")
IRIS_DEF_ATOM(atom_xor, uint32_t, ".xor.b32", "r")
IRIS_DEF_ATOM(atom_xor, uint64_t, ".xor.b64", "l")
IRIS_DEF_ATOM(atom_min, int32_t, ".min.s32", "r")
IRIS_DEF_ATOM(atom_min, uint32_t, ".min.u32", "r")
IRIS_DEF_ATOM(atom_min, int64_t, ".min.s64", "l")
IRIS_DEF_ATOM(atom_min, uint64_t, ".min.u64", "l")
IRIS_DEF_ATOM(atom_max, int32_t, ".max.s32", "r")
IRIS_DEF_ATOM(atom_max, uint32_t, ".max.u32", "r")
IRIS_DEF_ATOM(atom_max, int64_t, ".max.s64", "l")
IRIS_DEF_ATOM(atom_max, uint64_t, ".max.u64", "l")
IRIS_DEF_ATOM(atom_xchg, uint32_t, ".exch.b32", "r")
IRIS_DEF_ATOM(atom_xchg, uint64_t, ".exch.b64", "l")
#undef IRIS_DEF_ATOM
template <Sem S, Scope P> IRIS_D int64_t atom_add(int64_t* p, int64_t v) {
  return (int64_t)atom_add<S, P>((uint64_t*)p, (uint64_t)v);
}
template <Sem S, Scope P> IRIS_D uint16_t atom_add_f16(uint16_t* p, uint16_t v) {
  uint16_t old;
  IRIS_ATOM(".add.noftz.f16 %0, [%1], %2;", "=h"(old), "l"(p), "h"(v))
  return old;
}
template <Sem S, Scope P> IRIS_D uint16_t atom_add_bf16(uint16_t* p, uint16_t v) {
  uint16_t old;
  IRIS_ATOM(".add.noftz.bf16 %0, [%1], %2;", "=h"(old), "l"(p), "h"(v))
  return old;
}
template <Sem S, Scope P> IRIS_D uint32_t atom_cas(uint32_t* p, uint32_t cmp, uint32_t v) {
  uint32_t old;
  IRIS_ATOM(".cas.b32 %0, [%1], %2, %3;", "=r"(old), "l"(p), "r"(cmp), "r"(v))
  return old;
}
template <Sem S, Scope P> IRIS_D uint64_t atom_cas(uint64_t* p, uint64_t cmp, uint64_t v) {
  uint64_t old;
  IRIS_ATOM(".cas.b64 %0, [%1], %2, %3;", "=l"(old), "l"(p), "l"(cmp), "l"(v))
  return old;
}
#undef IRIS_ATOM
#undef IRIS_ATOM_SCOPES
#undef IRIS_ATOM_ONE

#else  // ------------------------------------------------------------ host twin (CPU backend)
template <CacheOp C, bool V, class U> inline U ld_raw(const U* p) {
  if constexpr (sizeof(U) == 16) { U v; __builtin_memcpy(&v, p, 16); return v; }
  else return __atomic_load_n(p, __ATOMIC_RELAXED);
}
template <CacheOp C, class U> inline void st_raw(U* p, U v) {
  if constexpr (sizeof(U) == 16) __builtin_memcpy(p, &v, 16);
  else __atomic_store_n(p, v, __ATOMIC_RELAXED);
}
template <Sem S> constexpr int host_order() {
  return S == Sem::relaxed ? __ATOMIC_RELAXED
         : S == Sem::acquire ? __ATOMIC_ACQUIRE
         : S == Sem::release ? __ATOMIC_RELEASE : __ATOMIC_ACQ_REL;
}
template <Sem S, Scope P, class T, class F> inline T host_rmw(T* p, F f) {
  if constexpr (sizeof(T) == 2) {  // 16-bit floats are handled by the caller on 16-bit words
    T old = __atomic_load_n(p, __ATOMIC_RELAXED);
    while (!__atomic_compare_exchange_n(p, &old, f(old), true, host_order<S>(), __ATOMIC_RELAXED)) {}
    return old;
  } else {
    using U = typename Bits<sizeof(T)>::type;
    U old = __atomic_load_n((U*)p, __ATOMIC_RELAXED);
    while (true) {
      U neu = bit_cast<U>(f(bit_cast<T>(old)));
      if (__atomic_compare_exchange_n((U*)p, &old, neu, true, host_order<S>(), __ATOMIC_RELAXED)) break;
    }
    return bit_cast<T>(old);
  }
}
template <Sem S, Scope P, class T> inline T atom_add(T* p, T v) { return host_rmw<S, P>(p, [v](T o) { return (T)(o + v); }); }
template <Sem S, Scope P, class T> inline T atom_and(T* p, T v) { return host_rmw<S, P>(p, [v](T o) { return (T)(o & v); }); }
template <Sem S, Scope P, class T> inline T atom_or(T* p, T v) { return host_rmw<S, P>(p, [v](T o) { return (T)(o | v); }); }
template <Sem S, Scope P, class T> inline T atom_xor(T* p, T v) { return host_rmw<S, P>(p, [v](T o) { return (T)(o ^ v); }); }
template <Sem S, Scope P, class T> inline T atom_min(T* p, T v) { return host_rmw<S, P>(p, [v](T o) { return o < v ? o : v; }); }
template <Sem S, Scope P, class T> inline T atom_max(T* p, T v) { return host_rmw<S, P>(p, [v](T o) { return o > v ? o : v; }); }
template <Sem S, Scope P, class T> inline T atom_xchg(T* p, T v) { return host_rmw<S, P>(p, [v](T) { return v; }); }
template <Sem S, Scope P, class T> inline T atom_cas(T* p, T cmp, T v) {
  T expected = cmp;
  __atomic_compare_exchange_n(p, &expected, v, false, host_order<S>(), __ATOMIC_RELAXED);
  return expected;
}
#endif

}  // namespace detail

// =========================================================================== per-thread element ops
// Load `*ptr` as seen on rank `from_rank` (ptr is a pointer into rank `to_rank`'s = the caller's heap).
template <class T, CacheOp C = CacheOp::none, bool Volatile = false>
IRIS_D T load(const T* ptr, int to_rank, int from_rank, const uint64_t* bases, bool pred = true, T other = T()) {
  if (!pred) return other;
  using U = typename detail::Bits<sizeof(T)>::type;
  const U* src = (const U*)translate(ptr, to_rank, from_rank, bases);
  return detail::bit_cast<T>(detail::ld_raw<C, Volatile>(src));
}
// Store `value` to `*ptr` on rank `to_rank` (ptr is a pointer into rank `from_rank`'s heap).
template <class T, CacheOp C = CacheOp::none>
IRIS_D void store(T* ptr, T value, int from_rank, int to_rank, const uint64_t* bases, bool pred = true) {
  if (!pred) return;
  using U = typename detail::Bits<sizeof(T)>::type;
  detail::st_raw<C>((U*)translate(ptr, from_rank, to_rank, bases), detail::bit_cast<U>(value));
}
// Copy one element from `src` on `from_rank` to `dst` on `to_rank`; both pointers are given in
// `cur_rank`'s address space and cur_rank must be one of the two (reference ops.py:134-214).
template <class T, CacheOp LC = CacheOp::none, CacheOp SC = CacheOp::none>
IRIS_D void copy(const T* src, T* dst, int from_rank, int to_rank, int cur_rank, const uint64_t* bases,
                 bool pred = true) {
  if (!pred) return;
  using U = typename detail::Bits<sizeof(T)>::type;
  const U* s = (const U*)translate(src, cur_rank, from_rank, bases);
  U* d = (U*)translate(dst, cur_rank, to_rank, bases);
  detail::st_raw<SC>(d, detail::ld_raw<LC, false>(s));
}
// get: remote load from `from_rank`, store into my own memory.
template <class T, CacheOp LC = CacheOp::none, CacheOp SC = CacheOp::none>
IRIS_D void get(const T* from_ptr, T* to_ptr, int from_rank, int to_rank, const uint64_t* bases, bool pred = true,
                T other = T()) {
  if (!pred) return;
  using U = typename detail::Bits<sizeof(T)>::type;
  const U* s = (const U*)translate(from_ptr, to_rank, from_rank, bases);
  detail::st_raw<SC>((U*)to_ptr, detail::ld_raw<LC, false>(s));
}
// put: load from my own memory, remote store on `to_rank`.
template <class T, CacheOp LC = CacheOp::none, CacheOp SC = CacheOp::none>
IRIS_D void put(const T* from_ptr, T* to_ptr, int from_rank, int to_rank, const uint64_t* bases, bool pred = true) {
  if (!pred) return;
  using U = typename detail::Bits<sizeof(T)>::type;
  U* d = (U*)translate(to_ptr, from_rank, to_rank, bases);
  detail::st_raw<SC>(d, detail::ld_raw<LC, false>((const U*)from_ptr));
}

#define IRIS_DEF_RMA_ATOMIC(NAME, IMPL)                                                                 \
  template <Sem S = Sem::acq_rel, Scope P = Scope::gpu, class T>                                          \
  IRIS_D T NAME(T* ptr, T val, int from_rank, int to_rank, const uint64_t* bases, bool pred = true) {     \
    if (!pred) return T();                                                                              \
    return detail::IMPL<S, P>(translate(ptr, from_rank, to_rank, bases), val);                           \
  }
IRIS_DEF_RMA_ATOMIC(atomic_add, atom_add)
IRIS_DEF_RMA_ATOMIC(atomic_and, atom_and)
IRIS_DEF_RMA_ATOMIC(atomic_or, atom_or)
IRIS_DEF_RMA_ATOMIC(atomic_xor, atom_xor)
IRIS_DEF_RMA_ATOMIC(atomic_min, atom_min)
IRIS_DEF_RMA_ATOMIC(atomic_max, atom_max)
#undef IRIS_DEF_RMA_ATOMIC
template <Sem S = Sem::acq_rel, Scope P = Scope::gpu, class T>
IRIS_D T atomic_sub(T* ptr, T val, int from_rank, int to_rank, const uint64_t* bases, bool pred = true) {
  if (!pred) return T();
  return detail::atom_add<S, P>(translate(ptr, from_rank, to_rank, bases), (T)(T(0) - val));
}
template <Sem S = Sem::acq_rel, Scope P = Scope::gpu, class T>
IRIS_D T atomic_xchg(T* ptr, T val, int from_rank, int to_rank, const uint64_t* bases, bool pred = true) {
  if (!pred) return T();
  using U = typename detail::Bits<sizeof(T)>::type;
  U old = detail::atom_xchg<S, P>((U*)translate(ptr, from_rank, to_rank, bases), detail::bit_cast<U>(val));
  return detail::bit_cast<T>(old);
}
template <Sem S = Sem::acq_rel, Scope P = Scope::gpu, class T>
IRIS_D T atomic_cas(T* ptr, T cmp, T val, int from_rank, int to_rank, const uint64_t* bases) {
  using U = typename detail::Bits<sizeof(T)>::type;
  U old = detail::atom_cas<S, P>((U*)translate(ptr, from_rank, to_rank, bases), detail::bit_cast<U>(cmp),
                                 detail::bit_cast<U>(val));
  return detail::bit_cast<T>(old);
}

// =========================================================================== cooperative ranges
// Copy `bytes` from src to dst with `nthreads` threads (thread `tid` of them), 16 bytes at a
// time when all three are 16-byte aligned, else bytewise. src/dst are final (already translated).
IRIS_D void copy_bytes(void* dst, const void* src, size_t bytes, int tid, int nthreads) {
  if ((((uint64_t)dst | (uint64_t)src | bytes) & 15) == 0) {
    const detail::U128* s = (const detail::U128*)src;
    detail::U128* d = (detail::U128*)dst;
    size_t n = bytes >> 4;
    size_t i = tid;
    // 4 independent 16-byte loads in flight per thread before the stores
    for (; i + 3 * (size_t)nthreads < n; i += 4 * (size_t)nthreads) {
      detail::U128 a = detail::ld_raw<CacheOp::none, false>(s + i);
      detail::U128 b = detail::ld_raw<CacheOp::none, false>(s + i + nthreads);
      detail::U128 c = detail::ld_raw<CacheOp::none, false>(s + i + 2 * (size_t)nthreads);
      detail::U128 e = detail::ld_raw<CacheOp::none, false>(s + i + 3 * (size_t)nthreads);
      detail::st_raw<CacheOp::none>(d + i, a);
      detail::st_raw<CacheOp::none>(d + i + nthreads, b);
      detail::st_raw<CacheOp::none>(d + i + 2 * (size_t)nthreads, c);
      detail::st_raw<CacheOp::none>(d + i + 3 * (size_t)nthreads, e);
    }
    for (; i < n; i += nthreads) detail::st_raw<CacheOp::none>(d + i, detail::ld_raw<CacheOp::none, false>(s + i));
  } else {
    const uint8_t* s = (const uint8_t*)src;
    uint8_t* d = (uint8_t*)dst;
    for (size_t i = tid; i < bytes; i += nthreads) d[i] = s[i];
  }
}
// put a contiguous block: local `src` -> `dst` (pointer into my heap) on `to_rank`.
template <class T>
IRIS_D void put_block(const DeviceContext& ctx, const T* src, T* dst, size_t n, int to_rank, int tid, int nthreads) {
  copy_bytes(ctx.remote(dst, to_rank), src, n * sizeof(T), tid, nthreads);
}
// get a contiguous block: `src` (pointer into my heap) on `from_rank` -> local `dst`.
template <class T>
IRIS_D void get_block(const DeviceContext& ctx, const T* src, T* dst, size_t n, int from_rank, int tid, int nthreads) {
  copy_bytes(dst, ctx.remote(src, from_rank), n * sizeof(T), tid, nthreads);
}

}  // namespace iris
