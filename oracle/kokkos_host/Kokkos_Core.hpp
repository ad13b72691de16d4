// A host-only stand-in for the part of the Kokkos programming model that the
// reference's evaluation path uses, so that the reference's own sources compile
// with g++ alone into a CPU library that the parity tests call as the checker.
//
// TEST INFRASTRUCTURE ONLY. Nothing in the product includes this file.
//
// It follows the published Kokkos API (View, parallel_for / reduce / scan over
// range and team policies, nested team ranges, reducers, atomics, deep_copy,
// mirrors, subviews) with the semantics of a host backend whose teams have one
// thread and one vector lane: every "parallel" construct runs its iterations in
// index order, or, when compiled with OpenMP, flat parallel_for loops and team
// leagues run their iterations on several host threads (what Kokkos' OpenMP
// backend does); reductions and scans always run in index order on one thread,
// so their sums have one fixed association.
// It is written from the API's documentation, not from Kokkos' sources.
#pragma once

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <memory>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define KOKKOS_LAMBDA [=]
#define KOKKOS_CLASS_LAMBDA [ =, *this ]
#define KOKKOS_INLINE_FUNCTION inline
#define KOKKOS_FORCEINLINE_FUNCTION inline
#define KOKKOS_FUNCTION
#define KOKKOS_DEFAULTED_FUNCTION
#define KOKKOS_ENABLE_SERIAL 1
#define KOKKOS_VERSION 50202

namespace Kokkos {

// ---------------------------------------------------------------- spaces ----
struct Serial;
struct HostSpace {
  using memory_space = HostSpace;
  using execution_space = Serial;
  static const char* name() { return "Host"; }
};
struct SharedHostPinnedSpace {
  using memory_space = SharedHostPinnedSpace;
  using execution_space = Serial;
  static const char* name() { return "HostPinned"; }
};
struct SharedSpace {
  using memory_space = SharedSpace;
  using execution_space = Serial;
  static const char* name() { return "Shared"; }
};
struct Serial {
  using memory_space = HostSpace;
  using execution_space = Serial;
  using scratch_memory_space = HostSpace;
  using array_layout = struct LayoutRight;
  void fence() const {}
  void fence(const std::string&) const {}
  static const char* name() { return "Serial"; }
  int concurrency() const {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
  }
  bool operator==(const Serial&) const { return true; }
  bool operator!=(const Serial&) const { return false; }
};
using DefaultExecutionSpace = Serial;
using DefaultHostExecutionSpace = Serial;

struct LayoutRight {};
struct LayoutLeft {};
struct LayoutStride {};
struct MemoryManaged {};
struct MemoryUnmanaged {};
template <unsigned>
struct MemoryTraits {};
enum : unsigned { Unmanaged = 1, RandomAccess = 2, Atomic = 4, Restrict = 8 };

template <unsigned A, unsigned B = 1>
struct LaunchBounds {};
namespace Experimental {
namespace WorkItemProperty {
struct HintLightWeight_t {};
struct HintHeavyWeight_t {};
struct None_t {};
constexpr HintLightWeight_t HintLightWeight{};
}  // namespace WorkItemProperty
}  // namespace Experimental

struct InitializationSettings {};
namespace detail {
inline bool& initialized() {
  static bool b = false;
  return b;
}
}  // namespace detail
inline void initialize() { detail::initialized() = true; }
inline void initialize(int&, char**) { detail::initialized() = true; }
inline void initialize(const InitializationSettings&) { detail::initialized() = true; }
inline void finalize() { detail::initialized() = false; }
inline bool is_initialized() { return detail::initialized(); }
inline bool is_finalized() { return false; }
inline void fence() {}
inline void fence(const std::string&) {}
struct ScopeGuard {
  ScopeGuard() { initialize(); }
  ScopeGuard(int&, char**) { initialize(); }
  ~ScopeGuard() { finalize(); }
};

namespace Tools {
inline bool profileLibraryLoaded() { return false; }
inline void beginParallelFor(const std::string&, uint32_t, uint64_t*) {}
inline void endParallelFor(uint64_t) {}
inline void pushRegion(const std::string&) {}
inline void popRegion() {}
}  // namespace Tools
namespace Profiling {
inline void pushRegion(const std::string&) {}
inline void popRegion() {}
}  // namespace Profiling

// ------------------------------------------------------------------ math ----
using std::abs;
using std::ceil;
using std::cos;
using std::exp;
using std::fabs;
using std::floor;
using std::fma;
using std::fmax;
using std::fmin;
using std::log;
using std::pow;
using std::round;
using std::sin;
using std::sqrt;
using std::tan;
using std::tanh;
using std::erf;
using std::log2;
using std::exp2;
using std::isnan;
using std::isfinite;
using std::isinf;
template <class T>
constexpr const T& max(const T& a, const T& b) { return a < b ? b : a; }
template <class T>
constexpr const T& min(const T& a, const T& b) { return b < a ? b : a; }
template <class T>
constexpr const T& clamp(const T& v, const T& lo, const T& hi) { return v < lo ? lo : (hi < v ? hi : v); }

template <class A, class B>
struct pair {
  A first;
  B second;
  pair() = default;
  pair(const A& a, const B& b) : first(a), second(b) {}
  template <class C, class D>
  pair(const std::pair<C, D>& p) : first(p.first), second(p.second) {}
};
template <class A, class B>
pair<A, B> make_pair(A a, B b) { return pair<A, B>(a, b); }

// --------------------------------------------------------------- atomics ----
// The loops that call these run on one host thread at a time per destination in
// the serial build; with OpenMP they go through std::atomic_ref-like builtins.
template <class T>
inline T atomic_fetch_add(T* p, T v) {
  if constexpr (std::is_integral_v<T>) {
    return __atomic_fetch_add(p, v, __ATOMIC_RELAXED);
  } else {
    T old, des;
    __atomic_load(p, &old, __ATOMIC_RELAXED);
    do { des = old + v; } while (!__atomic_compare_exchange(p, &old, &des, true, __ATOMIC_RELAXED, __ATOMIC_RELAXED));
    return old;
  }
}
template <class T, class U>
inline T atomic_fetch_add(T* p, U v) { return atomic_fetch_add(p, T(v)); }
template <class T, class U>
inline void atomic_add(T* p, U v) { (void) atomic_fetch_add(p, T(v)); }
template <class T>
inline void atomic_inc(T* p) { (void) atomic_fetch_add(p, T(1)); }
template <class T>
inline void atomic_increment(T* p) { (void) atomic_fetch_add(p, T(1)); }
template <class T, class U>
inline T atomic_fetch_max(T* p, U v) {
  T old, des;
  __atomic_load(p, &old, __ATOMIC_RELAXED);
  do { des = old < T(v) ? T(v) : old; } while (!__atomic_compare_exchange(p, &old, &des, true, __ATOMIC_RELAXED, __ATOMIC_RELAXED));
  return old;
}
template <class T, class U>
inline void atomic_max(T* p, U v) { (void) atomic_fetch_max(p, v); }
template <class T, class U>
inline T atomic_fetch_min(T* p, U v) {
  T old, des;
  __atomic_load(p, &old, __ATOMIC_RELAXED);
  do { des = T(v) < old ? T(v) : old; } while (!__atomic_compare_exchange(p, &old, &des, true, __ATOMIC_RELAXED, __ATOMIC_RELAXED));
  return old;
}
template <class T, class U>
inline void atomic_min(T* p, U v) { (void) atomic_fetch_min(p, v); }
template <class T>
inline T atomic_compare_exchange(T* p, T expected, T desired) {
  __atomic_compare_exchange(p, &expected, &desired, false, __ATOMIC_RELAXED, __ATOMIC_RELAXED);
  return expected;
}
template <class T>
inline T atomic_exchange(T* p, T v) {
  T old;
  __atomic_exchange(p, &v, &old, __ATOMIC_RELAXED);
  return old;
}
template <class T>
inline T atomic_load(const T* p) {
  T v;
  __atomic_load(const_cast<T*>(p), &v, __ATOMIC_RELAXED);
  return v;
}
template <class T>
inline void atomic_store(T* p, T v) { __atomic_store(p, &v, __ATOMIC_RELAXED); }
inline void memory_fence() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }

// ------------------------------------------------------------------ View ----
namespace detail {
template <class D>
struct data_type {
  using value = D;
  static constexpr int rank = 0;
};
template <class D>
struct data_type<D*> {
  using value = typename data_type<D>::value;
  static constexpr int rank = data_type<D>::rank + 1;
};
template <class... P>
struct pick_space {
  using type = HostSpace;
};
template <class P0, class... P>
struct pick_space<P0, P...> {
  using type = std::conditional_t<std::is_same_v<P0, SharedHostPinnedSpace> || std::is_same_v<P0, SharedSpace>, P0,
                                  typename pick_space<P...>::type>;
};
}  // namespace detail

struct WithoutInitializing_t {};
constexpr WithoutInitializing_t WithoutInitializing{};
struct SequentialHostInit_t {};
constexpr SequentialHostInit_t SequentialHostInit{};
struct ViewAllocProps {
  std::string label;
  bool init = true;
};
namespace detail {
inline void alloc_arg(ViewAllocProps& p, const std::string& s) { p.label = s; }
inline void alloc_arg(ViewAllocProps& p, const char* s) { p.label = s; }
inline void alloc_arg(ViewAllocProps& p, WithoutInitializing_t) { p.init = false; }
inline void alloc_arg(ViewAllocProps&, SequentialHostInit_t) {}
template <class X>
inline void alloc_arg(ViewAllocProps&, const X&) {}  // spaces, execution space instances
}  // namespace detail
template <class... A>
ViewAllocProps view_alloc(const A&... a) {
  ViewAllocProps p;
  (detail::alloc_arg(p, a), ...);
  return p;
}

struct ALL_t {};
constexpr ALL_t ALL{};

template <class DataType, class... Props>
class View {
 public:
  using value_type = typename detail::data_type<DataType>::value;
  using non_const_value_type = std::remove_const_t<value_type>;
  using const_value_type = std::add_const_t<value_type>;
  using pointer_type = value_type*;
  using reference_type = value_type&;
  using data_type = DataType;
  using memory_space = typename detail::pick_space<Props...>::type;
  using execution_space = Serial;
  using device_type = Serial;
  using array_layout = LayoutRight;
  using size_type = std::size_t;
  using traits = View;
  using HostMirror = View<DataType, Props...>;
  using host_mirror_type = HostMirror;
  using non_const_type = View<std::conditional_t<true, typename std::remove_const<value_type>::type, void>, Props...>;
  static constexpr int rank = detail::data_type<DataType>::rank;
  static constexpr int Rank = rank;
  static constexpr unsigned rank_dynamic = rank;
  static_assert(rank <= 4, "the stand-in has views of rank 0 to 4");

  View() = default;

  // Allocating constructors.
  explicit View(const std::string& label, std::size_t n0 = 0, std::size_t n1 = 0, std::size_t n2 = 0, std::size_t n3 = 0) {
    allocate(label, true, n0, n1, n2, n3);
  }
  explicit View(const char* label, std::size_t n0 = 0, std::size_t n1 = 0, std::size_t n2 = 0, std::size_t n3 = 0) {
    allocate(label, true, n0, n1, n2, n3);
  }
  explicit View(const ViewAllocProps& p, std::size_t n0 = 0, std::size_t n1 = 0, std::size_t n2 = 0, std::size_t n3 = 0) {
    allocate(p.label, p.init, n0, n1, n2, n3);
  }
  // Wrapping constructor: someone else's memory.
  View(pointer_type p, std::size_t n0 = 0, std::size_t n1 = 0, std::size_t n2 = 0, std::size_t n3 = 0) : ptr_(p) {
    set_extents(n0, n1, n2, n3);
  }
  // From a view of the same rank whose value type converts by qualification.
  template <class D2, class... P2,
            class = std::enable_if_t<detail::data_type<D2>::rank == rank &&
                                     std::is_convertible_v<typename detail::data_type<D2>::value*, value_type*>>>
  View(const View<D2, P2...>& o) : ptr_(o.data()), own_(o.owner()), label_(o.label()) {
    for (int d = 0; d < 4; ++d) ext_[d] = o.raw_extent(d), str_[d] = o.raw_stride(d);
  }

  template <class I0>
  reference_type operator()(I0 i) const {
    static_assert(rank == 1);
    return ptr_[std::size_t(i) * str_[0]];
  }
  reference_type operator()() const {
    static_assert(rank == 0);
    return *ptr_;
  }
  template <class I0, class I1>
  reference_type operator()(I0 i, I1 j) const {
    static_assert(rank == 2);
    return ptr_[std::size_t(i) * str_[0] + std::size_t(j) * str_[1]];
  }
  template <class I0, class I1, class I2>
  reference_type operator()(I0 i, I1 j, I2 k) const {
    static_assert(rank == 3);
    return ptr_[std::size_t(i) * str_[0] + std::size_t(j) * str_[1] + std::size_t(k) * str_[2]];
  }
  template <class I0, class I1, class I2, class I3>
  reference_type operator()(I0 i, I1 j, I2 k, I3 l) const {
    static_assert(rank == 4);
    return ptr_[std::size_t(i) * str_[0] + std::size_t(j) * str_[1] + std::size_t(k) * str_[2] + std::size_t(l) * str_[3]];
  }
  template <class I0>
  reference_type operator[](I0 i) const {
    static_assert(rank == 1);
    return ptr_[std::size_t(i) * str_[0]];
  }
  template <class... I>
  reference_type access(I... i) const { return (*this)(i...); }

  pointer_type data() const { return ptr_; }
  std::size_t extent(int d) const { return d < rank ? ext_[d] : 1; }
  int extent_int(int d) const { return int(extent(d)); }
  std::size_t size() const {
    std::size_t n = 1;
    for (int d = 0; d < rank; ++d) n *= ext_[d];
    return n;
  }
  // The distance, in elements, from the first element to one past the last.
  std::size_t span() const {
    if (size() == 0) return 0;
    std::size_t n = 1;
    for (int d = 0; d < rank; ++d) n += (ext_[d] - 1) * str_[d];
    return n;
  }
  bool span_is_contiguous() const { return span() == size(); }
  std::size_t stride(int d) const { return d < rank ? str_[d] : 0; }
  std::size_t stride_0() const { return stride(0); }
  std::size_t stride_1() const { return stride(1); }
  std::size_t stride_2() const { return stride(2); }
  const std::string& label() const { return label_; }
  bool is_allocated() const { return ptr_ != nullptr; }
  int use_count() const { return int(own_.use_count()); }

  // Internal, for conversions and subviews.
  const std::shared_ptr<void>& owner() const { return own_; }
  std::size_t raw_extent(int d) const { return ext_[d]; }
  std::size_t raw_stride(int d) const { return str_[d]; }
  void assign_raw(pointer_type p, const std::shared_ptr<void>& own, const std::string& label) {
    ptr_ = p, own_ = own, label_ = label;
  }
  void set_dim(int d, std::size_t e, std::size_t s) { ext_[d] = e, str_[d] = s; }

 private:
  void set_extents(std::size_t n0, std::size_t n1, std::size_t n2, std::size_t n3) {
    const std::size_t n[4] = {n0, n1, n2, n3};
    for (int d = 0; d < 4; ++d) ext_[d] = d < rank ? n[d] : 1;
    std::size_t s = 1;
    for (int d = rank - 1; d >= 0; --d) str_[d] = s, s *= ext_[d];
  }
  void allocate(const std::string& label, bool init, std::size_t n0, std::size_t n1, std::size_t n2, std::size_t n3) {
    set_extents(n0, n1, n2, n3);
    label_ = label;
    const std::size_t bytes = std::max<std::size_t>(size(), 1) * sizeof(non_const_value_type);
    void* raw = std::aligned_alloc(64, (bytes + 63) / 64 * 64);
    if (!raw) throw std::bad_alloc();
    if (init) std::memset(raw, 0, bytes);
    own_ = std::shared_ptr<void>(raw, [](void* q) { std::free(q); });
    ptr_ = reinterpret_cast<pointer_type>(raw);
  }

  pointer_type ptr_ = nullptr;
  std::size_t ext_[4] = {0, 0, 0, 0};
  std::size_t str_[4] = {0, 0, 0, 0};
  std::shared_ptr<void> own_;
  std::string label_;
};

template <class T>
struct is_view : std::false_type {};
template <class D, class... P>
struct is_view<View<D, P...>> : std::true_type {};
template <class T>
inline constexpr bool is_view_v = is_view<T>::value;

// ---------------------------------------------------------------- subview ----
namespace detail {
template <class A>
constexpr int keeps_dim() {
  return std::is_integral_v<std::decay_t<A>> ? 0 : 1;
}
template <class T, int R>
struct add_rank {
  using type = typename add_rank<T, R - 1>::type*;
};
template <class T>
struct add_rank<T, 0> {
  using type = T;
};
template <class V, class A>
inline void slice(const V& src, int d, const A& a, std::size_t& offset, std::size_t& e, std::size_t& s, bool& keep) {
  if constexpr (std::is_integral_v<A>) {
    offset += std::size_t(a) * src.raw_stride(d);
    keep = false;
  } else if constexpr (std::is_same_v<A, ALL_t>) {
    e = src.raw_extent(d), s = src.raw_stride(d), keep = true;
  } else {  // a pair [first, second)
    offset += std::size_t(a.first) * src.raw_stride(d);
    e = std::size_t(a.second) - std::size_t(a.first), s = src.raw_stride(d), keep = true;
  }
}
}  // namespace detail

template <class D, class... P, class... Args>
auto subview(const View<D, P...>& v, Args... args) {
  using V = View<D, P...>;
  static_assert(sizeof...(Args) == V::rank, "one slice argument per dimension");
  constexpr int R = (detail::keeps_dim<Args>() + ... + 0);
  using Out = View<typename detail::add_rank<typename V::value_type, R>::type, P...>;
  Out out;
  std::size_t offset = 0;
  int d = 0, o = 0;
  auto one = [&](const auto& a) {
    std::size_t e = 1, s = 0;
    bool keep = false;
    detail::slice(v, d, a, offset, e, s, keep);
    if (keep) out.set_dim(o++, e, s);
    ++d;
  };
  (one(args), ...);
  for (; o < 4; ++o) out.set_dim(o, 1, 0);
  out.assign_raw(v.data() ? v.data() + offset : nullptr, v.owner(), v.label());
  return out;
}

template <class V, class... Args>
using Subview = decltype(subview(std::declval<V>(), std::declval<Args>()...));

// -------------------------------------------------------------- deep_copy ----
namespace detail {
template <class V, class F>
inline void for_each_index(const V& v, F f) {
  const std::size_t n0 = V::rank > 0 ? v.raw_extent(0) : 1, n1 = V::rank > 1 ? v.raw_extent(1) : 1,
                    n2 = V::rank > 2 ? v.raw_extent(2) : 1, n3 = V::rank > 3 ? v.raw_extent(3) : 1;
  for (std::size_t i = 0; i < n0; ++i)
    for (std::size_t j = 0; j < n1; ++j)
      for (std::size_t k = 0; k < n2; ++k)
        for (std::size_t l = 0; l < n3; ++l)
          f(i * v.raw_stride(0) * (V::rank > 0) + j * v.raw_stride(1) * (V::rank > 1) + k * v.raw_stride(2) * (V::rank > 2) +
                l * v.raw_stride(3) * (V::rank > 3),
            i, j, k, l);
}
}  // namespace detail

template <class D1, class... P1, class D2, class... P2>
void deep_copy(const View<D1, P1...>& dst, const View<D2, P2...>& src) {
  using V1 = View<D1, P1...>;
  using V2 = View<D2, P2...>;
  static_assert(V1::rank == V2::rank, "deep_copy of views of different rank");
  using T = typename V1::non_const_value_type;
  if (dst.size() == 0 || (const void*) dst.data() == (const void*) src.data()) return;
  if constexpr (std::is_same_v<T, typename V2::non_const_value_type>)
    if (dst.span_is_contiguous() && src.span_is_contiguous()) {
      std::memmove((void*) dst.data(), (const void*) src.data(), dst.size() * sizeof(T));
      return;
    }
  detail::for_each_index(dst, [&](std::size_t off, std::size_t i, std::size_t j, std::size_t k, std::size_t l) {
    const std::size_t so = i * src.raw_stride(0) * (V2::rank > 0) + j * src.raw_stride(1) * (V2::rank > 1) +
                           k * src.raw_stride(2) * (V2::rank > 2) + l * src.raw_stride(3) * (V2::rank > 3);
    const_cast<T*>(dst.data())[off] = static_cast<T>(src.data()[so]);
  });
}
template <class D1, class... P1, class S, class = std::enable_if_t<!is_view_v<S> && std::is_convertible_v<S, typename View<D1, P1...>::non_const_value_type>>>
void deep_copy(const View<D1, P1...>& dst, const S& value) {
  using T = typename View<D1, P1...>::non_const_value_type;
  if (dst.size() == 0) return;
  if (dst.span_is_contiguous()) {
    std::fill_n(const_cast<T*>(dst.data()), dst.size(), T(value));
    return;
  }
  detail::for_each_index(dst, [&](std::size_t off, std::size_t, std::size_t, std::size_t, std::size_t) {
    const_cast<T*>(dst.data())[off] = T(value);
  });
}
// A rank-0 view into a scalar.
template <class S, class D2, class... P2, class = std::enable_if_t<!is_view_v<S> && View<D2, P2...>::rank == 0>>
void deep_copy(S& dst, const View<D2, P2...>& src) {
  dst = S(*src.data());
}
template <class A, class B>
void deep_copy(const Serial&, A&& dst, B&& src) {
  deep_copy(std::forward<A>(dst), std::forward<B>(src));
}

// ---------------------------------------------------------------- mirrors ----
template <class D, class... P>
View<D, P...> create_mirror_view(const View<D, P...>& v) { return v; }
template <class Space, class D, class... P, class = std::enable_if_t<!is_view_v<Space>>>
View<D, P...> create_mirror_view(const Space&, const View<D, P...>& v) { return v; }
template <class D, class... P>
View<D, P...> create_mirror_view(WithoutInitializing_t, const View<D, P...>& v) { return v; }
template <class Space, class D, class... P>
View<D, P...> create_mirror_view(WithoutInitializing_t, const Space&, const View<D, P...>& v) { return v; }
template <class Space, class D, class... P>
View<D, P...> create_mirror_view_and_copy(const Space&, const View<D, P...>& v, const std::string& = "") { return v; }
template <class D, class... P>
auto create_mirror(const View<D, P...>& v) {
  using V = View<D, P...>;
  View<typename detail::add_rank<typename V::non_const_value_type, V::rank>::type, P...> out(
      v.label(), v.extent(0), V::rank > 1 ? v.extent(1) : 0, V::rank > 2 ? v.extent(2) : 0, V::rank > 3 ? v.extent(3) : 0);
  return out;
}
template <class Space, class D, class... P, class = std::enable_if_t<!is_view_v<Space>>>
auto create_mirror(const Space&, const View<D, P...>& v) { return create_mirror(v); }

template <class D, class... P>
void resize(View<D, P...>& v, std::size_t n0 = 0, std::size_t n1 = 0, std::size_t n2 = 0, std::size_t n3 = 0) {
  View<D, P...> n(v.label(), n0, n1, n2, n3);
  using V = View<D, P...>;
  detail::for_each_index(n, [&](std::size_t off, std::size_t i, std::size_t j, std::size_t k, std::size_t l) {
    if (i < v.raw_extent(0) && (V::rank < 2 || j < v.raw_extent(1)) && (V::rank < 3 || k < v.raw_extent(2)) &&
        (V::rank < 4 || l < v.raw_extent(3)))
      n.data()[off] = v.data()[i * v.raw_stride(0) * (V::rank > 0) + j * v.raw_stride(1) * (V::rank > 1) +
                               k * v.raw_stride(2) * (V::rank > 2) + l * v.raw_stride(3) * (V::rank > 3)];
  });
  v = n;
}
template <class D, class... P>
void realloc(View<D, P...>& v, std::size_t n0 = 0, std::size_t n1 = 0, std::size_t n2 = 0, std::size_t n3 = 0) {
  const std::string label = v.label();
  v = View<D, P...>();
  v = View<D, P...>(label, n0, n1, n2, n3);
}

// --------------------------------------------------------------- policies ----
struct AUTO_t {};
constexpr AUTO_t AUTO{};

template <class... Props>
class RangePolicy {
 public:
  using execution_space = Serial;
  using index_type = long;
  using member_type = long;
  RangePolicy() = default;
  RangePolicy(long b, long e) : begin_(b), end_(e) {}
  RangePolicy(const Serial&, long b, long e) : begin_(b), end_(e) {}
  long begin() const { return begin_; }
  long end() const { return end_; }
  RangePolicy& set_chunk_size(int) { return *this; }

 private:
  long begin_ = 0, end_ = 0;
};

struct PerTeamValue {
  std::size_t v;
};
struct PerThreadValue {
  std::size_t v;
};
inline PerTeamValue PerTeam(std::size_t v) { return {v}; }
inline PerThreadValue PerThread(std::size_t v) { return {v}; }

// One team's scratch: a bump allocator over a buffer the launch owns.
class ScratchSpace {
 public:
  ScratchSpace(char* base, std::size_t bytes) : base_(base), end_(base + bytes), cur_(base) {}
  void* get_shmem(std::size_t bytes) const { return get_shmem_aligned(bytes, 8); }
  void* get_shmem_aligned(std::size_t bytes, std::size_t align) const {
    std::uintptr_t p = (reinterpret_cast<std::uintptr_t>(cur_) + align - 1) / align * align;
    char* q = reinterpret_cast<char*>(p);
    if (q + bytes > end_) return nullptr;
    cur_ = q + bytes;
    return q;
  }

 private:
  char *base_, *end_;
  mutable char* cur_;
};

class HostTeamMember {
 public:
  HostTeamMember(int league_rank, int league_size, char* s0, std::size_t b0, char* s1, std::size_t b1)
      : league_rank_(league_rank), league_size_(league_size), scratch0_(s0, b0), scratch1_(s1, b1) {}
  int league_rank() const { return league_rank_; }
  int league_size() const { return league_size_; }
  int team_rank() const { return 0; }
  int team_size() const { return 1; }
  void team_barrier() const {}
  const ScratchSpace& team_scratch(int level) const { return level == 0 ? scratch0_ : scratch1_; }
  const ScratchSpace& thread_scratch(int level) const { return team_scratch(level); }
  const ScratchSpace& team_shmem() const { return scratch0_; }
  template <class T>
  void team_broadcast(T&, int) const {}
  template <class T>
  T team_reduce(const T& v) const { return v; }
  template <class T>
  T team_scan(const T&) const { return T(0); }

 private:
  int league_rank_, league_size_;
  ScratchSpace scratch0_, scratch1_;
};

template <class... Props>
class TeamPolicy {
 public:
  using execution_space = Serial;
  using member_type = HostTeamMember;
  TeamPolicy() = default;
  template <class T = int, class V = int>
  TeamPolicy(int league, T, V = V()) : league_(league) {}
  template <class T = int, class V = int>
  TeamPolicy(const Serial&, int league, T, V = V()) : league_(league) {}
  int league_size() const { return league_; }
  int team_size() const { return 1; }
  int impl_vector_length() const { return 1; }
  TeamPolicy& set_scratch_size(int level, PerTeamValue t) {
    bytes_[level] = t.v;
    return *this;
  }
  TeamPolicy& set_scratch_size(int level, PerThreadValue t) {
    bytes_[level] = t.v;
    return *this;
  }
  TeamPolicy& set_scratch_size(int level, PerTeamValue t, PerThreadValue h) {
    bytes_[level] = t.v + h.v;
    return *this;
  }
  TeamPolicy& set_scratch_size(int level, PerThreadValue h, PerTeamValue t) { return set_scratch_size(level, t, h); }
  TeamPolicy& set_chunk_size(int) { return *this; }
  std::size_t scratch_size(int level) const { return bytes_[level]; }
  static int scratch_size_max(int level) { return level == 0 ? (1 << 20) : (1 << 30); }
  template <class F, class Tag>
  int team_size_max(const F&, const Tag&) const { return 1; }
  template <class F, class Tag>
  int team_size_recommended(const F&, const Tag&) const { return 1; }
  static int vector_length_max() { return 1; }

 private:
  int league_ = 0;
  std::size_t bytes_[2] = {0, 0};
};
struct ParallelForTag {};
struct ParallelReduceTag {};
struct ParallelScanTag {};

// Nested ranges over a team with one thread and one lane.
struct NestedRange {
  long begin, end;
};
template <class I>
NestedRange TeamThreadRange(const HostTeamMember&, I n) { return {0, long(n)}; }
template <class I, class J>
NestedRange TeamThreadRange(const HostTeamMember&, I b, J e) { return {long(b), long(e)}; }
template <class I>
NestedRange TeamVectorRange(const HostTeamMember&, I n) { return {0, long(n)}; }
template <class I, class J>
NestedRange TeamVectorRange(const HostTeamMember&, I b, J e) { return {long(b), long(e)}; }
template <class I>
NestedRange ThreadVectorRange(const HostTeamMember&, I n) { return {0, long(n)}; }
template <class I, class J>
NestedRange ThreadVectorRange(const HostTeamMember&, I b, J e) { return {long(b), long(e)}; }

struct SingleScope {};
inline SingleScope PerTeam(const HostTeamMember&) { return {}; }
inline SingleScope PerThread(const HostTeamMember&) { return {}; }
template <class F>
void single(const SingleScope&, const F& f) { f(); }
template <class F, class T>
void single(const SingleScope&, const F& f, T& value) { f(value); }

// ---------------------------------------------------------------- reducers ----
namespace detail {
template <class T, class Op>
class Reducer {
 public:
  using reducer = Reducer;
  using value_type = T;
  explicit Reducer(T& ref) : ref_(&ref) {}
  template <class D, class... P>
  explicit Reducer(const View<D, P...>& v) : ref_(const_cast<T*>(v.data())) {}
  T& reference() const { return *ref_; }
  void init(T& v) const { v = Op::identity(); }
  void join(T& a, const T& b) const { a = Op::apply(a, b); }

 private:
  T* ref_;
};
template <class T>
struct SumOp {
  static T identity() { return T(0); }
  static T apply(const T& a, const T& b) { return a + b; }
};
template <class T>
struct ProdOp {
  static T identity() { return T(1); }
  static T apply(const T& a, const T& b) { return a * b; }
};
template <class T>
struct MaxOp {
  static T identity() { return std::numeric_limits<T>::lowest(); }
  static T apply(const T& a, const T& b) { return a < b ? b : a; }
};
template <class T>
struct MinOp {
  static T identity() { return std::numeric_limits<T>::max(); }
  static T apply(const T& a, const T& b) { return b < a ? b : a; }
};
struct LAndOp {
  static int identity() { return 1; }
  static int apply(int a, int b) { return a && b; }
};
struct LOrOp {
  static int identity() { return 0; }
  static int apply(int a, int b) { return a || b; }
};
template <class R, class = void>
struct is_reducer : std::false_type {};
template <class R>
struct is_reducer<R, std::void_t<typename R::reducer>> : std::true_type {};
}  // namespace detail
template <class T, class Space = HostSpace>
struct Sum : detail::Reducer<T, detail::SumOp<T>> {
  using detail::Reducer<T, detail::SumOp<T>>::Reducer;
};
template <class T, class Space = HostSpace>
struct Prod : detail::Reducer<T, detail::ProdOp<T>> {
  using detail::Reducer<T, detail::ProdOp<T>>::Reducer;
};
template <class T, class Space = HostSpace>
struct Max : detail::Reducer<T, detail::MaxOp<T>> {
  using detail::Reducer<T, detail::MaxOp<T>>::Reducer;
};
template <class T, class Space = HostSpace>
struct Min : detail::Reducer<T, detail::MinOp<T>> {
  using detail::Reducer<T, detail::MinOp<T>>::Reducer;
};
template <class T, class Space = HostSpace>
struct LAnd : detail::Reducer<T, detail::LAndOp> {
  using detail::Reducer<T, detail::LAndOp>::Reducer;
};
template <class T, class Space = HostSpace>
struct LOr : detail::Reducer<T, detail::LOrOp> {
  using detail::Reducer<T, detail::LOrOp>::Reducer;
};
template <class T> Sum(T&) -> Sum<T>;
template <class T> Max(T&) -> Max<T>;
template <class T> Min(T&) -> Min<T>;

// ----------------------------------------------------------- parallel_for ----
namespace detail {
struct TeamScratch {
  std::vector<char> l0, l1;
};
template <class... P>
inline long range_begin(const RangePolicy<P...>& p) { return p.begin(); }
template <class... P>
inline long range_end(const RangePolicy<P...>& p) { return p.end(); }
template <class I, class = std::enable_if_t<std::is_integral_v<I>>>
inline long range_begin(I) { return 0; }
template <class I, class = std::enable_if_t<std::is_integral_v<I>>>
inline long range_end(I n) { return long(n); }

template <class T>
struct is_team_policy : std::false_type {};
template <class... P>
struct is_team_policy<TeamPolicy<P...>> : std::true_type {};

inline bool& in_parallel() {
  static thread_local bool b = false;
  return b;
}
}  // namespace detail

template <class Policy, class F>
void parallel_for(const std::string&, const Policy& policy, const F& f) {
  if constexpr (detail::is_team_policy<Policy>::value) {
    const int L = policy.league_size();
    const std::size_t b0 = policy.scratch_size(0) + 64, b1 = policy.scratch_size(1) + 64;
#if defined(_OPENMP)
    if (!detail::in_parallel() && L > 1) {
#pragma omp parallel
      {
        detail::in_parallel() = true;
        std::vector<char> s0(b0), s1(b1);
#pragma omp for schedule(static)
        for (int r = 0; r < L; ++r) f(HostTeamMember(r, L, s0.data(), b0, s1.data(), b1));
        detail::in_parallel() = false;
      }
      return;
    }
#endif
    std::vector<char> s0(b0), s1(b1);
    for (int r = 0; r < L; ++r) f(HostTeamMember(r, L, s0.data(), b0, s1.data(), b1));
  } else {
    const long b = detail::range_begin(policy), e = detail::range_end(policy);
#if defined(_OPENMP)
    if (!detail::in_parallel() && e - b > 1) {
#pragma omp parallel
      {
        detail::in_parallel() = true;
#pragma omp for schedule(static)
        for (long i = b; i < e; ++i) f(i);
        detail::in_parallel() = false;
      }
      return;
    }
#endif
    for (long i = b; i < e; ++i) f(i);
  }
}
template <class Policy, class F, class = std::enable_if_t<!std::is_convertible_v<Policy, std::string> && !std::is_same_v<Policy, NestedRange>>>
void parallel_for(const Policy& policy, const F& f) {
  parallel_for(std::string(), policy, f);
}
template <class F>
void parallel_for(const NestedRange& r, const F& f) {
  for (long i = r.begin; i < r.end; ++i) f(i);
}

// -------------------------------------------------------- parallel_reduce ----
namespace detail {
template <class Policy, class F, class T>
inline void reduce_loop(const Policy& policy, const F& f, T& acc) {
  if constexpr (is_team_policy<Policy>::value) {
    const int L = policy.league_size();
    const std::size_t b0 = policy.scratch_size(0) + 64, b1 = policy.scratch_size(1) + 64;
    std::vector<char> s0(b0), s1(b1);
    for (int r = 0; r < L; ++r) f(HostTeamMember(r, L, s0.data(), b0, s1.data(), b1), acc);
  } else if constexpr (std::is_same_v<Policy, NestedRange>) {
    for (long i = policy.begin; i < policy.end; ++i) f(i, acc);
  } else {
    const long b = range_begin(policy), e = range_end(policy);
    for (long i = b; i < e; ++i) f(i, acc);
  }
}
}  // namespace detail

template <class Policy, class F, class R>
void parallel_reduce(const std::string&, const Policy& policy, const F& f, R&& result) {
  using RT = std::decay_t<R>;
  if constexpr (detail::is_reducer<RT>::value) {
    typename RT::value_type acc;
    result.init(acc);
    detail::reduce_loop(policy, f, acc);
    result.reference() = acc;
  } else if constexpr (is_view_v<RT>) {
    using T = typename RT::non_const_value_type;
    T acc = T(0);
    detail::reduce_loop(policy, f, acc);
    *const_cast<T*>(result.data()) = acc;
  } else {
    RT acc = RT(0);
    detail::reduce_loop(policy, f, acc);
    result = acc;
  }
}
template <class Policy, class F, class R, class = std::enable_if_t<!std::is_convertible_v<Policy, std::string>>>
void parallel_reduce(const Policy& policy, const F& f, R&& result) {
  parallel_reduce(std::string(), policy, f, std::forward<R>(result));
}

// Several sums at once over a nested range (the results are summed, each from zero).
template <class F, class R0, class R1, class... Rs>
void parallel_reduce(const NestedRange& r, const F& f, R0& r0, R1& r1, Rs&... rs) {
  r0 = R0(0), r1 = R1(0), ((rs = Rs(0)), ...);
  for (long i = r.begin; i < r.end; ++i) f(i, r0, r1, rs...);
}

// ---------------------------------------------------------- parallel_scan ----
// f(i, partial, final): called once per index with final = true, `partial`
// holding the exclusive prefix on entry; f adds its own contribution.
namespace detail {
template <class Policy, class F, class T>
inline void scan_loop(const Policy& policy, const F& f, T& acc) {
  if constexpr (std::is_same_v<Policy, NestedRange>) {
    for (long i = policy.begin; i < policy.end; ++i) f(i, acc, true);
  } else {
    const long b = range_begin(policy), e = range_end(policy);
    for (long i = b; i < e; ++i) f(i, acc, true);
  }
}
template <class F>
struct scan_value;
template <class C, class R, class I, class T>
struct scan_value<R (C::*)(I, T&, bool) const> {
  using type = T;
};
template <class F>
using scan_value_t = typename scan_value<decltype(&F::operator())>::type;
}  // namespace detail

template <class Policy, class F>
void parallel_scan(const std::string&, const Policy& policy, const F& f) {
  detail::scan_value_t<F> acc{};
  detail::scan_loop(policy, f, acc);
}
template <class Policy, class F, class T, class = std::enable_if_t<!std::is_convertible_v<Policy, std::string>>>
void parallel_scan(const std::string&, const Policy& policy, const F& f, T& total) {
  if constexpr (is_view_v<T>) {
    typename T::non_const_value_type acc{};
    detail::scan_loop(policy, f, acc);
    *const_cast<typename T::non_const_value_type*>(total.data()) = acc;
  } else {
    T acc{};
    detail::scan_loop(policy, f, acc);
    total = acc;
  }
}
template <class Policy, class F, class = std::enable_if_t<!std::is_convertible_v<Policy, std::string>>>
void parallel_scan(const Policy& policy, const F& f) {
  parallel_scan(std::string(), policy, f);
}
template <class F, class T>
void parallel_scan(const NestedRange& r, const F& f, T& total) {
  T acc{};
  detail::scan_loop(r, f, acc);
  total = acc;
}

}  // namespace Kokkos
