// Host stand-in for Kokkos::sort (see Kokkos_Core.hpp in this folder): ascending
// sort of a rank-1 view. Test infrastructure only.
#pragma once
#include <Kokkos_Core.hpp>

namespace Kokkos {
template <class D, class... P>
void sort(const View<D, P...>& v) {
  static_assert(View<D, P...>::rank == 1, "sort takes a rank-1 view");
  if (v.stride(0) == 1) {
    std::sort(v.data(), v.data() + v.extent(0));
    return;
  }
  std::vector<typename View<D, P...>::non_const_value_type> t(v.extent(0));
  for (std::size_t i = 0; i < t.size(); ++i) t[i] = v(i);
  std::sort(t.begin(), t.end());
  for (std::size_t i = 0; i < t.size(); ++i) v(i) = t[i];
}
template <class D, class... P>
void sort(const Serial&, const View<D, P...>& v) { sort(v); }
}  // namespace Kokkos
