// Stand-in for absl::InlinedVector<T, N>: a std::vector with the same interface
// (the inline-capacity optimisation does not change results).
#pragma once
#include <cstddef>
#include <initializer_list>
#include <vector>
namespace absl {
template <class T, size_t N>
class InlinedVector : public std::vector<T> {
 public:
  using std::vector<T>::vector;
  InlinedVector() = default;
  InlinedVector(std::initializer_list<T> list) : std::vector<T>(list) {}
};
}  // namespace absl
