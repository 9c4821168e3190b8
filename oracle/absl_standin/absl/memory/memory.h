// Stand-in for absl::WrapUnique.
#pragma once
#include <memory>
namespace absl {
template <class T>
std::unique_ptr<T> WrapUnique(T* pointer) { return std::unique_ptr<T>(pointer); }
}  // namespace absl
