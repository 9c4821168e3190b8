// Stand-in for absl::Span<T>: pointer + length view, constructible from containers.
#pragma once
#include <cstddef>
#include <initializer_list>
#include <type_traits>
namespace absl {
template <class T>
class Span {
 public:
  using value_type = std::remove_cv_t<T>;
  constexpr Span() = default;
  constexpr Span(T* data, size_t size) : data_(data), size_(size) {}
  template <size_t N>
  constexpr Span(T (&array)[N]) : data_(array), size_(N) {}
  template <class C, class = decltype(std::declval<C&>().data()), class = decltype(std::declval<C&>().size()),
            class = std::enable_if_t<!std::is_same_v<std::decay_t<C>, Span>>>
  constexpr Span(C& container) : data_(container.data()), size_(container.size()) {}
  template <class C, class = decltype(std::declval<const C&>().data()), class = decltype(std::declval<const C&>().size()),
            class = std::enable_if_t<!std::is_same_v<std::decay_t<C>, Span> && std::is_const_v<T>>>
  constexpr Span(const C& container) : data_(container.data()), size_(container.size()) {}
  template <class U = T, class = std::enable_if_t<std::is_const_v<U>>>
  constexpr Span(std::initializer_list<value_type> list) : data_(list.begin()), size_(list.size()) {}
  constexpr T* data() const { return data_; }
  constexpr size_t size() const { return size_; }
  constexpr bool empty() const { return size_ == 0; }
  constexpr T& operator[](size_t i) const { return data_[i]; }
  constexpr T* begin() const { return data_; }
  constexpr T* end() const { return data_ + size_; }
  constexpr T& front() const { return data_[0]; }
  constexpr T& back() const { return data_[size_ - 1]; }
 private:
  T* data_ = nullptr;
  size_t size_ = 0;
};
template <class T>
constexpr Span<T> MakeSpan(T* data, size_t size) { return Span<T>(data, size); }
template <class C>
constexpr auto MakeSpan(C& c) -> Span<std::remove_pointer_t<decltype(c.data())>> {
  return Span<std::remove_pointer_t<decltype(c.data())>>(c.data(), c.size());
}
template <class T>
constexpr Span<const T> MakeConstSpan(const T* data, size_t size) { return Span<const T>(data, size); }
template <class C>
constexpr auto MakeConstSpan(const C& c) -> Span<const std::remove_pointer_t<decltype(c.data())>> {
  return Span<const std::remove_pointer_t<decltype(c.data())>>(c.data(), c.size());
}
}  // namespace absl
