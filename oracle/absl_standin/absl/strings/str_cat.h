// Stand-in for absl::StrCat: stream every argument into one std::string.
#pragma once
#include <sstream>
#include <string>
namespace absl {
template <class... Args>
std::string StrCat(const Args&... args) {
  std::ostringstream out;
  (out << ... << args);
  return out.str();
}
}  // namespace absl
