// Stand-in: absl::string_view is std::string_view.
#pragma once
#include <string_view>
namespace absl { using string_view = std::string_view; }
