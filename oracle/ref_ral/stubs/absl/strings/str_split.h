// TEST INFRASTRUCTURE.  Stand-in for the one abseil function the reference's
// context/common_context_impl.cc uses (the reference tree does not vendor
// abseil): split a string at every occurrence of a character, empty pieces kept.
#pragma once
#include <string>
#include <vector>

namespace absl {
inline std::vector<std::string> StrSplit(const std::string& text, char separator) {
  std::vector<std::string> pieces;
  size_t begin = 0;
  for (;;) {
    const size_t end = text.find(separator, begin);
    if (end == std::string::npos) {
      pieces.push_back(text.substr(begin));
      return pieces;
    }
    pieces.push_back(text.substr(begin, end - begin));
    begin = end + 1;
  }
}
}  // namespace absl
