// Shape maps and their text form "k=v,k=v". Grammar and failure behaviour are
// the reference's (bench/harness/shape_text.cpp:19-44, tools/kernelh/main.cpp:
// 242-266): strict decimal integers, no empty items, a malformed text parses to
// an empty map; printing is in key order.
#pragma once

#include <cstdint>
#include <map>
#include <string>

namespace kh {

using ShapeMap = std::map<std::string, int64_t>;

std::string shape_to_text(const ShapeMap &shape);
ShapeMap parse_shape_text(const std::string &text);

} // namespace kh
