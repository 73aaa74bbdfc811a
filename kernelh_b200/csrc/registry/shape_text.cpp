#include "shape_text.hpp"

#include <cerrno>
#include <cstdlib>

namespace kh {

std::string shape_to_text(const ShapeMap &shape) {
  std::string out;
  for (const auto &[k, v] : shape) {
    if (!out.empty()) out += ',';
    out += k + "=" + std::to_string(v);
  }
  return out;
}

ShapeMap parse_shape_text(const std::string &text) {
  ShapeMap out;
  size_t pos = 0;
  for (;;) {
    const size_t comma = text.find(',', pos);
    const std::string item = text.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos);
    const size_t eq = item.find('=');
    if (eq == std::string::npos || eq == 0 || eq + 1 >= item.size()) return {};
    const std::string value = item.substr(eq + 1);
    errno = 0;
    char *end = nullptr;
    const long long parsed = std::strtoll(value.c_str(), &end, 10);
    if (errno != 0 || end == value.c_str() || *end != '\0') return {};
    out[item.substr(0, eq)] = parsed;
    if (comma == std::string::npos) break;
    pos = comma + 1;
  }
  return out;
}

} // namespace kh
