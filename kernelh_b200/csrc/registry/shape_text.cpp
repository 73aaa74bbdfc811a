#include "shape_text.hpp"

#include <cctype>
#include <charconv>
#include <optional>
#include <string_view>

namespace kh {

std::string shape_to_text(const ShapeMap &shape) {
  std::string out;
  for (const auto &[k, v] : shape) {
    if (!out.empty()) out += ',';
    out += k + "=" + std::to_string(v);
  }
  return out;
}

namespace {

// A whole decimal integer that fits int64. Leading blanks and one '+' are
// tolerated because the C library conversion the reference's CLI relies on
// tolerates them; anything after the digits rejects the value.
std::optional<int64_t> whole_integer(std::string_view v) {
  while (!v.empty() && std::isspace(static_cast<unsigned char>(v.front()))) v.remove_prefix(1);
  if (v.size() > 1 && v.front() == '+' && v[1] != '-') v.remove_prefix(1);
  int64_t value = 0;
  const auto [stop, ec] = std::from_chars(v.data(), v.data() + v.size(), value, 10);
  if (ec != std::errc() || stop != v.data() + v.size() || v.empty()) return std::nullopt;
  return value;
}

} // namespace

ShapeMap parse_shape_text(const std::string &text) {
  ShapeMap out;
  std::string_view rest(text);
  bool more = true;
  while (more) {
    const size_t cut = rest.find(',');
    const std::string_view item = rest.substr(0, cut);
    more = cut != std::string_view::npos;
    if (more) rest.remove_prefix(cut + 1);
    const size_t sep = item.find('=');
    const bool has_key = sep != std::string_view::npos && sep > 0;
    const auto value = has_key ? whole_integer(item.substr(sep + 1)) : std::nullopt;
    if (!value) return {}; // one bad item voids the whole text
    out[std::string(item.substr(0, sep))] = *value; // a repeated key keeps the last value
  }
  return out;
}

} // namespace kh
