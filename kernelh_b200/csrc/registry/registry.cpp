#include "registry.hpp"

#include <map>
#include <mutex>
#include <stdexcept>

namespace kh {

void register_builtin_kernels(); // builtin_kernels.cpp

// Table emitted by the build step (cubin_blobs.cpp): one entry per kernel source.
const CodeObject *code_objects_begin();
extern const int kCodeObjectCount;

namespace {
std::mutex g_mu;
std::map<std::string, KernelRecord> &table() {
  static std::map<std::string, KernelRecord> t;
  return t;
}
// built-ins that a record registered from outside has displaced, kept for unregister_kernel
std::map<std::string, KernelRecord> &displaced() {
  static std::map<std::string, KernelRecord> t;
  return t;
}
bool g_builtins_done = false;
void ensure_builtins() {
  static std::once_flag once;
  std::call_once(once, [] {
    register_builtin_kernels();
    g_builtins_done = true;
  });
}
} // namespace

void register_kernel(KernelRecord record) {
  if (record.image) ensure_builtins(); // a record from outside lands on top of the built-ins, not under them
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = table().find(record.name);
  if (record.image && it != table().end() && !it->second.image) displaced()[record.name] = it->second;
  table()[record.name] = std::move(record);
}

bool unregister_kernel(const std::string &name) {
  ensure_builtins();
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = table().find(name);
  if (it == table().end() || !it->second.image) return false;
  table().erase(it);
  if (auto old = displaced().find(name); old != displaced().end()) {
    table()[name] = std::move(old->second);
    displaced().erase(old);
  }
  return true;
}

std::vector<std::string> registered_kernels() {
  ensure_builtins();
  std::lock_guard<std::mutex> lock(g_mu);
  std::vector<std::string> names;
  for (const auto &kv : table()) names.push_back(kv.first); // std::map iterates sorted
  return names;
}

const KernelRecord &find_kernel(const std::string &name) {
  ensure_builtins();
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = table().find(name);
    if (it != table().end()) return it->second;
  }
  std::string names;
  for (const std::string &n : registered_kernels()) {
    if (!names.empty()) names += ", ";
    names += n;
  }
  throw std::runtime_error("unknown kernel template '" + name + "'; registered kernels: " + names);
}

const CodeObject *find_code_object(const std::string &name) {
  const CodeObject *objects = code_objects_begin();
  for (int i = 0; i < kCodeObjectCount; ++i)
    if (name == objects[i].name) return &objects[i];
  return nullptr;
}

std::vector<std::string> code_object_names() {
  std::vector<std::string> out;
  const CodeObject *objects = code_objects_begin();
  for (int i = 0; i < kCodeObjectCount; ++i) out.emplace_back(objects[i].name);
  return out;
}

} // namespace kh
