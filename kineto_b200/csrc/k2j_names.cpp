// Host-side string table of the C ABI (k2j_names_*, k2j_intern_kernel_names): turns the kernel-name pointers of
// CUPTI activity buffers, as CUPTI wrote them, into ids of demangled names in a pool laid out for k2j_set_strings.
// Stands where the reference demangles the name of every kernel activity it logs, one std::string per activity
// (libkineto/src/CuptiActivity.h:297-300 -> libkineto/src/Demangle.cpp:33-53); here each distinct pointer is
// demangled once, and the walks over the buffers run on several threads.
#include "../../include/k2j.h"

#include <cxxabi.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <deque>
#include <string>
#include <string_view>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace k2j { uint32_t record_slots(uint32_t kind, uint32_t word1); }  // k2j.cu: 8-byte slots of a record, 0 = unknown kind

struct k2j_names {
  std::deque<std::string> store;                            // strings stay in place: the map's keys view them
  std::unordered_map<std::string_view, uint32_t> ids;
  std::vector<uint64_t> off{0};
  std::vector<uint8_t> data;
  std::unordered_map<const void*, uint32_t> by_pointer[2];  // [demangle] name pointer -> id
  uint32_t intern(std::string_view s) {
    auto it = ids.find(s);
    if (it != ids.end()) return it->second;
    const uint32_t id = (uint32_t)store.size();
    store.emplace_back(s);
    ids.emplace(std::string_view(store.back()), id);
    data.insert(data.end(), s.begin(), s.end());
    off.push_back(data.size());
    return id;
  }
};

namespace {
constexpr uint32_t kKindConcurrentKernel = 10;  // CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL
constexpr size_t kKernelNameOffset = 104;       // CUpti_ActivityKernel9::name
constexpr size_t kMaxSymbolSize = 8192;         // longer names are kept as they are (Demangle.cpp:31, :39-41)

// What the reference's demangle() returns for `name` (Demangle.cpp:33-53).
std::string demangled(const char* name, bool demangle) {
  if (!name) return std::string();
  if (!demangle || strlen(name) > kMaxSymbolSize) return std::string(name);
  int status = 0;
  size_t len = 0;
  char* d = abi::__cxa_demangle(name, nullptr, &len, &status);
  if (status != 0) return std::string(name);
  std::string out(d);
  free(d);
  return out;
}

struct Walk {
  std::vector<uint64_t> kernels;          // byte offsets of the kernel records of this slice of buffers
  std::vector<const void*> first_seen;    // distinct name pointers, in order of first sight
};
}  // namespace

extern "C" {

k2j_status k2j_names_create(k2j_names** out) {
  if (!out) return K2J_ERR_INVALID_ARGUMENT;
  *out = new k2j_names();
  return K2J_OK;
}

void k2j_names_destroy(k2j_names* names) { delete names; }

k2j_status k2j_names_intern(k2j_names* names, const char* s, uint64_t len, uint32_t* id) {
  if (!names || !id || (!s && len)) return K2J_ERR_INVALID_ARGUMENT;
  *id = names->intern(std::string_view(s ? s : "", (size_t)len));
  return K2J_OK;
}

k2j_status k2j_names_pool(const k2j_names* names, const uint64_t** off, const uint8_t** data, uint64_t* n_strings) {
  if (!names || !off || !data || !n_strings) return K2J_ERR_INVALID_ARGUMENT;
  *off = names->off.data();
  *data = names->data.data();
  *n_strings = names->off.size() - 1;
  return K2J_OK;
}

k2j_status k2j_intern_kernel_names(k2j_names* names, uint8_t* bytes, uint64_t n_bytes, const uint64_t* buftab,
                                   uint32_t n_buffers, int demangle, uint64_t* n_kernel_records) {
  if (!names || (!bytes && n_bytes) || (!buftab && n_buffers)) return K2J_ERR_INVALID_ARGUMENT;
  for (uint32_t b = 0; b < n_buffers; b++) {
    const uint64_t o = buftab[2 * b], v = buftab[2 * b + 1];
    if ((o & 7) || o > n_bytes || v > n_bytes - o) return K2J_ERR_INVALID_ARGUMENT;
  }
  uint64_t total = 0;
  for (uint32_t b = 0; b < n_buffers; b++) total += buftab[2 * b + 1];
  const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
  const size_t nt = std::max<size_t>(1, std::min<size_t>({(size_t)hw, (size_t)16, (size_t)n_buffers, (size_t)(total >> 22)}));
  std::vector<Walk> walks(nt);
  // buffers are dealt out in contiguous slices of about equal bytes, so "first seen" keeps the buffers' order
  std::vector<uint32_t> first(nt + 1, n_buffers);
  {
    uint64_t acc = 0; size_t t = 0; first[0] = 0;
    for (uint32_t b = 0; b < n_buffers && t + 1 < nt; b++) {
      acc += buftab[2 * b + 1];
      if (acc >= total * (t + 1) / nt) first[++t] = b + 1;
    }
  }
  auto walk = [&](size_t t) {
    Walk& w = walks[t];
    std::unordered_set<const void*> seen;
    const void* last = nullptr;
    for (uint32_t b = first[t]; b < first[t + 1]; b++) {
      const uint64_t base = buftab[2 * b], valid = buftab[2 * b + 1];
      uint64_t pos = 0;
      while (pos + 8 <= valid) {  // the walk of k2j_set_cupti: sized by kind, an unknown kind ends its buffer
        uint32_t kind, word1;
        memcpy(&kind, bytes + base + pos, 4);
        memcpy(&word1, bytes + base + pos + 4, 4);
        const uint64_t size = 8ull * k2j::record_slots(kind, word1);
        if (size == 0 || pos + size > valid) break;
        if (kind == kKindConcurrentKernel) {
          const void* p;
          memcpy(&p, bytes + base + pos + kKernelNameOffset, 8);
          w.kernels.push_back(base + pos);
          if (p != last && seen.insert(p).second) w.first_seen.push_back(p);  // launches of one kernel come in runs
          last = p;
        }
        pos += size;
      }
    }
  };
  auto on_threads = [&](auto&& fn) {
    std::vector<std::thread> threads;
    for (size_t t = 1; t < nt; t++) threads.emplace_back(fn, t);
    fn(0);
    for (auto& th : threads) th.join();
  };
  on_threads(walk);
  auto& ids = names->by_pointer[demangle ? 1 : 0];
  for (const Walk& w : walks)
    for (const void* p : w.first_seen)
      if (!ids.count(p)) ids.emplace(p, names->intern(demangled(static_cast<const char*>(p), demangle != 0)));
  auto rewrite = [&](size_t t) {
    const void* last = nullptr;
    uint64_t last_id = 0;
    bool have = false;
    for (uint64_t at : walks[t].kernels) {
      const void* p;
      memcpy(&p, bytes + at + kKernelNameOffset, 8);
      if (!have || p != last) { last = p; last_id = ids.find(p)->second; have = true; }
      memcpy(bytes + at + kKernelNameOffset, &last_id, 8);
    }
  };
  on_threads(rewrite);
  if (n_kernel_records) {
    *n_kernel_records = 0;
    for (const Walk& w : walks) *n_kernel_records += w.kernels.size();
  }
  return K2J_OK;
}

}  // extern "C"
