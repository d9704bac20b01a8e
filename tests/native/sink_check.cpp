// CPU harness around kineto_b200/csrc/k2j_sink.cuh: writes seeded random "events" through the emit pass's
// WindowSink into a host buffer, in random order and at every byte alignment, and compares the buffer with the
// plain concatenation of the events.  Window and output are ordinary host arrays here.
#include <cstdint>
#include <cstring>
#include <random>
#include <string>
#include <vector>
#include "k2j_sink.cuh"

namespace {
struct Op { int kind; uint64_t w; uint32_t len; std::vector<uint64_t> words; uint32_t skew; };
struct Event { std::vector<Op> ops; std::string text; };

std::string bytes_of(uint64_t w, uint32_t len) {
  std::string s;
  for (uint32_t i = 0; i < len; i++) s += (char)((w >> (8 * i)) & 0xff);
  return s;
}
uint64_t masked(uint64_t w, uint32_t len) { return len >= 8 ? w : (len ? w & (~0ull >> (8 * (8 - len))) : 0); }
}  // namespace

extern "C" {
// Returns 0 when the buffer equals the expected text, else 1 + the offset of the first difference
// (or -1 when a sink reported a size mismatch).
int64_t sc_fuzz(uint64_t seed, int n_events, int max_ops, int max_copy) {
  std::mt19937_64 rng(seed);
  auto rnd = [&](uint64_t n) { return (uint64_t)(rng() % n); };
  auto printable = [&]() { uint64_t w = 0; for (int i = 0; i < 8; i++) w |= (uint64_t)(0x21 + rnd(0x5d)) << (8 * i); return w; };
  std::vector<Event> ev(n_events);
  std::string expected;
  std::vector<uint64_t> offs(n_events);
  for (int e = 0; e < n_events; e++) {
    Event& E = ev[e];
    auto add = [&](Op o, const std::string& t) { E.ops.push_back(std::move(o)); E.text += t; };
    add(Op{3, k2j::kEventHead8, 8, {}, 0}, bytes_of(k2j::kEventHead8, 8));
    add(Op{1, 0x22687022ull, 4, {}, 0}, "\"ph\"");  // no event is shorter than kMinEventBytes
    const int nops = (int)rnd(max_ops + 1);
    for (int k = 0; k < nops; k++) {
      const int kind = (int)rnd(6);
      if (kind == 0) { uint32_t len = (uint32_t)rnd(5); uint64_t w = masked(printable(), len); add(Op{0, w, len, {}, 0}, bytes_of(w, len)); }
      else if (kind == 1) { uint64_t w = masked(printable(), 4); add(Op{1, w, 4, {}, 0}, bytes_of(w, 4)); }
      else if (kind == 2) { uint32_t len = (uint32_t)rnd(9); uint64_t w = masked(printable(), len); add(Op{2, w, len, {}, 0}, bytes_of(w, len)); }
      else if (kind == 3) { uint64_t w = printable(); add(Op{3, w, 8, {}, 0}, bytes_of(w, 8)); }
      else {
        const uint32_t len = (uint32_t)rnd(max_copy + 1), skew = kind == 5 ? (uint32_t)rnd(8) : 0;
        Op o{kind, 0, len, {}, skew};
        o.words.resize((skew + len + 7) / 8 + 2);
        for (auto& x : o.words) x = printable();
        const char* p = reinterpret_cast<const char*>(o.words.data()) + skew;
        add(std::move(o), std::string(p, len));
      }
    }
    add(Op{2, 0x2C7D20200Aull, 5, {}, 0}, std::string("\n  },"));
    offs[e] = expected.size();
    expected += E.text;
  }
  const size_t total = expected.size();
  std::vector<uint8_t> raw(total + 128 + 32, 0xEE);
  uint8_t* out = raw.data() + (32 - (reinterpret_cast<uintptr_t>(raw.data()) & 31)) % 32;
  std::vector<int> order(n_events);
  for (int i = 0; i < n_events; i++) order[i] = i;
  for (int i = n_events - 1; i > 0; i--) std::swap(order[i], order[rnd(i + 1)]);
  static uint32_t window[k2j::kWinWords * k2j::kWinStride + k2j::kWinPadWords];  // lane 0 of a warp's interleaved windows
  bool size_ok = true;
  for (int e : order) {
    for (auto& x : window) x = 0xA5A5A5A5u;  // stale contents of an earlier event
    k2j::WindowSink s;
    uint8_t* dst = out + offs[e];
    s.init(dst, (uint32_t)ev[e].text.size(), window);
    uint32_t loose = 0;  // bytes appended since the last ensure()
    for (const Op& o : ev[e].ops) {
      if (o.kind < 4) {
        if (loose + o.len > 32 || rnd(4) == 0) { s.ensure(48); loose = 0; }
        loose += o.len;
      } else loose = 0;
      switch (o.kind) {
        case 0: s.put((uint32_t)o.w, (int)o.len); break;
        case 1: s.put4((uint32_t)o.w); break;
        case 2: s.put64(o.w, o.len); break;
        case 3: s.put8w(o.w); break;
        case 4: s.words(o.words.data(), o.len); break;
        default: s.bytes(reinterpret_cast<const uint8_t*>(o.words.data()) + o.skew, o.len); break;
      }
    }
    size_ok = s.finish(dst, (uint32_t)ev[e].text.size()) && size_ok;
  }
  if (!size_ok) return -1;
  for (size_t i = 0; i < total; i++)
    if (out[i] != (uint8_t)expected[i]) return 1 + (int64_t)i;
  return 0;
}
}
