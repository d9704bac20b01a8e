// TEST INFRASTRUCTURE — CPU restatement of libkineto's trace post-processing path, used only as the
// checker for the CUDA implementation (tests/, the smoke test, and bench.py's cpu_baseline leg).
// The product library never calls into this file.
//
// Parity status: PINNED.  tests/test_oracle_vs_reference.py compares this restatement byte for byte
// with the unmodified reference (oracle/_ref/ref_driver) on seeded traces, and tests/golden/ holds
// reference outputs for machines where the reference is not built.
//
// What is restated (reference file:line, paths relative to the reference project):
//   pass 1  correlation maps            libkineto/src/CuptiActivityProfiler.cpp:256-302
//   pass 2  record dispatch             libkineto/src/CuptiActivityProfiler.cpp:532-588
//           runtime / driver records    libkineto/src/CuptiActivityProfiler.cpp:304-358
//           GPU records, window, spans  libkineto/src/GenericActivityProfiler.cpp:329-340, :397-435
//   CPU ops                             libkineto/src/GenericActivityProfiler.cpp:234-275
//   timestamps                          libkineto/src/CuptiTimestamp.h:29-51, src/ApproximateClock.cpp:83-90
//   names                               libkineto/src/CuptiActivity.h:297-300, :586-602, :682-687
//   args fragments                      libkineto/src/CuptiActivity.h:499-576, :604-622, :643-672,
//                                       :694-712, :758-765;  include/TypedMetadataJson.h:38-205
//   occupancy                           libkineto/src/DeviceProperties.cpp:161-222 (NVIDIA's
//                                       cuda_occupancy.h from the CUDA toolkit, as the reference uses)
//   JSON text                           libkineto/src/output_json.cpp:72-126, :144-153, :193-203,
//                                       :237-259, :318-345, :837-1021
//   user-annotation spans               libkineto/src/GenericActivityProfiler.cpp:277-327
//   synchronisation / CUDA event records libkineto/src/CuptiActivityProfiler.cpp:221-254, :379-514,
//                                       libkineto/src/CuptiActivity.h:180-411, output_json.cpp:914-943, :1006-1012
//
// Output: the "activities" part of the trace file, i.e. every event written between the header /
// metadata rows and the CPU trace span: CPU-op events, then GPU-side events in buffer order, then
// gpu_user_annotation spans (ActivityTrace::save order, libkineto/src/output_membuf.h:91-107).
#include <algorithm>
#include <charconv>
#include <cinttypes>
#include <climits>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include <cuda_occupancy.h>

#include "trace_file.h"
#include "../kineto_b200/csrc/k2j_cupti_sizes.h"  // generated from cupti_activity.h: record size per activity kind

namespace {

enum : uint32_t { K_MEMCPY = 1, K_MEMSET = 2, K_DRIVER = 4, K_RUNTIME = 5, K_KERNEL = 10, K_OVERHEAD = 17, K_MEMCPY2 = 22, K_CUDA_EVENT = 36, K_SYNC = 38, K_EXTCORR = 39 };
enum : int { T_CPU_OP = 0, T_GPU_USER_ANNOTATION = 2, T_GPU_MEMCPY = 3, T_GPU_MEMSET = 4, T_KERNEL = 5, T_RUNTIME = 7,
             T_DRIVER = 8, T_CPU_INSTANT = 9, T_OVERHEAD = 11, T_CUDA_SYNC = 15, T_CUDA_EVENT = 16, T_MTIA_COUNTERS = 17, T_XPU_RUNTIME = 21, T_XPU_DRIVER = 22,
             T_PU1_RUNTIME = 24, T_PU1_DRIVER = 25, T_XPU_SCOPE = 26, T_HW_COUNTERS = 28, T_COUNT = 29 };
const char* kTypeNames[T_COUNT] = {  // libkineto/include/ActivityType.h:80-112
    "cpu_op", "user_annotation", "gpu_user_annotation", "gpu_memcpy", "gpu_memset", "kernel",
    "external_correlation", "cuda_runtime", "cuda_driver", "cpu_instant_event", "python_function",
    "overhead", "mtia_runtime", "mtia_ccp_events", "mtia_insight", "cuda_sync", "cuda_event",
    "mtia_counters", "glow_runtime", "cuda_profiler_range", "hpu_op", "xpu_runtime", "xpu_driver",
    "collective_comm", "privateuse1_runtime", "privateuse1_driver", "xpu_scope_profiler", "xpu_sync",
    "hardware_counters"};

size_t recSize(uint32_t kind) {
  switch (kind) {
    case K_KERNEL: return 208;
    case K_MEMCPY: return 88;
    case K_MEMCPY2: return 96;
    case K_MEMSET: return 88;
    case K_RUNTIME: case K_DRIVER: return 40;
    case K_EXTCORR: return 24;
    case K_OVERHEAD: return 56;  // CUpti_ActivityOverhead3
    case K_SYNC: return 40;      // CUpti_ActivitySynchronization
    case K_CUDA_EVENT: return 56;  // CUpti_ActivityCudaEvent2
    // kinds the reference only counts (CuptiActivityProfiler.cpp:583-587): the record sizes of the CUDA 12.9 CUPTI
    // headers, so that the walk can step over them; 0 for a kind the headers do not define
    default: return kind < (uint32_t)k2j::kCuptiKinds ? 8u * k2j::kCuptiRecordSlots[kind] : 0;
  }
}

template <class T> T rd(const uint8_t* p, size_t off) { T v; memcpy(&v, p + off, sizeof(T)); return v; }

struct Counters {  // GenericActivityProfiler::ErrorCounts, libkineto/src/GenericActivityProfiler.h:528-535
  uint64_t out_of_range = 0, blocklisted_runtime = 0, invalid_external_correlation = 0, unexpected = 0;
  uint64_t x_events = 0, flow_events = 0, records = 0;
};

// ---- runtime/driver callback classification: libkineto/src/CuptiCbidRegistry.cpp:53-258 ----
bool rtFlow(uint32_t c) {
  switch (c) { case 211: case 269: case 272: case 430: case 311: case 131: case 165: case 147: return true; }
  return c >= 31 && c <= 52;
}
bool rtBlocked(uint32_t c) { return c == 17 || c == 16 || c == 10 || c == 133 || c == 134 || c == 136; }
bool drRegistered(uint32_t c) { return c == 307 || c == 652 || c == 549 || c == 551 || c == 552 || c == 550 || c == 554 || c == 555; }
bool drFlow(uint32_t c) { return c == 307 || c == 652; }

const char* memcpyKindStr(uint8_t k) {  // libkineto/src/cupti_strings.cpp:15-41
  static const char* n[] = {nullptr, "HtoD", "DtoH", "HtoA", "AtoH", "AtoA", "AtoD", "DtoA", "DtoD", "HtoH", "PtoP"};
  return (k >= 1 && k <= 10) ? n[k] : "<unknown>";
}
const char* memoryKindStr(uint32_t k) {  // libkineto/src/cupti_strings.cpp:43-66
  static const char* n[] = {"Unknown", "Pageable", "Pinned", "Device", "Array", "Managed", "Device Static", "Managed Static"};
  if (k <= 7) return n[k];
  if (k == 0x7fffffff) return "Force Int";
  return "Unrecognized";
}

// ---- text helpers ----
void appendI(std::string& s, int64_t v) { char b[24]; auto r = std::to_chars(b, b + 24, v); s.append(b, r.ptr); }
void appendU(std::string& s, uint64_t v) { char b[24]; auto r = std::to_chars(b, b + 24, v); s.append(b, r.ptr); }

// Default "{}" formatting of a double in {fmt}: shortest round-trip digits; fixed notation when the
// decimal exponent is in [-4, 16), otherwise d[.ddd]e±XX with at least two exponent digits.
void appendFmtDouble(std::string& s, double v) {
  if (std::isnan(v)) { s += std::signbit(v) ? "-nan" : "nan"; return; }
  if (std::isinf(v)) { s += v < 0 ? "-inf" : "inf"; return; }
  if (std::signbit(v)) { s += '-'; v = -v; }
  if (v == 0) { s += '0'; return; }
  char b[64];
  auto r = std::to_chars(b, b + 64, v, std::chars_format::scientific);
  std::string t(b, r.ptr);  // d[.ddd]e[+-]XX
  size_t epos = t.find('e');
  int e10 = atoi(t.c_str() + epos + 1);
  std::string digits;
  for (size_t i = 0; i < epos; i++) if (t[i] != '.') digits += t[i];
  int nd = (int)digits.size();
  if (e10 < -4 || e10 >= 16) {
    s += digits[0];
    if (nd > 1) { s += '.'; s.append(digits, 1, std::string::npos); }
    s += 'e';
    s += e10 < 0 ? '-' : '+';
    int a = e10 < 0 ? -e10 : e10;
    if (a < 10) s += '0';
    appendI(s, a);
    return;
  }
  if (e10 >= nd - 1) {           // integer: digits then zeros
    s += digits;
    s.append(e10 - (nd - 1), '0');
  } else if (e10 >= 0) {         // d.d with point inside
    s.append(digits, 0, e10 + 1);
    s += '.';
    s.append(digits, e10 + 1, std::string::npos);
  } else {                       // 0.000ddd
    s += "0.";
    s.append(-e10 - 1, '0');
    s += digits;
  }
}
void appendDoubleValue(std::string& s, double v) {  // TypedMetadataJson.h:172-178
  if (std::isfinite(v)) { appendFmtDouble(s, v); return; }
  s += '"'; appendFmtDouble(s, v); s += '"';
}

struct Frag {  // JsonTypedMetadataVisitor
  std::string j; bool first = true;
  void key(const char* k) { if (!first) j += ", "; first = false; j += '"'; j += k; j += "\": "; }
  void key(const std::string& k) { key(k.c_str()); }
  void i64(const char* k, int64_t v) { key(k); appendI(j, v); }
  void u64(const char* k, uint64_t v) { key(k); appendU(j, v); }
  void dbl(const char* k, double v) { key(k); appendDoubleValue(j, v); }
  void str(const char* k, const char* v) { key(k); j += '"'; j += v; j += '"'; }
  void beginDict(const char* k) { key(k); j += '{'; first = true; }
  void endDict() { j += '}'; first = false; }
};

void sanitize(std::string& v) {  // output_json.cpp:72-78
  std::string o; o.reserve(v.size());
  for (char c : v) { if (c == '\n') continue; o += (c == '\\') ? '/' : c; }
  v.swap(o);
}
std::string eventName(std::string n) {  // output_json.cpp:946-949
  if (n == "kernel") n = "Kernel";
  sanitize(n);
  for (unsigned char c : n) if (c < 0x20 || c > 0x7e) { n = "unknown"; break; }
  std::string o;
  for (char c : n) { if (c == '"') o += '\\'; o += c; }
  return o;
}
bool allSpace(const std::string& s) { for (unsigned char c : s) if (!isspace(c)) return false; return true; }

void appendTs(std::string& s, int64_t ns) {  // fmtTs, output_json.cpp:124-126
  appendI(s, ns / 1000);
  s += '.';
  int64_t r = ns % 1000;
  char b[8];
  snprintf(b, sizeof b, "%03" PRId64, r);  // "{:03}" pads to width 3 including a minus sign
  s += b;
}
int64_t sanitizeTid(int64_t t) { return t == INT64_MIN ? 0 : (t < 0 ? -t : t); }

struct Out {
  std::string buf;
  int64_t base;
  Counters* c;
  std::set<int64_t> syncRows;  // syncStreamMetadataEmitted_, output_json.cpp:919-920
  int64_t rel(int64_t t) const { int64_t r = t - base; return r < 0 ? 0 : r; }
  void xEvent(const char* cat, const std::string& name, int64_t pid, int64_t tid, int64_t ts, int64_t dur, const std::string& args) {
    buf += "\n  {\n    \"ph\": \"X\",\n    \"cat\": \""; buf += cat;
    buf += "\",\n    \"name\": \""; buf += name;
    buf += "\",\n    \"pid\": "; appendI(buf, pid);
    buf += ",\n    \"tid\": "; appendI(buf, tid);
    buf += ",\n    \"ts\": "; appendTs(buf, ts);
    buf += ",\n    \"dur\": "; appendTs(buf, dur);
    buf += "\n    ";
    if (!args.empty()) { buf += ",\n    \"args\": {\n      "; buf += args; buf += "\n    }"; }
    buf += "\n  },";
    c->x_events++;
  }
  // writeInstantEvent, libkineto/src/output_json.cpp:261-293, as handleGenericInstantEvent (:660-676) calls it:
  // scope "t", name and metadata exactly as the activity holds them (nothing is sanitised or escaped here).
  void instant(const char* cat, const std::string& name, int64_t pid, int64_t tid, int64_t ts, const std::string& md) {
    buf += "\n  {\n    \"ph\": \"i\",\n    \n    \"cat\": \""; buf += cat;
    buf += "\",\n    \"s\": \"t\",\n    \"name\": \""; buf += name;
    buf += "\",\n    \"pid\": "; appendI(buf, pid);
    buf += ",\n    \"tid\": "; appendI(buf, tid);
    buf += ",\n    \"ts\": "; appendTs(buf, ts);
    buf += "\n    ";
    if (!md.empty() && !allSpace(md)) { buf += ",\n    \"args\": {\n      "; buf += md; buf += "\n    }"; }
    buf += "\n  },";
    c->x_events++;  // counted with the complete events
  }
  // writeCounterEvent, libkineto/src/output_json.cpp:294-316: `pid` is text (a number, or a quoted track name)
  void counter(const char* cat, const std::string& name, const std::string& pid, int64_t tid, int64_t ts, const std::string& args) {
    buf += "\n  {\n    \"ph\": \"C\",\n    \"cat\": \""; buf += cat;
    buf += "\",\n    \"name\": \""; buf += name;
    buf += "\",\n    \"pid\": "; buf += pid;
    buf += ",\n    \"tid\": "; appendI(buf, tid);
    buf += ",\n    \"ts\": "; appendTs(buf, ts);
    buf += ",\n    \"args\": {\n      "; buf += args; buf += "\n    }\n  },";
  }
  void flow(char ph, int64_t id, int64_t pid, int64_t tid, int64_t ts, const char* name) {
    buf += "\n  {\n    \"ph\": \""; buf += ph;
    buf += "\",\n    \"id\": "; appendI(buf, id);
    buf += ",\n    \"pid\": "; appendI(buf, pid);
    buf += ",\n    \"tid\": "; appendI(buf, tid);
    buf += ",\n    \"ts\": "; appendTs(buf, ts);
    buf += ",\n    \"cat\": \""; buf += name; buf += "\",\n    \"name\": \""; buf += name; buf += "\"\n    ";
    if (ph == 'f') buf += ", \"bp\": \"e\"";
    buf += "\n  },";
    c->flow_events++;
  }
};

// handleActivity, output_json.cpp:837-963, for the event shapes this path produces.
struct Event {
  int type; std::string name; int64_t ts, dur, device, resource; bool hasLinked; int64_t linkedId;
  int64_t corrId; std::string md; int64_t flowId; int flowType; bool flowStart;
  bool streamSync = false;  // a CUDA_SYNC activity named "Stream Sync": shown on a row of its own
  std::string extra;        // collective arguments of a kernel launched by record_param_comms: appended as they are
};
constexpr int64_t kSyncStreamTidOffset = 1000000;  // output_json.h:237
void emit(Out& o, const Event& e) {
  int64_t ts = e.ts, dur = e.dur < 0 ? 0 : e.dur;
  if (e.type == T_GPU_USER_ANNOTATION) { ts -= 1; dur += 2; }
  int external = 0;
  if (e.hasLinked) external = (int)e.linkedId;
  else {
    switch (e.type) {
      case T_GPU_MEMCPY: case T_GPU_MEMSET: case T_KERNEL: case T_RUNTIME: case T_DRIVER:
      case T_XPU_RUNTIME: case T_XPU_DRIVER: case T_PU1_RUNTIME: case T_PU1_DRIVER: break;
      default: external = (int)e.corrId;
    }
  }
  std::string args;
  if (external != 0) { args += "\"External id\": "; appendI(args, external); }
  std::string md = e.md;
  sanitize(md);
  if (!md.empty() && !allSpace(md)) { if (!args.empty()) args += ","; args += md; }
  args += e.extra;  // every entry brings its own leading comma: a kernel's own metadata is never empty
  int64_t resource = e.resource;
  if (e.streamSync) {  // output_json.cpp:914-943: two metadata rows the first time a (device, row) pair shows up
    const int64_t syncTid = resource + kSyncStreamTidOffset;
    if (o.syncRows.insert((int64_t)((uint64_t)e.device << 32) | syncTid).second) {
      const int64_t mt = o.rel(ts);
      for (int k = 0; k < 2; k++) {
        o.buf += k == 0 ? "\n  {\n    \"name\": \"thread_name\", \"ph\": \"M\", \"ts\": " : "\n  {\n    \"name\": \"thread_sort_index\", \"ph\": \"M\", \"ts\": ";
        appendTs(o.buf, mt);
        o.buf += ", \"pid\": "; appendI(o.buf, e.device);
        o.buf += ", \"tid\": "; appendI(o.buf, syncTid);
        o.buf += k == 0 ? ",\n    \"args\": {\n      \"name\": \"stream " : ",\n    \"args\": {\n      \"sort_index\": ";
        appendI(o.buf, resource);
        o.buf += k == 0 ? " (sync)\"\n    }\n  }," : "\n    }\n  },";
      }
    }
    resource = syncTid;
  }
  o.xEvent(kTypeNames[e.type], eventName(e.name), e.device, sanitizeTid(resource), o.rel(ts), dur, args);
  if (e.flowId > 0) {
    const char* fname = e.flowType == 1 ? "fwdbwd" : e.flowType == 2 ? "ac2g" : nullptr;
    if (fname) o.flow(e.flowStart ? 's' : 'f', e.flowId, e.device, sanitizeTid(resource), o.rel(e.ts), fname);
  }
}

struct Conv {  // the converter lambda of ApproximateClock.cpp:83-90 with fixed constants
  int mode; int64_t t0; uint64_t t0a; long double scale;
  int64_t operator()(uint64_t t) const {
    if (mode == 0) return (int64_t)t;
    return t > t0a ? static_cast<int64_t>(static_cast<double>(t - t0a) * scale) + t0 : 0;
  }
};

struct Run {
  const K2JTraceFile& tf;
  k2jt_params p;
  Counters c;
  Out out;
  Conv conv;
  std::unordered_map<int64_t, int64_t> cpuCorr, userCorr;
  std::unordered_map<int64_t, size_t> activityMap;  // op id -> op row (last writer wins)
  std::unordered_map<int64_t, bool> globalOps;        // sharded traces: ids of all shards' ops
  std::map<int32_t, int32_t> tidMap;
  struct Span { int64_t start, end; size_t op; int64_t device, resource; };
  std::map<std::pair<int64_t, int64_t>, std::unordered_map<int64_t, Span>> userSpans;
  size_t seg[3] = {0, 0, 0};
  // synchronisation records: context -> device (first writer wins), (context, event) -> CUDA event records
  // ordered by correlation id, the (device, stream) pairs that showed GPU work, deferred stream-wait events
  std::unordered_map<uint32_t, uint32_t> ctxToDev;
  struct WaitInfo { uint32_t stream, corr; };
  std::map<std::pair<uint32_t, uint32_t>, std::vector<WaitInfo>> waitEvents;
  std::set<std::pair<int64_t, int64_t>> seenStreams;
  std::vector<const uint8_t*> deferred;

  explicit Run(const K2JTraceFile& f) : tf(f), p(*f.ptr<k2jt_params>("PARAMS")) {
    out.base = p.base_time_ns; out.c = &c;
    conv = Conv{p.ts_mode, p.conv_t0, p.conv_t0_approx, ldexpl((long double)p.conv_scale_mant, p.conv_scale_exp - 63)};
  }

  std::string opMetadata(size_t i) {
    const uint32_t* off = tf.ptr<uint32_t>("OPMDOFF");
    const k2jt_md_entry* md = tf.ptr<k2jt_md_entry>("MDENT");
    Frag f;
    for (uint32_t e = off[i]; e < off[i + 1]; e++) {
      f.key(tf.str(md[e].key));
      switch (md[e].type) {
        case 0: appendI(f.j, (int64_t)md[e].value); break;
        case 1: appendU(f.j, md[e].value); break;
        case 2: { double d; memcpy(&d, &md[e].value, 8); appendDoubleValue(f.j, d); break; }
        case 3: f.j += md[e].value ? "true" : "false"; break;
        case 4: f.j += '"'; f.j += tf.str((uint32_t)md[e].value); f.j += '"'; break;
        case 5: f.j += tf.str((uint32_t)md[e].value); break;
      }
    }
    return f.j;
  }
  // handleCounterEvent, libkineto/src/output_json.cpp:679-716: the activity's counter values (entries of type 6)
  void counterEvents(const Event& e, size_t i) {
    const uint32_t* off = tf.ptr<uint32_t>("OPMDOFF");
    const k2jt_md_entry* md = tf.ptr<k2jt_md_entry>("MDENT");
    std::string all;
    for (uint32_t k = off[i]; k < off[i + 1]; k++) {
      if (md[k].type != 6) continue;
      double d; memcpy(&d, &md[k].value, 8);
      std::string v; appendFmtDouble(v, d);
      if (e.type == T_HW_COUNTERS) {
        std::string pid = "\"GPU "; appendI(pid, e.device); pid += " Counters\"";
        out.counter(kTypeNames[e.type], tf.str(md[k].key), pid, sanitizeTid(e.resource), out.rel(e.ts), "\"\": " + v);
      } else {
        if (!all.empty()) all += ",";
        all += "\""; all += tf.str(md[k].key); all += "\": "; all += v;
      }
    }
    if (e.type != T_HW_COUNTERS) {
      std::string pid; appendI(pid, e.device);
      out.counter(kTypeNames[e.type], e.name, pid, sanitizeTid(e.resource), out.rel(e.ts), all);
    }
  }

  void cpuOps() {
    size_t n = tf.count<int64_t>("OPSTART");
    for (size_t i = 0; i < n; i++) {
      Event e;
      e.type = tf.ptr<int32_t>("OPTYPE")[i];
      e.name = tf.str(tf.ptr<uint32_t>("OPNAME")[i]);
      e.ts = tf.ptr<int64_t>("OPSTART")[i];
      e.dur = tf.ptr<int64_t>("OPEND")[i] - e.ts;
      e.device = tf.ptr<int32_t>("OPDEV")[i];
      // processCpuTrace rewrites device 0 to the process id right after handing the op to the logger
      // (GenericActivityProfiler.cpp:263-271); the in-memory logger only holds a pointer, so the file
      // written by ActivityTrace::save() shows the rewritten value.
      if (p.mode == 1 && e.device == 0) e.device = p.pid;
      e.resource = tf.ptr<int64_t>("OPRES")[i];
      e.hasLinked = false; e.linkedId = 0;
      e.corrId = tf.ptr<int32_t>("OPID")[i];
      e.md = opMetadata(i);
      e.flowId = tf.ptr<uint32_t>("OPFLOW")[i];
      uint8_t ft = tf.ptr<uint8_t>("OPFLOWT")[i];
      e.flowType = ft & 0xf; e.flowStart = (ft >> 4) & 1;
      // processCpuTrace logs an op only if its type is selected (GenericActivityProfiler.cpp:248);
      // the default selection is types 0..17, GPU_USER_ANNOTATION being switchable by flags bit 0.
      const bool selected = p.mode == 0 || (e.type < 18 && (e.type != T_GPU_USER_ANNOTATION || (p.flags & 1)));
      // an activity that had not ended when the trace stopped ends with the capture window (processCpuTrace,
      // GenericActivityProfiler.cpp:255-258; the "finished": false entry it gains is listed with its metadata)
      if (p.mode == 1 && selected && e.dur < 0) e.dur = p.window_end_ns - e.ts;
      if (selected && e.type == T_CPU_INSTANT)  // handleActivity's early exit, libkineto/src/output_json.cpp:842-845
        out.instant(kTypeNames[e.type], e.name, e.device, sanitizeTid(e.resource), out.rel(e.ts), e.md);
      else if (selected && (e.type == T_MTIA_COUNTERS || e.type == T_XPU_SCOPE || e.type == T_HW_COUNTERS))
        counterEvents(e, i);  // :846-855
      else if (selected) emit(out, e);
      activityMap[e.corrId] = i;
      // recordThreadInfo(resourceId, getThreadId, deviceId), GenericActivityProfiler.cpp:272: only keys
      // of this process are ever looked up; sysTid is an int32 parameter.
      if (e.device == p.pid) tidMap.emplace(tf.ptr<int32_t>("OPTHR")[i], (int32_t)e.resource);
    }
  }

  bool linked(uint32_t corr, int64_t* id) {  // linkedActivity(int32_t, ...), GenericActivityProfiler.cpp:397-408
    auto it = cpuCorr.find((int64_t)(int32_t)corr);
    if (it == cpuCorr.end()) return false;
    if (globalJoin()) {
      if (!globalOps.count(it->second)) return false;
      *id = it->second;
      return true;
    }
    auto it2 = activityMap.find(it->second);
    if (it2 == activityMap.end()) return false;
    *id = tf.ptr<int32_t>("OPID")[it2->second];
    return true;
  }
  // Collective metadata copied from the linked record_param_comms CPU op onto a kernel event
  // (ChromeTraceLogger::appendCollectiveArgs, libkineto/src/output_json.cpp:718-801; handleActivity :900-906).
  // Values are the op's metadata rendered by metadataValueToString (libkineto/src/GenericTraceActivity.cpp:20-47);
  // nothing here is sanitised.  Ops of other shards carry no metadata here, so sharded runs do not enrich.
  std::string mdValue(size_t row, const char* key, bool* found = nullptr) {
    const uint32_t* off = tf.ptr<uint32_t>("OPMDOFF");
    const k2jt_md_entry* md = tf.ptr<k2jt_md_entry>("MDENT");
    for (uint32_t e = off[row]; e < off[row + 1]; e++) {
      if (tf.str(md[e].key) != key) continue;
      if (found) *found = true;
      std::string v;
      switch (md[e].type) {
        case 0: appendI(v, (int64_t)md[e].value); break;
        case 1: appendU(v, md[e].value); break;
        case 2: { double d; memcpy(&d, &md[e].value, 8); appendFmtDouble(v, d); break; }
        case 3: v = md[e].value ? "true" : "false"; break;
        default: v = tf.str((uint32_t)md[e].value); break;
      }
      return v;
    }
    return "";
  }
  static std::string stripQuotes(std::string v) {
    if (v.size() >= 2 && v.front() == '"' && v.back() == '"') { v.pop_back(); v.erase(0, 1); }
    return v;
  }
  std::string collectiveArgs(uint32_t corr) {
    if (globalJoin()) return "";
    auto it = cpuCorr.find((int64_t)(int32_t)corr);
    if (it == cpuCorr.end()) return "";
    auto it2 = activityMap.find(it->second);
    if (it2 == activityMap.end()) return "";
    const size_t row = it2->second;
    if (tf.str(tf.ptr<uint32_t>("OPNAME")[row]) != "record_param_comms") return "";
    std::string a;
    auto raw = [&](const char* k, const std::string& v) { a += ",\""; a += k; a += "\": "; a += v; };
    auto quoted = [&](const char* k, const std::string& v) { a += ",\""; a += k; a += "\": \""; a += v; a += "\""; };
    const std::string name = stripQuotes(mdValue(row, "Collective name")), inMsg = mdValue(row, "In msg nelems"),
                      outMsg = mdValue(row, "Out msg nelems"), groupSize = mdValue(row, "Group size"),
                      dtype = stripQuotes(mdValue(row, "dtype"));
    if (!name.empty() && !inMsg.empty() && !outMsg.empty() && !groupSize.empty() && !dtype.empty()) {
      quoted("Collective name", name); raw("In msg nelems", inMsg); raw("Out msg nelems", outMsg); raw("Group size", groupSize);
      quoted("dtype", dtype);
    }
    const std::string inStart = stripQuotes(mdValue(row, "Input Tensors start")), outStart = stripQuotes(mdValue(row, "Output Tensors start"));
    if (!inStart.empty()) quoted("Input Tensors start", inStart);
    if (!outStart.empty()) quoted("Output Tensors start", outStart);
    const std::string inSplit = stripQuotes(mdValue(row, "In split size")), outSplit = stripQuotes(mdValue(row, "Out split size"));
    if (!inSplit.empty() && !outSplit.empty()) { quoted("In split size", inSplit); quoted("Out split size", outSplit); }
    for (const char* k : {"Process Group Name", "Process Group Description", "Process Group Ranks"}) {
      const std::string v = stripQuotes(mdValue(row, k));
      if (!v.empty()) quoted(k, v);
    }
    for (const char* k : {"Dst Rank", "Src Rank", "Seq", "Comms Id"}) {
      const std::string v = mdValue(row, k);
      if (!v.empty()) raw(k, v);
    }
    return a;
  }
  bool outOfRange(int64_t ts, int64_t dur) {
    bool oor = ts < p.window_start_ns || (ts + dur) > p.window_end_ns;
    if (oor) c.out_of_range++;
    return oor;
  }

  template <class F>
  void forEachRecord(F f) {
    const uint8_t* cu = tf.ptr<uint8_t>("CUPTI");
    const uint64_t* bt = tf.ptr<uint64_t>("BUFTAB");
    size_t nb = tf.count<uint64_t>("BUFTAB") / 2;
    for (size_t b = 0; b < nb; b++) {
      size_t pos = bt[2 * b], end = pos + bt[2 * b + 1];
      while (pos < end) {
        uint32_t kind = rd<uint32_t>(cu, pos);
        size_t sz = recSize(kind);
        f(cu + pos, kind);
        if (!sz) break;  // unknown kind: length unknown, rest of the buffer cannot be walked
        pos += sz;
      }
    }
  }

  // Sharded traces: the correlation maps and the CPU-op id set come from the arrays gathered from all
  // shards (sections GEXT: {external id, correlation id | external kind << 32} pairs; GOPS: op ids).
  bool globalJoin() const { return tf.has("GEXT") || tf.has("GOPS"); }
  void pass1Global() {
    const uint64_t* g = tf.ptr<uint64_t>("GEXT");
    for (size_t i = 0; i < tf.count<uint64_t>("GEXT") / 2; i++) {
      int64_t ext = (int64_t)g[2 * i];
      int64_t corr = (uint32_t)g[2 * i + 1];
      uint32_t ek = (uint32_t)(g[2 * i + 1] >> 32);
      if (ek == 3) cpuCorr[corr] = ext;
      else if (ek == 4) userCorr[corr] = ext;
    }
    const int32_t* ids = tf.ptr<int32_t>("GOPS");
    for (size_t i = 0; i < tf.count<int32_t>("GOPS"); i++) globalOps[ids[i]] = true;
    // invalid external kinds are counted by the shard that owns the record
    forEachRecord([&](const uint8_t* r, uint32_t kind) {
      if (kind == K_EXTCORR) { uint32_t ek = rd<uint32_t>(r, 4); if (ek != 3 && ek != 4) c.invalid_external_correlation++; }
    });
  }
  void noteCtx(uint32_t ctx, uint32_t dev) { ctxToDev.emplace(ctx, dev); }  // updateCtxToDeviceId, CuptiActivityProfiler.cpp:221-239
  void pass1Sync() {  // the rest of buildProcessingState, CuptiActivityProfiler.cpp:256-287
    forEachRecord([&](const uint8_t* r, uint32_t kind) {
      switch (kind) {
        case K_KERNEL: noteCtx(rd<uint32_t>(r, 44), rd<uint32_t>(r, 40)); break;
        case K_MEMCPY: case K_MEMSET: noteCtx(rd<uint32_t>(r, 36), rd<uint32_t>(r, 32)); break;
        case K_MEMCPY2: noteCtx(rd<uint32_t>(r, 48), rd<uint32_t>(r, 44)); noteCtx(rd<uint32_t>(r, 56), rd<uint32_t>(r, 52)); break;
        case K_CUDA_EVENT: {  // updateWaitEventMap, :243-254: kept sorted by correlation id, a new record goes before its equals
          auto& v = waitEvents[{rd<uint32_t>(r, 8), rd<uint32_t>(r, 16)}];
          const uint32_t corr = rd<uint32_t>(r, 4);
          auto pos = std::lower_bound(v.begin(), v.end(), corr, [](const WaitInfo& w, uint32_t c) { return w.corr < c; });
          v.insert(pos, WaitInfo{rd<uint32_t>(r, 12), corr});
          break;
        }
        default: break;
      }
    });
  }
  uint32_t ctxDevice(uint32_t ctx) const { auto it = ctxToDev.find(ctx); return it == ctxToDev.end() ? 0 : it->second; }
  static int32_t streamForTrace(uint32_t s) { return (int32_t)s; }  // streamIdForTrace, CuptiActivity.h:316-323
  static const char* syncTypeStr(uint32_t t) {  // libkineto/src/cupti_strings.cpp:137-151
    return t == 1 ? "Event Sync" : t == 2 ? "Stream Wait Event" : t == 3 ? "Stream Sync" : t == 4 ? "Context Sync" : "Unknown Sync";
  }
  void cudaEventRecord(const uint8_t* r) {  // handleCudaEventActivity, CuptiActivityProfiler.cpp:404-434
    Event e; e.type = T_CUDA_EVENT; e.name = "cudaEvent";
    const uint32_t corr = rd<uint32_t>(r, 4), ctx = rd<uint32_t>(r, 8), stream = rd<uint32_t>(r, 12);
    e.ts = conv(rd<uint64_t>(r, 40)); e.dur = 1;
    e.device = ctxDevice(ctx); e.resource = streamForTrace(stream);
    e.hasLinked = linked(corr, &e.linkedId);
    e.corrId = corr; e.flowId = corr; e.flowType = 2; e.flowStart = false;
    if (outOfRange(e.ts, e.dur)) return;
    Frag f;
    f.u64("event_id", rd<uint32_t>(r, 16)); f.i64("stream", streamForTrace(stream)); f.u64("correlation", corr);
    f.i64("device", e.device); f.u64("context", ctx);
    e.md = f.j;
    emit(out, e);
  }
  void logSync(const uint8_t* r) {  // the log_event functor of handleCudaSyncActivity, CuptiActivityProfiler.cpp:464-486
    const uint32_t type = rd<uint32_t>(r, 4), corr = rd<uint32_t>(r, 24), ctx = rd<uint32_t>(r, 28), stream = rd<uint32_t>(r, 32);
    const uint32_t event = rd<uint32_t>(r, 36);
    int32_t srcStream = -1, srcCorr = -1;
    const bool eventSync = type == 1 || type == 2;
    if (eventSync) {  // getWaitEventInfo, :379-402: the last record whose correlation id is not above the query's
      auto it = waitEvents.find({ctx, event});
      if (it != waitEvents.end()) {
        const auto& v = it->second;
        auto pos = std::upper_bound(v.begin(), v.end(), corr, [](uint32_t c, const WaitInfo& w) { return c < w.corr; });
        if (pos != v.begin()) { srcStream = (int32_t)std::prev(pos)->stream; srcCorr = (int32_t)std::prev(pos)->corr; }
      }
    }
    Event e; e.type = T_CUDA_SYNC; e.name = syncTypeStr(type);
    const uint64_t st = rd<uint64_t>(r, 8), en = rd<uint64_t>(r, 16);
    e.ts = conv(st); e.dur = p.ts_mode ? conv(en) - conv(st) : (int64_t)(en - st);
    e.device = ctxDevice(ctx); e.resource = streamForTrace(stream);
    e.hasLinked = linked(corr, &e.linkedId);
    e.corrId = corr; e.flowId = corr; e.flowType = 2; e.flowStart = false;
    e.streamSync = type == 3;
    if (outOfRange(e.ts, e.dur)) return;
    Frag f;
    f.str("cuda_sync_kind", syncTypeStr(type));
    if (eventSync) {
      f.i64("wait_on_stream", srcStream); f.i64("wait_on_cuda_event_record_corr_id", srcCorr); f.u64("wait_on_cuda_event_id", event);
    }
    f.i64("stream", streamForTrace(stream)); f.u64("correlation", corr); f.i64("device", e.device); f.u64("context", ctx);
    e.md = f.j;
    emit(out, e);
  }
  void syncRecord(const uint8_t* r) {  // handleCudaSyncActivity: stream-wait events wait for the end of the pass
    if (rd<uint32_t>(r, 4) == 2) deferred.push_back(r);
    else logSync(r);
  }
  void deferredSyncs() {  // logDeferredEvents, CuptiActivityProfiler.cpp:502-514
    for (const uint8_t* r : deferred)
      if (seenStreams.count({(int64_t)ctxDevice(rd<uint32_t>(r, 28)), (int64_t)rd<uint32_t>(r, 32)})) logSync(r);
  }
  void pass1() {
    forEachRecord([&](const uint8_t* r, uint32_t kind) {
      if (kind != K_EXTCORR) return;
      uint32_t ek = rd<uint32_t>(r, 4);
      int64_t ext = (int64_t)rd<uint64_t>(r, 8);
      int64_t corr = rd<uint32_t>(r, 16);
      if (ek == 3) cpuCorr[corr] = ext;
      else if (ek == 4) userCorr[corr] = ext;
      else c.invalid_external_correlation++;
    });
  }

  void apiRecord(const uint8_t* r, bool driver) {
    uint32_t cbid = rd<uint32_t>(r, 4);
    if (!driver) { if (rtBlocked(cbid)) { c.blocklisted_runtime++; return; } }
    else if (!drRegistered(cbid)) return;
    Event e;
    e.type = driver ? T_DRIVER : T_RUNTIME;
    const uint32_t* nt = tf.ptr<uint32_t>(driver ? "DRNAME" : "RTNAME");
    size_t nn = tf.count<uint32_t>(driver ? "DRNAME" : "RTNAME");
    e.name = cbid < nn ? tf.str(nt[cbid]) : "INVALID";
    uint64_t s = rd<uint64_t>(r, 8), en = rd<uint64_t>(r, 16);
    e.ts = conv(s);
    e.dur = p.ts_mode ? conv(en) - conv(s) : (int64_t)(en - s);
    int32_t tid = (int32_t)rd<uint32_t>(r, 28);
    auto it = tidMap.find(tid);
    if (it != tidMap.end()) tid = it->second;
    e.device = p.pid; e.resource = tid;
    uint32_t corr = rd<uint32_t>(r, 32);
    e.hasLinked = linked(corr, &e.linkedId);
    e.corrId = corr;
    if (outOfRange(e.ts, e.dur)) return;
    Frag f;
    f.u64("cbid", cbid); f.u64("correlation", corr);
    e.md = f.j;
    e.flowId = corr; e.flowType = 2; e.flowStart = driver ? drFlow(cbid) : rtFlow(cbid);
    emit(out, e);
  }

  void gpuCommon(Event& e, uint32_t corr, uint64_t s, uint64_t en, int64_t device, int64_t stream) {
    e.ts = conv(s);
    e.dur = p.ts_mode ? conv(en) - conv(s) : (int64_t)(en - s);
    e.device = device; e.resource = stream;
    e.hasLinked = linked(corr, &e.linkedId);
    e.corrId = corr; e.flowId = corr; e.flowType = 2; e.flowStart = false;
  }
  void afterGpu(const Event& e) {  // GenericActivityProfiler.cpp:419, :424-434
    seenStreams.insert({e.device, e.resource});
    if (!(p.flags & 1)) return;
    auto it = userCorr.find(e.corrId);
    if (it == userCorr.end()) return;
    auto it2 = activityMap.find(it->second);
    if (it2 == activityMap.end()) return;
    int64_t opId = tf.ptr<int32_t>("OPID")[it2->second];
    auto& m = userSpans[{e.device, e.resource}];
    auto f = m.find(opId);
    if (f == m.end()) f = m.insert({opId, Span{e.ts, e.ts + e.dur, it2->second, e.device, e.resource}}).first;
    Span& sp = f->second;
    if (e.ts < sp.start || sp.start == 0) sp.start = e.ts;
    sp.end = std::max(e.ts + e.dur, sp.end);
  }
  void graphAndChannel(Frag& f, uint32_t graphId, uint64_t node, uint32_t ch, uint32_t chType) {
    f.u64("graph id", graphId); f.u64("graph node id", node); f.u64("channel", ch); f.i64("channel_type", (int64_t)chType);
  }

  void kernelRecord(const uint8_t* r) {
    Event e; e.type = T_KERNEL;
    uint32_t dev = rd<uint32_t>(r, 40), ctx = rd<uint32_t>(r, 44), stream = rd<uint32_t>(r, 48), corr = rd<uint32_t>(r, 92);
    gpuCommon(e, corr, rd<uint64_t>(r, 16), rd<uint64_t>(r, 24), dev, stream);
    if (outOfRange(e.ts, e.dur)) return;
    e.name = tf.str((uint32_t)rd<uint64_t>(r, 104));
    int32_t gx = rd<int32_t>(r, 52), gy = rd<int32_t>(r, 56), gz = rd<int32_t>(r, 60);
    int32_t bx = rd<int32_t>(r, 64), by = rd<int32_t>(r, 68), bz = rd<int32_t>(r, 72);
    int32_t ssm = rd<int32_t>(r, 76), dsm = rd<int32_t>(r, 80);
    uint16_t regs = rd<uint16_t>(r, 6);
    const k2jt_device_props* dp = tf.ptr<k2jt_device_props>("DEVPROPS");
    int smCount = dev < (uint32_t)p.n_devices ? dp[dev].num_sms : 0;
    // blocksPerSm / warpsPerSm, DeviceProperties.cpp:161-174 (32-bit wrapping products, float math)
    int32_t gridProd = (int32_t)((uint32_t)gx * (uint32_t)gy * (uint32_t)gz);
    int32_t blockProd = (int32_t)((uint32_t)bx * (uint32_t)by * (uint32_t)bz);
    float bps = smCount == 0 ? INFINITY : gridProd / static_cast<float>(smCount);
    float wps = bps * blockProd / 32;
    // computeOccupancyMetrics, DeviceProperties.cpp:176-222
    cudaOccResult occ{};  // zero-initialised like OccupancyMetrics' default member
    float occupancy = -1.0f;  // OccupancyMetrics default, DeviceProperties.h:54
    if (dev < (uint32_t)p.n_devices) {
      float blocksPerSm = -1.0f;
      if (smCount != 0) blocksPerSm = gridProd / static_cast<float>(smCount);
      cudaOccFuncAttributes fa;
      fa.maxThreadsPerBlock = INT_MAX; fa.numRegs = regs; fa.sharedSizeBytes = ssm;
      fa.partitionedGCConfig = PARTITIONED_GC_OFF; fa.shmemLimitConfig = FUNC_SHMEM_LIMIT_DEFAULT;
      fa.maxDynamicSharedSizeBytes = 0;
      fa.numBlockBarriers = 0;
      const cudaOccDeviceState st = {};
      cudaOccDeviceProp prop;
      prop.computeMajor = dp[dev].major; prop.computeMinor = dp[dev].minor;
      prop.maxThreadsPerBlock = dp[dev].max_threads_per_block;
      prop.maxThreadsPerMultiprocessor = dp[dev].max_threads_per_sm;
      prop.regsPerBlock = dp[dev].regs_per_block; prop.regsPerMultiprocessor = dp[dev].regs_per_sm;
      prop.warpSize = dp[dev].warp_size; prop.sharedMemPerBlock = dp[dev].smem_per_block;
      prop.sharedMemPerMultiprocessor = dp[dev].smem_per_sm; prop.numSms = dp[dev].num_sms;
      prop.sharedMemPerBlockOptin = dp[dev].smem_per_block_optin;
      prop.reservedSharedMemPerBlock = dp[dev].reserved_smem_per_block;
      cudaOccError status = cudaOccMaxActiveBlocksPerMultiprocessor(&occ, &prop, &fa, &st, blockProd, (size_t)dsm);
      if (status == CUDA_OCC_SUCCESS) {
        float eff = std::min<float>((float)occ.activeBlocksPerMultiprocessor, blocksPerSm);
        occupancy = eff * blockProd / static_cast<float>(dp[dev].max_threads_per_sm);
      }
    }
    Frag f;
    f.u64("queued", rd<uint64_t>(r, 120)); f.i64("device", dev); f.u64("context", ctx); f.i64("stream", stream);
    f.u64("correlation", corr); f.u64("registers per thread", regs);
    f.i64("shared memory", (int64_t)(int32_t)((uint32_t)ssm + (uint32_t)dsm));
    f.dbl("blocks per SM", (double)bps); f.dbl("warps per SM", (double)wps);
    f.key("grid"); f.j += '['; appendI(f.j, gx); f.j += ", "; appendI(f.j, gy); f.j += ", "; appendI(f.j, gz); f.j += ']';
    f.key("block"); f.j += '['; appendI(f.j, bx); f.j += ", "; appendI(f.j, by); f.j += ", "; appendI(f.j, bz); f.j += ']';
    f.i64("est. achieved occupancy %", (int64_t)std::lround(occupancy * 100.0));
    f.beginDict("occupancy");
    f.i64("activeBlocksPerMultiprocessor", occ.activeBlocksPerMultiprocessor);
    {
      std::string lf;
      unsigned fac = occ.limitingFactors;
      if (fac == 0) lf = "none";
      else {
        const std::pair<unsigned, const char*> k[] = {{OCC_LIMIT_WARPS, "WARPS"}, {OCC_LIMIT_REGISTERS, "REGS"},
            {OCC_LIMIT_SHARED_MEMORY, "SMEM"}, {OCC_LIMIT_BLOCKS, "BLOCKS"}, {OCC_LIMIT_BARRIERS, "BARRIERS"}};
        for (auto& [m, n] : k) if (fac & m) { if (!lf.empty()) lf += "|"; lf += n; }
      }
      f.str("limitingFactors", lf.c_str());
    }
    f.i64("blockLimitRegs", occ.blockLimitRegs); f.i64("blockLimitSharedMem", occ.blockLimitSharedMem);
    f.i64("blockLimitWarps", occ.blockLimitWarps); f.i64("blockLimitBlocks", occ.blockLimitBlocks);
    f.i64("blockLimitBarriers", occ.blockLimitBarriers);
    f.i64("allocatedRegistersPerBlock", occ.allocatedRegistersPerBlock);
    f.u64("allocatedSharedMemPerBlock", occ.allocatedSharedMemPerBlock);
    f.endDict();
    graphAndChannel(f, rd<uint32_t>(r, 156), rd<uint64_t>(r, 144), rd<uint32_t>(r, 168), rd<uint32_t>(r, 172));
    e.md = f.j;
    e.extra = collectiveArgs(corr);
    emit(out, e);
    afterGpu(e);
  }

  void bandwidth(Frag& f, uint64_t bytes, int64_t dur) {  // CuptiActivity.h:460-470
    if (dur == 0) return;
    f.dbl("memory bandwidth (GB/s)", static_cast<double>(bytes) / static_cast<double>(dur));
  }
  std::string memcpyName(const uint8_t* r) {
    return std::string("Memcpy ") + memcpyKindStr(r[4]) + " (" + memoryKindStr(r[5]) + " -> " + memoryKindStr(r[6]) + ")";
  }
  void memcpyRecord(const uint8_t* r) {
    Event e; e.type = T_GPU_MEMCPY;
    uint32_t dev = rd<uint32_t>(r, 32), ctx = rd<uint32_t>(r, 36), stream = rd<uint32_t>(r, 40), corr = rd<uint32_t>(r, 44);
    gpuCommon(e, corr, rd<uint64_t>(r, 16), rd<uint64_t>(r, 24), dev, stream);
    if (outOfRange(e.ts, e.dur)) return;
    e.name = memcpyName(r);
    uint64_t bytes = rd<uint64_t>(r, 8);
    Frag f;
    f.i64("device", dev); f.u64("context", ctx); f.i64("stream", stream); f.u64("correlation", corr); f.u64("bytes", bytes);
    bandwidth(f, bytes, e.dur);
    graphAndChannel(f, rd<uint32_t>(r, 72), rd<uint64_t>(r, 64), rd<uint32_t>(r, 76), rd<uint32_t>(r, 80));
    e.md = f.j; emit(out, e); afterGpu(e);
  }
  void memcpy2Record(const uint8_t* r) {
    Event e; e.type = T_GPU_MEMCPY;
    uint32_t dev = rd<uint32_t>(r, 32), ctx = rd<uint32_t>(r, 36), stream = rd<uint32_t>(r, 40), corr = rd<uint32_t>(r, 60);
    gpuCommon(e, corr, rd<uint64_t>(r, 16), rd<uint64_t>(r, 24), dev, stream);
    if (outOfRange(e.ts, e.dur)) return;
    e.name = memcpyName(r);
    uint64_t bytes = rd<uint64_t>(r, 8);
    Frag f;
    f.u64("fromDevice", rd<uint32_t>(r, 44)); f.u64("inDevice", dev); f.u64("toDevice", rd<uint32_t>(r, 52));
    f.u64("fromContext", rd<uint32_t>(r, 48)); f.u64("inContext", ctx); f.u64("toContext", rd<uint32_t>(r, 56));
    f.i64("stream", stream); f.u64("correlation", corr); f.u64("bytes", bytes);
    bandwidth(f, bytes, e.dur);
    graphAndChannel(f, rd<uint32_t>(r, 80), rd<uint64_t>(r, 72), rd<uint32_t>(r, 84), rd<uint32_t>(r, 88));
    e.md = f.j; emit(out, e); afterGpu(e);
  }
  void memsetRecord(const uint8_t* r) {
    Event e; e.type = T_GPU_MEMSET;
    uint32_t dev = rd<uint32_t>(r, 32), ctx = rd<uint32_t>(r, 36), stream = rd<uint32_t>(r, 40), corr = rd<uint32_t>(r, 44);
    gpuCommon(e, corr, rd<uint64_t>(r, 16), rd<uint64_t>(r, 24), dev, stream);
    if (outOfRange(e.ts, e.dur)) return;
    e.name = std::string("Memset (") + memoryKindStr(rd<uint16_t>(r, 50)) + ")";
    uint64_t bytes = rd<uint64_t>(r, 8);
    Frag f;
    f.i64("device", dev); f.u64("context", ctx); f.i64("stream", stream); f.u64("correlation", corr); f.u64("bytes", bytes);
    bandwidth(f, bytes, e.dur);
    graphAndChannel(f, rd<uint32_t>(r, 72), rd<uint64_t>(r, 64), rd<uint32_t>(r, 76), rd<uint32_t>(r, 80));
    e.md = f.j; emit(out, e); afterGpu(e);
  }

  // handleOverheadActivity (libkineto/src/CuptiActivityProfiler.cpp:360-377) with OverheadActivity
  // (libkineto/src/CuptiActivity.h:144-179): device -1, resource 0, no correlation id, no metadata, no link.
  static const char* overheadKindStr(uint32_t k) {  // libkineto/src/cupti_strings.cpp:68-97
    switch (k) {
      case 0: return "Unknown";
      case 1: return "Driver Compiler";
      case 1u << 16: return "Buffer Flush";
      case 2u << 16: return "Instrumentation";
      case 3u << 16: return "Resource";
      case 4u << 16: return "Runtime Triggered Module Loading";
      case 5u << 16: return "Lazy Function Loading";
      case 6u << 16: return "Command Buffer Full";
      case 7u << 16: return "Activity Buffer Request";
      case 0x7fffffffu: return "Force Int";
      default: return "Unrecognized";
    }
  }
  void overheadRecord(const uint8_t* r) {
    Event e; e.type = T_OVERHEAD;
    e.name = overheadKindStr(rd<uint32_t>(r, 4));
    const uint64_t st = rd<uint64_t>(r, 24), en = rd<uint64_t>(r, 32);
    e.ts = conv(st); e.dur = p.ts_mode ? conv(en) - conv(st) : (int64_t)(en - st);
    e.device = -1; e.resource = 0; e.hasLinked = false; e.linkedId = 0; e.corrId = 0;
    e.flowId = 0; e.flowType = 0; e.flowStart = false;
    if (outOfRange(e.ts, e.dur)) return;
    emit(out, e);
  }

  int64_t recordStart(const uint8_t* r, uint32_t kind) {
    switch (kind) {
      case K_OVERHEAD: return conv(rd<uint64_t>(r, 24));
      case K_RUNTIME: case K_DRIVER: return conv(rd<uint64_t>(r, 8));
      case K_KERNEL: case K_MEMCPY: case K_MEMCPY2: case K_MEMSET: return conv(rd<uint64_t>(r, 16));
      case K_SYNC: return conv(rd<uint64_t>(r, 8));
      case K_CUDA_EVENT: return conv(rd<uint64_t>(r, 40));
      default: return INT64_MIN;
    }
  }
  void pass2() {
    // flags bit 1: the records are first put in stable order of their converted start timestamp (the
    // reference itself never sorts: this equals running it on pre-sorted buffers).
    std::vector<std::pair<const uint8_t*, uint32_t>> recs;
    forEachRecord([&](const uint8_t* r, uint32_t kind) { recs.push_back({r, kind}); });
    if (p.flags & 2) {
      std::stable_sort(recs.begin(), recs.end(), [&](const auto& a, const auto& b) {
        return recordStart(a.first, a.second) < recordStart(b.first, b.second);
      });
    }
    for (auto& [r, kind] : recs) {
      c.records++;
      switch (kind) {
        case K_EXTCORR: break;
        case K_RUNTIME: apiRecord(r, false); break;
        case K_DRIVER: apiRecord(r, true); break;
        case K_KERNEL: kernelRecord(r); break;
        case K_MEMCPY: memcpyRecord(r); break;
        case K_MEMCPY2: memcpy2Record(r); break;
        case K_MEMSET: memsetRecord(r); break;
        case K_OVERHEAD: overheadRecord(r); break;
        case K_SYNC: syncRecord(r); break;
        case K_CUDA_EVENT: cudaEventRecord(r); break;
        default: c.unexpected++; break;
      }
    }
    deferredSyncs();
  }

  void annotations() {  // GpuUserEventMap::logEvents, GenericActivityProfiler.cpp:320-327
    for (auto& [key, m] : userSpans)
      for (auto& [opId, sp] : m) {
        Event e; e.type = T_GPU_USER_ANNOTATION;
        e.name = tf.str(tf.ptr<uint32_t>("OPNAME")[sp.op]);
        e.ts = sp.start; e.dur = sp.end - sp.start; e.device = sp.device; e.resource = sp.resource;
        e.hasLinked = false; e.linkedId = 0; e.corrId = opId; e.flowId = 0; e.flowType = 0; e.flowStart = false;
        emit(out, e);
      }
  }

  void run() {
    const int32_t* tm = tf.ptr<int32_t>("TIDMAP");
    for (size_t i = 0; i < tf.count<int32_t>("TIDMAP") / 2; i++) tidMap.emplace(tm[2 * i], tm[2 * i + 1]);
    cpuOps();
    seg[0] = out.buf.size();
    if (p.mode != 0) { if (globalJoin()) pass1Global(); else pass1(); pass1Sync(); pass2(); }
    seg[1] = out.buf.size();
    if (p.mode != 0) annotations();
    seg[2] = out.buf.size();
  }
};

} // namespace

extern "C" {

// Runs the restatement over a trace container held in memory.  On success returns 0, stores a
// malloc'd buffer with the activities text in *out (caller frees with k2j_oracle_free) and fills
// stats[0..9] = {out bytes, cpu-op segment end, gpu segment end, X events, flow events, records,
// out_of_range, blocklisted_runtime, invalid_external_correlation, unexpected kinds}.
int k2j_oracle_run_file(const char* path, char** out, uint64_t* stats) {
  try {
    K2JTraceFile tf(path);
    Run r(tf);
    r.run();
    *out = (char*)malloc(r.out.buf.size() + 1);
    memcpy(*out, r.out.buf.data(), r.out.buf.size());
    stats[0] = r.out.buf.size(); stats[1] = r.seg[0]; stats[2] = r.seg[1];
    stats[3] = r.c.x_events; stats[4] = r.c.flow_events; stats[5] = r.c.records;
    stats[6] = r.c.out_of_range; stats[7] = r.c.blocklisted_runtime; stats[8] = r.c.invalid_external_correlation;
    stats[9] = r.c.unexpected;
    return 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "k2j_oracle: %s\n", e.what());
    return 1;
  }
}
void k2j_oracle_free(char* p) { free(p); }

// "{}" formatting of doubles, exposed so the formatting rule can be checked in isolation.
int k2j_oracle_fmt_double(double v, char* buf, int cap) {
  std::string s;
  appendFmtDouble(s, v);
  if ((int)s.size() >= cap) return -1;
  memcpy(buf, s.c_str(), s.size() + 1);
  return (int)s.size();
}
}
