// See output_b200.h.  Reference behaviour being matched (paths relative to the reference project):
//   file layout and host-written rows   libkineto/src/output_json.cpp:214-235, :261-292, :445-479, :507-658, :1066-1108
//   arrival order of the calls          libkineto/src/output_membuf.h:91-107 (save) and
//                                       libkineto/src/GenericActivityProfiler.cpp:178-275, :655-740 (direct)
#include "output_b200.h"

#include <fmt/format.h>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <thread>
#include <typeinfo>

#include <cuda_runtime_api.h>

#include "CuptiActivity.h"
#include "EnvMetadata.h"
#include "GenericTraceActivity.h"
#include "Logger.h"
#include "ThreadUtil.h"
#include "TraceSpan.h"
#include "TypedMetadataJson.h"
#include "cupti_strings.h"
#include "output_json.h"

#include "k2j.h"

namespace KINETO_NAMESPACE {

namespace {

void sanitize(std::string& v) {  // backslash -> slash, newlines dropped
  std::string o;
  o.reserve(v.size());
  for (char c : v) {
    if (c == '\n') continue;
    o += c == '\\' ? '/' : c;
  }
  v.swap(o);
}
void escapeQuotes(std::string& v) {
  std::string o;
  o.reserve(v.size() + 8);
  for (char c : v) {
    if (c == '"') o += '\\';
    o += c;
  }
  v.swap(o);
}
std::string ts(int64_t ns) { return fmt::format("{}.{:03}", ns / 1000, ns % 1000); }
int64_t rel(int64_t t) {
  int64_t r = t - ChromeTraceBaseTime::singleton().get();
  return r < 0 ? 0 : r;
}
int64_t absTid(int64_t t) { return t == INT64_MIN ? 0 : (t < 0 ? -t : t); }

std::string metaRow(const std::string& name, int64_t time, const std::string& pid, const std::string& tid,
                    const std::string& key, const std::string& value) {
  return fmt::format(
      "\n  {{\n    \"ph\": \"M\",\n    \"name\": \"{}\",\n    \"ts\": {},\n    \"pid\": {},\n    \"tid\": {},\n    \"args\": {{\n      \"{}\": {}\n    }}\n  }},",
      name, ts(time), pid, tid, key, value);
}
std::string instantRow(const std::string& name, const std::string& pid, const std::string& tid, int64_t time, bool last) {
  return fmt::format(
      "\n  {{\n    \"ph\": \"i\",\n    \n    \"s\": \"g\",\n    \"name\": \"{}\",\n    \"pid\": {},\n    \"tid\": {},\n    \"ts\": {}\n    \n  }}{}",
      name, pid, tid, ts(time), last ? "" : ",");
}

// Typed metadata of a GenericTraceActivity in visit order.
struct MdCollector final : public libkineto::ITypedMetadataVisitor {
  // Keys and string values are views into the visited activity (alive for the duration of the visit and of the
  // interning that follows); only rendered collections own their text.
  struct Entry { std::string_view key; uint32_t type; uint64_t value; std::string_view text; };
  std::vector<Entry> entries;
  std::deque<std::string> owned;
  void visitValue(const MetadataField<int64_t>& f, int64_t v) override { entries.push_back({f.name, K2J_MD_INT64, (uint64_t)v, {}}); }
  void visitValue(const MetadataField<double>& f, double v) override {
    uint64_t b; memcpy(&b, &v, 8);
    entries.push_back({f.name, K2J_MD_DOUBLE, b, {}});
  }
  void visitValue(const MetadataField<bool>& f, bool v) override { entries.push_back({f.name, K2J_MD_BOOL, v ? 1u : 0u, {}}); }
  void visitValue(const MetadataField<std::string>& f, std::string_view v) override { entries.push_back({f.name, K2J_MD_STRING, 0, v}); }
  void visitValue(const MetadataField<std::vector<int64_t>>& f, const std::vector<int64_t>& v) override { raw(f.name, v); }
  void visitValue(const MetadataField<std::vector<std::string>>& f, const std::vector<std::string>& v) override { raw(f.name, v); }
  void visitValue(const MetadataField<RawJson>& f, const RawJson& v) override { entries.push_back({f.name, K2J_MD_RAWJSON, 0, v.value}); }
  void visitValue(const MetadataField<uint64_t>& f, uint64_t v) override { entries.push_back({f.name, K2J_MD_UINT64, v, {}}); }
  void visitValue(const MetadataField<InputShapes>& f, const InputShapes& v) override { raw(f.name, v); }
  void visitUnsupported(std::string_view name) override { entries.push_back({name, K2J_MD_STRING, 0, "<unsupported metadata type>"}); }
  void beginDict(std::string_view) override {}
  void endDict() override {}
  template <class T> void raw(std::string_view name, const T& v) {  // collections: text once, as the reference renders them
    owned.emplace_back();
    libkineto::internal::JsonTypedMetadataVisitor::appendArray(owned.back(), v);
    entries.push_back({name, K2J_MD_RAWJSON, 0, owned.back()});
  }
};

}  // namespace

// Wall-clock breakdown of the logger's host side, printed at finalizeTrace when K2J_SHIM_TIMING is set.
struct Stopwatch {
  double total = 0;
  std::chrono::steady_clock::time_point t0;
  void start() { t0 = std::chrono::steady_clock::now(); }
  void stop() { total += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count(); }
};
struct Timed {
  Stopwatch& w;
  explicit Timed(Stopwatch& sw) : w(sw) { w.start(); }
  ~Timed() { w.stop(); }
};

// k2j contexts outlive the loggers that use them: a logger is created per ActivityTrace::save(), while a context's
// workspaces on the GPU are grow-only and cost tens of milliseconds to allocate.  A finished logger hands its
// context back; the next logger on that device takes it.  Contexts are kept until the process exits.
struct ContextPool {
  static std::mutex& mu() { static std::mutex m; return m; }
  // the occupancy fields need the properties of every device: read once per process, not once per flush
  static const std::vector<k2j_device_props>& deviceProps() {
    static const std::vector<k2j_device_props> props = [] {
      std::vector<k2j_device_props> v;
      int ndev = 0;
      if (cudaGetDeviceCount(&ndev) != cudaSuccess) ndev = 0;
      for (int i = 0; i < ndev; i++) {
        cudaDeviceProp dp;
        if (cudaGetDeviceProperties(&dp, i) != cudaSuccess) break;
        v.push_back({dp.major, dp.minor, dp.maxThreadsPerBlock, dp.maxThreadsPerMultiProcessor, dp.regsPerBlock,
                     dp.regsPerMultiprocessor, dp.warpSize, dp.multiProcessorCount, dp.sharedMemPerBlock,
                     dp.sharedMemPerBlockOptin, dp.sharedMemPerMultiprocessor, dp.reservedSharedMemPerBlock});
      }
      return v;
    }();
    return props;
  }
  static std::vector<std::pair<int, k2j_ctx*>>& free() { static std::vector<std::pair<int, k2j_ctx*>> v; return v; }
  static k2j_ctx* take(int device) {
    {
      std::lock_guard<std::mutex> g(mu());
      auto& v = free();
      for (size_t i = 0; i < v.size(); i++)
        if (v[i].first == device) { k2j_ctx* c = v[i].second; v.erase(v.begin() + i); return c; }
    }
    k2j_ctx* c = nullptr;
    return k2j_create(device, nullptr, &c) == K2J_OK ? c : nullptr;
  }
  static void give(int device, k2j_ctx* c) {
    if (!c) return;
    std::lock_guard<std::mutex> g(mu());
    free().push_back({device, c});
  }
};

struct B200TraceLogger::Impl {
  Stopwatch tOps, tRecords, tSetup, tRun, tWrite;
  std::string fileName, tempFileName;
  FILE* out = nullptr;
  k2j_ctx* ctx = nullptr;
  int device = 0;

  // string pool shared by all runs
  struct SvHash {
    using is_transparent = void;
    size_t operator()(std::string_view v) const { return std::hash<std::string_view>{}(v); }
  };
  std::unordered_map<std::string, uint32_t, SvHash, std::equal_to<>> ids;  // looked up by view: no copy per call
  std::vector<uint64_t> poolOff{0};
  std::vector<uint8_t> poolData;
  uint32_t intern(std::string_view s) {
    auto it = ids.find(s);
    if (it != ids.end()) return it->second;
    uint32_t id = (uint32_t)ids.size();
    ids.emplace(std::string(s), id);
    poolData.insert(poolData.end(), s.begin(), s.end());
    poolOff.push_back(poolData.size());
    return id;
  }
  std::unordered_map<const void*, uint32_t> kernelNameIds;  // raw name pointer -> id of the demangled name
  std::vector<uint32_t> rtNames, drNames;                    // cbid -> string id (filled on demand)
  uint32_t invalidId = 0;

  // one run = CPU-side activities followed by CUPTI records, in arrival order
  struct Run {
    std::vector<int64_t> start, end, resource;
    std::vector<int32_t> id, dev, thread, type;
    std::vector<uint32_t> name, flow, mdoff{0};
    std::vector<uint8_t> flowt;
    std::vector<k2j_md_entry> md;
    // The run's record bytes, written once by the threads that packed them (no zero fill, no regrowth).  In front
    // go the records that only feed lookups (their timestamps lie before the window, so they print nothing): what
    // the profiler had already resolved for a synchronisation activity when it reached the logger - its context's
    // device, the CUDA event record it waits on - restated as the records that make the device-side lookups give
    // the same answer.
    std::unique_ptr<uint8_t[]> cupti;
    size_t cuptiBytes = 0;
    // ids of the CPU-side activities of this run: a bitmap for the usual small non-negative ids, a set for the rest
    std::vector<uint64_t> opIdBits;
    std::unordered_set<int32_t> opIdRest;
    void noteOp(int32_t id) {
      if (id >= 0 && id < (1 << 28)) {
        const size_t w = (size_t)id >> 6;
        if (w >= opIdBits.size()) opIdBits.resize(std::max(w + 1, opIdBits.size() * 2), 0);
        opIdBits[w] |= 1ull << (id & 63);
      } else opIdRest.insert(id);
    }
    bool hasOp(int32_t id) const {
      if (id >= 0 && id < (1 << 28)) { const size_t w = (size_t)id >> 6; return w < opIdBits.size() && ((opIdBits[w] >> (id & 63)) & 1); }
      return opIdRest.count(id) != 0;
    }
    bool hasCupti = false;
  };
  Run run;
  std::vector<int32_t> tidPairs;
  std::unordered_map<int32_t, bool> tidSeen;

  void text(const std::string& s) {
    flushRun();
    if (out) fwrite(s.data(), 1, s.size(), out);
  }
  std::vector<int32_t> linkedIds;
  // What ChromeTraceLogger::appendCollectiveMetadata (libkineto/src/output_json.cpp:803-835) keeps for the trailer:
  // the job's rank and size from the first collective of the default process group, and every process group seen.
  // Host work per collective kernel; the kernel event's own collective arguments are written by the GPU path.
  DistributedInfo distInfo;
  std::unordered_map<std::string, pgConfig> pgMap;
  static std::string stripQuotes(std::string v) {
    if (v.size() >= 2 && v.front() == '"' && v.back() == '"') { v.pop_back(); v.erase(0, 1); }
    return v;
  }
  void noteCollective(const libkineto::ITraceActivity& op) {
    const std::string groupSize = op.getMetadataValue("Group size");
    std::string pgName = stripQuotes(op.getMetadataValue("Process Group Name"));
    std::string pgDesc = stripQuotes(op.getMetadataValue("Process Group Description"));
    std::string ranks = stripQuotes(op.getMetadataValue("Process Group Ranks"));
    if (distInfo.backend.empty() && pgDesc == "default_pg") {
      distInfo.backend = "nccl";
      distInfo.rank = op.getMetadataValue("Rank");
      distInfo.world_size = groupSize;
      distInfo.nccl_version = "unknown";
    }
    pgConfig cfg;
    cfg.pg_name = pgName; cfg.pg_desc = std::move(pgDesc); cfg.backend_config = "cuda:nccl"; cfg.pg_size = groupSize;
    cfg.ranks = std::move(ranks);
    pgMap.insert({pgName, cfg});
  }

  // ---- CUPTI wrappers: gathered as pointers, packed when the run is flushed ----
  // A wrapper stays alive and in place until the trace is finalised (the reference's own in-memory logger keeps
  // the same pointers, libkineto/src/output_membuf.h:59-63), so turning wrappers into record bytes can wait for
  // the flush and be split over threads: each thread packs a contiguous slice into a Piece, and the pieces are
  // merged in order, which keeps every "first one wins" / "last one wins" rule of the serial order.
  struct Piece {
    std::vector<uint8_t> cupti, prefix;
    std::vector<int32_t> linkedIds;
    std::vector<const libkineto::ITraceActivity*> collectives;     // linked record_param_comms ops, in order
    std::vector<int32_t> tidPairs;                                   // first sighting of each thread id, in order
    std::unordered_map<int32_t, bool> tidSeen;
    std::vector<uint32_t> rtCbids, drCbids;                          // callback ids met (distinct)
    std::vector<bool> rtSeen, drSeen;
    std::unordered_map<const void*, uint32_t> nameIds;               // raw kernel name pointer -> local id
    std::vector<const void*> namePtrs;
    std::vector<std::string> names;                                  // demangled, by local id
    std::vector<uint32_t> kernelOffsets;                             // kernel records in `cupti` (their name field holds a local id)
    std::vector<uint32_t> global;                                    // local name id -> pool id, set by mergePiece
    std::unordered_map<uint32_t, bool> ctxDeclared;
    size_t skipped = 0;
    std::string firstSkippedName;
    template <class T> void append(const T& rec) {
      const uint8_t* q = reinterpret_cast<const uint8_t*>(&rec);
      cupti.insert(cupti.end(), q, q + sizeof(T));
    }
    template <class T> void appendPrefix(const T& rec) {
      const uint8_t* q = reinterpret_cast<const uint8_t*>(&rec);
      prefix.insert(prefix.end(), q, q + sizeof(T));
    }
  };
  std::vector<const libkineto::ITraceActivity*> pending;
  // ---- CPU-side activities: gathered as pointers too, turned into columns when the run is flushed ----
  // The profiler keeps them alive and in place until the trace is finalised (GenericActivityProfiler.cpp:249-254;
  // the in-memory logger replays its own copies, which live as long as it does, output_membuf.h:64-66, :91-107),
  // so visiting their metadata - one unordered_map walk and several interned strings per activity - can be split
  // over threads like the wrappers: each thread fills the columns of a contiguous slice with string ids of its
  // own, and the slices are appended in order with their ids mapped to pool ids.  A caller that hands over
  // activities that do not outlive the call sets copyOps (environment K2J_SHIM_COPY_OPS=1): they are then turned
  // into columns at once, on the calling thread.
  std::vector<const libkineto::GenericTraceActivity*> pendingOps;
  bool copyOps = false;
  struct OpPiece {
    std::vector<int64_t> start, end, resource;
    std::vector<int32_t> id, dev, thread, type;
    std::vector<uint32_t> name, flow, mdoff;
    std::vector<uint8_t> flowt;
    std::vector<k2j_md_entry> md;
    std::unordered_map<std::string_view, uint32_t> ids;   // views into the live activities or into `owned`
    std::vector<std::string_view> strs;
    std::deque<std::string> owned;
    uint32_t local(std::string_view v) {
      auto it = ids.find(v);
      if (it != ids.end()) return it->second;
      const uint32_t k = (uint32_t)strs.size();
      ids.emplace(v, k); strs.push_back(v);
      return k;
    }
  };
  void opColumns(const libkineto::GenericTraceActivity& op, OpPiece& p) const;
  void packOps();
  size_t* skippedOut = nullptr;
  void packOne(const libkineto::ITraceActivity& a, Piece& p) const;
  void mergePiece(Piece& p);
  void packPending();

  bool flushRun();
};

// One CPU-side activity into the columns of its piece (string ids are the piece's own).
void B200TraceLogger::Impl::opColumns(const libkineto::GenericTraceActivity& op, OpPiece& p) const {
  p.start.push_back(op.startTime); p.end.push_back(op.endTime); p.id.push_back(op.id); p.dev.push_back(op.device);
  p.resource.push_back(op.resource); p.thread.push_back(op.threadId); p.type.push_back((int32_t)op.activityType);
  p.name.push_back(p.local(op.activityName)); p.flow.push_back(op.flow.id);
  p.flowt.push_back((uint8_t)(op.flow.type | (op.flow.start << 4)));
  MdCollector mc;
  op.visitTypedMetadata(mc);
  for (auto& e : mc.entries) {
    k2j_md_entry k{p.local(e.key), e.type, e.value};
    if (e.type == K2J_MD_STRING || e.type == K2J_MD_RAWJSON) {
      // text rendered for this visit (collections) lives in the collector: the piece takes it over
      bool ownedText = false;
      for (const std::string& o : mc.owned) if (o.data() == e.text.data()) { ownedText = true; break; }
      if (ownedText) { p.owned.emplace_back(e.text); k.value = p.local(p.owned.back()); }
      else k.value = p.local(e.text);
    }
    p.md.push_back(k);
  }
  for (const auto& cv : op.counterValues()) {  // counter events (output_json.cpp:679-716): name and value, in order
    uint64_t bits; const double v = cv.second; memcpy(&bits, &v, 8);
    p.md.push_back(k2j_md_entry{p.local(cv.first), K2J_MD_COUNTER, bits});
  }
  p.mdoff.push_back((uint32_t)p.md.size());
}

void B200TraceLogger::Impl::packOps() {
  if (pendingOps.empty()) return;
  Timed timed(tOps);
  std::vector<const libkineto::GenericTraceActivity*> acts;
  acts.swap(pendingOps);
  const size_t n = acts.size();
  const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
  const size_t nt = n < 20000 ? 1 : std::min<size_t>({(size_t)hw, (size_t)16, n / 10000});
  std::vector<OpPiece> pieces(nt);
  auto work = [&](size_t t) {
    const size_t lo = n * t / nt, hi = n * (t + 1) / nt;
    OpPiece& p = pieces[t];
    p.start.reserve(hi - lo); p.md.reserve(4 * (hi - lo));
    for (size_t i = lo; i < hi; i++) opColumns(*acts[i], p);
  };
  if (nt == 1) work(0);
  else {
    std::vector<std::thread> threads;
    for (size_t t = 1; t < nt; t++) threads.emplace_back(work, t);
    work(0);
    for (auto& th : threads) th.join();
  }
  Run& r = run;
  for (OpPiece& p : pieces) {  // in order: ids of the piece become pool ids, its columns follow the run's
    std::vector<uint32_t> global(p.strs.size());
    for (size_t i = 0; i < p.strs.size(); i++) global[i] = intern(p.strs[i]);
    const uint32_t mdBase = (uint32_t)r.md.size();
    r.start.insert(r.start.end(), p.start.begin(), p.start.end()); r.end.insert(r.end.end(), p.end.begin(), p.end.end());
    r.resource.insert(r.resource.end(), p.resource.begin(), p.resource.end()); r.id.insert(r.id.end(), p.id.begin(), p.id.end());
    r.dev.insert(r.dev.end(), p.dev.begin(), p.dev.end()); r.thread.insert(r.thread.end(), p.thread.begin(), p.thread.end());
    r.type.insert(r.type.end(), p.type.begin(), p.type.end()); r.flow.insert(r.flow.end(), p.flow.begin(), p.flow.end());
    r.flowt.insert(r.flowt.end(), p.flowt.begin(), p.flowt.end());
    for (uint32_t v : p.name) r.name.push_back(global[v]);
    for (uint32_t v : p.mdoff) r.mdoff.push_back(mdBase + v);
    for (k2j_md_entry e : p.md) {
      e.key = global[e.key];
      if (e.type == K2J_MD_STRING || e.type == K2J_MD_RAWJSON) e.value = global[(size_t)e.value];
      r.md.push_back(e);
    }
    for (int32_t v : p.id) r.noteOp(v);
  }
}

bool B200TraceLogger::Impl::flushRun() {
  packOps();
  packPending();
  Run r;
  std::swap(r, run);
  std::vector<int32_t> links;
  std::swap(links, linkedIds);
  const size_t nops = r.start.size();
  if (nops == 0 && r.cuptiBytes == 0) return true;
  if (!ctx || !out) return false;
  // CPU ops a record is linked to may have been logged in an earlier run: make them joinable here as
  // unselected activities (type bit cleared below), which take part in the join but print nothing.
  const uint32_t kHidden = 27;  // XPU_SYNC: never produced on this path; its type bit is left clear
  for (int32_t idv : links) {
    r.start.push_back(0); r.end.push_back(0); r.resource.push_back(0); r.id.push_back(idv); r.dev.push_back(0);
    r.thread.push_back(0); r.type.push_back((int32_t)kHidden); r.name.push_back(0); r.flow.push_back(0);
    r.flowt.push_back(0); r.mdoff.push_back(r.mdoff.back());
  }
  k2j_params p{};
  p.base_time_ns = ChromeTraceBaseTime::singleton().get();
  p.window_start_ns = 1;  // records arrive already filtered by the profiler; lookup-only records carry timestamp 0
  p.window_end_ns = INT64_MAX;
  p.pid = processId();
  p.ts_mode = 0;  // CuptiActivity<T>::timestamp() was not used: raw timestamps are converted below
  p.flags = 0;
  p.activity_type_mask = ~(1u << kHidden);
  const std::vector<k2j_device_props>& props = ContextPool::deviceProps();
  p.n_devices = (int32_t)props.size();
  k2j_ops ops{};
  const size_t n = r.start.size();
  ops.n_ops = n; ops.start_ns = r.start.data(); ops.end_ns = r.end.data(); ops.id = r.id.data(); ops.device = r.dev.data();
  ops.resource = r.resource.data(); ops.thread = r.thread.data(); ops.type = r.type.data(); ops.name = r.name.data();
  ops.flow_id = r.flow.data(); ops.flow_info = r.flowt.data(); ops.md_off = r.mdoff.data(); ops.md = r.md.data();
  const uint64_t buftab[2] = {0, r.cuptiBytes};
  k2j_result res;
  tSetup.start();
  bool ok = k2j_set_params(ctx, &p, props.data()) == K2J_OK &&
            k2j_set_strings(ctx, poolOff.data(), poolData.data(), poolOff.size() - 1) == K2J_OK &&
            k2j_set_cbid_names(ctx, rtNames.data(), (uint32_t)rtNames.size(), drNames.data(), (uint32_t)drNames.size()) == K2J_OK &&
            k2j_set_thread_map(ctx, tidPairs.data(), (uint32_t)(tidPairs.size() / 2)) == K2J_OK &&
            k2j_set_ops(ctx, &ops) == K2J_OK &&
            k2j_set_cupti(ctx, r.cupti.get(), r.cuptiBytes, buftab, r.cuptiBytes ? 1 : 0) == K2J_OK;
  tSetup.stop();
  tRun.start();
  ok = ok && k2j_run(ctx, &res) == K2J_OK;
  tRun.stop();
  if (!ok) {
    LOG(ERROR) << "B200TraceLogger: " << k2j_last_error(ctx);
    return false;
  }
  // the text goes from the device to the file in chunks, the copy of one overlapping the write of the one before
  Timed timed(tWrite);
  fflush(out);
  if (k2j_write_output(ctx, fileno(out), nullptr) != K2J_OK) {
    LOG(ERROR) << "B200TraceLogger: " << k2j_last_error(ctx);
    return false;
  }
  return true;
}

B200TraceLogger::B200TraceLogger(const std::string& traceFileName, int cudaDevice) : impl_(new Impl) {
  impl_->fileName = traceFileName.empty() ? fmt::format("/tmp/libkineto_activities_{}.json", processId()) : traceFileName;
  impl_->tempFileName = impl_->fileName + ".tmp";
  impl_->device = cudaDevice;
  impl_->out = fopen(impl_->tempFileName.c_str(), "wb");
  if (!impl_->out) PLOG(ERROR) << "Failed to open '" << impl_->fileName << "'";
  impl_->skippedOut = &skipped_;
  impl_->ctx = ContextPool::take(cudaDevice);
  if (!impl_->ctx) {
    // No GPU path, and deliberately no CPU path: like ChromeTraceLogger with an unopened file, every
    // handler returns without writing.
    LOG(ERROR) << "B200TraceLogger: cannot create a k2j context on CUDA device " << cudaDevice;
    impl_->ctx = nullptr;
    if (impl_->out) { fclose(impl_->out); impl_->out = nullptr; remove(impl_->tempFileName.c_str()); }
  }
  impl_->invalidId = impl_->intern("INVALID");
  const char* copy = getenv("K2J_SHIM_COPY_OPS");
  impl_->copyOps = copy && *copy && *copy != '0';
}

B200TraceLogger::~B200TraceLogger() {
  if (impl_->out) fclose(impl_->out);
  ContextPool::give(impl_->device, impl_->ctx);
}

void B200TraceLogger::handleTraceStart(const std::unordered_map<std::string, std::string>& metadata,
                                       const std::string& device_properties) {
  if (!impl_->out) return;
  std::string s = fmt::format(" {{\n    \"schemaVersion\": {},\n    \"deviceProperties\": [{}],\n    ", 1, device_properties);
  auto combined = libkineto::getEnvMetadata();  // environment first, caller's metadata wins (output_json.cpp:433-443)
  for (const auto& [k, v] : metadata) combined[k] = v;
  for (const auto& [k, v] : combined) {
    std::string sv = v;
    sanitize(sv);
    s += fmt::format("\n      \"{}\": {},", k, sv);
  }
  std::string unit = "ms";
#ifdef DISPLAY_TRACE_IN_NS
  unit = "ns";
#endif
  s += fmt::format("\n    \"displayTimeUnit\": \"{}\",\n    \"baseTimeNanoseconds\": {},\n    \"traceEvents\": [\n    ", unit,
                   ChromeTraceBaseTime::singleton().get());
  impl_->text(s);
}

void B200TraceLogger::handleDeviceInfo(const DeviceInfo& info, int64_t time) {
  if (!impl_->out) return;
  std::string name = info.name, label = info.label;
  sanitize(name); escapeQuotes(name); sanitize(label); escapeQuotes(label);
  time = rel(time);
  const std::string pid = std::to_string(info.id);
  impl_->text(metaRow("process_name", time, pid, "0", "name", "\"" + name + "\"") +
              metaRow("process_labels", time, pid, "0", "labels", "\"" + label + "\"") +
              metaRow("process_sort_index", time, pid, "0", "sort_index", std::to_string(info.sortIndex)));
}

void B200TraceLogger::handleResourceInfo(const ResourceInfo& info, int64_t time) {
  if (!impl_->out) return;
  std::string name = info.name;
  if (info.resourceType == ResourceType::HOST_THREAD) name = fmt::format("thread {} ({})", info.id, info.name);
  sanitize(name); escapeQuotes(name);
  time = rel(time);
  const std::string pid = std::to_string(info.deviceId), tid = std::to_string(absTid(info.id));
  impl_->text(metaRow("thread_name", time, pid, tid, "name", "\"" + name + "\"") +
              metaRow("thread_sort_index", time, pid, tid, "sort_index", std::to_string(info.sortIndex)));
}

void B200TraceLogger::handleOverheadInfo(const OverheadInfo& info, int64_t time) {
  if (!impl_->out) return;
  std::string name = info.name;
  sanitize(name); escapeQuotes(name);
  time = rel(time);
  impl_->text(metaRow("process_name", time, "-1", "0", "name", "\"" + name + "\"") +
              metaRow("process_sort_index", time, "-1", "0", "sort_index", std::to_string(0x100000All)));
}

void B200TraceLogger::handleTraceSpan(const TraceSpan& span) {
  if (!impl_->out) return;
  const int64_t start = rel(span.startTime);
  const int64_t dur = span.endTime == 0 ? 0 : span.endTime - span.startTime;
  std::string s = fmt::format(
      "\n  {{\n    \"ph\": \"X\",\n    \"cat\": \"Trace\",\n    \"name\": \"{}{} ({})\",\n    \"pid\": \"Spans\",\n    \"tid\": \"{}\",\n    \"ts\": {},\n    \"dur\": {}\n    ,\n    \"args\": {{\n      \"Op count\": {}\n    }}\n  }},",
      span.prefix, span.name, span.iteration, span.name, ts(start), ts(dur), span.opCount);
  s += metaRow("process_sort_index", start, "\"Spans\"", "0", "sort_index", std::to_string(0x20000000ll));
  s += instantRow(fmt::format("Iteration Start: {}", span.name), "\"Traces\"", fmt::format("\"Trace {}\"", span.name), start, false);
  impl_->text(s);
}

void B200TraceLogger::handleGenericActivity(const libkineto::GenericTraceActivity& op) {
  if (!impl_->out) return;
  Impl& m = *impl_;
  if (m.run.hasCupti) m.flushRun();  // a run is CPU-side activities followed by CUPTI records
  m.pendingOps.push_back(&op);
  if (m.copyOps) m.packOps();        // the activity may not outlive this call: into columns now
}

void B200TraceLogger::handleActivity(const libkineto::ITraceActivity& a) {
  if (!impl_->out) return;
  Impl& m = *impl_;
  // The wrapper classes of the CUPTI path are gathered and packed at the flush; everything else is tried as a
  // GenericTraceActivity now (it belongs to the columns of CPU-side activities, which are filled in arrival order).
  const std::type_info& ti = typeid(a);
  const bool wrapper = ti == typeid(GpuActivity<CUpti_ActivityKernelType>) || ti == typeid(RuntimeActivity) ||
                       ti == typeid(GpuActivity<CUpti_ActivityMemcpyType>) || ti == typeid(GpuActivity<CUpti_ActivityMemsetType>) ||
                       ti == typeid(GpuActivity<CUpti_ActivityMemcpyPtoPType>) || ti == typeid(DriverActivity) ||
                       ti == typeid(OverheadActivity) || ti == typeid(CudaSyncActivity) || ti == typeid(CudaEventActivity);
  if (!wrapper) {
    if (auto* g = dynamic_cast<const libkineto::GenericTraceActivity*>(&a)) { handleGenericActivity(*g); return; }
  }
  m.pending.push_back(&a);   // classes derived from the wrappers, and foreign classes, are sorted out by packOne
  m.run.hasCupti = true;
}

// One wrapper into its piece: the record with converted timestamps, in front of it the EXTERNAL_CORRELATION record
// that restates linkedActivity(), and the side information the merge needs.  Reads shared state only.
void B200TraceLogger::Impl::packOne(const libkineto::ITraceActivity& a, Piece& p) const {
  const libkineto::ActivityType ty = a.type();
  auto convert = [](auto& rec) {  // timestamps as the wrapper reports them (CuptiTimestamp.h:29-51)
    const uint64_t s = rec.start, e = rec.end;
    const int64_t cs = convertCuptiTimestamp(s);
    rec.start = (uint64_t)cs;
    rec.end = (uint64_t)(cs + convertCuptiDuration(s, e));
  };
  auto link = [&]() {
    const libkineto::ITraceActivity* l = a.linkedActivity();
    if (!l) return l;
    CUpti_ActivityExternalCorrelation e;
    memset(&e, 0, sizeof e);
    e.kind = CUPTI_ACTIVITY_KIND_EXTERNAL_CORRELATION;
    e.externalKind = CUPTI_EXTERNAL_CORRELATION_KIND_CUSTOM0;
    e.externalId = (uint64_t)l->correlationId();
    e.correlationId = (uint32_t)a.correlationId();
    p.append(e);
    // an op logged in an earlier run is made joinable again (see flushRun); one of this run keeps its own row, so
    // that its name and metadata stay reachable from the records linked to it
    if (!run.hasOp((int32_t)l->correlationId())) p.linkedIds.push_back((int32_t)l->correlationId());
    return l;
  };
  auto thread = [&](uint32_t tid) {
    if (p.tidSeen.count((int32_t)tid)) return;
    p.tidSeen[(int32_t)tid] = true;
    p.tidPairs.push_back((int32_t)tid); p.tidPairs.push_back((int32_t)a.resourceId());
  };
  auto cbid = [](std::vector<uint32_t>& list, std::vector<bool>& seen, uint32_t c) {
    if (c >= seen.size()) seen.resize(c + 1, false);
    if (!seen[c]) { seen[c] = true; list.push_back(c); }
  };
  auto declare = [&](uint32_t ctx, uint32_t device) {  // contextIdtoDeviceId's answer as the context's first writer
    if (p.ctxDeclared.count(ctx)) return;
    p.ctxDeclared[ctx] = true;
    CUpti_ActivityMemsetType ms;
    memset(&ms, 0, sizeof ms);
    ms.kind = CUPTI_ACTIVITY_KIND_MEMSET;
    ms.contextId = ctx; ms.deviceId = device;
    p.appendPrefix(ms);
  };
  if (auto* k = ty == ActivityType::CONCURRENT_KERNEL ? dynamic_cast<const GpuActivity<CUpti_ActivityKernelType>*>(&a) : nullptr) {
    const libkineto::ITraceActivity* l = link();
    if (l) {  // a collective's CPU op: compared in place where the name is a member, no string per kernel
      auto* g = dynamic_cast<const libkineto::GenericTraceActivity*>(l);
      if (g ? g->activityName == "record_param_comms" : l->name() == "record_param_comms") p.collectives.push_back(l);
    }
    CUpti_ActivityKernelType rec = k->raw();
    convert(rec);
    auto it = p.nameIds.find(rec.name);
    uint32_t id;
    if (it != p.nameIds.end()) id = it->second;
    else {
      id = (uint32_t)p.names.size();
      p.nameIds[rec.name] = id;
      p.namePtrs.push_back(rec.name);
      p.names.push_back(a.name());
    }
    uint64_t id64 = id;
    memcpy(&rec.name, &id64, 8);
    p.kernelOffsets.push_back((uint32_t)p.cupti.size());
    p.append(rec);
  } else if (auto* c = ty == ActivityType::GPU_MEMCPY ? dynamic_cast<const GpuActivity<CUpti_ActivityMemcpyType>*>(&a) : nullptr) {
    link();
    CUpti_ActivityMemcpyType rec = c->raw();
    convert(rec);
    p.append(rec);
  } else if (auto* c2 = ty == ActivityType::GPU_MEMCPY ? dynamic_cast<const GpuActivity<CUpti_ActivityMemcpyPtoPType>*>(&a) : nullptr) {
    link();
    CUpti_ActivityMemcpyPtoPType rec = c2->raw();
    convert(rec);
    p.append(rec);
  } else if (auto* s = ty == ActivityType::GPU_MEMSET ? dynamic_cast<const GpuActivity<CUpti_ActivityMemsetType>*>(&a) : nullptr) {
    link();
    CUpti_ActivityMemsetType rec = s->raw();
    convert(rec);
    p.append(rec);
  } else if (auto* rt = ty == ActivityType::CUDA_RUNTIME ? dynamic_cast<const RuntimeActivity*>(&a) : nullptr) {
    link();
    CUpti_ActivityAPI rec = rt->raw();
    convert(rec);
    cbid(p.rtCbids, p.rtSeen, rec.cbid);
    thread(rec.threadId);
    p.append(rec);
  } else if (auto* dr = ty == ActivityType::CUDA_DRIVER ? dynamic_cast<const DriverActivity*>(&a) : nullptr) {
    link();
    CUpti_ActivityAPI rec = dr->raw();
    convert(rec);
    cbid(p.drCbids, p.drSeen, rec.cbid);
    thread(rec.threadId);
    p.append(rec);
  } else if (auto* ov = ty == ActivityType::OVERHEAD ? dynamic_cast<const OverheadActivity*>(&a) : nullptr) {
    // the wrapper holds the 40-byte prefix of the record (CUpti_ActivityOverhead); the GPU path takes the
    // record as CUPTI writes it today (CUpti_ActivityOverhead3, 56 bytes)
    CUpti_ActivityOverhead3 rec;
    memset(&rec, 0, sizeof rec);
    memcpy(&rec, &ov->raw(), sizeof(CUpti_ActivityOverhead));
    convert(rec);
    p.append(rec);
  } else if (auto* sy = ty == ActivityType::CUDA_SYNC ? dynamic_cast<const CudaSyncActivity*>(&a) : nullptr) {
    link();
    CUpti_ActivitySynchronization rec = sy->raw();
    convert(rec);
    declare(rec.contextId, (uint32_t)a.deviceId());
    if (isEventSync(rec.type)) {
      // the CUDA event record the profiler found (CuptiActivityProfiler.cpp:452-461) is only visible as metadata
      MdCollector mc;
      a.visitTypedMetadata(mc);
      int64_t srcStream = -1, srcCorr = -1;
      for (auto& e : mc.entries) {
        if (e.key == "wait_on_stream") srcStream = (int64_t)e.value;
        else if (e.key == "wait_on_cuda_event_record_corr_id") srcCorr = (int64_t)e.value;
      }
      if (srcCorr != -1 || srcStream != -1) {
        CUpti_ActivityCudaEventType ev;
        memset(&ev, 0, sizeof ev);
        ev.kind = CUPTI_ACTIVITY_KIND_CUDA_EVENT;
        ev.correlationId = (uint32_t)srcCorr; ev.contextId = rec.contextId; ev.streamId = (uint32_t)srcStream;
        ev.eventId = rec.cudaEventId;
        p.appendPrefix(ev);
      }
    }
    p.append(rec);
  } else if (auto* ce = ty == ActivityType::CUDA_EVENT ? dynamic_cast<const CudaEventActivity*>(&a) : nullptr) {
    link();
    CUpti_ActivityCudaEventType rec = ce->raw();
    rec.deviceTimestamp = (uint64_t)convertCuptiTimestamp(rec.deviceTimestamp);
    declare(rec.contextId, (uint32_t)a.deviceId());
    p.append(rec);
  } else {
    // Foreign activity classes are not handled by the GPU path; there is no CPU path to fall back to, so they
    // are counted and reported.
    if (p.skipped++ == 0) p.firstSkippedName = a.name();
  }
}

// A piece joins the run: local kernel-name ids get pool ids, first sightings stay first sightings.  Its record
// bytes are moved by the threads afterwards (packPending).
void B200TraceLogger::Impl::mergePiece(Piece& p) {
  p.global.resize(p.names.size());
  for (size_t i = 0; i < p.names.size(); i++) {
    auto it = kernelNameIds.find(p.namePtrs[i]);
    p.global[i] = it != kernelNameIds.end() ? it->second : (kernelNameIds[p.namePtrs[i]] = intern(p.names[i]));
  }
  linkedIds.insert(linkedIds.end(), p.linkedIds.begin(), p.linkedIds.end());
  for (const libkineto::ITraceActivity* op : p.collectives) noteCollective(*op);
  for (size_t i = 0; i + 1 < p.tidPairs.size(); i += 2) {
    if (tidSeen.count(p.tidPairs[i])) continue;
    tidSeen[p.tidPairs[i]] = true;
    tidPairs.push_back(p.tidPairs[i]); tidPairs.push_back(p.tidPairs[i + 1]);
  }
  auto names = [&](std::vector<uint32_t>& tab, const std::vector<uint32_t>& cbids, bool driver) {
    for (uint32_t c : cbids) {
      if (c >= tab.size()) tab.resize(c + 1, invalidId);
      if (tab[c] == invalidId) tab[c] = intern(driver ? driverCbidName(c) : runtimeCbidName(c));
    }
  };
  names(rtNames, p.rtCbids, false);
  names(drNames, p.drCbids, true);
  if (p.skipped) {
    if (*skippedOut == 0) LOG(ERROR) << "B200TraceLogger: unsupported activity class for '" << p.firstSkippedName << "'; skipped";
    *skippedOut += p.skipped;
  }
}

void B200TraceLogger::Impl::packPending() {
  if (pending.empty()) return;
  Timed timed(tRecords);
  std::vector<const libkineto::ITraceActivity*> acts;
  acts.swap(pending);
  const size_t n = acts.size();
  const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
  const size_t nt = n < 50000 ? 1 : std::min<size_t>({(size_t)hw, (size_t)16, n / 25000});
  std::vector<Piece> pieces(nt);
  auto onThreads = [&](auto&& fn) {
    if (nt == 1) { fn(0); return; }
    std::vector<std::thread> threads;
    for (size_t t = 1; t < nt; t++) threads.emplace_back(fn, t);
    fn(0);
    for (auto& th : threads) th.join();
  };
  onThreads([&](size_t t) {
    const size_t lo = n * t / nt, hi = n * (t + 1) / nt;
    Piece& p = pieces[t];
    p.cupti.reserve((hi - lo) * 160);
    for (size_t i = lo; i < hi; i++) packOne(*acts[i], p);
  });
  // where each piece's bytes go: all lookup-only records first, then the records, both in piece order
  std::vector<size_t> prefixAt(nt), recordsAt(nt);
  size_t total = 0;
  for (size_t t = 0; t < nt; t++) { prefixAt[t] = total; total += pieces[t].prefix.size(); }
  for (size_t t = 0; t < nt; t++) { recordsAt[t] = total; total += pieces[t].cupti.size(); }
  for (Piece& p : pieces) mergePiece(p);
  run.cupti.reset(new uint8_t[total ? total : 1]);
  run.cuptiBytes = total;
  uint8_t* dst = run.cupti.get();
  onThreads([&](size_t t) {
    Piece& p = pieces[t];
    for (uint32_t off : p.kernelOffsets) {
      uint8_t* field = p.cupti.data() + off + offsetof(CUpti_ActivityKernelType, name);
      uint64_t id;
      memcpy(&id, field, 8);
      id = p.global[(size_t)id];
      memcpy(field, &id, 8);
    }
    if (!p.prefix.empty()) memcpy(dst + prefixAt[t], p.prefix.data(), p.prefix.size());
    if (!p.cupti.empty()) memcpy(dst + recordsAt[t], p.cupti.data(), p.cupti.size());
  });
}

void B200TraceLogger::finalizeTrace(const Config&, std::unique_ptr<ActivityBuffers> /*buffers*/, int64_t endTime) {
  if (!impl_->out) {
    LOG(ERROR) << "Failed to write to log file!";
    return;
  }
  std::string fileName = impl_->fileName;
  sanitize(fileName);
  std::string s = instantRow("Record Window End", "\"\"", "\"\"", rel(endTime), true);
  s += "\n  ],";
  if (!impl_->distInfo.backend.empty()) {  // addOnDemandDistMetadata, output_json.cpp:1030-1064
    const DistributedInfo& di = impl_->distInfo;
    s += fmt::format("\n  \"distributedInfo\": {{\"backend\": \"{}\", \"rank\": {}, \"world_size\": {}, \"pg_count\": {}, \"pg_config\": [",
                     di.backend, di.rank, di.world_size, std::to_string(impl_->pgMap.size()));
    bool first = true;
    for (const auto& el : impl_->pgMap) {
      if (!first) s += ",";
      s += fmt::format("{{\"pg_name\": \"{}\", \"pg_desc\": \"{}\", \"backend_config\": \"{}\", \"pg_size\": {}, \"ranks\": \"{}\"}}",
                       el.second.pg_name, el.second.pg_desc, el.second.backend_config, el.second.pg_size, el.second.ranks);
      first = false;
    }
    s += fmt::format("], \"nccl_version\": \"{}\"}},", di.nccl_version);
  }
  s += fmt::format("\"traceName\": \"{}\" }}", fileName);
  impl_->text(s);
  if (getenv("K2J_SHIM_TIMING"))
    fprintf(stderr, "B200TraceLogger host seconds: cpu activities %.3f, cupti activities %.3f, set inputs %.3f, k2j_run %.3f, copy + write %.3f\n",
            impl_->tOps.total, impl_->tRecords.total, impl_->tSetup.total, impl_->tRun.total, impl_->tWrite.total);
  fclose(impl_->out);
  impl_->out = nullptr;
  remove(impl_->fileName.c_str());
  if (rename(impl_->tempFileName.c_str(), impl_->fileName.c_str()) != 0)
    PLOG(ERROR) << "Failed to rename " << impl_->tempFileName << " to " << impl_->fileName;
}

}  // namespace KINETO_NAMESPACE
