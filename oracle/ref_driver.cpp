// TEST INFRASTRUCTURE — drives the UNMODIFIED reference (libkineto, compiled from the reference
// tree by oracle/Makefile) over one synthetic trace container and writes the Chrome-trace JSON it
// produces.  Nothing here is product code and the product never links or executes it.
//
// mode 0 follows the reference benchmark's timed region (benchmarks/json_output_benchmark.cpp:217-244):
//   ChromeTraceLogger(path); handleTraceStart({}, ""); handleGenericActivity per op; finalizeTrace.
// mode 1 follows the reference integration test (libkineto/test/CuptiActivityProfilerTest.cpp:320-346,
//   :468-603): a CuptiActivityApi subclass replays raw CUPTI records, CPU ops arrive through
//   transferCpuTrace, processTrace fills a MemoryTraceLogger and ActivityTrace::save() writes the file.
//
// usage: ref_driver <trace.k2jt> <out.json> [--repeat N] [--events-only <out.events>]
//        ref_driver --md-order key1 key2 ...   (prints GenericTraceActivity metadata visit order)
//        ref_driver --cbid-names <out.txt>     (prints "R|D <cbid> <name>" for every callback id)
//        ref_driver --version
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <memory>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>
#include <cupti.h>
#include <fmt/format.h>

#include "ActivityLoggerFactory.h"
#include "ActivityTrace.h"
#include "ApproximateClock.h"
#include "Config.h"
#include "CuptiActivity.h"
#include "CuptiActivityApi.h"
#include "CuptiActivityProfiler.h"
#include "CuptiTimestamp.h"
#include "GenericTraceActivity.h"
#include "Logger.h"
#include "ThreadUtil.h"
#include "cupti_strings.h"
#include "libkineto.h"
#include "output_json.h"
#include "output_membuf.h"

#include "trace_file.h"

using namespace libkineto;

extern "C" void k2j_fake_set_device_count(int n);
extern "C" cudaDeviceProp* k2j_fake_device_prop(int i);
extern "C" void k2j_fake_set_pid(int pid);
extern "C" void k2j_fake_set_now_ns(long long ns);

#include "../kineto_b200/csrc/k2j_cupti_sizes.h"  // generated from cupti_activity.h: record size per activity kind

namespace {

size_t recordSize(uint32_t kind) {
  switch (kind) {
    case CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL: return sizeof(CUpti_ActivityKernel9);
    case CUPTI_ACTIVITY_KIND_MEMCPY: return sizeof(CUpti_ActivityMemcpy5);
    case CUPTI_ACTIVITY_KIND_MEMCPY2: return sizeof(CUpti_ActivityMemcpyPtoP4);
    case CUPTI_ACTIVITY_KIND_MEMSET: return sizeof(CUpti_ActivityMemset4);
    case CUPTI_ACTIVITY_KIND_RUNTIME:
    case CUPTI_ACTIVITY_KIND_DRIVER: return sizeof(CUpti_ActivityAPI);
    case CUPTI_ACTIVITY_KIND_EXTERNAL_CORRELATION: return sizeof(CUpti_ActivityExternalCorrelation);
    case CUPTI_ACTIVITY_KIND_OVERHEAD: return sizeof(CUpti_ActivityOverhead3);  // what CUPTI 12.9 writes; the reference reads its 40-byte prefix
    case CUPTI_ACTIVITY_KIND_SYNCHRONIZATION: return sizeof(CUpti_ActivitySynchronization);
    case CUPTI_ACTIVITY_KIND_CUDA_EVENT: return sizeof(CUpti_ActivityCudaEvent2);
    // kinds the reference only counts: stepped over by the size of the kind's record in the CUPTI headers
    default: return kind < (uint32_t)k2j::kCuptiKinds ? 8u * k2j::kCuptiRecordSlots[kind] : 0;
  }
}

// Replays the synthetic buffers exactly like the reference test's MockCuptiActivities.
class ReplayCuptiActivities : public CuptiActivityApi {
 public:
  bool isAvailable(uint32_t& version) const override {
    version = 0;
    return true;
  }
  const std::pair<int, size_t> processActivities(
      CuptiActivityBufferMap&,
      const std::function<void(const CUpti_Activity*)>& handler) override {
    size_t bytes = 0;
    for (const CUpti_Activity* act : records) handler(act);
    return {(int)records.size(), bytes};
  }
  std::unique_ptr<CuptiActivityBufferMap> activityBuffers() override {
    auto map = std::make_unique<CuptiActivityBufferMap>();
    auto buf = std::make_unique<CuptiActivityBuffer>(100);
    uint8_t* addr = buf->data();
    (*map)[addr] = std::move(buf);
    return map;
  }
  std::vector<const CUpti_Activity*> records;
};

void addMetadata(GenericTraceActivity& op, const K2JTraceFile& tf, const k2jt_md_entry& e) {
  const std::string key = tf.str(e.key);
  switch (e.type) {
    case 0: op.addTypedMetadata(key, TypedValue{(int64_t)e.value}); break;
    case 1: op.addTypedMetadata(key, TypedValue{(uint64_t)e.value}); break;
    case 2: { double d; memcpy(&d, &e.value, 8); op.addTypedMetadata(key, TypedValue{d}); break; }
    case 3: op.addTypedMetadata(key, TypedValue{e.value != 0}); break;
    case 4: op.addMetadataQuoted(key, tf.str((uint32_t)e.value)); break;
    case 5: op.addTypedMetadata(key, TypedValue{RawJson{tf.str((uint32_t)e.value)}}); break;
    case 6: { double d; memcpy(&d, &e.value, 8); op.addCounterValue(key, d); break; }
    default: throw std::runtime_error("bad metadata type");
  }
}

// Records the key order a GenericTraceActivity visits its metadata in.
class OrderVisitor final : public ITypedMetadataVisitor {
 public:
  std::vector<std::string> keys;
 private:
  void visitValue(const MetadataField<int64_t>& f, int64_t) override { keys.emplace_back(f.name); }
  void visitValue(const MetadataField<double>& f, double) override { keys.emplace_back(f.name); }
  void visitValue(const MetadataField<bool>& f, bool) override { keys.emplace_back(f.name); }
  void visitValue(const MetadataField<std::string>& f, std::string_view) override { keys.emplace_back(f.name); }
  void visitValue(const MetadataField<std::vector<int64_t>>& f, const std::vector<int64_t>&) override { keys.emplace_back(f.name); }
  void visitValue(const MetadataField<std::vector<std::string>>& f, const std::vector<std::string>&) override { keys.emplace_back(f.name); }
  void visitValue(const MetadataField<RawJson>& f, const RawJson&) override { keys.emplace_back(f.name); }
  void visitValue(const MetadataField<uint64_t>& f, uint64_t) override { keys.emplace_back(f.name); }
  void visitValue(const MetadataField<InputShapes>& f, const InputShapes&) override { keys.emplace_back(f.name); }
  void visitUnsupported(std::string_view n) override { keys.emplace_back(n); }
  void beginDict(std::string_view) override {}
  void endDict() override {}
};

void fillOp(GenericTraceActivity& op, const K2JTraceFile& tf, size_t i) {
  op.startTime = tf.ptr<int64_t>("OPSTART")[i];
  op.endTime = tf.ptr<int64_t>("OPEND")[i];
  op.id = tf.ptr<int32_t>("OPID")[i];
  op.device = tf.ptr<int32_t>("OPDEV")[i];
  op.resource = tf.ptr<int64_t>("OPRES")[i];
  op.threadId = tf.ptr<int32_t>("OPTHR")[i];
  op.flow.id = tf.ptr<uint32_t>("OPFLOW")[i];
  const uint8_t ft = tf.ptr<uint8_t>("OPFLOWT")[i];
  op.flow.type = ft & 0xf;
  op.flow.start = (ft >> 4) & 1;
  const uint32_t* mdoff = tf.ptr<uint32_t>("OPMDOFF");
  const k2jt_md_entry* md = tf.ptr<k2jt_md_entry>("MDENT");
  // The container lists entries in VISIT order.  Inserting them in reverse reproduces that order in
  // the reference's unordered_map (a new node goes to the front of the list, or to the front of its
  // bucket's run, which for a valid visit order is the same place); verified below.
  for (uint32_t e = mdoff[i + 1]; e > mdoff[i]; e--) if (md[e - 1].type != 6) addMetadata(op, tf, md[e - 1]);
  for (uint32_t e = mdoff[i]; e < mdoff[i + 1]; e++) if (md[e].type == 6) addMetadata(op, tf, md[e]);  // counter values: a list, in order
  if (mdoff[i + 1] - mdoff[i] > 1) {
    OrderVisitor v;
    op.visitTypedMetadata(v);
    for (uint32_t e = mdoff[i], k = 0; e < mdoff[i + 1]; e++) {
      if (md[e].type == 6) continue;
      if (v.keys[k++] != tf.str(md[e].key)) {
        fprintf(stderr, "metadata order mismatch at op %zu: container has '%s', reference visits '%s'\n",
                i, tf.str(md[e].key).c_str(), v.keys[k - 1].c_str());
        exit(3);
      }
    }
  }
}

void setupFakes(const K2JTraceFile& tf, const k2jt_params& p) {
  const k2jt_device_props* dp = tf.ptr<k2jt_device_props>("DEVPROPS");
  k2j_fake_set_device_count(p.n_devices);
  for (int i = 0; i < p.n_devices; i++) {
    cudaDeviceProp* c = k2j_fake_device_prop(i);
    memset(c, 0, sizeof(*c));
    strncpy(c->name, dp[i].name, sizeof(c->name) - 1);
    c->major = dp[i].major;
    c->minor = dp[i].minor;
    c->maxThreadsPerBlock = dp[i].max_threads_per_block;
    c->maxThreadsPerMultiProcessor = dp[i].max_threads_per_sm;
    c->regsPerBlock = dp[i].regs_per_block;
    c->regsPerMultiprocessor = dp[i].regs_per_sm;
    c->warpSize = dp[i].warp_size;
    c->multiProcessorCount = dp[i].num_sms;
    c->sharedMemPerBlock = dp[i].smem_per_block;
    c->sharedMemPerBlockOptin = dp[i].smem_per_block_optin;
    c->sharedMemPerMultiprocessor = dp[i].smem_per_sm;
    c->reservedSharedMemPerBlock = dp[i].reserved_smem_per_block;
    c->totalGlobalMem = dp[i].total_global_mem;
  }
  k2j_fake_set_pid(p.pid);
  // Any instant inside the 7 889 238 s period that starts at base_time gives that base time.
  k2j_fake_set_now_ns(p.base_time_ns + 1000000000LL);
  if (ChromeTraceBaseTime::singleton().get() != p.base_time_ns) {
    fprintf(stderr, "base time %lld is not a period boundary (reference computes %lld)\n",
            (long long)p.base_time_ns, (long long)ChromeTraceBaseTime::singleton().get());
    exit(4);
  }
  if (processId() != p.pid) {
    fprintf(stderr, "pid pin failed\n");
    exit(4);
  }
}

double runMode0(const K2JTraceFile& tf, const k2jt_params& p, const std::string& out) {
  const size_t n = tf.count<int64_t>("OPSTART");
  TraceSpan span(p.window_start_ns, p.window_end_ns, "benchmark_trace");
  std::vector<GenericTraceActivity> acts;
  acts.reserve(n);
  for (size_t i = 0; i < n; i++) {
    GenericTraceActivity op(span, (ActivityType)tf.ptr<int32_t>("OPTYPE")[i], tf.str(tf.ptr<uint32_t>("OPNAME")[i]));
    fillOp(op, tf, i);
    acts.push_back(std::move(op));
  }
  auto t0 = std::chrono::steady_clock::now();
  {
    ChromeTraceLogger logger(out);
    std::unordered_map<std::string, std::string> metadata;
    logger.handleTraceStart(metadata, "");
    for (const auto& a : acts) logger.handleGenericActivity(a);
    const Config config;
    logger.finalizeTrace(config, nullptr, p.window_end_ns);
  }
  auto t1 = std::chrono::steady_clock::now();
  return std::chrono::duration<double>(t1 - t0).count();
}

double runMode1(const K2JTraceFile& tf, const k2jt_params& p, const std::string& out) {
  // Mutable copy of the raw records: kernel name fields become real pointers.
  std::vector<uint8_t> cupti(tf.ptr<uint8_t>("CUPTI"), tf.ptr<uint8_t>("CUPTI") + tf.count<uint8_t>("CUPTI"));
  const size_t nstr = tf.count<uint64_t>("POOLOFF") ? tf.count<uint64_t>("POOLOFF") - 1 : 0;
  std::vector<std::string> names(nstr);
  for (size_t i = 0; i < nstr; i++) names[i] = tf.str((uint32_t)i);

  ReplayCuptiActivities cuptiApi;
  const uint64_t* bt = tf.ptr<uint64_t>("BUFTAB");
  const size_t nbuf = tf.count<uint64_t>("BUFTAB") / 2;
  for (size_t b = 0; b < nbuf; b++) {
    size_t pos = bt[2 * b], end = bt[2 * b] + bt[2 * b + 1];
    while (pos < end) {
      auto* rec = reinterpret_cast<CUpti_Activity*>(&cupti[pos]);
      size_t sz = recordSize(rec->kind);
      if (sz == 0) {
        // Unknown kinds are still handed to the reference (it counts them); size unknown => stop buffer.
        cuptiApi.records.push_back(rec);
        break;
      }
      if (rec->kind == CUPTI_ACTIVITY_KIND_CONCURRENT_KERNEL) {
        auto* k = reinterpret_cast<CUpti_ActivityKernel9*>(rec);
        uint64_t id;
        memcpy(&id, &k->name, 8);
        k->name = names.at(id).c_str();
      }
      cuptiApi.records.push_back(rec);
      pos += sz;
    }
  }

  Config cfg;
  cfg.validate(std::chrono::system_clock::now());
  if (!(p.flags & 1)) {
    auto types = cfg.selectedActivityTypes();
    types.erase(ActivityType::GPU_USER_ANNOTATION);
    cfg.setSelectedActivityTypes(types);
  }
  ActivityLoggerFactory loggerFactory;
  loggerFactory.addProtocol("file", [](const std::string& url) {
    return std::unique_ptr<ActivityLogger>(new ChromeTraceLogger(url));
  });

  CuptiActivityProfiler profiler(cuptiApi, /*cpuOnly=*/false);
  auto tp = [](int64_t ns) {
    return std::chrono::time_point<std::chrono::system_clock>(
        std::chrono::duration_cast<std::chrono::system_clock::duration>(std::chrono::nanoseconds(ns)));
  };
  profiler.configure(cfg, tp(p.window_start_ns));
  profiler.startTrace(tp(p.window_start_ns));
  profiler.stopTrace(tp(p.window_end_ns));

  use_cupti_tsc() = true;
  if (p.ts_mode == 0) {
    get_time_converter() = [](approx_time_t t) { return t; };
  } else {
    // Same expression as the lambda returned by ApproximateClockToUnixTimeConverter::makeConverter
    // (libkineto/src/ApproximateClock.cpp:83-90), with fixed instead of measured constants.
    long double scale_factor = ldexpl((long double)p.conv_scale_mant, p.conv_scale_exp - 63);
    time_t t0 = p.conv_t0;
    approx_time_t t0_approx = p.conv_t0_approx;
    get_time_converter() = [=](approx_time_t t_approx) {
      return t_approx > t0_approx
          ? static_cast<time_t>(static_cast<double>(t_approx - t0_approx) * scale_factor) + t0
          : 0;
    };
  }

  const int32_t* tm = tf.ptr<int32_t>("TIDMAP");
  for (size_t i = 0; i < tf.count<int32_t>("TIDMAP") / 2; i++) {
    profiler.recordThreadInfo(/*sysTid=*/tm[2 * i + 1], /*tid=*/tm[2 * i], /*pid=*/p.pid);
  }

  const size_t nops = tf.count<int64_t>("OPSTART");
  if (nops) {
    auto cpu = std::make_unique<CpuTraceBuffer>();
    cpu->span = TraceSpan(p.window_start_ns, p.window_end_ns, "Synthetic trace");
    cpu->gpuOpCount = 0;
    for (size_t i = 0; i < nops; i++) {
      GenericTraceActivity op(cpu->span, (ActivityType)tf.ptr<int32_t>("OPTYPE")[i], tf.str(tf.ptr<uint32_t>("OPNAME")[i]));
      fillOp(op, tf, i);
      cpu->emplace_activity(std::move(op));
      cpu->span.opCount++;
    }
    profiler.transferCpuTrace(std::move(cpu));
  }

  auto t0 = std::chrono::steady_clock::now();
  auto logger = std::make_unique<MemoryTraceLogger>(cfg);
  profiler.processTrace(*logger);
  ActivityTrace trace(std::move(logger), loggerFactory);
  trace.save(out);
  auto t1 = std::chrono::steady_clock::now();
  profiler.reset();
  return std::chrono::duration<double>(t1 - t0).count();
}

} // namespace

int main(int argc, char** argv) {
  SET_LOG_SEVERITY_LEVEL(ERROR);
  if (argc >= 2 && std::string(argv[1]) == "--version") {
    printf("fmt %d cuda %d cupti_api %d long_double_mant_dig %d\n", FMT_VERSION, CUDA_VERSION, CUPTI_API_VERSION, __LDBL_MANT_DIG__);
    return 0;
  }
  if (argc >= 2 && std::string(argv[1]) == "--md-order") {
    static TraceSpan span(0, 0, "x");
    GenericTraceActivity op(span, ActivityType::CPU_OP, "x");
    for (int i = 2; i < argc; i++) op.addTypedMetadata(argv[i], TypedValue{(int64_t)i});
    OrderVisitor v;
    op.visitTypedMetadata(v);
    for (auto& k : v.keys) printf("%s\n", k.c_str());
    return 0;
  }
  if (argc >= 3 && std::string(argv[1]) == "--cbid-names") {
    FILE* f = fopen(argv[2], "w");
    for (uint32_t c = 0; c < (uint32_t)CUPTI_RUNTIME_TRACE_CBID_SIZE; c++) fprintf(f, "R %u %s\n", c, runtimeCbidName(c).c_str());
    for (uint32_t c = 0; c < (uint32_t)CUPTI_DRIVER_TRACE_CBID_SIZE; c++) fprintf(f, "D %u %s\n", c, driverCbidName(c).c_str());
    fclose(f);
    return 0;
  }
  if (argc < 3) {
    fprintf(stderr, "usage: ref_driver <trace.k2jt> <out.json> [--repeat N]\n");
    return 2;
  }
  int repeat = 1;
  for (int i = 3; i + 1 < argc; i++) {
    if (std::string(argv[i]) == "--repeat") repeat = atoi(argv[i + 1]);
  }
  try {
    K2JTraceFile tf(argv[1]);
    const k2jt_params p = *tf.ptr<k2jt_params>("PARAMS");
    setupFakes(tf, p);
    double best = 1e30, sum = 0;
    for (int r = 0; r < repeat; r++) {
      double s = p.mode == 0 ? runMode0(tf, p, argv[2]) : runMode1(tf, p, argv[2]);
      best = std::min(best, s);
      sum += s;
    }
    printf("{\"seconds_mean\": %.6f, \"seconds_min\": %.6f, \"repeat\": %d, \"fmt_version\": %d}\n",
           sum / repeat, best, repeat, FMT_VERSION);
  } catch (const std::exception& e) {
    fprintf(stderr, "ref_driver: %s\n", e.what());
    return 1;
  }
  return 0;
}
