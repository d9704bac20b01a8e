// B200TraceLogger — the libkineto::ActivityLogger that writes the Chrome-trace file through libk2j.
//
// This is the file a libkineto maintainer adds next to src/output_json.{h,cpp}; it compiles against
// libkineto's own headers (include/output_base.h, src/CuptiActivity.h) and links libk2j.so.  It is a
// drop-in for ChromeTraceLogger behind both creation paths of the reference:
//   loggerFactory.addProtocol("file", [](const std::string& p) { return std::make_unique<B200TraceLogger>(p); });
// (libkineto/src/ActivityProfilerController.cpp:108-129, libkineto/src/ActivityLoggerFactory.h:33-61).
//
// Division of labour: every activity event ("X" and flow events) is formatted on the GPU by libk2j;
// the O(devices + threads + spans) text around them — header, metadata rows, trace spans, trailer —
// is written here, in the order the calls arrive, exactly as ChromeTraceLogger orders its output.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "output_base.h"

struct k2j_ctx;

namespace KINETO_NAMESPACE {

class B200TraceLogger : public libkineto::ActivityLogger {
 public:
  explicit B200TraceLogger(const std::string& traceFileName, int cudaDevice = 0);
  ~B200TraceLogger() override;

  void handleDeviceInfo(const DeviceInfo& info, int64_t time) override;
  void handleResourceInfo(const ResourceInfo& info, int64_t time) override;
  void handleOverheadInfo(const OverheadInfo& info, int64_t time) override;
  void handleTraceSpan(const TraceSpan& span) override;
  void handleActivity(const libkineto::ITraceActivity& activity) override;
  void handleGenericActivity(const libkineto::GenericTraceActivity& activity) override;
  void handleTraceStart(const std::unordered_map<std::string, std::string>& metadata,
                        const std::string& device_properties) override;
  void finalizeMemoryTrace(const std::string&, const Config&) override {}
  void finalizeTrace(const Config& config, std::unique_ptr<ActivityBuffers> buffers, int64_t endTime) override;

  // Number of activities that could not be handed to the GPU path (unsupported activity classes).
  size_t skippedActivities() const { return skipped_; }

 private:
  struct Impl;
  std::unique_ptr<Impl> impl_;
  size_t skipped_ = 0;
};

}  // namespace KINETO_NAMESPACE
