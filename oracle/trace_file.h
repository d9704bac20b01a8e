// TEST INFRASTRUCTURE — reader for the synthetic-trace container shared by the two CPU checkers
// (ref_driver.cpp, which feeds the unmodified reference, and k2j_oracle.cpp, our restatement).
// The product library never includes this file; its inputs arrive as plain pointers through the
// C ABI declared in include/k2j.h.  The Python writer is kineto_b200/tracefile.py.
//
// Container layout (little endian):
//   char     magic[8] = "K2JTRACE"
//   uint32   version  = 1
//   uint32   n_sections
//   section table: n_sections x { char tag[8]; uint64 offset; uint64 size_bytes; }
//   section payloads, each 64-byte aligned
//
// Sections (all optional except PARAMS); element types in brackets:
//   PARAMS   [k2jt_params x1]
//   DEVPROPS [k2jt_device_props x n_devices]
//   POOLOFF  [uint64 x (n_strings+1)]   POOLDATA [bytes]          shared string pool
//   CUPTI    [bytes]  raw CUPTI activity records, packed back to back, 8-byte aligned.
//            The 8-byte `name` pointer field of kernel records holds a string-pool id instead.
//   BUFTAB   [uint64 x 2 x n_buffers]  (byte offset into CUPTI, valid size) per drained buffer
//   TIDMAP   [int32 x 2 x n_threads]   (CUPTI thread id, system thread id)
//   RTNAME   [uint32 x n_rt_cbids]  string-pool id of the runtime callback name per cbid
//   DRNAME   [uint32 x n_dr_cbids]  same for the driver domain
//   OPSTART/OPEND [int64]  OPID [int32]  OPDEV [int32]  OPRES [int64]  OPTHR [int32]
//   OPTYPE [int32: libkineto ActivityType value]  OPNAME [uint32 pool id]
//   OPFLOW [uint32 flow id]  OPFLOWT [uint8: flow type | (start << 4)]
//   OPMDOFF [uint32 x (n_ops+1)]  MDENT [k2jt_md_entry]   per-op typed metadata in visit order
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#pragma pack(push, 1)
struct k2jt_params {
  int64_t base_time_ns;     // ChromeTraceBaseTime value
  int64_t window_start_ns;  // captureWindowStartTime_
  int64_t window_end_ns;    // captureWindowEndTime_
  int32_t pid;              // processId()
  int32_t mode;             // 0: ops straight into the JSON logger (json_output_benchmark style)
                            // 1: processTrace into MemoryTraceLogger, then ActivityTrace::save()
  int32_t ts_mode;          // 0: CUPTI timestamps already unix ns; 1: TSC affine conversion
  int32_t flags;            // bit0: GPU_USER_ANNOTATION enabled; bit1: stable sort by start ts
  int64_t conv_t0;          // converter: t0 (unix ns)
  uint64_t conv_t0_approx;  // converter: t0 in ticks
  uint64_t conv_scale_mant; // converter: x87 80-bit scale factor, 64-bit significand
  int32_t conv_scale_exp;   //            and unbiased exponent: scale = mant * 2^(exp-63)
  int32_t n_devices;
};
struct k2jt_device_props {  // the cudaDeviceProp fields the path reads
  int32_t major, minor;
  int32_t max_threads_per_block, max_threads_per_sm;
  int32_t regs_per_block, regs_per_sm;
  int32_t warp_size, num_sms;
  uint64_t smem_per_block, smem_per_block_optin, smem_per_sm, reserved_smem_per_block;
  uint64_t total_global_mem;
  char name[64];
};
struct k2jt_md_entry {
  uint32_t key;   // string-pool id of the key
  uint32_t type;  // 0 int64, 1 uint64, 2 double (bit pattern), 3 bool, 4 quoted string (pool id),
                  // 5 raw JSON text (pool id)
  uint64_t value;
};
#pragma pack(pop)

struct K2JTraceFile {
  std::vector<uint8_t> blob;
  std::map<std::string, std::pair<uint64_t, uint64_t>> sec;

  explicit K2JTraceFile(const std::string& path) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) throw std::runtime_error("cannot open " + path);
    fseek(f, 0, SEEK_END);
    long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    blob.resize(n);
    if (fread(blob.data(), 1, n, f) != (size_t)n) throw std::runtime_error("short read");
    fclose(f);
    if (n < 16 || memcmp(blob.data(), "K2JTRACE", 8) != 0) throw std::runtime_error("bad magic");
    uint32_t ver, ns;
    memcpy(&ver, &blob[8], 4);
    memcpy(&ns, &blob[12], 4);
    if (ver != 1) throw std::runtime_error("bad version");
    for (uint32_t i = 0; i < ns; i++) {
      const uint8_t* e = &blob[16 + 24 * i];
      char tag[9] = {0};
      memcpy(tag, e, 8);
      uint64_t off, sz;
      memcpy(&off, e + 8, 8);
      memcpy(&sz, e + 16, 8);
      if (off + sz > (uint64_t)n) throw std::runtime_error("section out of range");
      sec[tag] = {off, sz};
    }
  }
  bool has(const char* tag) const { return sec.count(tag) != 0; }
  template <class T>
  const T* ptr(const char* tag) const {
    auto it = sec.find(tag);
    return it == sec.end() ? nullptr : reinterpret_cast<const T*>(&blob[it->second.first]);
  }
  template <class T>
  size_t count(const char* tag) const {
    auto it = sec.find(tag);
    return it == sec.end() ? 0 : it->second.second / sizeof(T);
  }
  std::string str(uint32_t id) const {
    const uint64_t* off = ptr<uint64_t>("POOLOFF");
    const char* data = ptr<char>("POOLDATA");
    return std::string(data + off[id], data + off[id + 1]);
  }
};
