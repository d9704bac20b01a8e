// Device side of libk2j: record segmentation, join tables, the size pass, the device-wide scan and
// the emit pass.  All kernels are plain streaming integer/byte kernels for sm_100a; the bound is HBM
// bandwidth (there is no dense contraction anywhere on this path).
//
// Data flow (one run):
//   k_escape_pool    per distinct string: JSON-sanitised copies (name flavour, metadata flavour)
//   k_seg_chunks     per 4 KiB chunk of every CUPTI buffer: record length per 8-byte slot, and for
//                    each of the 26 possible entry slots the slot at which a walk leaves the chunk
//   k_seg_compose    per buffer: chains the exit maps -> true entry slot of every chunk
//   k_seg_count      per chunk: walk from the true entry, count records per class
//   k_scan_*         exclusive scans (chunk counts, later event sizes)
//   k_seg_write      per chunk: walk again, fill the per-class work lists, insert
//                    EXTERNAL_CORRELATION records into the correlation tables (last writer wins)
//   k_build_ops      CPU-op id -> row table (last writer wins)
//   k_events<Count>  one thread per event, class-sorted: exact JSON byte length of the event
//   k_events<Write>  same traversal, bytes go straight to their final offset
#pragma once
#include <cuda_runtime.h>
#include <cuda_occupancy.h>
#include <limits.h>
#include <stdint.h>

#include "k2j_format.cuh"

namespace k2j {

// ---- record classes ---------------------------------------------------------------------------
enum : int { C_API = 0, C_KERNEL = 1, C_MEMCPY = 2, C_MEMCPY2 = 3, C_MEMSET = 4, C_EXT = 5,
             C_EXT_USER = 6 /* slot class only: EXTERNAL_CORRELATION of kind CUSTOM1; counted in C_EXT too */,
             C_NCLASS = 6,
             C_EVENTS = 6 /* column 6 of the count matrix: records that own an event slot */,
             C_UNEXPECTED = 7 /* column 7: records of unknown kind */,
             C_USER = 8 /* column 8: CUSTOM1 correlation records */, C_NCOL = 9, C_OP = 9 };
enum : uint32_t { K_MEMCPY = 1, K_MEMSET = 2, K_DRIVER = 4, K_RUNTIME = 5, K_KERNEL = 10, K_MEMCPY2 = 22, K_EXTCORR = 39 };

constexpr int kChunkSlots = 512;            // 4 KiB of 8-byte slots
constexpr int kMaxEntry = 26;               // longest record is 208 B = 26 slots
constexpr uint8_t kExitTerminate = 254;     // the walk hit a record it cannot size
constexpr uint8_t kEntryNone = 255;         // chunk is unreachable

// size/8 | class<<5 for a record kind; 0 = unknown
__device__ __forceinline__ uint32_t slot_code(uint32_t kind, uint32_t word1) {
  switch (kind) {
    case K_KERNEL: return 26u | (C_KERNEL << 5);
    case K_MEMCPY: return 11u | (C_MEMCPY << 5);
    case K_MEMCPY2: return 12u | (C_MEMCPY2 << 5);
    case K_MEMSET: return 11u | (C_MEMSET << 5);
    case K_RUNTIME: case K_DRIVER: return 5u | (C_API << 5);
    case K_EXTCORR: return 3u | ((word1 == 4u ? C_EXT_USER : C_EXT) << 5);  // word1 = externalKind
    default: return 0u;
  }
}

struct DevProps {
  int32_t major, minor, max_threads_per_block, max_threads_per_sm, regs_per_block, regs_per_sm, warp_size, num_sms;
  uint64_t smem_per_block, smem_per_block_optin, smem_per_sm, reserved_smem_per_block;
};

struct Counters {
  unsigned long long x_events, flow_events, out_of_range, blocklisted_runtime, invalid_external_correlation,
      unexpected, name_bytes, device_check, n_user;
};

struct MdEntry { uint32_t key, type; uint64_t value; };
struct ExtRec { uint64_t external_id; uint32_t correlation_id; uint32_t external_kind; };
struct SpanRec { int64_t start, end; uint64_t first_event; uint32_t device, stream; int32_t op_id; uint32_t op_row; };

struct Dev {
  // scalars
  int64_t base, win_start, win_end;
  int32_t pid, ts_mode, flags, n_devices; uint32_t type_mask;
  int64_t conv_t0; uint64_t conv_t0a, conv_mant; int32_t conv_exp;
  const DevProps* props;
  // strings
  const uint64_t* pool_off; const uint8_t* pool_data; uint32_t n_strings;
  uint32_t* esc_name_len; uint32_t* esc_md_len; uint8_t* esc_name; uint8_t* esc_md;
  const uint32_t* rt_names; uint32_t n_rt; const uint32_t* dr_names; uint32_t n_dr;
  const int32_t* tid_pairs; uint32_t n_tid_pairs; unsigned long long* tid_tab; uint32_t tid_mask;
  // CUPTI bytes and segmentation
  const uint8_t* cupti; uint64_t cupti_bytes;
  const uint64_t* buf_off; const uint64_t* buf_valid; const uint32_t* buf_chunk_base; uint32_t n_buf, n_chunks;
  uint8_t* slot_code;      // per 8-byte slot of the CUPTI bytes
  uint8_t* exit_map;       // n_chunks x 32
  uint8_t* chunk_entry;    // n_chunks
  uint32_t* chunk_cnt;     // C_NCOL columns x n_chunks
  uint64_t* chunk_base;    // C_NCOL columns x n_chunks (exclusive scan of chunk_cnt)
  // CPU ops
  uint64_t n_ops;
  const int64_t* op_start; const int64_t* op_end; const int32_t* op_id; const int32_t* op_device;
  const int64_t* op_resource; const int32_t* op_thread; const int32_t* op_type; const uint32_t* op_name; const uint32_t* op_flow;
  const uint8_t* op_flowt; const uint32_t* op_mdoff; const MdEntry* md;
  // EXTERNAL_CORRELATION records in processing order, compacted: the local shard's (ext_local) and
  // the array the tables are built from (ext_all: the same array, or all shards' arrays gathered)
  ExtRec* ext_local; const ExtRec* ext_all; uint64_t n_ext_all;
  const int32_t* join_op_ids; uint64_t n_join_ops;  // CPU-op ids the join sees (local or gathered)
  // join tables: 64-bit entries (key << 32 | value + 1), 0 = empty
  unsigned long long* corr_tab; uint32_t corr_mask;
  unsigned long long* user_tab; uint32_t user_mask;
  unsigned long long* op_tab; uint32_t op_mask;
  // user-annotation spans (GpuUserEventMap): (device, stream) set, then (set slot, op id) -> span
  unsigned long long* ds_tab; uint32_t ds_mask;
  unsigned long long* span_key; unsigned long long* span_nstart; unsigned long long* span_end;
  unsigned long long* span_nfirst; uint32_t* span_row; uint32_t span_mask;  // span_key == nullptr: off
  // work lists (class-sorted) and per-event arrays
  uint32_t* work_slot; uint32_t* work_ev; uint64_t cls_begin[C_NCLASS]; uint64_t cls_count[C_NCLASS];
  uint64_t ops_begin; uint64_t n_work;
  uint32_t* ev_size; const uint64_t* ev_off; uint64_t n_events;
  uint8_t* out; uint64_t out_cap;
  Counters* counters;
};

// Flag bit 2: CPU-side activities with device 0 show under the process id (the pid-0 override of
// GenericActivityProfiler.cpp:263-271 as seen through ActivityTrace::save()).
__device__ __forceinline__ int32_t op_pid(const Dev& d, int32_t device) { return (device == 0 && (d.flags & 4)) ? d.pid : device; }
__device__ __forceinline__ uint64_t esc_name_pos(const Dev& d, uint32_t id) { return ((2 * d.pool_off[id] + 7) & ~7ull) + 16ull * id; }
__device__ __forceinline__ uint64_t esc_md_pos(const Dev& d, uint32_t id) { return ((d.pool_off[id] + 7) & ~7ull) + 8ull * id; }

// ---- hashing ----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t hash32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
// Inserts key -> value; among equal keys the largest value stays (values are positions, so that is
// the last writer in processing order: std::unordered_map::operator[] assignment semantics,
// libkineto/src/CuptiActivityProfiler.cpp:293-296, GenericActivityProfiler.cpp:262).
__device__ __forceinline__ bool tab_insert(unsigned long long* tab, uint32_t mask, uint32_t key, uint32_t value) {
  const unsigned long long entry = ((unsigned long long)key << 32) | (unsigned long long)(value + 1u);
  uint32_t i = hash32(key) & mask;
  for (uint32_t probes = 0; probes <= mask; probes++) {
    unsigned long long old = tab[i];
    if (old == 0) {
      old = atomicCAS(&tab[i], 0ull, entry);
      if (old == 0) return true;
    }
    if ((uint32_t)(old >> 32) == key) { atomicMax(&tab[i], entry); return true; }
    i = (i + 1) & mask;
  }
  return false;
}
// Same, but the smallest value stays (first writer wins: recordThreadInfo only inserts when the key is
// absent, libkineto/src/GenericActivityProfiler.h:256-267).
__device__ __forceinline__ bool tab_insert_min(unsigned long long* tab, uint32_t mask, uint32_t key, uint32_t value) {
  const unsigned long long entry = ((unsigned long long)key << 32) | (unsigned long long)(value + 1u);
  uint32_t i = hash32(key) & mask;
  for (uint32_t probes = 0; probes <= mask; probes++) {
    unsigned long long old = tab[i];
    if (old == 0) {
      old = atomicCAS(&tab[i], 0ull, entry);
      if (old == 0) return true;
    }
    if ((uint32_t)(old >> 32) == key) { if (old > entry) atomicMin(&tab[i], entry); return true; }
    i = (i + 1) & mask;
  }
  return false;
}
// Returns value or 0xFFFFFFFF.
__device__ __forceinline__ uint32_t tab_find(const unsigned long long* tab, uint32_t mask, uint32_t key) {
  if (tab == nullptr) return 0xFFFFFFFFu;
  uint32_t i = hash32(key) & mask;
  for (uint32_t probes = 0; probes <= mask; probes++) {
    unsigned long long e = tab[i];
    if (e == 0) return 0xFFFFFFFFu;
    if ((uint32_t)(e >> 32) == key) return (uint32_t)e - 1u;
    i = (i + 1) & mask;
  }
  return 0xFFFFFFFFu;
}

// ---- string pool escaping -----------------------------------------------------------------------
// One warp per string.  Name flavour (output_json.cpp:946-949): "kernel" -> "Kernel"; '\\' -> '/';
// '\n' dropped; any remaining byte outside 0x20..0x7e turns the whole name into "unknown"; '"' gets a
// backslash.  Metadata flavour (output_json.cpp:896-897): only '\\' -> '/' and '\n' dropped.
__global__ void k_escape_pool(Dev d) {
  const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (warp >= d.n_strings) return;
  const uint64_t b = d.pool_off[warp], e = d.pool_off[warp + 1];
  const uint32_t len = (uint32_t)(e - b);
  const uint8_t* src = d.pool_data + b;
  uint8_t* dn = d.esc_name + esc_name_pos(d, warp);
  uint8_t* dm = d.esc_md + esc_md_pos(d, warp);
  bool is_kernel = false;
  if (len == 6) {
    is_kernel = src[0] == 'k' && src[1] == 'e' && src[2] == 'r' && src[3] == 'n' && src[4] == 'e' && src[5] == 'l';
  }
  uint32_t on = 0, om = 0;
  bool bad = false;
  for (uint32_t base = 0; base < len; base += 32) {
    const uint32_t i = base + lane;
    const bool in = i < len;
    uint8_t c = in ? src[i] : 0;
    if (c == '\\') c = '/';
    const bool keep = in && c != '\n';
    const bool quote = keep && c == '"';
    const bool nonprint = keep && (c < 0x20 || c > 0x7e);
    const uint32_t keep_m = __ballot_sync(0xffffffffu, keep);
    const uint32_t quote_m = __ballot_sync(0xffffffffu, quote);
    bad |= __ballot_sync(0xffffffffu, nonprint) != 0;
    const uint32_t lt = (1u << lane) - 1u;
    if (keep) {
      const uint32_t pm = om + __popc(keep_m & lt);
      dm[pm] = c;
      const uint32_t pn = on + __popc(keep_m & lt) + __popc(quote_m & lt);
      if (quote) { dn[pn] = '\\'; dn[pn + 1] = c; }
      else dn[pn] = (is_kernel && i == 0) ? 'K' : c;
    }
    om += __popc(keep_m);
    on += __popc(keep_m) + __popc(quote_m);
  }
  __syncwarp();
  if (bad) {
    if (lane < 7) dn[lane] = "unknown"[lane];
    on = 7;
  }
  if (lane == 0) { d.esc_name_len[warp] = on; d.esc_md_len[warp] = om; }
}

// ---- segmentation -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t find_buffer(const Dev& d, uint32_t chunk) {
  uint32_t lo = 0, hi = d.n_buf;  // buf_chunk_base has n_buf + 1 entries
  while (hi - lo > 1) { uint32_t mid = (lo + hi) >> 1; if (d.buf_chunk_base[mid] <= chunk) lo = mid; else hi = mid; }
  return lo;
}

struct ChunkGeom { uint64_t slot0; uint32_t nvalid; bool last; };
__device__ __forceinline__ ChunkGeom chunk_geom(const Dev& d, uint32_t chunk) {
  const uint32_t b = find_buffer(d, chunk);
  const uint32_t c = chunk - d.buf_chunk_base[b];
  const uint64_t buf_slots = d.buf_valid[b] >> 3;
  ChunkGeom g;
  g.slot0 = (d.buf_off[b] >> 3) + (uint64_t)c * kChunkSlots;
  const uint64_t rem = buf_slots - (uint64_t)c * kChunkSlots;
  g.nvalid = rem < (uint64_t)kChunkSlots ? (uint32_t)rem : (uint32_t)kChunkSlots;
  g.last = (chunk + 1 == d.buf_chunk_base[b + 1]);
  return g;
}

constexpr int kSegWarps = 8;

// One warp per chunk: slot codes and exit map.
__global__ void __launch_bounds__(kSegWarps * 32) k_seg_chunks(Dev d) {
  __shared__ uint8_t s_code[kSegWarps][kChunkSlots];
  const uint32_t w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t chunk = blockIdx.x * kSegWarps + w;
  if (chunk >= d.n_chunks) return;
  const ChunkGeom g = chunk_geom(d, chunk);
  const uint2* words = reinterpret_cast<const uint2*>(d.cupti);
#pragma unroll
  for (int j = 0; j < kChunkSlots / 128; j++) {
    const uint32_t s = 4 * (lane + 32 * j);
    uint32_t packed = 0;
#pragma unroll
    for (int q = 0; q < 4; q++) {
      uint32_t code = 0;
      if (s + q < g.nvalid) { const uint2 w2 = words[g.slot0 + s + q]; code = slot_code(w2.x, w2.y); }
      packed |= code << (8 * q);
    }
    *reinterpret_cast<uint32_t*>(&s_code[w][s]) = packed;
    if (s < g.nvalid) {
      uint8_t* dst = d.slot_code + g.slot0 + s;
      if (((g.slot0 + s) & 3) == 0 && s + 4 <= g.nvalid) *reinterpret_cast<uint32_t*>(dst) = packed;
      else { for (int q = 0; q < 4; q++) if (s + q < g.nvalid) dst[q] = (uint8_t)(packed >> (8 * q)); }
    }
  }
  __syncwarp();
  uint8_t code = kEntryNone;
  if (lane < kMaxEntry) {
    uint32_t pos = lane;
    code = 0;
    // Bounded: every step advances by at least 3 slots.
    for (int it = 0; it < kChunkSlots; it++) {
      if (pos >= g.nvalid) { code = g.last ? (pos == g.nvalid ? 0 : kExitTerminate) : (uint8_t)(pos - g.nvalid); break; }
      const uint32_t n = s_code[w][pos] & 31u;
      if (n == 0) { code = kExitTerminate; break; }
      pos += n;
    }
  }
  d.exit_map[(uint64_t)chunk * 32 + lane] = code;
}

// One block per buffer: chain the exit maps.
__global__ void __launch_bounds__(256) k_seg_compose(Dev d) {
  constexpr int kTile = 1024;
  __shared__ uint8_t s_map[kTile * 32];
  __shared__ uint32_t s_entry;
  const uint32_t b = blockIdx.x;
  const uint32_t c0 = d.buf_chunk_base[b], c1 = d.buf_chunk_base[b + 1];
  if (threadIdx.x == 0) s_entry = 0;
  for (uint32_t t0 = c0; t0 < c1; t0 += kTile) {
    const uint32_t n = min((uint32_t)kTile, c1 - t0);
    __syncthreads();
    const uint4* src = reinterpret_cast<const uint4*>(d.exit_map + (uint64_t)t0 * 32);
    uint4* dst = reinterpret_cast<uint4*>(s_map);
    for (uint32_t i = threadIdx.x; i < n * 2; i += blockDim.x) dst[i] = src[i];
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t e = s_entry;
      for (uint32_t c = 0; c < n; c++) {
        d.chunk_entry[t0 + c] = (uint8_t)e;
        if (e != kEntryNone) {
          const uint8_t x = s_map[c * 32 + e];
          e = (x >= kMaxEntry) ? kEntryNone : x;
        }
      }
      s_entry = e;
    }
  }
}

// Walk helper: lane 0 of a warp walks one chunk from its true entry.  `visit(pos, code)` is called per
// record that starts in the chunk.  Returns false if the walk ended on an unknown kind.
template <class F>
__device__ __forceinline__ void walk_chunk(const uint8_t* codes, uint32_t entry, const ChunkGeom& g, F visit) {
  uint32_t pos = entry;
  for (int it = 0; it < kChunkSlots && pos < g.nvalid; it++) {
    const uint32_t code = codes[pos];
    const uint32_t n = code & 31u;
    if (n == 0 || (g.last && pos + n > g.nvalid)) { visit(pos, 0u); return; }  // unknown kind or overrun
    visit(pos, code);
    pos += n;
  }
}

__device__ __forceinline__ void load_codes(const Dev& d, const ChunkGeom& g, uint8_t* s, uint32_t lane) {
  for (uint32_t i = lane; i < (uint32_t)kChunkSlots; i += 32) s[i] = i < g.nvalid ? d.slot_code[g.slot0 + i] : 0;
  __syncwarp();
}

__global__ void __launch_bounds__(kSegWarps * 32) k_seg_count(Dev d) {
  __shared__ uint8_t s_code[kSegWarps][kChunkSlots];
  const uint32_t w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t chunk = blockIdx.x * kSegWarps + w;
  if (chunk >= d.n_chunks) return;
  const ChunkGeom g = chunk_geom(d, chunk);
  const uint32_t entry = d.chunk_entry[chunk];
  uint32_t cnt[C_NCOL];
#pragma unroll
  for (int i = 0; i < C_NCOL; i++) cnt[i] = 0;
  if (entry != kEntryNone) {
    load_codes(d, g, s_code[w], lane);
    if (lane == 0) {
      walk_chunk(s_code[w], entry, g, [&](uint32_t, uint32_t code) {
        if (code == 0) { cnt[C_UNEXPECTED]++; return; }
        uint32_t cls = code >> 5;
        cnt[C_USER] += (cls == (uint32_t)C_EXT_USER);
        if (cls == (uint32_t)C_EXT_USER) cls = C_EXT;
#pragma unroll
        for (int i = 0; i < C_NCLASS; i++) cnt[i] += (cls == (uint32_t)i);
        cnt[C_EVENTS] += (cls != (uint32_t)C_EXT);
      });
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < C_NCOL; i++) d.chunk_cnt[(uint64_t)i * d.n_chunks + chunk] = cnt[i];
  }
}

__global__ void __launch_bounds__(kSegWarps * 32) k_seg_write(Dev d) {
  __shared__ uint8_t s_code[kSegWarps][kChunkSlots];
  __shared__ uint16_t s_pos[kSegWarps][kChunkSlots / 3 + 2];
  __shared__ uint16_t s_rank[kSegWarps][kChunkSlots / 3 + 2];
  __shared__ uint16_t s_evrank[kSegWarps][kChunkSlots / 3 + 2];
  __shared__ uint32_t s_n[kSegWarps];
  const uint32_t w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t chunk = blockIdx.x * kSegWarps + w;
  if (chunk >= d.n_chunks) return;
  const uint32_t entry = d.chunk_entry[chunk];
  if (entry == kEntryNone) return;
  const ChunkGeom g = chunk_geom(d, chunk);
  load_codes(d, g, s_code[w], lane);
  if (lane == 0) {
    uint32_t cnt[C_NCLASS];
#pragma unroll
    for (int i = 0; i < C_NCLASS; i++) cnt[i] = 0;
    uint32_t n = 0, ev = 0;
    walk_chunk(s_code[w], entry, g, [&](uint32_t pos, uint32_t code) {
      if (code == 0) return;
      uint32_t cls = code >> 5;
      if (cls == (uint32_t)C_EXT_USER) cls = C_EXT;
      uint32_t r = 0;
#pragma unroll
      for (int i = 0; i < C_NCLASS; i++) if (cls == (uint32_t)i) r = cnt[i]++;
      s_pos[w][n] = (uint16_t)(pos | (cls << 12));
      s_rank[w][n] = (uint16_t)r;
      s_evrank[w][n] = (uint16_t)ev;
      ev += (cls != (uint32_t)C_EXT);
      n++;
    });
    s_n[w] = n;
  }
  __syncwarp();
  const uint32_t n = s_n[w];
  const uint64_t ev_base = d.n_ops + d.chunk_base[(uint64_t)C_EVENTS * d.n_chunks + chunk];
  for (uint32_t i = lane; i < n; i += 32) {
    const uint32_t pos = s_pos[w][i] & 0xfffu, cls = s_pos[w][i] >> 12;
    const uint64_t slot = g.slot0 + pos;
    if (cls == (uint32_t)C_EXT) {
      const uint8_t* r = d.cupti + slot * 8;
      ExtRec e;
      e.external_kind = *reinterpret_cast<const uint32_t*>(r + 4);
      e.external_id = *reinterpret_cast<const uint64_t*>(r + 8);
      e.correlation_id = *reinterpret_cast<const uint32_t*>(r + 16);
      d.ext_local[d.chunk_base[(uint64_t)C_EXT * d.n_chunks + chunk] + s_rank[w][i]] = e;
    } else {
      const uint64_t dst = d.cls_begin[cls] + d.chunk_base[(uint64_t)cls * d.n_chunks + chunk] + s_rank[w][i];
      d.work_slot[dst] = (uint32_t)slot;
      d.work_ev[dst] = (uint32_t)(ev_base + s_evrank[w][i]);
    }
  }
}

// CUPTI thread id -> system thread id.  Priority order: the explicit pairs, then every CPU-side activity
// of this process in order (processCpuTrace -> recordThreadInfo(resourceId, getThreadId, deviceId),
// libkineto/src/GenericActivityProfiler.cpp:272); the first writer of a thread id wins.
__global__ void k_build_tids(Dev d) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (uint64_t)d.n_tid_pairs + d.n_ops) return;
  uint32_t key;
  if (i < d.n_tid_pairs) key = (uint32_t)d.tid_pairs[2 * i];
  else {
    const uint64_t j = i - d.n_tid_pairs;
    if (op_pid(d, d.op_device[j]) != d.pid) return;
    key = (uint32_t)d.op_thread[j];
  }
  if (!tab_insert_min(d.tid_tab, d.tid_mask, key, (uint32_t)i)) atomicAdd(&d.counters->device_check, 1ull);
}
// CPU-op id -> position (last writer wins): activityMap_[id] = op, GenericActivityProfiler.cpp:262.
__global__ void k_build_ops(Dev d) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.n_join_ops) return;
  if (!tab_insert(d.op_tab, d.op_mask, (uint32_t)d.join_op_ids[i], (uint32_t)i)) atomicAdd(&d.counters->device_check, 1ull);
}
// correlation id -> index of the winning EXTERNAL_CORRELATION record (handleCorrelationActivity,
// CuptiActivityProfiler.cpp:290-302).  `count_invalid`: only the shard that owns a record counts it.
__global__ void k_build_corr(Dev d, uint64_t own_begin, uint64_t own_end) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.n_ext_all) return;
  const ExtRec e = d.ext_all[i];
  bool ok = true;
  if (e.external_kind == 3u) ok = tab_insert(d.corr_tab, d.corr_mask, e.correlation_id, (uint32_t)i);
  else if (e.external_kind == 4u) { ok = tab_insert(d.user_tab, d.user_mask, e.correlation_id, (uint32_t)i); atomicAdd(&d.counters->n_user, 1ull); }
  else if (i >= own_begin && i < own_end) atomicAdd(&d.counters->invalid_external_correlation, 1ull);
  if (!ok) atomicAdd(&d.counters->device_check, 1ull);
}

// ---- exclusive scan: u32 in -> u64 out, `gridDim.y` independent columns -----------------------------
constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;

__device__ __forceinline__ uint64_t block_exclusive_scan(uint64_t v, uint64_t* total) {
  __shared__ uint64_t s_warp[kScanThreads / 32];
  const uint32_t lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  uint64_t x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { uint64_t y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= (uint32_t)o) x += y; }
  __syncthreads();
  if (lane == 31) s_warp[w] = x;
  __syncthreads();
  uint64_t base = 0, tot = 0;
#pragma unroll
  for (int i = 0; i < kScanThreads / 32; i++) { if ((uint32_t)i < w) base += s_warp[i]; tot += s_warp[i]; }
  *total = tot;
  return base + x - v;
}

__global__ void __launch_bounds__(kScanThreads) k_scan_reduce(const uint32_t* in, uint64_t n, uint64_t col_stride, uint64_t* block_sums, uint32_t n_blocks) {
  const uint32_t* src = in + (uint64_t)blockIdx.y * col_stride;
  const uint64_t base = (uint64_t)blockIdx.x * kScanTile;
  uint64_t s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; k++) {
    const uint64_t i = base + (uint64_t)k * kScanThreads + threadIdx.x;
    if (i < n) s += src[i];
  }
  uint64_t tot;
  block_exclusive_scan(s, &tot);
  if (threadIdx.x == 0) block_sums[(uint64_t)blockIdx.y * n_blocks + blockIdx.x] = tot;
}
// One block per column scans the block sums in place (exclusive) and stores the column total.
__global__ void __launch_bounds__(kScanThreads) k_scan_sums(uint64_t* block_sums, uint32_t n_blocks, uint64_t* totals) {
  uint64_t* p = block_sums + (uint64_t)blockIdx.x * n_blocks;
  uint64_t carry = 0;
  for (uint32_t b0 = 0; b0 < n_blocks; b0 += kScanThreads) {
    const uint32_t i = b0 + threadIdx.x;
    const uint64_t v = i < n_blocks ? p[i] : 0;
    uint64_t tot;
    const uint64_t ex = block_exclusive_scan(v, &tot);
    if (i < n_blocks) p[i] = carry + ex;
    carry += tot;
    __syncthreads();
  }
  if (threadIdx.x == 0) totals[blockIdx.x] = carry;
}
__global__ void __launch_bounds__(kScanThreads) k_scan_apply(const uint32_t* in, uint64_t n, uint64_t col_stride, const uint64_t* block_sums, uint32_t n_blocks, uint64_t* out) {
  const uint32_t* src = in + (uint64_t)blockIdx.y * col_stride;
  uint64_t* dst = out + (uint64_t)blockIdx.y * col_stride;
  const uint64_t base = (uint64_t)blockIdx.x * kScanTile + (uint64_t)threadIdx.x * kScanItems;
  uint32_t v[kScanItems];
  uint64_t s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; k++) { const uint64_t i = base + k; v[k] = i < n ? src[i] : 0; s += v[k]; }
  uint64_t tot;
  uint64_t ex = block_exclusive_scan(s, &tot) + block_sums[(uint64_t)blockIdx.y * n_blocks + blockIdx.x];
#pragma unroll
  for (int k = 0; k < kScanItems; k++) { const uint64_t i = base + k; if (i < n) dst[i] = ex; ex += v[k]; }
}

// ---- output sink: 16-byte vector stores straight to the final position ----------------------------------
// Bytes are gathered in a 64-bit shift register, completed 32-bit words go to a 4-word staging slot
// of this lane in shared memory (word k of lane l lives at index k*32+l: conflict free), and every
// fourth word the slot leaves as one 16-byte store.  Only the first and last 16-byte block of an
// event are written with narrower stores, so neighbouring events never overwrite each other.
struct GlobalSink {
  static constexpr bool kCounting = false;
  uint64_t acc; int n; int k; int head; uint32_t* slot; uint4* p;
  __device__ __forceinline__ void init(uint8_t* dst, uint32_t* lane_slot) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(dst);
    const int phase = (int)(a & 15);
    p = reinterpret_cast<uint4*>(a - phase);
    k = phase >> 2; n = phase & 3; acc = 0; head = phase; slot = lane_slot;
  }
  __device__ __forceinline__ void store_partial(int from, int to) {
    uint8_t* b = reinterpret_cast<uint8_t*>(p);
    int i = from;
    while (i < to) {
      const uint32_t w = slot[(i >> 2) * 32];
      if ((i & 3) == 0 && i + 4 <= to) { *reinterpret_cast<uint32_t*>(b + i) = w; i += 4; }
      else { b[i] = (uint8_t)(w >> ((i & 3) * 8)); i++; }
    }
  }
  __device__ __forceinline__ void word(uint32_t x) {
    slot[(k & 3) * 32] = x;
    k++;
    if ((k & 3) == 0) {
      if (head) { store_partial(head, 16); head = 0; }
      else *p = make_uint4(slot[0], slot[32], slot[64], slot[96]);
      p++;
    }
  }
  __device__ __forceinline__ void put(uint32_t w, int len) {
    acc |= (uint64_t)w << (n * 8);
    n += len;
    if (n >= 4) { word((uint32_t)acc); acc >>= 32; n -= 4; }
  }
  __device__ __forceinline__ void skip(uint32_t) {}
  template <int N> __device__ __forceinline__ void lit(const Lit<N>& l) {
#pragma unroll
    for (int i = 0; i < N / 4; i++) put(l.w[i], 4);
    if (N % 4) put(l.w[N / 4], N % 4);
  }
  __device__ __forceinline__ void finish() {
    const int have = (k & 3) * 4 + n;
    if (n) slot[(k & 3) * 32] = (uint32_t)acc;
    if (have > head) store_partial(head, have);
  }
};

// ---- event formatting ---------------------------------------------------------------------------------------
K2J_CONST_TABLE char kTypeNames[29][24] = {  // libkineto/include/ActivityType.h:80-112
    "cpu_op", "user_annotation", "gpu_user_annotation", "gpu_memcpy", "gpu_memset", "kernel",
    "external_correlation", "cuda_runtime", "cuda_driver", "cpu_instant_event", "python_function",
    "overhead", "mtia_runtime", "mtia_ccp_events", "mtia_insight", "cuda_sync", "cuda_event",
    "mtia_counters", "glow_runtime", "cuda_profiler_range", "hpu_op", "xpu_runtime", "xpu_driver",
    "collective_comm", "privateuse1_runtime", "privateuse1_driver", "xpu_scope_profiler", "xpu_sync",
    "hardware_counters"};
K2J_CONST_TABLE char kMemcpyKind[12][12] = {  // libkineto/src/cupti_strings.cpp:15-41
    "<unknown>", "HtoD", "DtoH", "HtoA", "AtoH", "AtoA", "AtoD", "DtoA", "DtoD", "HtoH", "PtoP", "<unknown>"};
K2J_CONST_TABLE char kMemoryKind[9][16] = {  // libkineto/src/cupti_strings.cpp:43-66
    "Unknown", "Pageable", "Pinned", "Device", "Array", "Managed", "Device Static", "Managed Static", "Unrecognized"};

template <class S> __device__ __forceinline__ void put_cstr(S& s, const char* c) {
  for (int i = 0; c[i]; i++) put_char(s, c[i]);
}
// Copies an escaped pool string (8-byte aligned, padded to a multiple of 4 readable bytes).
template <class S> __device__ __forceinline__ void put_pool(S& s, const uint8_t* src, uint32_t len) {
  if (S::kCounting) { s.skip(len); return; }
  const uint32_t* w = reinterpret_cast<const uint32_t*>(src);
  uint32_t i = 0;
  for (; i + 4 <= len; i += 4) s.put(w[i >> 2], 4);
  if (i < len) s.put(w[i >> 2] & (0xFFFFFFFFu >> (8 * (4 - (len - i)))), (int)(len - i));
}
template <class S> __device__ __forceinline__ void put_name(S& s, const Dev& d, uint32_t id, unsigned long long* name_bytes) {
  if (id >= d.n_strings) { atomicAdd(&d.counters->device_check, 1ull); return; }
  const uint32_t len = d.esc_name_len[id];
  put_pool(s, d.esc_name + esc_name_pos(d, id), len);
  *name_bytes += len;
}
template <class S> __device__ __forceinline__ void put_mdstr(S& s, const Dev& d, uint32_t id) {
  if (id >= d.n_strings) { atomicAdd(&d.counters->device_check, 1ull); return; }
  put_pool(s, d.esc_md + esc_md_pos(d, id), d.esc_md_len[id]);
}

__device__ __forceinline__ int64_t conv_ts(const Dev& d, uint64_t t) {
  return d.ts_mode ? tsc_to_ns(t, d.conv_t0a, d.conv_t0, d.conv_mant, d.conv_exp) : (int64_t)t;
}
__device__ __forceinline__ int64_t conv_dur(const Dev& d, uint64_t s, uint64_t e) {
  return d.ts_mode ? conv_ts(d, e) - conv_ts(d, s) : (int64_t)(e - s);
}
__device__ __forceinline__ int64_t rel_ts(const Dev& d, int64_t t) { const int64_t r = t - d.base; return r < 0 ? 0 : r; }
__device__ __forceinline__ int64_t abs_tid(int64_t t) { return t == INT64_MIN ? 0 : (t < 0 ? -t : t); }

// linkedActivity(int32_t correlationId, cpuCorrelationMap_) (GenericActivityProfiler.cpp:397-408):
// the id is sign-extended before the lookup while keys were stored zero-extended, so ids >= 2^31
// never match; the external id must equal a CPU-op id exactly as a 64-bit value.
__device__ __forceinline__ bool linked_op(const Dev& d, uint32_t corr, int32_t* op_id) {
  if (corr & 0x80000000u) return false;
  const uint32_t idx = tab_find(d.corr_tab, d.corr_mask, corr);
  if (idx == 0xFFFFFFFFu) return false;
  const int64_t ext = (int64_t)d.ext_all[idx].external_id;
  if (ext != (int64_t)(int32_t)ext) return false;
  if (tab_find(d.op_tab, d.op_mask, (uint32_t)(int32_t)ext) == 0xFFFFFFFFu) return false;
  *op_id = (int32_t)ext;  // the linked op's correlationId() is the key it was found under
  return true;
}

// GenericActivityProfiler::handleGpuActivity's user-annotation step (GenericActivityProfiler.cpp:424-434)
// with GpuUserEventMap::insertOrExtendEvent (:292-311): per (device, stream) and annotation op the span
// [min start, max end] over the GPU activities correlated to it.  Runs in the size pass only.
__device__ __forceinline__ void span_update(const Dev& d, uint32_t corr, uint32_t dev, uint32_t stream, int64_t ts,
                                            int64_t dur, uint64_t ev) {
  if (d.span_key == nullptr) return;
  const uint32_t idx = tab_find(d.user_tab, d.user_mask, corr);
  if (idx == 0xFFFFFFFFu) return;
  const int64_t ext = (int64_t)d.ext_all[idx].external_id;
  if (ext != (int64_t)(int32_t)ext) return;
  const uint32_t row = tab_find(d.op_tab, d.op_mask, (uint32_t)(int32_t)ext);
  if (row == 0xFFFFFFFFu) return;
  // (device, stream) -> slot
  const unsigned long long dskey = (((unsigned long long)dev << 32) | stream) + 1ull;
  uint32_t i = hash32(dev * 0x9E3779B1u ^ stream) & d.ds_mask;
  uint32_t probes = 0;
  for (; probes <= d.ds_mask; probes++) {
    unsigned long long old = d.ds_tab[i];
    if (old == 0) old = atomicCAS(&d.ds_tab[i], 0ull, dskey);
    if (old == 0 || old == dskey) break;
    i = (i + 1) & d.ds_mask;
  }
  if (probes > d.ds_mask) { atomicAdd(&d.counters->device_check, 1ull); return; }
  const unsigned long long key = ((unsigned long long)(i + 1u) << 32) | (uint32_t)(int32_t)ext;
  uint32_t j = hash32((i + 1u) * 0x85EBCA6Bu ^ (uint32_t)(int32_t)ext) & d.span_mask;
  for (probes = 0; probes <= d.span_mask; probes++) {
    unsigned long long old = d.span_key[j];
    if (old == 0) old = atomicCAS(&d.span_key[j], 0ull, key);
    if (old == 0 || old == key) break;
    j = (j + 1) & d.span_mask;
  }
  if (probes > d.span_mask) { atomicAdd(&d.counters->device_check, 1ull); return; }
  // min start / first event are kept as max of the complement so that zero-filled memory is "unset"
  atomicMax(&d.span_nstart[j], ~(unsigned long long)ts);
  atomicMax(&d.span_end[j], (unsigned long long)(ts + dur));
  atomicMax(&d.span_nfirst[j], ~(unsigned long long)ev);
  d.span_row[j] = row;
}

struct Tally { uint32_t x, flow; unsigned long long name_bytes; uint64_t ev; };

// Shared tail of an "X" event after the name: pid, tid, ts, dur and the opening of args.
template <class S> __device__ __forceinline__ void x_mid(S& s, int64_t pid, int64_t tid, int64_t ts_rel, int64_t dur) {
  K2J_LIT(s, "\",\n    \"pid\": "); put_i64(s, pid);
  K2J_LIT(s, ",\n    \"tid\": "); put_i64(s, tid);
  K2J_LIT(s, ",\n    \"ts\": "); put_ts(s, ts_rel);
  K2J_LIT(s, ",\n    \"dur\": "); put_ts(s, dur);
  K2J_LIT(s, "\n    ");
}
template <class S> __device__ __forceinline__ void flow_event(S& s, bool start, bool fwdbwd, uint64_t id, int64_t pid, int64_t tid, int64_t ts_rel) {
  if (start) K2J_LIT(s, "\n  {\n    \"ph\": \"s\",\n    \"id\": "); else K2J_LIT(s, "\n  {\n    \"ph\": \"f\",\n    \"id\": ");
  put_u64(s, id);
  K2J_LIT(s, ",\n    \"pid\": "); put_i64(s, pid);
  K2J_LIT(s, ",\n    \"tid\": "); put_i64(s, tid);
  K2J_LIT(s, ",\n    \"ts\": "); put_ts(s, ts_rel);
  if (fwdbwd) K2J_LIT(s, ",\n    \"cat\": \"fwdbwd\",\n    \"name\": \"fwdbwd\"\n    ");
  else K2J_LIT(s, ",\n    \"cat\": \"ac2g\",\n    \"name\": \"ac2g\"\n    ");
  if (!start) K2J_LIT(s, ", \"bp\": \"e\"");
  K2J_LIT(s, "\n  },");
}
template <class S> __device__ __forceinline__ void args_open_ext(S& s, bool has_ext, int32_t ext) {
  K2J_LIT(s, ",\n    \"args\": {\n      ");
  if (has_ext) { K2J_LIT(s, "\"External id\": "); put_i64(s, ext); put_char(s, ','); }
}
template <class S> __device__ __forceinline__ void graph_channel(S& s, uint32_t graph, uint64_t node, uint32_t ch, uint32_t cht) {
  K2J_LIT(s, ", \"graph id\": "); put_u64(s, graph);
  K2J_LIT(s, ", \"graph node id\": "); put_u64(s, node);
  K2J_LIT(s, ", \"channel\": "); put_u64(s, ch);
  K2J_LIT(s, ", \"channel_type\": "); put_u64(s, cht);
}
template <class S> __device__ __forceinline__ void bandwidth(S& s, uint64_t bytes, int64_t dur) {
  if (dur == 0) return;  // addBandwidthTypedMetadata, CuptiActivity.h:460-470
  K2J_LIT(s, ", \"memory bandwidth (GB/s)\": ");
  put_double_value(s, __ddiv_rn(__ull2double_rn(bytes), __ll2double_rn(dur)));
}

__device__ __forceinline__ bool out_of_range(const Dev& d, int64_t ts, int64_t dur) {
  return ts < d.win_start || (ts + dur) > d.win_end;
}

// ---- runtime / driver API record (handleRuntimeActivity / handleDriverActivity) ----
template <class S> __device__ __forceinline__ bool ev_api(S& s, const Dev& d, const uint8_t* r, Tally& t, uint32_t* filt) {
  // 40-byte records are only 8-byte aligned: 64-bit loads
  const uint2 a = *reinterpret_cast<const uint2*>(r);        // kind, cbid
  const uint64_t st = *reinterpret_cast<const uint64_t*>(r + 8), en = *reinterpret_cast<const uint64_t*>(r + 16);
  const uint2 b = *reinterpret_cast<const uint2*>(r + 24);   // processId, threadId
  const uint32_t corr = *reinterpret_cast<const uint32_t*>(r + 32);
  const bool driver = a.x == K_DRIVER;
  const uint32_t cbid = a.y;
  bool flow_start;
  if (!driver) {
    // CuptiCbidRegistry.cpp:127-161 blocklist; :57-122 flow-starting callbacks
    if (cbid == 17u || cbid == 16u || cbid == 10u || cbid == 133u || cbid == 134u || cbid == 136u) { *filt = 1; return false; }
    flow_start = cbid == 211u || cbid == 269u || cbid == 272u || cbid == 430u || cbid == 311u || cbid == 131u ||
                 cbid == 165u || cbid == 147u || (cbid >= 31u && cbid <= 52u);
  } else {
    // CuptiCbidRegistry.cpp:166-207: only these driver callbacks are tracked
    if (!(cbid == 307u || cbid == 652u || (cbid >= 549u && cbid <= 552u) || cbid == 554u || cbid == 555u)) return false;
    flow_start = cbid == 307u || cbid == 652u;
  }
  const int64_t ts = conv_ts(d, st), dur = conv_dur(d, st, en);
  if (out_of_range(d, ts, dur)) { *filt = 2; return false; }
  int32_t tid = (int32_t)b.y;
  {  // resourceInfo_.find({processId(), tid}), CuptiActivityProfiler.cpp:315-319
    const uint32_t idx = tab_find(d.tid_tab, d.tid_mask, (uint32_t)tid);
    if (idx != 0xFFFFFFFFu) tid = idx < d.n_tid_pairs ? d.tid_pairs[2 * idx + 1] : (int32_t)d.op_resource[idx - d.n_tid_pairs];
  }
  int32_t ext = 0;
  const bool has_ext = linked_op(d, corr, &ext) && ext != 0;
  if (driver) K2J_LIT(s, "\n  {\n    \"ph\": \"X\",\n    \"cat\": \"cuda_driver\",\n    \"name\": \"");
  else K2J_LIT(s, "\n  {\n    \"ph\": \"X\",\n    \"cat\": \"cuda_runtime\",\n    \"name\": \"");
  const uint32_t ntab = driver ? d.n_dr : d.n_rt;
  if (cbid < ntab) put_name(s, d, (driver ? d.dr_names : d.rt_names)[cbid], &t.name_bytes);
  else K2J_LIT(s, "INVALID");
  const int64_t tid_out = abs_tid(tid), ts_rel = rel_ts(d, ts);
  x_mid(s, d.pid, tid_out, ts_rel, dur < 0 ? 0 : dur);
  args_open_ext(s, has_ext, ext);
  K2J_LIT(s, "\"cbid\": "); put_u64(s, cbid);
  K2J_LIT(s, ", \"correlation\": "); put_u64(s, corr);
  K2J_LIT(s, "\n    }\n  },");
  t.x++;
  if (corr > 0) { flow_event(s, flow_start, false, corr, d.pid, tid_out, ts_rel); t.flow++; }
  return true;
}

// ---- kernel record (GpuActivity<Kernel>, CuptiActivity.h:499-576) ----
template <class S> __device__ __forceinline__ bool ev_kernel(S& s, const Dev& d, const uint8_t* r, Tally& t, uint32_t* filt) {
  const uint64_t st = *reinterpret_cast<const uint64_t*>(r + 16), en = *reinterpret_cast<const uint64_t*>(r + 24);
  const int64_t ts = conv_ts(d, st), dur = conv_dur(d, st, en);
  if (out_of_range(d, ts, dur)) { *filt = 2; return false; }
  const uint32_t dev = *reinterpret_cast<const uint32_t*>(r + 40), ctx = *reinterpret_cast<const uint32_t*>(r + 44);
  const uint32_t stream = *reinterpret_cast<const uint32_t*>(r + 48), corr = *reinterpret_cast<const uint32_t*>(r + 92);
  const int32_t gx = *reinterpret_cast<const int32_t*>(r + 52), gy = *reinterpret_cast<const int32_t*>(r + 56), gz = *reinterpret_cast<const int32_t*>(r + 60);
  const int32_t bx = *reinterpret_cast<const int32_t*>(r + 64), by = *reinterpret_cast<const int32_t*>(r + 68), bz = *reinterpret_cast<const int32_t*>(r + 72);
  const int32_t ssm = *reinterpret_cast<const int32_t*>(r + 76), dsm = *reinterpret_cast<const int32_t*>(r + 80);
  const uint32_t regs = *reinterpret_cast<const uint16_t*>(r + 6);
  const uint32_t name_id = (uint32_t)*reinterpret_cast<const uint64_t*>(r + 104);
  int32_t ext = 0;
  const bool has_ext = linked_op(d, corr, &ext) && ext != 0;

  // blocksPerSm / warpsPerSm / computeOccupancyMetrics (DeviceProperties.cpp:161-222): 32-bit wrapping
  // products, single-precision arithmetic without contraction.
  const int32_t grid_prod = (int32_t)((uint32_t)gx * (uint32_t)gy * (uint32_t)gz);
  const int32_t block_prod = (int32_t)((uint32_t)bx * (uint32_t)by * (uint32_t)bz);
  const bool have_dev = dev < (uint32_t)d.n_devices;
  const int sm_count = have_dev ? d.props[dev].num_sms : 0;
  const float bps = sm_count == 0 ? __int_as_float(0x7f800000) : __fdiv_rn(__int2float_rn(grid_prod), __int2float_rn(sm_count));
  const float wps = __fdiv_rn(__fmul_rn(bps, __int2float_rn(block_prod)), 32.0f);
  cudaOccResult occ;
  occ.activeBlocksPerMultiprocessor = 0; occ.limitingFactors = 0; occ.blockLimitRegs = 0; occ.blockLimitWarps = 0;
  occ.blockLimitSharedMem = 0; occ.blockLimitBlocks = 0; occ.blockLimitBarriers = 0; occ.allocatedRegistersPerBlock = 0;
  occ.allocatedSharedMemPerBlock = 0; occ.partitionedGCConfig = PARTITIONED_GC_OFF;
  float occupancy = -1.0f;  // OccupancyMetrics default (DeviceProperties.h:54)
  if (have_dev) {
    const DevProps& dp = d.props[dev];
    const float blocks_per_sm = sm_count != 0 ? __fdiv_rn(__int2float_rn(grid_prod), __int2float_rn(sm_count)) : -1.0f;
    cudaOccFuncAttributes fa;
    fa.maxThreadsPerBlock = INT_MAX; fa.numRegs = (int)regs; fa.sharedSizeBytes = (size_t)(int64_t)ssm;
    fa.partitionedGCConfig = PARTITIONED_GC_OFF; fa.shmemLimitConfig = FUNC_SHMEM_LIMIT_DEFAULT;
    fa.maxDynamicSharedSizeBytes = 0; fa.numBlockBarriers = 0;
    cudaOccDeviceState state;
    cudaOccDeviceProp prop;
    prop.computeMajor = dp.major; prop.computeMinor = dp.minor; prop.maxThreadsPerBlock = dp.max_threads_per_block;
    prop.maxThreadsPerMultiprocessor = dp.max_threads_per_sm; prop.regsPerBlock = dp.regs_per_block;
    prop.regsPerMultiprocessor = dp.regs_per_sm; prop.warpSize = dp.warp_size; prop.sharedMemPerBlock = dp.smem_per_block;
    prop.sharedMemPerMultiprocessor = dp.smem_per_sm; prop.numSms = dp.num_sms;
    prop.sharedMemPerBlockOptin = dp.smem_per_block_optin; prop.reservedSharedMemPerBlock = dp.reserved_smem_per_block;
    const cudaOccError status = cudaOccMaxActiveBlocksPerMultiprocessor(&occ, &prop, &fa, &state, block_prod, (size_t)(int64_t)dsm);
    if (status == CUDA_OCC_SUCCESS) {
      const float eff = fminf(__int2float_rn(occ.activeBlocksPerMultiprocessor), blocks_per_sm);
      occupancy = __fdiv_rn(__fmul_rn(eff, __int2float_rn(block_prod)), __int2float_rn(dp.max_threads_per_sm));
    }
  }
  const long long occ_pct = llround(__dmul_rn((double)occupancy, 100.0));

  K2J_LIT(s, "\n  {\n    \"ph\": \"X\",\n    \"cat\": \"kernel\",\n    \"name\": \"");
  put_name(s, d, name_id, &t.name_bytes);
  const int64_t ts_rel = rel_ts(d, ts);
  x_mid(s, (int64_t)dev, (int64_t)stream, ts_rel, dur < 0 ? 0 : dur);
  args_open_ext(s, has_ext, ext);
  K2J_LIT(s, "\"queued\": "); put_u64(s, *reinterpret_cast<const uint64_t*>(r + 120));
  K2J_LIT(s, ", \"device\": "); put_u64(s, dev);
  K2J_LIT(s, ", \"context\": "); put_u64(s, ctx);
  K2J_LIT(s, ", \"stream\": "); put_u64(s, stream);
  K2J_LIT(s, ", \"correlation\": "); put_u64(s, corr);
  K2J_LIT(s, ", \"registers per thread\": "); put_u64(s, regs);
  K2J_LIT(s, ", \"shared memory\": "); put_i64(s, (int64_t)(int32_t)((uint32_t)ssm + (uint32_t)dsm));
  K2J_LIT(s, ", \"blocks per SM\": "); put_double_value(s, (double)bps);
  K2J_LIT(s, ", \"warps per SM\": "); put_double_value(s, (double)wps);
  K2J_LIT(s, ", \"grid\": ["); put_i64(s, gx); K2J_LIT(s, ", "); put_i64(s, gy); K2J_LIT(s, ", "); put_i64(s, gz);
  K2J_LIT(s, "], \"block\": ["); put_i64(s, bx); K2J_LIT(s, ", "); put_i64(s, by); K2J_LIT(s, ", "); put_i64(s, bz);
  K2J_LIT(s, "], \"est. achieved occupancy %\": "); put_i64(s, occ_pct);
  K2J_LIT(s, ", \"occupancy\": {\"activeBlocksPerMultiprocessor\": "); put_i64(s, occ.activeBlocksPerMultiprocessor);
  K2J_LIT(s, ", \"limitingFactors\": \"");
  {  // limitingFactorsToString, CuptiActivity.h:476-497
    const unsigned f = occ.limitingFactors;
    if (f == 0) K2J_LIT(s, "none");
    else {
      bool first = true;
      if (f & OCC_LIMIT_WARPS) { K2J_LIT(s, "WARPS"); first = false; }
      if (f & OCC_LIMIT_REGISTERS) { if (!first) put_char(s, '|'); K2J_LIT(s, "REGS"); first = false; }
      if (f & OCC_LIMIT_SHARED_MEMORY) { if (!first) put_char(s, '|'); K2J_LIT(s, "SMEM"); first = false; }
      if (f & OCC_LIMIT_BLOCKS) { if (!first) put_char(s, '|'); K2J_LIT(s, "BLOCKS"); first = false; }
      if (f & OCC_LIMIT_BARRIERS) { if (!first) put_char(s, '|'); K2J_LIT(s, "BARRIERS"); first = false; }
    }
  }
  K2J_LIT(s, "\", \"blockLimitRegs\": "); put_i64(s, occ.blockLimitRegs);
  K2J_LIT(s, ", \"blockLimitSharedMem\": "); put_i64(s, occ.blockLimitSharedMem);
  K2J_LIT(s, ", \"blockLimitWarps\": "); put_i64(s, occ.blockLimitWarps);
  K2J_LIT(s, ", \"blockLimitBlocks\": "); put_i64(s, occ.blockLimitBlocks);
  K2J_LIT(s, ", \"blockLimitBarriers\": "); put_i64(s, occ.blockLimitBarriers);
  K2J_LIT(s, ", \"allocatedRegistersPerBlock\": "); put_i64(s, occ.allocatedRegistersPerBlock);
  K2J_LIT(s, ", \"allocatedSharedMemPerBlock\": "); put_u64(s, (uint64_t)occ.allocatedSharedMemPerBlock);
  put_char(s, '}');
  graph_channel(s, *reinterpret_cast<const uint32_t*>(r + 156), *reinterpret_cast<const uint64_t*>(r + 144),
                *reinterpret_cast<const uint32_t*>(r + 168), *reinterpret_cast<const uint32_t*>(r + 172));
  K2J_LIT(s, "\n    }\n  },");
  t.x++;
  if (corr > 0) { flow_event(s, false, false, corr, (int64_t)dev, (int64_t)stream, ts_rel); t.flow++; }
  if (S::kCounting) span_update(d, corr, dev, stream, ts, dur, t.ev);
  return true;
}

template <class S> __device__ __forceinline__ void memcpy_name(S& s, uint32_t kind, uint32_t src, uint32_t dst) {
  K2J_LIT(s, "Memcpy "); put_cstr(s, kMemcpyKind[kind <= 10 ? kind : 11]);
  K2J_LIT(s, " ("); put_cstr(s, kMemoryKind[src <= 7 ? src : 8]);
  K2J_LIT(s, " -> "); put_cstr(s, kMemoryKind[dst <= 7 ? dst : 8]);
  put_char(s, ')');
}

// ---- memcpy / memcpy2 / memset records (CuptiActivity.h:604-712) ----
template <class S, int CLS> __device__ __forceinline__ bool ev_mem(S& s, const Dev& d, const uint8_t* r, Tally& t, uint32_t* filt) {
  const uint64_t st = *reinterpret_cast<const uint64_t*>(r + 16), en = *reinterpret_cast<const uint64_t*>(r + 24);
  const int64_t ts = conv_ts(d, st), dur = conv_dur(d, st, en);
  if (out_of_range(d, ts, dur)) { *filt = 2; return false; }
  const uint64_t bytes = *reinterpret_cast<const uint64_t*>(r + 8);
  const uint32_t dev = *reinterpret_cast<const uint32_t*>(r + 32), ctx = *reinterpret_cast<const uint32_t*>(r + 36);
  const uint32_t stream = *reinterpret_cast<const uint32_t*>(r + 40);
  const uint32_t corr = *reinterpret_cast<const uint32_t*>(r + (CLS == C_MEMCPY2 ? 60 : 44));
  int32_t ext = 0;
  const bool has_ext = linked_op(d, corr, &ext) && ext != 0;
  if (CLS == C_MEMSET) {
    K2J_LIT(s, "\n  {\n    \"ph\": \"X\",\n    \"cat\": \"gpu_memset\",\n    \"name\": \"Memset (");
    const uint32_t mk = *reinterpret_cast<const uint16_t*>(r + 50);
    put_cstr(s, kMemoryKind[mk <= 7 ? mk : 8]);
    put_char(s, ')');
  } else {
    K2J_LIT(s, "\n  {\n    \"ph\": \"X\",\n    \"cat\": \"gpu_memcpy\",\n    \"name\": \"");
    memcpy_name(s, r[4], r[5], r[6]);
  }
  const int64_t ts_rel = rel_ts(d, ts);
  x_mid(s, (int64_t)dev, (int64_t)stream, ts_rel, dur < 0 ? 0 : dur);
  args_open_ext(s, has_ext, ext);
  if (CLS == C_MEMCPY2) {
    K2J_LIT(s, "\"fromDevice\": "); put_u64(s, *reinterpret_cast<const uint32_t*>(r + 44));
    K2J_LIT(s, ", \"inDevice\": "); put_u64(s, dev);
    K2J_LIT(s, ", \"toDevice\": "); put_u64(s, *reinterpret_cast<const uint32_t*>(r + 52));
    K2J_LIT(s, ", \"fromContext\": "); put_u64(s, *reinterpret_cast<const uint32_t*>(r + 48));
    K2J_LIT(s, ", \"inContext\": "); put_u64(s, ctx);
    K2J_LIT(s, ", \"toContext\": "); put_u64(s, *reinterpret_cast<const uint32_t*>(r + 56));
  } else {
    K2J_LIT(s, "\"device\": "); put_u64(s, dev);
    K2J_LIT(s, ", \"context\": "); put_u64(s, ctx);
  }
  K2J_LIT(s, ", \"stream\": "); put_u64(s, stream);
  K2J_LIT(s, ", \"correlation\": "); put_u64(s, corr);
  K2J_LIT(s, ", \"bytes\": "); put_u64(s, bytes);
  bandwidth(s, bytes, dur);
  constexpr int g = CLS == C_MEMCPY2 ? 8 : 0;
  graph_channel(s, *reinterpret_cast<const uint32_t*>(r + 72 + g), *reinterpret_cast<const uint64_t*>(r + 64 + g),
                *reinterpret_cast<const uint32_t*>(r + 76 + g), *reinterpret_cast<const uint32_t*>(r + 80 + g));
  K2J_LIT(s, "\n    }\n  },");
  t.x++;
  if (corr > 0) { flow_event(s, false, false, corr, (int64_t)dev, (int64_t)stream, ts_rel); t.flow++; }
  if (S::kCounting) span_update(d, corr, dev, stream, ts, dur, t.ev);
  return true;
}

// ---- CPU-side activity (ChromeTraceLogger::handleActivity for a GenericTraceActivity) ----
template <class S> __device__ __forceinline__ bool ev_op(S& s, const Dev& d, uint64_t i, Tally& t) {
  const int32_t type = d.op_type[i];
  if ((uint32_t)type >= 29u) { atomicAdd(&d.counters->device_check, 1ull); return false; }
  if (!((d.type_mask >> type) & 1u)) return false;  // type not selected: joins, but is not logged
  if (type == 9 || type == 17 || type == 26 || type == 28) {  // instant / counter events: not implemented
    atomicAdd(&d.counters->device_check, 1ull);
    return false;
  }
  int64_t ts = d.op_start[i];
  int64_t dur = d.op_end[i] - ts;
  if (dur < 0) dur = 0;
  const int64_t flow_ts = ts;
  if (type == 2) { ts -= 1; dur += 2; }  // GPU_USER_ANNOTATION, output_json.cpp:862-869
  // External id, output_json.cpp:871-895: no linked activity on this path; excluded types print none.
  int32_t ext = 0;
  const bool excluded = type == 3 || type == 4 || type == 5 || type == 7 || type == 8 || type == 21 || type == 22 || type == 24 || type == 25;
  if (!excluded) ext = d.op_id[i];
  const uint32_t m0 = d.op_mdoff[i], m1 = d.op_mdoff[i + 1];
  K2J_LIT(s, "\n  {\n    \"ph\": \"X\",\n    \"cat\": \"");
  put_cstr(s, kTypeNames[type]);
  K2J_LIT(s, "\",\n    \"name\": \"");
  put_name(s, d, d.op_name[i], &t.name_bytes);
  const int64_t pid = op_pid(d, d.op_device[i]), tid = abs_tid(d.op_resource[i]);
  x_mid(s, pid, tid, rel_ts(d, ts), dur);
  if (ext != 0 || m1 > m0) {
    K2J_LIT(s, ",\n    \"args\": {\n      ");
    if (ext != 0) { K2J_LIT(s, "\"External id\": "); put_i64(s, ext); if (m1 > m0) put_char(s, ','); }
    for (uint32_t e = m0; e < m1; e++) {  // JsonTypedMetadataVisitor, TypedMetadataJson.h:72-158
      const MdEntry md = d.md[e];
      if (e > m0) K2J_LIT(s, ", ");
      put_char(s, '"'); put_mdstr(s, d, md.key); K2J_LIT(s, "\": ");
      switch (md.type) {
        case 0: put_i64(s, (int64_t)md.value); break;
        case 1: put_u64(s, md.value); break;
        case 2: put_double_value(s, __longlong_as_double((long long)md.value)); break;
        case 3: if (md.value) K2J_LIT(s, "true"); else K2J_LIT(s, "false"); break;
        case 4: put_char(s, '"'); put_mdstr(s, d, (uint32_t)md.value); put_char(s, '"'); break;
        default: put_mdstr(s, d, (uint32_t)md.value); break;
      }
    }
    K2J_LIT(s, "\n    }");
  }
  K2J_LIT(s, "\n  },");
  t.x++;
  const uint32_t fid = d.op_flow[i];
  const uint32_t ft = d.op_flowt[i] & 0xfu;
  if (fid > 0 && (ft == 1u || ft == 2u)) {  // handleGenericLink, output_json.cpp:973-995
    flow_event(s, (d.op_flowt[i] >> 4) & 1u, ft == 1u, fid, pid, tid, rel_ts(d, flow_ts));
    t.flow++;
  }
  return true;
}

constexpr int kEventThreads = 128;

// One thread per work item.  Work items are class-sorted (each class padded to a multiple of 32),
// so a warp formats events of one shape.  WRITE = false: store the byte length; WRITE = true: write
// the bytes at ev_off[event].
template <bool WRITE>
__global__ void __launch_bounds__(kEventThreads) k_events(Dev d) {
  __shared__ uint32_t s_stage[kEventThreads * 4];
  __shared__ unsigned long long s_cnt[8];
  if (threadIdx.x < 8) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  const uint64_t i = (uint64_t)blockIdx.x * kEventThreads + threadIdx.x;
  Tally t; t.x = 0; t.flow = 0; t.name_bytes = 0; t.ev = 0;
  uint32_t filt = 0;
  if (i < d.n_work) {
    int cls;
    uint64_t j;
    if (i >= d.ops_begin) { cls = C_OP; j = i - d.ops_begin; }
    else {
      cls = 0;
#pragma unroll
      for (int c = 1; c < C_EXT; c++) if (i >= d.cls_begin[c]) cls = c;
      j = i - d.cls_begin[cls];
      if (j >= d.cls_count[cls]) cls = -1;  // padding
    }
    if (cls == C_OP && j >= d.n_ops) cls = -1;
    if (cls >= 0) {
      const uint64_t ev = cls == C_OP ? j : d.work_ev[i];
      t.ev = ev;
      const uint8_t* r = cls == C_OP ? nullptr : d.cupti + (uint64_t)d.work_slot[i] * 8;
      if (!WRITE) {
        CountSink s;
        switch (cls) {
          case C_API: ev_api(s, d, r, t, &filt); break;
          case C_KERNEL: ev_kernel(s, d, r, t, &filt); break;
          case C_MEMCPY: ev_mem<CountSink, C_MEMCPY>(s, d, r, t, &filt); break;
          case C_MEMCPY2: ev_mem<CountSink, C_MEMCPY2>(s, d, r, t, &filt); break;
          case C_MEMSET: ev_mem<CountSink, C_MEMSET>(s, d, r, t, &filt); break;
          default: ev_op(s, d, j, t); break;
        }
        d.ev_size[ev] = filt ? 0u : s.n;
      } else {
        const uint32_t size = d.ev_size[ev];
        if (size) {
          const uint64_t off = d.ev_off[ev];
          if (off + size > d.out_cap) { atomicAdd(&d.counters->device_check, 1ull); }
          else {
            GlobalSink s;
            s.init(d.out + off, &s_stage[(threadIdx.x >> 5) * 128 + (threadIdx.x & 31)]);
            switch (cls) {
              case C_API: ev_api(s, d, r, t, &filt); break;
              case C_KERNEL: ev_kernel(s, d, r, t, &filt); break;
              case C_MEMCPY: ev_mem<GlobalSink, C_MEMCPY>(s, d, r, t, &filt); break;
              case C_MEMCPY2: ev_mem<GlobalSink, C_MEMCPY2>(s, d, r, t, &filt); break;
              case C_MEMSET: ev_mem<GlobalSink, C_MEMSET>(s, d, r, t, &filt); break;
              default: ev_op(s, d, j, t); break;
            }
            s.finish();
          }
        }
      }
    }
  }
  if (!WRITE) {  // counters are tallied once, in the size pass
    if (t.x) atomicAdd(&s_cnt[0], (unsigned long long)t.x);
    if (t.flow) atomicAdd(&s_cnt[1], (unsigned long long)t.flow);
    if (filt == 2) atomicAdd(&s_cnt[2], 1ull);
    if (filt == 1) atomicAdd(&s_cnt[3], 1ull);
    if (t.name_bytes) atomicAdd(&s_cnt[4], t.name_bytes);
    __syncthreads();
    if (threadIdx.x == 0) {
      if (s_cnt[0]) atomicAdd(&d.counters->x_events, s_cnt[0]);
      if (s_cnt[1]) atomicAdd(&d.counters->flow_events, s_cnt[1]);
      if (s_cnt[2]) atomicAdd(&d.counters->out_of_range, s_cnt[2]);
      if (s_cnt[3]) atomicAdd(&d.counters->blocklisted_runtime, s_cnt[3]);
      if (s_cnt[4]) atomicAdd(&d.counters->name_bytes, s_cnt[4]);
    }
  }
}

// ---- user-annotation spans: collect, then format in the order the host determined ----
__global__ void k_span_collect(Dev d, SpanRec* out, unsigned int* n_out) {
  const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j > d.span_mask) return;
  const unsigned long long key = d.span_key[j];
  if (key == 0) return;
  const unsigned long long ds = d.ds_tab[(uint32_t)(key >> 32) - 1u] - 1ull;
  SpanRec r;
  r.start = (int64_t)~d.span_nstart[j];
  r.end = (int64_t)d.span_end[j];
  r.first_event = ~d.span_nfirst[j];
  r.device = (uint32_t)(ds >> 32); r.stream = (uint32_t)ds;
  r.op_id = (int32_t)(uint32_t)key; r.op_row = d.span_row[j];
  out[atomicAdd(n_out, 1u)] = r;
}

// One thread per span, in emission order: the gpu_user_annotation event that
// GpuUserEventMap::logEvents hands to the logger (GenericActivityProfiler.cpp:277-290, :320-327;
// output_json.cpp:862-895: starts 1 ns earlier, lasts 2 ns longer, "External id" is the op's id).
template <bool WRITE>
__global__ void __launch_bounds__(kEventThreads) k_annotations(Dev d, const SpanRec* spans, uint32_t n, uint32_t* sizes,
                                                               const uint64_t* offs, uint64_t out_base) {
  __shared__ uint32_t s_stage[kEventThreads * 4];
  const uint32_t i = blockIdx.x * kEventThreads + threadIdx.x;
  if (i >= n) return;
  const SpanRec r = spans[i];
  int64_t dur = r.end - r.start;
  if (dur < 0) dur = 0;
  unsigned long long nb = 0;
  auto body = [&](auto& s) {
    K2J_LIT(s, "\n  {\n    \"ph\": \"X\",\n    \"cat\": \"gpu_user_annotation\",\n    \"name\": \"");
    if (r.op_row < d.n_ops) put_name(s, d, d.op_name[r.op_row], &nb);
    x_mid(s, (int64_t)r.device, (int64_t)r.stream, rel_ts(d, r.start - 1), dur + 2);
    if (r.op_id != 0) { K2J_LIT(s, ",\n    \"args\": {\n      \"External id\": "); put_i64(s, r.op_id); K2J_LIT(s, "\n    }"); }
    K2J_LIT(s, "\n  },");
  };
  if (!WRITE) { CountSink s; body(s); sizes[i] = s.n; }
  else {
    GlobalSink s;
    s.init(d.out + out_base + offs[i], &s_stage[(threadIdx.x >> 5) * 128 + (threadIdx.x & 31)]);
    body(s);
    s.finish();
  }
}

}  // namespace k2j
