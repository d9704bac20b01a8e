// Device side of libk2j: record segmentation, join tables, the size pass, the device-wide scan and
// the emit pass.  All kernels are plain streaming integer/byte kernels for sm_100a; the bound is HBM
// bandwidth (there is no dense contraction anywhere on this path).
//
// Data flow (one run):
//   k_escape_pool    per distinct string: JSON-sanitised copies (name flavour, metadata flavour)
//   k_seg_chunks     per 4 KiB chunk of every CUPTI buffer: record length per 8-byte slot, and for
//                    each of the 26 possible entry slots the slot at which a walk leaves the chunk
//                    and the records per class it meets
//   k_seg_compose    per buffer: chains the exit maps -> true entry slot of every chunk -> its counts
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

#include "k2j_cupti_sizes.h"
#include "k2j_format.cuh"
#include "k2j_sink.cuh"

namespace k2j {

// ---- record classes ---------------------------------------------------------------------------
enum : int { C_API = 0, C_KERNEL = 1, C_MEMCPY = 2, C_MEMCPY2 = 3, C_MEMSET = 4, C_OVERHEAD = 5,
             C_SYNC = 6 /* synchronisation records logged where they stand */, C_CUDAEVENT = 7,
             C_WAIT = 8 /* stream-wait-event synchronisation records: logged after everything else */, C_EXT = 9,
             C_EXT_USER = 10 /* slot class only: EXTERNAL_CORRELATION of kind CUSTOM1; counted in C_EXT too */,
             C_NCLASS = 10,
             C_UNEXPECTED = 10 /* column 10 of the count matrix: records of unknown kind */,
             C_USER = 11 /* column 11: CUSTOM1 correlation records */,
             C_EVENTS = 12 /* column 12: records that own an event slot in buffer order (classes C_API .. C_CUDAEVENT) */,
             C_NCOL = 13, C_NPACKED = 12 /* columns a walk counts (8 bits each, three words) */, C_OP = 13 };
enum : uint32_t { K_MEMCPY = 1, K_MEMSET = 2, K_DRIVER = 4, K_RUNTIME = 5, K_KERNEL = 10, K_OVERHEAD = 17, K_MEMCPY2 = 22,
                  K_CUDA_EVENT = 36, K_SYNC = 38, K_EXTCORR = 39 };
constexpr int kChunkSlots = 512;            // 4 KiB of 8-byte slots
constexpr int kMaxEntry = 26;               // longest record is 208 B = 26 slots
constexpr uint8_t kExitTerminate = 254;     // the walk hit a record it cannot size
constexpr uint8_t kEntryNone = 255;         // chunk is unreachable

// Slot code of a record: size/8 in the low five bits, a group number in the high three; 0 = unknown kind.  Eleven
// slot classes share eight groups: classes of one group differ in size, so (group, size) names the class.
constexpr uint32_t kCodeApi = 5u | (0u << 5), kCodeKernel = 26u | (1u << 5), kCodeMemcpy = 11u | (2u << 5),
                   kCodeMemcpy2 = 12u | (3u << 5), kCodeMemset = 11u | (4u << 5), kCodeOverhead = 7u | (5u << 5),
                   kCodeExt = 3u | (6u << 5), kCodeExtUser = 3u | (7u << 5),
                   kCodeSync = 5u | (1u << 5) /* CUpti_ActivitySynchronization, 40 bytes */, kCodeWait = 5u | (2u << 5),
                   kCodeCudaEvent = 7u | (1u << 5) /* CUpti_ActivityCudaEvent2, 56 bytes */;
static_assert(kCodeWait == kCodeSync + 32u && kCodeExtUser == kCodeExt + 32u, "the decode adds one group for these");
__host__ __device__ constexpr uint32_t slot_code(uint32_t kind, uint32_t word1) {
  switch (kind) {
    case K_KERNEL: return kCodeKernel;
    case K_MEMCPY: return kCodeMemcpy;
    case K_MEMCPY2: return kCodeMemcpy2;
    case K_MEMSET: return kCodeMemset;
    case K_RUNTIME: case K_DRIVER: return kCodeApi;
    case K_OVERHEAD: return kCodeOverhead;  // CUpti_ActivityOverhead3, 56 bytes
    case K_EXTCORR: return word1 == 4u ? kCodeExtUser : kCodeExt;  // word1 = externalKind
    case K_SYNC: return word1 == 2u ? kCodeWait : kCodeSync;       // word1 = type; 2 = STREAM_WAIT_EVENT
    case K_CUDA_EVENT: return kCodeCudaEvent;
    default: return 0u;
  }
}
// A kind the path does not format (the reference counts it and goes on, CuptiActivityProfiler.cpp:583-587): the walk
// steps over it by the size of the kind's record in the CUPTI headers.  Its code has no class: group 0, or group 3
// for the one length that group 0 uses already.  0: a kind the headers do not know; it ends the walk of its buffer.
__host__ __device__ constexpr uint32_t skip_code_of_slots(uint32_t n) { return n == 0u ? 0u : (n == (kCodeApi & 31u) ? n | (3u << 5) : n); }
struct SkipCodes { uint8_t c[kCuptiKinds]; };
constexpr SkipCodes make_skip_codes() {
  SkipCodes t{};
  for (int k = 0; k < kCuptiKinds; k++) t.c[k] = slot_code((uint32_t)k, 0u) != 0u ? 0 : (uint8_t)skip_code_of_slots(kCuptiRecordSlots[k]);
  return t;
}
__constant__ SkipCodes g_skip_codes = make_skip_codes();
// Slot class (C_API .. C_EXT_USER) of a slot code; 0xff for codes no record has.
__host__ __device__ constexpr uint32_t code_slot_class(uint32_t code) {
  switch (code) {
    case kCodeApi: return C_API;
    case kCodeKernel: return C_KERNEL;
    case kCodeMemcpy: return C_MEMCPY;
    case kCodeMemcpy2: return C_MEMCPY2;
    case kCodeMemset: return C_MEMSET;
    case kCodeOverhead: return C_OVERHEAD;
    case kCodeSync: return C_SYNC;
    case kCodeCudaEvent: return C_CUDAEVENT;
    case kCodeWait: return C_WAIT;
    case kCodeExt: return C_EXT;
    case kCodeExtUser: return C_EXT_USER;
    default: return 0xffu;
  }
}

struct DevProps {
  int32_t major, minor, max_threads_per_block, max_threads_per_sm, regs_per_block, regs_per_sm, warp_size, num_sms;
  uint64_t smem_per_block, smem_per_block_optin, smem_per_sm, reserved_smem_per_block;
};

struct Counters {
  unsigned long long x_events, flow_events, out_of_range, blocklisted_runtime, invalid_external_correlation,
      unexpected, name_bytes, device_check, n_user, n_coll, guests;
};

struct MdEntry { uint32_t key, type; uint64_t value; };
struct ExtRec { uint64_t external_id; uint32_t correlation_id; uint32_t external_kind; };
struct SpanRec { int64_t start, end; uint64_t first_event; uint32_t device, stream; int32_t op_id; uint32_t op_row; };
struct EvtRec { uint64_t key; uint32_t corr, stream; };  // a CUDA event record: key = context << 32 | event id

struct Dev {
  // scalars
  int64_t base, win_start, win_end;
  int32_t pid, ts_mode, flags, n_devices; uint32_t type_mask;
  int64_t conv_t0; uint64_t conv_t0a, conv_mant; int32_t conv_exp;
  const DevProps* props;
  // strings
  const uint64_t* pool_off; const uint8_t* pool_data; uint32_t n_strings;
  uint32_t* esc_name_len; uint32_t* esc_md_len; uint8_t* esc_name; uint8_t* esc_md;
  uint8_t* str_class;      // per pool string: 0, 1 = "record_param_comms", 2 + k = the k-th collective metadata key
  const uint32_t* has_comms;  // non-zero when a CPU-side activity of this run is named record_param_comms (nullptr: no enrichment)
  const uint32_t* rt_names; uint32_t n_rt; const uint32_t* dr_names; uint32_t n_dr;
  const int32_t* tid_pairs; uint32_t n_tid_pairs; unsigned long long* tid_tab; uint32_t tid_mask;
  // CUPTI bytes and segmentation
  const uint8_t* cupti; uint64_t cupti_bytes;
  const uint64_t* buf_off; const uint64_t* buf_valid; const uint32_t* buf_chunk_base; uint32_t n_buf, n_chunks;
  uint8_t* slot_code;      // per 8-byte slot of the CUPTI bytes
  uint8_t* exit_map;       // n_chunks x 32
  uint32_t* walk_cnt;      // n_chunks x 32 x 3: packed class counts of the walk from each entry slot
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
  // n_ext_all / n_join_ops are index ranges.  With several shards the arrays are what an all-gather of equal-sized
  // rows left: row r (shard r) starts join_pitch bytes after row r - 1, holds join_counts[2 r] records and
  // join_counts[2 r + 1] ids, and index i means entry i % stride of row i / stride (so indices still grow in
  // processing order).  One shard: one row, join_counts == nullptr, every index valid.
  ExtRec* ext_local; const ExtRec* ext_all; uint64_t n_ext_all;
  const int32_t* join_op_ids; uint64_t n_join_ops;  // CPU-op ids the join sees (local or gathered)
  uint32_t ext_stride, ops_stride; uint64_t join_pitch; const uint64_t* join_counts;
  // with rows, this shard's own records and ids are read from its own arrays (ext_local, op_id), never from its row: the
  // rows may then hold, for every OTHER shard, only the records some shard other than their owner can want
  uint32_t own_rank; uint64_t own_n_ext, own_n_ops;
  // CPU-op ids of the other shards as bitmaps of their id ranges (nullptr: as lists, see join_op_ids): row r holds one
  // bit per id from op_bits_meta[2 r] on, op_bits_meta[2 r + 1] bits; the join only asks whether an id exists
  const uint32_t* op_bits; uint64_t op_bits_pitch; const int64_t* op_bits_meta; uint32_t op_bits_world;
  // sharded runs: bit sets (by hash) of the correlation ids this shard's events carry and of the CPU-op ids
  // the matching records name; keys outside them are not inserted.  nullptr: insert everything.
  uint32_t* need_corr; uint32_t need_corr_mask; uint32_t* need_op; uint32_t need_op_mask;
  // join tables: 64-bit entries (key << 32 | value + 1), 0 = empty
  unsigned long long* corr_tab; uint32_t corr_mask;
  // Correlation id 0 has no table entry (an entry's resolved form, key << 32 | linked id, would be the empty-slot
  // marker for it): [0] the winning CUSTOM0 record's position + 1, [1] after k_resolve_corr bit 33 "links to a
  // CPU op", low half that op's id.
  unsigned long long* corr0;
  unsigned long long* user_tab; uint32_t user_mask;
  unsigned long long* op_tab; uint32_t op_mask;
  // user-annotation spans (GpuUserEventMap): (device, stream) set, then (set slot, op id) -> span
  unsigned long long* ds_tab; uint32_t ds_mask;
  unsigned long long* span_key; unsigned long long* span_nstart; unsigned long long* span_end;
  unsigned long long* span_nfirst; uint32_t* span_row; uint32_t span_mask;  // span_key == nullptr: off
  // work lists (class-sorted) and per-event arrays
  uint32_t* work_slot; uint32_t* work_ev; uint64_t cls_begin[C_NCLASS]; uint64_t cls_count[C_NCLASS];
  uint64_t ops_begin; uint64_t n_work;
  uint64_t work_origin;    // first work item of this launch (0, or the first deferred synchronisation record)
  const uint32_t* work_indirect; uint64_t n_indirect;  // this launch handles the listed work items only (nullptr: a range)
  uint32_t* coll_list;     // work items of the kernel events that carry collective metadata, appended by the size pass
  int32_t wait_pass;       // size pass over the deferred synchronisation records only
  uint64_t wait_ev_base;   // event number of the first deferred synchronisation record
  // synchronisation records: context -> first record naming it, CUDA event records sorted by (context, event,
  // correlation id, position), (device, stream) pairs with GPU work in the window, first stream sync of every row
  unsigned long long* ctx_tab; uint32_t ctx_mask;
  const EvtRec* evt; uint32_t n_evt;
  unsigned long long* seen_tab; uint32_t seen_mask;
  unsigned long long* row_key; uint32_t* row_first; uint32_t row_mask;
  uint32_t* corr_zero;     // one bit per correlation-table slot: the entry links to a CPU op whose id is 0
  uint32_t* ev_size; const uint64_t* ev_off; uint64_t n_events;
  int32_t* ev_ext;        // per event: id of the linked CPU op found by the size pass (0 = none)
  uint8_t* out; uint64_t out_cap;  // address of output byte 0 (of the whole text), bytes of the whole text
  // Sharded traces: records in front of guest_front (a slot index) and from guest_back on are other shards' records
  // that only feed this shard's lookups (contexts, CUDA event records, streams with GPU work, first stream syncs):
  // they run through the size pass like any record, print nothing and are not counted.  None: 0 and 0xFFFFFFFF.
  uint32_t guest_front, guest_back;
  // Sharded traces: the last n_guest_ops CPU-side activities are other shards' record_param_comms ops, present only
  // so that kernels they launched find their collective metadata: never logged, not part of the join keys.
  // coll_tab (sharded runs): id -> row of the record_param_comms ops among this shard's rows and the guests.
  uint64_t n_guest_ops; unsigned long long* coll_tab; uint32_t coll_mask;
  uint64_t tile_begin, tile_end;   // this launch writes the events whose text starts in [tile_begin, tile_end): the whole
                                   // text, or one slab of a tiled run (then `out` points outside the slab for other bytes)
  Counters* counters;
};

// Flag bit 2: CPU-side activities with device 0 show under the process id (the pid-0 override of
// GenericActivityProfiler.cpp:263-271 as seen through ActivityTrace::save()).
__device__ __forceinline__ int32_t op_pid(const Dev& d, int32_t device) { return (device == 0 && (d.flags & 4)) ? d.pid : device; }
__device__ __forceinline__ uint64_t esc_name_pos(const Dev& d, uint32_t id) { return ((2 * d.pool_off[id] + 7) & ~7ull) + 16ull * id; }
__device__ __forceinline__ uint64_t esc_md_pos(const Dev& d, uint32_t id) { return ((d.pool_off[id] + 7) & ~7ull) + 8ull * id; }

// Entry i of the gathered EXTERNAL_CORRELATION records / CPU-op ids; false: past the end of its row.
__device__ __forceinline__ bool ext_at(const Dev& d, uint64_t i, ExtRec* out) {
  if (d.join_counts == nullptr) { *out = d.ext_all[i]; return true; }
  const uint32_t r = (uint32_t)(i / d.ext_stride), j = (uint32_t)(i - (uint64_t)r * d.ext_stride);
  if (r == d.own_rank) { if ((uint64_t)j >= d.own_n_ext) return false; *out = d.ext_local[j]; return true; }
  if ((uint64_t)j >= d.join_counts[2 * r]) return false;
  *out = *reinterpret_cast<const ExtRec*>(reinterpret_cast<const uint8_t*>(d.ext_all) + (uint64_t)r * d.join_pitch + (uint64_t)j * sizeof(ExtRec));
  return true;
}
__device__ __forceinline__ bool op_id_at(const Dev& d, uint64_t i, uint32_t* out) {
  if (d.join_counts == nullptr) { *out = (uint32_t)d.join_op_ids[i]; return true; }
  const uint32_t r = (uint32_t)(i / d.ops_stride), j = (uint32_t)(i - (uint64_t)r * d.ops_stride);
  if (r == d.own_rank) { if ((uint64_t)j >= d.own_n_ops) return false; *out = (uint32_t)d.op_id[j]; return true; }
  if ((uint64_t)j >= d.join_counts[2 * r + 1]) return false;
  *out = (uint32_t)*reinterpret_cast<const int32_t*>(reinterpret_cast<const uint8_t*>(d.join_op_ids) + (uint64_t)r * d.join_pitch + (uint64_t)j * 4u);
  return true;
}

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
// Strings the collective enrichment looks for (libkineto/src/output_json.cpp:34-52): the CPU op's name, then the
// metadata keys in the order appendCollectiveArgs (:718-801) reads them.
constexpr int kCollKeys = 16;
__constant__ char g_coll_str[1 + kCollKeys][28] = {
    "record_param_comms", "Collective name", "In msg nelems", "Out msg nelems", "Group size", "dtype", "Input Tensors start",
    "Output Tensors start", "In split size", "Out split size", "Process Group Name", "Process Group Description",
    "Process Group Ranks", "Dst Rank", "Src Rank", "Seq", "Comms Id"};
__constant__ uint8_t g_coll_len[1 + kCollKeys] = {18, 15, 13, 14, 10, 5, 19, 20, 13, 14, 18, 25, 19, 8, 8, 3, 8};
__global__ void k_escape_pool(Dev d) {
  const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (warp >= d.n_strings) return;
  const uint64_t b = d.pool_off[warp], e = d.pool_off[warp + 1];
  const uint32_t len = (uint32_t)(e - b);
  const uint8_t* src = d.pool_data + b;
  uint8_t* dn = d.esc_name + esc_name_pos(d, warp);
  uint8_t* dm = d.esc_md + esc_md_pos(d, warp);
  {  // class of the string for the collective enrichment: a byte-wise match against seventeen short constants
    const uint8_t raw = lane < len ? src[lane] : 0;
    uint32_t cls = 0;
    if (len >= 3 && len <= 25) {
      for (int k = 0; k <= kCollKeys; k++) {
        const bool same = len == g_coll_len[k] && (lane >= len || raw == (uint8_t)g_coll_str[k][lane]);
        if (__all_sync(0xffffffffu, same)) cls = 1u + (uint32_t)k;
      }
    }
    if (lane == 0) d.str_class[warp] = (uint8_t)cls;
  }
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

// Class column of a slot code for the count matrix (C_EXT_USER counts as C_EXT; see C_USER).
__device__ __forceinline__ uint32_t code_class(uint32_t code) {
  const uint32_t cls = code_slot_class(code);
  return cls == (uint32_t)C_EXT_USER ? (uint32_t)C_EXT : cls;
}

// One warp per chunk: slot codes; then lane e (< 26) walks the chunk as if it were entered at slot e
// and leaves behind where that walk exits (the exit map) and how many records of each class it met
// (twelve 8-bit counts packed in three words: a 4 KiB chunk holds at most 170 records).  Kind -> code and
// class -> count increments come from two small tables in shared memory, so neither the decode nor
// the walk branches on the record kind.
__global__ void __launch_bounds__(kSegWarps * 32) k_seg_chunks(Dev d) {
  __shared__ uint8_t s_code[kSegWarps][kChunkSlots];
  __shared__ uint8_t s_kind[64];     // slot code of record kinds 0..63 (CUSTOM1 correlation records add one class)
  __shared__ uint32_t s_inc[256][3]; // per slot code: increments of the three packed count words
  static_assert(kSegWarps * 32 == 256, "one thread per slot code");
  if (threadIdx.x < 64) { const uint32_t c = slot_code(threadIdx.x, 0u); s_kind[threadIdx.x] = (uint8_t)(c != 0u ? c : g_skip_codes.c[threadIdx.x]); }
  {
    const uint32_t sc = code_slot_class(threadIdx.x), cls = sc == (uint32_t)C_EXT_USER ? (uint32_t)C_EXT : sc;
    uint32_t inc[3] = {0u, 0u, 0u};
    if (sc != 0xffu) {
      inc[cls >> 2] = 1u << (8 * (cls & 3u));
      if (sc == (uint32_t)C_EXT_USER) inc[C_USER >> 2] += 1u << (8 * (C_USER & 3));
    } else if ((threadIdx.x & 31u) != 0u) inc[C_UNEXPECTED >> 2] = 1u << (8 * (C_UNEXPECTED & 3));  // a record that is stepped over
    s_inc[threadIdx.x][0] = inc[0]; s_inc[threadIdx.x][1] = inc[1]; s_inc[threadIdx.x][2] = inc[2];
  }
  __syncthreads();
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
      if (s + q < g.nvalid) {
        const uint2 w2 = words[g.slot0 + s + q];
        code = w2.x < 64u ? s_kind[w2.x] : 0u;
        code += (w2.x == K_EXTCORR && w2.y == 4u) ? 1u << 5 : 0u;  // externalKind CUSTOM1: the next group
        code += (w2.x == K_SYNC && w2.y == 2u) ? 1u << 5 : 0u;     // a stream-wait event: the next group
      }
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
  uint32_t c0 = 0, c1 = 0, c2 = 0;  // 8-bit counts of columns 0-3, 4-7, 8-11
  if (lane < kMaxEntry) {
    uint32_t pos = lane;
    code = 0;
    // Bounded: every step advances by at least 3 slots.
    for (int it = 0; it < kChunkSlots; it++) {
      if (pos >= g.nvalid) { code = g.last ? 0 : (uint8_t)(pos - g.nvalid); break; }
      const uint32_t sc = s_code[w][pos];
      const uint32_t n = sc & 31u;
      if (n == 0 || (g.last && pos + n > g.nvalid)) { code = kExitTerminate; c2 += 1u << (8 * (C_UNEXPECTED - 8)); break; }
      const uint32_t* inc = s_inc[sc];
      c0 += inc[0]; c1 += inc[1]; c2 += inc[2];
      pos += n;
    }
  }
  d.exit_map[(uint64_t)chunk * 32 + lane] = code;
  uint32_t* cw = d.walk_cnt + ((uint64_t)chunk * 32 + lane) * 3;
  cw[0] = c0; cw[1] = c1; cw[2] = c2;
}

// One block per buffer: chain the exit maps to the true entry slot of every chunk, then copy the counts
// of the walk that started there into the count matrix.  The chain over a tile of 1024 chunks runs in
// three short phases instead of 1024 dependent steps: (A) for each of 32 segments of 32 chunks and each
// possible entry, where a walk leaves the segment; (B) one thread chains the 32 segment maps;
// (C) one lane per segment walks its 32 chunks from the segment's true entry.
__global__ void __launch_bounds__(256) k_seg_compose(Dev d) {
  constexpr int kTile = 1024, kSeg = 32;
  __shared__ uint8_t s_map[kTile * 32];
  __shared__ uint8_t s_ent[kTile];
  __shared__ uint8_t s_segmap[kTile / kSeg][32];
  __shared__ uint8_t s_segent[kTile / kSeg];
  __shared__ uint32_t s_entry;
  const uint32_t b = blockIdx.x;
  const uint32_t c0 = d.buf_chunk_base[b], c1 = d.buf_chunk_base[b + 1];
  if (threadIdx.x == 0) s_entry = 0;
  auto step = [&](uint32_t e, uint32_t c, uint32_t n) -> uint32_t {  // entry of chunk c+1 given the entry of chunk c
    if (e == kEntryNone || c >= n) return e;
    const uint8_t x = s_map[c * 32 + e];
    return x >= kMaxEntry ? (uint32_t)kEntryNone : (uint32_t)x;
  };
  for (uint32_t t0 = c0; t0 < c1; t0 += kTile) {
    const uint32_t n = min((uint32_t)kTile, c1 - t0);
    __syncthreads();
    const uint4* src = reinterpret_cast<const uint4*>(d.exit_map + (uint64_t)t0 * 32);
    uint4* dst = reinterpret_cast<uint4*>(s_map);
    for (uint32_t i = threadIdx.x; i < n * 2; i += blockDim.x) dst[i] = src[i];
    __syncthreads();
    // (A) 32 segments x 26 entries independent chains of 32 steps
    for (uint32_t q = threadIdx.x; q < (kTile / kSeg) * 32; q += blockDim.x) {
      const uint32_t seg = q >> 5, e0 = q & 31u;
      uint32_t e = e0 < (uint32_t)kMaxEntry ? e0 : (uint32_t)kEntryNone;
      for (uint32_t c = seg * kSeg; c < (seg + 1) * kSeg; c++) e = step(e, c, n);
      s_segmap[seg][e0] = (uint8_t)e;
    }
    __syncthreads();
    // (B) chain the segments
    if (threadIdx.x == 0) {
      uint32_t e = s_entry;
      for (uint32_t seg = 0; seg < kTile / kSeg; seg++) {
        s_segent[seg] = (uint8_t)e;
        if (e != kEntryNone) e = s_segmap[seg][e];
      }
      s_entry = e;
    }
    __syncthreads();
    // (C) entries of the chunks of each segment
    if (threadIdx.x < kTile / kSeg) {
      const uint32_t seg = threadIdx.x;
      uint32_t e = s_segent[seg];
      for (uint32_t c = seg * kSeg; c < (seg + 1) * kSeg; c++) { s_ent[c] = (uint8_t)e; e = step(e, c, n); }
    }
    __syncthreads();
    for (uint32_t c = threadIdx.x; c < n; c += blockDim.x) {
      const uint32_t e = s_ent[c];
      d.chunk_entry[t0 + c] = (uint8_t)e;
      uint32_t w0 = 0, w1 = 0, w2 = 0;
      if (e != kEntryNone) {
        const uint32_t* cw = d.walk_cnt + ((uint64_t)(t0 + c) * 32 + e) * 3;
        w0 = cw[0]; w1 = cw[1]; w2 = cw[2];
      }
#pragma unroll
      for (int i = 0; i < 4; i++) d.chunk_cnt[(uint64_t)i * d.n_chunks + t0 + c] = (w0 >> (8 * i)) & 0xffu;
#pragma unroll
      for (int i = 0; i < 4; i++) d.chunk_cnt[(uint64_t)(4 + i) * d.n_chunks + t0 + c] = (w1 >> (8 * i)) & 0xffu;
#pragma unroll
      for (int i = 0; i < C_NPACKED - 8; i++) d.chunk_cnt[(uint64_t)(8 + i) * d.n_chunks + t0 + c] = (w2 >> (8 * i)) & 0xffu;
      // records that own an event slot in buffer order: classes C_API .. C_CUDAEVENT = the bytes of w0 and w1
      d.chunk_cnt[(uint64_t)C_EVENTS * d.n_chunks + t0 + c] = (((w0 & 0x00ff00ffu) + ((w0 >> 8) & 0x00ff00ffu) +
                                                                 (w1 & 0x00ff00ffu) + ((w1 >> 8) & 0x00ff00ffu)) * 0x00010001u) >> 16;
    }
  }
}

// Copies the chunk's slot codes to shared memory as 32-bit words; the chunk's first code lands at the
// returned byte offset (0..3) of `s`, which holds kChunkSlots + 4 bytes.
__device__ __forceinline__ uint32_t load_codes(const Dev& d, const ChunkGeom& g, uint8_t* s, uint32_t lane) {
  const uint64_t a0 = g.slot0 & ~3ull;
  const uint32_t off = (uint32_t)(g.slot0 & 3ull);
  const uint32_t nwords = (off + g.nvalid + 3u) >> 2;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(d.slot_code + a0);
  for (uint32_t i = lane; i < (uint32_t)(kChunkSlots + 4) / 4; i += 32) reinterpret_cast<uint32_t*>(s)[i] = i < nwords ? src[i] : 0u;
  __syncwarp();
  return off;
}

// One warp per chunk.  Lane 0 walks the chunk from its true entry and notes where records start; the
// warp then ranks the records within their class (32 at a time, by ballot) and writes the per-class
// work lists and the compacted EXTERNAL_CORRELATION records.
__global__ void __launch_bounds__(kSegWarps * 32) k_seg_write(Dev d) {
  __shared__ __align__(4) uint8_t s_code[kSegWarps][kChunkSlots + 4];
  __shared__ uint16_t s_pos[kSegWarps][kChunkSlots / 3 + 2];
  __shared__ uint32_t s_n[kSegWarps];
  __shared__ uint64_t s_base[kSegWarps][C_NCLASS];
  const uint32_t w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t chunk = blockIdx.x * kSegWarps + w;
  if (chunk >= d.n_chunks) return;
  const uint32_t entry = d.chunk_entry[chunk];
  if (entry == kEntryNone) return;
  const ChunkGeom g = chunk_geom(d, chunk);
  const uint8_t* codes = s_code[w] + load_codes(d, g, s_code[w], lane);
  if (lane == 0) {
    uint32_t n = 0, pos = entry;
    for (int it = 0; it < kChunkSlots && pos < g.nvalid; it++) {  // bounded: every step advances by at least 3 slots
      const uint32_t len = codes[pos] & 31u;
      if (len == 0 || (g.last && pos + len > g.nvalid)) break;    // unknown kind or overrun: the walk ends
      s_pos[w][n++] = (uint16_t)pos;
      pos += len;
    }
    s_n[w] = n;
  }
  __syncwarp();
  const uint32_t n = s_n[w];
  // next free position of every class (work list, or the compacted EXTERNAL_CORRELATION array)
  if (lane < (uint32_t)C_NCLASS) s_base[w][lane] = d.chunk_base[(uint64_t)lane * d.n_chunks + chunk] + (lane == (uint32_t)C_EXT ? 0 : d.cls_begin[lane]);
  __syncwarp();
  uint64_t ev_base = d.n_ops + d.chunk_base[(uint64_t)C_EVENTS * d.n_chunks + chunk];
  const uint32_t lt = (1u << lane) - 1u;
  for (uint32_t i0 = 0; i0 < n; i0 += 32) {
    const uint32_t i = i0 + lane;
    const uint32_t pos = i < n ? s_pos[w][i] : 0u;
    const uint32_t cls = i < n ? code_class(codes[pos]) : 0xffu;
    const bool on = cls != 0xffu;  // records of kinds that are only stepped over own nothing
    const uint32_t evm = __ballot_sync(0xffffffffu, on && cls < (uint32_t)C_WAIT);
    // rank within the class: the lanes holding records of one class find each other in one step
    const uint32_t peers = __match_any_sync(0xffffffffu, cls);
    const uint64_t dst = on ? s_base[w][cls] + __popc(peers & lt) : 0;
    __syncwarp();
    if (on && (peers & lt) == 0u) s_base[w][cls] += __popc(peers);
    __syncwarp();
    if (on) {
      const uint64_t slot = g.slot0 + pos;
      if (cls == (uint32_t)C_EXT) {
        const uint8_t* r = d.cupti + slot * 8;
        ExtRec e;
        e.external_kind = *reinterpret_cast<const uint32_t*>(r + 4);
        e.external_id = *reinterpret_cast<const uint64_t*>(r + 8);
        e.correlation_id = *reinterpret_cast<const uint32_t*>(r + 16);
        d.ext_local[dst] = e;
      } else {
        d.work_slot[dst] = (uint32_t)slot;
        // deferred records are numbered after every other event, in the order they stand in the buffers
        d.work_ev[dst] = cls == (uint32_t)C_WAIT ? (uint32_t)(d.wait_ev_base + (dst - d.cls_begin[C_WAIT])) : (uint32_t)(ev_base + __popc(evm & lt));
      }
    }
    ev_base += __popc(evm);
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
    if (j >= d.n_ops - d.n_guest_ops || op_pid(d, d.op_device[j]) != d.pid) return;  // guest rows extend no map
    key = (uint32_t)d.op_thread[j];
  }
  if (!tab_insert_min(d.tid_tab, d.tid_mask, key, (uint32_t)i)) atomicAdd(&d.counters->device_check, 1ull);
}
// A key owns two bits of one 32-bit word (one memory access per test or set): with eight bits of table per
// marked key about one word bit in eight is set and a foreign key passes with probability of about 1 in 60,
// from a table small enough to stay in the L2 while the gathered keys stream past it.
__device__ __forceinline__ uint32_t bit_pair(uint32_t h) { return (1u << (h & 31u)) | (1u << (h >> 27)); }
__device__ __forceinline__ bool bit_test(const uint32_t* bits, uint32_t mask, uint32_t key) {
  const uint32_t h = hash32(key ^ 0x9E3779B9u), m = bit_pair(h);
  return (bits[(h & mask) >> 5] & m) == m;
}
__device__ __forceinline__ void bit_set(uint32_t* bits, uint32_t mask, uint32_t key) {
  const uint32_t h = hash32(key ^ 0x9E3779B9u);
  atomicOr(&bits[(h & mask) >> 5], bit_pair(h));
}
// Sharded runs: marks the correlation id of every GPU-side record of this shard.  With the gathered
// arrays of W shards each rank would otherwise insert W times its own share of keys into its tables,
// although its events can only ever look up their own correlation ids.
__global__ void k_mark_corr(Dev d) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.ops_begin) return;
  int cls = 0;
#pragma unroll
  for (int c = 1; c < C_EXT; c++) if (i >= d.cls_begin[c]) cls = c;
  if (i - d.cls_begin[cls] >= d.cls_count[cls] || cls == C_OVERHEAD) return;  // padding; overhead records join nothing
  const uint8_t* r = d.cupti + (uint64_t)d.work_slot[i] * 8;
  const int off = cls == C_API ? 32 : cls == C_KERNEL ? 92 : cls == C_MEMCPY2 ? 60 : cls == C_CUDAEVENT ? 4 : (cls == C_SYNC || cls == C_WAIT) ? 24 : 44;
  bit_set(d.need_corr, d.need_corr_mask, *reinterpret_cast<const uint32_t*>(r + off));
}
// ---- sending join keys only where they can be wanted ----
// Every shard publishes the filter k_mark_corr fills (the correlation ids its events carry).  k_flag_wanted marks this
// shard's EXTERNAL_CORRELATION records (kinds the join uses) whose correlation id hits the filter of at least one other
// shard - each filter is asked on its own: their union would be so dense with many shards that half of all keys
// passed - and after a scan of the marks k_take_wanted copies them out in their order, which is all that "the last
// record of a correlation id wins" needs: positions only have to grow along a shard's records.
__global__ void k_flag_wanted(Dev d, const uint32_t* filters, uint64_t pitch_words, uint32_t world, uint32_t rank, uint32_t mask, uint64_t n,
                              uint32_t* flags) {
  const uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  const ExtRec e = d.ext_local[j];
  bool wanted = false;
  if (e.external_kind == 3u || e.external_kind == 4u)
    for (uint32_t r = 0; r < world && !wanted; r++)
      if (r != rank) wanted = bit_test(filters + (uint64_t)r * pitch_words, mask, e.correlation_id);
  flags[j] = wanted ? 1u : 0u;
}
__global__ void k_take_wanted(Dev d, const uint32_t* flags, const uint64_t* at, uint64_t n, ExtRec* out) {
  const uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n || flags[j] == 0u) return;
  out[at[j]] = d.ext_local[j];
}
// Is any CPU-side activity of this run named record_param_comms (bit 0: kernel events look at their linked op's
// name only if so), is any an instant event (bit 1)?
__global__ void k_find_comms(Dev d, uint32_t* flag, int comms_on) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.n_ops) return;
  const uint32_t name = d.op_name[i];
  if (comms_on && name < d.n_strings && d.str_class[name] == 1u) atomicOr(flag, 1u);
  const int type = d.op_type[i];
  if (type == 9 || type == 17 || type == 26 || type == 28) atomicOr(flag, 2u);  // instant and counter events: written by the same extra launch
}
// Sharded runs: id -> row of the record_param_comms ops of this shard and of the guest rows (the last row wins).
__global__ void k_build_coll(Dev d) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.n_ops) return;
  const uint32_t name = d.op_name[i];
  if (name >= d.n_strings || d.str_class[name] != 1u) return;
  if (!tab_insert(d.coll_tab, d.coll_mask, (uint32_t)d.op_id[i], (uint32_t)i)) atomicAdd(&d.counters->device_check, 1ull);
}
// CPU-op id -> position (last writer wins): activityMap_[id] = op, GenericActivityProfiler.cpp:262.
__global__ void k_build_ops(Dev d, uint64_t first, uint64_t last) {
  const uint64_t i = first + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  uint32_t id = 0u;
  const bool in = i < last && op_id_at(d, i, &id);
  const bool valid = in && (d.need_op == nullptr || bit_test(d.need_op, d.need_op_mask, id));
  // Ids repeat (every memory event of a PyTorch trace carries id 0): of the lanes of a warp that hold one id only the
  // last, which is the one that must win, goes to the table, so a run of equal ids costs one atomic per warp.
  const uint32_t peers = __match_any_sync(0xffffffffu, id) & __ballot_sync(0xffffffffu, valid);
  if (!valid || (threadIdx.x & 31u) != 31u - (uint32_t)__clz((int)peers)) return;
  if (!tab_insert(d.op_tab, d.op_mask, id, (uint32_t)i)) atomicAdd(&d.counters->device_check, 1ull);
}
// correlation id -> index of the winning EXTERNAL_CORRELATION record (handleCorrelationActivity,
// CuptiActivityProfiler.cpp:290-302).  `count_invalid`: only the shard that owns a record counts it.
__global__ void k_build_corr(Dev d, uint64_t own_begin, uint64_t own_end) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  ExtRec e;
  if (i >= d.n_ext_all || !ext_at(d, i, &e)) return;
  bool ok = true;
  if (e.external_kind == 3u) {
    if (d.need_corr != nullptr) {
      // this shard's own records are nearly all wanted by its own events: they go in untested
      if ((i < own_begin || i >= own_end) && !bit_test(d.need_corr, d.need_corr_mask, e.correlation_id)) return;
      if ((int64_t)e.external_id == (int64_t)(int32_t)e.external_id) bit_set(d.need_op, d.need_op_mask, (uint32_t)e.external_id);
    }
    if (e.correlation_id == 0u) atomicMax(&d.corr0[0], (unsigned long long)i + 1ull);
    else ok = tab_insert(d.corr_tab, d.corr_mask, e.correlation_id, (uint32_t)i);
  } else if (e.external_kind == 4u) {
    atomicAdd(&d.counters->n_user, 1ull);
    // user-annotation spans: the same filter as above when the keys of several shards were gathered
    if (d.user_tab != nullptr &&
        (d.need_corr == nullptr || (i >= own_begin && i < own_end) || bit_test(d.need_corr, d.need_corr_mask, e.correlation_id))) {
      if (d.need_op != nullptr && (int64_t)e.external_id == (int64_t)(int32_t)e.external_id) bit_set(d.need_op, d.need_op_mask, (uint32_t)e.external_id);
      ok = tab_insert(d.user_tab, d.user_mask, e.correlation_id, (uint32_t)i);
    }
  } else if (i >= own_begin && i < own_end) atomicAdd(&d.counters->invalid_external_correlation, 1ull);
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

struct CountSink2 : CountSink {
  __device__ __forceinline__ void put4(uint32_t) { n += 4; }
  __device__ __forceinline__ void put64(uint64_t, uint32_t len) { n += len; }
  __device__ __forceinline__ void words(const uint64_t*, uint32_t len) { n += len; }
  __device__ __forceinline__ void bytes(const uint8_t*, uint32_t len) { n += len; }
  __device__ __forceinline__ void ensure(uint32_t) {}
};

// ---- event programs ------------------------------------------------------------------------------------
// An event is a fixed sequence of fields, each a literal followed by a value.  The sequence of a
// record class is data (a table in constant memory), so all classes share one small formatting loop
// and the lanes of a warp, which format events of one class, run it in lock step.  A field's value
// is read from the thread's area in shared memory: the staged record itself, with the values that
// are computed rather than stored (converted times, the linked op, occupancy ...) written by the
// class's gather step into parts of the record that no field reads.
enum : uint8_t { T_NONE = 0, T_U64, T_I64, T_TS, T_DBL, T_NAME, T_CSTR, T_MD /* the metadata entries of a CPU-side activity */,
                 T_COLL = 11 /* collective metadata copied from the linked record_param_comms op */,
                 T_RAWSTR = 12 /* a pool string as it is */, T_RAWSTRIP /* ... minus one surrounding pair of quotes */,
                 T_MDRAW /* metadata entries with keys and strings as they are */,
                 T_MDCNT /* the counter values of a counter event: "name": value,... */,
                 T_HWC /* one whole counter event per counter value (HARDWARE_COUNTERS) */ };
enum : uint8_t { VK_U32 = 0, VK_I32 /* sign-extended */, VK_64 };
struct FieldSrc { const char* lit; uint8_t type; uint8_t vk; uint16_t voff; };
struct FieldDesc { uint16_t off, len; uint8_t type, vk; uint16_t voff; };

constexpr int c_strlen(const char* s) { int n = 0; while (s[n]) n++; return n; }
template <int NF> constexpr int prog_words(const FieldSrc (&src)[NF]) {  // 64-bit words
  int w = 0;
  for (int f = 0; f < NF; f++) w += (c_strlen(src[f].lit) + 7) / 8;
  return w + 1;  // one spare word: a copy reads one word past the literal
}
template <int NF, int NW> struct Prog {
  FieldDesc f[NF];
  uint64_t w[NW];
};
template <int NF, int NW> constexpr Prog<NF, NW> make_prog(const FieldSrc (&src)[NF]) {
  Prog<NF, NW> p{};
  int pos = 0;
  for (int f = 0; f < NF; f++) {
    const int n = c_strlen(src[f].lit);
    p.f[f].off = (uint16_t)pos; p.f[f].len = (uint16_t)n; p.f[f].type = src[f].type; p.f[f].vk = src[f].vk; p.f[f].voff = src[f].voff;
    for (int i = 0; i < n; i++) p.w[pos + i / 8] |= (uint64_t)(unsigned char)src[f].lit[i] << (8 * (i % 8));
    pos += (n + 7) / 8;
  }
  return p;
}
#define XHEAD(cat) "\n  {\n    \"ph\": \"X\",\n    \"cat\": \"" cat "\",\n    \"name\": \""
#define FLOW_TAIL "\n  },"

// Byte offsets inside a thread's area.  R_: a field of the record as CUPTI wrote it.  S_: a computed
// value, stored over record bytes that nothing reads (or past the record's end).
// -- runtime / driver API record (40 bytes) --
enum : int { AR_CBID = 4, AS_TS = 8, AS_DUR = 16, AS_PID = 24, AS_TID = 28, AR_CORR = 32, AS_EXT = 36, AS_NAME = 40 };
enum : int { A_HEAD_RT, A_HEAD_DR, A_NAME, A_INVALID, A_PID, A_TID, A_TS, A_DUR, A_ARGS, A_EXT, A_EXTC, A_CBID, A_CORR, A_CLOSE,
             A_FLOW_S, A_FLOW_F, A_FPID, A_FTID, A_FTS, A_FCAT, A_FBP, A_FEND, A_COUNT };
#define K2J_API_FIELDS \
    {XHEAD("cuda_runtime"), T_NONE}, {XHEAD("cuda_driver"), T_NONE}, {"", T_NAME, VK_U32, AS_NAME}, {"INVALID", T_NONE}, \
    {"\",\n    \"pid\": ", T_I64, VK_I32, AS_PID}, {",\n    \"tid\": ", T_I64, VK_U32, AS_TID}, {",\n    \"ts\": ", T_TS, VK_64, AS_TS}, \
    {",\n    \"dur\": ", T_TS, VK_64, AS_DUR}, \
    {"\n    ,\n    \"args\": {\n      ", T_NONE}, {"\"External id\": ", T_I64, VK_I32, AS_EXT}, {",", T_NONE}, \
    {"\"cbid\": ", T_U64, VK_U32, AR_CBID}, {", \"correlation\": ", T_U64, VK_U32, AR_CORR}, {"\n    }\n  },", T_NONE}, \
    {"\n  {\n    \"ph\": \"s\",\n    \"id\": ", T_U64, VK_U32, AR_CORR}, {"\n  {\n    \"ph\": \"f\",\n    \"id\": ", T_U64, VK_U32, AR_CORR}, \
    {",\n    \"pid\": ", T_I64, VK_I32, AS_PID}, {",\n    \"tid\": ", T_I64, VK_U32, AS_TID}, {",\n    \"ts\": ", T_TS, VK_64, AS_TS}, \
    {",\n    \"cat\": \"ac2g\",\n    \"name\": \"ac2g\"\n    ", T_NONE}, {", \"bp\": \"e\"", T_NONE}, {FLOW_TAIL, T_NONE}

// -- kernel record (GpuActivity<Kernel>, libkineto/src/CuptiActivity.h:499-576; 208 bytes) --
enum : int { KS_COLLROW = 0 /* row of the linked record_param_comms op */, KS_REGS = 8, KS_SMEM = 12, KS_TS = 16, KS_DUR = 24, KS_BPS = 32, KR_DEV = 40, KR_CTX = 44, KR_STREAM = 48, KR_GRID = 52,
             KR_BLOCK = 64, KS_PCT = 84, KS_ACTIVE = 88, KR_CORR = 92, KS_EXT = 96, KS_LIMIT = 100, KR_NAME = 104, KS_LREGS = 108,
             KS_LSMEM = 112, KS_LWARPS = 116, KR_QUEUED = 120, KS_WPS = 128, KS_LBLOCKS = 136, KS_LBARR = 140, KR_NODE = 144,
             KS_AREGS = 152, KR_GRAPH = 156, KS_ASMEM = 160, KR_CHAN = 168, KR_CHTYPE = 172 };
enum : int { K_HEAD, K_PID, K_TID, K_TS, K_DUR, K_ARGS, K_EXT, K_EXTC, K_QUEUED, K_DEV, K_CTX, K_STREAM, K_CORR, K_REGS, K_SMEM,
             K_BPS, K_WPS, K_GX, K_GY, K_GZ, K_BX, K_BY, K_BZ, K_OCCPCT, K_ACTIVE, K_LIMIT, K_LREGS, K_LSMEM, K_LWARPS, K_LBLOCKS,
             K_LBARR, K_AREGS, K_ASMEM, K_GRAPH, K_NODE, K_CHAN, K_CHTYPE, K_COLL, K_CLOSE, K_FLOW, K_FPID, K_FTID, K_FTS, K_FEND, K_COUNT };
#define K2J_KERNEL_FIELDS \
    {XHEAD("kernel"), T_NAME, VK_U32, KR_NAME}, {"\",\n    \"pid\": ", T_U64, VK_U32, KR_DEV}, {",\n    \"tid\": ", T_U64, VK_U32, KR_STREAM}, \
    {",\n    \"ts\": ", T_TS, VK_64, KS_TS}, {",\n    \"dur\": ", T_TS, VK_64, KS_DUR}, {"\n    ,\n    \"args\": {\n      ", T_NONE}, \
    {"\"External id\": ", T_I64, VK_I32, KS_EXT}, {",", T_NONE}, \
    {"\"queued\": ", T_U64, VK_64, KR_QUEUED}, {", \"device\": ", T_U64, VK_U32, KR_DEV}, {", \"context\": ", T_U64, VK_U32, KR_CTX}, \
    {", \"stream\": ", T_U64, VK_U32, KR_STREAM}, {", \"correlation\": ", T_U64, VK_U32, KR_CORR}, \
    {", \"registers per thread\": ", T_U64, VK_U32, KS_REGS}, {", \"shared memory\": ", T_I64, VK_I32, KS_SMEM}, \
    {", \"blocks per SM\": ", T_DBL, VK_64, KS_BPS}, {", \"warps per SM\": ", T_DBL, VK_64, KS_WPS}, \
    {", \"grid\": [", T_I64, VK_I32, KR_GRID}, {", ", T_I64, VK_I32, KR_GRID + 4}, {", ", T_I64, VK_I32, KR_GRID + 8}, \
    {"], \"block\": [", T_I64, VK_I32, KR_BLOCK}, {", ", T_I64, VK_I32, KR_BLOCK + 4}, {", ", T_I64, VK_I32, KR_BLOCK + 8}, \
    {"], \"est. achieved occupancy %\": ", T_I64, VK_I32, KS_PCT}, \
    {", \"occupancy\": {\"activeBlocksPerMultiprocessor\": ", T_I64, VK_I32, KS_ACTIVE}, {", \"limitingFactors\": \"", T_CSTR, VK_U32, KS_LIMIT}, \
    {"\", \"blockLimitRegs\": ", T_I64, VK_I32, KS_LREGS}, {", \"blockLimitSharedMem\": ", T_I64, VK_I32, KS_LSMEM}, \
    {", \"blockLimitWarps\": ", T_I64, VK_I32, KS_LWARPS}, {", \"blockLimitBlocks\": ", T_I64, VK_I32, KS_LBLOCKS}, \
    {", \"blockLimitBarriers\": ", T_I64, VK_I32, KS_LBARR}, {", \"allocatedRegistersPerBlock\": ", T_I64, VK_I32, KS_AREGS}, \
    {", \"allocatedSharedMemPerBlock\": ", T_U64, VK_64, KS_ASMEM}, {"}, \"graph id\": ", T_U64, VK_U32, KR_GRAPH}, \
    {", \"graph node id\": ", T_U64, VK_64, KR_NODE}, {", \"channel\": ", T_U64, VK_U32, KR_CHAN}, \
    {", \"channel_type\": ", T_U64, VK_U32, KR_CHTYPE}, {"", T_COLL, VK_U32, KS_COLLROW}, {"\n    }\n  },", T_NONE}, \
    {"\n  {\n    \"ph\": \"f\",\n    \"id\": ", T_U64, VK_U32, KR_CORR}, {",\n    \"pid\": ", T_U64, VK_U32, KR_DEV}, \
    {",\n    \"tid\": ", T_U64, VK_U32, KR_STREAM}, {",\n    \"ts\": ", T_TS, VK_64, KS_TS}, \
    {",\n    \"cat\": \"ac2g\",\n    \"name\": \"ac2g\"\n    , \"bp\": \"e\"\n  },", T_NONE}

// -- memcpy / memcpy2 / memset records (libkineto/src/CuptiActivity.h:586-712; 88 / 96 / 88 bytes).  The
// fields whose position differs between the layouts are copied to common slots past the record. --
enum : int { MR_BYTES = 8, MS_TS = 16, MS_DUR = 24, MR_DEV = 32, MR_CTX = 36, MR_STREAM = 40, MR_FROMDEV = 44, MR_FROMCTX = 48,
             MR_TODEV = 52, MR_TOCTX = 56, MS_KIND0 = 100, MS_KIND1 = 104, MS_KIND2 = 108, MS_EXT = 112, MS_BW = 120, MS_GRAPH = 128,
             MS_NODE = 136, MS_CHAN = 144, MS_CHTYPE = 148, MS_CORR = 152 };
enum : int { M_CPY_KIND, M_CPY_SRC, M_CPY_DST, M_SET_KIND, M_PID, M_TID, M_TS, M_DUR, M_ARGS, M_EXT, M_EXTC, M_FROMDEV, M_INDEV,
             M_TODEV, M_FROMCTX, M_INCTX, M_TOCTX, M_DEV, M_CTX, M_STREAM, M_CORR, M_BYTES, M_BW, M_GRAPH, M_NODE, M_CHAN, M_CHTYPE,
             M_CLOSE, M_FLOW, M_FPID, M_FTID, M_FTS, M_FEND, M_COUNT };
#define K2J_MEM_FIELDS \
    {XHEAD("gpu_memcpy") "Memcpy ", T_CSTR, VK_U32, MS_KIND0}, {" (", T_CSTR, VK_U32, MS_KIND1}, {" -> ", T_CSTR, VK_U32, MS_KIND2}, \
    {XHEAD("gpu_memset") "Memset (", T_CSTR, VK_U32, MS_KIND0}, \
    {")\",\n    \"pid\": ", T_U64, VK_U32, MR_DEV}, {",\n    \"tid\": ", T_U64, VK_U32, MR_STREAM}, {",\n    \"ts\": ", T_TS, VK_64, MS_TS}, \
    {",\n    \"dur\": ", T_TS, VK_64, MS_DUR}, \
    {"\n    ,\n    \"args\": {\n      ", T_NONE}, {"\"External id\": ", T_I64, VK_I32, MS_EXT}, {",", T_NONE}, \
    {"\"fromDevice\": ", T_U64, VK_U32, MR_FROMDEV}, {", \"inDevice\": ", T_U64, VK_U32, MR_DEV}, {", \"toDevice\": ", T_U64, VK_U32, MR_TODEV}, \
    {", \"fromContext\": ", T_U64, VK_U32, MR_FROMCTX}, {", \"inContext\": ", T_U64, VK_U32, MR_CTX}, {", \"toContext\": ", T_U64, VK_U32, MR_TOCTX}, \
    {"\"device\": ", T_U64, VK_U32, MR_DEV}, {", \"context\": ", T_U64, VK_U32, MR_CTX}, \
    {", \"stream\": ", T_U64, VK_U32, MR_STREAM}, {", \"correlation\": ", T_U64, VK_U32, MS_CORR}, {", \"bytes\": ", T_U64, VK_64, MR_BYTES}, \
    {", \"memory bandwidth (GB/s)\": ", T_DBL, VK_64, MS_BW}, \
    {", \"graph id\": ", T_U64, VK_U32, MS_GRAPH}, {", \"graph node id\": ", T_U64, VK_64, MS_NODE}, {", \"channel\": ", T_U64, VK_U32, MS_CHAN}, \
    {", \"channel_type\": ", T_U64, VK_U32, MS_CHTYPE}, \
    {"\n    }\n  },", T_NONE}, \
    {"\n  {\n    \"ph\": \"f\",\n    \"id\": ", T_U64, VK_U32, MS_CORR}, {",\n    \"pid\": ", T_U64, VK_U32, MR_DEV}, \
    {",\n    \"tid\": ", T_U64, VK_U32, MR_STREAM}, {",\n    \"ts\": ", T_TS, VK_64, MS_TS}, \
    {",\n    \"cat\": \"ac2g\",\n    \"name\": \"ac2g\"\n    , \"bp\": \"e\"\n  },", T_NONE}

// -- CPU-side activity (no record: every value is a slot): head, metadata entries, tail --
enum : int { OS_CAT = 0, OS_NAME = 4, OS_PID = 8, OS_EXT = 12, OS_TID = 16, OS_TS = 24, OS_DUR = 32, OS_ROW = 40, OS_FLOW = 44, OS_FTS = 48 };
enum : int { O_CAT, O_NAME, O_CNAME /* a constant-string name instead of a pool name */,
             I_HEAD, I_NAME /* an instant event: libkineto/src/output_json.cpp:261-293, :660-676 */,
             C_HEAD, C_NAME /* a counter event: libkineto/src/output_json.cpp:294-316, :679-716 */, H_ALL /* HARDWARE_COUNTERS: one event per value */,
             O_PID, O_TID, O_TS, O_DUR, O_PAD, O_ARGS,
             O_EXT, O_EXTC, O_MD, I_MD /* the same entries, nothing sanitised */, C_MD /* counter values */,
             P_ARGS_CLOSE, P_CLOSE, P_FLOW_S, P_FLOW_F, P_FPID, P_FTID, P_FTS, P_FWDBWD, P_AC2G, P_FBP, P_FEND, O_COUNT };
#define K2J_OPHEAD_FIELDS \
    {"\n  {\n    \"ph\": \"X\",\n    \"cat\": \"", T_CSTR, VK_U32, OS_CAT}, {"\",\n    \"name\": \"", T_NAME, VK_U32, OS_NAME}, \
    {"\",\n    \"name\": \"", T_CSTR, VK_U32, OS_NAME}, \
    {"\n  {\n    \"ph\": \"i\",\n    \n    \"cat\": \"", T_CSTR, VK_U32, OS_CAT}, {"\",\n    \"s\": \"t\",\n    \"name\": \"", T_RAWSTR, VK_U32, OS_NAME}, \
    {"\n  {\n    \"ph\": \"C\",\n    \"cat\": \"", T_CSTR, VK_U32, OS_CAT}, {"\",\n    \"name\": \"", T_RAWSTR, VK_U32, OS_NAME}, {"", T_HWC, VK_U32, OS_ROW}, \
    {"\",\n    \"pid\": ", T_I64, VK_I32, OS_PID}, \
    {",\n    \"tid\": ", T_I64, VK_64, OS_TID}, {",\n    \"ts\": ", T_TS, VK_64, OS_TS}, {",\n    \"dur\": ", T_TS, VK_64, OS_DUR}, {"\n    ", T_NONE}, \
    {",\n    \"args\": {\n      ", T_NONE}, {"\"External id\": ", T_I64, VK_I32, OS_EXT}, {",", T_NONE}
#define K2J_OPTAIL_FIELDS \
    {"\n    }", T_NONE}, {"\n  },", T_NONE}, {"\n  {\n    \"ph\": \"s\",\n    \"id\": ", T_U64, VK_U32, OS_FLOW}, \
    {"\n  {\n    \"ph\": \"f\",\n    \"id\": ", T_U64, VK_U32, OS_FLOW}, {",\n    \"pid\": ", T_I64, VK_I32, OS_PID}, \
    {",\n    \"tid\": ", T_I64, VK_64, OS_TID}, {",\n    \"ts\": ", T_TS, VK_64, OS_FTS}, \
    {",\n    \"cat\": \"fwdbwd\",\n    \"name\": \"fwdbwd\"\n    ", T_NONE}, {",\n    \"cat\": \"ac2g\",\n    \"name\": \"ac2g\"\n    ", T_NONE}, \
    {", \"bp\": \"e\"", T_NONE}, {FLOW_TAIL, T_NONE}

// -- gpu_user_annotation span --
enum : int { NS_NAME = 0, NS_PID = 4, NS_TID = 8, NS_EXT = 12, NS_TS = 16, NS_DUR = 24 };
enum : int { N_HEAD, N_PID, N_TID, N_TS, N_DUR, N_PAD, N_EXT, N_ARGS_CLOSE, N_CLOSE, N_COUNT };
#define K2J_ANN_FIELDS \
    {XHEAD("gpu_user_annotation"), T_NAME, VK_U32, NS_NAME}, {"\",\n    \"pid\": ", T_U64, VK_U32, NS_PID}, \
    {",\n    \"tid\": ", T_U64, VK_U32, NS_TID}, {",\n    \"ts\": ", T_TS, VK_64, NS_TS}, \
    {",\n    \"dur\": ", T_TS, VK_64, NS_DUR}, {"\n    ", T_NONE}, {",\n    \"args\": {\n      \"External id\": ", T_I64, VK_I32, NS_EXT}, \
    {"\n    }", T_NONE}, {"\n  },", T_NONE}


// -- synchronisation record (CudaSyncActivity, libkineto/src/CuptiActivity.h:181-211, :325-373; 40 bytes) and CUDA
// event record (CudaEventActivity, :233-262, :375-411; its fields are copied to the same slots).  A stream sync
// sits on a row of its own, and the first one of a row is preceded by two metadata rows
// (libkineto/src/output_json.cpp:914-943). --
enum : int { YS_TS = 8, YS_DUR = 16, YR_CORR = 24, YR_CTX = 28, YS_STREAM = 32, YR_EVENT = 36, YS_PID = 40, YS_EXT = 44, YS_TID = 48,
             YS_NAME = 56, YS_SRCSTREAM = 60, YS_SRCCORR = 64, YS_ROWTID = 72 };
enum : int { Y_MROW1, Y_MPID1, Y_MTID1, Y_MNAME, Y_MROW2, Y_MPID2, Y_MTID2, Y_MSORT, Y_MEND, Y_HEAD_SYNC, Y_HEAD_EVENT, Y_PID, Y_TID,
             Y_TS, Y_DUR, Y_ARGS, Y_EXT, Y_EXTC, Y_KIND, Y_WSTREAM, Y_WCORR, Y_WEVENT, Y_EVENTID, Y_STREAM_A, Y_STREAM_B, Y_CORR,
             Y_DEV, Y_CTX, Y_CLOSE, Y_FLOW, Y_FPID, Y_FTID, Y_FTS, Y_FEND, Y_COUNT };
#define K2J_SYNC_FIELDS \
    {"\n  {\n    \"name\": \"thread_name\", \"ph\": \"M\", \"ts\": ", T_TS, VK_64, YS_TS}, {", \"pid\": ", T_U64, VK_U32, YS_PID}, \
    {", \"tid\": ", T_I64, VK_64, YS_ROWTID}, {",\n    \"args\": {\n      \"name\": \"stream ", T_I64, VK_I32, YS_STREAM}, \
    {" (sync)\"\n    }\n  },\n  {\n    \"name\": \"thread_sort_index\", \"ph\": \"M\", \"ts\": ", T_TS, VK_64, YS_TS}, \
    {", \"pid\": ", T_U64, VK_U32, YS_PID}, {", \"tid\": ", T_I64, VK_64, YS_ROWTID}, \
    {",\n    \"args\": {\n      \"sort_index\": ", T_I64, VK_I32, YS_STREAM}, {"\n    }\n  },", T_NONE}, \
    {XHEAD("cuda_sync"), T_CSTR, VK_U32, YS_NAME}, {XHEAD("cuda_event") "cudaEvent", T_NONE}, \
    {"\",\n    \"pid\": ", T_U64, VK_U32, YS_PID}, {",\n    \"tid\": ", T_U64, VK_64, YS_TID}, {",\n    \"ts\": ", T_TS, VK_64, YS_TS}, \
    {",\n    \"dur\": ", T_TS, VK_64, YS_DUR}, {"\n    ,\n    \"args\": {\n      ", T_NONE}, \
    {"\"External id\": ", T_I64, VK_I32, YS_EXT}, {",", T_NONE}, {"\"cuda_sync_kind\": \"", T_CSTR, VK_U32, YS_NAME}, \
    {"\", \"wait_on_stream\": ", T_I64, VK_I32, YS_SRCSTREAM}, {", \"wait_on_cuda_event_record_corr_id\": ", T_I64, VK_I32, YS_SRCCORR}, \
    {", \"wait_on_cuda_event_id\": ", T_U64, VK_U32, YR_EVENT}, {"\"event_id\": ", T_U64, VK_U32, YR_EVENT}, \
    {", \"stream\": ", T_I64, VK_I32, YS_STREAM}, {"\", \"stream\": ", T_I64, VK_I32, YS_STREAM}, \
    {", \"correlation\": ", T_U64, VK_U32, YR_CORR}, {", \"device\": ", T_U64, VK_U32, YS_PID}, {", \"context\": ", T_U64, VK_U32, YR_CTX}, \
    {"\n    }\n  },", T_NONE}, \
    {"\n  {\n    \"ph\": \"f\",\n    \"id\": ", T_U64, VK_U32, YR_CORR}, {",\n    \"pid\": ", T_U64, VK_U32, YS_PID}, \
    {",\n    \"tid\": ", T_U64, VK_64, YS_TID}, {",\n    \"ts\": ", T_TS, VK_64, YS_TS}, \
    {",\n    \"cat\": \"ac2g\",\n    \"name\": \"ac2g\"\n    , \"bp\": \"e\"\n  },", T_NONE}

// One table for everything: [api][kernel][mem][op head, metadata marker, op tail][annotation][sync][constant strings].
enum : int { CS_TYPE = 0, CS_MEMCPY_KIND = 29, CS_MEMORY_KIND = 41, CS_LIMIT = 50, CS_OVERHEAD = 82, CS_SYNC = 93, CS_COLL = 98,
             CS_HWC = 114 /* the pieces of a HARDWARE_COUNTERS event */, CS_COUNT = 120 };
#define K2J_CSTR_FIELDS \
    {"cpu_op", 0}, {"user_annotation", 0}, {"gpu_user_annotation", 0}, {"gpu_memcpy", 0}, {"gpu_memset", 0}, {"kernel", 0}, \
    {"external_correlation", 0}, {"cuda_runtime", 0}, {"cuda_driver", 0}, {"cpu_instant_event", 0}, {"python_function", 0}, \
    {"overhead", 0}, {"mtia_runtime", 0}, {"mtia_ccp_events", 0}, {"mtia_insight", 0}, {"cuda_sync", 0}, {"cuda_event", 0}, \
    {"mtia_counters", 0}, {"glow_runtime", 0}, {"cuda_profiler_range", 0}, {"hpu_op", 0}, {"xpu_runtime", 0}, \
    {"xpu_driver", 0}, {"collective_comm", 0}, {"privateuse1_runtime", 0}, {"privateuse1_driver", 0}, \
    {"xpu_scope_profiler", 0}, {"xpu_sync", 0}, {"hardware_counters", 0}, \
    {"<unknown>", 0}, {"HtoD", 0}, {"DtoH", 0}, {"HtoA", 0}, {"AtoH", 0}, {"AtoA", 0}, {"AtoD", 0}, {"DtoA", 0}, {"DtoD", 0}, \
    {"HtoH", 0}, {"PtoP", 0}, {"<unknown>", 0}, \
    {"Unknown", 0}, {"Pageable", 0}, {"Pinned", 0}, {"Device", 0}, {"Array", 0}, {"Managed", 0}, {"Device Static", 0}, \
    {"Managed Static", 0}, {"Unrecognized", 0}, \
    {"none", 0}, {"WARPS", 0}, {"REGS", 0}, {"WARPS|REGS", 0}, {"SMEM", 0}, {"WARPS|SMEM", 0}, {"REGS|SMEM", 0}, \
    {"WARPS|REGS|SMEM", 0}, {"BLOCKS", 0}, {"WARPS|BLOCKS", 0}, {"REGS|BLOCKS", 0}, {"WARPS|REGS|BLOCKS", 0}, \
    {"SMEM|BLOCKS", 0}, {"WARPS|SMEM|BLOCKS", 0}, {"REGS|SMEM|BLOCKS", 0}, {"WARPS|REGS|SMEM|BLOCKS", 0}, {"BARRIERS", 0}, \
    {"WARPS|BARRIERS", 0}, {"REGS|BARRIERS", 0}, {"WARPS|REGS|BARRIERS", 0}, {"SMEM|BARRIERS", 0}, \
    {"WARPS|SMEM|BARRIERS", 0}, {"REGS|SMEM|BARRIERS", 0}, {"WARPS|REGS|SMEM|BARRIERS", 0}, {"BLOCKS|BARRIERS", 0}, \
    {"WARPS|BLOCKS|BARRIERS", 0}, {"REGS|BLOCKS|BARRIERS", 0}, {"WARPS|REGS|BLOCKS|BARRIERS", 0}, \
    {"SMEM|BLOCKS|BARRIERS", 0}, {"WARPS|SMEM|BLOCKS|BARRIERS", 0}, {"REGS|SMEM|BLOCKS|BARRIERS", 0}, \
    {"WARPS|REGS|SMEM|BLOCKS|BARRIERS", 0}, \
    {"Unknown", 0}, {"Driver Compiler", 0}, {"Buffer Flush", 0}, {"Instrumentation", 0}, {"Resource", 0}, \
    {"Runtime Triggered Module Loading", 0}, {"Lazy Function Loading", 0}, {"Command Buffer Full", 0}, \
    {"Activity Buffer Request", 0}, {"Force Int", 0}, {"Unrecognized", 0}, \
    {"Unknown Sync", 0}, {"Event Sync", 0}, {"Stream Wait Event", 0}, {"Stream Sync", 0}, {"Context Sync", 0}, \
    {",\"Collective name\": ", 0}, {",\"In msg nelems\": ", 0}, {",\"Out msg nelems\": ", 0}, {",\"Group size\": ", 0}, \
    {",\"dtype\": ", 0}, {",\"Input Tensors start\": ", 0}, {",\"Output Tensors start\": ", 0}, {",\"In split size\": ", 0}, \
    {",\"Out split size\": ", 0}, {",\"Process Group Name\": ", 0}, {",\"Process Group Description\": ", 0}, \
    {",\"Process Group Ranks\": ", 0}, {",\"Dst Rank\": ", 0}, {",\"Src Rank\": ", 0}, {",\"Seq\": ", 0}, {",\"Comms Id\": ", 0}, \
    {"\n  {\n    \"ph\": \"C\",\n    \"cat\": \"hardware_counters\",\n    \"name\": \"", 0}, {"\",\n    \"pid\": \"GPU ", 0}, \
    {" Counters\",\n    \"tid\": ", 0}, {",\n    \"ts\": ", 0}, {",\n    \"args\": {\n      \"\": ", 0}, {"\n    }\n  },", 0}


constexpr int API_BASE = 0, KERNEL_BASE = API_BASE + A_COUNT, MEM_BASE = KERNEL_BASE + K_COUNT, OP_BASE = MEM_BASE + M_COUNT,
              ANN_BASE = OP_BASE + O_COUNT, SYNC_BASE = ANN_BASE + N_COUNT, CSTR_BASE = SYNC_BASE + Y_COUNT,
              FIELD_COUNT = CSTR_BASE + CS_COUNT;
constexpr FieldSrc kAllFields[] = {K2J_API_FIELDS, K2J_KERNEL_FIELDS, K2J_MEM_FIELDS, K2J_OPHEAD_FIELDS, {"", T_MD, VK_U32, OS_ROW},
                                   {"", T_MDRAW, VK_U32, OS_ROW}, {"", T_MDCNT, VK_U32, OS_ROW},
                                   K2J_OPTAIL_FIELDS, K2J_ANN_FIELDS, K2J_SYNC_FIELDS, K2J_CSTR_FIELDS};
static_assert(sizeof(kAllFields) / sizeof(kAllFields[0]) == FIELD_COUNT, "field table and enums disagree");
constexpr bool wide_values_aligned() {
  for (int f = 0; f < FIELD_COUNT; f++) if (kAllFields[f].vk == VK_64 && kAllFields[f].voff % 8 != 0) return false;
  return true;
}
static_assert(wide_values_aligned(), "64-bit values must sit at multiples of 8 (slot_value loads one aligned unit)");
constexpr int kAllWords = prog_words(kAllFields);
__constant__ Prog<FIELD_COUNT, kAllWords> g_fields = make_prog<FIELD_COUNT, kAllWords>(kAllFields);

// ---- value formatting ----------------------------------------------------------------------------------------
// Four zero-padded ASCII digits of x < 10^4, most significant digit in the low byte (32-bit SWAR).
__device__ __forceinline__ uint32_t ascii4(uint32_t x) {
  const uint32_t q = (x * 5243u) >> 19, r = x - q * 100u;          // x / 100, x % 100
  const uint32_t pk = q | (r << 16);
  const uint32_t t = ((pk * 103u) >> 10) & 0x000F000Fu;            // tens of both pairs
  return (t | ((pk - t * 10u) << 8)) | 0x30303030u;
}
// Decimal of v: inline paths below 10^4 and below 10^8 (nearly every field), out of line above.
template <class S> __device__ __forceinline__ void put_dec(S& s, uint64_t v) {
  if (S::kCounting) { s.skip((uint32_t)ndigits64(v)); return; }
  if (v < 10000ull) {
    const uint32_t x = (uint32_t)v;
    const int d = 1 + (x >= 10u) + (x >= 100u) + (x >= 1000u);
    s.put(ascii4(x) >> (8 * (4 - d)), d);
    return;
  }
  if (v < 100000000ull) {
    const uint32_t x = (uint32_t)v, hi = x / 10000u, lo = x - hi * 10000u;
    const int d = 1 + (hi >= 10u) + (hi >= 100u) + (hi >= 1000u);  // digits of the upper part (hi >= 1)
    s.put64((uint64_t)(ascii4(hi) >> (8 * (4 - d))) | ((uint64_t)ascii4(lo) << (8 * d)), d + 4);
    return;
  }
  put_u64(s, v);
}
template <class S> __device__ __forceinline__ void put_dbl(S& s, double v) { put_double_value(s, v); }
template <class S> __device__ __forceinline__ void put_sdec(S& s, int64_t v) {
  if (v < 0) { put_char(s, '-'); put_dec(s, 0ull - (uint64_t)v); }
  else put_dec(s, (uint64_t)v);
}
template <class S> __device__ __forceinline__ void put_ts2(S& s, int64_t ns) {  // "{}.{:03}" of ns/1000, ns%1000
  const uint64_t us = (uint64_t)ns / 1000ull;
  const uint32_t fr = (uint32_t)((uint64_t)ns - us * 1000ull);
  put_dec(s, us);
  if (S::kCounting) { s.skip(4); return; }
  const uint32_t a = (fr * 41u) >> 12, r = fr - a * 100u, b = (r * 103u) >> 10, c = r - b * 10u;
  s.put4(0x3030302Eu + (a << 8) + (b << 16) + (c << 24));
}

template <class S> __device__ __forceinline__ void put_pool_words(S& s, const uint8_t* src, uint32_t len) {
  s.words(reinterpret_cast<const uint64_t*>(src), len);  // sanitised pool strings start 8-byte aligned
}
template <class S> __device__ __forceinline__ void put_name(S& s, const Dev& d, uint32_t id, unsigned long long* name_bytes) {
  if (id >= d.n_strings) { atomicAdd(&d.counters->device_check, 1ull); return; }

  const uint32_t len = d.esc_name_len[id];
  put_pool_words(s, d.esc_name + esc_name_pos(d, id), len);
  *name_bytes += len;
}
template <class S> __device__ __forceinline__ void put_mdstr(S& s, const Dev& d, uint32_t id) {
  if (id >= d.n_strings) { atomicAdd(&d.counters->device_check, 1ull); return; }
  put_pool_words(s, d.esc_md + esc_md_pos(d, id), d.esc_md_len[id]);
}

__device__ __noinline__ int64_t tsc_convert(uint64_t t, uint64_t t0a, int64_t t0, uint64_t mant, int exp) {
  return tsc_to_ns(t, t0a, t0, mant, exp);
}
__device__ __forceinline__ int64_t conv_ts(const Dev& d, uint64_t t) {
  return d.ts_mode ? tsc_convert(t, d.conv_t0a, d.conv_t0, d.conv_mant, d.conv_exp) : (int64_t)t;
}
__device__ __forceinline__ int64_t conv_dur(const Dev& d, uint64_t s, uint64_t e) {
  return d.ts_mode ? conv_ts(d, e) - conv_ts(d, s) : (int64_t)(e - s);
}
__device__ __forceinline__ int64_t rel_ts(const Dev& d, int64_t t) { const int64_t r = t - d.base; return r < 0 ? 0 : r; }
__device__ __forceinline__ int64_t abs_tid(int64_t t) { return t == INT64_MIN ? 0 : (t < 0 ? -t : t); }
__device__ __forceinline__ bool out_of_range(const Dev& d, int64_t ts, int64_t dur) {
  return ts < d.win_start || (ts + dur) > d.win_end;
}

// linkedActivity(int32_t correlationId, cpuCorrelationMap_) (GenericActivityProfiler.cpp:397-408):
// the id is sign-extended before the lookup while keys were stored zero-extended, so ids >= 2^31
// never match; the external id must equal a CPU-op id exactly as a 64-bit value.
// k_resolve_corr does the two dependent lookups once per table entry and leaves the linked op's id
// (or 0) in the entry's low half, so that an event needs a single probe.
// Is there a CPU-side activity with this id (activityMap_.find, GenericActivityProfiler.cpp:397-408)?  The table holds
// this shard's ids (or every shard's, as lists); the other shards' ids may come as bitmaps instead.
struct OpBits { const uint32_t* bits; uint64_t pitch; const int64_t* meta; uint32_t world, own_rank; };
__device__ __forceinline__ OpBits op_bits_of(const Dev& d) { return OpBits{d.op_bits, d.op_bits_pitch, d.op_bits_meta, d.op_bits_world, d.own_rank}; }
__device__ __forceinline__ bool op_in_bitmaps(const OpBits b, int32_t id) {
  if (b.bits == nullptr) return false;
  for (uint32_t r = 0; r < b.world; r++) {
    if (r == b.own_rank) continue;
    const int64_t k = (int64_t)id - b.meta[2 * r];
    if (k >= 0 && k < b.meta[2 * r + 1] && ((b.bits[(uint64_t)r * b.pitch + (uint64_t)(k >> 5)] >> (k & 31)) & 1u)) return true;
  }
  return false;
}
__device__ __forceinline__ bool op_known(const Dev& d, int32_t id) {
  return tab_find(d.op_tab, d.op_mask, (uint32_t)id) != 0xFFFFFFFFu || op_in_bitmaps(op_bits_of(d), id);
}
__global__ void k_op_id_bits(Dev d, int64_t min_id, uint64_t n_bits, uint32_t* bits) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.n_ops - d.n_guest_ops) return;
  const int64_t k = (int64_t)d.op_id[i] - min_id;
  if (k < 0 || (uint64_t)k >= n_bits) { atomicAdd(&d.counters->device_check, 1ull); return; }
  atomicOr(&bits[k >> 5], 1u << (k & 31));
}
__global__ void k_resolve_corr(Dev d) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0u && d.corr0[0] != 0ull) {  // correlation id 0
    ExtRec z; ext_at(d, d.corr0[0] - 1ull, &z);
    const int64_t ext = (int64_t)z.external_id;
    const bool linked = ext == (int64_t)(int32_t)ext && op_known(d, (int32_t)ext);
    d.corr0[1] = linked ? ((1ull << 33) | (unsigned long long)(uint32_t)(int32_t)ext) : 0ull;
  }
  if (i > d.corr_mask) return;
  const unsigned long long e = d.corr_tab[i];
  if (e == 0) return;
  ExtRec rec; ext_at(d, (uint32_t)e - 1u, &rec);
  const int64_t ext = (int64_t)rec.external_id;
  uint32_t id = 0;
  if (ext == (int64_t)(int32_t)ext && op_known(d, (int32_t)ext))
  {
    id = (uint32_t)(int32_t)ext;  // the linked op's correlationId() is the key it was found under
    if (id == 0u && d.corr_zero != nullptr) atomicOr(&d.corr_zero[i >> 5], 1u << (i & 31u));  // linked, to the op whose id is 0
  }
  d.corr_tab[i] = (e & 0xFFFFFFFF00000000ull) | id;
}
// The first probe is split off so that callers can issue its load early, next to other loads.
__device__ __forceinline__ unsigned long long linked_op_peek(const Dev& d, uint32_t corr) {
  if ((corr & 0x80000000u) || d.corr_tab == nullptr) return 0ull;
  return d.corr_tab[hash32(corr) & d.corr_mask];
}
__device__ __forceinline__ void linked_op(const Dev& d, uint32_t corr, unsigned long long first, int32_t* op_id) {
  if ((corr & 0x80000000u) || d.corr_tab == nullptr) return;
  if (corr == 0u) { const unsigned long long z = d.corr0[1]; if ((z >> 33) & 1ull) *op_id = (int32_t)(uint32_t)z; return; }
  uint32_t i = hash32(corr) & d.corr_mask;
  unsigned long long e = first;
  for (uint32_t probes = 0; probes <= d.corr_mask; probes++) {
    if (e == 0) return;  // an empty slot
    if ((uint32_t)(e >> 32) == corr) { *op_id = (int32_t)(uint32_t)e; return; }
    i = (i + 1) & d.corr_mask;
    e = d.corr_tab[i];
  }
}

// GenericActivityProfiler::handleGpuActivity's user-annotation step (GenericActivityProfiler.cpp:424-434)
// with GpuUserEventMap::insertOrExtendEvent (:292-311): per (device, stream) and annotation op the span
// [min start, max end] over the GPU activities correlated to it.  Runs in the size pass only.
// Out of line (rare), with the tables it touches passed by value: a reference to the kernel's parameter block would
// make every thread of the size pass copy that block (about 1 KB) into local memory at kernel entry.
struct SpanArgs {
  const unsigned long long* user_tab; uint32_t user_mask; const ExtRec* ext_all; uint32_t ext_stride; uint64_t join_pitch;  // rows of an all-gather: see Dev
  const ExtRec* ext_local; uint32_t own_rank; OpBits op_bits;
  const unsigned long long* op_tab; uint32_t op_mask;
  unsigned long long* ds_tab; uint32_t ds_mask; unsigned long long* span_key; unsigned long long* span_nstart;
  unsigned long long* span_end; unsigned long long* span_nfirst; uint32_t* span_row; uint32_t span_mask; Counters* counters;
};
__device__ __forceinline__ SpanArgs span_args(const Dev& d) {
  return SpanArgs{d.user_tab, d.user_mask, d.ext_all, d.join_counts != nullptr ? d.ext_stride : 0u, d.join_pitch, d.ext_local, d.own_rank, op_bits_of(d), d.op_tab, d.op_mask, d.ds_tab, d.ds_mask, d.span_key, d.span_nstart,
                  d.span_end, d.span_nfirst, d.span_row, d.span_mask, d.counters};
}
__device__ __noinline__ void span_update(const SpanArgs d, uint32_t corr, uint32_t dev, uint32_t stream, int64_t ts,
                                         int64_t dur, uint64_t ev) {
  const uint32_t idx = tab_find(d.user_tab, d.user_mask, corr);
  if (idx == 0xFFFFFFFFu) return;
  // (the table only holds positions of records that exist, so no count is looked at here)
  const ExtRec* rec = d.ext_stride == 0u ? d.ext_all + idx
                      : idx / d.ext_stride == d.own_rank ? d.ext_local + idx % d.ext_stride
                      : reinterpret_cast<const ExtRec*>(reinterpret_cast<const uint8_t*>(d.ext_all) + (uint64_t)(idx / d.ext_stride) * d.join_pitch) + idx % d.ext_stride;
  const int64_t ext = (int64_t)rec->external_id;
  if (ext != (int64_t)(int32_t)ext) return;
  const uint32_t row = tab_find(d.op_tab, d.op_mask, (uint32_t)(int32_t)ext);
  if (row == 0xFFFFFFFFu && !op_in_bitmaps(d.op_bits, (int32_t)ext)) return;  // (several shards: the row is not used, only that the op exists)
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

// ---- synchronisation and CUDA event records: the lookups of CuptiActivityProfiler.cpp:221-254, :379-402, :502-514 ----
// A set of 64-bit keys (0 = empty slot).  Returns the key's slot, or 0xFFFFFFFF if absent (or the table is full).
__device__ __forceinline__ uint32_t set64_slot(unsigned long long* tab, uint32_t mask, unsigned long long key, bool insert) {
  uint32_t i = hash32((uint32_t)(key >> 32) * 0x9E3779B1u ^ (uint32_t)key) & mask;
  for (uint32_t probes = 0; probes <= mask; probes++) {
    unsigned long long old = tab[i];
    if (old == 0) {
      if (!insert) return 0xFFFFFFFFu;
      old = atomicCAS(&tab[i], 0ull, key);
      if (old == 0) return i;
    }
    if (old == key) return i;
    i = (i + 1) & mask;
  }
  return 0xFFFFFFFFu;
}
__device__ __forceinline__ unsigned long long dev_stream_key(uint32_t dev, uint32_t stream) {
  return (((unsigned long long)dev << 32) | stream) + 1ull;
}
// seenDeviceStreams_ (GenericActivityProfiler.cpp:419): streams with a kernel, copy or memset inside the window.
__device__ __forceinline__ void seen_insert(const Dev& d, uint32_t dev, uint32_t stream) {
  if (set64_slot(d.seen_tab, d.seen_mask, dev_stream_key(dev, stream), true) == 0xFFFFFFFFu) atomicAdd(&d.counters->device_check, 1ull);
}
// ctxToDeviceId (CuptiActivityProfiler.cpp:221-239): the first kernel, copy or memset record that names a context
// decides its device; a peer-to-peer copy names its source context, then its destination context.  Values are
// record positions, so the smallest one is the first writer in processing order.
__global__ void k_build_ctx(Dev d) {
  const uint64_t i = d.cls_begin[C_KERNEL] + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.cls_begin[C_OVERHEAD]) return;
  int cls = C_KERNEL;
#pragma unroll
  for (int c = C_MEMCPY; c <= C_MEMSET; c++) if (i >= d.cls_begin[c]) cls = c;
  if (i - d.cls_begin[cls] >= d.cls_count[cls]) return;  // padding
  const uint32_t slot = d.work_slot[i];
  const uint8_t* r = d.cupti + (uint64_t)slot * 8;
  bool ok;
  if (cls == C_MEMCPY2) {
    ok = tab_insert_min(d.ctx_tab, d.ctx_mask, *reinterpret_cast<const uint32_t*>(r + 48), slot);
    ok = tab_insert_min(d.ctx_tab, d.ctx_mask, *reinterpret_cast<const uint32_t*>(r + 56), slot) && ok;
  } else ok = tab_insert_min(d.ctx_tab, d.ctx_mask, *reinterpret_cast<const uint32_t*>(r + (cls == C_KERNEL ? 44 : 36)), slot);
  if (!ok) atomicAdd(&d.counters->device_check, 1ull);
}
// contextIdtoDeviceId (CuptiActivityProfiler.cpp:527-530): device 0 for a context no record names.
__device__ __forceinline__ uint32_t ctx_device(const Dev& d, uint32_t ctx) {
  const uint32_t slot = tab_find(d.ctx_tab, d.ctx_mask, ctx);
  if (slot == 0xFFFFFFFFu) return 0u;
  const uint8_t* r = d.cupti + (uint64_t)slot * 8;
  const uint32_t kind = *reinterpret_cast<const uint32_t*>(r);
  if (kind == K_KERNEL) return *reinterpret_cast<const uint32_t*>(r + 40);
  if (kind == K_MEMCPY2) return *reinterpret_cast<const uint32_t*>(r + (*reinterpret_cast<const uint32_t*>(r + 48) == ctx ? 44 : 52));
  return *reinterpret_cast<const uint32_t*>(r + 32);
}
// Sort keys of the CUDA event records (work items of class C_CUDAEVENT, in processing order).  Stage 0: the
// correlation id; stage 1, on the result of the first sort: context << 32 | event id.  Both sorts are stable, so
// records end up ordered by (context, event, correlation id, position).
__global__ void k_evt_keys(Dev d, uint64_t* keys, uint32_t* vals, int stage) {
  const uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= d.cls_count[C_CUDAEVENT]) return;
  const uint32_t j = stage == 0 ? (uint32_t)p : vals[p];
  const uint8_t* r = d.cupti + (uint64_t)d.work_slot[d.cls_begin[C_CUDAEVENT] + j] * 8;
  if (stage == 0) { keys[p] = *reinterpret_cast<const uint32_t*>(r + 4); vals[p] = j; }
  else keys[p] = ((uint64_t)*reinterpret_cast<const uint32_t*>(r + 8) << 32) | *reinterpret_cast<const uint32_t*>(r + 16);
}
__global__ void k_evt_finish(Dev d, const uint64_t* keys, const uint32_t* vals, EvtRec* out) {
  const uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= d.cls_count[C_CUDAEVENT]) return;
  const uint8_t* r = d.cupti + (uint64_t)d.work_slot[d.cls_begin[C_CUDAEVENT] + vals[p]] * 8;
  EvtRec e;
  e.key = keys[p]; e.corr = *reinterpret_cast<const uint32_t*>(r + 4); e.stream = *reinterpret_cast<const uint32_t*>(r + 12);
  out[p] = e;
}
// getWaitEventInfo (CuptiActivityProfiler.cpp:379-402) over updateWaitEventMap's vectors (:243-254): among the
// records of (context, event) the largest correlation id not above the query's; among records with that id the
// one that came first (a new record is inserted before its equals, and the last of the equals is taken).
__device__ __forceinline__ bool wait_event_find(const Dev& d, uint32_t ctx, uint32_t event, uint32_t corr, int32_t* stream, int32_t* rcorr) {
  if (d.evt == nullptr || d.n_evt == 0) return false;
  const uint64_t key = ((uint64_t)ctx << 32) | event;
  uint32_t lo = 0, hi = d.n_evt;
  for (int it = 0; it < 34 && lo < hi; it++) {  // first record above (key, corr)
    const uint32_t mid = lo + ((hi - lo) >> 1);
    const EvtRec r = d.evt[mid];
    if (r.key < key || (r.key == key && r.corr <= corr)) lo = mid + 1; else hi = mid;
  }
  if (lo == 0) return false;
  const EvtRec last = d.evt[lo - 1];
  if (last.key != key) return false;
  uint32_t lo2 = 0, hi2 = lo - 1;
  for (int it = 0; it < 34 && lo2 < hi2; it++) {  // first record not below (key, last.corr)
    const uint32_t mid = lo2 + ((hi2 - lo2) >> 1);
    const EvtRec r = d.evt[mid];
    if (r.key < key || (r.key == key && r.corr < last.corr)) lo2 = mid + 1; else hi2 = mid;
  }
  const EvtRec first = d.evt[lo2];
  *stream = (int32_t)first.stream; *rcorr = (int32_t)first.corr;
  return true;
}
// linkedActivity for record types that print their own correlation id when nothing is linked: tells "linked to the
// CPU op whose id is 0" from "not linked" (k_resolve_corr leaves 0 in the entry for both and marks the former).
__device__ __forceinline__ bool linked_op_full(const Dev& d, uint32_t corr, int32_t* id) {
  if ((corr & 0x80000000u) || d.corr_tab == nullptr) return false;
  if (corr == 0u) { const unsigned long long z = d.corr0[1]; if ((z >> 33) & 1ull) { *id = (int32_t)(uint32_t)z; return true; } return false; }
  uint32_t i = hash32(corr) & d.corr_mask;
  for (uint32_t probes = 0; probes <= d.corr_mask; probes++) {
    const unsigned long long e = d.corr_tab[i];
    if (e == 0) return false;
    if ((uint32_t)(e >> 32) == corr) {
      if ((uint32_t)e != 0u) { *id = (int32_t)(uint32_t)e; return true; }
      if (d.corr_zero != nullptr && ((d.corr_zero[i >> 5] >> (i & 31u)) & 1u)) { *id = 0; return true; }
      return false;
    }
    i = (i + 1) & d.corr_mask;
  }
  return false;
}

struct Tally { uint32_t x, flow; unsigned long long name_bytes; uint64_t ev; uint64_t work; };

// A thread's area in shared memory: the staged record plus value slots (see the S_ offsets above).
constexpr int kRecStride = 23;              // 8-byte units per thread: 22 for the part of the longest record (Kernel9) that
                                            // fields read (176 of its 208 bytes); odd, so that 64-bit reads of 32 lanes
                                            // fall in distinct banks
constexpr int kAreaWords = 2 * kRecStride;  // the same in 32-bit words
__device__ __forceinline__ uint32_t a32(const uint32_t* a, int off) { return a[off >> 2]; }
__device__ __forceinline__ uint64_t a64(const uint32_t* a, int off) { return (uint64_t)a[off >> 2] | ((uint64_t)a[(off >> 2) + 1] << 32); }
__device__ __forceinline__ void s32(uint32_t* a, int off, uint32_t v) { a[off >> 2] = v; }
__device__ __forceinline__ void s64(uint32_t* a, int off, uint64_t v) { a[off >> 2] = (uint32_t)v; a[(off >> 2) + 1] = (uint32_t)(v >> 32); }
// value of a field: 32 bits zero- or sign-extended, or 64 bits (no branches)
// One 64-bit load of the aligned unit that holds the value: areas are an odd number of units apart, so the 64-bit
// loads of a warp touch every bank pair once, while 32-bit loads at that stride would collide two ways.  (64-bit
// values sit at multiples of 8.)
__device__ __forceinline__ uint64_t slot_value(const uint32_t* a, uint32_t voff, uint32_t vk) {
  const uint64_t u = reinterpret_cast<const uint64_t*>(a)[voff >> 3];
  const uint32_t lo = (voff & 4u) ? (uint32_t)(u >> 32) : (uint32_t)u;
  uint32_t hi = vk == VK_I32 ? (uint32_t)((int32_t)lo >> 31) : 0u;
  if (vk == VK_64) hi = (uint32_t)(u >> 32);
  return (uint64_t)lo | ((uint64_t)hi << 32);
}

// Each gather reads the staged record in `a`, writes the computed slots and returns the set of fields
// the event prints; 0 if the record produces no event (`*filt`: 1 blocklisted, 2 outside the window).
// `counting`: the size pass, which also finds the linked CPU op; the emit pass gets it as `ext_known`.

// handleRuntimeActivity / handleDriverActivity (libkineto/src/CuptiActivityProfiler.cpp:304-358)
__device__ __forceinline__ uint64_t gather_api(const Dev& d, uint32_t* a, Tally& t, uint32_t* filt, bool counting, int32_t* ext_io) {
  const uint32_t kind = a32(a, 0), cbid = a32(a, AR_CBID);
  const uint64_t st = a64(a, 8), en = a64(a, 16);
  const uint32_t corr = a32(a, AR_CORR);
  const bool driver = kind == K_DRIVER;
  // issue the independent table loads together, before the checks that consume them
  int32_t tid = (int32_t)a32(a, 28);
  const uint32_t tid_slot = hash32((uint32_t)tid) & d.tid_mask;
  const unsigned long long tid_first = d.tid_tab[tid_slot];
  const unsigned long long corr_first = counting ? linked_op_peek(d, corr) : 0ull;
  const uint32_t ntab = driver ? d.n_dr : d.n_rt;
  const bool named = cbid < ntab;
  const uint32_t name_id = named ? (driver ? d.dr_names : d.rt_names)[cbid] : 0u;
  bool flow_start;
  if (!driver) {
    // CuptiCbidRegistry.cpp:127-161 blocklist; :57-122 flow-starting callbacks
    if (cbid == 17u || cbid == 16u || cbid == 10u || cbid == 133u || cbid == 134u || cbid == 136u) { *filt = 1; return 0; }
    flow_start = cbid == 211u || cbid == 269u || cbid == 272u || cbid == 430u || cbid == 311u || cbid == 131u ||
                 cbid == 165u || cbid == 147u || (cbid >= 31u && cbid <= 52u);
  } else {
    // CuptiCbidRegistry.cpp:166-207: only these driver callbacks are tracked
    if (!(cbid == 307u || cbid == 652u || (cbid >= 549u && cbid <= 552u) || cbid == 554u || cbid == 555u)) return 0;
    flow_start = cbid == 307u || cbid == 652u;
  }
  const int64_t ts = conv_ts(d, st), dur = conv_dur(d, st, en);
  if (out_of_range(d, ts, dur)) { *filt = 2; return 0; }
  {  // resourceInfo_.find({processId(), tid}), CuptiActivityProfiler.cpp:315-319
    uint32_t idx = 0xFFFFFFFFu, i = tid_slot;
    unsigned long long e = tid_first;
    for (uint32_t probes = 0; probes <= d.tid_mask && e != 0; probes++) {
      if ((uint32_t)(e >> 32) == (uint32_t)tid) { idx = (uint32_t)e - 1u; break; }
      i = (i + 1) & d.tid_mask;
      e = d.tid_tab[i];
    }
    if (idx != 0xFFFFFFFFu) tid = idx < d.n_tid_pairs ? d.tid_pairs[2 * idx + 1] : (int32_t)d.op_resource[idx - d.n_tid_pairs];
  }
  int32_t ext = *ext_io;
  if (counting) { linked_op(d, corr, corr_first, &ext); *ext_io = ext; }
  const bool has_ext = ext != 0;
  s64(a, AS_TS, (uint64_t)rel_ts(d, ts)); s64(a, AS_DUR, (uint64_t)(dur < 0 ? 0 : dur));
  s32(a, AS_PID, (uint32_t)d.pid); s32(a, AS_TID, (uint32_t)abs_tid(tid)); s32(a, AS_EXT, (uint32_t)ext);
  s32(a, AS_NAME, name_id);
  uint64_t p = 0;
  auto on = [&](int f) { p |= 1ull << f; };
  on(driver ? A_HEAD_DR : A_HEAD_RT); on(named ? A_NAME : A_INVALID);
  on(A_PID); on(A_TID); on(A_TS); on(A_DUR); on(A_ARGS);
  if (has_ext) { on(A_EXT); on(A_EXTC); }
  on(A_CBID); on(A_CORR); on(A_CLOSE);
  t.x++;
  if (corr > 0) {
    on(flow_start ? A_FLOW_S : A_FLOW_F); on(A_FPID); on(A_FTID); on(A_FTS); on(A_FCAT);
    if (!flow_start) on(A_FBP);
    on(A_FEND);
    t.flow++;
  }
  return p;
}

// computeOccupancyMetrics (libkineto/src/DeviceProperties.cpp:176-222) with NVIDIA's occupancy calculator.
__device__ __forceinline__ void occupancy_metrics(const Dev& d, uint32_t dev, bool have_dev, int sm_count, int32_t grid_prod,
                                               int32_t block_prod, uint32_t regs, int32_t ssm, int32_t dsm, cudaOccResult* out,
                                               float* occupancy_out) {
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
  *out = occ;
  *occupancy_out = occupancy;
}

// GpuActivity<Kernel> (libkineto/src/CuptiActivity.h:499-576)
__device__ __forceinline__ uint64_t gather_kernel(const Dev& d, uint32_t* a, Tally& t, uint32_t* filt, bool counting, int32_t* ext_io) {
  const unsigned long long corr_first = counting ? linked_op_peek(d, a32(a, KR_CORR)) : 0ull;  // issued early
  const uint64_t st = a64(a, 16), en = a64(a, 24);
  const int64_t ts = conv_ts(d, st), dur = conv_dur(d, st, en);
  if (out_of_range(d, ts, dur)) { *filt = 2; return 0; }
  const uint32_t dev = a32(a, KR_DEV), stream = a32(a, KR_STREAM), corr = a32(a, KR_CORR);
  const int32_t gx = (int32_t)a32(a, KR_GRID), gy = (int32_t)a32(a, KR_GRID + 4), gz = (int32_t)a32(a, KR_GRID + 8);
  const int32_t bx = (int32_t)a32(a, KR_BLOCK), by = (int32_t)a32(a, KR_BLOCK + 4), bz = (int32_t)a32(a, KR_BLOCK + 8);
  const int32_t ssm = (int32_t)a32(a, 76), dsm = (int32_t)a32(a, 80);
  const uint32_t regs = a32(a, 4) >> 16;  // registersPerThread: 16 bits at byte 6
  int32_t ext = *ext_io;
  if (counting) { linked_op(d, corr, corr_first, &ext); *ext_io = ext; }
  const bool has_ext = ext != 0;
  // blocksPerSm / warpsPerSm (DeviceProperties.cpp:161-174): 32-bit wrapping products, single-precision
  // arithmetic without contraction.
  const int32_t grid_prod = (int32_t)((uint32_t)gx * (uint32_t)gy * (uint32_t)gz);
  const int32_t block_prod = (int32_t)((uint32_t)bx * (uint32_t)by * (uint32_t)bz);
  const bool have_dev = dev < (uint32_t)d.n_devices;
  const int sm_count = have_dev ? d.props[dev].num_sms : 0;
  const float bps = sm_count == 0 ? __int_as_float(0x7f800000) : __fdiv_rn(__int2float_rn(grid_prod), __int2float_rn(sm_count));
  const float wps = __fdiv_rn(__fmul_rn(bps, __int2float_rn(block_prod)), 32.0f);
  cudaOccResult occ;
  float occupancy;
  occupancy_metrics(d, dev, have_dev, sm_count, grid_prod, block_prod, regs, ssm, dsm, &occ, &occupancy);
  s32(a, KS_PCT, (uint32_t)(int32_t)llround(__dmul_rn((double)occupancy, 100.0)));
  s32(a, KS_ACTIVE, (uint32_t)occ.activeBlocksPerMultiprocessor); s32(a, KS_LIMIT, (uint32_t)(CS_LIMIT + (int)(occ.limitingFactors & 31u)));
  s32(a, KS_LREGS, (uint32_t)occ.blockLimitRegs); s32(a, KS_LSMEM, (uint32_t)occ.blockLimitSharedMem);
  s32(a, KS_LWARPS, (uint32_t)occ.blockLimitWarps); s32(a, KS_LBLOCKS, (uint32_t)occ.blockLimitBlocks);
  s32(a, KS_LBARR, (uint32_t)occ.blockLimitBarriers); s32(a, KS_AREGS, (uint32_t)occ.allocatedRegistersPerBlock);
  s64(a, KS_ASMEM, (uint64_t)occ.allocatedSharedMemPerBlock);
  s64(a, KS_BPS, (uint64_t)__double_as_longlong((double)bps)); s64(a, KS_WPS, (uint64_t)__double_as_longlong((double)wps));
  s64(a, KS_TS, (uint64_t)rel_ts(d, ts)); s64(a, KS_DUR, (uint64_t)(dur < 0 ? 0 : dur));
  s32(a, KS_REGS, regs); s32(a, KS_SMEM, (uint32_t)ssm + (uint32_t)dsm); s32(a, KS_EXT, (uint32_t)ext);
  uint64_t p = ((1ull << K_COUNT) - 1ull) & ~(1ull << K_COLL);  // every field except the optional ones below
  if (!has_ext) p &= ~((1ull << K_EXT) | (1ull << K_EXTC));
  else if (d.has_comms != nullptr && (*d.has_comms & 1u) != 0u) {
    // a kernel launched by a record_param_comms op carries that op's collective metadata (output_json.cpp:900-906)
    // (one shard: the op the join found; several: the join's table holds positions in the gathered keys, and the
    // collective ops of this shard's rows and of the guest rows have a table of their own)
    const uint32_t row = d.coll_tab != nullptr ? tab_find(d.coll_tab, d.coll_mask, (uint32_t)ext) : tab_find(d.op_tab, d.op_mask, (uint32_t)ext);
    if (row < d.n_ops && d.op_name[row] < d.n_strings && d.str_class[d.op_name[row]] == 1u) {
      p |= 1ull << K_COLL; s32(a, KS_COLLROW, row);
      if (counting && d.coll_list != nullptr) d.coll_list[atomicAdd(&d.counters->n_coll, 1ull)] = (uint32_t)t.work;  // for the extra emit launch
    }
  }
  t.x++;
  if (corr > 0) t.flow++;
  else p &= ~((1ull << K_FLOW) | (1ull << K_FPID) | (1ull << K_FTID) | (1ull << K_FTS) | (1ull << K_FEND));
  if (counting && d.seen_tab != nullptr) seen_insert(d, dev, stream);
  if (counting && d.span_key != nullptr) span_update(span_args(d), corr, dev, stream, ts, dur, t.ev);
  return p;
}

// memcpy / memcpy2 / memset records (libkineto/src/CuptiActivity.h:586-712)
template <int CLS>
__device__ __forceinline__ uint64_t gather_mem(const Dev& d, uint32_t* a, Tally& t, uint32_t* filt, bool counting, int32_t* ext_io) {
  const uint64_t st = a64(a, 16), en = a64(a, 24);
  const int64_t ts = conv_ts(d, st), dur = conv_dur(d, st, en);
  if (out_of_range(d, ts, dur)) { *filt = 2; return 0; }
  const uint64_t bytes = a64(a, MR_BYTES);
  const uint32_t dev = a32(a, MR_DEV), stream = a32(a, MR_STREAM);
  constexpr int g = CLS == C_MEMCPY2 ? 8 : 0;  // byte shift of the trailing fields in the peer-to-peer layout
  const uint32_t corr = a32(a, CLS == C_MEMCPY2 ? 60 : 44);
  int32_t ext = *ext_io;
  if (counting) { linked_op(d, corr, linked_op_peek(d, corr), &ext); *ext_io = ext; }
  const bool has_ext = ext != 0;
  const uint32_t w1 = a32(a, 4);
  const uint64_t node = a64(a, 64 + g);
  const uint32_t graph = a32(a, 72 + g), chan = a32(a, 76 + g), chtype = a32(a, 80 + g);
  if (CLS == C_MEMSET) {
    const uint32_t k = a32(a, 48) >> 16;  // memoryKind: 16 bits at byte 50
    s32(a, MS_KIND0, CS_MEMORY_KIND + (k <= 7 ? k : 8));
  } else {
    const uint32_t k0 = w1 & 0xffu, k1 = (w1 >> 8) & 0xffu, k2 = (w1 >> 16) & 0xffu;  // copyKind, srcKind, dstKind
    s32(a, MS_KIND0, CS_MEMCPY_KIND + (k0 <= 10 ? k0 : 11));
    s32(a, MS_KIND1, CS_MEMORY_KIND + (k1 <= 7 ? k1 : 8));
    s32(a, MS_KIND2, CS_MEMORY_KIND + (k2 <= 7 ? k2 : 8));
  }
  s64(a, MS_TS, (uint64_t)rel_ts(d, ts)); s64(a, MS_DUR, (uint64_t)(dur < 0 ? 0 : dur));
  s32(a, MS_EXT, (uint32_t)ext); s32(a, MS_CORR, corr);
  s32(a, MS_GRAPH, graph); s64(a, MS_NODE, node); s32(a, MS_CHAN, chan); s32(a, MS_CHTYPE, chtype);
  uint64_t p = 0;
  auto on = [&](int f) { p |= 1ull << f; };
  if (CLS == C_MEMSET) on(M_SET_KIND); else { on(M_CPY_KIND); on(M_CPY_SRC); on(M_CPY_DST); }
  on(M_PID); on(M_TID); on(M_TS); on(M_DUR); on(M_ARGS);
  if (has_ext) { on(M_EXT); on(M_EXTC); }
  if (CLS == C_MEMCPY2) { on(M_FROMDEV); on(M_INDEV); on(M_TODEV); on(M_FROMCTX); on(M_INCTX); on(M_TOCTX); }
  else { on(M_DEV); on(M_CTX); }
  on(M_STREAM); on(M_CORR); on(M_BYTES);
  if (dur != 0) {  // addBandwidthTypedMetadata, CuptiActivity.h:460-470
    on(M_BW);
    s64(a, MS_BW, (uint64_t)__double_as_longlong(__ddiv_rn(__ull2double_rn(bytes), __ll2double_rn(dur))));
  }
  on(M_GRAPH); on(M_NODE); on(M_CHAN); on(M_CHTYPE); on(M_CLOSE);
  t.x++;
  if (corr > 0) { on(M_FLOW); on(M_FPID); on(M_FTID); on(M_FTS); on(M_FEND); t.flow++; }
  if (counting && d.seen_tab != nullptr) seen_insert(d, dev, stream);
  if (counting && d.span_key != nullptr) span_update(span_args(d), corr, dev, stream, ts, dur, t.ev);
  return p;
}

// handleOverheadActivity (libkineto/src/CuptiActivityProfiler.cpp:360-377) with OverheadActivity
// (libkineto/src/CuptiActivity.h:144-179, names libkineto/src/cupti_strings.cpp:68-97): device -1, resource 0,
// no correlation id, no metadata, no flow.  The event has the shape of a CPU-side activity without
// arguments, so it uses that field program with a constant-string name.
__device__ __forceinline__ uint64_t gather_overhead(const Dev& d, uint32_t* a, Tally& t, uint32_t* filt) {
  const uint32_t kind = a32(a, 4);
  const uint64_t st = a64(a, 24), en = a64(a, 32);
  const int64_t ts = conv_ts(d, st), dur = conv_dur(d, st, en);
  if (out_of_range(d, ts, dur)) { *filt = 2; return 0; }
  uint32_t idx = 10;  // "Unrecognized"
  if (kind <= 1u) idx = kind;
  else if ((kind & 0xffffu) == 0u && (kind >> 16) >= 1u && (kind >> 16) <= 7u) idx = 1u + (kind >> 16);
  else if (kind == 0x7fffffffu) idx = 9;
  s32(a, OS_CAT, (uint32_t)(CS_TYPE + 11)); s32(a, OS_NAME, (uint32_t)CS_OVERHEAD + idx); s32(a, OS_PID, 0xFFFFFFFFu);
  s32(a, OS_EXT, 0u); s64(a, OS_TID, 0ull); s64(a, OS_TS, (uint64_t)rel_ts(d, ts)); s64(a, OS_DUR, (uint64_t)(dur < 0 ? 0 : dur));
  t.x++;
  return (1ull << O_CAT) | (1ull << O_CNAME) | (1ull << O_PID) | (1ull << O_TID) | (1ull << O_TS) | (1ull << O_DUR) |
         (1ull << O_PAD) | (1ull << P_CLOSE);
}

// Reads a synchronisation or CUDA event record into registers (the two layouts differ).
struct SyncFields { uint32_t type, corr, ctx, stream, event; uint64_t start, end; };
template <int CLS> __device__ __forceinline__ SyncFields sync_fields(const uint32_t* a) {
  SyncFields f;
  if (CLS == C_CUDAEVENT) {  // CUpti_ActivityCudaEvent2: the device timestamp is the start, the duration is 1 ns
    f.type = 0; f.corr = a32(a, 4); f.ctx = a32(a, 8); f.stream = a32(a, 12); f.event = a32(a, 16); f.start = a64(a, 40); f.end = 0;
  } else {
    f.type = a32(a, 4); f.start = a64(a, 8); f.end = a64(a, 16); f.corr = a32(a, 24); f.ctx = a32(a, 28); f.stream = a32(a, 32);
    f.event = a32(a, 36);
  }
  return f;
}
// handleCudaSyncActivity / handleCudaEventActivity (libkineto/src/CuptiActivityProfiler.cpp:404-500) with
// CudaSyncActivity / CudaEventActivity (libkineto/src/CuptiActivity.h:325-411).  A deferred record (C_WAIT) is
// dropped, before the window check, when its stream showed no GPU work (logDeferredEvents, :502-514).
template <int CLS>
__device__ __forceinline__ uint64_t gather_sync(const Dev& d, uint32_t* a, Tally& t, uint32_t* filt, bool counting, int32_t* ext_io) {
  const SyncFields f = sync_fields<CLS>(a);
  const uint32_t dev = ctx_device(d, f.ctx);
  if (CLS == C_WAIT && counting &&
      (d.seen_tab == nullptr || set64_slot(d.seen_tab, d.seen_mask, dev_stream_key(dev, f.stream), false) == 0xFFFFFFFFu))
    return 0;
  const int64_t ts = conv_ts(d, f.start), dur = CLS == C_CUDAEVENT ? 1 : conv_dur(d, f.start, f.end);
  if (out_of_range(d, ts, dur)) { *filt = 2; return 0; }
  int32_t ext = *ext_io;
  if (counting) {  // "External id": the linked op's id, else the record's own correlation id (output_json.cpp:871-895)
    int32_t id = 0;
    ext = linked_op_full(d, f.corr, &id) ? id : (int32_t)f.corr;
    *ext_io = ext;
  }
  const bool event_sync = CLS != C_CUDAEVENT && (f.type == 1u || f.type == 2u);  // isEventSync, CuptiActivity.h:308-312
  int64_t tid = (int64_t)(int32_t)f.stream;  // streamIdForTrace: "no stream" shows as -1
  uint64_t p = 0;
  auto on = [&](int fl) { p |= 1ull << fl; };
  if (CLS == C_SYNC && f.type == 3u) {  // a stream sync: own row, announced once
    tid += 1000000;  // kSyncStreamTidOffset, output_json.h:237
    s64(a, YS_ROWTID, (uint64_t)tid);
    const uint32_t slot = d.row_key != nullptr ? set64_slot(d.row_key, d.row_mask, dev_stream_key(dev, f.stream), false) : 0xFFFFFFFFu;
    if (slot != 0xFFFFFFFFu && d.row_first[slot] == (uint32_t)t.ev) {
      on(Y_MROW1); on(Y_MPID1); on(Y_MTID1); on(Y_MNAME); on(Y_MROW2); on(Y_MPID2); on(Y_MTID2); on(Y_MSORT); on(Y_MEND);
    }
  }
  if (event_sync) {
    int32_t src_stream = -1, src_corr = -1;
    wait_event_find(d, f.ctx, f.event, f.corr, &src_stream, &src_corr);
    s32(a, YS_SRCSTREAM, (uint32_t)src_stream); s32(a, YS_SRCCORR, (uint32_t)src_corr);
  }
  s64(a, YS_TS, (uint64_t)rel_ts(d, ts)); s64(a, YS_DUR, (uint64_t)(dur < 0 ? 0 : dur));
  s32(a, YR_CORR, f.corr); s32(a, YR_CTX, f.ctx); s32(a, YS_STREAM, f.stream); s32(a, YR_EVENT, f.event);
  s32(a, YS_PID, dev); s32(a, YS_EXT, (uint32_t)ext); s64(a, YS_TID, (uint64_t)abs_tid(tid));
  s32(a, YS_NAME, (uint32_t)CS_SYNC + (f.type >= 1u && f.type <= 4u ? f.type : 0u));
  on(CLS == C_CUDAEVENT ? Y_HEAD_EVENT : Y_HEAD_SYNC); on(Y_PID); on(Y_TID); on(Y_TS); on(Y_DUR); on(Y_ARGS);
  if (ext != 0) { on(Y_EXT); on(Y_EXTC); }
  if (CLS == C_CUDAEVENT) { on(Y_EVENTID); on(Y_STREAM_A); }
  else {
    on(Y_KIND);
    if (event_sync) { on(Y_WSTREAM); on(Y_WCORR); on(Y_WEVENT); on(Y_STREAM_A); } else on(Y_STREAM_B);
  }
  on(Y_CORR); on(Y_DEV); on(Y_CTX); on(Y_CLOSE);
  t.x++;
  if (f.corr > 0) { on(Y_FLOW); on(Y_FPID); on(Y_FTID); on(Y_FTS); on(Y_FEND); t.flow++; }
  return p;
}
// Which stream sync comes first on its row, in emission order: the smallest event number per (device, stream)
// among the stream syncs that are logged.
__global__ void k_sync_rows(Dev d) {
  const uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= d.cls_count[C_SYNC]) return;
  const uint64_t i = d.cls_begin[C_SYNC] + j;
  const uint32_t* r = reinterpret_cast<const uint32_t*>(d.cupti + (uint64_t)d.work_slot[i] * 8);
  if (r[1] != 3u) return;
  const uint64_t st = (uint64_t)r[2] | ((uint64_t)r[3] << 32), en = (uint64_t)r[4] | ((uint64_t)r[5] << 32);
  if (out_of_range(d, conv_ts(d, st), conv_dur(d, st, en))) return;
  const uint32_t slot = set64_slot(d.row_key, d.row_mask, dev_stream_key(ctx_device(d, r[7]), r[8]), true);
  if (slot == 0xFFFFFFFFu) { atomicAdd(&d.counters->device_check, 1ull); return; }
  atomicMin(&d.row_first[slot], d.work_ev[i]);
}

// ---- what other shards of a trace need from this one for their synchronisation and CUDA event records ----
// The reference fills its lookup maps from the whole trace before it logs anything (buildProcessingState,
// CuptiActivityProfiler.cpp:256-302; seenDeviceStreams_ and the once-per-row metadata during logging).  A shard's part
// of those maps is carried by a few of its own records, exported verbatim: per context the first kernel / copy /
// memset record (ctxToDeviceId), per (device, stream) the first such record inside the window (seenDeviceStreams_),
// per (context, stream) the first stream synchronisation inside the window (the row announcement), and every CUDA
// event record (waitEventMap).  k_export_select finds the per-key first records (smallest slot), k_export_list
// gathers their slots and sizes, the host orders them, k_export_copy writes the records.
__global__ void k_export_select(Dev d, unsigned long long* pair_key, uint32_t* pair_first, unsigned long long* sync_key, uint32_t* sync_first,
                                uint32_t mask) {
  const uint64_t i = d.cls_begin[C_KERNEL] + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.cls_begin[C_SYNC] + d.cls_count[C_SYNC]) return;
  int cls = C_KERNEL;
#pragma unroll
  for (int c = C_MEMCPY; c <= C_SYNC; c++) if (i >= d.cls_begin[c]) cls = c;
  if (i - d.cls_begin[cls] >= d.cls_count[cls] || (cls > C_MEMSET && cls != C_SYNC)) return;  // padding, other classes
  const uint32_t slot = d.work_slot[i];
  const uint32_t* r = reinterpret_cast<const uint32_t*>(d.cupti + (uint64_t)slot * 8);
  unsigned long long key;
  uint64_t st, en;
  if (cls == C_SYNC) {
    if (r[1] != 3u) return;  // stream synchronisations only
    st = (uint64_t)r[2] | ((uint64_t)r[3] << 32); en = (uint64_t)r[4] | ((uint64_t)r[5] << 32);
    key = dev_stream_key(r[7], r[8]);  // (context, stream): the device is only known once all shards' contexts are
  } else {
    st = (uint64_t)r[4] | ((uint64_t)r[5] << 32); en = (uint64_t)r[6] | ((uint64_t)r[7] << 32);
    key = cls == C_KERNEL ? dev_stream_key(r[10], r[12]) : dev_stream_key(r[8], r[10]);  // (device, stream)
  }
  if (out_of_range(d, conv_ts(d, st), conv_dur(d, st, en))) return;
  unsigned long long* keys = cls == C_SYNC ? sync_key : pair_key;
  const uint32_t at = set64_slot(keys, mask, key, true);
  if (at == 0xFFFFFFFFu) { atomicAdd(&d.counters->device_check, 1ull); return; }
  atomicMin(&(cls == C_SYNC ? sync_first : pair_first)[at], slot);
}
// One thread per table slot of the three tables: the slot and the length of every record to export.
__global__ void k_export_list(Dev d, const unsigned long long* pair_key, const uint32_t* pair_first, const unsigned long long* sync_key,
                              const uint32_t* sync_first, uint32_t mask, unsigned long long* list, uint32_t* n_list, uint32_t cap) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  uint32_t slot = 0xFFFFFFFFu;
  if (i <= d.ctx_mask) { const unsigned long long e = d.ctx_tab[i]; if (e != 0) slot = (uint32_t)e - 1u; }
  else if (i - (d.ctx_mask + 1u) <= mask) { const uint32_t j = i - (d.ctx_mask + 1u); if (pair_key[j] != 0) slot = pair_first[j]; }
  else if (i - (d.ctx_mask + 1u) - (mask + 1u) <= mask) { const uint32_t j = i - (d.ctx_mask + 1u) - (mask + 1u); if (sync_key[j] != 0) slot = sync_first[j]; }
  if (slot == 0xFFFFFFFFu) return;
  const uint32_t* r = reinterpret_cast<const uint32_t*>(d.cupti + (uint64_t)slot * 8);
  const uint32_t len = (slot_code(r[0], r[1]) & 31u) * 8u;
  const uint32_t at = atomicAdd(n_list, 1u);
  if (at < cap) list[at] = ((unsigned long long)slot << 32) | len;
}
// `list`: (slot << 32 | byte offset in dst) per record, lengths from the records' kinds; then the CUDA event records.
__global__ void k_export_copy(Dev d, const unsigned long long* list, uint32_t n_list, uint8_t* dst, uint64_t events_at) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t* src;
  uint64_t* out;
  if (i < n_list) {
    src = reinterpret_cast<const uint64_t*>(d.cupti + (list[i] >> 32) * 8);
    out = reinterpret_cast<uint64_t*>(dst + (uint32_t)list[i]);
  } else if (i - n_list < d.cls_count[C_CUDAEVENT]) {
    src = reinterpret_cast<const uint64_t*>(d.cupti + (uint64_t)d.work_slot[d.cls_begin[C_CUDAEVENT] + (i - n_list)] * 8);
    out = reinterpret_cast<uint64_t*>(dst + events_at + (i - n_list) * 56u);
  } else return;
  const uint32_t* r = reinterpret_cast<const uint32_t*>(src);
  const uint32_t words = slot_code(r[0], r[1]) & 31u;
  for (uint32_t k = 0; k < words; k++) out[k] = src[k];
}

// CPU-side activity: ChromeTraceLogger::handleActivity for a GenericTraceActivity (output_json.cpp:837-963)
__device__ __forceinline__ uint64_t gather_op(const Dev& d, uint64_t i, uint32_t* a, Tally& t) {
  if (i >= d.n_ops - d.n_guest_ops) return 0;  // a guest row: looked up, never logged
  const int32_t type = d.op_type[i];
  if ((uint32_t)type >= 29u) { atomicAdd(&d.counters->device_check, 1ull); return 0; }
  if (!((d.type_mask >> type) & 1u)) return 0;  // type not selected: joins, but is not logged
  if (type == 17 || type == 26 || type == 28) {  // counter events: handleCounterEvent, output_json.cpp:679-716 (no duration, no flow, raw text)
    s32(a, OS_CAT, (uint32_t)(CS_TYPE + type)); s32(a, OS_NAME, d.op_name[i]); s32(a, OS_PID, (uint32_t)op_pid(d, d.op_device[i]));
    s64(a, OS_TID, (uint64_t)abs_tid(d.op_resource[i])); s64(a, OS_TS, (uint64_t)rel_ts(d, d.op_start[i])); s32(a, OS_ROW, (uint32_t)i);
    if (type == 28) {  // HARDWARE_COUNTERS: one event per counter value, on a track named after the device
      bool any = false;
      for (uint32_t e = d.op_mdoff[i]; e < d.op_mdoff[i + 1]; e++) any = any || d.md[e].type == 6u;
      return any ? (1ull << H_ALL) : 0ull;
    }
    return (1ull << C_HEAD) | (1ull << C_NAME) | (1ull << O_PID) | (1ull << O_TID) | (1ull << O_TS) | (1ull << O_ARGS) | (1ull << C_MD) |
           (1ull << P_ARGS_CLOSE) | (1ull << P_CLOSE);
  }
  if (type == 9) {  // CPU_INSTANT_EVENT: handleGenericInstantEvent, output_json.cpp:660-676 (no duration, no flow, raw text)
    s32(a, OS_CAT, (uint32_t)(CS_TYPE + type)); s32(a, OS_NAME, d.op_name[i]); s32(a, OS_PID, (uint32_t)op_pid(d, d.op_device[i]));
    s64(a, OS_TID, (uint64_t)abs_tid(d.op_resource[i])); s64(a, OS_TS, (uint64_t)rel_ts(d, d.op_start[i])); s32(a, OS_ROW, (uint32_t)i);
    uint64_t pi = (1ull << I_HEAD) | (1ull << I_NAME) | (1ull << O_PID) | (1ull << O_TID) | (1ull << O_TS) | (1ull << O_PAD) | (1ull << P_CLOSE);
    if (d.op_mdoff[i + 1] > d.op_mdoff[i]) pi |= (1ull << O_ARGS) | (1ull << I_MD) | (1ull << P_ARGS_CLOSE);
    t.x++;
    return pi;
  }
  int64_t ts = d.op_start[i];
  int64_t dur = d.op_end[i] - ts;
  // an activity that had not ended when the trace stopped ends with the capture window (processCpuTrace,
  // GenericActivityProfiler.cpp:255-258; its "finished": false entry is part of its metadata like any other)
  if (dur < 0 && (d.flags & 8)) dur = d.win_end - ts;
  if (dur < 0) dur = 0;
  const int64_t flow_ts = ts;
  if (type == 2) { ts -= 1; dur += 2; }  // GPU_USER_ANNOTATION, output_json.cpp:862-869
  // External id, output_json.cpp:871-895: no linked activity on this path; excluded types print none.
  int32_t ext = 0;
  const bool excluded = type == 3 || type == 4 || type == 5 || type == 7 || type == 8 || type == 21 || type == 22 || type == 24 || type == 25;
  if (!excluded) ext = d.op_id[i];
  const bool has_md = d.op_mdoff[i + 1] > d.op_mdoff[i];
  const bool has_args = ext != 0 || has_md;
  const uint32_t flow = d.op_flow[i];
  s32(a, OS_CAT, (uint32_t)(CS_TYPE + type)); s32(a, OS_NAME, d.op_name[i]); s32(a, OS_PID, (uint32_t)op_pid(d, d.op_device[i]));
  s32(a, OS_EXT, (uint32_t)ext); s64(a, OS_TID, (uint64_t)abs_tid(d.op_resource[i]));
  s64(a, OS_TS, (uint64_t)rel_ts(d, ts)); s64(a, OS_DUR, (uint64_t)dur); s32(a, OS_ROW, (uint32_t)i); s32(a, OS_FLOW, flow);
  s64(a, OS_FTS, (uint64_t)rel_ts(d, flow_ts));
  uint64_t p = 0;
  auto on = [&](int f) { p |= 1ull << f; };
  on(O_CAT); on(O_NAME); on(O_PID); on(O_TID); on(O_TS); on(O_DUR); on(O_PAD);
  if (has_args) on(O_ARGS);
  if (ext != 0) { on(O_EXT); if (has_md) on(O_EXTC); }
  if (has_md) on(O_MD);
  if (has_args) on(P_ARGS_CLOSE);
  on(P_CLOSE);
  t.x++;
  const uint32_t ft = d.op_flowt[i] & 0xfu;
  if (flow > 0 && (ft == 1u || ft == 2u)) {  // handleGenericLink, output_json.cpp:973-995
    const bool start = (d.op_flowt[i] >> 4) & 1u;
    on(start ? P_FLOW_S : P_FLOW_F); on(P_FPID); on(P_FTID); on(P_FTS); on(ft == 1u ? P_FWDBWD : P_AC2G);
    if (!start) on(P_FBP);
    on(P_FEND);
    t.flow++;
  }
  return p;
}

// ChromeTraceLogger::appendCollectiveArgs (libkineto/src/output_json.cpp:718-801) for the CPU op in row `row`: the
// op's metadata values rendered as metadataValueToString does (libkineto/src/GenericTraceActivity.cpp:20-47), string
// values with one surrounding pair of quotes stripped where the reference strips it, nothing sanitised.  Every
// entry is written as ,"key": value (ArgsBuilder::addRaw / addQuoted, :161-170).
constexpr uint32_t kCollStrip = 0x0FF1u;   // keys whose string value loses one surrounding pair of quotes (and is quoted again)
// The op's entry for key k, or 0xFFFFFFFF.
__device__ __forceinline__ uint32_t coll_entry(const Dev& d, uint32_t row, uint32_t k) {
  uint32_t found = 0xFFFFFFFFu;
  for (uint32_t e = d.op_mdoff[row], m1 = d.op_mdoff[row + 1]; e < m1; e++) {
    const uint32_t key = d.md[e].key;
    if (key < d.n_strings && d.str_class[key] == 2u + k) found = e;
  }
  return found;
}
// [begin, end) of a string value in the pool, one surrounding pair of quotes stripped on request.
__device__ __forceinline__ void coll_text(const Dev& d, uint32_t id, bool strip, uint64_t* b, uint64_t* e) {
  uint64_t lo = 0, hi = 0;
  if (id < d.n_strings) { lo = d.pool_off[id]; hi = d.pool_off[id + 1]; }
  if (strip && hi - lo >= 2 && d.pool_data[lo] == '"' && d.pool_data[hi - 1] == '"') { lo++; hi--; }
  *b = lo; *e = hi;
}
// Bit k set: key k is written.  Numbers and booleans are never empty; a string is empty when nothing is left of it.
// The first five keys are written together or not at all, and so are the two split sizes.
// *ents: four bits per key, the entry's position among the op's entries (15: look it up again).
__device__ __forceinline__ uint32_t coll_mask(const Dev& d, uint32_t row, uint64_t* ents) {
  uint32_t mask = 0;
  uint64_t packed = 0;
  const uint32_t e0 = d.op_mdoff[row];
  for (uint32_t e = e0, m1 = d.op_mdoff[row + 1]; e < m1; e++) {
    const MdEntry md = d.md[e];
    const uint32_t cls = md.key < d.n_strings ? d.str_class[md.key] : 0u;
    if (cls < 2u) continue;
    const uint32_t k = cls - 2u;
    bool nonempty = true;
    if (md.type >= 4u) { uint64_t b, e2; coll_text(d, (uint32_t)md.value, (kCollStrip >> k) & 1u, &b, &e2); nonempty = e2 > b; }
    mask = nonempty ? (mask | (1u << k)) : (mask & ~(1u << k));
    const uint64_t pos = e - e0 < 15u ? e - e0 : 15u;
    packed = (packed & ~(15ull << (4 * k))) | (pos << (4 * k));
  }
  *ents = packed;
  if ((mask & 0x1Fu) != 0x1Fu) mask &= ~0x1Fu;
  if ((mask & 0x180u) != 0x180u) mask &= ~0x180u;
  return mask;
}

// The counter values of the CPU-side activity in row `row` (metadata entries of type 6: name, double).
// handleCounterEvent (libkineto/src/output_json.cpp:679-716): MTIA_COUNTERS / XPU_SCOPE_PROFILER print them as one
// argument list, "name": value joined by commas; HARDWARE_COUNTERS prints one whole event per value, named after
// the counter, on the track "GPU <device> Counters", its single argument named "".  Values are fmt's "{}" of the
// double, names are copied as they are.
template <class S> __device__ __forceinline__ void put_cstr(S& s, uint32_t index) {
  const FieldDesc cs = g_fields.f[CSTR_BASE + index];
  s.words(g_fields.w + cs.off, cs.len);
}
template <class S>
__device__ __forceinline__ void put_counters(S& s, const Dev& d, uint32_t row, bool hw) {
  bool first = true;
  for (uint32_t e = d.op_mdoff[row], m1 = d.op_mdoff[row + 1]; e < m1; e++) {
    const MdEntry md = d.md[e];
    if (md.type != 6u) continue;
    uint64_t b = 0, e2 = 0;
    coll_text(d, md.key, false, &b, &e2);
    const double x = __longlong_as_double((long long)md.value);
    s.ensure(48);
    if (hw) {
      put_cstr(s, CS_HWC + 0); s.bytes(d.pool_data + b, (uint32_t)(e2 - b));
      put_cstr(s, CS_HWC + 1); s.ensure(48); put_sdec(s, (int64_t)op_pid(d, d.op_device[row]));
      put_cstr(s, CS_HWC + 2); s.ensure(48); put_sdec(s, abs_tid(d.op_resource[row]));
      put_cstr(s, CS_HWC + 3); s.ensure(48); put_ts2(s, rel_ts(d, d.op_start[row]));
      put_cstr(s, CS_HWC + 4); s.ensure(48);
      if (double_is_finite(x)) put_double(s, x); else put_nonfinite(s, x);
      put_cstr(s, CS_HWC + 5);
    } else {
      if (!first) put_char(s, ',');
      put_char(s, '"'); s.bytes(d.pool_data + b, (uint32_t)(e2 - b)); s.put(0x203A22u, 3);  // "\": "
      s.ensure(48);
      if (double_is_finite(x)) put_double(s, x); else put_nonfinite(s, x);
    }
    first = false;
  }
}

// The value that follows a field's literal.  T_MD (CPU-side activities only) formats the typed metadata
// entries of the op (JsonTypedMetadataVisitor, libkineto/include/TypedMetadataJson.h:72-158): each entry
// is mapped onto one of the value types, so the kernel holds one copy of every formatter.
enum : int { T_BOOL = 8, T_MDSTR, T_QMDSTR };
// ENSURE = false: the caller has asked the sink for room for a number; fields that loop over entries or copy
// strings still ask for themselves.
template <class S, bool COLL = true, bool ENSURE = true>
__device__ __forceinline__ void put_value(S& s, const Dev& d, int type, uint64_t v, unsigned long long* name_bytes) {
  if (type == T_NONE) return;
  if (COLL && (type == T_MDCNT || type == T_HWC)) { put_counters(s, d, (uint32_t)v, type == T_HWC); return; }
  // Two field types loop over the entries of a CPU-side activity: its own metadata (T_MD) and the collective keys
  // copied onto a kernel (T_COLL).  Every other type takes the switch once.
  uint32_t e = 0, m1 = 0, m0 = 0, cmask = 0;
  uint64_t cents = 0;
  const bool coll = COLL && type == T_COLL, raw_md = COLL && type == T_MDRAW;
  const bool md_mode = type == T_MD || coll || raw_md;
  if (md_mode) {
    if (!coll) { m0 = e = d.op_mdoff[v]; m1 = d.op_mdoff[v + 1]; if (e >= m1) return; }
    else { m0 = (uint32_t)v; cmask = coll_mask(d, m0, &cents); if (!cmask) return; m1 = d.op_mdoff[m0]; }
  }
  bool more = false, close_quote = false;
  do {
    if (ENSURE || md_mode) s.ensure(48);  // a number takes at most 24 bytes; quotes and separators around it come out of the sink's slack
    if (md_mode) {
      if (!coll) {
        close_quote = false;
        const MdEntry md = d.md[e];
        if (e > m0) s.put(0x202Cu, 2);  // ", "
        put_char(s, '"');
        if (raw_md) { uint64_t b, e2; coll_text(d, md.key, false, &b, &e2); s.bytes(d.pool_data + b, (uint32_t)(e2 - b)); }
        else put_mdstr(s, d, md.key);
        s.put(0x203A22u, 3);  // "\": "
        v = md.value;
        type = md.type == 0 ? T_I64 : md.type == 1 ? T_U64 : md.type == 2 ? T_DBL : md.type == 3 ? T_BOOL : md.type == 4 ? T_QMDSTR : T_MDSTR;
        if (raw_md && md.type >= 4u) { type = T_RAWSTR; close_quote = md.type == 4u; if (close_quote) put_char(s, '"'); }
        more = ++e < m1;
      } else {  // the next collective key: its literal, then the op's value through the formatters below
        const uint32_t k = (uint32_t)__ffs((int)cmask) - 1u;
        cmask &= cmask - 1u;
        const uint32_t pos = (uint32_t)(cents >> (4 * k)) & 15u;
        const MdEntry md = d.md[pos < 15u ? m1 + pos : coll_entry(d, m0, k)];
        const FieldDesc cs = g_fields.f[CSTR_BASE + CS_COLL + k];
        s.words(g_fields.w + cs.off, cs.len);
        close_quote = (kCollStrip >> k) & 1u;
        if (close_quote) put_char(s, '"');
        v = md.value;
        type = md.type == 0 ? T_I64 : md.type == 1 ? T_U64 : md.type == 2 ? T_DBL : md.type == 3 ? T_BOOL : close_quote ? T_RAWSTRIP : T_RAWSTR;
        more = cmask != 0u;
      }
    }
    switch (type) {
      case T_U64: case T_I64: case T_TS: {
        uint64_t mag = v;
        uint32_t fr = 0;
        if (type == T_I64 && (int64_t)v < 0) { put_char(s, '-'); mag = 0ull - v; }
        if (type == T_TS) { mag = v / 1000ull; fr = (uint32_t)(v - mag * 1000ull); }  // "{}.{:03}" of ns/1000, ns%1000
        put_dec(s, mag);
        if (type == T_TS) {
          if (S::kCounting) s.skip(4);
          else {
            const uint32_t x = (fr * 41u) >> 12, r = fr - x * 100u, y = (r * 103u) >> 10, z = r - y * 10u;
            s.put4(0x3030302Eu + (x << 8) + (y << 16) + (z << 24));
          }
        }
        break;
      }
      case T_DBL: {
        const double x = __longlong_as_double((long long)v);
        // a collective value is the plain text of the number ("inf", "-nan"), not the JSON visitor's quoted form
        if (COLL && coll && !double_is_finite(x)) put_nonfinite(s, x); else put_dbl(s, x);
        break;
      }
      case T_NAME: put_name(s, d, (uint32_t)v, name_bytes); break;
      case T_CSTR: { const FieldDesc cs = g_fields.f[CSTR_BASE + (uint32_t)v]; s.words(g_fields.w + cs.off, cs.len); break; }
      case T_BOOL: if (v) s.put4(0x65757274u); else s.put64(0x65736C6166ull, 5); break;  // true / false
      default: {  // T_MDSTR, T_QMDSTR, T_RAWSTR, T_RAWSTRIP
        if (type == T_QMDSTR) put_char(s, '"');
        if (COLL && type >= T_RAWSTR) {
          uint64_t b, e2;
          coll_text(d, (uint32_t)v, type == T_RAWSTRIP, &b, &e2);
          s.bytes(d.pool_data + b, (uint32_t)(e2 - b));
        } else put_mdstr(s, d, (uint32_t)v);
        if (type == T_QMDSTR || close_quote) put_char(s, '"');
        break;
      }
    }
    if (md_mode && close_quote && type < T_RAWSTR) put_char(s, '"');  // a quoted number (strings close their own quote)
  } while (md_mode && more);
}

// Emit pass: walks the set bits of `present`.  Descriptor and value of the NEXT field are fetched before
// the current one is formatted, so their latency hides behind the formatting work.
template <class S, bool COLL = true>
__device__ __forceinline__ void run_fields(S& s, const Dev& d, const uint32_t* a, int base, uint64_t present,
                                           unsigned long long* name_bytes) {
  if (!present) return;
  int f = __ffsll((long long)present) - 1;
  present &= present - 1;
  FieldDesc fd = g_fields.f[base + f];
  uint64_t v = slot_value(a, fd.voff, fd.vk);
  while (true) {
    const bool more = present != 0;
    FieldDesc fdn = fd;
    uint64_t vn = 0;
    if (more) {
      f = __ffsll((long long)present) - 1;
      present &= present - 1;
      fdn = g_fields.f[base + f];
      vn = slot_value(a, fdn.voff, fdn.vk);
    }
    s.words(g_fields.w + fd.off, fd.len);
    put_value<S, COLL>(s, d, fd.type, v, name_bytes);
    if (!more) break;
    fd = fdn; v = vn;
  }
}

// Size pass: the same fields as straight-line code.  Field types, literal lengths and value slots are
// compile-time constants here, so each present field costs its value's digit count and one addition.
constexpr int field_word_offset(int i) {  // position of field i's literal in g_fields.w (as make_prog lays it out)
  int w = 0;
  for (int f = 0; f < i; f++) w += (c_strlen(kAllFields[f].lit) + 7) / 8;
  return w;
}
constexpr uint32_t longest_constant_string() {  // among those a T_CSTR value can name (the counter-event pieces are written by put_counters)
  uint32_t m = 0;
  for (int f = CSTR_BASE; f < CSTR_BASE + CS_HWC; f++) if ((uint32_t)c_strlen(kAllFields[f].lit) > m) m = (uint32_t)c_strlen(kAllFields[f].lit);
  return m;
}
// Most bytes a field's value can take; 0xffff for values of any length (names, metadata entries), which ask the
// sink for room themselves.
constexpr uint32_t value_max_bytes(int type, int vk) {
  switch (type) {
    case T_NONE: return 0;
    case T_U64: return vk == VK_64 ? 20u : 10u;
    case T_I64: return vk == VK_64 ? 20u : 11u;
    case T_TS: return 24u;       // up to 20 digits, '.', three digits
    case T_DBL: return 26u;      // 24 characters of a finite value; a non-finite one is shorter, in quotes
    case T_CSTR: return longest_constant_string();
    default: return 0xffffu;
  }
}
template <int I> struct FieldInfo {
  static constexpr int type = kAllFields[I].type;
  static constexpr uint32_t len = (uint32_t)c_strlen(kAllFields[I].lit);
  static constexpr uint32_t voff = kAllFields[I].voff;
  static constexpr uint32_t vk = kAllFields[I].vk;
  static constexpr int woff = field_word_offset(I);
  static constexpr uint32_t vmax = value_max_bytes(kAllFields[I].type, kAllFields[I].vk);
};
template <int BASE, int F, int NF, class S>
__device__ __forceinline__ void count_fields(S& s, const Dev& d, const uint32_t* a, uint64_t present, unsigned long long* name_bytes) {
  if constexpr (F < NF) {
    if ((present >> F) & 1ull) {
      s.n += FieldInfo<BASE + F>::len;
      if constexpr (FieldInfo<BASE + F>::type != T_NONE)
        put_value(s, d, FieldInfo<BASE + F>::type, slot_value(a, FieldInfo<BASE + F>::voff, FieldInfo<BASE + F>::vk), name_bytes);
    }
    count_fields<BASE, F + 1, NF>(s, d, a, present, name_bytes);
  }
}
// Emit pass, hot record classes: the sink is asked for room once per group of fields whose longest possible text
// fits the group size, not once per field; the groups are fixed at compile time.
constexpr uint32_t kGroupBytes = 88;
static_assert(kGroupBytes + 32 + kWinSlack <= (uint32_t)kWinBytes, "a group must fit a window that has just been flushed");
// First field of a group?  (Walks the class's fields from its first one, as the field loop does.)
constexpr bool group_starts_at(int base, int first, int f) {
  uint32_t acc = 0xffffu;  // the first field always starts a group
  bool starts = true;
  for (int g = first; g <= f; g++) {
    const uint32_t v = value_max_bytes(kAllFields[base + g].type, kAllFields[base + g].vk);
    const uint32_t need = (uint32_t)c_strlen(kAllFields[base + g].lit) + (v == 0xffffu ? 0u : v);
    starts = acc == 0xffffu || acc + need > kGroupBytes;
    if (starts) acc = need; else acc += need;
    if (v == 0xffffu) acc = 0xffffu;  // after a value of any length the next field asks again
  }
  return starts;
}
// Bytes the group starting at field f can take (f starts a group).
constexpr uint32_t group_bytes_from(int base, int f, int nf) {
  uint32_t acc = 0;
  for (int g = f; g < nf; g++) {
    const uint32_t v = value_max_bytes(kAllFields[base + g].type, kAllFields[base + g].vk);
    const uint32_t need = (uint32_t)c_strlen(kAllFields[base + g].lit) + (v == 0xffffu ? 0u : v);
    if (g > f && acc + need > kGroupBytes) break;
    acc += need;
    if (v == 0xffffu) break;
  }
  return acc;
}
// Number formatting of the hot classes' field loop: one out-of-line copy of each formatter per kernel, so that a
// field costs a call instead of a copy of the formatter (with the formatters inlined the kernel is bound by
// instruction fetch).  The sink travels in registers: window, position and open word in, position
// and open word out; nothing here flushes, the caller has asked for the room.
__device__ __forceinline__ WindowSink sink_at(uint32_t* win, uint32_t pos, uint32_t carry) {
  WindowSink s;
  s.win = win; s.pos = pos; s.carry = carry; s.w0 = 0; s.head = 0; s.gbase = nullptr;
  return s;
}
__device__ __forceinline__ uint64_t sink_state(const WindowSink& s) { return (uint64_t)s.pos | ((uint64_t)s.carry << 32); }
__device__ __noinline__ uint64_t app_u64(uint32_t* win, uint32_t pos, uint32_t carry, uint64_t v) {
  WindowSink s = sink_at(win, pos, carry);
  put_dec(s, v);
  return sink_state(s);
}
__device__ __noinline__ uint64_t app_u32(uint32_t* win, uint32_t pos, uint32_t carry, uint32_t v) {
  WindowSink s = sink_at(win, pos, carry);
  if (v < 10000u) {
    const int n = 1 + (v >= 10u) + (v >= 100u) + (v >= 1000u);
    s.put(ascii4(v) >> (8 * (4 - n)), n);
  } else if (v < 100000000u) {
    const uint32_t hi = v / 10000u, lo = v - hi * 10000u;
    const int n = 1 + (hi >= 10u) + (hi >= 100u) + (hi >= 1000u);
    s.put64((uint64_t)(ascii4(hi) >> (8 * (4 - n))) | ((uint64_t)ascii4(lo) << (8 * n)), (uint32_t)(n + 4));
  } else {  // 9 or 10 digits
    const uint32_t hi = v / 100000000u, lo = v - hi * 100000000u;
    const int n = 1 + (hi >= 10u);
    s.put(ascii4(hi) >> (8 * (4 - n)), n);
    s.put64(ascii8(lo), 8u);
  }
  return sink_state(s);
}
__device__ __noinline__ uint64_t app_i32(uint32_t* win, uint32_t pos, uint32_t carry, int32_t v) {
  WindowSink s = sink_at(win, pos, carry);
  uint32_t mag = (uint32_t)v;
  if (v < 0) { put_char(s, '-'); mag = 0u - mag; }
  return app_u32(win, s.pos, s.carry, mag);
}
__device__ __noinline__ uint64_t app_i64(uint32_t* win, uint32_t pos, uint32_t carry, int64_t v) {
  WindowSink s = sink_at(win, pos, carry);
  put_sdec(s, v);
  return sink_state(s);
}
__device__ __noinline__ uint64_t app_ts(uint32_t* win, uint32_t pos, uint32_t carry, uint64_t ns) {
  WindowSink s = sink_at(win, pos, carry);
  put_ts2(s, (int64_t)ns);
  return sink_state(s);
}
__device__ __noinline__ uint64_t app_dbl(uint32_t* win, uint32_t pos, uint32_t carry, uint64_t bits) {
  WindowSink s = sink_at(win, pos, carry);
  put_dbl(s, __longlong_as_double((long long)bits));
  return sink_state(s);
}
// a constant string of the field table (at most longest_constant_string() bytes)
__device__ __noinline__ uint64_t app_cstr(uint32_t* win, uint32_t pos, uint32_t carry, uint32_t index) {
  WindowSink s = sink_at(win, pos, carry);
  const FieldDesc cs = g_fields.f[CSTR_BASE + index];
  const uint64_t* w = g_fields.w + cs.off;
  for (uint32_t k = 0; k < ((uint32_t)cs.len >> 3); k++) s.put8w(w[k]);
  const uint32_t rem = cs.len & 7u;
  if (rem) s.put64(w[cs.len >> 3], rem);  // the table pads with zero bytes
  return sink_state(s);
}
// Emit pass, the same fields as a loop: all lanes of a warp are at the same field at the same time, so the field's
// descriptor and the words of its literal are warp-uniform constant loads, the loop's body is small enough to stay
// in the instruction cache, and lanes whose event lacks a field sit out one iteration.  Descriptor (64 bits):
// literal word offset 0..11, literal length 12..19, operation 20..23, value slot offset 24..35, group bytes 36..43
// (non-zero: the field starts a group, see kGroupBytes), value type 44..49.
enum : uint32_t { OP_NONE = 0, OP_U32, OP_I32, OP_U64, OP_I64, OP_TS, OP_DBL, OP_CSTR, OP_OTHER };
constexpr uint32_t field_op(int type, int vk) {
  switch (type) {
    case T_NONE: return OP_NONE;
    case T_U64: return vk == VK_64 ? OP_U64 : OP_U32;
    case T_I64: return vk == VK_64 ? OP_I64 : (vk == VK_I32 ? OP_I32 : OP_U32);
    case T_TS: return OP_TS;
    case T_DBL: return OP_DBL;
    case T_CSTR: return OP_CSTR;
    default: return OP_OTHER;
  }
}
struct LoopDescs { uint64_t d[FIELD_COUNT]; };
constexpr void fill_class_descs(LoopDescs& t, int base, int nf) {
  for (int f = 0; f < nf; f++) {
    const FieldSrc& src = kAllFields[base + f];
    const uint64_t grp = group_starts_at(base, 0, f) ? group_bytes_from(base, f, nf) : 0;
    t.d[base + f] = (uint64_t)field_word_offset(base + f) | ((uint64_t)c_strlen(src.lit) << 12) | ((uint64_t)field_op(src.type, src.vk) << 20) |
                    ((uint64_t)src.voff << 24) | (grp << 36) | ((uint64_t)src.type << 44);  // type: 6 bits
  }
}
constexpr LoopDescs make_loop_descs() {
  LoopDescs t{};
  fill_class_descs(t, API_BASE, A_COUNT); fill_class_descs(t, KERNEL_BASE, K_COUNT); fill_class_descs(t, MEM_BASE, M_COUNT);
  fill_class_descs(t, OP_BASE, O_COUNT);
  return t;
}
constexpr uint32_t longest_group(const LoopDescs& t) {
  uint32_t m = 0;
  for (int f = 0; f < FIELD_COUNT; f++) if (((t.d[f] >> 36) & 0xffu) > m) m = (uint32_t)(t.d[f] >> 36) & 0xffu;
  return m;
}
// a field that is longer than a group on its own still has to fit behind the open block of a flushed window
static_assert(longest_group(make_loop_descs()) + 32 + 8 <= (uint32_t)kWinBytes && longest_group(make_loop_descs()) < 256, "group does not fit the window");
__constant__ LoopDescs g_loop = make_loop_descs();
template <int BASE, int NF>
__device__ __forceinline__ void loop_fields(WindowSink& s, const Dev& d, const uint32_t* a, uint64_t present, unsigned long long* name_bytes) {
#pragma unroll 1
  for (int f = 0; f < NF; f++) {
    const bool on = (present >> f) & 1ull;
    const uint64_t desc = g_loop.d[BASE + f];
    const uint32_t grp = (uint32_t)(desc >> 36) & 0xffu;
    if (grp != 0u) s.ensure(grp);  // also when no lane has the field: the group's other fields rely on it
    if (on) {
      const uint32_t len = (uint32_t)(desc >> 12) & 0xffu;
      if (len != 0u) {
        const uint64_t* w = g_fields.w + ((uint32_t)desc & 0xfffu);
        const uint32_t ph = s.pos & 3u, sft = ph << 3, nw = (len + 7u) >> 3;
        uint32_t* p = s.win + (s.pos >> 2) * (uint32_t)kWinStride;
        uint32_t c = s.carry, t0 = 0, t1 = 0;
#pragma unroll 1
        for (uint32_t k = 0; k < nw; k++) {  // whole words; the table pads every literal with zero bytes
          const uint64_t x = w[k];
          const uint32_t lo = (uint32_t)x, hi = (uint32_t)(x >> 32);
          t0 = c | (lo << sft); t1 = funnel_l(lo, hi, sft);
          p[0] = t0; p[kWinStride] = t1;
          c = funnel_l(hi, 0u, sft);
          p += 2 * kWinStride;
        }
        const uint32_t rem = len & 7u;  // bytes of the last word copied that belong to the literal (0: all eight)
        const uint32_t k = rem == 0u ? 2u : (ph + rem) >> 2;  // words that last copy completed
        s.carry = k == 0u ? t0 : (k == 1u ? t1 : c);
        s.pos += len;
      }
      const uint32_t op = (uint32_t)(desc >> 20) & 0xfu, voff = (uint32_t)(desc >> 24) & 0xfffu;
      if (op != OP_NONE) {
        uint64_t st;
        if (op == OP_U32) st = app_u32(s.win, s.pos, s.carry, a[voff >> 2]);
        else if (op == OP_I32) st = app_i32(s.win, s.pos, s.carry, (int32_t)a[voff >> 2]);
        else if (op == OP_TS) st = app_ts(s.win, s.pos, s.carry, reinterpret_cast<const uint64_t*>(a)[voff >> 3]);
        else if (op == OP_U64) st = app_u64(s.win, s.pos, s.carry, reinterpret_cast<const uint64_t*>(a)[voff >> 3]);
        else if (op == OP_CSTR) st = app_cstr(s.win, s.pos, s.carry, a[voff >> 2]);
        else if (op == OP_DBL) st = app_dbl(s.win, s.pos, s.carry, reinterpret_cast<const uint64_t*>(a)[voff >> 3]);
        else if (op == OP_I64) st = app_i64(s.win, s.pos, s.carry, (int64_t)reinterpret_cast<const uint64_t*>(a)[voff >> 3]);
        else {  // names, metadata entries: they ask the sink for room themselves
          put_value<WindowSink, false, true>(s, d, (int)((uint32_t)(desc >> 44) & 0x3fu), (uint64_t)a[voff >> 2], name_bytes);
          st = sink_state(s);
        }
        s.pos = (uint32_t)st; s.carry = (uint32_t)(st >> 32);
      }
    }
  }
}
constexpr int kEventThreads = 128;
constexpr size_t events_smem_bytes(bool write) {
  return (size_t)kEventThreads * kRecStride * 8 + (write ? ((size_t)kEventThreads * kWinWords + kWinPadWords) * 4 : 0);
}

// COLL (emit pass only): this launch writes the kernel events that carry collective metadata, and only those; the
// launch without it writes everything else and holds no code for them.  Returns false when the event is left to
// the other launch.
template <class S, bool COLL = true>
__device__ __forceinline__ bool format_event(S& s, const Dev& d, int cls, uint32_t* a, uint64_t j, Tally& t, uint32_t* filt, int32_t* ext) {
  unsigned long long* nb = &t.name_bytes;
  if constexpr (S::kCounting) {
    uint64_t p;
    switch (cls) {  // straight-line field code per class
      case C_API: if ((p = gather_api(d, a, t, filt, true, ext))) count_fields<API_BASE, 0, A_COUNT>(s, d, a, p, nb); break;
      case C_KERNEL: if ((p = gather_kernel(d, a, t, filt, true, ext))) count_fields<KERNEL_BASE, 0, K_COUNT>(s, d, a, p, nb); break;
      case C_MEMCPY: if ((p = gather_mem<C_MEMCPY>(d, a, t, filt, true, ext))) count_fields<MEM_BASE, 0, M_COUNT>(s, d, a, p, nb); break;
      case C_MEMCPY2: if ((p = gather_mem<C_MEMCPY2>(d, a, t, filt, true, ext))) count_fields<MEM_BASE, 0, M_COUNT>(s, d, a, p, nb); break;
      case C_MEMSET: if ((p = gather_mem<C_MEMSET>(d, a, t, filt, true, ext))) count_fields<MEM_BASE, 0, M_COUNT>(s, d, a, p, nb); break;
      case C_OVERHEAD: if ((p = gather_overhead(d, a, t, filt))) count_fields<OP_BASE, 0, O_COUNT>(s, d, a, p, nb); break;
      case C_SYNC: if ((p = gather_sync<C_SYNC>(d, a, t, filt, true, ext))) count_fields<SYNC_BASE, 0, Y_COUNT>(s, d, a, p, nb); break;
      case C_WAIT: if ((p = gather_sync<C_WAIT>(d, a, t, filt, true, ext))) count_fields<SYNC_BASE, 0, Y_COUNT>(s, d, a, p, nb); break;
      case C_CUDAEVENT: if ((p = gather_sync<C_CUDAEVENT>(d, a, t, filt, true, ext))) count_fields<SYNC_BASE, 0, Y_COUNT>(s, d, a, p, nb); break;
      default: if ((p = gather_op(d, j, a, t))) count_fields<OP_BASE, 0, O_COUNT>(s, d, a, p, nb); break;
    }
  } else {
    uint64_t p;
    int base;
    switch (cls) {  // one copy of the field loop for all classes
      case C_API: p = gather_api(d, a, t, filt, false, ext); base = API_BASE; break;
      case C_KERNEL: p = gather_kernel(d, a, t, filt, false, ext); base = KERNEL_BASE; break;
      case C_MEMCPY: p = gather_mem<C_MEMCPY>(d, a, t, filt, false, ext); base = MEM_BASE; break;
      case C_MEMCPY2: p = gather_mem<C_MEMCPY2>(d, a, t, filt, false, ext); base = MEM_BASE; break;
      case C_MEMSET: p = gather_mem<C_MEMSET>(d, a, t, filt, false, ext); base = MEM_BASE; break;
      case C_OVERHEAD: p = gather_overhead(d, a, t, filt); base = OP_BASE; break;
      case C_SYNC: p = gather_sync<C_SYNC>(d, a, t, filt, false, ext); base = SYNC_BASE; break;
      case C_WAIT: p = gather_sync<C_WAIT>(d, a, t, filt, false, ext); base = SYNC_BASE; break;
      case C_CUDAEVENT: p = gather_sync<C_CUDAEVENT>(d, a, t, filt, false, ext); base = SYNC_BASE; break;
      default: p = gather_op(d, j, a, t); base = OP_BASE; break;
    }
    // rare shapes: kernels with collective metadata, instant events
    const bool rare = (cls == C_KERNEL && ((p >> K_COLL) & 1ull) != 0) ||
                      (cls == C_OP && (p & ((1ull << I_HEAD) | (1ull << C_HEAD) | (1ull << H_ALL))) != 0);
    if (rare != COLL) return false;
    if constexpr (COLL) run_fields<S, COLL>(s, d, a, base, p, nb);
    else {
      // the classes nearly all events belong to run compile-time field code; the others share the table-driven loop
      if (base == API_BASE) loop_fields<API_BASE, A_COUNT>(s, d, a, p, nb);
      else if (base == KERNEL_BASE) loop_fields<KERNEL_BASE, K_COUNT>(s, d, a, p, nb);
      else if (base == MEM_BASE) loop_fields<MEM_BASE, M_COUNT>(s, d, a, p, nb);
      else if (cls == C_OP) loop_fields<OP_BASE, O_COUNT>(s, d, a, p, nb);
      else run_fields<S, COLL>(s, d, a, base, p, nb);
    }
  }
  return true;
}

// 8-byte units staged of a record of each class (C_API .. C_OVERHEAD): whole records, except the kernel record's unread tail
__device__ __forceinline__ uint32_t class_units(int cls) {
  return cls == C_KERNEL ? 22u : cls == C_MEMCPY2 ? 12u : (cls == C_API || cls == C_SYNC || cls == C_WAIT) ? 5u
         : (cls == C_OVERHEAD || cls == C_CUDAEVENT) ? 7u : 11u;
}

// One thread per work item.  Work items are class-sorted (each class padded to a multiple of 32),
// so a warp formats events of one shape.  WRITE = false: store the byte length; WRITE = true: write
// the bytes at ev_off[event].  Either pass first copies the 32 records of a warp into shared memory
// with coalesced loads (lane = 8-byte unit of a record); all later reads of record fields and of the
// values computed from them are shared-memory reads at table-given offsets.
template <bool WRITE, bool COLL = false>
__global__ void __launch_bounds__(kEventThreads, WRITE ? 5 : 8) k_events(Dev d) {
  // dynamic shared memory (events_smem_bytes): the threads' record areas, then (emit pass) their output windows
  extern __shared__ uint64_t s_dyn[];
  uint64_t* const s_rec = s_dyn;
  uint32_t* const s_win = reinterpret_cast<uint32_t*>(s_dyn + kEventThreads * kRecStride);  // per warp: [kWinWords][32 lanes]; a pad after the last warp
  __shared__ unsigned long long s_cnt[8];
  if (!WRITE) {
    if (threadIdx.x < 8) s_cnt[threadIdx.x] = 0;
    __syncthreads();
  }
  uint64_t i = d.work_origin + (uint64_t)blockIdx.x * kEventThreads + threadIdx.x;
  if (d.work_indirect != nullptr) i = i < d.n_indirect ? (uint64_t)d.work_indirect[i] : d.n_work;
  Tally t; t.x = 0; t.flow = 0; t.name_bytes = 0; t.ev = 0; t.work = i;
  uint32_t filt = 0;
  int cls = -1;
  uint64_t j = 0;
  if (i < d.n_work) {
    if (i >= d.ops_begin) { cls = C_OP; j = i - d.ops_begin; }
    else {
      cls = 0;
#pragma unroll
      for (int c = 1; c < C_EXT; c++) if (i >= d.cls_begin[c]) cls = c;
      j = i - d.cls_begin[cls];
      if (j >= d.cls_count[cls]) cls = -1;  // padding
    }
    if (cls == C_OP && j >= d.n_ops) cls = -1;
    // deferred synchronisation records are sized in a pass of their own, once the streams with GPU work are known
    if (!WRITE && (cls == C_WAIT) != (d.wait_pass != 0)) cls = -1;
  }
  uint64_t ev = 0;
  const uint8_t* r = nullptr;
  bool guest = false;
  uint32_t size = 0;
  uint64_t off = 0;
  int32_t ext = 0;
  if (cls >= 0) {
    ev = cls == C_OP ? j : d.work_ev[i];
    t.ev = ev;
    if (cls != C_OP) {
      const uint32_t slot = d.work_slot[i];
      r = d.cupti + (uint64_t)slot * 8;
      guest = slot < d.guest_front || slot >= d.guest_back;
    }
    if (WRITE) {
      size = d.ev_size[ev];
      if (size) {
        off = d.ev_off[ev];
        if (cls != C_OP) ext = d.ev_ext[ev];
        if (off < d.tile_begin || off >= d.tile_end) size = 0;  // another slab's event
        else if (size < kMinEventBytes || off + size > d.out_cap) { atomicAdd(&d.counters->device_check, 1ull); size = 0; }
      }
      if (!size) { r = nullptr; cls = -1; }
    }
  }
  {
    // stage this warp's records: every lane's class is the warp's class (or none).  Asynchronous
    // 8-byte copies, so all of a warp's record loads are in flight together and take no registers.
    const uint32_t lane = threadIdx.x & 31u, wbase = threadIdx.x & ~31u;
    const int cls0 = __reduce_max_sync(0xffffffffu, cls);
    if (cls0 >= 0 && cls0 != C_OP) {
      const uint32_t nu = class_units(cls0), rpi = 32u / nu;
      const uint32_t sub = lane / nu, unit = lane - sub * nu;
      const unsigned long long mine = (unsigned long long)reinterpret_cast<uintptr_t>(r);
      const uint32_t sdst = (uint32_t)__cvta_generic_to_shared(&s_rec[(wbase + sub) * kRecStride + unit]);
      for (uint32_t k = 0; k < 32u; k += rpi) {
        const uint32_t rec = k + sub;
        const unsigned long long src = __shfl_sync(0xffffffffu, mine, rec & 31u);
        if (sub < rpi && rec < 32u && src != 0ull)
          asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(sdst + k * (uint32_t)(kRecStride * 8)), "l"(src + 8ull * unit) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncwarp();
    }
  }
  uint32_t* area = reinterpret_cast<uint32_t*>(&s_rec[threadIdx.x * kRecStride]);
  if (cls >= 0) {
    if (!WRITE) {
      CountSink2 s;
      format_event(s, d, cls, area, j, t, &filt, &ext);
      if (guest) { filt = 3u; t.x = 0; t.flow = 0; t.name_bytes = 0; }  // another shard's record: looked at, never written
      d.ev_size[ev] = filt ? 0u : s.n;
      if (cls != C_OP) d.ev_ext[ev] = ext;
    } else {
      WindowSink s;
      s.init(d.out + off, size, s_win + (threadIdx.x >> 5) * (kWinWords * kWinStride) + (threadIdx.x & 31u));
      if (format_event<WindowSink, COLL>(s, d, cls, area, j, t, &filt, &ext) && !s.finish(d.out + off, size))
        atomicAdd(&d.counters->device_check, 1ull);
    }
  }
  if (!WRITE) {  // counters are tallied once, in the size pass: warp sums, then one shared atomic per warp
    const uint32_t wx = __reduce_add_sync(0xffffffffu, t.x), wf = __reduce_add_sync(0xffffffffu, t.flow);
    const uint32_t wo = __reduce_add_sync(0xffffffffu, filt == 2u ? 1u : 0u), wb = __reduce_add_sync(0xffffffffu, filt == 1u ? 1u : 0u);
    const uint32_t wn = __reduce_add_sync(0xffffffffu, (uint32_t)t.name_bytes);  // a name is far shorter than 2^27 bytes
    const uint32_t wg = __reduce_add_sync(0xffffffffu, filt == 3u ? 1u : 0u);
    if ((threadIdx.x & 31u) == 0) {
      if (wx) atomicAdd(&s_cnt[0], (unsigned long long)wx);
      if (wf) atomicAdd(&s_cnt[1], (unsigned long long)wf);
      if (wo) atomicAdd(&s_cnt[2], (unsigned long long)wo);
      if (wb) atomicAdd(&s_cnt[3], (unsigned long long)wb);
      if (wn) atomicAdd(&s_cnt[4], (unsigned long long)wn);
      if (wg) atomicAdd(&s_cnt[5], (unsigned long long)wg);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      if (s_cnt[0]) atomicAdd(&d.counters->x_events, s_cnt[0]);
      if (s_cnt[1]) atomicAdd(&d.counters->flow_events, s_cnt[1]);
      if (s_cnt[2]) atomicAdd(&d.counters->out_of_range, s_cnt[2]);
      if (s_cnt[3]) atomicAdd(&d.counters->blocklisted_runtime, s_cnt[3]);
      if (s_cnt[4]) atomicAdd(&d.counters->name_bytes, s_cnt[4]);
      if (s_cnt[5]) atomicAdd(&d.counters->guests, s_cnt[5]);
    }
  }
}

// ---- tiled runs: which events and which work items belong to each slab of the output ----
// Slab t holds the events whose text starts in [t * slab, (t + 1) * slab).  bounds is a (n_tiles + 1) x
// kTileCols table: column 0 the first event of the slab, column 1 its first byte, columns 2 + c the first work
// item of class c (C_API .. C_WAIT) whose event belongs to the slab or a later one.  Work items of a class are
// in event order unless events were sorted by start time (then the launches of a slab cover whole classes
// and the kernels skip the other slabs' events by their offsets).
constexpr int kTileCols = 2 + C_EXT;
__global__ void k_tile_bounds(Dev d, uint64_t slab, uint32_t n_tiles, uint64_t total, uint64_t* bounds) {
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t > n_tiles) return;
  uint64_t e = d.n_events;
  if (t < n_tiles) {  // first event that starts at or after t * slab
    const uint64_t target = (uint64_t)t * slab;
    uint64_t lo = 0, hi = d.n_events;
    for (int it = 0; it < 40 && lo < hi; it++) { const uint64_t mid = lo + ((hi - lo) >> 1); if (d.ev_off[mid] < target) lo = mid + 1; else hi = mid; }
    e = lo;
  }
  uint64_t* row = bounds + (uint64_t)t * kTileCols;
  row[0] = e;
  row[1] = e < d.n_events ? d.ev_off[e] : total;
  for (int c = 0; c < C_EXT; c++) {  // first work item of the class whose event number is >= e
    uint64_t lo = d.cls_begin[c], hi = d.cls_begin[c] + d.cls_count[c];
    for (int it = 0; it < 40 && lo < hi; it++) { const uint64_t mid = lo + ((hi - lo) >> 1); if ((uint64_t)d.work_ev[mid] < e) lo = mid + 1; else hi = mid; }
    row[2 + c] = lo;
  }
}

// ---- optional ordering by start timestamp ----
// Sort key of every GPU-side event: converted start time relative to the window start (records outside
// the window emit nothing, their position does not matter).  Values are the buffer-order event numbers.
__global__ void k_sort_keys(Dev d, uint64_t* keys, uint32_t* vals, uint64_t span) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.ops_begin) return;
  int cls = 0;
#pragma unroll
  for (int c = 1; c < C_EXT; c++) if (i >= d.cls_begin[c]) cls = c;
  if (i - d.cls_begin[cls] >= d.cls_count[cls]) return;  // padding
  const uint8_t* r = d.cupti + (uint64_t)d.work_slot[i] * 8;
  const int64_t ts = conv_ts(d, *reinterpret_cast<const uint64_t*>(r + ((cls == C_API || cls == C_SYNC || cls == C_WAIT) ? 8
                                                                         : cls == C_OVERHEAD ? 24 : cls == C_CUDAEVENT ? 40 : 16)));
  uint64_t key = 0;
  if (ts >= d.win_start) { key = (uint64_t)(ts - d.win_start); if (key > span) key = span + 1; }
  if (cls == C_WAIT) key += span + 2;  // deferred records stay behind everything else
  const uint32_t e = d.work_ev[i] - (uint32_t)d.n_ops;
  keys[e] = key;
  vals[e] = e;
}
__global__ void k_sort_remap(Dev d, const uint32_t* rank) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= d.ops_begin) return;
  int cls = 0;
#pragma unroll
  for (int c = 1; c < C_EXT; c++) if (i >= d.cls_begin[c]) cls = c;
  if (i - d.cls_begin[cls] >= d.cls_count[cls]) return;
  d.work_ev[i] = (uint32_t)d.n_ops + rank[d.work_ev[i] - (uint32_t)d.n_ops];
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
  __shared__ uint64_t s_area[kEventThreads * 4];  // 32 bytes per span, 8-byte aligned for slot_value's 64-bit loads
  __shared__ uint32_t s_win[WRITE ? kEventThreads * kWinWords + kWinPadWords : 1];
  const uint32_t i = blockIdx.x * kEventThreads + threadIdx.x;
  if (i >= n) return;
  const SpanRec r = spans[i];
  int64_t dur = r.end - r.start;
  if (dur < 0) dur = 0;
  unsigned long long nb = 0;
  uint32_t* a = reinterpret_cast<uint32_t*>(&s_area[threadIdx.x * 4]);
  s32(a, NS_NAME, r.op_row < d.n_ops ? d.op_name[r.op_row] : 0xFFFFFFFFu); s32(a, NS_PID, r.device); s32(a, NS_TID, r.stream);
  s32(a, NS_EXT, (uint32_t)r.op_id); s64(a, NS_TS, (uint64_t)rel_ts(d, r.start - 1)); s64(a, NS_DUR, (uint64_t)(dur + 2));
  uint64_t p = (1ull << N_COUNT) - 1ull;
  if (r.op_id == 0) p &= ~((1ull << N_EXT) | (1ull << N_ARGS_CLOSE));
  if (!WRITE) { CountSink2 s; count_fields<ANN_BASE, 0, N_COUNT>(s, d, a, p, &nb); sizes[i] = s.n; }
  else {
    const uint32_t size = sizes[i];
    uint8_t* dst = d.out + out_base + offs[i];
    if (size < kMinEventBytes || out_base + offs[i] + size > d.out_cap) { atomicAdd(&d.counters->device_check, 1ull); return; }
    WindowSink s;
    s.init(dst, size, s_win + (threadIdx.x >> 5) * (kWinWords * kWinStride) + (threadIdx.x & 31u));
    run_fields(s, d, a, ANN_BASE, p, &nb);
    if (!s.finish(dst, size)) atomicAdd(&d.counters->device_check, 1ull);
  }
}

}  // namespace k2j
