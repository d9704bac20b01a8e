// Host side of libk2j: the C ABI of include/k2j.h over the kernels in k2j_kernels.cuh.
// One context owns a stream, grow-only device workspaces and the staged inputs of one trace.
#include "../../include/k2j.h"

#include <cuda_runtime.h>
#include <errno.h>
#include <unistd.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "k2j_kernels.cuh"
#include "k2j_sort.cuh"

namespace k2j {
// 8-byte slots of a record of `kind` (word1 = its second 32-bit word): kinds the path formats by the structures the
// reference reads them as, every other kind by the CUPTI headers' structure; 0 = a kind the headers do not define.
uint32_t record_slots(uint32_t kind, uint32_t word1) {
  if (kind >= (uint32_t)kCuptiKinds) return 0;
  const uint32_t code = slot_code(kind, word1);
  return code ? (code & 31u) : kCuptiRecordSlots[kind];
}
}  // namespace k2j

using namespace k2j;

namespace {

// Grow-only device allocation.
struct DevBuf {
  void* p = nullptr;
  size_t cap = 0;
  cudaError_t reserve(size_t bytes) {
    if (bytes <= cap) return cudaSuccess;
    if (p) cudaFree(p);
    p = nullptr; cap = 0;
    size_t want = bytes + bytes / 8 + 256;
    cudaError_t e = cudaMalloc(&p, want);
    if (e == cudaSuccess) cap = want;
    return e;
  }
  void release() { if (p) cudaFree(p); p = nullptr; cap = 0; }
  template <class T> T* as() const { return reinterpret_cast<T*>(p); }
};

// An input array: either caller-owned device memory used in place, or a staged copy of host memory.
struct Input {
  DevBuf own;
  const void* dev = nullptr;
  size_t bytes = 0;
};

}  // namespace

struct k2j_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  std::string err;
  k2j_params params{};
  bool have_params = false;
  std::vector<DevProps> props;
  DevBuf d_props;
  Input pool_off, pool_data, rt_names, dr_names, tid_pairs, cupti;
  Input op_start, op_end, op_id, op_device, op_resource, op_thread, op_type, op_name, op_flow, op_flowt, op_mdoff, op_md;
  uint64_t n_strings = 0, n_ops = 0, n_md = 0, cupti_bytes = 0;
  uint32_t n_rt = 0, n_dr = 0, n_tid = 0, n_buf = 0, n_chunks = 0;
  bool strings_dirty = true;
  std::vector<uint64_t> h_buf_off, h_buf_valid;
  std::vector<uint32_t> h_buf_chunk_base;
  DevBuf d_buf_off, d_buf_valid, d_buf_chunk_base;
  DevBuf esc_name, esc_md, esc_name_len, esc_md_len, walk_cnt, need_corr, need_op;
  DevBuf slot_code, exit_map, chunk_entry, chunk_cnt, chunk_base, scan_sums, scan_totals;
  DevBuf ds_tab, span_key, span_nstart, span_end, span_nfirst, span_row, span_out, span_cnt, ann_size, ann_off;
  DevBuf sort_keys[2], sort_vals[2], sort_hist, sort_base, sort_rank;
  DevBuf tid_tab, corr_tab, user_tab, op_tab, work_slot, work_ev, ev_size, ev_off, ev_ext, out, counters;
  uint64_t* h_totals = nullptr;   // pinned, 32 words: [0, C_NCOL) column totals, 20 text bytes, 21 bytes of CPU-op text, 22 annotation bytes, 23 sort, 24 scan entry point, 25 the record_param_comms flag, 26 kernel events with collective metadata
  Counters* h_counters = nullptr; // pinned
  void* h_stage[2] = {nullptr, nullptr};            // pinned staging buffers of k2j_write_output
  cudaEvent_t stage_ev[2] = {nullptr, nullptr};
  cudaEvent_t ev[8]{};
  uint64_t out_bytes = 0;
  bool ran = false, segmented = false, have_global_join = false;
  Dev d{};
  uint64_t totals[C_NCOL] = {0};
  uint32_t launches = 0;
  DevBuf ext_local;
  DevBuf slab[2], tile_bounds;                       // tiled runs: two output slabs, the slab table
  cudaStream_t copy_stream = nullptr;                // device-to-host copies of finished slabs
  cudaEvent_t slab_done[2] = {nullptr, nullptr}, slab_free[2] = {nullptr, nullptr};
  bool streamed = false;                             // the last run handed its text on slab by slab: no resident output
  DevBuf ctx_tab, evt_recs, seen_tab, row_key, row_first, corr_zero;  // synchronisation records
  DevBuf str_class, comms_flag, coll_list;                            // collective enrichment
  DevBuf corr0;                                                       // correlation id 0 (see Dev::corr0)
  const void* g_ext = nullptr; uint64_t g_n_ext = 0, g_own_begin = 0;
  const int32_t* g_op_ids = nullptr; uint64_t g_n_ops = 0;
  uint64_t guest_front_bytes = 0, guest_back_bytes = ~0ull; bool guests_declared = false;  // k2j_set_guest_ranges
  DevBuf exp_keys, exp_first, exp_list, exp_out, coll_tab;
  uint64_t n_guest_ops = 0;                                           // k2j_set_guest_ops
  std::vector<SpanRec> partial_spans;                                 // sharded runs: this shard's parts of the user-annotation spans
  uint32_t g_ext_stride = 0, g_ops_stride = 0, g_world = 1, g_rank = 0; uint64_t g_pitch = 0; const uint64_t* g_counts = nullptr;  // rows of an all-gather
  const uint32_t* g_op_bits = nullptr; uint64_t g_op_bits_pitch = 0; const int64_t* g_op_bits_meta = nullptr;  // k2j_set_global_op_bits
  int join_user_hint = -1;                                            // k2j_set_join_user_records: -1 not told
  uint32_t* need_bits = nullptr; uint64_t need_n_bits = 0;             // the caller's filter from k2j_join_need_bits, valid for this segmentation
};

namespace {

k2j_status fail(k2j_ctx* c, k2j_status st, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (c) c->err = buf;
  return st;
}
#define K2J_CUDA(ctx, call)                                                                       \
  do {                                                                                            \
    cudaError_t _e = (call);                                                                      \
    if (_e != cudaSuccess) return fail(ctx, K2J_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(_e)); \
  } while (0)

bool is_device_ptr(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// Stages `bytes` of `src`: device memory is referenced, host memory is copied on the context stream.
k2j_status stage(k2j_ctx* c, Input& in, const void* src, size_t bytes) {
  in.bytes = bytes;
  if (bytes == 0) { in.dev = nullptr; return K2J_OK; }
  if (!src) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null input array");
  if (is_device_ptr(src)) { in.dev = src; return K2J_OK; }
  K2J_CUDA(c, in.own.reserve(bytes));
  K2J_CUDA(c, cudaMemcpyAsync(in.own.p, src, bytes, cudaMemcpyHostToDevice, c->stream));
  in.dev = in.own.p;
  return K2J_OK;
}

uint32_t pow2_at_least(uint64_t n) {
  uint32_t p = 16;
  while (p < n && p < (1u << 31)) p <<= 1;
  return p;
}

struct Scan {
  static uint32_t blocks(uint64_t n) { return (uint32_t)((n + kScanTile - 1) / kScanTile); }
};

// Exclusive scan of `cols` columns of n u32 each (column stride n) into u64; totals land in
// totals[0..cols).  Three launches.
k2j_status run_scan(k2j_ctx* c, const uint32_t* in, uint64_t n, uint32_t cols, uint64_t* out, uint64_t* totals, uint32_t* launches) {
  const uint32_t nb = std::max<uint32_t>(1, Scan::blocks(n));
  K2J_CUDA(c, c->scan_sums.reserve((size_t)nb * cols * 8));
  uint64_t* sums = c->scan_sums.as<uint64_t>();
  k_scan_reduce<<<dim3(nb, cols), kScanThreads, 0, c->stream>>>(in, n, n, sums, nb);
  k_scan_sums<<<cols, kScanThreads, 0, c->stream>>>(sums, nb, totals);
  k_scan_apply<<<dim3(nb, cols), kScanThreads, 0, c->stream>>>(in, n, n, sums, nb, out);
  *launches += 3;
  K2J_CUDA(c, cudaGetLastError());
  return K2J_OK;
}

// Workspaces of the radix sort for n pairs.
k2j_status sort_reserve(k2j_ctx* c, uint64_t n) {
  const uint32_t tiles = (uint32_t)((n + kSortTile - 1) / kSortTile);
  for (int i = 0; i < 2; i++) {
    K2J_CUDA(c, c->sort_keys[i].reserve(n * 8));
    K2J_CUDA(c, c->sort_vals[i].reserve(n * 4));
  }
  K2J_CUDA(c, c->sort_hist.reserve((size_t)tiles * 256 * 4));
  K2J_CUDA(c, c->sort_base.reserve((size_t)tiles * 256 * 8));
  return K2J_OK;
}
// Stable sort of the n pairs in sort_keys[*cur] / sort_vals[*cur] by the low 8 * passes bits of the key; *cur names
// the buffers that hold the result.
k2j_status sort_passes(k2j_ctx* c, uint64_t n, int passes, int* cur_io) {
  cudaStream_t s = c->stream;
  const uint32_t tiles = (uint32_t)((n + kSortTile - 1) / kSortTile);
  int cur = *cur_io;
  for (int pass = 0; pass < passes; pass++) {
    k_rs_hist<<<tiles, kSortThreads, 0, s>>>(c->sort_keys[cur].as<uint64_t>(), n, 8 * pass, c->sort_hist.as<uint32_t>(), tiles);
    c->launches++;
    k2j_status st = run_scan(c, c->sort_hist.as<uint32_t>(), (uint64_t)tiles * 256, 1, c->sort_base.as<uint64_t>(),
                             c->scan_totals.as<uint64_t>() + 23, &c->launches);
    if (st) return st;
    k_rs_scatter<<<tiles, kSortThreads, 0, s>>>(c->sort_keys[cur].as<uint64_t>(), c->sort_vals[cur].as<uint32_t>(), n, 8 * pass,
                                                c->sort_base.as<uint64_t>(), tiles, c->sort_keys[cur ^ 1].as<uint64_t>(),
                                                c->sort_vals[cur ^ 1].as<uint32_t>());
    c->launches++;
    cur ^= 1;
  }
  *cur_io = cur;
  K2J_CUDA(c, cudaGetLastError());
  return K2J_OK;
}

// CUDA event records ordered by (context, event, correlation id, position): two stable sorts, by correlation id
// and then by context << 32 | event id.  The lookups of synchronisation records search the result.
k2j_status sort_cuda_events(k2j_ctx* c, uint64_t n) {
  cudaStream_t s = c->stream;
  Dev& d = c->d;
  k2j_status st = sort_reserve(c, n);
  if (st) return st;
  K2J_CUDA(c, c->evt_recs.reserve(n * sizeof(EvtRec)));
  const uint32_t blocks = (uint32_t)((n + 255) / 256);
  int cur = 0;
  k_evt_keys<<<blocks, 256, 0, s>>>(d, c->sort_keys[cur].as<uint64_t>(), c->sort_vals[cur].as<uint32_t>(), 0);
  c->launches++;
  if ((st = sort_passes(c, n, 4, &cur))) return st;
  k_evt_keys<<<blocks, 256, 0, s>>>(d, c->sort_keys[cur].as<uint64_t>(), c->sort_vals[cur].as<uint32_t>(), 1);
  c->launches++;
  if ((st = sort_passes(c, n, 8, &cur))) return st;
  k_evt_finish<<<blocks, 256, 0, s>>>(d, c->sort_keys[cur].as<uint64_t>(), c->sort_vals[cur].as<uint32_t>(), c->evt_recs.as<EvtRec>());
  c->launches++;
  K2J_CUDA(c, cudaGetLastError());
  d.evt = c->evt_recs.as<EvtRec>(); d.n_evt = (uint32_t)n;
  return K2J_OK;
}

// Stable LSD radix sort of the GPU-side events by start timestamp; afterwards work_ev holds sorted ranks.
k2j_status sort_gpu_events(k2j_ctx* c, uint64_t n) {
  cudaStream_t s = c->stream;
  Dev& d = c->d;
  const uint64_t span = (uint64_t)(c->params.window_end_ns - c->params.window_start_ns);
  const uint64_t max_key = c->totals[C_WAIT] ? 2 * span + 3 : span + 1;  // deferred records sort behind the rest
  int bits = 1;
  while (bits < 64 && (max_key >> bits)) bits++;
  const int passes = (bits + 7) / 8;
  k2j_status st0 = sort_reserve(c, n);
  if (st0) return st0;
  K2J_CUDA(c, c->sort_rank.reserve(n * 4));
  const uint32_t wl_blocks = (uint32_t)((d.ops_begin + 255) / 256);
  k_sort_keys<<<wl_blocks, 256, 0, s>>>(d, c->sort_keys[0].as<uint64_t>(), c->sort_vals[0].as<uint32_t>(), span);
  c->launches++;
  int cur = 0;
  if ((st0 = sort_passes(c, n, passes, &cur))) return st0;
  k_rs_invert<<<(uint32_t)((n + 255) / 256), 256, 0, s>>>(c->sort_vals[cur].as<uint32_t>(), n, c->sort_rank.as<uint32_t>());
  k_sort_remap<<<wl_blocks, 256, 0, s>>>(d, c->sort_rank.as<uint32_t>());
  c->launches += 2;
  K2J_CUDA(c, cudaGetLastError());
  return K2J_OK;
}

// Collects the span table, puts the spans in the order GpuUserEventMap::logEvents walks them — a
// std::map over (device, stream), and inside it a std::unordered_map<int64_t, ...> over the op id,
// filled in order of first use (libkineto/src/GenericActivityProfiler.h:341-346, .cpp:320-327) — and
// sizes their events.  Host work is O(distinct annotations).
// The span table as a list on the host (no order).
k2j_status collect_spans(k2j_ctx* c, uint32_t span_cap, std::vector<SpanRec>* spans) {
  cudaStream_t s = c->stream;
  Dev& d = c->d;
  K2J_CUDA(c, c->span_out.reserve((size_t)span_cap * sizeof(SpanRec)));
  K2J_CUDA(c, c->span_cnt.reserve(16));
  K2J_CUDA(c, cudaMemsetAsync(c->span_cnt.p, 0, 4, s));
  k_span_collect<<<(span_cap + 255) / 256, 256, 0, s>>>(d, c->span_out.as<SpanRec>(), c->span_cnt.as<unsigned int>());
  c->launches++;
  unsigned int n = 0;
  K2J_CUDA(c, cudaMemcpyAsync(&n, c->span_cnt.p, 4, cudaMemcpyDeviceToHost, s));
  K2J_CUDA(c, cudaStreamSynchronize(s));
  spans->resize(n);
  if (n == 0) return K2J_OK;
  K2J_CUDA(c, cudaMemcpyAsync(spans->data(), c->span_out.p, (size_t)n * sizeof(SpanRec), cudaMemcpyDeviceToHost, s));
  K2J_CUDA(c, cudaStreamSynchronize(s));
  return K2J_OK;
}
k2j_status size_annotations(k2j_ctx* c, const std::vector<SpanRec>& spans, uint32_t* n_out, uint64_t* bytes_out);
k2j_status order_annotations(k2j_ctx* c, uint32_t span_cap, uint32_t* n_out, uint64_t* bytes_out) {
  std::vector<SpanRec> spans;
  k2j_status st = collect_spans(c, span_cap, &spans);
  if (st) return st;
  return size_annotations(c, spans, n_out, bytes_out);
}
// Puts spans in logging order (see above), leaves them in span_out and sizes their events (ann_size, ann_off).
k2j_status size_annotations(k2j_ctx* c, const std::vector<SpanRec>& spans, uint32_t* n_out, uint64_t* bytes_out) {
  cudaStream_t s = c->stream;
  Dev& d = c->d;
  const unsigned int n = (unsigned int)spans.size();
  *n_out = n; *bytes_out = 0;
  if (n == 0) return K2J_OK;
  K2J_CUDA(c, c->span_out.reserve((size_t)n * sizeof(SpanRec)));
  std::map<std::pair<int64_t, int64_t>, std::vector<const SpanRec*>> by_stream;
  for (const SpanRec& r : spans) by_stream[{(int64_t)r.device, (int64_t)r.stream}].push_back(&r);
  std::vector<SpanRec> ordered;
  ordered.reserve(n);
  for (auto& kv : by_stream) {
    auto& v = kv.second;
    std::sort(v.begin(), v.end(), [](const SpanRec* a, const SpanRec* b) { return a->first_event < b->first_event; });
    std::unordered_map<int64_t, const SpanRec*> m;
    for (const SpanRec* r : v) m.insert({(int64_t)r->op_id, r});
    for (auto& e : m) ordered.push_back(*e.second);
  }
  K2J_CUDA(c, cudaMemcpyAsync(c->span_out.p, ordered.data(), (size_t)n * sizeof(SpanRec), cudaMemcpyHostToDevice, s));
  K2J_CUDA(c, c->ann_size.reserve((size_t)n * 4));
  K2J_CUDA(c, c->ann_off.reserve((size_t)n * 8));
  k_annotations<false><<<(n + kEventThreads - 1) / kEventThreads, kEventThreads, 0, s>>>(
      d, c->span_out.as<SpanRec>(), n, c->ann_size.as<uint32_t>(), nullptr, 0);
  c->launches++;
  K2J_CUDA(c, cudaGetLastError());
  k2j_status st = run_scan(c, c->ann_size.as<uint32_t>(), n, 1, c->ann_off.as<uint64_t>(), c->scan_totals.as<uint64_t>() + 22, &c->launches);
  if (st) return st;
  K2J_CUDA(c, cudaMemcpyAsync(c->h_totals + 22, c->scan_totals.as<uint64_t>() + 22, 8, cudaMemcpyDeviceToHost, s));
  K2J_CUDA(c, cudaStreamSynchronize(s));  // also covers `ordered`, which goes out of scope
  *bytes_out = c->h_totals[22];
  return K2J_OK;
}

}  // namespace

extern "C" {

const char* k2j_version(void) { return "k2j 0.1 (sm_100a)"; }

k2j_status k2j_create(int device, void* stream, k2j_ctx** out) {
  if (!out) return K2J_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { cudaGetLastError(); return K2J_ERR_CUDA; }
  if (device < 0 || device >= n) return K2J_ERR_INVALID_ARGUMENT;
  if (cudaSetDevice(device) != cudaSuccess) return K2J_ERR_CUDA;
  k2j_ctx* c = new k2j_ctx();
  c->device = device;
  if (stream) c->stream = (cudaStream_t)stream;
  else {
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) { delete c; return K2J_ERR_CUDA; }
    c->own_stream = true;
  }
  bool ok = cudaMallocHost((void**)&c->h_totals, 32 * sizeof(uint64_t)) == cudaSuccess &&
            cudaMallocHost((void**)&c->h_counters, sizeof(Counters)) == cudaSuccess &&
            c->counters.reserve(sizeof(Counters)) == cudaSuccess && c->scan_totals.reserve(32 * 8) == cudaSuccess;
  for (auto& e : c->ev) ok = ok && cudaEventCreate(&e) == cudaSuccess;
  // the emit kernels' shared memory (record areas + output windows) is above the 48 KiB that needs no opt-in
  ok = ok && cudaFuncSetAttribute(k_events<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)events_smem_bytes(true)) == cudaSuccess &&
       cudaFuncSetAttribute(k_events<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)events_smem_bytes(true)) == cudaSuccess;
  if (!ok) { k2j_destroy(c); return K2J_ERR_CUDA; }
  *out = c;
  return K2J_OK;
}

void k2j_destroy(k2j_ctx* c) {
  if (!c) return;
  cudaSetDevice(c->device);
  if (c->stream) cudaStreamSynchronize(c->stream);
  for (Input* in : {&c->pool_off, &c->pool_data, &c->rt_names, &c->dr_names, &c->tid_pairs, &c->op_thread, &c->cupti,
                    &c->op_start, &c->op_end, &c->op_id, &c->op_device, &c->op_resource, &c->op_type, &c->op_name,
                    &c->op_flow, &c->op_flowt, &c->op_mdoff, &c->op_md})
    in->own.release();
  for (DevBuf* b : {&c->d_props, &c->d_buf_off, &c->d_buf_valid, &c->d_buf_chunk_base, &c->esc_name, &c->esc_md,
                    &c->esc_name_len, &c->esc_md_len, &c->walk_cnt, &c->need_corr, &c->need_op, &c->slot_code, &c->exit_map, &c->chunk_entry, &c->chunk_cnt,
                    &c->chunk_base, &c->scan_sums, &c->scan_totals, &c->ds_tab, &c->span_key, &c->span_nstart, &c->span_end, &c->span_nfirst, &c->span_row,
                    &c->span_out, &c->span_cnt, &c->ann_size, &c->ann_off, &c->sort_keys[0], &c->sort_keys[1], &c->sort_vals[0],
                    &c->sort_vals[1], &c->sort_hist, &c->sort_base, &c->sort_rank, &c->tid_tab, &c->corr_tab, &c->user_tab, &c->op_tab,
                    &c->work_slot, &c->work_ev, &c->ev_size, &c->ev_off, &c->ev_ext, &c->out, &c->counters, &c->ext_local, &c->ctx_tab, &c->evt_recs,
                    &c->seen_tab, &c->row_key, &c->row_first, &c->corr_zero, &c->str_class, &c->comms_flag, &c->coll_list, &c->corr0,
                    &c->exp_keys, &c->exp_first, &c->exp_list, &c->exp_out, &c->coll_tab})
    b->release();
  if (c->h_totals) cudaFreeHost(c->h_totals);
  if (c->h_counters) cudaFreeHost(c->h_counters);
  for (int i = 0; i < 2; i++) {
    if (c->h_stage[i]) cudaFreeHost(c->h_stage[i]);
    if (c->stage_ev[i]) cudaEventDestroy(c->stage_ev[i]);
  }
  for (auto& e : c->ev) if (e) cudaEventDestroy(e);
  for (int i = 0; i < 2; i++) {
    c->slab[i].release();
    if (c->slab_done[i]) cudaEventDestroy(c->slab_done[i]);
    if (c->slab_free[i]) cudaEventDestroy(c->slab_free[i]);
  }
  c->tile_bounds.release();
  if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
  if (c->own_stream && c->stream) cudaStreamDestroy(c->stream);
  delete c;
}

const char* k2j_last_error(const k2j_ctx* c) { return c ? c->err.c_str() : "null context"; }

k2j_status k2j_set_params(k2j_ctx* c, const k2j_params* p, const k2j_device_props* props) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!p || p->n_devices < 0 || p->n_devices > 4096 || (p->n_devices > 0 && !props))
    return fail(c, K2J_ERR_INVALID_ARGUMENT, "bad params");
  if (p->ts_mode != 0 && p->ts_mode != 1) return fail(c, K2J_ERR_INVALID_ARGUMENT, "ts_mode must be 0 or 1");
  if (p->ts_mode == 1 && !(p->conv_scale_mant >> 63))
    return fail(c, K2J_ERR_INVALID_ARGUMENT, "converter scale must be a normalised 64-bit significand");
  K2J_CUDA(c, cudaSetDevice(c->device));
  c->params = *p;
  c->props.resize(p->n_devices);
  for (int i = 0; i < p->n_devices; i++) {
    DevProps& d = c->props[i];
    d.major = props[i].major; d.minor = props[i].minor;
    d.max_threads_per_block = props[i].max_threads_per_block; d.max_threads_per_sm = props[i].max_threads_per_sm;
    d.regs_per_block = props[i].regs_per_block; d.regs_per_sm = props[i].regs_per_sm;
    d.warp_size = props[i].warp_size; d.num_sms = props[i].num_sms;
    d.smem_per_block = props[i].smem_per_block; d.smem_per_block_optin = props[i].smem_per_block_optin;
    d.smem_per_sm = props[i].smem_per_sm; d.reserved_smem_per_block = props[i].reserved_smem_per_block;
  }
  K2J_CUDA(c, c->d_props.reserve(std::max<size_t>(1, c->props.size()) * sizeof(DevProps)));
  if (!c->props.empty())
    K2J_CUDA(c, cudaMemcpyAsync(c->d_props.p, c->props.data(), c->props.size() * sizeof(DevProps), cudaMemcpyHostToDevice, c->stream));
  K2J_CUDA(c, cudaStreamSynchronize(c->stream));  // c->props may be resized by the next call
  c->have_params = true;
  return K2J_OK;
}

k2j_status k2j_set_strings(k2j_ctx* c, const uint64_t* off, const uint8_t* data, uint64_t n) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (n >= 0xFFFFFFF0ull) return fail(c, K2J_ERR_INVALID_ARGUMENT, "too many strings");
  if (n > 0 && !off) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null string offsets");
  K2J_CUDA(c, cudaSetDevice(c->device));
  c->n_strings = n;
  c->strings_dirty = true;
  uint64_t total = 0;
  if (n > 0) {
    if (is_device_ptr(off)) K2J_CUDA(c, cudaMemcpy(&total, off + n, 8, cudaMemcpyDeviceToHost));
    else total = off[n];
  }
  k2j_status st = stage(c, c->pool_off, off, (n + 1) * 8);
  if (st) return st;
  st = stage(c, c->pool_data, data, total);
  if (st) return st;
  // closed-form capacities of the two sanitised flavours (see esc_name_pos / esc_md_pos)
  K2J_CUDA(c, c->esc_name.reserve(2 * total + 16 * (n + 1) + 16));
  K2J_CUDA(c, c->esc_md.reserve(total + 8 * (n + 1) + 16));
  K2J_CUDA(c, c->esc_name_len.reserve((n + 1) * 4));
  K2J_CUDA(c, c->esc_md_len.reserve((n + 1) * 4));
  K2J_CUDA(c, c->str_class.reserve(n + 1));
  return K2J_OK;
}

k2j_status k2j_set_cbid_names(k2j_ctx* c, const uint32_t* rt, uint32_t n_rt, const uint32_t* dr, uint32_t n_dr) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  K2J_CUDA(c, cudaSetDevice(c->device));
  c->n_rt = n_rt; c->n_dr = n_dr;
  k2j_status st = stage(c, c->rt_names, rt, (size_t)n_rt * 4);
  if (st) return st;
  return stage(c, c->dr_names, dr, (size_t)n_dr * 4);
}

k2j_status k2j_set_thread_map(k2j_ctx* c, const int32_t* pairs, uint32_t n) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (n > 0 && !pairs) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null thread map");
  if (n > 0 && is_device_ptr(pairs)) return fail(c, K2J_ERR_INVALID_ARGUMENT, "thread map must be host memory");
  K2J_CUDA(c, cudaSetDevice(c->device));
  c->n_tid = n;
  k2j_status st = stage(c, c->tid_pairs, pairs, (size_t)n * 8);
  if (st) return st;
  return K2J_OK;
}

k2j_status k2j_set_ops(k2j_ctx* c, const k2j_ops* o) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!o) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null ops");
  if (o->n_ops >= 0x7FFFFFF0ull) return fail(c, K2J_ERR_INVALID_ARGUMENT, "too many CPU activities");
  K2J_CUDA(c, cudaSetDevice(c->device));
  const uint64_t n = o->n_ops;
  c->n_ops = n;
  c->n_guest_ops = 0;  // new rows: k2j_set_guest_ops says again which of them are guests
  uint64_t n_md = 0;
  if (n > 0) {
    if (!o->md_off) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null md_off");
    uint32_t last = 0;
    if (is_device_ptr(o->md_off)) K2J_CUDA(c, cudaMemcpy(&last, o->md_off + n, 4, cudaMemcpyDeviceToHost));
    else last = o->md_off[n];
    n_md = last;
  }
  c->n_md = n_md;
  k2j_status st;
#define STAGE(field, src, bytes) if ((st = stage(c, c->field, src, bytes)) != K2J_OK) return st
  STAGE(op_start, o->start_ns, n * 8); STAGE(op_end, o->end_ns, n * 8); STAGE(op_id, o->id, n * 4);
  STAGE(op_device, o->device, n * 4); STAGE(op_resource, o->resource, n * 8); STAGE(op_thread, o->thread, n * 4);
  STAGE(op_type, o->type, n * 4);
  STAGE(op_name, o->name, n * 4); STAGE(op_flow, o->flow_id, n * 4); STAGE(op_flowt, o->flow_info, n);
  STAGE(op_mdoff, o->md_off, n ? (n + 1) * 4 : 0); STAGE(op_md, o->md, n_md * sizeof(k2j_md_entry));
#undef STAGE
  return K2J_OK;
}

k2j_status k2j_set_cupti(k2j_ctx* c, const uint8_t* bytes, uint64_t n_bytes, const uint64_t* buftab, uint32_t n_buf) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (n_bytes > (32ull << 30)) return fail(c, K2J_ERR_INVALID_ARGUMENT, "more than 32 GiB of CUPTI records in one call");
  if (n_buf > 0 && (!buftab || !bytes)) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null CUPTI buffers");
  if (n_buf > 0 && is_device_ptr(buftab)) return fail(c, K2J_ERR_INVALID_ARGUMENT, "buffer table must be host memory");
  K2J_CUDA(c, cudaSetDevice(c->device));
  c->h_buf_off.clear(); c->h_buf_valid.clear(); c->h_buf_chunk_base.assign(1, 0);
  uint64_t chunks = 0;
  for (uint32_t b = 0; b < n_buf; b++) {
    const uint64_t off = buftab[2 * b], valid = buftab[2 * b + 1];
    if ((off & 7) || (valid & 7)) return fail(c, K2J_ERR_INVALID_ARGUMENT, "buffer %u: offset/size not 8-byte aligned", b);
    if (off > n_bytes || valid > n_bytes - off) return fail(c, K2J_ERR_INVALID_ARGUMENT, "buffer %u: out of range", b);
    if (valid == 0) continue;
    c->h_buf_off.push_back(off); c->h_buf_valid.push_back(valid);
    chunks += (valid + kChunkSlots * 8 - 1) / (kChunkSlots * 8);
    if (chunks >= 0xFFFFFFF0ull) return fail(c, K2J_ERR_INVALID_ARGUMENT, "too many chunks");
    c->h_buf_chunk_base.push_back((uint32_t)chunks);
  }
  c->n_buf = (uint32_t)c->h_buf_off.size();
  c->n_chunks = (uint32_t)chunks;
  c->guest_front_bytes = 0; c->guest_back_bytes = ~0ull; c->guests_declared = false;
  c->cupti_bytes = n_bytes;
  k2j_status st = stage(c, c->cupti, bytes, n_bytes);
  if (st) return st;
  K2J_CUDA(c, c->d_buf_off.reserve(std::max<size_t>(8, c->n_buf * 8)));
  K2J_CUDA(c, c->d_buf_valid.reserve(std::max<size_t>(8, c->n_buf * 8)));
  K2J_CUDA(c, c->d_buf_chunk_base.reserve((c->n_buf + 1) * 4));
  if (c->n_buf) {
    K2J_CUDA(c, cudaMemcpyAsync(c->d_buf_off.p, c->h_buf_off.data(), c->n_buf * 8, cudaMemcpyHostToDevice, c->stream));
    K2J_CUDA(c, cudaMemcpyAsync(c->d_buf_valid.p, c->h_buf_valid.data(), c->n_buf * 8, cudaMemcpyHostToDevice, c->stream));
  }
  K2J_CUDA(c, cudaMemcpyAsync(c->d_buf_chunk_base.p, c->h_buf_chunk_base.data(), (c->n_buf + 1) * 4, cudaMemcpyHostToDevice, c->stream));
  return K2J_OK;
}

k2j_status k2j_segment(k2j_ctx* c, k2j_segment_info* info) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->have_params) return fail(c, K2J_ERR_STATE, "k2j_set_params has not been called");
  K2J_CUDA(c, cudaSetDevice(c->device));
  c->ran = false; c->segmented = false; c->have_global_join = false; c->need_bits = nullptr;
  cudaStream_t s = c->stream;
  c->launches = 0;

  Dev& d = c->d;
  d = Dev{};
  d.base = c->params.base_time_ns; d.win_start = c->params.window_start_ns; d.win_end = c->params.window_end_ns;
  d.pid = c->params.pid; d.ts_mode = c->params.ts_mode; d.flags = c->params.flags; d.n_devices = c->params.n_devices; d.type_mask = c->params.activity_type_mask;
  d.conv_t0 = c->params.conv_t0; d.conv_t0a = c->params.conv_t0_approx; d.conv_mant = c->params.conv_scale_mant;
  d.conv_exp = c->params.conv_scale_exp;
  d.props = c->d_props.as<DevProps>();
  d.pool_off = (const uint64_t*)c->pool_off.dev; d.pool_data = (const uint8_t*)c->pool_data.dev; d.n_strings = (uint32_t)c->n_strings;
  d.esc_name = c->esc_name.as<uint8_t>(); d.esc_md = c->esc_md.as<uint8_t>();
  d.esc_name_len = c->esc_name_len.as<uint32_t>(); d.esc_md_len = c->esc_md_len.as<uint32_t>();
  d.str_class = c->str_class.as<uint8_t>();
  d.rt_names = (const uint32_t*)c->rt_names.dev; d.n_rt = c->n_rt; d.dr_names = (const uint32_t*)c->dr_names.dev; d.n_dr = c->n_dr;
  d.tid_pairs = (const int32_t*)c->tid_pairs.dev; d.n_tid_pairs = c->n_tid;
  d.cupti = (const uint8_t*)c->cupti.dev; d.cupti_bytes = c->cupti_bytes;
  d.buf_off = c->d_buf_off.as<uint64_t>(); d.buf_valid = c->d_buf_valid.as<uint64_t>();
  d.buf_chunk_base = c->d_buf_chunk_base.as<uint32_t>(); d.n_buf = c->n_buf; d.n_chunks = c->n_chunks;
  d.n_ops = c->n_ops;
  d.op_start = (const int64_t*)c->op_start.dev; d.op_end = (const int64_t*)c->op_end.dev; d.op_id = (const int32_t*)c->op_id.dev;
  d.op_device = (const int32_t*)c->op_device.dev; d.op_resource = (const int64_t*)c->op_resource.dev;
  d.op_thread = (const int32_t*)c->op_thread.dev;
  d.op_type = (const int32_t*)c->op_type.dev; d.op_name = (const uint32_t*)c->op_name.dev; d.op_flow = (const uint32_t*)c->op_flow.dev;
  d.op_flowt = (const uint8_t*)c->op_flowt.dev; d.op_mdoff = (const uint32_t*)c->op_mdoff.dev; d.md = (const MdEntry*)c->op_md.dev;
  d.counters = c->counters.as<Counters>();
  d.n_guest_ops = c->n_guest_ops; d.coll_tab = nullptr;
  d.guest_front = (uint32_t)(c->guest_front_bytes / 8);
  d.guest_back = c->guest_back_bytes == ~0ull ? 0xFFFFFFFFu : (uint32_t)(c->guest_back_bytes / 8);

  K2J_CUDA(c, cudaMemsetAsync(c->counters.p, 0, sizeof(Counters), s));
  K2J_CUDA(c, cudaEventRecord(c->ev[0], s));

  // ---- string pool: sanitised copies (once per pool) ----
  if (c->strings_dirty && c->n_strings) {
    const uint32_t blocks = (uint32_t)((c->n_strings * 32 + 255) / 256);
    k_escape_pool<<<blocks, 256, 0, s>>>(d);
    c->launches++;
    c->strings_dirty = false;
  }

  // ---- segmentation ----
  const uint32_t nch = c->n_chunks;
  const uint32_t seg_blocks = (nch + kSegWarps - 1) / kSegWarps;
  uint64_t* totals = c->totals;
  for (int i = 0; i < C_NCOL; i++) totals[i] = 0;
  if (nch) {
    K2J_CUDA(c, c->slot_code.reserve(c->cupti_bytes / 8 + 64));
    K2J_CUDA(c, c->exit_map.reserve((size_t)nch * 32));
    K2J_CUDA(c, c->walk_cnt.reserve((size_t)nch * 32 * 3 * 4));
    K2J_CUDA(c, c->chunk_entry.reserve(nch));
    K2J_CUDA(c, c->chunk_cnt.reserve((size_t)nch * C_NCOL * 4));
    K2J_CUDA(c, c->chunk_base.reserve((size_t)nch * C_NCOL * 8));
    d.slot_code = c->slot_code.as<uint8_t>(); d.exit_map = c->exit_map.as<uint8_t>(); d.walk_cnt = c->walk_cnt.as<uint32_t>();
    d.chunk_entry = c->chunk_entry.as<uint8_t>(); d.chunk_cnt = c->chunk_cnt.as<uint32_t>();
    d.chunk_base = c->chunk_base.as<uint64_t>();
    k_seg_chunks<<<seg_blocks, kSegWarps * 32, 0, s>>>(d);
    k_seg_compose<<<c->n_buf, 256, 0, s>>>(d);
    c->launches += 2;
    K2J_CUDA(c, cudaGetLastError());
    k2j_status st = run_scan(c, d.chunk_cnt, nch, C_NCOL, d.chunk_base, c->scan_totals.as<uint64_t>(), &c->launches);
    if (st) return st;
    K2J_CUDA(c, cudaMemcpyAsync(c->h_totals, c->scan_totals.p, C_NCOL * 8, cudaMemcpyDeviceToHost, s));
    K2J_CUDA(c, cudaStreamSynchronize(s));
    for (int i = 0; i < C_NCOL; i++) totals[i] = c->h_totals[i];
  }

  // ---- class-sorted work lists, compacted EXTERNAL_CORRELATION records ----
  uint64_t pos = 0;
  for (int cls = 0; cls < C_NCLASS; cls++) {
    d.cls_begin[cls] = pos;
    d.cls_count[cls] = cls == C_EXT ? 0 : totals[cls];
    pos += (d.cls_count[cls] + 31) & ~31ull;
  }
  d.ops_begin = pos;
  d.n_work = pos + c->n_ops;
  d.n_events = c->n_ops + totals[C_EVENTS] + totals[C_WAIT];
  d.wait_ev_base = c->n_ops + totals[C_EVENTS];
  if (d.n_events >= 0xFFFFFFF0ull) return fail(c, K2J_ERR_INVALID_ARGUMENT, "more than 2^32 events in one call");
  K2J_CUDA(c, c->work_slot.reserve(std::max<uint64_t>(1, pos) * 4));
  K2J_CUDA(c, c->work_ev.reserve(std::max<uint64_t>(1, pos) * 4));
  K2J_CUDA(c, c->ext_local.reserve(std::max<uint64_t>(1, totals[C_EXT]) * sizeof(ExtRec)));
  d.work_slot = c->work_slot.as<uint32_t>(); d.work_ev = c->work_ev.as<uint32_t>();
  d.ext_local = c->ext_local.as<ExtRec>();
  if (nch) { k_seg_write<<<seg_blocks, kSegWarps * 32, 0, s>>>(d); c->launches++; }
  K2J_CUDA(c, cudaGetLastError());
  K2J_CUDA(c, cudaEventRecord(c->ev[1], s));
  c->segmented = true;
  if (info) {
    info->n_records = totals[C_EVENTS] + totals[C_WAIT] + totals[C_EXT] + totals[C_UNEXPECTED];
    info->n_external = totals[C_EXT];
    info->external_records = reinterpret_cast<const k2j_external_record*>(d.ext_local);
    info->n_ops = c->n_ops - c->n_guest_ops;
    info->n_user_external = totals[C_USER];
    info->op_ids = d.op_id;
    K2J_CUDA(c, cudaStreamSynchronize(s));  // the arrays above are complete when this returns
  }
  return K2J_OK;
}

k2j_status k2j_set_global_join(k2j_ctx* c, const void* ext_all, uint64_t n_ext_all, uint64_t own_begin,
                               const int32_t* op_ids_all, uint64_t n_ops_all) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->segmented) return fail(c, K2J_ERR_STATE, "k2j_segment has not run");
  if ((n_ext_all && !ext_all) || (n_ops_all && !op_ids_all)) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null join arrays");
  if ((n_ext_all && !is_device_ptr(ext_all)) || (n_ops_all && !is_device_ptr(op_ids_all)))
    return fail(c, K2J_ERR_INVALID_ARGUMENT, "gathered join arrays must be device memory");
  if (n_ext_all >= 0xFFFFFFF0ull || n_ops_all >= 0xFFFFFFF0ull || own_begin + c->totals[C_EXT] > n_ext_all)
    return fail(c, K2J_ERR_INVALID_ARGUMENT, "gathered join arrays out of range");
  c->g_ext = ext_all; c->g_n_ext = n_ext_all; c->g_own_begin = own_begin;
  c->g_op_ids = op_ids_all; c->g_n_ops = n_ops_all;
  c->g_counts = nullptr; c->g_world = 1; c->g_rank = 0; c->g_op_bits = nullptr; c->join_user_hint = -1;
  c->have_global_join = true;
  return K2J_OK;
}

k2j_status k2j_set_global_join_rows(k2j_ctx* c, const void* ext_rows, uint64_t ext_stride, const int32_t* op_id_rows, uint64_t ops_stride,
                                    uint64_t row_pitch_bytes, const uint64_t* counts, uint32_t world, uint32_t rank) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->segmented) return fail(c, K2J_ERR_STATE, "k2j_segment has not run");
  if (!ext_rows || !op_id_rows || !counts || world == 0 || rank >= world) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null join rows");
  if (!is_device_ptr(ext_rows) || !is_device_ptr(op_id_rows) || !is_device_ptr(counts))
    return fail(c, K2J_ERR_INVALID_ARGUMENT, "gathered join rows must be device memory");
  if (ext_stride == 0 || ops_stride == 0 || ext_stride * world >= 0xFFFFFFF0ull || ops_stride * world >= 0xFFFFFFF0ull ||
      c->totals[C_EXT] > ext_stride || c->n_ops - c->n_guest_ops > ops_stride || (row_pitch_bytes & 7))
    return fail(c, K2J_ERR_INVALID_ARGUMENT, "join rows: stride smaller than this shard's share, or out of range");
  c->g_ext = ext_rows; c->g_n_ext = ext_stride * world; c->g_own_begin = ext_stride * rank;
  c->g_op_ids = op_id_rows; c->g_n_ops = ops_stride * world;
  c->g_ext_stride = (uint32_t)ext_stride; c->g_ops_stride = (uint32_t)ops_stride; c->g_pitch = row_pitch_bytes;
  c->g_counts = counts; c->g_world = world; c->g_rank = rank; c->g_op_bits = nullptr; c->join_user_hint = -1;
  c->have_global_join = true;
  return K2J_OK;
}

k2j_status k2j_set_join_user_records(k2j_ctx* c, int any) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->have_global_join) return fail(c, K2J_ERR_STATE, "k2j_set_global_join has not been called");
  c->join_user_hint = any ? 1 : 0;
  return K2J_OK;
}

k2j_status k2j_op_id_bits(k2j_ctx* c, int64_t min_id, uint64_t n_bits, void* bits) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->segmented) return fail(c, K2J_ERR_STATE, "k2j_segment has not run");
  if (!bits || !is_device_ptr(bits) || n_bits == 0 || (n_bits & 31) || n_bits > (1ull << 33))
    return fail(c, K2J_ERR_INVALID_ARGUMENT, "op id bits: device memory, a multiple of 32 bits, at most 2^33");
  K2J_CUDA(c, cudaSetDevice(c->device));
  cudaStream_t s = c->stream;
  const Dev& d = c->d;
  K2J_CUDA(c, cudaMemsetAsync(bits, 0, n_bits / 8, s));
  K2J_CUDA(c, cudaMemsetAsync(d.counters, 0, sizeof(Counters), s));
  const uint64_t n = c->n_ops - c->n_guest_ops;
  if (n) { k_op_id_bits<<<(uint32_t)((n + 255) / 256), 256, 0, s>>>(d, min_id, n_bits, static_cast<uint32_t*>(bits)); c->launches++; }
  K2J_CUDA(c, cudaGetLastError());
  K2J_CUDA(c, cudaMemcpyAsync(c->h_counters, d.counters, sizeof(Counters), cudaMemcpyDeviceToHost, s));
  K2J_CUDA(c, cudaStreamSynchronize(s));
  if (c->h_counters->device_check) return fail(c, K2J_ERR_INVALID_ARGUMENT, "op id bits: an id of this shard lies outside [min_id, min_id + n_bits)");
  return K2J_OK;
}

k2j_status k2j_set_global_op_bits(k2j_ctx* c, const void* bit_rows, uint64_t row_pitch_bytes, const int64_t* meta) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->have_global_join || !c->g_counts) return fail(c, K2J_ERR_STATE, "k2j_set_global_join_rows has not been called");
  if (!bit_rows || !meta || !is_device_ptr(bit_rows) || !is_device_ptr(meta) || (row_pitch_bytes & 3))
    return fail(c, K2J_ERR_INVALID_ARGUMENT, "op id bits: device memory, rows a multiple of 4 bytes apart");
  c->g_op_bits = static_cast<const uint32_t*>(bit_rows); c->g_op_bits_pitch = row_pitch_bytes; c->g_op_bits_meta = meta;
  return K2J_OK;
}

k2j_status k2j_join_need_bits(k2j_ctx* c, void* bits, uint64_t n_bits) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->segmented) return fail(c, K2J_ERR_STATE, "k2j_segment has not run");
  if (!bits || !is_device_ptr(bits) || n_bits < 1024 || (n_bits & (n_bits - 1)) || n_bits > (1ull << 32))
    return fail(c, K2J_ERR_INVALID_ARGUMENT, "need bits: device memory and a power of two between 2^10 and 2^32 bits");
  K2J_CUDA(c, cudaSetDevice(c->device));
  cudaStream_t s = c->stream;
  Dev d = c->d;
  d.need_corr = static_cast<uint32_t*>(bits); d.need_corr_mask = (uint32_t)(n_bits - 1);
  K2J_CUDA(c, cudaMemsetAsync(bits, 0, n_bits / 8, s));
  if (d.ops_begin) { k_mark_corr<<<(uint32_t)((d.ops_begin + 255) / 256), 256, 0, s>>>(d); c->launches++; }
  K2J_CUDA(c, cudaGetLastError());
  c->need_bits = static_cast<uint32_t*>(bits); c->need_n_bits = n_bits;  // k2j_emit tests the gathered keys against the same filter
  return K2J_OK;
}

k2j_status k2j_filter_join_keys(k2j_ctx* c, const void* need_rows, uint64_t row_pitch_bytes, uint64_t n_bits, uint32_t world, uint32_t rank,
                                void* out_records, uint64_t capacity, uint64_t* n_out) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->segmented) return fail(c, K2J_ERR_STATE, "k2j_segment has not run");
  const uint64_t n = c->totals[C_EXT];
  if (!need_rows || !is_device_ptr(need_rows) || !n_out || !is_device_ptr(n_out) || world == 0 || rank >= world || n_bits < 1024 ||
      (n_bits & (n_bits - 1)) || n_bits > (1ull << 32) || (row_pitch_bytes & 3) || row_pitch_bytes < n_bits / 8 ||
      (n && (!out_records || !is_device_ptr(out_records))) || capacity < n)
    return fail(c, K2J_ERR_INVALID_ARGUMENT, "filter: device memory, a power-of-two filter size, room for every record of this shard");
  K2J_CUDA(c, cudaSetDevice(c->device));
  cudaStream_t s = c->stream;
  const Dev& d = c->d;
  K2J_CUDA(c, c->ev_size.reserve(std::max<uint64_t>(1, n) * 4));   // scratch: marks and their scan (free between segment and emit)
  K2J_CUDA(c, c->ev_off.reserve(std::max<uint64_t>(1, n) * 8));
  if (n) {
    k_flag_wanted<<<(uint32_t)((n + 255) / 256), 256, 0, s>>>(d, static_cast<const uint32_t*>(need_rows), row_pitch_bytes / 4, world, rank,
                                                             (uint32_t)(n_bits - 1), n, c->ev_size.as<uint32_t>());
    c->launches++;
    K2J_CUDA(c, cudaGetLastError());
    k2j_status st = run_scan(c, c->ev_size.as<uint32_t>(), n, 1, c->ev_off.as<uint64_t>(), c->scan_totals.as<uint64_t>() + 27, &c->launches);
    if (st) return st;
    k_take_wanted<<<(uint32_t)((n + 255) / 256), 256, 0, s>>>(d, c->ev_size.as<uint32_t>(), c->ev_off.as<uint64_t>(), n, static_cast<ExtRec*>(out_records));
    c->launches++;
    K2J_CUDA(c, cudaMemcpyAsync(n_out, c->scan_totals.as<uint64_t>() + 27, 8, cudaMemcpyDeviceToDevice, s));
  } else K2J_CUDA(c, cudaMemsetAsync(n_out, 0, 8, s));
  K2J_CUDA(c, cudaGetLastError());
  return K2J_OK;
}

k2j_status k2j_set_guest_ranges(k2j_ctx* c, uint64_t front_end_bytes, uint64_t back_begin_bytes) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if ((front_end_bytes & 7) || (back_begin_bytes & 7) || front_end_bytes > back_begin_bytes || back_begin_bytes > c->cupti_bytes)
    return fail(c, K2J_ERR_INVALID_ARGUMENT, "guest ranges: not 8-byte aligned, crossing, or past the end of the CUPTI bytes");
  for (size_t b = 0; b < c->h_buf_off.size(); b++) {  // a buffer is a guest buffer or this shard's own, never both
    const uint64_t lo = c->h_buf_off[b], hi = lo + c->h_buf_valid[b];
    const bool own = lo >= front_end_bytes && hi <= back_begin_bytes, guest = hi <= front_end_bytes || lo >= back_begin_bytes;
    if (!own && !guest) return fail(c, K2J_ERR_INVALID_ARGUMENT, "guest ranges: buffer %zu straddles a boundary", b);
  }
  c->guest_front_bytes = front_end_bytes; c->guest_back_bytes = back_begin_bytes; c->guests_declared = true;
  c->segmented = false;  // the next k2j_segment picks the ranges up
  return K2J_OK;
}

k2j_status k2j_partial_spans(k2j_ctx* c, const k2j_span** spans, uint64_t* n_spans) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!spans || !n_spans) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null result pointers");
  if (!c->ran && !c->streamed) return fail(c, K2J_ERR_STATE, "no completed run");
  static_assert(sizeof(k2j_span) == sizeof(SpanRec), "k2j_span is SpanRec");
  *spans = reinterpret_cast<const k2j_span*>(c->partial_spans.data());
  *n_spans = c->partial_spans.size();
  return K2J_OK;
}

k2j_status k2j_append_spans(k2j_ctx* c, const k2j_span* spans, uint64_t n_spans, uint64_t* n_bytes) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->ran) return fail(c, K2J_ERR_STATE, "no completed run whose text is in the context");
  if ((!spans && n_spans) || n_spans >= 0x7FFFFFF0ull) return fail(c, K2J_ERR_INVALID_ARGUMENT, "bad span list");
  K2J_CUDA(c, cudaSetDevice(c->device));
  cudaStream_t s = c->stream;
  Dev& d = c->d;
  std::vector<SpanRec> list(n_spans);
  if (n_spans) memcpy(list.data(), spans, n_spans * sizeof(SpanRec));
  for (const SpanRec& r : list)
    if (r.op_row != 0xFFFFFFFFu && r.op_row >= c->n_ops) return fail(c, K2J_ERR_INVALID_ARGUMENT, "span names a row past the CPU-side activities");
  uint32_t n = 0;
  uint64_t ann_bytes = 0;
  K2J_CUDA(c, cudaMemsetAsync(d.counters, 0, sizeof(Counters), s));
  k2j_status st = size_annotations(c, list, &n, &ann_bytes);
  if (st) return st;
  if (ann_bytes) {
    if (c->out.cap < c->out_bytes + ann_bytes + 64) {  // the text so far moves into a larger allocation
      DevBuf bigger;
      K2J_CUDA(c, bigger.reserve(c->out_bytes + ann_bytes + 64));
      if (c->out_bytes) K2J_CUDA(c, cudaMemcpyAsync(bigger.p, c->out.p, c->out_bytes, cudaMemcpyDeviceToDevice, s));
      K2J_CUDA(c, cudaStreamSynchronize(s));
      c->out.release();
      c->out = bigger;
    }
    d.out = c->out.as<uint8_t>(); d.out_cap = c->out_bytes + ann_bytes;
    k_annotations<true><<<(n + kEventThreads - 1) / kEventThreads, kEventThreads, 0, s>>>(
        d, c->span_out.as<SpanRec>(), n, c->ann_size.as<uint32_t>(), c->ann_off.as<uint64_t>(), c->out_bytes);
    c->launches++;
    K2J_CUDA(c, cudaGetLastError());
  }
  K2J_CUDA(c, cudaMemcpyAsync(c->h_counters, d.counters, sizeof(Counters), cudaMemcpyDeviceToHost, s));
  K2J_CUDA(c, cudaStreamSynchronize(s));
  if (c->h_counters->device_check) { c->ran = false; return fail(c, K2J_ERR_DEVICE_CHECK, "a device-side check failed while the spans were written"); }
  c->out_bytes += ann_bytes;
  if (n_bytes) *n_bytes = ann_bytes;
  return K2J_OK;
}

k2j_status k2j_set_guest_ops(k2j_ctx* c, uint64_t n_guest_ops) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (n_guest_ops > c->n_ops) return fail(c, K2J_ERR_INVALID_ARGUMENT, "more guest rows than CPU-side activities");
  c->n_guest_ops = n_guest_ops;
  c->segmented = false;
  return K2J_OK;
}

k2j_status k2j_export_lookup_records(k2j_ctx* c, const void** records, uint64_t* n_bytes) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!records || !n_bytes) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null result pointers");
  if (!c->segmented) return fail(c, K2J_ERR_STATE, "k2j_segment has not run");
  if (c->guests_declared) return fail(c, K2J_ERR_STATE, "lookup records are exported from a shard's own buffers, before guests are added");
  K2J_CUDA(c, cudaSetDevice(c->device));
  cudaStream_t s = c->stream;
  Dev d = c->d;
  const uint64_t* totals = c->totals;
  constexpr uint32_t kCtxCap = 1u << 14, kKeyCap = 1u << 16, kListCap = kCtxCap + 2 * kKeyCap;
  K2J_CUDA(c, c->ctx_tab.reserve((size_t)kCtxCap * 8));
  K2J_CUDA(c, c->exp_keys.reserve((size_t)kKeyCap * 8 * 2));
  K2J_CUDA(c, c->exp_first.reserve((size_t)kKeyCap * 4 * 2 + 16));
  K2J_CUDA(c, c->exp_list.reserve((size_t)kListCap * 8));
  d.ctx_tab = c->ctx_tab.as<unsigned long long>(); d.ctx_mask = kCtxCap - 1;
  unsigned long long* pair_key = c->exp_keys.as<unsigned long long>();
  unsigned long long* sync_key = pair_key + kKeyCap;
  uint32_t* pair_first = c->exp_first.as<uint32_t>();
  uint32_t* sync_first = pair_first + kKeyCap;
  uint32_t* n_list = sync_first + kKeyCap;
  K2J_CUDA(c, cudaMemsetAsync(d.ctx_tab, 0, (size_t)kCtxCap * 8, s));
  K2J_CUDA(c, cudaMemsetAsync(pair_key, 0, (size_t)kKeyCap * 8 * 2, s));
  K2J_CUDA(c, cudaMemsetAsync(pair_first, 0xFF, (size_t)kKeyCap * 4 * 2, s));
  K2J_CUDA(c, cudaMemsetAsync(n_list, 0, 16, s));
  K2J_CUDA(c, cudaMemsetAsync(d.counters, 0, sizeof(Counters), s));
  const uint64_t n_named = d.cls_begin[C_OVERHEAD] - d.cls_begin[C_KERNEL];
  if (n_named) k_build_ctx<<<(uint32_t)((n_named + 255) / 256), 256, 0, s>>>(d);
  const uint64_t n_sel = d.cls_begin[C_SYNC] + d.cls_count[C_SYNC] - d.cls_begin[C_KERNEL];
  if (n_sel) k_export_select<<<(uint32_t)((n_sel + 255) / 256), 256, 0, s>>>(d, pair_key, pair_first, sync_key, sync_first, kKeyCap - 1);
  k_export_list<<<(kListCap + 255) / 256, 256, 0, s>>>(d, pair_key, pair_first, sync_key, sync_first, kKeyCap - 1,
                                                       c->exp_list.as<unsigned long long>(), n_list, kListCap);
  K2J_CUDA(c, cudaGetLastError());
  uint32_t n = 0;
  K2J_CUDA(c, cudaMemcpyAsync(&n, n_list, 4, cudaMemcpyDeviceToHost, s));
  K2J_CUDA(c, cudaMemcpyAsync(c->h_counters, d.counters, sizeof(Counters), cudaMemcpyDeviceToHost, s));
  K2J_CUDA(c, cudaStreamSynchronize(s));
  if (c->h_counters->device_check || n > kListCap)
    return fail(c, K2J_ERR_DEVICE_CHECK, "more contexts or (device, stream) pairs than the export tables hold");
  // in processing order, each record once: a record's place among the exported ones decides ties between them
  std::vector<unsigned long long> list(n);
  if (n) K2J_CUDA(c, cudaMemcpy(list.data(), c->exp_list.p, (size_t)n * 8, cudaMemcpyDeviceToHost));
  std::sort(list.begin(), list.end());
  list.erase(std::unique(list.begin(), list.end()), list.end());
  uint64_t at = 0;
  for (auto& e : list) { const uint32_t len = (uint32_t)e; e = (e & 0xFFFFFFFF00000000ull) | at; at += len; }
  if (at >= (1ull << 32)) return fail(c, K2J_ERR_UNSUPPORTED, "more than 4 GiB of lookup records");
  const uint64_t n_events = totals[C_CUDAEVENT], total = at + 56 * n_events;
  K2J_CUDA(c, c->exp_out.reserve(std::max<uint64_t>(8, total)));
  if (!list.empty()) K2J_CUDA(c, cudaMemcpyAsync(c->exp_list.p, list.data(), list.size() * 8, cudaMemcpyHostToDevice, s));
  if (list.size() + n_events)
    k_export_copy<<<(uint32_t)((list.size() + n_events + 255) / 256), 256, 0, s>>>(d, c->exp_list.as<unsigned long long>(), (uint32_t)list.size(),
                                                                              c->exp_out.as<uint8_t>(), at);
  K2J_CUDA(c, cudaGetLastError());
  K2J_CUDA(c, cudaStreamSynchronize(s));  // `list` is read by the upload above; the records are complete when this returns
  *records = c->exp_out.p;
  *n_bytes = total;
  return K2J_OK;
}

}  // extern "C"

namespace {

// Where a tiled run sends its text.
struct TileSink {
  int mode = 0;              // 0: the whole text stays in the context; 1: host memory; 2: a file descriptor
  uint8_t* host = nullptr;   // mode 1
  uint64_t capacity = 0;
  int fd = -1;               // mode 2
  uint64_t slab_bytes = 0;
};
constexpr uint64_t kSlabMargin = 1ull << 20;   // a slab holds the events that START in its range: room for the last one's end
constexpr uint64_t kSlabPad = 64;              // bytes in front of a slab's text (an event's first store may begin before it)

k2j_status stream_bytes(k2j_ctx* c, const uint8_t* src, int fd, bool positioned, uint64_t file_offset, uint64_t total, cudaStream_t stream);

// The emit launches for the events whose text starts in [d.tile_begin, d.tile_end).  `ranges`: per class the work
// items to look at ([begin, end) pairs, C_API .. C_WAIT, then the CPU-side activities); nullptr: everything.
k2j_status launch_emit(k2j_ctx* c, const Dev& d, const uint64_t* ranges, bool instant, uint64_t n_coll, cudaStream_t s) {
  auto launch = [&](uint64_t begin, uint64_t end) {
    if (end <= begin) return;
    Dev dr = d;
    dr.work_origin = begin; dr.n_work = end;
    k_events<true><<<(uint32_t)((end - begin + kEventThreads - 1) / kEventThreads), kEventThreads, events_smem_bytes(true), s>>>(dr);
    c->launches++;
  };
  if (!ranges) launch(0, d.n_work);
  else for (int k = 0; k <= C_EXT; k++) launch(ranges[2 * k], ranges[2 * k + 1]);
  if (instant && c->n_ops) {
    // instant events: the same extra launch over the CPU-side activities
    Dev di = d;
    di.work_origin = ranges ? ranges[2 * C_EXT] : d.ops_begin;
    di.n_work = ranges ? ranges[2 * C_EXT + 1] : d.n_work;
    if (di.n_work > di.work_origin) {
      k_events<true, true><<<(uint32_t)((di.n_work - di.work_origin + kEventThreads - 1) / kEventThreads), kEventThreads, events_smem_bytes(true), s>>>(di);
      c->launches++;
    }
  }
  if (n_coll != 0) {
    // kernel events that carry collective metadata: a launch of their own over the work items the size pass
    // listed, so that the launch above holds no code for them
    Dev dk = d;
    dk.work_indirect = d.coll_list; dk.n_indirect = n_coll;
    k_events<true, true><<<(uint32_t)((dk.n_indirect + kEventThreads - 1) / kEventThreads), kEventThreads, events_smem_bytes(true), s>>>(dk);
    c->launches++;
  }
  K2J_CUDA(c, cudaGetLastError());
  return K2J_OK;
}

k2j_status emit_core(k2j_ctx* c, k2j_result* res, const TileSink& sink) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!res) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null result");
  if (!c->segmented) return fail(c, K2J_ERR_STATE, "k2j_segment has not run");
  K2J_CUDA(c, cudaSetDevice(c->device));
  memset(res, 0, sizeof *res);
  c->ran = false; c->streamed = false;
  cudaStream_t s = c->stream;
  Dev& d = c->d;
  const uint64_t* totals = c->totals;
  const uint64_t n_gpu_events = totals[C_EVENTS] + totals[C_WAIT];
  const uint64_t n_sync = totals[C_SYNC] + totals[C_WAIT], n_cuda_events = totals[C_CUDAEVENT];
  if (n_sync + n_cuda_events > 0 && c->have_global_join && !c->guests_declared)
    return fail(c, K2J_ERR_UNSUPPORTED, "synchronisation and CUDA event records of a sharded trace need the other shards' lookup records "
                                        "(k2j_export_lookup_records, k2j_set_guest_ranges)");
  K2J_CUDA(c, cudaEventRecord(c->ev[6], s));
  // every counter belongs to the emit step (segmentation counts through its scan columns): a second k2j_emit after
  // one k2j_segment starts from zero, and an earlier failed check does not fail this run
  K2J_CUDA(c, cudaMemsetAsync(d.counters, 0, sizeof(Counters), s));

  // ---- join tables ----
  uint64_t own_begin = 0, own_end = totals[C_EXT];
  if (c->have_global_join) {
    d.ext_all = (const ExtRec*)c->g_ext; d.n_ext_all = c->g_n_ext;
    d.join_op_ids = c->g_op_ids; d.n_join_ops = c->g_n_ops;
    d.join_counts = c->g_counts; d.ext_stride = c->g_ext_stride; d.ops_stride = c->g_ops_stride; d.join_pitch = c->g_pitch;
    d.own_rank = c->g_counts ? c->g_rank : 0xFFFFFFFFu; d.own_n_ext = totals[C_EXT]; d.own_n_ops = c->n_ops - c->n_guest_ops;
    d.op_bits = c->g_op_bits; d.op_bits_pitch = c->g_op_bits_pitch / 4; d.op_bits_meta = c->g_op_bits_meta; d.op_bits_world = c->g_world;
    own_begin = c->g_own_begin; own_end = own_begin + totals[C_EXT];
  } else {
    d.ext_all = d.ext_local; d.n_ext_all = totals[C_EXT];
    d.join_op_ids = d.op_id; d.n_join_ops = c->n_ops - c->n_guest_ops;
    d.join_counts = nullptr; d.own_rank = 0xFFFFFFFFu; d.op_bits = nullptr;
  }
  K2J_CUDA(c, c->ev_size.reserve(std::max<uint64_t>(1, d.n_events) * 4));
  K2J_CUDA(c, c->ev_off.reserve(std::max<uint64_t>(1, d.n_events) * 8));
  K2J_CUDA(c, c->ev_ext.reserve(std::max<uint64_t>(1, d.n_events) * 4));
  d.ev_size = c->ev_size.as<uint32_t>(); d.ev_off = c->ev_off.as<uint64_t>(); d.ev_ext = c->ev_ext.as<int32_t>();
  // With gathered keys only those this shard's events can look up enter its tables (see k_mark_corr), so the tables
  // are sized by the shard: its events, plus the share of foreign keys the marking lets through by chance.
  const bool filter = c->have_global_join;
  // (a filtered table holds at most the bound below, usually about half of it: 1.4 slots per possible key are enough)
  // (the shard's own records go in untested)
  const uint32_t corr_cap = filter ? pow2_at_least(14 * std::min<uint64_t>(d.n_ext_all, totals[C_EXT] + n_gpu_events + d.n_ext_all / 16 + 1024) / 10 + 2)
                                   : pow2_at_least(2 * d.n_ext_all + 2);
  const uint32_t op_cap = filter ? pow2_at_least(14 * std::min<uint64_t>(d.n_join_ops, n_gpu_events + d.n_join_ops / 16 + 1024) / 10 + 2)
                                 : pow2_at_least(2 * d.n_join_ops + 2);
  K2J_CUDA(c, c->corr_tab.reserve((size_t)corr_cap * 8));
  K2J_CUDA(c, c->user_tab.reserve((size_t)corr_cap * 8));
  K2J_CUDA(c, c->op_tab.reserve((size_t)op_cap * 8));
  d.corr_tab = c->corr_tab.as<unsigned long long>(); d.corr_mask = corr_cap - 1;
  d.user_tab = c->user_tab.as<unsigned long long>(); d.user_mask = corr_cap - 1;
  d.op_tab = c->op_tab.as<unsigned long long>(); d.op_mask = op_cap - 1;
  K2J_CUDA(c, cudaMemsetAsync(d.corr_tab, 0, (size_t)corr_cap * 8, s));
  K2J_CUDA(c, c->corr0.reserve(16));
  d.corr0 = c->corr0.as<unsigned long long>();
  K2J_CUDA(c, cudaMemsetAsync(d.corr0, 0, 16, s));
  // the user-annotation table is only written and read when CUSTOM1 correlation records exist
  // (several shards: another shard's CUSTOM1 records may name this shard's events, so the local count says nothing,
  // unless the caller has said that no shard holds any)
  const bool user_records = c->have_global_join ? c->join_user_hint != 0 : totals[C_USER] > 0;
  if (user_records) K2J_CUDA(c, cudaMemsetAsync(d.user_tab, 0, (size_t)corr_cap * 8, s));
  else d.user_tab = nullptr;
  K2J_CUDA(c, cudaMemsetAsync(d.op_tab, 0, (size_t)op_cap * 8, s));
  const uint32_t tid_cap = std::max<uint32_t>(16384, pow2_at_least(4ull * c->n_tid));
  K2J_CUDA(c, c->tid_tab.reserve((size_t)tid_cap * 8));
  d.tid_tab = c->tid_tab.as<unsigned long long>(); d.tid_mask = tid_cap - 1;
  K2J_CUDA(c, cudaMemsetAsync(d.tid_tab, 0, (size_t)tid_cap * 8, s));
  if (c->n_tid + c->n_ops) { k_build_tids<<<(uint32_t)((c->n_tid + c->n_ops + 255) / 256), 256, 0, s>>>(d); c->launches++; }
  // user-annotation span tables (single-shard runs only)
  const bool spans_on = (c->params.flags & K2J_FLAG_USER_ANNOTATIONS) && user_records;
  d.span_key = nullptr;
  uint32_t span_cap = 0;
  if (spans_on) {
    span_cap = pow2_at_least(2 * (c->have_global_join ? std::min<uint64_t>(c->g_n_ext, n_gpu_events) : totals[C_USER]) + 16);
    const uint32_t ds_cap = 1u << 16;
    K2J_CUDA(c, c->ds_tab.reserve((size_t)ds_cap * 8));
    K2J_CUDA(c, c->span_key.reserve((size_t)span_cap * 8));
    K2J_CUDA(c, c->span_nstart.reserve((size_t)span_cap * 8));
    K2J_CUDA(c, c->span_end.reserve((size_t)span_cap * 8));
    K2J_CUDA(c, c->span_nfirst.reserve((size_t)span_cap * 8));
    K2J_CUDA(c, c->span_row.reserve((size_t)span_cap * 4));
    d.ds_tab = c->ds_tab.as<unsigned long long>(); d.ds_mask = ds_cap - 1;
    d.span_key = c->span_key.as<unsigned long long>(); d.span_nstart = c->span_nstart.as<unsigned long long>();
    d.span_end = c->span_end.as<unsigned long long>(); d.span_nfirst = c->span_nfirst.as<unsigned long long>();
    d.span_row = c->span_row.as<uint32_t>(); d.span_mask = span_cap - 1;
    K2J_CUDA(c, cudaMemsetAsync(d.ds_tab, 0, (size_t)ds_cap * 8, s));
    K2J_CUDA(c, cudaMemsetAsync(d.span_key, 0, (size_t)span_cap * 8, s));
    K2J_CUDA(c, cudaMemsetAsync(d.span_nstart, 0, (size_t)span_cap * 8, s));
    K2J_CUDA(c, cudaMemsetAsync(d.span_end, 0, (size_t)span_cap * 8, s));
    K2J_CUDA(c, cudaMemsetAsync(d.span_nfirst, 0, (size_t)span_cap * 8, s));
  }
  d.need_corr = nullptr; d.need_op = nullptr;
  if (filter) {
    const uint32_t corr_bits = std::max<uint32_t>(1u << 20, pow2_at_least(8 * std::max<uint64_t>(1, n_gpu_events)));
    const uint32_t op_bits = corr_bits;
    K2J_CUDA(c, c->need_op.reserve(op_bits / 8));
    d.need_op = c->need_op.as<uint32_t>(); d.need_op_mask = op_bits - 1;
    K2J_CUDA(c, cudaMemsetAsync(d.need_op, 0, op_bits / 8, s));
    if (c->need_bits) {  // the filter the caller had filled for the exchange (k2j_join_need_bits): the same marks
      d.need_corr = c->need_bits; d.need_corr_mask = (uint32_t)(c->need_n_bits - 1);
    } else {
      K2J_CUDA(c, c->need_corr.reserve(corr_bits / 8));
      d.need_corr = c->need_corr.as<uint32_t>(); d.need_corr_mask = corr_bits - 1;
      K2J_CUDA(c, cudaMemsetAsync(d.need_corr, 0, corr_bits / 8, s));
      if (d.ops_begin) { k_mark_corr<<<(uint32_t)((d.ops_begin + 255) / 256), 256, 0, s>>>(d); c->launches++; }
    }
  }
  // collective enrichment: kernels look at their linked op's name only if some op is a record_param_comms call;
  // ops of other shards carry no metadata here, so sharded runs do not enrich
  d.has_comms = nullptr;
  if (c->n_ops && c->n_strings) {
    K2J_CUDA(c, c->comms_flag.reserve(16));
    K2J_CUDA(c, cudaMemsetAsync(c->comms_flag.p, 0, 4, s));
    k_find_comms<<<(uint32_t)((c->n_ops + 255) / 256), 256, 0, s>>>(d, c->comms_flag.as<uint32_t>(), 1);
    c->launches++;
    d.has_comms = c->comms_flag.as<uint32_t>();
    if (c->have_global_join) {
      // several shards: the join's table holds positions in the gathered keys, so the record_param_comms ops that carry
      // metadata here (this shard's rows and the guest rows) get an id -> row table of their own
      const uint32_t coll_cap = pow2_at_least(2 * c->n_ops + 16);
      K2J_CUDA(c, c->coll_tab.reserve((size_t)coll_cap * 8));
      d.coll_tab = c->coll_tab.as<unsigned long long>(); d.coll_mask = coll_cap - 1;
      K2J_CUDA(c, cudaMemsetAsync(d.coll_tab, 0, (size_t)coll_cap * 8, s));
      k_build_coll<<<(uint32_t)((c->n_ops + 255) / 256), 256, 0, s>>>(d);
      c->launches++;
    }
  }
  d.work_indirect = nullptr; d.n_indirect = 0; d.coll_list = nullptr;
  if (d.has_comms && totals[C_KERNEL]) {
    K2J_CUDA(c, c->coll_list.reserve(totals[C_KERNEL] * 4));
    d.coll_list = c->coll_list.as<uint32_t>();
  }
  // synchronisation and CUDA event records: their lookup structures exist only when such records do
  d.ctx_tab = nullptr; d.evt = nullptr; d.n_evt = 0; d.seen_tab = nullptr; d.row_key = nullptr; d.row_first = nullptr; d.corr_zero = nullptr;
  d.work_origin = 0; d.wait_pass = 0;
  if (n_sync + n_cuda_events > 0) {
    K2J_CUDA(c, c->corr_zero.reserve(corr_cap / 8 + 8));
    d.corr_zero = c->corr_zero.as<uint32_t>();
    K2J_CUDA(c, cudaMemsetAsync(d.corr_zero, 0, corr_cap / 8 + 8, s));
    const uint32_t ctx_cap = 1u << 14;   // distinct CUDA contexts of one trace: a few per device
    K2J_CUDA(c, c->ctx_tab.reserve((size_t)ctx_cap * 8));
    d.ctx_tab = c->ctx_tab.as<unsigned long long>(); d.ctx_mask = ctx_cap - 1;
    K2J_CUDA(c, cudaMemsetAsync(d.ctx_tab, 0, (size_t)ctx_cap * 8, s));
    const uint64_t n_named = d.cls_begin[C_OVERHEAD] - d.cls_begin[C_KERNEL];
    if (n_named) { k_build_ctx<<<(uint32_t)((n_named + 255) / 256), 256, 0, s>>>(d); c->launches++; }
    if (n_sync && n_cuda_events) {
      k2j_status st = sort_cuda_events(c, n_cuda_events);
      if (st) return st;
    }
    if (totals[C_WAIT]) {
      const uint32_t seen_cap = 1u << 16;  // (device, stream) pairs
      K2J_CUDA(c, c->seen_tab.reserve((size_t)seen_cap * 8));
      d.seen_tab = c->seen_tab.as<unsigned long long>(); d.seen_mask = seen_cap - 1;
      K2J_CUDA(c, cudaMemsetAsync(d.seen_tab, 0, (size_t)seen_cap * 8, s));
    }
    if (totals[C_SYNC]) {
      const uint32_t row_cap = pow2_at_least(2 * totals[C_SYNC] + 16);
      K2J_CUDA(c, c->row_key.reserve((size_t)row_cap * 8));
      K2J_CUDA(c, c->row_first.reserve((size_t)row_cap * 4));
      d.row_key = c->row_key.as<unsigned long long>(); d.row_first = c->row_first.as<uint32_t>(); d.row_mask = row_cap - 1;
      K2J_CUDA(c, cudaMemsetAsync(d.row_key, 0, (size_t)row_cap * 8, s));
      K2J_CUDA(c, cudaMemsetAsync(d.row_first, 0xFF, (size_t)row_cap * 4, s));
    }
  }
  if (d.n_ext_all) { k_build_corr<<<(uint32_t)((d.n_ext_all + 255) / 256), 256, 0, s>>>(d, own_begin, own_end); c->launches++; }
  if (d.op_bits != nullptr) {  // the other shards' ids came as bitmaps: the table holds this shard's own ids only
    const uint64_t first = (uint64_t)c->g_ops_stride * c->g_rank, last = first + d.own_n_ops;
    if (last > first) { k_build_ops<<<(uint32_t)((last - first + 255) / 256), 256, 0, s>>>(d, first, last); c->launches++; }
  } else if (d.n_join_ops) { k_build_ops<<<(uint32_t)((d.n_join_ops + 255) / 256), 256, 0, s>>>(d, 0, d.n_join_ops); c->launches++; }
  if (d.n_ext_all) { k_resolve_corr<<<(corr_cap + 255) / 256, 256, 0, s>>>(d); c->launches++; }
  K2J_CUDA(c, cudaGetLastError());
  K2J_CUDA(c, cudaEventRecord(c->ev[2], s));

  // ---- optional: GPU-side events in stable order of their start timestamp ----
  if ((c->params.flags & K2J_FLAG_SORT_BY_START) && n_gpu_events > 1) {
    k2j_status st = sort_gpu_events(c, n_gpu_events);
    if (st) return st;
  }
  // the first stream sync of every (device, stream) row, in emission order
  if (totals[C_SYNC]) { k_sync_rows<<<(uint32_t)((totals[C_SYNC] + 255) / 256), 256, 0, s>>>(d); c->launches++; }

  // ---- size pass, scan, emit pass ----
  uint64_t total_bytes = 0, ann_bytes = 0;
  uint32_t n_spans = 0;
  if (d.n_work) {
    const uint32_t ev_blocks = (uint32_t)((d.n_work + kEventThreads - 1) / kEventThreads);
    k_events<false><<<ev_blocks, kEventThreads, events_smem_bytes(false), s>>>(d);
    c->launches++;
    if (totals[C_WAIT]) {  // deferred synchronisation records: sized once every stream with GPU work is known
      Dev dw = d;
      dw.wait_pass = 1; dw.work_origin = d.cls_begin[C_WAIT];
      dw.n_work = d.cls_begin[C_WAIT] + ((totals[C_WAIT] + 31) & ~31ull);
      k_events<false><<<(uint32_t)((dw.n_work - dw.work_origin + kEventThreads - 1) / kEventThreads), kEventThreads, events_smem_bytes(false), s>>>(dw);
      c->launches++;
    }
    K2J_CUDA(c, cudaGetLastError());
    K2J_CUDA(c, cudaEventRecord(c->ev[3], s));
    k2j_status st = run_scan(c, d.ev_size, d.n_events, 1, c->ev_off.as<uint64_t>(), c->scan_totals.as<uint64_t>() + 20, &c->launches);
    if (st) return st;
    K2J_CUDA(c, cudaMemcpyAsync(c->h_totals + 20, c->scan_totals.as<uint64_t>() + 20, 8, cudaMemcpyDeviceToHost, s));
    if (n_gpu_events)
      K2J_CUDA(c, cudaMemcpyAsync(c->h_totals + 21, c->ev_off.as<uint64_t>() + c->n_ops, 8, cudaMemcpyDeviceToHost, s));
    c->h_totals[25] = 0;
    if (d.has_comms) K2J_CUDA(c, cudaMemcpyAsync(c->h_totals + 25, d.has_comms, 4, cudaMemcpyDeviceToHost, s));
    c->h_totals[26] = 0;
    if (d.coll_list) K2J_CUDA(c, cudaMemcpyAsync(c->h_totals + 26, &d.counters->n_coll, 8, cudaMemcpyDeviceToHost, s));
    K2J_CUDA(c, cudaEventRecord(c->ev[4], s));
    K2J_CUDA(c, cudaStreamSynchronize(s));
    total_bytes = c->h_totals[20];
    c->partial_spans.clear();
    if (spans_on && c->have_global_join) {
      // several shards: this shard's part of every span waits for the caller to merge it with the other shards' parts
      // (k2j_partial_spans, k2j_append_spans); nothing is written here
      k2j_status st2 = collect_spans(c, span_cap, &c->partial_spans);
      if (st2) return st2;
    } else if (spans_on) {
      k2j_status st2 = order_annotations(c, span_cap, &n_spans, &ann_bytes);
      if (st2) return st2;
    }
    (void)ev_blocks;
    const bool instant = (c->h_totals[25] & 2) != 0;
    const uint64_t n_coll = c->h_totals[26];
    d.out_cap = total_bytes + ann_bytes;
    K2J_CUDA(c, cudaEventRecord(c->ev[7], s));
    if (sink.mode == 0) {
      // ---- the whole text stays in the context ----
      K2J_CUDA(c, c->out.reserve(total_bytes + ann_bytes + 64));
      d.out = c->out.as<uint8_t>(); d.tile_begin = 0; d.tile_end = total_bytes;
      if (total_bytes) { k2j_status st3 = launch_emit(c, d, nullptr, instant, n_coll, s); if (st3) return st3; }
      if (ann_bytes) {
        k_annotations<true><<<(n_spans + kEventThreads - 1) / kEventThreads, kEventThreads, 0, s>>>(
            d, c->span_out.as<SpanRec>(), n_spans, c->ann_size.as<uint32_t>(), c->ann_off.as<uint64_t>(), total_bytes);
        c->launches++;
      }
      K2J_CUDA(c, cudaGetLastError());
    } else {
      // ---- tiled: slab t holds the events whose text starts in [t * slab, (t + 1) * slab); while slab t travels to
      // the host (or the file) slab t + 1 is being written ----
      if (sink.mode == 1 && (sink.capacity < total_bytes + ann_bytes || (!sink.host && total_bytes + ann_bytes)))
        return fail(c, K2J_ERR_INVALID_ARGUMENT, "destination too small: the text has %llu bytes", (unsigned long long)(total_bytes + ann_bytes));
      const uint64_t slab = sink.slab_bytes ? std::max<uint64_t>(sink.slab_bytes, 4ull << 20) : (256ull << 20);
      const uint64_t n_tiles64 = (total_bytes + slab - 1) / slab;
      if (n_tiles64 > 1000000ull) return fail(c, K2J_ERR_INVALID_ARGUMENT, "slab size too small for this trace");
      const uint32_t n_tiles = (uint32_t)n_tiles64;
      for (int i = 0; i < 2; i++) {
        K2J_CUDA(c, c->slab[i].reserve(std::min<uint64_t>(slab, total_bytes + ann_bytes) + kSlabMargin + kSlabPad + 64));
        if (!c->slab_done[i]) K2J_CUDA(c, cudaEventCreateWithFlags(&c->slab_done[i], cudaEventDisableTiming));
        if (!c->slab_free[i]) K2J_CUDA(c, cudaEventCreateWithFlags(&c->slab_free[i], cudaEventDisableTiming));
      }
      if (!c->copy_stream) K2J_CUDA(c, cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking));
      std::vector<uint64_t> bounds((size_t)(n_tiles + 1) * kTileCols);
      if (n_tiles) {
        K2J_CUDA(c, c->tile_bounds.reserve(bounds.size() * 8));
        k_tile_bounds<<<(n_tiles + 1 + 127) / 128, 128, 0, s>>>(d, slab, n_tiles, total_bytes, c->tile_bounds.as<uint64_t>());
        c->launches++;
        K2J_CUDA(c, cudaMemcpyAsync(bounds.data(), c->tile_bounds.p, bounds.size() * 8, cudaMemcpyDeviceToHost, s));
        K2J_CUDA(c, cudaStreamSynchronize(s));
      }
      const bool sorted = (c->params.flags & K2J_FLAG_SORT_BY_START) != 0;
      uint64_t file_pos = 0;
      // hands slab `k` (bytes [b0, b1) of the text) on; `wait_emit`: the slab's launches are recorded in slab_done[k & 1]
      auto hand_on = [&](uint32_t k, uint64_t b0, uint64_t b1) -> k2j_status {
        const uint8_t* src = c->slab[k & 1].as<uint8_t>() + kSlabPad;
        if (sink.mode == 1) {
          K2J_CUDA(c, cudaStreamWaitEvent(c->copy_stream, c->slab_done[k & 1], 0));
          if (b1 > b0) K2J_CUDA(c, cudaMemcpyAsync(sink.host + b0, src, b1 - b0, cudaMemcpyDeviceToHost, c->copy_stream));
          K2J_CUDA(c, cudaEventRecord(c->slab_free[k & 1], c->copy_stream));
        } else {
          K2J_CUDA(c, cudaEventSynchronize(c->slab_done[k & 1]));
          k2j_status st4 = stream_bytes(c, src, sink.fd, false, 0, b1 - b0, c->copy_stream);
          if (st4) return st4;
          file_pos += b1 - b0;
          K2J_CUDA(c, cudaEventRecord(c->slab_free[k & 1], c->copy_stream));
        }
        return K2J_OK;
      };
      const uint32_t n_slabs = n_tiles + (ann_bytes ? 1u : 0u);
      for (uint32_t t = 0; t < n_slabs; t++) {
        if (t >= 2) K2J_CUDA(c, cudaStreamWaitEvent(s, c->slab_free[t & 1], 0));  // the slab's previous text has left
        if (t < n_tiles) {
          const uint64_t* r0 = &bounds[(size_t)t * kTileCols];
          const uint64_t* r1 = r0 + kTileCols;
          if (r1[1] - r0[1] > slab + kSlabMargin) return fail(c, K2J_ERR_UNSUPPORTED, "an event of more than %llu bytes", (unsigned long long)kSlabMargin);
          d.tile_begin = r0[1]; d.tile_end = r1[1];
          d.out = c->slab[t & 1].as<uint8_t>() + kSlabPad - r0[1];
          uint64_t ranges[2 * (C_EXT + 1)];
          for (int k = 0; k < C_EXT; k++) {
            ranges[2 * k] = sorted ? d.cls_begin[k] : r0[2 + k];
            ranges[2 * k + 1] = sorted ? d.cls_begin[k] + d.cls_count[k] : r1[2 + k];
          }
          ranges[2 * C_EXT] = d.ops_begin + std::min<uint64_t>(r0[0], c->n_ops);   // CPU-side activities are events 0 .. n_ops
          ranges[2 * C_EXT + 1] = d.ops_begin + std::min<uint64_t>(r1[0], c->n_ops);
          k2j_status st3 = launch_emit(c, d, ranges, instant, n_coll, s);
          if (st3) return st3;
        } else {  // the user-annotation spans come last, as a slab of their own
          d.tile_begin = total_bytes; d.tile_end = total_bytes + ann_bytes;
          d.out = c->slab[t & 1].as<uint8_t>() + kSlabPad - total_bytes;
          k_annotations<true><<<(n_spans + kEventThreads - 1) / kEventThreads, kEventThreads, 0, s>>>(
              d, c->span_out.as<SpanRec>(), n_spans, c->ann_size.as<uint32_t>(), c->ann_off.as<uint64_t>(), total_bytes);
          c->launches++;
          K2J_CUDA(c, cudaGetLastError());
        }
        K2J_CUDA(c, cudaEventRecord(c->slab_done[t & 1], s));
        if (t >= 1) {  // slab t - 1 leaves while slab t is being written
          k2j_status st4 = hand_on(t - 1, t - 1 < n_tiles ? bounds[(size_t)(t - 1) * kTileCols + 1] : total_bytes,
                                   t - 1 < n_tiles ? bounds[(size_t)t * kTileCols + 1] : total_bytes + ann_bytes);
          if (st4) return st4;
        }
      }
      if (n_slabs) {
        const uint32_t t = n_slabs - 1;
        k2j_status st4 = hand_on(t, t < n_tiles ? bounds[(size_t)t * kTileCols + 1] : total_bytes,
                                 t < n_tiles ? bounds[(size_t)(t + 1) * kTileCols + 1] : total_bytes + ann_bytes);
        if (st4) return st4;
      }
      K2J_CUDA(c, cudaStreamSynchronize(c->copy_stream));
      (void)file_pos;
    }
  } else {
    K2J_CUDA(c, cudaEventRecord(c->ev[3], s));
    K2J_CUDA(c, cudaEventRecord(c->ev[4], s));
    K2J_CUDA(c, cudaEventRecord(c->ev[7], s));
  }
  K2J_CUDA(c, cudaEventRecord(c->ev[5], s));
  K2J_CUDA(c, cudaMemcpyAsync(c->h_counters, c->counters.p, sizeof(Counters), cudaMemcpyDeviceToHost, s));
  K2J_CUDA(c, cudaStreamSynchronize(s));

  res->out_bytes = total_bytes + ann_bytes;
  res->annotation_bytes = ann_bytes;
  res->ops_bytes = n_gpu_events ? c->h_totals[21] : total_bytes;
  res->n_records = totals[C_EVENTS] + totals[C_WAIT] + totals[C_EXT] + totals[C_UNEXPECTED] - c->h_counters->guests;
  res->x_events = c->h_counters->x_events + (ann_bytes ? n_spans : 0);
  res->flow_events = c->h_counters->flow_events;
  res->out_of_range_events = c->h_counters->out_of_range;
  res->blocklisted_runtime_events = c->h_counters->blocklisted_runtime;
  res->invalid_external_correlation_events = c->h_counters->invalid_external_correlation;
  res->unexpected_cuda_events = totals[C_UNEXPECTED];
  res->in_bytes = 208 * totals[C_KERNEL] + 88 * totals[C_MEMCPY] + 96 * totals[C_MEMCPY2] + 88 * totals[C_MEMSET] +
                  40 * totals[C_API] + 24 * totals[C_EXT] + 56 * totals[C_OVERHEAD] + 40 * (totals[C_SYNC] + totals[C_WAIT]) +
                  56 * totals[C_CUDAEVENT];
  res->name_bytes = c->h_counters->name_bytes;
  res->kernel_launches = c->launches;
  cudaEventElapsedTime(&res->ms_segment, c->ev[0], c->ev[1]);
  cudaEventElapsedTime(&res->ms_join, c->ev[6], c->ev[2]);
  cudaEventElapsedTime(&res->ms_size, c->ev[2], c->ev[3]);
  cudaEventElapsedTime(&res->ms_scan, c->ev[3], c->ev[4]);
  cudaEventElapsedTime(&res->ms_emit, c->ev[7], c->ev[5]);
  res->ms_total = res->ms_segment + res->ms_join + res->ms_size + res->ms_scan + res->ms_emit;
  c->out_bytes = total_bytes + ann_bytes;
  if (c->h_counters->device_check)
    return fail(c, K2J_ERR_DEVICE_CHECK, "%llu device-side checks failed (string id, table or output bound)",
                (unsigned long long)c->h_counters->device_check);
  c->ran = sink.mode == 0;  // only a run that completed without a failed check leaves text to serve
  c->streamed = sink.mode != 0;
  return K2J_OK;
}

}  // namespace

extern "C" {

k2j_status k2j_emit(k2j_ctx* c, k2j_result* res) { return emit_core(c, res, TileSink{}); }

k2j_status k2j_emit_to_host(k2j_ctx* c, void* host_dst, uint64_t capacity, uint64_t slab_bytes, k2j_result* res) {
  TileSink sink;
  sink.mode = 1; sink.host = static_cast<uint8_t*>(host_dst); sink.capacity = capacity; sink.slab_bytes = slab_bytes;
  return emit_core(c, res, sink);
}

k2j_status k2j_emit_to_fd(k2j_ctx* c, int fd, uint64_t slab_bytes, k2j_result* res) {
  if (c && fd < 0) return fail(c, K2J_ERR_INVALID_ARGUMENT, "bad file descriptor");
  TileSink sink;
  sink.mode = 2; sink.fd = fd; sink.slab_bytes = slab_bytes;
  return emit_core(c, res, sink);
}

k2j_status k2j_run(k2j_ctx* c, k2j_result* res) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!res) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null result");
  k2j_status st = k2j_segment(c, nullptr);
  if (st) return st;
  return k2j_emit(c, res);
}

k2j_status k2j_exclusive_scan_u32(k2j_ctx* c, const uint32_t* sizes, uint64_t n, uint64_t* offsets, uint64_t* total) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!total || (n && (!sizes || !offsets))) return fail(c, K2J_ERR_INVALID_ARGUMENT, "null scan argument");
  if (n && (!is_device_ptr(sizes) || !is_device_ptr(offsets))) return fail(c, K2J_ERR_INVALID_ARGUMENT, "scan arrays must be device memory");
  K2J_CUDA(c, cudaSetDevice(c->device));
  *total = 0;
  if (n == 0) return K2J_OK;
  uint32_t launches = 0;
  k2j_status st = run_scan(c, sizes, n, 1, offsets, c->scan_totals.as<uint64_t>() + 24, &launches);
  if (st) return st;
  K2J_CUDA(c, cudaMemcpyAsync(c->h_totals + 24, c->scan_totals.as<uint64_t>() + 24, 8, cudaMemcpyDeviceToHost, c->stream));
  K2J_CUDA(c, cudaStreamSynchronize(c->stream));
  *total = c->h_totals[24];
  return K2J_OK;
}

k2j_status k2j_output(k2j_ctx* c, const void** p, uint64_t* n) {
  if (!c || !p || !n) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->ran) return fail(c, K2J_ERR_STATE, "no completed run");
  *p = c->out.p; *n = c->out_bytes;
  return K2J_OK;
}

k2j_status k2j_copy_output(k2j_ctx* c, void* dst, uint64_t cap) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->ran) return fail(c, K2J_ERR_STATE, "no completed run");
  if (cap < c->out_bytes || (!dst && c->out_bytes)) return fail(c, K2J_ERR_INVALID_ARGUMENT, "destination too small");
  K2J_CUDA(c, cudaSetDevice(c->device));
  if (c->out_bytes) K2J_CUDA(c, cudaMemcpyAsync(dst, c->out.p, c->out_bytes, cudaMemcpyDeviceToHost, c->stream));
  K2J_CUDA(c, cudaStreamSynchronize(c->stream));
  return K2J_OK;
}

k2j_status k2j_copy_output_async(k2j_ctx* c, void* dst, uint64_t cap) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->ran) return fail(c, K2J_ERR_STATE, "no completed run");
  if (cap < c->out_bytes || (!dst && c->out_bytes)) return fail(c, K2J_ERR_INVALID_ARGUMENT, "destination too small");
  K2J_CUDA(c, cudaSetDevice(c->device));
  if (c->out_bytes) K2J_CUDA(c, cudaMemcpyAsync(dst, c->out.p, c->out_bytes, cudaMemcpyDeviceToHost, c->stream));
  return K2J_OK;
}

// Streams bytes [begin, begin + total) of the output to `fd` in chunks through the two pinned staging buffers: the
// copy of chunk i overlaps the write of chunk i - 1.  `positioned`: pwrite at file_offset, else write at the
// descriptor's position.
}  // extern "C"
namespace {
k2j_status stream_bytes(k2j_ctx* c, const uint8_t* src, int fd, bool positioned, uint64_t file_offset, uint64_t total, cudaStream_t stream) {
  constexpr size_t kChunk = 16u << 20;
  for (int i = 0; i < 2; i++) {
    if (!c->h_stage[i]) K2J_CUDA(c, cudaMallocHost(&c->h_stage[i], kChunk));
    if (!c->stage_ev[i]) K2J_CUDA(c, cudaEventCreateWithFlags(&c->stage_ev[i], cudaEventDisableTiming));
  }
  int io_errno = 0;
  auto write_all = [&](const char* p, size_t n, uint64_t off) -> bool {
    while (n) {
      const ssize_t w = positioned ? pwrite(fd, p, n, (off_t)off) : write(fd, p, n);
      if (w < 0) { if (errno == EINTR) continue; io_errno = errno; return false; }
      if (w == 0) { io_errno = EIO; return false; }  // no progress on a non-empty write
      p += w; n -= (size_t)w; off += (uint64_t)w;
    }
    return true;
  };
  const uint64_t n_chunks = (total + kChunk - 1) / kChunk;
  bool io_ok = true;
  cudaError_t e = cudaSuccess;
  for (uint64_t i = 0; i <= n_chunks && e == cudaSuccess; i++) {
    if (i < n_chunks) {  // chunk i starts its way to the host ...
      const size_t len = (size_t)std::min<uint64_t>(kChunk, total - i * kChunk);
      e = cudaMemcpyAsync(c->h_stage[i & 1], src + i * kChunk, len, cudaMemcpyDeviceToHost, stream);
      if (e == cudaSuccess) e = cudaEventRecord(c->stage_ev[i & 1], stream);
    }
    if (i > 0 && e == cudaSuccess) {  // ... while chunk i - 1, which has arrived, goes to the file
      e = cudaEventSynchronize(c->stage_ev[(i - 1) & 1]);
      const size_t len = (size_t)std::min<uint64_t>(kChunk, total - (i - 1) * kChunk);
      if (e == cudaSuccess && io_ok && !write_all(static_cast<const char*>(c->h_stage[(i - 1) & 1]), len, file_offset + (i - 1) * kChunk))
        io_ok = false;  // keep draining the copies
    }
  }
  if (e != cudaSuccess) {
    cudaStreamSynchronize(stream);  // no copy into the staging buffers stays in flight behind this call
    return fail(c, K2J_ERR_CUDA, "streaming the output: %s", cudaGetErrorString(e));
  }
  if (!io_ok) return fail(c, K2J_ERR_IO, "write: %s", strerror(io_errno));
  return K2J_OK;
}
}  // namespace
extern "C" {

k2j_status k2j_write_output(k2j_ctx* c, int fd, uint64_t* written) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->ran) return fail(c, K2J_ERR_STATE, "no completed run");
  if (fd < 0) return fail(c, K2J_ERR_INVALID_ARGUMENT, "bad file descriptor");
  K2J_CUDA(c, cudaSetDevice(c->device));
  k2j_status st = stream_bytes(c, c->out.as<uint8_t>(), fd, false, 0, c->out_bytes, c->stream);
  if (st) return st;
  if (written) *written = c->out_bytes;
  return K2J_OK;
}

k2j_status k2j_write_output_at(k2j_ctx* c, int fd, uint64_t file_offset, uint64_t begin, uint64_t n_bytes) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  if (!c->ran) return fail(c, K2J_ERR_STATE, "no completed run");
  if (fd < 0) return fail(c, K2J_ERR_INVALID_ARGUMENT, "bad file descriptor");
  if (begin > c->out_bytes || n_bytes > c->out_bytes - begin) return fail(c, K2J_ERR_INVALID_ARGUMENT, "range outside the output");
  K2J_CUDA(c, cudaSetDevice(c->device));
  return stream_bytes(c, c->out.as<uint8_t>() + begin, fd, true, file_offset, n_bytes, c->stream);
}

k2j_status k2j_synchronize(k2j_ctx* c) {
  if (!c) return K2J_ERR_INVALID_ARGUMENT;
  K2J_CUDA(c, cudaSetDevice(c->device));
  K2J_CUDA(c, cudaStreamSynchronize(c->stream));
  return K2J_OK;
}

}  // extern "C"
