/* k2j — C ABI of the B200 trace post-processing library (libk2j.so).
 *
 * One context turns the raw inputs of libkineto's post-processing step into the Chrome-trace JSON
 * text of every activity event, byte-identical to what the reference's ChromeTraceLogger writes for
 * the same inputs.  Every entry point returns a k2j_status, never throws, never aborts.  A context
 * is used by one thread at a time (the same contract as libkineto/src/output_json.h:62-63).
 *
 * Each declaration names the part of the reference it stands in for (paths relative to the
 * reference project).  Array arguments may be host or device memory: device memory is used in
 * place, host memory is copied to the GPU on the context's stream (asynchronously when it is
 * pinned).  Either way the arrays must stay valid and unchanged until k2j_run returns.
 *
 * Device memory handed to the library (input arrays, the gathered join arrays, scan inputs) is read by
 * kernels on the context's stream: its contents must be complete before the call that uses them, or be
 * produced by work that is ordered before the context's stream (the same stream, or an event the stream
 * waits on).  A caller that fills such arrays on another stream (NCCL, a framework's current stream)
 * either passes that stream to k2j_create or synchronises it first; the library inserts no such wait.
 */
#ifndef K2J_H_
#define K2J_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct k2j_ctx k2j_ctx;

typedef enum {
  K2J_OK = 0,
  K2J_ERR_INVALID_ARGUMENT = 1, /* null pointer, misaligned or out-of-range table entry */
  K2J_ERR_CUDA = 2,             /* a CUDA runtime call failed; see k2j_last_error */
  K2J_ERR_UNSUPPORTED = 3,      /* input uses a feature this build does not implement */
  K2J_ERR_STATE = 4,            /* call order violated (e.g. output requested before a run) */
  K2J_ERR_DEVICE_CHECK = 5,     /* a kernel's own bounds/consistency check tripped */
  K2J_ERR_IO = 6                /* writing the output to a file descriptor failed */
} k2j_status;

/* Scalars of one trace.
 * base_time_ns        ChromeTraceBaseTime::get()             libkineto/src/output_json.h:265-279
 * window_*            captureWindowStartTime_/EndTime_       libkineto/src/GenericActivityProfiler.cpp:329-340
 * pid                 processId(), the "pid" of runtime rows libkineto/src/CuptiActivity.h:93-95
 * ts_mode, conv_*     0: CUPTI timestamps are unix ns; 1: the affine TSC converter with a long-double
 *                     scale = conv_scale_mant * 2^(conv_scale_exp-63)
 *                                                            libkineto/src/ApproximateClock.cpp:83-90
 * flags               K2J_FLAG_*
 * activity_type_mask  bit t set: CPU-side activities of libkineto::ActivityType t are logged
 *                     (derivedConfig_->profileActivityTypes(), GenericActivityProfiler.cpp:248);
 *                     unselected activities still take part in the join                              */
typedef struct {
  int64_t base_time_ns;
  int64_t window_start_ns;
  int64_t window_end_ns;
  int32_t pid;
  int32_t ts_mode;
  int32_t flags;
  int32_t n_devices;
  int64_t conv_t0;
  uint64_t conv_t0_approx;
  uint64_t conv_scale_mant;
  int32_t conv_scale_exp;
  uint32_t activity_type_mask;
} k2j_params;

#define K2J_FLAG_USER_ANNOTATIONS 1 /* GPU_USER_ANNOTATION selected (GenericActivityProfiler.cpp:424) */
#define K2J_FLAG_SORT_BY_START 2     /* GPU-side events in stable order of their start timestamp (64-bit
                                       radix sort).  The reference never sorts: the output equals the
                                       reference's on buffers pre-sorted that way. */
#define K2J_FLAG_PID0_OVERRIDE 4    /* CPU activities with device 0 are shown under params.pid: what
                                       ActivityTrace::save() writes after the pid-0 override of
                                       GenericActivityProfiler.cpp:263-271 */
#define K2J_FLAG_UNFINISHED_OPS 8   /* CPU activities whose end precedes their start had not ended when the trace
                                       stopped: they end at window_end_ns (processCpuTrace,
                                       GenericActivityProfiler.cpp:255-258).  The "finished": false entry such an
                                       activity gains there is part of its metadata like any other: the caller lists
                                       it (K2J_MD_RAWJSON, text false) where the fixed-up activity visits it.  Without
                                       the flag (a logger driven directly) such an activity lasts 0 ns. */

/* cudaDeviceProp fields read by blocksPerSm / warpsPerSm / computeOccupancyMetrics
 * (libkineto/src/DeviceProperties.cpp:161-222). */
typedef struct {
  int32_t major, minor;
  int32_t max_threads_per_block, max_threads_per_sm;
  int32_t regs_per_block, regs_per_sm;
  int32_t warp_size, num_sms;
  uint64_t smem_per_block, smem_per_block_optin, smem_per_sm, reserved_smem_per_block;
} k2j_device_props;

/* One typed metadata entry of a CPU-side activity, in the order the activity visits them
 * (GenericTraceActivity::visitTypedMetadata, libkineto/include/GenericTraceActivity.h:160-170). */
typedef struct {
  uint32_t key;   /* string id */
  uint32_t type;  /* K2J_MD_* */
  uint64_t value; /* int64 / uint64 / double bits / bool / string id */
} k2j_md_entry;
enum { K2J_MD_INT64 = 0, K2J_MD_UINT64 = 1, K2J_MD_DOUBLE = 2, K2J_MD_BOOL = 3, K2J_MD_STRING = 4, K2J_MD_RAWJSON = 5,
       K2J_MD_COUNTER = 6 /* a counter value (GenericTraceActivity::counterValues(), name and double bits) of an activity
                             of type MTIA_COUNTERS, XPU_SCOPE_PROFILER or HARDWARE_COUNTERS, in the list's order after
                             the other entries; such activities are written as counter events
                             (libkineto/src/output_json.cpp:679-716) and their other entries are not printed */ };

/* Columns of the CPU-side activities (libkineto::GenericTraceActivity fields,
 * libkineto/include/GenericTraceActivity.h:173-192): all arrays have n_ops elements except
 * md_off (n_ops + 1) and md (md_off[n_ops]). */
typedef struct {
  uint64_t n_ops;
  const int64_t* start_ns;
  const int64_t* end_ns;
  const int32_t* id;        /* correlationId() */
  const int32_t* device;    /* deviceId(): the pid column */
  const int64_t* resource;  /* resourceId(): the tid column */
  const int32_t* thread;    /* getThreadId() */
  const int32_t* type;      /* libkineto::ActivityType value */
  const uint32_t* name;     /* string id */
  const uint32_t* flow_id;
  const uint8_t* flow_info; /* flow.type | flow.start << 4 */
  const uint32_t* md_off;
  const k2j_md_entry* md;
} k2j_ops;

/* Result of a run.  The error counters mirror GenericActivityProfiler::ErrorCounts
 * (libkineto/src/GenericActivityProfiler.h:528-535). */
typedef struct {
  uint64_t out_bytes;   /* total JSON bytes produced */
  uint64_t ops_bytes;   /* bytes of the CPU-activity events (they come first) */
  uint64_t n_records;   /* CUPTI records walked */
  uint64_t x_events;    /* "ph": "X" events written */
  uint64_t flow_events; /* "ph": "s"/"f" events written */
  uint64_t out_of_range_events;
  uint64_t blocklisted_runtime_events;
  uint64_t invalid_external_correlation_events;
  uint64_t unexpected_cuda_events;
  uint64_t in_bytes;    /* CUPTI record bytes consumed */
  uint64_t name_bytes;  /* escaped name bytes copied into events */
  uint64_t annotation_bytes; /* bytes of the gpu_user_annotation events (they come last) */
  uint32_t kernel_launches; /* GPU kernels this run launched */
  uint32_t reserved;
  float ms_segment;     /* device time of each stage, CUDA events on the context's stream */
  float ms_join;
  float ms_size;
  float ms_scan;
  float ms_emit;
  float ms_total;
} k2j_result;

/* Creates a context on CUDA device `device`.  `stream` is a cudaStream_t to run on, or NULL for a
 * stream owned by the context (non-blocking: not ordered with the default stream; a caller that works on the
 * default stream passes cudaStreamLegacy or cudaStreamPerThread, not the NULL handle).  No reference counterpart: the reference keeps this state in the
 * profiler and logger objects. */
k2j_status k2j_create(int device, void* stream, k2j_ctx** out);
void k2j_destroy(k2j_ctx* ctx);
/* Text of the last failure on this context. */
const char* k2j_last_error(const k2j_ctx* ctx);

/* Trace scalars and per-device properties (n_props = params->n_devices entries). */
k2j_status k2j_set_params(k2j_ctx* ctx, const k2j_params* params, const k2j_device_props* props);

/* The string pool every string id refers to: n_strings strings, string i = data[off[i], off[i+1]).
 * Kernel names are the demangled names (libkineto/src/CuptiActivity.h:297-300); the library applies
 * the JSON sanitising and escaping of libkineto/src/output_json.cpp:72-112 itself. */
k2j_status k2j_set_strings(k2j_ctx* ctx, const uint64_t* off, const uint8_t* data, uint64_t n_strings);

/* String ids of runtimeCbidName(cbid) / driverCbidName(cbid) per callback id
 * (libkineto/src/cupti_strings.cpp:106-132); ids past the end render as "INVALID". */
k2j_status k2j_set_cbid_names(k2j_ctx* ctx, const uint32_t* runtime, uint32_t n_runtime,
                              const uint32_t* driver, uint32_t n_driver);

/* (CUPTI thread id, system thread id) pairs: the resourceInfo_ lookup of
 * CuptiActivityProfiler::handleRuntimeActivity (libkineto/src/CuptiActivityProfiler.cpp:315-319).
 * For duplicate thread ids the first pair wins, as recordThreadInfo does.  CPU-side activities whose
 * device equals params.pid extend the map with (thread, resource) in order, after these pairs
 * (libkineto/src/GenericActivityProfiler.cpp:272).  At most a few thousand distinct threads. */
k2j_status k2j_set_thread_map(k2j_ctx* ctx, const int32_t* pairs, uint32_t n_pairs);

/* CPU-side activities: what GenericActivityProfiler::processCpuTrace iterates
 * (libkineto/src/GenericActivityProfiler.cpp:234-275). */
k2j_status k2j_set_ops(k2j_ctx* ctx, const k2j_ops* ops);

/* The drained CUPTI activity buffers: what CuptiActivityApi::processActivities iterates
 * (libkineto/src/CuptiActivityApi.cpp:235-246).  `buftab` holds (byte offset, valid bytes) per
 * buffer, in processing order; records are packed back to back, 8-byte aligned, sized by kind.
 * The `name` field of kernel records holds a string id. At most 32 GiB per call.
 * Kinds that are sized and formatted: CONCURRENT_KERNEL (CUpti_ActivityKernel9), MEMCPY (Memcpy5), MEMCPY2
 * (MemcpyPtoP4), MEMSET (Memset4), RUNTIME / DRIVER (ActivityAPI), EXTERNAL_CORRELATION, OVERHEAD (Overhead3),
 * SYNCHRONIZATION (ActivitySynchronization) and CUDA_EVENT (CudaEvent2)
 * (libkineto/src/CuptiActivityProfiler.cpp:532-588).  A record of any other kind that the CUDA 12.9 CUPTI headers
 * define is stepped over by the size of that kind's structure and counted in unexpected_cuda_events, as the
 * reference counts it (:583-587); a kind the headers do not define ends the walk of its buffer (counted once). */
k2j_status k2j_set_cupti(k2j_ctx* ctx, const uint8_t* bytes, uint64_t n_bytes, const uint64_t* buftab,
                         uint32_t n_buffers);

/* Runs the pipeline: segment -> join tables -> size -> scan -> emit.  Replaces the per-record work
 * of CuptiActivityProfiler::processGpuActivities (libkineto/src/CuptiActivityProfiler.cpp:189-220)
 * plus ChromeTraceLogger::handleActivity (libkineto/src/output_json.cpp:837-963) for every event. */
k2j_status k2j_run(k2j_ctx* ctx, k2j_result* result);

/* The same work in two steps, for traces sharded by contiguous record range over several GPUs (one
 * context per GPU).  k2j_segment walks this shard's buffers and compacts its EXTERNAL_CORRELATION
 * records (k2j_external_record, processing order).  The caller all-gathers those arrays and the CPU
 * activity ids of all shards in shard order (NCCL) and hands the result to k2j_set_global_join, so
 * that the correlation maps of CuptiActivityProfiler::buildProcessingState
 * (libkineto/src/CuptiActivityProfiler.cpp:256-302) and activityMap_ cover the whole trace;
 * `own_begin` is the index of this shard's first record in the gathered array.  k2j_emit then
 * builds the tables and produces this shard's text.  Without k2j_set_global_join the join sees only
 * the local shard (k2j_run = k2j_segment + k2j_emit). */
typedef struct {
  uint64_t external_id;
  uint32_t correlation_id;
  uint32_t external_kind;
} k2j_external_record;
typedef struct {
  uint64_t n_records;
  uint64_t n_external;
  const k2j_external_record* external_records; /* device memory, n_external entries */
  uint64_t n_ops;
  const int32_t* op_ids;                       /* device memory, n_ops entries */
  uint64_t n_user_external;                    /* how many of the n_external records are of kind CUSTOM1 (user annotations) */
} k2j_segment_info;
k2j_status k2j_segment(k2j_ctx* ctx, k2j_segment_info* info);
k2j_status k2j_set_global_join(k2j_ctx* ctx, const void* external_all, uint64_t n_external_all, uint64_t own_begin,
                               const int32_t* op_ids_all, uint64_t n_ops_all);
/* k2j_set_global_join for arrays left as an all-gather of equal-sized rows delivers them, so that nothing has to
 * be compacted (or counted on the host) between the collective and the run: row r (shard r) lies row_pitch_bytes
 * after row r - 1; a row's records start at ext_rows + r * pitch, its ids at op_id_rows + r * pitch; ext_stride /
 * ops_stride are the entries a row has room for, counts[2 r] / counts[2 r + 1] (device memory, written by the same
 * exchange) the entries it holds.  Tables are then sized for this shard's own events. */
k2j_status k2j_set_global_join_rows(k2j_ctx* ctx, const void* ext_rows, uint64_t ext_stride, const int32_t* op_id_rows,
                                    uint64_t ops_stride, uint64_t row_pitch_bytes, const uint64_t* counts, uint32_t world,
                                    uint32_t rank);
/* Sending join keys only where they can be wanted.  With k2j_set_global_join_rows a shard reads its OWN records
 * and ids from its own arrays, never from its row, so the row a shard contributes only has to hold what other
 * shards can want.  k2j_join_need_bits (after k2j_segment) fills `bits` (device memory, n_bits a power of two,
 * the same on every shard; about 4 bits per GPU-side record keep false hits near 2 %) with the filter of the
 * correlation ids this shard's events carry; `bits` must stay as it is until k2j_emit has run, which tests the
 * gathered keys against it.  The caller all-gathers the filters; k2j_filter_join_keys then
 * writes to `out_records` (device memory, room for `capacity` >= this shard's n_external records), in their order,
 * those of this shard's EXTERNAL_CORRELATION records whose correlation id hits the filter of at least one OTHER
 * shard (`need_rows`: the gathered filters, row_pitch_bytes apart), and their number to `n_out` (device memory, on
 * the context's stream).  These records, followed by the CPU-op ids, are the row to all-gather: positions still
 * grow along a shard's records, which is all that "the last record of a correlation id wins" needs, and counts[2 r]
 * is the number of records row r holds.  Nothing of the result changes; the bytes a rank receives no longer grow
 * with the number of shards times the shard size.  No reference counterpart. */
k2j_status k2j_join_need_bits(k2j_ctx* ctx, void* bits, uint64_t n_bits);
/* The CPU-op ids of the other shards as bitmaps.  The join only asks whether an activity with a given id exists
 * anywhere in the trace (activityMap_.find, libkineto/src/GenericActivityProfiler.cpp:397-408), and the ids of a
 * shard usually fill a narrow range: k2j_op_id_bits (after k2j_segment) sets, in `bits` (device memory, n_bits a
 * multiple of 32), bit id - min_id for every CPU-side activity of this shard (guest rows excluded; an id outside the
 * range is K2J_ERR_INVALID_ARGUMENT).  After k2j_set_global_join_rows, k2j_set_global_op_bits hands over the gathered
 * bitmaps (row r of `bit_rows`, row_pitch_bytes apart, with meta[2 r] = its min_id and meta[2 r + 1] = its n_bits;
 * device memory): the op ids of the rows given to k2j_set_global_join_rows are then not read, and only this shard's
 * own ids enter its table.  Forgotten by the next k2j_set_global_join*. */
k2j_status k2j_op_id_bits(k2j_ctx* ctx, int64_t min_id, uint64_t n_bits, void* bits);
k2j_status k2j_set_global_op_bits(k2j_ctx* ctx, const void* bit_rows, uint64_t row_pitch_bytes, const int64_t* meta);

/* ---- sharded traces: what crosses shards besides the join keys ---- */

/* Sharded traces whose shards hold synchronisation or CUDA event records.  The reference fills the lookups
 * those records use from the WHOLE trace before it logs anything: context -> device from the first kernel, copy
 * or memset record that names the context (libkineto/src/CuptiActivityProfiler.cpp:221-239), (context, event) ->
 * CUDA event record (:241-254, :379-402), the streams that showed GPU work inside the window, which gate deferred
 * stream-wait records (:502-514), and the once-per-row announcement in front of a row's first stream
 * synchronisation (libkineto/src/output_json.cpp:917-943).  A shard's share of that knowledge is carried by a few
 * of its own records.  k2j_export_lookup_records (after k2j_segment) returns them, copied verbatim and in
 * processing order into one CUPTI buffer in device memory of the context (valid until its next call): per context
 * its first kernel / copy / memset record, per (device, stream) the first such record inside the window, per
 * (context, stream) the first stream synchronisation inside the window, and every CUDA event record.  The caller
 * all-gathers the shards' buffers and gives each shard, through k2j_set_cupti, the lower shards' buffers in front of
 * its own buffers and the higher shards' behind them, then names the two byte ranges with k2j_set_guest_ranges
 * (records below `front_end_bytes` and from `back_begin_bytes` on are guests; buffers must not straddle either
 * boundary; k2j_set_cupti forgets the ranges).  Guest records take part in every lookup exactly as if the shard had
 * met them itself, print nothing and are not counted.  Then k2j_segment, the join exchange and k2j_emit as usual.
 * Without declared guest ranges a sharded run with such records is K2J_ERR_UNSUPPORTED. */
k2j_status k2j_export_lookup_records(k2j_ctx* ctx, const void** records, uint64_t* n_bytes);
k2j_status k2j_set_guest_ranges(k2j_ctx* ctx, uint64_t front_end_bytes, uint64_t back_begin_bytes);

/* Sharded traces with collectives.  A kernel launched by a record_param_comms CPU op prints that op's collective
 * metadata (libkineto/src/output_json.cpp:718-801, :900-906), and the op may belong to another shard.  The caller
 * appends the other shards' record_param_comms ops (id, name and metadata entries; their strings added to the pool)
 * behind its own rows in k2j_set_ops and says how many of the last rows are such guests: guest rows are found by the
 * kernels that need them, are never logged, extend no map and are not among the op ids k2j_segment reports.
 * k2j_set_ops resets the count to 0.  Ids of record_param_comms ops are taken to be used by no other op of the
 * trace (the reference would take the last op with that id, whatever its name).  Guest rows also serve as the
 * named rows of k2j_append_spans below. */
k2j_status k2j_set_guest_ops(k2j_ctx* ctx, uint64_t n_guest_ops);

/* Sharded traces with user annotations.  A gpu_user_annotation span covers, per (device, stream) and annotation
 * op, the GPU activities correlated to that op (libkineto/src/GenericActivityProfiler.cpp:292-327), wherever in the
 * trace they are, and the reference logs the spans after every other activity.  With K2J_FLAG_USER_ANNOTATIONS a
 * sharded run (k2j_set_global_join*) writes no spans; after k2j_emit, k2j_partial_spans returns this shard's part
 * of every span (host memory of the context, valid until its next run; first_event is the shard's own event
 * number; op_row is not meaningful).  The caller merges the parts of all shards - smallest start, largest end,
 * first_event ordered by (shard, event number) - names for each span the row of its op among the LAST shard's
 * CPU-side activities (its own or guest rows, k2j_set_guest_ops; 0xFFFFFFFF: no name), and hands the list to
 * k2j_append_spans on the last shard's context, which appends their events, in the reference's order
 * (libkineto/src/GenericActivityProfiler.h:341-346), to the text k2j_emit left there. */
typedef struct {
  int64_t start_ns, end_ns;
  uint64_t first_event;
  uint32_t device, stream;
  int32_t op_id;
  uint32_t op_row;
} k2j_span;
k2j_status k2j_partial_spans(k2j_ctx* ctx, const k2j_span** spans, uint64_t* n_spans);
k2j_status k2j_append_spans(k2j_ctx* ctx, const k2j_span* spans, uint64_t n_spans, uint64_t* n_bytes);
/* A sharded run keeps tables for the spans whenever K2J_FLAG_USER_ANNOTATIONS is set, since another shard's CUSTOM1
 * records may name this shard's events.  A caller that knows no shard holds such a record (the sum of
 * n_user_external over the shards is 0) says so with k2j_set_join_user_records(ctx, 0) after k2j_set_global_join*, and
 * the run then neither clears nor fills those tables (CUSTOM1 records that turn up all the same are ignored).
 * Forgotten by the next k2j_set_global_join*. */
k2j_status k2j_set_join_user_records(k2j_ctx* ctx, int any);

k2j_status k2j_filter_join_keys(k2j_ctx* ctx, const void* need_rows, uint64_t row_pitch_bytes, uint64_t n_bits, uint32_t world,
                                uint32_t rank, void* out_records, uint64_t capacity, uint64_t* n_out);
k2j_status k2j_emit(k2j_ctx* ctx, k2j_result* result);

/* k2j_emit for traces whose text should not be held whole on the device: the text is produced in slabs of
 * about `slab_bytes` (0: 256 MiB; two slabs are kept) and each slab leaves as soon as it is complete, while the
 * next one is being written.  k2j_emit_to_host copies every slab to its place in `host_dst` (the whole text,
 * result->out_bytes <= capacity; pinned memory lets the copies overlap the kernels): several contexts, one per
 * GPU, so fill their parts of one host buffer.  k2j_emit_to_fd writes the slabs to `fd` at its current position,
 * through the pinned staging buffers of k2j_write_output.  Afterwards the context holds no text (k2j_output and
 * the copy / write calls return K2J_ERR_STATE).  An event longer than 1 MiB is K2J_ERR_UNSUPPORTED here.
 * Stand where the reference streams events into its file as it produces them
 * (libkineto/src/output_json.cpp:237-259, :485-492): the reference never holds the text either. */
k2j_status k2j_emit_to_host(k2j_ctx* ctx, void* host_dst, uint64_t capacity, uint64_t slab_bytes, k2j_result* result);
k2j_status k2j_emit_to_fd(k2j_ctx* ctx, int fd, uint64_t slab_bytes, k2j_result* result);

/* The device-wide exclusive scan of the pipeline on its own: offsets[i] = sizes[0] + ... + sizes[i-1]
 * and *total = the sum, for n 32-bit sizes in device memory (offsets: n 64-bit values in device
 * memory).  It is the step that turns per-event byte lengths into final output positions; callers
 * that place several shards' text themselves use it for their own size tables.  The reference has no
 * such step: its logger appends to one std::ofstream (libkineto/src/output_json.cpp:246-257).
 * Scratch for the block sums comes from the context's grow-only workspace. */
k2j_status k2j_exclusive_scan_u32(k2j_ctx* ctx, const uint32_t* sizes, uint64_t n, uint64_t* offsets, uint64_t* total);

/* The same scan for callers that cannot allocate (no counterpart in the reference).  Profiler
 * callbacks that run during context teardown or under the allocator's lock, and processes whose
 * device memory is wholly owned by a framework's caching allocator, cannot let a library call
 * cudaMalloc; this entry point never allocates or frees: its block-sum scratch is a fixed array inside
 * the library image (about 64 KiB of device memory per GPU that loads the library, held until exit).
 * `sizes`, `offsets` and `total` are DEVICE pointers (total: one uint64 written by the GPU); the work is
 * queued on `stream` (a cudaStream_t, NULL = default stream) of `device` and is not waited for.
 * n above K2J_NOALLOC_SCAN_MAX is rejected with K2J_ERR_INVALID_ARGUMENT.  The first call on a device
 * looks up the scratch address and should come before any stream capture on that device.  All calls
 * on a device share the scratch: calls whose kernels could overlap on the GPU race and must be
 * ordered by the caller; nothing in the scratch needs clearing between calls.  With CUDA's default lazy
 * module loading the driver sets the kernels and the array up (and allocates for them) when they are first
 * used: one call with n >= 1 per device, or CUDA_MODULE_LOADING=EAGER, belongs before any region that must
 * not allocate.  The looked-up address does not survive cudaDeviceReset: do not use the entry point across
 * one.  The caller's current device is the same after the call as before. */
#define K2J_NOALLOC_SCAN_MAX (1ull << 24)
k2j_status k2j_exclusive_scan_u32_noalloc(int device, void* stream, const uint32_t* sizes, uint64_t n,
                                          uint64_t* offsets, uint64_t* total);

/* Device pointer and size of the text produced by the last run (valid until the next run). */
k2j_status k2j_output(k2j_ctx* ctx, const void** device_ptr, uint64_t* n_bytes);
/* Copies the text to host memory (pinned memory makes the copy asynchronous up to its final wait). */
k2j_status k2j_copy_output(k2j_ctx* ctx, void* host_dst, uint64_t capacity);
/* The same copy, only enqueued on the context's stream: it returns before the bytes have arrived.
 * k2j_synchronize (or any later call that waits on the stream) completes it; the context's output must
 * not be overwritten by another run before that.  A caller with two contexts can so keep the copy of
 * one trace running while the next trace is uploaded and formatted (no reference counterpart: the
 * reference writes its file synchronously, libkineto/src/output_json.cpp:1098-1107). */
k2j_status k2j_copy_output_async(k2j_ctx* ctx, void* host_dst, uint64_t capacity);
/* Writes the text to an open file descriptor at its current position: the device-to-host copy runs in chunks
 * through two pinned staging buffers of the context, so the copy of one chunk overlaps the write() of the one
 * before it, and the text is never held whole in host memory.  `written` (optional) receives the byte count.
 * Stands where the reference streams its events into an ofstream (libkineto/src/output_json.cpp:485-492,
 * :237-259); the caller keeps the reference's temporary-file-then-rename protocol (:1098-1107).
 * A failed write() returns K2J_ERR_IO with errno's text as the context's last error. */
k2j_status k2j_write_output(k2j_ctx* ctx, int fd, uint64_t* written);
/* The same for the bytes [begin, begin + n_bytes) of the text, written with pwrite at `file_offset` (the
 * descriptor's position is neither used nor moved).  Several contexts, in one process or in several, so fill
 * disjoint parts of one file: the shards of a trace write their CPU-op events and their GPU-side events where
 * they belong in the whole trace's text (the reference is single-process and has no counterpart;
 * libkineto/src/output_membuf.h:91-107 fixes the order of the parts). */
k2j_status k2j_write_output_at(k2j_ctx* ctx, int fd, uint64_t file_offset, uint64_t begin, uint64_t n_bytes);
/* Waits for everything enqueued on the context's stream. */
k2j_status k2j_synchronize(k2j_ctx* ctx);

/* ---- host-side string table: for callers that hold the drained buffers as CUPTI wrote them ----
 * In such a buffer the `name` field of a kernel record is a `const char*` into CUPTI's memory, and the reference
 * demangles it for every activity it logs (libkineto/src/CuptiActivity.h:297-300, libkineto/src/Demangle.cpp:33-53).
 * k2j_intern_kernel_names walks the buffers (the (byte offset, valid bytes) table of k2j_set_cupti, records sized
 * by kind the same way) IN PLACE and replaces each CONCURRENT_KERNEL record's name pointer by the id of its
 * name in `names` - demangled as Demangle.cpp does when `demangle` is non-zero (names above 8192 bytes and names
 * the demangler rejects are kept; a null pointer is the empty string) - so that the bytes can go to k2j_set_cupti
 * as they are.  Each distinct pointer is demangled once; buffers are walked on up to 16 host threads; ids are
 * given in order of first sight, so the result does not depend on the thread count.  The pointers must be
 * readable NUL-terminated strings when the call is made (CUPTI keeps them for the life of the module).  No GPU work.
 * k2j_names_intern gives the id of any other string of the trace (CPU-op names, metadata keys and values, callback
 * names); k2j_names_pool returns the pool in the layout k2j_set_strings takes (valid until the next call that
 * adds a string).  One table per trace; not thread-safe. */
typedef struct k2j_names k2j_names;
k2j_status k2j_names_create(k2j_names** out);
void k2j_names_destroy(k2j_names* names);
k2j_status k2j_names_intern(k2j_names* names, const char* s, uint64_t len, uint32_t* id);
k2j_status k2j_names_pool(const k2j_names* names, const uint64_t** off, const uint8_t** data, uint64_t* n_strings);
k2j_status k2j_intern_kernel_names(k2j_names* names, uint8_t* bytes, uint64_t n_bytes, const uint64_t* buftab,
                                   uint32_t n_buffers, int demangle, uint64_t* n_kernel_records);

/* Library version string. */
const char* k2j_version(void);

#ifdef __cplusplus
}
#endif
#endif /* K2J_H_ */
