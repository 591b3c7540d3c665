/*
 * recflex_b200.h — C ABI of librecflex_b200.so: the fused multi-feature
 * embedding-bag forward (sum pooling, per-feature outputs concatenated into
 * one [batch, sum(dim_f)] fp32 matrix) for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *  - Every function returns 0 on success and a negative EB_ERR_* code on
 *    failure; eb_last_error() returns a thread-local message for the last
 *    failure.  No C++ exception crosses this boundary.
 *  - The caller owns every buffer.  The library allocates device memory only
 *    inside eb_create() (a descriptor table of a few KB per handle, released
 *    by eb_destroy()) and eb_peer_alloc(); all per-call scratch lives in the
 *    caller's `workspace`.
 *  - Every launch goes to the `stream` argument (a cudaStream_t passed as
 *    void*, so that this header needs no CUDA include).
 *  - A handle is not thread-safe: use one handle per host thread / stream.
 *
 * Each entry point names the piece of the RecFlex reference it replaces
 * (paths are relative to the RecFlex repository root).
 */
#ifndef RECFLEX_B200_H_
#define RECFLEX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EB_OK 0
#define EB_ERR_INVALID_ARG (-1)
#define EB_ERR_CUDA (-2)
#define EB_ERR_WORKSPACE_TOO_SMALL (-3)
#define EB_ERR_BAD_INPUT (-4)      /* device-side input check failed (index out of range, offsets not monotone) */
#define EB_ERR_UNSUPPORTED (-5)
#define EB_ERR_TOO_LARGE (-6)

/* table_dtype values */
#define EB_F32 0
#define EB_F16 1
/* out_dtype values (eb_set_output_dtype): element type of the pooled output */
#define EB_OUT_F32 0
#define EB_OUT_BF16 1
#define EB_OUT_F16 2
/* index_dtype values (values and offsets share one dtype, as in torch.nn.EmbeddingBag) */
#define EB_I32 0
#define EB_I64 1

/*
 * Per-feature schedule kinds.  They play the role of the reference's schedule
 * classes (examples/schedules/*.py + examples/csrc/include/*_kernel.cuh):
 *   EB_SCHED_GROUP  a sub-warp group of `row_bytes/16` lanes owns one bag and
 *                   walks it serially (thread-per-bag for 16-byte rows); no
 *                   cross-lane reduction.  Replaces ws::SparseSegmentReduce
 *                   (warp_per_sample_kernel.cuh:10-82) and the one-hot row copy
 *                   onehot::GatherSegments (onehot_kernel.cuh:14-87).
 *   EB_SCHED_WARP   a whole warp owns one bag; its 32/(row_bytes/16) row slots
 *                   each take a contiguous run of the bag (indices fetched 2 or
 *                   4 at a time) and are combined with warp shuffles.  For
 *                   long, evenly sized bags.  These features are pooled by a
 *                   separate lean kernel (one CTA per 8 bags, 8 CTAs per SM, two
 *                   or four rows per lane in flight: unroll <= 2 -> 2, else 4)
 *                   launched right before the fused kernel.  Replaces
 *                   obms::SparseSegmentReduce
 *                   (one_block_multi_sample_kernel.cuh:16-108) and, for long
 *                   bags, ws::SparseSegmentReduce.
 *   EB_SCHED_FLAT   a warp streams the flattened index list of a run of bags,
 *                   dealing consecutive entries round-robin to its row slots,
 *                   keeps `unroll` rows per lane in flight regardless of bag
 *                   boundaries and resolves the boundaries with a segmented
 *                   warp reduction.  Replaces rbk::SparseSegmentSum
 *                   (reduce_by_key_kernel.cuh:185-366) without its inter-block
 *                   barrier and without leaving empty bags unwritten.
 *   EB_SCHED_STREAM the same flattened stream cut into one contiguous piece per
 *                   row slot; each slot walks its piece serially (no reduction
 *                   inside a piece), bags cut by a piece boundary are patched
 *                   once per 32 bags with a segmented shuffle scan.  Load
 *                   balanced over indices like rbk:: and mbs::
 *                   (multi_block_per_sample_kernel.cuh:17-112) but with neither
 *                   atomics nor scans in the inner loop.
 *   EB_SCHED_PIPE   EB_SCHED_STREAM with the rows in flight kept in a per-warp
 *                   shared-memory ring filled by per-lane cp.async copies
 *                   (unroll 2 / 4 / 6 / 8 -> 4 / 3 / 2 / 2 macro-steps deep:
 *                   8, 12, 12 or 16 rows per lane in flight) instead of in
 *                   registers: more bytes in flight per lane, fewer registers;
 *                   costs 48 KB (64 KB at unroll 8) of shared memory per CTA, so
 *                   at most 4 (3) CTAs per SM run (a higher occupancy setting is
 *                   honoured only up to what fits).  No counterpart in the
 *                   reference.
 *   EB_SCHED_AUTO   the library's default: EB_SCHED_STREAM with four rows in flight, whatever the feature
 *                   looks like.  Choosing per feature from dim, dtype and bag lengths is the tuner's job
 *                   (recflex_b200/tuning.py), which replaces this default.
 */
#define EB_SCHED_AUTO 0
#define EB_SCHED_GROUP 1
#define EB_SCHED_WARP 2
#define EB_SCHED_FLAT 3
#define EB_SCHED_STREAM 4
#define EB_SCHED_PIPE 5

typedef struct eb_handle eb_handle;

/* One feature's schedule = the reference's (ScheduleBase subclass, params NamedTuple)
 * pair (RecFlex/code_emitter/schedule_base.py:54-87). */
typedef struct eb_schedule {
  int32_t kind;          /* EB_SCHED_* */
  int32_t unroll;        /* rows per lane and macro-step: 1, 2, 4 or 8, or 6 with EB_SCHED_PIPE (0 = auto); batches with 64-bit indices always run at 4 */
  int32_t vec_bytes;     /* bytes per lane per row load: 16 (0 = auto; rows that are not 16-byte multiples use the element-wise fallback) */
  int32_t bags_per_tile; /* bags bound to one warp per tile; 0 = chosen on the device from the batch's mean bag length */
} eb_schedule;

/*
 * Create a handle for `num_features` embedding tables that live on `device`.
 * rows[f] x dims[f] row-major, dtype table_dtype[f] (EB_F32 / EB_F16),
 * table_ptrs[f] = device pointer.  The tables must stay allocated and in place
 * for the life of the handle.
 * Replaces FeatEmbed.__init__ + torch.ops.recom.get_gpu_pointers_array
 * (RecFlex/rec_modules.py:57-76, RecFlex/sched_basic_csrc/gpu_pointers_array.cc:16-25).
 */
int eb_create(eb_handle** out, int device, int num_features, const int64_t* rows,
              const int32_t* dims, const int32_t* table_dtype,
              const void* const* table_ptrs);

/* Release the handle and its device descriptor table. */
int eb_destroy(eb_handle* h);

/* Sum of dims = width of one output row (FeatEmbed.output_units, rec_modules.py:74-76). */
int eb_output_units(const eb_handle* h, int64_t* units);

/*
 * Set every feature's schedule and the CTAs-per-SM occupancy (1..8, 0 = keep)
 * of the fused kernel.  Replaces the code generation + compilation of one
 * FusedKnl per schedule assignment (RecFlex/code_emitter/codegen.py:221-383,
 * 474-494): every schedule variant is already compiled into the library.
 */
int eb_set_schedules(eb_handle* h, const eb_schedule* per_feature, int occupancy);

/* Read back the schedules in force (after AUTO resolution) and the occupancy. */
int eb_get_schedules(const eb_handle* h, eb_schedule* per_feature, int* occupancy);

/* Bytes of device scratch one forward call needs (independent of the batch size). */
int eb_workspace_bytes(const eb_handle* h, size_t* bytes);

/*
 * Persistent CTAs the fused kernel runs at `occupancy` CTAs per SM
 * (0 = the handle's current occupancy).  Replaces
 * torch.ops.recom.get_max_concurrent_blocks
 * (RecFlex/code_emitter/codegen.py:446-452, RecFlex/sched_basic_csrc/include/utils.cuh:6-21).
 */
int eb_max_concurrent_ctas(const eb_handle* h, int occupancy, int* ctas);

/*
 * The fused forward.  values_ptrs[f] / offsets_ptrs[f] are DEVICE pointers to
 * feature f's indices (nnz_f entries) and bag offsets (batch entries, or
 * batch+1 when offsets_have_end != 0, the last one being nnz_f).  nnz[f] is a
 * HOST array with each feature's index count (ignored, may be NULL, when
 * offsets_have_end != 0).  out is a DEVICE fp32 matrix [batch, out_ld] whose
 * first eb_output_units() columns receive the pooled rows (out_ld >= units
 * lets a caller write into a slice of a wider buffer).  Every element of those
 * columns is written; empty bags pool to 0.
 * Replaces recom_host.preprocess's tiling/task mapping + torch.ops.recom.process
 * (RecFlex/code_emitter/codegen.py:90-181, 387-444;
 *  RecFlex/sched_basic_csrc/task_mapping.cu:6-18) — the block-to-feature binding
 * is computed on the device from the batch itself.
 */
int eb_forward(eb_handle* h, int64_t batch, const void* const* values_ptrs,
               const void* const* offsets_ptrs, const int64_t* nnz, int index_dtype,
               int offsets_have_end, float* out, int64_t out_ld, void* workspace,
               size_t workspace_bytes, void* stream);

/*
 * Same, for one packed (jagged) batch: `values` holds all features' indices
 * back to back in feature order, `offsets` is a [num_features, batch+1] matrix
 * of per-feature offsets (each row starts at 0 and ends at nnz_f; in eb_forward
 * a feature's first offset may be any position of its index list).  Both are
 * DEVICE pointers; nothing is uploaded per call.
 * Replaces the packed d_arg_buffers / d_arg_buffer_offsets arguments of
 * FusedKnl (RecFlex/code_emitter/codegen.py:144-160, 318-331).
 */
int eb_forward_packed(eb_handle* h, int64_t batch, const void* values, const void* offsets,
                      int index_dtype, float* out, int64_t out_ld, void* workspace,
                      size_t workspace_bytes, void* stream);

/*
 * End-to-end call with HOST buffers (pinned memory recommended): copies the
 * packed batch to `staging` (device scratch of at least eb_host_staging_bytes),
 * runs the fused forward and copies the [batch, units] result back to host_out.
 * Returns after enqueueing; the caller synchronises `stream`.
 * Replaces FeatProcessEmbed.forward's upload + launch
 * (RecFlex/rec_modules.py:27-42, 127-133).
 */
int eb_forward_host(eb_handle* h, int64_t batch, const void* host_values, int64_t total_nnz,
                    const void* host_offsets, int index_dtype, float* host_out,
                    void* staging, size_t staging_bytes, void* workspace,
                    size_t workspace_bytes, void* stream);
int eb_host_staging_bytes(const eb_handle* h, int64_t batch, int64_t total_nnz,
                          int index_dtype, size_t* bytes);

/*
 * The fused forward with per-feature device time, the counterpart of
 * `timing=True` (RecFlex/code_emitter/codegen.py:301-316, 396-401;
 * RecFlex/rec_modules.py:96-109): each tile's clock64() delta is summed per
 * feature and converted to nanoseconds with the device's nominal (maximum) SM
 * clock, as the reference converts its clock() deltas with cudaDevAttrClockRate.
 * The figures rank a feature's schedules against each other; they are not
 * absolute times whenever the SM clock runs below its maximum.  per_feature_ns
 * is a HOST array of num_features doubles; the call synchronises `stream`.
 */
int eb_forward_timed(eb_handle* h, int64_t batch, const void* const* values_ptrs,
                     const void* const* offsets_ptrs, const int64_t* nnz, int index_dtype,
                     int offsets_have_end, float* out, int64_t out_ld, void* workspace,
                     size_t workspace_bytes, void* stream, double* per_feature_ns);

/*
 * Kernel timing.  eb_kernel_timing(h, 1) makes every later forward record a
 * CUDA event pair around its kernels: the binding kernel, the warp-per-bag
 * kernel when a feature uses it, and the fused kernel (a ring of 256 pairs).  eb_kernel_times() waits for the
 * recorded pairs, writes the elapsed milliseconds of each launch since the
 * previous read (oldest first, at most `cap`) and clears the ring.  This is the
 * in-process counterpart of the reference's global-stage measurement, the
 * FusedKnl total from `nsys stats --report gpukernsum`
 * (RecFlex/parser.py:71-85, RecFlex/tuning/measure.py:98-122).
 */
int eb_kernel_timing(eb_handle* h, int enable);
int eb_kernel_times(eb_handle* h, float* ms, int cap, int* count);

/*
 * Copy the device status word of the last forward that used `workspace` and
 * return EB_ERR_BAD_INPUT when the kernel met an index outside [0, rows) or a
 * decreasing offset (such entries are skipped, never dereferenced).
 * Synchronises `stream`.  The reference performs no such check.
 */
int eb_check_status(eb_handle* h, void* workspace, void* stream);

/*
 * The run-time binding of the last forward that used `workspace`: how many bags
 * the device bound to one warp tile, per feature (HOST array of num_features
 * entries; ceil(batch / bags_per_tile[f]) is the feature's tile count).
 * Synchronises `stream`.  The counterpart of reading the per-batch block counts
 * of the reference's host preprocess (RecFlex/tuning/measure.py measure_task_blocks,
 * used by Tuner.tune_fixed_thread_binding, RecFlex/tuning/tuner.py:312-357).
 */
int eb_last_binding(eb_handle* h, void* workspace, void* stream, int32_t* bags_per_tile);

/*
 * Fill a table with the library's counter-based synthetic weights: element
 * (row, col) of a table with `seed` is a fixed integer hash mapped to an
 * approximately normal value of standard deviation `std`; any row can be
 * regenerated on any device or on the CPU without storing the table.
 * Stands in for torch.randn table creation (RecFlex/rec_modules.py:64-68).
 */
int eb_fill_table(void* table, int64_t rows, int32_t dim, int32_t table_dtype, uint64_t seed,
                  float std, int device, void* stream);

/*
 * Place the features' outputs at arbitrary columns: feature f writes columns
 * [first_column[f], first_column[f] + dim_f) of an output row that is `units`
 * wide (NULL restores the default, features side by side).  Used by the sharded
 * path, where a rank's features go to their canonical columns of the global
 * [batch, sum of all dims] layout.  No counterpart in the reference, whose
 * column offsets are compile-time constants (d_embed_dim_offsets,
 * RecFlex/code_emitter/codegen.py:287-292).
 */
int eb_set_output_columns(eb_handle* h, const int32_t* first_column, int64_t units);

/*
 * Fused pooling + exchange for table-wise sharding (no counterpart in the
 * reference): like eb_forward, but sample b of the batch is stored into the
 * output matrix of rank b / (batch / world), at row b % (batch / world).
 * peer_out[r] is THIS process's device pointer to rank r's [batch / world,
 * out_ld] fp32 matrix (its own for r == its rank, peers' through
 * eb_peer_open), so the pooled rows cross NVLink as plain stores from the
 * kernel that computes them and no all-to-all or re-layout pass follows.
 * batch / world must be a multiple of 32, world <= 16.  The kernel never waits
 * on another GPU; the caller orders consumers after ALL ranks' kernels (for
 * example with an all-reduce on the same stream) and must not let a rank start
 * step k + 2 into a buffer a peer may still be reading from step k.
 */
int eb_forward_peers(eb_handle* h, int64_t batch, const void* const* values_ptrs,
                     const void* const* offsets_ptrs, const int64_t* nnz, int index_dtype,
                     int offsets_have_end, float* const* peer_out, int world, int64_t out_ld,
                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * Bags far longer than the rest.  A bag whose rows add up to `min_bytes` or
 * more (default 1 MB; 0 switches the mechanism off) is not pooled by the warp
 * that meets it, where it would be the kernel's tail: the EB_SCHED_STREAM /
 * EB_SCHED_PIPE walk hands it to a second kernel launched right after the fused
 * one, in which many warps pool segments of the bag and the warp that finishes
 * the last segment adds the partial sums in segment order (no atomics on the
 * data, the same bits on every run).  This is the library's block-per-bag
 * schedule; it replaces mbs::SparseSegmentReduceCore
 * (examples/csrc/include/multi_block_per_sample_kernel.cuh:17-112), which adds
 * its tiles with atomicAdd into an output it never zeroes.  At most 256 bags
 * per call are handed over (further ones are pooled in place); batches with
 * 64-bit indices, rows wider than 512 bytes, the chunked order of
 * eb_forward_exchange and eb_forward_packed_noalloc pool every bag in place.
 * The second kernel costs a few microseconds per call when no bag is long.
 */
int eb_set_long_bag_split(eb_handle* h, int64_t min_bytes);

/*
 * Element type of the pooled output (no counterpart in the reference, whose
 * output is hard-wired to fp32, RecFlex/code_emitter/codegen.py:416-421).
 * EB_OUT_F32 is the default and the contract the parity tests pin.
 * EB_OUT_BF16 / EB_OUT_F16 make every forward of this handle write its sums,
 * still accumulated in fp32, rounded to nearest even into 2-byte elements:
 * `out`, `out_ld` and the output buffers of the other entry points then count
 * such elements (pass the buffer cast to float*).  Meant for consumers that
 * cast anyway (the first linear layer of RecFlex/rec_modules.py:143-179's
 * RecomModel in bf16): it halves the bytes written, downloaded and exchanged.
 * A bag that the stream / pipe schedules cut in two has its first part rounded
 * once more on the way; empty bags are exactly 0 in every type.
 */
int eb_set_output_dtype(eb_handle* h, int out_dtype);

/*
 * Pooling + exchange through the copy engines for table-wise sharding (no
 * counterpart in the reference).  This rank pools ITS features for the whole
 * batch into `send` ([batch, send_ld] elements of the output dtype, this GPU's
 * memory) in ONE launch whose tile order walks the batch in `chunks` pieces:
 * sample b belongs to destination rank b / (batch / world), and piece k holds
 * rows [k, k + 1) * batch / (world * chunks) of every destination.  As soon as
 * the kernel has finished a piece (a device flag the kernel raises; the copy
 * streams wait for it with a stream memory operation, the host is not
 * involved), the `copy_streams` (1 to 16 streams of the caller; destinations
 * are dealt over them so that several copy engines work at once) copy the
 * piece's rows to every other rank: rank d receives them in peer_out[d]
 * ([batch / world, out_ld] elements, THIS process's pointer to rank d's
 * matrix, see eb_peer_open) at columns [out_col, out_col + output units), rows
 * in batch order.  This rank's own samples never enter the send buffer: the
 * kernel stores them straight into peer_out[rank].  The copies of piece k run
 * while piece k + 1 is pooled.  A kernel launched right after the
 * pooling kernel raises every flag, so the copy stream can never wait longer
 * than the pooling runs.  The caller orders consumers after `stream` (own
 * samples) and all ranks' copy streams, and must not reuse `send` before the
 * copy streams are done with it.
 * batch must be a multiple of world * chunks; world <= 16, chunks <= 64.
 * The flags live in `workspace` and count calls: zero-fill a workspace once
 * before its first use here.
 * Returns EB_ERR_UNSUPPORTED when the driver has no stream memory operations.
 */
int eb_forward_exchange(eb_handle* h, int64_t batch, const void* const* values_ptrs,
                        const void* const* offsets_ptrs, const int64_t* nnz, int index_dtype,
                        int offsets_have_end, float* send, int64_t send_ld, float* const* peer_out,
                        int world, int rank, int64_t out_ld, int64_t out_col, int chunks,
                        void* workspace, size_t workspace_bytes, void* stream,
                        void* const* copy_streams, int num_copy_streams);

/*
 * Who ships the finished pieces of eb_forward_exchange (no counterpart in the
 * reference).  EB_EXCHANGE_COPY_ENGINES (default): cudaMemcpy2DAsync /
 * cudaMemcpyAsync on the copy streams.  EB_EXCHANGE_SM_PUSH: a small kernel on
 * the first copy stream (128-thread CTAs that fit beside the pooling kernel's),
 * whose warps load 512-byte runs of the send buffer and store them to the peer,
 * so that full lines cross NVLink; needs rows, leading dimensions and column
 * offsets that are multiples of 16 bytes and falls back to the copy engines
 * otherwise.
 */
#define EB_EXCHANGE_COPY_ENGINES 0
#define EB_EXCHANGE_SM_PUSH 1
int eb_set_exchange_engine(eb_handle* h, int engine);

/*
 * Splits eb_forward_exchange between the two ways a row can travel (no
 * counterpart in the reference): the rows for the `hops` ranks to the right of
 * this one (rank + 1 ... rank + hops, modulo world) are stored by the pooling
 * kernel straight into those ranks' result blocks, like this rank's own rows;
 * only the remaining destinations go through the send buffer and the copy
 * streams.  Kernel stores and copy engines are limited by different things, so
 * together they can move more than either alone.  0 (default): every other
 * rank is served by copies; world - 1 or more: none is.
 */
int eb_set_exchange_direct(eb_handle* h, int hops);

/*
 * Overlap of the two pooling kernels (no counterpart in the reference, whose
 * single generated kernel holds every schedule).  0 (the default): features on
 * EB_SCHED_WARP are pooled by their own kernel, then the fused kernel pools the
 * rest, both on the caller's stream.  n > 0: the fused kernel is launched first
 * on n CTAs per SM (never more than the occupancy given to eb_set_schedules)
 * and the warp-per-bag kernel runs beside it on a stream the handle owns,
 * forked from and joined back into the caller's stream with events, so the
 * caller sees the usual stream order.  Only used when some, but not all,
 * features are on EB_SCHED_WARP; eb_forward_timed keeps the serial order.
 */
int eb_set_kernel_overlap(eb_handle* h, int fused_ctas_per_sm);

/*
 * Order in which eb_forward_peers walks the batch (no counterpart in the
 * reference).  enabled != 0 (the default): consecutive tiles of a feature are
 * dealt round-robin over the destination ranks, so that every GPU of the node
 * stores to all the others at any moment.  0: batch order, i.e. rank 0's rows
 * first on every GPU.  The results are the same either way.
 */
int eb_set_peer_interleave(eb_handle* h, int enabled);

/*
 * Device buffers other processes of this node can map (CUDA IPC): eb_peer_alloc
 * allocates `bytes` on `device` and fills a 64-byte handle to send to the other
 * ranks; eb_peer_open maps a peer's handle into this process (the returned
 * pointer is valid on `device`); eb_peer_close unmaps; eb_peer_free releases an
 * eb_peer_alloc buffer.  These are the only other allocating calls besides
 * eb_create.
 */
int eb_peer_alloc(int device, size_t bytes, void** ptr, unsigned char* handle64);
int eb_peer_open(int device, const unsigned char* handle64, void** ptr);
int eb_peer_close(int device, void* ptr);
int eb_peer_free(int device, void* ptr);

/*
 * Column placement for table-wise sharding (no counterpart in the reference,
 * which has no multi-GPU data path): after the all-to-all of pooled outputs a
 * rank holds, back to back, one block [rows, sum(dim of sender s's features)]
 * per sender.  This copies every feature's columns to its canonical place in
 * dst [rows, dst_ld].  `segments` is a DEVICE array of num_segments records
 * {int64 src_off; int32 src_ld; int32 dst_col; int32 width; int32 pad}: element
 * offset (from src) of the feature's first column in row 0 of its block, the
 * block's row length, the destination column and the feature's dim.
 */
int eb_place_columns(const float* src, float* dst, int64_t rows, int64_t dst_ld, int32_t num_segments,
                     const void* segments, int device, void* stream);

/*
 * Device-side ingestion of a lengths-based jagged batch: `lengths` is a DEVICE
 * [num_features, batch] matrix of bag lengths (values and lengths share one
 * integer dtype); writes the DEVICE [num_features, batch + 1] offsets matrix
 * eb_forward_packed expects (row f = exclusive prefix sum of feature f's
 * lengths, last entry = nnz_f).  Replaces the offsets part of the host
 * preprocess (examples/csrc/warp_per_sample_preprocess.cu:14-33: the running
 * segment_offsets) for inputs that arrive as lengths.
 */
int eb_offsets_from_lengths(const void* lengths, void* offsets, int32_t num_features, int64_t batch,
                            int index_dtype, int device, void* stream);

/*
 * Host-side parser of the reference's text input: `text` holds `batch` lines
 * separated by '\n' (one bag per line, indices separated by any non-digit
 * character, an empty line is an empty bag).  Writes the indices to values_out
 * (capacity values_cap) and batch+1 offsets to offsets_out; *nnz_out receives
 * the index count.  Replaces ws::StringSplitToInt
 * (examples/csrc/warp_per_sample_preprocess.cu:6-38).
 */
int eb_parse_bags(const char* text, size_t text_len, int64_t batch, int32_t* values_out,
                  int64_t values_cap, int32_t* offsets_out, int64_t* nnz_out);

/*
 * The packed fused forward for callers that cannot allocate device memory at
 * all: a plugin inside a server whose memory pool owns every byte and treats a
 * driver allocation as an error, a sandbox that forbids allocation calls, or a
 * latency path where an allocation's implicit device synchronisation is not
 * acceptable.  Those callers can use neither eb_create() (it allocates the
 * descriptor table) nor a workspace of their own.  This entry point has no
 * counterpart in the reference, whose launcher allocates per call
 * (RecFlex/code_emitter/codegen.py:416-421).
 *
 * It takes the tables directly (same meaning as eb_create's arguments), one
 * packed batch (as eb_forward_packed) and the output, and calls no cudaMalloc,
 * cudaFree or other allocating routine.  Descriptors and scratch live in one
 * array built into the library image (about 121 KB of device memory on every
 * GPU that loads the library, until the process exits), which bounds it to
 * EB_NOALLOC_MAX_FEATURES features: more are refused with EB_ERR_TOO_LARGE.
 * Schedules are the library defaults at 4 CTAs per SM.
 *
 * All calls on a GPU share that array and it keeps the previous call's
 * contents; each call rewrites the descriptors and its binding kernel resets
 * the counters and the status word, so back-to-back calls on one stream are
 * safe, while calls whose kernels overlap on the GPU (other streams) race.
 * On the host, calls for one GPU are serialised by a lock and every GPU has
 * its own staging buffer, so threads driving different GPUs do not interfere.
 * The first call on each device resolves the array's device address
 * (cudaGetSymbolAddress); make that first call before any stream capture
 * begins.  Every call stages its descriptors through host memory that the next
 * call overwrites, so a call is refused (EB_ERR_UNSUPPORTED) while its stream
 * is being captured.  At most 16 devices per process.
 *
 * eb_noalloc_check_status reads the status word of the last call on `device`
 * out of the built-in array (the role eb_check_status plays for a handle's
 * workspace): EB_ERR_BAD_INPUT when that call met an index outside [0, rows)
 * or offsets that had to be clamped.  Synchronises `stream`; allocates nothing.
 */
#define EB_NOALLOC_MAX_FEATURES 1024
int eb_forward_packed_noalloc(int device, int num_features, const int64_t* rows, const int32_t* dims,
                              const int32_t* table_dtype, const void* const* table_ptrs, int64_t batch,
                              const void* values, const void* offsets, int index_dtype, float* out,
                              int64_t out_ld, void* stream);
int eb_noalloc_check_status(int device, void* stream);

/* Message of the calling thread's last failure ("" if none). */
const char* eb_last_error(void);

/* Library version string and the SM architecture it was compiled for. */
const char* eb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* RECFLEX_B200_H_ */
