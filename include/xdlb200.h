/*
 * xdlb200.h - C ABI of libxdlb200.so: hand-written sm_100a CUDA kernels for the
 * CTR-inference hot path of Blaze (alibaba/x-deeplearning, directory blaze/).
 *
 * Conventions
 *   - every pointer named in an argument struct is a DEVICE pointer unless its
 *     comment says "host";
 *   - every entry point returns 0 when the work was enqueued on `stream`, and a
 *     negative xb_status when an argument was rejected (nothing is launched);
 *     xb_last_error() returns the reason for the calling thread;
 *   - nothing here synchronises the stream, and the compute entry points do not
 *     allocate: scratch memory is passed in by the caller;
 *   - data types use Blaze's DataType numbering (blaze/blaze/proto/blaze.proto:6-20).
 *
 * Each entry point names the reference interface (path inside the reference
 * project, file:line) that a Blaze CUDA operator would replace with it.
 */
#ifndef XDLB200_H_
#define XDLB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* xb_stream_t; /* cudaStream_t */

enum xb_status {
  XB_OK = 0,
  XB_ERR_ARG = -1,       /* bad argument (shape, dtype, alignment, null pointer) */
  XB_ERR_UNSUPPORTED = -2,
  XB_ERR_CUDA = -3,      /* a CUDA runtime/driver call failed */
  XB_ERR_SCRATCH = -4,   /* scratch buffer too small */
  XB_ERR_LIMIT = -5      /* size beyond a documented maximum */
};

enum xb_dtype {
  XB_F32 = 1,
  XB_I32 = 2,
  XB_I64 = 10,
  XB_F16 = 12,
  XB_BF16 = 14,          /* extension: not a Blaze type */
  XB_REC64 = 110         /* extension, id lists only: 8-byte routing records (segment << 32) | row, the row is used */
};

/* Reason of the last non-zero return on this thread ("" if none). */
const char* xb_last_error(void);
/* Library version and the SM architecture the kernels were compiled for. */
const char* xb_version(void);
/* Device-side status of the tensor-core kernels on the current device. Every
 * wait inside them (mbarrier, TMEM) is bounded; a wait that runs out records
 * (site << 8 | 1) and the kernel tears down and returns instead of hanging.
 * *status is 0 when no wait ever ran out. Synchronise the stream first.
 * xb_device_status_clear() resets the word. */
int xb_device_status(int* status);
int xb_device_status_clear(void);
/* Maps the status word of the current device into host memory and returns its address (one small pinned
 * allocation per device, made by the first call; later calls return the same address). After a stream
 * synchronisation *host_word != 0 says what xb_device_status would, without a device-to-host copy, so a
 * serving loop can test it after every request. Once a wait has run out, later waits on that device give
 * up after a few microseconds until xb_device_status_clear is called (it resets the mirror too): a
 * long-lived process must clear the word when it has reported the failure. No counterpart in the
 * reference, whose kernels have no bounded waits. */
int xb_device_status_mirror(const volatile int** host_word);

/* ------------------------------------------------------------------------- */
/* Embedding tables in HBM.
 * Replaces the in-memory image of QuickEmbeddingDict (hash table + weight blob,
 * blaze/blaze/store/quick_embedding/quick_embedding_dict.h:18-110).
 * Rows are stored at a fixed pitch that is a multiple of 16 bytes so a row is
 * fetched with 128-bit loads. The key index is open addressing over
 * (key,row) slots; with slot_keys == NULL keys are row numbers. */
typedef struct xb_table_desc {
  const void* weights;          /* row r at weights + r * row_pitch_bytes */
  int64_t rows;
  int32_t dim;
  int32_t dtype;                /* XB_F32 or XB_F16 storage */
  int64_t row_pitch_bytes;      /* multiple of 16 */
  const int64_t* slot_keys;     /* [slots] or NULL for identity keys */
  const int32_t* slot_rows;     /* [slots], -1 = empty */
  int64_t slots;                /* power of two */
} xb_table_desc;

/* Pitch the library uses for a (dim, dtype) table. */
int64_t xb_table_row_pitch(int32_t dim, int32_t dtype);
/* Allocates device memory and uploads a table. `weights_host` is row-major
 * [rows, dim] fp32 on the HOST and is converted to `dtype`; `keys_host`
 * ([rows] int64, host) may be NULL for identity keys. On success *out owns
 * the device buffers until xb_table_destroy. A repeated key keeps its first row. */
int xb_table_create(xb_table_desc** out, int64_t rows, int32_t dim, int32_t dtype,
                    const float* weights_host, const int64_t* keys_host);
/* Replica of a table that lives on device `src_device`, on the CURRENT device (device-to-device copies; the
 * host image is not needed again). One serving process holds one replica per device it serves
 * (blaze/blaze/api/cpp_api/predictor_manager_impl.cc:142-177 creates predictors per device id). */
int xb_table_clone(xb_table_desc** out, const xb_table_desc* src, int32_t src_device);
void xb_table_destroy(xb_table_desc* t);
/* Host-side builder of the open-addressing index: fills slot_keys/slot_rows
 * (host arrays of `slots` entries, slots a power of two >= 2*rows). */
int xb_table_build_index_host(const int64_t* keys_host, int64_t rows, int64_t slots,
                              int64_t* slot_keys_host, int32_t* slot_rows_host);

/* ------------------------------------------------------------------------- */
/* Embedding pooling.
 * Replaces SparsePuller::Get (blaze/blaze/store/sparse_puller.h:77-83) as
 * implemented by QuickEmbeddingDict::Get
 * (blaze/blaze/store/quick_embedding/quick_embedding_dict.cc:89-147) with the
 * kSum/kAvg/kAssign processors (udf_processor.h:41-151). One xb_pool_group is one
 * SparsePullerInput/SparsePullerOutput pair; xb_pool_item is one
 * SparsePullerInput::Param + SparsePullerOutput::OutItem. */
enum { XB_UDF_SUM = 0, XB_UDF_AVG = 1, XB_UDF_ASSIGN = 2 };
enum { XB_TRUNC_ORDER = 0, XB_TRUNC_REVERSE = 1 };
#define XB_MAX_POOL_ITEMS 4
#define XB_MAX_POOL_GROUPS 32   /* groups per call; call again for more */

typedef struct xb_pool_item {
  int32_t udf;             /* XB_UDF_* */
  int32_t trunc_dir;       /* XB_TRUNC_*, kAssign only */
  int32_t trunc_num;       /* kAssign only */
  int32_t assign_stride;   /* elements between assigned rows; 0 = dim (Blaze layout) */
  void* out;               /* at the item's column offset inside its block */
  int64_t stride;          /* block row stride, elements */
} xb_pool_item;

typedef struct xb_pool_group {
  const xb_table_desc* table;  /* HOST pointer; NULL = table-name miss: outputs are zero-filled */
  const void* ids;             /* [n_ids] */
  const void* values;          /* [n_ids] per-id weights (values_dtype), NULL = all 1.0 */
  const int32_t* segments;     /* [batch] counts, or [batch+1] exclusive offsets into ids (they need not start
                                  at 0: several groups may share one id buffer) */
  int64_t n_ids;               /* ids the group's segments cover; with offsets it only sizes the work split,
                                  so an estimate is enough when the exact number is not known on the host */
  int64_t batch;
  int32_t dim;                 /* the group's configured dim (EmbeddingFeatureGroupConfig.dim); must
                                  equal table->dim when the table exists */
  int32_t id_dtype;            /* XB_I64 or XB_I32 (XB_REC64: routing records as received by an owner rank) */
  int32_t segments_are_offsets;
  int32_t out_dtype;           /* XB_F32 or XB_F16 */
  int32_t n_items;
  int32_t values_dtype;        /* XB_F32 (0 also means fp32) or XB_F16 */
  xb_pool_item items[XB_MAX_POOL_ITEMS];
} xb_pool_group;

/* Bytes of scratch xb_embedding_pool needs for these groups (offsets of the
 * groups that pass counts). */
size_t xb_embedding_pool_scratch_bytes(const xb_pool_group* groups, int32_t n_groups);
/* Every output element of every item is written (zero where nothing pools),
 * so the caller needs no memset (the reference op memsets first,
 * blaze/blaze/operator/sparse_op/embedding/embedding_op.h:181). */
int xb_embedding_pool(const xb_pool_group* groups, int32_t n_groups, void* scratch,
                      size_t scratch_bytes, xb_stream_t stream);

/* xb_embedding_pool for callers that cannot hand over device scratch: an operator
 * that runs inside someone else's memory plan (a serving process whose device
 * memory was carved up at start-up, a plug-in that is given input and output
 * buffers and nothing else, code running while the framework's allocator is
 * locked) has nowhere to get the offsets buffer from and may not call cudaMalloc.
 * This entry point has no counterpart in the reference. It keeps the
 * counts->offsets scratch in a 1 MiB array that is part of the library image
 * (every GPU that loads the library holds that 1 MiB until the process exits),
 * and it calls no allocator of any kind.
 *   - Limit: xb_embedding_pool_scratch_bytes(groups, n_groups) must not exceed
 *     xb_embedding_pool_static_max_bytes(); a larger request is rejected with
 *     XB_ERR_LIMIT before anything is launched. Every group that passes counts
 *     takes 4*(batch+1) bytes of offsets rounded up to 256 PLUS the partial sums
 *     of the multi-block scan (4 bytes per 8192 samples, rounded up to 256), so
 *     size by that function, not by the offsets alone. Groups that pass
 *     exclusive offsets need none.
 *   - The first call on each device looks the array's address up; make that
 *     first call outside any stream capture.
 *   - All calls share the one array and it keeps whatever the previous call
 *     left. Nothing in it has to start at zero (every offset that is read is
 *     written by the same call first), but two calls that overlap on the GPU
 *     (different streams, or another thread) race on it: serialise them.
 * Inputs, outputs and results are exactly those of xb_embedding_pool. */
size_t xb_embedding_pool_static_max_bytes(void);
int xb_embedding_pool_static(const xb_pool_group* groups, int32_t n_groups, xb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Row-sharded embedding tables (tables too large for one GPU). The reference has no
 * multi-device path (Blaze is single-process, blaze/blaze/api/cpp_api/
 * predictor_manager_impl.cc:142-177); these entry points are the device side of the
 * exchange this project adds around xb_embedding_pool:
 *   rule    owner = (uint64)id % shards, local row = (uint64)id / shards
 *   step 1  xb_route_ids: bucket a rank's ids by owner with a stable counting sort;
 *           out_rows / out_values / out_tags hold bucket 0, then bucket 1, ...;
 *           out_tags[i] is the segment number (index into seg_offsets) the id belongs to;
 *           owner_counts[w] = size of bucket w (device, int64).
 *           With out_tags == NULL, out_rows receives packed records instead, (segment << 32) | local row
 *           (8 bytes per id on the wire instead of 12; local rows and segment numbers below 2^31), which
 *           xb_unpack_routed splits at the owner into int32 rows (xb_embedding_pool takes XB_I32 ids) and tags
 *   step 2  (caller) all-to-all of the buckets
 *   step 3  xb_tag_counts: segment lengths of what an owner received from one source rank
 *           (tags arrive in ascending order), then xb_embedding_pool over the local shard
 *           with identity keys -> partial sums [segments of every source, dim] fp32
 *   step 4  (caller) all-to-all of the partial sums back to the sources
 *   step 5  xb_shard_combine: out[sample, group*dim + e] = sum over owners 0..shards-1, in
 *           that fixed order, of partial[owner][group*rows + sample][e]; with avg != 0 the
 *           sum is multiplied by (float)(1.0 / seg_len) as kAvg does. */
size_t xb_route_scratch_bytes(int64_t n_ids, int32_t shards);
int xb_route_ids(const int64_t* ids, const float* values, const int32_t* seg_offsets, int64_t segments,
                 int64_t n_ids, int32_t shards, int64_t* out_rows, float* out_values, int32_t* out_tags,
                 int64_t* owner_counts, void* scratch, size_t scratch_bytes, xb_stream_t stream);
int xb_unpack_routed(const int64_t* packed, int64_t n, int32_t* rows, int32_t* tags, xb_stream_t stream);
int xb_tag_counts(const int32_t* tags, int64_t n, int32_t* counts, int64_t n_counts, xb_stream_t stream);
/* Step 3 for everything an owner received, in two calls instead of one per source rank and one pooling group per
 * (source, table) built by the caller. source_counts (HOST, [sources]) are the lengths of the source ranks' slices
 * of `tags`; counts[s * segments + t] receives the length of segment t of source s. xb_shard_pool then pools, for
 * every source s and table t, the segments [sum(table_segments[:t]), +table_segments[t]) of that source against
 * tables[t] (HOST arrays of n_tables entries); offsets [sources * S + 1] are the exclusive offsets of all
 * (source, segment) pairs into `rows` (S = sum(table_segments)); out [sources * S, dim] in out_dtype: XB_F32 (the
 * 1e-5 bar of fp32 models) or XB_F16 (a model whose tables and activations are fp16: each partial sum is rounded
 * once, which halves the bytes of the return exchange). xb_shard_combine takes the same dtype as partial_dtype and
 * always accumulates in fp32. Tags outside [0, segments) - they come from a peer - are ignored by the counting
 * kernels. */
int xb_tag_counts_sources(const int32_t* tags, const int64_t* source_counts, int32_t sources, int32_t* counts,
                          int64_t segments, xb_stream_t stream);
int xb_shard_pool(const xb_table_desc* const* tables, const int64_t* table_segments, int32_t n_tables,
                  const void* rows, int32_t row_dtype, int64_t n_rows, const float* values, const int32_t* offsets,
                  int32_t sources, int32_t dim, void* out, int32_t out_dtype, xb_stream_t stream);
int xb_shard_combine(const void* partial, int32_t partial_dtype, int32_t shards, int64_t segments, int32_t dim,
                     const int32_t* seg_len, int32_t avg, void* out, int64_t out_stride, int64_t groups,
                     int32_t out_dtype, xb_stream_t stream);

/* Fixed-capacity variant of step 1 for an exchange that never reads bucket sizes back to the host: bucket w starts
 * at out_records + w * bucket_cap, its slot 0 holds the number of packed records that follow (at most
 * bucket_cap - 1); a bucket that would not fit raises *overflow (device int, e.g. mapped host memory) and is cut.
 * xb_unpack_routed_padded splits `sources` received buckets into rows and tags in place (slots past a bucket's
 * count get tag -1, which the counting kernels ignore). xb_scan_counts turns n_arrays count arrays of `batch`
 * entries (counts_stride apart) into exclusive offsets of batch + 1 entries (offsets_stride apart).
 * xb_shard_pool_padded is xb_shard_pool over that layout: offsets [sources][S + 1] count from each source's
 * first record. */
int xb_route_ids_padded(const int64_t* ids, const int32_t* seg_offsets, int64_t segments, int64_t n_ids, int32_t shards,
                        int64_t bucket_cap, int64_t* out_records, int32_t* overflow, void* scratch, size_t scratch_bytes,
                        xb_stream_t stream);
int xb_unpack_routed_padded(const int64_t* packed, int32_t sources, int64_t bucket_cap, int32_t* rows, int32_t* tags,
                            xb_stream_t stream);
size_t xb_scan_counts_scratch_bytes(int32_t n_arrays, int64_t batch);
int xb_scan_counts(const int32_t* counts, int64_t counts_stride, int32_t* offsets, int64_t offsets_stride, int32_t n_arrays,
                   int64_t batch, void* scratch, size_t scratch_bytes, xb_stream_t stream);
int xb_shard_pool_padded(const xb_table_desc* const* tables, const int64_t* table_segments, int32_t n_tables,
                         const int32_t* rows, int64_t bucket_cap, const int32_t* offsets, int32_t sources,
                         int64_t n_rows_estimate, int32_t dim, void* out, int32_t out_dtype, xb_stream_t stream);
/* The same two steps without an unpacked copy of the received buckets: segment lengths counted from the records
 * themselves (counts [sources * segments], zeroed here), and pooling that reads the records as its id list. */
int xb_record_counts_padded(const int64_t* packed, int32_t sources, int64_t bucket_cap, int32_t* counts, int64_t segments,
                            xb_stream_t stream);
int xb_shard_pool_records(const xb_table_desc* const* tables, const int64_t* table_segments, int32_t n_tables,
                          const int64_t* records, int64_t bucket_cap, const int32_t* offsets, int32_t sources,
                          int64_t n_rows_estimate, int32_t dim, void* out, int32_t out_dtype, xb_stream_t stream);


/* The whole sharded step behind one call, with the two exchanges done by NCCL from inside the library (bound at
 * run time: libnccl.so.2 is needed only by processes that create a context for more than one rank). A context
 * belongs to one rank = one process and device; it owns every buffer of a step (allocated at creation) and its
 * NCCL communicator. xb_shard_unique_id makes the 128-byte communicator id on one rank; the caller hands it to
 * the others (any transport) and every rank calls xb_shard_ctx_create with it.
 *   tables[t]          this rank's shard of table t (identity keys: row = local row), all of `dim`
 *   table_segments[t]  segments of table t per step on THIS rank (feature groups of t x samples of this rank)
 *   max_ids            most ids one step of this rank may carry
 *   capacity_factor    bucket capacity = factor x max_ids / world (+ header): head room for owners that hold hot
 *                      rows; a step that exceeds it reports overflow = 1 through xb_shard_ctx_status
 * xb_sharded_pool enqueues the step on `stream` and returns; nothing in it waits for the device. ids / seg_offsets
 * as for xb_route_ids (segments numbered table after table, group-major inside a table); out [rows, >= groups * dim]
 * receives sum-pooled vectors, out[sample, g * dim + e] for segment g * rows + sample. xb_a2a_route and
 * xb_a2a_return are the two exchanges alone (ids out, partial sums back) for callers that run the owner-side
 * kernels themselves. xb_shard_ctx_status is read after the caller synchronised the stream: *overflow != 0 says
 * the last steps dropped ids (raise capacity_factor); an NCCL asynchronous error is returned as XB_ERR_CUDA. */
typedef struct xb_shard_ctx xb_shard_ctx;
typedef struct xb_shard_config {
  int32_t rank, world;
  int32_t dim;
  int32_t n_tables;
  const xb_table_desc* const* tables;   /* HOST array of HOST pointers */
  const int64_t* table_segments;        /* HOST */
  int64_t max_ids;
  int32_t partial_dtype;                /* XB_F32 or XB_F16 */
  float capacity_factor;                /* <= 1 means 1 */
} xb_shard_config;
int xb_shard_unique_id(void* id128);
int64_t xb_shard_bucket_capacity(int64_t max_ids, int32_t world, float capacity_factor);
int xb_shard_ctx_create(xb_shard_ctx** out, const void* unique_id128, const xb_shard_config* cfg);
void xb_shard_ctx_destroy(xb_shard_ctx* ctx);
int xb_sharded_pool(xb_shard_ctx* ctx, const int64_t* ids, const int32_t* seg_offsets, int64_t n_ids, int64_t groups,
                    int32_t avg, void* out, int64_t out_stride, int32_t out_dtype, xb_stream_t stream);
/* The same step in two halves, so that a caller can overlap the id exchange of step i+1 with the pooling of step i
 * (no reference counterpart): xb_sharded_pool_begin buckets the ids and enqueues their exchange on `stream`;
 * xb_sharded_pool_finish takes the oldest begun step, makes `stream` wait for that exchange and enqueues the rest.
 * At most two steps may be begun and not finished; every rank must issue begin and finish calls in the same order
 * (exchanges of one communicator run in issue order); the id and offset arrays of a begun step stay untouched
 * until its work has run. xb_sharded_pool is begin followed by finish on one stream. */
int xb_sharded_pool_begin(xb_shard_ctx* ctx, const int64_t* ids, const int32_t* seg_offsets, int64_t n_ids, xb_stream_t stream);
int xb_sharded_pool_finish(xb_shard_ctx* ctx, int64_t groups, int32_t avg, void* out, int64_t out_stride, int32_t out_dtype,
                           xb_stream_t stream);
/* xb_sharded_pool_finish itself in two parts, for a third pipeline stage: xb_sharded_pool_pool (segment lengths, owner
 * pooling, exchange of the partial sums; waits for the step's id exchange) and xb_sharded_pool_combine (waits for the
 * step's partial-sum exchange). Two steps may be pooled and not combined. With begin(i+2), pool(i+1), combine(i) issued
 * in that order on three streams, both exchanges of a step overlap kernels of its neighbours. */
int xb_sharded_pool_pool(xb_shard_ctx* ctx, xb_stream_t stream);
int xb_sharded_pool_combine(xb_shard_ctx* ctx, int64_t groups, int32_t avg, void* out, int64_t out_stride, int32_t out_dtype,
                            xb_stream_t stream);


int xb_a2a_route(xb_shard_ctx* ctx, const int64_t* ids, const int32_t* seg_offsets, int64_t n_ids, xb_stream_t stream);
int xb_a2a_return(xb_shard_ctx* ctx, xb_stream_t stream);
int xb_shard_ctx_status(xb_shard_ctx* ctx, int32_t* overflow);
int64_t xb_shard_ctx_bucket_capacity(const xb_shard_ctx* ctx);
size_t xb_shard_ctx_device_bytes(const xb_shard_ctx* ctx);
/* Optional phase timing of xb_sharded_pool (no reference counterpart): when enabled, the call records seven events on
 * its stream; after a stream synchronisation xb_shard_ctx_phase_ms gives the milliseconds of the last call's six
 * phases: bucket ids by owner, exchange ids, segment lengths + offsets, pool, exchange partial sums, combine. */
int xb_shard_ctx_profile(xb_shard_ctx* ctx, int32_t enable);
int xb_shard_ctx_phase_ms(xb_shard_ctx* ctx, float* ms6);


/* Measurement aid (no reference counterpart): gathers the `n` rows `row_ids` of `table` (rows of at most 64 bytes) and
 * discards them. Timed by the caller, it gives the rate at which this GPU can fetch rows at random addresses - the
 * ceiling of a pooling kernel on a table that does not fit L2. `sink` is one float of device memory. */
int xb_gather_probe(const xb_table_desc* table, const int32_t* row_ids, int64_t n, float* sink, xb_stream_t stream);

/* Self-test of the bounded waits (no counterpart in the reference): launches one warp that waits on a barrier
 * nothing will ever signal and gives up after `limit_cycles`. Afterwards xb_device_status reports a non-zero
 * word (site 99) until xb_device_status_clear, and every other entry point keeps working. */
int xb_selftest_wait_timeout(int64_t limit_cycles, xb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* GEMM family with fused bias + activation epilogue.
 * Replaces GemmOp::RunOnDevice (blaze/blaze/operator/op/gemm_op.h:33-107),
 * FusedParallelGemmOp::RunOnDevice (blaze/blaze/operator/fused_op/
 * fused_parallel_gemm_op.h:43-133), the strided-batched calls behind MatMul /
 * FusedParallelMatMul (blaze/blaze/math/gemm.h:50-79, math/broadcast.h:156-381)
 * and, through `epilogue`, a following Dice / PRelu / Sigmoid operator
 * (operator/op/dice_op.cu:11-21, prelu_op.cu:10-23, sigmoid_op.cu:11-17).
 *   Y[b] = act(alpha * op(A[b]) * op(B[b]) + beta * bias[b]),  b < batch
 * All matrices are row-major with explicit leading dimensions; a batch stride of
 * 0 re-uses the operand for every b (shared A of FusedParallelGemm). Y may point
 * at a column offset of a wider matrix (ldy > N) which gives axis-1 concat of the
 * branches for free. */
enum { XB_EPI_NONE = 0, XB_EPI_PRELU = 1, XB_EPI_DICE = 2, XB_EPI_SIGMOID = 3 };
enum { XB_BIAS_NONE = 0, XB_BIAS_ROW = 1 /* [N] */, XB_BIAS_FULL = 2 /* [M,N] */ };
enum { XB_GEMM_AUTO = 0, XB_GEMM_SIMT = 1, XB_GEMM_TCGEN05 = 2 };

typedef struct xb_gemm_args {
  int32_t M, N, K;
  int32_t trans_a, trans_b;
  float alpha, beta;
  const void* A; int64_t lda; int64_t stride_a;
  const void* B; int64_t ldb; int64_t stride_b;
  const void* bias; int64_t ldbias; int64_t stride_bias; int32_t bias_kind;
  void* Y; int64_t ldy; int64_t stride_y;
  int32_t batch;
  int32_t ab_dtype;        /* XB_F32, XB_F16 or XB_BF16: A and B */
  int32_t bias_dtype;      /* dtype of bias */
  int32_t y_dtype;
  int32_t epilogue;        /* XB_EPI_* */
  const float* ep_a;       /* PRelu: slopes [ep_count]; Dice: gamma [N] */
  const float* ep_b;       /* Dice: mean [N] */
  const float* ep_c;       /* Dice: var [N] */
  int32_t ep_count;        /* PRelu: number of slopes (1 = shared, else N) */
  int32_t dice_nosqrt;
  int64_t stride_ep;       /* per-batch stride of ep_a/b/c, elements (0 = shared) */
  int32_t engine;          /* XB_GEMM_AUTO picks tcgen05 when the layout allows */
  int64_t bias_row_group;  /* XB_BIAS_FULL only: rows of Y that share one bias row (output row m reads bias
                              row m / bias_row_group); 0 or 1 = one bias row per output row. This is the
                              broadcast add of PrunedGemmOp (blaze/blaze/operator/op/pruned_gemm_op.h:106-152:
                              the one-row partial product added to every row), applied per group of rows so
                              that several requests share a launch. */
} xb_gemm_args;

int xb_gemm(const xb_gemm_args* args, xb_stream_t stream);
/* 1 when XB_GEMM_AUTO would run these arguments on the tcgen05 engine. */
int xb_gemm_uses_tcgen05(const xb_gemm_args* args);

/* Pack a row-major [K,N] weight into the K-major [N, ldk] layout (ldk >= K,
 * multiple of 8, zero padded) the tcgen05 engine reads, with dtype conversion.
 * Done once when constants are loaded (blaze/blaze/operator/op/constant_fill_op.h:20-37). */
int xb_pack_weight_kmajor(const void* W, int32_t w_dtype, int32_t K, int32_t N, int64_t ldw,
                          void* out, int32_t out_dtype, int64_t ldk, int32_t batch,
                          int64_t stride_w, int64_t stride_out, xb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Fused DIN attention unit.
 * Replaces rows 7-16 of the shipped DIN graph
 * (blaze/tools/example_model/din/model/graph_ulf.txt: Sub, Mul, BroadcastTo x2,
 * Concat, Gemm x3 with activations, Where, Softmax, MatMul) - operators
 * blaze/blaze/operator/op/elementwise_op.h:63-307, concat_op.h:34-131,
 * gemm_op.h:33-107, softmax_op.cc:21-78, matmul_op.h:31-144.
 * For request r: q[r] [n_cand, d], k[r] [T, d];
 *   x = [q, k, q-k, q*k] (4d), s = W2'act(W1'act(W0'x+b0)+b1)+b2,
 *   out[n] = sum_t s[n,t] * k[t]     (optionally masked softmax over t first).
 * The 4d-wide concat is built in shared memory and never written to HBM. */
enum { XB_ACT_NONE = 0, XB_ACT_SIGMOID = 1, XB_ACT_DICE = 2 };
/* `engine` of xb_din_att_args takes XB_GEMM_AUTO / XB_GEMM_SIMT / XB_GEMM_TCGEN05 or this value: the tcgen05
 * engine that regroups layer 1 as q x (Wq + Wd + diag(k_t) Wp) and runs two steps per MMA (needs `packed`). */
enum { XB_ATT_ENGINE_PAIR = 3,
       /* the tcgen05 engine that splits layer 1 into (Wq + Wd) q + Wp (q * k_t) + [(Wk - Wd) k_t + b0], the last
        * term once per request: half the MMAs per step, persistent CTAs. XB_GEMM_AUTO picks it when `packed` is
        * given and the shape fits; XB_GEMM_TCGEN05 keeps the per-step engine. */
       XB_ATT_ENGINE_SPLIT = 4 };

typedef struct xb_din_att_weights {
  /* K-major packed fp16 weights: W0 [h0, 4d], W1 [h1, h0]; W2 fp32 [h1] */
  const void* W0; const void* W1; const float* W2;
  const float *b0, *b1;  float b2;
  const float *gamma0, *mean0, *var0;   /* Dice, [h0] */
  const float *gamma1, *mean1, *var1;   /* Dice, [h1] */
  const void* packed;                   /* optional: output of xb_din_attention_pack for these weights and
                                           `act`; saves re-laying the operands out in every CTA */
} xb_din_att_weights;

typedef struct xb_din_att_args {
  const void* q;  int64_t ldq;          /* fp16 [requests*n_cand, d] */
  const void* k;  int64_t ldk;          /* fp16 [requests*T, d] */
  const int32_t* seq_len;               /* [requests] valid steps, NULL = T */
  void* out; int64_t ldo;               /* fp16 [requests*n_cand, d] */
  float* scores;                        /* optional fp32 [requests*n_cand, T], NULL to skip */
  int32_t requests, n_cand, T, d, h0, h1;
  int32_t act;                          /* XB_ACT_* */
  int32_t use_softmax;                  /* masked softmax over t (shipped graph) */
  int32_t engine;                       /* XB_GEMM_AUTO / _SIMT / _TCGEN05 */
  xb_din_att_weights w;
} xb_din_att_args;

int xb_din_attention(const xb_din_att_args* args, xb_stream_t stream);
/* Lays the weights of `args` (d, h0, h1, act, w.*) out once in the form the tcgen05 engine keeps in
 * shared memory. xb_din_attention_packed_bytes returns 0 for shapes that engine does not take. */
size_t xb_din_attention_packed_bytes(int32_t d, int32_t h0, int32_t h1);
int xb_din_attention_pack(const xb_din_att_args* args, void* packed, size_t bytes, xb_stream_t stream);

/* Fused assembly of the DIN tower input. Replaces rows 17-22 of the shipped DIN
 * graph (ReduceSum over the behaviour rows, Mul, Concat, Fuse x2:
 * blaze/blaze/operator/op/reduce_sum_op.h:17-86, elementwise_op.h:63-307,
 * concat_op.h:34-131, fuse_op.h:28-83). For request r and candidate n:
 *   X[r*n_cand+n] = [user[r] (du) | q | his_sum[r] | q*his_sum[r] | att | q-his_sum[r] | 0...]
 * with his_sum[r] = sum_t k[r,t]; columns [du+5d, ldx) are zero-filled so X can
 * feed the tcgen05 GEMM engine (ldx a multiple of 8). All tensors fp16. */
int xb_din_tower_input(const void* user, int64_t ldu, const void* q, int64_t ldq, const void* k,
                       int64_t ldk, const void* att, int64_t ldatt, void* X, int64_t ldx,
                       int32_t requests, int32_t n_cand, int32_t T, int32_t d, int32_t du,
                       xb_stream_t stream);
/* The same features split the way PrunedGemmOp wants its two operands
 * (blaze/blaze/operator/op/pruned_gemm_op.h:1-10: [A|B] x [C;D] = A x C + B x D): the columns that are
 * equal for every candidate of a request go once per request into
 *   Xu[r]           = [user[r] (du) | his_sum[r] (d) | 0...]            [requests, ldxu]
 * and the per-candidate columns into
 *   Xc[r*n_cand+n]  = [q | q*his_sum[r] | att | q-his_sum[r] | 0...]    [requests*n_cand, ldxc]. */
int xb_din_tower_input_split(const void* user, int64_t ldu, const void* q, int64_t ldq, const void* k,
                             int64_t ldk, const void* att, int64_t ldatt, void* Xu, int64_t ldxu, void* Xc,
                             int64_t ldxc, int32_t requests, int32_t n_cand, int32_t T, int32_t d, int32_t du,
                             xb_stream_t stream);

/* Fused DIN tower: the assembly above, the tower MLP du+5d -> n1 -> n2 -> n3 with Dice after the first
 * two layers, and the final softmax, in one tcgen05 kernel (plus a small per-request kernel). Replaces
 * rows 17-29 of the shipped DIN graph: the Concat / Fuse rows above, three Gemm rows with bias
 * (blaze/blaze/operator/op/gemm_op.h:33-107), two Dice rows (dice_op.cu:11-21) and Softmax
 * (softmax_op.cc:21-78). The first layer is computed as PrunedGemmOp does
 * (blaze/blaze/operator/op/pruned_gemm_op.h:1-163): the [user | his_sum] columns once per request.
 * Weights are the model's fp16 constants in Blaze's [K, N] layout; biases and Dice parameters fp32.
 * prob [requests*n_cand, n3] fp32: softmax over n3 (softmax != 0) or the fp16-rounded logits. */
typedef struct xb_din_tower_args {
  const void* user; int64_t ldu;        /* [requests, du] fp16 */
  const void* q; int64_t ldq;           /* [requests*n_cand, d] fp16 */
  const void* k; int64_t ldk;           /* [requests*T, d] fp16 */
  const void* att; int64_t ldatt;       /* [requests*n_cand, d] fp16 */
  float* prob;
  int32_t requests, n_cand, T, d, du, n1, n2, n3;
  const void* W1; const float* b1; const float* gamma1; const float* mean1; const float* var1;   /* [du+5d, n1] */
  const void* W2; const float* b2; const float* gamma2; const float* mean2; const float* var2;   /* [n1, n2] */
  const void* W3; const float* b3;                                                              /* [n2, n3] */
  int32_t softmax;
  const void* packed;                   /* image written by xb_din_tower_pack */
} xb_din_tower_args;

/* 0 for shapes the kernel does not take (d <= 64, n1 <= 256, n2 <= 128, n3 <= 8). */
size_t xb_din_tower_packed_bytes(int32_t d, int32_t n1, int32_t n2, int32_t n3);
/* Lays the weights out once in the form the kernel keeps in shared memory (needs d, du, n1..n3, W*, b2, b3,
 * gamma*, mean*, var*). */
int xb_din_tower_pack(const xb_din_tower_args* args, void* packed, size_t bytes, xb_stream_t stream);
/* Per-launch scratch: his_sum [requests, d] and the per-request product [requests, n1], fp32. */
size_t xb_din_tower_workspace_bytes(int32_t requests, int32_t d, int32_t n1);
int xb_din_tower(const xb_din_tower_args* args, void* workspace, size_t workspace_bytes, xb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Recurrent layers of the DIEN-style model. x, y [batch, T, H] in `dtype` (XB_F32 or
 * XB_F16); weights and biases in the same dtype; H <= 64.
 * xb_gru replaces GRUOp (blaze/blaze/operator/op/gru_op.h:41-158, CPU kernel
 * gru_op.cc:33-93, CUDA kernels gru_op.cu): i2h, h2h [H, 3H] with gate order
 * (r, z, candidate), h' = c + z (h - c); leading steps whose first H input
 * pre-activations are all zero emit zeros.
 * xb_augru has no operator in Blaze; it follows the training-side cell
 * (xdl-algorithm-solution/DIEN/script/utils.py:139-207): Wg [2H, 2H], Wc [2H, H],
 * att [batch, T] attention scores, u' = (1 - att) u, h' = u' h + (1 - u') c. */
int xb_gru(const void* x, void* y, int64_t batch, int32_t T, int32_t H, const void* i2h, const void* h2h,
           const void* i2h_bias, const void* h2h_bias, int32_t dtype, xb_stream_t stream);
int xb_augru(const void* x, const void* att, void* y, int64_t batch, int32_t T, int32_t H, const void* Wg,
             const void* bg, const void* Wc, const void* bc, int32_t dtype, xb_stream_t stream);
/* The AUGRU as the DIEN-style model uses it: every candidate of a request walks the request's own sequence
 * x [requests, T, H] with its own scores att [requests * n_cand, T], and only the final state
 * y_final [requests * n_cand, H] is kept. All tensors fp16. `engine`: XB_GEMM_AUTO / _SIMT / _TCGEN05; the tcgen05
 * engine (one CTA per 128 candidates, both per-candidate products as MMAs with the state in tensor memory, the
 * request-side terms x_t Wg_x + bg and x_t Wc_x + bc computed once per request) takes an even H <= 64 whose padding
 * to a multiple of 8 leaves at least 4 slots (H = 36 does). Same cell as xb_augru. */
int xb_augru_shared(const void* x, const void* att, void* y_final, int32_t requests, int32_t n_cand, int32_t T, int32_t H,
                    const void* Wg, const void* bg, const void* Wc, const void* bc, int32_t engine, xb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Stand-alone operators for graphs that were not fused. x/y share `dtype`;
 * per-column parameters share it too (Blaze keeps them in the model dtype). */
/* DiceOp, blaze/blaze/operator/op/dice_op.h:41-98 */
int xb_dice(const void* x, void* y, int64_t rows, int32_t c, const void* gamma, const void* mean,
            const void* var, int32_t nosqrt, int32_t dtype, xb_stream_t stream);
/* PReluOp, blaze/blaze/operator/op/prelu_op.h:25-64 */
int xb_prelu(const void* x, void* y, int64_t size, const void* w, int64_t inner, int32_t dtype,
             int32_t w_dtype, xb_stream_t stream);
/* SigmoidOp, blaze/blaze/operator/op/sigmoid_op.cu:11-17 */
int xb_sigmoid(const void* x, void* y, int64_t size, int32_t dtype, xb_stream_t stream);
/* SoftmaxOp, blaze/blaze/operator/op/softmax_op.cu:25-67: softmax over c with outer n, inner w */
int xb_softmax(const void* x, void* y, int64_t n, int32_t c, int64_t w, int32_t dtype, xb_stream_t stream);
/* BatchNormalizationOp (inference), blaze/blaze/operator/op/batch_normalization_op.cu:12 */
int xb_batchnorm(const void* x, void* y, int64_t size, int32_t c, const void* gamma, const void* beta,
                 const void* mean, const void* var, float eps, int32_t nosqrt, int32_t dtype,
                 xb_stream_t stream);
/* Elementwise with numpy broadcasting over <= 4 dims,
 * blaze/blaze/operator/op/elementwise_op.h:63-307. `where`: a is int32 condition. */
enum { XB_EW_ADD = 0, XB_EW_SUB, XB_EW_MUL, XB_EW_DIV, XB_EW_MAX, XB_EW_MIN, XB_EW_EQ, XB_EW_NE,
       XB_EW_BROADCAST_TO, XB_EW_WHERE };
int xb_elementwise(int32_t op, const void* a, const int64_t* a_strides, const void* b,
                   const int64_t* b_strides, const void* c, const int64_t* c_strides, void* y,
                   const int64_t* y_shape /* 4 dims */, int32_t dtype, xb_stream_t stream);
/* Strided 2-D copy with dtype conversion: Concat / Slice / Split / Fuse /
 * FusedSliceConcat are expressed as one or more of these
 * (blaze/blaze/operator/op/concat_op.cu:32-43, slice_op.cu:10, fuse_op.cu:10-18,
 * fused_op/fused_slice_concat_op.cu:24-140). src row stride 0 broadcasts one row. */
int xb_copy2d(const void* src, int64_t src_ld, int32_t src_dtype, void* dst, int64_t dst_ld,
              int32_t dst_dtype, int64_t rows, int64_t cols, xb_stream_t stream);
/* Many flat device-to-device copies in one launch: the merge and split steps of request batching
 * (Batching::CopyDataToMergedNet, blaze/blaze/scheduler/batching.cc:117-129, issues one cudaMemcpyAsync per input
 * blob and request; stacking 32 requests of a 39-input net is 1248 of them). `items` is a DEVICE array of n_items
 * descriptors (the caller copies it there, e.g. from pinned memory on the same stream); max_bytes is the largest
 * `bytes` among them (it sizes the grid). Source and destination ranges must not overlap. */
typedef struct xb_copy_item {
  const void* src;
  void* dst;
  int64_t bytes;
} xb_copy_item;
int xb_copy_segments(const xb_copy_item* items, int32_t n_items, int64_t max_bytes, xb_stream_t stream);
/* ReduceSum over the middle axis of [outer, r, inner], blaze/blaze/math/reduce.cu:12-113 */
int xb_reduce_sum(const void* x, void* y, int64_t outer, int64_t r, int64_t inner, int32_t dtype,
                  xb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* XDLB200_H_ */
