// Row-sharded embedding pooling as one call: the whole step of the large-table configuration (route ->
// id exchange -> owner pooling -> partial-sum exchange -> combine) behind the C ABI, with NCCL called from
// here. Nothing in a step synchronises with the host:
//   * ids travel in fixed-capacity buckets (one per destination, slot 0 = record count), so the all-to-all
//     is an equal split whose sizes the host knows without reading the bucket sizes back; a bucket that
//     would overflow raises a flag the caller checks after its own stream synchronisation;
//   * every buffer is allocated once, when the context is created.
// NCCL is bound at run time (dlopen of libnccl.so.2): a process that never shards tables does not need it,
// and inside a PyTorch process the already loaded NCCL is the one that gets used.
//
// The reference has no multi-device path (Blaze is single-process, blaze/blaze/api/cpp_api/
// predictor_manager_impl.cc:142-177); the plug-in point is its SparsePuller interface
// (blaze/blaze/store/sparse_puller.h:77-105), which the host runtime's sharded puller implements on this.
#include <dlfcn.h>

#include <algorithm>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "xb_common.cuh"

namespace xb {
namespace {

// ---- NCCL, bound at run time -----------------------------------------------------------------------------
typedef struct ncclComm* ncclComm_t;
struct NcclUniqueId { char internal[128]; };
enum { kNcclSuccess = 0, kNcclInProgress = 7, kNcclInt8 = 0 };

struct NcclApi {
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*Send)(const void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*Recv)(void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  bool ok = false;
  std::string why;
  NcclApi() {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) { why = std::string("libnccl.so.2 could not be loaded: ") + dlerror(); return; }
    bool all = true;
    auto bind = [&](const char* name, void** fn) { *fn = dlsym(h, name); all = all && *fn != nullptr; };
    bind("ncclGetUniqueId", (void**)&GetUniqueId);
    bind("ncclCommInitRank", (void**)&CommInitRank);
    bind("ncclCommDestroy", (void**)&CommDestroy);
    bind("ncclGroupStart", (void**)&GroupStart);
    bind("ncclGroupEnd", (void**)&GroupEnd);
    bind("ncclSend", (void**)&Send);
    bind("ncclRecv", (void**)&Recv);
    bind("ncclCommGetAsyncError", (void**)&CommGetAsyncError);
    bind("ncclGetErrorString", (void**)&GetErrorString);
    ok = all;
    if (!ok) why = "libnccl.so.2 lacks an entry point this library needs";
  }
};
NcclApi& nccl() {
  static NcclApi api;
  return api;
}

#define XB_NCCL(call)                                                                                \
  do {                                                                                               \
    int r__ = (call);                                                                                \
    if (r__ != kNcclSuccess) return fail(XB_ERR_CUDA, "%s failed: %s", #call, nccl().GetErrorString(r__)); \
  } while (0)

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace
}  // namespace xb

using namespace xb;

struct xb_shard_ctx {
  int rank = 0, world = 1, dim = 0, n_tables = 0, partial_dtype = XB_F32, device = 0;
  std::vector<const xb_table_desc*> tables;
  std::vector<int64_t> table_segments;
  int64_t S = 0;              // segments of one rank, all tables
  int64_t max_ids = 0, cap = 0;
  ncclComm_t comm = nullptr;
  // device buffers, allocated once
  char* arena = nullptr;
  size_t arena_bytes = 0;
  int64_t *send = nullptr, *recv = nullptr;         // [world * cap] packed records: the slot in use
  int64_t *send2[2] = {nullptr, nullptr}, *recv2[2] = {nullptr, nullptr};   // two slots: a begun step and the one before it
  int64_t slot_ids[2] = {0, 0};                     // ids of the step each slot holds
  cudaEvent_t slot_ready[2] = {nullptr, nullptr};   // recorded when a slot's id exchange has been enqueued
  cudaEvent_t slot_free[2] = {nullptr, nullptr};    // recorded when the pooling that reads a slot has been enqueued
  int begun = 0, finished = 0;                      // steps begun / finished so far (begun - finished <= 2)
  int32_t *counts = nullptr, *offsets = nullptr;    // [world * S], [world * (S + 1)]
  char *partial = nullptr, *back = nullptr;         // [world * S * dim] partial sums (partial_dtype): the slot in use
  char *partial2[2] = {nullptr, nullptr}, *back2[2] = {nullptr, nullptr};   // two slots: a pooled step and the one before it
  cudaEvent_t back_ready[2] = {nullptr, nullptr};   // recorded when a slot's partial-sum exchange has been enqueued
  cudaEvent_t back_free[2] = {nullptr, nullptr};    // recorded when the combine that reads a slot has been enqueued
  int pooled = 0;                                   // steps whose middle part has been enqueued (finished counts combines)
  void* route_scratch = nullptr; size_t route_scratch_bytes = 0;
  void* scan_scratch = nullptr; size_t scan_scratch_bytes = 0;
  int32_t* overflow_dev = nullptr;                  // device view of the mapped flag
  volatile int32_t* overflow_host = nullptr;
  // optional phase timing: events recorded at the phase boundaries of the last xb_sharded_pool call
  bool profile = false;
  cudaEvent_t ev[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
};

static inline void mark(xb_shard_ctx* c, int i, cudaStream_t stream) {
  if (c->profile) cudaEventRecord(c->ev[i], stream);
}

extern "C" int xb_shard_unique_id(void* id128) {
  XB_REQUIRE(id128, XB_ERR_ARG, "xb_shard_unique_id: null pointer");
  XB_REQUIRE(nccl().ok, XB_ERR_UNSUPPORTED, "xb_shard_unique_id: %s", nccl().why.c_str());
  NcclUniqueId id;
  XB_NCCL(nccl().GetUniqueId(&id));
  memcpy(id128, &id, sizeof(id));
  return 0;
}

extern "C" void xb_shard_ctx_destroy(xb_shard_ctx* c) {
  if (!c) return;
  if (c->comm) nccl().CommDestroy(c->comm);
  if (c->arena) cudaFree(c->arena);
  if (c->overflow_host) cudaFreeHost((void*)c->overflow_host);
  for (cudaEvent_t e : c->ev)
    if (e) cudaEventDestroy(e);
  for (cudaEvent_t e : c->slot_ready)
    if (e) cudaEventDestroy(e);
  for (cudaEvent_t e : c->slot_free)
    if (e) cudaEventDestroy(e);
  for (cudaEvent_t e : c->back_ready)
    if (e) cudaEventDestroy(e);
  for (cudaEvent_t e : c->back_free)
    if (e) cudaEventDestroy(e);
  delete c;
}

extern "C" int64_t xb_shard_bucket_capacity(int64_t max_ids, int32_t world, float capacity_factor) {
  if (max_ids < 0 || world < 1) return 0;
  const double f = capacity_factor > 1.f ? capacity_factor : 1.f;
  const int64_t mean = (max_ids + world - 1) / world;
  int64_t cap = (int64_t)(mean * f) + 1 + 64;                  // + the header slot + slack for tiny inputs
  return (cap + 511) / 512 * 512;
}

extern "C" int xb_shard_ctx_create(xb_shard_ctx** out, const void* unique_id128, const xb_shard_config* cfg) {
  XB_REQUIRE(out && cfg, XB_ERR_ARG, "xb_shard_ctx_create: null argument");
  XB_REQUIRE(cfg->world >= 1 && cfg->world <= 16 && cfg->rank >= 0 && cfg->rank < cfg->world, XB_ERR_ARG,
             "xb_shard_ctx_create: rank %d of %d (at most 16 shards)", cfg->rank, cfg->world);
  XB_REQUIRE(cfg->n_tables >= 1 && cfg->tables && cfg->table_segments && cfg->dim >= 1 && cfg->max_ids >= 0, XB_ERR_ARG,
             "xb_shard_ctx_create: bad table list");
  XB_REQUIRE(cfg->partial_dtype == XB_F32 || cfg->partial_dtype == XB_F16, XB_ERR_UNSUPPORTED,
             "xb_shard_ctx_create: partial dtype %d", cfg->partial_dtype);
  XB_REQUIRE(cfg->world == 1 || unique_id128, XB_ERR_ARG, "xb_shard_ctx_create: a communicator id is needed for %d ranks", cfg->world);
  std::unique_ptr<xb_shard_ctx, void (*)(xb_shard_ctx*)> c(new xb_shard_ctx(), xb_shard_ctx_destroy);
  c->rank = cfg->rank; c->world = cfg->world; c->dim = cfg->dim; c->n_tables = cfg->n_tables;
  c->partial_dtype = cfg->partial_dtype; c->max_ids = cfg->max_ids;
  XB_CUDA(cudaGetDevice(&c->device));
  for (int t = 0; t < cfg->n_tables; ++t) {
    XB_REQUIRE(cfg->tables[t] && cfg->table_segments[t] >= 0, XB_ERR_ARG, "xb_shard_ctx_create: table %d", t);
    XB_REQUIRE(cfg->tables[t]->dim == cfg->dim && cfg->tables[t]->slot_keys == nullptr, XB_ERR_ARG,
               "xb_shard_ctx_create: table %d must have dim %d and identity keys (local rows)", t, cfg->dim);
    XB_REQUIRE(cfg->tables[t]->rows < ((int64_t)1 << 31) - 1, XB_ERR_LIMIT, "xb_shard_ctx_create: shard %d has too many rows", t);
    c->tables.push_back(cfg->tables[t]);
    c->table_segments.push_back(cfg->table_segments[t]);
    c->S += cfg->table_segments[t];
  }
  XB_REQUIRE(c->S < ((int64_t)1 << 31) / cfg->world, XB_ERR_LIMIT, "xb_shard_ctx_create: too many segments");
  c->cap = xb_shard_bucket_capacity(cfg->max_ids, cfg->world, cfg->capacity_factor);
  XB_REQUIRE(c->cap * cfg->world < ((int64_t)1 << 31), XB_ERR_LIMIT, "xb_shard_ctx_create: too many ids per step");
  const int W = c->world;
  const size_t esz = c->partial_dtype == XB_F32 ? 4 : 2;
  c->route_scratch_bytes = xb_route_scratch_bytes(c->max_ids, W);
  const int groups_per_scan = std::min(W, XB_MAX_POOL_GROUPS);
  c->scan_scratch_bytes = xb_scan_counts_scratch_bytes(groups_per_scan, c->S);
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t at = off; off += align256(bytes); return at; };
  const size_t o_send = take((size_t)W * c->cap * 8), o_recv = take((size_t)W * c->cap * 8);
  const size_t o_send1 = take((size_t)W * c->cap * 8), o_recv1 = take((size_t)W * c->cap * 8);
  const size_t o_counts = take((size_t)W * c->S * 4), o_offsets = take((size_t)W * (c->S + 1) * 4);
  const size_t o_partial = take((size_t)W * c->S * c->dim * esz), o_back = take((size_t)W * c->S * c->dim * esz);
  const size_t o_partial1 = take((size_t)W * c->S * c->dim * esz), o_back1 = take((size_t)W * c->S * c->dim * esz);
  const size_t o_route = take(c->route_scratch_bytes), o_scan = take(c->scan_scratch_bytes);
  c->arena_bytes = off;
  XB_CUDA(cudaMalloc(reinterpret_cast<void**>(&c->arena), c->arena_bytes));
  c->send2[0] = reinterpret_cast<int64_t*>(c->arena + o_send); c->recv2[0] = reinterpret_cast<int64_t*>(c->arena + o_recv);
  c->send2[1] = reinterpret_cast<int64_t*>(c->arena + o_send1); c->recv2[1] = reinterpret_cast<int64_t*>(c->arena + o_recv1);
  c->send = c->send2[0]; c->recv = c->recv2[0];
  for (cudaEvent_t& e : c->slot_ready) XB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  for (cudaEvent_t& e : c->slot_free) XB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  c->counts = reinterpret_cast<int32_t*>(c->arena + o_counts); c->offsets = reinterpret_cast<int32_t*>(c->arena + o_offsets);
  c->partial2[0] = c->arena + o_partial; c->back2[0] = c->arena + o_back;
  c->partial2[1] = c->arena + o_partial1; c->back2[1] = c->arena + o_back1;
  c->partial = c->partial2[0]; c->back = c->back2[0];
  for (cudaEvent_t& e : c->back_ready) XB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  for (cudaEvent_t& e : c->back_free) XB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  c->route_scratch = c->arena + o_route; c->scan_scratch = c->arena + o_scan;
  int32_t* flag = nullptr;
  XB_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&flag), 64, cudaHostAllocMapped | cudaHostAllocPortable));
  *flag = 0;
  c->overflow_host = flag;
  XB_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&c->overflow_dev), flag, 0));
  if (W > 1) {
    XB_REQUIRE(nccl().ok, XB_ERR_UNSUPPORTED, "xb_shard_ctx_create: %s", nccl().why.c_str());
    NcclUniqueId id;
    memcpy(&id, unique_id128, sizeof(id));
    XB_NCCL(nccl().CommInitRank(&c->comm, W, id, c->rank));
  }
  *out = c.release();
  return 0;
}

// slice w of `send` goes to rank w, slice w of `recv` comes from rank w; `bytes` per slice
static int all_to_all_equal(xb_shard_ctx* c, const void* send, void* recv, size_t bytes, cudaStream_t stream) {
  if (c->world == 1) {
    XB_CUDA(cudaMemcpyAsync(recv, send, bytes, cudaMemcpyDeviceToDevice, stream));
    return 0;
  }
  XB_NCCL(nccl().GroupStart());
  for (int w = 0; w < c->world; ++w) {
    XB_NCCL(nccl().Send(static_cast<const char*>(send) + (size_t)w * bytes, bytes, kNcclInt8, w, c->comm, stream));
    XB_NCCL(nccl().Recv(static_cast<char*>(recv) + (size_t)w * bytes, bytes, kNcclInt8, w, c->comm, stream));
  }
  XB_NCCL(nccl().GroupEnd());
  return 0;
}

extern "C" int xb_a2a_route(xb_shard_ctx* c, const int64_t* ids, const int32_t* seg_offsets, int64_t n_ids, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(c && seg_offsets && n_ids >= 0 && (n_ids == 0 || ids), XB_ERR_ARG, "xb_a2a_route: bad arguments");
  XB_REQUIRE(n_ids <= c->max_ids, XB_ERR_LIMIT, "xb_a2a_route: %lld ids, the context was sized for %lld", (long long)n_ids,
             (long long)c->max_ids);
  mark(c, 0, stream);
  if (int rc = xb_route_ids_padded(ids, seg_offsets, c->S, n_ids, c->world, c->cap, c->send, c->overflow_dev, c->route_scratch,
                                   c->route_scratch_bytes, stream)) return rc;
  mark(c, 1, stream);
  return all_to_all_equal(c, c->send, c->recv, (size_t)c->cap * 8, stream);
}

extern "C" int xb_a2a_return(xb_shard_ctx* c, xb_stream_t stream_) {
  XB_REQUIRE(c, XB_ERR_ARG, "xb_a2a_return: null context");
  const size_t esz = c->partial_dtype == XB_F32 ? 4 : 2;
  return all_to_all_equal(c, c->partial, c->back, (size_t)c->S * c->dim * esz, (cudaStream_t)stream_);
}

// First half of a step: bucket the ids by owner and exchange the buckets. Two steps may be begun before the first is
// finished (two sets of exchange buffers), so a caller can overlap the id exchange of step i+1 with the pooling of
// step i: begin(i+1) on one stream, finish(i) on another, always in that order on every rank (the exchanges of one
// communicator run in the order they were issued). All begin calls go to one stream, all finish calls to one stream.
// `ids` and `seg_offsets` must stay valid until the work enqueued here has run.
extern "C" int xb_sharded_pool_begin(xb_shard_ctx* c, const int64_t* ids, const int32_t* seg_offsets, int64_t n_ids,
                                     xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(c, XB_ERR_ARG, "xb_sharded_pool_begin: null context");
  int dev = -1;
  XB_CUDA(cudaGetDevice(&dev));
  XB_REQUIRE(dev == c->device, XB_ERR_ARG, "xb_sharded_pool_begin: the context belongs to device %d, current device is %d", c->device, dev);
  XB_REQUIRE(c->begun - c->pooled < 2, XB_ERR_ARG, "xb_sharded_pool_begin: two steps are already in flight; finish one first");
  const int slot = c->begun & 1;
  c->send = c->send2[slot]; c->recv = c->recv2[slot];
  // the step that used this slot two begins ago has been finished (checked above): its pooling, which reads the
  // slot's receive buffer, may still be running on another stream
  if (c->begun >= 2) XB_CUDA(cudaStreamWaitEvent(stream, c->slot_free[slot], 0));
  if (int rc = xb_a2a_route(c, ids, seg_offsets, n_ids, stream)) return rc;      // 1. bucket + exchange
  XB_CUDA(cudaEventRecord(c->slot_ready[slot], stream));
  c->slot_ids[slot] = n_ids;
  ++c->begun;
  return 0;
}

// Middle part of the oldest begun step, on `stream` (which is made to wait for that step's id exchange): segment
// lengths and offsets per source, owner pooling, exchange of the partial sums. Two steps may be pooled before the
// first is combined (two sets of partial-sum buffers). All calls of this function go to one stream.
extern "C" int xb_sharded_pool_pool(xb_shard_ctx* c, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(c, XB_ERR_ARG, "xb_sharded_pool_pool: null context");
  XB_REQUIRE(c->begun > c->pooled, XB_ERR_ARG, "xb_sharded_pool_pool: no step has been begun");
  XB_REQUIRE(c->pooled - c->finished < 2, XB_ERR_ARG, "xb_sharded_pool_pool: two pooled steps are waiting for their combine");
  const int W = c->world;
  const int slot = c->pooled & 1;
  const int64_t* recv = c->recv2[slot];
  const int64_t n_ids = c->slot_ids[slot];
  c->partial = c->partial2[slot]; c->back = c->back2[slot];
  XB_CUDA(cudaStreamWaitEvent(stream, c->slot_ready[slot], 0));
  // the combine that read this slot's partial sums two steps ago may still be running on another stream
  if (c->pooled >= 2) XB_CUDA(cudaStreamWaitEvent(stream, c->back_free[slot], 0));
  mark(c, 2, stream);
  // 2. at the owner: segment lengths per source from the received records, offsets per source
  if (int rc = xb_record_counts_padded(recv, W, c->cap, c->counts, c->S, stream)) return rc;
  for (int s0 = 0; s0 < W; s0 += XB_MAX_POOL_GROUPS) {
    const int n = std::min(W - s0, (int)XB_MAX_POOL_GROUPS);
    if (int rc = xb_scan_counts(c->counts + (int64_t)s0 * c->S, c->S, c->offsets + (int64_t)s0 * (c->S + 1), c->S + 1, n, c->S,
                                c->scan_scratch, c->scan_scratch_bytes, stream)) return rc;
  }
  mark(c, 3, stream);
  // 3. pool every (source, table) segment range against that table's shard
  if (int rc = xb_shard_pool_records(c->tables.data(), c->table_segments.data(), c->n_tables, recv, c->cap, c->offsets, W,
                                     n_ids, c->dim, c->partial, c->partial_dtype, stream)) return rc;
  XB_CUDA(cudaEventRecord(c->slot_free[slot], stream));
  mark(c, 4, stream);
  // 4. partial sums back to the sources
  if (int rc = xb_a2a_return(c, stream)) return rc;
  XB_CUDA(cudaEventRecord(c->back_ready[slot], stream));
  mark(c, 5, stream);
  ++c->pooled;
  return 0;
}

// Last part of the oldest pooled step, on `stream` (which is made to wait for that step's partial-sum exchange):
// the owner-ordered combine into `out`.
extern "C" int xb_sharded_pool_combine(xb_shard_ctx* c, int64_t groups, int32_t avg, void* out, int64_t out_stride,
                                       int32_t out_dtype, xb_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  XB_REQUIRE(c && out && groups >= 1 && c->S % groups == 0, XB_ERR_ARG, "xb_sharded_pool_combine: bad arguments");
  XB_REQUIRE(c->pooled > c->finished, XB_ERR_ARG, "xb_sharded_pool_combine: no pooled step is waiting");
  XB_REQUIRE(!avg, XB_ERR_UNSUPPORTED, "xb_sharded_pool: average pooling needs the segment lengths; use kSum and scale");
  const int slot = c->finished & 1;
  XB_CUDA(cudaStreamWaitEvent(stream, c->back_ready[slot], 0));
  // 5. owner-ordered combine
  const int rc = xb_shard_combine(c->back2[slot], c->partial_dtype, c->world, c->S, c->dim, nullptr, 0, out, out_stride, groups,
                                  out_dtype, stream);
  XB_CUDA(cudaEventRecord(c->back_free[slot], stream));
  mark(c, 6, stream);
  ++c->finished;
  return rc;
}

// Middle and last part of the oldest begun step on one stream.
extern "C" int xb_sharded_pool_finish(xb_shard_ctx* c, int64_t groups, int32_t avg, void* out, int64_t out_stride,
                                      int32_t out_dtype, xb_stream_t stream) {
  XB_REQUIRE(c && out && groups >= 1 && c->S % groups == 0, XB_ERR_ARG, "xb_sharded_pool_finish: bad arguments");
  XB_REQUIRE(c->begun > c->finished, XB_ERR_ARG, "xb_sharded_pool_finish: no step has been begun");
  XB_REQUIRE(!avg, XB_ERR_UNSUPPORTED, "xb_sharded_pool: average pooling needs the segment lengths; use kSum and scale");
  if (c->pooled == c->finished)
    if (int rc = xb_sharded_pool_pool(c, stream)) return rc;
  return xb_sharded_pool_combine(c, groups, avg, out, out_stride, out_dtype, stream);
}

// The whole step on one stream.
extern "C" int xb_sharded_pool(xb_shard_ctx* c, const int64_t* ids, const int32_t* seg_offsets, int64_t n_ids, int64_t groups,
                               int32_t avg, void* out, int64_t out_stride, int32_t out_dtype, xb_stream_t stream) {
  XB_REQUIRE(c && out && groups >= 1 && c->S % groups == 0, XB_ERR_ARG, "xb_sharded_pool: bad arguments");
  XB_REQUIRE(!avg, XB_ERR_UNSUPPORTED, "xb_sharded_pool: average pooling needs the segment lengths; use kSum and scale");
  XB_REQUIRE(c->begun == c->finished, XB_ERR_ARG, "xb_sharded_pool: a step begun with xb_sharded_pool_begin is still open");
  if (int rc = xb_sharded_pool_begin(c, ids, seg_offsets, n_ids, stream)) return rc;
  return xb_sharded_pool_finish(c, groups, avg, out, out_stride, out_dtype, stream);
}

// Phase timing of xb_sharded_pool: off by default (seven event records per call when on).
extern "C" int xb_shard_ctx_profile(xb_shard_ctx* c, int32_t enable) {
  XB_REQUIRE(c, XB_ERR_ARG, "xb_shard_ctx_profile: null context");
  if (enable)
    for (cudaEvent_t& e : c->ev)
      if (!e) XB_CUDA(cudaEventCreate(&e));
  c->profile = enable != 0;
  return 0;
}

// Milliseconds of the six phases of the last profiled call, after the caller has synchronised its stream:
// bucket ids by owner, exchange ids, segment lengths + offsets, pool, exchange partial sums, combine.
extern "C" int xb_shard_ctx_phase_ms(xb_shard_ctx* c, float* ms6) {
  XB_REQUIRE(c && ms6 && c->profile, XB_ERR_ARG, "xb_shard_ctx_phase_ms: profiling is off");
  for (int i = 0; i < 6; ++i) XB_CUDA(cudaEventElapsedTime(&ms6[i], c->ev[i], c->ev[i + 1]));
  return 0;
}

extern "C" int xb_shard_ctx_status(xb_shard_ctx* c, int32_t* overflow) {
  XB_REQUIRE(c && overflow, XB_ERR_ARG, "xb_shard_ctx_status: null argument");
  *overflow = *c->overflow_host;
  if (*overflow) *c->overflow_host = 0;
  if (c->comm) {
    int async_err = kNcclSuccess;
    XB_NCCL(nccl().CommGetAsyncError(c->comm, &async_err));
    XB_REQUIRE(async_err == kNcclSuccess || async_err == kNcclInProgress, XB_ERR_CUDA, "xb_shard_ctx_status: NCCL reports %s",
               nccl().GetErrorString(async_err));
  }
  return 0;
}

extern "C" int64_t xb_shard_ctx_bucket_capacity(const xb_shard_ctx* c) { return c ? c->cap : 0; }
extern "C" size_t xb_shard_ctx_device_bytes(const xb_shard_ctx* c) { return c ? c->arena_bytes : 0; }
