// Sparse pullers of the B200 runtime.
//
//  "b200_sparse_puller" / "qed_sparse_puller": embedding tables resident in HBM.
//      Tables come from a QED file written by Blaze's EmbeddingBuilder (byte format:
//      blaze/blaze/store/quick_embedding/version_verifier.cc:9-72, trie.cc:70-124,
//      hashtable.cc:73-118, weight_blob.h:65-98) or from AddTable(). The file does
//      not record a table's dim (Blaze takes it from the model's EmbeddingConfig), so
//      a file table is uploaded on its first use, when the dim is known.
//  "mock_sparse_puller": no table; every id "hits" a row of ones, so the pooled value is
//      the per-id weight broadcast over dim (blaze/blaze/store/mock_sparse_puller.cc:56-133).
#include <cstring>
#include <fstream>

#include "runtime.h"

namespace blaze {
namespace store {
namespace {

struct FileTable {
  std::vector<std::pair<uint64_t, uint64_t>> entries;   // (key, byte offset into blob)
  std::string blob;
};

class B200SparsePuller : public SparsePuller {
 public:
  ~B200SparsePuller() override {
    for (auto& kv : tables_)
      for (auto& r : kv.second) xb_table_destroy(r.desc);
  }

  Status Load(const std::string& url) override {
    std::ifstream is(url, std::ios::binary);
    if (!is.is_open()) { LOG_ERROR("load quick embedding dict failed! url: ", url); return kFail; }
    char magic[31];
    is.read(magic, 31);
    if (!is.good() || strncmp(magic, "ALIMAMA_MODEL_SERVING_EMBEDDING", 31) != 0) {
      LOG_ERROR("load verifier failed! url: ", url);
      return kFail;
    }
    uint32_t version = 0;
    is.read((char*)&version, 4);
    if (!is.good() || version / 1000 != 2 || version % 1000 > 1) {
      LOG_ERROR("unknown value type of dict url: ", url, " version: ", version);
      return kFail;
    }
    file_fp16_ = version % 1000 == 1;
    uint64_t trie_size = 0;
    is.read((char*)&trie_size, 8);
    if (!is.good() || trie_size > (1u << 28)) { LOG_ERROR("load trie failed! url: ", url); return kFail; }
    std::string trie(trie_size, '\0');
    is.read(&trie[0], trie_size);
    if (!is.good()) { LOG_ERROR("load trie failed! url: ", url); return kFail; }
    std::unordered_map<uint16_t, std::string> gid_name;
    if (!WalkTrie(trie, 0, "", &gid_name, 0)) { LOG_ERROR("load trie failed! url: ", url); return kFail; }
    uint16_t gid;
    while (is.read((char*)&gid, 2)) {
      FileTable ft;
      uint32_t bucket_size = 0;
      is.read((char*)&bucket_size, 4);
      if (!is.good()) return Fail("hashtable", url, gid);
      is.seekg((std::streamoff)bucket_size * 8, std::ios::cur);      // the bucket directory is not needed
      uint64_t byte_size = 0;
      is.read((char*)&byte_size, 8);
      if (!is.good() || byte_size % 16 != 0) return Fail("hashtable", url, gid);
      ft.entries.resize(byte_size / 16);
      if (byte_size) is.read((char*)ft.entries.data(), byte_size);
      if (!is.good()) return Fail("hashtable", url, gid);
      uint64_t blob_size = 0;
      is.read((char*)&blob_size, 8);
      if (!is.good()) return Fail("weight blob", url, gid);
      ft.blob.resize(blob_size);
      if (blob_size) is.read(&ft.blob[0], blob_size);
      if (!is.good()) return Fail("weight blob", url, gid);
      auto it = gid_name.find(gid);
      if (it != gid_name.end()) file_tables_[it->second] = std::move(ft);
    }
    return kOK;
  }

  Status AddTable(const std::string& name, int64_t rows, int dim, int storage_dtype, const float* w,
                  const int64_t* keys) override {
    std::lock_guard<std::mutex> lock(mu_);
    if (tables_.count(name)) { LOG_ERROR("table ", name, " already registered"); return kFail; }
    Resident r;
    CUDA_CHECK(cudaGetDevice(&r.device));
    if (xb_table_create(&r.desc, rows, dim, storage_dtype, w, keys) != 0) {
      LOG_ERROR("xb_table_create failed: ", xb_last_error());
      return kFail;
    }
    tables_[name].push_back(r);
    return kOK;
  }

  Status GetAsync(const std::vector<SparsePullerInput>& input, std::vector<SparsePullerOutput>& output, int device_id,
                  cudaStream_t stream, int* launches) override {
    if (input.size() != output.size()) return kFail;
    std::vector<xb_pool_group> groups;
    for (size_t i = 0; i < input.size(); ++i) {
      const SparsePullerInput& in = input[i];
      const SparsePullerOutput& out = output[i];
      if (in.in_item.size() != out.out_item.size()) return kFail;
      if (in.in_item.empty() || in.key_num == nullptr) continue;      // feature group without inputs
      if (in.in_item.size() > XB_MAX_POOL_ITEMS) { LOG_ERROR("more than ", XB_MAX_POOL_ITEMS, " blocks read one feature group"); return kFail; }
      xb_pool_group g;
      memset(&g, 0, sizeof(g));
      g.table = Find(in.name, in.dim, device_id);                     // nullptr: table-name miss -> zeros
      g.ids = in.key; g.values = in.value; g.values_dtype = in.value_type;
      g.segments = reinterpret_cast<const int32_t*>(in.key_num);
      g.n_ids = (int64_t)in.key_size; g.batch = (int64_t)in.key_num_size;
      g.dim = in.dim; g.id_dtype = in.key_type; g.out_dtype = in.value_type;
      if (in.num_type != kInt32) { LOG_ERROR("Unsupported num type:", in.num_type); return kFail; }
      g.n_items = (int)in.in_item.size();
      for (int k = 0; k < g.n_items; ++k) {
        g.items[k].udf = in.in_item[k].udf_type;
        g.items[k].trunc_dir = in.in_item[k].trunc_direction;
        g.items[k].trunc_num = in.in_item[k].trunc_num;
        g.items[k].out = out.out_item[k].out;
        g.items[k].stride = (int64_t)out.out_item[k].stride;
      }
      groups.push_back(g);
    }
    for (size_t b = 0; b < groups.size(); b += XB_MAX_POOL_GROUPS) {
      const int n = (int)std::min<size_t>(XB_MAX_POOL_GROUPS, groups.size() - b);
      const size_t need = xb_embedding_pool_scratch_bytes(groups.data() + b, n);
      void* scratch = Scratch(device_id, need);
      if (xb_embedding_pool(groups.data() + b, n, scratch, need, stream) != 0) {
        LOG_ERROR("xb_embedding_pool failed: ", xb_last_error());
        return kFail;
      }
      *launches += 2;
    }
    return kOK;
  }

 protected:
  struct Resident {
    xb_table_desc* desc = nullptr;
    int device = 0;
  };

  static Status Fail(const char* what, const std::string& url, int gid) {
    LOG_ERROR("load ", what, " failed! url: ", url, " gid: ", gid);
    return kFail;
  }

  // depth-first walk of the serialized trie; a node with value != 0xFF names a table
  static bool WalkTrie(const std::string& bytes, uint32_t off, const std::string& prefix,
                       std::unordered_map<uint16_t, std::string>* out, int depth) {
    if (depth > 256 || (size_t)off + 3 > bytes.size()) return false;
    uint16_t value;
    memcpy(&value, bytes.data() + off, 2);
    const uint8_t branches = (uint8_t)bytes[off + 2];
    if (value != 0xFF) (*out)[value] = prefix;
    size_t pos = off + 3;
    for (int i = 0; i < branches; ++i) {
      if (pos + 5 > bytes.size()) return false;
      const char c = bytes[pos];
      uint32_t child;
      memcpy(&child, bytes.data() + pos + 1, 4);
      pos += 5;
      if (!WalkTrie(bytes, child, prefix + c, out, depth + 1)) return false;
    }
    return true;
  }

  const xb_table_desc* Find(const std::string& name, int dim, int device_id) {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = tables_.find(name);
    if (it == tables_.end()) {
      auto f = file_tables_.find(name);
      if (f == file_tables_.end()) return nullptr;
      // first use of a file table: now the dim is known, build the dense image and upload it
      const FileTable& ft = f->second;
      const size_t es = file_fp16_ ? 2 : 4;
      const int64_t rows = (int64_t)ft.entries.size();
      if (rows == 0) return nullptr;
      std::vector<float> w((size_t)rows * dim);
      std::vector<int64_t> keys(rows);
      for (int64_t r = 0; r < rows; ++r) {
        keys[r] = (int64_t)ft.entries[r].first;
        const uint64_t off = ft.entries[r].second;
        BLAZE_CONDITION_THROW(off + (uint64_t)dim * es <= ft.blob.size(), "table ", name, ": dim ", dim,
                              " reads past the weight blob");
        for (int c = 0; c < dim; ++c) {
          if (file_fp16_) {
            uint16_t h;
            memcpy(&h, ft.blob.data() + off + 2 * c, 2);
            w[r * dim + c] = HalfBitsToFloat(h);
          } else {
            memcpy(&w[r * dim + c], ft.blob.data() + off + 4 * c, 4);
          }
        }
      }
      Resident res;
      res.device = device_id;
      CUDA_CHECK(cudaSetDevice(device_id));
      BLAZE_CONDITION_THROW(xb_table_create(&res.desc, rows, dim, file_fp16_ ? XB_F16 : XB_F32, w.data(), keys.data()) == 0,
                            "xb_table_create failed: ", xb_last_error());
      it = tables_.emplace(name, std::vector<Resident>{res}).first;
      file_tables_.erase(f);
    }
    for (const Resident& r : it->second)
      if (r.device == device_id) return r.desc;
    // first use on another device of this process: one replica per device, copied device to device
    // (one PredictorManager serves CreatePredictor(type, device_id) for any device id)
    Resident rep;
    rep.device = device_id;
    CUDA_CHECK(cudaSetDevice(device_id));
    const Resident& src = it->second.front();
    BLAZE_CONDITION_THROW(xb_table_clone(&rep.desc, src.desc, src.device) == 0, "table ", name, ": replica on device ",
                          device_id, " failed: ", xb_last_error());
    it->second.push_back(rep);
    return rep.desc;
  }

  void* Scratch(int device, size_t bytes) {
    // one scratch buffer per (thread, device): predictors are per-thread and their kernels run in stream order
    thread_local std::unordered_map<int, std::pair<void*, size_t>> bufs;
    auto& b = bufs[device];
    if (b.second < bytes) {
      if (b.first) { CUDA_CHECK(cudaDeviceSynchronize()); cudaFree(b.first); }
      const size_t cap = std::max<size_t>(bytes, 1 << 16);
      CUDA_CHECK(cudaMalloc(&b.first, cap));
      b.second = cap;
    }
    return b.first;
  }

  std::mutex mu_;
  std::unordered_map<std::string, std::vector<Resident>> tables_;   // one replica per device that used the table
  std::unordered_map<std::string, FileTable> file_tables_;
  bool file_fp16_ = false;
};

// "b200_sharded_sparse_puller": tables too large for one GPU, row-sharded over the ranks of one box (one process
// per GPU). The Embedding operator's groups are pooled by ONE xb_sharded_pool call: ids routed to the owners,
// pooled there, partial sums returned and combined, the two exchanges done by NCCL inside the kernel library.
// It takes what the large-table configuration needs: every feature group of the operator feeds one kSum item,
// all tables have one dim, the items of a table's groups are adjacent and the whole operator writes one block
// (group g at column g * dim). Per-id weights are NOT routed: every id counts with weight 1.0, whatever the
// `.values` input holds (the configuration feeds ones).
class ShardedSparsePuller : public B200SparsePuller {
 public:
  ~ShardedSparsePuller() override {
    if (ctx_) xb_shard_ctx_destroy(ctx_);
    for (void* p : {(void*)ids_, (void*)counts_, (void*)offsets_, (void*)items_dev_, scan_scratch_}) if (p) cudaFree(p);
    if (items_host_) cudaFreeHost(items_host_);
  }

  Status InitSharded(int rank, int world, const void* unique_id, int64_t max_ids_per_step, int partial_dtype,
                     float capacity_factor) override {
    if (world < 1 || rank < 0 || rank >= world || max_ids_per_step <= 0) return kFail;
    rank_ = rank; world_ = world; max_ids_ = max_ids_per_step; partial_dtype_ = partial_dtype; factor_ = capacity_factor;
    if (unique_id) { uid_.assign((const char*)unique_id, (const char*)unique_id + 128); }
    return kOK;
  }

  Status AddDeviceShard(const std::string& name, int64_t rows, int dim, int storage_dtype, const void* device_weights,
                        int64_t pitch_bytes) override {
    std::lock_guard<std::mutex> lock(mu_);
    if (tables_.count(name) || borrowed_.count(name)) { LOG_ERROR("table ", name, " already registered"); return kFail; }
    std::unique_ptr<xb_table_desc> d(new xb_table_desc());
    memset(d.get(), 0, sizeof(xb_table_desc));
    d->weights = device_weights; d->rows = rows; d->dim = dim; d->dtype = storage_dtype; d->row_pitch_bytes = pitch_bytes;
    borrowed_[name] = std::move(d);
    return kOK;
  }

  Status GetAsync(const std::vector<SparsePullerInput>& input, std::vector<SparsePullerOutput>& output, int device_id,
                  cudaStream_t stream, int* launches) override {
    if (world_ == 0) { LOG_ERROR("sharded puller used before InitSharded"); return kFail; }
    if (input.size() != output.size() || input.empty()) return kFail;
    const size_t G = input.size();
    const int dim = input[0].dim;
    const size_t B = input[0].key_num_size;
    const int vtype = input[0].value_type;
    const size_t esz = vtype == kFloat16 ? 2 : 4;
    char* base = reinterpret_cast<char*>(output[0].out_item.empty() ? nullptr : output[0].out_item[0].out);
    int64_t n_ids = 0;
    std::vector<std::string> table_order;
    std::vector<int64_t> table_groups;
    for (size_t g = 0; g < G; ++g) {
      const SparsePullerInput& in = input[g];
      const bool shape_ok = in.in_item.size() == 1 && output[g].out_item.size() == 1 && in.in_item[0].udf_type == kSum &&
                            in.dim == dim && in.key_num_size == B && in.key_type == kInt64 && in.num_type == kInt32 &&
                            output[g].out_item[0].stride == output[0].out_item[0].stride &&
                            reinterpret_cast<char*>(output[g].out_item[0].out) == base + g * dim * esz;
      if (!shape_ok) {
        LOG_ERROR("sharded puller: feature group ", g, " is outside what it takes (one kSum item per group, one dim, "
                  "int64 ids, int32 counts, one output block with group g at column g * dim)");
        return kFail;
      }
      if (table_order.empty() || table_order.back() != in.name) {
        for (const auto& t : table_order)
          if (t == in.name) { LOG_ERROR("sharded puller: the groups of table ", in.name, " are not adjacent"); return kFail; }
        table_order.push_back(in.name);
        table_groups.push_back(0);
      }
      ++table_groups.back();
      n_ids += (int64_t)in.key_size;
    }
    if (n_ids > max_ids_) { LOG_ERROR("sharded puller: ", n_ids, " ids in one step, InitSharded allowed ", max_ids_); return kFail; }
    CUDA_CHECK(cudaSetDevice(device_id));
    if (!ctx_ || batch_ != B || tables_sig_ != table_order || groups_sig_ != table_groups) {
      if (ctx_) { CUDA_CHECK(cudaDeviceSynchronize()); xb_shard_ctx_destroy(ctx_); ctx_ = nullptr; }
      std::vector<const xb_table_desc*> descs;
      std::vector<int64_t> segs;
      for (size_t t = 0; t < table_order.size(); ++t) {
        const xb_table_desc* d = Shard(table_order[t], dim, device_id);
        if (!d) { LOG_ERROR("sharded puller: no shard of table ", table_order[t], " on this rank"); return kFail; }
        descs.push_back(d);
        segs.push_back(table_groups[t] * (int64_t)B);
      }
      xb_shard_config cfg;
      memset(&cfg, 0, sizeof(cfg));
      cfg.rank = rank_; cfg.world = world_; cfg.dim = dim; cfg.n_tables = (int)descs.size();
      cfg.tables = descs.data(); cfg.table_segments = segs.data(); cfg.max_ids = max_ids_;
      cfg.partial_dtype = partial_dtype_; cfg.capacity_factor = factor_;
      if (xb_shard_ctx_create(&ctx_, uid_.empty() ? nullptr : uid_.data(), &cfg) != 0) {
        LOG_ERROR("xb_shard_ctx_create failed: ", xb_last_error());
        return kFail;
      }
      batch_ = B; tables_sig_ = table_order; groups_sig_ = table_groups;
      // staging for the operator's inputs as one routing problem: ids and counts of all groups back to back
      for (void** p : {(void**)&ids_, (void**)&counts_, (void**)&offsets_, (void**)&items_dev_, &scan_scratch_}) {
        if (*p) cudaFree(*p);
        *p = nullptr;
      }
      CUDA_CHECK(cudaMalloc((void**)&ids_, (size_t)max_ids_ * 8));
      CUDA_CHECK(cudaMalloc((void**)&counts_, G * B * 4));
      CUDA_CHECK(cudaMalloc((void**)&offsets_, (G * B + 1) * 4));
      CUDA_CHECK(cudaMalloc((void**)&items_dev_, 2 * G * sizeof(xb_copy_item)));
      scan_bytes_ = xb_scan_counts_scratch_bytes(1, (int64_t)(G * B));
      CUDA_CHECK(cudaMalloc(&scan_scratch_, std::max<size_t>(scan_bytes_, 256)));
      if (items_host_) cudaFreeHost(items_host_);
      CUDA_CHECK(cudaHostAlloc((void**)&items_host_, 2 * G * sizeof(xb_copy_item), cudaHostAllocDefault));
    }
    // one descriptor-table copy gathers the ids and the counts of every group (the pinned table is reused: the
    // previous call's copy of it must have been consumed, which by now it long has)
    if (consumed_recorded_) CUDA_CHECK(cudaEventSynchronize(Consumed()));
    int64_t at = 0, max_bytes = 0;
    for (size_t g = 0; g < G; ++g) {
      items_host_[2 * g] = {input[g].key, ids_ + at, (int64_t)input[g].key_size * 8};
      items_host_[2 * g + 1] = {input[g].key_num, counts_ + g * B, (int64_t)B * 4};
      max_bytes = std::max<int64_t>(max_bytes, std::max<int64_t>((int64_t)input[g].key_size * 8, (int64_t)B * 4));
      at += (int64_t)input[g].key_size;
    }
    CUDA_CHECK(cudaMemcpyAsync(items_dev_, items_host_, 2 * G * sizeof(xb_copy_item), cudaMemcpyHostToDevice, stream));
    XB_CHECK(xb_copy_segments(items_dev_, (int)(2 * G), max_bytes, stream));
    CUDA_CHECK(cudaEventRecord(Consumed(), stream));
    consumed_recorded_ = true;
    XB_CHECK(xb_scan_counts(counts_, 0, offsets_, 0, 1, (int64_t)(G * B), scan_scratch_, scan_bytes_, stream));
    if (xb_sharded_pool(ctx_, ids_, offsets_, n_ids, (int64_t)G, 0, base, (int64_t)output[0].out_item[0].stride,
                        vtype, stream) != 0) {
      LOG_ERROR("xb_sharded_pool failed: ", xb_last_error());
      return kFail;
    }
    *launches += 12;
    return kOK;
  }

  // after the caller synchronised its stream: did a step drop ids because a bucket overflowed?
  bool Overflowed() {
    int32_t f = 0;
    return ctx_ && xb_shard_ctx_status(ctx_, &f) == 0 && f != 0;
  }

 private:
  const xb_table_desc* Shard(const std::string& name, int dim, int device_id) {
    {
      std::lock_guard<std::mutex> lock(mu_);
      auto b = borrowed_.find(name);
      if (b != borrowed_.end()) return b->second.get();
    }
    return Find(name, dim, device_id);
  }
  cudaEvent_t Consumed() {
    if (!consumed_) cudaEventCreateWithFlags(&consumed_, cudaEventDisableTiming);
    return consumed_;
  }

  int rank_ = 0, world_ = 0, partial_dtype_ = XB_F16;
  int64_t max_ids_ = 0;
  float factor_ = 2.f;
  std::vector<char> uid_;
  xb_shard_ctx* ctx_ = nullptr;
  size_t batch_ = 0;
  std::vector<std::string> tables_sig_;
  std::vector<int64_t> groups_sig_;
  std::unordered_map<std::string, std::unique_ptr<xb_table_desc>> borrowed_;
  int64_t* ids_ = nullptr;
  int32_t *counts_ = nullptr, *offsets_ = nullptr;
  xb_copy_item *items_dev_ = nullptr, *items_host_ = nullptr;
  void* scan_scratch_ = nullptr;
  size_t scan_bytes_ = 0;
  cudaEvent_t consumed_ = nullptr;
  bool consumed_recorded_ = false;
};

class MockSparsePuller : public B200SparsePuller {
 public:
  Status Load(const std::string&) override { return kOK; }
  Status GetAsync(const std::vector<SparsePullerInput>& input, std::vector<SparsePullerOutput>& output, int device_id,
                  cudaStream_t stream, int* launches) override {
    // every key resolves to row 0 of a one-row table of ones of the group's dim
    std::vector<SparsePullerInput> in = input;
    size_t max_ids = 0;
    for (const auto& g : in) max_ids = std::max(max_ids, g.key_size);
    void* zeros = Zeros(device_id, max_ids * 8, stream);
    for (auto& g : in) {
      if (g.in_item.empty()) continue;
      g.name = "__ones_" + std::to_string(g.dim);
      {
        std::lock_guard<std::mutex> lock(mu_);
        if (!tables_.count(g.name)) {
          std::vector<float> ones(g.dim, 1.0f);
          Resident r;
          r.device = device_id;
          BLAZE_CONDITION_THROW(xb_table_create(&r.desc, 1, g.dim, XB_F32, ones.data(), nullptr) == 0, xb_last_error());
          tables_[g.name].push_back(r);
        }
      }
      g.key = zeros;
      g.key_type = kInt64;
    }
    return B200SparsePuller::GetAsync(in, output, device_id, stream, launches);
  }

 private:
  void* Zeros(int device, size_t bytes, cudaStream_t stream) {
    thread_local std::unordered_map<int, std::pair<void*, size_t>> bufs;
    auto& b = bufs[device];
    if (b.second < bytes) {
      if (b.first) { CUDA_CHECK(cudaDeviceSynchronize()); cudaFree(b.first); }
      const size_t cap = std::max<size_t>(bytes, 1 << 12);
      CUDA_CHECK(cudaMalloc(&b.first, cap));
      b.second = cap;
    }
    CUDA_CHECK(cudaMemsetAsync(b.first, 0, std::max<size_t>(bytes, 8), stream));
    return b.first;
  }
};

SparsePuller* CreateB200() { return new B200SparsePuller(); }
SparsePuller* CreateMock() { return new MockSparsePuller(); }
SparsePuller* CreateSharded() { return new ShardedSparsePuller(); }

struct RegisterAll {
  RegisterAll() {
    SparsePullerCreationRegisterer::Get()->Register("b200_sparse_puller", CreateB200);
    SparsePullerCreationRegisterer::Get()->Register("qed_sparse_puller", CreateB200);
    SparsePullerCreationRegisterer::Get()->Register("mock_sparse_puller", CreateMock);
    SparsePullerCreationRegisterer::Get()->Register("b200_sharded_sparse_puller", CreateSharded);
  }
} g_register_all;

}  // namespace
}  // namespace store
}  // namespace blaze
