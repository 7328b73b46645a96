// C glue around the UNMODIFIED reference sparse store (QuickEmbeddingDict).
//
// TEST INFRASTRUCTURE ONLY: linked into oracle/_ref/libqed_ref.so together with
// the reference's own store sources, compiled where they lie. It lets the
// parity tests and the CPU-baseline leg of the benchmark run the reference's
// pooling loop (blaze/blaze/store/quick_embedding/quick_embedding_dict.cc:89-147)
// on the same arrays the CUDA path consumes.
//
// Tables are written to a QED file the same way the reference's own unit test
// does (blaze/blaze/test/store/quick_embedding/quick_embedding_dict_test.cc:30-79)
// and then loaded with QuickEmbeddingDict::Load.
#include <cstdint>
#include <cstring>
#include <fstream>
#include <memory>
#include <string>
#include <vector>

#include "blaze/store/quick_embedding/quick_embedding_dict.h"
#include "blaze/common/types.h"

using namespace blaze;
using namespace blaze::store;

extern "C" {

// Write `ntables` fp32 tables to `path`. Table t has nrows[t] rows of dims[t]
// floats, keys[t][r] is the int64 key of row r.
int ref_qed_build(const char* path, int ntables, const char* const* names,
                  const int* dims, const int64_t* nrows,
                  const int64_t* const* keys, const float* const* weights) {
  VersionVerifier verifier(DictValueType::fp32);
  BulkLoadTrie trie;
  for (int t = 0; t < ntables; ++t) trie.PreInsert(names[t], (uint16_t)t);
  if (!trie.BulkLoad()) return -1;
  std::ofstream os(path, std::ios::binary);
  if (!os.is_open()) return -2;
  if (!verifier.Dump(&os)) return -3;
  if (!trie.Dump(&os)) return -4;
  for (int t = 0; t < ntables; ++t) {
    std::unique_ptr<BulkLoadHashTable> ht(new BulkLoadHashTable());
    WeightBlob<float> blob;
    if (!blob.AllocateMemory((size_t)nrows[t] * dims[t])) return -5;
    for (int64_t r = 0; r < nrows[t]; ++r) {
      float* w = nullptr;
      uint64_t off = blob.InsertWeights(dims[t], &w);
      if (w == nullptr) return -6;
      memcpy(w, weights[t] + r * dims[t], sizeof(float) * dims[t]);
      ht->PreInsert((uint64_t)keys[t][r], off);
    }
    uint16_t gid = (uint16_t)t;
    os.write((char*)&gid, sizeof(gid));
    if (!ht->BulkLoad()) return -7;
    if (!ht->Dump(&os)) return -8;
    if (!blob.Dump(&os)) return -9;
  }
  os.close();
  return 0;
}

void* ref_qed_open(const char* path) {
  QuickEmbeddingDict* d = new QuickEmbeddingDict();
  if (d->Load(path) != kOK) { delete d; return nullptr; }
  return d;
}

void ref_qed_close(void* h) { delete reinterpret_cast<QuickEmbeddingDict*>(h); }

// One feature group, n_items output blocks. udf: 0 sum, 1 avg, 2 assign.
// Outputs must be zeroed by the caller where the reference op would memset
// them (blaze/blaze/operator/sparse_op/embedding/embedding_op.h:181).
int ref_qed_get(void* h, const char* table, int dim, const int64_t* keys,
                const float* values, const int32_t* key_num, int64_t batch,
                int n_items, const int* udf, const int* trunc_dir,
                const int* trunc_num, float* const* outs,
                const int64_t* strides) {
  QuickEmbeddingDict* d = reinterpret_cast<QuickEmbeddingDict*>(h);
  std::vector<SparsePullerInput> in(1);
  std::vector<SparsePullerOutput> out(1);
  in[0].name = table;
  in[0].key = (void*)keys;
  in[0].value = (void*)values;
  in[0].key_num = (void*)key_num;
  in[0].key_num_size = (size_t)batch;
  in[0].key_type = blaze::kInt64;
  in[0].value_type = blaze::kFloat;
  in[0].num_type = blaze::kInt32;
  in[0].dim = dim;
  for (int k = 0; k < n_items; ++k) {
    SparsePullerInput::Param p;
    p.udf_type = (UDFType)udf[k];
    p.trunc_direction = (TruncDirection)trunc_dir[k];
    p.trunc_num = trunc_num[k];
    in[0].in_item.push_back(p);
    SparsePullerOutput::OutItem o;
    o.out = outs[k];
    o.stride = (size_t)strides[k];
    out[0].out_item.push_back(o);
  }
  try {
    return (int)d->Get(in, out);
  } catch (...) {
    return -100;
  }
}

}  // extern "C"
