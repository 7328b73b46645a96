/* C API of the B200 host runtime: the entry points of Blaze's
 * blaze/blaze/api/c_api/c_api_predictor.h and c_api_error.h with the same names
 * and argument meaning (0 = success, -1 = failure, reason through
 * Blaze_GetLastErrorString), plus Blaze_B200_* extensions for registering
 * in-memory embedding tables and text NetDefs (used by tests and benchmarks). */
#ifndef BLAZE_B200_C_API_PREDICTOR_H_
#define BLAZE_B200_C_API_PREDICTOR_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* PredictorManagerHandle;
typedef void* PredictorHandle;

const char* Blaze_GetLastErrorString(void);

int Blaze_InitScheduler(int enable_batching, int max_batch_size, int batch_timeout_micros, int num_threads_for_cpu,
                        int num_threads_for_cuda, int num_threads_for_pipe);
int Blaze_PredictorManagerCreate(PredictorManagerHandle* handle);
int Blaze_PredictorManagerDelete(PredictorManagerHandle handle);
int Blaze_PredictorManagerSetDataType(PredictorManagerHandle handle, int data_type);
int Blaze_PredictorManagerSetRunMode(PredictorManagerHandle handle, const char* run_mode);
int Blaze_LoadSparseModelWeight(PredictorManagerHandle handle, const char* sparse_model_weight_file);
int Blaze_PredcitorManagerLoadModel(PredictorManagerHandle handle, const char* blaze_model_file, int optimization_pass);
int Blaze_PredictorManagerLoadDeepNetModel(PredictorManagerHandle handle, const char* deepnet_conf_file,
                                           const char* deepnet_param_file, int optimization_pass);
int Blaze_PredictorCreate(PredictorManagerHandle predictor_mgr, int device_type, int device_id, PredictorHandle* handle);
int Blaze_PredictorDelete(PredictorHandle handle);
int Blaze_PredictorReshapeInput(PredictorHandle handle, const char* name, const int* data, int num);
int Blaze_PredictorFeed(PredictorHandle handle, const char* name, void* data, int len);
int Blaze_PredictorForward(PredictorHandle handle);
int Blaze_PredictorOutputShape(PredictorHandle handle, const char* name, size_t* ndim, size_t** shape);
int Blaze_PredictorOutputDataType(PredictorHandle handle, const char* name, int* data_type);
int Blaze_PredictorOutput(PredictorHandle handle, const char* name, void* data, size_t len);
int Blaze_PredictorParamName(PredictorHandle handle, size_t* ndim, const char*** name);
int Blaze_PredictorParamShape(PredictorHandle handle, const char* name, size_t* ndim, size_t** shape);
int Blaze_PredictorParamDataType(PredictorHandle handle, const char* name, int* data_type);
int Blaze_PredictorParam(PredictorHandle handle, const char* name, void* data, size_t len);
int Blaze_PredictorListInputNames(PredictorHandle handle, size_t* ndim, const char*** names);
int Blaze_PredictorListOutputNames(PredictorHandle handle, size_t* ndim, const char*** names);
int Blaze_PredictorRegisterObservers(PredictorHandle handle, size_t ndim, const char** names);
int Blaze_PredictorDumpObservers(PredictorHandle handle, size_t* ndim, const char*** key, const char*** value);

/* ---- extensions ---------------------------------------------------------- */
/* Model given as NetDef text (protobuf text format) instead of a file. */
int Blaze_B200_LoadModelFromText(PredictorManagerHandle handle, const char* netdef_text, int optimization_pass);
/* Sparse puller of the given registered type ("b200_sparse_puller", "qed_sparse_puller",
 * "mock_sparse_puller"); uri may be NULL for types that need no file. */
int Blaze_B200_LoadSparseModelWeight(PredictorManagerHandle handle, const char* uri, const char* type);
/* Registers an in-memory fp32 [rows, dim] table (host pointers) with the manager's puller
 * (type b200/qed); storage_dtype 1 = fp32, 12 = fp16; keys may be NULL (row numbers). */
int Blaze_B200_AddTable(PredictorManagerHandle handle, const char* table_name, int64_t rows, int dim,
                        int storage_dtype, const float* weights, const int64_t* keys);
/* Feed whose source is already in device memory (no host staging). */
/* Row-sharded tables (tables too large for one GPU; one process per GPU of a box). Load the puller
 * "b200_sharded_sparse_puller" (Blaze_B200_LoadSparseModelWeight(handle, NULL, type)), make the 128-byte communicator
 * id on one rank with Blaze_B200_ShardUniqueId and hand it to the others, call Blaze_B200_ShardedInit on every rank,
 * then register this rank's shards: row r of a table lives on rank r % world at local row r / world. An Embedding
 * operator over such tables is pooled by one xb_sharded_pool call (see include/xdlb200.h). */
int Blaze_B200_ShardUniqueId(void* unique_id128);
int Blaze_B200_ShardedInit(PredictorManagerHandle handle, int rank, int world, const void* unique_id128,
                           int64_t max_ids_per_step, int partial_dtype, float capacity_factor);
/* A shard that already lives in device memory (rows x dim elements of storage_dtype, pitch_bytes apart). The caller
 * keeps the memory alive while predictors exist. */
int Blaze_B200_AddDeviceShard(PredictorManagerHandle handle, const char* table_name, int64_t rows, int dim,
                              int storage_dtype, const void* device_weights, int64_t pitch_bytes);
/* Operator types of the model the manager holds (after the optimization passes when LoadModel ran them), comma
 * separated, into `buffer`. Returns 0, or the capacity needed when `buffer` is NULL or too small. */
int Blaze_B200_ModelOpTypes(PredictorManagerHandle handle, char* buffer, size_t capacity);
int Blaze_B200_PredictorFeedDevice(PredictorHandle handle, const char* name, const void* device_data, size_t len);
/* Device pointer of an output (valid until the next Forward); no device-to-host copy. */
int Blaze_B200_PredictorOutputDevice(PredictorHandle handle, const char* name, void** device_data, size_t* len);
/* Number of kernel-library calls issued by the last Forward. */
int Blaze_B200_PredictorLastLaunchCount(PredictorHandle handle, int* count);
/* Predictor::Forward(cb): with batching switched on by Blaze_InitScheduler the call returns at once and
 * cb(arg) runs on the batch thread when this predictor's outputs are ready (requests of several
 * predictors of one model are stacked into one run); without batching the net runs before the call
 * returns and cb(arg) is called from it. */
int Blaze_B200_PredictorForwardAsync(PredictorHandle handle, void (*cb)(void*), void* arg);
/* The batch the queue would close on `n_tasks` waiting requests, without running anything: rows[t * n_inputs + j]
 * is the first dimension of request t's j-th per-sample input. Writes the positions that run together with
 * request 0 (at most max_tasks, request 0 included) and returns how many; -1 on bad arguments. */
int Blaze_B200_PlanBatch(const int64_t* rows, int n_tasks, int n_inputs, int max_tasks, int* picked);
/* Merged runs so far and the requests they carried (process-wide). */
int Blaze_B200_BatchingStats(int64_t* batches, int64_t* tasks);

#ifdef __cplusplus
}
#endif
#endif
