// C glue around the UNMODIFIED reference Workspace / Net / operators on their CPU path.
//
// TEST INFRASTRUCTURE ONLY: linked into oracle/_ref/libblaze_cpu.so by oracle/build_ref_dense.sh together with the
// reference's own sources, compiled where they lie. It lets the parity tests and the reference arm of the
// benchmark run a text-format NetDef the way the reference's operator tests do
// (blaze/blaze/test/operator/operator_test_common.h:19-32: Workspace::CreateNet(file) then Net::Run), with the
// inputs fed as PredictorImpl::Feed does (blaze/blaze/api/cpp_api/predictor_impl.cc:95-137).
//
// The CBLAS entry points the reference calls (blaze/blaze/math/gemm.cc:26-79, 313-326) are defined here: they
// forward to an OpenBLAS found at run time (the reference links an unpinned OpenBLAS,
// blaze/blaze/CMakeLists.txt:58) or, when none is found, to a plain k-ascending fp32 loop. refnet_blas() says which.
#include <dlfcn.h>
#include <glob.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "cblas.h"
#include "blaze/common/blob.h"
#include "blaze/graph/net.h"
#include "blaze/graph/workspace.h"
#include "blaze/store/sparse_puller.h"

namespace {

typedef void (*sgemm_fn)(CBLAS_ORDER, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, int, int, int, float, const float*, int,
                         const float*, int, float, float*, int);
typedef void (*dgemm_fn)(CBLAS_ORDER, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, int, int, int, double, const double*, int,
                         const double*, int, double, double*, int);
typedef void (*sgemv_fn)(CBLAS_ORDER, CBLAS_TRANSPOSE, int, int, float, const float*, int, const float*, int, float,
                         float*, int);
typedef void (*dgemv_fn)(CBLAS_ORDER, CBLAS_TRANSPOSE, int, int, double, const double*, int, const double*, int,
                         double, double*, int);
typedef void (*threads_fn)(int);

struct Blas {
  sgemm_fn sgemm = nullptr;
  dgemm_fn dgemm = nullptr;
  sgemv_fn sgemv = nullptr;
  dgemv_fn dgemv = nullptr;
  std::string name = "naive k-ascending loops (no OpenBLAS found)";
  Blas() {
    // XDL_OPENBLAS=<file> wins; "none" forces the plain loops
    const char* env = getenv("XDL_OPENBLAS");
    std::vector<std::string> cands;
    if (env && *env) {
      if (strcmp(env, "none") == 0) return;
      cands.push_back(env);
    } else {
      // LP64 builds that ship with the image's Python packages: scipy's (symbols prefixed scipy_), OpenCV's
      const char* pats[] = {"/opt/*/.venv/lib/python3*/site-packages/scipy.libs/libscipy_openblas-*.so",
                            "/opt/*/.venv/lib/python3*/site-packages/opencv_python_headless.libs/libopenblas*.so*",
                            "/usr/lib/x86_64-linux-gnu/libopenblas.so*", "/usr/lib/x86_64-linux-gnu/openblas*/libopenblas*.so*"};
      for (const char* pat : pats) {
        glob_t g;
        if (glob(pat, 0, nullptr, &g) == 0)
          for (size_t i = 0; i < g.gl_pathc; ++i) cands.push_back(g.gl_pathv[i]);
        globfree(&g);
      }
    }
    for (const auto& path : cands) {
      void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
      if (!h) continue;
      for (const char* prefix : {"", "scipy_"}) {
        const std::string pre(prefix);
        sgemm_fn s = (sgemm_fn)dlsym(h, (pre + "cblas_sgemm").c_str());
        dgemm_fn d = (dgemm_fn)dlsym(h, (pre + "cblas_dgemm").c_str());
        sgemv_fn sv = (sgemv_fn)dlsym(h, (pre + "cblas_sgemv").c_str());
        dgemv_fn dv = (dgemv_fn)dlsym(h, (pre + "cblas_dgemv").c_str());
        if (s && d && sv && dv) {
          sgemm = s; dgemm = d; sgemv = sv; dgemv = dv;
          // one BLAS thread per net, as a Blaze predictor runs (parallelism comes from predictors on host threads)
          threads_fn t = (threads_fn)dlsym(h, (pre + "openblas_set_num_threads").c_str());
          if (t) t(1);
          name = "OpenBLAS " + path + " (1 thread per call)";
          return;
        }
      }
      dlclose(h);
    }
  }
};
Blas& blas() {
  static Blas b;
  return b;
}

template <typename T>
void naive_gemm(CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int M, int N, int K, T alpha, const T* A, int lda, const T* B,
                int ldb, T beta, T* C, int ldc) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      T acc = 0;
      for (int k = 0; k < K; ++k) {
        const T a = ta == CblasNoTrans ? A[(size_t)m * lda + k] : A[(size_t)k * lda + m];
        const T b = tb == CblasNoTrans ? B[(size_t)k * ldb + n] : B[(size_t)n * ldb + k];
        acc += a * b;
      }
      C[(size_t)m * ldc + n] = alpha * acc + (beta == 0 ? 0 : beta * C[(size_t)m * ldc + n]);
    }
}
template <typename T>
void naive_gemv(CBLAS_TRANSPOSE ta, int M, int N, T alpha, const T* A, int lda, const T* x, int incx, T beta, T* y, int incy) {
  const int rows = ta == CblasNoTrans ? M : N, cols = ta == CblasNoTrans ? N : M;
  for (int r = 0; r < rows; ++r) {
    T acc = 0;
    for (int c = 0; c < cols; ++c) acc += (ta == CblasNoTrans ? A[(size_t)r * lda + c] : A[(size_t)c * lda + r]) * x[(size_t)c * incx];
    y[(size_t)r * incy] = alpha * acc + (beta == 0 ? 0 : beta * y[(size_t)r * incy]);
  }
}

}  // namespace

extern "C" {

void cblas_sgemm(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int M, int N, int K, float alpha, const float* A,
                 int lda, const float* B, int ldb, float beta, float* C, int ldc) {
  if (blas().sgemm) blas().sgemm(o, ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
  else naive_gemm<float>(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}
void cblas_dgemm(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int M, int N, int K, double alpha, const double* A,
                 int lda, const double* B, int ldb, double beta, double* C, int ldc) {
  if (blas().dgemm) blas().dgemm(o, ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
  else naive_gemm<double>(ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}
void cblas_sgemv(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, int M, int N, float alpha, const float* A, int lda, const float* x,
                 int incx, float beta, float* y, int incy) {
  if (blas().sgemv) blas().sgemv(o, ta, M, N, alpha, A, lda, x, incx, beta, y, incy);
  else naive_gemv<float>(ta, M, N, alpha, A, lda, x, incx, beta, y, incy);
}
void cblas_dgemv(CBLAS_ORDER o, CBLAS_TRANSPOSE ta, int M, int N, double alpha, const double* A, int lda, const double* x,
                 int incx, double beta, double* y, int incy) {
  if (blas().dgemv) blas().dgemv(o, ta, M, N, alpha, A, lda, x, incx, beta, y, incy);
  else naive_gemv<double>(ta, M, N, alpha, A, lda, x, incx, beta, y, incy);
}

const char* refnet_blas(void) { return blas().name.c_str(); }

struct RefNet {
  blaze::Workspace ws;
  std::shared_ptr<blaze::Net> net;
  std::string error;
};
static thread_local std::string g_refnet_error;
const char* refnet_last_error(void) { return g_refnet_error.c_str(); }

// net_file: text-format NetDef. qed_file (may be NULL or ""): a QED file for the Embedding operators, served by
// the reference's own "qed_sparse_puller" (blaze/blaze/store/quick_embedding/quick_embedding_dict.cc:153).
void* refnet_create(const char* net_file, const char* qed_file) {
  std::unique_ptr<RefNet> r(new RefNet());
  try {
    if (qed_file && *qed_file) {
      // one loaded dictionary per file, shared by every net of the process (a PredictorManager holds one
      // puller for all its predictors, blaze/blaze/api/cpp_api/predictor_manager_impl.cc)
      static std::mutex mu;
      static std::map<std::string, std::shared_ptr<blaze::store::SparsePuller>> loaded;
      std::lock_guard<std::mutex> lock(mu);
      std::shared_ptr<blaze::store::SparsePuller>& puller = loaded[qed_file];
      if (!puller) {
        puller.reset(blaze::store::SparsePullerCreationRegisterer::Get()->CreateSparsePuller("qed_sparse_puller"));
        if (!puller) { g_refnet_error = "qed_sparse_puller is not registered"; return nullptr; }
        if (puller->Load(qed_file) != blaze::store::kOK) {
          puller.reset();
          g_refnet_error = "QED file did not load";
          return nullptr;
        }
      }
      r->ws.SetSparsePuller(puller);
    }
    r->net = r->ws.CreateNet(net_file);
    if (!r->net) { g_refnet_error = "CreateNet returned null"; return nullptr; }
  } catch (const std::exception& e) {
    g_refnet_error = e.what();
    return nullptr;
  }
  return r.release();
}

void refnet_destroy(void* h) { delete reinterpret_cast<RefNet*>(h); }

// Reshape + copy, as PredictorImpl::ReshapeInput / Feed do for a CPU blob.
int refnet_feed(void* h, const char* name, const int64_t* shape, int ndim, const void* data, size_t bytes) {
  RefNet* r = reinterpret_cast<RefNet*>(h);
  try {
    blaze::Blob* b = r->net->external_input_blob(name);
    if (!b) { g_refnet_error = std::string("no external input ") + name; return -1; }
    std::vector<size_t> s(shape, shape + ndim);
    b->Reshape(s);
    const size_t need = b->size() * blaze::DataTypeSize(b->data_type());
    if (need != bytes) { g_refnet_error = std::string("feed of ") + name + ": byte count differs"; return -2; }
    if (bytes) memcpy(b->as<char>(), data, bytes);
  } catch (const std::exception& e) {
    g_refnet_error = e.what();
    return -3;
  }
  return 0;
}

int refnet_run(void* h) {
  RefNet* r = reinterpret_cast<RefNet*>(h);
  try {
    return r->net->Run() ? 0 : -1;
  } catch (const std::exception& e) {
    g_refnet_error = e.what();
    return -3;
  }
}

// shape[8], returns the data type (blaze DataType numbering) or a negative error; copies min(bytes, cap)
int refnet_output(void* h, const char* name, int64_t* shape, int* ndim, void* data, size_t cap, size_t* bytes) {
  RefNet* r = reinterpret_cast<RefNet*>(h);
  try {
    blaze::Blob* b = r->net->external_output_blob(name);
    if (!b) { g_refnet_error = std::string("no external output ") + name; return -1; }
    const auto& s = b->shape();
    *ndim = (int)s.size();
    for (size_t i = 0; i < s.size() && i < 8; ++i) shape[i] = (int64_t)s[i];
    *bytes = b->size() * blaze::DataTypeSize(b->data_type());
    if (data && cap) memcpy(data, b->as<char>(), *bytes < cap ? *bytes : cap);
    return (int)b->data_type();
  } catch (const std::exception& e) {
    g_refnet_error = e.what();
    return -3;
  }
}

}  // extern "C"
