// Library runtime shared by every kernel unit: thread-local error message, device query, programmatic-dependent-launch
// switches, version string.  Kept apart from the dispatchers so that a library linked from a subset of the units loads.
#include <stdarg.h>
#include <stdlib.h>

#include "common.cuh"

namespace b200p {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return B200P_ERR_CUDA;
}

// 0 off, 1 every kernel, 2 only the tensor-path GEMM (B200P_PDL overrides the default at load time)
static int g_pdl = [] { const char* e = getenv("B200P_PDL"); return e ? atoi(e) : 2; }();
static int g_sm_count = -1;
static int g_cc_major = -1;

static int query_device() {
  if (g_cc_major >= 0) return B200P_OK;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  cudaDeviceProp p;
  e = cudaGetDeviceProperties(&p, dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceProperties");
  g_cc_major = p.major;
  g_sm_count = p.multiProcessorCount;
  return B200P_OK;
}

// per-class PDL mask for the non-GEMM kernels (see common.cuh); B200P_PDL=1 means every class
static int g_pdl_mask = [] { const char* e = getenv("B200P_PDL_MASK"); return e ? atoi(e) : 0; }();
static thread_local int g_pdl_class = 0;
void pdl_set_class(int cls) { g_pdl_class = cls; }
bool pdl_enabled() { return g_pdl == 1 || (g_pdl_mask & g_pdl_class) != 0; }
bool pdl_enabled_gemm() { return g_pdl != 0; }

int sm_count() {
  query_device();
  return g_sm_count > 0 ? g_sm_count : 148;
}

}  // namespace b200p

using namespace b200p;

// 0.3: dense GEMM, ragged batches, gated delta rule and latent attention entry points added to the 0.2 ABI
extern "C" const char* b200p_version(void) { return "b200parallm 0.3 (sm_100a)"; }
extern "C" const char* b200p_last_error(void) { return g_err; }

extern "C" int b200p_arch_check(void) {
  int rc = query_device();
  if (rc) return rc;
  B200P_REQUIRE(g_cc_major == 10, B200P_ERR_ARCH, "device compute capability %d.x is not sm_100", g_cc_major);
  return B200P_OK;
}

extern "C" int b200p_sm_count(void) {
  int rc = query_device();
  if (rc) return rc;
  return g_sm_count;
}

extern "C" int b200p_set_pdl(int enabled) {
  g_pdl = enabled;
  return B200P_OK;
}

