// Error plumbing shared by every entry point of the C ABI.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/flagtree_b200.h"

namespace ftb {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return FTB_OK;
  set_last_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
  return FTB_ERR_CUDA;
}

}  // namespace ftb

extern "C" FTB_API int ftb_abi_version(void) { return 1; }
extern "C" FTB_API const char* ftb_last_error_string(void) { return ftb::g_last_error; }
// Size of the argument structs as the library was compiled: bindings compare it with their mirror.
extern "C" FTB_API int ftb_sizeof_sparse_mla_args(void) { return static_cast<int>(sizeof(ftb_sparse_mla_args)); }
extern "C" FTB_API int ftb_sizeof_gemm_args(void) { return static_cast<int>(sizeof(ftb_gemm_args)); }
extern "C" FTB_API int ftb_sizeof_gemm_fp8_args(void) { return static_cast<int>(sizeof(ftb_gemm_fp8_args)); }
extern "C" FTB_API int ftb_sizeof_sparse_mla_merge_args(void) { return static_cast<int>(sizeof(ftb_sparse_mla_merge_args)); }
extern "C" FTB_API int ftb_sizeof_kv_cache_write_args(void) { return static_cast<int>(sizeof(ftb_kv_cache_write_args)); }
extern "C" FTB_API int ftb_sizeof_topk_args(void) { return static_cast<int>(sizeof(ftb_topk_args)); }
