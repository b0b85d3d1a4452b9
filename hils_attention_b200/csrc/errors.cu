// Error text of the C ABI (one buffer per host thread) and library identification.
#include <stdarg.h>

#include "common.cuh"

namespace hils {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
  return HILS_ERR_CUDA;
}

}  // namespace hils

namespace hils {
int take_status_sparse_tc();
int take_status_swa_tc();
int take_status_sparse_cm();
int take_status_topk_tc();
int take_status_logz_tc();
int take_status_paged();
}  // namespace hils

extern "C" int hils_version(void) { return 100; }

// Device-side error words written by kernels whose bounded waits expired (0 = none).  Reading them
// synchronises the device and clears them.
extern "C" int hils_take_device_status(void) {
  const int a = hils::take_status_sparse_tc();
  const int b = hils::take_status_swa_tc();
  const int c = hils::take_status_sparse_cm();
  const int d = hils::take_status_topk_tc();
  const int e = hils::take_status_logz_tc();
  const int f = hils::take_status_paged();
  if (a < 0 || b < 0 || c < 0 || d < 0 || e < 0 || f < 0) return -1;
  return a != 0 ? a : (b != 0 ? b : (c != 0 ? c : (d != 0 ? d : (e != 0 ? e : f))));
}
extern "C" const char* hils_last_error(void) { return hils::g_err; }
