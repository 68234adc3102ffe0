// Error plumbing of the C ABI: a thread-local message buffer behind sgl_last_error().
#include "common.cuh"

namespace sgl {
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
}  // namespace sgl

extern "C" const char* sgl_last_error(void) { return sgl::g_err; }

extern "C" const char* sgl_build_info(void) { return "libsgl_b200 0.1 (sm_100a, CUDA " SGL_STR(CUDART_VERSION) ")"; }
