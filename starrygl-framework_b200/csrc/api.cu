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

// ---------------------------------------------------------------------------------------------------------------
// CUDA-graph helpers: capture a sequence of this library's (asynchronous) calls once, replay it with one launch.
// ---------------------------------------------------------------------------------------------------------------
extern "C" int sgl_graph_capture_begin(void* stream) {
  SGL_CUDA_CHECK(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
  return SGL_OK;
}

extern "C" int sgl_graph_capture_end(void* stream, void** out_exec) {
  SGL_REQUIRE(out_exec, SGL_ERR_ARG, "graph_capture_end: out_exec is null");
  cudaGraph_t graph = nullptr;
  SGL_CUDA_CHECK(cudaStreamEndCapture((cudaStream_t)stream, &graph));
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    sgl::set_error("cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
    return SGL_ERR_CUDA;
  }
  *out_exec = exec;
  return SGL_OK;
}

extern "C" int sgl_graph_launch(void* exec, const void* copy_src, void* copy_dst, size_t copy_bytes, void* stream) {
  SGL_REQUIRE(exec, SGL_ERR_ARG, "graph_launch: exec is null");
  if (copy_bytes) SGL_CUDA_CHECK(cudaMemcpyAsync(copy_dst, copy_src, copy_bytes, cudaMemcpyDefault, (cudaStream_t)stream));
  SGL_CUDA_CHECK(cudaGraphLaunch((cudaGraphExec_t)exec, (cudaStream_t)stream));
  return SGL_OK;
}

extern "C" int sgl_graph_destroy(void* exec) {
  if (exec) SGL_CUDA_CHECK(cudaGraphExecDestroy((cudaGraphExec_t)exec));
  return SGL_OK;
}
