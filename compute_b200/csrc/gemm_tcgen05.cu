// tcgen05 / TMEM / TMA GEMM for DotGeneral (placeholder until the kernel lands).
#include "common.cuh"

namespace cb {

bool dot_tc_supports(const cb_dot_desc& d, std::string* why) {
  if (why) *why = "not built yet";
  return false;
}
int dot_tc_plan(cb_plan* p) { return fail(CB_ERR_NOT_IMPLEMENTED, "DotGeneral tcgen05 kernel is not built yet"); }
int dot_tc_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  return fail(CB_ERR_NOT_IMPLEMENTED, "DotGeneral tcgen05 kernel is not built yet");
}

}  // namespace cb
