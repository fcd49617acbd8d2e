// Flash-style tensor-core attention (placeholder until the kernel lands).
#include "common.cuh"

namespace cb {

bool sdpa_flash_supports(const cb_sdpa_desc& d, std::string* why) {
  if (why) *why = "not built yet";
  return false;
}
int sdpa_flash_plan(cb_plan* p) { return fail(CB_ERR_NOT_IMPLEMENTED, "flash attention kernel is not built yet"); }
int sdpa_flash_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  return fail(CB_ERR_NOT_IMPLEMENTED, "flash attention kernel is not built yet");
}

}  // namespace cb
