// FusedScaledDotProductAttention plan: validation (the checks of buildSDPANode,
// internal/gobackend/fusedops/sdpa.go:98-210 of the reference) and kernel selection.
#include "common.cuh"

namespace cb {

struct SdpaParams;
int sdpa_fill_params(const cb_sdpa_desc& d, SdpaParams* p);
int sdpa_generic_plan(cb_plan* p);
bool sdpa_tile_supports(const cb_sdpa_desc& d);
int sdpa_tile_plan(cb_plan* p);
int sdpa_tile_launch(const cb_plan* p, const void* const* in, void* const* out, cudaStream_t s);
int sdpa_generic_launch(const cb_plan* p, const void* const* in, void* const* out, cudaStream_t s);
bool sdpa_flash_supports(const cb_sdpa_desc& d, std::string* why);
int sdpa_flash_plan(cb_plan* p);
int sdpa_flash_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
bool sdpa_decode_supports(const cb_sdpa_desc& d, std::string* why);
int sdpa_decode_plan(cb_plan* p);
int sdpa_decode_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);
int sdpa_validate_operands(const cb_sdpa_desc& d);

int sdpa_plan(cb_plan* p) {
  cb_sdpa_desc& d = p->sdpa;
  const char* op = "FusedScaledDotProductAttention";
  if (d.dtype == CB_F8E4M3FN || d.dtype == CB_F8E5M2)
    return fail(CB_ERR_NOT_IMPLEMENTED, "%s: float8 input dtype %s is not implemented", op, dtype_name(d.dtype));
  if (d.dtype != CB_F32 && d.dtype != CB_F64 && d.dtype != CB_BF16 && d.dtype != CB_F16)
    return fail(CB_ERR_INVALID_ARG, "%s: unsupported dtype %s", op, dtype_name(d.dtype));
  if (d.B < 0 || d.S < 0 || d.Skv < 0 || d.D < 0) return fail(CB_ERR_INVALID_ARG, "%s: negative dimension", op);
  if (d.Hq <= 0 || d.Hkv <= 0 || d.Hq % d.Hkv != 0)
    return fail(CB_ERR_INVALID_ARG, "%s: numHeads (%lld) must be positive and divisible by numKVHeads (%lld)", op,
                (long long)d.Hq, (long long)d.Hkv);
  if (d.layout != CB_LAYOUT_BHSD && d.layout != CB_LAYOUT_BSHD) return fail(CB_ERR_INVALID_ARG, "%s: unknown axes layout %d", op, d.layout);
  if (d.mask_kind < CB_MASK_NONE || d.mask_kind > CB_MASK_ADDITIVE) return fail(CB_ERR_INVALID_ARG, "%s: unknown mask kind", op);
  CB_TRY(sdpa_validate_operands(d));
  p->n_inputs = 3 + (d.mask_kind != CB_MASK_NONE ? 1 : 0) + (d.has_seq_lens ? 2 : 0) + (d.bias_rank > 0 ? 1 : 0);
  p->n_outputs = 1;
  int variant = d.variant;
  std::string why;
  const bool flash_ok = sdpa_flash_supports(d, &why);
  std::string why_decode;
  const bool decode_ok = sdpa_decode_supports(d, &why_decode);
  // long query tiles go to the tensor-core kernel, a few query tokens over a long cache to the streaming kernel
  // everything else with at least half a tile of query rows to the tiled CUDA-core kernel, the rest to the row kernel
  if (variant == CB_SDPA_AUTO)
    variant = flash_ok ? CB_SDPA_FLASH : (decode_ok ? CB_SDPA_DECODE : (sdpa_tile_supports(d) ? CB_SDPA_TILE : CB_SDPA_GENERIC));
  if (variant == CB_SDPA_TILE) {
    if (!sdpa_tile_supports(d)) return fail(CB_ERR_NOT_IMPLEMENTED, "%s tiled kernel: float32 / bfloat16 / float16, head_dim 32, 64 or 128, at least 16 query rows", op);
    p->variant = variant;
    return sdpa_tile_plan(p);
  }
  if (variant == CB_SDPA_DECODE) {
    if (!decode_ok) return fail(CB_ERR_NOT_IMPLEMENTED, "%s decode kernel: %s", op, why_decode.c_str());
    p->variant = variant;
    return sdpa_decode_plan(p);
  }
  if (variant == CB_SDPA_FLASH) {
    if (!flash_ok) return fail(CB_ERR_NOT_IMPLEMENTED, "%s flash kernel: %s", op, why.c_str());
    p->variant = variant;
    return sdpa_flash_plan(p);
  }
  p->variant = CB_SDPA_GENERIC;
  return sdpa_generic_plan(p);
}

int sdpa_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  if (p->variant == CB_SDPA_FLASH) return sdpa_flash_launch(p, in, out, ws, s);
  if (p->variant == CB_SDPA_DECODE) return sdpa_decode_launch(p, in, out, ws, s);
  if (p->variant == CB_SDPA_TILE) return sdpa_tile_launch(p, in, out, s);
  return sdpa_generic_launch(p, in, out, s);
}

}  // namespace cb
