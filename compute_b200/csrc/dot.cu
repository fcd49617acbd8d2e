// DotGeneral plan: validation and kernel selection by shape and dtype
// (the role of FindRegisteredImplementation / execDotGeneral in the reference:
// internal/gobackend/dot/registration.go:101-118, dot.go:375-393).
#include "common.cuh"

namespace cb {

bool dot_generic_supports(int in_dtype, int out_dtype);
int dot_generic_launch(const cb_dot_desc& d, const void* const* in, void* const* out, cudaStream_t s);
bool dot_generic_supports_epilogue(int in_dtype);
bool dot_tc_supports(const cb_dot_desc& d, std::string* why);
int dot_tc_plan(cb_plan* p);
int dot_tc_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s);

int dot_plan(cb_plan* p) {
  cb_dot_desc& d = p->dot;
  if (d.B < 0 || d.M < 0 || d.N < 0 || d.K < 0) return fail(CB_ERR_INVALID_ARG, "DotGeneral: negative dimension");
  const int od = d.out_dtype ? d.out_dtype : d.in_dtype;
  if (d.activation < CB_ACT_NONE || d.activation > CB_ACT_TANH) return fail(CB_ERR_INVALID_ARG, "FusedDense: unknown activation %d", d.activation);
  const bool dense = d.has_bias || d.activation != CB_ACT_NONE;
  if (dense && !dot_generic_supports_epilogue(d.in_dtype))
    return fail(CB_ERR_NOT_IMPLEMENTED, "FusedDense: dtype %s", dtype_name(d.in_dtype));
  p->n_inputs = 2 + (d.has_bias ? 1 : 0);
  p->n_outputs = 1;
  int variant = d.variant;
  std::string why;
  const bool tc_ok = dot_tc_supports(d, &why);
  if (variant == CB_DOT_AUTO) variant = tc_ok ? CB_DOT_TCGEN05 : CB_DOT_GENERIC;
  if (variant == CB_DOT_TCGEN05 || variant == CB_DOT_TCGEN05_EXACT) {
    if (!tc_ok) return fail(CB_ERR_NOT_IMPLEMENTED, "DotGeneral tcgen05 kernel: %s", why.c_str());
    p->variant = variant;
    return dot_tc_plan(p);
  }
  if (!dot_generic_supports(d.in_dtype, od))
    return fail(CB_ERR_NOT_IMPLEMENTED, "no DotGeneral implementation found for layout=%s and dtypes=%s,%s",
                d.rhs_transposed ? "Transposed" : "NonTransposed", dtype_name(d.in_dtype), dtype_name(od));
  p->variant = CB_DOT_GENERIC;
  p->blocks = (int)(((d.N + 63) / 64) * ((d.M + 63) / 64) * d.B);
  p->threads = 256;
  p->name = std::string("dot_generic_") + dtype_name(d.in_dtype) + "_" + dtype_name(od) + (d.rhs_transposed ? "_nt" : "_nn") + (dense ? "_dense" : "");
  return CB_OK;
}

int dot_launch(const cb_plan* p, const void* const* in, void* const* out, void* ws, cudaStream_t s) {
  if (p->variant == CB_DOT_TCGEN05 || p->variant == CB_DOT_TCGEN05_EXACT) return dot_tc_launch(p, in, out, ws, s);
  return dot_generic_launch(p->dot, in, out, s);
}

}  // namespace cb
