/*
 * CPU oracle for the cudabackend hot path — TEST INFRASTRUCTURE ONLY.
 * See oracle.h for what each function restates and how parity is pinned.
 * Nothing here is part of the shipped library.
 */
#include "oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ */
/* half-precision scalar types                                        */
/* ------------------------------------------------------------------ */

static inline uint32_t f32_bits(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float bits_f32(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

/* bfloat16.go:30-39: NaN/Inf keep their top 16 bits; everything else gets
 * 0x7FFF + lsb added before the shift (round to nearest, ties to even). */
uint16_t orc_bf16_from_f32(float x) {
  uint32_t b = f32_bits(x);
  if ((b & 0x7F800000u) == 0x7F800000u) return (uint16_t)(b >> 16);
  b += 0x7FFFu + ((b >> 16) & 1u);
  return (uint16_t)(b >> 16);
}
float orc_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

void orc_bf16_from_f32_n(const float* in, uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = orc_bf16_from_f32(in[i]);
}
void orc_bf16_to_f32_n(const uint16_t* in, float* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = orc_bf16_to_f32(in[i]);
}

/* float16.go:103-165: IEEE binary16 with round-to-nearest-even, overflow to
 * infinity, gradual underflow, flush below 2^-25. */
uint16_t orc_f16_from_f32(float x) {
  uint32_t b = f32_bits(x);
  uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
  int e = (int)((b >> 23) & 0xFFu);
  uint32_t man = b & 0x007FFFFFu;
  if (e == 0xFF) {
    if (man == 0) return (uint16_t)(sign | 0x7C00u);
    return (uint16_t)(sign | 0x7C00u | (uint16_t)(man >> 13) | 1u);
  }
  e -= 127;
  if (e > 15) return (uint16_t)(sign | 0x7C00u);
  if (e < -24) return sign;
  if (e < -14) {
    man |= 0x00800000u;
    unsigned shift = (unsigned)(14 - e);
    man >>= (shift - 1);
    man = (man & 1u) ? (man >> 1) + 1u : (man >> 1);
    return (uint16_t)(sign | (uint16_t)man);
  }
  uint16_t re = (uint16_t)((e + 15) << 10);
  uint16_t rm = (uint16_t)(man >> 13);
  if (man & 0x1000u) {
    if ((man & 0x0FFFu) != 0 || (rm & 1u)) {
      rm++;
      if (rm & 0x0400u) {
        rm = 0;
        re = (uint16_t)(re + 0x0400u);
        if (re >= 0x7C00u) return (uint16_t)(sign | 0x7C00u);
      }
    }
  }
  return (uint16_t)(sign | re | rm);
}

float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  int e = (h & 0x7C00u) >> 10;
  uint32_t man = h & 0x03FFu;
  if (e == 0x1F) return bits_f32(sign | 0x7F800000u | (man << 13));
  if (e == 0) {
    if (man == 0) return bits_f32(sign);
    while ((man & 0x0400u) == 0) { man <<= 1; e--; }
    e++;
    man &= 0x03FFu;
  }
  return bits_f32(sign | ((uint32_t)(e - 15 + 127) << 23) | (man << 13));
}

int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------ */
/* activations (dense.go:176-205, gelu.go:113-118)                    */
/* ------------------------------------------------------------------ */

void orc_activation_f32(float* d, size_t n, int activation) {
  switch (activation) {
    case ORC_ACT_NONE: break;
    case ORC_ACT_GELU: {
      const float inv_sqrt2 = (float)(1.0 / sqrt(2.0));
      for (size_t i = 0; i < n; i++) {
        float x = d[i];
        float h = x * 0.5f;
        d[i] = h * (1.0f + (float)erf((double)(x * inv_sqrt2)));
      }
      break;
    }
    case ORC_ACT_RELU:
      for (size_t i = 0; i < n; i++) if (d[i] < 0) d[i] = 0;
      break;
    case ORC_ACT_SILU:
      for (size_t i = 0; i < n; i++) {
        float x = d[i];
        d[i] = x / (1.0f + (float)exp((double)(-x)));
      }
      break;
    case ORC_ACT_HARDSWISH: {
      const float sixth = (float)(1.0 / 6.0);
      for (size_t i = 0; i < n; i++) {
        float x = d[i];
        float g = x * sixth + 0.5f;
        if (g < 0.0f) g = 0.0f;
        if (g > 1.0f) g = 1.0f;
        d[i] = x * g;
      }
      break;
    }
    case ORC_ACT_TANH:
      for (size_t i = 0; i < n; i++) d[i] = (float)tanh((double)d[i]);
      break;
    default: break;
  }
}

/* ------------------------------------------------------------------ */
/* fused quantized dense, Linear scheme, int8/uint8 weights           */
/* ------------------------------------------------------------------ */

/* One reference work unit: row m, columns [n0,n1)  (quantizeddense.go:617-649).
 * Order of operations per element: bias first, then k ascending,
 * out += (x * float(w)) * s            (symmetric)
 * out += x * (float(w) * s + zp)       (with zero points)
 * every operation rounded to f32 on its own. */
static void qdense_unit(const float* x, const int8_t* ws, const uint8_t* wu,
                        const float* scales, const float* zps, const float* bias,
                        float* out, int64_t m, int64_t n0, int64_t n1,
                        int64_t K, int64_t N, int64_t bs, int64_t nblk) {
  float* o = out + m * N;
  for (int64_t n = n0; n < n1; n++) o[n] = bias ? bias[n] : 0.0f;
  for (int64_t k = 0; k < K; k++) {
    const float xv = x[m * K + k];
    const float* srow = scales + k * nblk;
    const float* zrow = zps ? zps + k * nblk : NULL;
    int64_t blk = n0 / bs;
    int64_t next = (blk + 1) * bs;
    for (int64_t n = n0; n < n1; n++) {
      if (n >= next) { blk++; next += bs; }
      const float wf = ws ? (float)ws[k * N + n] : (float)wu[k * N + n];
      if (zrow) {
        float dq = wf * srow[blk];
        dq = dq + zrow[blk];
        float p = xv * dq;
        o[n] = o[n] + p;
      } else {
        float p = xv * wf;
        p = p * srow[blk];
        o[n] = o[n] + p;
      }
    }
  }
}

void orc_qdense_linear(const float* x, const void* w, int w_unsigned,
                       const float* scales, const float* zero_points,
                       const float* bias, float* out,
                       int64_t M, int64_t K, int64_t N, int64_t block_size,
                       int activation, int threads) {
  const int8_t* ws = w_unsigned ? NULL : (const int8_t*)w;
  const uint8_t* wu = w_unsigned ? (const uint8_t*)w : NULL;
  const int64_t nblk = (N + block_size - 1) / block_size;
  const int64_t min_chunk = 4096; /* geluMinParallelizeChunk, gelu.go:90 */
  if (threads <= 1 || M * K * N <= min_chunk) {
    for (int64_t m = 0; m < M; m++)
      qdense_unit(x, ws, wu, scales, zero_points, bias, out, m, 0, N, K, N, block_size, nblk);
  } else if (M > 1) {
#pragma omp parallel for num_threads(threads) schedule(dynamic, 1)
    for (int64_t m = 0; m < M; m++)
      qdense_unit(x, ws, wu, scales, zero_points, bias, out, m, 0, N, K, N, block_size, nblk);
  } else {
    int64_t tile = min_chunk / K;
    if (tile < 1) tile = 1;
    const int64_t ntiles = (N + tile - 1) / tile;
#pragma omp parallel for num_threads(threads) schedule(dynamic, 16)
    for (int64_t t = 0; t < ntiles; t++) {
      int64_t n0 = t * tile, n1 = n0 + tile;
      if (n1 > N) n1 = N;
      qdense_unit(x, ws, wu, scales, zero_points, bias, out, 0, n0, n1, K, N, block_size, nblk);
    }
  }
  /* the reference applies the activation single-threaded over the whole output */
  orc_activation_f32(out, (size_t)(M * N), activation);
}

/* ------------------------------------------------------------------ */
/* packed 4-bit weights and the NF4 scheme                            */
/* ------------------------------------------------------------------ */

/* Int4 / Uint4 storage: two elements per byte over the flat element order, the low nibble first;
 * Int4 nibbles 8..15 mean -8..-1 (internal/gobackend/ops/convertdtype.go:199-226).  The reference
 * unpacks such weights to one int8 / uint8 per element before the dense op
 * (fusedops/quantizeddense.go:420-450), so the Linear scheme on packed weights is
 * orc_unpack_* followed by orc_qdense_linear. */
void orc_unpack_int4(const uint8_t* packed, int8_t* dst, size_t n_bytes) {
  for (size_t i = 0; i < n_bytes; i++) {
    int lo = packed[i] & 0x0F;
    if (lo >= 8) lo -= 16;
    const int hi = (int8_t)packed[i] >> 4; /* arithmetic shift keeps the sign */
    dst[2 * i] = (int8_t)lo;
    dst[2 * i + 1] = (int8_t)hi;
  }
}
void orc_unpack_uint4(const uint8_t* packed, uint8_t* dst, size_t n_bytes) {
  for (size_t i = 0; i < n_bytes; i++) {
    dst[2 * i] = packed[i] & 0x0F;
    dst[2 * i + 1] = packed[i] >> 4;
  }
}

/* The 16 NormalFloat4 values of QLoRA (Dettmers et al. 2023, appendix E), as float32; the
 * reference holds the same table (fused_ops.go:114-121). */
static const float orc_nf4_table[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
const float* orc_nf4_values(void) { return orc_nf4_table; }

/* NF4 scheme (quantizeddense.go:586-609): the low four bits of every (unpacked) weight index the
 * table; per element, k ascending:  out += (x * table[w & 15]) * s, each operation rounded to f32;
 * bias first; no zero points.  `w` holds one byte per element (int8 or uint8: only the low nibble
 * is used). */
static void qdense_nf4_unit(const float* x, const uint8_t* w, const float* scales, const float* bias,
                            float* out, int64_t m, int64_t n0, int64_t n1,
                            int64_t K, int64_t N, int64_t bs, int64_t nblk) {
  float* o = out + m * N;
  for (int64_t n = n0; n < n1; n++) o[n] = bias ? bias[n] : 0.0f;
  for (int64_t k = 0; k < K; k++) {
    const float xv = x[m * K + k];
    const float* srow = scales + k * nblk;
    int64_t blk = n0 / bs;
    int64_t next = (blk + 1) * bs;
    for (int64_t n = n0; n < n1; n++) {
      if (n >= next) { blk++; next += bs; }
      float p = xv * orc_nf4_table[w[k * N + n] & 0x0F];
      p = p * srow[blk];
      o[n] = o[n] + p;
    }
  }
}

void orc_qdense_nf4(const float* x, const void* w, const float* scales, const float* bias, float* out,
                    int64_t M, int64_t K, int64_t N, int64_t block_size, int activation, int threads) {
  const int64_t nblk = (N + block_size - 1) / block_size;
  (void)threads; /* the work split does not change any element's arithmetic */
  for (int64_t m = 0; m < M; m++)
    qdense_nf4_unit(x, (const uint8_t*)w, scales, bias, out, m, 0, N, K, N, block_size, nblk);
  orc_activation_f32(out, (size_t)(M * N), activation);
}

/* ------------------------------------------------------------------ */
/* GGML block formats Q4_0, Q8_0, IQ4_NL, Q4_K, Q6_K                  */
/* ------------------------------------------------------------------ */

/* Type codes of compute.GGMLQuantType (fused_ops.go:132-145); values and bytes per block (:148-176). */
enum { ORC_GGML_Q4_0 = 0, ORC_GGML_Q8_0 = 1, ORC_GGML_IQ4_NL = 2, ORC_GGML_Q4_K = 5, ORC_GGML_Q6_K = 7 };
int orc_ggml_values_per_block(int t) { return (t == ORC_GGML_Q4_0 || t == ORC_GGML_Q8_0 || t == ORC_GGML_IQ4_NL) ? 32 : (t == ORC_GGML_Q4_K || t == ORC_GGML_Q6_K) ? 256 : 0; }
int orc_ggml_bytes_per_block(int t) {
  switch (t) { case ORC_GGML_Q4_0: case ORC_GGML_IQ4_NL: return 18; case ORC_GGML_Q8_0: return 34; case ORC_GGML_Q4_K: return 144; case ORC_GGML_Q6_K: return 210; default: return 0; }
}
/* compute.IQ4NLLookupTable (fused_ops.go:127-130) */
static const float orc_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

/* getScaleMinK4 (quantizeddense_ggml.go:219-228): the 6-bit scale and min of sub-block j from the 12 packed bytes */
static void orc_scale_min_k4(int j, const uint8_t* sc, uint8_t* scale, uint8_t* min) {
  if (j < 4) { *scale = sc[j] & 63; *min = sc[j + 4] & 63; }
  else { *scale = (uint8_t)((sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4)); *min = (uint8_t)((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)); }
}

/* quantizeddense_ggml.go:157-302.  A row is K / values_per_block blocks; fp16 fields are little-endian.
 *   Q8_0 (34 bytes): d, 32 int8: value i = d * q[i].
 *   Q4_0 (18 bytes): d, 16 bytes: value i = d * (low nibble of q[i] - 8), value 16 + i = d * (high nibble - 8).
 *   IQ4_NL: as Q4_0 with table[nibble] in place of nibble - 8.
 *   Q4_K (144 bytes): d, dmin, 12 bytes of 6-bit scales / mins, 128 nibble bytes; 4 chunks of 64 values: the low nibbles
 *     of 32 bytes with (scale, min) 2c, then their high nibbles with 2c + 1; value = (d * scale) * nibble - dmin * min.
 *   Q6_K (210 bytes): ql[128], qh[64], int8 scales[16], d; two halves of 128 values; value = (d * scale) * (q - 32)
 *     with q = 4 low bits from ql, 2 high bits from qh. */
void orc_ggml_dequant_row(const uint8_t* data, float* out, int64_t K, int ggml_type) {
  const int vpb = orc_ggml_values_per_block(ggml_type), bb = orc_ggml_bytes_per_block(ggml_type);
  if (!vpb) return;
  const int64_t nblocks = K / vpb;
  for (int64_t b = 0; b < nblocks; b++) {
    const uint8_t* blk = data + b * bb;
    float* o = out + b * vpb;
    if (ggml_type == ORC_GGML_Q8_0) {
      const float d = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
      for (int i = 0; i < 32; i++) o[i] = d * (float)(int8_t)blk[2 + i];
    } else if (ggml_type == ORC_GGML_Q4_0 || ggml_type == ORC_GGML_IQ4_NL) {
      const float d = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
      const uint8_t* qs = blk + 2;
      for (int i = 0; i < 16; i++) {
        if (ggml_type == ORC_GGML_Q4_0) {
          o[i] = d * (float)((int)(qs[i] & 0x0F) - 8);
          o[16 + i] = d * (float)((int)(qs[i] >> 4) - 8);
        } else {
          o[i] = d * orc_iq4nl[qs[i] & 0x0F];
          o[16 + i] = d * orc_iq4nl[qs[i] >> 4];
        }
      }
    } else if (ggml_type == ORC_GGML_Q4_K) {
      const float d = orc_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
      const float dmin = orc_f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
      const uint8_t* scales = blk + 4;
      const uint8_t* qs = blk + 16;
      int idx = 0;
      for (int chunk = 0; chunk < 4; chunk++) {
        uint8_t sc1, m1, sc2, m2;
        orc_scale_min_k4(2 * chunk, scales, &sc1, &m1);
        orc_scale_min_k4(2 * chunk + 1, scales, &sc2, &m2);
        const float d1 = d * (float)sc1, min1 = dmin * (float)m1;
        const float d2 = d * (float)sc2, min2 = dmin * (float)m2;
        for (int l = 0; l < 32; l++) { const float t = d1 * (float)(qs[chunk * 32 + l] & 0xF); o[idx++] = t - min1; }
        for (int l = 0; l < 32; l++) { const float t = d2 * (float)(qs[chunk * 32 + l] >> 4); o[idx++] = t - min2; }
      }
    } else {  /* Q6_K */
      const uint8_t* ql = blk;
      const uint8_t* qh = blk + 128;
      const int8_t* sc = (const int8_t*)(blk + 192);
      const float d = orc_f16_to_f32((uint16_t)(blk[208] | (blk[209] << 8)));
      for (int half = 0; half < 2; half++) {
        for (int l = 0; l < 32; l++) {
          const int is = l / 16;
          const int q1 = (int)(int8_t)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
          const int q2 = (int)(int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
          const int q3 = (int)(int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
          const int q4 = (int)(int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
          float t;
          t = d * (float)sc[is];     o[l]      = t * (float)q1;
          t = d * (float)sc[is + 2]; o[l + 32] = t * (float)q2;
          t = d * (float)sc[is + 4]; o[l + 64] = t * (float)q3;
          t = d * (float)sc[is + 6]; o[l + 96] = t * (float)q4;
        }
        o += 128; ql += 64; qh += 32; sc += 8;
      }
    }
  }
}

/* quantizeddense_ggml.go:98-131: per output, the row is dequantised, dot = sum_k x[k] * w[k] in one
 * float, k ascending; then + bias[n]; the activation over the whole output last (:89). */
void orc_qdense_ggml(const float* x, const uint8_t* w, const float* bias, float* out,
                     int64_t M, int64_t K, int64_t N, int ggml_type, int activation) {
  const int vpb = orc_ggml_values_per_block(ggml_type);
  const int64_t bytes_per_row = vpb ? K / vpb * orc_ggml_bytes_per_block(ggml_type) : 0;
  float* row = (float*)malloc((size_t)(K > 0 ? K : 1) * sizeof(float));
  for (int64_t n = 0; n < N; n++) {
    orc_ggml_dequant_row(w + n * bytes_per_row, row, K, ggml_type);
    for (int64_t m = 0; m < M; m++) {
      float dot = 0.0f;
      for (int64_t k = 0; k < K; k++) { const float p = x[m * K + k] * row[k]; dot = dot + p; }
      out[m * N + n] = dot;
      if (bias) out[m * N + n] += bias[n];
    }
  }
  free(row);
  orc_activation_f32(out, (size_t)(M * N), activation);
}

/* execQuantizedEmbeddingLookup (quantizeddense.go:455-499): out[i, :] = the dequantised row indices[i] of the table;
 * returns the position of the first index outside [0, vocab) (the reference returns an error there), or -1. */
int64_t orc_embedding_lookup(const uint8_t* table, const int64_t* indices, float* out, int64_t vocab, int64_t n_indices,
                             int64_t K, int ggml_type) {
  const int vpb = orc_ggml_values_per_block(ggml_type);
  const int64_t bytes_per_row = vpb ? K / vpb * orc_ggml_bytes_per_block(ggml_type) : 0;
  for (int64_t i = 0; i < n_indices; i++) {
    if (indices[i] < 0 || indices[i] >= vocab) return i;
    orc_ggml_dequant_row(table + indices[i] * bytes_per_row, out + i * K, K, ggml_type);
  }
  return -1;
}

/* ------------------------------------------------------------------ */
/* FusedSoftmax, FusedGelu, FusedLayerNorm                            */
/* ------------------------------------------------------------------ */

/* softmax.go:83-118: x viewed as [outer, L, inner]; per line: max, exp(x - max) summed in index
 * order, scaled by 1 / sum.  (The reference's float32 path uses its fastmath.Exp32 approximation;
 * this restatement uses libm, and comparisons carry a tolerance.) */
#define ORC_SOFTMAX(NAME, T, EXPF)                                                          \
  void NAME(const T* x, T* y, int64_t outer, int64_t L, int64_t inner) {                    \
    for (int64_t o = 0; o < outer; o++)                                                     \
      for (int64_t in = 0; in < inner; in++) {                                              \
        const int64_t base = o * L * inner + in;                                            \
        T mx = (T)(-INFINITY);                                                              \
        for (int64_t i = 0; i < L; i++) if (x[base + i * inner] > mx) mx = x[base + i * inner]; \
        T sum = 0;                                                                          \
        for (int64_t i = 0; i < L; i++) { y[base + i * inner] = (T)EXPF(x[base + i * inner] - mx); sum += y[base + i * inner]; } \
        const T inv = (T)1 / sum;                                                           \
        for (int64_t i = 0; i < L; i++) y[base + i * inner] *= inv;                         \
      }                                                                                     \
  }
ORC_SOFTMAX(orc_softmax_f32, float, expf)
ORC_SOFTMAX(orc_softmax_f64, double, exp)

/* gelu.go:113-126: exact x/2 (1 + erf(x / sqrt 2)), or the tanh form; erf / tanh evaluated in double
 * and rounded to T, the surrounding arithmetic in T. */
void orc_gelu_f32(const float* x, float* y, size_t n, int exact) {
  const float inv_sqrt2 = (float)(1.0 / sqrt(2.0)), c = (float)sqrt(2.0 / M_PI);
  for (size_t i = 0; i < n; i++) {
    const float v = x[i];
    if (exact) y[i] = v * 0.5f * (1.0f + (float)erf((double)(v * inv_sqrt2)));
    else { const float inner = c * (v + 0.044715f * v * v * v); y[i] = v * 0.5f * (1.0f + (float)tanh((double)inner)); }
  }
}
void orc_gelu_f64(const double* x, double* y, size_t n, int exact) {
  const double inv_sqrt2 = 1.0 / sqrt(2.0), c = sqrt(2.0 / M_PI);
  for (size_t i = 0; i < n; i++) {
    const double v = x[i];
    if (exact) y[i] = v * 0.5 * (1.0 + erf(v * inv_sqrt2));
    else { const double inner = c * (v + 0.044715 * v * v * v); y[i] = v * 0.5 * (1.0 + tanh(inner)); }
  }
}

/* layernorm.go:129-168 (trailing axes): per row mean, variance of the differences (both summed in
 * index order, divided by L), invStd = T(1 / sqrt(double(var) + eps)), then gamma and beta. */
#define ORC_LAYERNORM(NAME, T)                                                              \
  void NAME(const T* x, const T* gamma, const T* beta, T* y, int64_t rows, int64_t L, double eps) { \
    for (int64_t r = 0; r < rows; r++) {                                                    \
      const T* xr = x + r * L;                                                              \
      T sum = 0;                                                                            \
      for (int64_t i = 0; i < L; i++) sum += xr[i];                                         \
      const T mean = sum / (T)L;                                                            \
      T vs = 0;                                                                             \
      for (int64_t i = 0; i < L; i++) { const T d = xr[i] - mean; vs += d * d; }            \
      const T var = vs / (T)L;                                                              \
      const T inv_std = (T)(1.0 / sqrt((double)var + eps));                                 \
      for (int64_t i = 0; i < L; i++) {                                                     \
        T v = (xr[i] - mean) * inv_std;                                                     \
        if (gamma) v *= gamma[i];                                                           \
        if (beta) v += beta[i];                                                             \
        y[r * L + i] = v;                                                                   \
      }                                                                                     \
    }                                                                                       \
  }
ORC_LAYERNORM(orc_layernorm_f32, float)
ORC_LAYERNORM(orc_layernorm_f64, double)

/* ------------------------------------------------------------------ */
/* DotGeneral                                                         */
/* ------------------------------------------------------------------ */

static int is_float_dtype(int d) { return d == ORC_F16 || d == ORC_F32 || d == ORC_F64 || d == ORC_BF16; }
static int is_half_dtype(int d) { return d == ORC_F16 || d == ORC_BF16; }
static int is_int_dtype(int d) { return d >= ORC_I8 && d <= ORC_U64; }

static size_t dtype_size(int d) {
  switch (d) {
    case ORC_BOOL: case ORC_I8: case ORC_U8: return 1;
    case ORC_I16: case ORC_U16: case ORC_F16: case ORC_BF16: return 2;
    case ORC_I32: case ORC_U32: case ORC_F32: return 4;
    case ORC_I64: case ORC_U64: case ORC_F64: return 8;
    default: return 0;
  }
}

static double load_as_double(const void* p, int d, int64_t i) {
  switch (d) {
    case ORC_F64: return ((const double*)p)[i];
    case ORC_F32: return (double)((const float*)p)[i];
    case ORC_BF16: return (double)orc_bf16_to_f32(((const uint16_t*)p)[i]);
    case ORC_F16: return (double)orc_f16_to_f32(((const uint16_t*)p)[i]);
    case ORC_I8: return (double)((const int8_t*)p)[i];
    case ORC_U8: return (double)((const uint8_t*)p)[i];
    case ORC_I16: return (double)((const int16_t*)p)[i];
    case ORC_U16: return (double)((const uint16_t*)p)[i];
    case ORC_I32: return (double)((const int32_t*)p)[i];
    case ORC_U32: return (double)((const uint32_t*)p)[i];
    case ORC_I64: return (double)((const int64_t*)p)[i];
    case ORC_U64: return (double)((const uint64_t*)p)[i];
    default: return 0.0;
  }
}

static int64_t load_as_i64(const void* p, int d, int64_t i) {
  switch (d) {
    case ORC_I8: return ((const int8_t*)p)[i];
    case ORC_U8: return ((const uint8_t*)p)[i];
    case ORC_I16: return ((const int16_t*)p)[i];
    case ORC_U16: return ((const uint16_t*)p)[i];
    case ORC_I32: return ((const int32_t*)p)[i];
    case ORC_U32: return ((const uint32_t*)p)[i];
    case ORC_I64: return ((const int64_t*)p)[i];
    case ORC_U64: return (int64_t)((const uint64_t*)p)[i];
    default: return 0;
  }
}

/* value -> value rounded to float dtype d (as a double). */
static double round_to_dtype(double v, int d) {
  switch (d) {
    case ORC_F64: return v;
    case ORC_F32: return (double)(float)v;
    case ORC_BF16: return (double)orc_bf16_to_f32(orc_bf16_from_f32((float)v));
    case ORC_F16: return (double)orc_f16_to_f32(orc_f16_from_f32((float)v));
    default: return v;
  }
}

static void store_float(void* p, int d, int64_t i, double v) {
  switch (d) {
    case ORC_F64: ((double*)p)[i] = v; break;
    case ORC_F32: ((float*)p)[i] = (float)v; break;
    case ORC_BF16: ((uint16_t*)p)[i] = orc_bf16_from_f32((float)v); break;
    case ORC_F16: ((uint16_t*)p)[i] = orc_f16_from_f32((float)v); break;
    default: break;
  }
}

static void store_int(void* p, int d, int64_t i, int64_t v) {
  switch (d) {
    case ORC_I8: ((int8_t*)p)[i] = (int8_t)v; break;
    case ORC_U8: ((uint8_t*)p)[i] = (uint8_t)v; break;
    case ORC_I16: ((int16_t*)p)[i] = (int16_t)v; break;
    case ORC_U16: ((uint16_t*)p)[i] = (uint16_t)v; break;
    case ORC_I32: ((int32_t*)p)[i] = (int32_t)v; break;
    case ORC_U32: ((uint32_t*)p)[i] = (uint32_t)v; break;
    case ORC_I64: ((int64_t*)p)[i] = v; break;
    case ORC_U64: ((uint64_t*)p)[i] = (uint64_t)v; break;
    default: break;
  }
}

/* Offsets (in elements) of every multi-index over `axes` (row-major in the
 * order the axes are listed). Returns count; *offs malloc'ed. */
static int64_t axis_offsets(const int64_t* dims, const int64_t* strides,
                            const int* axes, int n_axes, int64_t** offs) {
  int64_t count = 1;
  for (int i = 0; i < n_axes; i++) count *= dims[axes[i]];
  *offs = (int64_t*)malloc(sizeof(int64_t) * (size_t)(count > 0 ? count : 1));
  for (int64_t lin = 0; lin < count; lin++) {
    int64_t rem = lin, off = 0;
    for (int i = n_axes - 1; i >= 0; i--) {
      int64_t d = dims[axes[i]];
      off += (rem % d) * strides[axes[i]];
      rem /= d;
    }
    (*offs)[lin] = off;
  }
  return count;
}

int orc_dot_general(int in_dtype, const void* lhs, int lhs_rank, const int64_t* lhs_dims,
                    const int* lhs_contract, const int* lhs_batch,
                    const void* rhs, int rhs_rank, const int64_t* rhs_dims,
                    const int* rhs_contract, const int* rhs_batch,
                    int n_contract, int n_batch,
                    int acc_dtype, int out_dtype, void* out, int acc_f64) {
  if (lhs_rank > 16 || rhs_rank > 16 || dtype_size(in_dtype) == 0) return -1;
  if (out_dtype == 0) out_dtype = in_dtype;
  for (int i = 0; i < n_contract; i++)
    if (lhs_dims[lhs_contract[i]] != rhs_dims[rhs_contract[i]]) return -1;
  for (int i = 0; i < n_batch; i++)
    if (lhs_dims[lhs_batch[i]] != rhs_dims[rhs_batch[i]]) return -1;

  /* dtype the normalised op computes in (dot.go:207-217, :340-372) */
  int comp = in_dtype;      /* dtype inputs are (re)rounded to */
  int acc = in_dtype;       /* accumulation dtype */
  if (is_half_dtype(in_dtype)) acc = ORC_F32;
  if (acc_dtype != 0 && acc_dtype != in_dtype && acc_dtype != acc) {
    comp = acc_dtype;
    acc = is_half_dtype(acc_dtype) ? ORC_F32 : acc_dtype;
  }
  const int float_path = is_float_dtype(comp);
  if (float_path != is_float_dtype(in_dtype) && !is_int_dtype(in_dtype)) return -2;

  int64_t ls[16], rs[16];
  { int64_t s = 1; for (int i = lhs_rank - 1; i >= 0; i--) { ls[i] = s; s *= lhs_dims[i]; } }
  { int64_t s = 1; for (int i = rhs_rank - 1; i >= 0; i--) { rs[i] = s; s *= rhs_dims[i]; } }
  int lcross[16], rcross[16], nlc = 0, nrc = 0;
  for (int a = 0; a < lhs_rank; a++) {
    int used = 0;
    for (int i = 0; i < n_contract; i++) used |= (lhs_contract[i] == a);
    for (int i = 0; i < n_batch; i++) used |= (lhs_batch[i] == a);
    if (!used) lcross[nlc++] = a;
  }
  for (int a = 0; a < rhs_rank; a++) {
    int used = 0;
    for (int i = 0; i < n_contract; i++) used |= (rhs_contract[i] == a);
    for (int i = 0; i < n_batch; i++) used |= (rhs_batch[i] == a);
    if (!used) rcross[nrc++] = a;
  }
  int64_t *lb, *rb, *lc, *rc, *lk, *rk;
  const int64_t nB = axis_offsets(lhs_dims, ls, lhs_batch, n_batch, &lb);
  axis_offsets(rhs_dims, rs, rhs_batch, n_batch, &rb);
  const int64_t nM = axis_offsets(lhs_dims, ls, lcross, nlc, &lc);
  const int64_t nN = axis_offsets(rhs_dims, rs, rcross, nrc, &rc);
  const int64_t nK = axis_offsets(lhs_dims, ls, lhs_contract, n_contract, &lk);
  axis_offsets(rhs_dims, rs, rhs_contract, n_contract, &rk);

#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t b = 0; b < nB; b++) {
    for (int64_t i = 0; i < nM; i++) {
      for (int64_t j = 0; j < nN; j++) {
        const int64_t lo = lb[b] + lc[i], ro = rb[b] + rc[j];
        const int64_t oi = (b * nM + i) * nN + j;
        if (float_path) {
          double result;
          if (acc_f64 || acc == ORC_F64) {
            double s = 0.0;
            for (int64_t c = 0; c < nK; c++) {
              double a = round_to_dtype(load_as_double(lhs, in_dtype, lo + lk[c]), comp);
              double bb = round_to_dtype(load_as_double(rhs, in_dtype, ro + rk[c]), comp);
              s += a * bb;
            }
            result = s;
          } else {
            float s = 0.0f;
            for (int64_t c = 0; c < nK; c++) {
              float a = (float)round_to_dtype(load_as_double(lhs, in_dtype, lo + lk[c]), comp);
              float bb = (float)round_to_dtype(load_as_double(rhs, in_dtype, ro + rk[c]), comp);
              float p = a * bb;
              s = s + p;
            }
            result = (double)s;
          }
          if (is_float_dtype(out_dtype)) store_float(out, out_dtype, oi, result);
          else store_int(out, out_dtype, oi, (int64_t)result);
        } else {
          int64_t s = 0;
          for (int64_t c = 0; c < nK; c++)
            s += load_as_i64(lhs, in_dtype, lo + lk[c]) * load_as_i64(rhs, in_dtype, ro + rk[c]);
          if (is_float_dtype(out_dtype)) store_float(out, out_dtype, oi, (double)s);
          else store_int(out, out_dtype, oi, s);
        }
      }
    }
  }
  free(lb); free(rb); free(lc); free(rc); free(lk); free(rk);
  return 0;
}

/* ------------------------------------------------------------------ */
/* scaled dot-product attention                                       */
/* ------------------------------------------------------------------ */

/* sdpaComputeMaskStrides, sdpa.go:309-329 */
static void mask_strides(int rank, const int64_t* d, int64_t* bstride, int64_t* hstride) {
  *bstride = 0; *hstride = 0;
  if (rank == 3) {
    if (d[0] > 1) *bstride = d[1] * d[2];
  } else if (rank == 4) {
    if (d[0] > 1) *bstride = d[1] * d[2] * d[3];
    if (d[1] > 1) *hstride = d[2] * d[3];
  }
}

/* One (batch, kv head) group: sdpaGeneric, sdpa.go:373-519. */
static void sdpa_group(const float* q, const float* k, const float* v,
                       int64_t q_off, int64_t kv_off, int64_t q_seq_stride, int64_t kv_seq_stride,
                       int64_t q_group_stride,
                       const float* add_mask, const uint8_t* bool_mask, int64_t mask_group_stride,
                       const float* add_bias, int64_t bias_group_stride,
                       float* scores, float* out,
                       int64_t group, int64_t S, int64_t Skv, int64_t D, float scale, int causal,
                       int64_t q_limit, int64_t kv_limit) {
  for (int64_t g = 0; g < group; g++) {
    const int64_t gq = q_off + g * q_group_stride;
    for (int64_t qi = 0; qi < S; qi++) {
      const int64_t row = gq + qi * q_seq_stride;
      if (qi >= q_limit) {               /* padded query row -> zeros */
        for (int64_t d = 0; d < D; d++) out[row + d] = 0.0f;
        continue;
      }
      float* sc = scores + (g * S + qi) * Skv;
      const int64_t mrow = g * mask_group_stride + qi * Skv;
      const int64_t brow = g * bias_group_stride + qi * Skv;
      int64_t live = Skv < kv_limit ? Skv : kv_limit;
      if (causal && qi + 1 < live) live = qi + 1;
      float row_max = -INFINITY;
      for (int64_t j = 0; j < Skv; j++) sc[j] = 0.0f;
      for (int64_t j = 0; j < live; j++) {
        if (bool_mask && !bool_mask[mrow + j]) continue;
        float dot = 0.0f;
        const float* kr = k + kv_off + j * kv_seq_stride;
        for (int64_t d = 0; d < D; d++) {
          float p = q[row + d] * kr[d];
          dot = dot + p;
        }
        float s = dot * scale;
        if (add_bias) s = s + add_bias[brow + j];
        if (add_mask) s = s + add_mask[mrow + j];
        sc[j] = s;
        if (s > row_max) row_max = s;
      }
      float sum = 0.0f;
      for (int64_t j = 0; j < live; j++) {
        if (bool_mask && !bool_mask[mrow + j]) continue;
        sc[j] = (float)exp((double)(sc[j] - row_max));
        sum = sum + sc[j];
      }
      const float inv = (sum != 0.0f) ? 1.0f / sum : 0.0f;  /* all-masked row -> zeros */
      for (int64_t j = 0; j < live; j++) {
        if (bool_mask && !bool_mask[mrow + j]) sc[j] = 0.0f;
        else sc[j] = sc[j] * inv;
      }
      for (int64_t d = 0; d < D; d++) {
        float acc = 0.0f;
        for (int64_t j = 0; j < live; j++) {
          if (bool_mask && !bool_mask[mrow + j]) continue;
          float p = sc[j] * v[kv_off + j * kv_seq_stride + d];
          acc = acc + p;
        }
        out[row + d] = acc;
      }
    }
  }
}

static void sdpa_impl(const float* q, const float* k, const float* v,
                      const void* mask, int mask_is_bool, int mask_rank, const int64_t* mask_dims,
                      const float* bias, int bias_rank, const int64_t* bias_dims,
                      const int32_t* q_len, const int32_t* kv_len, float* out,
                      int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t Skv, int64_t D,
                      int bshd, double scale, int causal,
                      int64_t b0, int64_t b1, int64_t h0, int64_t h1) {
  const int64_t group = Hq / Hkv;
  int64_t q_seq, kv_seq, q_head, kv_head, q_batch, kv_batch;
  if (bshd) {   /* [B,S,H,D], sdpa.go:554-566 */
    q_seq = Hq * D; kv_seq = Hkv * D; q_head = D; kv_head = D;
    q_batch = S * Hq * D; kv_batch = Skv * Hkv * D;
  } else {      /* [B,H,S,D], sdpa.go:567-578 */
    q_seq = D; kv_seq = D; q_head = S * D; kv_head = Skv * D;
    q_batch = Hq * S * D; kv_batch = Hkv * Skv * D;
  }
  int64_t mb = 0, mh = 0, bb = 0, bh = 0;
  if (mask) mask_strides(mask_rank, mask_dims, &mb, &mh);
  if (bias) mask_strides(bias_rank, bias_dims, &bb, &bh);
  float* scores = (float*)malloc(sizeof(float) * (size_t)(group * S * Skv > 0 ? group * S * Skv : 1));
  for (int64_t b = b0; b < b1; b++) {
    int64_t q_limit = S, kv_limit = Skv;
    if (q_len) { int64_t l = q_len[b]; q_limit = l < 0 ? 0 : (l > S ? S : l); }
    if (kv_len) { int64_t l = kv_len[b]; kv_limit = l < 0 ? 0 : (l > Skv ? Skv : l); }
    for (int64_t h = h0; h < h1; h++) {
      const int64_t q_off = b * q_batch + h * group * q_head;
      const int64_t kv_off = b * kv_batch + h * kv_head;
      const float* am = NULL; const uint8_t* bm = NULL; int64_t mgs = 0;
      if (mask) {
        const int64_t off = b * mb + h * group * mh;
        if (mh > 0 && group > 1) mgs = mh;
        if (mask_is_bool) bm = (const uint8_t*)mask + off; else am = (const float*)mask + off;
      }
      const float* ab = NULL; int64_t bgs = 0;
      if (bias) {
        ab = bias + b * bb + h * group * bh;
        if (bh > 0 && group > 1) bgs = bh;
      }
      sdpa_group(q, k, v, q_off, kv_off, q_seq, kv_seq, q_head, am, bm, mgs, ab, bgs,
                 scores, out, group, S, Skv, D, (float)scale, causal, q_limit, kv_limit);
    }
  }
  free(scores);
}

void orc_sdpa_f32(const float* q, const float* k, const float* v,
                  const void* mask, int mask_is_bool, int mask_rank, const int64_t* mask_dims,
                  const float* bias, int bias_rank, const int64_t* bias_dims,
                  const int32_t* q_len, const int32_t* kv_len, float* out,
                  int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t Skv, int64_t D,
                  int bshd, double scale, int causal) {
  if (scale == 0.0) scale = 1.0 / sqrt((double)D);   /* sdpa.go:155-158 */
  sdpa_impl(q, k, v, mask, mask_is_bool, mask_rank, mask_dims, bias, bias_rank, bias_dims,
            q_len, kv_len, out, B, Hq, Hkv, S, Skv, D, bshd, scale, causal, 0, B, 0, Hkv);
}

void orc_sdpa_f32_slice(const float* q, const float* k, const float* v, float* out,
                        int64_t B, int64_t Hq, int64_t Hkv, int64_t S, int64_t Skv, int64_t D,
                        int bshd, double scale, int causal,
                        int64_t b0, int64_t b1, int64_t h0, int64_t h1) {
  if (scale == 0.0) scale = 1.0 / sqrt((double)D);
  sdpa_impl(q, k, v, NULL, 0, 0, NULL, NULL, 0, NULL, NULL, NULL, out,
            B, Hq, Hkv, S, Skv, D, bshd, scale, causal, b0, b1, h0, h1);
}

/* ------------------------------------------------------------------ */
/* blocked f32 GEMM (timed CPU baseline for DotGeneral)               */
/* ------------------------------------------------------------------ */

#define GB_MR 4
#define GB_NR 32
#define GB_KC 128
#define GB_MC 24
#define GB_NC 512

/* Register-tile update: acc[MR][NR] += Apanel[kc][MR] (x) Bpanel[kc][NR].
 * Cloned per ISA so the prebuilt library runs on whatever host it lands on. */
__attribute__((target_clones("avx512f", "avx2,fma", "default")))
static void gb_micro(const float* ap, const float* bp, float* c, int64_t ldc, int64_t kc,
                     int64_t mr, int64_t nr, int overwrite) {
  float acc[GB_MR][GB_NR];
  for (int i = 0; i < GB_MR; i++)
    for (int j = 0; j < GB_NR; j++) acc[i][j] = 0.0f;
  for (int64_t p = 0; p < kc; p++) {
    const float* a = ap + p * GB_MR;
    const float* b = bp + p * GB_NR;
    for (int i = 0; i < GB_MR; i++) {
      const float av = a[i];
      for (int j = 0; j < GB_NR; j++) acc[i][j] += av * b[j];
    }
  }
  for (int64_t i = 0; i < mr; i++)
    for (int64_t j = 0; j < nr; j++) {
      if (overwrite) c[i * ldc + j] = acc[i][j];
      else c[i * ldc + j] += acc[i][j];
    }
}

void orc_gemm_f32_blocked(const float* A, const float* B, float* C,
                          int64_t M, int64_t K, int64_t N, int threads) {
  if (threads < 1) threads = 1;
  const int64_t n_jc = (N + GB_NC - 1) / GB_NC;
#pragma omp parallel num_threads(threads)
  {
    float* bpack = (float*)aligned_alloc(64, sizeof(float) * GB_KC * GB_NC);
    float* apack = (float*)aligned_alloc(64, sizeof(float) * GB_KC * (GB_MC + GB_MR));
#pragma omp for schedule(dynamic, 1)
    for (int64_t jc_i = 0; jc_i < n_jc; jc_i++) {
      const int64_t jc = jc_i * GB_NC;
      const int64_t nc = (N - jc) < GB_NC ? (N - jc) : GB_NC;
      for (int64_t pc = 0; pc < K; pc += GB_KC) {
        const int64_t kc = (K - pc) < GB_KC ? (K - pc) : GB_KC;
        /* pack rhs panel: [ceil(nc/NR)][kc][NR], zero padded */
        for (int64_t jr = 0; jr < nc; jr += GB_NR) {
          float* dst = bpack + (jr / GB_NR) * kc * GB_NR;
          for (int64_t p = 0; p < kc; p++)
            for (int64_t j = 0; j < GB_NR; j++)
              dst[p * GB_NR + j] = (jr + j < nc) ? B[(pc + p) * N + jc + jr + j] : 0.0f;
        }
        for (int64_t ic = 0; ic < M; ic += GB_MC) {
          const int64_t mc = (M - ic) < GB_MC ? (M - ic) : GB_MC;
          for (int64_t ir = 0; ir < mc; ir += GB_MR) {
            float* dst = apack + (ir / GB_MR) * kc * GB_MR;
            for (int64_t p = 0; p < kc; p++)
              for (int64_t i = 0; i < GB_MR; i++)
                dst[p * GB_MR + i] = (ir + i < mc) ? A[(ic + ir + i) * K + pc + p] : 0.0f;
          }
          for (int64_t jr = 0; jr < nc; jr += GB_NR)
            for (int64_t ir = 0; ir < mc; ir += GB_MR) {
              const int64_t mr = (mc - ir) < GB_MR ? (mc - ir) : GB_MR;
              const int64_t nr = (nc - jr) < GB_NR ? (nc - jr) : GB_NR;
              gb_micro(apack + (ir / GB_MR) * kc * GB_MR, bpack + (jr / GB_NR) * kc * GB_NR,
                       C + (ic + ir) * N + jc + jr, N, kc, mr, nr, pc == 0);
            }
        }
      }
    }
    free(bpack);
    free(apack);
  }
}
