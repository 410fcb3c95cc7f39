/*
 * CPU oracle for the quantized-matmul hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, the arithmetic of the
 * reference's device kernels so that the CUDA path can be checked against it. It is
 * never linked into, imported by or called from the product library; only the test
 * suite, the smoke check and the benchmark's cpu_baseline / reference arm may use it.
 *
 * Parity pins: the codec and the quantizer are pinned bit-exactly against the
 * reference's own helper functions compiled for the host (oracle/build.py) and
 * against the reference tests' golden vectors (tests/test_oracle_golden.py). The
 * NVFP4 quantizer has no counterpart in the reference: parity unpinned for it.
 *
 * Every function cites the reference file:line it follows (paths inside the
 * reference project).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

static inline float bits_to_float(uint32_t bits) {
  float value;
  memcpy(&value, &bits, sizeof value);
  return value;
}

static inline uint32_t float_to_bits(float value) {
  uint32_t bits;
  memcpy(&bits, &value, sizeof bits);
  return bits;
}

/* kernels/mxfp8.cu:1-3 — bf16 is the upper half of an fp32. */
ORACLE_API float oracle_bf16_to_float(uint16_t value) {
  return bits_to_float((uint32_t)value << 16);
}

/* kernels/mxfp8.cu:5-9 — round to nearest even by adding 0x7fff + lsb; no NaN case. */
ORACLE_API uint16_t oracle_float_to_bf16(float value) {
  uint32_t bits = float_to_bits(value);
  bits += 0x7fffu + ((bits >> 16) & 1u);
  return (uint16_t)(bits >> 16);
}

/* IEEE binary16 helpers for the f16 GEMV and the int4 extension (round to nearest even). */
ORACLE_API float oracle_f16_to_float(uint16_t value) {
  uint32_t sign = (uint32_t)(value & 0x8000u) << 16;
  uint32_t exponent = (value >> 10) & 0x1fu;
  uint32_t mantissa = value & 0x3ffu;
  if (exponent == 0) {
    float magnitude = ldexpf((float)mantissa, -24);
    return sign ? -magnitude : magnitude;
  }
  if (exponent == 31) return bits_to_float(sign | 0x7f800000u | (mantissa << 13));
  return bits_to_float(sign | ((exponent + 112u) << 23) | (mantissa << 13));
}

ORACLE_API uint16_t oracle_float_to_f16(float value) {
  uint32_t bits = float_to_bits(value);
  uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
  uint32_t magnitude = bits & 0x7fffffffu;
  if (magnitude >= 0x7f800000u) return sign | (magnitude > 0x7f800000u ? 0x7e00u : 0x7c00u);
  if (magnitude >= 0x477ff000u) return sign | 0x7c00u; /* rounds to infinity */
  if (magnitude < 0x33000001u) return sign;            /* rounds to zero */
  int exponent = (int)(magnitude >> 23) - 127;
  uint32_t mantissa = (magnitude & 0x7fffffu) | 0x800000u;
  int shift = exponent < -14 ? 13 + (-14 - exponent) : 13;
  uint32_t kept = mantissa >> shift;
  uint32_t rest = mantissa & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rest > half || (rest == half && (kept & 1u))) ++kept;
  if (exponent < -14) return sign | (uint16_t)kept;
  return sign | (uint16_t)(((uint32_t)(exponent + 15) << 10) + (kept - 0x400u));
}

/* kernels/mxfp8.cu:11-23 — E4M3 (finite-only variant): bias 7, 0x7f/0xff are NaN. */
ORACLE_API float oracle_e4m3(uint8_t value) {
  uint32_t magnitude = value & 0x7fu;
  uint32_t exponent = magnitude >> 3;
  uint32_t mantissa = magnitude & 7u;
  if (exponent == 15u && mantissa == 7u) return bits_to_float(0x7fc00000u);
  float decoded = exponent == 0u
                      ? ldexpf((float)mantissa, -9)
                      : ldexpf(1.0f + (float)mantissa * 0.125f, (int)exponent - 7);
  return (value & 0x80u) == 0u ? decoded : -decoded;
}

/* kernels/mxfp8.cu:25-29 — E8M0 power-of-two scale, 255 is NaN. */
ORACLE_API float oracle_e8m0(uint8_t value) {
  return value == 255u ? bits_to_float(0x7fc00000u) : ldexpf(1.0f, (int)value - 127);
}

/* kernels/mxfp8.cu:31-53 — fp32 -> E4M3, nearest even, saturating at 448 (0x7e). */
ORACLE_API uint8_t oracle_encode_e4m3(float value) {
  uint8_t sign = (float_to_bits(value) >> 31) == 0u ? 0u : 0x80u;
  float magnitude = fabsf(value);
  if (magnitude == 0.0f) return sign;
  if (magnitude >= 448.0f) return sign | 0x7eu;
  if (magnitude < 0.015625f) {
    uint32_t mantissa = (uint32_t)nearbyintf(magnitude * 512.0f);
    return sign | (uint8_t)(mantissa < 8u ? mantissa : 8u);
  }
  int exponent = ilogbf(magnitude);
  uint32_t encoded_exponent = (uint32_t)(exponent + 7);
  uint32_t mantissa = (uint32_t)nearbyintf((ldexpf(magnitude, -exponent) - 1.0f) * 8.0f);
  if (mantissa == 8u) {
    ++encoded_exponent;
    mantissa = 0u;
  }
  if (encoded_exponent >= 15u) {
    encoded_exponent = 15u;
    if (mantissa > 6u) mantissa = 6u;
  }
  return sign | (uint8_t)((encoded_exponent << 3) | mantissa);
}

/*
 * kernels/mxfp8.cu:55-67 and sys/native/fp4_vector_sm120.cu:32-39 — byte offset of scale
 * (row, column) in the 128-row x 4-column swizzled atoms both block-scaled formats share.
 */
ORACLE_API uint32_t oracle_scale_offset(uint32_t row, uint32_t column, uint32_t columns) {
  uint32_t column_tiles = (columns + 3u) / 4u;
  uint32_t row_tile = row / 128u;
  uint32_t row_in_tile = row % 128u;
  uint32_t row_quarter = row_in_tile / 32u;
  uint32_t row_lane = row_in_tile % 32u;
  uint32_t column_tile = column / 4u;
  uint32_t column_in_tile = column % 4u;
  return ((((row_tile * column_tiles + column_tile) * 32u + row_lane) * 4u + row_quarter) * 4u +
          column_in_tile);
}

/* src/cutlass/mxfp8.rs:45-50 — padded bytes of a swizzled scale buffer. */
ORACLE_API size_t oracle_scale_bytes(size_t rows, size_t columns) {
  return ((rows + 127u) / 128u) * 128u * (((columns + 3u) / 4u) * 4u);
}

/*
 * kernels/mxfp8.cu:69-96 — bf16 -> MXFP8. One E8M0 scale per 32 consecutive columns:
 * exponent = clamp(ceil(log2(max(amax / 448, 2^-127))) + 127, 0, 254), codes are
 * encode_e4m3(value / 2^(exponent - 127)); the scale byte goes straight to its swizzled
 * slot. `scales` must be pre-zeroed by the caller (src/mxfp8/tensor_core.rs:183).
 * NaN elements do not take part in amax (fmaxf semantics, kernels/mxfp8.cu:81-84).
 */
ORACLE_API void oracle_mxfp8_quantize_bf16(const uint16_t* input, uint8_t* output, uint8_t* scales,
                                           uint32_t rows, uint32_t columns) {
  uint32_t groups = columns / 32u;
  for (uint32_t row = 0; row < rows; ++row) {
    for (uint32_t group = 0; group < groups; ++group) {
      const uint16_t* block = input + (size_t)row * columns + (size_t)group * 32u;
      float maximum = 0.0f;
      int seen = 0;
      for (uint32_t lane = 0; lane < 32u; ++lane) {
        float magnitude = fabsf(oracle_bf16_to_float(block[lane]));
        maximum = seen ? fmaxf(maximum, magnitude) : magnitude;
        seen = 1;
      }
      float requested = fmaxf(maximum / 448.0f, 5.87747175e-39f);
      int exponent = (int)ceilf(log2f(requested)) + 127;
      if (exponent > 254) exponent = 254;
      if (exponent < 0) exponent = 0;
      float scale = ldexpf(1.0f, exponent - 127);
      uint8_t* codes = output + (size_t)row * columns + (size_t)group * 32u;
      for (uint32_t lane = 0; lane < 32u; ++lane) {
        codes[lane] = oracle_encode_e4m3(oracle_bf16_to_float(block[lane]) / scale);
      }
      scales[oracle_scale_offset(row, group, groups)] = (uint8_t)exponent;
    }
  }
}

/* kernels/mxfp8.cu:98-109 — row-major [rows, columns] scales into the swizzled layout. */
ORACLE_API void oracle_swizzle_scales(const uint8_t* input, uint8_t* output, uint32_t rows,
                                      uint32_t columns) {
  for (uint32_t row = 0; row < rows; ++row) {
    for (uint32_t column = 0; column < columns; ++column) {
      output[oracle_scale_offset(row, column, columns)] = input[(size_t)row * columns + column];
    }
  }
}

/*
 * kernels/mxfp8.cu:111-153 (and the 4-token variant :155-217) — weight-only MXFP8:
 * out[t, n] = bf16(sum_k x[t,k] * e4m3(w[n,k]) * 2^(s[n,k/32]-127)), fp32 sum with the
 * per-term order x * w * scale. Scales are row-major [n, k/32]; weights are little-endian
 * u32 words holding four codes each.
 */
ORACLE_API void oracle_mxfp8_bf16_matmul(const uint16_t* input, const uint32_t* weight,
                                         const uint8_t* scales, uint16_t* output, uint32_t tokens,
                                         uint32_t input_features, uint32_t output_features) {
  uint32_t words = input_features / 4u;
  uint32_t groups = input_features / 32u;
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t token = 0; token < tokens; ++token) {
    for (uint32_t row = 0; row < output_features; ++row) {
      float sum = 0.0f;
      for (uint32_t column = 0; column < input_features; ++column) {
        uint32_t packed = weight[(size_t)row * words + column / 4u];
        uint8_t code = (uint8_t)(packed >> ((column & 3u) * 8u));
        float x = oracle_bf16_to_float(input[(size_t)token * input_features + column]);
        float scale = oracle_e8m0(scales[(size_t)row * groups + column / 32u]);
        sum += x * oracle_e4m3(code) * scale;
      }
      output[(size_t)token * output_features + row] = oracle_float_to_bf16(sum);
    }
  }
}

/*
 * kernels/mxfp8.cu:219-271 — routed bank GEMV with optional bf16 bias; an out-of-range
 * expert writes 0.
 */
ORACLE_API void oracle_mxfp8_bf16_gathered(const uint16_t* input, const uint32_t* weight,
                                           const uint8_t* scales, const uint16_t* bias,
                                           const uint32_t* selected, uint16_t* output,
                                           uint32_t assignments, uint32_t matrices, uint32_t rows,
                                           uint32_t columns, uint32_t selections_per_input,
                                           uint32_t has_bias) {
  uint32_t words = columns / 4u;
  uint32_t groups = columns / 32u;
  for (uint32_t assignment = 0; assignment < assignments; ++assignment) {
    uint32_t matrix = selected[assignment];
    for (uint32_t row = 0; row < rows; ++row) {
      if (matrix >= matrices) {
        output[(size_t)assignment * rows + row] = oracle_float_to_bf16(0.0f);
        continue;
      }
      size_t matrix_row = (size_t)matrix * rows + row;
      uint32_t input_row = assignment / selections_per_input;
      float sum = 0.0f;
      for (uint32_t column = 0; column < columns; ++column) {
        uint32_t packed = weight[matrix_row * words + column / 4u];
        uint8_t code = (uint8_t)(packed >> ((column & 3u) * 8u));
        float x = oracle_bf16_to_float(input[(size_t)input_row * columns + column]);
        float scale = oracle_e8m0(scales[matrix_row * groups + column / 32u]);
        sum += x * oracle_e4m3(code) * scale;
      }
      float value = sum + (has_bias == 0u ? 0.0f : oracle_bf16_to_float(bias[matrix_row]));
      output[(size_t)assignment * rows + row] = oracle_float_to_bf16(value);
    }
  }
}

/* kernels/mxfp8.cu:273-296 — selected-row dequantisation times output_scale. */
ORACLE_API void oracle_mxfp8_embedding_bf16(const uint32_t* weight, const uint8_t* scales,
                                            const uint32_t* selected, uint16_t* output,
                                            uint32_t selected_start, uint32_t tokens,
                                            uint32_t vocab, uint32_t hidden, float output_scale) {
  uint32_t words = hidden / 4u;
  uint32_t groups = hidden / 32u;
  for (uint32_t token = 0; token < tokens; ++token) {
    uint32_t row = selected[selected_start + token];
    if (row >= vocab) continue;
    for (uint32_t column = 0; column < hidden; ++column) {
      uint32_t packed = weight[(size_t)row * words + column / 4u];
      uint8_t code = (uint8_t)(packed >> ((column & 3u) * 8u));
      float scale = oracle_e8m0(scales[(size_t)row * groups + column / 32u]);
      output[(size_t)token * hidden + column] =
          oracle_float_to_bf16(oracle_e4m3(code) * scale * output_scale);
    }
  }
}

/*
 * Dequantise an MXFP8 operand ([rows, k] codes, swizzled E8M0 scales per 32 columns) to
 * fp32: code * 2^(s-127). Format from kernels/mxfp8.cu:11-29,55-67; operand roles from
 * sys/native/mxfp8_sm120.cu:17-48 (A row-major [M,K], B "column-major" = [N,K] K-contiguous).
 */
ORACLE_API void oracle_mxfp8_dequantize(const uint8_t* codes, const uint8_t* scales, float* output,
                                        uint32_t rows, uint32_t k) {
  uint32_t groups = k / 32u;
#pragma omp parallel for schedule(static)
  for (uint32_t row = 0; row < rows; ++row) {
    for (uint32_t column = 0; column < k; ++column) {
      float scale = oracle_e8m0(scales[oracle_scale_offset(row, column / 32u, groups)]);
      output[(size_t)row * k + column] = oracle_e4m3(codes[(size_t)row * k + column]) * scale;
    }
  }
}

/*
 * C[M,N] = bf16(A[M,K] . B[N,K]^T) on fp32 operands, fp32 accumulation
 * (sys/native/mxfp8_sm120.cu:17-48: fp32 accumulator, alpha 1, beta 0, bf16 output).
 * Cache-blocked, OpenMP over row blocks. Used for every dequantise-then-matmul check and
 * as the timed CPU baseline.
 */
ORACLE_API void oracle_gemm_nt_f32(const float* a, const float* b, float* c, uint32_t m,
                                   uint32_t n, uint32_t k) {
  enum { BM = 32, BN = 64, BK = 256 };
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (uint32_t m0 = 0; m0 < m; m0 += BM) {
    for (uint32_t n0 = 0; n0 < n; n0 += BN) {
      float tile[BM][BN];
      memset(tile, 0, sizeof tile);
      uint32_t m1 = m0 + BM < m ? m0 + BM : m;
      uint32_t n1 = n0 + BN < n ? n0 + BN : n;
      for (uint32_t k0 = 0; k0 < k; k0 += BK) {
        uint32_t k1 = k0 + BK < k ? k0 + BK : k;
        for (uint32_t i = m0; i < m1; ++i) {
          const float* a_row = a + (size_t)i * k;
          for (uint32_t j = n0; j < n1; ++j) {
            const float* b_row = b + (size_t)j * k;
            float sum = 0.0f;
            for (uint32_t p = k0; p < k1; ++p) sum += a_row[p] * b_row[p];
            tile[i - m0][j - n0] += sum;
          }
        }
      }
      for (uint32_t i = m0; i < m1; ++i) {
        for (uint32_t j = n0; j < n1; ++j) c[(size_t)i * n + j] = tile[i - m0][j - n0];
      }
    }
  }
}

ORACLE_API void oracle_f32_to_bf16(const float* input, uint16_t* output, size_t count) {
  for (size_t index = 0; index < count; ++index) output[index] = oracle_float_to_bf16(input[index]);
}

ORACLE_API void oracle_bf16_to_f32(const uint16_t* input, float* output, size_t count) {
  for (size_t index = 0; index < count; ++index) output[index] = oracle_bf16_to_float(input[index]);
}

/* MXFP8 block-scaled GEMM, dequantise-then-matmul (sys/native/mxfp8_sm120.cu:17-48,137-156). */
ORACLE_API int oracle_mxfp8_gemm(const uint8_t* a, const uint8_t* a_scales, const uint8_t* b,
                                 const uint8_t* b_scales, uint16_t* c, uint32_t m, uint32_t n,
                                 uint32_t k) {
  float* a_f = (float*)malloc((size_t)m * k * sizeof(float));
  float* b_f = (float*)malloc((size_t)n * k * sizeof(float));
  float* c_f = (float*)malloc((size_t)m * n * sizeof(float));
  if (!a_f || !b_f || !c_f) {
    free(a_f); free(b_f); free(c_f);
    return -2;
  }
  oracle_mxfp8_dequantize(a, a_scales, a_f, m, k);
  oracle_mxfp8_dequantize(b, b_scales, b_f, n, k);
  oracle_gemm_nt_f32(a_f, b_f, c_f, m, n, k);
  oracle_f32_to_bf16(c_f, c, (size_t)m * n);
  free(a_f); free(b_f); free(c_f);
  return 0;
}

/* ---------------------------------------------------------------------------------------
 * NVFP4: E2M1 codes (two per byte, even k in the low nibble) with one UE4M3 scale per 16.
 * ------------------------------------------------------------------------------------- */

/* sys/native/fp4_vector_sm120.cu:41-79 (cvt e2m1x2) and sys/native/marlin/repack.cu:32-34. */
ORACLE_API float oracle_e2m1(uint8_t nibble) {
  static const float magnitudes[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  float magnitude = magnitudes[nibble & 7u];
  return (nibble & 8u) ? -magnitude : magnitude;
}

/* sys/native/fp4_vector_sm120.cu:81-83 — UE4M3: the E4M3 bit pattern read as unsigned. */
ORACLE_API float oracle_ue4m3(uint8_t value) { return oracle_e4m3(value & 0x7fu); }

/* sys/native/fp4_vector_sm120.cu:32-39 — scale (row, 16-wide column block) for K columns. */
ORACLE_API uint32_t oracle_fp4_scale_index(uint32_t row, uint32_t scale_column, uint32_t k) {
  uint32_t blocks_k = k / 64u;
  uint32_t row_block = ((row >> 7) * blocks_k) << 9;
  uint32_t row_offset = ((row & 31u) << 4) + (((row & 127u) >> 5) << 2);
  uint32_t column_offset = ((scale_column >> 2) << 9) + (scale_column & 3u);
  return row_block + row_offset + column_offset;
}

ORACLE_API void oracle_nvfp4_dequantize(const uint8_t* codes, const uint8_t* scales, float* output,
                                        uint32_t rows, uint32_t k) {
#pragma omp parallel for schedule(static)
  for (uint32_t row = 0; row < rows; ++row) {
    for (uint32_t column = 0; column < k; ++column) {
      uint8_t byte = codes[((size_t)row * k + column) / 2u];
      uint8_t nibble = (column & 1u) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xfu);
      float scale = oracle_ue4m3(scales[oracle_fp4_scale_index(row, column / 16u, k)]);
      output[(size_t)row * k + column] = oracle_e2m1(nibble) * scale;
    }
  }
}

/*
 * sys/native/fp4_vector_sm120.cu:85-125 — y[n] = bf16(alpha * sum_blocks dot16 * sx * sw),
 * FP4 x FP4, M = 1, fp32 accumulation; each 16-wide dot is formed first and then scaled
 * by the product of the two block scales.
 */
ORACLE_API void oracle_fp4_vector(const uint8_t* input, const uint8_t* input_scales,
                                  const uint8_t* weight, const uint8_t* weight_scales,
                                  uint16_t* output, uint32_t n, uint32_t k, float alpha) {
#pragma omp parallel for schedule(static)
  for (uint32_t row = 0; row < n; ++row) {
    float accumulator = 0.0f;
    for (uint32_t block = 0; block < k / 16u; ++block) {
      float dot = 0.0f;
      for (uint32_t item = 0; item < 16u; ++item) {
        uint32_t column = block * 16u + item;
        uint8_t xb = input[column / 2u];
        uint8_t wb = weight[((size_t)row * k + column) / 2u];
        uint8_t xn = (column & 1u) ? (uint8_t)(xb >> 4) : (uint8_t)(xb & 0xfu);
        uint8_t wn = (column & 1u) ? (uint8_t)(wb >> 4) : (uint8_t)(wb & 0xfu);
        dot = oracle_e2m1(xn) * oracle_e2m1(wn) + dot;
      }
      float scales = oracle_ue4m3(input_scales[oracle_fp4_scale_index(0, block, k)]) *
                     oracle_ue4m3(weight_scales[oracle_fp4_scale_index(row, block, k)]);
      accumulator += dot * scales;
    }
    output[row] = oracle_float_to_bf16(accumulator * alpha);
  }
}

/*
 * bf16 activations x NVFP4 weights, M small: y[m, n] = bf16(global * sum_k x * e2m1(w) * sw).
 * The reference's analogue is the Marlin NVFP4 dense path, whose effective numerics are
 * fp32 accumulation of x * (e2m1 * s) followed by the global scale before the bf16 round
 * (sys/native/marlin/vendor/dense_template.h:355-359,1655-1658).
 */
ORACLE_API void oracle_nvfp4_gemv_bf16(const uint16_t* input, const uint8_t* weight,
                                       const uint8_t* weight_scales, uint16_t* output, uint32_t m,
                                       uint32_t n, uint32_t k, float global_scale) {
#pragma omp parallel for schedule(static)
  for (uint32_t row = 0; row < n; ++row) {
    for (uint32_t token = 0; token < m; ++token) {
      float accumulator = 0.0f;
      for (uint32_t column = 0; column < k; ++column) {
        uint8_t wb = weight[((size_t)row * k + column) / 2u];
        uint8_t wn = (column & 1u) ? (uint8_t)(wb >> 4) : (uint8_t)(wb & 0xfu);
        float scale = oracle_ue4m3(weight_scales[oracle_fp4_scale_index(row, column / 16u, k)]);
        float x = oracle_bf16_to_float(input[(size_t)token * k + column]);
        accumulator += x * (oracle_e2m1(wn) * scale);
      }
      output[(size_t)token * n + row] = oracle_float_to_bf16(accumulator * global_scale);
    }
  }
}

/* Nearest-even fp32 -> UE4M3 (non-negative input), saturating at 448; via the E4M3 encoder. */
ORACLE_API uint8_t oracle_encode_ue4m3(float value) {
  if (!(value > 0.0f)) return 0u;
  return (uint8_t)(oracle_encode_e4m3(value) & 0x7fu);
}

/* Nearest-even fp32 -> E2M1 nibble, saturating at +-6. Ties go to the even code. */
ORACLE_API uint8_t oracle_encode_e2m1(float value) {
  uint8_t sign = (float_to_bits(value) >> 31) ? 8u : 0u;
  float magnitude = fabsf(value);
  uint8_t code;
  if (!(magnitude == magnitude)) code = 7u;
  else if (magnitude <= 0.25f) code = 0u;
  else if (magnitude < 0.75f) code = 1u;
  else if (magnitude <= 1.25f) code = 2u;
  else if (magnitude < 1.75f) code = 3u;
  else if (magnitude <= 2.5f) code = 4u;
  else if (magnitude < 3.5f) code = 5u;
  else if (magnitude <= 5.0f) code = 6u;
  else code = 7u;
  return sign | code;
}

/*
 * bf16 -> NVFP4. NO COUNTERPART IN THE REFERENCE (its tests feed constant bytes,
 * tests/cutlass/fp4/mod.rs:21-24): parity unpinned; this function is the written spec.
 *   global = amax_tensor / (448 * 6)            (1.0 when the tensor is all zero)
 *   s_blk  = rne_ue4m3(amax_blk / (6 * global)) (one per 16 columns, swizzled layout)
 *   code   = rne_e2m1(x * r), r = 1 / (ue4m3(s_blk) * global) rounded to fp32 once per block
 *            (x / (ue4m3(s_blk) * global) where r overflows), saturating at +-6; 0 when s_blk is 0
 * All divisions and products are fp32. Returns the global scale through *global_scale.
 */
static void nvfp4_quantize_rows(const uint16_t* input, uint8_t* codes, uint8_t* scales,
                                float global, uint32_t rows, uint32_t k);

ORACLE_API void oracle_nvfp4_quantize_bf16(const uint16_t* input, uint8_t* codes, uint8_t* scales,
                                           float* global_scale, uint32_t rows, uint32_t k) {
  float amax = 0.0f;
  for (size_t index = 0; index < (size_t)rows * k; ++index) {
    float magnitude = fabsf(oracle_bf16_to_float(input[index]));
    if (magnitude > amax) amax = magnitude;
  }
  float global = amax > 0.0f ? amax / 2688.0f : 1.0f;
  *global_scale = global;
  nvfp4_quantize_rows(input, codes, scales, global, rows, k);
}

/* The same block scales and codes for a global scale the caller fixed beforehand (a calibrated
 * activation scale shared by several tensors): steps 2 and 3 of the spec above. */
ORACLE_API void oracle_nvfp4_quantize_bf16_scaled(const uint16_t* input, uint8_t* codes,
                                                  uint8_t* scales, float global_scale,
                                                  uint32_t rows, uint32_t k) {
  nvfp4_quantize_rows(input, codes, scales, global_scale, rows, k);
}

static void nvfp4_quantize_rows(const uint16_t* input, uint8_t* codes, uint8_t* scales,
                                float global, uint32_t rows, uint32_t k) {
  for (uint32_t row = 0; row < rows; ++row) {
    for (uint32_t block = 0; block < k / 16u; ++block) {
      const uint16_t* values = input + (size_t)row * k + (size_t)block * 16u;
      float block_max = 0.0f;
      for (uint32_t item = 0; item < 16u; ++item) {
        float magnitude = fabsf(oracle_bf16_to_float(values[item]));
        if (magnitude > block_max) block_max = magnitude;
      }
      uint8_t scale_code = oracle_encode_ue4m3(block_max / (6.0f * global));
      scales[oracle_fp4_scale_index(row, block, k)] = scale_code;
      float denominator = oracle_ue4m3(scale_code) * global;
      volatile float inverse = 1.0f / denominator;        /* rounded to fp32 here, once */
      int by_product = inverse <= 3.402823466e38f;
      for (uint32_t item = 0; item < 16u; item += 2u) {
        uint8_t low = 0u, high = 0u;
        if (scale_code != 0u) {
          float first = oracle_bf16_to_float(values[item]);
          float second = oracle_bf16_to_float(values[item + 1u]);
          low = oracle_encode_e2m1(by_product ? first * inverse : first / denominator);
          high = oracle_encode_e2m1(by_product ? second * inverse : second / denominator);
        }
        codes[((size_t)row * k + (size_t)block * 16u + item) / 2u] = (uint8_t)(low | (high << 4));
      }
    }
  }
}

/* ---------------------------------------------------------------------------------------
 * Dense GEMV and grouped GEMM
 * ------------------------------------------------------------------------------------- */

/*
 * sys/native/dense_vector_sm120.cu:50-132 — y = alpha * W x + beta * y, fp32 FMA chain,
 * output rounded to the element type. data_type: 0 = f16, 1 = bf16.
 */
ORACLE_API void oracle_dense_vector(int data_type, const uint16_t* input, const uint16_t* weight,
                                    uint16_t* output, uint32_t n, uint32_t k, float alpha,
                                    float beta) {
#pragma omp parallel for schedule(static)
  for (uint32_t row = 0; row < n; ++row) {
    float sum = 0.0f;
    for (uint32_t column = 0; column < k; ++column) {
      float x = data_type ? oracle_bf16_to_float(input[column]) : oracle_f16_to_float(input[column]);
      float w = data_type ? oracle_bf16_to_float(weight[(size_t)row * k + column])
                          : oracle_f16_to_float(weight[(size_t)row * k + column]);
      sum = fmaf(x, w, sum);
    }
    float result = alpha * sum;
    if (beta != 0.0f) {
      float previous = data_type ? oracle_bf16_to_float(output[row]) : oracle_f16_to_float(output[row]);
      result = fmaf(beta, previous, result);
    }
    output[row] = data_type ? oracle_float_to_bf16(result) : oracle_float_to_f16(result);
  }
}

/*
 * sys/native/variable_grouped_bf16_sm120.cu:18-33 — per group g the first
 * min(rows[g], max_rows) rows starting at offsets[g] of the compact A [capacity, K] are
 * multiplied by W_g^T ([N, K]) into the same rows of C [capacity, N]; fp32 accumulation,
 * C = acc + beta * C, bf16 out. Rows no group covers are left untouched.
 */
ORACLE_API void oracle_variable_grouped_bf16(const uint16_t* input, const uint16_t* weights,
                                             const uint32_t* rows, const uint32_t* offsets,
                                             uint16_t* output, uint32_t groups, uint32_t max_rows,
                                             uint32_t n, uint32_t k, float beta) {
  for (uint32_t group = 0; group < groups; ++group) {
    uint32_t row_count = rows[group] < max_rows ? rows[group] : max_rows;
    size_t offset = offsets[group];
    const uint16_t* w = weights + (size_t)group * n * k;
#pragma omp parallel for collapse(2) schedule(static)
    for (uint32_t row = 0; row < row_count; ++row) {
      for (uint32_t column = 0; column < n; ++column) {
        const uint16_t* a_row = input + (offset + row) * k;
        const uint16_t* w_row = w + (size_t)column * k;
        float sum = 0.0f;
        for (uint32_t p = 0; p < k; ++p) {
          sum += oracle_bf16_to_float(a_row[p]) * oracle_bf16_to_float(w_row[p]);
        }
        uint16_t* destination = output + (offset + row) * n + column;
        if (beta != 0.0f) sum += beta * oracle_bf16_to_float(*destination);
        *destination = oracle_float_to_bf16(sum);
      }
    }
  }
}

ORACLE_API int oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
