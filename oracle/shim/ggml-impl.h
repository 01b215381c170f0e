/*
 * Build-time stand-in for the two names the reference's quantized-matmul sources
 * take from ggml (an empty, un-vendored submodule of the reference):
 *   GGML_FP32_TO_FP16 / GGML_FP16_TO_FP32 : IEEE binary16 round-to-nearest-even
 *   GGML_RESTRICT                         : restrict qualifier
 * Written from that contract; no ggml source is reproduced.  Used only by
 * oracle/Makefile when compiling the reference objects into oracle/_ref/.
 */
#pragma once
#include <immintrin.h>
#include <stdint.h>
typedef uint16_t ggml_fp16_t;
#define GGML_RESTRICT __restrict__
#define GGML_FP32_TO_FP16(x) ((uint16_t)_cvtss_sh((x), 0))
#define GGML_FP16_TO_FP32(x) (_cvtsh_ss((x)))
