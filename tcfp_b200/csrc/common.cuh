// Shared device helpers for the TCFP-12 hot-path kernels (sm_100a).
//
// Everything that decides a quantized byte lives here so that the weight
// quantizer, the activation/gradient quantizer and the tests agree on one
// definition.  All float arithmetic that feeds a rounding decision uses the
// explicit round-to-nearest intrinsics: a contracted FMA would change W_lo
// and the error buffer relative to the reference's op-by-op torch chain
// (tcfp/core.py:99-106, tcfp/nn/__init__.py:364-383).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tcfp {

constexpr float kE4M3Max = 448.0f;     // tcfp/core.py:29
constexpr float kE5M2Max = 57344.0f;   // tcfp/core.py:35
constexpr float kAmaxFloor = 1e-12f;   // tcfp/core.py:100, tcfp/kernels.py:251

// ---- FP8 encode / decode ---------------------------------------------------
template <bool E5M2>
__device__ __forceinline__ uint8_t encode_fp8(float x) {
  // round-to-nearest-even with saturation; callers clamp first so saturation
  // only matters for the deliberately out-of-range probes of the SR search.
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
}

template <bool E5M2>
__device__ __forceinline__ float decode_fp8(uint8_t c) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, E5M2 ? __NV_E5M2 : __NV_E4M3);
  return __half2float(__half(h));
}

// two values per conversion instruction; low byte = first value
template <bool E5M2>
__device__ __forceinline__ uint32_t encode_fp8x2(float a, float b) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
}

// Decode by placing the 7 magnitude bits at the top of a float's exponent /
// mantissa field and rescaling: exact for normals and subnormals alike
// (E4M3: bias 7 -> times 2^120; E5M2: bias 15 -> times 2^112).
template <bool E5M2>
__device__ __forceinline__ float decode_fp8_fast(uint32_t c) {
  const uint32_t mag = E5M2 ? ((c & 0x7Fu) << 21) : ((c & 0x7Fu) << 20);
  const float scale = E5M2 ? 5.192296858534828e33f /* 2^112 */ : 1.329227995784916e36f /* 2^120 */;
  const float v = __fmul_rn(__uint_as_float(mag), scale);
  return __uint_as_float(__float_as_uint(v) | ((c & 0x80u) << 24));
}

// two codes (low 16 bits of c) -> two floats through the hardware converter:
// fp8x2 -> f16x2 is exact, f16 -> f32 is exact
template <bool E5M2>
__device__ __forceinline__ float2 decode_fp8x2(uint32_t c) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(c & 0xFFFFu), E5M2 ? __NV_E5M2 : __NV_E4M3);
  return __half22float2(__half2(h));
}

__device__ __forceinline__ float clampf(float x, float lim) {
  return fminf(fmaxf(x, -lim), lim);
}

// ---- power-of-two block exponent ------------------------------------------
// e = max(ceil(log2(max(amax,1e-12) / fmax)), -126)   (tcfp/kernels.py:250-256)
// evaluated the way the reference's Triton kernels evaluate it on the GPU:
// the float32 "/" is the PTX instruction div.full.f32 (an approximate
// division: for these operands amax * RN(1/fmax), one ulp above the IEEE
// quotient for many amax), the log2 is the full-precision float32 log2.  Both
// are issued here as the same operations, so the exponents agree with the
// reference kernel bit for bit, including amax values a few ulps above
// fmax * 2^k where an IEEE division would land on the other side of the
// integer.
//
// Fast form for fmax = 1.75 * 2^P (448: P = 8, 57344: P = 15).  With
// amax = 2^a (1+f): f < 0.75 puts the quotient in (2^(a-P-1), 2^(a-P)]
// (the top of that range rounds to 2^(a-P) exactly), so e = a-P;
// f >= 0.75 + 256 ulps gives a quotient safely above 2^(a-P), so e = a-P+1;
// the sliver in between goes through the full rule.
__device__ __forceinline__ int block_exponent(float amax, float fmax);
template <bool E5M2>
__device__ __forceinline__ int block_exponent_fast(float amax) {
  constexpr int P = E5M2 ? 15 : 8;
  amax = fmaxf(amax, kAmaxFloor);
  const uint32_t b = __float_as_uint(amax);
  const int a = (int)(b >> 23) - 127;
  const uint32_t m = b & 0x7FFFFFu;
  int e;
  if (m < 0x600000u) e = a - P;
  else if (m >= 0x600000u + 256u) e = a - P + 1;
  else return block_exponent(amax, E5M2 ? kE5M2Max : kE4M3Max);
  return e < -126 ? -126 : e;
}

__device__ __forceinline__ float div_full_f32(float a, float b) {
  float q;
  asm("div.full.f32 %0, %1, %2;" : "=f"(q) : "f"(a), "f"(b));
  return q;
}

__device__ __forceinline__ int block_exponent(float amax, float fmax) {
  amax = fmaxf(amax, kAmaxFloor);
  const float q = div_full_f32(amax, fmax);
  const int e = (int)ceilf(log2f(q));
  return e < -126 ? -126 : e;
}

// 2^e as float for e in [-149, 127] (exact, subnormals included)
__device__ __forceinline__ float exp2_int(int e) {
  if (e >= -126) return __uint_as_float((uint32_t)(e + 127) << 23);
  return __uint_as_float(1u << (e + 149));
}

// ---- Philox4x32-10 ---------------------------------------------------------
// The four output words of philox4x32-10(key = seed, counter = (ctr_lo, ctr_hi, 0, 0)).
// High and low halves of the round products as separate 32-bit multiplies:
// measured faster on sm_100 than forming the 64-bit products.
__device__ __forceinline__ uint4 philox4x32_10(uint64_t seed, uint64_t ctr) {
  uint32_t c0 = (uint32_t)ctr, c1 = (uint32_t)(ctr >> 32), c2 = 0u, c3 = 0u;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hb = __umulhi(0xCD9E8D57u, c2), lb = 0xCD9E8D57u * c2;
    const uint32_t ha = __umulhi(0xD2511F53u, c0), la = 0xD2511F53u * c0;
    c0 = hb ^ c1 ^ k0;
    c2 = ha ^ c3 ^ k1;
    c1 = lb;
    c3 = la;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// word -> uniform in [0,1): reinterpret as int32, x<0 -> -x-1, times 4.6566127342e-10f
__device__ __forceinline__ float philox_word_to_uniform(uint32_t w) {
  int32_t x = (int32_t)w;
  if (x < 0) x = -x - 1;
  return __fmul_rn((float)x, 4.6566127342e-10f);
}

// Block path: u = f(FIRST word of philox(seed, ctr)).  This is the stream
// tl.rand(seed, offset) produces, which the reference's block quantizer draws
// at offset n*K + k (tcfp/kernels.py:415-417).
__device__ __forceinline__ float philox_uniform(uint64_t seed, uint64_t ctr) {
  return philox_word_to_uniform(philox4x32_10(seed, ctr).x);
}

// Per-tensor paths (the reference draws torch.rand_like there, which nothing
// else can reproduce; the stream is this library's definition): element j
// takes word (j & 3) of philox(seed, j >> 2), so one generator call serves
// four elements.  Fills the uniforms of elements base .. base + 3.
__device__ __forceinline__ void philox_uniform_x4(uint64_t seed, uint64_t base, float u[4]) {
  const uint4 a = philox4x32_10(seed, base >> 2);
  const int sh = (int)(base & 3u);
  if (sh == 0) {
    u[0] = philox_word_to_uniform(a.x); u[1] = philox_word_to_uniform(a.y);
    u[2] = philox_word_to_uniform(a.z); u[3] = philox_word_to_uniform(a.w);
    return;
  }
  // a window that straddles two generator calls (stream offsets that are not multiples of four)
  const uint4 b = philox4x32_10(seed, (base >> 2) + 1);
  uint32_t w0, w1, w2, w3;
  if (sh == 1) { w0 = a.y; w1 = a.z; w2 = a.w; w3 = b.x; }
  else if (sh == 2) { w0 = a.z; w1 = a.w; w2 = b.x; w3 = b.y; }
  else { w0 = a.w; w1 = b.x; w2 = b.y; w3 = b.z; }
  u[0] = philox_word_to_uniform(w0); u[1] = philox_word_to_uniform(w1);
  u[2] = philox_word_to_uniform(w2); u[3] = philox_word_to_uniform(w3);
}

// ---- stochastic rounding, two variants -------------------------------------
// Variant of the block kernel (tcfp/kernels.py:398-423).  x is already
// clamped to +-448.
__device__ __forceinline__ uint8_t sr_block_e4m3(float x, float u) {
  uint8_t rtn = encode_fp8<false>(x);
  float rtn_f = decode_fp8<false>(rtn);
  float diff = __fsub_rn(x, rtn_f);
  float dir = diff >= 0.f ? 1.f : -1.f;
  float abs_rtn = fmaxf(fabsf(rtn_f), kAmaxFloor);
  float nudge = __fmul_rn(__fmul_rn(dir, abs_rtn), 0.25f);
  uint8_t other = encode_fp8<false>(__fadd_rn(rtn_f, nudge));
  float other_f = decode_fp8<false>(other);
  float span = fabsf(__fsub_rn(other_f, rtn_f));
  float gap = fmaxf(span, 1e-45f);
  float frac = fminf(__fdiv_rn(fabsf(diff), gap), 1.0f);
  bool exact = (fabsf(diff) < 1e-45f) || (span < 1e-45f);
  if (exact) return rtn;
  return (u < frac) ? other : rtn;
}

// Variant of the per-tensor path (tcfp/core.py:418-464).
__device__ __forceinline__ uint8_t sr_tensor_e4m3(float x, float u) {
  uint8_t lo = encode_fp8<false>(x);
  float lo_f = decode_fp8<false>(lo);
  float d = __fsub_rn(x, lo_f);
  if (x == lo_f) return lo;
  float dir = d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f);
  uint8_t hi = encode_fp8<false>(__fadd_rn(lo_f, __fmul_rn(dir, 0.0078125f)));
  if (decode_fp8<false>(hi) == lo_f) {
    float abs_lo = fmaxf(fabsf(lo_f), 0.015625f);
    float big = __fmul_rn(__fmul_rn(dir, abs_lo), 0.25f);
    float probe = __fadd_rn(lo_f, big);
    // torch's float -> float8_e4m3fn cast does not saturate: anything that
    // rounds past 448 (|probe| > 464) becomes NaN, every comparison with it
    // is false and the reference keeps the round-to-nearest code.
    if (fabsf(probe) > 464.0f) return lo;
    hi = encode_fp8<false>(probe);
  }
  float hi_f = decode_fp8<false>(hi);
  float gap = fmaxf(fabsf(__fsub_rn(hi_f, lo_f)), 1e-45f);
  float frac = fminf(fmaxf(__fdiv_rn(fabsf(d), gap), 0.f), 1.f);
  return (u < frac) ? hi : lo;
}

// ---- packed E8M0 scale-factor layout ---------------------------------------
// The tensor-core block-scaled MMA takes one E8M0 byte per (row, 32-wide K
// block).  Scale factors of 128 rows x 4 consecutive scale blocks form one
// 512-byte chunk: byte (r0*16 + r1*4 + j) for row = 32*r1 + r0 and scale
// block j.  Chunks are ordered [row_block][k_group].  Exponent e is stored
// biased (e + 127); the -128 sentinel becomes 0 (2^-127).
__device__ __forceinline__ uint8_t e8m0_from_exp(int e) {
  return e <= -127 ? (uint8_t)0 : (uint8_t)(e + 127);
}
__host__ __device__ __forceinline__ size_t sf_chunk_offset(int64_t row, int64_t kb, int64_t k_groups) {
  int64_t rb = row >> 7, r1 = (row >> 5) & 3, r0 = row & 31;
  int64_t kg = kb >> 2, j = kb & 3;
  return (size_t)((rb * k_groups + kg) * 512 + r0 * 16 + r1 * 4 + j);
}

}  // namespace tcfp
