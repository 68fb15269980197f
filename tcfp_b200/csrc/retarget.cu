// Block-scaled weights re-targeted for the input-gradient GEMM.
//
// Forward, W (D_out, D_in) carries one power-of-two scale per (row, 32/64/128
// wide block of D_in): the contraction of  y = x . W^T  runs along D_in, so
// the block-scaled tensor-core MMA applies the scales itself.  Backward,
// dX = g . W  contracts along D_out, where those scales change from one
// contraction element to the next (tcfp/kernels.py:1146-1189 dequantizes the
// operands to FP32 and multiplies in TF32 for that reason).
//
// This kernel rewrites the quantized weight once per weight version into the
// orientation the backward contraction wants, so that dX runs on the same FP8
// block-scaled MMA as the forward:
//
//   codes (R = D_out, C = D_in), exponents s[c / bs][r]         (reference layout)
//     ->  codes_t (C, R)   one E4M3 code per element, TRANSPOSED (K-major for dX)
//         t[r / bs][c]     one exponent per (output column c, block of bs rows)
//
//   t[kb][c]      = max over the rows r of block kb of s[c / bs][r]   (sentinel rows excluded)
//   codes_t[c][r] = E4M3( value(codes[r][c]) * 2^(s[c / bs][r] - t[r / bs][c]) )
//
// The exponent shift is <= 0, so nothing overflows; a value is changed only
// when the shift pushes it below E4M3's subnormal step 2^-9 (relative to a
// block whose largest row reaches 2^8): an absolute error of at most
// 2^-10 * 2^t on elements more than 2^15 times smaller than the block's
// range.  Everything else is exact.
//
// Tile: 128 x 128 codes per CTA.  A thread owns 4 x 4 micro-tiles: four
// coalesced 32-bit row loads, a byte transpose in registers, four 32-bit
// stores into an XOR-swizzled shared tile, and coalesced 128-byte row stores
// of the transposed tile.
#include "common.cuh"
#include "launch.h"

namespace tcfp {
namespace {

constexpr int kTile = 128;
constexpr int kThreads = 256;

template <int BS>
__global__ void __launch_bounds__(kThreads)
block_retarget_kernel(const uint8_t* __restrict__ codes_hi, const uint8_t* __restrict__ codes_lo,
                      const int8_t* __restrict__ exp_hi, const int8_t* __restrict__ exp_lo,
                      uint8_t* __restrict__ out_hi, uint8_t* __restrict__ out_lo, int8_t* __restrict__ t_hi,
                      int8_t* __restrict__ t_lo, int64_t R, int64_t C) {
  constexpr int kColBlocks = kTile / BS;   // source column blocks (scale blocks of the forward) per tile
  constexpr int kRowGroups = kTile / BS;   // groups of BS source rows (scale blocks of the backward) per tile
  __shared__ __align__(16) int8_t s_e[kColBlocks][kTile];
  __shared__ int s_t[kColBlocks][kRowGroups];
  __shared__ uint32_t s_tile[kTile * 32];

  const bool lo_plane = blockIdx.y != 0;
  const uint8_t* codes = lo_plane ? codes_lo : codes_hi;
  const int8_t* exps = lo_plane ? exp_lo : exp_hi;
  uint8_t* out = lo_plane ? out_lo : out_hi;
  int8_t* t_plane = lo_plane ? t_lo : t_hi;

  const int64_t tiles_c = (C + kTile - 1) / kTile;
  const int64_t r0 = (int64_t)(blockIdx.x / tiles_c) * kTile;
  const int64_t c0 = (int64_t)(blockIdx.x % tiles_c) * kTile;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- the tile's codes first: 16 independent 32-bit loads per thread, in flight while the exponents are staged.
  //      4 x 4 micro-tiles: rows 4*(warp + 8*i) .. +3, columns 4*lane .. +3
  uint32_t raw_all[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rw = warp + 8 * i;                 // row word: rows 4*rw .. 4*rw + 3
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
      const int64_t row = r0 + 4 * rw + rr, col = c0 + 4 * lane;
      raw_all[i][rr] = (row < R && col < C) ? __ldg(reinterpret_cast<const uint32_t*>(codes + row * C + col)) : 0u;
    }
  }

  // ---- exponents of the tile: s[c / bs][r]; -128 marks an all-zero residual block
  if (threadIdx.x < kColBlocks * kRowGroups) s_t[threadIdx.x / kRowGroups][threadIdx.x % kRowGroups] = -127;
  __syncthreads();
  for (int i = threadIdx.x; i < kColBlocks * kTile; i += kThreads) {
    const int cb = i / kTile, r = i % kTile;
    const int64_t col_block = c0 / BS + cb;
    int8_t e = -128;
    if (r0 + r < R && col_block * BS < C) e = exps[col_block * R + r0 + r];
    s_e[cb][r] = e;
    // a warp holds 32 consecutive rows of one column block, i.e. (part of) one group of BS rows
    const int m = __reduce_max_sync(0xFFFFFFFFu, e == -128 ? -127 : (int)e);
    if (lane == 0) atomicMax(&s_t[cb][r / BS], m);
  }
  __syncthreads();

  const int cb = (4 * lane) / BS;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rw = warp + 8 * i;
    const int g = (4 * rw) / BS;
    const int t = s_t[cb][g];
    uint32_t w[4];
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
      const uint32_t raw = raw_all[i][rr];
      const int e = (int)s_e[cb][4 * rw + rr];
      const int shift = e - t;                    // <= 0 for live rows
      const float f = (e == -128 || shift < -126) ? 0.f : exp2_int(shift);
      const float2 d01 = decode_fp8x2<false>(raw), d23 = decode_fp8x2<false>(raw >> 16);
      w[rr] = encode_fp8x2<false>(d01.x * f, d01.y * f) | (encode_fp8x2<false>(d23.x * f, d23.y * f) << 16);
    }
    // byte transpose: word j gathers byte j of the four rows
    const uint32_t a01 = __byte_perm(w[0], w[1], 0x5140), b01 = __byte_perm(w[0], w[1], 0x7362);
    const uint32_t a23 = __byte_perm(w[2], w[3], 0x5140), b23 = __byte_perm(w[2], w[3], 0x7362);
    const uint32_t o0 = __byte_perm(a01, a23, 0x5410), o1 = __byte_perm(a01, a23, 0x7632);
    const uint32_t o2 = __byte_perm(b01, b23, 0x5410), o3 = __byte_perm(b01, b23, 0x7632);
    const int n = 4 * lane;                      // transposed-tile rows n .. n + 3 share the swizzle key `lane`
    s_tile[(n + 0) * 32 + (rw ^ lane)] = o0;
    s_tile[(n + 1) * 32 + (rw ^ lane)] = o1;
    s_tile[(n + 2) * 32 + (rw ^ lane)] = o2;
    s_tile[(n + 3) * 32 + (rw ^ lane)] = o3;
  }
  __syncthreads();

  // ---- transposed tile out: row n of the tile is 128 contiguous bytes of codes_t
#pragma unroll 4
  for (int k = 0; k < kTile / 8; ++k) {
    const int n = warp * (kTile / 8) + k;
    const int64_t orow = c0 + n, ocol = r0 + 4 * lane;
    if (orow < C && ocol < R)
      *reinterpret_cast<uint32_t*>(out + orow * R + ocol) = s_tile[n * 32 + (lane ^ (n >> 2))];
  }
  // ---- exponents of the transposed operand: t[(r0 / bs + g)][c0 + n]
  for (int i = threadIdx.x; i < kRowGroups * kTile; i += kThreads) {
    const int g = i / kTile, n = i % kTile;
    const int64_t kb = r0 / BS + g;
    if (kb * BS < R && c0 + n < C) t_plane[kb * C + c0 + n] = (int8_t)s_t[n / BS][g];
  }
}

}  // namespace
}  // namespace tcfp

using namespace tcfp;

extern "C" int32_t tcfp_block_retarget(const uint8_t* w_hi, const uint8_t* w_lo, const int8_t* exp_hi,
                                       const int8_t* exp_lo, uint8_t* hi_t, uint8_t* lo_t, int8_t* t_hi, int8_t* t_lo,
                                       int64_t R, int64_t C, int32_t block_size, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!w_hi || !exp_hi || !hi_t || !t_hi) return fail(TCFP_ERR_INVALID, "block_retarget: NULL pointer");
  const bool has_lo = w_lo != nullptr;
  if (has_lo && (!exp_lo || !lo_t || !t_lo)) return fail(TCFP_ERR_INVALID, "block_retarget: the residual needs all of its four arrays");
  if (block_size != 32 && block_size != 64 && block_size != 128)
    return fail(TCFP_ERR_INVALID, "block_size must be 32, 64, or 128, got %d", block_size);
  if (R <= 0 || C <= 0 || R % block_size != 0 || C % block_size != 0)
    return fail(TCFP_ERR_INVALID, "block_retarget: both dimensions (%lld, %lld) must be divisible by block_size (%d)",
                (long long)R, (long long)C, block_size);
  if (((uintptr_t)w_hi | (uintptr_t)w_lo | (uintptr_t)hi_t | (uintptr_t)lo_t) & 3u)
    return fail(TCFP_ERR_INVALID, "block_retarget: code arrays must be 4-byte aligned");
  const int64_t tiles = ((R + kTile - 1) / kTile) * ((C + kTile - 1) / kTile);
  if (tiles > 0x7FFFFFFF) return fail(TCFP_ERR_UNSUPPORTED, "block_retarget: tensor too large");
  const dim3 grid((unsigned)tiles, has_lo ? 2u : 1u, 1u);
  switch (block_size) {
    case 32: block_retarget_kernel<32><<<grid, kThreads, 0, stream>>>(w_hi, w_lo, exp_hi, exp_lo, hi_t, lo_t, t_hi, t_lo, R, C); break;
    case 64: block_retarget_kernel<64><<<grid, kThreads, 0, stream>>>(w_hi, w_lo, exp_hi, exp_lo, hi_t, lo_t, t_hi, t_lo, R, C); break;
    default: block_retarget_kernel<128><<<grid, kThreads, 0, stream>>>(w_hi, w_lo, exp_hi, exp_lo, hi_t, lo_t, t_hi, t_lo, R, C); break;
  }
  CUDA_TRY(cudaGetLastError());
  return TCFP_OK;
}
