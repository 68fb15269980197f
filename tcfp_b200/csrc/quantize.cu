// K1 / K2: HBM-bound quantizers of the TCFP-12 hot path (sm_100a).
//
//   dual_quantize_block_kernel   W(+e) -> W_hi, W_lo, two exponent planes, e'
//                                (tcfp/kernels.py:288-459 + the torch error
//                                update at :1867-1873, in ONE pass)
//   quantize_block_kernel        x -> FP8 codes + exponent plane
//                                (tcfp/kernels.py:205-275)
//   pt_* kernels                 per-tensor scaling: a grid-level amax pass
//                                followed by the quantizing pass(es)
//                                (tcfp/core.py:85-158, nn/__init__.py:343-383)
//
// Layout: every CTA owns a tile of 32 rows x 512 columns; a warp owns four
// rows and walks a row in 128-column segments, one 128-bit load per lane, so
// that a scale block of 32/64/128 columns is a group of 8/16/32 lanes and its
// amax is a handful of shuffles.  The tile's exponents are staged in shared
// memory and written out as 32-byte runs of the (K/bs, rows) planes.
#include "common.cuh"
#include "launch.h"

namespace tcfp {

namespace {

// Block quantizers: one CTA per 32-row tile, launched in tile order.  A grid of
// resident CTAs looping over tiles (to trim the partial last wave: 2048 tiles
// on 592 CTA slots are 3.46 waves) was built and measured at 8192^2 -- a
// contiguous tile range per CTA: error-feedback kernel 156 -> 181 us, bf16
// activations 45 -> 38 us; round-robin tiles with the remainder dealt in
// quarter tiles: 156 -> 169 us and 45 -> 44 us, and 20 % slower on the
// 32768 x 4096 / 32768 x 1536 bf16 tensors of a decoder step (likely reason:
// CTAs retiring and starting at their own pace overlap one tile's stores with
// the next one's loads, which a loop with a barrier per tile does not).  The
// plain launch stays.
constexpr int kTileRows = 32;
constexpr int kTileCols = 512;
constexpr int kThreads = 256;

struct f4 { float v[4]; };

template <bool BF16>
__device__ __forceinline__ f4 load4(const void* base, size_t idx) {
  f4 r;
  if constexpr (BF16) {
    uint2 raw = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + idx));
    r.v[0] = __uint_as_float(raw.x << 16);
    r.v[1] = __uint_as_float(raw.x & 0xFFFF0000u);
    r.v[2] = __uint_as_float(raw.y << 16);
    r.v[3] = __uint_as_float(raw.y & 0xFFFF0000u);
  } else {
    float4 raw = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx));
    r.v[0] = raw.x; r.v[1] = raw.y; r.v[2] = raw.z; r.v[3] = raw.w;
  }
  return r;
}

__device__ __forceinline__ f4 load4f(const float* base, size_t idx) {
  float4 raw = *reinterpret_cast<const float4*>(base + idx);
  f4 r; r.v[0] = raw.x; r.v[1] = raw.y; r.v[2] = raw.z; r.v[3] = raw.w;
  return r;
}

__device__ __forceinline__ void store4f(float* base, size_t idx, const f4& x) {
  *reinterpret_cast<float4*>(base + idx) = make_float4(x.v[0], x.v[1], x.v[2], x.v[3]);
}

__device__ __forceinline__ uint32_t pack4(uint8_t a, uint8_t b, uint8_t c, uint8_t d) {
  return (uint32_t)a | ((uint32_t)b << 8) | ((uint32_t)c << 16) | ((uint32_t)d << 24);
}

// max of a non-negative value over aligned groups of GROUP lanes.  A whole
// warp uses one integer warp-reduce (non-negative floats order like their bit
// patterns); for smaller groups the reduce instruction's throughput loses to
// a shuffle tree (measured: block 32 with 8-lane groups 170 vs 153 us at 8192^2).
template <int GROUP>
__device__ __forceinline__ float group_max(float v) {
  if constexpr (GROUP == 32) {
    return __uint_as_float(__reduce_max_sync(0xFFFFFFFFu, __float_as_uint(v)));
  } else {
#pragma unroll
    for (int o = GROUP / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
  }
}

__device__ __forceinline__ float amax4(const f4& x) {
  return fmaxf(fmaxf(fabsf(x.v[0]), fabsf(x.v[1])), fmaxf(fabsf(x.v[2]), fabsf(x.v[3])));
}

// Writes the staged exponents of one tile: planes (K/bs, rows) and, when
// requested, the packed E8M0 chunks.
template <int BS, int TILE_COLS = kTileCols>
__device__ __forceinline__ void flush_tile_scales(const int8_t (*s_exp)[kTileRows], int8_t* plane,
                                                  uint8_t* sf, int64_t rows, int64_t K, int64_t row0,
                                                  int64_t col0) {
  constexpr int kBlocksPerTile = TILE_COLS / BS;
  const int64_t num_kb = K / BS;
  const int64_t kb0 = col0 / BS;
  const int r = threadIdx.x & 31;
  const int64_t row = row0 + r;
  for (int b = threadIdx.x >> 5; b < kBlocksPerTile; b += kThreads / 32) {
    int64_t kb = kb0 + b;
    if (kb < num_kb && row < rows) plane[kb * rows + row] = s_exp[b][r];
  }
  if (sf != nullptr) {
    const int64_t k_groups = (num_kb + 3) >> 2;
    for (int g = threadIdx.x >> 5; g < (kBlocksPerTile + 3) / 4; g += kThreads / 32) {
      int64_t kb = kb0 + 4 * g;
      if (kb < num_kb && row < rows) {
        uint8_t by[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          by[j] = (kb + j < num_kb && 4 * g + j < kBlocksPerTile) ? e8m0_from_exp((int)s_exp[4 * g + j][r])
                                                                  : (uint8_t)127;
        *reinterpret_cast<uint32_t*>(sf + sf_chunk_offset(row, kb, k_groups)) = pack4(by[0], by[1], by[2], by[3]);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// K1a: block-scaled dual quantizer
// ---------------------------------------------------------------------------
template <int BS, bool W_BF16, int MODE>
__global__ void __launch_bounds__(kThreads, (MODE == TCFP_Q_NONE) ? 5 : 4)
dual_quantize_block_kernel(const void* __restrict__ w, float* err, uint8_t* __restrict__ w_hi,
                           uint8_t* __restrict__ w_lo, int8_t* __restrict__ exp_hi,
                           int8_t* __restrict__ exp_lo, uint8_t* __restrict__ sf_hi,
                           uint8_t* __restrict__ sf_lo, int64_t N, int64_t K, uint64_t seed,
                           uint64_t offset) {
  constexpr int GROUP = BS / 4;
  constexpr bool HAS_ERR = (MODE == TCFP_Q_EF || MODE == TCFP_Q_EF_READONLY);
  constexpr int kBlocksPerTile = kTileCols / BS;
  __shared__ int8_t s_hi[kBlocksPerTile][kTileRows];
  __shared__ int8_t s_lo[kBlocksPerTile][kTileRows];

  const int64_t tiles_k = (K + kTileCols - 1) / kTileCols;
  const int64_t row0 = (int64_t)(blockIdx.x / tiles_k) * kTileRows;
  const int64_t col0 = (int64_t)(blockIdx.x % tiles_k) * kTileCols;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

#pragma unroll 1
  for (int rr = 0; rr < 4; ++rr) {
    const int r_local = warp * 4 + rr;
    const int64_t row = row0 + r_local;
    f4 wv[4], ev[4];
    bool ok[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int64_t col = col0 + s * 128 + lane * 4;
      ok[s] = (row < N) && (col < K);
      if (ok[s]) {
        wv[s] = load4<W_BF16>(w, (size_t)row * K + col);
        if constexpr (HAS_ERR) ev[s] = load4f(err, (size_t)row * K + col);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) { wv[s].v[i] = 0.f; ev[s].v[i] = 0.f; }
      }
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int64_t col = col0 + s * 128 + lane * 4;
      f4 wc;
#pragma unroll
      for (int i = 0; i < 4; ++i) wc.v[i] = HAS_ERR ? __fadd_rn(wv[s].v[i], ev[s].v[i]) : wv[s].v[i];
      // --- W_hi
      const int e_hi = block_exponent_fast<false>(group_max<GROUP>(amax4(wc)));
      const float inv_hi = exp2_int(e_hi), fwd_hi = exp2_int(-e_hi);
      // the saturating cast makes the reference's clamp to +-448 implicit
      const uint32_t ph = encode_fp8x2<false>(__fmul_rn(wc.v[0], fwd_hi), __fmul_rn(wc.v[1], fwd_hi)) |
                          (encode_fp8x2<false>(__fmul_rn(wc.v[2], fwd_hi), __fmul_rn(wc.v[3], fwd_hi)) << 16);
      f4 hdq, res;
      {
        const float2 d01 = decode_fp8x2<false>(ph), d23 = decode_fp8x2<false>(ph >> 16);
        hdq.v[0] = __fmul_rn(d01.x, inv_hi); hdq.v[1] = __fmul_rn(d01.y, inv_hi);
        hdq.v[2] = __fmul_rn(d23.x, inv_hi); hdq.v[3] = __fmul_rn(d23.y, inv_hi);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) res.v[i] = __fsub_rn(wc.v[i], hdq.v[i]);
      // --- W_lo
      const float amax_lo = group_max<GROUP>(amax4(res));
      const bool zero_res = amax_lo < kAmaxFloor;
      const int e_lo = block_exponent_fast<false>(amax_lo);
      const float fwd_lo = zero_res ? 1.0f : exp2_int(-e_lo);
      uint32_t pl;
      if constexpr (MODE == TCFP_Q_SRR) {
        uint8_t cl[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float x = clampf(__fmul_rn(res.v[i], fwd_lo), kE4M3Max);
          float u = philox_uniform(seed, offset + (uint64_t)row * (uint64_t)K + (uint64_t)(col + i));
          cl[i] = sr_block_e4m3(x, u);
        }
        pl = pack4(cl[0], cl[1], cl[2], cl[3]);
      } else {
        pl = encode_fp8x2<false>(__fmul_rn(res.v[0], fwd_lo), __fmul_rn(res.v[1], fwd_lo)) |
             (encode_fp8x2<false>(__fmul_rn(res.v[2], fwd_lo), __fmul_rn(res.v[3], fwd_lo)) << 16);
      }
      if (ok[s]) {
        const size_t idx = (size_t)row * K + col;
        *reinterpret_cast<uint32_t*>(w_hi + idx) = ph;
        *reinterpret_cast<uint32_t*>(w_lo + idx) = pl;
        if constexpr (MODE == TCFP_Q_EF) {
          // e' = W - deq(hi) - deq(lo), from the stored codes, against the
          // original weight (tcfp/kernels.py:1870-1873).  The sentinel plane
          // value -128 dequantizes with 2^-128; its codes are all zero.
          const float inv_lo = zero_res ? exp2_int(-128) : exp2_int(e_lo);
          f4 en;
          const float2 l01 = decode_fp8x2<false>(pl), l23 = decode_fp8x2<false>(pl >> 16);
          const float ld[4] = {l01.x, l01.y, l23.x, l23.y};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float t = __fsub_rn(wv[s].v[i], hdq.v[i]);
            en.v[i] = __fsub_rn(t, __fmul_rn(ld[i], inv_lo));
          }
          store4f(err, idx, en);
        }
      }
      if ((lane % GROUP) == 0) {
        const int b = (s * 128 + lane * 4) / BS;
        s_hi[b][r_local] = (int8_t)e_hi;
        s_lo[b][r_local] = zero_res ? (int8_t)-128 : (int8_t)e_lo;
      }
    }
  }
  __syncthreads();
  flush_tile_scales<BS>(s_hi, exp_hi, sf_hi, N, K, row0, col0);
  flush_tile_scales<BS>(s_lo, exp_lo, sf_lo, N, K, row0, col0);
}

// ---------------------------------------------------------------------------
// K2: block-scaled single quantizer (activations E4M3, gradients E5M2)
// One 128-bit load per lane: 4 float32 or 8 bfloat16 values, so a tile is 512
// or 1024 columns wide and a scale block is a group of BS/4 or BS/8 lanes.
// ---------------------------------------------------------------------------
// With COLSUM the kernel also produces the column sums of x (the bias
// gradient when x is the output gradient, tcfp/nn/__init__.py:558, 753, which
// the reference takes in a separate full pass): a CTA walks kColsumRowTiles
// row tiles, keeps per-thread partial sums of its columns, folds the eight
// warps' partials in a fixed order and writes one row of `partial`
// ((row groups) x C floats); colsum_reduce_kernel adds the row groups, again
// in a fixed order, so the result does not depend on scheduling.
constexpr int kColsumRowTiles = 8;

template <int BS, bool X_BF16, bool E5M2, bool COLSUM = false>
__global__ void __launch_bounds__(kThreads)
quantize_block_kernel(const void* __restrict__ x, uint8_t* __restrict__ out, int8_t* __restrict__ exps,
                      uint8_t* __restrict__ sf, __nv_bfloat16* __restrict__ deq, int64_t R, int64_t C,
                      float* __restrict__ partial = nullptr) {
  constexpr int VEC = X_BF16 ? 8 : 4;
  constexpr int GROUP = BS / VEC;
  constexpr int SEG = 32 * VEC;             // columns one warp covers per load
  constexpr int TILE_COLS = 4 * SEG;
  constexpr int kBlocksPerTile = TILE_COLS / BS;
  constexpr int RT = COLSUM ? kColsumRowTiles : 1;
  __shared__ int8_t s_e[kBlocksPerTile][kTileRows];
  __shared__ float s_sum[COLSUM ? kThreads / 32 : 1][COLSUM ? TILE_COLS : 1];

  const int64_t tiles_c = (C + TILE_COLS - 1) / TILE_COLS;
  const int64_t row_group = (int64_t)(blockIdx.x / tiles_c);
  const int64_t col0 = (int64_t)(blockIdx.x % tiles_c) * TILE_COLS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float acc[COLSUM ? 4 : 1][COLSUM ? VEC : 1];
  if constexpr (COLSUM) {
#pragma unroll
    for (int s = 0; s < 4; ++s)
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[s][i] = 0.f;
  }

#pragma unroll 1
  for (int rt = 0; rt < RT; ++rt) {
  const int64_t row0 = (row_group * RT + rt) * kTileRows;
  if (COLSUM && row0 >= R) break;
#pragma unroll 1
  for (int rr = 0; rr < 4; ++rr) {
    const int r_local = warp * 4 + rr;
    const int64_t row = row0 + r_local;
    float xv[4][VEC];
    bool ok[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int64_t col = col0 + s * SEG + lane * VEC;
      ok[s] = (row < R) && (col < C);
      if (ok[s]) {
        if constexpr (X_BF16) {
          uint4 raw = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + (size_t)row * C + col));
          const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            xv[s][2 * i] = __uint_as_float(wds[i] << 16);
            xv[s][2 * i + 1] = __uint_as_float(wds[i] & 0xFFFF0000u);
          }
        } else {
          float4 raw = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + (size_t)row * C + col));
          xv[s][0] = raw.x; xv[s][1] = raw.y; xv[s][2] = raw.z; xv[s][3] = raw.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) xv[s][i] = 0.f;
      }
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int64_t col = col0 + s * SEG + lane * VEC;
      float am = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) am = fmaxf(am, fabsf(xv[s][i]));
      if constexpr (COLSUM) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[s][i] = __fadd_rn(acc[s][i], xv[s][i]);
      }
      const int e = block_exponent_fast<E5M2>(group_max<GROUP>(am));
      const float fwd = exp2_int(-e), inv = exp2_int(e);
      uint32_t pc[VEC / 4];
#pragma unroll
      for (int h = 0; h < VEC / 4; ++h)
        pc[h] = encode_fp8x2<E5M2>(__fmul_rn(xv[s][4 * h], fwd), __fmul_rn(xv[s][4 * h + 1], fwd)) |
                (encode_fp8x2<E5M2>(__fmul_rn(xv[s][4 * h + 2], fwd), __fmul_rn(xv[s][4 * h + 3], fwd)) << 16);
      if (ok[s]) {
        const size_t idx = (size_t)row * C + col;
        if constexpr (VEC == 8) *reinterpret_cast<uint2*>(out + idx) = make_uint2(pc[0], pc[1]);
        else *reinterpret_cast<uint32_t*>(out + idx) = pc[0];
        if (deq != nullptr) {
          uint32_t dq[VEC / 2];
#pragma unroll
          for (int i = 0; i < VEC / 2; ++i) {
            const uint32_t word = pc[i / 2] >> (16 * (i & 1));
            __nv_bfloat162 pr = __floats2bfloat162_rn(__fmul_rn(decode_fp8_fast<E5M2>(word), inv),
                                                     __fmul_rn(decode_fp8_fast<E5M2>(word >> 8), inv));
            dq[i] = *reinterpret_cast<uint32_t*>(&pr);
          }
          if constexpr (VEC == 8) *reinterpret_cast<uint4*>(deq + idx) = make_uint4(dq[0], dq[1], dq[2], dq[3]);
          else *reinterpret_cast<uint2*>(deq + idx) = make_uint2(dq[0], dq[1]);
        }
      }
      if ((lane % GROUP) == 0) s_e[(s * SEG + lane * VEC) / BS][r_local] = (int8_t)e;
    }
  }
  __syncthreads();
  flush_tile_scales<BS, TILE_COLS>(s_e, exps, sf, R, C, row0, col0);
  if constexpr (COLSUM) __syncthreads();      // the next row tile rewrites s_e
  }
  if constexpr (COLSUM) {
#pragma unroll
    for (int s = 0; s < 4; ++s)
#pragma unroll
      for (int i = 0; i < VEC; ++i) s_sum[warp][s * SEG + lane * VEC + i] = acc[s][i];
    __syncthreads();
    for (int c = threadIdx.x; c < TILE_COLS; c += kThreads) {
      float t = s_sum[0][c];
#pragma unroll
      for (int w = 1; w < kThreads / 32; ++w) t = __fadd_rn(t, s_sum[w][c]);
      if (col0 + c < C) partial[row_group * C + col0 + c] = t;
    }
  }
}

// Per-tensor path: one read of x yields its amax (the quantizer's scale) and
// the column sums.  256 rows x 512 columns per CTA, two rows in flight per
// column group.
constexpr int kAcRows = 256;
constexpr int kAcCols = 512;

template <bool X_BF16>
__global__ void __launch_bounds__(kThreads)
amax_colsum_kernel(const void* __restrict__ x, int64_t R, int64_t C, unsigned int* amax_word,
                   float* __restrict__ partial) {
  __shared__ float s_part[kAcCols];
  __shared__ float s_m[kThreads / 32];
  const int cl = threadIdx.x & 127, rl = threadIdx.x >> 7;
  const int64_t col = (int64_t)blockIdx.x * kAcCols + 4 * cl;
  const int64_t r_begin = (int64_t)blockIdx.y * kAcRows;
  const int64_t r_end = r_begin + kAcRows < R ? r_begin + kAcRows : R;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, m = 0.f;
  if (col < C) {
#pragma unroll 4
    for (int64_t r = r_begin + rl; r < r_end; r += 2) {
      const f4 v = load4<X_BF16>(x, (size_t)r * C + col);
      a0 = __fadd_rn(a0, v.v[0]); a1 = __fadd_rn(a1, v.v[1]); a2 = __fadd_rn(a2, v.v[2]); a3 = __fadd_rn(a3, v.v[3]);
      m = fmaxf(m, amax4(v));
    }
  }
  if (rl == 1) { s_part[4 * cl] = a0; s_part[4 * cl + 1] = a1; s_part[4 * cl + 2] = a2; s_part[4 * cl + 3] = a3; }
  m = group_max<32>(m);
  if ((threadIdx.x & 31) == 0) s_m[threadIdx.x >> 5] = m;
  __syncthreads();
  if (rl == 0 && col < C) {
    float* dst = partial + (size_t)blockIdx.y * C + col;
    dst[0] = __fadd_rn(a0, s_part[4 * cl]); dst[1] = __fadd_rn(a1, s_part[4 * cl + 1]);
    dst[2] = __fadd_rn(a2, s_part[4 * cl + 2]); dst[3] = __fadd_rn(a3, s_part[4 * cl + 3]);
  }
  if (threadIdx.x == 0) {
    for (int i = 1; i < kThreads / 32; ++i) m = fmaxf(m, s_m[i]);
    atomicMax(amax_word, __float_as_uint(m));
  }
}

// out[c] = sum over the row groups of partial[g][c], in order
__global__ void colsum_reduce_kernel(const float* __restrict__ partial, int64_t groups, int64_t C, float* __restrict__ out) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float t = 0.f;
  for (int64_t g = 0; g < groups; ++g) t = __fadd_rn(t, partial[g * C + c]);
  out[c] = t;
}

// exponent plane -> packed chunks, one thread per (row, k_group)
__global__ void pack_scales_kernel(const int8_t* __restrict__ exps, uint8_t* __restrict__ sf, int64_t rows,
                                   int64_t num_kb) {
  const int64_t k_groups = (num_kb + 3) >> 2;
  const int64_t rows_pad = (rows + 127) & ~(int64_t)127;
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows_pad * k_groups) return;
  const int64_t row = t % rows_pad, kg = t / rows_pad;
  uint8_t by[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int64_t kb = kg * 4 + j;
    by[j] = (row < rows && kb < num_kb) ? e8m0_from_exp((int)exps[kb * rows + row]) : (uint8_t)127;
  }
  *reinterpret_cast<uint32_t*>(sf + sf_chunk_offset(row, kg * 4, k_groups)) = pack4(by[0], by[1], by[2], by[3]);
}

// block-scaled codes -> bf16 values.  VEC = 16: one 128-bit load of codes and
// two 128-bit stores per thread (16 codes never straddle a scale block);
// VEC = 4 serves arrays that are only 4-byte aligned.  (Two groups per thread,
// half the tensor apart, measured slower inside a training step: 2.39 vs 2.06 ms
// over its 16 launches.)
template <int BS, bool E5M2, int VEC>
__global__ void __launch_bounds__(256)
block_dequantize_bf16_kernel(const uint8_t* __restrict__ codes, const int8_t* __restrict__ exps,
                             __nv_bfloat16* __restrict__ out, int64_t rows, int64_t K, int sentinel_zero) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t idx = t * VEC;
  if (idx >= rows * K) return;
  const int64_t row = idx / K, col = idx % K;
  const int e = (int)__ldg(exps + (col / BS) * rows + row);
  const float s = (sentinel_zero && e == -128) ? 0.f : exp2_int(e);
  uint32_t words[VEC / 4];
  if constexpr (VEC == 16) {
    const uint4 c = __ldg(reinterpret_cast<const uint4*>(codes + idx));
    words[0] = c.x; words[1] = c.y; words[2] = c.z; words[3] = c.w;
  } else {
    words[0] = __ldg(reinterpret_cast<const uint32_t*>(codes + idx));
  }
  uint32_t o[VEC / 2];
#pragma unroll
  for (int w = 0; w < VEC / 4; ++w) {
    const float2 d01 = decode_fp8x2<E5M2>(words[w]), d23 = decode_fp8x2<E5M2>(words[w] >> 16);
    __nv_bfloat162 p0 = __floats2bfloat162_rn(d01.x * s, d01.y * s);
    __nv_bfloat162 p1 = __floats2bfloat162_rn(d23.x * s, d23.y * s);
    o[2 * w] = *reinterpret_cast<uint32_t*>(&p0);
    o[2 * w + 1] = *reinterpret_cast<uint32_t*>(&p1);
  }
  if constexpr (VEC == 16) {
    uint4* dst = reinterpret_cast<uint4*>(out + idx);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  } else {
    *reinterpret_cast<uint2*>(out + idx) = make_uint2(o[0], o[1]);
  }
}

// FP32 -> bf16 head + bf16 tail (x = head + tail to 16 significant bits):
// head = bf16(x), tail = bf16(x - head).  One read of x, two bf16 writes
// (8 B/elem) for what three elementwise torch passes do in 22 B/elem.
__global__ void __launch_bounds__(256)
split_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ head, __nv_bfloat16* __restrict__ tail,
                  int64_t nvec) {
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(x) + v);
    const float xs[4] = {a.x, a.y, a.z, a.w};
    uint32_t h[2], t[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const __nv_bfloat16 h0 = __float2bfloat16_rn(xs[2 * i]), h1 = __float2bfloat16_rn(xs[2 * i + 1]);
      const __nv_bfloat16 t0 = __float2bfloat16_rn(__fsub_rn(xs[2 * i], __bfloat162float(h0)));
      const __nv_bfloat16 t1 = __float2bfloat16_rn(__fsub_rn(xs[2 * i + 1], __bfloat162float(h1)));
      h[i] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
      t[i] = (uint32_t)__bfloat16_as_ushort(t0) | ((uint32_t)__bfloat16_as_ushort(t1) << 16);
    }
    reinterpret_cast<uint2*>(head)[v] = make_uint2(h[0], h[1]);
    reinterpret_cast<uint2*>(tail)[v] = make_uint2(t[0], t[1]);
  }
}

// ---------------------------------------------------------------------------
// Per-tensor scaling: flat passes over the tensor, 4 x 128-bit loads in flight
// per thread.  `reverse` walks the chunks backwards so that a pass starts on
// the tail the previous pass left in L2.
// ---------------------------------------------------------------------------
constexpr int kPtUnroll = 4;
constexpr int kPtChunk = kThreads * kPtUnroll;  // vectors of 4 elements per CTA iteration

// workspace words: [0] amax(W+e) bits, [1] amax(residual) bits
template <bool X_BF16, bool HAS_ERR>
__global__ void __launch_bounds__(kThreads)
pt_amax_kernel(const void* __restrict__ x, const float* __restrict__ err, int64_t nvec, unsigned int* ws) {
  float m = 0.f;
  const int64_t nchunks = (nvec + kPtChunk - 1) / kPtChunk;
  for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
    f4 xv[kPtUnroll], ev[kPtUnroll];
    bool ok[kPtUnroll];
#pragma unroll
    for (int u = 0; u < kPtUnroll; ++u) {
      int64_t v = c * kPtChunk + u * kThreads + threadIdx.x;
      ok[u] = v < nvec;
      if (ok[u]) {
        xv[u] = load4<X_BF16>(x, (size_t)v * 4);
        if constexpr (HAS_ERR) ev[u] = load4f(err, (size_t)v * 4);
      }
    }
#pragma unroll
    for (int u = 0; u < kPtUnroll; ++u) {
      if (!ok[u]) continue;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float w = HAS_ERR ? __fadd_rn(xv[u].v[i], ev[u].v[i]) : xv[u].v[i];
        m = fmaxf(m, fabsf(w));
      }
    }
  }
  m = group_max<32>(m);
  __shared__ float s_m[kThreads / 32];
  if ((threadIdx.x & 31) == 0) s_m[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kThreads / 32; ++i) m = fmaxf(m, s_m[i]);
    atomicMax(ws, __float_as_uint(m));  // non-negative floats order like their bits
  }
}

// scale = FP8_MAX / amax as torch evaluates ``python_float / tensor``
// (tcfp/core.py:100-101): reciprocal of the tensor, then times the scalar --
// two roundings, not one division.
__device__ __forceinline__ float pt_scale(float amax, float fmax) {
  return __fmul_rn(__frcp_rn(fmaxf(amax, kAmaxFloor)), fmax);
}

// single-tensor quantize pass (activations / gradients)
template <bool X_BF16, bool E5M2, bool SR>
__global__ void __launch_bounds__(kThreads)
pt_quantize_kernel(const void* __restrict__ x, uint8_t* __restrict__ out, float* __restrict__ scale_out,
                   int64_t nvec, const unsigned int* ws, const float* amax_in, const float* scale_in,
                   uint64_t seed, uint64_t offset) {
  constexpr float FMAX = E5M2 ? kE5M2Max : kE4M3Max;
  float scale;
  if (scale_in) {
    scale = *scale_in;
  } else {
    const float amax = amax_in ? *amax_in : __uint_as_float(ws[0]);
    if constexpr (X_BF16) {
      // a bf16 tensor keeps its amax, the clamp, the reciprocal and the
      // product with FP8_MAX in bf16 (tcfp/core.py:100-101 on a bf16 input);
      // only the final scale is widened to float32
      const float a = __bfloat162float(__float2bfloat16_rn(fmaxf(amax, kAmaxFloor)));
      const float r = __bfloat162float(__float2bfloat16_rn(__frcp_rn(a)));
      scale = __bfloat162float(__float2bfloat16_rn(__fmul_rn(r, FMAX)));
    } else {
      scale = pt_scale(amax, FMAX);
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) scale_out[0] = __fdiv_rn(1.0f, scale);
  const int64_t nchunks = (nvec + kPtChunk - 1) / kPtChunk;
  for (int64_t cc = blockIdx.x; cc < nchunks; cc += gridDim.x) {
    const int64_t c = nchunks - 1 - cc;
    f4 xv[kPtUnroll];
    bool ok[kPtUnroll];
#pragma unroll
    for (int u = 0; u < kPtUnroll; ++u) {
      int64_t v = c * kPtChunk + u * kThreads + threadIdx.x;
      ok[u] = v < nvec;
      if (ok[u]) xv[u] = load4<X_BF16>(x, (size_t)v * 4);
    }
#pragma unroll
    for (int u = 0; u < kPtUnroll; ++u) {
      if (!ok[u]) continue;
      int64_t v = c * kPtChunk + u * kThreads + threadIdx.x;
      uint32_t pq;
      if constexpr (SR && !E5M2) {
        uint8_t q[4];
        float un[4];
        philox_uniform_x4(seed, offset + (uint64_t)v * 4u, un);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float xs = clampf(__fmul_rn(xv[u].v[i], scale), FMAX);
          q[i] = sr_tensor_e4m3(xs, un[i]);
        }
        pq = pack4(q[0], q[1], q[2], q[3]);
      } else {
        pq = encode_fp8x2<E5M2>(__fmul_rn(xv[u].v[0], scale), __fmul_rn(xv[u].v[1], scale)) |
             (encode_fp8x2<E5M2>(__fmul_rn(xv[u].v[2], scale), __fmul_rn(xv[u].v[3], scale)) << 16);
      }
      *reinterpret_cast<uint32_t*>(out + (size_t)v * 4) = pq;
    }
  }
}

// pass 2 of the weight path: W_hi codes + residual amax
template <bool W_BF16, bool HAS_ERR>
__global__ void __launch_bounds__(kThreads)
pt_hi_kernel(const void* __restrict__ w, const float* __restrict__ err, uint8_t* __restrict__ w_hi, int64_t nvec,
             unsigned int* ws, const float* amax_hi_in) {
  const float amax = amax_hi_in ? *amax_hi_in : __uint_as_float(ws[0]);
  const float scale = pt_scale(amax, kE4M3Max);
  const float inv = __fdiv_rn(1.0f, scale);
  float m = 0.f;
  const int64_t nchunks = (nvec + kPtChunk - 1) / kPtChunk;
  for (int64_t cc = blockIdx.x; cc < nchunks; cc += gridDim.x) {
    const int64_t c = nchunks - 1 - cc;  // reverse: start on what pass 1 left in L2
    f4 xv[kPtUnroll], ev[kPtUnroll];
    bool ok[kPtUnroll];
#pragma unroll
    for (int u = 0; u < kPtUnroll; ++u) {
      int64_t v = c * kPtChunk + u * kThreads + threadIdx.x;
      ok[u] = v < nvec;
      if (ok[u]) {
        xv[u] = load4<W_BF16>(w, (size_t)v * 4);
        if constexpr (HAS_ERR) ev[u] = load4f(err, (size_t)v * 4);
      }
    }
#pragma unroll
    for (int u = 0; u < kPtUnroll; ++u) {
      if (!ok[u]) continue;
      int64_t v = c * kPtChunk + u * kThreads + threadIdx.x;
      f4 wc;
#pragma unroll
      for (int i = 0; i < 4; ++i) wc.v[i] = HAS_ERR ? __fadd_rn(xv[u].v[i], ev[u].v[i]) : xv[u].v[i];
      const uint32_t pq = encode_fp8x2<false>(__fmul_rn(wc.v[0], scale), __fmul_rn(wc.v[1], scale)) |
                          (encode_fp8x2<false>(__fmul_rn(wc.v[2], scale), __fmul_rn(wc.v[3], scale)) << 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float r = __fsub_rn(wc.v[i], __fmul_rn(decode_fp8_fast<false>(pq >> (8 * i)), inv));
        m = fmaxf(m, fabsf(r));
      }
      *reinterpret_cast<uint32_t*>(w_hi + (size_t)v * 4) = pq;
    }
  }
  m = group_max<32>(m);
  __shared__ float s_m[kThreads / 32];
  if ((threadIdx.x & 31) == 0) s_m[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kThreads / 32; ++i) m = fmaxf(m, s_m[i]);
    atomicMax(ws + 1, __float_as_uint(m));
  }
}

// final pass: W_lo codes and the new error.  With FUSED_HI the pass also
// produces W_hi (both scales known up front: delayed scaling with a predicted
// residual amax), making the whole quantizer one read of W and e.
template <bool W_BF16, int MODE, bool FUSED_HI>
__global__ void __launch_bounds__(kThreads)
pt_lo_kernel(const void* __restrict__ w, float* err, uint8_t* w_hi, uint8_t* __restrict__ w_lo,
             float* __restrict__ scale_hi, float* __restrict__ scale_lo, float* __restrict__ amax_out,
             int64_t nvec, unsigned int* ws, const float* amax_hi_in, const float* amax_lo_in, uint64_t seed,
             uint64_t offset) {
  constexpr bool HAS_ERR = (MODE == TCFP_Q_EF || MODE == TCFP_Q_EF_READONLY);
  const float amax_hi = amax_hi_in ? *amax_hi_in : __uint_as_float(ws[0]);
  const float sc_hi = pt_scale(amax_hi, kE4M3Max);
  const float inv_hi = __fdiv_rn(1.0f, sc_hi);
  const float amax_lo = amax_lo_in ? *amax_lo_in : __uint_as_float(ws[1]);
  const float sc_lo = pt_scale(amax_lo, kE4M3Max);
  const float inv_lo = __fdiv_rn(1.0f, sc_lo);
  if (!FUSED_HI && blockIdx.x == 0 && threadIdx.x == 0) {
    scale_hi[0] = inv_hi;
    scale_lo[0] = inv_lo;
    if (amax_out) { amax_out[0] = __uint_as_float(ws[0]); amax_out[1] = __uint_as_float(ws[1]); }
  }
  float m = 0.f;
  const int64_t nchunks = (nvec + kPtChunk - 1) / kPtChunk;
  for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
    f4 xv[kPtUnroll], ev[kPtUnroll];
    uint32_t hv[kPtUnroll];
    bool ok[kPtUnroll];
#pragma unroll
    for (int u = 0; u < kPtUnroll; ++u) {
      int64_t v = c * kPtChunk + u * kThreads + threadIdx.x;
      ok[u] = v < nvec;
      if (ok[u]) {
        xv[u] = load4<W_BF16>(w, (size_t)v * 4);
        if constexpr (HAS_ERR) ev[u] = load4f(err, (size_t)v * 4);
        if constexpr (!FUSED_HI) hv[u] = *reinterpret_cast<const uint32_t*>(w_hi + (size_t)v * 4);
      }
    }
#pragma unroll
    for (int u = 0; u < kPtUnroll; ++u) {
      if (!ok[u]) continue;
      int64_t v = c * kPtChunk + u * kThreads + threadIdx.x;
      uint8_t qh[4], ql[4];
      f4 en;
      float un[4];
      if constexpr (MODE == TCFP_Q_SRR) philox_uniform_x4(seed, offset + (uint64_t)v * 4u, un);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float wc = HAS_ERR ? __fadd_rn(xv[u].v[i], ev[u].v[i]) : xv[u].v[i];
        if constexpr (FUSED_HI) qh[i] = encode_fp8<false>(__fmul_rn(wc, sc_hi));
        else qh[i] = (uint8_t)(hv[u] >> (8 * i));
        float hdeq = __fmul_rn(decode_fp8_fast<false>(qh[i]), inv_hi);
        float r = __fsub_rn(wc, hdeq);
        if constexpr (FUSED_HI) m = fmaxf(m, fabsf(r));
        float xs = clampf(__fmul_rn(r, sc_lo), kE4M3Max);
        if constexpr (MODE == TCFP_Q_SRR) {
          ql[i] = sr_tensor_e4m3(xs, un[i]);
        } else {
          ql[i] = encode_fp8<false>(xs);
        }
        if constexpr (MODE == TCFP_Q_EF) {
          // tcfp/nn/__init__.py:379-382: W - (hi*inv_hi + lo*inv_lo)
          float recon = __fadd_rn(hdeq, __fmul_rn(decode_fp8_fast<false>(ql[i]), inv_lo));
          en.v[i] = __fsub_rn(xv[u].v[i], recon);
        }
      }
      if constexpr (FUSED_HI) *reinterpret_cast<uint32_t*>(w_hi + (size_t)v * 4) = pack4(qh[0], qh[1], qh[2], qh[3]);
      *reinterpret_cast<uint32_t*>(w_lo + (size_t)v * 4) = pack4(ql[0], ql[1], ql[2], ql[3]);
      if constexpr (MODE == TCFP_Q_EF) store4f(err, (size_t)v * 4, en);
    }
  }
  if constexpr (FUSED_HI) {
    m = group_max<32>(m);
    __shared__ float s_m[kThreads / 32];
    if ((threadIdx.x & 31) == 0) s_m[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 1; i < kThreads / 32; ++i) m = fmaxf(m, s_m[i]);
      atomicMax(ws + 1, __float_as_uint(m));
    }
  }
}

// writes the scalar outputs of the fused path after the grid has finished
__global__ void pt_finalize_kernel(float* scale_hi, float* scale_lo, float* amax_out, const unsigned int* ws,
                                   const float* amax_hi_in, const float* amax_lo_in) {
  const float amax_hi = amax_hi_in ? *amax_hi_in : __uint_as_float(ws[0]);
  const float amax_lo = amax_lo_in ? *amax_lo_in : __uint_as_float(ws[1]);
  scale_hi[0] = __fdiv_rn(1.0f, pt_scale(amax_hi, kE4M3Max));
  scale_lo[0] = __fdiv_rn(1.0f, pt_scale(amax_lo, kE4M3Max));
  if (amax_out) { amax_out[0] = __uint_as_float(ws[0]); amax_out[1] = __uint_as_float(ws[1]); }
}

int flat_grid(int64_t nvec) {
  int64_t nchunks = (nvec + kPtChunk - 1) / kPtChunk;
  int64_t cap = (int64_t)sm_count() * 8;
  return (int)(nchunks < cap ? (nchunks > 0 ? nchunks : 1) : cap);
}

#define DISPATCH_BS(bs, ...)                         \
  switch (bs) {                                      \
    case 32: { constexpr int BS = 32; __VA_ARGS__; } break;   \
    case 64: { constexpr int BS = 64; __VA_ARGS__; } break;   \
    case 128: { constexpr int BS = 128; __VA_ARGS__; } break; \
    default: return fail(TCFP_ERR_INVALID, "block_size must be 32, 64, or 128, got %d", (int)(bs)); \
  }

#define DISPATCH_BOOL(flag, NAME, ...)                \
  if (flag) { constexpr bool NAME = true; __VA_ARGS__; } \
  else { constexpr bool NAME = false; __VA_ARGS__; }

#define DISPATCH_MODE(mode, ...)                                                       \
  switch (mode) {                                                                      \
    case TCFP_Q_NONE: { constexpr int MODE = TCFP_Q_NONE; __VA_ARGS__; } break;        \
    case TCFP_Q_EF: { constexpr int MODE = TCFP_Q_EF; __VA_ARGS__; } break;            \
    case TCFP_Q_EF_READONLY: { constexpr int MODE = TCFP_Q_EF_READONLY; __VA_ARGS__; } break; \
    case TCFP_Q_SRR: { constexpr int MODE = TCFP_Q_SRR; __VA_ARGS__; } break;          \
    default: return fail(TCFP_ERR_INVALID, "unknown quantizer mode %d", (int)(mode));  \
  }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace tcfp

using namespace tcfp;

extern "C" size_t tcfp_dual_quantize_workspace_bytes(void) { return 256; }

extern "C" int32_t tcfp_absmax(const void* x, int32_t x_dtype, const float* err, int64_t numel, float* amax_out,
                               void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!x || !amax_out) return fail(TCFP_ERR_INVALID, "absmax: NULL pointer");
  if (numel <= 0 || numel % 4 != 0) return fail(TCFP_ERR_INVALID, "absmax: numel must be a positive multiple of 4");
  if (x_dtype != TCFP_F32 && x_dtype != TCFP_BF16) return fail(TCFP_ERR_INVALID, "absmax: input must be float32 or bfloat16");
  const bool bf16 = (x_dtype == TCFP_BF16);
  if (((uintptr_t)x & (bf16 ? 7 : 15)) || (err && !aligned16(err))) return fail(TCFP_ERR_INVALID, "absmax: misaligned tensor");
  const int64_t nvec = numel / 4;
  CUDA_TRY(cudaMemsetAsync(amax_out, 0, 4, stream));
  // the bits of a non-negative float order like unsigned integers, so the
  // output word doubles as the atomic-max target
  DISPATCH_BOOL(bf16, X_BF16, DISPATCH_BOOL(err != nullptr, HAS_ERR,
    pt_amax_kernel<X_BF16, HAS_ERR><<<flat_grid(nvec), kThreads, 0, stream>>>(x, err, nvec, (unsigned int*)amax_out)));
  CUDA_TRY(cudaGetLastError());
  return TCFP_OK;
}

extern "C" size_t tcfp_sf_packed_bytes(int64_t rows, int64_t K, int32_t block_size) {
  if (rows <= 0 || K <= 0 || block_size <= 0) return 0;
  int64_t num_kb = K / block_size;
  return (size_t)(((rows + 127) / 128) * ((num_kb + 3) / 4) * 512);
}

extern "C" int32_t tcfp_dual_quantize(const void* w, int32_t w_dtype, float* err, uint8_t* w_hi, uint8_t* w_lo,
                                      void* scale_hi, void* scale_lo, uint8_t* sf_hi, uint8_t* sf_lo, int64_t N,
                                      int64_t K, int32_t block_size, int32_t mode, uint64_t seed, uint64_t offset,
                                      const float* amax_hi_in, const float* amax_lo_in, float* amax_out,
                                      void* workspace, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!w || !w_hi || !w_lo || !scale_hi || !scale_lo) return fail(TCFP_ERR_INVALID, "dual_quantize: NULL pointer");
  if (N <= 0 || K <= 0) return fail(TCFP_ERR_INVALID, "dual_quantize: empty shape (%lld, %lld)", (long long)N, (long long)K);
  if (w_dtype != TCFP_F32 && w_dtype != TCFP_BF16) return fail(TCFP_ERR_INVALID, "dual_quantize: weight must be float32 or bfloat16");
  const bool has_err = (mode == TCFP_Q_EF || mode == TCFP_Q_EF_READONLY);
  if (has_err && !err) return fail(TCFP_ERR_INVALID, "dual_quantize: error-feedback mode needs an error buffer");
  if (!has_err && err) return fail(TCFP_ERR_INVALID, "dual_quantize: stochastic_lo / no-EF modes and error_buf are mutually exclusive");
  if (K % 4 != 0 || !aligned16(w) || (err && !aligned16(err)) || ((uintptr_t)w_hi & 3) || ((uintptr_t)w_lo & 3))
    return fail(TCFP_ERR_INVALID, "dual_quantize: tensors must be contiguous, 16-byte aligned, K %% 4 == 0");
  const bool bf16 = (w_dtype == TCFP_BF16);

  if (block_size != 0) {
    if (block_size != 32 && block_size != 64 && block_size != 128)
      return fail(TCFP_ERR_INVALID, "block_size must be 32, 64, or 128, got %d", block_size);
    if (K % block_size != 0)
      return fail(TCFP_ERR_INVALID, "K (%lld) must be divisible by block_size (%d)", (long long)K, block_size);
    const int64_t num_kb = K / block_size;
    if ((sf_hi || sf_lo) && (num_kb % 4 != 0)) {
      // chunk tails beyond the last scale block must hold a finite scale
      size_t bytes = tcfp_sf_packed_bytes(N, K, block_size);
      if (sf_hi) CUDA_TRY(cudaMemsetAsync(sf_hi, 127, bytes, stream));
      if (sf_lo) CUDA_TRY(cudaMemsetAsync(sf_lo, 127, bytes, stream));
    }
    const int64_t tiles = ((N + kTileRows - 1) / kTileRows) * ((K + kTileCols - 1) / kTileCols);
    if (tiles > 0x7FFFFFFF) return fail(TCFP_ERR_UNSUPPORTED, "dual_quantize: tensor too large");
    DISPATCH_BS(block_size, DISPATCH_BOOL(bf16, W_BF16, DISPATCH_MODE(mode,
      dual_quantize_block_kernel<BS, W_BF16, MODE><<<(unsigned)tiles, kThreads, 0, stream>>>(
          w, err, w_hi, w_lo, (int8_t*)scale_hi, (int8_t*)scale_lo, sf_hi, sf_lo, N, K, seed, offset))));
    CUDA_TRY(cudaGetLastError());
    return TCFP_OK;
  }

  // ---- per-tensor
  if (!workspace) return fail(TCFP_ERR_INVALID, "dual_quantize: per-tensor scaling needs a workspace");
  unsigned int* ws = (unsigned int*)workspace;
  const int64_t nvec = N * K / 4;
  const int grid = flat_grid(nvec);
  CUDA_TRY(cudaMemsetAsync(ws, 0, 8, stream));
  // pass 1: amax(W + e), skipped when the caller supplies the amax to use
  if (!amax_hi_in) {
    DISPATCH_BOOL(bf16, W_BF16, DISPATCH_BOOL(has_err, HAS_ERR,
      pt_amax_kernel<W_BF16, HAS_ERR><<<grid, kThreads, 0, stream>>>(w, err, nvec, ws)));
  }
  if (amax_lo_in) {
    DISPATCH_BOOL(bf16, W_BF16, DISPATCH_MODE(mode,
      pt_lo_kernel<W_BF16, MODE, true><<<grid, kThreads, 0, stream>>>(
          w, err, w_hi, w_lo, (float*)scale_hi, (float*)scale_lo, amax_out, nvec, ws, amax_hi_in, amax_lo_in, seed, offset)));
    pt_finalize_kernel<<<1, 1, 0, stream>>>((float*)scale_hi, (float*)scale_lo, amax_out, ws, amax_hi_in, amax_lo_in);
  } else {
    DISPATCH_BOOL(bf16, W_BF16, DISPATCH_BOOL(has_err, HAS_ERR,
      pt_hi_kernel<W_BF16, HAS_ERR><<<grid, kThreads, 0, stream>>>(w, err, w_hi, nvec, ws, amax_hi_in)));
    DISPATCH_BOOL(bf16, W_BF16, DISPATCH_MODE(mode,
      pt_lo_kernel<W_BF16, MODE, false><<<grid, kThreads, 0, stream>>>(
          w, err, w_hi, w_lo, (float*)scale_hi, (float*)scale_lo, amax_out, nvec, ws, amax_hi_in, amax_lo_in, seed, offset)));
  }
  CUDA_TRY(cudaGetLastError());
  return TCFP_OK;
}

extern "C" int32_t tcfp_quantize(const void* x, int32_t x_dtype, uint8_t* out, void* scale_out, uint8_t* sf_out,
                                 void* deq_bf16_out, int64_t R, int64_t C, int32_t block_size, int32_t fmt,
                                 const float* amax_in, const float* scale_in, int32_t stochastic, uint64_t seed,
                                 uint64_t offset, void* workspace, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!x || !out || !scale_out) return fail(TCFP_ERR_INVALID, "quantize: NULL pointer");
  if (R <= 0 || C <= 0) return fail(TCFP_ERR_INVALID, "quantize: empty shape (%lld, %lld)", (long long)R, (long long)C);
  if (x_dtype != TCFP_F32 && x_dtype != TCFP_BF16) return fail(TCFP_ERR_INVALID, "quantize: input must be float32 or bfloat16");
  if (fmt != TCFP_E4M3 && fmt != TCFP_E5M2) return fail(TCFP_ERR_INVALID, "quantize: unknown FP8 format %d", fmt);
  const bool bf16 = (x_dtype == TCFP_BF16), e5m2 = (fmt == TCFP_E5M2);
  if (C % 4 != 0 || ((uintptr_t)x & (bf16 ? 7 : 15)) || ((uintptr_t)out & 3))
    return fail(TCFP_ERR_INVALID, "quantize: tensors must be contiguous, aligned, C %% 4 == 0");
  if (block_size != 0 && bf16 && (((uintptr_t)x & 15) || ((uintptr_t)out & 7) || ((uintptr_t)deq_bf16_out & 15)))
    return fail(TCFP_ERR_INVALID, "quantize: bfloat16 block quantization needs 16-byte aligned tensors");
  if (stochastic && (block_size != 0 || e5m2))
    return fail(TCFP_ERR_UNSUPPORTED, "quantize: stochastic rounding is per-tensor E4M3 only");
  if (block_size != 0) {
    if (block_size != 32 && block_size != 64 && block_size != 128)
      return fail(TCFP_ERR_INVALID, "block_size must be 32, 64, or 128, got %d", block_size);
    if (C % block_size != 0)
      return fail(TCFP_ERR_INVALID, "K (%lld) must be divisible by block_size (%d)", (long long)C, block_size);
    if (sf_out && ((C / block_size) % 4 != 0))
      CUDA_TRY(cudaMemsetAsync(sf_out, 127, tcfp_sf_packed_bytes(R, C, block_size), stream));
    const int64_t tile_cols = bf16 ? 2 * kTileCols : kTileCols;
    const int64_t tiles = ((R + kTileRows - 1) / kTileRows) * ((C + tile_cols - 1) / tile_cols);
    if (tiles > 0x7FFFFFFF) return fail(TCFP_ERR_UNSUPPORTED, "quantize: tensor too large");
    DISPATCH_BS(block_size, DISPATCH_BOOL(bf16, X_BF16, DISPATCH_BOOL(e5m2, E5M2,
      quantize_block_kernel<BS, X_BF16, E5M2><<<(unsigned)tiles, kThreads, 0, stream>>>(
          x, out, (int8_t*)scale_out, sf_out, (__nv_bfloat16*)deq_bf16_out, R, C))));
    CUDA_TRY(cudaGetLastError());
    return TCFP_OK;
  }
  const bool given = amax_in || scale_in;
  if (!workspace && !given) return fail(TCFP_ERR_INVALID, "quantize: per-tensor scaling needs a workspace");
  unsigned int* ws = (unsigned int*)workspace;
  const int64_t nvec = R * C / 4;
  const int grid = flat_grid(nvec);
  if (!given) {
    CUDA_TRY(cudaMemsetAsync(ws, 0, 8, stream));
    DISPATCH_BOOL(bf16, X_BF16, pt_amax_kernel<X_BF16, false><<<grid, kThreads, 0, stream>>>(x, nullptr, nvec, ws));
  }
  if (stochastic) {
    DISPATCH_BOOL(bf16, X_BF16,
      pt_quantize_kernel<X_BF16, false, true><<<grid, kThreads, 0, stream>>>(x, out, (float*)scale_out, nvec, ws, amax_in, scale_in, seed, offset));
  } else {
    DISPATCH_BOOL(bf16, X_BF16, DISPATCH_BOOL(e5m2, E5M2,
      pt_quantize_kernel<X_BF16, E5M2, false><<<grid, kThreads, 0, stream>>>(x, out, (float*)scale_out, nvec, ws, amax_in, scale_in, 0, 0)));
  }
  CUDA_TRY(cudaGetLastError());
  return TCFP_OK;
}

extern "C" size_t tcfp_colsum_workspace_bytes(int64_t R, int64_t C) {
  if (R <= 0 || C <= 0) return 0;
  // one row of partial sums per 256 input rows (both scaling modes), plus the amax words
  return (size_t)(((R + 255) / 256) * C) * sizeof(float) + 256;
}

extern "C" int32_t tcfp_quantize_colsum(const void* x, int32_t x_dtype, uint8_t* out, void* scale_out, uint8_t* sf_out,
                                        int64_t R, int64_t C, int32_t block_size, int32_t fmt, float* colsum_out,
                                        void* workspace, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!x || !out || !scale_out || !colsum_out || !workspace) return fail(TCFP_ERR_INVALID, "quantize_colsum: NULL pointer");
  if (R <= 0 || C <= 0) return fail(TCFP_ERR_INVALID, "quantize_colsum: empty shape (%lld, %lld)", (long long)R, (long long)C);
  if (x_dtype != TCFP_F32 && x_dtype != TCFP_BF16) return fail(TCFP_ERR_INVALID, "quantize_colsum: input must be float32 or bfloat16");
  if (fmt != TCFP_E4M3 && fmt != TCFP_E5M2) return fail(TCFP_ERR_INVALID, "quantize_colsum: unknown FP8 format %d", fmt);
  const bool bf16 = (x_dtype == TCFP_BF16), e5m2 = (fmt == TCFP_E5M2);
  if (C % 4 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)out & 7) || ((uintptr_t)workspace & 15) || (bf16 && C % 8 != 0))
    return fail(TCFP_ERR_INVALID, "quantize_colsum: tensors must be contiguous and 16-byte aligned, C %% 4 == 0 (8 for bfloat16)");
  float* partial = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + 256);
  unsigned int* ws = reinterpret_cast<unsigned int*>(workspace);
  int64_t groups;
  if (block_size != 0) {
    if (block_size != 32 && block_size != 64 && block_size != 128)
      return fail(TCFP_ERR_INVALID, "block_size must be 32, 64, or 128, got %d", block_size);
    if (C % block_size != 0)
      return fail(TCFP_ERR_INVALID, "K (%lld) must be divisible by block_size (%d)", (long long)C, block_size);
    if (sf_out && ((C / block_size) % 4 != 0))
      CUDA_TRY(cudaMemsetAsync(sf_out, 127, tcfp_sf_packed_bytes(R, C, block_size), stream));
    const int64_t tile_cols = bf16 ? 2 * kTileCols : kTileCols;
    groups = (R + kTileRows * kColsumRowTiles - 1) / (kTileRows * kColsumRowTiles);
    const int64_t ctas = groups * ((C + tile_cols - 1) / tile_cols);
    if (ctas > 0x7FFFFFFF) return fail(TCFP_ERR_UNSUPPORTED, "quantize_colsum: tensor too large");
    DISPATCH_BS(block_size, DISPATCH_BOOL(bf16, X_BF16, DISPATCH_BOOL(e5m2, E5M2,
      quantize_block_kernel<BS, X_BF16, E5M2, true><<<(unsigned)ctas, kThreads, 0, stream>>>(
          x, out, (int8_t*)scale_out, sf_out, nullptr, R, C, partial))));
  } else {
    groups = (R + kAcRows - 1) / kAcRows;
    if (groups > 65535) return fail(TCFP_ERR_UNSUPPORTED, "quantize_colsum: more than 16M rows");
    CUDA_TRY(cudaMemsetAsync(ws, 0, 8, stream));
    const dim3 grid((unsigned)((C + kAcCols - 1) / kAcCols), (unsigned)groups, 1);
    DISPATCH_BOOL(bf16, X_BF16, amax_colsum_kernel<X_BF16><<<grid, kThreads, 0, stream>>>(x, R, C, ws, partial));
    const int64_t nvec = R * C / 4;
    DISPATCH_BOOL(bf16, X_BF16, DISPATCH_BOOL(e5m2, E5M2,
      pt_quantize_kernel<X_BF16, E5M2, false><<<flat_grid(nvec), kThreads, 0, stream>>>(
          x, out, (float*)scale_out, nvec, ws, nullptr, nullptr, 0, 0)));
  }
  colsum_reduce_kernel<<<(unsigned)((C + 255) / 256), 256, 0, stream>>>(partial, groups, C, colsum_out);
  CUDA_TRY(cudaGetLastError());
  return TCFP_OK;
}

extern "C" int32_t tcfp_pack_scales(const int8_t* exps, uint8_t* sf_out, int64_t rows, int64_t K, int32_t block_size,
                                    void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!exps || !sf_out) return fail(TCFP_ERR_INVALID, "pack_scales: NULL pointer");
  if (block_size != 32 && block_size != 64 && block_size != 128)
    return fail(TCFP_ERR_INVALID, "block_size must be 32, 64, or 128, got %d", block_size);
  if (rows <= 0 || K <= 0 || K % block_size != 0)
    return fail(TCFP_ERR_INVALID, "K (%lld) must be divisible by block_size (%d)", (long long)K, block_size);
  const int64_t num_kb = K / block_size;
  const int64_t total = ((rows + 127) / 128 * 128) * ((num_kb + 3) / 4);
  pack_scales_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(exps, sf_out, rows, num_kb);
  CUDA_TRY(cudaGetLastError());
  return TCFP_OK;
}

extern "C" int32_t tcfp_block_dequantize_bf16(const uint8_t* codes, const int8_t* exps, void* out_bf16, int64_t rows,
                                              int64_t K, int32_t block_size, int32_t fmt, int32_t sentinel_zero,
                                              void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!codes || !exps || !out_bf16) return fail(TCFP_ERR_INVALID, "block_dequantize: NULL pointer");
  if (rows <= 0 || K <= 0 || K % 4 != 0) return fail(TCFP_ERR_INVALID, "block_dequantize: bad shape");
  if (K % (block_size > 0 ? block_size : 1) != 0)
    return fail(TCFP_ERR_INVALID, "K (%lld) must be divisible by block_size (%d)", (long long)K, block_size);
  const bool wide = (((uintptr_t)codes | (uintptr_t)out_bf16) & 15u) == 0 && K % 16 == 0;
  const int64_t threads = rows * K / (wide ? 16 : 4);
  if ((threads + 255) / 256 > 0x7FFFFFFF) return fail(TCFP_ERR_UNSUPPORTED, "block_dequantize: tensor too large");
  const unsigned grid = (unsigned)((threads + 255) / 256);
  const bool e5m2 = (fmt == TCFP_E5M2);
  if (wide) {
    DISPATCH_BS(block_size, DISPATCH_BOOL(e5m2, E5M2,
      block_dequantize_bf16_kernel<BS, E5M2, 16><<<grid, 256, 0, stream>>>(codes, exps, (__nv_bfloat16*)out_bf16, rows, K, sentinel_zero)));
  } else {
    DISPATCH_BS(block_size, DISPATCH_BOOL(e5m2, E5M2,
      block_dequantize_bf16_kernel<BS, E5M2, 4><<<grid, 256, 0, stream>>>(codes, exps, (__nv_bfloat16*)out_bf16, rows, K, sentinel_zero)));
  }
  CUDA_TRY(cudaGetLastError());
  return TCFP_OK;
}

extern "C" int32_t tcfp_split_bf16(const float* x, void* head_bf16, void* tail_bf16, int64_t n, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (!x || !head_bf16 || !tail_bf16) return fail(TCFP_ERR_INVALID, "split_bf16: NULL pointer");
  if (n <= 0 || n % 4 != 0) return fail(TCFP_ERR_INVALID, "split_bf16: element count (%lld) must be a positive multiple of 4", (long long)n);
  if (((uintptr_t)x & 15u) || (((uintptr_t)head_bf16 | (uintptr_t)tail_bf16) & 7u))
    return fail(TCFP_ERR_INVALID, "split_bf16: input must be 16-byte aligned, outputs 8-byte aligned");
  const int64_t nvec = n / 4;
  const int64_t want = (nvec + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  split_bf16_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, stream>>>(
      x, (__nv_bfloat16*)head_bf16, (__nv_bfloat16*)tail_bf16, nvec);
  CUDA_TRY(cudaGetLastError());
  return TCFP_OK;
}
