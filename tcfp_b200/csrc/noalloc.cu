// Block-scaled dual GEMM for callers that cannot allocate device memory.
//
// The regular route from reference-layout scales (int8 exponent planes of
// shape (K/bs, rows)) to the tensor-core GEMM needs three scratch arrays for
// the re-packed E8M0 scale factors; tcfp_pack_scales() writes them into
// buffers the caller allocated.  Some callers have no allocator to ask: code
// running inside a region where cudaMalloc is forbidden or would synchronise
// (a latency-critical serving loop, a plugin that was handed only its input
// and output buffers by a host framework that owns all device memory).  For
// them this file keeps the scratch in a fixed array that is part of the
// library image.
#include <mutex>

#include "launch.h"

namespace {

// 2 MiB per operand: enough for an 8192 x 8192 operand at block size 32
// (64 row blocks x 64 K groups x 512 B).  Every GPU that loads the library
// holds these 6 MiB until the process exits.
constexpr size_t kRegionBytes = 2u << 20;
static __device__ __align__(256) unsigned char g_static_sf_scratch[3 * kRegionBytes];

std::mutex g_mu;
unsigned char* g_scratch_ptr[64] = {nullptr};

// The array's name is only a host-side handle; the device address has to be
// asked for, once per device, while that device is current.
int scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return tcfp::fail(TCFP_ERR_UNSUPPORTED, "static scratch: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(&p, g_static_sf_scratch));
    g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_ptr[dev];
  return TCFP_OK;
}

}  // namespace

extern "C" size_t tcfp_static_scratch_bytes_per_operand(void) { return kRegionBytes; }

extern "C" int32_t tcfp_block_dual_gemm_static(const uint8_t* a, const int8_t* exp_a, const uint8_t* w_hi,
                                               const int8_t* exp_hi, const uint8_t* w_lo, const int8_t* exp_lo,
                                               const float* bias, void* out, int32_t out_dtype, int64_t M, int64_t N,
                                               int64_t K, int32_t block_size, void* stream) {
  if (!a || !exp_a || !w_hi || !exp_hi || !out) return tcfp::fail(TCFP_ERR_INVALID, "block_dual_gemm_static: NULL pointer");
  if ((w_lo == nullptr) != (exp_lo == nullptr))
    return tcfp::fail(TCFP_ERR_INVALID, "block_dual_gemm_static: w_lo and exp_lo go together");
  if (block_size != 32 && block_size != 64 && block_size != 128)
    return tcfp::fail(TCFP_ERR_INVALID, "block_size must be 32, 64, or 128, got %d", block_size);
  if (M <= 0 || N <= 0 || K <= 0 || K % block_size != 0)
    return tcfp::fail(TCFP_ERR_INVALID, "block_dual_gemm_static: bad shape M=%lld N=%lld K=%lld", (long long)M,
                      (long long)N, (long long)K);
  // everything the GEMM entry point would refuse is refused here, before the first
  // pack kernel runs: a rejected call must leave the shared scratch as it found it
  if (out_dtype != TCFP_F32 && out_dtype != TCFP_BF16)
    return tcfp::fail(TCFP_ERR_INVALID, "block_dual_gemm_static: output must be float32 or bfloat16");
  if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF || (K % 16) != 0 || (N % (out_dtype == TCFP_BF16 ? 8 : 4)) != 0 ||
      (((uintptr_t)a | (uintptr_t)w_hi | (uintptr_t)w_lo | (uintptr_t)out) & 15u))
    return tcfp::fail(TCFP_ERR_INVALID,
                      "block_dual_gemm_static: operands need 16-byte aligned base pointers and row pitches");
  const size_t need_a = tcfp_sf_packed_bytes(M, K, block_size);
  const size_t need_w = tcfp_sf_packed_bytes(N, K, block_size);
  if (need_a > kRegionBytes || need_w > kRegionBytes)
    return tcfp::fail(TCFP_ERR_UNSUPPORTED,
                      "block_dual_gemm_static: packed scale factors need %zu / %zu bytes, the built-in scratch holds %zu "
                      "per operand; use tcfp_pack_scales + tcfp_block_dual_gemm with caller-allocated buffers",
                      need_a, need_w, kRegionBytes);
  unsigned char* base = nullptr;
  int rc = scratch_for_current_device(&base);
  if (rc != TCFP_OK) return rc;
  uint8_t* sf_a = base;
  uint8_t* sf_hi = base + kRegionBytes;
  uint8_t* sf_lo = base + 2 * kRegionBytes;
  // the pack kernel writes every byte of the chunks it covers, padding
  // included, so nothing left by an earlier call can leak into this one
  if ((rc = tcfp_pack_scales(exp_a, sf_a, M, K, block_size, stream)) != TCFP_OK) return rc;
  if ((rc = tcfp_pack_scales(exp_hi, sf_hi, N, K, block_size, stream)) != TCFP_OK) return rc;
  if (w_lo && (rc = tcfp_pack_scales(exp_lo, sf_lo, N, K, block_size, stream)) != TCFP_OK) return rc;
  return tcfp_block_dual_gemm(a, sf_a, w_hi, sf_hi, w_lo, w_lo ? sf_lo : nullptr, bias, out, out_dtype, M, N, K,
                              block_size, stream);
}
