/*
 * tcfp_b200 -- C ABI of the B200 (sm_100a) TCFP-12 linear-layer hot path.
 *
 * This header is the whole drop-in boundary: plain pointers, sizes and enums,
 * no framework types.  It replaces the two native/JIT surfaces of the
 * reference project:
 *
 *   - the pybind11 module built from tcfp/csrc/fused_dual_gemm.{h,cu} and
 *     tcfp/csrc/fused_dual_gemm_bind.cpp (``forward`` / ``backward_dx``,
 *     loaded by tcfp/cuda_ext.py:155-282), and
 *   - the Triton kernels and their Python launch wrappers in tcfp/kernels.py
 *     (``fused_dual_gemm_forward`` :1545, ``fused_dual_gemm_backward_dx``
 *     :1604, ``block_quantize_fp8`` :1675, ``fused_dual_quantize_fp8`` :1749,
 *     ``fused_block_scaled_dual_gemm_forward`` :1939,
 *     ``fused_block_scaled_backward_dx`` :2326), plus the torch elementwise
 *     chains of tcfp/core.py:85-158 and tcfp/nn/__init__.py:343-383.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in ``_host``;
 *     a parameter documented "nullable" may be NULL;
 *   - matrices are dense row-major; weights are (N, K) = (out, in) as in
 *     ``nn.Linear``;
 *   - every entry point returns 0 on success or a negative TCFP_ERR_* code,
 *     never throws, never traps the device; the text of the last failure on
 *     the calling thread is available through tcfp_last_error();
 *   - work is enqueued on ``stream`` (a cudaStream_t passed as void*) of the
 *     CURRENT device; nothing synchronises unless documented;
 *   - the library never allocates device memory: scratch comes in through
 *     ``workspace`` arguments sized by tcfp_*_workspace_bytes().
 */
#ifndef TCFP_B200_H_
#define TCFP_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
#define TCFP_OK                 0
#define TCFP_ERR_INVALID       -1   /* bad argument (shape, enum, NULL, alignment) */
#define TCFP_ERR_UNSUPPORTED   -2   /* valid request this build cannot serve      */
#define TCFP_ERR_CUDA          -3   /* a CUDA runtime/driver call failed          */
#define TCFP_ERR_DEVICE        -4   /* a kernel reported a bounded wait that ran out */

/* ---- enums ------------------------------------------------------------- */
typedef enum { TCFP_F32 = 0, TCFP_BF16 = 1 } tcfp_dtype;
typedef enum { TCFP_E4M3 = 0, TCFP_E5M2 = 1 } tcfp_fp8;

/* error-feedback / rounding mode of the weight dual quantizer */
typedef enum {
  TCFP_Q_NONE = 0,        /* no error buffer, round-to-nearest W_lo            */
  TCFP_Q_EF = 1,          /* read error buffer, write the new error in place   */
  TCFP_Q_EF_READONLY = 2, /* read error buffer, leave it untouched
                             (update_ef == False, tcfp/nn/__init__.py:378,607) */
  TCFP_Q_SRR = 3          /* no buffer, stochastic rounding of W_lo            */
} tcfp_qmode;

/* ---- library ----------------------------------------------------------- */
/* version as 10000*major + 100*minor + patch */
int32_t tcfp_version(void);
/* copies the calling thread's last error text (NUL-terminated) into buf */
int32_t tcfp_last_error(char* buf, size_t n);
/*
 * No counterpart in the reference.  The GEMM kernels are persistent: one CTA
 * (pair) per SM for the whole launch, so a collective's kernel queued beside
 * one finds no SM to run on until the GEMM ends.  tcfp_set_sm_reserve(n) makes
 * the GEMM entry points called afterwards FROM THE SAME HOST THREAD size their
 * grids for (SM count - n) SMs, leaving n for the collective; 0 restores the
 * full grid.  Returns the previous value (>= 0), or TCFP_ERR_INVALID.
 */
int32_t tcfp_set_sm_reserve(int32_t n);

/* Synchronises ``stream`` and returns TCFP_ERR_DEVICE if any kernel of this
 * library recorded a timed-out wait since the last call (and clears the
 * record).  The hot path never calls this; tests and debug builds do. */
int32_t tcfp_check_device_status(void* stream);
/* Launches one CTA that waits limit_ns (at most 100 ms) on a barrier nothing
 * signals, so that the give-up path -- status word set, kernel returns, the
 * context stays usable -- can be tested without any real failure. */
int32_t tcfp_selftest_bounded_wait(uint64_t limit_ns, void* stream);

/* ---- K1: weight dual quantizer ----------------------------------------- */
/*
 * W (N,K) [+ FP32 error buffer] -> W_hi, W_lo (E4M3 codes, (N,K) bytes),
 * their scales, and the updated error buffer.
 *
 * block_size == 0  : per-tensor scaling.  Replaces steps 1-4 of
 *     _TCFP12TensorCoreFunction.forward (tcfp/nn/__init__.py:343-383) and the
 *     to_fp8_e4m3 / to_fp8_e4m3_sr chains (tcfp/core.py:85-134, 418-464).
 *     scale_hi / scale_lo receive ONE float each: the inverse scale
 *     (1 / (448 / amax)) exactly as torch computes it.
 *     amax_hi_in / amax_lo_in (nullable, 1 float each) override the fresh
 *     amax (delayed scaling, tcfp/nn/__init__.py:250-309); amax_out
 *     (nullable, 2 floats) receives the current un-clamped amax of W+e
 *     (0 when amax_hi_in was supplied, use tcfp_absmax for it) and of the
 *     residual.
 * block_size in {32,64,128}: power-of-two block scaling along K.  Replaces
 *     fused_dual_quantize_fp8 (tcfp/kernels.py:1749-1875).  scale_hi /
 *     scale_lo receive int8 exponent planes of shape (K/bs, N); -128 marks a
 *     zero-residual block.  sf_hi / sf_lo (nullable) additionally receive the
 *     same exponents as biased E8M0 bytes in the 512-byte chunk layout the
 *     tensor-core GEMM consumes (see tcfp_sf_packed_bytes()).
 *
 * err is read for EF / EF_READONLY and written for EF; it must be NULL for
 * NONE and SRR.  SRR draws u = philox4x32-10(key=seed, ctr=offset + n*K + k).
 * workspace: tcfp_dual_quantize_workspace_bytes() bytes (per-tensor only).
 */
int32_t tcfp_dual_quantize(const void* w, int32_t w_dtype, float* err,
                           uint8_t* w_hi, uint8_t* w_lo,
                           void* scale_hi, void* scale_lo,
                           uint8_t* sf_hi, uint8_t* sf_lo,
                           int64_t N, int64_t K, int32_t block_size,
                           int32_t mode, uint64_t seed, uint64_t offset,
                           const float* amax_hi_in, const float* amax_lo_in,
                           float* amax_out, void* workspace, void* stream);
size_t tcfp_dual_quantize_workspace_bytes(void);

/* amax_out[0] = max |x[i] (+ err[i])| over numel elements (err nullable).
 * Replaces the ``tensor.abs().max()`` reductions of tcfp/core.py:100 and
 * tcfp/nn/__init__.py:282 where the caller needs the value before the
 * quantizing pass (delayed scaling). */
int32_t tcfp_absmax(const void* x, int32_t x_dtype, const float* err,
                    int64_t numel, float* amax_out, void* stream);

/* ---- K2: activation / gradient quantizer ------------------------------- */
/*
 * x (R,C) f32|bf16 -> FP8 codes (R,C).
 * block_size == 0: per-tensor, scale_out = 1 float inverse scale; replaces
 *     to_fp8_e4m3 / to_fp8_e5m2 (tcfp/core.py:85-106, 137-158); amax_in
 *     (nullable) overrides the fresh amax, scale_in (nullable, wins over
 *     amax_in) is used directly as the forward scale -- the ``scale=``
 *     argument of the reference functions; stochastic != 0 (E4M3 only)
 *     rounds stochastically with u = philox(seed, offset + i), replacing
 *     to_fp8_e4m3_sr (tcfp/core.py:109-134, 418-464); workspace as above.
 * block_size in {32,64,128}: replaces block_quantize_fp8
 *     (tcfp/kernels.py:1675-1722); scale_out = int8 (C/bs, R); sf_out
 *     (nullable) = packed E8M0 copy; deq_bf16_out (nullable) = the
 *     dequantized value code*2^e as bf16 (exact), consumed by the
 *     block-scaled dX GEMM.
 */
int32_t tcfp_quantize(const void* x, int32_t x_dtype, uint8_t* out,
                      void* scale_out, uint8_t* sf_out, void* deq_bf16_out,
                      int64_t R, int64_t C, int32_t block_size, int32_t fmt,
                      const float* amax_in, const float* scale_in,
                      int32_t stochastic, uint64_t seed, uint64_t offset,
                      void* workspace, void* stream);

/* bytes of the packed E8M0 scale-factor array for a (rows, K) operand */
size_t tcfp_sf_packed_bytes(int64_t rows, int64_t K, int32_t block_size);
/*
 * tcfp_quantize of a gradient that ALSO returns its column sums -- the bias
 * gradient, which the reference takes with a separate full pass over the
 * gradient (grad_2d.sum(dim=0), tcfp/nn/__init__.py:558, 753).  block_size 0:
 * one pass yields the amax and the sums, the cast follows (tcfp/core.py:
 * 137-158); block_size 32/64/128: the block quantizer accumulates the sums as
 * it goes (tcfp/kernels.py:205-275).  colsum_out: C floats.  The summation
 * order is fixed (per 256-row group, then the groups in order), so repeated
 * calls return identical bits.  workspace: tcfp_colsum_workspace_bytes(R, C)
 * bytes of device memory, 16-byte aligned.
 */
size_t tcfp_colsum_workspace_bytes(int64_t R, int64_t C);
int32_t tcfp_quantize_colsum(const void* x, int32_t x_dtype, uint8_t* out,
                             void* scale_out, uint8_t* sf_out, int64_t R,
                             int64_t C, int32_t block_size, int32_t fmt,
                             float* colsum_out, void* workspace, void* stream);

/* int8 exponent plane (K/bs, rows) -> packed E8M0 chunks (for callers that
 * hold only the reference-layout planes) */
int32_t tcfp_pack_scales(const int8_t* exps, uint8_t* sf_out, int64_t rows,
                         int64_t K, int32_t block_size, void* stream);
/* block-scaled FP8 codes + int8 exponents -> bf16 values (exact);
 * replaces block_dequantize_fp8 (tcfp/kernels.py:1725-1746) for the
 * backward operands.  sentinel_zero != 0 maps exponent -128 to scale 0. */
int32_t tcfp_block_dequantize_bf16(const uint8_t* codes, const int8_t* exps,
                                   void* out_bf16, int64_t rows, int64_t K,
                                   int32_t block_size, int32_t fmt,
                                   int32_t sentinel_zero, void* stream);

/* FP32 -> bf16 head + bf16 tail (x = head + tail to 16 significant bits:
 * head = bf16(x), tail = bf16(x - head)), the operand form tcfp_bf16_dw_gemm
 * takes for an FP32 gradient.  n elements, n % 4 == 0.  No reference
 * counterpart: the reference multiplies the FP32 gradient as it is
 * (tcfp/nn/__init__.py:744-750). */
int32_t tcfp_split_bf16(const float* x, void* head_bf16, void* tail_bf16,
                        int64_t n, void* stream);

/* ---- K3: fused dual GEMM ----------------------------------------------- */
/*
 * Per-tensor scaled.  trans_b == 0 (forward, "NT"):
 *     out(M,N) = (A . W_hi^T) * (s_a*s_hi) + (A . W_lo^T) * (s_a*s_lo)
 *   with A (M,K) FP8, W_* (N,K) E4M3.  Replaces
 *   tcfp::fused_dual_fp8_gemm_forward (tcfp/csrc/fused_dual_gemm.h:25-32) and
 *   fused_dual_gemm_forward (tcfp/kernels.py:1545-1601).
 * trans_b == 1 (backward dX, "NN"):
 *     out(M,N) = (A . W_hi) * (s_a*s_hi) + (A . W_lo) * (s_a*s_lo)
 *   with A (M,K) FP8 (E5M2 gradients), W_* (K,N) E4M3 in their native
 *   (out,in) layout -- no transposed copy.  Replaces
 *   tcfp::fused_dual_fp8_gemm_backward_dx (fused_dual_gemm.h:42-48) and
 *   fused_dual_gemm_backward_dx (tcfp/kernels.py:1604-1666).
 * w_lo / s_lo may both be NULL (single GEMM, "abd" backward,
 * tcfp/nn/__init__.py:499-508).  s_* point at one device float each.
 * bias (nullable, N floats) is added in the epilogue.  out_dtype f32|bf16.
 * All leading dimensions must make rows 16-byte aligned (M,N,K % 16 == 0).
 */
int32_t tcfp_dual_gemm(const uint8_t* a, int32_t a_fmt,
                       const uint8_t* w_hi, const uint8_t* w_lo,
                       const float* s_a, const float* s_hi, const float* s_lo,
                       const float* bias, void* out, int32_t out_dtype,
                       int64_t M, int64_t N, int64_t K, int32_t trans_b,
                       void* stream);

/*
 * Weight gradient in FP8:  dW(n_out, k_in) = (g^T . x) * (s_g*s_x)  with
 * g (tokens, n_out) FP8 (E5M2 gradients) and x (tokens, k_in) E4M3, both in
 * their forward layouts -- the transposes are smem-descriptor bits, not
 * copies.  Replaces torch._scaled_mm(grad_fp8.t().contiguous(),
 * ensure_column_major(act_fp8)) at tcfp/nn/__init__.py:546-555.
 */
int32_t tcfp_dw_gemm(const uint8_t* g, int32_t g_fmt, const uint8_t* x,
                     const float* s_g, const float* s_x, void* out,
                     int32_t out_dtype, int64_t tokens, int64_t n_out,
                     int64_t k_in, void* stream);

/*
 * Block-scaled forward:
 *   out[m,n] = sum_kb 2^sa[kb,m] * (2^shi[kb,n] * A_kb.Whi_kb + 2^slo[kb,n] * A_kb.Wlo_kb)
 * A (M,K) E4M3, W_* (N,K) E4M3, scale factors as packed E8M0 chunk arrays
 * (tcfp_pack_scales / the sf_* outputs of the quantizers).  Replaces
 * fused_block_scaled_dual_gemm_forward (tcfp/kernels.py:1939-2028).
 */
int32_t tcfp_block_dual_gemm(const uint8_t* a, const uint8_t* sf_a,
                             const uint8_t* w_hi, const uint8_t* sf_hi,
                             const uint8_t* w_lo, const uint8_t* sf_lo,
                             const float* bias, void* out, int32_t out_dtype,
                             int64_t M, int64_t N, int64_t K,
                             int32_t block_size, void* stream);

/*
 * Block-scaled forward with the activation quantizer fused into the GEMM
 * prologue: x (M,K) bf16 is block-quantized to E4M3 + E8M0 inside the K loop
 * by converter warps (same bytes as tcfp_quantize(block_size) produces) and
 * multiplied against W_hi / W_lo as in tcfp_block_dual_gemm.  act_codes_out
 * (M,K) and act_exps_out (K/bs, M) int8 -- both or neither -- receive the
 * quantized activation for the backward pass, written by the CTAs of the
 * first column tile only.  Every column tile re-quantizes its A tiles, so
 * this pays for narrow layers only.  Replaces
 * fused_act_quant_dual_gemm_forward (tcfp/kernels.py:2031-2149, kernel
 * :826-1041), which the reference dispatches for N <= 512
 * (tcfp/nn/__init__.py:620-640).
 */
int32_t tcfp_block_dual_gemm_fused_act(const void* x_bf16, const uint8_t* w_hi,
                                       const uint8_t* sf_hi, const uint8_t* w_lo,
                                       const uint8_t* sf_lo, const float* bias,
                                       void* out, int32_t out_dtype,
                                       uint8_t* act_codes_out,
                                       int8_t* act_exps_out, int64_t M,
                                       int64_t N, int64_t K, int32_t block_size,
                                       void* stream);

/*
 * No counterpart in the reference.  Same result as tcfp_pack_scales (x3)
 * followed by tcfp_block_dual_gemm, for callers that hold the scales as
 * reference-layout int8 exponent planes (K/bs, rows) and cannot allocate the
 * packed scale-factor buffers: a plugin given only its input and output
 * buffers, or code on a path where cudaMalloc is off limits.  The packed
 * scales go into a 6 MiB array built into the library (2 MiB per operand,
 * tcfp_static_scratch_bytes_per_operand(); every GPU that loads the library
 * carries it).  Operands whose packed scales exceed 2 MiB (more than
 * 8192 x 8192 at block 32) are refused with TCFP_ERR_UNSUPPORTED.  This call
 * allocates nothing.  The first call on each device looks up the array's
 * device address -- make that call before starting any stream capture.  All
 * calls on a device share the one array: two calls whose kernels can overlap
 * on the GPU (different streams) race; serialise them.
 */
int32_t tcfp_block_dual_gemm_static(const uint8_t* a, const int8_t* exp_a,
                                    const uint8_t* w_hi, const int8_t* exp_hi,
                                    const uint8_t* w_lo, const int8_t* exp_lo,
                                    const float* bias, void* out,
                                    int32_t out_dtype, int64_t M, int64_t N,
                                    int64_t K, int32_t block_size,
                                    void* stream);
size_t tcfp_static_scratch_bytes_per_operand(void);

/*
 * Block-scaled input gradient on the FP8 tensor-core path, in two steps.
 *
 * tcfp_block_retarget: rewrites a block-quantized weight (R = D_out rows,
 * C = D_in columns; exponents exp_* in the reference layout (C/bs, R)) into the
 * orientation the backward contraction needs: codes TRANSPOSED to (C, R) and
 * one exponent per (column c, block of bs rows), written as planes t_* of
 * shape (R/bs, C) -- the reference layout of an operand with rows = C and
 * K = R, ready for tcfp_pack_scales.  t = max of the rows' exponents in the
 * block; each code is re-encoded as value * 2^(s - t).  Exact except where the
 * down-shift drops below E4M3's subnormal step (absolute error <= 2^-10 * 2^t).
 * The -128 sentinel of the residual plane contributes zeros.  w_lo and its
 * three companions may all be NULL.  Depends only on the quantized weight: do
 * it once per weight version and reuse it across micro-batches.
 *
 * tcfp_block_dx_gemm:
 *   out(M, D_in) = sum_kb 2^sg[kb,m] * (2^t_hi[kb,n] * G_kb.HiT_kb + 2^t_lo[kb,n] * G_kb.LoT_kb)
 * with G (M, D_out) E5M2 block-quantized along D_out and the retargeted
 * operands (D_in, D_out); all scale factors as packed chunk arrays.  Together
 * they replace fused_block_scaled_backward_dx (tcfp/kernels.py:2326-2425,
 * kernel :1051-1205), which dequantizes to FP32 and multiplies in TF32.
 */
int32_t tcfp_block_retarget(const uint8_t* w_hi, const uint8_t* w_lo,
                            const int8_t* exp_hi, const int8_t* exp_lo,
                            uint8_t* hi_t, uint8_t* lo_t, int8_t* t_hi,
                            int8_t* t_lo, int64_t R, int64_t C,
                            int32_t block_size, void* stream);
int32_t tcfp_block_dx_gemm(const uint8_t* g, const uint8_t* sf_g,
                           const uint8_t* w_hi_t, const uint8_t* sf_hi_t,
                           const uint8_t* w_lo_t, const uint8_t* sf_lo_t,
                           void* out, int32_t out_dtype, int64_t M,
                           int64_t d_in, int64_t d_out, int32_t block_size,
                           void* stream);

/*
 * BF16 dual GEMM on exactly dequantized operands:
 *   trans_b == 1: out(M,N) = A(M,K) . (B_hi(K,N) + B_lo(K,N))   (block dX)
 *   trans_b == 0: out(M,N) = A(M,K) . (B_hi(N,K) + B_lo(N,K))^T
 * Replaces fused_block_scaled_backward_dx (tcfp/kernels.py:2326-2425), whose
 * per-contraction-element weight scales cannot ride an FP8 block-scaled MMA.
 */
int32_t tcfp_bf16_dual_gemm(const void* a, const void* b_hi, const void* b_lo,
                            const float* bias, void* out, int32_t out_dtype,
                            int64_t M, int64_t N, int64_t K, int32_t trans_b,
                            void* stream);

/*
 * Weight gradient of the block-scaled layer on the bf16 tensor-core path:
 *     out(k_in, n_out) = x^T . (g_hi + g_lo)
 * x (tokens, k_in) bf16 (the exactly dequantized saved activation, or the bf16
 * input), g_hi / g_lo (tokens, n_out) the bf16 head and tail of the FP32
 * gradient (g = g_hi + g_lo to 16 significant bits; g_lo nullable).  The
 * result is dW TRANSPOSED.  Replaces the FP32 ``grad.t() @ activation``
 * matmuls at tcfp/nn/__init__.py:744-750 at tensor-core speed.
 */
int32_t tcfp_bf16_dw_gemm(const void* x, const void* g_hi, const void* g_lo,
                          void* out, int32_t out_dtype, int64_t tokens,
                          int64_t k_in, int64_t n_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TCFP_B200_H_ */
