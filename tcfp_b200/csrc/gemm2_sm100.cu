// K3, two-SM form: the fused dual GEMM on CTA pairs (tcgen05 cta_group::2).
//
// A cluster of two CTAs owns a 256 x 128 output tile.  Each CTA stages its own
// 128 rows of A and HALF of the B operand, and the leader CTA issues
// tcgen05.mma.cta_group::2 instructions that read both halves: per SM the
// shared-memory and L2 traffic of the B operand is halved relative to the
// one-SM kernel (32 KB instead of 48 KB per K stage), which is what the
// one-SM kernel is limited by at 8192^3.
//
// Two accumulation layouts:
//   CONCAT (per-tensor scales; hi and lo need different FP32 factors):
//       one MMA 256 x 256 per K step; CTA 0 stages the W_hi tile, CTA 1 the
//       W_lo tile; accumulator columns [0,128) = A.W_hi, [128,256) = A.W_lo.
//       Without W_lo the two halves are two adjacent 128-column tiles of W.
//   SUM (block-scaled MXF8 and exactly dequantized BF16; no epilogue factors):
//       two MMAs 256 x 128 per K step into the SAME 128 accumulator columns;
//       each CTA stages 64 rows of W_hi and 64 rows of W_lo.
//   A single bf16 product (the weight gradient of a bf16 output gradient) has
//   no second operand to sum, and a 256 x 128 tile would pull 24 KB per CTA
//   from L2 for every four MMAs (96 B per clock per SM, more than L2 delivers):
//   it runs in the CONCAT layout as a 256 x 256 tile (KIND_BF16_WIDE, 64 B per
//   clock per SM, the same as the dual kinds).
//
// Roles per CTA as in the one-SM kernel (warp 0 TMA, warp 1 MMA/TMEM, warps
// 2-5 epilogue).  Both producers signal the LEADER's full barrier; the
// leader's tcgen05.commit multicasts to the empty / accumulator-full barriers
// of both CTAs; both epilogues arrive on the leader's accumulator-empty
// barrier.  No TMA multicast is used anywhere.
//
// Every wait is bounded; see sm100_ptx.cuh.
#include <cuda.h>

#include "common.cuh"
#include "launch.h"
#include "sm100_ptx.cuh"

namespace tcfp {
namespace {

constexpr int BM = 128;   // rows per CTA (256 per pair)
constexpr int BN = 128;   // output columns per accumulator half
constexpr int kThreads = 192;
constexpr int kATile = 16384;
constexpr int kBTile = 16384;         // per CTA: its half of the B operand(s)
constexpr int kStageBytes = kATile + kBTile;
constexpr int kSfStage = 3 * 512;
constexpr int kPieceBytes = 16384;    // 128 rows x 128 B of staged output
constexpr int kGroupM = 8;            // default rasterisation group, in units of 256-row tile rows
constexpr int KIND_BF16_WIDE = 3;     // bf16 operands, CONCAT layout (single product, 256 x 256 tile)

__host__ __device__ constexpr bool is_bf16_kind(int kind) { return kind == KIND_BF16 || kind == KIND_BF16_WIDE; }

struct Gemm2Params {
  int M, N, K;
  int k_stages;
  int has_lo;
  int a_fmt;
  int block_size;
  int group_m;
  const float* s_a;
  const float* s_hi;
  const float* s_lo;
  const float* bias;
  unsigned int* status;
};

// ---- cluster helpers --------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion is counted on a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ void tc_cp_sf_pair(uint32_t tmem_addr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}

template <int KIND>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accum, uint32_t sfa, uint32_t sfb) {
  if constexpr (KIND == KIND_F8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
        : "memory");
  } else if constexpr (is_bf16_kind(KIND)) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum), "r"(sfa), "r"(sfb)
        : "memory");
  }
}

template <int KIND>
struct Traits2 {
  static constexpr bool kSum = (KIND == KIND_MXF8 || KIND == KIND_BF16);
  static constexpr int kElemBytes = is_bf16_kind(KIND) ? 2 : 1;
  static constexpr int kStageK = 128 / kElemBytes;
  static constexpr int kMmaK = 32 / kElemBytes;
  static constexpr int kStages = (KIND == KIND_MXF8) ? 5 : 6;
  static constexpr int kAccCols = kSum ? 128 : 256;   // TMEM columns per accumulator buffer
  static constexpr int kSfColBase = 2 * kAccCols;     // MXF8: scale factors behind the two buffers
};

template <int KIND>
__host__ __device__ constexpr int smem_bytes2() {
  return 1024 + Traits2<KIND>::kStages * kStageBytes + 2 * kPieceBytes +
         (KIND == KIND_MXF8 ? Traits2<KIND>::kStages * kSfStage : 0) + 256;
}

// tile id -> (256-row block, column block); M fastest inside groups of kGroupM
__device__ __forceinline__ void tile_coords2(int tile, int tiles_m, int tiles_n, int group_m, int& mb, int& nb) {
  const int per_group = group_m * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int gm = min(tiles_m - first_m, group_m);
  const int in_group = tile - group * per_group;
  mb = first_m + in_group % gm;
  nb = in_group / gm;
}

template <int KIND, bool B_MN, bool OUT_BF16, bool A_MN = false>
__global__ void __launch_bounds__(kThreads, 1)
dual_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_bhi,
                      const __grid_constant__ CUtensorMap tm_blo, const __grid_constant__ CUtensorMap tm_out,
                      const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfhi,
                      const __grid_constant__ CUtensorMap tm_sflo, const Gemm2Params p) {
  using T = Traits2<KIND>;
  constexpr int kStages = T::kStages;
  constexpr bool kSum = T::kSum;
  constexpr uint32_t kTmemCols = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint8_t* staging = stage_base + kStages * kStageBytes;
  uint8_t* sf_base = staging + 2 * kPieceBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sf_base + (KIND == KIND_MXF8 ? kStages * kSfStage : 0));
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = smem_u32(bars + kStages);
  const uint32_t bar_tfull = smem_u32(bars + 2 * kStages);
  const uint32_t bar_tempty = smem_u32(bars + 2 * kStages + 2);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  // column blocks are 128 wide, except CONCAT without W_lo which covers 256
  const int tile_n = (!kSum && !p.has_lo) ? 2 * BN : BN;
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + tile_n - 1) / tile_n;
  const int num_tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 8);   // one arrival per epilogue warp of both CTAs
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tm_a);
    prefetch_tmap(&tm_bhi);
    prefetch_tmap(&tm_blo);
    prefetch_tmap(&tm_out);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before anything remote touches them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ======================= TMA producer (both CTAs) =======================
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      // bytes ONE CTA delivers per stage
      uint32_t cta_bytes = kATile;
      if constexpr (!kSum) cta_bytes += kBTile;                          // hi (rank 0) or lo / second tile (rank 1)
      else cta_bytes += (p.has_lo ? 2 : 1) * (kBTile / 2);
      if constexpr (KIND == KIND_MXF8) cta_bytes += (p.has_lo ? 3 : 2) * 512;
      const int kg_per = (KIND == KIND_MXF8) ? (p.block_size / 32) : 1;
      bool live = true;
      for (int tile = pair; live && tile < num_tiles; tile += num_pairs) {
        int mb, nb;
        tile_coords2(tile, tiles_m, tiles_n, p.group_m, mb, nb);
        const int row0 = mb * 2 * BM + (int)rank * BM;
        for (int ks = 0; ks < p.k_stages; ++ks) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status)) { live = false; break; }
          const uint32_t full_leader = mapa(bar_full + 8 * stage, 0);
          if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * cta_bytes);
          const uint32_t sa = smem_u32(stage_base + stage * kStageBytes);
          const uint32_t sb = sa + kATile;
          const int k0 = ks * T::kStageK;
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, &tm_a, k0, row0, full_leader);
          } else {
            // A stored transposed, (K, M) row-major: one box per 128-byte-wide group of its M columns
            constexpr int kABoxes = T::kElemBytes;
#pragma unroll
            for (int b = 0; b < kABoxes; ++b)
              tma_load_2d_pair(sa + b * (kATile / kABoxes), &tm_a, row0 + b * (128 / T::kElemBytes), k0, full_leader);
          }
          if constexpr (!kSum) {
            // this CTA's half of the 256 MMA columns
            const CUtensorMap* map = (p.has_lo && rank == 1) ? &tm_blo : &tm_bhi;
            const int n0 = nb * tile_n + ((!p.has_lo && rank == 1) ? BN : 0);
            if constexpr (!B_MN) {
              tma_load_2d_pair(sb, map, k0, n0, full_leader);
            } else {
              // (K, N) row-major: one box per 128-byte-wide group of this CTA's 128 columns
              constexpr int kBBoxes = T::kElemBytes;
#pragma unroll
              for (int b = 0; b < kBBoxes; ++b)
                tma_load_2d_pair(sb + b * (kBTile / kBBoxes), map, n0 + b * (128 / T::kElemBytes), k0, full_leader);
            }
          } else {
            // 64 of the 128 MMA columns of each operand
            const int n0 = nb * BN + (int)rank * (BN / 2);
            if constexpr (!B_MN) {
              tma_load_2d_pair(sb, &tm_bhi, k0, n0, full_leader);
              if (p.has_lo) tma_load_2d_pair(sb + kBTile / 2, &tm_blo, k0, n0, full_leader);
            } else {
              tma_load_2d_pair(sb, &tm_bhi, n0, k0, full_leader);
              if (p.has_lo) tma_load_2d_pair(sb + kBTile / 2, &tm_blo, n0, k0, full_leader);
            }
          }
          if constexpr (KIND == KIND_MXF8) {
            const int k_groups = ((p.K / p.block_size) + 3) / 4;
            const int kg = (ks * 4) / kg_per / 4;
            const uint32_t ssf = smem_u32(sf_base + stage * kSfStage);
            tma_load_2d_pair(ssf, &tm_sfa, 0, (mb * 2 + (int)rank) * k_groups + kg, full_leader);
            tma_load_2d_pair(ssf + 512, &tm_sfhi, 0, nb * k_groups + kg, full_leader);
            if (p.has_lo) tma_load_2d_pair(ssf + 1024, &tm_sflo, 0, nb * k_groups + kg, full_leader);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ======================= MMA issuer (leader CTA only) =======================
    if (rank == 0 && elect_one()) {
      const uint32_t n_mma = kSum ? BN : 2 * BN;
      uint32_t idesc;
      if constexpr (KIND == KIND_MXF8) {
        idesc = ((uint32_t)p.a_fmt << 7) | ((B_MN ? 1u : 0u) << 16) | ((n_mma >> 3) << 17) | (1u << 23) |
                ((uint32_t)((2 * BM) >> 4) << 24);
      } else {
        const uint32_t fa = is_bf16_kind(KIND) ? 1u : (uint32_t)p.a_fmt;
        const uint32_t fb = is_bf16_kind(KIND) ? 1u : 0u;
        idesc = (1u << 4) | (fa << 7) | (fb << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                ((n_mma >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
      }
      static_assert(!(A_MN && KIND == KIND_MXF8), "block-scaled kind takes A K-major");
      constexpr uint32_t kALbo = A_MN ? (uint32_t)(kATile / T::kElemBytes) : 16u;
      constexpr uint32_t kAKStep = A_MN ? (uint32_t)(T::kMmaK * 128) : 32u;
      // B: every CTA holds (n_mma / 2) columns of each MMA's B operand.
      //   K-major : rows of 128 B, 8-row groups 1024 B apart.
      //   MN-major: 128-byte-wide column groups (CONCAT fp8: one of 128 cols; SUM bf16: one of 64 cols;
      //             CONCAT bf16: two of 64 cols, LBO apart).
      constexpr uint32_t kBLbo = (B_MN && !kSum && T::kElemBytes == 2) ? (uint32_t)(kBTile / 2) : 16u;
      constexpr uint32_t kBKStep = B_MN ? (uint32_t)(T::kMmaK * 128) : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool live = true;
      for (int tile = pair; live && tile < num_tiles; tile += num_pairs) {
        if (!mbar_wait(bar_tempty + 8 * buf, buf_phase ^ 1, abort_flag, p.status)) { live = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * T::kAccCols);
        for (int ks = 0; ks < p.k_stages; ++ks) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status)) { live = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(stage_base + stage * kStageBytes);
          const uint32_t sb = sa + kATile;
          uint32_t tsfa = 0, tsfb_hi = 0, tsfb_lo = 0;
          int sf_first = 0, sf_shift = 0;
          if constexpr (KIND == KIND_MXF8) {
            const uint32_t ssf = smem_u32(sf_base + stage * kSfStage);
            tsfa = tmem_base + (uint32_t)(T::kSfColBase + stage * 16);
            tsfb_hi = tsfa + 4;
            tsfb_lo = tsfa + 8;
            tc_cp_sf_pair(tsfa, make_desc(ssf, 0, 128, 0));
            tc_cp_sf_pair(tsfb_hi, make_desc(ssf + 512, 0, 128, 0));
            if (p.has_lo) tc_cp_sf_pair(tsfb_lo, make_desc(ssf + 1024, 0, 128, 0));
            if (p.block_size == 32) { sf_first = 0; sf_shift = 0; }
            else if (p.block_size == 64) { sf_first = 2 * (ks & 1); sf_shift = 1; }
            else { sf_first = ks & 3; sf_shift = 2; }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t adesc = make_desc(sa + j * kAKStep, kALbo, 1024, 2);
            uint32_t id = idesc;
            if constexpr (KIND == KIND_MXF8) {
              const uint32_t sfid = (uint32_t)(sf_first + (j >> sf_shift));
              id |= (sfid << 29) | (sfid << 4);
            }
            const uint64_t bdesc = make_desc(sb + j * kBKStep, kBLbo, 1024, 2);
            tc_mma_pair<KIND>(d_tmem, adesc, bdesc, id, (ks | j) != 0 ? 1u : 0u, tsfa, tsfb_hi);
            if constexpr (kSum) {
              if (p.has_lo) {
                const uint64_t bdesc_lo = make_desc(sb + kBTile / 2 + j * kBKStep, kBLbo, 1024, 2);
                tc_mma_pair<KIND>(d_tmem, adesc, bdesc_lo, id, 1u, tsfa, tsfb_lo);
              }
            }
          }
          tc_commit_pair(bar_empty + 8 * stage);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!live) break;
        tc_commit_pair(bar_tfull + 8 * buf);
        if (++buf == 2) { buf = 0; buf_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ======================= epilogue (both CTAs, own 128 rows) =======================
    const int q = warp & 3;
    const int r_local = q * 32 + lane;
    const bool issuer = (threadIdx.x == 64);
    float c_hi = 1.f, c_lo = 1.f;
    if constexpr (KIND == KIND_F8) {
      const float sa = __ldg(p.s_a);
      c_hi = sa * __ldg(p.s_hi);
      c_lo = p.has_lo ? sa * __ldg(p.s_lo) : c_hi;
    }
    const bool dual_concat = !kSum && p.has_lo;
    const int n_pieces = tile_n / 32;
    constexpr int kPieceCols = OUT_BF16 ? 64 : 32;     // output columns per 128-byte staging row
    int buf = 0;
    uint32_t buf_phase = 0;
    int pending = 0;          // TMA stores in flight (issuer only)
    int sbuf = 0;             // staging buffer for the next store
    bool live = true;
    for (int tile = pair; live && tile < num_tiles; tile += num_pairs) {
      int mb, nb;
      tile_coords2(tile, tiles_m, tiles_n, p.group_m, mb, nb);
      const int row0 = mb * 2 * BM + (int)rank * BM;
      if (!mbar_wait(bar_tfull + 8 * buf, buf_phase, abort_flag, p.status)) { live = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * T::kAccCols);
#pragma unroll 1
      for (int g = 0; g < n_pieces; ++g) {
        uint32_t vh[32], vl[32];
        tmem_ld32(t_row + g * 32, vh);
        if (dual_concat) tmem_ld32(t_row + BN + g * 32, vl);
        tmem_ld_wait();
        if (g == n_pieces - 1) {
          // last read of this accumulator: hand it back to the leader's MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(mapa(bar_tempty + 8 * buf, 0));
        }
        float o[32];
        const float cg = (!dual_concat && g >= 4) ? c_lo : c_hi;   // second tile of a 256-wide single GEMM
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(vh[i]) * cg;
          if (dual_concat) v = fmaf(__uint_as_float(vl[i]), c_lo, v);
          o[i] = v;
        }
        const int n0 = nb * tile_n + g * 32;
        if (p.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (n0 + i < p.N) o[i] += __ldg(p.bias + n0 + i);
        }
        // a staging buffer may be rewritten once the store issued two pieces ago has read it
        const bool new_row = OUT_BF16 ? ((g & 1) == 0) : true;
        if (new_row) {
          if (issuer && pending >= 2) { bulk_wait_read1(); pending = 1; }
          epi_bar_sync();
        }
        uint8_t* piece = staging + sbuf * kPieceBytes + r_local * 128;
        if constexpr (!OUT_BF16) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float4 v4 = make_float4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
            *reinterpret_cast<float4*>(piece + ((c ^ (r_local & 7)) << 4)) = v4;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            __nv_bfloat162 b0 = __floats2bfloat162_rn(o[8 * c], o[8 * c + 1]);
            __nv_bfloat162 b1 = __floats2bfloat162_rn(o[8 * c + 2], o[8 * c + 3]);
            __nv_bfloat162 b2 = __floats2bfloat162_rn(o[8 * c + 4], o[8 * c + 5]);
            __nv_bfloat162 b3 = __floats2bfloat162_rn(o[8 * c + 6], o[8 * c + 7]);
            uint4 v4;
            v4.x = *reinterpret_cast<uint32_t*>(&b0);
            v4.y = *reinterpret_cast<uint32_t*>(&b1);
            v4.z = *reinterpret_cast<uint32_t*>(&b2);
            v4.w = *reinterpret_cast<uint32_t*>(&b3);
            const int cc = (g & 1) * 4 + c;
            *reinterpret_cast<uint4*>(piece + ((cc ^ (r_local & 7)) << 4)) = v4;
          }
        }
        const bool row_done = OUT_BF16 ? ((g & 1) == 1 || g == n_pieces - 1) : true;
        if (row_done) {
          fence_async_smem();
          epi_bar_sync();
          if (issuer) {
            const int nst = OUT_BF16 ? (nb * tile_n + (g >> 1) * kPieceCols) : n0;
            if (nst < p.N && row0 < p.M) {
              tma_store_2d(&tm_out, smem_u32(staging + sbuf * kPieceBytes), nst, row0);
              bulk_commit();
              ++pending;
            }
          }
          sbuf ^= 1;
        }
      }
      if (++buf == 2) { buf = 0; buf_phase ^= 1; }
    }
    if (issuer) bulk_wait0();
  }

  // ======================= teardown =======================
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 20; ++i) __nanosleep(1000);
  }
  cluster_sync_all();   // the peer may still be reading operands / signalling barriers of this CTA
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode2() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// A tensor map is a pure function of (address, shape, box, type, swizzle).  A
// training step launches the same GEMMs on the same buffers over and over (the
// caching allocator hands back the same addresses), so the encoded maps are
// kept in a small per-thread direct-mapped table instead of being re-encoded
// by the driver on every launch (seven per launch).
struct MapKey {
  const void* ptr;
  int64_t rows, cols;
  int32_t box_cols, box_rows, dt, swz, elem_bytes;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box_cols == o.box_cols && box_rows == o.box_rows &&
           dt == o.dt && swz == o.swz && elem_bytes == o.elem_bytes;
  }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool valid;
};
constexpr int kMapSlots = 512;

int make_map2(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* ptr, int64_t rows, int64_t cols,
              int box_cols, int box_rows, CUtensorMapSwizzle swz) {
  static thread_local MapSlot table[kMapSlots] = {};
  const MapKey key{ptr, rows, cols, box_cols, box_rows, (int32_t)dt, (int32_t)swz, elem_bytes};
  uint64_t h = reinterpret_cast<uintptr_t>(ptr) >> 4;
  h ^= (uint64_t)rows * 0x9E3779B97F4A7C15ull ^ (uint64_t)cols * 0xC2B2AE3D27D4EB4Full ^ (uint64_t)(box_rows * 131 + box_cols) ^
       ((uint64_t)dt << 40) ^ ((uint64_t)swz << 48);
  h ^= h >> 29;
  MapSlot& slot = table[h % kMapSlots];
  if (slot.valid && slot.key == key) {
    *map = slot.map;
    return TCFP_OK;
  }
  EncodeTiledFn enc = get_encode2();
  if (!enc) return fail(TCFP_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) || ((cols * elem_bytes) & 15))
    return fail(TCFP_ERR_INVALID, "GEMM operands need 16-byte aligned base pointers and row pitches");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(cols * elem_bytes)};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TCFP_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  slot.key = key;
  slot.map = *map;
  slot.valid = true;
  return TCFP_OK;
}

template <int KIND, bool B_MN, bool OUT_BF16, bool A_MN = false>
int launch2(const void* a, const void* b_hi, const void* b_lo, const void* sf_a, const void* sf_hi, const void* sf_lo,
            void* out, Gemm2Params p, cudaStream_t stream) {
  using T = Traits2<KIND>;
  const CUtensorMapDataType dt = is_bf16_kind(KIND) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const int eb = T::kElemBytes;
  const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tm_a, tm_bhi, tm_blo, tm_out, tm_sfa, tm_sfhi, tm_sflo;
  int rc;
  if (!A_MN) rc = make_map2(&tm_a, dt, eb, a, p.M, p.K, T::kStageK, BM, sw);
  else rc = make_map2(&tm_a, dt, eb, a, p.K, p.M, 128 / eb, T::kStageK, sw);
  if (rc != TCFP_OK) return rc;
  const int b_rows = T::kSum ? BN / 2 : BN;    // B rows (columns of the output) one CTA stages per operand
  if (!B_MN) {
    if ((rc = make_map2(&tm_bhi, dt, eb, b_hi, p.N, p.K, T::kStageK, b_rows, sw)) != TCFP_OK) return rc;
    if ((rc = make_map2(&tm_blo, dt, eb, b_lo ? b_lo : b_hi, p.N, p.K, T::kStageK, b_rows, sw)) != TCFP_OK) return rc;
  } else {
    // boxes are one 128-byte swizzle row wide; a CTA whose share is 256 bytes wide loads two
    if ((b_rows * eb) % 128 != 0) return fail(TCFP_ERR_UNSUPPORTED, "pair kernel: this operand layout is not tiled");
    if ((rc = make_map2(&tm_bhi, dt, eb, b_hi, p.K, p.N, 128 / eb, T::kStageK, sw)) != TCFP_OK) return rc;
    if ((rc = make_map2(&tm_blo, dt, eb, b_lo ? b_lo : b_hi, p.K, p.N, 128 / eb, T::kStageK, sw)) != TCFP_OK) return rc;
  }
  if (OUT_BF16) rc = make_map2(&tm_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, p.M, p.N, 64, BM, sw);
  else rc = make_map2(&tm_out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, out, p.M, p.N, 32, BM, sw);
  if (rc != TCFP_OK) return rc;
  tm_sfa = tm_a; tm_sfhi = tm_a; tm_sflo = tm_a;
  if (KIND == KIND_MXF8) {
    // packed scale factors as a (chunks x 128 words) matrix, one 512-byte chunk per row
    const int64_t kg = ((p.K / p.block_size) + 3) / 4;
    const int64_t chunks_a = ((p.M + 127) / 128) * kg, chunks_b = ((p.N + 127) / 128) * kg;
    const CUtensorMapSwizzle none = CU_TENSOR_MAP_SWIZZLE_NONE;
    if ((rc = make_map2(&tm_sfa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, sf_a, chunks_a, 128, 128, 1, none)) != TCFP_OK) return rc;
    if ((rc = make_map2(&tm_sfhi, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, sf_hi, chunks_b, 128, 128, 1, none)) != TCFP_OK) return rc;
    if ((rc = make_map2(&tm_sflo, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, sf_lo ? sf_lo : sf_hi, chunks_b, 128, 128, 1, none)) != TCFP_OK) return rc;
  }

  p.status = device_status_ptr();
  // rows of tiles swept together before moving to the next column band: a larger group re-reads the B
  // operand from HBM fewer times (8192^3: 16 instead of 8 cut the per-tensor forward from 0.740 to 0.720 ms
  // and its dX from 0.724 to 0.702 ms; the block-scaled kind measured no better, 32 measured worse for all)
  p.group_m = (KIND == KIND_F8) ? 2 * kGroupM : kGroupM;
  p.k_stages = (p.K + T::kStageK - 1) / T::kStageK;
  p.has_lo = b_lo != nullptr;
  constexpr int smem = smem_bytes2<KIND>();
  auto kern = dual_gemm_pair_kernel<KIND, B_MN, OUT_BF16, A_MN>;
  static bool configured[64] = {false};  // per template instance and device
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(TCFP_ERR_UNSUPPORTED, "device index %d out of range", dev);
  if (!configured[dev]) {
    CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev] = true;
  }
  const int tile_n = (!T::kSum && !p.has_lo) ? 2 * BN : BN;
  const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + tile_n - 1) / tile_n);
  const int max_pairs = gemm_sm_budget() / 2;
  const int pairs = tiles < max_pairs ? tiles : max_pairs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tm_a, tm_bhi, tm_blo, tm_out, tm_sfa, tm_sfhi, tm_sflo, p));
  return TCFP_OK;
}

}  // namespace

// Entry points used by the C ABI functions in gemm_sm100.cu.  kind: KIND_*.
int pair_gemm_dispatch(int kind, bool a_mn, bool b_mn, bool out_bf16, const void* a, const void* b_hi, const void* b_lo,
                       const void* sf_a, const void* sf_hi, const void* sf_lo, void* out, int M, int N, int K, int a_fmt,
                       int block_size, const float* s_a, const float* s_hi, const float* s_lo, const float* bias,
                       cudaStream_t stream) {
  Gemm2Params p{};
  p.M = M; p.N = N; p.K = K;
  p.a_fmt = a_fmt;
  p.block_size = block_size;
  p.s_a = s_a; p.s_hi = s_hi; p.s_lo = s_lo; p.bias = bias;
#define TCFP_PAIR(KIND, BMN)                                                                              \
  return out_bf16 ? launch2<KIND, BMN, true>(a, b_hi, b_lo, sf_a, sf_hi, sf_lo, out, p, stream)           \
                  : launch2<KIND, BMN, false>(a, b_hi, b_lo, sf_a, sf_hi, sf_lo, out, p, stream)
  if (a_mn) {
    if (!b_mn || kind == KIND_MXF8) return fail(TCFP_ERR_UNSUPPORTED, "pair kernel: transposed A is built for the weight gradients only");
    if (kind == KIND_BF16 && b_lo == nullptr)
      return out_bf16 ? launch2<KIND_BF16_WIDE, true, true, true>(a, b_hi, b_lo, sf_a, sf_hi, sf_lo, out, p, stream)
                      : launch2<KIND_BF16_WIDE, true, false, true>(a, b_hi, b_lo, sf_a, sf_hi, sf_lo, out, p, stream);
    if (kind == KIND_BF16)
      return out_bf16 ? launch2<KIND_BF16, true, true, true>(a, b_hi, b_lo, sf_a, sf_hi, sf_lo, out, p, stream)
                      : launch2<KIND_BF16, true, false, true>(a, b_hi, b_lo, sf_a, sf_hi, sf_lo, out, p, stream);
    return out_bf16 ? launch2<KIND_F8, true, true, true>(a, b_hi, b_lo, sf_a, sf_hi, sf_lo, out, p, stream)
                    : launch2<KIND_F8, true, false, true>(a, b_hi, b_lo, sf_a, sf_hi, sf_lo, out, p, stream);
  }
  if (kind == KIND_F8) { if (b_mn) { TCFP_PAIR(KIND_F8, true); } else { TCFP_PAIR(KIND_F8, false); } }
  if (kind == KIND_MXF8) { TCFP_PAIR(KIND_MXF8, false); }
  if (kind == KIND_BF16) { if (b_mn) { TCFP_PAIR(KIND_BF16, true); } else { TCFP_PAIR(KIND_BF16, false); } }
#undef TCFP_PAIR
  return fail(TCFP_ERR_INVALID, "pair kernel: unknown kind %d", kind);
}

}  // namespace tcfp
