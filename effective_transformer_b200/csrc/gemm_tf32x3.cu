// fp32 projections on the tensor cores without giving up fp32 accuracy:
//   C[M,N] = epilogue(A[M,K] * W[K,N] (+ bias)),  fp32 in, fp32 out.
// tcgen05 has no fp32 x fp32 MMA; kind::tf32 keeps 11 significand bits of each
// operand.  Every operand is therefore split into two tf32 numbers,
//   x = hi + lo,  hi = rn_tf32(x),  lo = x - hi  (exact in fp32, |lo| <= 2^-12 |x|),
// and the product is taken as  hi*hi + hi*lo + lo*hi  with fp32 accumulation in
// TMEM: the dropped lo*lo term and the rounding of lo are of relative size
// 2^-22, i.e. the result is as accurate as an fp32 FMA chain (the 1e-4 * RMS
// gate of the fp32 path needs about 2^-17).  A stage of the shared-memory ring
// holds the four operand tiles of one 32-wide k-block (A_hi, A_lo, W_hi, W_lo)
// and feeds the three products from them: four tiles fetched per three MMA
// groups instead of six, because the kernel is bound by the L2 -> SM traffic.
// W_hi / W_lo ([N,K], K-major) are made once when weights are registered; A_hi /
// A_lo by split_tf32_kernel in front of each projection.  Replaces the fp32
// cublasGemmEx call sites of the reference's layer functor
// (tf_op/bert_transformer_op.cu.cc:110-141,200-209,215-225,229-240) for the
// FP32 OperationType (common.h:26).
//
// Kernel structure as in gemm_tcgen05.cu (one persistent CTA per SM, 320
// threads: TMA producer warp, MMA issuer warp, eight epilogue warps; 3-stage
// shared-memory ring, a stage = four [128 x 32] fp32 tiles with the 128-byte
// swizzle), every wait bounded.  The accumulation differs: see the
// note on units in front of the kernel.
#include "common.cuh"
#include "ptx_sm100.cuh"

#include <cstdlib>
#include <mutex>

namespace etb {

namespace {

using namespace ptx;

constexpr int BM = 128;
constexpr int BK = 32;     // 32 fp32 = 128 bytes = one swizzle row
constexpr int UMMA_K = 8;  // kind::tf32: 8 elements = 32 bytes per instruction
constexpr int kEpilogueWarps = 8;
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr int kNumThreads = 64 + kEpilogueThreads;

constexpr int kStagingFloatsPerWarp = 32 * 32;  // epilogue staging: 32 rows x 32 columns per warp
constexpr int kStagingBytes = kEpilogueWarps * kStagingFloatsPerWarp * 4;

constexpr int BN = 128;    // four TMEM blocks of BN columns hold the units in flight
struct Cfg {
  static constexpr int kStages = 3;
  static constexpr int kABytes = BM * BK * 4;
  static constexpr int kBBytes = BN * BK * 4;
  static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;  // A_hi, A_lo, W_hi, W_lo
  static constexpr int kNumBars = 2 * kStages + 2 * 4 + 1;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + kStagingBytes;
  static constexpr int kTmemCols = 4 * BN;
};

enum Site : int {
  kSiteProducerEmpty = 1,
  kSiteProducerDrain = 2,
  kSiteMmaTmemEmpty = 3,
  kSiteMmaFull = 4,
  kSiteMmaDrain = 5,
  kSiteEpilogueFull = 6,
  kSiteSmemAlign = 7,
};

// Instruction descriptor for kind::tf32: bits [4,6) D format (1 = f32), [7,10) A
// format and [10,13) B format (2 = tf32), A and B K-major, [17,23) N >> 3,
// [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_tf32_f32acc(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Epilogue store of one warp: 32 rows (one per lane) x 32 columns of finished sums.
// Bias and activation are applied in the row-per-thread layout; the values then
// pass through a 32 x 32 float staging buffer of the warp (4 KB, 16-byte groups
// swizzled by row: conflict-free both ways) so that every global store
// instruction covers whole 128-byte row segments (4 rows x 128 bytes) instead of
// 32 rows x 16 bytes.  c_lo given: the result is written already split for the
// projection that reads it next, rn_tf32 half to C and remainder to c_lo.

template <int EPI>
__device__ __forceinline__ void store_chunk(float* stage, const float* vals, float* __restrict__ C,
                                            float* __restrict__ c_lo, const float* __restrict__ bias, int N,
                                            int row0, int col, int M, int lane) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    float f[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) f[e] = vals[g * 4 + e];
    if (EPI != kEpiNone) {
      float fb[4];
      VecTraits<float>::unpack(ld_global_v4(bias + col + g * 4), fb);
#pragma unroll
      for (int e = 0; e < 4; ++e) f[e] += fb[e];
    }
    if (EPI == kEpiBiasGelu) {
#pragma unroll
      for (int e = 0; e < 4; ++e) f[e] = gelu_tanh(f[e]);
    } else if (EPI == kEpiBiasTanh) {
#pragma unroll
      for (int e = 0; e < 4; ++e) f[e] = tanhf(f[e]);
    }
    *reinterpret_cast<float4*>(stage + lane * 32 + ((g ^ (lane & 7)) << 2)) = make_float4(f[0], f[1], f[2], f[3]);
  }
  __syncwarp();
  const int g = lane & 7;
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    const int r = t * 4 + (lane >> 3);
    const float4 v = *reinterpret_cast<const float4*>(stage + r * 32 + ((g ^ (r & 7)) << 2));
    const int row = row0 + r;
    if (row < M) {
      const size_t off = static_cast<size_t>(row) * N + col + g * 4;
      if (c_lo == nullptr) {
        *reinterpret_cast<float4*>(C + off) = v;
      } else {
        const float4 hi = make_float4(rn_tf32(v.x), rn_tf32(v.y), rn_tf32(v.z), rn_tf32(v.w));
        *reinterpret_cast<float4*>(C + off) = hi;
        *reinterpret_cast<float4*>(c_lo + off) = make_float4(v.x - hi.x, v.y - hi.y, v.z - hi.z, v.w - hi.w);
      }
    }
  }
  __syncwarp();  // the buffer is reused by the next chunk
}

// The same for 32 rows x 16 columns (2 KB of staging): a store instruction covers
// 8 rows x 64 bytes.
template <int EPI>
__device__ __forceinline__ void store_chunk16(float* stage, const float* vals, float* __restrict__ C,
                                              float* __restrict__ c_lo, const float* __restrict__ bias, int N,
                                              int row0, int col, int M, int lane) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float f[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) f[e] = vals[g * 4 + e];
    if (EPI != kEpiNone) {
      float fb[4];
      VecTraits<float>::unpack(ld_global_v4(bias + col + g * 4), fb);
#pragma unroll
      for (int e = 0; e < 4; ++e) f[e] += fb[e];
    }
    if (EPI == kEpiBiasGelu) {
#pragma unroll
      for (int e = 0; e < 4; ++e) f[e] = gelu_tanh(f[e]);
    } else if (EPI == kEpiBiasTanh) {
#pragma unroll
      for (int e = 0; e < 4; ++e) f[e] = tanhf(f[e]);
    }
    *reinterpret_cast<float4*>(stage + lane * 16 + ((g ^ ((lane >> 1) & 3)) << 2)) = make_float4(f[0], f[1], f[2], f[3]);
  }
  __syncwarp();
  const int g = lane & 3;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int r = t * 8 + (lane >> 2);
    const float4 v = *reinterpret_cast<const float4*>(stage + r * 16 + ((g ^ ((r >> 1) & 3)) << 2));
    const int row = row0 + r;
    if (row < M) {
      const size_t off = static_cast<size_t>(row) * N + col + g * 4;
      if (c_lo == nullptr) {
        *reinterpret_cast<float4*>(C + off) = v;
      } else {
        const float4 hi = make_float4(rn_tf32(v.x), rn_tf32(v.y), rn_tf32(v.z), rn_tf32(v.w));
        *reinterpret_cast<float4*>(C + off) = hi;
        *reinterpret_cast<float4*>(c_lo + off) = make_float4(v.x - hi.x, v.y - hi.y, v.z - hi.z, v.w - hi.w);
      }
    }
  }
  __syncwarp();  // the buffer is reused by the next chunk
}

// hi = rn_tf32(x), lo = x - hi, four elements per thread and iteration.  hi or lo
// may be the same array as x (each element is read, then written, by one thread).
__global__ void __launch_bounds__(256)
split_tf32_kernel(const float* x, float* hi, float* lo,
                  const int* __restrict__ rows_ptr, int max_rows, int cols) {
  pdl_wait();
  pdl_trigger();
  int rows = rows_ptr != nullptr ? *rows_ptr : max_rows;
  rows = rows < 0 ? 0 : (rows > max_rows ? max_rows : rows);
  const long long n4 = static_cast<long long>(rows) * cols / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const Vec16 v = ld_global_v4(x + i * 4);
    float f[4], h[4], l[4];
    VecTraits<float>::unpack(v, f);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      h[e] = rn_tf32(f[e]);
      l[e] = f[e] - h[e];
    }
    st_global_v4(hi + i * 4, VecTraits<float>::pack(h));
    st_global_v4(lo + i * 4, VecTraits<float>::pack(l));
  }
}

// One tile = 128 x BN of C.  Its K/32 k-blocks are cut into units of kUnitKb
// k-blocks (three products each); a unit is accumulated from zero in one of four
// TMEM blocks of BN columns (used round-robin), and the epilogue warps add
// finished units into fp32 registers.  Reason: the tensor core adds into its fp32
// accumulator with truncation, so a single chain over all 3K/8 instructions
// drifts by about 1e-4 relative at K = 3072; 72-instruction chains summed with
// round-to-nearest stay at the level of an fp32 FMA loop.  The unit is also the
// slack of the pipeline: the issuer runs (number of blocks) units ahead of the
// epilogue warps, which must fit a tile's bias / activation / store phase into
// that time; with units of 3 k-blocks the issuer waited for TMEM 19-27 % of a
// K = 768 projection.  Draining a unit overlaps the MMAs of
// the next ones, so the issuer never waits for the epilogue in steady state.
constexpr int kUnitKb = 6;
constexpr int kTmemBlocks = 4;

template <int EPI>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmap_a_hi, const __grid_constant__ CUtensorMap tmap_a_lo,
                   const __grid_constant__ CUtensorMap tmap_w_hi, const __grid_constant__ CUtensorMap tmap_w_lo,
                   float* __restrict__ C, float* __restrict__ c_lo, const float* __restrict__ bias,
                   const int* __restrict__ m_ptr, int max_m, int N, int K, int* status_word, int reverse_m) {
  using cfg = Cfg;
  constexpr int S = cfg::kStages;

  // The prologue (barriers, TMEM) touches no global memory: it runs before the
  // wait on the preceding kernel, under that kernel's tail.
  pdl_trigger();

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t tiles_addr = smem_u32(smem_raw);
  if ((tiles_addr & 1023u) != 0u) {
    pdl_wait();  // no CTA leaves before the preceding kernel has completed
    if (threadIdx.x == 0) report_timeout(status_word, kKernelGemmTc, kSiteSmemAlign);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + S * cfg::kStageBytes);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
  auto tmem_full_bar = [&](int a) { return bar0 + 8u * (2 * S + a); };
  auto tmem_empty_bar = [&](int a) { return bar0 + 8u * (2 * S + kTmemBlocks + a); };
  const uint32_t drain_bar = bar0 + 8u * (2 * S + 2 * kTmemBlocks);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + cfg::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < kTmemBlocks; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), kEpilogueThreads);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_wait();  // M and the A rows come from earlier kernels
  int M = *m_ptr;
  M = M < 0 ? 0 : (M > max_m ? max_m : M);
  const int m_tiles = (M + BM - 1) / BM;
  const int n_tiles = N / BN;
  const int num_tiles = m_tiles * n_tiles;  // 0: every role's loop is empty
  const int num_kb = K / BK;
  const int units_per_tile = (num_kb + kUnitKb - 1) / kUnitKb;

  auto fail = [&](int site) {
    *abort_flag = 1;
    report_timeout(status_word, kKernelGemmTc, site);
  };

  if (warp == 0) {
    // ------------------------- TMA producer -------------------------
    if (lane == 0) {
      prefetch_tensormap(&tmap_a_hi);
      prefetch_tensormap(&tmap_a_lo);
      prefetch_tensormap(&tmap_w_hi);
      prefetch_tensormap(&tmap_w_lo);
      uint32_t stage = 0, phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m_lin = tile / n_tiles, n_tile = tile - m_lin * n_tiles;
        const int m_tile = reverse_m ? m_tiles - 1 - m_lin : m_lin;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            fail(kSiteProducerEmpty);
            ok = false;
            break;
          }
          const uint32_t a_dst = tiles_addr + stage * cfg::kStageBytes;
          const uint32_t b_dst = a_dst + 2 * cfg::kABytes;
          mbar_arrive_expect_tx(full_bar(stage), cfg::kStageBytes);
          tma_load_2d(a_dst, &tmap_a_hi, kb * BK, m_tile * BM, full_bar(stage));
          tma_load_2d(b_dst, &tmap_w_hi, kb * BK, n_tile * BN, full_bar(stage));
          tma_load_2d(b_dst + cfg::kBBytes, &tmap_w_lo, kb * BK, n_tile * BN, full_bar(stage));
          tma_load_2d(a_dst + cfg::kABytes, &tmap_a_lo, kb * BK, m_tile * BM, full_bar(stage));
          ++issued;
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // copies still in flight must land before the CTA's shared memory goes away
      const long long pending = issued < S ? issued : S;
      for (long long i = 0; i < pending; ++i) {
        const long long f = issued - 1 - i;
        if (!mbar_wait(full_bar(static_cast<int>(f % S)), static_cast<uint32_t>((f / S) & 1), abort_flag) &&
            *abort_flag == 0)
          fail(kSiteProducerDrain);
      }
    }
  } else if (warp == 1) {
    // ------------------------- MMA issuer -------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_tf32_f32acc(BM, BN);
      uint32_t stage = 0, phase = 0;
      uint32_t unit = 0;  // running over all tiles of this CTA: TMEM block = unit % 4
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb0 = 0; kb0 < num_kb && ok; kb0 += kUnitKb, ++unit) {
          const int blk = unit % kTmemBlocks;
          const uint32_t blk_phase = (unit / kTmemBlocks) & 1u;
          if (!mbar_wait(tmem_empty_bar(blk), blk_phase ^ 1u, abort_flag)) {
            fail(kSiteMmaTmemEmpty);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + blk * BN;
          const int kb1 = min(kb0 + kUnitKb, num_kb);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
              fail(kSiteMmaFull);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_addr = tiles_addr + stage * cfg::kStageBytes;
            const uint64_t a_hi = make_kmajor_sw128_desc(a_addr);
            const uint64_t a_lo = make_kmajor_sw128_desc(a_addr + cfg::kABytes);
            const uint64_t w_hi = make_kmajor_sw128_desc(a_addr + 2 * cfg::kABytes);
            const uint64_t w_lo = make_kmajor_sw128_desc(a_addr + 2 * cfg::kABytes + cfg::kBBytes);
            // 8 fp32 = 32 bytes inside the swizzle row: +2 in the address field
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_tf32_ss(d_tmem, a_hi + 2u * k, w_hi + 2u * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) umma_tf32_ss(d_tmem, a_hi + 2u * k, w_lo + 2u * k, idesc, 1u);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) umma_tf32_ss(d_tmem, a_lo + 2u * k, w_hi + 2u * k, idesc, 1u);
            umma_commit(empty_bar(stage));
            if (++stage == S) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok) umma_commit(tmem_full_bar(blk));
        }
      }
      umma_commit(drain_bar);  // all MMAs must have retired before TMEM is freed
      if (!mbar_wait(drain_bar, 0u, abort_flag) && *abort_flag == 0) fail(kSiteMmaDrain);
    }
  } else {
    // ------------------------- epilogue -------------------------
    // warp w reads TMEM lanes [32*(w%4), +32) (one output row per thread) and one
    // half (64) of the tile's columns, kept as a running fp32 sum in registers.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int kCols = BN / 2;
    float* stage = reinterpret_cast<float*>(smem_raw + S * cfg::kStageBytes + cfg::kBarrierBytes) +
                   (warp - 2) * kStagingFloatsPerWarp;
    uint32_t unit = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m_lin = tile / n_tiles, n_tile = tile - m_lin * n_tiles;
      const int m_tile = reverse_m ? m_tiles - 1 - m_lin : m_lin;
      const int col0 = n_tile * BN + half * kCols;
      float sum[kCols];
#pragma unroll
      for (int e = 0; e < kCols; ++e) sum[e] = 0.f;
      for (int ui = 0; ui < units_per_tile; ++ui, ++unit) {
        const int blk = unit % kTmemBlocks;
        const uint32_t blk_phase = (unit / kTmemBlocks) & 1u;
        const bool got = mbar_wait(tmem_full_bar(blk), blk_phase, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) fail(kSiteEpilogueFull);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + blk * BN + half * kCols;
        uint32_t r[kCols];
        tmem_ld_32x32b_x32(t_row, r);
        tmem_ld_32x32b_x32(t_row + 32, r + 32);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(tmem_empty_bar(blk));  // the unit is in registers: hand the TMEM block back
#pragma unroll
        for (int e = 0; e < kCols; ++e) sum[e] += __uint_as_float(r[e]);
      }
      if (!ok) break;
#pragma unroll
      for (int ch = 0; ch < kCols / 32; ++ch)
        store_chunk<EPI>(stage, sum + ch * 32, C, c_lo, bias, N, m_tile * BM + quad * 32, col0 + ch * 32, M, lane);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------------------
// CTA-pair variant (N % 256 == 0): a cluster of two CTAs computes a 256 x 256
// tile with tcgen05.mma cta_group::2.  Per k-block each CTA fetches A_hi / A_lo
// for its 128 rows and W_hi / W_lo for 128 of the tile's 256 W rows: 64 KB per
// 3 x 4 instructions of 128 x 256 x 8 per CTA, half of the L2 -> SM traffic per
// FLOP of the single-CTA kernel, which is what bounds that kernel.  No load is
// multicast.  The accumulator of a unit is a 256-column TMEM block in each CTA;
// the 512 columns hold two blocks, drained by the epilogue warps (64 running
// sums per thread) while the other block accumulates.  Barriers as in the
// fp16 pair kernel: full[] and tmem_empty[] live in CTA 0, empty[] and
// tmem_full[] in both (CTA 0's MMA thread commits to both).  The last round of
// tiles is cut into 256 x 128 units when it would occupy at most half of the
// pairs (pair_units()).
// ---------------------------------------------------------------------------
constexpr int BM2 = 2 * BM;
constexpr int BN2 = 256;
constexpr int kPairBlocks = 2;
// Sixteen epilogue warps (four per TMEM lane quadrant, a quarter of the columns each): with
// eight, a thread holds 128 running sums and the bias / GELU / split / store phase of a tile,
// squeezed into the remaining registers with two warps per scheduler, took about 27 k cycles
// per tile of the GELU projection, more than the two accumulation units (18 k cycles) the
// issuer can run ahead.
constexpr int kPairEpilogueWarps = 16;
constexpr int kPairThreads = 64 + kPairEpilogueWarps * 32;
constexpr int kPairStagingFloatsPerWarp = 32 * 16;  // 32 rows x 16 columns
struct PairCfg {
  static constexpr int kStages = 3;
  static constexpr int kABytes = BM * BK * 4;          // this CTA's 128 rows of A_hi (and of A_lo)
  static constexpr int kBBytes = (BN2 / 2) * BK * 4;   // this CTA's 128 rows of W_hi (and of W_lo)
  static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;
  static constexpr int kNumBars = 2 * kStages + 2 * kPairBlocks + 1;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + kPairEpilogueWarps * kPairStagingFloatsPerWarp * 4;
  static constexpr int kTmemCols = kPairBlocks * BN2;
};

__device__ __forceinline__ void umma_tf32_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_tf32x3_pair_kernel(const __grid_constant__ CUtensorMap tmap_a_hi, const __grid_constant__ CUtensorMap tmap_a_lo,
                        const __grid_constant__ CUtensorMap tmap_w_hi, const __grid_constant__ CUtensorMap tmap_w_lo,
                        const __grid_constant__ CUtensorMap tmap_w_hi_half,
                        const __grid_constant__ CUtensorMap tmap_w_lo_half, float* __restrict__ C,
                        float* __restrict__ c_lo, const float* __restrict__ bias, const int* __restrict__ m_ptr,
                        int max_m, int N, int K, int* status_word, int reverse_m) {
  using cfg = PairCfg;
  constexpr int S = cfg::kStages;

  // The prologue touches no global memory: it runs before the wait on the preceding kernel.
  pdl_trigger();
  const uint32_t rank = cluster_ctarank();  // 0 issues the MMAs
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t tiles_addr = smem_u32(smem_raw);
  if ((tiles_addr & 1023u) != 0u) {  // same layout in both CTAs: uniform for the pair
    pdl_wait();  // no CTA leaves before the preceding kernel has completed
    if (threadIdx.x == 0) report_timeout(status_word, kKernelGemmTc, kSiteSmemAlign);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + S * cfg::kStageBytes);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
  auto tmem_full_bar = [&](int a) { return bar0 + 8u * (2 * S + a); };
  auto tmem_empty_bar = [&](int a) { return bar0 + 8u * (2 * S + kPairBlocks + a); };
  const uint32_t drain_bar = bar0 + 8u * (2 * S + 2 * kPairBlocks);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + cfg::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < kPairBlocks; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 2 * kPairEpilogueWarps);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), cfg::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  pdl_wait();  // M and the A rows come from earlier kernels
  int M = *m_ptr;
  M = M < 0 ? 0 : (M > max_m ? max_m : M);
  const int m_tiles = (M + BM2 - 1) / BM2;
  const int n_tiles = N / BN2;
  const int num_tiles = m_tiles * n_tiles;  // 0: every role's loop is empty
  const int num_kb = K / BK;
  const int units_per_tile = (num_kb + kUnitKb - 1) / kUnitKb;  // accumulation units, not work units
  int num_units;
  const int full_tiles = pair_units(num_tiles, num_pairs, &num_units);

  auto fail = [&](int site) {
    *abort_flag = 1;
    report_timeout(status_word, kKernelGemmTc, site);
  };

  if (warp == 0) {
    // ------------------------- TMA producer (both CTAs) -------------------------
    if (lane == 0) {
      prefetch_tensormap(&tmap_a_hi);
      prefetch_tensormap(&tmap_a_lo);
      prefetch_tensormap(&tmap_w_hi);
      prefetch_tensormap(&tmap_w_lo);
      uint32_t stage = 0, phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int u = pair_id; u < num_units && ok; u += num_pairs) {
        const PairUnit pu = pair_unit(u, full_tiles, n_tiles, m_tiles, reverse_m);
        const int a_row = pu.m_tile * BM2 + static_cast<int>(rank) * BM;
        const int b_row = pu.col0 + static_cast<int>(rank) * (pu.ncols / 2);
        const bool whole = pu.ncols == BN2;
        const uint32_t stage_tx = 2u * (2u * cfg::kABytes + (whole ? 2u * cfg::kBBytes : cfg::kBBytes));
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            fail(kSiteProducerEmpty);
            ok = false;
            break;
          }
          const uint32_t a_dst = tiles_addr + stage * cfg::kStageBytes;
          const uint32_t b_dst = a_dst + 2 * cfg::kABytes;
          const uint32_t full0 = mapa_shared(full_bar(stage), 0);
          if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), stage_tx);
          tma_load_2d_pair(a_dst, &tmap_a_hi, kb * BK, a_row, full0);
          tma_load_2d_pair(b_dst, whole ? &tmap_w_hi : &tmap_w_hi_half, kb * BK, b_row, full0);
          tma_load_2d_pair(b_dst + cfg::kBBytes, whole ? &tmap_w_lo : &tmap_w_lo_half, kb * BK, b_row, full0);
          tma_load_2d_pair(a_dst + cfg::kABytes, &tmap_a_lo, kb * BK, a_row, full0);
          ++issued;
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (rank == 0) {
        // full[] counts both CTAs' bytes: once these phases are complete no copy
        // of the pair is in flight; the peer learns it at the closing cluster barrier.
        const long long pending = issued < S ? issued : S;
        for (long long i = 0; i < pending; ++i) {
          const long long f = issued - 1 - i;
          if (!mbar_wait(full_bar(static_cast<int>(f % S)), static_cast<uint32_t>((f / S) & 1), abort_flag) &&
              *abort_flag == 0)
            fail(kSiteProducerDrain);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------- MMA issuer (CTA 0 only) -------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_whole = make_idesc_tf32_f32acc(BM2, BN2);
      constexpr uint32_t idesc_half = make_idesc_tf32_f32acc(BM2, BN2 / 2);
      uint32_t stage = 0, phase = 0;
      uint32_t unit = 0;  // accumulation units over all work units of this pair: TMEM block = unit % 2
      bool ok = true;
      for (int u = pair_id; u < num_units && ok; u += num_pairs) {
        const uint32_t idesc = u < full_tiles ? idesc_whole : idesc_half;
        for (int kb0 = 0; kb0 < num_kb && ok; kb0 += kUnitKb, ++unit) {
          const int blk = unit % kPairBlocks;
          const uint32_t blk_phase = (unit / kPairBlocks) & 1u;
          if (!mbar_wait(tmem_empty_bar(blk), blk_phase ^ 1u, abort_flag)) {
            fail(kSiteMmaTmemEmpty);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + blk * BN2;
          const int kb1 = min(kb0 + kUnitKb, num_kb);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
              fail(kSiteMmaFull);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_addr = tiles_addr + stage * cfg::kStageBytes;
            const uint64_t a_hi = make_kmajor_sw128_desc(a_addr);
            const uint64_t a_lo = make_kmajor_sw128_desc(a_addr + cfg::kABytes);
            const uint64_t w_hi = make_kmajor_sw128_desc(a_addr + 2 * cfg::kABytes);
            const uint64_t w_lo = make_kmajor_sw128_desc(a_addr + 2 * cfg::kABytes + cfg::kBBytes);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_tf32_ss_pair(d_tmem, a_hi + 2u * k, w_hi + 2u * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) umma_tf32_ss_pair(d_tmem, a_hi + 2u * k, w_lo + 2u * k, idesc, 1u);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) umma_tf32_ss_pair(d_tmem, a_lo + 2u * k, w_hi + 2u * k, idesc, 1u);
            umma_commit_pair(empty_bar(stage));
            umma_commit_pair(mapa_shared(empty_bar(stage), 1));
            if (++stage == S) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok) {
            umma_commit_pair(tmem_full_bar(blk));
            umma_commit_pair(mapa_shared(tmem_full_bar(blk), 1));
          }
        }
      }
      umma_commit_pair(drain_bar);
      if (!mbar_wait(drain_bar, 0u, abort_flag) && *abort_flag == 0) fail(kSiteMmaDrain);
    }
  } else {
    // ------------------------- epilogue (both CTAs) -------------------------
    // warp w reads TMEM lanes [32*(w%4), +32) (one output row per thread) and one
    // quarter of the unit's columns (64, or 32 in a half-width unit), kept as
    // running fp32 sums in registers.
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;
    constexpr int kCols = BN2 / 4;
    float* stage = reinterpret_cast<float*>(smem_raw + S * cfg::kStageBytes + cfg::kBarrierBytes) +
                   (warp - 2) * kPairStagingFloatsPerWarp;
    uint32_t unit = 0;
    bool ok = true;
    for (int u = pair_id; u < num_units && ok; u += num_pairs) {
      const PairUnit pu = pair_unit(u, full_tiles, n_tiles, m_tiles, reverse_m);
      const int wcols = pu.ncols / 4;        // this warp's columns
      const int chunks = wcols / 16;
      const int col0 = pu.col0 + part * wcols;
      float sum[kCols];
#pragma unroll
      for (int e = 0; e < kCols; ++e) sum[e] = 0.f;
      for (int ui = 0; ui < units_per_tile; ++ui, ++unit) {
        const int blk = unit % kPairBlocks;
        const uint32_t blk_phase = (unit / kPairBlocks) & 1u;
        const bool got = mbar_wait(tmem_full_bar(blk), blk_phase, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {
          if (lane == 0) fail(kSiteEpilogueFull);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + blk * BN2 + part * wcols;
#pragma unroll
        for (int ch = 0; ch < kCols / 16; ++ch)
          if (ch < chunks) {
            uint32_t r[16];
            tmem_ld_32x32b_x16(t_row + ch * 16, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) sum[ch * 16 + e] += __uint_as_float(r[e]);
          }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_shared(tmem_empty_bar(blk), 0));  // the block goes back to the issuer
      }
      if (!ok) break;
      const int row0 = pu.m_tile * BM2 + static_cast<int>(rank) * BM + quad * 32;
#pragma unroll
      for (int ch = 0; ch < kCols / 16; ++ch)
        if (ch < chunks) store_chunk16<EPI>(stage, sum + ch * 16, C, c_lo, bias, N, row0, col0 + ch * 16, M, lane);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still touch its barriers or TMEM
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, cfg::kTmemCols);
  }
}

bool encode_2d_f32_sw128(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                         TensorMapCache* cache) {
  if (cache != nullptr) {
    if (const CUtensorMap* hit = cache->find(4, base, rows, cols, cols, box_rows, BK)) {
      *map = *hit;
      return true;
    }
  }
  EncodeTiledFn fn = get_encode_tiled();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 4};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box,
                        elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache != nullptr) cache->insert(4, base, rows, cols, cols, box_rows, BK, *map);
  return true;
}

template <int EPI>
cudaError_t launch_epi(const CUtensorMap& tah, const CUtensorMap& tal, const CUtensorMap& twh, const CUtensorMap& twl,
                       const float* bias, float* c, float* c_lo, const int* m_ptr, int max_m, int n, int k,
                       int* status_word, int reverse_m, cudaStream_t stream) {
  static PerDeviceOnce once;  // function attributes are per device
  const cudaError_t once_err = once.run([] {
    cudaError_t attr_err = cudaFuncSetAttribute(gemm_tf32x3_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    Cfg::kSmemBytes);
    return attr_err;
  });
  if (once_err != cudaSuccess) return once_err;
  const long long max_tiles = static_cast<long long>((max_m + BM - 1) / BM) * (n / BN);
  long long grid = sm_count();
  if (grid > max_tiles) grid = max_tiles;
  if (grid < 1) grid = 1;
  return launch_pdl(gemm_tf32x3_kernel<EPI>, dim3(static_cast<int>(grid)), dim3(kNumThreads), Cfg::kSmemBytes, stream,
                    tah, tal, twh, twl, c, c_lo, bias, m_ptr, max_m, n, k, status_word, reverse_m);
}

template <int EPI>
cudaError_t launch_pair_epi(const CUtensorMap& tah, const CUtensorMap& tal, const CUtensorMap& twh,
                            const CUtensorMap& twl, const CUtensorMap& twhh, const CUtensorMap& twlh, const float* bias,
                            float* c, float* c_lo, const int* m_ptr, int max_m, int n, int k, int* status_word,
                            int reverse_m, cudaStream_t stream) {
  static PerDeviceOnce once;  // function attributes are per device
  const cudaError_t once_err = once.run([] {
    cudaError_t attr_err = cudaFuncSetAttribute(gemm_tf32x3_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    PairCfg::kSmemBytes);
    return attr_err;
  });
  if (once_err != cudaSuccess) return once_err;
  const long long max_tiles = static_cast<long long>((max_m + BM2 - 1) / BM2) * (n / BN2);
  long long pairs = sm_count() / 2;
  if (pairs > max_tiles) pairs = max_tiles;
  if (pairs < 1) pairs = 1;
  return launch_pdl(gemm_tf32x3_pair_kernel<EPI>, dim3(static_cast<int>(2 * pairs)), dim3(kPairThreads),
                    PairCfg::kSmemBytes, stream, tah, tal, twh, twl, twhh, twlh, c, c_lo, bias, m_ptr, max_m, n, k,
                    status_word, reverse_m);
}

}  // namespace

cudaError_t launch_split_tf32(const float* x, float* hi, float* lo, const int* rows_ptr, int max_rows, int cols,
                              cudaStream_t stream) {
  if (max_rows <= 0 || cols <= 0) return cudaSuccess;
  if ((cols % 4) != 0) return cudaErrorInvalidValue;
  const long long n4 = static_cast<long long>(max_rows) * cols / 4;
  long long ctas = (n4 + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (ctas > cap) ctas = cap;
  return launch_pdl(split_tf32_kernel, dim3(static_cast<int>(ctas)), dim3(256), 0, stream, x, hi, lo, rows_ptr,
                    max_rows, cols);
}

cudaError_t launch_gemm_tf32x3(const float* a_hi, const float* a_lo, const float* w_hi, const float* w_lo,
                               const float* bias, float* c, const int* m_ptr, int max_m, int n, int k,
                               int epilogue, int* status_word, cudaStream_t stream, bool reverse_m, float* c_lo,
                               TensorMapCache* maps) {
  if (max_m <= 0) return cudaSuccess;
  if (n <= 0 || k <= 0 || (n % 128) != 0 || (k % BK) != 0) return cudaErrorInvalidValue;
  for (const void* p : {static_cast<const void*>(a_hi), static_cast<const void*>(a_lo),
                        static_cast<const void*>(w_hi), static_cast<const void*>(w_lo),
                        static_cast<const void*>(c)})
    if (p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u)) return cudaErrorMisalignedAddress;
  if (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 15u)) return cudaErrorMisalignedAddress;
  if (c_lo != nullptr && (reinterpret_cast<uintptr_t>(c_lo) & 15u)) return cudaErrorMisalignedAddress;
  if (epilogue != kEpiNone && bias == nullptr) return cudaErrorInvalidValue;
  CUtensorMap tah, tal, twh, twl;
  if (!encode_2d_f32_sw128(&tah, a_hi, static_cast<uint64_t>(max_m), static_cast<uint64_t>(k), BM, maps) ||
      !encode_2d_f32_sw128(&tal, a_lo, static_cast<uint64_t>(max_m), static_cast<uint64_t>(k), BM, maps) ||
      !encode_2d_f32_sw128(&twh, w_hi, static_cast<uint64_t>(n), static_cast<uint64_t>(k), BN, maps) ||
      !encode_2d_f32_sw128(&twl, w_lo, static_cast<uint64_t>(n), static_cast<uint64_t>(k), BN, maps))
    return cudaErrorInvalidValue;
  const int rev = reverse_m ? 1 : 0;
  // The pair kernel needs enough 256 x 256 tiles at capacity to occupy the pairs; below that
  // the 128 x 128 tiles of the one-CTA kernel spread a small batch over more SMs.
  const long long pair_tiles = static_cast<long long>((max_m + BM2 - 1) / BM2) * (n / BN2);
  if ((n % BN2) == 0 && pair_tiles >= sm_count() / 2) {
    // the W maps above (128-row boxes) serve whole tiles; half-width units take 64 rows per CTA
    CUtensorMap twhh, twlh;
    if (!encode_2d_f32_sw128(&twhh, w_hi, static_cast<uint64_t>(n), static_cast<uint64_t>(k), 64, maps) ||
        !encode_2d_f32_sw128(&twlh, w_lo, static_cast<uint64_t>(n), static_cast<uint64_t>(k), 64, maps))
      return cudaErrorInvalidValue;
#define ETB_PAIR_CASE(E) \
  case E:                \
    return launch_pair_epi<E>(tah, tal, twh, twl, twhh, twlh, bias, c, c_lo, m_ptr, max_m, n, k, status_word, rev, \
                              stream)
    switch (epilogue) {
      ETB_PAIR_CASE(kEpiNone);
      ETB_PAIR_CASE(kEpiBias);
      ETB_PAIR_CASE(kEpiBiasGelu);
      ETB_PAIR_CASE(kEpiBiasTanh);
      default:
        return cudaErrorInvalidValue;
    }
#undef ETB_PAIR_CASE
  }
#define ETB_CASE(E) \
  case E:           \
    return launch_epi<E>(tah, tal, twh, twl, bias, c, c_lo, m_ptr, max_m, n, k, status_word, rev, stream)
  switch (epilogue) {
    ETB_CASE(kEpiNone);
    ETB_CASE(kEpiBias);
    ETB_CASE(kEpiBiasGelu);
    ETB_CASE(kEpiBiasTanh);
    default:
      return cudaErrorInvalidValue;
  }
#undef ETB_CASE
}

}  // namespace etb
