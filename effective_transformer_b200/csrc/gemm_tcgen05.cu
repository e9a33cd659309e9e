// Dense projections on the 5th-generation tensor cores:
//   C[M,N] = epilogue(A[M,K] * Wp[N,K]^T (+ bias)),  fp16 in, fp32 accumulate in
//   TMEM, fp16 out.
// Replaces the cublasGemmEx call sites of the reference's layer functor
// (tf_op/bert_transformer_op.cu.cc:110-141,200-209,215-225,229-240) and folds
// add_bias_act (cuda/cuda_kernels.cu:88-134) / the bias half of
// add_QKV_bias_padding (cuda/attention.cu:106-175) into the epilogue.
//
// Structure (one persistent CTA per SM, 320 threads):
//   warp 0   TMA producer: A tile [128 x 64] and W tile [BN x 64] per k-block
//            into a kStages-deep shared-memory ring (128-byte swizzle)
//   warp 1   MMA issuer: tcgen05.mma cta_group::1 kind::f16, M=128, N=BN, K=16,
//            accumulating into one of two TMEM buffers of BN columns
//   warps 2-9 epilogue: tcgen05.ld of the finished accumulator (one TMEM lane
//            quadrant and one half of the columns per warp), bias in fp32,
//            optional GELU / tanh / residual add, staged through shared memory
//            to coalesced stores of C, overlapping the next tile's main loop
// The kernel every BERT projection uses is the CTA-pair variant further down
// (N a multiple of 256); this one covers N = 128 (mod 256).
// M is read from device memory, so no host synchronisation is needed between
// the padding-offset kernel and the projections.  Every mbarrier wait is
// bounded; on expiry the kernel records a code in the status word, all roles
// unwind, TMEM is freed and the kernel returns.
#include "common.cuh"
#include "ptx_sm100.cuh"

#include <cstdlib>
#include <mutex>

namespace etb {

namespace {

using namespace ptx;

constexpr int BM = 128;
constexpr int BK = 64;  // 64 fp16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kEpilogueWarps = 8;  // two per TMEM lane quadrant, each owning half of the tile's columns
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr int kNumThreads = 64 + kEpilogueThreads;

constexpr int kStagingPerWarp = 32 * 128;  // 32 rows x 128 bytes (64 fp16 columns)

// ---- LayerNorm inside the GEMM kernel (kEpiResidualLayerNorm, kEpiLayerNorm) -----------------
// A 32-row block of C can be normalised once all N of its columns are stored, by up to six warps of
// three CTA pairs.  Roles in a CTA of these variants:
//   epilogue warps   store their part of a unit, raise a shared-memory flag, go on
//   counting warp    (one more warp) sees the flags, makes the flagged stores visible to the GPU with
//                    ONE fence for all of them (a fence costs a round trip to L2: too long for every
//                    epilogue warp to wait for it per tile), adds each part's columns to the global
//                    counter of its row block, and publishes the blocks whose count it completed in a
//                    queue of the CTA
//   epilogue warps   normalise four rows each of every published block, in place, in the time they
//                    would otherwise spend waiting for their next accumulator
__host__ __device__ constexpr bool has_ln(int epi) { return epi == kEpiResidualLayerNorm || epi == kEpiLayerNorm; }
// what the accumulator epilogue itself does for an epilogue kind
__host__ __device__ constexpr int base_epi(int epi) {
  return epi == kEpiResidualLayerNorm ? kEpiBiasResidual : epi == kEpiLayerNorm ? kEpiNone : epi;
}
__host__ __device__ constexpr int threads_of(int epi) { return kNumThreads + (has_ln(epi) ? 32 : 0); }
constexpr int kLnRowsPerWarp = 32 / kEpilogueWarps;  // a 32-row block is shared out among the epilogue warps
constexpr int kLnQueue = 32;                         // published blocks a CTA can hold before the slowest warp has done its rows

// LayerNorm of RB consecutive rows of c [*, n] in place by one warp, n = 256 * VPL: lane l holds
// the 16-byte vectors j * 32 + l of a row, statistics in fp32 in two passes over the registers,
// as add_bias_input_layernorm_kernel does (same arithmetic in the same order).  The RB rows are
// worked on side by side (no branch between them), so that one row's dependent chains -- the
// running sums, the shuffles -- hide behind the others'.  Only the first nrows (1..RB) rows
// exist: the others repeat the last one (same values stored to the same place again).
// ADD: x = c + (residual + bias) first.  Rows are read through L2 (other CTAs wrote them).
template <int VPL, bool ADD, int RB>
__device__ __forceinline__ void ln_rows(__half* c, const __half* residual, const __half* bias,
                                        const __half* gamma, const __half* beta, int n, int nrows, float eps,
                                        int lane) {
  const float inv_n = 1.0f / static_cast<float>(n);
  size_t off[RB];
  float x[RB][VPL][8];
  {
    Vec16 vc[RB][VPL], vr[ADD ? RB : 1][VPL];
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      off[r] = static_cast<size_t>(r < nrows ? r : nrows - 1) * n + lane * 8;
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        vc[r][j] = ld_global_cg_v4(c + off[r] + j * 256);
        if (ADD) vr[r][j] = ld_global_nc_v4(residual + off[r] + j * 256);
      }
    }
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      float fb[8];
      if (ADD) VecTraits<__half>::unpack(ld_global_v4(bias + lane * 8 + j * 256), fb);
#pragma unroll
      for (int r = 0; r < RB; ++r) {
        VecTraits<__half>::unpack(vc[r][j], x[r][j]);
        if (ADD) {
          float fi[8];
          VecTraits<__half>::unpack(vr[r][j], fi);
#pragma unroll
          for (int e = 0; e < 8; ++e) x[r][j][e] += fi[e] + fb[e];
        }
      }
    }
  }
  float mean[RB], rstd[RB];
#pragma unroll
  for (int r = 0; r < RB; ++r) {
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) sum += x[r][j][e];
    mean[r] = sum;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
#pragma unroll
    for (int r = 0; r < RB; ++r) mean[r] += __shfl_xor_sync(0xffffffffu, mean[r], o);
#pragma unroll
  for (int r = 0; r < RB; ++r) {
    mean[r] *= inv_n;
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float dlt = x[r][j][e] - mean[r];
        sq += dlt * dlt;
      }
    rstd[r] = sq;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
#pragma unroll
    for (int r = 0; r < RB; ++r) rstd[r] += __shfl_xor_sync(0xffffffffu, rstd[r], o);
#pragma unroll
  for (int r = 0; r < RB; ++r) rstd[r] = rsqrtf(rstd[r] * inv_n + eps);
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    float fg[8], fbe[8];
    VecTraits<__half>::unpack(ld_global_v4(gamma + lane * 8 + j * 256), fg);
    VecTraits<__half>::unpack(ld_global_v4(beta + lane * 8 + j * 256), fbe);
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      float y[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = (x[r][j][e] - mean[r]) * rstd[r] * fg[e] + fbe[e];
      st_global_v4(c + off[r] + j * 256, VecTraits<__half>::pack(y));
    }
  }
}

template <int BN>
struct Cfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kNumBars = 2 * kStages + 5;
  static constexpr int kStagingBytes = kEpilogueWarps * kStagingPerWarp;
  static constexpr int kColsPerWarp = BN / 2;
  static constexpr int kBiasBytes = kEpilogueWarps * kColsPerWarp * 2;  // per-warp fp16 bias slice
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBiasBytes + 256 /*barriers*/;
  static constexpr int kTmemCols = 2 * BN;
};

// tanh-form GELU on a pair of fp16 values (x + bias was formed in fp32 and
// rounded once).  The reference's half kernel does the same step in half2
// (cuda/cuda_kernels.cu:38-51); here the tanh is the hardware f16x2
// approximation too.  Large |x| saturates cleanly: tanh(+-inf) = +-1.
__device__ __forceinline__ uint32_t gelu_tanh_half2(uint32_t xbits) {
  const __half2 x = *reinterpret_cast<const __half2*>(&xbits);
  const __half2 c1 = __float2half2_rn(0.7978845608028654f);
  const __half2 c2 = __float2half2_rn(0.7978845608028654f * 0.044715f);
  const __half2 u = __hmul2(x, __hfma2(__hmul2(x, x), c2, c1));
  const uint32_t ubits = *reinterpret_cast<const uint32_t*>(&u);
  uint32_t tbits;
  asm("tanh.approx.f16x2 %0, %1;" : "=r"(tbits) : "r"(ubits));
  const __half2 th = *reinterpret_cast<const __half2*>(&tbits);
  const __half2 hx = __hmul2(x, __float2half2_rn(0.5f));
  const __half2 y = __hfma2(hx, th, hx);
  return *reinterpret_cast<const uint32_t*>(&y);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, const Vec16& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ Vec16 ld_shared_v4(uint32_t addr) {
  Vec16 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t hadd2_u(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t half2_of(float x) {
  const __half2 h = __float2half2_rn(x);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// What the deferred-LayerNorm epilogues need beside the accumulator.
struct NormCtx {
  // kEpiNormIn(Gelu): C = rstd * acc + bias[n] + nm * csum[n], nm = -rstd * mu
  // The whole epilogue runs in the TMEM phase, one row per thread, with bias and csum of the chunk's 64
  // columns side by side in the warp's 256 staging bytes.
  float rstd = 1.f;               // of this thread's row
  uint32_t nm2_own = 0u;          // -rstd * mu of this thread's row, as an fp16 pair
  const __half* bias_g = nullptr; // bias / csum at the warp's first column
  const __half* csum_g = nullptr;
  Vec16 stage0 = {0u, 0u, 0u, 0u};  // lanes 0-7: bias, lanes 8-15: csum of chunk 0 (requested before the accumulator wait)
  // kEpiNormResidual, rows 4 i + (lane >> 3) of the coalesced phase
  float mu_i[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float rstd_i[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
  // gamma / beta of this lane's eight columns per 64-column chunk, as fp16 pairs (ones / zeros without)
  Vec16 g2[2] = {{0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u}, {0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u}};
  Vec16 be2[2] = {{0u, 0u, 0u, 0u}, {0u, 0u, 0u, 0u}};
  float* stats = nullptr;         // stats_out at (first row of the warp, first 64-column piece of the warp)
  int s2 = 0;                     // floats per row of stats_out
};

// v[i] summed over the 8 lanes of a group (lanes 8g .. 8g+7): afterwards v[0] of the lane with
// piece p (= lane & 7) holds the total of index p.  7 shuffles instead of 24.
__device__ __forceinline__ void group_transpose_sum(float (&v)[8], int piece) {
#pragma unroll
  for (int h = 4; h >= 1; h >>= 1) {
    const bool upper = (piece & h) != 0;
#pragma unroll
    for (int j = 0; j < h; ++j) {
      const float send = upper ? v[j] : v[j + h];
      const float keep = upper ? v[j + h] : v[j];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, send, h);
    }
  }
}

// Epilogue of one warp for one finished accumulator: its 32 rows (TMEM lanes
// starting at the lane field of t_row) x kCols columns.  Per 64-column chunk:
// TMEM -> registers (one row per thread) -> bias/GELU in fp32 -> fp16 -> the
// warp's swizzled staging buffer -> coalesced global stores (one instruction
// writes 4 full 128-byte row segments).  `release` runs once all TMEM reads of
// the warp have completed.  rows_valid = M - (first row of this warp).
template <int EPI, typename Release>
__device__ __forceinline__ void epilogue_warp_tile(uint32_t t_row, __half* ctile, int N, int rows_valid,
                                                   uint32_t bias_s, uint32_t buf, int lane, int chunks,
                                                   const __half* rtile, Release release, const NormCtx& nc = NormCtx()) {
  Vec16 staged = nc.stage0;
#pragma unroll 1
  for (int c = 0; c < chunks; ++c) {
    uint32_t r[64];
    tmem_ld_32x32b_x32(t_row + c * 64, r);
    tmem_ld_32x32b_x32(t_row + c * 64 + 32, r + 32);
    if (EPI == kEpiNormIn || EPI == kEpiNormInGelu) {
      if (lane < 16) st_shared_v4(bias_s + lane * 16, staged);
      if (c + 1 < chunks && lane < 16)  // the next chunk's, under this chunk's work
        staged = ld_global_nc_v4((lane < 8 ? nc.bias_g : nc.csum_g) + (c + 1) * 64 + (lane & 7) * 8);
      __syncwarp();
    }
    tmem_ld_wait();
    if (c == chunks - 1) {
      // the accumulator now lives in registers: hand the TMEM buffer back
      tc_fence_before();
      release();
    }
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[p * 8 + e]);
      if (EPI == kEpiNormIn || EPI == kEpiNormInGelu) {
        // rstd * acc + bias[n] + nm * csum[n] (then the GELU): the scaling in fp32, the two sums on
        // fp16 pairs; bias and csum of the chunk's columns lie side by side in the warp's staging bytes
        const Vec16 b2 = ld_shared_v4(bias_s + p * 16);
        const Vec16 c2 = ld_shared_v4(bias_s + 128 + p * 16);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] *= nc.rstd;
        const Vec16 a2 = VecTraits<__half>::pack(f);
        Vec16 o;
        o.x = hfma2_u(nc.nm2_own, c2.x, hadd2_u(a2.x, b2.x));
        o.y = hfma2_u(nc.nm2_own, c2.y, hadd2_u(a2.y, b2.y));
        o.z = hfma2_u(nc.nm2_own, c2.z, hadd2_u(a2.z, b2.z));
        o.w = hfma2_u(nc.nm2_own, c2.w, hadd2_u(a2.w, b2.w));
        if (EPI == kEpiNormInGelu) {
          o.x = gelu_tanh_half2(o.x);
          o.y = gelu_tanh_half2(o.y);
          o.z = gelu_tanh_half2(o.z);
          o.w = gelu_tanh_half2(o.w);
        }
        st_shared_v4(buf + lane * 128 + ((p ^ (lane & 7)) << 4), o);
        continue;
      } else if (EPI != kEpiNone) {
        float fb[8];
        VecTraits<__half>::unpack(ld_shared_v4(bias_s + (c * 64 + p * 8) * 2), fb);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += fb[e];
      }
      if (EPI == kEpiBiasTanh) {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = tanhf(f[e]);
      }
      Vec16 o = VecTraits<__half>::pack(f);
      if (EPI == kEpiBiasGelu) {
        o.x = gelu_tanh_half2(o.x);
        o.y = gelu_tanh_half2(o.y);
        o.z = gelu_tanh_half2(o.z);
        o.w = gelu_tanh_half2(o.w);
      }
      st_shared_v4(buf + lane * 128 + ((p ^ (lane & 7)) << 4), o);
    }
    __syncwarp();
    if (EPI == kEpiNormResidual) {
      // The residual is LN(rtile), taken here where a warp instruction covers four whole 128-byte row
      // segments; the statistics of the rows as they are stored go out beside them.
      const int piece = lane & 7, g = lane >> 3;
      Vec16 res[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = 4 * i + g;
        if (rr < rows_valid) res[i] = ld_global_nc_v4(rtile + static_cast<size_t>(rr) * N + c * 64 + piece * 8);
      }
      // gamma, beta of this lane's eight columns as fp16 pairs (fetched before the accumulator
      // arrived)
      const Vec16 g2 = c == 0 ? nc.g2[0] : nc.g2[1], be2 = c == 0 ? nc.be2[0] : nc.be2[1];
      float s1[8], s2[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = 4 * i + g;
        const Vec16 v = ld_shared_v4(buf + rr * 128 + ((piece ^ (rr & 7)) << 4));
        s1[i] = 0.f, s2[i] = 0.f;
        if (rr < rows_valid) {
          // (res - mu) * rstd in fp32: a row whose mean dwarfs its spread has res * rstd and mu * rstd in
          // the thousands and their difference of order one; then * gamma + beta and the sum on fp16 pairs
          float fr[8];
          VecTraits<__half>::unpack(res[i], fr);
          const float rs = nc.rstd_i[i], nmr = -nc.mu_i[i] * nc.rstd_i[i];
#pragma unroll
          for (int e = 0; e < 8; ++e) fr[e] = fmaf(fr[e], rs, nmr);
          const Vec16 d2 = VecTraits<__half>::pack(fr);
          Vec16 o;
          o.x = hadd2_u(v.x, hfma2_u(d2.x, g2.x, be2.x));
          o.y = hadd2_u(v.y, hfma2_u(d2.y, g2.y, be2.y));
          o.z = hadd2_u(v.z, hfma2_u(d2.z, g2.z, be2.z));
          o.w = hadd2_u(v.w, hfma2_u(d2.w, g2.w, be2.w));
          st_global_v4(ctile + static_cast<size_t>(rr) * N + c * 64 + piece * 8, o);
          float fx[8];
          VecTraits<__half>::unpack(o, fx);  // the statistics are those of the stored values
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            s1[i] += fx[e];
            s2[i] = fmaf(fx[e], fx[e], s2[i]);
          }
        }
      }
      group_transpose_sum(s1, piece);
      group_transpose_sum(s2, piece);
      const int rr = 4 * piece + g;  // the row whose totals this lane now holds
      if (rr < rows_valid)
        *reinterpret_cast<float2*>(nc.stats + static_cast<size_t>(rr) * nc.s2 + 2 * c) = make_float2(s1[0], s2[0]);
    } else if (EPI == kEpiBiasResidual) {
      // the residual is added here, where a warp instruction covers four whole 128-byte row
      // segments (one row per thread, as in the TMEM phase, would scatter 32 lines per load)
      Vec16 res[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = 4 * i + (lane >> 3), piece = lane & 7;
        if (rr < rows_valid) res[i] = ld_global_nc_v4(rtile + static_cast<size_t>(rr) * N + c * 64 + piece * 8);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = 4 * i + (lane >> 3), piece = lane & 7;
        const Vec16 v = ld_shared_v4(buf + rr * 128 + ((piece ^ (rr & 7)) << 4));
        if (rr < rows_valid) {
          float fv[8], fr[8];
          VecTraits<__half>::unpack(v, fv);
          VecTraits<__half>::unpack(res[i], fr);
#pragma unroll
          for (int e = 0; e < 8; ++e) fv[e] += fr[e];
          st_global_v4(ctile + static_cast<size_t>(rr) * N + c * 64 + piece * 8, VecTraits<__half>::pack(fv));
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int rr = 4 * i + (lane >> 3), piece = lane & 7;
        const Vec16 v = ld_shared_v4(buf + rr * 128 + ((piece ^ (rr & 7)) << 4));
        if (rr < rows_valid) st_global_v4(ctile + static_cast<size_t>(rr) * N + c * 64 + piece * 8, v);
      }
    }
    __syncwarp();  // the staging buffer is rewritten by the next chunk / tile
  }
}

enum Site : int {
  kSiteProducerEmpty = 1,
  kSiteProducerDrain = 2,
  kSiteMmaTmemEmpty = 3,
  kSiteMmaFull = 4,
  kSiteMmaDrain = 5,
  kSiteEpilogueFull = 6,
  kSiteSmemAlign = 7,
  kSiteLnMailbox = 8,
};

template <int BN, int EPI>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b, __half* __restrict__ C,
                    const __half* __restrict__ bias, const __half* __restrict__ residual,
                    const int* __restrict__ m_ptr, int max_m, int N, int K, int* status_word, int reverse_m) {
  using cfg = Cfg<BN>;
  constexpr int S = cfg::kStages;

  // The prologue (barriers, TMEM) touches no global memory: it runs before the
  // wait on the preceding kernel, under that kernel's tail.
  pdl_trigger();

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t tiles_addr = smem_u32(smem_raw);
  if ((tiles_addr & 1023u) != 0u) {  // the swizzled tiles need 1024-byte alignment
    pdl_wait();  // no CTA leaves before the preceding kernel has completed
    if (threadIdx.x == 0) report_timeout(status_word, kKernelGemmTc, kSiteSmemAlign);
    return;
  }
  uint8_t* tiles = smem_raw;
  const uint32_t staging_addr = tiles_addr + S * cfg::kStageBytes;
  const uint32_t bias_addr = staging_addr + cfg::kStagingBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + S * cfg::kStageBytes + cfg::kStagingBytes + cfg::kBiasBytes);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
  auto tmem_full_bar = [&](int a) { return bar0 + 8u * (2 * S + a); };
  auto tmem_empty_bar = [&](int a) { return bar0 + 8u * (2 * S + 2 + a); };
  const uint32_t drain_bar = bar0 + 8u * (2 * S + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + cfg::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
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
  const int num_kb = (K + BK - 1) / BK;

  auto fail = [&](int site) {
    *abort_flag = 1;
    report_timeout(status_word, kKernelGemmTc, site);
  };

  if (warp == 0) {
    // ------------------------- TMA producer -------------------------
    if (lane == 0) {
      prefetch_tensormap(&tmap_a);
      prefetch_tensormap(&tmap_b);
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
          const uint32_t b_dst = a_dst + cfg::kABytes;
          mbar_arrive_expect_tx(full_bar(stage), cfg::kStageBytes);
          tma_load_2d(a_dst, &tmap_a, kb * BK, m_tile * BM, full_bar(stage));
          tma_load_2d(b_dst, &tmap_b, kb * BK, n_tile * BN, full_bar(stage));
          ++issued;
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // Copies still in flight must land before the CTA's shared memory goes away.
      const long long pending = issued < S ? issued : S;
      for (long long i = 0; i < pending; ++i) {
        const long long f = issued - 1 - i;
        if (!mbar_wait(full_bar(static_cast<int>(f % S)), static_cast<uint32_t>((f / S) & 1),
                       abort_flag) && *abort_flag == 0)
          fail(kSiteProducerDrain);
      }
    }
  } else if (warp == 1) {
    // ------------------------- MMA issuer -------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16_f32acc(BM, BN);
      uint32_t stage = 0, phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag)) {
          fail(kSiteMmaTmemEmpty);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            fail(kSiteMmaFull);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = tiles_addr + stage * cfg::kStageBytes;
          const uint64_t adesc = make_kmajor_sw128_desc(a_addr);
          const uint64_t bdesc = make_kmajor_sw128_desc(a_addr + cfg::kABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing K by 16 fp16 = 32 bytes inside the swizzle row: +2 in the address field
            umma_f16_ss(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(tmem_full_bar(acc));
      }
      // All MMAs must have retired before TMEM is freed.
      umma_commit(drain_bar);
      if (!mbar_wait(drain_bar, 0u, abort_flag) && *abort_flag == 0) fail(kSiteMmaDrain);
    }
  } else {
    // ------------------------- epilogue -------------------------
    // Eight warps: warp w works on TMEM lanes [32*(w%4), +32) (the rows it may
    // access) and on one half of the tile's columns, two warps per scheduler
    // so that TMEM, shared-memory and MUFU latencies overlap.
    const int quad = warp & 3;
    const int ew = warp - 2;            // 0..7
    const int half = ew >> 2;           // which half of the columns
    constexpr int kCols = cfg::kColsPerWarp;
    const uint32_t buf = staging_addr + ew * kStagingPerWarp;
    const uint32_t bias_s = bias_addr + ew * (kCols * 2);
    int it = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int m_lin = tile / n_tiles, n_tile = tile - m_lin * n_tiles;
        const int m_tile = reverse_m ? m_tiles - 1 - m_lin : m_lin;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int col0 = n_tile * BN + half * kCols;
      if (EPI != kEpiNone) {
        // this warp's bias slice -> shared memory (read back as broadcasts)
        if (lane < kCols / 8) st_shared_v4(bias_s + lane * 16, ld_global_v4(bias + col0 + lane * 8));
        __syncwarp();
      }
      // every lane polls; the vote makes the outcome uniform and reconverges the
      // warp for the .sync.aligned TMEM loads below
      const bool got = mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) fail(kSiteEpilogueFull);
        break;
      }
      tc_fence_after();
      const int row0 = m_tile * BM + quad * 32;
      const uint32_t t_row =
          tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN + half * kCols;
      __half* ctile = C + static_cast<size_t>(row0) * N + col0;
      const __half* rtile = EPI == kEpiBiasResidual ? residual + static_cast<size_t>(row0) * N + col0 : nullptr;
      epilogue_warp_tile<EPI>(t_row, ctile, N, M - row0, bias_s, buf, lane, kCols / 64, rtile,
                              [&] { mbar_arrive(tmem_empty_bar(acc)); });
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
// CTA-pair variant: a cluster of two CTAs (one per SM of a TPC) computes a
// 256 x 256 tile with tcgen05.mma cta_group::2.  Each CTA loads 128 rows of A
// and 128 of the tile's 256 W rows per k-block (32 KB instead of 48 KB per
// 128 x 256 of output, i.e. one third less L2 -> shared-memory traffic per
// FLOP) and keeps the 128 x 256 accumulator of its own rows in its own TMEM.
// CTA 0 of the pair issues the MMAs for both; barriers that cross the pair:
//   full[s]      lives in CTA 0, counts the TMA bytes of both CTAs
//   empty[s]     one per CTA, CTA 0's MMA thread commits to both
//   tmem_full[a] one per CTA, CTA 0's MMA thread commits to both
//   tmem_empty[a] lives in CTA 0, one arrival per epilogue warp of both CTAs
// No load is multicast: each CTA fetches its own operand rows.
//
// Work units and the last wave.  Tiles are dealt round-robin to the pairs, so
// when num_tiles is not a multiple of the number of pairs the last round
// keeps only `rem` pairs busy for a whole tile time.  If rem is at most half
// of the pairs, each of those tiles is cut into two 256 x 128 units (MMA with
// N = 128, each CTA loading 64 W rows): the last round then takes half a tile
// time.  BERT-base at T = 39 778: 468 tiles of the N = 768 projections on 74
// pairs = 6.32 rounds -> 6.5 instead of 7.
// ---------------------------------------------------------------------------
struct PairCfg {
  static constexpr int BN = 256;
  static constexpr int kStages = 6;
  static constexpr int kABytes = BM * BK * 2;          // this CTA's 128 A rows
  static constexpr int kBBytes = (BN / 2) * BK * 2;    // this CTA's 128 W rows
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kNumBars = 2 * kStages + 5;
  static constexpr int kStagingBytes = kEpilogueWarps * kStagingPerWarp;
  static constexpr int kColsPerWarp = BN / 2;
  static constexpr int kBiasBytes = kEpilogueWarps * kColsPerWarp * 2;
  // barriers (2 * kStages + 5), the TMEM slot, the abort flag and the words of the LayerNorm work sharing
  static constexpr int kControlBytes = 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBiasBytes + kControlBytes;
  static_assert(kNumBars * 8 + 8 + (3 * kEpilogueWarps + kLnQueue + 2) * 4 <= kControlBytes, "control block too small");
  static_assert(kSmemBytes <= 232448, "more than 227 KB of shared memory");
  static constexpr int kTmemCols = 2 * BN;
};

// VPL: 16-byte vectors of a C row per lane in the LayerNorm warps (N / 256); 0 for the other epilogues.
template <int EPI, int VPL>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(threads_of(EPI), 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_b_half, __half* __restrict__ C,
                         const __half* __restrict__ bias, const __half* __restrict__ residual,
                         const int* __restrict__ m_ptr, int max_m, int N, int K, int* status_word,
                         int reverse_m, const GemmLayerNorm ln) {
  using cfg = PairCfg;
  constexpr int S = cfg::kStages;
  constexpr int BN = cfg::BN;
  constexpr int BM2 = 2 * BM;

  // The prologue (barriers, TMEM, cluster sync) touches no global memory: it runs
  // before the wait on the preceding kernel, under that kernel's tail.
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
  uint8_t* tiles = smem_raw;
  const uint32_t staging_addr = tiles_addr + S * cfg::kStageBytes;
  const uint32_t bias_addr = staging_addr + cfg::kStagingBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + S * cfg::kStageBytes + cfg::kStagingBytes + cfg::kBiasBytes);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (S + s); };
  auto tmem_full_bar = [&](int a) { return bar0 + 8u * (2 * S + a); };
  auto tmem_empty_bar = [&](int a) { return bar0 + 8u * (2 * S + 2 + a); };
  const uint32_t drain_bar = bar0 + 8u * (2 * S + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + cfg::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // LayerNorm variants.  Per epilogue warp e: ep_units[e] = units whose stores it has issued,
  // ep_final[e] = it has left its loop, ln_seen[e] = published blocks it has done its rows of.
  // The queue: q_row[i % kLnQueue] = first row of the i-th published block, *q_tail = how many are
  // published, *q_closed = the counting warp will publish no more.
  volatile int* ep_units = reinterpret_cast<volatile int*>(tmem_slot + 2);
  volatile int* ep_final = ep_units + kEpilogueWarps;
  volatile int* ln_seen = ep_final + kEpilogueWarps;
  volatile int* q_row = ln_seen + kEpilogueWarps;
  volatile int* q_tail = q_row + kLnQueue;
  volatile int* q_closed = q_tail + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 2 * kEpilogueWarps);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    for (int e = 0; e < 3 * kEpilogueWarps + kLnQueue + 2; ++e) ep_units[e] = 0;
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
  const int n_tiles = N / BN;
  const int num_tiles = m_tiles * n_tiles;  // 0: every role's loop is empty
  const int num_kb = (K + BK - 1) / BK;
  // last round cut into half-width units when it occupies at most half of the pairs
  int num_units;
  const int full_tiles = pair_units(num_tiles, num_pairs, &num_units);
  const bool split = num_units != full_tiles;

  auto fail = [&](int site) {
    *abort_flag = 1;
    report_timeout(status_word, kKernelGemmTc, site);
  };

  if (warp == 0) {
    // ------------------------- TMA producer (both CTAs) -------------------------
    if (lane == 0) {
      prefetch_tensormap(&tmap_a);
      prefetch_tensormap(&tmap_b);
      if (split) prefetch_tensormap(&tmap_b_half);
      uint32_t stage = 0, phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int u = pair_id; u < num_units && ok; u += num_pairs) {
        const PairUnit pu = pair_unit(u, full_tiles, n_tiles, m_tiles, reverse_m);
        const int a_row = pu.m_tile * BM2 + static_cast<int>(rank) * BM;
        const int b_row = pu.col0 + static_cast<int>(rank) * (pu.ncols / 2);
        const bool whole = pu.ncols == BN;
        const uint32_t stage_tx = 2u * (cfg::kABytes + (whole ? cfg::kBBytes : cfg::kBBytes / 2));
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            fail(kSiteProducerEmpty);
            ok = false;
            break;
          }
          const uint32_t a_dst = tiles_addr + stage * cfg::kStageBytes;
          const uint32_t b_dst = a_dst + cfg::kABytes;
          const uint32_t full0 = mapa_shared(full_bar(stage), 0);
          if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), stage_tx);
          tma_load_2d_pair(a_dst, &tmap_a, kb * BK, a_row, full0);
          tma_load_2d_pair(b_dst, whole ? &tmap_b : &tmap_b_half, kb * BK, b_row, full0);
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
          if (!mbar_wait(full_bar(static_cast<int>(f % S)), static_cast<uint32_t>((f / S) & 1),
                         abort_flag) && *abort_flag == 0)
            fail(kSiteProducerDrain);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------- MMA issuer (CTA 0 only) -------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_whole = make_idesc_f16_f32acc(BM2, BN);
      constexpr uint32_t idesc_half = make_idesc_f16_f32acc(BM2, BN / 2);
      uint32_t stage = 0, phase = 0;
      int it = 0;
      bool ok = true;
      for (int u = pair_id; u < num_units && ok; u += num_pairs, ++it) {
        const uint32_t idesc = u < full_tiles ? idesc_whole : idesc_half;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag)) {
          fail(kSiteMmaTmemEmpty);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            fail(kSiteMmaFull);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = tiles_addr + stage * cfg::kStageBytes;
          const uint64_t adesc = make_kmajor_sw128_desc(a_addr);
          const uint64_t bdesc = make_kmajor_sw128_desc(a_addr + cfg::kABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16_ss_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(empty_bar(stage));
          umma_commit_pair(mapa_shared(empty_bar(stage), 1));
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          umma_commit_pair(tmem_full_bar(acc));
          umma_commit_pair(mapa_shared(tmem_full_bar(acc), 1));
        }
      }
      umma_commit_pair(drain_bar);
      if (!mbar_wait(drain_bar, 0u, abort_flag) && *abort_flag == 0) fail(kSiteMmaDrain);
    }
  } else if (warp < 2 + kEpilogueWarps) {
    // ------------------------- epilogue (both CTAs) -------------------------
    constexpr int kBase = base_epi(EPI);
    constexpr bool kLn = has_ln(EPI);
    const int quad = warp & 3;
    const int ew = warp - 2;
    const int half = ew >> 2;
    constexpr int kCols = cfg::kColsPerWarp;
    const uint32_t buf = staging_addr + ew * kStagingPerWarp;
    const uint32_t bias_s = bias_addr + ew * (kCols * 2);

    // ---- LayerNorm variants: this warp's four rows of every published block ----
    int seen = 0;  // published blocks this warp has done
    auto ln_poll = [&]() -> bool {
      bool any = false;
      if constexpr (kLn) {
        const int tail = *q_tail;  // one shared-memory read for the whole warp
        // The counting warp saw the complete block (device scope) before it published it to this
        // CTA (CTA-scope release); this warp's reads, which go to L2, are ordered behind that.
        if (seen != tail) __threadfence_block();
        for (; seen != tail; ++seen) {
          any = true;
          const int first = q_row[seen % kLnQueue] + ew * kLnRowsPerWarp;
          const int nrows = min(kLnRowsPerWarp, M - first);
          if (nrows > 0) {
            __half* crow = C + static_cast<size_t>(first) * N;
            const __half* rrow = residual + static_cast<size_t>(first) * N;
            constexpr int RB = VPL <= 3 ? kLnRowsPerWarp : kLnRowsPerWarp / 2;
#pragma unroll 1
            for (int r0 = 0; r0 < nrows; r0 += RB)
              ln_rows<(VPL > 0 ? VPL : 1), EPI == kEpiLayerNorm, RB>(
                  crow + static_cast<size_t>(r0) * N, rrow + static_cast<size_t>(r0) * N, bias, ln.gamma, ln.beta, N,
                  min(RB, nrows - r0), ln.eps, lane);
          }
        }
        if (any) {
          __syncwarp();
          if (lane == 0) ln_seen[ew] = seen;  // the queue slot may be reused once every warp is past it
        }
      }
      return any;
    };

    // Deferred-LayerNorm variants: the partial sums of one row, (sum, sum of squares) per 64-column
    // piece, as they come from memory; which row depends on the phase that uses them (see below).
    constexpr bool kDeferred = kBase == kEpiNormIn || kBase == kEpiNormInGelu || kBase == kEpiNormResidual;
    constexpr int kStatVecs = VPL > 0 ? VPL : 1;  // float4s of a row's partial sums: width / 128 (the launcher's VPL)
    float4 raw[kDeferred ? kStatVecs : 1];
    auto stat_row = [&](const PairUnit& pu) {
      const int r0 = pu.m_tile * BM2 + static_cast<int>(rank) * BM + quad * 32;
      return kBase == kEpiNormResidual ? r0 + 4 * (lane & 7) + (lane >> 3) : r0 + lane;
    };
    auto request_stats = [&](int u) {
      if constexpr (kDeferred) {
        if (ln.stats_in == nullptr || u >= num_units) return;
        const int row = stat_row(pair_unit(u, full_tiles, n_tiles, m_tiles, reverse_m));
        if (row >= M) return;
        const float4* p = reinterpret_cast<const float4*>(ln.stats_in + static_cast<size_t>(row) * (2 * ln.stat_slots));
#pragma unroll
        for (int j = 0; j < kStatVecs; ++j)
          if (2 * j < ln.stat_slots) raw[j] = p[j];
      }
    };
    request_stats(pair_id);

    int it = 0;
    for (int u = pair_id; u < num_units; u += num_pairs, ++it) {
      const PairUnit pu = pair_unit(u, full_tiles, n_tiles, m_tiles, reverse_m);
      const int m_tile = pu.m_tile;
      const int wcols = pu.ncols / 2;  // columns of this warp: 128, or 64 in a half-width unit
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const int col0 = pu.col0 + half * wcols;
      if (kBase != kEpiNone && kBase != kEpiNormIn && kBase != kEpiNormInGelu) {
        if (lane < wcols / 8) st_shared_v4(bias_s + lane * 16, ld_global_v4(bias + col0 + lane * 8));
        __syncwarp();
      }
      // The row statistics of this unit were requested a unit ago (the loads are a global-memory
      // latency that would otherwise sit in front of every epilogue: the K = H projections leave the
      // epilogue warps no slack); reduce them now and request the next unit's.
      const int row0 = m_tile * BM2 + static_cast<int>(rank) * BM + quad * 32;
      NormCtx nc;
      if constexpr (kDeferred) {
        float mu = 0.f, rstd = 1.f;
        if (ln.stats_in != nullptr && stat_row(pu) < M) {
          float s1 = 0.f, s2 = 0.f;
#pragma unroll
          for (int j = 0; j < kStatVecs; ++j)
            if (2 * j < ln.stat_slots) {
              s1 += raw[j].x + raw[j].z;
              s2 += raw[j].y + raw[j].w;
            }
          const float inv = 1.0f / static_cast<float>(kBase == kEpiNormResidual ? N : K);
          mu = s1 * inv;
          rstd = rsqrtf(fmaxf(s2 * inv - mu * mu, 0.f) + ln.eps);
        }
        request_stats(u + num_pairs);
        if constexpr (kBase == kEpiNormResidual) {
          // lane (g, piece) worked out the statistics of residual row 4 * piece + g; the coalesced
          // phase needs those of rows 4 i + g, which the lanes of its own group hold
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            nc.mu_i[i] = __shfl_sync(0xffffffffu, mu, (lane & ~7) + i);
            nc.rstd_i[i] = __shfl_sync(0xffffffffu, rstd, (lane & ~7) + i);
          }
          if (ln.gamma != nullptr) {
            nc.g2[0] = ld_global_nc_v4(ln.gamma + col0 + (lane & 7) * 8);
            nc.be2[0] = ld_global_nc_v4(ln.beta + col0 + (lane & 7) * 8);
            if (wcols > 64) {
              nc.g2[1] = ld_global_nc_v4(ln.gamma + col0 + 64 + (lane & 7) * 8);
              nc.be2[1] = ld_global_nc_v4(ln.beta + col0 + 64 + (lane & 7) * 8);
            }
          }
          nc.s2 = 2 * (N / 64);
          nc.stats = ln.stats_out + static_cast<size_t>(row0) * nc.s2 + 2 * (col0 / 64);
        } else {
          // this thread's row of A is normalised on the way out
          nc.rstd = rstd;
          const float nm = -rstd * mu;
          nc.nm2_own = half2_of(nm);
          nc.bias_g = bias + col0;
          nc.csum_g = ln.csum + col0;
          if (lane < 16) nc.stage0 = ld_global_nc_v4((lane < 8 ? nc.bias_g : nc.csum_g) + (lane & 7) * 8);
        }
      }
      bool got;
      if constexpr (kLn) {
        // wait for the accumulator, normalising published rows meanwhile
        got = true;
        unsigned long long t0 = 0;
        for (uint32_t spin = 1;; ++spin) {
          if (__all_sync(0xffffffffu, mbar_test_wait(tmem_full_bar(acc), acc_phase))) break;
          if (ln_poll()) {
            t0 = 0;
          } else if ((spin & 63u) == 0u) {
            bool stop = *abort_flag != 0;
            const unsigned long long now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitTimeoutNs) stop = true;
            if (__any_sync(0xffffffffu, stop)) {
              got = false;
              break;
            }
          }
        }
      } else {
        got = __all_sync(0xffffffffu, mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag));
      }
      if (!got) {
        if (lane == 0) fail(kSiteEpilogueFull);
        break;
      }
      tc_fence_after();
      const uint32_t t_row =
          tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN + half * wcols;
      __half* ctile = C + static_cast<size_t>(row0) * N + col0;
      const uint32_t empty0 = mapa_shared(tmem_empty_bar(acc), 0);
      const __half* rtile = (kBase == kEpiBiasResidual || kBase == kEpiNormResidual)
                                ? residual + static_cast<size_t>(row0) * N + col0
                                : nullptr;
      epilogue_warp_tile<kBase>(t_row, ctile, N, M - row0, bias_s, buf, lane, wcols / 64, rtile, [&] {
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(empty0);
      }, nc);
      if constexpr (kLn) {
        // this unit's stores are issued: tell the counting warp (CTA-scope release of all lanes' stores)
        __threadfence_block();
        __syncwarp();
        if (lane == 0) ep_units[ew] = it + 1;
      }
    }
    if constexpr (kLn) {
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        ep_final[ew] = 1;
      }
      // stay until the counting warp has published its last block and this warp has done its rows
      // of all of them (q_closed is read before the queue: a block is published before the flag)
      unsigned long long t0 = 0;
      for (;;) {
        const int closed = *q_closed;
        const bool any = ln_poll();
        if (closed != 0 && !any) break;
        if (any) {
          t0 = 0;
          continue;
        }
        __nanosleep(64);
        const unsigned long long now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        if (__any_sync(0xffffffffu, now - t0 > 2 * kWaitTimeoutNs || *abort_flag != 0)) break;
      }
    }
  } else if constexpr (has_ln(EPI)) {
    // ------------------------- counting warp (both CTAs, LayerNorm variants) -------------------------
    // Lane e < 8 follows epilogue warp e through the unit schedule, which it can compute itself.
    const int e = lane & (kEpilogueWarps - 1);
    const bool tracker = lane < kEpilogueWarps;
    const int quad = e & 3;  // epilogue warp e is warp e + 2: TMEM lane quadrant (e + 2) & 3
    const int equad = (e + 2) & 3;
    (void)quad;
    int counted = 0;         // units of warp e already added to the row counters
    int published = 0;       // blocks this CTA has published (same value in every lane)
    unsigned long long t0 = 0;
    bool give_up = false;
    for (;;) {
      // flags first, then "final": a warp raises its last flag before it sets final
      const int final_e = tracker ? ep_final[e] : 1;
      const int units_e = tracker ? ep_units[e] : 0;
      const bool pending = tracker && units_e > counted;
      const unsigned pend_mask = __ballot_sync(0xffffffffu, pending);
      if (pend_mask != 0u) {
        t0 = 0;
        // One device-scope fence for every flagged store: the flags were raised behind CTA-scope
        // fences of the storing warps, so this fence orders those stores before the counts below.
        __threadfence();
        int last_row = -1;
        if (pending) {
          const int u = pair_id + counted * num_pairs;
          const PairUnit pu = pair_unit(u, full_tiles, n_tiles, m_tiles, reverse_m);
          const int row0 = pu.m_tile * BM2 + static_cast<int>(rank) * BM + equad * 32;
          const int wcols = pu.ncols / 2;
          const int before = atomicAdd(ln.counters + (row0 >> 5), wcols);
          if (before + wcols == N) {  // this part completed the 32 rows: every column is in L2
            ln.counters[row0 >> 5] = 0;  // nobody else touches it any more: zero again for the next launch
            if (row0 < M) last_row = row0;
          }
          ++counted;
        }
        // publish the completed blocks, one queue slot each, in lane order
        const unsigned post_mask = __ballot_sync(0xffffffffu, last_row >= 0);
        if (post_mask != 0u) {
          const int nposts = __popc(post_mask);
          // room in the queue: every epilogue warp must be past the slots about to be overwritten
          for (;;) {
            int slowest = tracker ? ln_seen[e] : 0x7fffffff;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) slowest = min(slowest, __shfl_xor_sync(0xffffffffu, slowest, o));
            if (published + nposts - slowest <= kLnQueue) break;
            __nanosleep(64);
            const unsigned long long now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            if (__any_sync(0xffffffffu, now - t0 > kWaitTimeoutNs || *abort_flag != 0)) {
              give_up = true;
              break;
            }
          }
          if (give_up) {
            if (lane == 0) fail(kSiteLnMailbox);
            break;
          }
          t0 = 0;
          if (last_row >= 0) {
            const int slot = published + __popc(post_mask & ((1u << lane) - 1u));
            q_row[slot % kLnQueue] = last_row;
          }
          published += nposts;
          __threadfence_block();  // acquire of the counts above, release of the queue entries
          __syncwarp();
          if (lane == 0) *q_tail = published;
        }
        continue;
      }
      // nothing flagged: finished when every epilogue warp has left its loop (and all its flags are counted)
      if (__all_sync(0xffffffffu, final_e != 0)) break;
      __nanosleep(32);
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (__any_sync(0xffffffffu, now - t0 > 4 * kWaitTimeoutNs || *abort_flag != 0)) break;
    }
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      *q_closed = 1;
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

template <int EPI, int VPL>
cudaError_t launch_pair_epi(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tbh,
                            const __half* bias, const __half* residual, __half* c,
                            const int* m_ptr, int max_m, int n, int k, int* status_word, int reverse_m,
                            const GemmLayerNorm& ln, cudaStream_t stream) {
  using cfg = PairCfg;
  static PerDeviceOnce once;  // function attributes are per device
  const cudaError_t once_err = once.run([] {
    return cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<EPI, VPL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                cfg::kSmemBytes);
  });
  if (once_err != cudaSuccess) return once_err;
  const long long max_tiles = static_cast<long long>((max_m + 2 * BM - 1) / (2 * BM)) * (n / cfg::BN);
  long long pairs = sm_count() / 2;
  if (pairs > max_tiles) pairs = max_tiles;
  if (pairs < 1) pairs = 1;
  return launch_pdl(gemm_tcgen05_pair_kernel<EPI, VPL>, dim3(static_cast<int>(2 * pairs)), dim3(threads_of(EPI)),
                    cfg::kSmemBytes, stream, ta, tb, tbh, c, bias, residual, m_ptr, max_m, n, k, status_word, reverse_m,
                    ln);
}

// LayerNorm variants: one instantiation per row width (N / 256 vectors per lane).
template <int EPI>
cudaError_t launch_pair_ln(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tbh,
                           const __half* bias, const __half* residual, __half* c, const int* m_ptr, int max_m,
                           int n, int k, int* status_word, int reverse_m, const GemmLayerNorm& ln,
                           cudaStream_t stream) {
#define ETB_LN_CASE(V)                                                                                            \
  case V:                                                                                                         \
    return launch_pair_epi<EPI, V>(ta, tb, tbh, bias, residual, c, m_ptr, max_m, n, k, status_word, reverse_m, ln, \
                                   stream)
  switch (n >> 8) {
    ETB_LN_CASE(1);
    ETB_LN_CASE(2);
    ETB_LN_CASE(3);
    ETB_LN_CASE(4);
    default:
      return cudaErrorInvalidValue;
  }
#undef ETB_LN_CASE
}

// Deferred-LayerNorm variants: one instantiation per width of the normalised rows (width / 128 float4s
// of partial sums per row; widths up to 1024, the limit of the fp16 handle's LayerNorm anyway).
template <int EPI>
cudaError_t launch_pair_norm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tbh,
                             const __half* bias, const __half* residual, __half* c, const int* m_ptr, int max_m,
                             int n, int k, int* status_word, int reverse_m, const GemmLayerNorm& ln,
                             cudaStream_t stream) {
#define ETB_NORM_CASE(V)                                                                                          \
  case V:                                                                                                         \
    return launch_pair_epi<EPI, V>(ta, tb, tbh, bias, residual, c, m_ptr, max_m, n, k, status_word, reverse_m, ln, \
                                   stream)
  const int width = EPI == kEpiNormResidual ? n : k;
  switch (width / 128) {
    ETB_NORM_CASE(2);
    ETB_NORM_CASE(4);
    ETB_NORM_CASE(6);
    ETB_NORM_CASE(8);
    default:
      return cudaErrorInvalidValue;
  }
#undef ETB_NORM_CASE
}

cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tbh,
                        const __half* bias, const __half* residual, __half* c,
                        const int* m_ptr, int max_m, int n, int k, int epilogue, int* status_word,
                        int reverse_m, const GemmLayerNorm& ln, cudaStream_t stream) {
#define ETB_PAIR_CASE(E)                                                                                      \
  case E:                                                                                                     \
    return launch_pair_epi<E, 0>(ta, tb, tbh, bias, residual, c, m_ptr, max_m, n, k, status_word, reverse_m, ln, \
                                 stream)
  switch (epilogue) {
    ETB_PAIR_CASE(kEpiNone);
    ETB_PAIR_CASE(kEpiBias);
    ETB_PAIR_CASE(kEpiBiasGelu);
    ETB_PAIR_CASE(kEpiBiasTanh);
    ETB_PAIR_CASE(kEpiBiasResidual);
    case kEpiNormIn:
      return launch_pair_norm<kEpiNormIn>(ta, tb, tbh, bias, residual, c, m_ptr, max_m, n, k, status_word, reverse_m,
                                          ln, stream);
    case kEpiNormInGelu:
      return launch_pair_norm<kEpiNormInGelu>(ta, tb, tbh, bias, residual, c, m_ptr, max_m, n, k, status_word,
                                              reverse_m, ln, stream);
    case kEpiNormResidual:
      return launch_pair_norm<kEpiNormResidual>(ta, tb, tbh, bias, residual, c, m_ptr, max_m, n, k, status_word,
                                                reverse_m, ln, stream);
    case kEpiResidualLayerNorm:
      return launch_pair_ln<kEpiResidualLayerNorm>(ta, tb, tbh, bias, residual, c, m_ptr, max_m, n, k, status_word,
                                                   reverse_m, ln, stream);
    case kEpiLayerNorm:
      return launch_pair_ln<kEpiLayerNorm>(ta, tb, tbh, bias, residual, c, m_ptr, max_m, n, k, status_word,
                                           reverse_m, ln, stream);
    default:
      return cudaErrorInvalidValue;
  }
#undef ETB_PAIR_CASE
}

template <int BN, int EPI>
cudaError_t launch_bn_epi(const CUtensorMap& ta, const CUtensorMap& tb, const __half* bias, const __half* residual, __half* c,
                          const int* m_ptr, int max_m, int n, int k, int* status_word, int reverse_m,
                          cudaStream_t stream) {
  using cfg = Cfg<BN>;
  static PerDeviceOnce once;  // function attributes are per device
  const cudaError_t once_err = once.run([] {
    cudaError_t attr_err = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, cfg::kSmemBytes);
    return attr_err;
  });
  if (once_err != cudaSuccess) return once_err;
  const long long max_tiles = static_cast<long long>((max_m + BM - 1) / BM) * (n / BN);
  long long grid = sm_count();
  if (grid > max_tiles) grid = max_tiles;
  if (grid < 1) grid = 1;
  return launch_pdl(gemm_tcgen05_kernel<BN, EPI>, dim3(static_cast<int>(grid)), dim3(kNumThreads),
                    cfg::kSmemBytes, stream, ta, tb, c, bias, residual, m_ptr, max_m, n, k, status_word, reverse_m);
}

template <int BN>
cudaError_t launch_bn(const CUtensorMap& ta, const CUtensorMap& tb, const __half* bias, const __half* residual, __half* c,
                      const int* m_ptr, int max_m, int n, int k, int epilogue, int* status_word,
                      int reverse_m, cudaStream_t stream) {
  switch (epilogue) {
    case kEpiNone:
      return launch_bn_epi<BN, kEpiNone>(ta, tb, bias, residual, c, m_ptr, max_m, n, k, status_word, reverse_m, stream);
    case kEpiBias:
      return launch_bn_epi<BN, kEpiBias>(ta, tb, bias, residual, c, m_ptr, max_m, n, k, status_word, reverse_m, stream);
    case kEpiBiasGelu:
      return launch_bn_epi<BN, kEpiBiasGelu>(ta, tb, bias, residual, c, m_ptr, max_m, n, k, status_word, reverse_m, stream);
    case kEpiBiasTanh:
      return launch_bn_epi<BN, kEpiBiasTanh>(ta, tb, bias, residual, c, m_ptr, max_m, n, k, status_word, reverse_m, stream);
    case kEpiBiasResidual:
      return launch_bn_epi<BN, kEpiBiasResidual>(ta, tb, bias, residual, c, m_ptr, max_m, n, k, status_word,
                                                 reverse_m, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

const CUtensorMap* TensorMapCache::find(int dtype_tag, const void* base, uint64_t rows, uint64_t cols,
                                        uint64_t row_stride, uint32_t box_rows, uint32_t box_cols) {
  const auto it = entries_.find(Key{dtype_tag, base, rows, cols, row_stride, box_rows, box_cols});
  return it == entries_.end() ? nullptr : &it->second;
}

void TensorMapCache::insert(int dtype_tag, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride,
                            uint32_t box_rows, uint32_t box_cols, const CUtensorMap& map) {
  if (entries_.size() >= kMaxEntries) entries_.clear();
  entries_[Key{dtype_tag, base, rows, cols, row_stride, box_rows, box_cols}] = map;
}

bool encode_2d_fp16_sw128(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                          uint64_t row_stride_elems, uint32_t box_rows, uint32_t box_cols,
                          TensorMapCache* cache) {
  if (cache != nullptr) {
    if (const CUtensorMap* hit = cache->find(2, base, rows, cols, row_stride_elems, box_rows, box_cols)) {
      *map = *hit;
      return true;
    }
  }
  EncodeTiledFn fn = get_encode_tiled();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_stride_elems * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims,
                        strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (cache != nullptr) cache->insert(2, base, rows, cols, row_stride_elems, box_rows, box_cols, *map);
  return true;
}

cudaError_t launch_gemm_tcgen05(const __half* a, const __half* w_packed, const __half* bias,
                                __half* c, const int* m_ptr, int max_m, int n, int k, int epilogue,
                                int* status_word, cudaStream_t stream, bool reverse_m, const __half* residual,
                                TensorMapCache* maps, const GemmLayerNorm* ln) {
  if (max_m <= 0) return cudaSuccess;
  if (n <= 0 || k <= 0 || (n % 128) != 0 || (k % 8) != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a) & 15u) || (reinterpret_cast<uintptr_t>(w_packed) & 15u) ||
      (reinterpret_cast<uintptr_t>(c) & 15u) || (bias && (reinterpret_cast<uintptr_t>(bias) & 15u)))
    return cudaErrorMisalignedAddress;
  if (epilogue != kEpiNone && bias == nullptr) return cudaErrorInvalidValue;
  const bool needs_residual = epilogue == kEpiBiasResidual || epilogue == kEpiResidualLayerNorm ||
                              epilogue == kEpiLayerNorm || epilogue == kEpiNormResidual;
  if (needs_residual && (residual == nullptr || (reinterpret_cast<uintptr_t>(residual) & 15u)))
    return cudaErrorInvalidValue;
  GemmLayerNorm lnp;
  if (has_ln(epilogue)) {
    if (ln == nullptr || ln->gamma == nullptr || ln->beta == nullptr || ln->counters == nullptr ||
        !gemm_layernorm_supported(n))
      return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(ln->gamma) & 15u) || (reinterpret_cast<uintptr_t>(ln->beta) & 15u))
      return cudaErrorMisalignedAddress;
    lnp = *ln;
  }
  if (is_deferred_norm(epilogue)) {
    // the pair kernel only; statistics in 64-column pieces of rows whose width is a multiple of 128
    if (ln == nullptr || (n % 256) != 0) return cudaErrorInvalidValue;
    const int width = epilogue == kEpiNormResidual ? n : k;  // of the tensor the statistics describe
    if ((width % 256) != 0 || width > 1024) return cudaErrorInvalidValue;
    if (ln->stats_in != nullptr &&
        (ln->stat_slots != width / 64 || (reinterpret_cast<uintptr_t>(ln->stats_in) & 15u)))
      return cudaErrorInvalidValue;
    if (epilogue == kEpiNormResidual) {
      if (ln->stats_out == nullptr || (reinterpret_cast<uintptr_t>(ln->stats_out) & 7u)) return cudaErrorInvalidValue;
      if ((ln->gamma == nullptr) != (ln->beta == nullptr)) return cudaErrorInvalidValue;
      if (ln->gamma != nullptr &&
          ((reinterpret_cast<uintptr_t>(ln->gamma) & 15u) || (reinterpret_cast<uintptr_t>(ln->beta) & 15u)))
        return cudaErrorMisalignedAddress;
    } else {
      if (ln->csum == nullptr || (reinterpret_cast<uintptr_t>(ln->csum) & 15u)) return cudaErrorInvalidValue;
    }
    lnp = *ln;
  }
  const int bn = (n % 256 == 0) ? 256 : 128;
  const bool pair = bn == 256;
  CUtensorMap ta, tb;
  if (!encode_2d_fp16_sw128(&ta, a, static_cast<uint64_t>(max_m), static_cast<uint64_t>(k),
                            static_cast<uint64_t>(k), BM, BK, maps))
    return cudaErrorInvalidValue;
  if (!encode_2d_fp16_sw128(&tb, w_packed, static_cast<uint64_t>(n), static_cast<uint64_t>(k),
                            static_cast<uint64_t>(k), static_cast<uint32_t>(pair ? 128 : bn), BK, maps))
    return cudaErrorInvalidValue;
  const int rev = reverse_m ? 1 : 0;
  if (pair) {
    CUtensorMap tbh;  // 64 W rows per CTA: the half-width units of the last round
    if (!encode_2d_fp16_sw128(&tbh, w_packed, static_cast<uint64_t>(n), static_cast<uint64_t>(k),
                              static_cast<uint64_t>(k), 64, BK, maps))
      return cudaErrorInvalidValue;
    return launch_pair(ta, tb, tbh, bias, residual, c, m_ptr, max_m, n, k, epilogue, status_word, rev, lnp, stream);
  }
  return launch_bn<128>(ta, tb, bias, residual, c, m_ptr, max_m, n, k, epilogue, status_word, rev, stream);
}

}  // namespace etb
