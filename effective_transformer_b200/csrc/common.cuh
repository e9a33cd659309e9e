// Shared device/host helpers for the sm_100a encoder kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <string>
#include <utility>

namespace etb {

class TensorMapCache;  // ptx_sm100.cuh: tensor maps a handle keeps between launches

// Text returned by et_last_error(NULL): errors of calls that take no handle.
void set_global_error(const std::string& msg);

// ---- launch geometry ------------------------------------------------------
constexpr int kNumSMsB200 = 148;

constexpr int kMaxDevices = 64;

// Index of the current device, or -1.
inline int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

// SM count of the current device (cached per device: a process may hold handles on several GPUs).
inline int sm_count() {
  static std::atomic<int> cached[kMaxDevices] = {};
  const int dev = current_device();
  if (dev < 0) return kNumSMsB200;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = kNumSMsB200;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// One-time set-up per device.  A kernel's function attributes (the opt-in to more than 48 KB of
// dynamic shared memory) belong to the device that was current when they were set, so a launcher
// that serves handles on several GPUs of one process has to set them once on each.
class PerDeviceOnce {
 public:
  template <typename F>
  cudaError_t run(F&& setup) {
    const int dev = current_device();
    if (dev < 0) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mutex_);
    if (!done_[dev]) {
      err_[dev] = setup();
      done_[dev] = true;
    }
    return err_[dev];
  }

 private:
  std::mutex mutex_;
  bool done_[kMaxDevices] = {};
  cudaError_t err_[kMaxDevices] = {};
};

// ---- programmatic dependent launch ---------------------------------------
// Consecutive kernels of a pass are launched with the programmatic-stream-
// serialization attribute: the next kernel's CTAs may be scheduled, and run
// their set-up (shared-memory carve-up, barrier init, TMEM allocation), while
// the previous kernel drains.  The contract that makes this safe:
//   * every CTA of such a kernel executes pdl_wait() before its first access
//     to global memory and before any exit path (it returns once the previous
//     kernel has completed and its writes are visible);
//   * pdl_trigger() only lets the next kernel start being scheduled earlier; it
//     carries no ordering.
// Without the launch attribute both instructions are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ETB_PDL=0 launches everything with full stream serialization (A/B measurements).
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("ETB_PDL");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

// kernel<<<grid, block, smem, stream>>>(args...) with the attribute above.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

// ---- device status word ---------------------------------------------------
// A kernel whose bounded wait expires records (kernel id << 8 | site) once.
enum KernelId : int { kKernelGemmTc = 1, kKernelAttnTc = 2, kKernelSelfTest = 15 };

__device__ __forceinline__ void report_timeout(int* status_word, int kernel_id, int site) {
  if (status_word != nullptr) atomicCAS(status_word, 0, (kernel_id << 8) | site);
}

// x rounded to tf32 (11 significand bits, round to nearest), as an fp32 number.
__device__ __forceinline__ float rn_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// ---- 16-byte vector access ------------------------------------------------
struct alignas(16) Vec16 {
  uint32_t x, y, z, w;
};

__device__ __forceinline__ Vec16 ld_global_nc_v4(const void* p) {
  Vec16 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Through L2 only: for rows that other CTAs of the same kernel have just written.
__device__ __forceinline__ Vec16 ld_global_cg_v4(const void* p) {
  Vec16 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ Vec16 ld_global_v4(const void* p) {
  return *reinterpret_cast<const Vec16*>(p);
}
__device__ __forceinline__ void st_global_v4(void* p, const Vec16& v) {
  *reinterpret_cast<Vec16*>(p) = v;
}
__device__ __forceinline__ void st_global_cs_v4(void* p, const Vec16& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// Elements of T held by one 16-byte vector.
template <typename T>
struct VecTraits;
template <>
struct VecTraits<float> {
  static constexpr int kElems = 4;
  __device__ static void unpack(const Vec16& v, float* f) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  __device__ static Vec16 pack(const float* f) {
    Vec16 v;
    v.x = __float_as_uint(f[0]);
    v.y = __float_as_uint(f[1]);
    v.z = __float_as_uint(f[2]);
    v.w = __float_as_uint(f[3]);
    return v;
  }
};
template <>
struct VecTraits<__half> {
  static constexpr int kElems = 8;
  __device__ static void unpack(const Vec16& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 t = __half22float2(h);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ static Vec16 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    Vec16 v;
    v.x = w[0];
    v.y = w[1];
    v.z = w[2];
    v.w = w[3];
    return v;
  }
};

// ---- math -----------------------------------------------------------------
// tanh-form GELU with the constants of the reference kernel
// (cuda/cuda_kernels.cu:29-37); evaluated in fp32.
__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  // 0.5 (1 + tanh u) = 1 / (1 + exp(-2u)): one exponential and one reciprocal, relative
  // error of a few 1e-6; exp overflow (x below about -10) gives x / inf = -0, the limit.
  return __fdividef(x, 1.0f + __expf(-2.0f * u));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- kernel launchers implemented in the .cu files -------------------------
// Every launcher returns the cudaError_t of the launch.  `t_ptr` is a device
// pointer to the valid-token count; kernels never need it on the host.

cudaError_t launch_padding_offsets(const int* mask, int batch, int seq, int* prefix_sum,
                                   int* valid_word_num, int* batch_idx, int* word_idx,
                                   int* seq_len_out, int* cu_seqlens, int* padding_offset,
                                   int* scratch, cudaStream_t stream);
cudaError_t launch_seq_bounds_from_batch_idx(const int* batch_idx, const int* t_ptr, int batch,
                                             int max_tokens, int* cu_seqlens, cudaStream_t stream);
template <typename T>
cudaError_t launch_remove_padding(const T* from, const int* batch_idx, const int* word_idx,
                                  const int* t_ptr, T* to, int batch, int seq, int hidden,
                                  cudaStream_t stream);
template <typename T>
cudaError_t launch_restore_padding(const T* from, const int* batch_idx, const int* word_idx,
                                   const int* t_ptr, T* to, int batch, int seq, int hidden,
                                   cudaStream_t stream);
template <typename T>
cudaError_t launch_add_qkv_bias_transpose(const T* q, const T* bq, const T* k, const T* bk,
                                          const T* v, const T* bv, T* out, const int* t_ptr,
                                          int max_tokens, int heads, int d, cudaStream_t stream);
template <typename T>
cudaError_t launch_add_bias_gelu(T* out, const T* bias, const int* t_ptr, int max_tokens, int n,
                                 cudaStream_t stream);
// split_hi / split_lo (fp32 only, both or neither): the normalised rows are also written as
// rn_tf32 half and remainder, the input format of the fp32 projections on the tensor cores.
template <typename T>
cudaError_t launch_add_bias_input_layernorm(T* out, const T* input, const T* bias, const T* gamma,
                                            const T* beta, const int* t_ptr, int max_tokens, int n,
                                            float eps, cudaStream_t stream, bool reverse = false,
                                            T* split_hi = nullptr, T* split_lo = nullptr);
// Embedding rows + LayerNorm for valid tokens only, written packed [T, n].
// token_type_ids / type_table / pos_table may be null.
template <typename T>
cudaError_t launch_embedding_layernorm(const int* input_ids, const int* token_type_ids,
                                       const int* batch_idx, const int* word_idx, const int* t_ptr,
                                       const T* word_table, int vocab, const T* type_table,
                                       int type_vocab, const T* pos_table, const T* gamma,
                                       const T* beta, T* out, int batch, int seq, int n, float eps,
                                       cudaStream_t stream);
// out[b] = packed[cu_seqlens[b]] (zero row for an empty sequence); *count_out = batch.
cudaError_t launch_gather_first_tokens(const void* packed, const int* cu_seqlens, void* out, int batch,
                                       int max_tokens, int row_bytes, int* count_out,
                                       cudaStream_t stream);
// Weight repacking (runs once per layer when weights are registered).
template <typename T>
cudaError_t launch_transpose(const T* src, T* dst, int rows, int cols, cudaStream_t stream);
template <typename T>
cudaError_t launch_copy_columns(const T* src, T* dst, int rows, int cols, int dst_ld, int dst_col0,
                                cudaStream_t stream);

// kEpiBiasTanh is the pooler's activation (sample/tensorflow/modeling.py:224-232).
// kEpiBiasResidual adds a [M,N] tensor (the layer's residual input) besides the bias, so that
// the LayerNorm behind the projection reads one tensor instead of two.
// kEpiResidualLayerNorm / kEpiLayerNorm (tcgen05 GEMM with N a multiple of 256 up to 1024 only): the
// bias + residual + LayerNorm behind the projection (cuda/cuda_kernels.cu:157-236) runs inside the
// GEMM kernel.  The row block of C whose last column tile has just been stored is normalised in
// place by warps of the same kernel while the rows are still in L2, so no LayerNorm kernel is
// launched and the pre-LayerNorm tensor is never read back from HBM.  kEpiResidualLayerNorm adds
// bias and residual in the GEMM epilogue (as kEpiBiasResidual); kEpiLayerNorm leaves the epilogue
// bare and adds them when the rows are normalised.
//
// kEpiNormIn / kEpiNormInGelu / kEpiNormResidual: the LayerNorm is never materialised.  A projection
// whose input is LN(x) = (x - mu) * rstd * gamma + beta runs on the un-normalised x with gamma folded
// into its weights (W' = diag(gamma) W with centred columns, see fold_layernorm_kernel):
// LN(x) W + b = rstd * (x W' - mu * colsum(W')) + (beta W + b), and the row's mu, rstd come from partial
// sums the producer of x left beside it.
//   kEpiNormIn(Gelu)   C = act(rstd[r] * (acc - mu[r] * csum[n]) + bias[n])
//   kEpiNormResidual   C = acc + bias[n] + ((res[r,n] - mu[r]) * rstd[r] * gamma[n] + beta[n]), i.e. the residual
//                      is the LayerNorm of `residual`, taken on the fly; and the kernel leaves the sum and
//                      the sum of squares of every 64-column piece of every row of C (as stored, after
//                      rounding) in `stats_out`, for the consumers of LN(C).
enum Epilogue : int {
  kEpiNone = 0, kEpiBias = 1, kEpiBiasGelu = 2, kEpiBiasTanh = 3, kEpiBiasResidual = 4,
  kEpiResidualLayerNorm = 5, kEpiLayerNorm = 6, kEpiNormIn = 7, kEpiNormInGelu = 8, kEpiNormResidual = 9
};

// LayerNorm parameters of the two fused epilogues.  `counters`: one int per 32 rows of the 256-row
// tiles that cover C (8 * ceil(max_m / 256) of them), zero before the launch; the kernel leaves
// them zero again.
// Deferred variants (kEpiNorm*): `stats_in` [rows, 2 * stat_slots] holds (sum, sum of squares) per
// 64-column piece of the rows of the normalised tensor (stat_slots = its width / 64; rows rounded up
// to the 256-row tile), null = the tensor is used as it is (mu = 0, rstd = 1); `csum` [N] = column
// sums of the folded weights; `stats_out` [rows, 2 * N / 64]; gamma / beta null = ones / zeros.
struct GemmLayerNorm {
  const __half* gamma = nullptr;
  const __half* beta = nullptr;
  float eps = 1e-6f;
  int* counters = nullptr;
  const float* stats_in = nullptr;
  int stat_slots = 0;
  const __half* csum = nullptr;
  float* stats_out = nullptr;
};
__host__ __device__ constexpr bool is_deferred_norm(int epi) {
  return epi == kEpiNormIn || epi == kEpiNormInGelu || epi == kEpiNormResidual;
}

// LayerNorm parameters folded into the projection that consumes it (kEpiNormIn): w_packed [N,K]
// K-major -> w_folded = w * gamma[k] with the mean over k taken from every output row (it multiplies
// sum_k (x_k - mu) = 0), csum[n] = sum_k w_folded as stored (what fp16 rounding leaves of zero),
// bias_folded = bias + beta W.
cudaError_t launch_fold_layernorm(const __half* w_packed, const __half* bias, const __half* gamma,
                                  const __half* beta, __half* w_folded, __half* csum, __half* bias_folded, int n,
                                  int k, cudaStream_t stream);
// CUDA-core GEMM: C[M,N] = epi(A[M,K] * W[K,N]); W row-major [K,N].
template <typename T>
cudaError_t launch_gemm_simt(const T* a, const T* w, const T* bias, T* c, const int* m_ptr,
                             int max_m, int n, int k, int epilogue, cudaStream_t stream);
// CUDA-core attention on the packed layout.  ctx_lo (fp32 only): the output is
// written split for the tf32 projection behind it, rn_tf32 half to ctx, remainder to ctx_lo.
// cu_seqlens_k given: cross-attention, sequence b's keys / values are rows
// [cu_seqlens_k[b], cu_seqlens_k[b+1]) of k / v (row stride kv_token_stride, at most max_seq_k of them).
template <typename T>
cudaError_t launch_attention_simt(const T* q, const T* k, const T* v, long long token_stride,
                                  long long head_stride, T* ctx, const int* cu_seqlens, int batch,
                                  int max_seq, int heads, int d, cudaStream_t stream, T* ctx_lo = nullptr,
                                  const int* cu_seqlens_k = nullptr, long long kv_token_stride = 0,
                                  int max_seq_k = 0);
// Self-attention of the fp32 handle on tensor cores at fp32 accuracy (mma.sync tf32, three products
// per fp32 product); same layout and arguments as launch_attention_simt<float>.
cudaError_t launch_attention_tf32x3(const float* q, const float* k, const float* v, long long token_stride,
                                    long long head_stride, float* ctx, const int* cu_seqlens, int batch,
                                    int max_seq, int heads, int d, cudaStream_t stream, float* ctx_lo = nullptr);
// The same under a general [B, S, S] mask with the reference op's semantics
// (padded keys take part with K = V = 0).  pos_row[b*S+p] = packed row of
// position p or -1, made by launch_position_rows (a memset and one kernel).
cudaError_t launch_position_rows(const int* batch_idx, const int* word_idx, const int* t_ptr, int batch,
                                 int seq, int* pos_row, cudaStream_t stream);
template <typename T>
cudaError_t launch_attention_masked_simt(const T* q, const T* k, const T* v, long long token_stride,
                                         long long head_stride, T* ctx, const T* attr_mask,
                                         const int* cu_seqlens, const int* word_idx, const int* pos_row,
                                         int batch, int seq, int heads, int d, cudaStream_t stream);
// Tensor-core attention (TMA-fed, mma.sync), fp16.  q/k/v hold max_tokens rows.
cudaError_t launch_attention_tc(const __half* q, const __half* k, const __half* v,
                                long long token_stride, long long head_stride, __half* ctx,
                                const int* cu_seqlens, int batch, int max_seq, int max_tokens, int heads,
                                int d, int* status_word, cudaStream_t stream, TensorMapCache* maps = nullptr);
// tcgen05 attention for sequences of at most 128 tokens: a plan (sequences
// packed into 128-row tiles) made once per batch, then one launch per layer.
// attr_mask given ([B, seq, seq], 1 = attend; with batch_idx / word_idx of the packed rows): a
// general mask with the reference op's semantics (padded keys take part with K = V = 0).
size_t attention_plan_ints(int batch, int max_tokens);
cudaError_t launch_attention_plan(const int* cu_seqlens, int batch, int max_tokens, int* plan,
                                  cudaStream_t stream);
cudaError_t launch_attention_tcgen05(const __half* q, const __half* k, const __half* v,
                                     long long token_stride, long long head_stride, __half* ctx,
                                     const int* plan, int batch, int max_tokens, int heads, int d,
                                     int* status_word, cudaStream_t stream, bool reverse = false,
                                     TensorMapCache* maps = nullptr, const __half* attr_mask = nullptr,
                                     const int* batch_idx = nullptr, const int* word_idx = nullptr, int seq = 0);
// fp32 GEMM on the tensor cores by the three-product tf32 split (gemm_tf32x3.cu):
// x = hi + lo with hi = rn_tf32(x); hi/lo may alias x.  rows_ptr null = max_rows.
cudaError_t launch_split_tf32(const float* x, float* hi, float* lo, const int* rows_ptr, int max_rows, int cols,
                              cudaStream_t stream);
// a_hi/a_lo [max_m, K], w_hi/w_lo [N, K] (K-major); C = epi(A * W^T (+ bias)), fp32.
// c_lo given: the result is written already split, rn_tf32 half to c and remainder to c_lo.
cudaError_t launch_gemm_tf32x3(const float* a_hi, const float* a_lo, const float* w_hi, const float* w_lo,
                               const float* bias, float* c, const int* m_ptr, int max_m, int n, int k,
                               int epilogue, int* status_word, cudaStream_t stream, bool reverse_m = false,
                               float* c_lo = nullptr, TensorMapCache* maps = nullptr);
// tcgen05 GEMM, fp16 in / fp32 accumulate / fp16 out.  w_packed is [N,K].
// reverse_m: row tiles are visited from the last to the first.  A kernel that
// consumes what the previous kernel has just written finds the rows written
// last still in L2 if it starts with them, so consecutive kernels of a layer
// alternate their direction.
cudaError_t launch_gemm_tcgen05(const __half* a, const __half* w_packed, const __half* bias,
                                __half* c, const int* m_ptr, int max_m, int n, int k, int epilogue,
                                int* status_word, cudaStream_t stream, bool reverse_m = false,
                                const __half* residual = nullptr, TensorMapCache* maps = nullptr,
                                const GemmLayerNorm* ln = nullptr);
// Whether the fused LayerNorm epilogues can serve a projection of n output columns.
inline bool gemm_layernorm_supported(int n) { return n > 0 && n % 256 == 0 && n <= 1024; }


// One CTA whose bounded wait (2 ms) runs out on purpose; it records (kKernelSelfTest << 8 | 1).
cudaError_t launch_selftest_wait_timeout(int* status_word, cudaStream_t stream);

// ---- work units of the CTA-pair GEMMs ---------------------------------------
// Tiles of 256 x 256 are dealt round-robin to the pairs.  When the last round
// would keep at most half of the pairs busy, each of its tiles is cut into two
// 256 x 128 units: units [0, full_tiles) are whole tiles, the rest are halves.
struct PairUnit {
  int m_tile;  // 256-row tile
  int col0;    // first output column
  int ncols;   // 256 (whole tile) or 128 (half of a last-round tile)
};
__device__ __forceinline__ PairUnit pair_unit(int u, int full_tiles, int n_tiles, int m_tiles, int reverse_m) {
  int tile = u, half = -1;
  if (u >= full_tiles) {
    const int r = u - full_tiles;
    tile = full_tiles + (r >> 1);
    half = r & 1;
  }
  const int m_lin = tile / n_tiles, n_tile = tile - m_lin * n_tiles;
  PairUnit pu;
  pu.m_tile = reverse_m ? m_tiles - 1 - m_lin : m_lin;
  pu.col0 = n_tile * 256 + (half > 0 ? 128 : 0);
  pu.ncols = half < 0 ? 256 : 128;
  return pu;
}
// Splits `num_tiles` for `num_pairs` pairs: returns the number of whole-tile
// units, *num_units = all units.
__device__ __forceinline__ int pair_units(int num_tiles, int num_pairs, int* num_units) {
  const int rem = num_tiles % num_pairs;
  const bool split = rem > 0 && 2 * rem <= num_pairs;
  const int full_tiles = split ? num_tiles - rem : num_tiles;
  *num_units = full_tiles + (split ? 2 * rem : 0);
  return full_tiles;
}

}  // namespace etb
