// Fused element-wise kernels on the packed [T, *] layout: QKV bias + head
// transpose, bias + GELU, bias + residual + LayerNorm, and the weight
// repacking helpers.  They replace add_QKV_bias_padding (cuda/attention.cu:
// 106-242), add_bias_act and add_bias_input_layernorm (cuda/cuda_kernels.cu:
// 88-271).  All arithmetic is fp32; every global access is a 16-byte vector.
#include "common.cuh"

namespace etb {

namespace {

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 8;

__device__ __forceinline__ int clamp_tokens(const int* t_ptr, int max_tokens) {
  const int t = *t_ptr;
  return t < 0 ? 0 : (t > max_tokens ? max_tokens : t);
}

// out[which][head][token][0:d] = src_which[token][head*d : head*d+d] + bias_which[...]
template <typename T>
__global__ void __launch_bounds__(kThreads)
add_qkv_bias_transpose_kernel(const T* __restrict__ q, const T* __restrict__ bq,
                              const T* __restrict__ k, const T* __restrict__ bk,
                              const T* __restrict__ v, const T* __restrict__ bv,
                              T* __restrict__ out, const int* __restrict__ t_ptr, int max_tokens,
                              int heads, int d) {
  constexpr int E = VecTraits<T>::kElems;
  const int t = clamp_tokens(t_ptr, max_tokens);
  const int hidden = heads * d;
  const int vpr = hidden / E;   // vectors per row
  const int vph = d / E;        // vectors per head
  const long long total = static_cast<long long>(t) * vpr;
  const T* srcs[3] = {q, k, v};
  const T* biases[3] = {bq, bk, bv};
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int token = static_cast<int>(i / vpr);
    const int c = static_cast<int>(i - static_cast<long long>(token) * vpr);
    const int head = c / vph, within = c - head * vph;
    Vec16 x[3], b[3];
#pragma unroll
    for (int w = 0; w < 3; ++w) {
      x[w] = ld_global_nc_v4(srcs[w] + static_cast<size_t>(token) * hidden + c * E);
      b[w] = ld_global_v4(biases[w] + c * E);
    }
#pragma unroll
    for (int w = 0; w < 3; ++w) {
      float fx[E], fb[E];
      VecTraits<T>::unpack(x[w], fx);
      VecTraits<T>::unpack(b[w], fb);
#pragma unroll
      for (int e = 0; e < E; ++e) fx[e] += fb[e];
      T* dst = out + ((static_cast<size_t>(w) * heads + head) * max_tokens + token) * d + within * E;
      st_global_v4(dst, VecTraits<T>::pack(fx));
    }
  }
}

// out[token][c] = gelu(out[token][c] + bias[c]) in place.
template <typename T>
__global__ void __launch_bounds__(kThreads)
add_bias_gelu_kernel(T* __restrict__ out, const T* __restrict__ bias, const int* __restrict__ t_ptr,
                     int max_tokens, int n) {
  constexpr int E = VecTraits<T>::kElems;
  constexpr int kBatch = 4;
  const int t = clamp_tokens(t_ptr, max_tokens);
  const int vpr = n / E;
  const long long total = static_cast<long long>(t) * vpr;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < total;
       i0 += stride * kBatch) {
    Vec16 x[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const long long i = i0 + j * stride;
      if (i < total) x[j] = ld_global_v4(out + i * E);
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const long long i = i0 + j * stride;
      if (i < total) {
        const int c = static_cast<int>(i % vpr);
        float fx[E], fb[E];
        VecTraits<T>::unpack(x[j], fx);
        VecTraits<T>::unpack(ld_global_v4(bias + c * E), fb);
#pragma unroll
        for (int e = 0; e < E; ++e) fx[e] = gelu_tanh(fx[e] + fb[e]);
        st_global_v4(out + i * E, VecTraits<T>::pack(fx));
      }
    }
  }
}

// out[row] = LN(out[row] + input[row] + bias) * gamma + beta (kHasInput false:
// LN(out[row]) alone, for a producer that added them itself), one warp per row,
// the row held in registers (fp32) between the two statistics passes.
// A warp fetches kRows rows at a time before it works on the first: the kernel is
// bound by the bytes it has in flight (about 35 KB per SM are needed to cover the
// HBM latency at full bandwidth), and one 1.5 KB row per warp is too few of them.
// bias / gamma / beta are re-read per row: they stay L1-resident, and not
// keeping them in registers raises the number of resident warps.
template <typename T, int kVPL, int kRows, bool kHasInput>
__global__ void __launch_bounds__(kThreads, (kVPL <= 4 ? 2 : 1))
add_bias_input_layernorm_kernel(T* __restrict__ out, const T* __restrict__ input,
                                const T* __restrict__ bias, const T* __restrict__ gamma,
                                const T* __restrict__ beta, const int* __restrict__ t_ptr,
                                int max_tokens, int n, float eps, int reverse, T* __restrict__ split_hi,
                                T* __restrict__ split_lo) {
  pdl_wait();
  pdl_trigger();
  constexpr int E = VecTraits<T>::kElems;
  const int t = clamp_tokens(t_ptr, max_tokens);
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * (kThreads / 32);
  const int vpr = n / E;
  const float inv_n = 1.0f / static_cast<float>(n);

  for (int r0 = warp; r0 < t; r0 += nwarps * kRows) {
    Vec16 vo[kRows][kVPL], vi[kHasInput ? kRows : 1][kVPL];
    int rows[kRows];
#pragma unroll
    for (int k = 0; k < kRows; ++k) {
      const int r = r0 + k * nwarps;
      rows[k] = r < t ? (reverse ? t - 1 - r : r) : -1;  // last rows first: they are the freshest in L2
      if (rows[k] >= 0) {
        const T* orow = out + static_cast<size_t>(rows[k]) * n;
#pragma unroll
        for (int j = 0; j < kVPL; ++j) {
          const int c = j * 32 + lane;
          if (c < vpr) {
            vo[k][j] = ld_global_v4(orow + c * E);
            if (kHasInput) vi[k][j] = ld_global_nc_v4(input + static_cast<size_t>(rows[k]) * n + c * E);
          }
        }
      }
    }
#pragma unroll
    for (int k = 0; k < kRows; ++k) {
      if (rows[k] < 0) continue;  // uniform over the warp
      T* orow = out + static_cast<size_t>(rows[k]) * n;
      float x[kVPL][E];
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < kVPL; ++j) {
        const int c = j * 32 + lane;
        if (c < vpr) {
          float fo[E];
          VecTraits<T>::unpack(vo[k][j], fo);
          if (kHasInput) {
            float fi[E], fb[E];
            VecTraits<T>::unpack(vi[k][j], fi);
            VecTraits<T>::unpack(ld_global_v4(bias + c * E), fb);
#pragma unroll
            for (int e = 0; e < E; ++e) fo[e] += fi[e] + fb[e];
          }
#pragma unroll
          for (int e = 0; e < E; ++e) {
            x[j][e] = fo[e];
            sum += x[j][e];
          }
        } else {
#pragma unroll
          for (int e = 0; e < E; ++e) x[j][e] = 0.f;
        }
      }
      const float mean = warp_sum(sum) * inv_n;
      float sq = 0.f;
#pragma unroll
      for (int j = 0; j < kVPL; ++j) {
        const int c = j * 32 + lane;
        if (c < vpr) {
#pragma unroll
          for (int e = 0; e < E; ++e) {
            const float dlt = x[j][e] - mean;
            sq += dlt * dlt;
          }
        }
      }
      const float rstd = rsqrtf(warp_sum(sq) * inv_n + eps);
#pragma unroll
      for (int j = 0; j < kVPL; ++j) {
        const int c = j * 32 + lane;
        if (c < vpr) {
          float fg[E], fbe[E], y[E];
          VecTraits<T>::unpack(ld_global_v4(gamma + c * E), fg);
          VecTraits<T>::unpack(ld_global_v4(beta + c * E), fbe);
#pragma unroll
          for (int e = 0; e < E; ++e) y[e] = (x[j][e] - mean) * rstd * fg[e] + fbe[e];
          st_global_v4(orow + c * E, VecTraits<T>::pack(y));
          if constexpr (sizeof(T) == 4) {
            if (split_hi != nullptr) {  // fp32 tensor path: the next projection's input, already split
              float hi[E], lo[E];
#pragma unroll
              for (int e = 0; e < E; ++e) {
                hi[e] = rn_tf32(y[e]);
                lo[e] = y[e] - hi[e];
              }
              const size_t off = static_cast<size_t>(rows[k]) * n + c * E;
              st_global_v4(split_hi + off, VecTraits<T>::pack(hi));
              st_global_v4(split_lo + off, VecTraits<T>::pack(lo));
            }
          }
        }
      }
    }
  }
}

template <typename T>
__global__ void transpose_kernel(const T* __restrict__ src, T* __restrict__ dst, int rows, int cols) {
  __shared__ T tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[i][threadIdx.x] = src[static_cast<size_t>(r) * cols + c];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[static_cast<size_t>(c) * rows + r] = tile[threadIdx.x][i];
  }
}

template <typename T>
__global__ void copy_columns_kernel(const T* __restrict__ src, T* __restrict__ dst, int rows,
                                    int cols, int dst_ld, int dst_col0) {
  const long long total = static_cast<long long>(rows) * cols;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols, c = i - r * cols;
    dst[r * dst_ld + dst_col0 + c] = src[i];
  }
}

inline int grid_for(long long work_items) {
  long long ctas = (work_items + kThreads - 1) / kThreads;
  const long long cap = static_cast<long long>(sm_count()) * kCtasPerSm;
  if (ctas > cap) ctas = cap;
  return ctas < 1 ? 1 : static_cast<int>(ctas);
}


// LayerNorm folded into the projection behind it.  For LN(x) = (x - mu) * rstd * gamma + beta and
// y = LN(x) W + b:   y = rstd * sum_k (x_k - mu) V_kn + b'_n   with V = diag(gamma) W, b' = b + beta W.
// Since sum_k (x_k - mu) = 0, any constant may be taken from a column of V: the folded weights are
// the CENTRED columns  W'_kn = V_kn - mean_k V_kn,  so that  y = rstd * (x W' - mu * csum) + b'  with
// csum_n = sum_k W'_kn, which is only what rounding W' to fp16 leaves (~1e-4): the large term
// mu * colsum(V), which a row with |mu| >> sigma would have to cancel against x V in the epilogue, is
// gone, and the cancellation happens inside the tensor core's fp32 accumulation instead.
// W is the packed [N, K] K-major copy; one CTA per output row n.
__global__ void __launch_bounds__(256)
fold_layernorm_kernel(const __half* __restrict__ w, const __half* __restrict__ bias,
                      const __half* __restrict__ gamma, const __half* __restrict__ beta, __half* __restrict__ wf,
                      __half* __restrict__ csum, __half* __restrict__ bias_f, int k) {
  const int n = blockIdx.x;
  const __half* wrow = w + static_cast<size_t>(n) * k;
  __half* frow = wf + static_cast<size_t>(n) * k;
  __shared__ float red[2][8];
  __shared__ float mean_s;
  auto block_sum2 = [&](float a, float b, float& ta, float& tb) {
    a = warp_sum(a);
    b = warp_sum(b);
    __syncthreads();  // red[] may still be read from the previous use
    if ((threadIdx.x & 31) == 0) red[0][threadIdx.x >> 5] = a, red[1][threadIdx.x >> 5] = b;
    __syncthreads();
    ta = 0.f, tb = 0.f;
    for (int i = 0; i < 8; ++i) ta += red[0][i], tb += red[1][i];
  };
  float v_sum = 0.f, bw = 0.f;
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    const float wv = __half2float(wrow[j]);
    v_sum += wv * __half2float(gamma[j]);
    bw += __half2float(beta[j]) * wv;
  }
  float tv, tb;
  block_sum2(v_sum, bw, tv, tb);
  if (threadIdx.x == 0) mean_s = tv / static_cast<float>(k);
  __syncthreads();
  const float mean = mean_s;
  float s = 0.f;
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    const __half f = __float2half_rn(__half2float(wrow[j]) * __half2float(gamma[j]) - mean);
    frow[j] = f;
    s += __half2float(f);
  }
  float ts, unused;
  block_sum2(s, 0.f, ts, unused);
  if (threadIdx.x == 0) {
    csum[n] = __float2half_rn(ts);
    bias_f[n] = __float2half_rn(__half2float(bias[n]) + tb);
  }
}

}  // namespace

template <typename T>
cudaError_t launch_add_qkv_bias_transpose(const T* q, const T* bq, const T* k, const T* bk,
                                          const T* v, const T* bv, T* out, const int* t_ptr,
                                          int max_tokens, int heads, int d, cudaStream_t stream) {
  constexpr int E = VecTraits<T>::kElems;
  if (max_tokens <= 0) return cudaSuccess;
  if (d % E != 0) return cudaErrorInvalidValue;
  const long long work = static_cast<long long>(max_tokens) * (heads * d / E);
  add_qkv_bias_transpose_kernel<T><<<grid_for(work), kThreads, 0, stream>>>(
      q, bq, k, bk, v, bv, out, t_ptr, max_tokens, heads, d);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_add_bias_gelu(T* out, const T* bias, const int* t_ptr, int max_tokens, int n,
                                 cudaStream_t stream) {
  constexpr int E = VecTraits<T>::kElems;
  if (max_tokens <= 0) return cudaSuccess;
  if (n % E != 0) return cudaErrorInvalidValue;
  const long long work = static_cast<long long>(max_tokens) * (n / E) / 4 + 1;
  add_bias_gelu_kernel<T><<<grid_for(work), kThreads, 0, stream>>>(out, bias, t_ptr, max_tokens, n);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_add_bias_input_layernorm(T* out, const T* input, const T* bias, const T* gamma,
                                            const T* beta, const int* t_ptr, int max_tokens, int n,
                                            float eps, cudaStream_t stream, bool reverse, T* split_hi,
                                            T* split_lo) {
  constexpr int E = VecTraits<T>::kElems;
  if (max_tokens <= 0) return cudaSuccess;
  if ((split_hi == nullptr) != (split_lo == nullptr) || (split_hi != nullptr && sizeof(T) != 4))
    return cudaErrorInvalidValue;
  if (n % E != 0 || n <= 0) return cudaErrorInvalidValue;
  const int vpl = (n / E + 31) / 32;
  const bool has_input = input != nullptr;
  if (has_input && bias == nullptr) return cudaErrorInvalidValue;
  cudaError_t le = cudaSuccess;
  // One wave of CTAs, as many as are resident at once (the kernel's warps loop over the rows):
  // with more, the later waves start as the first ones end and the kernel has a long tail.
  // Rows a warp has in flight: about 18 vectors of 16 bytes per lane.
#define ETB_LN_ONE(V, R, HAS)                                                                                  \
  do {                                                                                                         \
    auto kernel = add_bias_input_layernorm_kernel<T, V, R, HAS>;                                               \
    static std::atomic<int> resident[kMaxDevices] = {};                                                        \
    const int dev = current_device();                                                                          \
    int per_sm = dev >= 0 ? resident[dev].load(std::memory_order_relaxed) : 0;                                 \
    if (per_sm == 0) {                                                                                         \
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0) != cudaSuccess ||        \
          per_sm < 1)                                                                                          \
        per_sm = 1;                                                                                            \
      if (dev >= 0) resident[dev].store(per_sm, std::memory_order_relaxed);                                    \
    }                                                                                                          \
    const long long rows_per_cta = static_cast<long long>(kThreads / 32) * R;                                  \
    long long ctas = (max_tokens + rows_per_cta - 1) / rows_per_cta;                                           \
    const long long cap = static_cast<long long>(sm_count()) * per_sm;                                         \
    if (ctas > cap) ctas = cap;                                                                                \
    le = launch_pdl(kernel, dim3(static_cast<int>(ctas)), dim3(kThreads), 0, stream, out, input, bias, gamma,  \
                    beta, t_ptr, max_tokens, n, eps, reverse ? 1 : 0, split_hi, split_lo);                     \
  } while (0)
#define ETB_LN(V, R_IN, R_NO)              \
  do {                                     \
    if (has_input) ETB_LN_ONE(V, R_IN, true); \
    else ETB_LN_ONE(V, R_NO, false);       \
  } while (0)
  if (vpl <= 1) ETB_LN(1, 4, 8);
  else if (vpl <= 2) ETB_LN(2, 4, 8);
  else if (vpl <= 3) ETB_LN(3, 2, 4);
  else if (vpl <= 4) ETB_LN(4, 2, 4);
  else if (vpl <= 6) ETB_LN(6, 1, 2);
  else if (vpl <= 8) ETB_LN(8, 1, 1);
  else return cudaErrorInvalidValue;
#undef ETB_LN
#undef ETB_LN_ONE
  return le;
}

template <typename T>
cudaError_t launch_transpose(const T* src, T* dst, int rows, int cols, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  transpose_kernel<T><<<grid, block, 0, stream>>>(src, dst, rows, cols);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_copy_columns(const T* src, T* dst, int rows, int cols, int dst_ld, int dst_col0,
                                cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  copy_columns_kernel<T><<<grid_for(static_cast<long long>(rows) * cols), kThreads, 0, stream>>>(
      src, dst, rows, cols, dst_ld, dst_col0);
  return cudaGetLastError();
}

#define ETB_INST(T)                                                                              \
  template cudaError_t launch_add_qkv_bias_transpose<T>(const T*, const T*, const T*, const T*,  \
                                                        const T*, const T*, T*, const int*, int, \
                                                        int, int, cudaStream_t);                 \
  template cudaError_t launch_add_bias_gelu<T>(T*, const T*, const int*, int, int, cudaStream_t); \
  template cudaError_t launch_add_bias_input_layernorm<T>(T*, const T*, const T*, const T*,      \
                                                          const T*, const int*, int, int, float, \
                                                          cudaStream_t, bool, T*, T*);           \
  template cudaError_t launch_transpose<T>(const T*, T*, int, int, cudaStream_t);                \
  template cudaError_t launch_copy_columns<T>(const T*, T*, int, int, int, int, cudaStream_t);
ETB_INST(float)
ETB_INST(__half)
#undef ETB_INST

cudaError_t launch_fold_layernorm(const __half* w_packed, const __half* bias, const __half* gamma,
                                  const __half* beta, __half* w_folded, __half* csum, __half* bias_folded, int n,
                                  int k, cudaStream_t stream) {
  if (n <= 0 || k <= 0) return cudaErrorInvalidValue;
  fold_layernorm_kernel<<<n, 256, 0, stream>>>(w_packed, bias, gamma, beta, w_folded, csum, bias_folded, k);
  return cudaGetLastError();
}

}  // namespace etb
