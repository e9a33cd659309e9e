// CUDA-core self-attention on the packed, variable-length layout: one CTA per
// (sequence, head), one query row per thread, keys streamed through shared
// memory in blocks of 64 with an online softmax.  fp32 arithmetic throughout:
// this is the attention of the fp32 handle.  It replaces the padded batched
// GEMMs + softmax_kernel + transpose_rm_padding sequence of the reference
// (tf_op/bert_transformer_op.cu.cc:158-191, cuda/attention.cu:249-492); no
// padded position is loaded or computed.
// A second kernel evaluates the same block under a general [B, S, S] attention
// mask (any dtype of the handle), for callers whose mask is not the key-only
// tile of the input mask.
#include "common.cuh"

namespace etb {

namespace {

constexpr int kD = 64;        // size_per_head
constexpr int kKeyBlock = 64;
constexpr int kThreads = 128;

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(kThreads)
attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                      long long token_stride, long long head_stride, T* __restrict__ ctx,
                      const int* __restrict__ cu_seqlens, int heads, int max_seq, float scale) {
  const int b = blockIdx.x / heads, head = blockIdx.x % heads;
  const int lo = cu_seqlens[b];
  int len = cu_seqlens[b + 1] - lo;
  if (len <= 0) return;
  if (len > max_seq) len = max_seq;  // corrupt bounds: stay inside the sequence budget

  __shared__ float Ks[kKeyBlock][kD + 1];
  __shared__ float Vs[kKeyBlock][kD];

  const size_t hoff = static_cast<size_t>(head) * head_stride;
  const int hidden = heads * kD;

  for (int q0 = 0; q0 < len; q0 += kThreads) {
    const int qi = q0 + threadIdx.x;
    const bool active = qi < len;
    float qr[kD], acc[kD];
    float m = -INFINITY, l = 0.f;
#pragma unroll
    for (int c = 0; c < kD; ++c) acc[c] = 0.f;
    if (active) {
      const T* qp = q + static_cast<size_t>(lo + qi) * token_stride + hoff;
#pragma unroll
      for (int c = 0; c < kD; ++c) qr[c] = to_f<T>(qp[c]) * scale;
    } else {
#pragma unroll
      for (int c = 0; c < kD; ++c) qr[c] = 0.f;
    }
    for (int k0 = 0; k0 < len; k0 += kKeyBlock) {
      const int nk = min(kKeyBlock, len - k0);
      __syncthreads();
      for (int idx = threadIdx.x; idx < nk * kD; idx += kThreads) {
        const int j = idx / kD, c = idx % kD;
        const size_t off = static_cast<size_t>(lo + k0 + j) * token_stride + hoff + c;
        Ks[j][c] = to_f<T>(k[off]);
        Vs[j][c] = to_f<T>(v[off]);
      }
      __syncthreads();
      if (active) {
        for (int j = 0; j < nk; ++j) {
          float s = 0.f;
#pragma unroll
          for (int c = 0; c < kD; ++c) s = fmaf(qr[c], Ks[j][c], s);
          if (s > m) {
            const float r = expf(m - s);  // exp(-inf) = 0 on the first key
            l *= r;
#pragma unroll
            for (int c = 0; c < kD; ++c) acc[c] *= r;
            m = s;
          }
          const float p = expf(s - m);
          l += p;
#pragma unroll
          for (int c = 0; c < kD; ++c) acc[c] = fmaf(p, Vs[j][c], acc[c]);
        }
      }
    }
    if (active) {
      const float inv = 1.0f / l;
      T* op = ctx + static_cast<size_t>(lo + qi) * hidden + head * kD;
#pragma unroll
      for (int c = 0; c < kD; ++c) op[c] = from_f<T>(acc[c] * inv);
    }
  }
}

// pos_row[b*S + p] = packed row of position p of sequence b, or -1 if padded.
__global__ void position_rows_kernel(const int* __restrict__ batch_idx, const int* __restrict__ word_idx,
                                     const int* __restrict__ t_ptr, int max_tokens, int seq,
                                     int* __restrict__ pos_row) {
  int t = *t_ptr;
  t = t < 0 ? 0 : (t > max_tokens ? max_tokens : t);
  for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < t; v += gridDim.x * blockDim.x) {
    const long long flat = static_cast<long long>(batch_idx[v]) * seq + word_idx[v];
    if (flat >= 0 && flat < max_tokens) pos_row[flat] = v;
  }
}

// Attention under a general [B, S, S] mask, with the semantics of the
// reference op (cuda/attention.cu:106-242 then :249-382): every query of a
// sequence sees all S key positions; a padded key has K = V = 0 (the op
// scatters valid rows into zero-filled buffers), so its score is 0 before the
// additive mask term (1 - m) * -10000.  One CTA per (sequence, head), one
// valid query per thread, key positions streamed in blocks of 64 through
// shared memory, online softmax in fp32.  A fallback: correctness first.
template <typename T>
__global__ void __launch_bounds__(kThreads)
attention_masked_simt_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                             long long token_stride, long long head_stride, T* __restrict__ ctx,
                             const T* __restrict__ attr_mask, const int* __restrict__ cu_seqlens,
                             const int* __restrict__ word_idx, const int* __restrict__ pos_row, int heads,
                             int seq, float scale) {
  const int b = blockIdx.x / heads, head = blockIdx.x % heads;
  const int lo = cu_seqlens[b];
  int len = cu_seqlens[b + 1] - lo;
  if (len <= 0) return;
  if (len > seq) len = seq;

  __shared__ float Ks[kKeyBlock][kD + 1];
  __shared__ float Vs[kKeyBlock][kD];
  __shared__ int rows[kKeyBlock];

  const size_t hoff = static_cast<size_t>(head) * head_stride;
  const int hidden = heads * kD;
  const int* prow = pos_row + static_cast<size_t>(b) * seq;

  for (int q0 = 0; q0 < len; q0 += kThreads) {
    const int qi = q0 + threadIdx.x;
    const bool active = qi < len;
    float qr[kD], acc[kD];
    float m = -INFINITY, l = 0.f;
    int qpos = 0;
#pragma unroll
    for (int c = 0; c < kD; ++c) acc[c] = 0.f;
    if (active) {
      const T* qp = q + static_cast<size_t>(lo + qi) * token_stride + hoff;
#pragma unroll
      for (int c = 0; c < kD; ++c) qr[c] = to_f<T>(qp[c]) * scale;
      qpos = word_idx[lo + qi];
      qpos = qpos < 0 ? 0 : (qpos >= seq ? seq - 1 : qpos);
    } else {
#pragma unroll
      for (int c = 0; c < kD; ++c) qr[c] = 0.f;
    }
    const T* mrow = attr_mask + (static_cast<size_t>(b) * seq + qpos) * seq;
    for (int k0 = 0; k0 < seq; k0 += kKeyBlock) {
      const int nk = min(kKeyBlock, seq - k0);
      __syncthreads();
      if (threadIdx.x < nk) rows[threadIdx.x] = prow[k0 + threadIdx.x];
      __syncthreads();
      for (int idx = threadIdx.x; idx < nk * kD; idx += kThreads) {
        const int j = idx / kD, c = idx % kD;
        const int r = rows[j];
        float kv = 0.f, vv = 0.f;
        if (r >= 0) {
          const size_t off = static_cast<size_t>(r) * token_stride + hoff + c;
          kv = to_f<T>(k[off]);
          vv = to_f<T>(v[off]);
        }
        Ks[j][c] = kv;
        Vs[j][c] = vv;
      }
      __syncthreads();
      if (active) {
        for (int j = 0; j < nk; ++j) {
          float s = 0.f;
#pragma unroll
          for (int c = 0; c < kD; ++c) s = fmaf(qr[c], Ks[j][c], s);
          s += (1.0f - to_f<T>(mrow[k0 + j])) * -10000.0f;
          if (s > m) {
            const float r = expf(m - s);
            l *= r;
#pragma unroll
            for (int c = 0; c < kD; ++c) acc[c] *= r;
            m = s;
          }
          const float p = expf(s - m);
          l += p;
#pragma unroll
          for (int c = 0; c < kD; ++c) acc[c] = fmaf(p, Vs[j][c], acc[c]);
        }
      }
    }
    if (active) {
      const float inv = 1.0f / l;
      T* op = ctx + static_cast<size_t>(lo + qi) * hidden + head * kD;
#pragma unroll
      for (int c = 0; c < kD; ++c) op[c] = from_f<T>(acc[c] * inv);
    }
  }
}

}  // namespace

cudaError_t launch_position_rows(const int* batch_idx, const int* word_idx, const int* t_ptr, int batch,
                                 int seq, int* pos_row, cudaStream_t stream) {
  const long long n = static_cast<long long>(batch) * seq;
  if (n <= 0) return cudaSuccess;
  if (n > 0x7fffffffLL) return cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(pos_row, 0xff, static_cast<size_t>(n) * sizeof(int), stream);  // all -1
  if (e != cudaSuccess) return e;
  long long ctas = (n + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (ctas > cap) ctas = cap;
  position_rows_kernel<<<static_cast<int>(ctas), 256, 0, stream>>>(batch_idx, word_idx, t_ptr,
                                                                   static_cast<int>(n), seq, pos_row);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_attention_masked_simt(const T* q, const T* k, const T* v, long long token_stride,
                                         long long head_stride, T* ctx, const T* attr_mask,
                                         const int* cu_seqlens, const int* word_idx, const int* pos_row,
                                         int batch, int seq, int heads, int d, cudaStream_t stream) {
  if (batch <= 0 || heads <= 0 || seq <= 0) return cudaSuccess;
  if (d != kD) return cudaErrorInvalidValue;
  const float scale = 1.0f / sqrtf(static_cast<float>(d));
  attention_masked_simt_kernel<T><<<batch * heads, kThreads, 0, stream>>>(
      q, k, v, token_stride, head_stride, ctx, attr_mask, cu_seqlens, word_idx, pos_row, heads, seq, scale);
  return cudaGetLastError();
}

template cudaError_t launch_attention_masked_simt<float>(const float*, const float*, const float*, long long,
                                                         long long, float*, const float*, const int*,
                                                         const int*, const int*, int, int, int, int,
                                                         cudaStream_t);
template cudaError_t launch_attention_masked_simt<__half>(const __half*, const __half*, const __half*,
                                                          long long, long long, __half*, const __half*,
                                                          const int*, const int*, const int*, int, int, int,
                                                          int, cudaStream_t);

template <typename T>
cudaError_t launch_attention_simt(const T* q, const T* k, const T* v, long long token_stride,
                                  long long head_stride, T* ctx, const int* cu_seqlens, int batch,
                                  int max_seq, int heads, int d, cudaStream_t stream) {
  if (batch <= 0 || heads <= 0) return cudaSuccess;
  if (d != kD) return cudaErrorInvalidValue;
  const float scale = 1.0f / sqrtf(static_cast<float>(d));
  attention_simt_kernel<T><<<batch * heads, kThreads, 0, stream>>>(
      q, k, v, token_stride, head_stride, ctx, cu_seqlens, heads, max_seq, scale);
  return cudaGetLastError();
}

template cudaError_t launch_attention_simt<float>(const float*, const float*, const float*,
                                                  long long, long long, float*, const int*, int,
                                                  int, int, int, cudaStream_t);
template cudaError_t launch_attention_simt<__half>(const __half*, const __half*, const __half*,
                                                   long long, long long, __half*, const int*, int,
                                                   int, int, int, cudaStream_t);

}  // namespace etb
