// CUDA-core self-attention on the packed, variable-length layout: one CTA per
// (sequence, head), one query row per thread, keys streamed through shared
// memory in blocks of 64 with an online softmax.  fp32 arithmetic throughout:
// this is the attention of the fp32 handle.  It replaces the padded batched
// GEMMs + softmax_kernel + transpose_rm_padding sequence of the reference
// (tf_op/bert_transformer_op.cu.cc:158-191, cuda/attention.cu:249-492); no
// padded position is loaded or computed.
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

}  // namespace

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
