// CUDA-core GEMM: C[M,N] = epilogue(A[M,K] * W[K,N] (+ bias)), fp32 FMA
// accumulation.  It is the dense projection of the fp32 handle (true fp32, no
// TF32) and replaces the cublasGemmEx SGEMM call sites of the reference
// (tf_op/bert_transformer_op.cu.cc:110-141,200-240).  W is row-major [in,out]
// exactly as the reference passes it, so no repacking is needed.
// 128x128x8 tiles, 256 threads, 8x8 outputs per thread, register prefetch of
// the next k-slab.  M is read from device memory.
#include "common.cuh"

namespace etb {

namespace {

constexpr int BM = 128, BN = 128, BK = 8, kThreads = 256;

template <typename T>
struct Load4;
template <>
struct Load4<float> {
  __device__ static void ld(const float* p, float* f) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  __device__ static void st(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};
template <>
struct Load4<__half> {
  __device__ static void ld(const __half* p, float* f) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
  __device__ static void st(__half* p, const float* f) {
    __half2 a = __floats2half2_rn(f[0], f[1]), b = __floats2half2_rn(f[2], f[3]);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&a);
    v.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = v;
  }
};

template <typename T>
__global__ void __launch_bounds__(kThreads)
gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ W, const T* __restrict__ bias,
                 T* __restrict__ C, const int* __restrict__ m_ptr, int max_m, int N, int K,
                 int epilogue) {
  int M = *m_ptr;
  M = M < 0 ? 0 : (M > max_m ? max_m : M);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  if (m0 >= M) return;

  __shared__ __align__(16) float As[2][BK][BM];
  __shared__ __align__(16) float Bs[2][BK][BN];

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  // global -> smem assignments
  const int a_row = tid >> 1, a_k = (tid & 1) * 4;   // A tile 128 x 8
  const int b_k = tid >> 5, b_n = (tid & 31) * 4;    // W tile 8 x 128

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  float ra[4], rb[4];
  auto load_slab = [&](int k0) {
    const int gr = m0 + a_row, gk = k0 + a_k;
    if (gr < M && gk < K) Load4<T>::ld(A + static_cast<size_t>(gr) * K + gk, ra);
    else ra[0] = ra[1] = ra[2] = ra[3] = 0.f;
    const int gkb = k0 + b_k, gn = n0 + b_n;
    if (gkb < K && gn < N) Load4<T>::ld(W + static_cast<size_t>(gkb) * N + gn, rb);
    else rb[0] = rb[1] = rb[2] = rb[3] = 0.f;
  };
  auto store_slab = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 4; ++i) As[buf][a_k + i][a_row] = ra[i];
    *reinterpret_cast<float4*>(&Bs[buf][b_k][b_n]) = make_float4(rb[0], rb[1], rb[2], rb[3]);
  };

  load_slab(0);
  store_slab(0);
  __syncthreads();
  const int nslabs = (K + BK - 1) / BK;
  for (int s = 0; s < nslabs; ++s) {
    const int buf = s & 1;
    if (s + 1 < nslabs) load_slab((s + 1) * BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[8], b[8];
      *reinterpret_cast<float4*>(&a[0]) = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
      *reinterpret_cast<float4*>(&a[4]) = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
      *reinterpret_cast<float4*>(&b[0]) = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
      *reinterpret_cast<float4*>(&b[4]) = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (s + 1 < nslabs) {
      store_slab(buf ^ 1);
      __syncthreads();
    }
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (r >= M) continue;
#pragma unroll
    for (int jh = 0; jh < 2; ++jh) {
      const int c = n0 + jh * 64 + tx * 4;
      if (c >= N) continue;
      float o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = acc[i][jh * 4 + j];
      if (epilogue != kEpiNone) {
        float fb[4];
        Load4<T>::ld(bias + c, fb);
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] += fb[j];
        if (epilogue == kEpiBiasGelu) {
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = gelu_tanh(o[j]);
        } else if (epilogue == kEpiBiasTanh) {
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = tanhf(o[j]);
        }
      }
      Load4<T>::st(C + static_cast<size_t>(r) * N + c, o);
    }
  }
}

}  // namespace

template <typename T>
cudaError_t launch_gemm_simt(const T* a, const T* w, const T* bias, T* c, const int* m_ptr,
                             int max_m, int n, int k, int epilogue, cudaStream_t stream) {
  if (max_m <= 0 || n <= 0) return cudaSuccess;
  if ((n % 4) != 0 || (k % 4) != 0 || k <= 0) return cudaErrorInvalidValue;
  dim3 grid((n + BN - 1) / BN, (max_m + BM - 1) / BM);
  gemm_simt_kernel<T><<<grid, kThreads, 0, stream>>>(a, w, bias, c, m_ptr, max_m, n, k, epilogue);
  return cudaGetLastError();
}

template cudaError_t launch_gemm_simt<float>(const float*, const float*, const float*, float*,
                                             const int*, int, int, int, int, cudaStream_t);
template cudaError_t launch_gemm_simt<__half>(const __half*, const __half*, const __half*, __half*,
                                              const int*, int, int, int, int, cudaStream_t);

}  // namespace etb
