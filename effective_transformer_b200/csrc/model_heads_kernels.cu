// The stages of the BERT model either side of the encoder stack, on the
// packed (padding-free) layout:
//   * embedding lookup + token-type row + position row + LayerNorm
//     (sample/tensorflow/modeling.py:380-521), evaluated for valid tokens only
//     and written straight into the packed [T, H] tensor, so the padded
//     [B, S, H] embedding output is never materialised.  The reference notes
//     that its padding removal "will be faster if placed in front of embedding"
//     (tf_op/bert_transformer_op.cu.cc:295-296); this is that placement.
//   * the pooler's first-token gather (modeling.py:224-229): row cu_seqlens[b]
//     of the packed tensor is the first token of sequence b.
// Both are pure HBM traffic: one warp per output row, 16-byte accesses.
#include "common.cuh"

namespace etb {

namespace {

constexpr int kThreads = 256;
constexpr int kCtasPerSm = 4;  // 64 registers x 256 threads: four CTAs are resident, the grid is one wave

__device__ __forceinline__ int clamp_tokens(const int* t_ptr, int max_tokens) {
  const int t = *t_ptr;
  return t < 0 ? 0 : (t > max_tokens ? max_tokens : t);
}

// out[v] = LN(word[ids[b,s]] + type[types[b,s]] + pos[s]) * gamma + beta for
// packed row v = (b, s).  An id outside its table contributes a zero row, as
// TensorFlow's GPU gather and one-hot matmul do.
template <typename T, int kVPL>
__global__ void __launch_bounds__(kThreads, (kVPL <= 4 ? kCtasPerSm : 1))
embedding_layernorm_kernel(const int* __restrict__ input_ids, const int* __restrict__ token_type_ids,
                           const int* __restrict__ batch_idx, const int* __restrict__ word_idx,
                           const int* __restrict__ t_ptr, const T* __restrict__ word_table, int vocab,
                           const T* __restrict__ type_table, int type_vocab,
                           const T* __restrict__ pos_table, const T* __restrict__ gamma,
                           const T* __restrict__ beta, T* __restrict__ out, int max_tokens, int seq,
                           int n, float eps) {
  pdl_wait();
  pdl_trigger();
  constexpr int E = VecTraits<T>::kElems;
  const int t = clamp_tokens(t_ptr, max_tokens);
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * (kThreads / 32);
  const int vpr = n / E;
  const float inv_n = 1.0f / static_cast<float>(n);

  // Row metadata (packed row -> position -> ids) is a chain of two dependent
  // loads; it is fetched one iteration ahead so that its latency hides behind
  // the row traffic of the current token.
  int id_n = -1, ty_n = -1, s_n = -1;
  auto fetch_meta = [&](int row) {
    id_n = ty_n = s_n = -1;
    if (row >= t) return;
    const int b = batch_idx[row], s = word_idx[row];
    const long long flat = static_cast<long long>(b) * seq + s;
    if (s < 0 || s >= seq || flat < 0 || flat >= max_tokens) return;  // corrupt index: zero rows
    s_n = s;
    id_n = input_ids[flat];
    ty_n = (type_table == nullptr) ? -1 : (token_type_ids == nullptr ? 0 : token_type_ids[flat]);
  };
  fetch_meta(warp);
  for (int row = warp; row < t; row += nwarps) {
    const int id = id_n, ty = ty_n, s = s_n;
    fetch_meta(row + nwarps);
    const T* wrow = (id >= 0 && id < vocab) ? word_table + static_cast<size_t>(id) * n : nullptr;
    const T* trow = (ty >= 0 && ty < type_vocab) ? type_table + static_cast<size_t>(ty) * n : nullptr;
    const T* prow = (pos_table != nullptr && s >= 0) ? pos_table + static_cast<size_t>(s) * n : nullptr;

    Vec16 vw[kVPL], vt[kVPL], vp[kVPL];
    const Vec16 zero = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int j = 0; j < kVPL; ++j) {
      const int c = j * 32 + lane;
      vw[j] = (c < vpr && wrow != nullptr) ? ld_global_nc_v4(wrow + c * E) : zero;
      vt[j] = (c < vpr && trow != nullptr) ? ld_global_v4(trow + c * E) : zero;
      vp[j] = (c < vpr && prow != nullptr) ? ld_global_v4(prow + c * E) : zero;
    }
    float x[kVPL][E];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kVPL; ++j) {
      float fw[E], ft[E], fp[E];
      VecTraits<T>::unpack(vw[j], fw);
      VecTraits<T>::unpack(vt[j], ft);
      VecTraits<T>::unpack(vp[j], fp);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        // the same association as the graph: (word + type) + position
        x[j][e] = (fw[e] + ft[e]) + fp[e];
        sum += x[j][e];
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
    T* orow = out + static_cast<size_t>(row) * n;
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
      }
    }
  }
}

// out[b] = packed[cu_seqlens[b]] for a sequence with tokens, a zero row for an
// empty one (the padded tensor the reference pools from holds zeros there,
// tf_op/bert_transformer_op.cu.cc:354-360).  One warp per sequence.  count_out
// (may be null) receives the number of rows written, for a GEMM that reads
// its row count from the device.
__global__ void __launch_bounds__(kThreads)
gather_first_tokens_kernel(const char* __restrict__ packed, const int* __restrict__ cu_seqlens,
                           char* __restrict__ out, int batch, int max_tokens, int row_bytes,
                           int* __restrict__ count_out) {
  pdl_wait();
  pdl_trigger();
  if (count_out != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *count_out = batch;
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * (kThreads / 32);
  const int nvec = row_bytes >> 4;
  const Vec16 zero = {0u, 0u, 0u, 0u};
  for (int b = warp; b < batch; b += nwarps) {
    const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1];
    const bool has = (hi > lo) && lo >= 0 && lo < max_tokens;
    const char* src = packed + static_cast<size_t>(has ? lo : 0) * row_bytes;
    char* dst = out + static_cast<size_t>(b) * row_bytes;
    for (int i = lane; i < nvec; i += 32)
      st_global_v4(dst + static_cast<size_t>(i) * 16,
                   has ? ld_global_nc_v4(src + static_cast<size_t>(i) * 16) : zero);
  }
}

}  // namespace

template <typename T>
cudaError_t launch_embedding_layernorm(const int* input_ids, const int* token_type_ids,
                                       const int* batch_idx, const int* word_idx, const int* t_ptr,
                                       const T* word_table, int vocab, const T* type_table,
                                       int type_vocab, const T* pos_table, const T* gamma,
                                       const T* beta, T* out, int batch, int seq, int n, float eps,
                                       cudaStream_t stream) {
  constexpr int E = VecTraits<T>::kElems;
  const long long max_tokens = static_cast<long long>(batch) * seq;
  if (max_tokens <= 0) return cudaSuccess;
  if (n <= 0 || n % E != 0 || max_tokens > 0x7fffffffLL) return cudaErrorInvalidValue;
  const int vpl = (n / E + 31) / 32;
  const long long rows_per_cta = kThreads / 32;
  long long ctas = (max_tokens + rows_per_cta - 1) / rows_per_cta;
  const long long cap = static_cast<long long>(sm_count()) * kCtasPerSm;
  if (ctas > cap) ctas = cap;
  const int grid = static_cast<int>(ctas);
  cudaError_t le = cudaSuccess;
#define ETB_EMB(V)                                                                                  \
  le = launch_pdl(embedding_layernorm_kernel<T, V>, dim3(grid), dim3(kThreads), 0, stream, input_ids, \
                  token_type_ids, batch_idx, word_idx, t_ptr, word_table, vocab, type_table, type_vocab, \
                  pos_table, gamma, beta, out, static_cast<int>(max_tokens), seq, n, eps)
  if (vpl <= 1) ETB_EMB(1);
  else if (vpl <= 2) ETB_EMB(2);
  else if (vpl <= 3) ETB_EMB(3);
  else if (vpl <= 4) ETB_EMB(4);
  else if (vpl <= 6) ETB_EMB(6);
  else if (vpl <= 8) ETB_EMB(8);
  else return cudaErrorInvalidValue;
#undef ETB_EMB
  return le;
}

cudaError_t launch_gather_first_tokens(const void* packed, const int* cu_seqlens, void* out, int batch,
                                       int max_tokens, int row_bytes, int* count_out,
                                       cudaStream_t stream) {
  if (batch <= 0) return cudaSuccess;
  if (row_bytes <= 0 || (row_bytes & 15) != 0) return cudaErrorInvalidValue;
  long long ctas = (batch + kThreads / 32 - 1) / (kThreads / 32);
  const long long cap = static_cast<long long>(sm_count()) * kCtasPerSm;
  if (ctas > cap) ctas = cap;
  return launch_pdl(gather_first_tokens_kernel, dim3(static_cast<int>(ctas)), dim3(kThreads), 0, stream,
                    static_cast<const char*>(packed), cu_seqlens, static_cast<char*>(out), batch, max_tokens,
                    row_bytes, count_out);
}

#define ETB_INST(T)                                                                               \
  template cudaError_t launch_embedding_layernorm<T>(const int*, const int*, const int*, const int*, \
                                                     const int*, const T*, int, const T*, int,    \
                                                     const T*, const T*, const T*, T*, int, int,  \
                                                     int, float, cudaStream_t);
ETB_INST(float)
ETB_INST(__half)
#undef ETB_INST

}  // namespace etb
