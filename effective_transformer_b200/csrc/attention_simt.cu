// CUDA-core self-attention on the packed, variable-length layout: one CTA per
// (sequence, head, 64 queries), a 4 x 8 register block of scores and of outputs
// per thread, keys streamed through shared memory in blocks of 64 with an
// online softmax.  fp32 arithmetic throughout: this is the attention of the
// fp32 handle.  It replaces the padded batched
// GEMMs + softmax_kernel + transpose_rm_padding sequence of the reference
// (tf_op/bert_transformer_op.cu.cc:158-191, cuda/attention.cu:249-492); no
// padded position is loaded or computed.
// A second kernel evaluates the same block under a general [B, S, S] attention
// mask (any dtype of the handle), for callers whose mask is not the key-only
// tile of the input mask.
#include "common.cuh"

#include <mutex>

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

// Tile sizes of attention_simt_kernel: 64 queries x 64 keys per pass, rows of
// 68 floats in shared memory (16-byte aligned, and the stride spreads the rows
// that one warp reads over different banks).
constexpr int kQB = 64;
constexpr int kKB = 64;
constexpr int kPad = kD + 4;
constexpr int kSimtSmemBytes = (kQB + 2 * kKB) * kPad * static_cast<int>(sizeof(float));

// 4 consecutive elements of a row as fp32; kVec: one 16-byte (fp32) or 8-byte
// (fp16) access, for which the launcher has checked the alignment.
template <typename T, bool kVec>
__device__ __forceinline__ float4 load4(const T* p) {
  if constexpr (kVec && sizeof(T) == 4) {
    return *reinterpret_cast<const float4*>(p);
  } else if constexpr (kVec) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
  } else {
    return make_float4(to_f<T>(p[0]), to_f<T>(p[1]), to_f<T>(p[2]), to_f<T>(p[3]));
  }
}
template <typename T, bool kVec>
__device__ __forceinline__ void store4(T* p, float a, float b, float c, float d) {
  if constexpr (kVec && sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
  } else if constexpr (kVec) {
    uint2 u;
    *reinterpret_cast<__half2*>(&u.x) = __floats2half2_rn(a, b);
    *reinterpret_cast<__half2*>(&u.y) = __floats2half2_rn(c, d);
    *reinterpret_cast<uint2*>(p) = u;
  } else {
    p[0] = from_f<T>(a), p[1] = from_f<T>(b), p[2] = from_f<T>(c), p[3] = from_f<T>(d);
  }
}

// Scores of NI row groups x NJ key groups of one thread: s[i][j] += Q[ty+16i] . K[tx+8j].
// NI and NJ are compile-time so that groups beyond the sequence cost no issue slots.
template <int NI, int NJ>
__device__ __forceinline__ void score_groups(const float (*Qs)[kPad], const float (*Ks)[kPad], int ty, int tx,
                                             float (&s)[4][8]) {
#pragma unroll 1
  for (int c = 0; c < kD; c += 4) {
    float4 qv[NI], kv[NJ];
#pragma unroll
    for (int i = 0; i < NI; ++i) qv[i] = *reinterpret_cast<const float4*>(&Qs[ty + 16 * i][c]);
#pragma unroll
    for (int j = 0; j < NJ; ++j) kv[j] = *reinterpret_cast<const float4*>(&Ks[tx + 8 * j][c]);
#pragma unroll
    for (int i = 0; i < NI; ++i)
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        s[i][j] = fmaf(qv[i].x, kv[j].x, s[i][j]);
        s[i][j] = fmaf(qv[i].y, kv[j].y, s[i][j]);
        s[i][j] = fmaf(qv[i].z, kv[j].z, s[i][j]);
        s[i][j] = fmaf(qv[i].w, kv[j].w, s[i][j]);
      }
  }
}
template <int NI>
__device__ __forceinline__ void score_rows(const float (*Qs)[kPad], const float (*Ks)[kPad], int ty, int tx, int nj,
                                           float (&s)[4][8]) {
  switch ((nj + 1) >> 1) {  // key groups in pairs
    case 1: score_groups<NI, 2>(Qs, Ks, ty, tx, s); break;
    case 2: score_groups<NI, 4>(Qs, Ks, ty, tx, s); break;
    case 3: score_groups<NI, 6>(Qs, Ks, ty, tx, s); break;
    default: score_groups<NI, 8>(Qs, Ks, ty, tx, s); break;
  }
}
// o[i][:] += P[ty+16i][0..nk4) . V[0..nk4)[cols of this thread] for NI row groups.
template <int NI>
__device__ __forceinline__ void weighted_values(const float (*Ps)[kPad], const float (*Vs)[kPad], int ty, int tx,
                                                int nk4, float (&o)[4][8]) {
#pragma unroll 1
  for (int j0 = 0; j0 < nk4; j0 += 4) {
    float pv[NI][4];
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const float4 x = *reinterpret_cast<const float4*>(&Ps[ty + 16 * i][j0]);
      pv[i][0] = x.x, pv[i][1] = x.y, pv[i][2] = x.z, pv[i][3] = x.w;
    }
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const float4 va = *reinterpret_cast<const float4*>(&Vs[j0 + jj][4 * tx]);
      const float4 vb = *reinterpret_cast<const float4*>(&Vs[j0 + jj][32 + 4 * tx]);
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        const float pj = pv[i][jj];
        o[i][0] = fmaf(pj, va.x, o[i][0]);
        o[i][1] = fmaf(pj, va.y, o[i][1]);
        o[i][2] = fmaf(pj, va.z, o[i][2]);
        o[i][3] = fmaf(pj, va.w, o[i][3]);
        o[i][4] = fmaf(pj, vb.x, o[i][4]);
        o[i][5] = fmaf(pj, vb.y, o[i][5]);
        o[i][6] = fmaf(pj, vb.z, o[i][6]);
        o[i][7] = fmaf(pj, vb.w, o[i][7]);
      }
    }
  }
}

// cu_seqlens_k null: self-attention (keys and values are the sequence's own rows).  Otherwise
// cross-attention: sequence b's queries are rows [cu_seqlens[b], cu_seqlens[b+1]) of q and its
// keys / values rows [cu_seqlens_k[b], cu_seqlens_k[b+1]) of k / v, which have their own row
// stride (from_seq_len != to_seq_len of sample/tensorflow/modeling.py:558-752 on packed tensors).
// One CTA per (sequence, head, block of 64 queries), 128 threads.  Thread
// (ty, tx) = (tid / 8, tid % 8) owns the 4 x 8 block of scores with rows
// ty + 16 i and keys tx + 8 j, then the 4 x 8 block of the output with the same
// rows and columns 4 tx + {0..3}, 32 + 4 tx + {0..3}.  Q, K and V tiles sit in
// shared memory; the probabilities overwrite the K tile.  Keys are walked in
// blocks of 64 with an online softmax, so any sequence length works.  Row and
// key groups beyond the sequence's length are skipped (the bounds are uniform
// for the CTA).
template <typename T, bool kVec>
__global__ void __launch_bounds__(kThreads, 4)
attention_simt_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                      long long token_stride, long long head_stride, T* __restrict__ ctx, T* __restrict__ ctx_lo,
                      const int* __restrict__ cu_seqlens, int heads, int max_seq, float scale,
                      const int* __restrict__ cu_seqlens_k, long long kv_token_stride, int max_seq_k) {
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x / heads, head = blockIdx.x % heads;
  const int lo = cu_seqlens[b];
  int len = cu_seqlens[b + 1] - lo;
  if (len > max_seq) len = max_seq;  // corrupt bounds: stay inside the sequence budget
  const int q0 = blockIdx.y * kQB;
  if (q0 >= len) return;
  // the keys' rows: the sequence's own, or those of the other tensor
  int klo = lo, klen = len;
  if (cu_seqlens_k != nullptr) {
    klo = cu_seqlens_k[b];
    klen = cu_seqlens_k[b + 1] - klo;
    klen = klen < 0 ? 0 : (klen > max_seq_k ? max_seq_k : klen);
  }

  extern __shared__ __align__(16) float simt_smem[];
  float(*Qs)[kPad] = reinterpret_cast<float(*)[kPad]>(simt_smem);
  float(*Ks)[kPad] = reinterpret_cast<float(*)[kPad]>(simt_smem + kQB * kPad);  // then the probabilities
  float(*Vs)[kPad] = reinterpret_cast<float(*)[kPad]>(simt_smem + (kQB + kKB) * kPad);

  const size_t hoff = static_cast<size_t>(head) * head_stride;
  const int hidden = heads * kD;
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
  const int nq = min(kQB, len - q0);
  const int ni = (nq + 15) >> 4;  // row groups in use

  // A 64 x 64 tile is 8 accesses of 4 elements per thread.  All loads of a tile are issued
  // before the first store to shared memory, so that a thread waits for memory once per tile
  // and not once per access.
  constexpr int kPerThread = kQB * (kD / 4) / kThreads;
  auto load_tile = [&](const T* base, long long stride, int first_row, int nrows, float4 (&buf)[kPerThread]) {
#pragma unroll
    for (int it = 0; it < kPerThread; ++it) {
      const int idx = it * kThreads + threadIdx.x;
      const int row = idx >> 4, c = (idx & 15) * 4;
      buf[it] = make_float4(0.f, 0.f, 0.f, 0.f);  // rows past the sequence: finite values
      if (row < nrows) buf[it] = load4<T, kVec>(base + static_cast<size_t>(first_row + row) * stride + hoff + c);
    }
  };
  auto store_tile = [&](float(*dst)[kPad], const float4 (&buf)[kPerThread], float mul) {
#pragma unroll
    for (int it = 0; it < kPerThread; ++it) {
      const int idx = it * kThreads + threadIdx.x;
      const int row = idx >> 4, c = (idx & 15) * 4;
      *reinterpret_cast<float4*>(&dst[row][c]) =
          make_float4(buf[it].x * mul, buf[it].y * mul, buf[it].z * mul, buf[it].w * mul);
    }
  };
  {
    // Q tile and the first block of K and V: one round trip to memory
    float4 qb[kPerThread], kb[kPerThread], vb[kPerThread];
    const int nk0 = min(kKB, klen);
    load_tile(q, token_stride, lo + q0, nq, qb);
    load_tile(k, kv_token_stride, klo, nk0, kb);
    load_tile(v, kv_token_stride, klo, nk0, vb);
    store_tile(Qs, qb, scale);
    store_tile(Ks, kb, 1.0f);
    store_tile(Vs, vb, 1.0f);
  }

  float o[4][8], m[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) o[i][e] = 0.f;
  }

  auto load_keys = [&](int k0, int nk) {
    float4 kb[kPerThread], vb[kPerThread];
    load_tile(k, kv_token_stride, klo + k0, nk, kb);
    load_tile(v, kv_token_stride, klo + k0, nk, vb);
    store_tile(Ks, kb, 1.0f);
    store_tile(Vs, vb, 1.0f);
  };

  for (int k0 = 0; k0 < klen; k0 += kKB) {
    const int nk = min(kKB, klen - k0);
    const int nj = (nk + 7) >> 3;      // key groups in use
    const int nk4 = (nk + 3) & ~3;
    if (k0 > 0) {
      __syncthreads();  // the previous block's probabilities and V rows are no longer read
      load_keys(k0, nk);
    }
    __syncthreads();

    float s[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) s[i][j] = 0.f;
    switch (ni) {
      case 1: score_rows<1>(Qs, Ks, ty, tx, nj, s); break;
      case 2: score_rows<2>(Qs, Ks, ty, tx, nj, s); break;
      case 3: score_rows<3>(Qs, Ks, ty, tx, nj, s); break;
      default: score_rows<4>(Qs, Ks, ty, tx, nj, s); break;
    }
    // online softmax: the 8 lanes with the same ty hold one row's 64 scores
    float r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i >= ni) break;  // uniform for the CTA; the 8 lanes of a row stay together
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (tx + 8 * j >= nk) s[i][j] = -INFINITY;
        mx = fmaxf(mx, s[i][j]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      const float m_new = fmaxf(m[i], mx);  // finite: every block has at least one key
      r[i] = expf(m[i] - m_new);            // exp(-inf) = 0 for the first block
      m[i] = m_new;
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[i][j] = expf(s[i][j] - m_new);
        sum += s[i][j];
      }
      l[i] = l[i] * r[i] + sum;  // this lane's share of the row sum
#pragma unroll
      for (int e = 0; e < 8; ++e) o[i][e] *= r[i];
    }
    __syncthreads();  // every thread has read its K rows: the tile becomes the probabilities
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) Ks[ty + 16 * i][tx + 8 * j] = s[i][j];
    __syncthreads();

    switch (ni) {
      case 1: weighted_values<1>(Ks, Vs, ty, tx, nk4, o); break;
      case 2: weighted_values<2>(Ks, Vs, ty, tx, nk4, o); break;
      case 3: weighted_values<3>(Ks, Vs, ty, tx, nk4, o); break;
      default: weighted_values<4>(Ks, Vs, ty, tx, nk4, o); break;
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float sum = l[i];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    const int row = ty + 16 * i;
    if (row < nq) {
      const float inv = sum > 0.f ? 1.0f / sum : 0.f;  // no key at all (cross-attention onto an empty sequence): zeros
      const size_t off = static_cast<size_t>(lo + q0 + row) * hidden + head * kD;
#pragma unroll
      for (int e = 0; e < 8; ++e) o[i][e] *= inv;
      if constexpr (sizeof(T) == 4) {
        if (ctx_lo != nullptr) {
          // split for the fp32 output projection on the tensor cores: tf32 half to ctx, remainder to ctx_lo
          float rem[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float hi = rn_tf32(o[i][e]);
            rem[e] = o[i][e] - hi;
            o[i][e] = hi;
          }
          store4<T, kVec>(ctx_lo + off + 4 * tx, rem[0], rem[1], rem[2], rem[3]);
          store4<T, kVec>(ctx_lo + off + 32 + 4 * tx, rem[4], rem[5], rem[6], rem[7]);
        }
      }
      store4<T, kVec>(ctx + off + 4 * tx, o[i][0], o[i][1], o[i][2], o[i][3]);
      store4<T, kVec>(ctx + off + 32 + 4 * tx, o[i][4], o[i][5], o[i][6], o[i][7]);
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
                                  int max_seq, int heads, int d, cudaStream_t stream, T* ctx_lo,
                                  const int* cu_seqlens_k, long long kv_token_stride, int max_seq_k) {
  if (batch <= 0 || heads <= 0) return cudaSuccess;
  if (cu_seqlens_k == nullptr) {
    kv_token_stride = token_stride;
    max_seq_k = max_seq;
  }
  if (d != kD) return cudaErrorInvalidValue;
  const float scale = 1.0f / sqrtf(static_cast<float>(d));
  if (max_seq <= 0) return cudaSuccess;
  static PerDeviceOnce once;  // function attributes are per device
  const cudaError_t once_err = once.run([] {
    cudaError_t attr_err = cudaFuncSetAttribute(attention_simt_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSimtSmemBytes);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(attention_simt_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSimtSmemBytes);
    return attr_err;
  });
  if (once_err != cudaSuccess) return once_err;
  // four elements per access when every row segment starts on such a boundary
  const uintptr_t mask = 4 * sizeof(T) - 1;
  const bool vec = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                     reinterpret_cast<uintptr_t>(ctx) | reinterpret_cast<uintptr_t>(ctx_lo)) & mask) == 0 &&
                   token_stride % 4 == 0 && head_stride % 4 == 0 && kv_token_stride % 4 == 0;
  const dim3 grid(batch * heads, (max_seq + kQB - 1) / kQB);
  return vec ? launch_pdl(attention_simt_kernel<T, true>, grid, dim3(kThreads), kSimtSmemBytes, stream, q, k, v,
                          token_stride, head_stride, ctx, ctx_lo, cu_seqlens, heads, max_seq, scale, cu_seqlens_k,
                          kv_token_stride, max_seq_k)
             : launch_pdl(attention_simt_kernel<T, false>, grid, dim3(kThreads), kSimtSmemBytes, stream, q, k, v,
                          token_stride, head_stride, ctx, ctx_lo, cu_seqlens, heads, max_seq, scale, cu_seqlens_k,
                          kv_token_stride, max_seq_k);
}

template cudaError_t launch_attention_simt<float>(const float*, const float*, const float*,
                                                  long long, long long, float*, const int*, int,
                                                  int, int, int, cudaStream_t, float*, const int*, long long, int);
template cudaError_t launch_attention_simt<__half>(const __half*, const __half*, const __half*,
                                                   long long, long long, __half*, const int*, int,
                                                   int, int, int, cudaStream_t, __half*, const int*, long long, int);

}  // namespace etb
