// Self-attention of the fp32 handle on tensor cores at fp32 accuracy.
//
// The packed, variable-length layout and the tiling are those of the CUDA-core
// kernel (attention_simt.cu): one CTA per (sequence, head, 64 queries), Q, K and V
// tiles in shared memory, keys walked in blocks of 64 with an online softmax.  The
// two contractions of a block, S = Q K^T and O += P V, run as mma.sync m16n8k8
// with tf32 operands and fp32 accumulators, every fp32 operand split into
// x = hi + lo, hi = round_to_tf32(x), and the product taken as
// hi*hi + hi*lo + lo*hi (the lo*lo term is below fp32's last place), the same
// split the fp32 projections use (gemm_tf32x3.cu).  Chains are short here (64
// terms per accumulator and block), so the accumulators stay in the MMA.
// Replaces the padded batched GEMMs + softmax_kernel + transpose_rm_padding
// sequence of the reference (tf_op/bert_transformer_op.cu.cc:158-191,
// cuda/attention.cu:249-492) for OperationType FP32; no padded position is loaded
// or computed.  Warp w of the four owns query rows [16 w, 16 w + 16) of the tile.
#include "common.cuh"

namespace etb {

namespace {

constexpr int kD = 64;
constexpr int kQB = 64, kKB = 64;
constexpr int kThreads = 128;
constexpr int kPadQK = kD + 4;  // Q / K rows: the fragment reads of a warp hit 32 different banks
constexpr int kPadV = kD + 8;   // V rows are read down a column per fragment: 8 t + g is conflict-free
constexpr int kSmemBytes = ((kQB + kKB) * kPadQK + kKB * kPadV) * static_cast<int>(sizeof(float));

// D += A * B, m16n8k8, tf32 operands (the low 13 bits of an operand are ignored), fp32 accumulate.
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  const float h = rn_tf32(x);
  hi = __float_as_uint(h);
  lo = __float_as_uint(x - h);
}
// c += a * b at fp32 accuracy: three tf32 products
__device__ __forceinline__ void mma_3x(float (&c)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4],
                                       const uint32_t (&bh)[2], const uint32_t (&bl)[2]) {
  mma_tf32(c, al, bh);
  mma_tf32(c, ah, bl);
  mma_tf32(c, ah, bh);
}

template <bool kVec>
__global__ void __launch_bounds__(kThreads, 4)
attention_tf32x3_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                        long long token_stride, long long head_stride, float* __restrict__ ctx,
                        float* __restrict__ ctx_lo, const int* __restrict__ cu_seqlens, int heads, int max_seq,
                        float scale) {
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x / heads, head = blockIdx.x % heads;
  const int lo = cu_seqlens[b];
  int len = cu_seqlens[b + 1] - lo;
  if (len > max_seq) len = max_seq;  // corrupt bounds: stay inside the sequence budget
  const int q0 = blockIdx.y * kQB;
  if (q0 >= len) return;

  extern __shared__ __align__(16) float tf_smem[];
  float(*Qs)[kPadQK] = reinterpret_cast<float(*)[kPadQK]>(tf_smem);
  float(*Ks)[kPadQK] = reinterpret_cast<float(*)[kPadQK]>(tf_smem + kQB * kPadQK);  // then the probabilities
  float(*Vs)[kPadV] = reinterpret_cast<float(*)[kPadV]>(tf_smem + (kQB + kKB) * kPadQK);

  const size_t hoff = static_cast<size_t>(head) * head_stride;
  const int hidden = heads * kD;
  const int nq = min(kQB, len - q0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;  // fragment coordinates: group (row / column) and thread in group
  const int rw = 16 * warp;               // first tile row of this warp
  const bool active = rw < nq;            // rows past the sequence are not computed (the warp still syncs)

  // A 64 x 64 tile is 8 accesses of 4 elements per thread, all issued before the first store to
  // shared memory, so that a thread waits for memory once per tile.
  constexpr int kPerThread = kQB * (kD / 4) / kThreads;
  auto load_tile = [&](const float* base, int first_row, int nrows, float4 (&buf)[kPerThread]) {
#pragma unroll
    for (int it = 0; it < kPerThread; ++it) {
      const int idx = it * kThreads + threadIdx.x;
      const int row = idx >> 4, c = (idx & 15) * 4;
      buf[it] = make_float4(0.f, 0.f, 0.f, 0.f);  // rows past the sequence: zeros (their probabilities are zero too)
      if (row < nrows) {
        const float* p = base + static_cast<size_t>(first_row + row) * token_stride + hoff + c;
        if constexpr (kVec) buf[it] = *reinterpret_cast<const float4*>(p);
        else buf[it] = make_float4(p[0], p[1], p[2], p[3]);
      }
    }
  };
  auto store_tile = [&](auto dst, const float4 (&buf)[kPerThread], float mul) {
#pragma unroll
    for (int it = 0; it < kPerThread; ++it) {
      const int idx = it * kThreads + threadIdx.x;
      const int row = idx >> 4, c = (idx & 15) * 4;
      *reinterpret_cast<float4*>(&dst[row][c]) =
          make_float4(buf[it].x * mul, buf[it].y * mul, buf[it].z * mul, buf[it].w * mul);
    }
  };
  {
    float4 qb[kPerThread], kb[kPerThread], vb[kPerThread];
    const int nk0 = min(kKB, len);
    load_tile(q, lo + q0, nq, qb);
    load_tile(k, lo, nk0, kb);
    load_tile(v, lo, nk0, vb);
    store_tile(Qs, qb, scale);
    store_tile(Ks, kb, 1.0f);
    store_tile(Vs, vb, 1.0f);
  }

  // accumulator fragments: element (row g, columns 2t, 2t+1) in [0], [1] and (row g + 8, same columns) in [2], [3]
  float o[8][4];
#pragma unroll
  for (int nb = 0; nb < 8; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nb][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};  // rows g and g + 8

  for (int k0 = 0; k0 < len; k0 += kKB) {
    const int nk = min(kKB, len - k0);
    const int nkb = (nk + 7) >> 3;  // 8-key blocks in use (uniform for the CTA)
    if (k0 > 0) {
      __syncthreads();  // the previous block's probabilities and V rows are no longer read
      float4 kb[kPerThread], vb[kPerThread];
      load_tile(k, lo + k0, nk, kb);
      load_tile(v, lo + k0, nk, vb);
      store_tile(Ks, kb, 1.0f);
      store_tile(Vs, vb, 1.0f);
    }
    __syncthreads();

    float s[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nb][e] = 0.f;
    if (active) {
      // ---- S = Q K^T: 8 steps of 8 along the head dimension ----
#pragma unroll 2
      for (int ks = 0; ks < kD / 8; ++ks) {
        uint32_t ah[4], al[4];
        split_tf32(Qs[rw + g][ks * 8 + t], ah[0], al[0]);
        split_tf32(Qs[rw + g + 8][ks * 8 + t], ah[1], al[1]);
        split_tf32(Qs[rw + g][ks * 8 + t + 4], ah[2], al[2]);
        split_tf32(Qs[rw + g + 8][ks * 8 + t + 4], ah[3], al[3]);
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
          if (nb < nkb) {
            uint32_t bh[2], bl[2];
            split_tf32(Ks[nb * 8 + g][ks * 8 + t], bh[0], bl[0]);
            split_tf32(Ks[nb * 8 + g][ks * 8 + t + 4], bh[1], bl[1]);
            mma_3x(s[nb], ah, al, bh, bl);
          }
        }
      }
      // ---- online softmax: the four lanes of a group hold one row's 64 scores ----
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float mx = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            if (nb * 8 + 2 * t + e >= nk) s[nb][2 * hh + e] = -INFINITY;
            mx = fmaxf(mx, s[nb][2 * hh + e]);
          }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m[hh], mx);  // finite: every block has at least one key
        const float r = expf(m[hh] - m_new);   // exp(-inf) = 0 for the first block
        m[hh] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float p = expf(s[nb][2 * hh + e] - m_new);
            s[nb][2 * hh + e] = p;
            sum += p;
          }
        l[hh] = l[hh] * r + sum;  // this lane's share of the row sum
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
          o[nb][2 * hh] *= r;
          o[nb][2 * hh + 1] *= r;
        }
      }
    }
    __syncthreads();  // every warp has read its K fragments: the tile becomes the probabilities
    if (active) {
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
        *reinterpret_cast<float2*>(&Ks[rw + g][nb * 8 + 2 * t]) = make_float2(s[nb][0], s[nb][1]);
        *reinterpret_cast<float2*>(&Ks[rw + g + 8][nb * 8 + 2 * t]) = make_float2(s[nb][2], s[nb][3]);
      }
      __syncwarp();  // a warp reads back only the probability rows it wrote itself
      // ---- O += P V: one step per 8 keys, 8 blocks of 8 output columns ----
#pragma unroll 2
      for (int ks = 0; ks < nkb; ++ks) {
        uint32_t ph[4], pl[4];
        split_tf32(Ks[rw + g][ks * 8 + t], ph[0], pl[0]);
        split_tf32(Ks[rw + g + 8][ks * 8 + t], ph[1], pl[1]);
        split_tf32(Ks[rw + g][ks * 8 + t + 4], ph[2], pl[2]);
        split_tf32(Ks[rw + g + 8][ks * 8 + t + 4], ph[3], pl[3]);
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
          uint32_t vh[2], vl[2];
          split_tf32(Vs[ks * 8 + t][nb * 8 + g], vh[0], vl[0]);
          split_tf32(Vs[ks * 8 + t + 4][nb * 8 + g], vh[1], vl[1]);
          mma_3x(o[nb], ph, pl, vh, vl);
        }
      }
    }
  }

  if (!active) return;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    float sum = l[hh];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const int row = rw + g + 8 * hh;
    if (row < nq) {
      const float inv = 1.0f / sum;
      const size_t off = static_cast<size_t>(lo + q0 + row) * hidden + head * kD + 2 * t;
#pragma unroll
      for (int nb = 0; nb < 8; ++nb) {
        float a = o[nb][2 * hh] * inv, c = o[nb][2 * hh + 1] * inv;
        if (ctx_lo != nullptr) {
          // split for the fp32 output projection on the tensor cores: tf32 half to ctx, remainder to ctx_lo
          const float ah = rn_tf32(a), ch = rn_tf32(c);
          if constexpr (kVec) *reinterpret_cast<float2*>(ctx_lo + off + nb * 8) = make_float2(a - ah, c - ch);
          else ctx_lo[off + nb * 8] = a - ah, ctx_lo[off + nb * 8 + 1] = c - ch;
          a = ah, c = ch;
        }
        if constexpr (kVec) *reinterpret_cast<float2*>(ctx + off + nb * 8) = make_float2(a, c);
        else ctx[off + nb * 8] = a, ctx[off + nb * 8 + 1] = c;
      }
    }
  }
}

}  // namespace

cudaError_t launch_attention_tf32x3(const float* q, const float* k, const float* v, long long token_stride,
                                    long long head_stride, float* ctx, const int* cu_seqlens, int batch,
                                    int max_seq, int heads, int d, cudaStream_t stream, float* ctx_lo) {
  if (batch <= 0 || heads <= 0 || max_seq <= 0) return cudaSuccess;
  if (d != kD) return cudaErrorInvalidValue;
  static PerDeviceOnce once;  // function attributes are per device
  const cudaError_t once_err = once.run([] {
    cudaError_t e = cudaFuncSetAttribute(attention_tf32x3_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_tf32x3_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kSmemBytes);
    return e;
  });
  if (once_err != cudaSuccess) return once_err;
  const float scale = 1.0f / sqrtf(static_cast<float>(d));
  // 16-byte row segments for the tile loads, 8-byte pairs for the stores
  const bool vec = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                     reinterpret_cast<uintptr_t>(ctx) | reinterpret_cast<uintptr_t>(ctx_lo)) & 15u) == 0 &&
                   token_stride % 4 == 0 && head_stride % 4 == 0;
  const dim3 grid(batch * heads, (max_seq + kQB - 1) / kQB);
  return vec ? launch_pdl(attention_tf32x3_kernel<true>, grid, dim3(kThreads), kSmemBytes, stream, q, k, v,
                          token_stride, head_stride, ctx, ctx_lo, cu_seqlens, heads, max_seq, scale)
             : launch_pdl(attention_tf32x3_kernel<false>, grid, dim3(kThreads), kSmemBytes, stream, q, k, v,
                          token_stride, head_stride, ctx, ctx_lo, cu_seqlens, heads, max_seq, scale);
}

}  // namespace etb
