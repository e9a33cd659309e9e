// Tensor-core self-attention on the packed, variable-length layout (fp16 in,
// fp32 softmax and accumulation, fp16 out).  One CTA per (sequence, head);
// each of its 4 warps owns 16 query rows at a time; keys/values stream through
// shared memory in blocks of 64 with an online softmax, so only the len_b
// valid keys of a sequence are ever loaded or multiplied.  Replaces the padded
// cublasGemmStridedBatchedEx QK^T / P*V pair, softmax_kernel and
// transpose_rm_padding of the reference (tf_op/bert_transformer_op.cu.cc:
// 158-191, cuda/attention.cu:249-492): the context is written directly in the
// packed [T, heads*d] layout.
#include "common.cuh"

namespace etb {

namespace {

constexpr int kD = 64;
constexpr int kQBlock = 64;    // 4 warps x 16 rows
constexpr int kKBlock = 64;
constexpr int kLd = kD + 8;    // padded row (144 bytes): conflict-free ldmatrix
constexpr int kThreads = 128;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

struct TileSrc {
  __half (*dst)[kLd];
  const __half* src;
  int rows;
};
// Copies `rows` rows of 64 fp16 (128 bytes) into each padded 64-row shared
// tile and zero-fills the rest.  All global loads of all tiles are issued
// before the first shared-memory store, so one memory latency covers them.
template <int kTiles>
__device__ __forceinline__ void load_tiles(const TileSrc (&t)[kTiles], long long token_stride) {
  constexpr int kPerThread = 64 * 8 / kThreads;  // 16-byte vectors per thread and tile
  Vec16 v[kTiles][kPerThread];
#pragma unroll
  for (int i = 0; i < kTiles; ++i) {
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
      const int idx = threadIdx.x + j * kThreads;
      const int r = idx >> 3, c = idx & 7;
      v[i][j] = Vec16{0u, 0u, 0u, 0u};
      if (r < t[i].rows) v[i][j] = ld_global_nc_v4(t[i].src + static_cast<size_t>(r) * token_stride + c * 8);
    }
  }
#pragma unroll
  for (int i = 0; i < kTiles; ++i) {
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
      const int idx = threadIdx.x + j * kThreads;
      *reinterpret_cast<Vec16*>(&t[i].dst[idx >> 3][(idx & 7) * 8]) = v[i][j];
    }
  }
}

__global__ void __launch_bounds__(kThreads, 4)
attention_tc_kernel(const __half* __restrict__ q, const __half* __restrict__ k,
                    const __half* __restrict__ v, long long token_stride, long long head_stride,
                    __half* __restrict__ ctx, const int* __restrict__ cu_seqlens, int heads,
                    int max_seq, float scale_log2e) {
  const int b = blockIdx.x / heads, head = blockIdx.x % heads;
  const int lo = cu_seqlens[b];
  int len = cu_seqlens[b + 1] - lo;
  if (len <= 0) return;
  if (len > max_seq) len = max_seq;

  __shared__ __align__(16) __half Qs[kQBlock][kLd];
  __shared__ __align__(16) __half Ks[kKBlock][kLd];
  __shared__ __align__(16) __half Vs[kKBlock][kLd];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const size_t hoff = static_cast<size_t>(head) * head_stride;
  const int hidden = heads * kD;

  for (int q0 = 0; q0 < len; q0 += kQBlock) {
    const int nq = min(kQBlock, len - q0);
    __syncthreads();  // previous iteration's readers of the tiles are done
    {
      // the Q block together with the first K/V block
      const TileSrc first[3] = {
          {Qs, q + static_cast<size_t>(lo + q0) * token_stride + hoff, nq},
          {Ks, k + static_cast<size_t>(lo) * token_stride + hoff, min(kKBlock, len)},
          {Vs, v + static_cast<size_t>(lo) * token_stride + hoff, min(kKBlock, len)}};
      load_tiles<3>(first, token_stride);
    }
    __syncthreads();
    const bool warp_active = warp * 16 < nq;

    // Q fragments for this warp's 16 rows: 4 k-steps of 16 dims
    uint32_t qa[4][4];
    if (warp_active) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = kk * 16 + (lane >> 4) * 8;
        ldmatrix_x4(smem_addr(&Qs[r][c]), qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
      }
    }
    float o[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    for (int k0 = 0; k0 < len; k0 += kKBlock) {
      const int nk = min(kKBlock, len - k0);
      if (k0 > 0) {
        __syncthreads();  // previous block's readers of Ks/Vs are done
        const TileSrc next[2] = {{Ks, k + static_cast<size_t>(lo + k0) * token_stride + hoff, nk},
                                 {Vs, v + static_cast<size_t>(lo + k0) * token_stride + hoff, nk}};
        load_tiles<2>(next, token_stride);
        __syncthreads();
      }
      if (!warp_active) continue;

      // S = Q K^T : 16 x 64 scores as 8 n-tiles of 8 keys
      float s[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll
        for (int kk2 = 0; kk2 < 2; ++kk2) {
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(smem_addr(&Ks[n * 8 + (lane & 7)][kk2 * 32 + (lane >> 3) * 8]), b0, b1, b2, b3);
          mma_16816(s[n], qa[kk2 * 2], b0, b1);
          mma_16816(s[n], qa[kk2 * 2 + 1], b2, b3);
        }
      }
      // scale, mask keys beyond the sequence, running max
      float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = n * 8 + t4 * 2 + (e & 1);
          const float val = (key < nk) ? s[n][e] * scale_log2e : -INFINITY;
          s[n][e] = val;
          m_new[e >> 1] = fmaxf(m_new[e >> 1], val);
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
        m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
      }
      float corr[2], psum[2] = {0.f, 0.f};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        corr[h] = exp2f(m_run[h] - m_new[h]);  // first block: exp2(-inf) = 0
        m_run[h] = m_new[h];
      }
      uint32_t pa[4][4];  // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p[e] = exp2f(s[n][e] - m_new[e >> 1]);
          psum[e >> 1] += p[e];
        }
        pa[n >> 1][(n & 1) * 2 + 0] = pack_half2(p[0], p[1]);
        pa[n >> 1][(n & 1) * 2 + 1] = pack_half2(p[2], p[3]);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * corr[h] + psum[h];
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        o[n][0] *= corr[0];
        o[n][1] *= corr[0];
        o[n][2] *= corr[1];
        o[n][3] *= corr[1];
      }
      // O += P V : k over 64 keys (4 steps), n over 64 dims (8 tiles, two per ldmatrix)
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
        for (int n2 = 0; n2 < 4; ++n2) {
          uint32_t b0, b1, b2, b3;
          const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int c = n2 * 16 + (lane >> 4) * 8;
          ldmatrix_x4_trans(smem_addr(&Vs[r][c]), b0, b1, b2, b3);
          mma_16816(o[n2 * 2], pa[kk], b0, b1);
          mma_16816(o[n2 * 2 + 1], pa[kk], b2, b3);
        }
      }
    }

    if (warp_active) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + g + h * 8;
        if (row < nq) {
          const float inv = 1.0f / l_run[h];
          __half* op = ctx + static_cast<size_t>(lo + q0 + row) * hidden + head * kD + t4 * 2;
#pragma unroll
          for (int n = 0; n < 8; ++n) {
            *reinterpret_cast<uint32_t*>(op + n * 8) =
                pack_half2(o[n][h * 2] * inv, o[n][h * 2 + 1] * inv);
          }
        }
      }
    }
  }
}

}  // namespace

cudaError_t launch_attention_tc(const __half* q, const __half* k, const __half* v,
                                long long token_stride, long long head_stride, __half* ctx,
                                const int* cu_seqlens, int batch, int max_seq, int heads, int d,
                                int* status_word, cudaStream_t stream) {
  (void)status_word;
  if (batch <= 0 || heads <= 0) return cudaSuccess;
  if (d != kD || (token_stride % 8) != 0 || (head_stride % 8) != 0) return cudaErrorInvalidValue;
  const float scale_log2e = (1.0f / sqrtf(static_cast<float>(d))) * 1.4426950408889634f;
  attention_tc_kernel<<<batch * heads, kThreads, 0, stream>>>(
      q, k, v, token_stride, head_stride, ctx, cu_seqlens, heads, max_seq, scale_log2e);
  return cudaGetLastError();
}

}  // namespace etb
