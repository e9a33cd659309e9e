// Tensor-core self-attention on the packed, variable-length layout (fp16 in,
// fp32 softmax and accumulation, fp16 out).  Replaces the padded
// cublasGemmStridedBatchedEx QK^T / P*V pair, softmax_kernel and
// transpose_rm_padding of the reference (tf_op/bert_transformer_op.cu.cc:
// 158-191, cuda/attention.cu:249-492): the context is written directly in the
// packed [T, heads*d] layout and only the valid keys of a sequence are ever
// loaded or multiplied.
//
// Persistent CTAs walk over (sequence, head) work items.  One thread feeds a
// double-buffered shared-memory area with TMA: 16-row x 64-column boxes
// (128-byte swizzle) of the item's Q, K and V rows, completion counted on an
// mbarrier, so the NEXT item streams in while the four warps compute the
// current one (16 query rows per warp, ldmatrix + mma.sync m16n8k16, online
// softmax in the exp2 domain).  Sequences longer than 64 tokens are processed
// in 64-row query blocks and 64-key blocks.  Every mbarrier wait is bounded.
#include "common.cuh"
#include "ptx_sm100.cuh"

#include <mutex>

namespace etb {

namespace {

using namespace ptx;

constexpr int kD = 64;
constexpr int kBlock = 64;          // query rows / keys per block (4 warps x 16 rows)
constexpr int kBoxRows = 16;        // rows per TMA box
constexpr int kBoxBytes = kBoxRows * kD * 2;   // 2048
constexpr int kTileBytes = kBlock * kD * 2;    // 8192: 64 rows of 128 bytes, swizzled
constexpr int kBufBytes = 3 * kTileBytes;      // Q, K, V
constexpr int kThreads = 128;
constexpr int kCtasPerSm = 4;
constexpr int kSmemBytes = 2 * kBufBytes + 64;  // two buffers + barriers

enum Site : int { kSiteItem = 1, kSiteBlock = 2, kSiteSmemAlign = 3 };

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
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void st_shared_zero16(uint32_t addr) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(addr), "r"(0u) : "memory");
}

struct Item {
  int lo, len, head;
};

// How (token, head) maps to TMA coordinates: x = head * x_per_head,
// y = head * y_per_head + token.
struct Coords {
  int x_per_head, y_per_head;
};

__global__ void __launch_bounds__(kThreads, kCtasPerSm)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, Coords co, __half* __restrict__ ctx,
                    const int* __restrict__ cu_seqlens, int batch, int heads, int max_seq,
                    float scale_log2e, int* status_word) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if ((base & 1023u) != 0u) {
    if (threadIdx.x == 0) report_timeout(status_word, kKernelAttnTc, kSiteSmemAlign);
    return;
  }
  const uint32_t bar0 = base + 2 * kBufBytes;          // full[0], full[1], block barrier
  const uint32_t block_bar = bar0 + 16;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + 2 * kBufBytes + 32);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const uint32_t sw = static_cast<uint32_t>(lane & 7);  // swizzle term of every ldmatrix row of this lane
  const int hidden = heads * kD;
  const int total = batch * heads;
  int i = blockIdx.x;
  if (i >= total) return;

  if (threadIdx.x == 0) {
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    mbar_init(block_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
  }
  __syncthreads();

  auto get_item = [&](int idx) {
    Item it;
    const int b = idx / heads;
    it.head = idx - b * heads;
    it.lo = cu_seqlens[b];
    const int len = cu_seqlens[b + 1] - it.lo;
    it.len = len < 0 ? 0 : (len > max_seq ? max_seq : len);
    return it;
  };
  // Thread 0: Q block q0 (optional) and K/V block k0 of an item -> buffer at
  // `buf_addr`, completion on `bar`.  An empty item still arrives once.
  auto issue = [&](const Item& it, uint32_t buf_addr, int q0, int k0, bool with_q, uint32_t bar) {
    const int bq = (with_q && it.len > q0) ? (min(kBlock, it.len - q0) + kBoxRows - 1) / kBoxRows : 0;
    const int bk = it.len > k0 ? (min(kBlock, it.len - k0) + kBoxRows - 1) / kBoxRows : 0;
    mbar_arrive_expect_tx(bar, static_cast<uint32_t>((bq + 2 * bk) * kBoxBytes));
    const int x = it.head * co.x_per_head, y = it.head * co.y_per_head + it.lo;
    for (int j = 0; j < bq; ++j)
      tma_load_2d(buf_addr + j * kBoxBytes, &tmap_q, x, y + q0 + j * kBoxRows, bar);
    for (int j = 0; j < bk; ++j) {
      tma_load_2d(buf_addr + kTileBytes + j * kBoxBytes, &tmap_k, x, y + k0 + j * kBoxRows, bar);
      tma_load_2d(buf_addr + 2 * kTileBytes + j * kBoxBytes, &tmap_v, x, y + k0 + j * kBoxRows, bar);
    }
  };

  Item cur = get_item(i);
  if (threadIdx.x == 0) issue(cur, base, 0, 0, true, bar0);
  uint32_t block_phase = 0;
  bool ok = true;

  for (int it_n = 0; i < total && ok; i += gridDim.x, ++it_n) {
    const int buf = it_n & 1;
    const uint32_t tq = base + buf * kBufBytes, tk = tq + kTileBytes, tv = tk + kTileBytes;
    const int inext = i + gridDim.x;
    Item nxt{0, 0, 0};
    if (inext < total) {
      nxt = get_item(inext);
      if (threadIdx.x == 0) issue(nxt, base + (buf ^ 1) * kBufBytes, 0, 0, true, bar0 + 8 * (buf ^ 1));
    }
    if (!mbar_wait(bar0 + 8 * buf, static_cast<uint32_t>((it_n >> 1) & 1), abort_flag)) {
      *abort_flag = 1;
      report_timeout(status_word, kKernelAttnTc, kSiteItem);
      ok = false;
    }
    ok = __syncthreads_and(ok);
    if (!ok) break;

    const int len = cur.len;
    for (int q0 = 0; q0 < len && ok; q0 += kBlock) {
      const int nq = min(kBlock, len - q0);
      if (q0 > 0) {
        // long sequence: fetch the next query block and restart at key block 0
        __syncthreads();
        if (threadIdx.x == 0) {
          fence_proxy_async_smem();
          issue(cur, tq, q0, 0, true, block_bar);
        }
        if (!mbar_wait(block_bar, block_phase, abort_flag)) {
          *abort_flag = 1;
          report_timeout(status_word, kKernelAttnTc, kSiteBlock);
          ok = false;
        }
        block_phase ^= 1u;
        ok = __syncthreads_and(ok);
        if (!ok) break;
      }
      const bool warp_active = warp * 16 < nq;

      uint32_t qa[4][4];  // Q fragments of this warp's 16 rows: 4 k-steps of 16 dims
      if (warp_active) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint32_t c = static_cast<uint32_t>(kk * 2 + (lane >> 4));
          ldmatrix_x4(tq + r * 128 + ((c ^ sw) << 4), qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
        }
      }
      float o[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
      float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

      for (int k0 = 0; k0 < len && ok; k0 += kBlock) {
        const int nk = min(kBlock, len - k0);
        if (k0 > 0) {
          __syncthreads();  // readers of the previous key block are done
          if (threadIdx.x == 0) {
            fence_proxy_async_smem();
            issue(cur, tq, q0, k0, false, block_bar);
          }
          if (!mbar_wait(block_bar, block_phase, abort_flag)) {
            *abort_flag = 1;
            report_timeout(status_word, kKernelAttnTc, kSiteBlock);
            ok = false;
          }
          block_phase ^= 1u;
          ok = __syncthreads_and(ok);
          if (!ok) break;
        }
        if (!warp_active) continue;

        // The last box may carry rows of the next sequence (or stale rows past the
        // last token): zero the V rows [nk, next multiple of 16) so that P = 0
        // meets a finite value there.  Every warp does it for itself.
        {
          const int pad = ((nk + 15) & ~15) - nk;
          for (int idx = lane; idx < pad * 8; idx += 32)
            st_shared_zero16(tv + (nk + (idx >> 3)) * 128 + ((idx & 7) << 4));
          __syncwarp();
        }

        // S = Q K^T : 16 x 64 scores as 8 n-tiles of 8 keys (tiles past nk are skipped)
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
          if (n * 8 < nk) {
            const int r = n * 8 + (lane & 7);
#pragma unroll
            for (int kk2 = 0; kk2 < 2; ++kk2) {
              uint32_t b0, b1, b2, b3;
              const uint32_t c = static_cast<uint32_t>(kk2 * 4 + (lane >> 3));
              ldmatrix_x4(tk + r * 128 + ((c ^ sw) << 4), b0, b1, b2, b3);
              mma_16816(s[n], qa[kk2 * 2], b0, b1);
              mma_16816(s[n], qa[kk2 * 2 + 1], b2, b3);
            }
          }
        }
        // mask keys beyond the sequence (only the last, partial n-tile has any), raw running max
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          if (n * 8 < nk) {
            if (n * 8 + 8 > nk) {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (n * 8 + t4 * 2 + (e & 1) >= nk) s[n][e] = -INFINITY;
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) m_new[e >> 1] = fmaxf(m_new[e >> 1], s[n][e]);
          }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
          m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
        }
        // p = 2^((s - m) * scale * log2(e)) as one FMA + one ex2 per score
        const float ms[2] = {-m_new[0] * scale_log2e, -m_new[1] * scale_log2e};
        float psum[2] = {0.f, 0.f};
        uint32_t pa[4][4];  // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          float p[4] = {0.f, 0.f, 0.f, 0.f};
          if (n * 8 < nk) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              p[e] = ex2_approx(fmaf(s[n][e], scale_log2e, ms[e >> 1]));
              psum[e >> 1] += p[e];
            }
          }
          pa[n >> 1][(n & 1) * 2 + 0] = pack_half2(p[0], p[1]);
          pa[n >> 1][(n & 1) * 2 + 1] = pack_half2(p[2], p[3]);
        }
        if (k0 > 0) {
          // rescale what earlier key blocks accumulated
          float corr[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            corr[h] = ex2_approx((m_run[h] - m_new[h]) * scale_log2e);
            l_run[h] *= corr[h];
          }
#pragma unroll
          for (int n = 0; n < 8; ++n) {
            o[n][0] *= corr[0];
            o[n][1] *= corr[0];
            o[n][2] *= corr[1];
            o[n][3] *= corr[1];
          }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          l_run[h] += psum[h];
          m_run[h] = m_new[h];
        }
        // O += P V : k over the keys (16 per step, steps past nk skipped), n over 64 dims
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          if (kk * 16 < nk) {
            const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
            for (int n2 = 0; n2 < 4; ++n2) {
              uint32_t b0, b1, b2, b3;
              const uint32_t c = static_cast<uint32_t>(n2 * 2 + (lane >> 4));
              ldmatrix_x4_trans(tv + r * 128 + ((c ^ sw) << 4), b0, b1, b2, b3);
              mma_16816(o[n2 * 2], pa[kk], b0, b1);
              mma_16816(o[n2 * 2 + 1], pa[kk], b2, b3);
            }
          }
        }
      }

      if (warp_active && ok) {
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
            __half* op = ctx + static_cast<size_t>(cur.lo + q0 + row) * hidden + cur.head * kD + t4 * 2;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
              *reinterpret_cast<uint32_t*>(op + n * 8) =
                  pack_half2(o[n][h * 2] * inv, o[n][h * 2 + 1] * inv);
            }
          }
        }
      }
    }
    __syncthreads();  // this buffer is refilled two items from now
    if (threadIdx.x == 0) fence_proxy_async_smem();
    cur = nxt;
  }
}

}  // namespace

cudaError_t launch_attention_tc(const __half* q, const __half* k, const __half* v,
                                long long token_stride, long long head_stride, __half* ctx,
                                const int* cu_seqlens, int batch, int max_seq, int max_tokens, int heads,
                                int d, int* status_word, cudaStream_t stream, TensorMapCache* maps) {
  if (batch <= 0 || heads <= 0 || max_tokens <= 0) return cudaSuccess;
  if (d != kD || token_stride < kD || (token_stride % 8) != 0 || (head_stride % 8) != 0 || head_stride < 0)
    return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15u)
    return cudaErrorMisalignedAddress;
  // Two layouts: heads side by side inside a token row (x moves with the head),
  // or one [max_tokens, 64] block per head (y moves with the head).
  Coords co;
  uint64_t cols, rows;
  if (static_cast<long long>(heads - 1) * head_stride + kD <= token_stride) {
    co = {static_cast<int>(head_stride), 0};
    cols = static_cast<uint64_t>(heads - 1) * head_stride + kD;
    rows = static_cast<uint64_t>(max_tokens);
  } else if (token_stride == kD && head_stride % token_stride == 0 && head_stride / token_stride >= max_tokens) {
    co = {0, static_cast<int>(head_stride / token_stride)};
    cols = kD;
    rows = static_cast<uint64_t>(heads - 1) * (head_stride / token_stride) + max_tokens;
  } else {
    return cudaErrorInvalidValue;
  }
  CUtensorMap tq, tk, tv;
  if (!encode_2d_fp16_sw128(&tq, q, rows, cols, static_cast<uint64_t>(token_stride), kBoxRows, kD, maps) ||
      !encode_2d_fp16_sw128(&tk, k, rows, cols, static_cast<uint64_t>(token_stride), kBoxRows, kD, maps) ||
      !encode_2d_fp16_sw128(&tv, v, rows, cols, static_cast<uint64_t>(token_stride), kBoxRows, kD, maps))
    return cudaErrorInvalidValue;
  static PerDeviceOnce once;  // function attributes are per device
  const cudaError_t once_err = once.run([] {
    cudaError_t attr_err = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBytes);
    return attr_err;
  });
  if (once_err != cudaSuccess) return once_err;
  const float scale_log2e = (1.0f / sqrtf(static_cast<float>(d))) * 1.4426950408889634f;
  const long long total = static_cast<long long>(batch) * heads;
  long long grid = static_cast<long long>(sm_count()) * kCtasPerSm;
  if (grid > total) grid = total;
  attention_tc_kernel<<<static_cast<int>(grid), kThreads, kSmemBytes, stream>>>(
      tq, tk, tv, co, ctx, cu_seqlens, batch, heads, max_seq, scale_log2e, status_word);
  return cudaGetLastError();
}

}  // namespace etb
