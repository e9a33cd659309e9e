// Self-attention on the packed, variable-length layout with the 5th-generation
// tensor cores (fp16 in, fp32 scores/softmax/accumulation, fp16 out), for
// sequences of up to 128 tokens.  Replaces the padded batched QK^T / softmax /
// P*V / transpose_rm_padding sequence of the reference
// (tf_op/bert_transformer_op.cu.cc:158-191, cuda/attention.cu:249-492).
//
// Whole sequences are packed greedily into tiles of at most 128 consecutive
// token rows (attention_plan_kernel, once per batch).  One work item is a
// (tile, head) pair:
//   TMA        Q, K, V rows of the tile -> shared memory (128-byte swizzle)
//   tcgen05    S = Q K^T, M = 128, N = rows rounded to 16, into TMEM
//   softmax    one thread per query row reads its row from TMEM, keeps only
//              the columns of its own sequence (block-diagonal mask), writes
//              P (fp16) to shared memory in the K-major operand layout
//   tcgen05    O = P V (V is the MN-major B operand), into TMEM
//   epilogue   O / rowsum -> fp16 -> packed context [T, heads*64]
// Keys of other sequences contribute exact zeros; padded positions do not
// exist in this layout at all.  Four CTAs per SM overlap the phases of four
// items.  Every mbarrier wait is bounded.
#include "common.cuh"
#include "ptx_sm100.cuh"

#include <mutex>

namespace etb {

namespace {

using namespace ptx;

constexpr int kD = 64;
constexpr int kTileRows = 128;
constexpr int kBoxRows = 32;
constexpr int kBoxBytes = kBoxRows * kD * 2;        // 4096
constexpr int kTileBytes = kTileRows * kD * 2;      // 16384: 128 rows of 128 bytes
constexpr int kThreads = 128;
// TMEM columns of a CTA: S in [0,128); the softmax overwrites it in place with P (fp16 pairs,
// columns [0,64): the pair of keys 2j, 2j+1 lands in column j, which it has already read), and
// O goes to [64,128) once every row has consumed its scores.
constexpr int kTmemCols = 128;
constexpr int kPCol = 0;
constexpr int kOCol = 64;
constexpr int kCtasPerSm = 4;    // 4 x 128 TMEM columns, 4 x 48 KB shared memory
// One {Q, K, V} buffer + barriers.  P never touches shared memory (it is the TMEM A operand
// of the second MMA), so the Q and K tiles are free as soon as S = Q K^T has completed and the
// V tile as soon as O = P V has: the next item's Q/K rows are loaded under this item's softmax
// and second MMA, its V rows under the epilogue and the next item's first MMA and softmax.
// Four CTAs per SM keep the phases of four items in flight.
constexpr int kBufBytes = 3 * kTileBytes;
constexpr int kSmemBytes = kBufBytes + 64;

enum Site : int { kSiteLoad = 1, kSiteScores = 2, kSiteContext = 3, kSiteSmemAlign = 4 };

// 32 lanes x 16 columns of 32-bit: thread i of the warp writes TMEM lane (lane field) + i.
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows = lanes, two fp16 per 32-bit column)
// is read from tensor memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
// kind::f16 instruction descriptor, fp32 accumulate, A K-major; B K-major or MN-major.
__device__ __forceinline__ uint32_t idesc_f16(int m, int n, bool b_mn_major) {
  return (1u << 4) | (b_mn_major ? (1u << 16) : 0u) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// Layout of the plan in device memory (ints):
//   [0] number of tiles   [4, 4+B) first token row of tile i   [4+B, 4+2B) rows of tile i
//   [4+2B, 4+2B+cap) first token of the sequence that owns token t   [.., +cap) one past its last token
//   [4+2B+2cap, +B+1) scratch of the planning kernel (first sequence of tile i)
__host__ __device__ inline size_t plan_ints(int batch, int max_tokens) {
  return 4 + 3 * static_cast<size_t>(batch) + 1 + 2 * static_cast<size_t>(max_tokens);
}

// One CTA: packs whole sequences greedily into tiles of <= 128 rows, then
// labels every token with its sequence's token range.
__global__ void attention_plan_kernel(const int* __restrict__ cu_seqlens, int batch, int max_tokens,
                                      int* __restrict__ plan) {
  pdl_wait();
  pdl_trigger();
  int* tile_start = plan + 4;
  int* tile_rows = plan + 4 + batch;
  int* seq_lo = plan + 4 + 2 * batch;
  int* seq_hi = seq_lo + max_tokens;
  // Greedy packing = following a chain: a tile that starts with sequence b ends
  // before next(b), the first sequence whose last token lies more than 128 rows
  // behind the tile's first token.  next() is found for every b in parallel (a
  // binary search over the sorted boundaries); only the walk along the chain,
  // one step per tile, is sequential.
  constexpr int kSharedSeqs = 8192;
  __shared__ int s_next[kSharedSeqs];
  int* next = batch <= kSharedSeqs ? s_next : seq_hi;   // larger batches: global scratch (slower walk)
  const bool scratch_ok = batch <= kSharedSeqs || batch <= max_tokens;
  auto cu = [&](int b) { return min(cu_seqlens[b], max_tokens); };
  if (scratch_ok) {
    for (int b = threadIdx.x; b < batch; b += blockDim.x) {
      const int limit = cu(b) + kTileRows;
      int lo_b = b, hi_b = batch;  // first j in [b, batch] with cu(j + 1) > limit (batch if none)
      while (lo_b < hi_b) {
        const int mid = (lo_b + hi_b) >> 1;
        if (cu(mid + 1) > limit) hi_b = mid; else lo_b = mid + 1;
      }
      next[b] = lo_b > b ? lo_b : b + 1;  // a sequence longer than a tile still advances
    }
  }
  __syncthreads();
  int* tile_seq = seq_hi + max_tokens;   // first sequence of every tile, then one end marker
  __shared__ int s_nt;
  if (threadIdx.x == 0) {
    // the sequential part touches shared memory only (plus fire-and-forget stores)
    int nt = 0;
    for (int b = 0; b < batch;) {
      int e;
      if (scratch_ok) {
        e = next[b];
      } else {
        const int limit = cu(b) + kTileRows;
        e = b;
        while (e < batch && cu(e + 1) <= limit) ++e;
        if (e == b) e = b + 1;
      }
      tile_seq[nt++] = b;
      b = e;
    }
    tile_seq[nt] = batch;
    s_nt = nt;
  }
  __syncthreads();
  {
    int nt = s_nt;
    for (int i = threadIdx.x; i < nt; i += blockDim.x) {
      const int first = cu(tile_seq[i]);
      int rows = cu(tile_seq[i + 1]) - first;
      rows = rows > kTileRows ? kTileRows : rows;  // longer sequences are not handled by this kernel
      tile_start[i] = first;
      tile_rows[i] = rows;
    }
    // only the last tile can be empty (nothing but empty sequences at the end of the batch)
    if (threadIdx.x == 0) {
      if (nt > 0 && cu(batch) - cu(tile_seq[nt - 1]) <= 0) --nt;
      plan[0] = nt;
    }
  }
  __syncthreads();  // next[] is dead: seq_hi may be written
  // one warp per sequence, lanes over its tokens: the label stores are coalesced
  // (a thread per sequence scatters 32 lines per store instruction and made this
  // loop the longest part of the kernel)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int b = warp; b < batch; b += nwarps) {
    int lo = cu_seqlens[b], hi = cu_seqlens[b + 1];
    lo = lo < 0 ? 0 : lo;
    hi = hi > max_tokens ? max_tokens : hi;
    for (int t = lo + lane; t < hi; t += 32) {
      seq_lo[t] = lo;
      seq_hi[t] = hi;
    }
  }
}

struct Coords {
  int x_per_head, y_per_head;  // TMA coordinates: x = head * x_per_head, y = head * y_per_head + token
};

// General [B, S, S] attention mask (kMask kernels): attr_mask[b][q][k] > 0.5 = query position q of
// sequence b may attend to key position k; batch_idx / word_idx give the sequence and the position of
// every packed row.  Semantics of the reference op (cuda/attention.cu:106-382): the score of a
// disallowed key gets -10000, and a PADDED key position takes part with K = V = 0 -- score 0, nothing
// added to the context, but its weight counts in the softmax denominator when the mask allows it.
struct MaskArgs {
  const __half* attr_mask;
  const int* batch_idx;
  const int* word_idx;
  int seq;
};

template <bool kMask>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, Coords co, __half* __restrict__ ctx,
                         const int* __restrict__ plan, int batch, int max_tokens, int heads,
                         float scale_log2e, int* status_word, int reverse, MaskArgs ma) {
  // The prologue (barriers, TMEM) touches no global memory: it runs before the
  // wait on the preceding kernel, under that kernel's tail.
  pdl_trigger();
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if ((base & 1023u) != 0u) {
    pdl_wait();  // no CTA leaves before the preceding kernel has completed
    if (threadIdx.x == 0) report_timeout(status_word, kKernelAttnTc, kSiteSmemAlign);
    return;
  }
  const int* tile_start = plan + 4;
  const int* tile_rows = plan + 4 + batch;
  const int* seq_lo = plan + 4 + 2 * batch;
  const int* seq_hi = seq_lo + max_tokens;

  const uint32_t bar_load0 = base + kBufBytes, bar_mma = bar_load0 + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + kBufBytes + 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + kBufBytes + 32);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = threadIdx.x;  // this thread's query row inside the tile = its TMEM lane
  const int hidden = heads * kD;

  if (threadIdx.x == 0) {
    mbar_init(bar_load0, 1);
    mbar_init(bar_load0 + 8, 1);
    mbar_init(bar_mma, 1);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);

  pdl_wait();  // the plan and the Q/K/V rows come from earlier kernels
  const int num_tiles = plan[0];
  const int total = num_tiles * heads;  // a CTA beyond it runs no item and frees its TMEM below

  uint32_t mma_phase = 0;
  bool ok = true;
  // Thread 0: Q and K rows of an item (barrier bar_qk) / its V rows (barrier bar_v).
  const uint32_t bar_qk = bar_load0, bar_v = bar_load0 + 8u;
  auto clamp_rows = [](int rows) { return rows < 1 ? 1 : (rows > kTileRows ? kTileRows : rows); };
  auto issue_qk = [&](int head_i, int first_row, int rows) {
    const int boxes = (clamp_rows(rows) + kBoxRows - 1) / kBoxRows;
    mbar_arrive_expect_tx(bar_qk, static_cast<uint32_t>(2 * boxes * kBoxBytes));
    const int x = head_i * co.x_per_head, y = head_i * co.y_per_head + first_row;
    for (int j = 0; j < boxes; ++j) {
      tma_load_2d(base + j * kBoxBytes, &tmap_q, x, y + j * kBoxRows, bar_qk);
      tma_load_2d(base + kTileBytes + j * kBoxBytes, &tmap_k, x, y + j * kBoxRows, bar_qk);
    }
  };
  auto issue_v = [&](int head_i, int first_row, int rows) {
    const int boxes = (clamp_rows(rows) + kBoxRows - 1) / kBoxRows;
    mbar_arrive_expect_tx(bar_v, static_cast<uint32_t>(boxes * kBoxBytes));
    const int x = head_i * co.x_per_head, y = head_i * co.y_per_head + first_row;
    for (int j = 0; j < boxes; ++j)
      tma_load_2d(base + 2 * kTileBytes + j * kBoxBytes, &tmap_v, x, y + j * kBoxRows, bar_v);
  };
  // An item's plan entries (tile bounds, then this row's sequence bounds) are two dependent
  // global loads.  They are fetched one item ahead in two steps, each issued where nothing needs
  // its result yet: the tile bounds under the wait for S = Q K^T, the sequence bounds under the
  // wait for O = P V.
  struct ItemMeta {
    int head, t0, n, lo, hi;
  };
  auto meta_tile = [&](int item_idx, ItemMeta& m) {   // step 1: issues two loads
    m = ItemMeta{0, 0, 1, 0, 0};
    if (item_idx >= total) return;
    const int li = reverse ? total - 1 - item_idx : item_idx;  // last tiles first: freshest in L2
    const int tile_i = li / heads;
    m.head = li - tile_i * heads;
    m.t0 = tile_start[tile_i];
    m.n = tile_rows[tile_i];
  };
  auto meta_row = [&](ItemMeta& m) {                  // step 2: needs step 1's results, issues two loads
    m.n = m.n < 1 ? 1 : (m.n > kTileRows ? kTileRows : m.n);
    if (r < m.n) {
      m.lo = seq_lo[m.t0 + r];
      m.hi = seq_hi[m.t0 + r];
    } else {
      m.lo = m.hi = m.t0;
    }
  };
  auto meta_finish = [&](ItemMeta& m) {               // this row's sequence, relative to the tile
    int lo = m.lo - m.t0, hi = m.hi - m.t0;
    m.lo = lo < 0 ? 0 : lo;
    m.hi = hi > m.n ? m.n : hi;
  };
  ItemMeta cur;
  meta_tile(blockIdx.x, cur);
  meta_row(cur);
  meta_finish(cur);
  if (threadIdx.x == 0 && static_cast<int>(blockIdx.x) < total) {
    issue_qk(cur.head, cur.t0, cur.n);
    issue_v(cur.head, cur.t0, cur.n);
  }
  int it_n = 0;
  auto wait_all = [&](uint32_t bar, uint32_t phase, int site) {
    bool got = mbar_wait(bar, phase, abort_flag);
    if (!got) {
      *abort_flag = 1;
      report_timeout(status_word, kKernelAttnTc, site);
    }
    return __syncthreads_and(got) != 0;
  };

  for (int item = blockIdx.x; item < total && ok; item += gridDim.x, ++it_n) {
    const int head = cur.head, t0 = cur.t0, n = cur.n;
    const int n16 = (n + 15) & ~15;
    const uint32_t sq = base, sk = sq + kTileBytes, sv = sk + kTileBytes;
    const uint32_t load_phase = static_cast<uint32_t>(it_n & 1);
    const bool has_next = item + static_cast<int>(gridDim.x) < total;

    const int lo = cur.lo, hi = cur.hi;
    // General mask: which of this row's own keys (tile columns lo..hi) it may attend to, one bit per tile
    // column, and how many PADDED key positions it may attend to (they only weigh in the denominator).
    // A row that may attend to nothing attends to everything: the same -10000 on every score cancels.
    uint32_t allow[4] = {0u, 0u, 0u, 0u};
    float n_pad = 0.f;
    if constexpr (kMask) {
      if (r < n && hi > lo) {
        const int token = t0 + r;
        const __half* mrow = ma.attr_mask +
            (static_cast<size_t>(ma.batch_idx[token]) * ma.seq + ma.word_idx[token]) * ma.seq;
        int total = 0;  // allowed key positions, valid or padded
        for (int j = 0; j < ma.seq; ++j) total += __half2float(mrow[j]) > 0.5f ? 1 : 0;
        int valid_allowed = 0;
        for (int c = lo; c < hi; ++c) {
          const int kpos = ma.word_idx[t0 + c];
          const bool a = total == 0 || __half2float(mrow[kpos]) > 0.5f;
          valid_allowed += a ? 1 : 0;
          if (a) {
            // static register indices: pick the word with a select chain
            const uint32_t bit = 1u << (c & 31);
            const int w = c >> 5;
            allow[0] |= w == 0 ? bit : 0u;
            allow[1] |= w == 1 ? bit : 0u;
            allow[2] |= w == 2 ? bit : 0u;
            allow[3] |= w == 3 ? bit : 0u;
          }
        }
        n_pad = static_cast<float>(total == 0 ? ma.seq - (hi - lo) : total - valid_allowed);
      }
    }
    ok = wait_all(bar_qk, load_phase, kSiteLoad);
    if (!ok) break;
    tc_fence_before();

    // ---- S = Q K^T ----
    if (threadIdx.x == 0) {
      tc_fence_after();
      const uint32_t idesc = idesc_f16(kTileRows, n16, false);
      const uint64_t qd = make_kmajor_sw128_desc(sq), kd = make_kmajor_sw128_desc(sk);
#pragma unroll
      for (int k = 0; k < kD / 16; ++k) umma_f16_ss(tmem_base, qd + 2u * k, kd + 2u * k, idesc, k != 0 ? 1u : 0u);
      umma_commit(bar_mma);
    }
    ItemMeta nxt;
    meta_tile(item + static_cast<int>(gridDim.x), nxt);
    ok = wait_all(bar_mma, mma_phase, kSiteScores);
    mma_phase ^= 1u;
    if (!ok) break;
    tc_fence_after();
    // Q and K are dead: the next item's Q/K rows stream in under the softmax and the second MMA
    if (threadIdx.x == 0 && has_next) issue_qk(nxt.head, nxt.t0, nxt.n);

    // ---- softmax over the row's own sequence; P -> tensor memory, over the scores it replaces ----
    const bool warp_has_rows = warp * 32 < n;
    float inv_l = 1.0f;
    if (warp_has_rows) {
      // columns any row of this warp needs, in 16-column chunks (uniform in the warp)
      int ulo = (r < n) ? lo : kTileRows, uhi = (r < n) ? hi : 0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        ulo = min(ulo, __shfl_xor_sync(0xffffffffu, ulo, o));
        uhi = max(uhi, __shfl_xor_sync(0xffffffffu, uhi, o));
      }
      ulo &= ~31;   // 32-column loads stay inside the 128 allocated columns
      uhi = (uhi + 15) & ~15;
      // (32 columns per TMEM load; a load may run up to 16 columns past n16, into
      // allocated columns whose values the range test discards)
      // Which of the 32 columns from c0 on this row attends to, one bit per column: the columns of its own
      // sequence (lo <= c < hi), or the bits the general mask left of them.  One bit test per element is
      // cheaper than a range test, and the kernel is bound by its instruction count as much as by HBM.
      auto chunk_bits = [&](int c0) -> uint32_t {
        if constexpr (kMask) {
          const int w = c0 >> 5;
          return w == 0 ? allow[0] : w == 1 ? allow[1] : w == 2 ? allow[2] : allow[3];
        } else {
          const int a = max(lo - c0, 0), b = min(hi - c0, 32);
          if (b <= a) return 0u;
          const uint32_t below_b = b >= 32 ? 0xffffffffu : (1u << b) - 1u;
          return below_b & ~((1u << a) - 1u);  // a < b <= 32, so a <= 31
        }
      };
      float m = -INFINITY;
      for (int c0 = ulo; c0 < uhi; c0 += 32) {
        uint32_t s32[32];
        tmem_ld_32x32b_x32(t_lane + c0, s32);
        tmem_ld_wait();
        const uint32_t aw = chunk_bits(c0);
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if ((aw >> e) & 1u) m = fmaxf(m, __uint_as_float(s32[e]));
      }
      if constexpr (kMask) {
        if (n_pad > 0.f) m = fmaxf(m, 0.f);  // a padded key the row may attend to has score 0
      }
      const float ms = (r < n && hi > lo) ? -m * scale_log2e : 0.f;
      float l = 0.f;
      for (int c0 = 0; c0 < n16; c0 += 32) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) pk[e] = 0u;
        if (c0 < uhi && c0 + 32 > ulo) {   // uniform in the warp
          uint32_t s32[32];
          tmem_ld_32x32b_x32(t_lane + c0, s32);
          tmem_ld_wait();
          const uint32_t aw = chunk_bits(c0);
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            float p2[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const float pe = ex2_approx(fmaf(__uint_as_float(s32[2 * e + u]), scale_log2e, ms));
              p2[u] = ((aw >> (2 * e + u)) & 1u) != 0u ? pe : 0.f;
              l += p2[u];
            }
            pk[e] = pack_half2(p2[0], p2[1]);
          }
        }
        // 32 keys = 16 packed columns; they overwrite score columns [c0/2, c0/2 + 16), all of
        // which this thread has read (c0/2 + 16 <= c0 + 32 and chunks are visited in order)
        tmem_st_32x32b_x16(t_lane + kPCol + (c0 >> 1), pk);
      }
      tmem_st_wait();
      if constexpr (kMask) l += n_pad * ex2_approx(ms);  // padded keys: score 0, V = 0
      inv_l = (l > 0.f) ? 1.0f / l : 0.f;
    }
    // this item's V rows were requested an item ago and have had the softmax to arrive.  Rows
    // [n, n16) may belong to the next tile or be stale: P is zero there, so make V finite there too.
    bool got_v = mbar_wait(bar_v, load_phase, abort_flag);
    if (!got_v) {
      *abort_flag = 1;
      report_timeout(status_word, kKernelAttnTc, kSiteLoad);
    }
    for (int idx = threadIdx.x; idx < (n16 - n) * 8; idx += kThreads)
      st_shared_v4(sv + (n + (idx >> 3)) * 128 + ((idx & 7) << 4), 0u, 0u, 0u, 0u);
    fence_proxy_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(got_v) != 0;
    if (!ok) break;

    // ---- O = P V ----
    if (threadIdx.x == 0) {
      tc_fence_after();
      const uint32_t idesc = idesc_f16(kTileRows, kD, true);
      for (int ks = 0; ks < n16 / 16; ++ks) {
        const uint64_t vd = make_kmajor_sw128_desc(sv + ks * 2048);  // MN-major: 16 keys = two 8-row groups
        // A = P from tensor memory: 16 keys = 8 packed columns per instruction
        umma_f16_ts(tmem_base + kOCol, tmem_base + kPCol + ks * 8, vd, idesc, ks != 0 ? 1u : 0u);
      }
      umma_commit(bar_mma);
    }
    meta_row(nxt);
    ok = wait_all(bar_mma, mma_phase, kSiteContext);
    mma_phase ^= 1u;
    if (!ok) break;
    tc_fence_after();
    // V is dead: the next item's V rows stream in under the epilogue and the next first MMA
    if (threadIdx.x == 0 && has_next) {
      fence_proxy_async_smem();  // orders the zero-fill stores above before the copy's writes
      issue_v(nxt.head, nxt.t0, nxt.n);
    }

    // ---- epilogue: O / l -> fp16 -> packed context ----
    if (warp_has_rows) {
      uint32_t ov[64];
      tmem_ld_32x32b_x32(t_lane + kOCol, ov);
      tmem_ld_32x32b_x32(t_lane + kOCol + 32, ov + 32);
      tmem_ld_wait();
      if (r < n) {
        __half* op = ctx + static_cast<size_t>(t0 + r) * hidden + head * kD;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t w[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            w[e] = pack_half2(__uint_as_float(ov[q4 * 16 + 2 * e]) * inv_l,
                              __uint_as_float(ov[q4 * 16 + 2 * e + 1]) * inv_l);
          asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(op + q4 * 16), "r"(w[0]),
                       "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                       : "memory");
        }
      }
    }
    tc_fence_before();
    __syncthreads();  // TMEM and the tiles are reused by the next item
    if (threadIdx.x == 0) fence_proxy_async_smem();
    meta_finish(nxt);
    cur = nxt;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

size_t attention_plan_ints(int batch, int max_tokens) { return plan_ints(batch, max_tokens); }

cudaError_t launch_attention_plan(const int* cu_seqlens, int batch, int max_tokens, int* plan,
                                  cudaStream_t stream) {
  if (batch <= 0) return cudaSuccess;
  const cudaError_t le = launch_pdl(attention_plan_kernel, dim3(1), dim3(1024), 0, stream, cu_seqlens, batch,
                                    max_tokens, plan);
  if (le != cudaSuccess) return le;
  return cudaGetLastError();
}

cudaError_t launch_attention_tcgen05(const __half* q, const __half* k, const __half* v,
                                     long long token_stride, long long head_stride, __half* ctx,
                                     const int* plan, int batch, int max_tokens, int heads, int d,
                                     int* status_word, cudaStream_t stream, bool reverse, TensorMapCache* maps,
                                     const __half* attr_mask, const int* batch_idx, const int* word_idx, int seq) {
  if (batch <= 0 || heads <= 0 || max_tokens <= 0) return cudaSuccess;
  if (d != kD || token_stride < kD || (token_stride % 8) != 0 || (head_stride % 8) != 0 || head_stride < 0)
    return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(ctx)) & 31u)
    return cudaErrorMisalignedAddress;
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
    cudaError_t attr_err = cudaFuncSetAttribute(attention_tcgen05_kernel<false>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(attention_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemBytes);
    return attr_err;
  });
  if (once_err != cudaSuccess) return once_err;
  const bool masked = attr_mask != nullptr;
  if (masked && (batch_idx == nullptr || word_idx == nullptr || seq <= 0 || seq > kTileRows))
    return cudaErrorInvalidValue;
  const MaskArgs ma{attr_mask, batch_idx, word_idx, seq};
  const float scale_log2e = (1.0f / sqrtf(static_cast<float>(d))) * 1.4426950408889634f;
  // every tile holds at least one sequence, so batch * heads bounds the item count
  long long grid = static_cast<long long>(sm_count()) * kCtasPerSm;
  const long long max_items = static_cast<long long>(batch) * heads;
  if (grid > max_items) grid = max_items;
  return masked ? launch_pdl(attention_tcgen05_kernel<true>, dim3(static_cast<int>(grid)), dim3(kThreads), kSmemBytes,
                             stream, tq, tk, tv, co, ctx, plan, batch, max_tokens, heads, scale_log2e, status_word,
                             reverse ? 1 : 0, ma)
                : launch_pdl(attention_tcgen05_kernel<false>, dim3(static_cast<int>(grid)), dim3(kThreads), kSmemBytes,
                             stream, tq, tk, tv, co, ctx, plan, batch, max_tokens, heads, scale_log2e, status_word,
                             reverse ? 1 : 0, ma);
}

}  // namespace etb
