// Padding bookkeeping: mask prefix sum -> per-token indices, remove padding,
// restore padding.  Replaces the scan / compress / restore kernels of the
// reference (cuda/cuda_kernels.cu:278-718) and the host logic around them
// (tf_op/bert_transformer_op.cu.cc:266-373).  All integer results are
// bit-exact with cumsum(mask) - mask.
#include "common.cuh"

#include <mutex>
#include <string>

#include "../../include/et_b200.h"

namespace etb {

namespace {

constexpr int kRowsPerCta = 8;  // one warp per mask row

// Pass 1: valid positions per mask row.
__global__ void __launch_bounds__(kRowsPerCta * 32)
seq_lengths_kernel(const int* __restrict__ mask, int batch, int seq, int* __restrict__ lens,
                   int* __restrict__ seq_len_out) {
  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x * kRowsPerCta + warp;
  if (b >= batch) return;
  const int* row = mask + static_cast<size_t>(b) * seq;
  int cnt = 0;
  for (int s = lane; s < seq; s += 32) cnt += (row[s] > 0) ? 1 : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if (lane == 0) {
    lens[b] = cnt;
    if (seq_len_out != nullptr) seq_len_out[b] = cnt;
  }
}

// Pass 2: row bases from the row lengths, then a ballot scan inside each row.
__global__ void __launch_bounds__(kRowsPerCta * 32)
padding_offsets_emit_kernel(const int* __restrict__ mask, const int* __restrict__ lens, int batch,
                            int seq, int* __restrict__ prefix_sum, int* __restrict__ valid_word_num,
                            int* __restrict__ batch_idx, int* __restrict__ word_idx,
                            int* __restrict__ cu_seqlens, int* __restrict__ padding_offset) {
  pdl_wait();
  pdl_trigger();
  __shared__ int s_part[kRowsPerCta];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r0 = blockIdx.x * kRowsPerCta;
  // tokens in all rows before this CTA's first row
  int acc = 0;
  for (int j = threadIdx.x; j < r0; j += blockDim.x) acc += lens[j];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) s_part[warp] = acc;
  __syncthreads();
  int base = 0;
#pragma unroll
  for (int w = 0; w < kRowsPerCta; ++w) base += s_part[w];
  const int b = r0 + warp;
  if (b >= batch) return;
  for (int w = 0; w < warp; ++w) base += lens[r0 + w];

  if (lane == 0 && cu_seqlens != nullptr) cu_seqlens[b] = base;
  const int* row = mask + static_cast<size_t>(b) * seq;
  int running = base;
  for (int s0 = 0; s0 < seq; s0 += 32) {
    const int s = s0 + lane;
    const bool valid = (s < seq) && (row[s] > 0);
    const unsigned bal = __ballot_sync(0xffffffffu, valid);
    const int pre = running + __popc(bal & ((1u << lane) - 1u));
    if (s < seq) {
      const size_t flat = static_cast<size_t>(b) * seq + s;
      if (prefix_sum != nullptr) prefix_sum[flat] = pre;
      if (valid) {
        if (batch_idx != nullptr) batch_idx[pre] = b;
        if (word_idx != nullptr) word_idx[pre] = s;
        if (padding_offset != nullptr) padding_offset[pre] = static_cast<int>(flat) - pre;
      }
    }
    running += __popc(bal);
  }
  if (b == batch - 1 && lane == 0) {
    if (cu_seqlens != nullptr) cu_seqlens[batch] = running;
    if (valid_word_num != nullptr) valid_word_num[0] = running;
  }
}

__global__ void empty_batch_kernel(int* valid_word_num, int* cu_seqlens) {
  pdl_wait();
  if (valid_word_num != nullptr) valid_word_num[0] = 0;
  if (cu_seqlens != nullptr) cu_seqlens[0] = 0;
}

// cu_seqlens from batch_idx alone (the layer op receives no other padding
// information): packed rows of one sequence are contiguous and ordered by b.
__global__ void seq_bounds_kernel(const int* __restrict__ batch_idx, const int* __restrict__ t_ptr,
                                  int batch, int max_tokens, int* __restrict__ cu_seqlens) {
  pdl_wait();
  pdl_trigger();
  int t = *t_ptr;
  t = t < 0 ? 0 : (t > max_tokens ? max_tokens : t);
  for (int v = blockIdx.x * blockDim.x + threadIdx.x; v <= t; v += gridDim.x * blockDim.x) {
    int prev = (v == 0) ? -1 : batch_idx[v - 1];
    int cur = (v == t) ? batch : batch_idx[v];
    prev = prev < -1 ? -1 : prev;
    cur = cur > batch ? batch : cur;
    for (int b = prev + 1; b <= cur; ++b) cu_seqlens[b] = v;
  }
}

constexpr int kCopyWarpsPerCta = 8;
constexpr int kCopyCtasPerSm = 8;

template <int kChunk>
__device__ __forceinline__ void warp_copy_row(const char* __restrict__ src, char* __restrict__ dst,
                                              int nvec, int lane) {
  for (int i0 = 0; i0 < nvec; i0 += 32 * kChunk) {
    Vec16 r[kChunk];
#pragma unroll
    for (int c = 0; c < kChunk; ++c) {
      const int i = i0 + c * 32 + lane;
      if (i < nvec) r[c] = ld_global_nc_v4(src + static_cast<size_t>(i) * 16);
    }
#pragma unroll
    for (int c = 0; c < kChunk; ++c) {
      const int i = i0 + c * 32 + lane;
      if (i < nvec) st_global_v4(dst + static_cast<size_t>(i) * 16, r[c]);
    }
  }
}

__device__ __forceinline__ void warp_zero_row(char* __restrict__ dst, int nvec, int lane) {
  const Vec16 z = {0u, 0u, 0u, 0u};
  for (int i = lane; i < nvec; i += 32) st_global_v4(dst + static_cast<size_t>(i) * 16, z);
}

// Packed row v <- padded row (batch_idx[v], word_idx[v]); one warp per row.
__global__ void __launch_bounds__(kCopyWarpsPerCta * 32)
remove_padding_kernel(const char* __restrict__ from, const int* __restrict__ batch_idx,
                      const int* __restrict__ word_idx, const int* __restrict__ t_ptr,
                      char* __restrict__ to, int max_rows, int seq, int row_bytes) {
  pdl_wait();
  pdl_trigger();
  int t = *t_ptr;
  t = t < 0 ? 0 : (t > max_rows ? max_rows : t);
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * kCopyWarpsPerCta + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * kCopyWarpsPerCta;
  const int nvec = row_bytes >> 4;
  for (int v = warp; v < t; v += nwarps) {
    const int b = batch_idx[v], s = word_idx[v];
    const size_t r = static_cast<size_t>(b) * seq + s;
    if (r >= static_cast<size_t>(max_rows)) continue;  // corrupt index: skip, never fault
    warp_copy_row<4>(from + r * row_bytes, to + static_cast<size_t>(v) * row_bytes, nvec, lane);
  }
}

// One pass over the padded output: item v < T copies packed row v to its
// padded row and zero-fills the gap of padded rows in front of it; item T
// zero-fills everything behind the last valid row.
__global__ void __launch_bounds__(kCopyWarpsPerCta * 32)
restore_padding_kernel(const char* __restrict__ from, const int* __restrict__ batch_idx,
                       const int* __restrict__ word_idx, const int* __restrict__ t_ptr,
                       char* __restrict__ to, int max_rows, int seq, int row_bytes) {
  pdl_wait();
  pdl_trigger();
  int t = *t_ptr;
  t = t < 0 ? 0 : (t > max_rows ? max_rows : t);
  const int lane = threadIdx.x & 31;
  const int warp = blockIdx.x * kCopyWarpsPerCta + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * kCopyWarpsPerCta;
  const int nvec = row_bytes >> 4;
  for (int v = warp; v <= t; v += nwarps) {
    long long prev = -1, cur = max_rows;
    if (v > 0) prev = static_cast<long long>(batch_idx[v - 1]) * seq + word_idx[v - 1];
    if (v < t) cur = static_cast<long long>(batch_idx[v]) * seq + word_idx[v];
    if (prev < -1 || prev >= max_rows) prev = max_rows;  // corrupt index: nothing to fill
    if (cur < 0 || cur > max_rows) cur = max_rows;
    for (long long r = prev + 1; r < cur; ++r)
      warp_zero_row(to + static_cast<size_t>(r) * row_bytes, nvec, lane);
    if (v < t && cur < max_rows)
      warp_copy_row<4>(from + static_cast<size_t>(v) * row_bytes,
                       to + static_cast<size_t>(cur) * row_bytes, nvec, lane);
  }
}

}  // namespace

cudaError_t launch_padding_offsets(const int* mask, int batch, int seq, int* prefix_sum,
                                   int* valid_word_num, int* batch_idx, int* word_idx,
                                   int* seq_len_out, int* cu_seqlens, int* padding_offset,
                                   int* scratch, cudaStream_t stream) {
  if (batch <= 0 || seq <= 0) {
    return launch_pdl(empty_batch_kernel, dim3(1), dim3(1), 0, stream, valid_word_num, cu_seqlens);
  }
  const int ctas = (batch + kRowsPerCta - 1) / kRowsPerCta;
  cudaError_t e = launch_pdl(seq_lengths_kernel, dim3(ctas), dim3(kRowsPerCta * 32), 0, stream, mask, batch, seq,
                             scratch, seq_len_out);
  if (e != cudaSuccess) return e;
  return launch_pdl(padding_offsets_emit_kernel, dim3(ctas), dim3(kRowsPerCta * 32), 0, stream, mask, scratch,
                    batch, seq, prefix_sum, valid_word_num, batch_idx, word_idx, cu_seqlens, padding_offset);
}

cudaError_t launch_seq_bounds_from_batch_idx(const int* batch_idx, const int* t_ptr, int batch,
                                             int max_tokens, int* cu_seqlens, cudaStream_t stream) {
  const int threads = 256;
  int ctas = (max_tokens + 1 + threads - 1) / threads;
  const int cap = sm_count() * 8;
  ctas = ctas < 1 ? 1 : (ctas > cap ? cap : ctas);
  return launch_pdl(seq_bounds_kernel, dim3(ctas), dim3(threads), 0, stream, batch_idx, t_ptr, batch, max_tokens,
                    cu_seqlens);
}

template <typename T>
cudaError_t launch_remove_padding(const T* from, const int* batch_idx, const int* word_idx,
                                  const int* t_ptr, T* to, int batch, int seq, int hidden,
                                  cudaStream_t stream) {
  const long long rows = static_cast<long long>(batch) * seq;
  if (rows <= 0) return cudaSuccess;
  const int row_bytes = hidden * static_cast<int>(sizeof(T));
  long long ctas = (rows + kCopyWarpsPerCta - 1) / kCopyWarpsPerCta;
  const long long cap = static_cast<long long>(sm_count()) * kCopyCtasPerSm;
  if (ctas > cap) ctas = cap;
  return launch_pdl(remove_padding_kernel, dim3(static_cast<int>(ctas)), dim3(kCopyWarpsPerCta * 32), 0, stream,
                    reinterpret_cast<const char*>(from), batch_idx, word_idx, t_ptr, reinterpret_cast<char*>(to),
                    static_cast<int>(rows), seq, row_bytes);
}

template <typename T>
cudaError_t launch_restore_padding(const T* from, const int* batch_idx, const int* word_idx,
                                   const int* t_ptr, T* to, int batch, int seq, int hidden,
                                   cudaStream_t stream) {
  const long long rows = static_cast<long long>(batch) * seq;
  if (rows <= 0) return cudaSuccess;
  const int row_bytes = hidden * static_cast<int>(sizeof(T));
  long long ctas = (rows + 1 + kCopyWarpsPerCta - 1) / kCopyWarpsPerCta;
  const long long cap = static_cast<long long>(sm_count()) * kCopyCtasPerSm;
  if (ctas > cap) ctas = cap;
  return launch_pdl(restore_padding_kernel, dim3(static_cast<int>(ctas)), dim3(kCopyWarpsPerCta * 32), 0, stream,
                    reinterpret_cast<const char*>(from), batch_idx, word_idx, t_ptr, reinterpret_cast<char*>(to),
                    static_cast<int>(rows), seq, row_bytes);
}

#define ETB_INST(T)                                                                              \
  template cudaError_t launch_remove_padding<T>(const T*, const int*, const int*, const int*, T*, \
                                                int, int, int, cudaStream_t);                    \
  template cudaError_t launch_restore_padding<T>(const T*, const int*, const int*, const int*,   \
                                                 T*, int, int, int, cudaStream_t);
ETB_INST(float)
ETB_INST(__half)
#undef ETB_INST

// ---------------------------------------------------------------------------
// et_padding_offsets_noalloc: the padding-offset computation for callers that
// must not allocate device memory.
//
// et_padding_offsets needs a scratch array of batch_size ints (the per-row
// token counts that pass 1 hands to pass 2) and leaves its allocation to the
// caller.  Some callers cannot provide one: a framework custom-op whose
// allocator may not be re-entered from the op, code that runs while a memory
// pool is frozen, or a plain C plug-in host that has no device allocator at
// all.  For them the scratch lives in the library image itself, as the
// file-scope device array below; every GPU that loads the library holds these
// ET_NOALLOC_MAX_BATCH * 4 bytes until the process exits.
//
// The array's name is only a host-side handle for the symbol: the device
// address is looked up with cudaGetSymbolAddress, once per device, with that
// device current, the first time the entry point runs there.
// ---------------------------------------------------------------------------
namespace {

static __device__ __align__(256) int g_noalloc_row_lengths[ET_NOALLOC_MAX_BATCH];

std::mutex g_noalloc_mutex;
int* g_noalloc_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device (set-up on first use).
cudaError_t noalloc_scratch(int** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    int* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_row_lengths);
    if (e != cudaSuccess) return e;
    if (p == nullptr) return cudaErrorInvalidSymbol;
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return cudaSuccess;
}

}  // namespace
}  // namespace etb

namespace {

int noalloc_impl(const int* mask, int batch_size, int seq_len, int* prefix_sum, int* valid_word_num,
                 int* batch_idx, int* word_idx, int* seq_len_out, int* cu_seqlens, int* padding_offset,
                 void* stream) {
  if (batch_size < 0 || seq_len < 0) {
    etb::set_global_error("et_padding_offsets_noalloc: negative batch_size or seq_len");
    return ET_INVALID_ARGUMENT;
  }
  if (batch_size > ET_NOALLOC_MAX_BATCH) {
    etb::set_global_error("et_padding_offsets_noalloc: batch_size " + std::to_string(batch_size) +
                          " exceeds ET_NOALLOC_MAX_BATCH (" + std::to_string(ET_NOALLOC_MAX_BATCH) +
                          "); use et_padding_offsets with caller-provided scratch");
    return ET_INVALID_ARGUMENT;
  }
  if (batch_size > 0 && seq_len > 0 && mask == nullptr) {
    etb::set_global_error("et_padding_offsets_noalloc: null mask");
    return ET_INVALID_ARGUMENT;
  }
  int* scratch = nullptr;
  cudaError_t e = etb::noalloc_scratch(&scratch);
  if (e != cudaSuccess) {
    etb::set_global_error(std::string("et_padding_offsets_noalloc: cudaGetSymbolAddress failed: ") +
                          cudaGetErrorString(e));
    return ET_CUDA_ERROR;
  }
  // Nothing in the scratch has to start at zero: pass 1 overwrites the first
  // batch_size entries before pass 2 reads them, and no other entry is read.
  e = etb::launch_padding_offsets(mask, batch_size, seq_len, prefix_sum, valid_word_num, batch_idx,
                                  word_idx, seq_len_out, cu_seqlens, padding_offset, scratch,
                                  static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    etb::set_global_error(std::string("et_padding_offsets_noalloc: launch failed: ") + cudaGetErrorString(e));
    return ET_CUDA_ERROR;
  }
  return ET_OK;
}

}  // namespace

extern "C" int et_padding_offsets_noalloc(const int* mask, int batch_size, int seq_len, int* prefix_sum,
                                          int* valid_word_num, int* batch_idx, int* word_idx,
                                          int* seq_len_out, int* cu_seqlens, int* padding_offset,
                                          void* stream) {
  // The error texts are std::strings: no exception (a failed host allocation) may cross the C ABI.
  try {
    return noalloc_impl(mask, batch_size, seq_len, prefix_sum, valid_word_num, batch_idx, word_idx, seq_len_out,
                        cu_seqlens, padding_offset, stream);
  } catch (...) {
    return ET_CUDA_ERROR;
  }
}
