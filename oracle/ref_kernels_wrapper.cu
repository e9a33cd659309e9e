// TEST INFRASTRUCTURE.  C entry points around the kernel launchers of the
// reference (declared in its cuda/cuda_kernels.h and cuda/attention.h), so that
// the tests can run the reference's own CUDA kernels - compiled unmodified from
// the reference checkout by oracle/build_ref.py - next to this repository's
// kernels and next to the CPU oracle.  Nothing here is part of the product and
// nothing of the reference's source is copied: this file only calls its
// public launcher templates.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "cuda/attention.h"
#include "cuda/cuda_kernels.h"

namespace et = effectivetransformer;

namespace {
inline int done() { return static_cast<int>(cudaGetLastError()); }
inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }
}  // namespace

extern "C" {

// d_out must hold 2 * length ints (the launcher keeps its scratch behind the
// result, as the input functor allocates it: tf_op/bert_transformer_op.cu.cc:279).
int ref_exclusive_scan(int* d_out, const int* d_in, int length, void* stream) {
  et::exclusiveScan_kernelLauncher(d_out, d_in, length, S(stream));
  return done();
}

// dtype: 0 = float, 1 = half (the two instantiations the reference ships)
int ref_compress_input(int dtype, const void* from, const int* mask, const int* prefix, void* to,
                       int* batch_idx, int* word_idx, int batch, int seq, int hidden, void* stream) {
  if (dtype == 1)
    et::compressBertInput_kernelLauncher<__half>(static_cast<const __half*>(from), mask, prefix,
                                                 static_cast<__half*>(to), batch_idx, word_idx, batch,
                                                 seq, hidden, S(stream));
  else
    et::compressBertInput_kernelLauncher<float>(static_cast<const float*>(from), mask, prefix,
                                                static_cast<float*>(to), batch_idx, word_idx, batch, seq,
                                                hidden, S(stream));
  return done();
}

int ref_restore_output(int dtype, void* to, const void* from, const int* batch_idx, const int* word_idx,
                       int valid_word_num, int seq, int hidden, void* stream) {
  if (dtype == 1)
    et::restoreBertOutput_kernelLauncher<__half>(static_cast<__half*>(to), static_cast<const __half*>(from),
                                                 batch_idx, word_idx, valid_word_num, seq, hidden, S(stream));
  else
    et::restoreBertOutput_kernelLauncher<float>(static_cast<float*>(to), static_cast<const float*>(from),
                                                batch_idx, word_idx, valid_word_num, seq, hidden, S(stream));
  return done();
}

int ref_add_bias_act(int dtype, void* out, const void* bias, int m, int n, void* stream) {
  if (dtype == 1)
    et::add_bias_act_kernelLauncher<__half>(static_cast<__half*>(out), static_cast<const __half*>(bias), m, n,
                                            S(stream));
  else
    et::add_bias_act_kernelLauncher<float>(static_cast<float*>(out), static_cast<const float*>(bias), m, n,
                                           S(stream));
  return done();
}

int ref_add_bias_input_layernorm(int dtype, void* out, const void* input, const void* bias, const void* gamma,
                                 const void* beta, int m, int n, void* stream) {
  if (dtype == 1)
    et::add_bias_input_layernorm_kernelLauncher<__half>(
        static_cast<__half*>(out), static_cast<const __half*>(input), static_cast<const __half*>(bias),
        static_cast<const __half*>(gamma), static_cast<const __half*>(beta), m, n, S(stream));
  else
    et::add_bias_input_layernorm_kernelLauncher<float>(
        static_cast<float*>(out), static_cast<const float*>(input), static_cast<const float*>(bias),
        static_cast<const float*>(gamma), static_cast<const float*>(beta), m, n, S(stream));
  return done();
}

int ref_add_qkv_bias_padding(int dtype, void* q, const void* bq, void* k, const void* bk, void* v,
                             const void* bv, void* q_buf, void* k_buf, void* v_buf, int valid_word_num,
                             int batch, int seq, int heads, int d, const int* batch_idx, const int* word_idx,
                             void* stream) {
  if (dtype == 1)
    et::cuda::add_QKV_bias_padding_kernelLauncher<__half>(
        static_cast<__half*>(q), static_cast<const __half*>(bq), static_cast<__half*>(k),
        static_cast<const __half*>(bk), static_cast<__half*>(v), static_cast<const __half*>(bv),
        static_cast<__half*>(q_buf), static_cast<__half*>(k_buf), static_cast<__half*>(v_buf), valid_word_num,
        batch, seq, heads, d, batch_idx, word_idx, S(stream));
  else
    et::cuda::add_QKV_bias_padding_kernelLauncher<float>(
        static_cast<float*>(q), static_cast<const float*>(bq), static_cast<float*>(k),
        static_cast<const float*>(bk), static_cast<float*>(v), static_cast<const float*>(bv),
        static_cast<float*>(q_buf), static_cast<float*>(k_buf), static_cast<float*>(v_buf), valid_word_num,
        batch, seq, heads, d, batch_idx, word_idx, S(stream));
  return done();
}

int ref_softmax(int dtype, void* qk_buf, const void* attr_mask, int batch, int heads, int seq, float scaler,
                void* stream) {
  if (dtype == 1)
    et::cuda::softmax_kernel_kernelLauncher<__half>(static_cast<__half*>(qk_buf),
                                                    static_cast<const __half*>(attr_mask), batch, heads, seq,
                                                    __float2half(scaler), S(stream));
  else
    et::cuda::softmax_kernel_kernelLauncher<float>(static_cast<float*>(qk_buf),
                                                   static_cast<const float*>(attr_mask), batch, heads, seq,
                                                   scaler, S(stream));
  return done();
}

int ref_transpose_rm_padding(int dtype, void* src, void* dst, int valid_word_num, int batch, int seq, int heads,
                             int d, const int* batch_idx, const int* word_idx, void* stream) {
  if (dtype == 1)
    et::cuda::transpose_rm_padding_kernelLauncher<__half>(static_cast<__half*>(src), static_cast<__half*>(dst),
                                                          valid_word_num, batch, seq, heads, d, batch_idx,
                                                          word_idx, S(stream));
  else
    et::cuda::transpose_rm_padding_kernelLauncher<float>(static_cast<float*>(src), static_cast<float*>(dst),
                                                         valid_word_num, batch, seq, heads, d, batch_idx,
                                                         word_idx, S(stream));
  return done();
}

}  // extern "C"
