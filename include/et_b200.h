/*
 * C ABI of the B200 (sm_100a) padding-free BERT encoder path.
 *
 * Every entry point takes plain pointers and sizes; device pointers are raw
 * CUDA device addresses, `stream` is a cudaStream_t passed as void*.  No C++
 * exception crosses this boundary: every function returns an et_status_t and
 * the text of the last error of a handle is available from et_last_error().
 *
 * The three operators mirror the reference's TensorFlow ops
 *   EffectiveTransformerInput   (tf_op/bert_transformer_op.cc:249-274)
 *   EffectiveTransformer        (tf_op/bert_transformer_op.cc:44-77)
 *   EffectiveTransformerOutput  (tf_op/bert_transformer_op.cc:359-380)
 * and the parameter structs mirror, field for field, the C++ encoder-layer
 * interface of tf_op/bert_transformer_op.h:50-128, so a framework shim is a
 * pointer copy.
 *
 * A handle is bound to one CUDA device, owns the repacked weights, the
 * workspace and a device status word, and is not re-entrant: calls on one
 * handle must be issued from one thread at a time (the reference serialises
 * its layer op with a mutex, tf_op/bert_transformer_op.cc:213).
 */
#ifndef ET_B200_H_
#define ET_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct et_handle_s* et_handle_t;

typedef enum {
  ET_OK = 0,
  ET_INVALID_ARGUMENT = 1,   /* reference: errors::InvalidArgument via OP_REQUIRES */
  ET_CUDA_ERROR = 2,         /* reference: check_cuda_error -> errors::Internal (common.h:73-81) */
  ET_WORKSPACE_TOO_SMALL = 3,
  ET_DEVICE_TIMEOUT = 4,     /* a bounded device-side wait expired; see et_device_status */
  ET_NOT_READY = 5           /* weights of a layer were never set */
} et_status_t;

/* Mirrors effectivetransformer::OperationType {FP32, HALF} (common.h:26). */
typedef enum { ET_FP32 = 0, ET_FP16 = 1 } et_dtype_t;

typedef struct {
  int dtype;            /* et_dtype_t: element type of activations AND weights */
  int num_layers;
  int head_num;         /* attr head_num       (tf_op/bert_transformer_op.cc:56) */
  int size_per_head;    /* attr size_per_head  (tf_op/bert_transformer_op.cc:57); must be 64 */
  int ffn_dim;          /* the reference hard-codes 4*hidden (tf_op/bert_transformer_op.cu.cc:215) */
  int max_batch_size;   /* attr batch_size: a maximum, the run-time batch may be smaller */
  int max_seq_len;      /* attr from_seq_len == to_seq_len */
  float layernorm_eps;  /* 0 selects the reference kernel's 1e-6 (cuda/cuda_kernels.cu:183) */
  int device;           /* CUDA device ordinal */
} et_config_t;

/* Mirrors TransformerParam (tf_op/bert_transformer_op.h:50-66). */
typedef struct {
  int batch_size;
  int from_seq_len;
  int to_seq_len;       /* must equal from_seq_len (tf_op/bert_transformer_op.cc:130-131) */
  int head_num;
  int size_per_head;
} et_transformer_param_t;

/* Mirrors EncoderInitParam<T> (tf_op/bert_transformer_op.h:68-96); T is the
 * handle's dtype.  Weight kernels are [in, out] row-major as TensorFlow's
 * dense layers store them.  If attr_kernel_Q is NULL the weights registered
 * with et_set_layer_weights for that layer are used and all other weight
 * fields are ignored; otherwise all 16 weight fields must be device pointers
 * and are repacked on `stream` before the layer runs.  attr_mask ([B,S,S]) is
 * accepted for signature compatibility and must be the key-only tile of the
 * input mask (sample/tensorflow/benchmark.py:59-61); it is not read unless the
 * handle is in general-mask mode (et_set_general_mask). */
typedef struct {
  const void* from_tensor;   /* packed [T, H] inside a [B,S,H]-sized buffer */
  const void* to_tensor;     /* must equal from_tensor (self-attention) */
  const void* attr_kernel_Q;
  const void* attr_kernel_K;
  const void* attr_kernel_V;
  const void* attr_bias_Q;
  const void* attr_bias_K;
  const void* attr_bias_V;
  const void* attr_mask;
  const void* attr_output_kernel;
  const void* attr_output_bias;
  const void* attr_output_layernorm_gamma;
  const void* attr_output_layernorm_beta;
  const void* inter_kernel;
  const void* inter_bias;
  const void* output_kernel;
  const void* output_bias;
  const void* output_layernorm_gamma;
  const void* output_layernorm_beta;
  const int* batch_idx;
  const int* word_idx;
  const int* valid_word_num;
  void* transformer_out;     /* packed [T, H]; may alias from_tensor */
  void* stream;              /* replaces cublas_handle + stream of the reference struct */
} et_encoder_param_t;

/* Mirrors EncoderInputInitParam<T> (tf_op/bert_transformer_op.h:98-112). */
typedef struct {
  const void* from_tensor;   /* [B, S, H] */
  const int* mask;           /* [B, S], 0/1 */
  int* valid_word_num;       /* [1] */
  int* batch_idx;            /* [B*S], first T entries written */
  int* word_idx;             /* [B*S], first T entries written */
  int batch_size;
  int from_seq_len;
  int head_num;
  int size_per_head;
  void* to_tensor;           /* [B,S,H]-sized buffer, first T rows written */
  void* stream;
} et_input_param_t;

/* Mirrors EncoderOutputInitParam<T> (tf_op/bert_transformer_op.h:114-128). */
typedef struct {
  const void* from_tensor;   /* packed [T, H] */
  const int* valid_word_num;
  const int* batch_idx;
  const int* word_idx;
  int batch_size;
  int from_seq_len;
  int head_num;
  int size_per_head;
  void* to_tensor;           /* [B, S, H]; padded rows are written as zero */
  void* stream;
} et_output_param_t;

/* ---- life cycle --------------------------------------------------------- */

/* Replaces the op constructors (tf_op/bert_transformer_op.cc:84-178): checks
 * the attributes, binds the device, allocates weights slots, workspace and
 * the status word. */
int et_create(const et_config_t* config, et_handle_t* out_handle);
int et_destroy(et_handle_t handle);
const char* et_last_error(et_handle_t handle);

/* Replaces the attr -> device weight tensors step of the layer op constructor
 * (tf_op/bert_transformer_op.cc:91-103).  `weights` holds 16 pointers in the
 * order of python/effective_transformer/__init__.py:55-74.  `on_host` != 0:
 * host arrays (copied synchronously); 0: device arrays.  The handle keeps its
 * own repacked copy; the caller's arrays are not referenced afterwards. */
int et_set_layer_weights(et_handle_t handle, int layer, const void* const* weights, int on_host);

/* Bytes of handle-owned workspace for a [B, S] batch (size_t arithmetic; the
 * reference's int formula overflows, tf_op/bert_transformer_op.cu.cc:75-77). */
int et_workspace_bytes(et_handle_t handle, int batch_size, int seq_len, size_t* out_bytes);
/* What et_create allocated for the handle's own (max_batch_size, max_seq_len):
 * equals et_workspace_bytes at that shape (both are read from one table). */
int et_workspace_allocated_bytes(et_handle_t handle, size_t* out_bytes);

/* ---- the three operators ------------------------------------------------ */

/* EffectiveTransformerInputOpFunctor::Compute
 * (tf_op/bert_transformer_op.cu.cc:266-331).  No host synchronisation. */
int et_input(et_handle_t handle, const et_input_param_t* param);

/* EffectiveTransformerOpFunctor::Compute (tf_op/bert_transformer_op.cu.cc:37-259). */
int et_layer(et_handle_t handle, int layer, const et_encoder_param_t* param,
             const et_transformer_param_t* t_param);

/* EffectiveTransformerOutputOpFunctor::Compute
 * (tf_op/bert_transformer_op.cu.cc:339-373). */
int et_output(et_handle_t handle, const et_output_param_t* param);

/* ---- whole path ---------------------------------------------------------- */

/* get_sequence_output (python/effective_transformer/__init__.py:32-84) as one
 * call: input op, num_layers layer ops, output op, all on `stream`, device
 * buffers.  `out` is [B,S,H].  Asynchronous; nothing is read back. */
int et_forward(et_handle_t handle, const void* from_tensor, const int* mask, void* out,
               int batch_size, int seq_len, void* stream);

/* General attention masks.  By default the layer op does not read attr_mask
 * (it must be the key-only tile of the input mask, as the reference's sample
 * builds it, and the fast kernels derive it from the sequence bounds).
 * et_set_general_mask(handle, 1) makes et_layer read attr_mask [B,S,S]
 * through et_attention_general_mask's kernel instead;
 * et_forward_general_mask is et_forward with such a mask. */
int et_set_general_mask(et_handle_t handle, int enable);
int et_forward_general_mask(et_handle_t handle, const void* from_tensor, const int* mask,
                            const void* attr_mask, void* out, int batch_size, int seq_len, void* stream);

/* et_forward with HOST buffers (pinned or pageable): copies from_tensor and mask to
 * the device, runs et_forward, copies the [B,S,H] result back and waits for
 * it, like one sess.run of sample/tensorflow/benchmark.py:114-124.
 * `valid_word_num_out` (may be NULL) receives T. */
int et_forward_host(et_handle_t handle, const void* from_tensor_host, const int* mask_host,
                    void* out_host, int batch_size, int seq_len, int* valid_word_num_out);

/* ---- the model around the stack: embeddings in front, pooler behind -------
 * The reference leaves both to TensorFlow (sample/tensorflow/modeling.py:
 * 380-521 and 224-232) and feeds its input op with the padded embedding output.
 * Here they run on the packed layout: embedding rows are gathered for valid
 * tokens only (the placement the reference itself recommends,
 * tf_op/bert_transformer_op.cu.cc:295-296) and the pooler reads first-token
 * rows straight from the packed tensor. */

/* Registers the embedding tables (copied; element type = the handle's dtype):
 * word_table [vocab_size, H]; type_table [type_vocab_size, H] or NULL
 * (use_token_type = False); position_table [max_position, H] or NULL
 * (use_position_embeddings = False); LayerNorm gamma/beta [H].
 * layernorm_eps 0 selects tf.contrib.layers.layer_norm's 1e-12. */
int et_set_embedding_weights(et_handle_t handle, const void* word_table, int vocab_size,
                             const void* type_table, int type_vocab_size, const void* position_table,
                             int max_position, const void* gamma, const void* beta, float layernorm_eps,
                             int on_host);

/* Registers the pooler's dense layer: kernel [H, H] ([in, out]) and bias [H]. */
int et_set_pooler_weights(et_handle_t handle, const void* kernel, const void* bias, int on_host);

/* BertModel (sample/tensorflow/modeling.py:107-235) at inference, device
 * buffers: input_ids / mask int32 [B,S]; token_type_ids int32 [B,S] or NULL
 * (all zero, modeling.py:159-160).  Outputs, each may be NULL:
 * sequence_out [B,S,H] (padded rows zero) and pooled_out [B,H] (needs pooler
 * weights).  A sequence without tokens pools a zero first-token row.  If both
 * are NULL the packed result stays in the handle (et_last_packed_output).
 * seq_len > max_position is rejected (tf.assert_less_equal, modeling.py:487).
 * Asynchronous on `stream`. */
int et_forward_ids(et_handle_t handle, const int* input_ids, const int* token_type_ids, const int* mask,
                   void* sequence_out, void* pooled_out, int batch_size, int seq_len, void* stream);

/* Same with HOST buffers; waits for the results.  Only ids and masks go up
 * (12 bytes per position) and only the requested outputs come back. */
int et_forward_ids_host(et_handle_t handle, const int* input_ids_host, const int* token_type_ids_host,
                        const int* mask_host, void* sequence_out_host, void* pooled_out_host,
                        int batch_size, int seq_len, int* valid_word_num_out);

/* The pooler alone on a packed tensor [T, H] (e.g. the last et_layer output):
 * pooled_out[b] = tanh(packed[cu_seqlens[b]] * kernel + bias).  cu_seqlens
 * NULL selects the array of the last et_input/et_forward* call on the handle. */
int et_pooler(et_handle_t handle, const void* packed, const int* cu_seqlens, void* pooled_out,
              int batch_size, int seq_len, void* stream);

/* Packed [T, H] result of the last et_forward* call (device pointer, valid
 * until the next call on the handle) and the device pointer to T. */
int et_last_packed_output(et_handle_t handle, const void** packed, const int** valid_word_num);

/* ---- CUDA-graph replay ------------------------------------------------------
 * The valid-token count never leaves the device, so one forward pass is a fixed
 * sequence of launches for given buffers and (B, S): it can be captured once
 * and replayed for every batch written into the same buffers, whatever its
 * mask.  That removes the host's launch cost (about 90 launches per 12-layer
 * pass), which dominates for small batches.  No reference counterpart.
 * et_graph_capture runs et_forward(from_tensor, mask, out, B, S) once on a
 * stream of the handle (so the buffers must hold a valid batch) and records
 * it; et_graph_capture_ids does the same for et_forward_ids.  A handle holds
 * one captured pass; capturing again replaces it; registering embedding or
 * pooler weights discards it.  et_graph_launch enqueues the pass on `stream`.
 * Per-kernel timing (et_set_profiling) does not see replayed kernels; their
 * launch counts are added per replay. */
int et_graph_capture(et_handle_t handle, const void* from_tensor, const int* mask, void* out,
                     int batch_size, int seq_len);
int et_graph_capture_ids(et_handle_t handle, const int* input_ids, const int* token_type_ids,
                         const int* mask, void* sequence_out, void* pooled_out, int batch_size,
                         int seq_len);
int et_graph_launch(et_handle_t handle, void* stream);
int et_graph_release(et_handle_t handle);

/* Reads the device status word (synchronises `stream`): 0 = no device-side
 * wait expired since the last call.  Non-zero encodes kernel id and wait site;
 * the word is cleared. */
int et_device_status(et_handle_t handle, void* stream, int* out_status);

/* Device arrays produced by the last et_input/et_forward on this handle:
 * cu_seqlens int32[B+1], seq_len int32[B], padding_offset int32[T],
 * prefix_sum int32[B*S].  Valid until the next call on the handle. */
int et_last_padding_info(et_handle_t handle, const int** cu_seqlens, const int** seq_len,
                         const int** padding_offset, const int** prefix_sum);

/* Per-kernel accounting.  Launch counts are always kept; with profiling
 * enabled a CUDA event is recorded on the launching stream after every
 * launcher call (and before the first one of an API call), so a kernel's time
 * runs from the end of the launch before it to its own end and the categories
 * add up to the whole call.  et_get_profile waits for the recorded events and
 * returns, per category, the summed device time in ms and the number of
 * kernels launched since the last reset. */
enum {
  ET_PROF_PADDING_OFFSETS = 0,
  ET_PROF_REMOVE_PADDING = 1,
  ET_PROF_GEMM_QKV = 2,
  ET_PROF_ATTENTION = 3,
  ET_PROF_GEMM_ATTN_OUT = 4,
  ET_PROF_LAYERNORM = 5,
  ET_PROF_GEMM_FFN1 = 6,
  ET_PROF_GEMM_FFN2 = 7,
  ET_PROF_RESTORE_PADDING = 8,
  ET_PROF_EMBEDDING = 9,
  ET_PROF_POOLER = 10,
  ET_PROF_NUM = 11
};
int et_set_profiling(et_handle_t handle, int enable);
int et_get_profile(et_handle_t handle, double* ms_out, long long* launches_out, int reset);

/* Utility for bindings without a CUDA runtime of their own: copies `bytes`
 * from device to host on `stream` and waits for it. */
int et_copy_to_host(void* dst_host, const void* src_device, size_t bytes, void* stream);

/* 0 (default): tensor-core kernels - tcgen05 GEMMs and attention for an fp16
 * handle, the tf32-split tcgen05 GEMM and the tf32-split mma.sync attention
 * for an fp32 handle.  1: CUDA-core GEMMs and attention for both
 * (plain fp32 FMA arithmetic; for debugging and as a second opinion). */
int et_set_debug_simt(et_handle_t handle, int use_simt);

/* 0 (default): no LayerNorm inside a projection kernel's own output rows (see
 * et_set_deferred_layernorm for what runs instead).
 * 1 (fp16 handles with hidden a multiple of 256 up to 1024): both LayerNorms run
 * inside the projection kernels (et_gemm_fused epilogues 6 and 5): 5 launches per
 * layer and no pre-LayerNorm tensor read back from HBM.  Same results (the same
 * arithmetic in the same order).  Measured on B200 it is slower at the benchmark
 * sizes, which is why it is opt-in.  Changing the setting drops recorded graphs. */
int et_set_fused_layernorm(et_handle_t handle, int enable);
/* 1 (default on fp16 handles whose hidden size, at most 1024, and ffn_dim are
 * multiples of 256):
 * inside the whole-stack calls (et_forward*, the graph and host-buffer
 * calls) no LayerNorm between the projections is materialised: the two
 * hidden-wide projections leave x + sublayer(x) and its row statistics, the
 * projections behind them run on weights with the LayerNorm's gamma folded in
 * (et_gemm_deferred_norm below), and only the last layer's LayerNorm runs as a
 * kernel: 5 launches per layer + 1 instead of 7.  et_layer always materialises
 * its output.  0, fp32 handles and the other widths: one add_bias_input_layernorm
 * kernel behind the attention-output and the second feed-forward projection, as
 * in the reference (tf_op/bert_transformer_op.cu.cc:211-213,242-246).
 * et_set_fused_layernorm(1) takes precedence.  Changing the setting drops
 * recorded graphs. */
int et_set_deferred_layernorm(et_handle_t handle, int enable);

/* Chunking of the host-buffer call (et_forward_host): number of chunks, share of
 * a middle chunk when the first and the last have 1 (0: the handle found that
 * chunking does not pay for the last shape and sends the batch in one piece),
 * and whether the handle has settled on it by its own measurement: calls of a
 * (batch, seq) shape start with 1:6:1; the first replayed call times the upload
 * and two passes of different size, a model of the copies nothing overlaps plus
 * the fixed cost of the extra passes proposes shares, and the proposal is kept if
 * two replayed calls with it beat two with 1:6:1.  ETB_HOST_MID_SHARE fixes the
 * share instead. */
int et_host_chunk_shares(et_handle_t handle, int* chunks, int* mid_share, int* measured);

/* Failure-detection self-test: launches one CTA whose bounded wait (2 ms, on a
 * barrier nobody arrives at; no copy or MMA in flight) runs out, so that it
 * records a code in the handle's status word and returns normally.  The next
 * et_device_status reports (15 << 8 | 1) and clears the word; the host-buffer
 * calls map a non-zero word to ET_DEVICE_TIMEOUT.  No reference counterpart. */
int et_selftest_wait_timeout(et_handle_t handle, void* stream);

/* ---- kernel-level entry points (one per reference launcher) --------------
 * dtype is an et_dtype_t; all pointers are device pointers; `valid_word_num`
 * is a DEVICE pointer to T (row counts are never read back to the host). */

/* exclusiveScan_kernelLauncher (cuda/cuda_kernels.cu:704-718) fused with the
 * index outputs of compress_bert_input (cuda/cuda_kernels.cu:292-299).  Any
 * output pointer may be NULL.  `scratch` must hold batch_size ints. */
int et_padding_offsets(const int* mask, int batch_size, int seq_len, int* prefix_sum,
                       int* valid_word_num, int* batch_idx, int* word_idx, int* seq_len_out,
                       int* cu_seqlens, int* padding_offset, int* scratch, void* stream);

/* et_padding_offsets for callers that cannot hand over device scratch.  It has
 * no counterpart in the reference (whose input functor takes its scratch from
 * TensorFlow's allocator).  Some hosts of this library cannot call cudaMalloc
 * or any allocator around the call: a framework op that must not re-enter its
 * own allocator, code running while a memory pool is frozen, a bare C plug-in
 * with no device allocator.  The per-row token counts that et_padding_offsets
 * keeps in `scratch` live instead in a device array that is part of the
 * library image: ET_NOALLOC_MAX_BATCH ints (64 KiB) on every GPU that loads
 * the library, until the process exits.  The call itself allocates nothing
 * (no cudaMalloc/cudaFree, no allocating library routine).
 *   - batch_size > ET_NOALLOC_MAX_BATCH is rejected with ET_INVALID_ARGUMENT
 *     (text in et_last_error(NULL)); seq_len is not limited.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress) and caches it; make that first call before any
 *     stream capture begins on that device.
 *   - All calls on a device share the one array.  Nothing in it has to be
 *     cleared between calls (each call overwrites the entries it reads), but
 *     two calls that overlap on the GPU (different streams) race: serialise
 *     them.  Outputs are those of et_padding_offsets, bit for bit. */
#define ET_NOALLOC_MAX_BATCH 16384
int et_padding_offsets_noalloc(const int* mask, int batch_size, int seq_len, int* prefix_sum,
                               int* valid_word_num, int* batch_idx, int* word_idx, int* seq_len_out,
                               int* cu_seqlens, int* padding_offset, void* stream);

/* compressBertInput_kernelLauncher (cuda/cuda_kernels.cu:340-372), copy part. */
int et_remove_padding(int dtype, const void* from_tensor, const int* batch_idx, const int* word_idx,
                      const int* valid_word_num, void* to_tensor, int batch_size, int seq_len,
                      int hidden, void* stream);

/* cudaMemsetAsync + restoreBertOutput_kernelLauncher
 * (tf_op/bert_transformer_op.cu.cc:354-360, cuda/cuda_kernels.cu:429-459) in one pass. */
int et_restore_padding(int dtype, const void* from_tensor, const int* batch_idx, const int* word_idx,
                       const int* valid_word_num, void* to_tensor, int batch_size, int seq_len,
                       int hidden, void* stream);

/* Embedding lookup + token-type and position rows + LayerNorm
 * (sample/tensorflow/modeling.py:380-521) for the valid tokens only: packed row
 * v = (batch_idx[v], word_idx[v]) receives
 * LN(word_table[input_ids[b,s]] + type_table[token_type_ids[b,s]] + position_table[s]).
 * token_type_ids NULL = all zero; type_table / position_table NULL = that term
 * is absent.  An id outside its table contributes a zero row (TensorFlow's GPU
 * gather / one-hot matmul).  The caller guarantees seq_len <= rows of
 * position_table. */
int et_embedding_layernorm(int dtype, const int* input_ids, const int* token_type_ids,
                           const int* batch_idx, const int* word_idx, const int* valid_word_num,
                           const void* word_table, int vocab_size, const void* type_table,
                           int type_vocab_size, const void* position_table, const void* gamma,
                           const void* beta, float eps, void* to_tensor, int batch_size, int seq_len,
                           int hidden, void* stream);

/* First-token rows of a packed tensor (sample/tensorflow/modeling.py:228):
 * out[b] = packed[cu_seqlens[b]], a zero row for a sequence without tokens. */
int et_gather_first_tokens(int dtype, const void* packed, const int* cu_seqlens, void* out,
                           int batch_size, int max_tokens, int hidden, void* stream);

/* add_QKV_bias_padding_kernelLauncher (cuda/attention.cu:106-242) without the
 * re-padding: q,k,v packed [T,H] + bias -> head-major packed [3, heads, max_tokens, d]. */
int et_add_qkv_bias_transpose(int dtype, const void* q, const void* bias_q, const void* k,
                              const void* bias_k, const void* v, const void* bias_v, void* qkv_out,
                              const int* valid_word_num, int max_tokens, int head_num,
                              int size_per_head, void* stream);

/* add_bias_act_kernelLauncher (cuda/cuda_kernels.cu:136-150): in place on [T, n]. */
int et_add_bias_gelu(int dtype, void* out, const void* bias, const int* valid_word_num,
                     int max_tokens, int n, void* stream);

/* add_bias_input_layernorm_kernelLauncher (cuda/cuda_kernels.cu:238-271): in place on out [T, n]. */
int et_add_bias_input_layernorm(int dtype, void* out, const void* input, const void* bias,
                                const void* gamma, const void* beta, const int* valid_word_num,
                                int max_tokens, int n, float eps, void* stream);

/* The attention block of the layer functor (batched QK^T, softmax_kernel,
 * batched P*V, transpose_rm_padding: tf_op/bert_transformer_op.cu.cc:158-191,
 * cuda/attention.cu:249-492) on the packed layout.  q/k/v are addressed as
 * base + token*token_stride + head*head_stride (elements): either heads side
 * by side inside a token row ([T, 3H] as the fused projection writes it) or
 * one [max_tokens, d] block per head; ctx is packed [T, heads*d].  q/k/v/ctx
 * hold max_tokens rows (rows past T are never needed, reads past max_tokens
 * never happen).  use_simt = 0: tensor cores (fp16: TMA-fed mma.sync, any
 * length; fp32: mma.sync with tf32 operands, three products per fp32 product,
 * fp32 accuracy); use_simt = 1: the CUDA-core kernel (plain fp32 FMA). */
int et_attention(int dtype, const void* q, const void* k, const void* v, long long token_stride,
                 long long head_stride, void* ctx, const int* cu_seqlens, int batch_size,
                 int max_seq_len, int max_tokens, int head_num, int size_per_head, int use_simt,
                 int* status_word, void* stream);

/* The attention block under a GENERAL [B,S,S] mask (element type = dtype,
 * 1 = attend), for callers whose mask is not the key-only tile of the input
 * mask (causal, banded, per-pair masks).  Semantics of the reference op
 * (cuda/attention.cu:106-242, 249-382): a query sees all S key positions,
 * score*1/sqrt(d) + (1 - m)*(-10000); padded key positions take part with
 * K = V = 0, exactly as the reference's zero-filled padded buffers make them.
 * CUDA-core kernel, fp32 arithmetic, any dtype and sequence length; fp16 with
 * seq_len <= 128 has a tensor-core form, et_attention_tiles_general_mask, which
 * the handle uses by itself.  pos_row_scratch: batch_size*seq_len ints. */
int et_attention_general_mask(int dtype, const void* q, const void* k, const void* v, long long token_stride,
                              long long head_stride, void* ctx, const void* attr_mask, const int* cu_seqlens,
                              const int* batch_idx, const int* word_idx, const int* valid_word_num,
                              int* pos_row_scratch, int batch_size, int seq_len, int head_num,
                              int size_per_head, void* stream);

/* Cross-attention on packed tensors: from_seq_len != to_seq_len of the
 * sample model's attention_layer (sample/tensorflow/modeling.py:558-752; the
 * layer op itself rejects it, tf_op/bert_transformer_op.cc:130-131, and so does
 * et_layer).  Sequence b's queries are rows [cu_seqlens_q[b], cu_seqlens_q[b+1])
 * of q (row stride q_token_stride), its keys and values rows
 * [cu_seqlens_k[b], cu_seqlens_k[b+1]) of k / v (row stride kv_token_stride);
 * head h at column h * head_stride; ctx is packed [Tq, heads * 64].  Softmax over
 * the to-sequence's own keys (the key-only mask of the to-tensor); a query whose
 * to-sequence is empty gets a zero row.  CUDA-core kernel, fp32 arithmetic. */
int et_attention_cross(int dtype, const void* q, long long q_token_stride, const void* k, const void* v,
                       long long kv_token_stride, long long head_stride, void* ctx, const int* cu_seqlens_q,
                       const int* cu_seqlens_k, int batch_size, int max_seq_q, int max_seq_k, int head_num,
                       int size_per_head, void* stream);

/* The same attention block on the tcgen05 tensor cores, fp16, for batches whose
 * sequences have at most 128 tokens (max_seq_len <= 128).  A plan packs whole
 * sequences into tiles of at most 128 token rows; it depends only on
 * cu_seqlens, so it is made once per batch (et_attention_plan) and reused by
 * every layer (et_attention_tiles).  `plan` holds
 * et_attention_plan_ints(batch_size, max_tokens) ints of device memory.
 * q/k/v/ctx as for et_attention, additionally 32-byte aligned. */
size_t et_attention_plan_ints(int batch_size, int max_tokens);
int et_attention_plan(const int* cu_seqlens, int batch_size, int max_tokens, int* plan, void* stream);
int et_attention_tiles(const void* q, const void* k, const void* v, long long token_stride,
                       long long head_stride, void* ctx, const int* plan, int batch_size, int max_seq_len,
                       int max_tokens, int head_num, int size_per_head, int* status_word, void* stream);
/* The same kernel under a general attention mask attr_mask [B, seq_len, seq_len]
 * (fp16, 1 = attend), semantics of the reference op's masked softmax
 * (cuda/attention.cu:106-382: disallowed keys get -10000; a padded key position
 * takes part with K = V = 0, i.e. it weighs in the denominator when the mask
 * allows it).  batch_idx / word_idx: sequence and position of every packed row
 * (outputs of et_padding_offsets).  seq_len <= 128.  A query that may attend to
 * nothing gets the softmax over all seq_len keys (the TF graph's result). */
int et_attention_tiles_general_mask(const void* q, const void* k, const void* v, long long token_stride,
                                    long long head_stride, void* ctx, const int* plan, const void* attr_mask,
                                    const int* batch_idx, const int* word_idx, int batch_size, int seq_len,
                                    int max_tokens, int head_num, int size_per_head, int* status_word,
                                    void* stream);

/* cublasGemmEx call sites of the layer functor
 * (tf_op/bert_transformer_op.cu.cc:110-141,200-209,215-225,229-240):
 * C[M,N] = epilogue(A[M,K] * W[K,N] (+ bias)), W row-major [in,out] as the
 * reference passes it.  epilogue: 0 none, 1 +bias, 2 gelu(+bias), 3 tanh(+bias)
 * (the pooler's dense layer, sample/tensorflow/modeling.py:229-232).  M is read
 * from the device (`m_ptr`), `max_m` bounds it.  The tcgen05 path needs
 * `w_packed` = the [N,K] K-major copy made by et_pack_weight (w may be NULL);
 * the CUDA-core path (use_simt, always for fp32) reads `w`. */
int et_gemm(int dtype, const void* a, const void* w, const void* w_packed, const void* bias, void* c,
            const int* m_ptr, int max_m, int n, int k, int epilogue, int use_simt, int* status_word,
            void* stream);
int et_pack_weight(int dtype, const void* w, void* w_packed, int k, int n, void* stream);

/* The tcgen05 GEMM (fp16) with the epilogues that take the layer's residual:
 *   4  C = A*W + bias + residual                      (the second feed-forward
 *      projection followed by a separate LayerNorm)
 *   5  C = LayerNorm(A*W + bias + residual), bias and residual added in the
 *      accumulator epilogue (tf_op/bert_transformer_op.cu.cc:229-246 in one kernel)
 *   6  the same result with bias and residual added where the rows are
 *      normalised (tf_op/bert_transformer_op.cu.cc:200-213 in one kernel)
 * For 5 and 6 (N a multiple of 256, at most 1024) every 32-row block of C is
 * normalised in place by the kernel as soon as its last column tile has been
 * stored: semantics of add_bias_input_layernorm (cuda/cuda_kernels.cu:157-236),
 * fp32 statistics, eps <= 0 means 1e-6.  `row_counters`: 8 * ceil(max_m / 256)
 * ints (one per 32 rows of the 256-row tiles), zero before the call; the kernel
 * leaves them zero.  `residual` is [max_m, N]
 * and must not alias c. */
int et_gemm_fused(const void* a, const void* w_packed, const void* bias, const void* residual,
                  const void* gamma, const void* beta, float eps, int* row_counters, void* c,
                  const int* m_ptr, int max_m, int n, int k, int epilogue, int* status_word, void* stream);

/* The LayerNorm that is never materialised.  A projection whose input is
 * LN(x) = (x - mu) * rstd * gamma + beta can run on x itself with gamma folded
 * into its weights: LN(x) W + b = rstd * (x W' - mu * colsum(W')) + (beta W + b),
 * W' = diag(gamma) W.  No counterpart in the reference, which runs
 * add_bias_input_layernorm (cuda/cuda_kernels.cu:157-271) as a kernel of its own
 * between the projections (tf_op/bert_transformer_op.cu.cc:211-213,242-246);
 * the handle uses these inside et_forward* when et_set_deferred_layernorm is on.
 * et_fold_layernorm: w_packed [N,K] (et_pack_weight), bias [N], gamma / beta [K]
 * -> w_folded [N,K] = gamma-scaled weights with the mean over K taken from every
 * output row (it multiplies sum_k (x_k - mu) = 0, and removes the large term
 * mu * colsum that would otherwise cancel in the epilogue), csum [N] = the row
 * sums fp16 rounding leaves, bias_folded [N] (fp16).
 * et_gemm_deferred_norm (fp16, n % 256 == 0): epilogue
 *   7  C = rstd[r] * (A W' - mu[r] * csum[n]) + bias[n]          (bias = bias_folded)
 *   8  the same, then GELU
 *   9  C = A W + bias[n] + LN(residual)[r,n], LN taken on the fly from `residual`
 *      [M,N] with gamma / beta [N] (NULL: ones / zeros); and stats_out
 *      [rows, 2 * N/64] receives (sum, sum of squares) of every 64-column piece
 *      of every stored row of C.
 * stats_in: such statistics of A's rows (7, 8: [rows, 2 * K/64]) or of
 * residual's rows (9: [rows, 2 * N/64]); NULL: mu = 0, rstd = 1.  Rows of the
 * statistics buffers: max_m rounded up to a multiple of 256. */
int et_fold_layernorm(const void* w_packed, const void* bias, const void* gamma, const void* beta, void* w_folded,
                      void* csum, void* bias_folded, int n, int k, void* stream);
int et_gemm_deferred_norm(const void* a, const void* w_packed, const void* bias, const void* csum,
                          const void* residual, const void* gamma, const void* beta, float eps,
                          const float* stats_in, float* stats_out, void* c, const int* m_ptr, int max_m, int n,
                          int k, int epilogue, int* status_word, void* stream);

/* The same call sites for the FP32 OperationType on the tensor cores, keeping
 * fp32 accuracy: every operand is split into two tf32 numbers, x = hi + lo with
 * hi = round_to_tf32(x) (et_split_tf32; hi or lo may be x itself), and the
 * product is hi*hi + hi*lo + lo*hi accumulated in fp32 - one tcgen05 kind::tf32
 * GEMM over a K axis three times as long.  a_hi/a_lo are [max_m, K], w_hi/w_lo
 * the halves of the [N, K] K-major copy made by et_pack_weight; N a multiple of
 * 128, K of 32; epilogue as for et_gemm.  No reference counterpart (the
 * reference's fp32 path is cuBLAS SGEMM). */
int et_split_tf32(const float* x, float* hi, float* lo, const int* rows_ptr, int max_rows, int cols,
                  void* stream);
int et_gemm_fp32_tensor(const float* a_hi, const float* a_lo, const float* w_hi, const float* w_lo,
                        const float* bias, float* c, const int* m_ptr, int max_m, int n, int k, int epilogue,
                        int* status_word, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* ET_B200_H_ */
