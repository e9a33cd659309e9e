// Host side of the encoder path and its C ABI (include/et_b200.h): handle,
// weight repacking, workspace, the three operators and the whole-path calls.
// It plays the role of the reference's GPU functors
// (tf_op/bert_transformer_op.cu.cc:33-373) without TensorFlow: the caller's
// stream and buffers come in through POD structs, work is only enqueued, and
// the valid-token count never travels to the host between kernels.
#include "../../include/et_b200.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <type_traits>
#include <utility>
#include <chrono>
#include <vector>

#include "common.cuh"
#include "ptx_sm100.cuh"

using namespace etb;

namespace {

inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct LayerWeights {
  // row-major [in, out] copies (QKV concatenated along out) for the CUDA-core GEMM
  void* wqkv = nullptr;  // [H, 3H]
  void* wo = nullptr;    // [H, H]
  void* w1 = nullptr;    // [H, F]
  void* w2 = nullptr;    // [F, H]
  // K-major [out, in] copies for the tcgen05 GEMM (fp16 handles only)
  void* wqkv_t = nullptr;  // [3H, H]
  void* wo_t = nullptr;    // [H, H]
  void* w1_t = nullptr;    // [F, H]
  void* w2_t = nullptr;    // [H, F]
  // fp32 handles: the K-major copies above hold rn_tf32(W) and these W - rn_tf32(W)
  // (the two halves of the three-product tf32 split, gemm_tf32x3.cu)
  void* wqkv_lo = nullptr;
  void* wo_lo = nullptr;
  void* w1_lo = nullptr;
  void* w2_lo = nullptr;
  void* bqkv = nullptr;    // [3H]
  void* bo = nullptr;
  void* ln1_gamma = nullptr;
  void* ln1_beta = nullptr;
  void* b1 = nullptr;      // [F]
  void* b2 = nullptr;
  void* ln2_gamma = nullptr;
  void* ln2_beta = nullptr;
  // fp16 handles, deferred LayerNorm: the two projections that consume a LayerNorm, with its gamma
  // folded into their weights (K-major [out, in]), the column sums of the folded weights, and
  // bias + beta W.  wqkv_f folds the LayerNorm that closes the layer BEFORE this one.
  void* wqkv_f = nullptr;
  void* cqkv = nullptr;
  void* bqkv_f = nullptr;
  void* w1_f = nullptr;
  void* c1 = nullptr;
  void* b1_f = nullptr;
  bool ready = false;
};

// Embedding tables and pooler weights (the stages in front of and behind the stack).
struct ModelWeights {
  void* word = nullptr;   // [vocab, H]
  void* type = nullptr;   // [type_vocab, H] or null
  void* pos = nullptr;    // [max_pos, H] or null
  void* emb_gamma = nullptr;
  void* emb_beta = nullptr;
  int vocab = 0, type_vocab = 0, max_pos = 0;
  float emb_eps = 1e-12f;
  bool emb_ready = false;
  void* pool_w = nullptr;    // [H, H] row-major [in, out]
  void* pool_w_t = nullptr;  // [H, H] K-major copy for the tcgen05 GEMM (fp16 handles)
  void* pool_b = nullptr;
  bool pool_ready = false;
  std::vector<void*> emb_allocs, pool_allocs;
};

struct Workspace {
  size_t cap_tokens = 0;  // rows every token buffer can hold (multiple of 128)
  void* x = nullptr;      // [cap, H]  packed activations (layer input/output)
  void* qkv = nullptr;    // [cap, 3H]
  void* ctx = nullptr;    // [cap, H]
  void* att = nullptr;    // [cap, H]
  void* ffn = nullptr;    // [cap, F]
  void* stage_in = nullptr;   // [B*S, H] device staging for the host-buffer call
  void* stage_out = nullptr;  // [B*S, H]
  int* stage_mask = nullptr;  // [B*S]
  int* stage_ids = nullptr;   // [B*S] token ids of the host-buffer model call
  int* stage_types = nullptr; // [B*S]
  void* first_tok = nullptr;  // [round_up(B,128), H] first-token rows (pooler input)
  void* pooled = nullptr;     // [round_up(B,128), H] pooler output staging
  int* pool_m = nullptr;      // device copy of the batch size (row count of the pooler GEMM)
  int* batch_idx = nullptr;
  int* word_idx = nullptr;
  int* padding_offset = nullptr;
  int* prefix_sum = nullptr;
  int* seq_len = nullptr;     // [B]
  int* cu_seqlens = nullptr;  // [B+1]
  int* lens_scratch = nullptr;
  int* attn_plan = nullptr;   // tile plan of the tcgen05 attention (made once per batch)
  int* pos_row = nullptr;     // [B*S] position -> packed row (general-mask attention)
  float* a_hi = nullptr;      // fp32 handles: [cap, H] tf32 halves of a projection's input
  float* a_lo = nullptr;
  float* ffn_lo = nullptr;    // fp32 handles: [cap, F] remainder of the GELU output (its tf32 half is in ffn)
  int* ln_counters = nullptr; // [cap / 32] column counts of the GEMMs that normalise their own output rows
  float* stats_x = nullptr;   // deferred LayerNorm: (sum, sum of squares) per 64-column piece of the rows of x
  float* stats_att = nullptr; // ... and of att
  int* valid_word_num = nullptr;
  int* status = nullptr;
  std::vector<void*> allocations;
};

// Every workspace buffer with its size for a (batch, seq) capacity: et_create allocates from this
// list and et_workspace_bytes adds it up, so the two cannot drift apart.
struct WsItem {
  void** slot;
  size_t bytes;
};
// Row counters of the GEMMs that normalise their own output: one per 32 rows of the 256-row tiles
// that cover `rows` rows.
inline size_t ln_counter_ints(size_t rows) { return round_up(rows, 256) / 32 + 8; }
inline size_t ws_round(size_t bytes) { return round_up(bytes == 0 ? 16 : bytes, 256); }

// The LayerNorm can be deferred into the projections around it (fp16 tensor-core path, every
// projection on the CTA-pair kernel, statistics in 64-column pieces of rows of 128 * j columns).
bool defer_eligible(const et_config_t& c) {
  const int H = c.head_num * c.size_per_head;
  // rows of up to 1024 columns: the epilogues hold a row's partial sums in registers (width / 128 vectors)
  return c.dtype == ET_FP16 && H % 256 == 0 && H <= 1024 && c.ffn_dim % 256 == 0 && c.num_layers > 0;
}

std::vector<WsItem> workspace_items(const et_config_t& c, size_t batch, size_t seq, Workspace& ws) {
  const size_t H = static_cast<size_t>(c.head_num) * c.size_per_head, f = c.ffn_dim;
  const size_t e = c.dtype == ET_FP16 ? 2 : 4;
  const size_t bs = batch * seq, cap = round_up(bs, 128), bpad = round_up(batch, 128);
  const bool f32 = c.dtype == ET_FP32;
  auto I = [](int** p) { return reinterpret_cast<void**>(p); };
  auto F = [](float** p) { return reinterpret_cast<void**>(p); };
  return {
      {&ws.x, cap * H * e}, {&ws.qkv, cap * 3 * H * e}, {&ws.ctx, cap * H * e}, {&ws.att, cap * H * e},
      {&ws.ffn, cap * f * e}, {&ws.stage_in, bs * H * e}, {&ws.stage_out, bs * H * e},
      {I(&ws.stage_mask), bs * 4}, {I(&ws.stage_ids), bs * 4}, {I(&ws.stage_types), bs * 4},
      {&ws.first_tok, bpad * H * e}, {&ws.pooled, bpad * H * e}, {I(&ws.pool_m), 4},
      {I(&ws.batch_idx), cap * 4}, {I(&ws.word_idx), cap * 4}, {I(&ws.padding_offset), cap * 4},
      {I(&ws.prefix_sum), cap * 4}, {I(&ws.seq_len), batch * 4}, {I(&ws.cu_seqlens), (batch + 1) * 4},
      {I(&ws.lens_scratch), batch * 4},
      {I(&ws.attn_plan), attention_plan_ints(static_cast<int>(batch), static_cast<int>(cap)) * 4},
      {I(&ws.pos_row), cap * 4},
      {F(&ws.a_hi), f32 ? cap * H * 4 : 0}, {F(&ws.a_lo), f32 ? cap * H * 4 : 0},
      {F(&ws.ffn_lo), f32 ? cap * f * 4 : 0},
      {I(&ws.ln_counters), ln_counter_ints(bs) * 4},
      {F(&ws.stats_x), defer_eligible(c) ? round_up(bs, 256) * (H / 64) * 2 * 4 : 0},
      {F(&ws.stats_att), defer_eligible(c) ? round_up(bs, 256) * (H / 64) * 2 * 4 : 0},
      {I(&ws.valid_word_num), 4}, {I(&ws.status), 4}};
}

}  // namespace

struct Profiler {
  bool enabled = false;
  long long launches[ET_PROF_NUM] = {};
  double ms[ET_PROF_NUM] = {};
  // A span ends with its own event and starts at the end event of the launch
  // before it in the same call (one record per launch instead of two); only
  // the first launch of a call records a start event of its own.
  struct Span { int cat; cudaEvent_t a, b; bool owns_a; };
  std::vector<Span> pending;
  std::vector<cudaEvent_t> free_events;
  cudaEvent_t chain = nullptr;       // end event of the previous launch of this call
  cudaStream_t chain_stream = nullptr;
  cudaEvent_t get() {
    if (!free_events.empty()) {
      cudaEvent_t e = free_events.back();
      free_events.pop_back();
      return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
  }
};

struct et_handle_s {
  et_config_t cfg{};
  Profiler prof;
  int hidden = 0;
  size_t esize = 0;
  float eps = 1e-6f;
  bool use_simt = false;
  bool general_mask = false;  // et_set_general_mask: et_layer reads attr_mask
  // Row order of consecutive kernels alternates ("snake"): a kernel that starts
  // with the rows its producer wrote last finds them in L2.  prev_ascending =
  // the previous kernel of the chain wrote its rows first-to-last.
  bool prev_ascending = true;
  // fp16 tensor-core path, et_set_fused_layernorm(1): bias + residual + LayerNorm run inside the two
  // N = hidden projection kernels (5 launches per layer instead of 7).  Off by default: measured on
  // B200 it breaks even behind the K = ffn_dim projection and loses behind the K = hidden one (the
  // eight epilogue warps of a CTA hide the LayerNorm's memory latency worse than the 16 warps per SM
  // of the LayerNorm kernel, and its L2 traffic slows the GEMM's operand loads).
  bool fuse_ln = false;
  // et_set_deferred_layernorm: inside a whole-stack call no LayerNorm between the projections is
  // materialised; producers leave row statistics, consumers run on folded weights (gemm_tcgen05.cu,
  // kEpiNorm*).  folded_ready: the folded weights match the layers' current weights.
  // defer_active: the stack being enqueued runs that way (set by stack_impl for run_layer).
  bool defer_ln = true;   // used where the configuration allows it (defer_eligible)
  bool folded_ready = false;
  bool defer_active = false;
  TensorMapCache maps;  // TMA descriptors of this handle's launches
  // general [B,S,S] mask of the pass being enqueued (null: key-only mask, fast kernels)
  const void* cur_attr_mask = nullptr;
  const int* cur_word_idx = nullptr;
  const int* cur_batch_idx = nullptr;
  std::vector<LayerWeights> layers;
  ModelWeights model;
  Workspace ws;
  cudaStream_t own_stream = nullptr;
  // host-buffer entry: copies run on their own streams so that the upload of
  // chunk i+1 and the download of chunk i-1 overlap the computation of chunk i
  static constexpr int kMaxChunks = 8;
  cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
  cudaEvent_t in_done[kMaxChunks] = {}, comp_done[kMaxChunks] = {};
  int host_chunks = 3;     // measured best on cfg2 (ETB_HOST_CHUNKS overrides)
  int host_mid_share = 6;  // share of a middle chunk when the first and the last have 1: 1:6:1
                           // (measured on cfg2: 2 -> 9.0 ms, 6 -> 8.8 ms, 8 -> 9.0 ms; ETB_HOST_MID_SHARE)
  bool host_share_auto = true;  // pick the middle share from the first call's measured copy and compute times
  bool host_share_measured = false;
  int tuned_batch = -1, tuned_seq = -1;  // shape the chunking was measured on (another shape measures again)
  // The model's choice is tried against the default shares on replayed calls (wall time of whole
  // calls, the best of two each): 0 = timing the default, 1 = timing the model's choice, 2 = settled.
  int tune_state = 0;
  int tune_replays = 0;
  int tune_model_share = 6;
  double tune_ms_default = 0.0, tune_ms_trial = 0.0;
  cudaEvent_t tune_ev[6] = {};  // upload start/end, pass start/end of the first and of the middle chunk
  size_t ws_bytes_allocated = 0;  // sum of the workspace buffers et_create allocated
  int* host_pinned = nullptr;  // [2 + kMaxChunks]: valid_word_num, status, per-chunk token counts
  // one captured forward pass (et_graph_capture*): replayed by et_graph_launch
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t graph_exec = nullptr;
  long long graph_launches[ET_PROF_NUM] = {};  // kernels per category inside the captured pass
  // et_forward_host replays one captured pass per chunk once the same
  // (batch, seq) shape has been seen twice in a row: the staging buffers are
  // fixed, so only the host's launch cost changes.  ETB_HOST_GRAPH=0 disables it.
  struct HostGraphs {
    int batch = -1, seq = -1, per = 0;  // per = number of chunks of the recorded shape
    int mid_share = 0;                  // chunk shares the graphs were recorded with
    bool simt = false;
    std::vector<cudaGraph_t> graphs;
    std::vector<cudaGraphExec_t> execs;
    std::vector<std::vector<long long>> launches;  // per chunk, per category
  } host_graphs;
  bool host_graph_enabled = true;
  int last_host_batch = -1, last_host_seq = -1;
  std::string last_error;
};

namespace {

thread_local std::string g_create_error;

}  // namespace
namespace etb {
void set_global_error(const std::string& msg) { g_create_error = msg; }
}  // namespace etb
namespace {

int set_error(et_handle_t h, int code, const std::string& msg) {
  if (h != nullptr) h->last_error = msg;
  else g_create_error = msg;
  return code;
}
int cuda_fail(et_handle_t h, cudaError_t e, const char* what) {
  return set_error(h, ET_CUDA_ERROR,
                   std::string("[ET][ERROR] CUDA runtime error: ") + cudaGetErrorString(e) + " in " + what);
}
// A kernel's bounded wait expired (status word != 0, already copied to host_pinned[1]): clear the
// word and the GEMMs' row counters (an aborted kernel may have left them half counted).
int device_timeout(et_handle_t h, cudaStream_t s);
#define ET_CUDA(h, expr)                                   \
  do {                                                     \
    cudaError_t e__ = (expr);                              \
    if (e__ != cudaSuccess) return cuda_fail(h, e__, #expr); \
  } while (0)

// Runs one launcher call; counts its kernels and, when profiling is on,
// times it with CUDA events on the launching stream.
#define ET_LAUNCH(h, cat, nkernels, stream, expr)                          \
  do {                                                                     \
    Profiler& pr__ = (h)->prof;                                            \
    cudaEvent_t ea__ = nullptr, eb__ = nullptr;                            \
    bool own__ = false;                                                    \
    if (pr__.enabled) {                                                    \
      eb__ = pr__.get();                                                   \
      if (pr__.chain != nullptr && pr__.chain_stream == (stream)) {        \
        ea__ = pr__.chain;                                                 \
      } else {                                                             \
        ea__ = pr__.get();                                                 \
        own__ = true;                                                      \
        if (ea__) cudaEventRecord(ea__, stream);                           \
      }                                                                    \
    }                                                                      \
    cudaError_t e__ = (expr);                                              \
    if (ea__ && eb__) {                                                    \
      cudaEventRecord(eb__, stream);                                       \
      pr__.pending.push_back({cat, ea__, eb__, own__});                    \
      pr__.chain = eb__;                                                   \
      pr__.chain_stream = (stream);                                        \
    }                                                                      \
    if (e__ != cudaSuccess) return cuda_fail(h, e__, #expr);               \
    pr__.launches[cat] += (nkernels);                                      \
  } while (0)

struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) ok = false;
    if (ok && prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// Clears the general-mask state of a pass on every way out of the call that set it, so that a
// call that fails half-way cannot leave the handle in general-mask mode for the next one.
struct MaskScope {
  et_handle_t h;
  MaskScope(et_handle_t handle, const void* attr_mask, const int* batch_idx, const int* word_idx) : h(handle) {
    h->cur_attr_mask = attr_mask;
    h->cur_batch_idx = batch_idx;
    h->cur_word_idx = word_idx;
  }
  ~MaskScope() {
    h->cur_attr_mask = nullptr;
    h->cur_batch_idx = nullptr;
    h->cur_word_idx = nullptr;
  }
};

int ws_alloc(et_handle_t h, void** p, size_t bytes) {
  bytes = ws_round(bytes);
  ET_CUDA(h, cudaMalloc(p, bytes));
  h->ws.allocations.push_back(*p);
  return ET_OK;
}

size_t workspace_bytes_for(const et_handle_s* h, size_t batch, size_t seq) {
  Workspace scratch;  // only the sizes are read
  size_t total = 0;
  for (const WsItem& it : workspace_items(h->cfg, batch, seq, scratch)) total += ws_round(it.bytes);
  return total;
}

template <typename T>
int pack_layer(et_handle_t h, LayerWeights& lw, const void* const* w, cudaStream_t s) {
  const int hid = h->hidden, f = h->cfg.ffn_dim;
  auto W = [&](int i) { return static_cast<const T*>(w[i]); };
  // row-major concat [H, 3H]
  for (int j = 0; j < 3; ++j)
    ET_CUDA(h, launch_copy_columns<T>(W(2 * j), static_cast<T*>(lw.wqkv), hid, hid, 3 * hid, j * hid, s));
  ET_CUDA(h, cudaMemcpyAsync(lw.wo, w[6], sizeof(T) * hid * hid, cudaMemcpyDeviceToDevice, s));
  ET_CUDA(h, cudaMemcpyAsync(lw.w1, w[10], sizeof(T) * hid * f, cudaMemcpyDeviceToDevice, s));
  ET_CUDA(h, cudaMemcpyAsync(lw.w2, w[12], sizeof(T) * f * hid, cudaMemcpyDeviceToDevice, s));
  if (lw.wqkv_t != nullptr) {
    for (int j = 0; j < 3; ++j)
      ET_CUDA(h, launch_transpose<T>(W(2 * j), static_cast<T*>(lw.wqkv_t) + static_cast<size_t>(j) * hid * hid,
                                     hid, hid, s));
    ET_CUDA(h, launch_transpose<T>(W(6), static_cast<T*>(lw.wo_t), hid, hid, s));
    ET_CUDA(h, launch_transpose<T>(W(10), static_cast<T*>(lw.w1_t), hid, f, s));
    ET_CUDA(h, launch_transpose<T>(W(12), static_cast<T*>(lw.w2_t), f, hid, s));
  }
  if (std::is_same<T, float>::value && lw.wqkv_lo != nullptr) {
    // in place: the K-major copy keeps rn_tf32(W), the second array gets the remainder
    struct { void* hi; void* lo; int rows, cols; } parts[] = {
        {lw.wqkv_t, lw.wqkv_lo, 3 * hid, hid}, {lw.wo_t, lw.wo_lo, hid, hid},
        {lw.w1_t, lw.w1_lo, f, hid}, {lw.w2_t, lw.w2_lo, hid, f}};
    for (auto& p : parts)
      ET_CUDA(h, launch_split_tf32(static_cast<const float*>(p.hi), static_cast<float*>(p.hi),
                                   static_cast<float*>(p.lo), nullptr, p.rows, p.cols, s));
  }
  for (int j = 0; j < 3; ++j)
    ET_CUDA(h, cudaMemcpyAsync(static_cast<T*>(lw.bqkv) + j * hid, w[2 * j + 1], sizeof(T) * hid,
                               cudaMemcpyDeviceToDevice, s));
  ET_CUDA(h, cudaMemcpyAsync(lw.bo, w[7], sizeof(T) * hid, cudaMemcpyDeviceToDevice, s));
  ET_CUDA(h, cudaMemcpyAsync(lw.ln1_beta, w[8], sizeof(T) * hid, cudaMemcpyDeviceToDevice, s));
  ET_CUDA(h, cudaMemcpyAsync(lw.ln1_gamma, w[9], sizeof(T) * hid, cudaMemcpyDeviceToDevice, s));
  ET_CUDA(h, cudaMemcpyAsync(lw.b1, w[11], sizeof(T) * f, cudaMemcpyDeviceToDevice, s));
  ET_CUDA(h, cudaMemcpyAsync(lw.b2, w[13], sizeof(T) * hid, cudaMemcpyDeviceToDevice, s));
  ET_CUDA(h, cudaMemcpyAsync(lw.ln2_beta, w[14], sizeof(T) * hid, cudaMemcpyDeviceToDevice, s));
  ET_CUDA(h, cudaMemcpyAsync(lw.ln2_gamma, w[15], sizeof(T) * hid, cudaMemcpyDeviceToDevice, s));
  lw.ready = true;
  return ET_OK;
}

int pack_layer_any(et_handle_t h, int layer, const void* const* w, cudaStream_t s) {
  LayerWeights& lw = h->layers[layer];
  return h->cfg.dtype == ET_FP16 ? pack_layer<__half>(h, lw, w, s) : pack_layer<float>(h, lw, w, s);
}

// Folded weights of every layer (deferred LayerNorm), once all layers have their weights.
int fold_all(et_handle_t h, cudaStream_t s) {
  h->folded_ready = false;
  if (!defer_eligible(h->cfg)) return ET_OK;
  for (const auto& lw : h->layers)
    if (!lw.ready) return ET_OK;
  const int hid = h->hidden, f = h->cfg.ffn_dim;
  auto H16 = [](const void* p) { return static_cast<const __half*>(p); };
  auto M16 = [](void* p) { return static_cast<__half*>(p); };
  for (size_t l = 0; l < h->layers.size(); ++l) {
    LayerWeights& lw = h->layers[l];
    ET_CUDA(h, launch_fold_layernorm(H16(lw.w1_t), H16(lw.b1), H16(lw.ln1_gamma), H16(lw.ln1_beta), M16(lw.w1_f),
                                     M16(lw.c1), M16(lw.b1_f), f, hid, s));
    if (l > 0) {
      const LayerWeights& prev = h->layers[l - 1];
      ET_CUDA(h, launch_fold_layernorm(H16(lw.wqkv_t), H16(lw.bqkv), H16(prev.ln2_gamma), H16(prev.ln2_beta),
                                       M16(lw.wqkv_f), M16(lw.cqkv), M16(lw.bqkv_f), 3 * hid, hid, s));
    }
  }
  h->folded_ready = true;
  return ET_OK;
}

// One encoder layer on the packed layout.  x_out may alias x_in.
// fp32 tensor path only: in_split_ready = the workspace's a_hi / a_lo already hold the tf32
// halves of x_in (the layer before wrote them); out_split = write those of x_out for the next
// layer.  Both are false for a layer called on its own, whose input may be anything.
template <typename T>
int run_layer(et_handle_t h, const LayerWeights& lw, const T* x_in, T* x_out, const int* t_ptr,
              int max_m, const int* cu_seqlens, int batch, int seq, cudaStream_t s,
              bool in_split_ready = false, bool out_split = false, int layer_index = -1) {
  const int hid = h->hidden, f = h->cfg.ffn_dim, heads = h->cfg.head_num, d = h->cfg.size_per_head;
  Workspace& ws = h->ws;
  T* qkv = static_cast<T*>(ws.qkv);
  T* ctx = static_cast<T*>(ws.ctx);
  T* att = static_cast<T*>(ws.att);
  T* ffn = static_cast<T*>(ws.ffn);
  auto B = [](const void* p) { return static_cast<const T*>(p); };
  const bool tc = std::is_same<T, __half>::value && !h->use_simt;
  const bool tc32 = std::is_same<T, float>::value && !h->use_simt;  // three-product tf32 split
  // direction for a kernel that can run either way / for one that only runs first-to-last
  auto turn = [&]() {
    const bool reverse = h->prev_ascending;
    h->prev_ascending = !reverse;
    return reverse;
  };
  auto forward_only = [&]() { h->prev_ascending = true; };

  // fp32 tensor path: a_lo_ready = the input already is its tf32 half with the remainder in
  // a_lo_ready (written so by the kernel before); c_lo = write the output split the same way.
  auto gemm = [&](const T* a, const void* w_rm, const void* w_t, const void* w_lo, const void* bias, T* c,
                  int n, int k, int epi, const float* a_lo_ready = nullptr, float* c_lo = nullptr) -> cudaError_t {
    if (tc)
      return launch_gemm_tcgen05(reinterpret_cast<const __half*>(a), static_cast<const __half*>(w_t),
                                 static_cast<const __half*>(bias), reinterpret_cast<__half*>(c), t_ptr,
                                 max_m, n, k, epi, ws.status, s, turn(), nullptr, &h->maps);
    if (tc32) {
      // w_t holds rn_tf32(W), w_lo the remainder; the input is split the same way first
      const float* a_hi = reinterpret_cast<const float*>(a);
      const float* a_lo = a_lo_ready;
      if (a_lo == nullptr) {
        cudaError_t e = launch_split_tf32(a_hi, ws.a_hi, ws.a_lo, t_ptr, max_m, k, s);
        if (e != cudaSuccess) return e;
        forward_only();
        a_hi = ws.a_hi, a_lo = ws.a_lo;
      }
      return launch_gemm_tf32x3(a_hi, a_lo, static_cast<const float*>(w_t), static_cast<const float*>(w_lo),
                                static_cast<const float*>(bias), reinterpret_cast<float*>(c), t_ptr, max_m, n, k,
                                epi, ws.status, s, turn(), c_lo, &h->maps);
    }
    forward_only();
    return launch_gemm_simt<T>(a, B(w_rm), B(bias), c, t_ptr, max_m, n, k, epi, s);
  };

  // fp32 tensor path: the CUDA-core attention writes its output split for the projection behind
  // it (the halves of the QKV input in a_hi / a_lo are no longer needed by then)
  T* ctx_lo = (tc32 && h->cur_attr_mask == nullptr) ? reinterpret_cast<T*>(ws.a_lo) : nullptr;
  // Q,K,V projections + bias in one GEMM -> [T, 3H]
  // Deferred LayerNorm (inside a whole-stack call): x_in holds the un-normalised sum the layer before
  // left, with its row statistics in ws.stats_x; no LayerNorm kernel runs between the projections.
  const bool deferred = tc && h->defer_active && layer_index >= 0;
  auto H16 = [](const void* p) { return static_cast<const __half*>(p); };
  const int stat_slots = hid / 64;
  if (deferred && layer_index > 0) {
    GemmLayerNorm nin;
    nin.eps = h->eps;
    nin.stats_in = ws.stats_x;
    nin.stat_slots = stat_slots;
    nin.csum = H16(lw.cqkv);
    ET_LAUNCH(h, ET_PROF_GEMM_QKV, 1, s,
              launch_gemm_tcgen05(H16(x_in), H16(lw.wqkv_f), H16(lw.bqkv_f), reinterpret_cast<__half*>(qkv), t_ptr,
                                  max_m, 3 * hid, hid, kEpiNormIn, ws.status, s, turn(), nullptr, &h->maps, &nin));
  } else if (tc32 && in_split_ready)
    ET_LAUNCH(h, ET_PROF_GEMM_QKV, 1, s,
              gemm(reinterpret_cast<const T*>(ws.a_hi), lw.wqkv, lw.wqkv_t, lw.wqkv_lo, lw.bqkv, qkv, 3 * hid, hid,
                   kEpiBias, ws.a_lo));
  else
    ET_LAUNCH(h, ET_PROF_GEMM_QKV, tc32 ? 2 : 1, s, gemm(x_in, lw.wqkv, lw.wqkv_t, lw.wqkv_lo, lw.bqkv, qkv, 3 * hid, hid, kEpiBias));
  // attention straight from the [T, 3H] buffer to packed context [T, H]
  const bool masked = h->cur_attr_mask != nullptr;
  if (masked && tc && seq <= 128)
    // general mask on the tensor cores: the packed-tile kernel with the mask read per (query, key)
    ET_LAUNCH(h, ET_PROF_ATTENTION, 1, s,
              launch_attention_tcgen05(reinterpret_cast<const __half*>(qkv),
                                       reinterpret_cast<const __half*>(qkv) + hid,
                                       reinterpret_cast<const __half*>(qkv) + 2 * hid, 3LL * hid, d,
                                       reinterpret_cast<__half*>(ctx), ws.attn_plan, batch, max_m, heads, d,
                                       ws.status, s, turn(), &h->maps,
                                       static_cast<const __half*>(h->cur_attr_mask), h->cur_batch_idx,
                                       h->cur_word_idx, seq));
  else if (masked)
    ET_LAUNCH(h, ET_PROF_ATTENTION, 1, s,
              launch_attention_masked_simt<T>(qkv, qkv + hid, qkv + 2 * hid, 3LL * hid, d, ctx,
                                              B(h->cur_attr_mask), cu_seqlens, h->cur_word_idx, ws.pos_row,
                                              batch, seq, heads, d, s));
  else if (tc && seq <= 128)
    ET_LAUNCH(h, ET_PROF_ATTENTION, 1, s,
              launch_attention_tcgen05(reinterpret_cast<const __half*>(qkv),
                                       reinterpret_cast<const __half*>(qkv) + hid,
                                       reinterpret_cast<const __half*>(qkv) + 2 * hid, 3LL * hid, d,
                                       reinterpret_cast<__half*>(ctx), ws.attn_plan, batch, max_m, heads, d,
                                       ws.status, s, turn(), &h->maps));
  else if (tc)
    ET_LAUNCH(h, ET_PROF_ATTENTION, 1, s, launch_attention_tc(reinterpret_cast<const __half*>(qkv),
                                   reinterpret_cast<const __half*>(qkv) + hid,
                                   reinterpret_cast<const __half*>(qkv) + 2 * hid, 3LL * hid, d,
                                   reinterpret_cast<__half*>(ctx), cu_seqlens, batch, seq, max_m, heads, d,
                                   ws.status, s, &h->maps));
  else if (tc32)
    // fp32 handle: tensor cores at fp32 accuracy (three tf32 products per product), as its projections
    ET_LAUNCH(h, ET_PROF_ATTENTION, 1, s,
              launch_attention_tf32x3(reinterpret_cast<const float*>(qkv), reinterpret_cast<const float*>(qkv) + hid,
                                      reinterpret_cast<const float*>(qkv) + 2 * hid, 3LL * hid, d,
                                      reinterpret_cast<float*>(ctx), cu_seqlens, batch, seq, heads, d, s,
                                      reinterpret_cast<float*>(ctx_lo)));
  else
    ET_LAUNCH(h, ET_PROF_ATTENTION, 1, s, launch_attention_simt<T>(qkv, qkv + hid, qkv + 2 * hid, 3LL * hid, d, ctx, cu_seqlens,
                                        batch, seq, heads, d, s, ctx_lo));
  if (!(tc && seq <= 128)) forward_only();
  // fp16 tensor-core path: bias + residual + LayerNorm run inside the projection kernels (rows are
  // normalised in place as soon as their last column tile has been stored), no LayerNorm launch
  if (deferred) {
    // attention output projection: + bias + LN(x_in) taken on the fly (the layer input itself in the
    // first layer); leaves the sum in att and its row statistics in ws.stats_att
    GemmLayerNorm n1;
    n1.eps = h->eps;
    n1.stat_slots = stat_slots;
    if (layer_index > 0) {
      const LayerWeights& prev = h->layers[layer_index - 1];
      n1.stats_in = ws.stats_x;
      n1.gamma = H16(prev.ln2_gamma);
      n1.beta = H16(prev.ln2_beta);
    }
    n1.stats_out = ws.stats_att;
    ET_LAUNCH(h, ET_PROF_GEMM_ATTN_OUT, 1, s,
              launch_gemm_tcgen05(H16(ctx), H16(lw.wo_t), H16(lw.bo), reinterpret_cast<__half*>(att), t_ptr, max_m,
                                  hid, hid, kEpiNormResidual, ws.status, s, turn(), H16(x_in), &h->maps, &n1));
    // first feed-forward projection of LN1(att): folded weights, statistics, GELU
    GemmLayerNorm n2;
    n2.eps = h->eps;
    n2.stats_in = ws.stats_att;
    n2.stat_slots = stat_slots;
    n2.csum = H16(lw.c1);
    ET_LAUNCH(h, ET_PROF_GEMM_FFN1, 1, s,
              launch_gemm_tcgen05(H16(att), H16(lw.w1_f), H16(lw.b1_f), reinterpret_cast<__half*>(ffn), t_ptr, max_m,
                                  f, hid, kEpiNormInGelu, ws.status, s, turn(), nullptr, &h->maps, &n2));
    // second: + bias + LN1(att) on the fly; leaves the sum in x_out and its statistics in ws.stats_x
    GemmLayerNorm n3;
    n3.eps = h->eps;
    n3.stats_in = ws.stats_att;
    n3.stat_slots = stat_slots;
    n3.gamma = H16(lw.ln1_gamma);
    n3.beta = H16(lw.ln1_beta);
    n3.stats_out = ws.stats_x;
    ET_LAUNCH(h, ET_PROF_GEMM_FFN2, 1, s,
              launch_gemm_tcgen05(H16(ffn), H16(lw.w2_t), H16(lw.b2), reinterpret_cast<__half*>(x_out), t_ptr, max_m,
                                  hid, f, kEpiNormResidual, ws.status, s, turn(), H16(att), &h->maps, &n3));
    return ET_OK;
  }
  const bool ln_in_gemm = tc && h->fuse_ln && gemm_layernorm_supported(hid);
  GemmLayerNorm gln;
  gln.eps = h->eps;
  gln.counters = ws.ln_counters;
  // attention output projection, then +bias +residual, LayerNorm
  // (fp32 tensor path: both LayerNorms also write their rows split for the projection behind them)
  T* ln_hi = tc32 ? reinterpret_cast<T*>(ws.a_hi) : nullptr;
  T* ln_lo = tc32 ? reinterpret_cast<T*>(ws.a_lo) : nullptr;
  if (ln_in_gemm) {
    gln.gamma = H16(lw.ln1_gamma);
    gln.beta = H16(lw.ln1_beta);
    ET_LAUNCH(h, ET_PROF_GEMM_ATTN_OUT, 1, s,
              launch_gemm_tcgen05(H16(ctx), H16(lw.wo_t), H16(lw.bo), reinterpret_cast<__half*>(att), t_ptr, max_m,
                                  hid, hid, kEpiLayerNorm, ws.status, s, turn(), H16(x_in), &h->maps, &gln));
  } else {
    ET_LAUNCH(h, ET_PROF_GEMM_ATTN_OUT, tc32 && ctx_lo == nullptr ? 2 : 1, s,
              gemm(ctx, lw.wo, lw.wo_t, lw.wo_lo, nullptr, att, hid, hid, kEpiNone,
                   reinterpret_cast<const float*>(ctx_lo)));
    ET_LAUNCH(h, ET_PROF_LAYERNORM, 1, s,
              launch_add_bias_input_layernorm<T>(att, x_in, B(lw.bo), B(lw.ln1_gamma), B(lw.ln1_beta), t_ptr, max_m,
                                                 hid, h->eps, s, turn(), ln_hi, ln_lo));
  }
  // feed-forward: bias + GELU fused into the first GEMM
  // (fp32 tensor path: the GELU output leaves the epilogue split for the second projection)
  ET_LAUNCH(h, ET_PROF_GEMM_FFN1, 1, s,
            gemm(tc32 ? reinterpret_cast<const T*>(ws.a_hi) : att, lw.w1, lw.w1_t, lw.w1_lo, lw.b1, ffn, f, hid,
                 kEpiBiasGelu, tc32 ? ws.a_lo : nullptr, tc32 ? ws.ffn_lo : nullptr));
  // fp16 tensor-core path: the second FFN projection adds its bias and the residual in its
  // epilogue (its K = F main loop leaves the epilogue warps idle time), so the LayerNorm
  // behind it reads one tensor instead of two.  The attention output projection (K = H) has
  // no such slack: there the rows' bias and residual are added where they are normalised.
  if (ln_in_gemm) {
    gln.gamma = H16(lw.ln2_gamma);
    gln.beta = H16(lw.ln2_beta);
    ET_LAUNCH(h, ET_PROF_GEMM_FFN2, 1, s,
              launch_gemm_tcgen05(H16(ffn), H16(lw.w2_t), H16(lw.b2), reinterpret_cast<__half*>(x_out), t_ptr, max_m,
                                  hid, f, kEpiResidualLayerNorm, ws.status, s, turn(), H16(att), &h->maps, &gln));
  } else if (tc) {
    ET_LAUNCH(h, ET_PROF_GEMM_FFN2, 1, s,
              launch_gemm_tcgen05(H16(ffn), H16(lw.w2_t), H16(lw.b2), reinterpret_cast<__half*>(x_out), t_ptr, max_m,
                                  hid, f, kEpiBiasResidual, ws.status, s, turn(), H16(att), &h->maps));
    ET_LAUNCH(h, ET_PROF_LAYERNORM, 1, s,
              launch_add_bias_input_layernorm<T>(x_out, nullptr, nullptr, B(lw.ln2_gamma), B(lw.ln2_beta), t_ptr,
                                                 max_m, hid, h->eps, s, turn()));
  } else {
    ET_LAUNCH(h, ET_PROF_GEMM_FFN2, 1, s,
              gemm(ffn, lw.w2, lw.w2_t, lw.w2_lo, nullptr, x_out, hid, f, kEpiNone, tc32 ? ws.ffn_lo : nullptr));
    const bool split2 = tc32 && out_split;
    ET_LAUNCH(h, ET_PROF_LAYERNORM, 1, s, launch_add_bias_input_layernorm<T>(x_out, att, B(lw.b2), B(lw.ln2_gamma), B(lw.ln2_beta),
                                                  t_ptr, max_m, hid, h->eps, s, turn(), split2 ? ln_hi : nullptr,
                                                  split2 ? ln_lo : nullptr));
  }
  return ET_OK;
}

int device_timeout(et_handle_t h, cudaStream_t s) {
  char msg[96];
  snprintf(msg, sizeof msg, "device-side wait expired, status word 0x%x", h->host_pinned[1]);
  cudaMemsetAsync(h->ws.status, 0, 4, s);
  cudaMemsetAsync(h->ws.ln_counters, 0, ln_counter_ints(h->ws.cap_tokens) * 4, s);
  cudaStreamSynchronize(s);
  return set_error(h, ET_DEVICE_TIMEOUT, msg);
}

int check_shape(et_handle_t h, int batch, int seq, int heads, int d) {
  if (batch < 0 || seq < 0) return set_error(h, ET_INVALID_ARGUMENT, "negative batch_size or seq_len");
  if (batch > h->cfg.max_batch_size)
    return set_error(h, ET_INVALID_ARGUMENT, "batch_size exceeds the handle's max_batch_size");
  if (seq > h->cfg.max_seq_len)
    return set_error(h, ET_INVALID_ARGUMENT, "seq_len exceeds the handle's max_seq_len");
  if (heads != h->cfg.head_num || d != h->cfg.size_per_head)
    return set_error(h, ET_INVALID_ARGUMENT, "head_num / size_per_head differ from the handle's");
  return ET_OK;
}

int input_impl(et_handle_t h, const et_input_param_t* p) {
  cudaStream_t s = static_cast<cudaStream_t>(p->stream);
  Workspace& ws = h->ws;
  ET_LAUNCH(h, ET_PROF_PADDING_OFFSETS, (p->batch_size > 0 && p->from_seq_len > 0) ? 2 : 1, s, launch_padding_offsets(p->mask, p->batch_size, p->from_seq_len, ws.prefix_sum,
                                    p->valid_word_num, p->batch_idx, p->word_idx, ws.seq_len,
                                    ws.cu_seqlens, ws.padding_offset, ws.lens_scratch, s));
  if (h->cfg.dtype == ET_FP16)
    ET_LAUNCH(h, ET_PROF_REMOVE_PADDING, 1, s, launch_remove_padding<__half>(static_cast<const __half*>(p->from_tensor), p->batch_idx,
                                             p->word_idx, p->valid_word_num,
                                             static_cast<__half*>(p->to_tensor), p->batch_size,
                                             p->from_seq_len, h->hidden, s));
  else
    ET_LAUNCH(h, ET_PROF_REMOVE_PADDING, 1, s, launch_remove_padding<float>(static_cast<const float*>(p->from_tensor), p->batch_idx,
                                            p->word_idx, p->valid_word_num,
                                            static_cast<float*>(p->to_tensor), p->batch_size,
                                            p->from_seq_len, h->hidden, s));
  return ET_OK;
}

int output_impl(et_handle_t h, const et_output_param_t* p) {
  cudaStream_t s = static_cast<cudaStream_t>(p->stream);
  if (h->cfg.dtype == ET_FP16)
    ET_LAUNCH(h, ET_PROF_RESTORE_PADDING, 1, s, launch_restore_padding<__half>(static_cast<const __half*>(p->from_tensor), p->batch_idx,
                                              p->word_idx, p->valid_word_num,
                                              static_cast<__half*>(p->to_tensor), p->batch_size,
                                              p->from_seq_len, h->hidden, s));
  else
    ET_LAUNCH(h, ET_PROF_RESTORE_PADDING, 1, s, launch_restore_padding<float>(static_cast<const float*>(p->from_tensor), p->batch_idx,
                                             p->word_idx, p->valid_word_num,
                                             static_cast<float*>(p->to_tensor), p->batch_size,
                                             p->from_seq_len, h->hidden, s));
  return ET_OK;
}

void graph_release(et_handle_t h);
int stack_impl(et_handle_t h, int batch, int seq, cudaStream_t s);
int restore_impl(et_handle_t h, void* out, int batch, int seq, cudaStream_t s);

int forward_impl(et_handle_t h, const void* from_tensor, const int* mask, void* out, int batch, int seq,
                 cudaStream_t s) {
  h->prof.chain = nullptr;  // other work may have been enqueued since the last call
  int rc = check_shape(h, batch, seq, h->cfg.head_num, h->cfg.size_per_head);
  if (rc != ET_OK) return rc;
  if (from_tensor == nullptr || mask == nullptr || out == nullptr)
    return set_error(h, ET_INVALID_ARGUMENT, "null tensor pointer");
  for (int l = 0; l < h->cfg.num_layers; ++l)
    if (!h->layers[l].ready) return set_error(h, ET_NOT_READY, "weights of a layer were never set");
  Workspace& ws = h->ws;
  et_input_param_t ip{};
  ip.from_tensor = from_tensor;
  ip.mask = mask;
  ip.valid_word_num = ws.valid_word_num;
  ip.batch_idx = ws.batch_idx;
  ip.word_idx = ws.word_idx;
  ip.batch_size = batch;
  ip.from_seq_len = seq;
  ip.head_num = h->cfg.head_num;
  ip.size_per_head = h->cfg.size_per_head;
  ip.to_tensor = ws.x;
  ip.stream = s;
  rc = input_impl(h, &ip);
  if (rc != ET_OK) return rc;
  rc = stack_impl(h, batch, seq, s);
  if (rc != ET_OK) return rc;
  return restore_impl(h, out, batch, seq, s);
}

// The layer stack in place on the packed tensor ws.x (attention tiles are
// planned once per batch).
int stack_impl(et_handle_t h, int batch, int seq, cudaStream_t s) {
  Workspace& ws = h->ws;
  int rc = ET_OK;
  h->prev_ascending = true;  // remove-padding / the embedding kernel write rows first-to-last
  const int max_m = batch * seq;
  const bool tiles = h->cfg.dtype == ET_FP16 && !h->use_simt && seq <= 128 && max_m > 0;
  if (tiles)  // the packed-tile attention serves key-only and general masks
    ET_LAUNCH(h, ET_PROF_PADDING_OFFSETS, 1, s,
              launch_attention_plan(ws.cu_seqlens, batch, max_m, ws.attn_plan, s));
  else if (h->cur_attr_mask != nullptr)
    ET_LAUNCH(h, ET_PROF_PADDING_OFFSETS, 1, s,
              launch_position_rows(ws.batch_idx, ws.word_idx, ws.valid_word_num, batch, seq, ws.pos_row, s));
  // No LayerNorm between the projections: x holds un-normalised sums from the first layer's end on,
  // and the last layer's LayerNorm is the one kernel that runs, behind the loop.
  h->defer_active =
      h->defer_ln && !h->fuse_ln && h->folded_ready && !h->use_simt && defer_eligible(h->cfg) && max_m > 0;
  for (int l = 0; l < h->cfg.num_layers; ++l) {
    if (h->cfg.dtype == ET_FP16)
      rc = run_layer<__half>(h, h->layers[l], static_cast<const __half*>(ws.x), static_cast<__half*>(ws.x),
                             ws.valid_word_num, max_m, ws.cu_seqlens, batch, seq, s, false, false, l);
    else
      rc = run_layer<float>(h, h->layers[l], static_cast<const float*>(ws.x), static_cast<float*>(ws.x),
                            ws.valid_word_num, max_m, ws.cu_seqlens, batch, seq, s, l > 0,
                            l + 1 < h->cfg.num_layers);
    if (rc != ET_OK) {
      h->defer_active = false;
      return rc;
    }
  }
  if (h->defer_active) {
    h->defer_active = false;
    const LayerWeights& last = h->layers.back();
    const bool reverse = h->prev_ascending;
    h->prev_ascending = !reverse;
    ET_LAUNCH(h, ET_PROF_LAYERNORM, 1, s,
              launch_add_bias_input_layernorm<__half>(static_cast<__half*>(ws.x), nullptr, nullptr,
                                                      static_cast<const __half*>(last.ln2_gamma),
                                                      static_cast<const __half*>(last.ln2_beta), ws.valid_word_num,
                                                      max_m, h->hidden, h->eps, s, reverse));
  }
  return ET_OK;
}

// Output op from the handle's packed tensor to a padded [B,S,H] buffer.
int restore_impl(et_handle_t h, void* out, int batch, int seq, cudaStream_t s) {
  Workspace& ws = h->ws;
  et_output_param_t op{};
  op.from_tensor = ws.x;
  op.valid_word_num = ws.valid_word_num;
  op.batch_idx = ws.batch_idx;
  op.word_idx = ws.word_idx;
  op.batch_size = batch;
  op.from_seq_len = seq;
  op.head_num = h->cfg.head_num;
  op.size_per_head = h->cfg.size_per_head;
  op.to_tensor = out;
  op.stream = s;
  return output_impl(h, &op);
}

// pooled_out[b] = tanh(packed[cu_seqlens[b]] * W + bias): first-token gather,
// then one GEMM whose epilogue adds the bias and applies tanh.
int pooler_impl(et_handle_t h, const void* packed, const int* cu_seqlens, void* pooled_out, int batch,
                int max_tokens, cudaStream_t s) {
  if (!h->model.pool_ready) return set_error(h, ET_NOT_READY, "pooler weights were never set");
  if (batch == 0) return ET_OK;
  Workspace& ws = h->ws;
  const ModelWeights& mw = h->model;
  const int hid = h->hidden;
  ET_LAUNCH(h, ET_PROF_POOLER, 1, s,
            launch_gather_first_tokens(packed, cu_seqlens, ws.first_tok, batch, max_tokens,
                                       hid * static_cast<int>(h->esize), ws.pool_m, s));
  if (h->cfg.dtype == ET_FP16 && !h->use_simt)
    ET_LAUNCH(h, ET_PROF_POOLER, 1, s,
              launch_gemm_tcgen05(static_cast<const __half*>(ws.first_tok), static_cast<const __half*>(mw.pool_w_t),
                                  static_cast<const __half*>(mw.pool_b), static_cast<__half*>(pooled_out),
                                  ws.pool_m, batch, hid, hid, kEpiBiasTanh, ws.status, s, false, nullptr, &h->maps));
  else if (h->cfg.dtype == ET_FP16)
    ET_LAUNCH(h, ET_PROF_POOLER, 1, s,
              launch_gemm_simt<__half>(static_cast<const __half*>(ws.first_tok), static_cast<const __half*>(mw.pool_w),
                                       static_cast<const __half*>(mw.pool_b), static_cast<__half*>(pooled_out),
                                       ws.pool_m, batch, hid, hid, kEpiBiasTanh, s));
  else
    ET_LAUNCH(h, ET_PROF_POOLER, 1, s,
              launch_gemm_simt<float>(static_cast<const float*>(ws.first_tok), static_cast<const float*>(mw.pool_w),
                                      static_cast<const float*>(mw.pool_b), static_cast<float*>(pooled_out),
                                      ws.pool_m, batch, hid, hid, kEpiBiasTanh, s));
  return ET_OK;
}

// Token ids -> embeddings of the valid tokens (packed) -> stack -> outputs.
int forward_ids_impl(et_handle_t h, const int* input_ids, const int* token_type_ids, const int* mask,
                     void* sequence_out, void* pooled_out, int batch, int seq, cudaStream_t s) {
  h->prof.chain = nullptr;
  int rc = check_shape(h, batch, seq, h->cfg.head_num, h->cfg.size_per_head);
  if (rc != ET_OK) return rc;
  if (input_ids == nullptr || mask == nullptr) return set_error(h, ET_INVALID_ARGUMENT, "null tensor pointer");
  const ModelWeights& mw = h->model;
  if (!mw.emb_ready) return set_error(h, ET_NOT_READY, "embedding weights were never set");
  if (pooled_out != nullptr && !mw.pool_ready) return set_error(h, ET_NOT_READY, "pooler weights were never set");
  if (mw.pos != nullptr && seq > mw.max_pos)
    return set_error(h, ET_INVALID_ARGUMENT, "seq_len exceeds max_position_embeddings");
  for (int l = 0; l < h->cfg.num_layers; ++l)
    if (!h->layers[l].ready) return set_error(h, ET_NOT_READY, "weights of a layer were never set");
  Workspace& ws = h->ws;
  ET_LAUNCH(h, ET_PROF_PADDING_OFFSETS, (batch > 0 && seq > 0) ? 2 : 1, s,
            launch_padding_offsets(mask, batch, seq, ws.prefix_sum, ws.valid_word_num, ws.batch_idx,
                                   ws.word_idx, ws.seq_len, ws.cu_seqlens, ws.padding_offset,
                                   ws.lens_scratch, s));
  if (h->cfg.dtype == ET_FP16) {
    auto H = [](const void* p) { return static_cast<const __half*>(p); };
    ET_LAUNCH(h, ET_PROF_EMBEDDING, 1, s,
              launch_embedding_layernorm<__half>(input_ids, token_type_ids, ws.batch_idx, ws.word_idx,
                                                 ws.valid_word_num, H(mw.word), mw.vocab, H(mw.type),
                                                 mw.type_vocab, H(mw.pos), H(mw.emb_gamma), H(mw.emb_beta),
                                                 static_cast<__half*>(ws.x), batch, seq, h->hidden,
                                                 mw.emb_eps, s));
  } else {
    auto F = [](const void* p) { return static_cast<const float*>(p); };
    ET_LAUNCH(h, ET_PROF_EMBEDDING, 1, s,
              launch_embedding_layernorm<float>(input_ids, token_type_ids, ws.batch_idx, ws.word_idx,
                                                ws.valid_word_num, F(mw.word), mw.vocab, F(mw.type),
                                                mw.type_vocab, F(mw.pos), F(mw.emb_gamma), F(mw.emb_beta),
                                                static_cast<float*>(ws.x), batch, seq, h->hidden,
                                                mw.emb_eps, s));
  }
  rc = stack_impl(h, batch, seq, s);
  if (rc != ET_OK) return rc;
  if (pooled_out != nullptr) {
    rc = pooler_impl(h, ws.x, ws.cu_seqlens, pooled_out, batch, batch * seq, s);
    if (rc != ET_OK) return rc;
  }
  if (sequence_out != nullptr) return restore_impl(h, sequence_out, batch, seq, s);
  return ET_OK;
}

// Copies `count` elements of the handle's dtype into a fresh device array.
int upload_array(et_handle_t h, void** dst, const void* src, size_t count, int on_host,
                 std::vector<void*>& owner, cudaStream_t s) {
  *dst = nullptr;
  if (src == nullptr) return ET_OK;
  void* p = nullptr;
  const size_t bytes = count * h->esize;
  ET_CUDA(h, cudaMalloc(&p, round_up(bytes == 0 ? 16 : bytes, 256)));
  owner.push_back(p);
  ET_CUDA(h, cudaMemcpyAsync(p, src, bytes, on_host ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice, s));
  *dst = p;
  return ET_OK;
}

// Cuts a batch into `chunks` runs of whole sequences.  The first and the last
// run get share 1, the others `mid_share`: the first upload and the last
// download are the two copies that nothing overlaps.
std::vector<std::pair<int, int>> plan_host_chunks(int batch, int chunks, int mid_share) {
  std::vector<std::pair<int, int>> out;
  if (batch <= 0) return out;
  if (chunks > batch) chunks = batch;
  if (chunks < 1) chunks = 1;
  if (mid_share < 1) mid_share = 1;
  const int units = chunks <= 2 ? chunks : 2 + mid_share * (chunks - 2);
  int b0 = 0;
  for (int c = 0; c < chunks; ++c) {
    const int share = (chunks <= 2 || c == 0 || c == chunks - 1) ? 1 : mid_share;
    int nb = static_cast<int>((static_cast<long long>(batch) * share + units - 1) / units);
    if (c == chunks - 1 || b0 + nb > batch) nb = batch - b0;
    if (nb <= 0) break;
    out.emplace_back(b0, nb);
    b0 += nb;
  }
  if (b0 < batch) out.back().second += batch - b0;
  return out;
}

void host_graphs_release(et_handle_t h) {
  et_handle_s::HostGraphs& hg = h->host_graphs;
  for (cudaGraphExec_t e : hg.execs) cudaGraphExecDestroy(e);
  for (cudaGraph_t g : hg.graphs) cudaGraphDestroy(g);
  hg.execs.clear();
  hg.graphs.clear();
  hg.launches.clear();
  hg.batch = hg.seq = -1;
}

// Captures forward_impl for every chunk of a host-buffer call (the stream is idle).
void host_graphs_build(et_handle_t h, int batch, int seq, const std::vector<std::pair<int, int>>& plan) {
  host_graphs_release(h);
  et_handle_s::HostGraphs& hg = h->host_graphs;
  Workspace& ws = h->ws;
  cudaStream_t s = h->own_stream;
  const size_t seq_bytes = static_cast<size_t>(seq) * h->hidden * h->esize;
  const std::string saved_error = h->last_error;
  bool ok = true;
  for (size_t c = 0; c < plan.size() && ok; ++c) {
    const int b0 = plan[c].first, nb = plan[c].second;
    long long before[ET_PROF_NUM];
    for (int i = 0; i < ET_PROF_NUM; ++i) before[i] = h->prof.launches[i];
    if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
      ok = false;
      break;
    }
    const int rc = forward_impl(h, static_cast<char*>(ws.stage_in) + b0 * seq_bytes,
                                ws.stage_mask + static_cast<size_t>(b0) * seq,
                                static_cast<char*>(ws.stage_out) + b0 * seq_bytes, nb, seq, s);
    cudaGraph_t g = nullptr;
    const cudaError_t e = cudaStreamEndCapture(s, &g);
    std::vector<long long> cnt(ET_PROF_NUM);
    for (int i = 0; i < ET_PROF_NUM; ++i) {
      cnt[i] = h->prof.launches[i] - before[i];
      h->prof.launches[i] = before[i];
    }
    cudaGraphExec_t ex = nullptr;
    if (rc != ET_OK || e != cudaSuccess || g == nullptr || cudaGraphInstantiate(&ex, g, 0) != cudaSuccess) {
      if (g) cudaGraphDestroy(g);
      ok = false;
      break;
    }
    hg.graphs.push_back(g);
    hg.execs.push_back(ex);
    hg.launches.push_back(cnt);
  }
  if (!ok) {
    cudaGetLastError();
    host_graphs_release(h);
    h->last_error = saved_error;
    h->host_graph_enabled = false;  // do not retry on every call
    return;
  }
  hg.batch = batch;
  hg.seq = seq;
  hg.per = static_cast<int>(plan.size());
  hg.mid_share = h->host_mid_share;
  hg.simt = h->use_simt;
}

}  // namespace

// =============================== C ABI =====================================
#define ET_TRY try {
#define ET_CATCH(h)                                                              \
  }                                                                              \
  catch (const std::bad_alloc&) { return set_error(h, ET_CUDA_ERROR, "host allocation failed"); } \
  catch (const std::exception& e) { return set_error(h, ET_CUDA_ERROR, e.what()); }             \
  catch (...) { return set_error(h, ET_CUDA_ERROR, "Runtime error"); }

extern "C" {

int et_create(const et_config_t* config, et_handle_t* out_handle) {
  et_handle_t h = nullptr;
  ET_TRY
  if (config == nullptr || out_handle == nullptr)
    return set_error(nullptr, ET_INVALID_ARGUMENT, "null config or out_handle");
  *out_handle = nullptr;
  const et_config_t& c = *config;
  if (c.dtype != ET_FP32 && c.dtype != ET_FP16)
    return set_error(nullptr, ET_INVALID_ARGUMENT, "dtype must be ET_FP32 or ET_FP16");
  if (c.num_layers <= 0 || c.head_num <= 0 || c.max_batch_size <= 0 || c.max_seq_len <= 0)
    return set_error(nullptr, ET_INVALID_ARGUMENT, "num_layers, head_num, max_batch_size, max_seq_len must be positive");
  if (c.size_per_head != 64)
    return set_error(nullptr, ET_INVALID_ARGUMENT, "size_per_head must be 64");
  const int hid = c.head_num * c.size_per_head;
  if (c.ffn_dim <= 0 || (c.ffn_dim % 128) != 0 || (hid % 128) != 0)
    return set_error(nullptr, ET_INVALID_ARGUMENT, "hidden and ffn_dim must be positive multiples of 128");
  // the LayerNorm and embedding kernels keep a row in the registers of one warp: 8 vectors of 16 bytes per lane
  if (hid > (c.dtype == ET_FP16 ? 2048 : 1024))
    return set_error(nullptr, ET_INVALID_ARGUMENT,
                     "hidden (head_num * size_per_head) is limited to 2048 for ET_FP16 and 1024 for ET_FP32");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || c.device < 0 || c.device >= ndev)
    return set_error(nullptr, ET_CUDA_ERROR, "no such CUDA device");
  DeviceGuard guard(c.device);
  if (!guard.ok) return set_error(nullptr, ET_CUDA_ERROR, "cudaSetDevice failed");
  cudaDeviceProp prop{};
  if (cudaGetDeviceProperties(&prop, c.device) != cudaSuccess || prop.major != 10)
    return set_error(nullptr, ET_CUDA_ERROR, "this library contains sm_100a code only: a B200-class GPU is required");

  h = new et_handle_s();
  h->cfg = c;
  h->hidden = hid;
  h->esize = c.dtype == ET_FP16 ? 2 : 4;
  h->eps = c.layernorm_eps > 0.f ? c.layernorm_eps : 1e-6f;
  h->use_simt = false;
  h->layers.resize(c.num_layers);
  auto bail = [&](int rc) {
    std::string msg = h->last_error;
    et_destroy(h);
    g_create_error = msg;
    return rc;
  };
  int rc = ET_OK;
  const size_t e = h->esize, f = c.ffn_dim;
  const size_t H = hid;
  for (auto& lw : h->layers) {
    struct { void** p; size_t n; } items[] = {
        {&lw.wqkv, 3 * H * H}, {&lw.wo, H * H}, {&lw.w1, H * f}, {&lw.w2, f * H},
        {&lw.bqkv, 3 * H}, {&lw.bo, H}, {&lw.ln1_gamma, H}, {&lw.ln1_beta, H},
        {&lw.b1, f}, {&lw.b2, H}, {&lw.ln2_gamma, H}, {&lw.ln2_beta, H}};
    for (auto& it : items)
      if ((rc = ws_alloc(h, it.p, it.n * e)) != ET_OK) return bail(rc);
    {  // K-major [out, in] copies for the tensor-core GEMMs (fp32: plus the tf32 remainders)
      struct { void** p; size_t n; } packed[] = {
          {&lw.wqkv_t, 3 * H * H}, {&lw.wo_t, H * H}, {&lw.w1_t, H * f}, {&lw.w2_t, f * H},
          {&lw.wqkv_lo, 3 * H * H}, {&lw.wo_lo, H * H}, {&lw.w1_lo, H * f}, {&lw.w2_lo, f * H}};
      const int count = c.dtype == ET_FP16 ? 4 : 8;
      for (int i = 0; i < count; ++i)
        if ((rc = ws_alloc(h, packed[i].p, packed[i].n * e)) != ET_OK) return bail(rc);
    }
    if (defer_eligible(c)) {
      struct { void** p; size_t n; } folded[] = {{&lw.wqkv_f, 3 * H * H}, {&lw.cqkv, 3 * H}, {&lw.bqkv_f, 3 * H},
                                                  {&lw.w1_f, H * f},       {&lw.c1, f},       {&lw.b1_f, f}};
      for (auto& it : folded)
        if ((rc = ws_alloc(h, it.p, it.n * e)) != ET_OK) return bail(rc);
    }
  }
  Workspace& ws = h->ws;
  ws.cap_tokens = round_up(static_cast<size_t>(c.max_batch_size) * c.max_seq_len, 128);
  for (const WsItem& b : workspace_items(c, static_cast<size_t>(c.max_batch_size),
                                         static_cast<size_t>(c.max_seq_len), ws))
    if ((rc = ws_alloc(h, b.slot, b.bytes)) != ET_OK) return bail(rc);
    else h->ws_bytes_allocated += ws_round(b.bytes);
  if (cudaMemset(ws.ln_counters, 0, ln_counter_ints(ws.cap_tokens) * 4) != cudaSuccess)
    return bail(cuda_fail(h, cudaGetLastError(), "cudaMemset"));
  if (cudaMemset(ws.status, 0, 4) != cudaSuccess || cudaMemset(ws.valid_word_num, 0, 4) != cudaSuccess)
    return bail(cuda_fail(h, cudaGetLastError(), "cudaMemset"));
  if (cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking) != cudaSuccess)
    return bail(cuda_fail(h, cudaGetLastError(), "cudaStreamCreate"));
  if (cudaStreamCreateWithFlags(&h->h2d_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&h->d2h_stream, cudaStreamNonBlocking) != cudaSuccess)
    return bail(cuda_fail(h, cudaGetLastError(), "cudaStreamCreate"));
  for (int i = 0; i < et_handle_s::kMaxChunks; ++i)
    if (cudaEventCreateWithFlags(&h->in_done[i], cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&h->comp_done[i], cudaEventDisableTiming) != cudaSuccess)
      return bail(cuda_fail(h, cudaGetLastError(), "cudaEventCreate"));
  if (const char* e = getenv("ETB_HOST_GRAPH")) h->host_graph_enabled = !(e[0] == '0');
  if (const char* e = getenv("ETB_HOST_CHUNKS")) {
    const int n = atoi(e);
    if (n >= 1 && n <= et_handle_s::kMaxChunks) h->host_chunks = n;
  }
  if (const char* e = getenv("ETB_HOST_MID_SHARE")) {  // fixes the shares; otherwise the first call measures
    const int n = atoi(e);
    if (n >= 1 && n <= 16) {
      h->host_mid_share = n;
      h->host_share_auto = false;
    }
  }
  for (auto& ev : h->tune_ev)
    if (cudaEventCreate(&ev) != cudaSuccess) return bail(cuda_fail(h, cudaGetLastError(), "cudaEventCreate"));
  if (cudaMallocHost(reinterpret_cast<void**>(&h->host_pinned),
                     (2 + et_handle_s::kMaxChunks) * sizeof(int)) != cudaSuccess)
    return bail(cuda_fail(h, cudaGetLastError(), "cudaMallocHost"));
  *out_handle = h;
  return ET_OK;
  ET_CATCH(nullptr)
}

int et_destroy(et_handle_t h) {
  if (h == nullptr) return ET_OK;
  DeviceGuard guard(h->cfg.device);
  cudaDeviceSynchronize();
  if (h->graph_exec) cudaGraphExecDestroy(h->graph_exec);
  if (h->graph) cudaGraphDestroy(h->graph);
  for (cudaGraphExec_t e : h->host_graphs.execs) cudaGraphExecDestroy(e);
  for (cudaGraph_t g : h->host_graphs.graphs) cudaGraphDestroy(g);
  for (void* p : h->ws.allocations) cudaFree(p);
  for (void* p : h->model.emb_allocs) cudaFree(p);
  for (void* p : h->model.pool_allocs) cudaFree(p);
  for (auto& sp : h->prof.pending) {
    if (sp.owns_a) cudaEventDestroy(sp.a);
    cudaEventDestroy(sp.b);
  }
  for (cudaEvent_t e : h->prof.free_events) cudaEventDestroy(e);
  for (int i = 0; i < et_handle_s::kMaxChunks; ++i) {
    if (h->in_done[i]) cudaEventDestroy(h->in_done[i]);
    if (h->comp_done[i]) cudaEventDestroy(h->comp_done[i]);
  }
  for (cudaEvent_t ev : h->tune_ev)
    if (ev) cudaEventDestroy(ev);
  if (h->own_stream) cudaStreamDestroy(h->own_stream);
  if (h->h2d_stream) cudaStreamDestroy(h->h2d_stream);
  if (h->d2h_stream) cudaStreamDestroy(h->d2h_stream);
  if (h->host_pinned) cudaFreeHost(h->host_pinned);
  delete h;
  return ET_OK;
}

const char* et_last_error(et_handle_t h) {
  return h != nullptr ? h->last_error.c_str() : g_create_error.c_str();
}

int et_set_debug_simt(et_handle_t h, int use_simt) {
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  h->use_simt = use_simt != 0;
  return ET_OK;
}

int et_set_fused_layernorm(et_handle_t h, int enable) {
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (h->fuse_ln != (enable != 0)) {
    DeviceGuard guard(h->cfg.device);
    cudaDeviceSynchronize();
    graph_release(h);        // recorded passes hold the other kernel sequence
    host_graphs_release(h);
  }
  h->fuse_ln = enable != 0;
  return ET_OK;
}

int et_set_deferred_layernorm(et_handle_t h, int enable) {
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (enable != 0 && !defer_eligible(h->cfg))
    return set_error(h, ET_INVALID_ARGUMENT,
                     "deferred LayerNorm needs an fp16 handle whose hidden size (at most 1024) and ffn_dim are multiples of 256");
  if (h->defer_ln != (enable != 0)) {
    DeviceGuard guard(h->cfg.device);
    cudaDeviceSynchronize();
    graph_release(h);        // recorded passes hold the other kernel sequence
    host_graphs_release(h);
  }
  h->defer_ln = enable != 0;
  return ET_OK;
}

int et_workspace_allocated_bytes(et_handle_t h, size_t* out_bytes) {
  if (h == nullptr || out_bytes == nullptr) return ET_INVALID_ARGUMENT;
  *out_bytes = h->ws_bytes_allocated;
  return ET_OK;
}

int et_host_chunk_shares(et_handle_t h, int* chunks, int* mid_share, int* measured) {
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (chunks) *chunks = h->host_chunks;
  if (mid_share) *mid_share = h->host_mid_share;
  if (measured) *measured = h->host_share_measured ? 1 : 0;
  return ET_OK;
}

int et_set_layer_weights(et_handle_t h, int layer, const void* const* weights, int on_host) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (layer < 0 || layer >= h->cfg.num_layers || weights == nullptr)
    return set_error(h, ET_INVALID_ARGUMENT, "layer out of range or null weights");
  for (int i = 0; i < 16; ++i)
    if (weights[i] == nullptr) return set_error(h, ET_INVALID_ARGUMENT, "null weight pointer");
  DeviceGuard guard(h->cfg.device);
  const size_t H = h->hidden, f = h->cfg.ffn_dim, e = h->esize;
  const size_t counts[16] = {H * H, H, H * H, H, H * H, H, H * H, H, H, H, H * f, f, f * H, H, H, H};
  const void* dev[16];
  std::vector<void*> temps;
  int rc = ET_OK;
  if (on_host) {
    for (int i = 0; i < 16 && rc == ET_OK; ++i) {
      void* p = nullptr;
      cudaError_t ce = cudaMalloc(&p, round_up(counts[i] * e, 256));
      if (ce == cudaSuccess) {
        temps.push_back(p);
        ce = cudaMemcpyAsync(p, weights[i], counts[i] * e, cudaMemcpyHostToDevice, h->own_stream);
      }
      if (ce != cudaSuccess) rc = cuda_fail(h, ce, "weight upload");
      dev[i] = p;
    }
  } else {
    for (int i = 0; i < 16; ++i) dev[i] = weights[i];
  }
  if (rc == ET_OK) rc = pack_layer_any(h, layer, dev, h->own_stream);
  if (rc == ET_OK) rc = fold_all(h, h->own_stream);  // once every layer has its weights
  cudaError_t se = cudaStreamSynchronize(h->own_stream);
  for (void* p : temps) cudaFree(p);
  if (rc == ET_OK && se != cudaSuccess) rc = cuda_fail(h, se, "cudaStreamSynchronize");
  return rc;
  ET_CATCH(h)
}

int et_workspace_bytes(et_handle_t h, int batch_size, int seq_len, size_t* out_bytes) {
  if (h == nullptr || out_bytes == nullptr) return ET_INVALID_ARGUMENT;
  if (batch_size < 0 || seq_len < 0) return set_error(h, ET_INVALID_ARGUMENT, "negative shape");
  *out_bytes = workspace_bytes_for(h, static_cast<size_t>(batch_size), static_cast<size_t>(seq_len));
  return ET_OK;
}

int et_input(et_handle_t h, const et_input_param_t* p) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (p == nullptr) return set_error(h, ET_INVALID_ARGUMENT, "null param");
  int rc = check_shape(h, p->batch_size, p->from_seq_len, p->head_num, p->size_per_head);
  if (rc != ET_OK) return rc;
  if (!p->from_tensor || !p->mask || !p->valid_word_num || !p->batch_idx || !p->word_idx || !p->to_tensor)
    return set_error(h, ET_INVALID_ARGUMENT, "null tensor pointer");
  DeviceGuard guard(h->cfg.device);
  h->prof.chain = nullptr;
  return input_impl(h, p);
  ET_CATCH(h)
}

int et_output(et_handle_t h, const et_output_param_t* p) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (p == nullptr) return set_error(h, ET_INVALID_ARGUMENT, "null param");
  int rc = check_shape(h, p->batch_size, p->from_seq_len, p->head_num, p->size_per_head);
  if (rc != ET_OK) return rc;
  if (!p->from_tensor || !p->valid_word_num || !p->batch_idx || !p->word_idx || !p->to_tensor)
    return set_error(h, ET_INVALID_ARGUMENT, "null tensor pointer");
  DeviceGuard guard(h->cfg.device);
  h->prof.chain = nullptr;
  return output_impl(h, p);
  ET_CATCH(h)
}

int et_layer(et_handle_t h, int layer, const et_encoder_param_t* p, const et_transformer_param_t* tp) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (p == nullptr || tp == nullptr) return set_error(h, ET_INVALID_ARGUMENT, "null param");
  if (layer < 0 || layer >= h->cfg.num_layers) return set_error(h, ET_INVALID_ARGUMENT, "layer out of range");
  if (tp->from_seq_len != tp->to_seq_len)
    return set_error(h, ET_INVALID_ARGUMENT, "only support from_seq_len == to_seq_len");
  int rc = check_shape(h, tp->batch_size, tp->from_seq_len, tp->head_num, tp->size_per_head);
  if (rc != ET_OK) return rc;
  if (!p->from_tensor || !p->transformer_out || !p->batch_idx || !p->word_idx || !p->valid_word_num)
    return set_error(h, ET_INVALID_ARGUMENT, "null tensor pointer");
  if (p->to_tensor != nullptr && p->to_tensor != p->from_tensor)
    return set_error(h, ET_INVALID_ARGUMENT, "to_tensor must equal from_tensor (self-attention)");
  DeviceGuard guard(h->cfg.device);
  h->prof.chain = nullptr;
  cudaStream_t s = static_cast<cudaStream_t>(p->stream);
  if (h->general_mask && p->attr_mask == nullptr)
    return set_error(h, ET_INVALID_ARGUMENT, "general-mask mode: attr_mask [B,S,S] is required");
  // from here on every return leaves the handle in key-only-mask mode again
  MaskScope mask_scope(h, h->general_mask ? p->attr_mask : nullptr, h->general_mask ? p->batch_idx : nullptr,
                       h->general_mask ? p->word_idx : nullptr);
  if (p->attr_kernel_Q != nullptr) {
    const void* w[16] = {p->attr_kernel_Q, p->attr_bias_Q, p->attr_kernel_K, p->attr_bias_K,
                         p->attr_kernel_V, p->attr_bias_V, p->attr_output_kernel, p->attr_output_bias,
                         p->attr_output_layernorm_beta, p->attr_output_layernorm_gamma, p->inter_kernel,
                         p->inter_bias, p->output_kernel, p->output_bias, p->output_layernorm_beta,
                         p->output_layernorm_gamma};
    for (int i = 0; i < 16; ++i)
      if (w[i] == nullptr) return set_error(h, ET_INVALID_ARGUMENT, "null weight pointer");
    rc = pack_layer_any(h, layer, w, s);
    if (rc != ET_OK) return rc;
  }
  if (!h->layers[layer].ready) return set_error(h, ET_NOT_READY, "weights of this layer were never set");
  const int batch = tp->batch_size, seq = tp->from_seq_len, max_m = batch * seq;
  ET_LAUNCH(h, ET_PROF_PADDING_OFFSETS, 1, s, launch_seq_bounds_from_batch_idx(p->batch_idx, p->valid_word_num, batch, max_m,
                                              h->ws.cu_seqlens, s));
  if (h->cfg.dtype == ET_FP16 && !h->use_simt && seq <= 128 && max_m > 0) {
    ET_LAUNCH(h, ET_PROF_PADDING_OFFSETS, 1, s,
              launch_attention_plan(h->ws.cu_seqlens, batch, max_m, h->ws.attn_plan, s));
  } else if (h->cur_attr_mask != nullptr) {
    ET_LAUNCH(h, ET_PROF_PADDING_OFFSETS, 1, s,
              launch_position_rows(p->batch_idx, p->word_idx, p->valid_word_num, batch, seq, h->ws.pos_row, s));
  }
  if (h->cfg.dtype == ET_FP16)
    rc = run_layer<__half>(h, h->layers[layer], static_cast<const __half*>(p->from_tensor),
                           static_cast<__half*>(p->transformer_out), p->valid_word_num, max_m,
                           h->ws.cu_seqlens, batch, seq, s);
  else
    rc = run_layer<float>(h, h->layers[layer], static_cast<const float*>(p->from_tensor),
                          static_cast<float*>(p->transformer_out), p->valid_word_num, max_m,
                          h->ws.cu_seqlens, batch, seq, s);
  return rc;
  ET_CATCH(h)
}

int et_forward(et_handle_t h, const void* from_tensor, const int* mask, void* out, int batch_size,
               int seq_len, void* stream) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  DeviceGuard guard(h->cfg.device);
  return forward_impl(h, from_tensor, mask, out, batch_size, seq_len, static_cast<cudaStream_t>(stream));
  ET_CATCH(h)
}

int et_set_general_mask(et_handle_t h, int enable) {
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  h->general_mask = enable != 0;
  return ET_OK;
}

int et_forward_general_mask(et_handle_t h, const void* from_tensor, const int* mask, const void* attr_mask,
                            void* out, int batch_size, int seq_len, void* stream) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (attr_mask == nullptr) return set_error(h, ET_INVALID_ARGUMENT, "attr_mask [B,S,S] is required");
  DeviceGuard guard(h->cfg.device);
  MaskScope mask_scope(h, attr_mask, h->ws.batch_idx, h->ws.word_idx);
  return forward_impl(h, from_tensor, mask, out, batch_size, seq_len, static_cast<cudaStream_t>(stream));
  ET_CATCH(h)
}

}  // extern "C"

namespace {

// Chunking of a host-buffer call from the measured times of one 3-chunk call: `up` ms for the
// whole upload (the download is taken to cost the same), a pass over a fraction x of the batch
// costs fixed + slope * x ms (fixed: the ~90 dependent launches of a pass, whatever its size).
// Timeline of shares 1:m:1 -- upload of chunk 0, then its pass while chunk 1 is uploaded, the
// passes of chunks 1 and 2, the download of chunk 2:
//   t(m) = up/(m+2) + max(pass(1/(m+2)), up*m/(m+2)) + pass(m/(m+2)) + pass(1/(m+2)) + up/(m+2)
// A wide middle chunk shortens the two copies nothing overlaps, until its own upload no longer
// hides behind the first chunk's pass (several processes sharing the host's PCIe switches).
// One chunk costs up + pass(1) + up: better for small batches, where the fixed cost of two more
// passes outweighs the overlapped copies.  Returns the middle share, or 0 for "do not chunk".
int best_host_chunking(double up, double fixed, double slope) {
  auto pass = [&](double x) { return fixed + slope * x; };
  int best = 0;
  double best_t = up + pass(1.0) + up;
  for (int m : {1, 2, 3, 4, 6, 8}) {
    const double d = m + 2;
    const double t = up / d + std::max(pass(1 / d), up * m / d) + pass(m / d) + pass(1 / d) + up / d;
    if (t < best_t - 1e-9) {
      best_t = t;
      best = m;
    }
  }
  return best;
}

int forward_host_body(et_handle_t h, const void* from_host, const int* mask_host, void* out_host,
                      int batch_size, int seq_len, int* valid_word_num_out) {
  Workspace& ws = h->ws;
  cudaStream_t s = h->own_stream;
  int rc = ET_OK;
  // The batch is cut into chunks of whole sequences (they are independent):
  // all uploads are queued on the upload stream at once, chunk i is computed
  // when its upload has landed, and its result goes back on the download
  // stream while chunk i+1 is being computed.
  const size_t seq_bytes = static_cast<size_t>(seq_len) * h->hidden * h->esize;
  int chunks = h->host_chunks;
  if (h->host_share_auto && h->host_share_measured && (h->tuned_batch != batch_size || h->tuned_seq != seq_len)) {
    h->host_share_measured = false;  // another shape: measure again, starting from the default shares
    h->host_mid_share = 6;
    h->tune_state = 0;
    h->tune_replays = 0;
    h->tune_model_share = 6;
  }
  if (h->host_share_auto && !h->host_share_measured &&
      (h->last_host_batch != batch_size || h->last_host_seq != seq_len)) {
    h->host_mid_share = 6;  // another shape while the shares were still being tried: start over
    h->tune_state = 0;
    h->tune_replays = 0;
    h->tune_model_share = 6;
  }
  if (static_cast<size_t>(batch_size) * seq_bytes < (8u << 20)) chunks = 1;  // too small to be worth it
  if ((h->host_share_measured || h->tune_state == 1) && h->host_mid_share == 0) chunks = 1;  // one piece
  const std::vector<std::pair<int, int>> plan =
      plan_host_chunks(batch_size, chunks, h->host_mid_share > 0 ? h->host_mid_share : 1);
  const int per = static_cast<int>(plan.size());
  int nchunks = 0;
  et_handle_s::HostGraphs& hg = h->host_graphs;
  const bool graphs_allowed = h->host_graph_enabled && !h->prof.enabled && h->cur_attr_mask == nullptr;
  const bool replay = graphs_allowed && hg.batch == batch_size && hg.seq == seq_len && hg.per == per &&
                      hg.mid_share == h->host_mid_share && hg.simt == h->use_simt && !hg.execs.empty();
  // The first REPLAYED chunked call measures the copy and pass times that choose the shares of the
  // calls to come: an eager pass over a small chunk is bound by its launches (and the first one by
  // one-time set-up), which overstates the fixed cost of a pass and chose too narrow a middle chunk.
  // If the shares change, the next call runs eagerly again and the one after records the new chunks.
  const bool tuning = h->host_share_auto && !h->host_share_measured && replay;
  const bool measure = tuning && h->tune_state == 0 && h->tune_replays == 0 && per >= 3 && h->tune_ev[0] != nullptr;
  const auto call_begin = std::chrono::steady_clock::now();
  if (measure) ET_CUDA(h, cudaEventRecord(h->tune_ev[0], h->h2d_stream));
  for (; nchunks < per; ++nchunks) {
    const size_t b0 = plan[nchunks].first, nb = plan[nchunks].second;
    ET_CUDA(h, cudaMemcpyAsync(static_cast<char*>(ws.stage_in) + b0 * seq_bytes,
                               static_cast<const char*>(from_host) + b0 * seq_bytes, nb * seq_bytes,
                               cudaMemcpyHostToDevice, h->h2d_stream));
    ET_CUDA(h, cudaMemcpyAsync(ws.stage_mask + static_cast<size_t>(b0) * seq_len,
                               mask_host + static_cast<size_t>(b0) * seq_len,
                               nb * seq_len * 4, cudaMemcpyHostToDevice, h->h2d_stream));
    ET_CUDA(h, cudaEventRecord(h->in_done[nchunks], h->h2d_stream));
  }
  if (measure) ET_CUDA(h, cudaEventRecord(h->tune_ev[1], h->h2d_stream));
  for (int c = 0; c < per; ++c) {
    const size_t b0 = plan[c].first;
    const int nb = plan[c].second;
    ET_CUDA(h, cudaStreamWaitEvent(s, h->in_done[c], 0));
    // the passes of the first and the middle chunk, each from the moment its upload has landed: two
    // sizes give the fixed cost of a pass and its cost per sequence
    if (measure && c <= 1) ET_CUDA(h, cudaEventRecord(h->tune_ev[2 + 2 * c], s));
    if (replay && c < static_cast<int>(hg.execs.size())) {
      ET_CUDA(h, cudaGraphLaunch(hg.execs[c], s));
      for (int i = 0; i < ET_PROF_NUM; ++i) h->prof.launches[i] += hg.launches[c][i];
    } else {
      rc = forward_impl(h, static_cast<char*>(ws.stage_in) + b0 * seq_bytes,
                        ws.stage_mask + static_cast<size_t>(b0) * seq_len,
                        static_cast<char*>(ws.stage_out) + b0 * seq_bytes, nb, seq_len, s);
      if (rc != ET_OK) return rc;
    }
    if (measure && c <= 1) ET_CUDA(h, cudaEventRecord(h->tune_ev[3 + 2 * c], s));
    ET_CUDA(h, cudaMemcpyAsync(&h->host_pinned[2 + c], ws.valid_word_num, 4, cudaMemcpyDeviceToHost, s));
    ET_CUDA(h, cudaEventRecord(h->comp_done[c], s));
    ET_CUDA(h, cudaStreamWaitEvent(h->d2h_stream, h->comp_done[c], 0));
    ET_CUDA(h, cudaMemcpyAsync(static_cast<char*>(out_host) + b0 * seq_bytes,
                               static_cast<char*>(ws.stage_out) + b0 * seq_bytes, nb * seq_bytes,
                               cudaMemcpyDeviceToHost, h->d2h_stream));
  }
  ET_CUDA(h, cudaMemcpyAsync(&h->host_pinned[1], ws.status, 4, cudaMemcpyDeviceToHost, s));
  ET_CUDA(h, cudaStreamSynchronize(s));
  ET_CUDA(h, cudaStreamSynchronize(h->d2h_stream));
  ET_CUDA(h, cudaStreamSynchronize(h->h2d_stream));
  int total_tokens = 0;
  for (int i = 0; i < nchunks; ++i) total_tokens += h->host_pinned[2 + i];
  if (valid_word_num_out) *valid_word_num_out = total_tokens;
  if (h->host_pinned[1] != 0) return device_timeout(h, s);
  if (measure) {
    float up_ms = 0.f, first_ms = 0.f, mid_ms = 0.f;
    const double x0 = static_cast<double>(plan[0].second) / batch_size, x1 = static_cast<double>(plan[1].second) / batch_size;
    h->tune_model_share = h->host_mid_share;
    if (cudaEventElapsedTime(&up_ms, h->tune_ev[0], h->tune_ev[1]) == cudaSuccess &&
        cudaEventElapsedTime(&first_ms, h->tune_ev[2], h->tune_ev[3]) == cudaSuccess &&
        cudaEventElapsedTime(&mid_ms, h->tune_ev[4], h->tune_ev[5]) == cudaSuccess && up_ms > 0.f && first_ms > 0.f &&
        mid_ms > 0.f && x1 > x0) {
      double slope = (mid_ms - first_ms) / (x1 - x0);
      if (slope < 0) slope = 0;
      double fixed = first_ms - slope * x0;
      if (fixed < 0) fixed = 0;
      h->tune_model_share = best_host_chunking(up_ms, fixed, slope);
    }
  }
  if (tuning) {
    // The model (copies and passes as straight lines) only proposes: its choice is kept if two
    // replayed calls with it beat two replayed calls with the default shares by more than 1 %.
    const double call_ms =
        std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - call_begin).count();
    double& best = h->tune_state == 0 ? h->tune_ms_default : h->tune_ms_trial;
    best = h->tune_replays == 0 ? call_ms : std::min(best, call_ms);
    if (++h->tune_replays >= 2) {
      h->tune_replays = 0;
      if (h->tune_state == 0 && h->tune_model_share != h->host_mid_share) {
        h->tune_state = 1;                            // the next calls run, record and replay the model's choice
        h->host_mid_share = h->tune_model_share;
      } else {
        if (h->tune_state == 1 && !(h->tune_ms_trial < 0.99 * h->tune_ms_default)) h->host_mid_share = 6;
        h->tune_state = 2;
        h->host_share_measured = true;
        h->tuned_batch = batch_size;
        h->tuned_seq = seq_len;
      }
    }
  }
  // second call in a row with this shape: record its chunks for the calls to come
  if (!replay && graphs_allowed && batch_size > 0 && h->last_host_batch == batch_size &&
      h->last_host_seq == seq_len && !measure)
    host_graphs_build(h, batch_size, seq_len, plan);  // best effort: on failure the eager path stays
  h->last_host_batch = batch_size;
  h->last_host_seq = seq_len;
  return ET_OK;
}

// Copies of a host-buffer call may still be running when an error is found: nothing of the call
// may touch the caller's buffers after it has returned.
void quiesce_host_call(et_handle_t h) {
  cudaStreamSynchronize(h->own_stream);
  cudaStreamSynchronize(h->h2d_stream);
  cudaStreamSynchronize(h->d2h_stream);
}

}  // namespace

extern "C" {

int et_forward_host(et_handle_t h, const void* from_host, const int* mask_host, void* out_host,
                    int batch_size, int seq_len, int* valid_word_num_out) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  int rc = check_shape(h, batch_size, seq_len, h->cfg.head_num, h->cfg.size_per_head);
  if (rc != ET_OK) return rc;
  if (!from_host || !mask_host || !out_host) return set_error(h, ET_INVALID_ARGUMENT, "null host pointer");
  DeviceGuard guard(h->cfg.device);
  rc = forward_host_body(h, from_host, mask_host, out_host, batch_size, seq_len, valid_word_num_out);
  if (rc != ET_OK) quiesce_host_call(h);
  return rc;
  ET_CATCH(h)
}

int et_set_embedding_weights(et_handle_t h, const void* word_table, int vocab_size, const void* type_table,
                             int type_vocab_size, const void* position_table, int max_position,
                             const void* gamma, const void* beta, float layernorm_eps, int on_host) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (word_table == nullptr || vocab_size <= 0 || gamma == nullptr || beta == nullptr)
    return set_error(h, ET_INVALID_ARGUMENT, "word_table, gamma and beta are required");
  if ((type_table != nullptr && type_vocab_size <= 0) || (position_table != nullptr && max_position <= 0))
    return set_error(h, ET_INVALID_ARGUMENT, "a table was given with a non-positive row count");
  DeviceGuard guard(h->cfg.device);
  ModelWeights& mw = h->model;
  cudaStream_t s = h->own_stream;
  ET_CUDA(h, cudaDeviceSynchronize());  // nothing may still read the tables being replaced
  graph_release(h);  // a captured pass holds the addresses of the tables being freed
  for (void* p : mw.emb_allocs) cudaFree(p);
  mw.emb_allocs.clear();
  mw.emb_ready = false;
  const size_t H = h->hidden;
  int rc = upload_array(h, &mw.word, word_table, static_cast<size_t>(vocab_size) * H, on_host, mw.emb_allocs, s);
  if (rc == ET_OK)
    rc = upload_array(h, &mw.type, type_table, static_cast<size_t>(type_vocab_size) * H, on_host, mw.emb_allocs, s);
  if (rc == ET_OK)
    rc = upload_array(h, &mw.pos, position_table, static_cast<size_t>(max_position) * H, on_host, mw.emb_allocs, s);
  if (rc == ET_OK) rc = upload_array(h, &mw.emb_gamma, gamma, H, on_host, mw.emb_allocs, s);
  if (rc == ET_OK) rc = upload_array(h, &mw.emb_beta, beta, H, on_host, mw.emb_allocs, s);
  cudaError_t se = cudaStreamSynchronize(s);
  if (rc == ET_OK && se != cudaSuccess) rc = cuda_fail(h, se, "cudaStreamSynchronize");
  if (rc != ET_OK) return rc;
  mw.vocab = vocab_size;
  mw.type_vocab = type_table ? type_vocab_size : 0;
  mw.max_pos = position_table ? max_position : 0;
  mw.emb_eps = layernorm_eps > 0.f ? layernorm_eps : 1e-12f;
  mw.emb_ready = true;
  return ET_OK;
  ET_CATCH(h)
}

int et_set_pooler_weights(et_handle_t h, const void* kernel, const void* bias, int on_host) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (kernel == nullptr || bias == nullptr) return set_error(h, ET_INVALID_ARGUMENT, "null weight pointer");
  DeviceGuard guard(h->cfg.device);
  ModelWeights& mw = h->model;
  cudaStream_t s = h->own_stream;
  ET_CUDA(h, cudaDeviceSynchronize());
  graph_release(h);
  for (void* p : mw.pool_allocs) cudaFree(p);
  mw.pool_allocs.clear();
  mw.pool_ready = false;
  mw.pool_w_t = nullptr;
  const size_t H = h->hidden;
  int rc = upload_array(h, &mw.pool_w, kernel, H * H, on_host, mw.pool_allocs, s);
  if (rc == ET_OK) rc = upload_array(h, &mw.pool_b, bias, H, on_host, mw.pool_allocs, s);
  if (rc == ET_OK && h->cfg.dtype == ET_FP16) {
    void* p = nullptr;
    ET_CUDA(h, cudaMalloc(&p, round_up(H * H * 2, 256)));
    mw.pool_allocs.push_back(p);
    mw.pool_w_t = p;
    ET_CUDA(h, launch_transpose<__half>(static_cast<const __half*>(mw.pool_w), static_cast<__half*>(p),
                                        h->hidden, h->hidden, s));
  }
  cudaError_t se = cudaStreamSynchronize(s);
  if (rc == ET_OK && se != cudaSuccess) rc = cuda_fail(h, se, "cudaStreamSynchronize");
  if (rc != ET_OK) return rc;
  mw.pool_ready = true;
  return ET_OK;
  ET_CATCH(h)
}

int et_forward_ids(et_handle_t h, const int* input_ids, const int* token_type_ids, const int* mask,
                   void* sequence_out, void* pooled_out, int batch_size, int seq_len, void* stream) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  DeviceGuard guard(h->cfg.device);
  return forward_ids_impl(h, input_ids, token_type_ids, mask, sequence_out, pooled_out, batch_size, seq_len,
                          static_cast<cudaStream_t>(stream));
  ET_CATCH(h)
}

}  // extern "C"

namespace {

int forward_ids_host_body(et_handle_t h, const int* ids_host, const int* types_host, const int* mask_host,
                          void* sequence_out_host, void* pooled_out_host, int batch_size, int seq_len,
                          int* valid_word_num_out) {
  Workspace& ws = h->ws;
  cudaStream_t s = h->own_stream;
  const size_t n = static_cast<size_t>(batch_size) * seq_len;
  ET_CUDA(h, cudaMemcpyAsync(ws.stage_ids, ids_host, n * 4, cudaMemcpyHostToDevice, s));
  ET_CUDA(h, cudaMemcpyAsync(ws.stage_mask, mask_host, n * 4, cudaMemcpyHostToDevice, s));
  if (types_host) ET_CUDA(h, cudaMemcpyAsync(ws.stage_types, types_host, n * 4, cudaMemcpyHostToDevice, s));
  const int rc = forward_ids_impl(h, ws.stage_ids, types_host ? ws.stage_types : nullptr, ws.stage_mask,
                                  sequence_out_host ? ws.stage_out : nullptr, pooled_out_host ? ws.pooled : nullptr,
                                  batch_size, seq_len, s);
  if (rc != ET_OK) return rc;
  if (pooled_out_host)
    ET_CUDA(h, cudaMemcpyAsync(pooled_out_host, ws.pooled, static_cast<size_t>(batch_size) * h->hidden * h->esize,
                               cudaMemcpyDeviceToHost, s));
  if (sequence_out_host)
    ET_CUDA(h, cudaMemcpyAsync(sequence_out_host, ws.stage_out, n * h->hidden * h->esize,
                               cudaMemcpyDeviceToHost, s));
  ET_CUDA(h, cudaMemcpyAsync(&h->host_pinned[0], ws.valid_word_num, 4, cudaMemcpyDeviceToHost, s));
  ET_CUDA(h, cudaMemcpyAsync(&h->host_pinned[1], ws.status, 4, cudaMemcpyDeviceToHost, s));
  ET_CUDA(h, cudaStreamSynchronize(s));
  if (valid_word_num_out) *valid_word_num_out = h->host_pinned[0];
  if (h->host_pinned[1] != 0) return device_timeout(h, s);
  return ET_OK;
}

}  // namespace

extern "C" {

int et_forward_ids_host(et_handle_t h, const int* ids_host, const int* types_host, const int* mask_host,
                        void* sequence_out_host, void* pooled_out_host, int batch_size, int seq_len,
                        int* valid_word_num_out) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  int rc = check_shape(h, batch_size, seq_len, h->cfg.head_num, h->cfg.size_per_head);
  if (rc != ET_OK) return rc;
  if (!ids_host || !mask_host) return set_error(h, ET_INVALID_ARGUMENT, "null host pointer");
  DeviceGuard guard(h->cfg.device);
  rc = forward_ids_host_body(h, ids_host, types_host, mask_host, sequence_out_host, pooled_out_host, batch_size,
                             seq_len, valid_word_num_out);
  if (rc != ET_OK) quiesce_host_call(h);
  return rc;
  ET_CATCH(h)
}

int et_pooler(et_handle_t h, const void* packed, const int* cu_seqlens, void* pooled_out, int batch_size,
              int seq_len, void* stream) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  int rc = check_shape(h, batch_size, seq_len, h->cfg.head_num, h->cfg.size_per_head);
  if (rc != ET_OK) return rc;
  if (packed == nullptr || pooled_out == nullptr) return set_error(h, ET_INVALID_ARGUMENT, "null tensor pointer");
  DeviceGuard guard(h->cfg.device);
  h->prof.chain = nullptr;
  return pooler_impl(h, packed, cu_seqlens ? cu_seqlens : h->ws.cu_seqlens, pooled_out, batch_size,
                     batch_size * seq_len, static_cast<cudaStream_t>(stream));
  ET_CATCH(h)
}

int et_last_packed_output(et_handle_t h, const void** packed, const int** valid_word_num) {
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (packed) *packed = h->ws.x;
  if (valid_word_num) *valid_word_num = h->ws.valid_word_num;
  return ET_OK;
}

}  // extern "C"

namespace {

void graph_release(et_handle_t h) {
  if (h->graph_exec) cudaGraphExecDestroy(h->graph_exec);
  if (h->graph) cudaGraphDestroy(h->graph);
  h->graph_exec = nullptr;
  h->graph = nullptr;
}

// Runs `pass` once eagerly (one-time function attributes, driver entry points
// and tensor-map encodes of first use happen outside the capture), then
// records the same pass on the handle's own stream into a graph.  The pass only
// enqueues kernels: the valid-token count stays on the device, so the graph
// depends on the buffers and on (B, S) but not on the batch's contents.
template <typename Pass>
int capture_pass(et_handle_t h, Pass pass) {
  graph_release(h);
  cudaStream_t s = h->own_stream;
  int rc = pass(s);
  if (rc != ET_OK) return rc;
  ET_CUDA(h, cudaStreamSynchronize(s));
  const bool was_profiling = h->prof.enabled;
  h->prof.enabled = false;  // event pairs inside a capture cannot be timed
  long long before[ET_PROF_NUM];
  for (int i = 0; i < ET_PROF_NUM; ++i) before[i] = h->prof.launches[i];
  cudaError_t e = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal);
  if (e != cudaSuccess) {
    h->prof.enabled = was_profiling;
    return cuda_fail(h, e, "cudaStreamBeginCapture");
  }
  rc = pass(s);
  cudaGraph_t g = nullptr;
  e = cudaStreamEndCapture(s, &g);
  h->prof.enabled = was_profiling;
  for (int i = 0; i < ET_PROF_NUM; ++i) {
    h->graph_launches[i] = h->prof.launches[i] - before[i];
    h->prof.launches[i] = before[i];  // nothing ran yet: launches are counted per replay
  }
  if (rc != ET_OK || e != cudaSuccess || g == nullptr) {
    if (g) cudaGraphDestroy(g);
    cudaGetLastError();
    return rc != ET_OK ? rc : cuda_fail(h, e, "cudaStreamEndCapture");
  }
  h->graph = g;
  e = cudaGraphInstantiate(&h->graph_exec, g, 0);
  if (e != cudaSuccess) {
    graph_release(h);
    return cuda_fail(h, e, "cudaGraphInstantiate");
  }
  return ET_OK;
}

}  // namespace

extern "C" {

int et_graph_capture(et_handle_t h, const void* from_tensor, const int* mask, void* out, int batch_size,
                     int seq_len) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  DeviceGuard guard(h->cfg.device);
  return capture_pass(h, [&](cudaStream_t s) {
    return forward_impl(h, from_tensor, mask, out, batch_size, seq_len, s);
  });
  ET_CATCH(h)
}

int et_graph_capture_ids(et_handle_t h, const int* input_ids, const int* token_type_ids, const int* mask,
                         void* sequence_out, void* pooled_out, int batch_size, int seq_len) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  DeviceGuard guard(h->cfg.device);
  return capture_pass(h, [&](cudaStream_t s) {
    return forward_ids_impl(h, input_ids, token_type_ids, mask, sequence_out, pooled_out, batch_size, seq_len, s);
  });
  ET_CATCH(h)
}

int et_graph_launch(et_handle_t h, void* stream) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (h->graph_exec == nullptr) return set_error(h, ET_NOT_READY, "no captured pass: call et_graph_capture first");
  DeviceGuard guard(h->cfg.device);
  ET_CUDA(h, cudaGraphLaunch(h->graph_exec, static_cast<cudaStream_t>(stream)));
  for (int i = 0; i < ET_PROF_NUM; ++i) h->prof.launches[i] += h->graph_launches[i];
  return ET_OK;
  ET_CATCH(h)
}

int et_graph_release(et_handle_t h) {
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  DeviceGuard guard(h->cfg.device);
  graph_release(h);
  return ET_OK;
}

int et_device_status(et_handle_t h, void* stream, int* out_status) {
  ET_TRY
  if (h == nullptr || out_status == nullptr) return ET_INVALID_ARGUMENT;
  DeviceGuard guard(h->cfg.device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  ET_CUDA(h, cudaMemcpyAsync(&h->host_pinned[1], h->ws.status, 4, cudaMemcpyDeviceToHost, s));
  ET_CUDA(h, cudaStreamSynchronize(s));
  *out_status = h->host_pinned[1];
  if (*out_status != 0) {
    ET_CUDA(h, cudaMemsetAsync(h->ws.status, 0, 4, s));
    // an aborted GEMM may have left its row counters half counted
    ET_CUDA(h, cudaMemsetAsync(h->ws.ln_counters, 0, ln_counter_ints(h->ws.cap_tokens) * 4, s));
    ET_CUDA(h, cudaStreamSynchronize(s));
  }
  return ET_OK;
  ET_CATCH(h)
}

int et_last_padding_info(et_handle_t h, const int** cu_seqlens, const int** seq_len,
                         const int** padding_offset, const int** prefix_sum) {
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  if (cu_seqlens) *cu_seqlens = h->ws.cu_seqlens;
  if (seq_len) *seq_len = h->ws.seq_len;
  if (padding_offset) *padding_offset = h->ws.padding_offset;
  if (prefix_sum) *prefix_sum = h->ws.prefix_sum;
  return ET_OK;
}

int et_set_profiling(et_handle_t h, int enable) {
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  h->prof.enabled = enable != 0;
  h->prof.chain = nullptr;
  return ET_OK;
}

int et_get_profile(et_handle_t h, double* ms_out, long long* launches_out, int reset) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  DeviceGuard guard(h->cfg.device);
  Profiler& pr = h->prof;
  for (auto& sp : pr.pending) {
    ET_CUDA(h, cudaEventSynchronize(sp.b));
    float ms = 0.f;
    ET_CUDA(h, cudaEventElapsedTime(&ms, sp.a, sp.b));
    pr.ms[sp.cat] += ms;
    if (sp.owns_a) pr.free_events.push_back(sp.a);
    pr.free_events.push_back(sp.b);
  }
  pr.pending.clear();
  pr.chain = nullptr;
  for (int i = 0; i < ET_PROF_NUM; ++i) {
    if (ms_out) ms_out[i] = pr.ms[i];
    if (launches_out) launches_out[i] = pr.launches[i];
    if (reset) {
      pr.ms[i] = 0.0;
      pr.launches[i] = 0;
    }
  }
  return ET_OK;
  ET_CATCH(h)
}

int et_copy_to_host(void* dst_host, const void* src_device, size_t bytes, void* stream) {
  if (bytes == 0) return ET_OK;
  if (dst_host == nullptr || src_device == nullptr) return ET_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(dst_host, src_device, bytes, cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return ET_CUDA_ERROR;
  return cudaStreamSynchronize(s) == cudaSuccess ? ET_OK : ET_CUDA_ERROR;
}

// ---- kernel-level entry points ---------------------------------------------
static int to_status(cudaError_t e) {
  if (e == cudaSuccess) return ET_OK;
  if (e == cudaErrorInvalidValue || e == cudaErrorMisalignedAddress) return ET_INVALID_ARGUMENT;
  return ET_CUDA_ERROR;
}

int et_padding_offsets(const int* mask, int batch_size, int seq_len, int* prefix_sum,
                       int* valid_word_num, int* batch_idx, int* word_idx, int* seq_len_out,
                       int* cu_seqlens, int* padding_offset, int* scratch, void* stream) {
  if (batch_size < 0 || seq_len < 0) return ET_INVALID_ARGUMENT;
  if (batch_size > 0 && seq_len > 0 && (mask == nullptr || scratch == nullptr)) return ET_INVALID_ARGUMENT;
  return to_status(launch_padding_offsets(mask, batch_size, seq_len, prefix_sum, valid_word_num, batch_idx,
                                          word_idx, seq_len_out, cu_seqlens, padding_offset, scratch,
                                          static_cast<cudaStream_t>(stream)));
}

#define ET_DISPATCH(dtype, CALL_HALF, CALL_FLOAT) \
  ((dtype) == ET_FP16 ? to_status(CALL_HALF) : (dtype) == ET_FP32 ? to_status(CALL_FLOAT) : ET_INVALID_ARGUMENT)

int et_remove_padding(int dtype, const void* from, const int* batch_idx, const int* word_idx,
                      const int* t_ptr, void* to, int batch, int seq, int hidden, void* stream) {
  if (!from || !batch_idx || !word_idx || !t_ptr || !to || batch < 0 || seq < 0 || hidden <= 0 ||
      (hidden * (dtype == ET_FP16 ? 2 : 4)) % 16 != 0)
    return ET_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return ET_DISPATCH(dtype,
                     launch_remove_padding<__half>(static_cast<const __half*>(from), batch_idx, word_idx, t_ptr,
                                                   static_cast<__half*>(to), batch, seq, hidden, s),
                     launch_remove_padding<float>(static_cast<const float*>(from), batch_idx, word_idx, t_ptr,
                                                  static_cast<float*>(to), batch, seq, hidden, s));
}

int et_restore_padding(int dtype, const void* from, const int* batch_idx, const int* word_idx,
                       const int* t_ptr, void* to, int batch, int seq, int hidden, void* stream) {
  if (!from || !batch_idx || !word_idx || !t_ptr || !to || batch < 0 || seq < 0 || hidden <= 0 ||
      (hidden * (dtype == ET_FP16 ? 2 : 4)) % 16 != 0)
    return ET_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return ET_DISPATCH(dtype,
                     launch_restore_padding<__half>(static_cast<const __half*>(from), batch_idx, word_idx, t_ptr,
                                                    static_cast<__half*>(to), batch, seq, hidden, s),
                     launch_restore_padding<float>(static_cast<const float*>(from), batch_idx, word_idx, t_ptr,
                                                   static_cast<float*>(to), batch, seq, hidden, s));
}

int et_add_qkv_bias_transpose(int dtype, const void* q, const void* bq, const void* k, const void* bk,
                              const void* v, const void* bv, void* out, const int* t_ptr, int max_tokens,
                              int heads, int d, void* stream) {
  if (!q || !bq || !k || !bk || !v || !bv || !out || !t_ptr || max_tokens < 0 || heads <= 0 || d <= 0)
    return ET_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define H_(p) static_cast<const __half*>(p)
#define F_(p) static_cast<const float*>(p)
  return ET_DISPATCH(dtype,
                     launch_add_qkv_bias_transpose<__half>(H_(q), H_(bq), H_(k), H_(bk), H_(v), H_(bv),
                                                           static_cast<__half*>(out), t_ptr, max_tokens, heads, d, s),
                     launch_add_qkv_bias_transpose<float>(F_(q), F_(bq), F_(k), F_(bk), F_(v), F_(bv),
                                                          static_cast<float*>(out), t_ptr, max_tokens, heads, d, s));
}

int et_add_bias_gelu(int dtype, void* out, const void* bias, const int* t_ptr, int max_tokens, int n,
                     void* stream) {
  if (!out || !bias || !t_ptr || max_tokens < 0 || n <= 0) return ET_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return ET_DISPATCH(dtype,
                     launch_add_bias_gelu<__half>(static_cast<__half*>(out), H_(bias), t_ptr, max_tokens, n, s),
                     launch_add_bias_gelu<float>(static_cast<float*>(out), F_(bias), t_ptr, max_tokens, n, s));
}

int et_add_bias_input_layernorm(int dtype, void* out, const void* input, const void* bias,
                                const void* gamma, const void* beta, const int* t_ptr, int max_tokens,
                                int n, float eps, void* stream) {
  if (!out || !input || !bias || !gamma || !beta || !t_ptr || max_tokens < 0 || n <= 0)
    return ET_INVALID_ARGUMENT;
  if (!(eps > 0.f)) eps = 1e-6f;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return ET_DISPATCH(dtype,
                     launch_add_bias_input_layernorm<__half>(static_cast<__half*>(out), H_(input), H_(bias),
                                                             H_(gamma), H_(beta), t_ptr, max_tokens, n, eps, s),
                     launch_add_bias_input_layernorm<float>(static_cast<float*>(out), F_(input), F_(bias),
                                                            F_(gamma), F_(beta), t_ptr, max_tokens, n, eps, s));
}

int et_embedding_layernorm(int dtype, const int* input_ids, const int* token_type_ids, const int* batch_idx,
                           const int* word_idx, const int* t_ptr, const void* word_table, int vocab_size,
                           const void* type_table, int type_vocab_size, const void* position_table,
                           const void* gamma, const void* beta, float eps, void* to_tensor, int batch, int seq,
                           int hidden, void* stream) {
  if (batch < 0 || seq < 0 || hidden <= 0 || (dtype != ET_FP16 && dtype != ET_FP32)) return ET_INVALID_ARGUMENT;
  if (batch == 0 || seq == 0) return ET_OK;  // no token, nothing to write
  if (!input_ids || !batch_idx || !word_idx || !t_ptr || !word_table || !gamma || !beta || !to_tensor ||
      vocab_size <= 0 || (type_table && type_vocab_size <= 0))
    return ET_INVALID_ARGUMENT;
  if (!(eps > 0.f)) eps = 1e-12f;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return ET_DISPATCH(dtype,
                     launch_embedding_layernorm<__half>(input_ids, token_type_ids, batch_idx, word_idx, t_ptr,
                                                        H_(word_table), vocab_size, H_(type_table),
                                                        type_vocab_size, H_(position_table), H_(gamma), H_(beta),
                                                        static_cast<__half*>(to_tensor), batch, seq, hidden, eps, s),
                     launch_embedding_layernorm<float>(input_ids, token_type_ids, batch_idx, word_idx, t_ptr,
                                                       F_(word_table), vocab_size, F_(type_table),
                                                       type_vocab_size, F_(position_table), F_(gamma), F_(beta),
                                                       static_cast<float*>(to_tensor), batch, seq, hidden, eps, s));
}

int et_gather_first_tokens(int dtype, const void* packed, const int* cu_seqlens, void* out, int batch_size,
                           int max_tokens, int hidden, void* stream) {
  if (!packed || !cu_seqlens || !out || batch_size < 0 || max_tokens < 0 || hidden <= 0 ||
      (dtype != ET_FP16 && dtype != ET_FP32))
    return ET_INVALID_ARGUMENT;
  return to_status(launch_gather_first_tokens(packed, cu_seqlens, out, batch_size, max_tokens,
                                              hidden * (dtype == ET_FP16 ? 2 : 4), nullptr,
                                              static_cast<cudaStream_t>(stream)));
}

int et_attention(int dtype, const void* q, const void* k, const void* v, long long token_stride,
                 long long head_stride, void* ctx, const int* cu_seqlens, int batch, int max_seq,
                 int max_tokens, int heads, int d, int use_simt, int* status_word, void* stream) {
  if (!q || !k || !v || !ctx || !cu_seqlens || batch < 0 || heads <= 0 || d != 64 || max_seq < 0 ||
      max_tokens < 0)
    return ET_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == ET_FP16 && !use_simt)
    return to_status(launch_attention_tc(H_(q), H_(k), H_(v), token_stride, head_stride,
                                         static_cast<__half*>(ctx), cu_seqlens, batch, max_seq, max_tokens,
                                         heads, d, status_word, s));
  if (dtype == ET_FP32 && !use_simt)
    return to_status(launch_attention_tf32x3(F_(q), F_(k), F_(v), token_stride, head_stride, static_cast<float*>(ctx),
                                             cu_seqlens, batch, max_seq, heads, d, s));
  return ET_DISPATCH(dtype,
                     launch_attention_simt<__half>(H_(q), H_(k), H_(v), token_stride, head_stride,
                                                   static_cast<__half*>(ctx), cu_seqlens, batch, max_seq, heads, d, s),
                     launch_attention_simt<float>(F_(q), F_(k), F_(v), token_stride, head_stride,
                                                  static_cast<float*>(ctx), cu_seqlens, batch, max_seq, heads, d, s));
}

int et_attention_cross(int dtype, const void* q, long long q_token_stride, const void* k, const void* v,
                       long long kv_token_stride, long long head_stride, void* ctx, const int* cu_seqlens_q,
                       const int* cu_seqlens_k, int batch, int max_seq_q, int max_seq_k, int heads, int d,
                       void* stream) {
  if (batch < 0 || heads <= 0 || d != 64 || max_seq_q < 0 || max_seq_k < 0 || (dtype != ET_FP16 && dtype != ET_FP32))
    return ET_INVALID_ARGUMENT;
  if (batch == 0 || max_seq_q == 0) return ET_OK;
  if (!q || !k || !v || !ctx || !cu_seqlens_q || !cu_seqlens_k) return ET_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return ET_DISPATCH(dtype,
                     launch_attention_simt<__half>(H_(q), H_(k), H_(v), q_token_stride, head_stride,
                                                   static_cast<__half*>(ctx), cu_seqlens_q, batch, max_seq_q, heads, d,
                                                   s, nullptr, cu_seqlens_k, kv_token_stride, max_seq_k),
                     launch_attention_simt<float>(F_(q), F_(k), F_(v), q_token_stride, head_stride,
                                                  static_cast<float*>(ctx), cu_seqlens_q, batch, max_seq_q, heads, d, s,
                                                  nullptr, cu_seqlens_k, kv_token_stride, max_seq_k));
}

int et_attention_general_mask(int dtype, const void* q, const void* k, const void* v, long long token_stride,
                              long long head_stride, void* ctx, const void* attr_mask, const int* cu_seqlens,
                              const int* batch_idx, const int* word_idx, const int* t_ptr, int* pos_row_scratch,
                              int batch, int seq, int heads, int d, void* stream) {
  if (batch < 0 || seq < 0 || heads <= 0 || d != 64 || (dtype != ET_FP16 && dtype != ET_FP32))
    return ET_INVALID_ARGUMENT;
  if (batch == 0 || seq == 0) return ET_OK;
  if (!q || !k || !v || !ctx || !attr_mask || !cu_seqlens || !batch_idx || !word_idx || !t_ptr || !pos_row_scratch)
    return ET_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int rc = to_status(launch_position_rows(batch_idx, word_idx, t_ptr, batch, seq, pos_row_scratch, s));
  if (rc != ET_OK) return rc;
  return ET_DISPATCH(dtype,
                     launch_attention_masked_simt<__half>(H_(q), H_(k), H_(v), token_stride, head_stride,
                                                          static_cast<__half*>(ctx), H_(attr_mask), cu_seqlens,
                                                          word_idx, pos_row_scratch, batch, seq, heads, d, s),
                     launch_attention_masked_simt<float>(F_(q), F_(k), F_(v), token_stride, head_stride,
                                                         static_cast<float*>(ctx), F_(attr_mask), cu_seqlens,
                                                         word_idx, pos_row_scratch, batch, seq, heads, d, s));
}

size_t et_attention_plan_ints(int batch_size, int max_tokens) {
  if (batch_size < 0 || max_tokens < 0) return 0;
  return attention_plan_ints(batch_size, max_tokens);
}

int et_attention_plan(const int* cu_seqlens, int batch_size, int max_tokens, int* plan, void* stream) {
  if (!cu_seqlens || !plan || batch_size < 0 || max_tokens < 0) return ET_INVALID_ARGUMENT;
  return to_status(launch_attention_plan(cu_seqlens, batch_size, max_tokens, plan,
                                         static_cast<cudaStream_t>(stream)));
}

int et_attention_tiles(const void* q, const void* k, const void* v, long long token_stride,
                       long long head_stride, void* ctx, const int* plan, int batch_size, int max_seq_len,
                       int max_tokens, int head_num, int size_per_head, int* status_word, void* stream) {
  if (!q || !k || !v || !ctx || !plan || batch_size < 0 || head_num <= 0 || size_per_head != 64 ||
      max_seq_len < 0 || max_seq_len > 128 || max_tokens < 0)
    return ET_INVALID_ARGUMENT;
  return to_status(launch_attention_tcgen05(H_(q), H_(k), H_(v), token_stride, head_stride,
                                            static_cast<__half*>(ctx), plan, batch_size, max_tokens, head_num,
                                            size_per_head, status_word, static_cast<cudaStream_t>(stream)));
}

int et_attention_tiles_general_mask(const void* q, const void* k, const void* v, long long token_stride,
                                    long long head_stride, void* ctx, const int* plan, const void* attr_mask,
                                    const int* batch_idx, const int* word_idx, int batch_size, int seq_len,
                                    int max_tokens, int head_num, int size_per_head, int* status_word,
                                    void* stream) {
  if (!q || !k || !v || !ctx || !plan || !attr_mask || !batch_idx || !word_idx || batch_size < 0 || head_num <= 0 ||
      size_per_head != 64 || seq_len <= 0 || seq_len > 128 || max_tokens < 0)
    return ET_INVALID_ARGUMENT;
  return to_status(launch_attention_tcgen05(H_(q), H_(k), H_(v), token_stride, head_stride,
                                            static_cast<__half*>(ctx), plan, batch_size, max_tokens, head_num,
                                            size_per_head, status_word, static_cast<cudaStream_t>(stream), false,
                                            nullptr, H_(attr_mask), batch_idx, word_idx, seq_len));
}

int et_gemm(int dtype, const void* a, const void* w, const void* w_packed, const void* bias, void* c,
            const int* m_ptr, int max_m, int n, int k, int epilogue, int use_simt, int* status_word,
            void* stream) {
  if (!a || !c || !m_ptr || max_m < 0 || n <= 0 || k <= 0 || epilogue < 0 || epilogue > 3)
    return ET_INVALID_ARGUMENT;
  if (epilogue != 0 && !bias) return ET_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == ET_FP16 && !use_simt) {
    if (!w_packed) return ET_INVALID_ARGUMENT;
    return to_status(launch_gemm_tcgen05(H_(a), H_(w_packed), H_(bias), static_cast<__half*>(c), m_ptr, max_m,
                                         n, k, epilogue, status_word, s));
  }
  if (!w) return ET_INVALID_ARGUMENT;
  return ET_DISPATCH(dtype,
                     launch_gemm_simt<__half>(H_(a), H_(w), H_(bias), static_cast<__half*>(c), m_ptr, max_m, n, k,
                                              epilogue, s),
                     launch_gemm_simt<float>(F_(a), F_(w), F_(bias), static_cast<float*>(c), m_ptr, max_m, n, k,
                                             epilogue, s));
}

int et_gemm_fused(const void* a, const void* w_packed, const void* bias, const void* residual, const void* gamma,
                  const void* beta, float eps, int* row_counters, void* c, const int* m_ptr, int max_m, int n,
                  int k, int epilogue, int* status_word, void* stream) {
  if (!a || !w_packed || !bias || !residual || !c || !m_ptr || max_m < 0 || n <= 0 || k <= 0)
    return ET_INVALID_ARGUMENT;
  if (epilogue != kEpiBiasResidual && epilogue != kEpiResidualLayerNorm && epilogue != kEpiLayerNorm)
    return ET_INVALID_ARGUMENT;
  GemmLayerNorm ln;
  if (epilogue != kEpiBiasResidual) {
    if (!gamma || !beta || !row_counters || !gemm_layernorm_supported(n)) return ET_INVALID_ARGUMENT;
    ln.gamma = H_(gamma);
    ln.beta = H_(beta);
    ln.eps = eps > 0.f ? eps : 1e-6f;
    ln.counters = row_counters;
  }
  return to_status(launch_gemm_tcgen05(H_(a), H_(w_packed), H_(bias), static_cast<__half*>(c), m_ptr, max_m, n, k,
                                       epilogue, status_word, static_cast<cudaStream_t>(stream), false,
                                       H_(residual), nullptr, &ln));
}

int et_fold_layernorm(const void* w_packed, const void* bias, const void* gamma, const void* beta, void* w_folded,
                      void* csum, void* bias_folded, int n, int k, void* stream) {
  if (!w_packed || !bias || !gamma || !beta || !w_folded || !csum || !bias_folded || n <= 0 || k <= 0)
    return ET_INVALID_ARGUMENT;
  return to_status(launch_fold_layernorm(H_(w_packed), H_(bias), H_(gamma), H_(beta), static_cast<__half*>(w_folded),
                                         static_cast<__half*>(csum), static_cast<__half*>(bias_folded), n, k,
                                         static_cast<cudaStream_t>(stream)));
}

int et_gemm_deferred_norm(const void* a, const void* w_packed, const void* bias, const void* csum,
                          const void* residual, const void* gamma, const void* beta, float eps,
                          const float* stats_in, float* stats_out, void* c, const int* m_ptr, int max_m, int n,
                          int k, int epilogue, int* status_word, void* stream) {
  if (!a || !w_packed || !bias || !c || !m_ptr || max_m < 0 || n <= 0 || k <= 0) return ET_INVALID_ARGUMENT;
  if (!is_deferred_norm(epilogue)) return ET_INVALID_ARGUMENT;
  GemmLayerNorm ln;
  ln.eps = eps > 0.f ? eps : 1e-6f;
  ln.stats_in = stats_in;
  ln.stat_slots = (epilogue == kEpiNormResidual ? n : k) / 64;
  ln.csum = H_(csum);
  ln.gamma = H_(gamma);
  ln.beta = H_(beta);
  ln.stats_out = stats_out;
  return to_status(launch_gemm_tcgen05(H_(a), H_(w_packed), H_(bias), static_cast<__half*>(c), m_ptr, max_m, n, k,
                                       epilogue, status_word, static_cast<cudaStream_t>(stream), false,
                                       H_(residual), nullptr, &ln));
}

int et_selftest_wait_timeout(et_handle_t h, void* stream) {
  ET_TRY
  if (h == nullptr) return ET_INVALID_ARGUMENT;
  DeviceGuard guard(h->cfg.device);
  ET_CUDA(h, launch_selftest_wait_timeout(h->ws.status, static_cast<cudaStream_t>(stream)));
  return ET_OK;
  ET_CATCH(h)
}

int et_split_tf32(const float* x, float* hi, float* lo, const int* rows_ptr, int max_rows, int cols,
                  void* stream) {
  if (max_rows < 0 || cols < 0) return ET_INVALID_ARGUMENT;
  if (max_rows == 0 || cols == 0) return ET_OK;
  if (!x || !hi || !lo) return ET_INVALID_ARGUMENT;
  return to_status(launch_split_tf32(x, hi, lo, rows_ptr, max_rows, cols, static_cast<cudaStream_t>(stream)));
}

int et_gemm_fp32_tensor(const float* a_hi, const float* a_lo, const float* w_hi, const float* w_lo,
                        const float* bias, float* c, const int* m_ptr, int max_m, int n, int k, int epilogue,
                        int* status_word, void* stream) {
  if (!m_ptr || max_m < 0 || n <= 0 || k <= 0 || epilogue < 0 || epilogue > 3) return ET_INVALID_ARGUMENT;
  if (epilogue != 0 && !bias) return ET_INVALID_ARGUMENT;
  if (max_m == 0) return ET_OK;
  if (!a_hi || !a_lo || !w_hi || !w_lo || !c) return ET_INVALID_ARGUMENT;
  return to_status(launch_gemm_tf32x3(a_hi, a_lo, w_hi, w_lo, bias, c, m_ptr, max_m, n, k, epilogue, status_word,
                                      static_cast<cudaStream_t>(stream)));
}

int et_pack_weight(int dtype, const void* w, void* w_packed, int k, int n, void* stream) {
  if (!w || !w_packed || k <= 0 || n <= 0) return ET_INVALID_ARGUMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return ET_DISPATCH(dtype, launch_transpose<__half>(H_(w), static_cast<__half*>(w_packed), k, n, s),
                     launch_transpose<float>(F_(w), static_cast<float*>(w_packed), k, n, s));
}
#undef H_
#undef F_

}  // extern "C"
