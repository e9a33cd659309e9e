"""TEST INFRASTRUCTURE - CPU oracle: a restatement of the reference's padded
TF-graph BERT encoder (sample/tensorflow/modeling.py) in torch-on-CPU.  Only
tests, the smoke check and the benchmark's CPU-baseline / reference leg may
import this module; the product path never does.

Parity status: the reference ships no tests, fixtures or golden vectors for
this path and its TF-1.15 graph cannot be imported here (TensorFlow is absent):
the whole-model function is UNPINNED by a run of the reference's TF graph.
What it is held to instead:
(a) the reference's own CUDA kernels, compiled unmodified from the reference
    checkout (oracle/build_ref.py) and run on the GPU box: LayerNorm, bias+GELU
    and the attention block (QKV bias + re-padding, softmax, head merge) agree
    with the per-kernel functions below within one rounding of the storage
    type (tests/test_reference_kernels_gpu.py);
(b) an independent implementation of the same architecture
    (tests/golden/make_golden.py, Hugging Face ``BertEncoder`` with the tanh
    GELU), to 5e-15 in float64;
(c) its own float64 evaluation;
(b) and (c) are stored in tests/golden/.

Third-party arithmetic the reference relies on and that is restated here from
its published definition: TensorFlow 1.15.3 ``tf.layers.dense`` (x @ W + b with
W of shape [in, out]), ``tf.nn.softmax`` (last axis), ``tf.tanh``/``tf.pow`` and
``tf.contrib.layers.layer_norm`` (biased variance over the last axis,
variance epsilon 1e-12, then * gamma + beta).

fp16 policy: inputs and weights are rounded to fp16 first, the arithmetic runs
in ``compute_dtype`` (float32 or float64).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

TF_LAYER_NORM_EPS = 1e-12      # tf.contrib.layers.layer_norm's variance_epsilon
DEVICE_LAYER_NORM_EPS = 1e-6   # cuda/cuda_kernels.cu:183,227


def _t(a, dtype) -> torch.Tensor:
    if isinstance(a, torch.Tensor):
        return a.to(dtype)
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype)


def gelu(x: torch.Tensor) -> torch.Tensor:
    """tanh form, sample/tensorflow/modeling.py:264-277."""
    cdf = 0.5 * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * torch.pow(x, 3))))
    return x * cdf


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor,
               eps: float = TF_LAYER_NORM_EPS) -> torch.Tensor:
    """sample/tensorflow/modeling.py:362-365 (last axis, learned gamma/beta)."""
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    return (x - mean) * torch.rsqrt(var + eps) * gamma + beta


def dense(x: torch.Tensor, kernel: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """tf.layers.dense: kernel is [in, out]."""
    return x @ kernel + bias


def attention_layer(x2d: torch.Tensor, attention_mask: Optional[torch.Tensor],
                    wq, bq, wk, bk, wv, bv, batch: int, seq: int, heads: int, d: int,
                    stages: Optional[Dict[str, torch.Tensor]] = None) -> torch.Tensor:
    """sample/tensorflow/modeling.py:558-752 with from_tensor == to_tensor.
    ``attention_mask`` is [B, S, S] (1 = attend)."""
    q = dense(x2d, wq, bq)                                   # :666-671
    k = dense(x2d, wk, bk)                                   # :674-679
    v = dense(x2d, wv, bv)                                   # :682-687
    if stages is not None:
        stages["q"], stages["k"], stages["v"] = q, k, v
    q = q.reshape(batch, seq, heads, d).permute(0, 2, 1, 3)  # :690-692
    k = k.reshape(batch, seq, heads, d).permute(0, 2, 1, 3)  # :695-696
    scores = torch.matmul(q, k.transpose(-1, -2)) * (1.0 / math.sqrt(float(d)))  # :701-703
    if attention_mask is not None:
        adder = (1.0 - attention_mask.unsqueeze(1)) * -10000.0   # :705-717
        scores = scores + adder
    probs = torch.softmax(scores, dim=-1)                    # :721
    v = v.reshape(batch, seq, heads, d).permute(0, 2, 1, 3)  # :728-733
    ctx = torch.matmul(probs, v)                             # :736
    ctx = ctx.permute(0, 2, 1, 3).reshape(batch * seq, heads * d)  # :739-745
    if stages is not None:
        stages["context"] = ctx
    return ctx


def transformer_model(from_tensor, attention_mask, weights: Sequence, heads: int, d: int,
                      compute_dtype=torch.float32, round_to_fp16: bool = False,
                      ln_eps: float = TF_LAYER_NORM_EPS,
                      layer0_stages: Optional[Dict[str, torch.Tensor]] = None,
                      all_layers: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """The padded encoder stack, sample/tensorflow/modeling.py:755-893.

    from_tensor [B, S, H]; attention_mask [B, S, S] or None; ``weights`` is the
    flat list of 16 arrays per layer in the order of
    python/effective_transformer/__init__.py:55-74.  Returns [B, S, H]."""
    def prep(a):
        if isinstance(a, torch.Tensor) and a.dtype == compute_dtype and not round_to_fp16:
            return a                                         # already in the working precision
        t = _t(a, torch.float32)
        if round_to_fp16:
            t = t.to(torch.float16).to(torch.float32)
        return t.to(compute_dtype)

    x = prep(from_tensor)
    batch, seq, hidden = x.shape
    assert hidden == heads * d
    mask = None if attention_mask is None else _t(attention_mask, compute_dtype)
    num_layers = len(weights) // 16
    prev = x.reshape(batch * seq, hidden)                    # :826
    for l in range(num_layers):
        w = [prep(a) for a in weights[l * 16:(l + 1) * 16]]
        stages = layer0_stages if (l == 0 and layer0_stages is not None) else None
        layer_input = prev
        ctx = attention_layer(layer_input, mask, w[0], w[1], w[2], w[3], w[4], w[5],
                              batch, seq, heads, d, stages)
        att = dense(ctx, w[6], w[7])                         # :855-858
        att = layer_norm(att + layer_input, w[9], w[8], ln_eps)   # :859-860
        inter = gelu(dense(att, w[10], w[11]))               # :863-868
        out = dense(inter, w[12], w[13])                     # :871-875
        out = layer_norm(out + att, w[15], w[14], ln_eps)    # :876-877
        if stages is not None:
            stages["attention_output"], stages["intermediate"], stages["layer_output"] = att, inter, out
        if all_layers is not None:
            all_layers.append(out.reshape(batch, seq, hidden))
        prev = out
    return prev.reshape(batch, seq, hidden)                  # :890-892


def embedding_lookup(input_ids, word_table: torch.Tensor) -> torch.Tensor:
    """sample/tensorflow/modeling.py:380-422: gather of word_table rows,
    [B, S] ids -> [B, S, H]."""
    ids = torch.from_numpy(np.asarray(input_ids).astype(np.int64))
    return word_table[ids]


def embedding_postprocessor(x: torch.Tensor, token_type_ids, type_table: Optional[torch.Tensor],
                            position_table: Optional[torch.Tensor], gamma: torch.Tensor,
                            beta: torch.Tensor, eps: float = TF_LAYER_NORM_EPS) -> torch.Tensor:
    """sample/tensorflow/modeling.py:425-521: + token-type rows (:471-484, the
    one-hot matmul is a row gather), + the first S position rows (:486-518),
    then LayerNorm (:520; dropout is the identity at inference)."""
    b, s, h = x.shape
    out = x
    if type_table is not None:
        tt = torch.from_numpy(np.asarray(token_type_ids).astype(np.int64))
        out = out + type_table[tt]
    if position_table is not None:
        assert s <= position_table.shape[0]                  # :487
        out = out + position_table[:s].unsqueeze(0)
    return layer_norm(out, gamma, beta, eps)


def pooler(sequence_output: torch.Tensor, kernel: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """sample/tensorflow/modeling.py:224-232: tanh(dense(first token)),
    [B, S, H] -> [B, H]."""
    return torch.tanh(dense(sequence_output[:, 0, :], kernel, bias))


def bert_model(heads, mask: np.ndarray, weights: Sequence, head_num: int, d: int,
               compute_dtype=torch.float32, round_to_fp16: bool = False,
               embedding_eps: float = TF_LAYER_NORM_EPS, ln_eps: float = TF_LAYER_NORM_EPS,
               zero_padded_rows: bool = False):
    """BertModel of sample/tensorflow/modeling.py:107-235 at inference:
    embeddings -> encoder stack -> pooler.  ``heads`` carries the ids and
    tables (an object with the fields of workloads.ModelHeads).  Returns
    (embedding_output [B,S,H], sequence_output [B,S,H], pooled_output [B,H]).

    ``zero_padded_rows``: the padding-free ops hand back zeros at padded
    positions (tf_op/bert_transformer_op.cu.cc:354-360), so a sequence whose
    first position is padding pools a zero row; set it to state that variant."""
    def prep(a):
        t = _t(a, torch.float32)
        if round_to_fp16:
            t = t.to(torch.float16).to(torch.float32)
        return t.to(compute_dtype)

    emb = embedding_lookup(heads.input_ids, prep(heads.word_table))
    emb = embedding_postprocessor(emb, heads.token_type_ids, prep(heads.type_table),
                                  prep(heads.position_table), prep(heads.ln_gamma),
                                  prep(heads.ln_beta), embedding_eps)
    if round_to_fp16:
        emb = emb.to(torch.float16).to(compute_dtype)        # the stage's output tensor is fp16
    b, s = mask.shape
    am = np.tile(mask, s).reshape(b, s, s)                   # modeling.py:524-555 for a key mask
    seq_out = transformer_model(emb, am, weights, head_num, d, compute_dtype=compute_dtype,
                                round_to_fp16=round_to_fp16, ln_eps=ln_eps)
    pool_in = seq_out
    if zero_padded_rows:
        pool_in = seq_out * torch.from_numpy(np.asarray(mask)).to(compute_dtype).unsqueeze(-1)
    pooled = pooler(pool_in, prep(heads.pooler_kernel), prep(heads.pooler_bias))
    return emb, seq_out, pooled


def valid_rows(y: torch.Tensor, mask: np.ndarray) -> torch.Tensor:
    """Rows of [B, S, H] at mask == 1 in (b, s) order: the comparison domain of
    sample/tensorflow/benchmark.py:105-112."""
    b, s, h = y.shape
    sel = torch.from_numpy(np.asarray(mask).ravel() > 0)
    return y.reshape(b * s, h)[sel]


# ----------------------------------------------------------------------------
# Per-kernel restatements (packed layout), used by the kernel-level parity tests
# ----------------------------------------------------------------------------

def add_bias_gelu(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """add_bias_act (cuda/cuda_kernels.cu:88-134): gelu(x + bias)."""
    return gelu(x + bias)


def add_bias_input_layernorm(out: torch.Tensor, inp: torch.Tensor, bias: torch.Tensor,
                             gamma: torch.Tensor, beta: torch.Tensor,
                             eps: float = DEVICE_LAYER_NORM_EPS) -> torch.Tensor:
    """add_bias_input_layernorm (cuda/cuda_kernels.cu:157-236):
    LN(out + input + bias) * gamma + beta with eps 1e-6."""
    return layer_norm(out + inp + bias, gamma, beta, eps)


def packed_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: np.ndarray,
                     heads: int, d: int) -> torch.Tensor:
    """Self-attention on packed [T, H] tensors, one softmax per (sequence,
    head) over that sequence's own tokens.  Equals the padded computation of
    modeling.py:690-745 restricted to valid rows when the 3-D mask is the
    key-only tile of the input mask (exp(-10000) underflows to zero)."""
    t = q.shape[0]
    out = torch.zeros_like(q)
    scale = 1.0 / math.sqrt(float(d))
    for b in range(len(cu_seqlens) - 1):
        lo, hi = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
        if hi <= lo:
            continue
        n = hi - lo
        qb = q[lo:hi].reshape(n, heads, d).permute(1, 0, 2)
        kb = k[lo:hi].reshape(n, heads, d).permute(1, 0, 2)
        vb = v[lo:hi].reshape(n, heads, d).permute(1, 0, 2)
        p = torch.softmax(torch.matmul(qb, kb.transpose(-1, -2)) * scale, dim=-1)
        out[lo:hi] = torch.matmul(p, vb).permute(1, 0, 2).reshape(n, heads * d)
    assert out.shape[0] == t
    return out


def cross_attention_padded(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, attention_mask: torch.Tensor,
                           heads: int, d: int) -> torch.Tensor:
    """The core of attention_layer with from_tensor != to_tensor (sample/tensorflow/modeling.py:
    690-745): q is [B, F, heads*d] (already projected), k and v [B, T, heads*d], attention_mask
    [B, F, T] (1 = attend).  Returns the context [B, F, heads*d]."""
    b, f, _ = q.shape
    t = k.shape[1]
    qh = q.reshape(b, f, heads, d).permute(0, 2, 1, 3)                      # :690-692
    kh = k.reshape(b, t, heads, d).permute(0, 2, 1, 3)                      # :695-696
    scores = torch.matmul(qh, kh.transpose(-1, -2)) * (1.0 / math.sqrt(float(d)))   # :701-703
    scores = scores + (1.0 - attention_mask.unsqueeze(1).to(q.dtype)) * -10000.0    # :705-717
    probs = torch.softmax(scores, dim=-1)                                    # :721
    vh = v.reshape(b, t, heads, d).permute(0, 2, 1, 3)                      # :728-733
    return torch.matmul(probs, vh).permute(0, 2, 1, 3).reshape(b, f, heads * d)     # :736-745


def packed_attention_general_mask(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                                  cu_seqlens: np.ndarray, word_idx: np.ndarray, attr_mask: torch.Tensor,
                                  seq: int, heads: int, d: int) -> torch.Tensor:
    """The attention block of the reference op under a general [B, S, S] mask:
    valid rows are scattered into zero-filled padded [B, heads, S, d] buffers
    (cuda/attention.cu:106-242, memset at tf_op/bert_transformer_op.cu.cc:146),
    so a padded key takes part with K = V = 0; softmax of
    score/sqrt(d) + (1 - m) * -10000 over all S keys (cuda/attention.cu:249-382,
    without the kernel's +1e-6 in the denominator); valid rows gathered back
    (cuda/attention.cu:388-492).  ``word_idx[v]`` is the position of packed row v."""
    out = torch.zeros_like(q)
    scale = 1.0 / math.sqrt(float(d))
    for b in range(len(cu_seqlens) - 1):
        lo, hi = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
        if hi <= lo:
            continue
        pos = torch.from_numpy(np.asarray(word_idx[lo:hi]).astype(np.int64))
        n = hi - lo
        qb = q[lo:hi].reshape(n, heads, d).permute(1, 0, 2)
        kp = torch.zeros(heads, seq, d, dtype=q.dtype)
        vp = torch.zeros(heads, seq, d, dtype=q.dtype)
        kp[:, pos] = k[lo:hi].reshape(n, heads, d).permute(1, 0, 2)
        vp[:, pos] = v[lo:hi].reshape(n, heads, d).permute(1, 0, 2)
        m = attr_mask[b][pos].to(q.dtype)                     # [n, S]: the mask rows of the valid queries
        scores = torch.matmul(qb, kp.transpose(-1, -2)) * scale + (1.0 - m).unsqueeze(0) * -10000.0
        p = torch.softmax(scores, dim=-1)
        out[lo:hi] = torch.matmul(p, vp).permute(1, 0, 2).reshape(n, heads * d)
    return out


def packed_encoder(x_packed, cu_seqlens: np.ndarray, weights: Sequence, heads: int, d: int,
                   compute_dtype=torch.float32, round_to_fp16: bool = False,
                   ln_eps: float = DEVICE_LAYER_NORM_EPS, attr_mask=None, word_idx=None,
                   seq: Optional[int] = None) -> torch.Tensor:
    """The same stack evaluated on the packed [T, H] layout in the order of the
    reference's layer functor (tf_op/bert_transformer_op.cu.cc:104-246).  With
    ``attr_mask`` [B, S, S] (plus ``word_idx`` and ``seq``) the attention block is
    packed_attention_general_mask, i.e. the op's behaviour under a general mask."""
    def prep(a):
        t = _t(a, torch.float32)
        if round_to_fp16:
            t = t.to(torch.float16).to(torch.float32)
        return t.to(compute_dtype)

    x = prep(x_packed)
    for l in range(len(weights) // 16):
        w = [prep(a) for a in weights[l * 16:(l + 1) * 16]]
        q, k, v = dense(x, w[0], w[1]), dense(x, w[2], w[3]), dense(x, w[4], w[5])
        if attr_mask is None:
            ctx = packed_attention(q, k, v, cu_seqlens, heads, d)
        else:
            ctx = packed_attention_general_mask(q, k, v, cu_seqlens, word_idx, _t(attr_mask, compute_dtype),
                                                seq, heads, d)
        att = add_bias_input_layernorm(ctx @ w[6], x, w[7], w[9], w[8], ln_eps)
        inter = add_bias_gelu(att @ w[10], w[11])
        x = add_bias_input_layernorm(inter @ w[12], att, w[13], w[15], w[14], ln_eps)
    return x
