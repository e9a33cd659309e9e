"""B200-native padding-free BERT encoder path.

Python mirror of the reference's package shim
(python/effective_transformer/__init__.py): the same three operators
(`effective_transformer_input`, `effective_transformer`,
`effective_transformer_output`) and `get_sequence_output`, with the same
argument meaning, on top of the C ABI in include/et_b200.h.  PyTorch is used
for device memory and streams only; all arithmetic runs in the sm_100a kernels
of libet_b200.so.  There is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _capi
from ._capi import EtError  # noqa: F401

__all__ = ["BertConfig", "EffectiveTransformer", "get_sequence_output", "EtError"]


@dataclass
class BertConfig:
    """The fields of sample/tensorflow/modeling.py's BertConfig that the
    encoder path reads (sample/tensorflow/bert_config.json)."""
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    vocab_size: int = 30522
    type_vocab_size: int = 2
    max_position_embeddings: int = 512


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class EffectiveTransformer:
    """One handle = the weights of all layers + workspace on one GPU.

    Replaces the three TF op kernels and their constructors
    (tf_op/bert_transformer_op.cc:84-447)."""

    def __init__(self, num_layers: int, head_num: int, size_per_head: int, ffn_dim: int,
                 max_batch_size: int, max_seq_length: int, dtype: torch.dtype = torch.float16,
                 device: int = 0, layernorm_eps: float = 0.0):
        if dtype not in (torch.float16, torch.float32):
            raise ValueError("dtype must be torch.float16 or torch.float32")
        self._lib = _capi.load()
        self.dtype = dtype
        self.np_dtype = np.float16 if dtype == torch.float16 else np.float32
        self.et_dtype = _capi.ET_FP16 if dtype == torch.float16 else _capi.ET_FP32
        self.num_layers, self.head_num, self.size_per_head = num_layers, head_num, size_per_head
        self.hidden, self.ffn_dim = head_num * size_per_head, ffn_dim
        self.max_batch_size, self.max_seq_length = max_batch_size, max_seq_length
        self.device = torch.device("cuda", device)
        cfg = _capi.Config(self.et_dtype, num_layers, head_num, size_per_head, ffn_dim,
                           max_batch_size, max_seq_length, layernorm_eps, device)
        handle = C.c_void_p()
        _capi.check(self._lib.et_create(C.byref(cfg), C.byref(handle)))
        self._h = handle

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.et_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- weights ---------------------------------------------------------
    def set_layer_weights(self, layer: int, weights: Sequence) -> None:
        """16 arrays in the order of python/effective_transformer/__init__.py:55-74
        (numpy arrays or torch tensors; converted to the handle's dtype)."""
        if len(weights) != 16:
            raise ValueError("a layer takes 16 weight arrays")
        host: List[np.ndarray] = []
        for w in weights:
            a = w.detach().cpu().numpy() if isinstance(w, torch.Tensor) else np.asarray(w)
            host.append(np.ascontiguousarray(a.astype(self.np_dtype, copy=False)))
        arr = (C.c_void_p * 16)(*[a.ctypes.data for a in host])
        _capi.check(self._lib.et_set_layer_weights(self._h, layer, arr, 1), self._h)

    def set_weights(self, weights_value: Sequence) -> None:
        if len(weights_value) != 16 * self.num_layers:
            raise ValueError("weights_value must hold 16 arrays per layer")
        for l in range(self.num_layers):
            self.set_layer_weights(l, weights_value[l * 16:(l + 1) * 16])

    def set_debug_simt(self, on: bool) -> None:
        _capi.check(self._lib.et_set_debug_simt(self._h, 1 if on else 0), self._h)

    def set_fused_layernorm(self, on: bool) -> None:
        """On: bias + residual + LayerNorm run inside the two hidden-wide projection kernels, on
        their own output rows (5 launches per layer); takes precedence over the deferred LayerNorm."""
        _capi.check(self._lib.et_set_fused_layernorm(self._h, 1 if on else 0), self._h)

    def set_deferred_layernorm(self, on: bool) -> None:
        """On (default where the widths allow it): the whole-stack calls materialise no LayerNorm
        between the projections (producers leave row statistics, consumers run on folded weights);
        only the last one runs as a kernel.  Off: a LayerNorm kernel behind each hidden-wide projection."""
        _capi.check(self._lib.et_set_deferred_layernorm(self._h, 1 if on else 0), self._h)

    def workspace_bytes(self, batch_size: int, seq_len: int) -> int:
        n = C.c_size_t(0)
        _capi.check(self._lib.et_workspace_bytes(self._h, batch_size, seq_len, C.byref(n)), self._h)
        return int(n.value)

    def workspace_allocated_bytes(self) -> int:
        n = C.c_size_t(0)
        _capi.check(self._lib.et_workspace_allocated_bytes(self._h, C.byref(n)), self._h)
        return int(n.value)

    def host_chunk_shares(self) -> Tuple[int, int, bool]:
        """(chunks, share of a middle chunk, whether the share was measured by the handle)."""
        c, m, f = C.c_int(0), C.c_int(0), C.c_int(0)
        _capi.check(self._lib.et_host_chunk_shares(self._h, C.byref(c), C.byref(m), C.byref(f)), self._h)
        return int(c.value), int(m.value), bool(f.value)

    def selftest_wait_timeout(self) -> None:
        """Launches the failure-detection self-test kernel (a 2 ms bounded wait that runs out)."""
        _capi.check(self._lib.et_selftest_wait_timeout(self._h, _stream()), self._h)

    def set_general_mask(self, on: bool) -> None:
        """When on, effective_transformer() reads its attention_mask [B,S,S] (dtype of
        the handle, 1 = attend) through the general-mask attention kernel; when off
        (default) the mask must be the key-only tile of input_mask and is not read."""
        _capi.check(self._lib.et_set_general_mask(self._h, 1 if on else 0), self._h)

    def forward_general_mask(self, from_tensor: torch.Tensor, input_mask: torch.Tensor,
                             attention_mask: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """forward() under a general [B,S,S] attention mask (semantics of the
        reference op: padded keys take part with K = V = 0)."""
        self._check_act(from_tensor, "from_tensor")
        self._check_act(attention_mask, "attention_mask")
        b, s, _ = from_tensor.shape
        if tuple(attention_mask.shape) != (b, s, s):
            raise ValueError("attention_mask must be [B, S, S]")
        mask = self._i32(input_mask)
        if out is None:
            out = torch.empty_like(from_tensor)
        _capi.check(self._lib.et_forward_general_mask(self._h, _ptr(from_tensor), _ptr(mask), _ptr(attention_mask),
                                                      _ptr(out), b, s, _stream()), self._h)
        return out

    # ---- the three operators ----------------------------------------------
    def _check_act(self, t: torch.Tensor, name: str) -> None:
        if t.dtype != self.dtype or not t.is_cuda or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous CUDA tensor of dtype {self.dtype}")

    def effective_transformer_input(self, from_tensor: torch.Tensor, input_mask: torch.Tensor
                                    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        """(from_tensor [B,S,H], mask int32 [B,S]) -> (to_tensor [B,S,H] with the
        first T rows packed, valid_word_num [1], batch_idx [B,S], word_idx [B,S])
        as tf_op/bert_transformer_op.cc:249-274."""
        self._check_act(from_tensor, "from_tensor")
        b, s, _ = from_tensor.shape
        mask = input_mask.to(torch.int32).contiguous()
        to_tensor = torch.empty_like(from_tensor)
        valid = torch.zeros(1, dtype=torch.int32, device=from_tensor.device)
        batch_idx = torch.zeros((b, s), dtype=torch.int32, device=from_tensor.device)
        word_idx = torch.zeros((b, s), dtype=torch.int32, device=from_tensor.device)
        p = _capi.InputParam(_ptr(from_tensor), _ptr(mask), _ptr(valid), _ptr(batch_idx), _ptr(word_idx),
                             b, s, self.head_num, self.size_per_head, _ptr(to_tensor), _stream())
        _capi.check(self._lib.et_input(self._h, C.byref(p)), self._h)
        return to_tensor, valid, batch_idx, word_idx

    def effective_transformer(self, layer_idx: int, from_tensor: torch.Tensor, to_tensor: torch.Tensor,
                              attention_mask: Optional[torch.Tensor], valid_word_num: torch.Tensor,
                              batch_idx: torch.Tensor, word_idx: torch.Tensor) -> torch.Tensor:
        """One encoder layer on the packed layout (tf_op/bert_transformer_op.cc:44-77);
        the layer's weights are those registered with set_layer_weights."""
        self._check_act(from_tensor, "from_tensor")
        if to_tensor.data_ptr() != from_tensor.data_ptr():
            raise ValueError("to_tensor must be from_tensor (self-attention)")
        b, s, _ = from_tensor.shape
        out = torch.empty_like(from_tensor)
        p = _capi.EncoderParam()
        p.from_tensor, p.to_tensor = _ptr(from_tensor), _ptr(to_tensor)
        p.attr_mask = _ptr(attention_mask)
        p.batch_idx, p.word_idx, p.valid_word_num = _ptr(batch_idx), _ptr(word_idx), _ptr(valid_word_num)
        p.transformer_out, p.stream = _ptr(out), _stream()
        tp = _capi.TransformerParam(b, s, s, self.head_num, self.size_per_head)
        _capi.check(self._lib.et_layer(self._h, layer_idx, C.byref(p), C.byref(tp)), self._h)
        return out

    def effective_transformer_output(self, from_tensor: torch.Tensor, valid_word_num: torch.Tensor,
                                     batch_idx: torch.Tensor, word_idx: torch.Tensor) -> torch.Tensor:
        """Packed [T,H] (inside a [B,S,H] tensor) -> padded [B,S,H], padding rows
        zero (tf_op/bert_transformer_op.cc:359-380)."""
        self._check_act(from_tensor, "from_tensor")
        b, s, _ = from_tensor.shape
        out = torch.empty_like(from_tensor)
        p = _capi.OutputParam(_ptr(from_tensor), _ptr(valid_word_num), _ptr(batch_idx), _ptr(word_idx),
                              b, s, self.head_num, self.size_per_head, _ptr(out), _stream())
        _capi.check(self._lib.et_output(self._h, C.byref(p)), self._h)
        return out

    # ---- whole path --------------------------------------------------------
    def forward(self, from_tensor: torch.Tensor, input_mask: torch.Tensor,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Input op, all layers, output op on the current stream (device tensors)."""
        self._check_act(from_tensor, "from_tensor")
        b, s, _ = from_tensor.shape
        if input_mask.dtype != torch.int32 or not input_mask.is_contiguous():
            input_mask = input_mask.to(torch.int32).contiguous()
        if out is None:
            out = torch.empty_like(from_tensor)
        _capi.check(self._lib.et_forward(self._h, _ptr(from_tensor), _ptr(input_mask), _ptr(out), b, s,
                                         _stream()), self._h)
        return out

    def forward_host(self, from_tensor: np.ndarray, input_mask: np.ndarray,
                     out: Optional[np.ndarray] = None) -> Tuple[np.ndarray, int]:
        """Same with host arrays: host->device copies, the forward pass and the
        device->host copy of the result happen inside the call."""
        if from_tensor.dtype != self.np_dtype or input_mask.dtype != np.int32:
            raise ValueError("from_tensor must have the handle's dtype and input_mask must be int32")
        from_tensor = np.ascontiguousarray(from_tensor)
        input_mask = np.ascontiguousarray(input_mask)
        b, s, _ = from_tensor.shape
        if out is None:
            out = np.empty_like(from_tensor)
        t = C.c_int(0)
        _capi.check(self._lib.et_forward_host(self._h, from_tensor.ctypes.data, input_mask.ctypes.data,
                                              out.ctypes.data, b, s, C.byref(t)), self._h)
        return out, int(t.value)

    # ---- the model around the stack ----------------------------------------
    def _host(self, a) -> Optional[np.ndarray]:
        if a is None:
            return None
        a = a.detach().cpu().numpy() if isinstance(a, torch.Tensor) else np.asarray(a)
        return np.ascontiguousarray(a.astype(self.np_dtype, copy=False))

    def set_embeddings(self, word_table, type_table, position_table, ln_gamma, ln_beta,
                       layernorm_eps: float = 0.0) -> None:
        """Tables of embedding_lookup / embedding_postprocessor
        (sample/tensorflow/modeling.py:380-521).  type_table / position_table may be
        None (use_token_type / use_position_embeddings = False)."""
        w, t, p = self._host(word_table), self._host(type_table), self._host(position_table)
        g, b = self._host(ln_gamma), self._host(ln_beta)
        for name, a in (("word_table", w), ("type_table", t), ("position_table", p)):
            if a is not None and (a.ndim != 2 or a.shape[1] != self.hidden):
                raise ValueError(f"{name} must be [rows, {self.hidden}]")
        _capi.check(self._lib.et_set_embedding_weights(
            self._h, w.ctypes.data, w.shape[0], None if t is None else t.ctypes.data,
            0 if t is None else t.shape[0], None if p is None else p.ctypes.data,
            0 if p is None else p.shape[0], g.ctypes.data, b.ctypes.data, layernorm_eps, 1), self._h)

    def set_pooler(self, kernel, bias) -> None:
        """The pooler's dense layer (sample/tensorflow/modeling.py:229-232): kernel [H, H] as [in, out]."""
        k, b = self._host(kernel), self._host(bias)
        if k.shape != (self.hidden, self.hidden) or b.shape != (self.hidden,):
            raise ValueError("pooler kernel must be [H, H] and bias [H]")
        _capi.check(self._lib.et_set_pooler_weights(self._h, k.ctypes.data, b.ctypes.data, 1), self._h)

    @staticmethod
    def _i32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if t is None or (t.dtype == torch.int32 and t.is_contiguous()):
            return t
        return t.to(torch.int32).contiguous()

    def forward_ids(self, input_ids: torch.Tensor, input_mask: torch.Tensor,
                    token_type_ids: Optional[torch.Tensor] = None, sequence_output: bool = True,
                    pooled_output: bool = False) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        """BertModel (sample/tensorflow/modeling.py:107-235) from token ids on the
        current stream: (get_sequence_output() [B,S,H] or None, get_pooled_output()
        [B,H] or None).  Embedding rows are gathered for valid tokens only."""
        ids, mask, types = self._i32(input_ids), self._i32(input_mask), self._i32(token_type_ids)
        b, s = ids.shape
        seq = torch.empty((b, s, self.hidden), dtype=self.dtype, device=ids.device) if sequence_output else None
        pooled = torch.empty((b, self.hidden), dtype=self.dtype, device=ids.device) if pooled_output else None
        _capi.check(self._lib.et_forward_ids(self._h, _ptr(ids), _ptr(types), _ptr(mask), _ptr(seq),
                                             _ptr(pooled), b, s, _stream()), self._h)
        return seq, pooled

    def forward_ids_host(self, input_ids: np.ndarray, input_mask: np.ndarray,
                         token_type_ids: Optional[np.ndarray] = None, sequence_output: bool = True,
                         pooled_output: bool = False):
        """Same with host int32 arrays; returns (sequence or None, pooled or None, T)."""
        arrs = [input_ids, input_mask] + ([token_type_ids] if token_type_ids is not None else [])
        if any(a.dtype != np.int32 for a in arrs):
            raise ValueError("ids and masks must be int32")
        ids, mask = np.ascontiguousarray(input_ids), np.ascontiguousarray(input_mask)
        types = None if token_type_ids is None else np.ascontiguousarray(token_type_ids)
        b, s = ids.shape
        seq = np.empty((b, s, self.hidden), dtype=self.np_dtype) if sequence_output else None
        pooled = np.empty((b, self.hidden), dtype=self.np_dtype) if pooled_output else None
        t = C.c_int(0)
        _capi.check(self._lib.et_forward_ids_host(
            self._h, ids.ctypes.data, None if types is None else types.ctypes.data, mask.ctypes.data,
            None if seq is None else seq.ctypes.data, None if pooled is None else pooled.ctypes.data,
            b, s, C.byref(t)), self._h)
        return seq, pooled, int(t.value)

    def pooler(self, packed: torch.Tensor, batch_size: int, seq_len: int,
               cu_seqlens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """tanh(dense(first token of every sequence)) read from a packed [T,H] tensor
        (sample/tensorflow/modeling.py:224-232); cu_seqlens None = those of the last
        input op on this handle."""
        self._check_act(packed, "packed")
        out = torch.empty((batch_size, self.hidden), dtype=self.dtype, device=packed.device)
        _capi.check(self._lib.et_pooler(self._h, _ptr(packed), _ptr(self._i32(cu_seqlens)), _ptr(out),
                                        batch_size, seq_len, _stream()), self._h)
        return out

    # ---- CUDA-graph replay --------------------------------------------------
    def capture(self, from_tensor: torch.Tensor, input_mask: torch.Tensor, out: torch.Tensor) -> None:
        """Records forward(from_tensor, input_mask, out) as a CUDA graph.  The three
        tensors are the graph's fixed buffers: write each new batch (any mask) into
        them and call replay().  input_mask must be int32 and contiguous."""
        self._check_act(from_tensor, "from_tensor")
        self._check_act(out, "out")
        if input_mask.dtype != torch.int32 or not input_mask.is_contiguous():
            raise ValueError("input_mask must be a contiguous int32 tensor (it is a fixed graph buffer)")
        b, s, _ = from_tensor.shape
        self._graph_buffers = (from_tensor, input_mask, out)   # keep them alive
        _capi.check(self._lib.et_graph_capture(self._h, _ptr(from_tensor), _ptr(input_mask), _ptr(out), b, s),
                    self._h)

    def capture_ids(self, input_ids: torch.Tensor, input_mask: torch.Tensor,
                    token_type_ids: Optional[torch.Tensor], sequence_out: Optional[torch.Tensor],
                    pooled_out: Optional[torch.Tensor]) -> None:
        """Records forward_ids on fixed buffers (all int32 inputs contiguous)."""
        for t in (input_ids, input_mask, token_type_ids):
            if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
                raise ValueError("ids and masks must be contiguous int32 tensors (fixed graph buffers)")
        b, s = input_ids.shape
        self._graph_buffers = (input_ids, input_mask, token_type_ids, sequence_out, pooled_out)
        _capi.check(self._lib.et_graph_capture_ids(self._h, _ptr(input_ids), _ptr(token_type_ids),
                                                   _ptr(input_mask), _ptr(sequence_out), _ptr(pooled_out), b, s),
                    self._h)

    def replay(self) -> None:
        """Enqueues the captured pass on the current stream."""
        _capi.check(self._lib.et_graph_launch(self._h, _stream()), self._h)

    def release_graph(self) -> None:
        _capi.check(self._lib.et_graph_release(self._h), self._h)
        self._graph_buffers = None

    def set_profiling(self, on: bool) -> None:
        _capi.check(self._lib.et_set_profiling(self._h, 1 if on else 0), self._h)

    def get_profile(self, reset: bool = True):
        """{category: (device ms, kernels launched)} since the last reset; the
        times are non-zero only while profiling is enabled."""
        n = len(_capi.PROF_NAMES)
        ms = (C.c_double * n)()
        cnt = (C.c_longlong * n)()
        _capi.check(self._lib.et_get_profile(self._h, ms, cnt, 1 if reset else 0), self._h)
        return {name: (float(ms[i]), int(cnt[i])) for i, name in enumerate(_capi.PROF_NAMES)}

    def device_status(self) -> int:
        st = C.c_int(0)
        _capi.check(self._lib.et_device_status(self._h, _stream(), C.byref(st)), self._h)
        return int(st.value)

    def last_padding_info(self, batch: int, tokens: int, seq: int):
        """cu_seqlens, seq_len, padding_offset, prefix_sum of the last input op
        as CPU int32 arrays."""
        ptrs = [C.c_void_p() for _ in range(4)]
        _capi.check(self._lib.et_last_padding_info(self._h, *[C.byref(p) for p in ptrs]), self._h)
        sizes = [batch + 1, batch, tokens, batch * seq]
        outs = []
        for p, n in zip(ptrs, sizes):
            host = np.empty(n, dtype=np.int32)
            _capi.check(self._lib.et_copy_to_host(host.ctypes.data, p.value, n * 4, _stream()), self._h)
            outs.append(host)
        return outs


def get_sequence_output(config, max_batch_size: int, max_seq_length: int, attention_mask,
                        input_mask: torch.Tensor, from_tensor: torch.Tensor, weights_value: Sequence,
                        engine: Optional[EffectiveTransformer] = None) -> torch.Tensor:
    """Same wiring as python/effective_transformer/__init__.py:32-84: the input
    op, one layer op per hidden layer (weights taken 16 at a time from
    `weights_value`), the output op.  `attention_mask` is accepted for
    signature compatibility; it must be the key-only tile of `input_mask`."""
    head_num = config.num_attention_heads
    size_per_head = int(config.hidden_size / config.num_attention_heads)
    num_layers = config.num_hidden_layers
    ffn = getattr(config, "intermediate_size", 4 * config.hidden_size)
    own = engine is None
    if own:
        engine = EffectiveTransformer(num_layers, head_num, size_per_head, ffn, max_batch_size,
                                      max_seq_length, dtype=from_tensor.dtype,
                                      device=from_tensor.device.index or 0)
        engine.set_weights(weights_value)
    try:
        # 1. rm padding
        x, valid_word_num, batch_idx, word_idx = engine.effective_transformer_input(from_tensor, input_mask)
        # 2. transformer loop
        for layer_idx in range(num_layers):
            x = engine.effective_transformer(layer_idx, x, x, attention_mask, valid_word_num, batch_idx,
                                             word_idx)
        # 3. pad back
        out = engine.effective_transformer_output(x, valid_word_num, batch_idx, word_idx)
        torch.cuda.current_stream().synchronize()
        return out
    finally:
        if own:
            engine.close()
