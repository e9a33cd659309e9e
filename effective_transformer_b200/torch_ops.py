"""The three operators as PyTorch custom ops.

The reference registers its operators with TensorFlow
(``EffectiveTransformerInput`` tf_op/bert_transformer_op.cc:249-274,
``EffectiveTransformer`` :44-77, ``EffectiveTransformerOutput`` :359-380, each
with a shape function) and loads them with ``tf.load_op_library``
(python/effective_transformer/__init__.py:24-30).  TensorFlow is not available
to this repository, PyTorch is: this module registers the same three operators,
with the same inputs, outputs and shape rules, in the dispatcher namespace
``effective_transformer_b200``.  They can be called eagerly, traced
(``torch.compile`` / ``torch.export`` see them as opaque ops with known output
shapes) and checked with ``torch.library.opcheck``.

Where the TF layer op takes its 16 weight tensors as op inputs, the PyTorch op
takes the id of an ``EffectiveTransformer`` engine (weights registered once with
``set_weights``) and a layer index: ``engine_id = register_engine(engine)``.

    import effective_transformer_b200.torch_ops as ops
    eid = ops.register_engine(engine)
    x, valid, bidx, widx = torch.ops.effective_transformer_b200.effective_transformer_input(eid, from_tensor, mask)
    for l in range(num_layers):
        x = torch.ops.effective_transformer_b200.effective_transformer(eid, l, x, x, None, valid, bidx, widx)
    out = torch.ops.effective_transformer_b200.effective_transformer_output(eid, x, valid, bidx, widx)
"""
from __future__ import annotations

import itertools
import weakref
from typing import Dict, List, Optional, Tuple

import torch
from torch import Tensor

_ENGINES: Dict[int, "weakref.ReferenceType"] = {}
_IDS = itertools.count(1)


def register_engine(engine) -> int:
    """Makes an EffectiveTransformer addressable from the ops; returns its id.
    Only a weak reference is kept: the caller owns the engine."""
    eid = next(_IDS)
    _ENGINES[eid] = weakref.ref(engine)
    return eid


def unregister_engine(engine_id: int) -> None:
    _ENGINES.pop(engine_id, None)


def _engine(engine_id: int):
    ref = _ENGINES.get(engine_id)
    eng = ref() if ref is not None else None
    if eng is None:
        raise RuntimeError(f"no live engine registered under id {engine_id}")
    return eng


def _check_bsh(t: Tensor, name: str) -> Tuple[int, int, int]:
    if t.dim() != 3:
        raise ValueError(f"{name} must be [batch, seq, hidden]")   # rank check of the TF shape functions
    return t.shape[0], t.shape[1], t.shape[2]


@torch.library.custom_op("effective_transformer_b200::effective_transformer_input", mutates_args=())
def effective_transformer_input(engine_id: int, from_tensor: Tensor, mask: Tensor) -> List[Tensor]:
    """(from_tensor [B,S,H], mask int32 [B,S]) -> [to_tensor [B,S,H] (first T rows packed),
    valid_word_num [1], batch_idx [B,S], word_idx [B,S]]."""
    return list(_engine(engine_id).effective_transformer_input(from_tensor, mask))


@effective_transformer_input.register_fake
def _(engine_id: int, from_tensor: Tensor, mask: Tensor) -> List[Tensor]:
    b, s, _h = _check_bsh(from_tensor, "from_tensor")
    if mask.dim() != 2 or mask.shape[0] != b or mask.shape[1] != s:
        raise ValueError("mask must be [batch, seq]")
    i32 = dict(dtype=torch.int32, device=from_tensor.device)
    return [torch.empty_like(from_tensor), torch.empty((1,), **i32), torch.empty((b, s), **i32),
            torch.empty((b, s), **i32)]


@torch.library.custom_op("effective_transformer_b200::effective_transformer", mutates_args=())
def effective_transformer(engine_id: int, layer_idx: int, from_tensor: Tensor, to_tensor: Tensor,
                          attention_mask: Optional[Tensor], valid_word_num: Tensor, batch_idx: Tensor,
                          word_idx: Tensor) -> Tensor:
    """One encoder layer on the packed layout; output shaped like from_tensor."""
    eng = _engine(engine_id)
    if to_tensor.data_ptr() != from_tensor.data_ptr():
        # the dispatcher may hand over two views of one buffer: compare storage, not identity
        raise ValueError("to_tensor must be from_tensor (self-attention)")
    return eng.effective_transformer(layer_idx, from_tensor, from_tensor, attention_mask, valid_word_num,
                                     batch_idx, word_idx)


@effective_transformer.register_fake
def _(engine_id: int, layer_idx: int, from_tensor: Tensor, to_tensor: Tensor, attention_mask: Optional[Tensor],
      valid_word_num: Tensor, batch_idx: Tensor, word_idx: Tensor) -> Tensor:
    b, s, _h = _check_bsh(from_tensor, "from_tensor")
    if tuple(to_tensor.shape) != tuple(from_tensor.shape):
        raise ValueError("only support from_seq_len == to_seq_len")   # tf_op/bert_transformer_op.cc:130-131
    if attention_mask is not None and tuple(attention_mask.shape) != (b, s, s):
        raise ValueError("attention_mask must be [batch, seq, seq]")
    return torch.empty_like(from_tensor)


@torch.library.custom_op("effective_transformer_b200::effective_transformer_output", mutates_args=())
def effective_transformer_output(engine_id: int, from_tensor: Tensor, valid_word_num: Tensor, batch_idx: Tensor,
                                 word_idx: Tensor) -> Tensor:
    """Packed [T,H] inside a [B,S,H] tensor -> padded [B,S,H] with zero padding rows."""
    return _engine(engine_id).effective_transformer_output(from_tensor, valid_word_num, batch_idx, word_idx)


@effective_transformer_output.register_fake
def _(engine_id: int, from_tensor: Tensor, valid_word_num: Tensor, batch_idx: Tensor, word_idx: Tensor) -> Tensor:
    _check_bsh(from_tensor, "from_tensor")
    return torch.empty_like(from_tensor)


def get_sequence_output(engine_id: int, num_layers: int, attention_mask: Optional[Tensor], input_mask: Tensor,
                        from_tensor: Tensor) -> Tensor:
    """The wiring of python/effective_transformer/__init__.py:42-82 on the registered ops."""
    ns = torch.ops.effective_transformer_b200
    x, valid, bidx, widx = ns.effective_transformer_input(engine_id, from_tensor, input_mask)
    for layer_idx in range(num_layers):
        x = ns.effective_transformer(engine_id, layer_idx, x, x, attention_mask, valid, bidx, widx)
    return ns.effective_transformer_output(engine_id, x, valid, bidx, widx)
