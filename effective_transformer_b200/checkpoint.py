"""Weights by name -> the positional lists the encoder path takes.

The reference never looks weights up by name: its shim slices
``weights_value`` 16 arrays at a time in TensorFlow's variable-creation order
(python/effective_transformer/__init__.py:55-74), and the sample model restores
variables from a checkpoint by their scope names
(sample/tensorflow/modeling.py:317-341, scopes at :171-232 and :828-877).  A
user who switches to this library has either such named arrays (exported from
a TF checkpoint to .npz, TensorFlow itself is not needed here) or a Hugging
Face ``BertModel`` state dict.  Both are mapped to

* ``weights_value``: 16 arrays per layer, kernels as [in, out], for
  ``EffectiveTransformer.set_weights``;
* ``ModelHeads``-like tables for ``set_embeddings`` / ``set_pooler``.

Pure numpy; nothing here touches the GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Tuple

import numpy as np

# Suffixes below "<encoder scope>/layer_<l>/" in the 16-per-layer order of
# python/effective_transformer/__init__.py:55-74.
TF_LAYER_SUFFIXES = (
    "attention/self/query/kernel", "attention/self/query/bias",
    "attention/self/key/kernel", "attention/self/key/bias",
    "attention/self/value/kernel", "attention/self/value/bias",
    "attention/output/dense/kernel", "attention/output/dense/bias",
    "attention/output/LayerNorm/beta", "attention/output/LayerNorm/gamma",
    "intermediate/dense/kernel", "intermediate/dense/bias",
    "output/dense/kernel", "output/dense/bias",
    "output/LayerNorm/beta", "output/LayerNorm/gamma",
)

# The same 16 slots in a Hugging Face BertModel state dict, below
# "encoder.layer.<l>."; True = a torch Linear weight [out, in] that must be
# transposed to the [in, out] kernel layout.
HF_LAYER_KEYS = (
    ("attention.self.query.weight", True), ("attention.self.query.bias", False),
    ("attention.self.key.weight", True), ("attention.self.key.bias", False),
    ("attention.self.value.weight", True), ("attention.self.value.bias", False),
    ("attention.output.dense.weight", True), ("attention.output.dense.bias", False),
    ("attention.output.LayerNorm.bias", False), ("attention.output.LayerNorm.weight", False),
    ("intermediate.dense.weight", True), ("intermediate.dense.bias", False),
    ("output.dense.weight", True), ("output.dense.bias", False),
    ("output.LayerNorm.bias", False), ("output.LayerNorm.weight", False),
)


@dataclass
class ModelTables:
    """Embedding tables, their LayerNorm and the pooler's dense layer; any
    group that the source does not hold is None."""
    word_table: Optional[np.ndarray] = None
    type_table: Optional[np.ndarray] = None
    position_table: Optional[np.ndarray] = None
    ln_gamma: Optional[np.ndarray] = None
    ln_beta: Optional[np.ndarray] = None
    pooler_kernel: Optional[np.ndarray] = None   # [in, out]
    pooler_bias: Optional[np.ndarray] = None


def tf_variable_names(num_layers: int, encoder_scope: str = "bert/encoder") -> List[str]:
    """Names of the 16 * num_layers encoder variables in positional order."""
    return [f"{encoder_scope}/layer_{l}/{s}" for l in range(num_layers) for s in TF_LAYER_SUFFIXES]


def _np(a) -> np.ndarray:
    if hasattr(a, "detach"):
        a = a.detach().cpu().numpy()
    return np.ascontiguousarray(np.asarray(a))


def _strip(name: str) -> str:
    return name[:-2] if name.endswith(":0") else name


def _check_layer(w: List[np.ndarray], layer: int) -> None:
    h = w[0].shape[0]
    f = w[10].shape[1]
    want = [(h, h), (h,), (h, h), (h,), (h, h), (h,), (h, h), (h,), (h,), (h,), (h, f), (f,), (f, h), (h,), (h,), (h,)]
    for i, (a, shp) in enumerate(zip(w, want)):
        if tuple(a.shape) != shp:
            raise ValueError(f"layer {layer}, slot {i} ({TF_LAYER_SUFFIXES[i]}): shape {tuple(a.shape)}, expected {shp}")


def weights_from_tf_variables(named: Mapping[str, object], num_layers: Optional[int] = None,
                              scope: str = "bert") -> Tuple[List[np.ndarray], ModelTables]:
    """``named`` maps TF variable names (with or without the ``:0`` suffix) to
    arrays, e.g. ``dict(np.load("bert.npz"))``.  Returns (weights_value, tables).
    ``num_layers`` None = as many ``layer_<l>`` scopes as are present."""
    v: Dict[str, np.ndarray] = {_strip(k): _np(a) for k, a in named.items()}
    enc = f"{scope}/encoder" if scope else "encoder"
    if num_layers is None:
        num_layers = 0
        while f"{enc}/layer_{num_layers}/{TF_LAYER_SUFFIXES[0]}" in v:
            num_layers += 1
        if num_layers == 0:
            raise KeyError(f"no variable named {enc}/layer_0/{TF_LAYER_SUFFIXES[0]}")
    weights: List[np.ndarray] = []
    for l in range(num_layers):
        layer = []
        for s in TF_LAYER_SUFFIXES:
            name = f"{enc}/layer_{l}/{s}"
            if name not in v:
                raise KeyError(f"missing variable {name}")
            layer.append(v[name])
        _check_layer(layer, l)
        weights.extend(layer)
    emb = f"{scope}/embeddings" if scope else "embeddings"
    pool = f"{scope}/pooler" if scope else "pooler"
    g = v.get
    tables = ModelTables(g(f"{emb}/word_embeddings"), g(f"{emb}/token_type_embeddings"),
                         g(f"{emb}/position_embeddings"), g(f"{emb}/LayerNorm/gamma"), g(f"{emb}/LayerNorm/beta"),
                         g(f"{pool}/dense/kernel"), g(f"{pool}/dense/bias"))
    return weights, tables


def weights_from_hf_state_dict(state_dict: Mapping[str, object], num_layers: Optional[int] = None,
                               prefix: str = "") -> Tuple[List[np.ndarray], ModelTables]:
    """From a Hugging Face ``BertModel.state_dict()`` (``prefix`` "bert." for a
    model with a head).  Linear weights are transposed to [in, out]."""
    sd = state_dict
    if num_layers is None:
        num_layers = 0
        while f"{prefix}encoder.layer.{num_layers}.{HF_LAYER_KEYS[0][0]}" in sd:
            num_layers += 1
        if num_layers == 0:
            raise KeyError(f"no key {prefix}encoder.layer.0.{HF_LAYER_KEYS[0][0]}")
    weights: List[np.ndarray] = []
    for l in range(num_layers):
        layer = []
        for key, transpose in HF_LAYER_KEYS:
            name = f"{prefix}encoder.layer.{l}.{key}"
            if name not in sd:
                raise KeyError(f"missing key {name}")
            a = _np(sd[name])
            layer.append(np.ascontiguousarray(a.T) if transpose else a)
        _check_layer(layer, l)
        weights.extend(layer)

    def g(key, transpose=False):
        name = prefix + key
        if name not in sd:
            return None
        a = _np(sd[name])
        return np.ascontiguousarray(a.T) if transpose else a

    tables = ModelTables(g("embeddings.word_embeddings.weight"), g("embeddings.token_type_embeddings.weight"),
                         g("embeddings.position_embeddings.weight"), g("embeddings.LayerNorm.weight"),
                         g("embeddings.LayerNorm.bias"), g("pooler.dense.weight", True), g("pooler.dense.bias"))
    return weights, tables


def to_tf_variables(weights_value, tables: Optional[ModelTables] = None, scope: str = "bert") -> Dict[str, np.ndarray]:
    """The inverse of weights_from_tf_variables (for exporting / round trips)."""
    if len(weights_value) % 16:
        raise ValueError("weights_value must hold 16 arrays per layer")
    names = tf_variable_names(len(weights_value) // 16, f"{scope}/encoder" if scope else "encoder")
    out = {n: _np(a) for n, a in zip(names, weights_value)}
    if tables is not None:
        emb = f"{scope}/embeddings" if scope else "embeddings"
        pool = f"{scope}/pooler" if scope else "pooler"
        for name, a in ((f"{emb}/word_embeddings", tables.word_table),
                        (f"{emb}/token_type_embeddings", tables.type_table),
                        (f"{emb}/position_embeddings", tables.position_table),
                        (f"{emb}/LayerNorm/gamma", tables.ln_gamma), (f"{emb}/LayerNorm/beta", tables.ln_beta),
                        (f"{pool}/dense/kernel", tables.pooler_kernel), (f"{pool}/dense/bias", tables.pooler_bias)):
            if a is not None:
                out[name] = _np(a)
    return out


def load_engine_weights(engine, weights_value, tables: Optional[ModelTables] = None) -> None:
    """Registers everything that is present with an EffectiveTransformer."""
    engine.set_weights(weights_value)
    if tables is None:
        return
    if tables.word_table is not None:
        engine.set_embeddings(tables.word_table, tables.type_table, tables.position_table, tables.ln_gamma,
                              tables.ln_beta)
    if tables.pooler_kernel is not None:
        engine.set_pooler(tables.pooler_kernel, tables.pooler_bias)
