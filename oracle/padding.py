"""TEST INFRASTRUCTURE - CPU oracle for the padding bookkeeping of the encoder
path.  Only tests, the smoke check and the benchmark's CPU-baseline leg may
import this module; the product path never does.

Parity status: the reference ships no tests, fixtures or golden vectors, so
this oracle is pinned against outputs of the reference itself: its scan,
compress and restore kernels, compiled unmodified from the reference checkout
(oracle/build_ref.py) and run on the GPU box, agree bit for bit with the
functions below (tests/test_reference_kernels_gpu.py).  Each function restates
the integer arithmetic of the reference kernels it cites, in numpy, for
arbitrary 0/1 masks.
"""
from __future__ import annotations

from typing import Dict

import numpy as np


def exclusive_scan(mask_flat: np.ndarray) -> np.ndarray:
    """Exclusive prefix sum of the flattened int mask.
    Restates exclusiveScan_kernelLauncher (cuda/cuda_kernels.cu:477-718): the
    Blelloch up/down sweep there computes exactly ``cumsum(x) - x`` in int32."""
    m = np.asarray(mask_flat, dtype=np.int64).ravel()
    return (np.cumsum(m) - m).astype(np.int32)


def valid_word_num(mask_flat: np.ndarray) -> int:
    """prefix[last] + (mask[last] == 1)
    (tf_op/bert_transformer_op.cu.cc:303-316)."""
    m = np.asarray(mask_flat).ravel()
    if m.size == 0:
        return 0
    pre = exclusive_scan(m)
    return int(pre[-1]) + (1 if int(m[-1]) == 1 else 0)


def padding_indices(mask: np.ndarray) -> Dict[str, np.ndarray]:
    """All integer outputs of the input op for a [B, S] 0/1 mask.

    batch_idx / word_idx follow compress_bert_input
    (cuda/cuda_kernels.cu:278-307): for every position with mask > 0.5 the
    packed row ``prefix[b, s]`` records (b, s).  Entries past the valid count
    are unspecified in the reference (never written); this oracle returns only
    the first T entries.  cu_seqlens[b] = prefix[b*S] and
    padding_offset[v] = batch_idx[v]*S + word_idx[v] - v are derived values.
    """
    mask = np.asarray(mask, dtype=np.int32)
    b, s = mask.shape
    flat = mask.ravel()
    prefix = exclusive_scan(flat)
    valid = flat > 0
    pos = np.nonzero(valid)[0].astype(np.int64)
    t = int(pos.size)
    batch_idx = (pos // s).astype(np.int32) if s else np.zeros(0, np.int32)
    word_idx = (pos % s).astype(np.int32) if s else np.zeros(0, np.int32)
    seq_len = mask.astype(np.int64).sum(axis=1).astype(np.int32)
    cu = np.zeros(b + 1, dtype=np.int32)
    cu[1:] = np.cumsum(seq_len)
    padding_offset = (pos - np.arange(t, dtype=np.int64)).astype(np.int32)
    return {
        "prefix_sum": prefix.reshape(b, s),
        "valid_word_num": np.array([valid_word_num(flat)], dtype=np.int32),
        "batch_idx": batch_idx,
        "word_idx": word_idx,
        "seq_len": seq_len,
        "cu_seqlens": cu,
        "padding_offset": padding_offset,
    }


def remove_padding(x: np.ndarray, mask: np.ndarray) -> np.ndarray:
    """[B, S, H] -> packed [T, H]; a bit-exact copy of the valid rows in
    (b, s) order (cuda/cuda_kernels.cu:300-306)."""
    b, s = mask.shape
    h = x.shape[-1]
    return np.ascontiguousarray(x.reshape(b * s, h)[np.asarray(mask).ravel() > 0])


def restore_padding(packed: np.ndarray, batch_idx: np.ndarray, word_idx: np.ndarray,
                    batch: int, seq_len: int) -> np.ndarray:
    """Zero [B, S, H] then scatter the packed rows back
    (tf_op/bert_transformer_op.cu.cc:354-360, cuda/cuda_kernels.cu:389-407)."""
    h = packed.shape[1]
    out = np.zeros((batch * seq_len, h), dtype=packed.dtype)
    t = batch_idx.shape[0]
    out[batch_idx.astype(np.int64) * seq_len + word_idx.astype(np.int64)] = packed[:t]
    return out.reshape(batch, seq_len, h)
