"""Helpers shared by the GPU parity tests: torch tensors for device memory,
calls through the C ABI (effective_transformer_b200._capi)."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from effective_transformer_b200 import _capi

DT = {torch.float16: _capi.ET_FP16, torch.float32: _capi.ET_FP32}


def lib():
    return _capi.load()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def dev(a, dtype=None) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda().contiguous()


def iptr(t):
    return None if t is None else t.data_ptr()


def ok(code: int) -> None:
    assert code == _capi.ET_OK, f"C ABI call failed: {_capi.STATUS_NAMES.get(code, code)}"


def padding_offsets(mask: torch.Tensor):
    """Runs et_padding_offsets on an int32 [B,S] CUDA mask and returns all outputs."""
    b, s = mask.shape
    n = max(b * s, 1)
    i32 = dict(dtype=torch.int32, device="cuda")
    out = {
        "prefix_sum": torch.full((n,), -7, **i32), "valid_word_num": torch.full((1,), -7, **i32),
        "batch_idx": torch.full((n,), -7, **i32), "word_idx": torch.full((n,), -7, **i32),
        "seq_len": torch.full((max(b, 1),), -7, **i32), "cu_seqlens": torch.full((b + 1,), -7, **i32),
        "padding_offset": torch.full((n,), -7, **i32),
    }
    scratch = torch.zeros(max(b, 1), **i32)
    ok(lib().et_padding_offsets(iptr(mask), b, s, iptr(out["prefix_sum"]), iptr(out["valid_word_num"]),
                                iptr(out["batch_idx"]), iptr(out["word_idx"]), iptr(out["seq_len"]),
                                iptr(out["cu_seqlens"]), iptr(out["padding_offset"]), iptr(scratch), stream()))
    torch.cuda.synchronize()
    return out


def status_word() -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device="cuda")
