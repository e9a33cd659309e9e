"""GPU test of et_padding_offsets_noalloc, the padding-offset entry point for
callers that cannot allocate device memory (a framework op that must not
re-enter its allocator, code running while a memory pool is frozen, a C plug-in
without a device allocator).  Its scratch is a fixed device array inside the
library instead of a caller buffer, so all it may differ in from
et_padding_offsets is where the per-row token counts are kept: every output
must be identical, bit for bit, on consecutive calls that reuse the array, and
equal to the CPU oracle of the padding bookkeeping (oracle/padding.py).  The
property the entry point is named for is checked too: the device's free memory
does not move across a call (after the first one, which resolves the array's
address).

The file name makes pytest collect it last, so a run that stops at the first
failure has already run every other test.  It also passes when run alone.
"""
import numpy as np
import pytest
import torch

from effective_transformer_b200 import _capi
from effective_transformer_b200 import workloads as W
from oracle import padding as P

from util import dev, iptr, lib, ok, padding_offsets, stream

pytestmark = pytest.mark.gpu

OUTPUTS = ("prefix_sum", "valid_word_num", "batch_idx", "word_idx", "seq_len", "cu_seqlens", "padding_offset")


def padding_offsets_noalloc(mask: torch.Tensor):
    """Same buffers and fill pattern as util.padding_offsets, but no scratch argument."""
    b, s = mask.shape
    n = max(b * s, 1)
    i32 = dict(dtype=torch.int32, device="cuda")
    out = {
        "prefix_sum": torch.full((n,), -7, **i32), "valid_word_num": torch.full((1,), -7, **i32),
        "batch_idx": torch.full((n,), -7, **i32), "word_idx": torch.full((n,), -7, **i32),
        "seq_len": torch.full((max(b, 1),), -7, **i32), "cu_seqlens": torch.full((b + 1,), -7, **i32),
        "padding_offset": torch.full((n,), -7, **i32),
    }
    ok(lib().et_padding_offsets_noalloc(iptr(mask), b, s, iptr(out["prefix_sum"]), iptr(out["valid_word_num"]),
                                        iptr(out["batch_idx"]), iptr(out["word_idx"]), iptr(out["seq_len"]),
                                        iptr(out["cu_seqlens"]), iptr(out["padding_offset"]), stream()))
    torch.cuda.synchronize()
    return out


def assert_equals_oracle(out, mask_np):
    """All integer outputs against oracle/padding.py, bit for bit."""
    b, s = mask_np.shape
    ref = P.padding_indices(mask_np)
    t = int(ref["valid_word_num"][0])
    assert int(out["valid_word_num"][0]) == t
    assert np.array_equal(out["cu_seqlens"].cpu().numpy(), ref["cu_seqlens"])
    if b * s == 0:
        return
    assert np.array_equal(out["prefix_sum"].cpu().numpy()[:b * s], ref["prefix_sum"].ravel())
    assert np.array_equal(out["seq_len"].cpu().numpy()[:b], ref["seq_len"])
    for k in ("batch_idx", "word_idx", "padding_offset"):
        got = out[k].cpu().numpy()
        assert np.array_equal(got[:t], ref[k]), k
        assert np.all(got[t:] == -7), k + ": wrote past the valid count"


def test_noalloc_matches_caller_scratch_entry_point_on_consecutive_calls():
    rng = np.random.RandomState(123)
    spec = W.WORKLOADS[2]
    masks = [
        W.prefix_mask(W.draw_lengths(spec, np.random.RandomState(spec.seed)), spec.max_seq_len),  # B=1000, S=64
        (rng.rand(37, 50) < 0.4).astype(np.int32),    # smaller batch right after: stale counts beyond row 37 stay unused
        (rng.rand(1000, 33) < 0.7).astype(np.int32),  # back to a large batch over the same array
        np.zeros((5, 9), np.int32),                   # nothing valid
    ]
    for m in masks:
        md = dev(m)
        want = padding_offsets(md)            # existing entry point, caller-provided scratch
        got = padding_offsets_noalloc(md)     # new entry point, scratch inside the library
        for k in OUTPUTS:
            assert torch.equal(got[k], want[k]), k
        assert_equals_oracle(got, m)


def test_noalloc_call_leaves_free_device_memory_unchanged():
    """After the first call on a device (which looks the array's address up) a call allocates
    nothing: free device memory as the driver reports it is the same before and after, and the
    torch allocator (the only other allocator in this process) is not asked either."""
    mask = dev((np.random.RandomState(7).rand(512, 48) < 0.6).astype(np.int32))
    b, s = mask.shape
    i32 = dict(dtype=torch.int32, device="cuda")
    bufs = [torch.zeros(b * s, **i32) for _ in range(4)] + [torch.zeros(1, **i32), torch.zeros(b, **i32),
                                                            torch.zeros(b + 1, **i32)]
    prefix, bidx, widx, poff, valid, slen, cu = bufs

    def call():
        ok(lib().et_padding_offsets_noalloc(iptr(mask), b, s, iptr(prefix), iptr(valid), iptr(bidx), iptr(widx),
                                            iptr(slen), iptr(cu), iptr(poff), stream()))
        torch.cuda.synchronize()

    call()                                   # first call on this device: set-up
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    for _ in range(3):
        call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert torch.cuda.memory_reserved() == reserved_before
    assert int(valid[0]) == int(mask.sum())


def test_noalloc_rejects_batches_beyond_the_fixed_scratch():
    assert _capi.NOALLOC_MAX_BATCH == 16384
    b = _capi.NOALLOC_MAX_BATCH + 1
    mask = torch.ones((b, 1), dtype=torch.int32, device="cuda")
    one = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib().et_padding_offsets_noalloc(iptr(mask), b, 1, None, iptr(one), None, None, None, None, None, stream())
    assert rc == _capi.ET_INVALID_ARGUMENT
    assert b"ET_NOALLOC_MAX_BATCH" in lib().et_last_error(None)
    # the largest accepted batch still works and agrees with the caller-scratch entry point
    mask = (torch.rand(_capi.NOALLOC_MAX_BATCH, 3, device="cuda") < 0.5).to(torch.int32)
    want, got = padding_offsets(mask), padding_offsets_noalloc(mask)
    for k in OUTPUTS:
        assert torch.equal(got[k], want[k]), k
