"""GPU parity tests, kernel by kernel, through the C ABI: every CUDA kernel is
compared with the CPU oracle on the same seeded inputs.  Integer and copy
kernels must be bit-exact; floating-point kernels are compared against the
oracle evaluated in float64 on the fp16/fp32-rounded inputs."""
import math

import numpy as np
import pytest
import torch

from effective_transformer_b200 import _capi
from effective_transformer_b200 import workloads as W
from oracle import bert_encoder as O
from oracle import padding as P

from util import DT, dev, iptr, lib, ok, padding_offsets, status_word, stream

pytestmark = pytest.mark.gpu


def _check_padding(mask_np):
    b, s = mask_np.shape
    out = padding_offsets(dev(mask_np.astype(np.int32)))
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


@pytest.mark.parametrize("b,s", [(1, 1), (3, 7), (8, 32), (5, 33), (100, 32), (17, 129), (1000, 64), (4096, 128)])
def test_padding_offsets_prefix_masks(b, s):
    rng = np.random.RandomState(b * 1000 + s)
    lens = rng.randint(0, s + 1, size=b)
    _check_padding(W.prefix_mask(lens.astype(np.int32), s))


@pytest.mark.parametrize("b,s,p", [(4, 16, 0.5), (64, 37, 0.3), (9, 1024, 0.9), (300, 65, 0.05)])
def test_padding_offsets_arbitrary_masks(b, s, p):
    rng = np.random.RandomState(7)
    _check_padding((rng.rand(b, s) < p).astype(np.int32))


def test_padding_offsets_edge_cases():
    _check_padding(np.zeros((6, 10), np.int32))            # nothing valid
    _check_padding(np.ones((6, 10), np.int32))             # nothing padded, last mask = 1
    m = np.zeros((4, 8), np.int32); m[3, 7] = 1            # only the very last position
    _check_padding(m)
    m = np.ones((4, 8), np.int32); m[3, 7] = 0             # last mask = 0
    _check_padding(m)
    _check_padding(np.zeros((0, 8), np.int32))             # empty batch
    cfg4 = W.WORKLOADS[4]
    lens = W.draw_lengths(cfg4, np.random.RandomState(cfg4.seed))
    _check_padding(W.prefix_mask(lens, cfg4.max_seq_len))  # 524 288 positions, skewed lengths


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("b,s,h", [(5, 12, 128), (8, 32, 768), (64, 64, 1024), (3, 5, 64)])
def test_remove_restore_padding_bit_exact(dtype, b, s, h):
    rng = np.random.RandomState(b + s + h)
    mask_np = (rng.rand(b, s) < 0.6).astype(np.int32)
    mask_np[0, :] = 0                                       # an empty sequence
    x = dev(rng.randn(b, s, h).astype(np.float32), dtype)
    idx = padding_offsets(dev(mask_np))
    t = int(idx["valid_word_num"][0])
    packed = torch.full((b, s, h), 77.0, dtype=dtype, device="cuda")
    ok(lib().et_remove_padding(DT[dtype], iptr(x), iptr(idx["batch_idx"]), iptr(idx["word_idx"]),
                               iptr(idx["valid_word_num"]), iptr(packed), b, s, h, stream()))
    torch.cuda.synchronize()
    ref = P.remove_padding(x.cpu().numpy(), mask_np)
    got = packed.cpu().numpy().reshape(b * s, h)
    assert np.array_equal(got[:t], ref)
    assert np.all(got[t:] == 77.0)                          # rows past T untouched
    restored = torch.full((b, s, h), 55.0, dtype=dtype, device="cuda")
    ok(lib().et_restore_padding(DT[dtype], iptr(packed), iptr(idx["batch_idx"]), iptr(idx["word_idx"]),
                                iptr(idx["valid_word_num"]), iptr(restored), b, s, h, stream()))
    torch.cuda.synchronize()
    ref_back = P.restore_padding(ref, idx["batch_idx"].cpu().numpy()[:t], idx["word_idx"].cpu().numpy()[:t], b, s)
    assert np.array_equal(restored.cpu().numpy(), ref_back)  # padded rows are exactly zero


def test_restore_padding_all_padding_and_no_padding():
    for fill in (0, 1):
        b, s, h = 4, 9, 64
        mask_np = np.full((b, s), fill, np.int32)
        x = dev(np.random.RandomState(1).randn(b, s, h).astype(np.float32), torch.float16)
        idx = padding_offsets(dev(mask_np))
        packed = torch.zeros_like(x)
        ok(lib().et_remove_padding(_capi.ET_FP16, iptr(x), iptr(idx["batch_idx"]), iptr(idx["word_idx"]),
                                   iptr(idx["valid_word_num"]), iptr(packed), b, s, h, stream()))
        out = torch.full_like(x, 9.0)
        ok(lib().et_restore_padding(_capi.ET_FP16, iptr(packed), iptr(idx["batch_idx"]), iptr(idx["word_idx"]),
                                    iptr(idx["valid_word_num"]), iptr(out), b, s, h, stream()))
        torch.cuda.synchronize()
        assert torch.equal(out, x * fill)


def _tol(dtype):
    # one rounding of an O(1..10) value in the output type
    return dict(rtol=2e-3, atol=2e-3) if dtype == torch.float16 else dict(rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("t,cap,heads", [(37, 64, 2), (1954, 3200, 12), (300, 300, 16)])
def test_add_qkv_bias_transpose(dtype, t, cap, heads):
    d, h = 64, heads * 64
    rng = np.random.RandomState(t)
    q, k, v = [dev(rng.randn(cap, h).astype(np.float32), dtype) for _ in range(3)]
    bq, bk, bv = [dev(rng.randn(h).astype(np.float32), dtype) for _ in range(3)]
    out = torch.full((3, heads, cap, d), 5.0, dtype=dtype, device="cuda")
    tn = dev(np.array([t], np.int32))
    ok(lib().et_add_qkv_bias_transpose(DT[dtype], iptr(q), iptr(bq), iptr(k), iptr(bk), iptr(v), iptr(bv),
                                       iptr(out), iptr(tn), cap, heads, d, stream()))
    torch.cuda.synchronize()
    for w, (x, bias) in enumerate(((q, bq), (k, bk), (v, bv))):
        ref = (x[:t].double() + bias.double()).reshape(t, heads, d).permute(1, 0, 2)
        torch.testing.assert_close(out[w, :, :t].double(), ref, **_tol(dtype))
    assert torch.all(out[:, :, t:] == 5.0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("t,cap,n", [(37, 64, 256), (1954, 3200, 3072), (129, 129, 4096)])
def test_add_bias_gelu(dtype, t, cap, n):
    rng = np.random.RandomState(n)
    x = dev((2.0 * rng.randn(cap, n)).astype(np.float32), dtype)
    bias = dev(rng.randn(n).astype(np.float32), dtype)
    ref = O.add_bias_gelu(x[:t].double(), bias.double())
    keep = x[t:].clone()
    tn = dev(np.array([t], np.int32))
    ok(lib().et_add_bias_gelu(DT[dtype], iptr(x), iptr(bias), iptr(tn), cap, n, stream()))
    torch.cuda.synchronize()
    torch.testing.assert_close(x[:t].double(), ref, **_tol(dtype))
    assert torch.equal(x[t:], keep)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("t,cap,n", [(37, 64, 128), (1954, 3200, 768), (200, 256, 1024), (50, 50, 2048)])
def test_add_bias_input_layernorm(dtype, t, cap, n):
    rng = np.random.RandomState(n + 1)
    if dtype == torch.float32 and n > 1024:
        # a row must fit one warp's registers: 8 x 16-byte vectors per lane
        z = torch.zeros(cap, n, device="cuda")
        tn = dev(np.array([t], np.int32))
        assert lib().et_add_bias_input_layernorm(DT[dtype], iptr(z), iptr(z), iptr(z), iptr(z), iptr(z),
                                                 iptr(tn), cap, n, 1e-6, stream()) == _capi.ET_INVALID_ARGUMENT
        return
    out = dev(rng.randn(cap, n).astype(np.float32), dtype)
    inp = dev(rng.randn(cap, n).astype(np.float32), dtype)
    bias, beta = [dev(0.5 * rng.randn(n).astype(np.float32), dtype) for _ in range(2)]
    gamma = dev((1 + 0.2 * rng.randn(n)).astype(np.float32), dtype)
    ref = O.add_bias_input_layernorm(out[:t].double(), inp[:t].double(), bias.double(), gamma.double(),
                                     beta.double(), eps=1e-6)
    keep = out[t:].clone()
    tn = dev(np.array([t], np.int32))
    ok(lib().et_add_bias_input_layernorm(DT[dtype], iptr(out), iptr(inp), iptr(bias), iptr(gamma), iptr(beta),
                                         iptr(tn), cap, n, 1e-6, stream()))
    torch.cuda.synchronize()
    torch.testing.assert_close(out[:t].double(), ref, **(dict(rtol=2e-3, atol=4e-3) if dtype == torch.float16
                                                       else dict(rtol=1e-5, atol=1e-5)))
    assert torch.equal(out[t:], keep)


def _gemm_case(dtype, m, cap, n, k, epi, use_simt, seed=0):
    rng = np.random.RandomState(seed + m + n + k)
    a = dev(rng.randn(cap, k).astype(np.float32), dtype)
    w = dev((rng.randn(k, n) / math.sqrt(k)).astype(np.float32), dtype)
    bias = dev(rng.randn(n).astype(np.float32), dtype)
    c = torch.full((cap, n), 3.0, dtype=dtype, device="cuda")
    wp = torch.empty((n, k), dtype=dtype, device="cuda")
    ok(lib().et_pack_weight(DT[dtype], iptr(w), iptr(wp), k, n, stream()))
    torch.cuda.synchronize()
    assert torch.equal(wp, w.t().contiguous())
    mt = dev(np.array([m], np.int32))
    st = status_word()
    ok(lib().et_gemm(DT[dtype], iptr(a), iptr(w), iptr(wp), iptr(bias) if epi else None, iptr(c), iptr(mt),
                     cap, n, k, epi, 1 if use_simt else 0, iptr(st), stream()))
    torch.cuda.synchronize()
    assert int(st[0]) == 0, f"device-side wait expired: status 0x{int(st[0]):x}"
    ref = a[:m].double() @ w.double()
    if epi >= 1:
        ref = ref + bias.double()
    if epi == 2:
        ref = O.gelu(ref)
    if dtype == torch.float16:
        torch.testing.assert_close(c[:m].double(), ref, rtol=2e-3, atol=3e-3)
    else:
        torch.testing.assert_close(c[:m].double(), ref, rtol=1e-5, atol=2e-5)
    assert torch.all(c[m:] == 3.0), "rows past M were written"


@pytest.mark.parametrize("m,cap,n,k", [(1, 1, 128, 64), (60, 60, 128, 128), (134, 256, 768, 768),
                                       (300, 384, 2304, 768), (257, 300, 768, 3072), (128, 128, 256, 64),
                                       (1000, 1000, 3072, 768), (0, 64, 256, 128)])
@pytest.mark.parametrize("epi", [0, 1, 2])
def test_gemm_tcgen05(m, cap, n, k, epi):
    _gemm_case(torch.float16, m, cap, n, k, epi, use_simt=False)


def test_gemm_tcgen05_many_tiles_per_cta():
    # more tiles than CTAs: exercises both TMEM accumulator buffers and ring wrap-around
    _gemm_case(torch.float16, 5000, 5000, 3072, 768, 2, use_simt=False)
    _gemm_case(torch.float16, 4111, 4200, 768, 3072, 0, use_simt=False)
    _gemm_case(torch.float16, 3000, 3000, 1152, 1024, 1, use_simt=False)   # N = 9 * 128: BN = 128 path


@pytest.mark.parametrize("epi", [0, 1, 2])
@pytest.mark.parametrize("m,n,k", [(6500, 768, 768),      # 78 tiles on 74 CTA pairs: 4 tiles left, cut in halves
                                   (9372, 768, 3072),     # 111 tiles: 37 left = exactly half of the pairs
                                   (9729, 768, 768),      # 117 tiles: 43 left, more than half: not cut
                                   (6401, 2304, 768)])    # 234 tiles: 12 left; a one-row last tile
def test_gemm_tcgen05_last_round_cut_into_half_width_units(m, n, k, epi):
    _gemm_case(torch.float16, m, m, n, k, epi, use_simt=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("m,cap,n,k", [(1, 1, 128, 64), (60, 60, 128, 128), (134, 256, 768, 768),
                                       (257, 300, 768, 3072), (300, 300, 2304, 768), (0, 64, 256, 128)])
@pytest.mark.parametrize("epi", [0, 1, 2])
def test_gemm_simt(dtype, m, cap, n, k, epi):
    _gemm_case(dtype, m, cap, n, k, epi, use_simt=True)


def _attention_case(dtype, lens, heads, use_simt, layout):
    d = 64
    h = heads * d
    lens = np.asarray(lens, np.int32)
    cu = np.zeros(len(lens) + 1, np.int32)
    cu[1:] = np.cumsum(lens)
    t = int(cu[-1])
    cap = max(t, 1)
    rng = np.random.RandomState(int(lens.sum()) + heads)
    if layout == "qkv":        # [T, 3H] as the fused projection writes it
        qkv = dev(rng.randn(cap, 3 * h).astype(np.float32), dtype)
        q, k, v = qkv[:, :h], qkv[:, h:2 * h], qkv[:, 2 * h:]
        qp, kp, vp = qkv.data_ptr(), qkv.data_ptr() + h * qkv.element_size(), qkv.data_ptr() + 2 * h * qkv.element_size()
        tstride, hstride = 3 * h, d
    elif layout == "unaligned":  # rows of 3H + 1 elements starting one element into the buffer
        wide = dev(rng.randn(cap, 3 * h + 1).astype(np.float32), dtype)
        es = wide.element_size()
        q, k, v = wide[:, 1:h + 1], wide[:, h + 1:2 * h + 1], wide[:, 2 * h + 1:]
        qp, kp, vp = wide.data_ptr() + es, wide.data_ptr() + (h + 1) * es, wide.data_ptr() + (2 * h + 1) * es
        tstride, hstride = 3 * h + 1, d
    else:                      # head-major [3, heads, cap, d] as et_add_qkv_bias_transpose writes it
        buf = dev(rng.randn(3, heads, cap, d).astype(np.float32), dtype)
        q, k, v = [buf[i].permute(1, 0, 2).reshape(cap, h) for i in range(3)]
        es = buf.element_size()
        qp, kp, vp = [buf.data_ptr() + i * heads * cap * d * es for i in range(3)]
        tstride, hstride = d, cap * d
    ctx = torch.full((cap, h), 2.0, dtype=dtype, device="cuda")
    st = status_word()
    ok(lib().et_attention(DT[dtype], qp, kp, vp, tstride, hstride, iptr(ctx), iptr(dev(cu)), len(lens),
                          int(lens.max()) if len(lens) else 0, cap, heads, d, 1 if use_simt else 0, iptr(st),
                          stream()))
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    ref = O.packed_attention(q[:t].double().cpu(), k[:t].double().cpu(), v[:t].double().cpu(), cu, heads, d)
    tol = dict(rtol=3e-3, atol=3e-3) if dtype == torch.float16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(ctx[:t].double().cpu(), ref, **tol)
    assert torch.all(ctx[t:] == 2.0)


LEN_CASES = [[1], [5, 1, 16, 0, 33], [64] * 3, [20, 23, 29, 8, 11, 11, 15, 17], [128, 1, 100, 127, 65, 64, 63],
             [200, 3, 129]]


@pytest.mark.parametrize("lens", LEN_CASES)
@pytest.mark.parametrize("layout", ["qkv", "headmajor"])
def test_attention_tensor_core(lens, layout):
    _attention_case(torch.float16, lens, 2, use_simt=False, layout=layout)


@pytest.mark.parametrize("lens", LEN_CASES)
@pytest.mark.parametrize("layout", ["qkv", "headmajor", "unaligned"])
def test_attention_fp32_on_tensor_cores_keeps_fp32_accuracy(lens, layout):
    """The fp32 handle's attention: mma.sync with tf32 operands, three products per fp32 product,
    held to the tolerance of the CUDA-core fp32 kernel (1e-5 against the float64 oracle)."""
    _attention_case(torch.float32, lens, 3, use_simt=False, layout=layout)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("lens", LEN_CASES)
def test_attention_simt(dtype, lens):
    _attention_case(dtype, lens, 3, use_simt=True, layout="qkv")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_attention_simt_rows_off_the_vector_boundary(dtype):
    """Row segments that do not start on a 16-byte (fp32) / 8-byte (fp16) boundary take the
    element-wise loads of the CUDA-core kernel."""
    _attention_case(dtype, [20, 23, 70, 8, 1], 3, use_simt=True, layout="unaligned")


def _attention_tiles_case(lens, heads, layout, seed=0):
    """et_attention_plan + et_attention_tiles (tcgen05, sequences of <= 128 tokens)."""
    d = 64
    h = heads * d
    lens = np.asarray(lens, np.int32)
    cu = np.zeros(len(lens) + 1, np.int32)
    cu[1:] = np.cumsum(lens)
    t = int(cu[-1])
    cap = max(t, 1) + 5          # a few stale rows behind the last token
    rng = np.random.RandomState(int(lens.sum()) + heads + seed)
    if layout == "qkv":
        qkv = dev(rng.randn(cap, 3 * h).astype(np.float32), torch.float16)
        qkv[t:] = float("nan")   # stale rows must never reach a valid output
        q, k, v = qkv[:, :h], qkv[:, h:2 * h], qkv[:, 2 * h:]
        qp, kp, vp = qkv.data_ptr(), qkv.data_ptr() + h * 2, qkv.data_ptr() + 2 * h * 2
        tstride, hstride = 3 * h, d
    else:
        buf = dev(rng.randn(3, heads, cap, d).astype(np.float32), torch.float16)
        buf[:, :, t:] = float("nan")
        q, k, v = [buf[i].permute(1, 0, 2).reshape(cap, h) for i in range(3)]
        qp, kp, vp = [buf.data_ptr() + i * heads * cap * d * 2 for i in range(3)]
        tstride, hstride = d, cap * d
    ctx = torch.full((cap, h), 2.0, dtype=torch.float16, device="cuda")
    st = status_word()
    cu_d = dev(cu)
    plan = torch.zeros(int(lib().et_attention_plan_ints(len(lens), cap)), dtype=torch.int32, device="cuda")
    ok(lib().et_attention_plan(iptr(cu_d), len(lens), cap, iptr(plan), stream()))
    ok(lib().et_attention_tiles(qp, kp, vp, tstride, hstride, iptr(ctx), iptr(plan), len(lens),
                                int(lens.max()) if len(lens) else 0, cap, heads, d, iptr(st), stream()))
    torch.cuda.synchronize()
    assert int(st[0]) == 0, f"device-side wait expired: status 0x{int(st[0]):x}"
    # the plan: whole sequences, at most 128 rows per tile, every token covered once
    pl = plan.cpu().numpy()
    nt, b = int(pl[0]), len(lens)
    starts, rows = pl[4:4 + nt], pl[4 + b:4 + b + nt]
    assert np.all(rows >= 1) and np.all(rows <= 128) and int(rows.sum()) == t
    assert np.all(np.isin(starts, cu)) and np.all(np.isin(starts + rows, cu))
    ref = O.packed_attention(q[:t].double().cpu(), k[:t].double().cpu(), v[:t].double().cpu(), cu, heads, d)
    torch.testing.assert_close(ctx[:t].double().cpu(), ref, rtol=3e-3, atol=3e-3)
    assert torch.all(ctx[t:] == 2.0)


TILE_LEN_CASES = [[1], [5, 1, 16, 0, 33], [64] * 3, [20, 23, 29, 8, 11, 11, 15, 17], [128, 1, 100, 127, 65, 64, 63],
                  [128] * 4, [1] * 300, [17] * 40 + [0] * 3 + [111]]


@pytest.mark.parametrize("lens", TILE_LEN_CASES)
@pytest.mark.parametrize("layout", ["qkv", "headmajor"])
def test_attention_tcgen05_tiles(lens, layout):
    _attention_tiles_case(lens, 2, layout)


def test_attention_tcgen05_tiles_benchmark_shapes():
    for cfg, heads in ((1, 12), (4, 16)):
        spec = W.WORKLOADS[cfg]
        lens = W.draw_lengths(spec, np.random.RandomState(spec.seed))[:400]
        _attention_tiles_case(lens, heads, "qkv", seed=cfg)


def test_attention_full_size_softmax_rows_sum_to_one():
    """cfg2 shape (B=1000, 12 heads): with V = 1 every context element must be 1
    (each probability row sums to one over the sequence's own keys only)."""
    spec = W.WORKLOADS[2]
    lens = W.draw_lengths(spec, np.random.RandomState(spec.seed))
    cu = np.zeros(len(lens) + 1, np.int32); cu[1:] = np.cumsum(lens)
    t, h = int(cu[-1]), 768
    qkv = torch.randn(t, 3 * h, dtype=torch.float16, device="cuda")
    qkv[:, 2 * h:] = 1.0
    ctx = torch.zeros(t, h, dtype=torch.float16, device="cuda")
    st = status_word()
    es = 2
    ok(lib().et_attention(_capi.ET_FP16, qkv.data_ptr(), qkv.data_ptr() + h * es, qkv.data_ptr() + 2 * h * es,
                          3 * h, 64, iptr(ctx), iptr(dev(cu)), len(lens), 64, t, 12, 64, 0, iptr(st), stream()))
    torch.cuda.synchronize()
    assert float((ctx.float() - 1.0).abs().max()) < 2e-3


@pytest.mark.parametrize("m,cap,n,k", [(1, 1, 128, 64), (60, 60, 128, 128), (134, 256, 768, 768),
                                       (300, 384, 2304, 768), (257, 300, 768, 3072), (128, 128, 256, 32),
                                       (1000, 1000, 3072, 768), (0, 64, 256, 128), (5000, 5000, 1152, 1024),
                                       (5000, 5000, 1024, 512),    # 80 pair tiles: the last round is cut in halves
                                       (9000, 10000, 768, 3072)])  # pair kernel, long K, M below capacity, 108 tiles
@pytest.mark.parametrize("epi", [0, 1, 2, 3])
def test_gemm_fp32_on_tensor_cores_keeps_fp32_accuracy(m, cap, n, k, epi):
    """The three-product tf32 split: same tolerance as the CUDA-core fp32 GEMM against the
    float64 product, and the split itself is exact (hi + lo == x, hi has 11 significand bits)."""
    rng = np.random.RandomState(m + n + k + epi)
    a = dev(rng.randn(cap, k).astype(np.float32))
    w = dev((rng.randn(k, n) / math.sqrt(k)).astype(np.float32))
    bias = dev(rng.randn(n).astype(np.float32))
    c = torch.full((cap, n), 3.0, dtype=torch.float32, device="cuda")
    w_hi = torch.empty((n, k), dtype=torch.float32, device="cuda")
    ok(lib().et_pack_weight(_capi.ET_FP32, iptr(w), iptr(w_hi), k, n, stream()))
    w_lo = torch.empty_like(w_hi)
    ok(lib().et_split_tf32(iptr(w_hi), iptr(w_hi), iptr(w_lo), None, n, k, stream()))     # in place
    a_hi, a_lo = torch.empty_like(a), torch.empty_like(a)
    mt = dev(np.array([m], np.int32))
    ok(lib().et_split_tf32(iptr(a), iptr(a_hi), iptr(a_lo), iptr(mt), cap, k, stream()))
    torch.cuda.synchronize()
    assert torch.equal(a_hi[:m] + a_lo[:m], a[:m])
    assert torch.equal(w_hi + w_lo, w.t().contiguous())
    assert bool(((a_hi[:m].view(torch.int32) & 0x1FFF) == 0).all())          # tf32: low 13 bits clear
    assert bool((a_lo[:m].abs() <= a[:m].abs() * 2.0 ** -11).all())
    st = status_word()
    ok(lib().et_gemm_fp32_tensor(iptr(a_hi), iptr(a_lo), iptr(w_hi), iptr(w_lo), iptr(bias) if epi else None,
                                 iptr(c), iptr(mt), cap, n, k, epi, iptr(st), stream()))
    torch.cuda.synchronize()
    assert int(st[0]) == 0, f"device-side wait expired: status 0x{int(st[0]):x}"
    ref = a[:m].double() @ w.double()
    if epi >= 1:
        ref = ref + bias.double()
    if epi == 2:
        ref = O.gelu(ref)
    if epi == 3:
        ref = torch.tanh(ref)
    torch.testing.assert_close(c[:m].double(), ref, rtol=1e-5, atol=2e-5)
    assert torch.all(c[m:] == 3.0), "rows past M were written"
    if m > 0:
        # a plain tf32 product (one term) would miss this tolerance by two orders of magnitude
        one_term = (a_hi[:m].double() @ w_hi.double().t())
        plain = a[:m].double() @ w.double()
        assert float((one_term - plain).abs().max()) > 20 * float((c[:m].double() - ref).abs().max()) or k < 128


# ---- epilogues that take the layer's residual: bias + residual, and the LayerNorm inside the GEMM -------
def _gemm_fused_case(m, cap, n, k, epi, seed=0, counters_check=True):
    """et_gemm_fused against the float64 oracle: C = A W + bias + residual (4), and its LayerNorm
    (5: bias/residual added in the accumulator epilogue, 6: added where the rows are normalised)."""
    rng = np.random.RandomState(seed + m + n + k + epi)
    h = torch.float16
    a = dev(rng.randn(cap, k).astype(np.float32), h)
    w = dev((rng.randn(k, n) / math.sqrt(k)).astype(np.float32), h)
    bias = dev(0.5 * rng.randn(n).astype(np.float32), h)
    res = dev(rng.randn(cap, n).astype(np.float32), h)
    gamma = dev((1 + 0.2 * rng.randn(n)).astype(np.float32), h)
    beta = dev(0.3 * rng.randn(n).astype(np.float32), h)
    c = torch.full((cap, n), 3.0, dtype=h, device="cuda")
    wp = torch.empty((n, k), dtype=h, device="cuda")
    ok(lib().et_pack_weight(DT[h], iptr(w), iptr(wp), k, n, stream()))
    counters = torch.zeros(8 * ((cap + 255) // 256) + 1, dtype=torch.int32, device="cuda")   # one per 32 rows of the 256-row tiles
    mt = dev(np.array([m], np.int32))
    st = status_word()
    ok(lib().et_gemm_fused(iptr(a), iptr(wp), iptr(bias), iptr(res), iptr(gamma), iptr(beta), 1e-6, iptr(counters),
                           iptr(c), iptr(mt), cap, n, k, epi, iptr(st), stream()))
    torch.cuda.synchronize()
    assert int(st[0]) == 0, f"device-side wait expired: status 0x{int(st[0]):x}"
    pre = a[:m].double() @ w.double() + bias.double() + res[:m].double()
    if epi == 4:
        torch.testing.assert_close(c[:m].double(), pre, rtol=2e-3, atol=4e-3)
    else:
        mean = pre.mean(-1, keepdim=True)
        var = ((pre - mean) ** 2).mean(-1, keepdim=True)
        ref = (pre - mean) / torch.sqrt(var + 1e-6) * gamma.double() + beta.double()
        # the pre-LayerNorm sum is stored in fp16 once (as the reference's half kernel adds in half2,
        # cuda/cuda_kernels.cu:214): one fp16 rounding of an O(1) value in front of the normalisation
        torch.testing.assert_close(c[:m].double(), ref, rtol=3e-3, atol=6e-3)
    assert torch.all(c[m:] == 3.0), "rows past M were written"
    if counters_check:
        assert int(counters.abs().sum()) == 0, "the row counters must be zero again after the launch"


@pytest.mark.parametrize("epi", [4, 5, 6])
@pytest.mark.parametrize("m,cap,n,k", [(1, 1, 256, 64), (134, 256, 768, 768), (257, 300, 768, 3072),
                                       (1000, 1000, 1024, 1024), (300, 384, 512, 128), (0, 64, 768, 128),
                                       (31, 64, 768, 768), (33, 33, 1024, 4096)])
def test_gemm_tcgen05_residual_and_layernorm_epilogues(m, cap, n, k, epi):
    _gemm_fused_case(m, cap, n, k, epi)


@pytest.mark.parametrize("epi", [4, 5, 6])
@pytest.mark.parametrize("m,n,k", [(6500, 768, 768),      # last round cut into half-width units
                                   (9372, 768, 3072),     # 37 tiles left = exactly half of the pairs
                                   (9729, 768, 768),      # 43 left: not cut
                                   (20000, 1024, 1024)])  # several rounds per pair: mailboxes are reused
def test_gemm_tcgen05_residual_and_layernorm_epilogues_many_tiles(m, n, k, epi):
    _gemm_fused_case(m, m, n, k, epi)


def test_gemm_layernorm_epilogue_equals_gemm_then_layernorm_kernel():
    """The rows the GEMM normalises itself are those of the two-kernel path: epilogue 4 followed by
    add_bias_input_layernorm on one tensor, and epilogue 0 followed by the kernel with bias and
    residual.  Same arithmetic in the same order; the compiler may contract a multiply-add in one
    kernel and not in the other, so a few elements differ by one fp16 unit in the last place."""
    rng = np.random.RandomState(5)
    m, n, k = 4973, 768, 768
    h = torch.float16
    a = dev(rng.randn(m, k).astype(np.float32), h)
    w = dev((rng.randn(k, n) / math.sqrt(k)).astype(np.float32), h)
    bias = dev(0.5 * rng.randn(n).astype(np.float32), h)
    res = dev(rng.randn(m, n).astype(np.float32), h)
    gamma = dev((1 + 0.2 * rng.randn(n)).astype(np.float32), h)
    beta = dev(0.3 * rng.randn(n).astype(np.float32), h)
    wp = torch.empty((n, k), dtype=h, device="cuda")
    ok(lib().et_pack_weight(DT[h], iptr(w), iptr(wp), k, n, stream()))
    mt = dev(np.array([m], np.int32))
    st = status_word()
    counters = torch.zeros(8 * ((m + 255) // 256), dtype=torch.int32, device="cuda")
    zero_bias = torch.zeros_like(bias)

    def fused(epi):
        c = torch.empty((m, n), dtype=h, device="cuda")
        ok(lib().et_gemm_fused(iptr(a), iptr(wp), iptr(bias), iptr(res), iptr(gamma), iptr(beta), 1e-6,
                               iptr(counters), iptr(c), iptr(mt), m, n, k, epi, iptr(st), stream()))
        return c

    # 5 == (4, then LayerNorm of one tensor)
    two = fused(4)
    ok(lib().et_add_bias_input_layernorm(DT[h], iptr(two), iptr(torch.zeros_like(two)), iptr(zero_bias), iptr(gamma),
                                         iptr(beta), iptr(mt), m, n, 1e-6, stream()))
    one = fused(5)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    assert int((one != two).sum()) <= m * n // 5000 and float((one.float() - two.float()).abs().max()) <= 4e-3
    # 6 == (plain GEMM, then LayerNorm with bias and residual)
    plain = torch.empty((m, n), dtype=h, device="cuda")
    ok(lib().et_gemm(DT[h], iptr(a), None, iptr(wp), None, iptr(plain), iptr(mt), m, n, k, 0, 0, iptr(st), stream()))
    ok(lib().et_add_bias_input_layernorm(DT[h], iptr(plain), iptr(res), iptr(bias), iptr(gamma), iptr(beta), iptr(mt),
                                         m, n, 1e-6, stream()))
    one = fused(6)
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    assert int((one != plain).sum()) <= m * n // 5000 and float((one.float() - plain.float()).abs().max()) <= 4e-3


# ---- the LayerNorm that is never materialised: folded into the consumer, statistics from the producer -----
def _row_stat_pieces(x16: torch.Tensor) -> torch.Tensor:
    """(sum, sum of squares) of every 64-column piece of every row, as the producer epilogue leaves them."""
    rows, width = x16.shape
    xs = x16.float().reshape(rows, width // 64, 64)
    return torch.stack([xs.sum(-1), (xs * xs).sum(-1)], dim=-1).reshape(rows, 2 * (width // 64)).contiguous()


def _deferred_consumer_case(m, cap, n, k, gelu, with_stats, seed=0):
    """epilogues 7 / 8: the projection of LN(x) computed from x, folded weights and x's row statistics."""
    rng = np.random.RandomState(seed + m + n + k)
    h = torch.float16
    x = dev((1.5 * rng.randn(cap, k) + 0.3).astype(np.float32), h)        # un-normalised rows with a mean
    w = dev((rng.randn(k, n) / math.sqrt(k)).astype(np.float32), h)
    bias = dev(0.5 * rng.randn(n).astype(np.float32), h)
    gamma = dev((1 + 0.2 * rng.randn(k)).astype(np.float32), h)
    beta = dev(0.3 * rng.randn(k).astype(np.float32), h)
    wp = torch.empty((n, k), dtype=h, device="cuda")
    ok(lib().et_pack_weight(DT[h], iptr(w), iptr(wp), k, n, stream()))
    wf, csum, bf = torch.empty_like(wp), torch.empty(n, dtype=h, device="cuda"), torch.empty(n, dtype=h, device="cuda")
    ok(lib().et_fold_layernorm(iptr(wp), iptr(bias), iptr(gamma), iptr(beta), iptr(wf), iptr(csum), iptr(bf), n, k,
                               stream()))
    torch.cuda.synchronize()
    # the fold itself: gamma folded in, then the mean over k taken from every output row (it multiplies
    # sum_k (x_k - mu) = 0); csum is what fp16 rounding leaves of the zero row sums
    v = wp.float() * gamma.float()[None, :]
    wf_ref = (v - v.mean(-1, keepdim=True)).half()
    assert float((wf.float() - wf_ref.float()).abs().max()) <= 2e-3 * float(v.abs().max())
    torch.testing.assert_close(csum.float(), wf.float().sum(-1), rtol=1e-2, atol=1e-3)
    assert float(csum.float().abs().max()) < 0.05
    torch.testing.assert_close(bf.double(), bias.double() + beta.double() @ w.double(), rtol=2e-3, atol=2e-3)
    rows_cap = (cap + 255) // 256 * 256
    stats = torch.zeros(rows_cap, 2 * (k // 64), dtype=torch.float32, device="cuda")
    stats[:cap] = _row_stat_pieces(x)
    c = torch.full((cap, n), 3.0, dtype=h, device="cuda")
    mt = dev(np.array([m], np.int32))
    st = status_word()
    ok(lib().et_gemm_deferred_norm(iptr(x), iptr(wf if with_stats else wp), iptr(bf if with_stats else bias),
                                   iptr(csum), None, None, None, 1e-6, iptr(stats) if with_stats else None, None,
                                   iptr(c), iptr(mt), cap, n, k, 8 if gelu else 7, iptr(st), stream()))
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    xd = x[:m].double()
    if with_stats:
        mean = xd.mean(-1, keepdim=True)
        var = ((xd - mean) ** 2).mean(-1, keepdim=True)
        y = (xd - mean) / torch.sqrt(var + 1e-6) * gamma.double() + beta.double()
    else:
        y = xd                                                             # no statistics: x is used as it is
    ref = y @ w.double() + bias.double()
    if gelu:
        ref = O.gelu(ref)
    torch.testing.assert_close(c[:m].double(), ref, rtol=4e-3, atol=8e-3)
    assert torch.all(c[m:] == 3.0), "rows past M were written"


@pytest.mark.parametrize("gelu", [False, True])
@pytest.mark.parametrize("with_stats", [True, False])
@pytest.mark.parametrize("m,cap,n,k", [(1, 1, 256, 256), (134, 256, 2304, 768), (257, 300, 3072, 768),
                                       (1000, 1000, 1024, 1024), (0, 64, 768, 256), (6500, 6500, 768, 768),
                                       (300, 300, 512, 512)])
def test_gemm_tcgen05_projection_of_a_layernorm_that_is_not_materialised(m, cap, n, k, gelu, with_stats):
    _deferred_consumer_case(m, cap, n, k, gelu, with_stats)


def _deferred_producer_case(m, cap, n, k, with_norm, seed=0):
    """epilogue 9: C = A W + bias + LN(residual) with the LayerNorm taken on the fly, and the statistics
    of the stored rows of C."""
    rng = np.random.RandomState(seed + m + n + k + 9)
    h = torch.float16
    a = dev(rng.randn(cap, k).astype(np.float32), h)
    w = dev((rng.randn(k, n) / math.sqrt(k)).astype(np.float32), h)
    bias = dev(0.5 * rng.randn(n).astype(np.float32), h)
    res = dev((1.5 * rng.randn(cap, n) + 0.3).astype(np.float32), h)
    gamma = dev((1 + 0.2 * rng.randn(n)).astype(np.float32), h)
    beta = dev(0.3 * rng.randn(n).astype(np.float32), h)
    wp = torch.empty((n, k), dtype=h, device="cuda")
    ok(lib().et_pack_weight(DT[h], iptr(w), iptr(wp), k, n, stream()))
    rows_cap = (cap + 255) // 256 * 256
    stats_in = torch.zeros(rows_cap, 2 * (n // 64), dtype=torch.float32, device="cuda")
    stats_in[:cap] = _row_stat_pieces(res)
    stats_out = torch.full((rows_cap, 2 * (n // 64)), -7.0, dtype=torch.float32, device="cuda")
    c = torch.full((cap, n), 3.0, dtype=h, device="cuda")
    mt = dev(np.array([m], np.int32))
    st = status_word()
    ok(lib().et_gemm_deferred_norm(iptr(a), iptr(wp), iptr(bias), None, iptr(res),
                                   iptr(gamma) if with_norm else None, iptr(beta) if with_norm else None, 1e-6,
                                   iptr(stats_in) if with_norm else None, iptr(stats_out), iptr(c), iptr(mt), cap, n,
                                   k, 9, iptr(st), stream()))
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    rd = res[:m].double()
    if with_norm:
        mean = rd.mean(-1, keepdim=True)
        var = ((rd - mean) ** 2).mean(-1, keepdim=True)
        rd = (rd - mean) / torch.sqrt(var + 1e-6) * gamma.double() + beta.double()
    ref = a[:m].double() @ w.double() + bias.double() + rd
    torch.testing.assert_close(c[:m].double(), ref, rtol=3e-3, atol=6e-3)
    assert torch.all(c[m:] == 3.0), "rows past M were written"
    # the statistics describe the rows as they were stored
    want = _row_stat_pieces(c[:m])
    torch.testing.assert_close(stats_out[:m], want, rtol=1e-5, atol=1e-4)
    assert torch.all(stats_out[m:] == -7.0), "statistics of rows past M were written"


@pytest.mark.parametrize("with_norm", [True, False])
@pytest.mark.parametrize("m,cap,n,k", [(1, 1, 256, 64), (134, 256, 768, 768), (257, 300, 768, 3072),
                                       (1000, 1000, 1024, 4096), (0, 64, 768, 128), (6500, 6500, 768, 768),
                                       (9372, 9372, 768, 3072)])
def test_gemm_tcgen05_residual_is_a_layernorm_taken_on_the_fly(m, cap, n, k, with_norm):
    _deferred_producer_case(m, cap, n, k, with_norm)


def test_deferred_layernorm_rows_with_a_large_mean_and_a_small_spread():
    """Rows whose mean dwarfs their spread (x = 60 + noise; one row constant, where rstd reaches
    1 / sqrt(eps)): LN(x) is O(1) while x W is in the hundreds.  The consumer (7) runs on weights with
    centred columns, so that no term with the row's mean is left to cancel in its epilogue; the
    producer (9) takes (res - mu) * rstd in fp32.  Both must stay close to the float64 LayerNorm.
    (The row statistics are fp32 sums and sums of squares: their variance is good to about
    1e-7 * (mu / sigma)^2 relative, i.e. to 4e-4 here; a ratio of a thousand would need another form.)"""
    rng = np.random.RandomState(3)
    h = torch.float16
    m, n, k = 300, 768, 768
    x = (60.0 + rng.randn(m, k)).astype(np.float32)
    x[7, :] = 60.0                                                         # zero variance
    x = dev(x, h)
    w = dev((rng.randn(k, n) / math.sqrt(k)).astype(np.float32), h)
    bias = dev(0.5 * rng.randn(n).astype(np.float32), h)
    gamma = dev((1 + 0.2 * rng.randn(k)).astype(np.float32), h)
    beta = dev(0.3 * rng.randn(k).astype(np.float32), h)
    wp = torch.empty((n, k), dtype=h, device="cuda")
    ok(lib().et_pack_weight(DT[h], iptr(w), iptr(wp), k, n, stream()))
    wf, csum, bf = torch.empty_like(wp), torch.empty(n, dtype=h, device="cuda"), torch.empty(n, dtype=h, device="cuda")
    ok(lib().et_fold_layernorm(iptr(wp), iptr(bias), iptr(gamma), iptr(beta), iptr(wf), iptr(csum), iptr(bf), n, k,
                               stream()))
    rows_cap = (m + 255) // 256 * 256
    stats = torch.zeros(rows_cap, 2 * (k // 64), dtype=torch.float32, device="cuda")
    stats[:m] = _row_stat_pieces(x)
    xd = x.double()
    mean = xd.mean(-1, keepdim=True)
    var = ((xd - mean) ** 2).mean(-1, keepdim=True)
    y = (xd - mean) / torch.sqrt(var + 1e-6) * gamma.double() + beta.double()
    mt = dev(np.array([m], np.int32))
    st = status_word()
    # consumer: projection of LN(x)
    c = torch.zeros((m, n), dtype=h, device="cuda")
    ok(lib().et_gemm_deferred_norm(iptr(x), iptr(wf), iptr(bf), iptr(csum), None, None, None, 1e-6, iptr(stats), None,
                                   iptr(c), iptr(mt), m, n, k, 7, iptr(st), stream()))
    torch.cuda.synchronize()
    ref = y @ w.double() + bias.double()
    assert torch.isfinite(c).all()
    torch.testing.assert_close(c.double(), ref, rtol=1e-2, atol=3e-2)
    # producer: A W + bias + LN(x) as the residual
    a = dev(rng.randn(m, k).astype(np.float32), h)
    stats_out = torch.zeros(rows_cap, 2 * (n // 64), dtype=torch.float32, device="cuda")
    c2 = torch.zeros((m, n), dtype=h, device="cuda")
    ok(lib().et_gemm_deferred_norm(iptr(a), iptr(wp), iptr(bias), None, iptr(x), iptr(gamma), iptr(beta), 1e-6,
                                   iptr(stats), iptr(stats_out), iptr(c2), iptr(mt), m, n, k, 9, iptr(st), stream()))
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    ref2 = a.double() @ w.double() + bias.double() + y
    assert torch.isfinite(c2).all()
    torch.testing.assert_close(c2.double(), ref2, rtol=1e-2, atol=3e-2)


def test_gemm_fused_rejects_what_it_cannot_do():
    z = torch.zeros(256, dtype=torch.float16, device="cuda")
    cnt = torch.zeros(8, dtype=torch.int32, device="cuda")
    mt = dev(np.array([1], np.int32))
    bad = _capi.ET_INVALID_ARGUMENT
    # N not a multiple of 256 / above 1024 for the LayerNorm epilogues, unknown epilogue, missing pointers
    assert lib().et_gemm_fused(iptr(z), iptr(z), iptr(z), iptr(z), iptr(z), iptr(z), 1e-6, iptr(cnt), iptr(z),
                               iptr(mt), 1, 128, 64, 5, None, stream()) == bad
    assert lib().et_gemm_fused(iptr(z), iptr(z), iptr(z), iptr(z), iptr(z), iptr(z), 1e-6, iptr(cnt), iptr(z),
                               iptr(mt), 1, 1280, 64, 6, None, stream()) == bad
    assert lib().et_gemm_fused(iptr(z), iptr(z), iptr(z), iptr(z), iptr(z), iptr(z), 1e-6, iptr(cnt), iptr(z),
                               iptr(mt), 1, 256, 64, 2, None, stream()) == bad
    assert lib().et_gemm_fused(iptr(z), iptr(z), iptr(z), iptr(z), iptr(z), iptr(z), 1e-6, None, iptr(z),
                               iptr(mt), 1, 256, 64, 5, None, stream()) == bad
    assert lib().et_gemm_fused(iptr(z), iptr(z), iptr(z), None, iptr(z), iptr(z), 1e-6, iptr(cnt), iptr(z),
                               iptr(mt), 1, 256, 64, 4, None, stream()) == bad


# ---- cross-attention: from_seq_len != to_seq_len on packed tensors ------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("lens_q,lens_k", [([5, 1, 16, 33], [7, 40, 3, 1]), ([64, 64, 2], [128, 1, 90]),
                                           ([10, 0, 4], [6, 9, 0]), ([130, 3], [70, 200])])
def test_cross_attention_against_the_padded_oracle(dtype, lens_q, lens_k):
    """et_attention_cross vs attention_layer with from_tensor != to_tensor (padded, key-only mask of
    the to-tensor), compared on the valid query rows.  A query whose to-sequence is empty gets zeros."""
    rng = np.random.RandomState(sum(lens_q) + 7 * sum(lens_k))
    heads, d = 3, 64
    h = heads * d
    lens_q, lens_k = np.array(lens_q, np.int32), np.array(lens_k, np.int32)
    b, f, t = len(lens_q), int(max(lens_q.max(), 1)), int(max(lens_k.max(), 1))
    cu_q = np.zeros(b + 1, np.int32); cu_q[1:] = np.cumsum(lens_q)
    cu_k = np.zeros(b + 1, np.int32); cu_k[1:] = np.cumsum(lens_k)
    tq, tk = int(cu_q[-1]), int(cu_k[-1])
    q = dev(rng.randn(tq + 3, h).astype(np.float32), dtype)
    kv = dev(rng.randn(tk + 2, 2 * h).astype(np.float32), dtype)       # K and V side by side: their own row stride
    ctx = torch.full((tq + 3, h), 2.0, dtype=dtype, device="cuda")
    cu_q_d, cu_k_d = dev(cu_q), dev(cu_k)
    ok(lib().et_attention_cross(DT[dtype], iptr(q), h, kv.data_ptr(), kv.data_ptr() + h * kv.element_size(), 2 * h, d,
                                iptr(ctx), iptr(cu_q_d), iptr(cu_k_d), b, f, t, heads, d, stream()))
    torch.cuda.synchronize()
    # padded oracle
    qp = torch.zeros(b, f, h, dtype=torch.float64)
    kp = torch.zeros(b, t, h, dtype=torch.float64)
    vp = torch.zeros(b, t, h, dtype=torch.float64)
    mask = torch.zeros(b, f, t, dtype=torch.float64)
    for i in range(b):
        qp[i, :lens_q[i]] = q[cu_q[i]:cu_q[i + 1]].double().cpu()
        kp[i, :lens_k[i]] = kv[cu_k[i]:cu_k[i + 1], :h].double().cpu()
        vp[i, :lens_k[i]] = kv[cu_k[i]:cu_k[i + 1], h:].double().cpu()
        mask[i, :, :lens_k[i]] = 1.0
    ref = O.cross_attention_padded(qp, kp, vp, mask, heads, d)
    tol = dict(rtol=3e-3, atol=3e-3) if dtype == torch.float16 else dict(rtol=1e-5, atol=1e-5)
    for i in range(b):
        got = ctx[cu_q[i]:cu_q[i + 1]].double().cpu()
        if lens_k[i] == 0:
            assert torch.all(got == 0)
        else:
            torch.testing.assert_close(got, ref[i, :lens_q[i]], **tol)
    assert torch.all(ctx[tq:] == 2.0)
