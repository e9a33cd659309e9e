"""GPU tests that run the REFERENCE's own CUDA kernels (cuda/cuda_kernels.cu and
cuda/attention.cu of the reference checkout, compiled unmodified for sm_100a by
oracle/build_ref.py into oracle/_ref/libet_ref_kernels.so) next to the CPU
oracle and next to this repository's kernels, on the same seeded inputs.

They pin the oracle to the reference at kernel level: the integer outputs
(scan, batch_idx, word_idx, valid count) and the copies must agree bit for bit;
LayerNorm, bias+GELU and the attention block (QKV bias + re-padding, softmax,
head merge; the two batched GEMMs in between are torch.matmul standing in for
cuBLAS) must agree within one rounding of the storage type.
Skipped when the checker library has not been built (no reference checkout)."""
import ctypes as C
import math
import os

import numpy as np
import pytest
import torch

from effective_transformer_b200 import _capi
from effective_transformer_b200 import workloads as W
from oracle import bert_encoder as O
from oracle import padding as P

from util import DT, dev, iptr, lib, ok, padding_offsets, status_word, stream

pytestmark = pytest.mark.gpu
REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                       "libet_ref_kernels.so")
_ref = None


def ref():
    global _ref
    if _ref is None:
        if not os.path.exists(REF_LIB):
            pytest.skip("oracle/_ref/libet_ref_kernels.so not built (needs the reference checkout)")
        _ref = C.CDLL(REF_LIB)
        vp, i32 = C.c_void_p, C.c_int
        sigs = {
            "ref_exclusive_scan": [vp, vp, i32, vp],
            "ref_compress_input": [i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, vp],
            "ref_restore_output": [i32, vp, vp, vp, vp, i32, i32, i32, vp],
            "ref_add_bias_act": [i32, vp, vp, i32, i32, vp],
            "ref_add_bias_input_layernorm": [i32, vp, vp, vp, vp, vp, i32, i32, vp],
            "ref_add_qkv_bias_padding": [i32] + [vp] * 9 + [i32] * 5 + [vp, vp, vp],
            "ref_softmax": [i32, vp, vp, i32, i32, i32, C.c_float, vp],
            "ref_transpose_rm_padding": [i32, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp],
        }
        for n, a in sigs.items():
            getattr(_ref, n).restype = i32
            getattr(_ref, n).argtypes = a
    return _ref


def rok(code):
    assert code == 0, f"reference launcher reported CUDA error {code}"


def ref_input_op(x, mask_np):
    """The reference's input functor (tf_op/bert_transformer_op.cu.cc:266-331) on its own kernels."""
    b, s = mask_np.shape
    n, h = b * s, x.shape[-1]
    mask = dev(mask_np.astype(np.int32))
    scan = torch.full((2 * n,), -7, dtype=torch.int32, device="cuda")
    rok(ref().ref_exclusive_scan(iptr(scan), iptr(mask), n, stream()))
    packed = torch.full_like(x, 77.0)
    bidx = torch.full((n,), -7, dtype=torch.int32, device="cuda")
    widx = torch.full((n,), -7, dtype=torch.int32, device="cuda")
    rok(ref().ref_compress_input(DT[x.dtype], iptr(x), iptr(mask), iptr(scan), iptr(packed), iptr(bidx), iptr(widx),
                                 b, s, h, stream()))
    torch.cuda.synchronize()
    prefix = scan[:n].cpu().numpy()
    valid = int(prefix[-1]) + (1 if int(mask_np.ravel()[-1]) == 1 else 0)    # the functor's host rule
    return prefix, valid, bidx, widx, packed


@pytest.mark.parametrize("case", ["cfg0", "cfg1", "cfg2", "arbitrary", "short", "last_zero"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_padding_path_against_reference_kernels(case, dtype):
    rng = np.random.RandomState(5)
    if case in ("cfg0", "cfg1", "cfg2"):
        spec = W.WORKLOADS[int(case[-1])]
        lens = W.draw_lengths(spec, np.random.RandomState(spec.seed))
        mask_np, h = W.prefix_mask(lens, spec.max_seq_len), 768
    elif case == "arbitrary":
        mask_np, h = (rng.rand(37, 61) < 0.5).astype(np.int32), 128      # 2257 positions: 2 blocks + remainder
    elif case == "short":
        mask_np, h = (rng.rand(3, 50) < 0.7).astype(np.int32), 64        # a single small scan
    else:
        mask_np, h = np.ones((4, 256), np.int32), 64                      # exactly one 1024 block ...
        mask_np[-1, -1] = 0                                                # ... ending in a pad position
    b, s = mask_np.shape
    x = dev(rng.randn(b, s, h).astype(np.float32), dtype)
    prefix, valid, bidx, widx, packed = ref_input_op(x, mask_np)
    want = P.padding_indices(mask_np)
    t = int(want["valid_word_num"][0])
    # reference kernels == CPU oracle
    assert np.array_equal(prefix, want["prefix_sum"].ravel()) and valid == t
    assert np.array_equal(bidx.cpu().numpy()[:t], want["batch_idx"])
    assert np.array_equal(widx.cpu().numpy()[:t], want["word_idx"])
    assert np.array_equal(packed.cpu().numpy().reshape(b * s, h)[:t], P.remove_padding(x.cpu().numpy(), mask_np))
    # this repository's kernels == reference kernels
    mine = padding_offsets(dev(mask_np))
    assert int(mine["valid_word_num"][0]) == valid
    assert np.array_equal(mine["prefix_sum"].cpu().numpy()[:b * s], prefix)
    assert torch.equal(mine["batch_idx"][:t], bidx[:t]) and torch.equal(mine["word_idx"][:t], widx[:t])
    my_packed = torch.full_like(x, 77.0)
    ok(lib().et_remove_padding(DT[dtype], iptr(x), iptr(mine["batch_idx"]), iptr(mine["word_idx"]),
                               iptr(mine["valid_word_num"]), iptr(my_packed), b, s, h, stream()))
    torch.cuda.synchronize()
    assert torch.equal(my_packed.reshape(b * s, h)[:t], packed.reshape(b * s, h)[:t])
    # output op: cudaMemsetAsync + restore kernel of the reference vs the fused kernel here
    ref_out = torch.full_like(x, 9.0)
    ref_out.zero_()                                                        # the functor's memset
    rok(ref().ref_restore_output(DT[dtype], iptr(ref_out), iptr(packed), iptr(bidx), iptr(widx), valid, s, h, stream()))
    my_out = torch.full_like(x, 9.0)
    ok(lib().et_restore_padding(DT[dtype], iptr(my_packed), iptr(mine["batch_idx"]), iptr(mine["word_idx"]),
                                iptr(mine["valid_word_num"]), iptr(my_out), b, s, h, stream()))
    torch.cuda.synchronize()
    assert torch.equal(my_out, ref_out)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("m,n", [(37, 768), (1954, 768), (130, 1024)])
def test_layernorm_against_reference_kernel(dtype, m, n):
    rng = np.random.RandomState(m + n)
    out0 = dev(rng.randn(m, n).astype(np.float32), dtype)
    inp = dev(rng.randn(m, n).astype(np.float32), dtype)
    bias, beta = [dev(0.5 * rng.randn(n).astype(np.float32), dtype) for _ in range(2)]
    gamma = dev((1 + 0.2 * rng.randn(n)).astype(np.float32), dtype)
    r_out, m_out = out0.clone(), out0.clone()
    rok(ref().ref_add_bias_input_layernorm(DT[dtype], iptr(r_out), iptr(inp), iptr(bias), iptr(gamma), iptr(beta),
                                           m, n, stream()))
    tn = dev(np.array([m], np.int32))
    ok(lib().et_add_bias_input_layernorm(DT[dtype], iptr(m_out), iptr(inp), iptr(bias), iptr(gamma), iptr(beta),
                                         iptr(tn), m, n, 1e-6, stream()))
    torch.cuda.synchronize()
    want = O.add_bias_input_layernorm(out0.double(), inp.double(), bias.double(), gamma.double(), beta.double(),
                                      eps=1e-6)
    # the reference's half kernel adds out+input+bias in fp16 before the statistics: one more rounding
    tol = dict(rtol=4e-3, atol=8e-3) if dtype == torch.float16 else dict(rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(r_out.double(), want, **tol)      # reference kernel vs oracle
    torch.testing.assert_close(m_out.double(), r_out.double(), **tol)   # ours vs reference kernel


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("m,n", [(37, 3072), (500, 3072), (64, 4096)])
def test_bias_gelu_against_reference_kernel(dtype, m, n):
    rng = np.random.RandomState(m + n)
    x0 = dev((2.0 * rng.randn(m, n)).astype(np.float32), dtype)
    bias = dev(rng.randn(n).astype(np.float32), dtype)
    r_out, m_out = x0.clone(), x0.clone()
    rok(ref().ref_add_bias_act(DT[dtype], iptr(r_out), iptr(bias), m, n, stream()))
    tn = dev(np.array([m], np.int32))
    ok(lib().et_add_bias_gelu(DT[dtype], iptr(m_out), iptr(bias), iptr(tn), m, n, stream()))
    torch.cuda.synchronize()
    want = O.add_bias_gelu(x0.double(), bias.double())
    # the reference's half kernel cubes in fp16 (cuda/cuda_kernels.cu:42): a few fp16 roundings
    tol = dict(rtol=6e-3, atol=6e-3) if dtype == torch.float16 else dict(rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(r_out.double(), want, **tol)
    torch.testing.assert_close(m_out.double(), r_out.double(), **tol)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("batch,seq,heads", [(6, 32, 2), (11, 64, 12), (3, 128, 4)])   # softmax v2 / v1 / 128-wide
def test_attention_block_against_reference_kernels(dtype, batch, seq, heads):
    d, h = 64, heads * 64
    rng = np.random.RandomState(batch * seq + heads)
    lens = rng.randint(1, seq + 1, size=batch).astype(np.int32)
    lens[0] = seq
    mask_np = W.prefix_mask(lens, seq)
    idx = padding_offsets(dev(mask_np))
    t = int(idx["valid_word_num"][0])
    q, k, v = [dev(rng.randn(t, h).astype(np.float32), dtype) for _ in range(3)]
    bq, bk, bv = [dev(0.3 * rng.randn(h).astype(np.float32), dtype) for _ in range(3)]
    # ---- reference: bias + re-padding + head transpose, QK^T, softmax, PV, head merge + un-padding
    qb, kb, vb = [torch.zeros(batch, heads, seq, d, dtype=dtype, device="cuda") for _ in range(3)]   # the memset
    rok(ref().ref_add_qkv_bias_padding(DT[dtype], iptr(q), iptr(bq), iptr(k), iptr(bk), iptr(v), iptr(bv), iptr(qb),
                                       iptr(kb), iptr(vb), t, batch, seq, heads, d, iptr(idx["batch_idx"]),
                                       iptr(idx["word_idx"]), stream()))
    scores = torch.matmul(qb, kb.transpose(-1, -2)).contiguous()             # stands in for cublasGemmStridedBatchedEx
    attr_mask = dev(W.attention_mask_from_input_mask(mask_np).astype(np.float32), dtype)
    rok(ref().ref_softmax(DT[dtype], iptr(scores), iptr(attr_mask), batch, heads, seq, 1.0 / math.sqrt(d), stream()))
    ctx_pad = torch.matmul(scores, vb).contiguous()
    r_ctx = torch.zeros(t, h, dtype=dtype, device="cuda")
    rok(ref().ref_transpose_rm_padding(DT[dtype], iptr(ctx_pad), iptr(r_ctx), t, batch, seq, heads, d,
                                       iptr(idx["batch_idx"]), iptr(idx["word_idx"]), stream()))
    # ---- this repository: bias + head transpose (no re-padding), attention on the packed layout
    tn = dev(np.array([t], np.int32))
    qkv_t = torch.zeros(3, heads, t, d, dtype=dtype, device="cuda")
    ok(lib().et_add_qkv_bias_transpose(DT[dtype], iptr(q), iptr(bq), iptr(k), iptr(bk), iptr(v), iptr(bv),
                                       iptr(qkv_t), iptr(tn), t, heads, d, stream()))
    m_ctx = torch.zeros(t, h, dtype=dtype, device="cuda")
    st = status_word()
    es = qkv_t.element_size()
    ptrs = [qkv_t.data_ptr() + i * heads * t * d * es for i in range(3)]
    if dtype == torch.float16:
        plan = torch.zeros(int(lib().et_attention_plan_ints(batch, t)), dtype=torch.int32, device="cuda")
        ok(lib().et_attention_plan(iptr(idx["cu_seqlens"]), batch, t, iptr(plan), stream()))
        ok(lib().et_attention_tiles(ptrs[0], ptrs[1], ptrs[2], d, t * d, iptr(m_ctx), iptr(plan), batch, seq, t,
                                    heads, d, iptr(st), stream()))
    else:
        ok(lib().et_attention(DT[dtype], ptrs[0], ptrs[1], ptrs[2], d, t * d, iptr(m_ctx), iptr(idx["cu_seqlens"]),
                              batch, seq, t, heads, d, 1, iptr(st), stream()))
    torch.cuda.synchronize()
    assert int(st[0]) == 0
    cu = idx["cu_seqlens"].cpu().numpy()
    want = O.packed_attention((q.double() + bq.double()).cpu(), (k.double() + bk.double()).cpu(),
                              (v.double() + bv.double()).cpu(), cu, heads, d)
    tol = dict(rtol=4e-3, atol=4e-3) if dtype == torch.float16 else dict(rtol=2e-5, atol=2e-5)
    torch.testing.assert_close(r_ctx.double().cpu(), want, **tol)            # reference kernels vs oracle
    torch.testing.assert_close(m_ctx.double().cpu(), r_ctx.double().cpu(), **tol)   # ours vs reference kernels


def reference_kernel_chain(x_pad, mask_np, weights, heads, dtype):
    """The reference's three functors replayed on its own kernels in its own order
    (tf_op/bert_transformer_op.cu.cc:104-246, 266-331, 339-373); the cublasGemmEx /
    cublasGemmStridedBatchedEx calls are torch.matmul."""
    b, s, h = x_pad.shape
    d = h // heads
    prefix, t, bidx, widx, packed = ref_input_op(x_pad, mask_np)
    x = packed.reshape(b * s, h)[:t].contiguous()
    attr_mask = dev(W.attention_mask_from_input_mask(mask_np).astype(np.float32), dtype)
    wd = [dev(np.asarray(w, np.float32), dtype) for w in weights]
    for l in range(len(weights) // 16):
        w = wd[l * 16:(l + 1) * 16]
        q, k, v = (x @ w[0]).contiguous(), (x @ w[2]).contiguous(), (x @ w[4]).contiguous()
        qb, kb, vb = [torch.zeros(b, heads, s, d, dtype=dtype, device="cuda") for _ in range(3)]
        rok(ref().ref_add_qkv_bias_padding(DT[dtype], iptr(q), iptr(w[1]), iptr(k), iptr(w[3]), iptr(v), iptr(w[5]),
                                           iptr(qb), iptr(kb), iptr(vb), t, b, s, heads, d, iptr(bidx), iptr(widx),
                                           stream()))
        scores = torch.matmul(qb, kb.transpose(-1, -2)).contiguous()
        rok(ref().ref_softmax(DT[dtype], iptr(scores), iptr(attr_mask), b, heads, s, 1.0 / math.sqrt(d), stream()))
        ctx_pad = torch.matmul(scores, vb).contiguous()
        attr_out = torch.zeros(t, h, dtype=dtype, device="cuda")
        rok(ref().ref_transpose_rm_padding(DT[dtype], iptr(ctx_pad), iptr(attr_out), t, b, s, heads, d, iptr(bidx),
                                           iptr(widx), stream()))
        att = (attr_out @ w[6]).contiguous()
        rok(ref().ref_add_bias_input_layernorm(DT[dtype], iptr(att), iptr(x), iptr(w[7]), iptr(w[9]), iptr(w[8]),
                                               t, h, stream()))
        inter = (att @ w[10]).contiguous()
        rok(ref().ref_add_bias_act(DT[dtype], iptr(inter), iptr(w[11]), t, inter.shape[1], stream()))
        out = (inter @ w[12]).contiguous()
        rok(ref().ref_add_bias_input_layernorm(DT[dtype], iptr(out), iptr(att), iptr(w[13]), iptr(w[15]), iptr(w[14]),
                                               t, h, stream()))
        x = out
    full = torch.zeros(b, s, h, dtype=dtype, device="cuda")
    pk = torch.zeros(b * s, h, dtype=dtype, device="cuda")
    pk[:t] = x
    rok(ref().ref_restore_output(DT[dtype], iptr(full), iptr(pk), iptr(bidx), iptr(widx), t, s, h, stream()))
    torch.cuda.synchronize()
    return full


@pytest.mark.parametrize("cfg", [0, 1])
def test_whole_path_against_reference_kernel_chain(cfg):
    """12 BERT-base layers (cfg0 fp32, cfg1 fp16): reference kernels in the reference's
    order vs the CPU oracle vs this library's et_forward, on valid tokens."""
    import effective_transformer_b200 as et
    spec = W.WORKLOADS[cfg]
    wl = W.make_workload(spec)
    fp16 = spec.dtype == "fp16"
    dtype = torch.float16 if fp16 else torch.float32
    x = dev(wl.from_tensor, dtype)
    y_ref = reference_kernel_chain(x, wl.mask, wl.weights, spec.shape.head_num, dtype)
    am = W.attention_mask_from_input_mask(wl.mask)
    y_orc = O.valid_rows(O.transformer_model(wl.from_tensor, am, wl.weights, 12, 64, compute_dtype=torch.float64,
                                             round_to_fp16=fp16), wl.mask)
    sh = spec.shape
    eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, sh.size_per_head, sh.ffn_dim, spec.batch,
                                  spec.max_seq_len, dtype=dtype)
    eng.set_weights(wl.weights)
    y_me = eng.forward(x, dev(wl.mask))
    torch.cuda.synchronize()
    r = O.valid_rows(y_ref.cpu().double(), wl.mask)
    m = O.valid_rows(y_me.cpu().double(), wl.mask)
    d_ref, d_me, d_cross = (r - y_orc).abs(), (m - y_orc).abs(), (m - r).abs()
    if fp16:
        # this library against the oracle: the stated gate
        assert float(d_me.max()) <= 2e-2 and float(d_me.mean()) <= 2e-3, (float(d_me.max()), float(d_me.mean()))
        # The reference's half kernels round more often (fp16 bias adds and cube, Q/K/V written
        # before the bias): its own chain sits at the edge of that gate (measured max 2.1e-2, mean
        # 1.5e-3 on cfg1), so it is held to twice the gate, and this library must not be further
        # from the oracle than the reference's kernels are.
        assert float(d_ref.max()) <= 4e-2 and float(d_ref.mean()) <= 4e-3, (float(d_ref.max()), float(d_ref.mean()))
        assert float(d_cross.max()) <= 4e-2 and float(d_cross.mean()) <= 4e-3
        assert float(d_me.mean()) <= float(d_ref.mean())
    else:
        rms = float(y_orc.pow(2).mean().sqrt())
        for dd, what in ((d_ref, "reference kernels vs oracle"), (d_me, "this library vs oracle"),
                         (d_cross, "this library vs reference kernels")):
            assert float(dd.max()) <= 1e-4 * rms, (what, float(dd.max()), rms)
    pad = torch.from_numpy(wl.mask.ravel() == 0)
    assert torch.all(y_ref.cpu().reshape(-1, sh.hidden)[pad] == 0) and torch.all(y_me.cpu().reshape(-1, sh.hidden)[pad] == 0)
    eng.close()
