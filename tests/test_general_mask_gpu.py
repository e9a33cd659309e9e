"""GPU tests of attention under a general [B, S, S] mask (causal, banded, random
per-pair, rows with nothing allowed, masks that let padded keys in), three ways
where the reference's kernels are available: the reference's own attention
chain (add_QKV_bias_padding, softmax_kernel, transpose_rm_padding compiled from
the reference checkout; the two batched GEMMs are torch.matmul), the CPU
oracle's restatement of that chain, and this library's packed kernel.
"""
import math
import os

import numpy as np
import pytest
import torch

import effective_transformer_b200 as et
from effective_transformer_b200 import _capi
from effective_transformer_b200 import workloads as W
from oracle import bert_encoder as O
from util import DT, dev, iptr, lib, ok, padding_offsets, stream

pytestmark = pytest.mark.gpu
REF_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                      "libet_ref_kernels.so")


def general_masks(mask_np: np.ndarray, rng) -> dict:
    """[B,S,S] float masks over a [B,S] input mask."""
    b, s = mask_np.shape
    key = np.tile(mask_np, s).reshape(b, s, s).astype(np.float32)
    causal = np.tril(np.ones((s, s), np.float32))[None] * key
    band = (np.abs(np.arange(s)[:, None] - np.arange(s)[None, :]) <= 3).astype(np.float32)[None] * key
    rand = (rng.rand(b, s, s) < 0.5).astype(np.float32) * key
    rand[:, np.arange(s), np.arange(s)] = key[:, 0, :]       # keep the diagonal of valid positions
    blocked = key.copy()
    blocked[:, 1, :] = 0                                      # query position 1 may attend to nothing
    leaky = np.ones((b, s, s), np.float32)                    # padded keys allowed: they count with K = V = 0
    return {"key_only": key, "causal": causal, "band": band, "random": rand, "blocked_row": blocked,
            "padded_keys_allowed": leaky}


def run_ours(dtype, q, k, v, attr, idx, batch, seq, heads):
    t, h = q.shape
    ctx = torch.full((t, h), float("nan"), dtype=dtype, device="cuda")
    scratch = torch.empty(batch * seq, dtype=torch.int32, device="cuda")
    ok(lib().et_attention_general_mask(DT[dtype], iptr(q), iptr(k), iptr(v), h, 64, iptr(ctx), iptr(attr),
                                       iptr(idx["cu_seqlens"]), iptr(idx["batch_idx"]), iptr(idx["word_idx"]),
                                       iptr(idx["valid_word_num"]), iptr(scratch), batch, seq, heads, 64, stream()))
    torch.cuda.synchronize()
    return ctx


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("prefix", [True, False], ids=["prefix_mask", "mask_with_holes"])
def test_general_mask_attention_three_ways(dtype, prefix):
    # seq = the reference softmax's block size: with idle threads its max reduction sees their
    # -1e-20 filler and a row with nothing allowed comes out as zeros instead of uniform
    batch, seq, heads, d = 5, 64, 3, 64
    h = heads * d
    rng = np.random.RandomState(21 + int(prefix))
    if prefix:
        lens = rng.randint(2, seq + 1, size=batch).astype(np.int32)
        lens[2] = 0
        mask_np = W.prefix_mask(lens, seq)
    else:
        mask_np = (rng.rand(batch, seq) < 0.7).astype(np.int32)
    idx = padding_offsets(dev(mask_np))
    t = int(idx["valid_word_num"][0])
    cu, widx = idx["cu_seqlens"].cpu().numpy(), idx["word_idx"].cpu().numpy()
    q, k, v = [dev(rng.randn(t, h).astype(np.float32), dtype) for _ in range(3)]
    have_ref = os.path.exists(REF_SO)
    if have_ref:
        from test_reference_kernels_gpu import ref, rok
    for name, m_np in general_masks(mask_np, rng).items():
        attr = dev(m_np, dtype)
        got = run_ours(dtype, q, k, v, attr, idx, batch, seq, heads)
        want = O.packed_attention_general_mask(q.double().cpu(), k.double().cpu(), v.double().cpu(), cu, widx,
                                               torch.from_numpy(m_np).double(), seq, heads, d)
        tol = dict(rtol=4e-3, atol=4e-3) if dtype == torch.float16 else dict(rtol=2e-5, atol=2e-5)
        if name == "blocked_row" and dtype == torch.float32:
            # score - 10000 in fp32 keeps 1e-3 of the score (as in the reference and in TF): the
            # weights of the all-masked row carry that rounding, the float64 oracle does not
            tol = dict(rtol=2e-3, atol=2e-3)
        torch.testing.assert_close(got.double().cpu(), want, msg=lambda s: f"{name}: ours vs oracle\n{s}", **tol)
        if name == "key_only":                               # the fast path's own semantics
            plain = O.packed_attention(q.double().cpu(), k.double().cpu(), v.double().cpu(), cu, heads, d)
            torch.testing.assert_close(want, plain, rtol=1e-9, atol=1e-9)
        if not have_ref:
            continue
        zero_bias = torch.zeros(h, dtype=dtype, device="cuda")
        qb, kb, vb = [torch.zeros(batch, heads, seq, d, dtype=dtype, device="cuda") for _ in range(3)]
        rok(ref().ref_add_qkv_bias_padding(DT[dtype], iptr(q), iptr(zero_bias), iptr(k),
                                           iptr(zero_bias), iptr(v), iptr(zero_bias), iptr(qb), iptr(kb),
                                           iptr(vb), t, batch, seq, heads, d, iptr(idx["batch_idx"]),
                                           iptr(idx["word_idx"]), stream()))
        scores = torch.matmul(qb, kb.transpose(-1, -2)).contiguous()
        rok(ref().ref_softmax(DT[dtype], iptr(scores), iptr(attr), batch, heads, seq, 1.0 / math.sqrt(d), stream()))
        ctx_pad = torch.matmul(scores, vb).contiguous()
        r_ctx = torch.zeros(t, h, dtype=dtype, device="cuda")
        rok(ref().ref_transpose_rm_padding(DT[dtype], iptr(ctx_pad), iptr(r_ctx), t, batch, seq, heads, d,
                                           iptr(idx["batch_idx"]), iptr(idx["word_idx"]), stream()))
        torch.cuda.synchronize()
        r64, g64, keep = r_ctx.double().cpu(), got.double().cpu(), torch.ones(t, dtype=torch.bool)
        if name == "blocked_row":
            # Where a query may attend to nothing every score is about -10000.  The reference's
            # blockReduceMax pads idle lanes with 0 (cuda/attention.cu:90), so its maximum is 0, every
            # exp underflows and the row comes out as 0 / 1e-6 = 0; the TF graph (and this library)
            # give the uniform average that softmax defines.  Checked as what it is.
            keep = torch.from_numpy(widx[:t] != 1)
            assert bool((r64[~keep] == 0).all())
        torch.testing.assert_close(r64[keep], want[keep], msg=lambda s: f"{name}: reference vs oracle\n{s}", **tol)
        torch.testing.assert_close(g64[keep], r64[keep], msg=lambda s: f"{name}: ours vs reference\n{s}", **tol)


@pytest.mark.parametrize("dtype", ["fp32", "fp16"])
def test_whole_path_under_a_general_mask(dtype):
    """Causal mask over the tiny model: forward_general_mask and the op-by-op wiring
    with set_general_mask against the packed oracle, which itself equals the padded
    TF-graph restatement when no padded key is let in."""
    spec = W.tiny_spec(dtype=dtype)
    wl = W.make_workload(spec, random_gamma_beta=True)
    sh = spec.shape
    b, s = wl.mask.shape
    tdt = torch.float16 if dtype == "fp16" else torch.float32
    causal = np.tril(np.ones((s, s), np.float32))[None] * W.attention_mask_from_input_mask(wl.mask)
    y_pad = O.transformer_model(wl.from_tensor, causal, wl.weights, sh.head_num, sh.size_per_head,
                                compute_dtype=torch.float64, round_to_fp16=(dtype == "fp16"))
    want = O.valid_rows(y_pad, wl.mask)
    # the packed oracle with the op's semantics gives the same rows (up to the LayerNorm epsilons)
    from oracle import padding as P
    pidx = P.padding_indices(wl.mask)
    x_valid = O.valid_rows(torch.from_numpy(wl.from_tensor), wl.mask)
    cu = np.concatenate([[0], np.cumsum(wl.lengths)]).astype(np.int32)
    y_packed = O.packed_encoder(x_valid, cu, wl.weights, sh.head_num, sh.size_per_head, compute_dtype=torch.float64,
                                round_to_fp16=(dtype == "fp16"), ln_eps=1e-12, attr_mask=causal,
                                word_idx=pidx["word_idx"], seq=s)
    assert float((y_packed - want).abs().max()) < 1e-9

    eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, sh.size_per_head, sh.ffn_dim, b, s, dtype=tdt)
    eng.set_weights(wl.weights)
    x = torch.from_numpy(wl.from_tensor).to(tdt).cuda()
    m = torch.from_numpy(wl.mask).cuda()
    am = torch.from_numpy(causal).to(tdt).cuda()
    y = eng.forward_general_mask(x, m, am)
    torch.cuda.synchronize()

    def check(y_dev):
        diff = (O.valid_rows(y_dev.cpu().double(), wl.mask) - want).abs()
        if dtype == "fp16":
            assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3
        else:
            assert float(diff.max()) <= 1e-4 * float(want.pow(2).mean().sqrt())
    check(y)
    # a causal mask must change the result with respect to the key-only mask
    assert not torch.equal(y, eng.forward(x, m))
    # op by op, as python/effective_transformer/__init__.py:42-82 wires it
    eng.set_general_mask(True)
    cfg = et.BertConfig(sh.hidden, sh.num_layers, sh.head_num, sh.ffn_dim)
    y_ops = et.get_sequence_output(cfg, b, s, am, m, x, wl.weights, engine=eng)
    assert torch.equal(y_ops, y)
    with pytest.raises(et.EtError) as e:
        et.get_sequence_output(cfg, b, s, None, m, x, wl.weights, engine=eng)
    assert e.value.code == _capi.ET_INVALID_ARGUMENT         # general-mask mode needs the mask
    eng.set_general_mask(False)
    assert torch.equal(et.get_sequence_output(cfg, b, s, None, m, x, wl.weights, engine=eng), eng.forward(x, m))
    eng.close()


@pytest.mark.parametrize("prefix", [True, False], ids=["prefix_mask", "mask_with_holes"])
@pytest.mark.parametrize("seq", [64, 128, 40])
def test_general_mask_attention_on_tensor_cores(prefix, seq):
    """et_attention_tiles_general_mask (the packed-tile tcgen05 kernel reading the mask per query and
    key) against the oracle's restatement of the reference op's masked attention, for every kind of
    mask, and against the CUDA-core general-mask kernel."""
    batch, heads, d = 9, 3, 64
    h = heads * d
    rng = np.random.RandomState(5 + seq + int(prefix))
    if prefix:
        lens = rng.randint(1, seq + 1, size=batch).astype(np.int32)
        lens[2] = 0
        lens[5] = seq
        mask_np = W.prefix_mask(lens, seq)
    else:
        mask_np = (rng.rand(batch, seq) < 0.7).astype(np.int32)
    idx = padding_offsets(dev(mask_np))
    t = int(idx["valid_word_num"][0])
    cu, widx = idx["cu_seqlens"].cpu().numpy(), idx["word_idx"].cpu().numpy()
    dtype = torch.float16
    qkv = dev(rng.randn(t + 5, 3 * h).astype(np.float32), dtype)
    q, k, v = qkv[:, :h], qkv[:, h:2 * h], qkv[:, 2 * h:]
    cap = t + 5
    plan = torch.zeros(int(lib().et_attention_plan_ints(batch, cap)), dtype=torch.int32, device="cuda")
    ok(lib().et_attention_plan(iptr(idx["cu_seqlens"]), batch, cap, iptr(plan), stream()))
    e = qkv.element_size()
    for name, m_np in general_masks(mask_np, rng).items():
        attr = dev(m_np, dtype)
        ctx = torch.full((cap, h), 2.0, dtype=dtype, device="cuda")
        st = torch.zeros(1, dtype=torch.int32, device="cuda")
        ok(lib().et_attention_tiles_general_mask(qkv.data_ptr(), qkv.data_ptr() + h * e, qkv.data_ptr() + 2 * h * e,
                                                 3 * h, 64, iptr(ctx), iptr(plan), iptr(attr), iptr(idx["batch_idx"]),
                                                 iptr(idx["word_idx"]), batch, seq, cap, heads, 64, iptr(st), stream()))
        torch.cuda.synchronize()
        assert int(st[0]) == 0
        want = O.packed_attention_general_mask(q[:t].double().cpu(), k[:t].double().cpu(), v[:t].double().cpu(), cu,
                                               widx, torch.from_numpy(m_np).double(), seq, heads, d)
        torch.testing.assert_close(ctx[:t].double().cpu(), want, rtol=4e-3, atol=4e-3,
                                   msg=lambda s: f"{name}: tensor-core kernel vs oracle\n{s}")
        assert torch.all(ctx[t:] == 2.0)
        simt = run_ours(dtype, q[:t].contiguous(), k[:t].contiguous(), v[:t].contiguous(), attr, idx, batch, seq, heads)
        torch.testing.assert_close(ctx[:t].float(), simt.float(), rtol=4e-3, atol=4e-3,
                                   msg=lambda s: f"{name}: tensor-core vs CUDA-core kernel\n{s}")
