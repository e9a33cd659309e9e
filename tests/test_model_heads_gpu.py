"""GPU parity tests of the stages either side of the encoder stack on the packed
layout: embedding lookup + token-type/position rows + LayerNorm for valid tokens
only (sample/tensorflow/modeling.py:380-521), the pooler (modeling.py:224-232),
and the model call from token ids that strings them around the stack.

Tolerances: the embedding stage is one LayerNorm of a three-term sum, so it is
held to one rounding of the storage type (fp32: 2e-6 * max|ref|, fp16: 1 fp16
ulp of the value + fp32 noise); model outputs use the gates of the stack
(fp32: 1e-4 * RMS, fp16: max 2e-2 / mean 2e-3).
"""
import os

import numpy as np
import pytest
import torch

import effective_transformer_b200 as et
from effective_transformer_b200 import _capi
from effective_transformer_b200 import workloads as W
from oracle import bert_encoder as O
from util import DT, dev, iptr, lib, ok, padding_offsets, status_word, stream

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FP32_REL_RMS = 1e-4
FP16_MAX_ABS, FP16_MEAN_ABS = 2e-2, 2e-3


def tiny_model_case(dtype="fp32"):
    spec = W.tiny_spec(dtype=dtype)
    wl = W.make_workload(spec, random_gamma_beta=True)
    lengths = wl.lengths.copy()
    lengths[3] = 0
    mask = W.prefix_mask(lengths, spec.max_seq_len)
    heads = W.make_model_heads(spec, lengths, 1000, 2, 64)
    return spec, wl, lengths, mask, heads


def oracle_embedding(heads, tdt, type_table=True, pos_table=True, eps=1e-12, ids=None, types=None):
    """float64 oracle on the values as stored in the tables' dtype."""
    r = lambda a: torch.from_numpy(a).to(tdt).double()
    ids = heads.input_ids if ids is None else ids
    x = O.embedding_lookup(ids, r(heads.word_table))
    return O.embedding_postprocessor(
        x, heads.token_type_ids if types is None else types, r(heads.type_table) if type_table else None,
        r(heads.position_table) if pos_table else None, r(heads.ln_gamma), r(heads.ln_beta), eps)


def run_embedding(heads, mask, tdt, use_types=True, type_table=True, pos_table=True, eps=1e-12, ids=None):
    b, s = mask.shape
    h = heads.word_table.shape[1]
    idx = padding_offsets(dev(mask))
    out = torch.full((max(b * s, 1), h), float("nan"), dtype=tdt, device="cuda")
    d = lambda a: dev(a, tdt)
    word, typ, pos = d(heads.word_table), d(heads.type_table), d(heads.position_table)
    g, be = d(heads.ln_gamma), d(heads.ln_beta)
    ids_d = dev(heads.input_ids if ids is None else ids)
    types_d = dev(heads.token_type_ids)
    ok(lib().et_embedding_layernorm(
        DT[tdt], iptr(ids_d), iptr(types_d) if use_types else None, iptr(idx["batch_idx"]), iptr(idx["word_idx"]),
        iptr(idx["valid_word_num"]), iptr(word), word.shape[0], iptr(typ) if type_table else None, typ.shape[0],
        iptr(pos) if pos_table else None, iptr(g), iptr(be), eps, iptr(out), b, s, h, stream()))
    torch.cuda.synchronize()
    return out, int(idx["valid_word_num"].item())


def assert_embedding_close(got: torch.Tensor, ref: torch.Tensor, tdt):
    diff = (got.double().cpu() - ref).abs()
    if tdt == torch.float32:
        assert float(diff.max()) <= 2e-6 * float(ref.abs().max()), float(diff.max())
    else:
        # one fp16 rounding of the result (relative 2^-11) plus fp32 evaluation noise
        bound = ref.abs() * 2.0 ** -11 + 1e-5
        assert bool((diff <= bound).all()), float((diff - bound).max())


@pytest.mark.parametrize("tdt", [torch.float32, torch.float16])
@pytest.mark.parametrize("variant", ["full", "no_type_ids", "no_type_table", "no_position"])
def test_embedding_layernorm_packed_matches_oracle(tdt, variant):
    spec, wl, lengths, mask, heads = tiny_model_case()
    kw = dict(use_types=variant != "no_type_ids", type_table=variant != "no_type_table",
              pos_table=variant != "no_position")
    out, t = run_embedding(heads, mask, tdt, **kw)
    assert t == int(lengths.sum())
    types = np.zeros_like(heads.token_type_ids) if variant == "no_type_ids" else None
    ref = oracle_embedding(heads, tdt, kw["type_table"], kw["pos_table"], types=types)
    assert_embedding_close(out[:t], O.valid_rows(ref, mask), tdt)
    assert bool(torch.isnan(out[t:].float()).all())          # rows past T are not touched


@pytest.mark.parametrize("tdt", [torch.float32, torch.float16])
def test_embedding_bert_base_width_and_device_eps(tdt):
    spec = W.WORKLOADS[1]
    lengths = W.draw_lengths(spec, np.random.RandomState(spec.seed))
    mask = W.prefix_mask(lengths, spec.max_seq_len)
    heads = W.make_model_heads(spec, lengths, vocab_size=4000)
    out, t = run_embedding(heads, mask, tdt, eps=1e-6)
    ref = oracle_embedding(heads, tdt, eps=1e-6)
    assert_embedding_close(out[:t], O.valid_rows(ref, mask), tdt)


def test_embedding_out_of_range_ids_contribute_zero_rows():
    spec, wl, lengths, mask, heads = tiny_model_case()
    ids = heads.input_ids.copy()
    ids[0, 0], ids[1, 1] = -5, 1000                          # below and past the 1000-row table
    out, t = run_embedding(heads, mask, torch.float32, ids=ids)
    safe = np.clip(ids, 0, 999)
    r = lambda a: torch.from_numpy(a).double()
    x = O.embedding_lookup(safe, r(heads.word_table))
    x[0, 0] = 0
    x[1, 1] = 0
    ref = O.embedding_postprocessor(x, heads.token_type_ids, r(heads.type_table), r(heads.position_table),
                                    r(heads.ln_gamma), r(heads.ln_beta))
    assert_embedding_close(out[:t], O.valid_rows(ref, mask), torch.float32)


def test_embedding_empty_batch_and_all_padding():
    spec, wl, lengths, mask, heads = tiny_model_case()
    zero_mask = np.zeros_like(mask)
    out, t = run_embedding(heads, zero_mask, torch.float16)
    assert t == 0 and bool(torch.isnan(out.float()).all())
    empty = W.make_model_heads(spec, np.zeros(0, np.int32), 1000, 2, 64)
    out, t = run_embedding(empty, np.zeros((0, spec.max_seq_len), np.int32), torch.float16)
    assert t == 0


@pytest.mark.parametrize("tdt", [torch.float32, torch.float16])
def test_gather_first_tokens_bit_exact(tdt):
    rng = np.random.RandomState(5)
    lengths = np.array([3, 0, 1, 7, 0, 0, 2], np.int32)
    cu = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    t, h = int(cu[-1]), 128
    packed = dev(rng.randn(t, h).astype(np.float32), tdt)
    out = torch.full((len(lengths), h), float("nan"), dtype=tdt, device="cuda")
    ok(lib().et_gather_first_tokens(DT[tdt], iptr(packed), iptr(dev(cu)), iptr(out), len(lengths), t, h, stream()))
    torch.cuda.synchronize()
    for b, n in enumerate(lengths):
        want = packed[cu[b]] if n > 0 else torch.zeros(h, dtype=tdt, device="cuda")
        assert torch.equal(out[b], want)


@pytest.mark.parametrize("tdt,use_simt", [(torch.float32, 1), (torch.float16, 1), (torch.float16, 0)])
def test_gemm_bias_tanh_epilogue(tdt, use_simt):
    rng = np.random.RandomState(11)
    m, n, k = 300, 256, 384
    a = dev(rng.randn(m, k).astype(np.float32), tdt)
    w = dev((0.05 * rng.randn(k, n)).astype(np.float32), tdt)
    bias = dev((0.1 * rng.randn(n)).astype(np.float32), tdt)
    wp = torch.empty((n, k), dtype=tdt, device="cuda")
    ok(lib().et_pack_weight(DT[tdt], iptr(w), iptr(wp), k, n, stream()))
    c = torch.empty((m, n), dtype=tdt, device="cuda")
    st = status_word()
    ok(lib().et_gemm(DT[tdt], iptr(a), iptr(w), iptr(wp), iptr(bias), iptr(c), iptr(dev(np.array([m], np.int32))),
                     m, n, k, 3, use_simt, iptr(st), stream()))
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    ref = torch.tanh(a.double().cpu() @ w.double().cpu() + bias.double().cpu())
    diff = (c.double().cpu() - ref).abs()
    assert float(diff.max()) <= (2e-5 if tdt == torch.float32 else 1.5e-3), float(diff.max())
    # an epilogue value past the last one is rejected
    assert lib().et_gemm(DT[tdt], iptr(a), iptr(w), iptr(wp), iptr(bias), iptr(c),
                         iptr(dev(np.array([m], np.int32))), m, n, k, 4, use_simt, iptr(st),
                         stream()) == _capi.ET_INVALID_ARGUMENT


def make_model_engine(spec, wl, heads, batch, simt=False):
    tdt = torch.float16 if spec.dtype == "fp16" else torch.float32
    sh = spec.shape
    eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, sh.size_per_head, sh.ffn_dim, batch,
                                  spec.max_seq_len, dtype=tdt)
    eng.set_weights(wl.weights)
    eng.set_embeddings(heads.word_table, heads.type_table, heads.position_table, heads.ln_gamma, heads.ln_beta)
    eng.set_pooler(heads.pooler_kernel, heads.pooler_bias)
    if simt:
        eng.set_debug_simt(True)
    return eng


def assert_model_parity(seq, pooled, ref_seq_valid, ref_pooled, mask, fp16):
    got = O.valid_rows(seq.detach().cpu().double(), mask)
    for g, r in ((got, ref_seq_valid.double()), (pooled.detach().cpu().double(), ref_pooled.double())):
        diff = (g - r).abs()
        if fp16:
            assert float(diff.max()) <= FP16_MAX_ABS and float(diff.mean()) <= FP16_MEAN_ABS, \
                (float(diff.max()), float(diff.mean()))
        else:
            rms = float(r.pow(2).mean().sqrt())
            assert float(diff.max()) <= FP32_REL_RMS * rms, (float(diff.max()), rms)
    b, s, h = seq.shape
    pad = torch.from_numpy(mask.ravel() == 0)
    assert torch.all(seq.detach().cpu().reshape(b * s, h)[pad] == 0)


@pytest.mark.parametrize("dtype,simt", [("fp32", False), ("fp32", True), ("fp16", True), ("fp16", False)])
def test_forward_ids_tiny_against_golden(dtype, simt):
    d = np.load(os.path.join(GOLD, "tiny_model_fp64.npz"))
    spec, wl, lengths, mask, heads = tiny_model_case(dtype)
    eng = make_model_engine(spec, wl, heads, mask.shape[0], simt)
    seq, pooled = eng.forward_ids(dev(heads.input_ids), dev(mask), dev(heads.token_type_ids),
                                  sequence_output=True, pooled_output=True)
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    sh = spec.shape
    if dtype == "fp32":
        ref_seq, ref_pool = torch.from_numpy(d["sequence_oracle64"]), torch.from_numpy(d["pooled_oracle64"]).clone()
    else:
        _, y, p = O.bert_model(heads, mask, wl.weights, sh.head_num, sh.size_per_head,
                               compute_dtype=torch.float64, round_to_fp16=True)
        ref_seq, ref_pool = O.valid_rows(y, mask), p
    # a sequence without tokens pools a zero first-token row: tanh(bias)
    ref_pool = ref_pool.clone()
    bias = torch.from_numpy(heads.pooler_bias)
    ref_pool[3] = torch.tanh((bias.half() if dtype == "fp16" else bias).double())
    assert_model_parity(seq, pooled, ref_seq, ref_pool, mask, dtype == "fp16")
    eng.close()


@pytest.mark.parametrize("cfg", [1, 2])
def test_forward_ids_equals_embedding_then_forward_bit_for_bit(cfg):
    """Size-independent property at the benchmark sizes: the model call from ids is
    the embedding kernel, the stack and the pooler on the same packed rows, so it
    must reproduce the three-step composition exactly."""
    spec = W.WORKLOADS[cfg]
    wl = W.make_workload(spec)
    heads = W.make_model_heads(spec, wl.lengths)
    eng = make_model_engine(spec, wl, heads, spec.batch)
    ids, mask, types = dev(heads.input_ids), dev(wl.mask), dev(heads.token_type_ids)
    seq, pooled = eng.forward_ids(ids, mask, types, sequence_output=True, pooled_output=True)
    torch.cuda.synchronize()
    # composition: packed embedding -> padded tensor -> forward (input op, stack, output op) -> pooler
    emb_packed, t = run_embedding(heads, wl.mask, torch.float16)
    assert t == wl.valid_tokens
    idx = padding_offsets(mask)
    b, s, h = spec.batch, spec.max_seq_len, spec.shape.hidden
    padded = torch.empty((b, s, h), dtype=torch.float16, device="cuda")
    ok(lib().et_restore_padding(_capi.ET_FP16, iptr(emb_packed), iptr(idx["batch_idx"]), iptr(idx["word_idx"]),
                                iptr(idx["valid_word_num"]), iptr(padded), b, s, h, stream()))
    seq2 = eng.forward(padded, mask)
    packed = torch.empty((b * s, h), dtype=torch.float16, device="cuda")
    ok(lib().et_remove_padding(_capi.ET_FP16, iptr(seq2), iptr(idx["batch_idx"]), iptr(idx["word_idx"]),
                               iptr(idx["valid_word_num"]), iptr(packed), b, s, h, stream()))
    pooled2 = eng.pooler(packed, b, s, idx["cu_seqlens"])
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    assert torch.equal(seq, seq2)
    assert torch.equal(pooled, pooled2)
    # first-token rule against the padded tensor, the way the reference's graph slices it
    first = seq[:, 0, :].double().cpu()
    ref = torch.tanh(first @ torch.from_numpy(heads.pooler_kernel).half().double()
                     + torch.from_numpy(heads.pooler_bias).half().double())
    assert float((pooled.double().cpu() - ref).abs().max()) <= 2e-3
    eng.close()


def test_forward_ids_host_equals_device_call_and_outputs_are_optional():
    spec = W.WORKLOADS[1]
    wl = W.make_workload(spec)
    heads = W.make_model_heads(spec, wl.lengths)
    eng = make_model_engine(spec, wl, heads, spec.batch)
    seq, pooled = eng.forward_ids(dev(heads.input_ids), dev(wl.mask), dev(heads.token_type_ids), True, True)
    torch.cuda.synchronize()
    seq_h, pooled_h, t = eng.forward_ids_host(heads.input_ids, wl.mask, heads.token_type_ids, True, True)
    assert t == wl.valid_tokens
    assert np.array_equal(seq_h, seq.cpu().numpy()) and np.array_equal(pooled_h, pooled.cpu().numpy())
    none_seq, pooled_only, t = eng.forward_ids_host(heads.input_ids, wl.mask, heads.token_type_ids, False, True)
    assert none_seq is None and np.array_equal(pooled_only, pooled_h)
    # token_type_ids omitted = all zero (modeling.py:159-160)
    seq0, _ = eng.forward_ids(dev(heads.input_ids), dev(wl.mask), None, True, False)
    seq0b, _ = eng.forward_ids(dev(heads.input_ids), dev(wl.mask), dev(np.zeros_like(heads.token_type_ids)), True, False)
    torch.cuda.synchronize()
    assert torch.equal(seq0, seq0b) and not torch.equal(seq0, seq)
    eng.close()


def test_model_call_errors():
    spec, wl, lengths, mask, heads = tiny_model_case("fp16")
    sh = spec.shape
    eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, sh.size_per_head, sh.ffn_dim, 5, spec.max_seq_len,
                                  dtype=torch.float16)
    eng.set_weights(wl.weights)
    ids, m = dev(heads.input_ids), dev(mask)
    with pytest.raises(et.EtError) as e:
        eng.forward_ids(ids, m)
    assert e.value.code == _capi.ET_NOT_READY               # no embedding tables yet
    eng.set_embeddings(heads.word_table, heads.type_table, heads.position_table[:8], heads.ln_gamma, heads.ln_beta)
    with pytest.raises(et.EtError) as e:
        eng.forward_ids(ids, m)                              # S = 12 > 8 position rows (modeling.py:487)
    assert e.value.code == _capi.ET_INVALID_ARGUMENT
    eng.set_embeddings(heads.word_table, heads.type_table, heads.position_table, heads.ln_gamma, heads.ln_beta)
    with pytest.raises(et.EtError) as e:
        eng.forward_ids(ids, m, pooled_output=True)
    assert e.value.code == _capi.ET_NOT_READY               # no pooler weights yet
    seq, _ = eng.forward_ids(ids, m)
    torch.cuda.synchronize()
    assert bool(torch.isfinite(seq.float()).all())
    with pytest.raises(ValueError):
        eng.set_pooler(heads.pooler_kernel[:, :64], heads.pooler_bias)
    eng.close()
