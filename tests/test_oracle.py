"""CPU tests: the oracle against the committed golden vectors, and the integer
oracle against first principles."""
import os

import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from effective_transformer_b200 import workloads as W
from oracle import bert_encoder as O
from oracle import padding as P

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_token_counts_match_fixture():
    d = np.load(os.path.join(GOLD, "token_counts.npz"))
    for spec in W.WORKLOADS:
        lens = W.draw_lengths(spec, np.random.RandomState(spec.seed))
        assert int(lens.sum()) == int(d[spec.name][0])
        assert int((lens.astype(np.int64) ** 2).sum()) == int(d[spec.name][1])
    assert int(d["cfg2_base_fp16_b1000_s64"][0]) == 39778


def test_tiny_oracle_matches_golden_and_independent_implementation():
    d = np.load(os.path.join(GOLD, "tiny_fp64.npz"))
    spec = W.tiny_spec()
    wl = W.make_workload(spec, random_gamma_beta=True)
    assert np.array_equal(wl.lengths, d["lengths"]) and np.array_equal(wl.mask, d["mask"])
    am = W.attention_mask_from_input_mask(wl.mask)
    stages = {}
    y = O.transformer_model(wl.from_tensor, am, wl.weights, spec.shape.head_num, spec.shape.size_per_head,
                            compute_dtype=torch.float64, layer0_stages=stages)
    yv = O.valid_rows(y, wl.mask).numpy()
    assert np.abs(yv - d["oracle64"]).max() < 1e-12
    assert np.abs(yv - d["independent"]).max() < 1e-12     # Hugging Face BertEncoder, float64
    for k, v in stages.items():
        assert np.abs(v.numpy() - d["stage_" + k]).max() < 1e-12
    # float32 evaluation (the timed CPU baseline) stays within 1e-4 * RMS of the float64 master
    y32 = O.transformer_model(wl.from_tensor, am, wl.weights, spec.shape.head_num, spec.shape.size_per_head,
                              compute_dtype=torch.float32)
    rms = float(np.sqrt((d["oracle64"] ** 2).mean()))
    assert np.abs(O.valid_rows(y32, wl.mask).numpy() - d["oracle64"]).max() < 1e-4 * rms


def test_cfg0_oracle_matches_golden():
    d = np.load(os.path.join(GOLD, "cfg0_fp64_subsampled.npz"))
    wl = W.make_workload(W.WORKLOADS[0])
    assert np.array_equal(wl.lengths, d["lengths"])
    am = W.attention_mask_from_input_mask(wl.mask)
    y = O.transformer_model(wl.from_tensor, am, wl.weights, 12, 64, compute_dtype=torch.float64)
    yv = O.valid_rows(y, wl.mask).numpy()[:, ::8]
    assert np.abs(yv - d["oracle64"]).max() < 1e-11
    assert np.abs(yv - d["independent"]).max() < 1e-11


def test_packed_encoder_equals_padded_encoder():
    """The padding-free formulation is the same function on valid tokens; the
    LayerNorm epsilon gap (1e-6 on the device vs 1e-12 in TF) is far inside tolerance."""
    spec = W.tiny_spec()
    wl = W.make_workload(spec, random_gamma_beta=True)
    am = W.attention_mask_from_input_mask(wl.mask)
    y = O.valid_rows(O.transformer_model(wl.from_tensor, am, wl.weights, 2, 64, compute_dtype=torch.float64),
                     wl.mask)
    idx = P.padding_indices(wl.mask)
    xp = P.remove_padding(wl.from_tensor, wl.mask)
    yp = O.packed_encoder(xp, idx["cu_seqlens"], wl.weights, 2, 64, compute_dtype=torch.float64,
                          ln_eps=O.TF_LAYER_NORM_EPS)
    assert float((y - yp).abs().max()) < 1e-10
    yp6 = O.packed_encoder(xp, idx["cu_seqlens"], wl.weights, 2, 64, compute_dtype=torch.float64,
                           ln_eps=O.DEVICE_LAYER_NORM_EPS)
    rms = float(y.pow(2).mean().sqrt())
    assert float((y - yp6).abs().max()) < 1e-5 * rms


def test_padding_indices_golden():
    d = np.load(os.path.join(GOLD, "tiny_fp64.npz"))
    idx = P.padding_indices(d["mask"])
    for k, v in idx.items():
        assert np.array_equal(v, d["idx_" + k]), k


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 6), st.integers(0, 70), st.integers(0, 2 ** 31 - 1))
def test_padding_indices_properties(b, s, seed):
    rng = np.random.RandomState(seed)
    mask = (rng.rand(b, s) < 0.6).astype(np.int32)     # arbitrary (non-prefix) masks are legal
    idx = P.padding_indices(mask)
    flat = mask.ravel()
    t = int(flat.sum())
    # exclusive scan, element by element
    run = 0
    for i, m in enumerate(flat):
        assert idx["prefix_sum"].ravel()[i] == run
        run += int(m)
    assert int(idx["valid_word_num"][0]) == t == idx["batch_idx"].size
    if s:
        pos = idx["batch_idx"].astype(np.int64) * s + idx["word_idx"]
        assert np.all(np.diff(pos) > 0) and np.all(flat[pos] == 1)
        assert np.array_equal(idx["padding_offset"], pos - np.arange(t))
    assert idx["cu_seqlens"][0] == 0 and idx["cu_seqlens"][-1] == t
    assert np.array_equal(np.diff(idx["cu_seqlens"]), idx["seq_len"])
    # remove -> restore round trip
    x = rng.randn(b, s, 8).astype(np.float32)
    back = P.restore_padding(P.remove_padding(x, mask), idx["batch_idx"], idx["word_idx"], b, s)
    assert np.array_equal(back, x * mask[:, :, None])


def test_valid_word_num_last_mask_rule():
    # exclusive scan + "last mask is 1" rule of the input functor
    assert P.valid_word_num(np.array([1, 0, 1, 1])) == 3
    assert P.valid_word_num(np.array([1, 0, 1, 0])) == 2
    assert P.valid_word_num(np.array([], dtype=np.int32)) == 0


def tiny_model_case():
    """The case of tests/golden/make_golden_heads.py (sequence 3 emptied)."""
    spec = W.tiny_spec()
    wl = W.make_workload(spec, random_gamma_beta=True)
    lengths = wl.lengths.copy()
    lengths[3] = 0
    mask = W.prefix_mask(lengths, spec.max_seq_len)
    heads = W.make_model_heads(spec, lengths, 1000, 2, 64)
    return spec, wl, lengths, mask, heads


def test_model_heads_oracle_matches_golden_and_independent_implementation():
    d = np.load(os.path.join(GOLD, "tiny_model_fp64.npz"))
    spec, wl, lengths, mask, heads = tiny_model_case()
    assert np.array_equal(mask, d["mask"]) and np.array_equal(heads.input_ids, d["input_ids"])
    assert np.array_equal(heads.token_type_ids, d["token_type_ids"])
    e, y, p = O.bert_model(heads, mask, wl.weights, spec.shape.head_num, spec.shape.size_per_head,
                           compute_dtype=torch.float64)
    for got, name in ((e.numpy(), "embedding"), (O.valid_rows(y, mask).numpy(), "sequence"), (p.numpy(), "pooled")):
        assert np.abs(got - d[name + "_oracle64"]).max() < 1e-12, name
        assert np.abs(got - d[name + "_independent"]).max() < 1e-12, name   # Hugging Face, float64


def test_embedding_stage_variants_and_pooler_of_empty_sequence():
    spec, wl, lengths, mask, heads = tiny_model_case()
    t = lambda a: torch.from_numpy(a).double()
    x = O.embedding_lookup(heads.input_ids, t(heads.word_table))
    full = O.embedding_postprocessor(x, heads.token_type_ids, t(heads.type_table), t(heads.position_table),
                                     t(heads.ln_gamma), t(heads.ln_beta))
    # hand-rolled row: word + type + position, then LN
    b, s = 1, 2
    row = (heads.word_table[heads.input_ids[b, s]].astype(np.float64)
           + heads.type_table[heads.token_type_ids[b, s]] + heads.position_table[s])
    row = (row - row.mean()) / np.sqrt(row.var() + 1e-12) * heads.ln_gamma + heads.ln_beta
    assert np.abs(full[b, s].numpy() - row).max() < 1e-12
    # use_token_type = False / use_position_embeddings = False drop exactly that term
    no_type = O.embedding_postprocessor(x, None, None, t(heads.position_table), t(heads.ln_gamma), t(heads.ln_beta))
    no_pos = O.embedding_postprocessor(x, heads.token_type_ids, t(heads.type_table), None, t(heads.ln_gamma),
                                       t(heads.ln_beta))
    assert not torch.allclose(no_type, full) and not torch.allclose(no_pos, full)
    # the zero-row variant: an empty sequence pools tanh(bias)
    _, _, pooled = O.bert_model(heads, mask, wl.weights, spec.shape.head_num, spec.shape.size_per_head,
                                compute_dtype=torch.float64, zero_padded_rows=True)
    assert np.abs(pooled[3].numpy() - np.tanh(heads.pooler_bias.astype(np.float64))).max() < 1e-12
    _, _, pooled_tf = O.bert_model(heads, mask, wl.weights, spec.shape.head_num, spec.shape.size_per_head,
                                   compute_dtype=torch.float64)
    keep = lengths > 0
    assert torch.equal(pooled[keep], pooled_tf[keep])
