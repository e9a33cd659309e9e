"""Weight loading by name (effective_transformer_b200/checkpoint.py): TF variable
names and Hugging Face state dicts -> the positional 16-per-layer order of
python/effective_transformer/__init__.py:55-74.  The mapping is pinned by running
a Hugging Face BertModel and the oracle / the GPU library on the converted weights."""
import numpy as np
import pytest
import torch

from effective_transformer_b200 import checkpoint as CK
from effective_transformer_b200 import workloads as W
from oracle import bert_encoder as O


def hf_model(layers=2, heads=2, ffn=256, vocab=500, positions=40, seed=0):
    from transformers import BertConfig, BertModel
    torch.manual_seed(seed)
    cfg = BertConfig(vocab_size=vocab, hidden_size=heads * 64, num_hidden_layers=layers, num_attention_heads=heads,
                     intermediate_size=ffn, max_position_embeddings=positions, type_vocab_size=2,
                     hidden_act="gelu_new", hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                     layer_norm_eps=1e-12)
    cfg._attn_implementation = "eager"
    m = BertModel(cfg).eval()
    with torch.no_grad():                                    # LayerNorm defaults are 1/0: make them matter
        for name, p in m.named_parameters():
            if "LayerNorm" in name:
                p.add_(0.1 * torch.randn_like(p))
    return m, cfg


def inputs(cfg, batch=4, seq=10, seed=1):
    rng = np.random.RandomState(seed)
    lengths = rng.randint(1, seq + 1, size=batch).astype(np.int32)
    lengths[0] = seq
    mask = W.prefix_mask(lengths, seq)
    ids = rng.randint(0, cfg.vocab_size, size=(batch, seq)).astype(np.int32)
    types = (rng.rand(batch, seq) < 0.5).astype(np.int32)
    return lengths, mask, ids, types


def as_heads(tables: CK.ModelTables, ids, types) -> W.ModelHeads:
    return W.ModelHeads(ids, types, tables.word_table, tables.type_table, tables.position_table, tables.ln_gamma,
                        tables.ln_beta, tables.pooler_kernel, tables.pooler_bias)


def test_tf_names_round_trip_and_errors():
    spec = W.tiny_spec()
    wl = W.make_workload(spec)
    heads = W.make_model_heads(spec, wl.lengths, 100, 2, 16)
    tables = CK.ModelTables(heads.word_table, heads.type_table, heads.position_table, heads.ln_gamma, heads.ln_beta,
                            heads.pooler_kernel, heads.pooler_bias)
    named = CK.to_tf_variables(wl.weights, tables)
    assert "bert/encoder/layer_1/attention/output/LayerNorm/gamma" in named
    assert "bert/embeddings/word_embeddings" in named and "bert/pooler/dense/kernel" in named
    assert len(CK.tf_variable_names(2)) == 32
    # ":0" suffixes and an unrelated variable are tolerated
    named2 = {k + ":0": v for k, v in named.items()}
    named2["global_step:0"] = np.zeros(1)
    w2, t2 = CK.weights_from_tf_variables(named2)
    assert len(w2) == len(wl.weights) and all(np.array_equal(a, b) for a, b in zip(w2, wl.weights))
    assert np.array_equal(t2.word_table, heads.word_table) and np.array_equal(t2.pooler_bias, heads.pooler_bias)
    # slot order: index 8 is the attention LayerNorm beta, 9 its gamma
    assert np.array_equal(w2[16 + 8], named["bert/encoder/layer_1/attention/output/LayerNorm/beta"])
    assert np.array_equal(w2[16 + 9], named["bert/encoder/layer_1/attention/output/LayerNorm/gamma"])
    missing = dict(named)
    del missing["bert/encoder/layer_0/intermediate/dense/bias"]
    with pytest.raises(KeyError):
        CK.weights_from_tf_variables(missing)
    bad = dict(named)
    bad["bert/encoder/layer_0/output/dense/kernel"] = bad["bert/encoder/layer_0/output/dense/kernel"].T
    with pytest.raises(ValueError):
        CK.weights_from_tf_variables(bad)
    # encoder-only checkpoints (no embeddings, no pooler) give empty tables
    enc_only = {k: v for k, v in named.items() if "/encoder/" in k}
    _, t3 = CK.weights_from_tf_variables(enc_only)
    assert t3.word_table is None and t3.pooler_kernel is None


def test_hf_state_dict_maps_onto_the_oracle():
    model, cfg = hf_model()
    lengths, mask, ids, types = inputs(cfg)
    weights, tables = CK.weights_from_hf_state_dict(model.double().state_dict())
    assert len(weights) == 32 and weights[10].shape == (128, 256)     # intermediate kernel is [in, out]
    with torch.no_grad():
        out = model(input_ids=torch.from_numpy(ids.astype(np.int64)),
                    attention_mask=torch.from_numpy(mask.astype(np.int64)),
                    token_type_ids=torch.from_numpy(types.astype(np.int64)))
    emb, seq, pooled = O.bert_model(as_heads(tables, ids, types), mask, weights, cfg.num_attention_heads, 64,
                                    compute_dtype=torch.float64)
    got, want = O.valid_rows(seq, mask), O.valid_rows(out.last_hidden_state, mask)
    assert float((got - want).abs().max()) < 1e-9
    assert float((pooled - out.pooler_output).abs().max()) < 1e-9
    # and through the TF naming
    w_tf, t_tf = CK.weights_from_tf_variables(CK.to_tf_variables(weights, tables))
    assert all(np.array_equal(a, b) for a, b in zip(w_tf, weights))
    assert np.array_equal(t_tf.position_table, tables.position_table)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_gpu_library_reproduces_a_hugging_face_bert_model(dtype):
    import effective_transformer_b200 as et
    model, cfg = hf_model(layers=3, heads=4, ffn=512, vocab=800, positions=64, seed=3)
    lengths, mask, ids, types = inputs(cfg, batch=9, seq=33, seed=4)
    if dtype == torch.float16:
        model = model.half().float()                         # the values the fp16 handle will hold
    weights, tables = CK.weights_from_hf_state_dict(model.state_dict())
    with torch.no_grad():
        ref = model.double()(input_ids=torch.from_numpy(ids.astype(np.int64)),
                             attention_mask=torch.from_numpy(mask.astype(np.int64)),
                             token_type_ids=torch.from_numpy(types.astype(np.int64)))
    eng = et.EffectiveTransformer(cfg.num_hidden_layers, cfg.num_attention_heads, 64, cfg.intermediate_size, 9, 33,
                                  dtype=dtype)
    CK.load_engine_weights(eng, weights, tables)
    seq, pooled = eng.forward_ids(torch.from_numpy(ids).cuda(), torch.from_numpy(mask).cuda(),
                                  torch.from_numpy(types).cuda(), sequence_output=True, pooled_output=True)
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    for got, want in ((O.valid_rows(seq.cpu().double(), mask), O.valid_rows(ref.last_hidden_state, mask)),
                      (pooled.cpu().double(), ref.pooler_output)):
        diff = (got - want).abs()
        if dtype == torch.float16:
            assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3, (float(diff.max()), float(diff.mean()))
        else:
            assert float(diff.max()) <= 1e-4 * float(want.pow(2).mean().sqrt()), float(diff.max())
    eng.close()
