"""Generates tiny_model_fp64.npz: the stages either side of the encoder stack
(embedding lookup + token-type and position rows + LayerNorm,
sample/tensorflow/modeling.py:380-521, and the pooler, modeling.py:224-232).
Run from the repository root:  python tests/golden/make_golden_heads.py

Two sources per tensor, as in make_golden.py:
  * ``oracle64``      - oracle/bert_encoder.py (bert_model) in float64;
  * ``independent``   - Hugging Face ``transformers`` BertEmbeddings, BertEncoder
    and BertPooler in float64 with the same seeded tables and weights.
The case: the "tiny" architecture (2 layers, 2 heads x 64, FFN 256, B=5, S=12)
with a 1000-word vocabulary, 2 token types and 64 positions.  Sequence 3 is
made empty so that the first-token rule for a sequence without tokens is part
of the fixture.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from effective_transformer_b200 import workloads as W  # noqa: E402
from oracle import bert_encoder as O  # noqa: E402
import make_golden as G  # noqa: E402

VOCAB, TYPES, POSITIONS = 1000, 2, 64


def tiny_model_case():
    spec = W.tiny_spec()
    wl = W.make_workload(spec, random_gamma_beta=True)
    lengths = wl.lengths.copy()
    lengths[3] = 0
    mask = W.prefix_mask(lengths, spec.max_seq_len)
    heads = W.make_model_heads(spec, lengths, VOCAB, TYPES, POSITIONS)
    return spec, wl, lengths, mask, heads


def independent_model(spec, wl, mask, heads):
    from transformers import BertConfig
    from transformers.models.bert.modeling_bert import BertEmbeddings, BertPooler
    sh = spec.shape
    cfg = BertConfig(vocab_size=VOCAB, hidden_size=sh.hidden, num_hidden_layers=sh.num_layers,
                     num_attention_heads=sh.head_num, intermediate_size=sh.ffn_dim,
                     max_position_embeddings=POSITIONS, type_vocab_size=TYPES,
                     hidden_act="gelu_new", hidden_dropout_prob=0.0,
                     attention_probs_dropout_prob=0.0, layer_norm_eps=1e-12, pad_token_id=0)
    emb = BertEmbeddings(cfg).double().eval()
    pool = BertPooler(cfg).double().eval()
    d = lambda a: torch.from_numpy(a).double()
    with torch.no_grad():
        emb.word_embeddings.weight.copy_(d(heads.word_table))
        emb.token_type_embeddings.weight.copy_(d(heads.type_table))
        emb.position_embeddings.weight.copy_(d(heads.position_table))
        emb.LayerNorm.weight.copy_(d(heads.ln_gamma))
        emb.LayerNorm.bias.copy_(d(heads.ln_beta))
        pool.dense.weight.copy_(d(heads.pooler_kernel).T)
        pool.dense.bias.copy_(d(heads.pooler_bias))
        e = emb(input_ids=torch.from_numpy(heads.input_ids.astype(np.int64)),
                token_type_ids=torch.from_numpy(heads.token_type_ids.astype(np.int64)))
        wl2 = W.Workload(spec, wl.lengths, mask, e.numpy(), wl.weights)
        # the encoder of make_golden.py, fed with this embedding output in float64
        y = G.independent_encoder_from(wl2, e)
        p = pool(y)
    return e, y, p


def main() -> None:
    spec, wl, lengths, mask, heads = tiny_model_case()
    sh = spec.shape
    e, y, p = O.bert_model(heads, mask, wl.weights, sh.head_num, sh.size_per_head,
                           compute_dtype=torch.float64)
    e_i, y_i, p_i = independent_model(spec, wl, mask, heads)
    for name, a, b in (("embedding", e, e_i), ("sequence", O.valid_rows(y, mask), O.valid_rows(y_i, mask)),
                       ("pooled", p, p_i)):
        print(f"{name}: oracle vs independent max|delta| = {float((a - b).abs().max()):.3e}")
    np.savez_compressed(
        os.path.join(HERE, "tiny_model_fp64.npz"),
        lengths=lengths, mask=mask, input_ids=heads.input_ids, token_type_ids=heads.token_type_ids,
        embedding_oracle64=e.numpy(), embedding_independent=e_i.numpy(),
        sequence_oracle64=O.valid_rows(y, mask).numpy(),
        sequence_independent=O.valid_rows(y_i, mask).numpy(),
        pooled_oracle64=p.numpy(), pooled_independent=p_i.numpy())
    print("wrote", os.path.join(HERE, "tiny_model_fp64.npz"))


if __name__ == "__main__":
    main()
