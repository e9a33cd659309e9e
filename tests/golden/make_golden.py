"""Generates the golden fixtures in this directory.  Run from the repository
root:  python tests/golden/make_golden.py

Two sources are stored side by side for every case:
  * ``oracle64``  - oracle/bert_encoder.py evaluated in float64;
  * ``independent`` - Hugging Face ``transformers`` BertEncoder (an independent
    implementation of the Google BERT encoder that the reference's
    sample/tensorflow/modeling.py also implements), float64, tanh GELU
    ("gelu_new"), LayerNorm eps 1e-12, loaded with the same seeded weights.
The reference's own TF-1.15 graph cannot be imported (TensorFlow is absent), so
these are the pins the oracle is held to.

Cases: "tiny" (2 layers, 2 heads x 64, FFN 256, B=5, S=12; full tensors and the
layer-0 intermediates) and "cfg0" (BERT-base fp32, B=8, S=32; valid rows, every
8th hidden column, to keep the file small).
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from effective_transformer_b200 import workloads as W  # noqa: E402
from oracle import bert_encoder as O  # noqa: E402
from oracle import padding as P  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def independent_encoder(wl: W.Workload) -> torch.Tensor:
    return independent_encoder_from(wl, torch.from_numpy(wl.from_tensor).double())


def independent_encoder_from(wl: W.Workload, x: torch.Tensor) -> torch.Tensor:
    """The independent encoder stack on a given float64 input [B, S, H] and wl.mask."""
    from transformers import BertConfig
    from transformers.models.bert.modeling_bert import BertEncoder
    sh = wl.spec.shape
    cfg = BertConfig(hidden_size=sh.hidden, num_hidden_layers=sh.num_layers,
                     num_attention_heads=sh.head_num, intermediate_size=sh.ffn_dim,
                     hidden_act="gelu_new", hidden_dropout_prob=0.0,
                     attention_probs_dropout_prob=0.0, layer_norm_eps=1e-12)
    cfg._attn_implementation = "eager"
    enc = BertEncoder(cfg).double().eval()
    with torch.no_grad():
        for l, layer in enumerate(enc.layer):
            w = [torch.from_numpy(a).double() for a in wl.weights[l * 16:(l + 1) * 16]]
            a = layer.attention
            a.self.query.weight.copy_(w[0].T); a.self.query.bias.copy_(w[1])
            a.self.key.weight.copy_(w[2].T); a.self.key.bias.copy_(w[3])
            a.self.value.weight.copy_(w[4].T); a.self.value.bias.copy_(w[5])
            a.output.dense.weight.copy_(w[6].T); a.output.dense.bias.copy_(w[7])
            a.output.LayerNorm.bias.copy_(w[8]); a.output.LayerNorm.weight.copy_(w[9])
            layer.intermediate.dense.weight.copy_(w[10].T); layer.intermediate.dense.bias.copy_(w[11])
            layer.output.dense.weight.copy_(w[12].T); layer.output.dense.bias.copy_(w[13])
            layer.output.LayerNorm.bias.copy_(w[14]); layer.output.LayerNorm.weight.copy_(w[15])
        am = torch.from_numpy(W.attention_mask_from_input_mask(wl.mask)).double()
        ext = (1.0 - am[:, None, :, :]) * -10000.0
        return enc(x, attention_mask=ext)[0]


def main() -> None:
    torch.manual_seed(0)
    # ---- tiny ----
    spec = W.tiny_spec()
    wl = W.make_workload(spec, random_gamma_beta=True)
    am = W.attention_mask_from_input_mask(wl.mask)
    stages = {}
    y = O.transformer_model(wl.from_tensor, am, wl.weights, spec.shape.head_num,
                            spec.shape.size_per_head, compute_dtype=torch.float64,
                            layer0_stages=stages)
    y_ind = independent_encoder(wl)
    idx = P.padding_indices(wl.mask)
    np.savez_compressed(
        os.path.join(HERE, "tiny_fp64.npz"),
        lengths=wl.lengths, mask=wl.mask,
        oracle64=O.valid_rows(y, wl.mask).numpy(),
        independent=O.valid_rows(y_ind, wl.mask).numpy(),
        **{"stage_" + k: v.numpy() for k, v in stages.items()},
        **{"idx_" + k: v for k, v in idx.items()})
    # ---- cfg0 ----
    spec0 = W.WORKLOADS[0]
    wl0 = W.make_workload(spec0)
    am0 = W.attention_mask_from_input_mask(wl0.mask)
    y0 = O.transformer_model(wl0.from_tensor, am0, wl0.weights, 12, 64, compute_dtype=torch.float64)
    y0_ind = independent_encoder(wl0)
    idx0 = P.padding_indices(wl0.mask)
    np.savez_compressed(
        os.path.join(HERE, "cfg0_fp64_subsampled.npz"),
        lengths=wl0.lengths,
        oracle64=O.valid_rows(y0, wl0.mask).numpy()[:, ::8],
        independent=O.valid_rows(y0_ind, wl0.mask).numpy()[:, ::8],
        rms=np.array([float(O.valid_rows(y0, wl0.mask).pow(2).mean().sqrt())]),
        **{"idx_" + k: v for k, v in idx0.items()})
    # ---- token counts of the five benchmark configurations ----
    counts = {}
    for s in W.WORKLOADS:
        rng = np.random.RandomState(s.seed)
        lens = W.draw_lengths(s, rng)
        counts[s.name] = np.array([int(lens.sum()), int((lens.astype(np.int64) ** 2).sum())])
    np.savez_compressed(os.path.join(HERE, "token_counts.npz"), **counts)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
