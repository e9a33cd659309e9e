"""Seeded synthetic workloads with the shapes and value distributions of the
reference's benchmark script (sample/tensorflow/benchmark.py:38-61).

The reference draws per-sequence lengths with
``np.random.randint(2*avg - max, max + 1)``, builds a prefix mask, draws the
embedding output from N(0,1) and lets TensorFlow initialise the encoder
variables.  Here everything comes from one legacy ``np.random.RandomState`` in
a fixed draw order so that every process (tests, benchmark, oracle) sees the
same tensors:

1. sequence lengths,
2. ``from_tensor`` ~ N(0,1) of shape [B, S, H],
3. per layer, the 16 arrays in the order of
   python/effective_transformer/__init__.py:55-74 (kernels 0.02*N(0,1) of
   shape [in, out], biases 0.02*N(0,1), LayerNorm beta = 0 and gamma = 1).

No external dataset is involved; none exists for this path.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import numpy as np

# Index of each array inside one layer's group of 16
# (python/effective_transformer/__init__.py:55-74).
W_Q_KERNEL, W_Q_BIAS, W_K_KERNEL, W_K_BIAS, W_V_KERNEL, W_V_BIAS = 0, 1, 2, 3, 4, 5
W_ATT_OUT_KERNEL, W_ATT_OUT_BIAS, W_ATT_LN_BETA, W_ATT_LN_GAMMA = 6, 7, 8, 9
W_INTER_KERNEL, W_INTER_BIAS, W_OUT_KERNEL, W_OUT_BIAS = 10, 11, 12, 13
W_OUT_LN_BETA, W_OUT_LN_GAMMA = 14, 15
WEIGHTS_PER_LAYER = 16


@dataclass(frozen=True)
class EncoderShape:
    """Architecture of the encoder stack (sample/tensorflow/bert_config.json)."""
    num_layers: int
    head_num: int
    size_per_head: int
    ffn_dim: int

    @property
    def hidden(self) -> int:
        return self.head_num * self.size_per_head


BERT_BASE = EncoderShape(num_layers=12, head_num=12, size_per_head=64, ffn_dim=3072)
BERT_LARGE = EncoderShape(num_layers=24, head_num=16, size_per_head=64, ffn_dim=4096)


@dataclass(frozen=True)
class WorkloadSpec:
    name: str
    shape: EncoderShape
    dtype: str            # "fp32" or "fp16"
    batch: int
    max_seq_len: int
    len_low: int          # randint(low, high) bounds; ignored when skewed
    len_high: int
    skewed: bool = False  # 90% lengths in [1,16], 10% in [100,128]
    seed: int = 0


# The five benchmark configurations (index = position in the list).
WORKLOADS = [
    WorkloadSpec("cfg0_base_fp32_b8_s32", BERT_BASE, "fp32", 8, 32, 8, 33),
    WorkloadSpec("cfg1_base_fp16_b100_s32", BERT_BASE, "fp16", 100, 32, 8, 33),
    WorkloadSpec("cfg2_base_fp16_b1000_s64", BERT_BASE, "fp16", 1000, 64, 16, 65),
    WorkloadSpec("cfg3_base_fp32_b500_s64", BERT_BASE, "fp32", 500, 64, 16, 65),
    WorkloadSpec("cfg4_large_fp16_b4096_s128_skewed", BERT_LARGE, "fp16", 4096, 128, 1, 17, skewed=True),
]


def tiny_spec(dtype: str = "fp32", layers: int = 2, heads: int = 2, ffn: int = 256,
              batch: int = 5, max_seq_len: int = 12, seed: int = 3) -> WorkloadSpec:
    """A small architecture for fast CPU-side checks."""
    return WorkloadSpec("tiny", EncoderShape(layers, heads, 64, ffn), dtype, batch,
                        max_seq_len, 1, max_seq_len + 1, seed=seed)


def draw_lengths(spec: WorkloadSpec, rng: np.random.RandomState) -> np.ndarray:
    b = spec.batch
    if spec.skewed:
        short = rng.randint(1, 17, size=b, dtype=np.int32)
        long_ = rng.randint(100, 129, size=b, dtype=np.int32)
        is_long = rng.rand(b) < 0.10
        return np.where(is_long, long_, short).astype(np.int32)
    return rng.randint(spec.len_low, spec.len_high, size=b, dtype=np.int32)


def prefix_mask(lengths: np.ndarray, max_seq_len: int) -> np.ndarray:
    """mask[b, :len_b] = 1 (sample/tensorflow/benchmark.py:47-49)."""
    return (np.arange(max_seq_len, dtype=np.int32)[None, :] < lengths[:, None]).astype(np.int32)


def attention_mask_from_input_mask(mask: np.ndarray) -> np.ndarray:
    """Key-only 3-D mask, tile(mask, S).reshape(B, S, S)
    (sample/tensorflow/benchmark.py:59-61)."""
    b, s = mask.shape
    return np.tile(mask, s).reshape(b, s, s)


def draw_layer_weights(shape: EncoderShape, rng: np.random.RandomState,
                       np_dtype=np.float32) -> List[np.ndarray]:
    h, f = shape.hidden, shape.ffn_dim
    k = lambda i, o: (0.02 * rng.randn(i, o)).astype(np_dtype)
    b = lambda o: (0.02 * rng.randn(o)).astype(np_dtype)
    w: List[Optional[np.ndarray]] = [None] * WEIGHTS_PER_LAYER
    w[W_Q_KERNEL], w[W_Q_BIAS] = k(h, h), b(h)
    w[W_K_KERNEL], w[W_K_BIAS] = k(h, h), b(h)
    w[W_V_KERNEL], w[W_V_BIAS] = k(h, h), b(h)
    w[W_ATT_OUT_KERNEL], w[W_ATT_OUT_BIAS] = k(h, h), b(h)
    w[W_ATT_LN_BETA], w[W_ATT_LN_GAMMA] = np.zeros(h, np_dtype), np.ones(h, np_dtype)
    w[W_INTER_KERNEL], w[W_INTER_BIAS] = k(h, f), b(f)
    w[W_OUT_KERNEL], w[W_OUT_BIAS] = k(f, h), b(h)
    w[W_OUT_LN_BETA], w[W_OUT_LN_GAMMA] = np.zeros(h, np_dtype), np.ones(h, np_dtype)
    return w  # type: ignore[return-value]


@dataclass
class Workload:
    spec: WorkloadSpec
    lengths: np.ndarray            # int32 [B]
    mask: np.ndarray               # int32 [B, S]
    from_tensor: np.ndarray        # float32 [B, S, H] (cast by the caller)
    weights: List[np.ndarray] = field(default_factory=list)   # 16 * L arrays, float32

    @property
    def valid_tokens(self) -> int:
        return int(self.lengths.sum())


def make_workload(spec: WorkloadSpec, with_weights: bool = True,
                  batch_override: Optional[int] = None,
                  random_gamma_beta: bool = False) -> Workload:
    """Materialise a workload.  ``batch_override`` keeps only the first
    sequences of the same draw (used for bounded CPU samples)."""
    rng = np.random.RandomState(spec.seed)
    lengths = draw_lengths(spec, rng)
    mask = prefix_mask(lengths, spec.max_seq_len)
    x = rng.randn(spec.batch, spec.max_seq_len, spec.shape.hidden).astype(np.float32)
    weights: List[np.ndarray] = []
    if with_weights:
        for _ in range(spec.shape.num_layers):
            weights.extend(draw_layer_weights(spec.shape, rng))
        if random_gamma_beta:
            # not part of the benchmark recipe: exercises gamma/beta in tests
            g = np.random.RandomState(spec.seed + 1000)
            for l in range(spec.shape.num_layers):
                for idx in (W_ATT_LN_GAMMA, W_OUT_LN_GAMMA):
                    weights[l * 16 + idx] = (1.0 + 0.1 * g.randn(spec.shape.hidden)).astype(np.float32)
                for idx in (W_ATT_LN_BETA, W_OUT_LN_BETA):
                    weights[l * 16 + idx] = (0.1 * g.randn(spec.shape.hidden)).astype(np.float32)
    if batch_override is not None and batch_override < spec.batch:
        lengths, mask, x = lengths[:batch_override], mask[:batch_override], x[:batch_override]
    return Workload(spec, lengths, mask, x, weights)


def make_workload_fast(spec: WorkloadSpec, with_input: bool = True) -> Workload:
    """The same lengths as ``make_workload`` (so the same valid-token count and tile packing) with
    inputs and weights of the same shapes and distributions drawn by numpy's float32 generator,
    which is several times faster than the legacy float64 draws: for timing passes over the large
    workloads, where the values only have to be well-scaled, not the canonical ones."""
    lengths = draw_lengths(spec, np.random.RandomState(spec.seed))
    mask = prefix_mask(lengths, spec.max_seq_len)
    g = np.random.default_rng(spec.seed)
    n = lambda *shape: g.standard_normal(shape, dtype=np.float32)
    # with_input=False: the caller draws the N(0,1) input itself (e.g. on the device); from_tensor is empty
    x = n(spec.batch, spec.max_seq_len, spec.shape.hidden) if with_input else np.zeros((0,), np.float32)
    h, f = spec.shape.hidden, spec.shape.ffn_dim
    weights: List[np.ndarray] = []
    for _ in range(spec.shape.num_layers):
        w: List[Optional[np.ndarray]] = [None] * WEIGHTS_PER_LAYER
        for kk, bb, (i, o) in ((W_Q_KERNEL, W_Q_BIAS, (h, h)), (W_K_KERNEL, W_K_BIAS, (h, h)),
                               (W_V_KERNEL, W_V_BIAS, (h, h)), (W_ATT_OUT_KERNEL, W_ATT_OUT_BIAS, (h, h)),
                               (W_INTER_KERNEL, W_INTER_BIAS, (h, f)), (W_OUT_KERNEL, W_OUT_BIAS, (f, h))):
            w[kk], w[bb] = 0.02 * n(i, o), 0.02 * n(o)
        w[W_ATT_LN_BETA], w[W_ATT_LN_GAMMA] = np.zeros(h, np.float32), np.ones(h, np.float32)
        w[W_OUT_LN_BETA], w[W_OUT_LN_GAMMA] = np.zeros(h, np.float32), np.ones(h, np.float32)
        weights.extend(w)  # type: ignore[arg-type]
    return Workload(spec, lengths, mask, x, weights)


@dataclass
class ModelHeads:
    """The pieces of sample/tensorflow/modeling.py's BertModel that sit either
    side of the encoder stack: token ids and the three embedding tables with
    their LayerNorm (modeling.py:380-521), and the pooler's dense layer
    (modeling.py:224-232)."""
    input_ids: np.ndarray        # int32 [B, S]
    token_type_ids: np.ndarray   # int32 [B, S]
    word_table: np.ndarray       # float32 [vocab, H]
    type_table: np.ndarray       # float32 [type_vocab, H]
    position_table: np.ndarray   # float32 [max_position, H]
    ln_gamma: np.ndarray         # float32 [H]
    ln_beta: np.ndarray          # float32 [H]
    pooler_kernel: np.ndarray    # float32 [H, H]  ([in, out])
    pooler_bias: np.ndarray      # float32 [H]


def make_model_heads(spec: WorkloadSpec, lengths: np.ndarray, vocab_size: int = 30522,
                     type_vocab_size: int = 2, max_position: int = 512,
                     table_scale: float = 0.02) -> ModelHeads:
    """Seeded ids and tables for the embedding / pooler stages.  Drawn from a
    RandomState of their own (seed + 7919) so that the encoder-stack draws of
    ``make_workload`` stay what they are.  Vocabulary, type and position sizes
    default to sample/tensorflow/bert_config.json; ``table_scale`` is the
    reference's initializer_range.  Each sequence gets segment 0 then segment 1,
    split at a random point, as sentence-pair inputs do."""
    rng = np.random.RandomState(spec.seed + 7919)
    b, s, h = len(lengths), spec.max_seq_len, spec.shape.hidden
    ids = rng.randint(0, vocab_size, size=(b, s)).astype(np.int32)
    split = (rng.rand(b) * (lengths + 1)).astype(np.int32)
    types = (np.arange(s, dtype=np.int32)[None, :] >= split[:, None]).astype(np.int32)
    types = np.minimum(types, type_vocab_size - 1).astype(np.int32)
    t = lambda *shape: (table_scale * rng.randn(*shape)).astype(np.float32)
    word, typ, pos = t(vocab_size, h), t(type_vocab_size, h), t(max_position, h)
    gamma = (1.0 + 0.1 * rng.randn(h)).astype(np.float32)
    beta = (0.1 * rng.randn(h)).astype(np.float32)
    return ModelHeads(ids, types, word, typ, pos, gamma, beta, t(h, h), t(h))


def algorithmic_flops(shape: EncoderShape, lengths: np.ndarray) -> float:
    """FLOPs of one forward pass counted on valid positions only:
    GEMMs 2*T*H*(3H + H + 2F) and attention 4*H*sum(len^2) per layer."""
    t = float(lengths.astype(np.int64).sum())
    l2 = float((lengths.astype(np.int64) ** 2).sum())
    h, f = shape.hidden, shape.ffn_dim
    per_layer = 2.0 * t * h * (3 * h + h + 2 * f) + 4.0 * h * l2
    return per_layer * shape.num_layers


def balanced_shards(lengths: np.ndarray, num_shards: int) -> Tuple[List[np.ndarray], np.ndarray]:
    """Assign sequences to shards so that valid-token counts are balanced
    (longest-first greedy).  Returns the per-shard sequence index arrays (each
    sorted ascending so that a shard keeps the batch order) and the per-shard
    token totals."""
    order = np.argsort(-lengths.astype(np.int64), kind="stable")
    loads = np.zeros(num_shards, dtype=np.int64)
    buckets: List[List[int]] = [[] for _ in range(num_shards)]
    for i in order:
        g = int(np.argmin(loads))
        buckets[g].append(int(i))
        loads[g] += int(lengths[i])
    return [np.array(sorted(b), dtype=np.int64) for b in buckets], loads
