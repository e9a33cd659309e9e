"""GPU parity tests of the whole path (input op -> layers -> output op) against
the CPU oracle, through the reference-shaped Python API and the C ABI.

Tolerances (valid tokens only, as sample/tensorflow/benchmark.py:105-112):
  fp32: max|delta| <= 1e-4 * RMS(oracle activations)
  fp16: max|delta| <= 2e-2 and mean|delta| <= 2e-3 after all layers
"""
import os

import numpy as np
import pytest
import torch

import effective_transformer_b200 as et
from effective_transformer_b200 import _capi
from effective_transformer_b200 import workloads as W
from oracle import bert_encoder as O
from oracle import padding as P

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

FP32_REL_RMS = 1e-4
FP16_MAX_ABS, FP16_MEAN_ABS = 2e-2, 2e-3


def make_engine(spec: W.WorkloadSpec, wl: W.Workload, simt: bool = False) -> et.EffectiveTransformer:
    dtype = torch.float16 if spec.dtype == "fp16" else torch.float32
    sh = spec.shape
    eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, sh.size_per_head, sh.ffn_dim,
                                  wl.mask.shape[0], spec.max_seq_len, dtype=dtype)
    eng.set_weights(wl.weights)
    if simt:
        eng.set_debug_simt(True)
    return eng


def run_forward(eng, wl):
    x = torch.from_numpy(wl.from_tensor).to(eng.dtype).cuda()
    m = torch.from_numpy(wl.mask).cuda()
    y = eng.forward(x, m)
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    return y


def assert_parity(y_dev: torch.Tensor, y_ref_valid: torch.Tensor, mask: np.ndarray, fp16: bool):
    got = O.valid_rows(y_dev.detach().cpu().double(), mask)
    ref = y_ref_valid.double()
    diff = (got - ref).abs()
    if fp16:
        assert float(diff.max()) <= FP16_MAX_ABS, f"max abs {float(diff.max())}"
        assert float(diff.mean()) <= FP16_MEAN_ABS, f"mean abs {float(diff.mean())}"
    else:
        rms = float(ref.pow(2).mean().sqrt())
        assert float(diff.max()) <= FP32_REL_RMS * rms, f"max abs {float(diff.max())} vs rms {rms}"
    # padded rows come back as exact zeros
    b, s, h = y_dev.shape
    pad = torch.from_numpy(mask.ravel() == 0)
    assert torch.all(y_dev.detach().cpu().reshape(b * s, h)[pad] == 0)


def oracle_valid(wl, spec, dtype64=False):
    am = W.attention_mask_from_input_mask(wl.mask)
    y = O.transformer_model(wl.from_tensor, am, wl.weights, spec.shape.head_num, spec.shape.size_per_head,
                            compute_dtype=torch.float64 if dtype64 else torch.float32,
                            round_to_fp16=(spec.dtype == "fp16"))
    return O.valid_rows(y, wl.mask)


@pytest.mark.parametrize("dtype,simt", [("fp32", False), ("fp32", True), ("fp16", True), ("fp16", False)])
def test_tiny_against_golden(dtype, simt):
    d = np.load(os.path.join(GOLD, "tiny_fp64.npz"))
    spec = W.tiny_spec(dtype=dtype)
    wl = W.make_workload(spec, random_gamma_beta=True)
    eng = make_engine(spec, wl, simt)
    y = run_forward(eng, wl)
    if dtype == "fp32":
        ref = torch.from_numpy(d["oracle64"])
    else:
        ref = oracle_valid(wl, spec, dtype64=True)
    assert_parity(y, ref, wl.mask, fp16=(dtype == "fp16"))
    eng.close()


def test_cfg0_fp32_against_golden():
    d = np.load(os.path.join(GOLD, "cfg0_fp64_subsampled.npz"))
    spec = W.WORKLOADS[0]
    wl = W.make_workload(spec)
    eng = make_engine(spec, wl)
    y = run_forward(eng, wl)
    got = O.valid_rows(y.cpu().double(), wl.mask).numpy()[:, ::8]
    assert np.abs(got - d["oracle64"]).max() <= FP32_REL_RMS * float(d["rms"][0])
    # integer outputs of the input op, bit-exact
    cu, sl, po, pre = eng.last_padding_info(spec.batch, wl.valid_tokens, spec.max_seq_len)
    assert np.array_equal(cu, d["idx_cu_seqlens"]) and np.array_equal(sl, d["idx_seq_len"])
    assert np.array_equal(po, d["idx_padding_offset"]) and np.array_equal(pre, d["idx_prefix_sum"].ravel())
    eng.close()


@pytest.mark.parametrize("simt", [False, True])
def test_cfg1_fp16_twelve_layers(simt):
    spec = W.WORKLOADS[1]
    wl = W.make_workload(spec)
    eng = make_engine(spec, wl, simt)
    y = run_forward(eng, wl)
    assert_parity(y, oracle_valid(wl, spec), wl.mask, fp16=True)
    eng.close()


@pytest.mark.parametrize("ranks", [2, 8])
def test_sharded_batch_reassembled_equals_the_oracle(ranks):
    """The multi-GPU split, emulated on one GPU: the batch is dealt to `ranks` shards by the planner
    the multi-rank benchmark uses, every shard runs through an engine of its own, and the outputs,
    put back in batch order by the gather's inverse permutation, meet the oracle of the whole batch."""
    from effective_transformer_b200.sharding import inverse_order
    spec = W.WORKLOADS[1]
    wl = W.make_workload(spec)
    shards, loads = W.balanced_shards(wl.lengths, ranks)
    assert int(loads.sum()) == wl.valid_tokens
    blocks = []
    for idx in shards:
        part = W.Workload(spec, wl.lengths[idx], wl.mask[idx], wl.from_tensor[idx], wl.weights)
        eng = make_engine(spec, part)
        blocks.append(run_forward(eng, part).cpu())
        eng.close()
    whole = torch.cat(blocks, dim=0)[torch.from_numpy(inverse_order(shards))]
    assert whole.shape[0] == spec.batch
    assert_parity(whole, oracle_valid(wl, spec), wl.mask, fp16=True)


def test_operator_api_matches_forward_and_reference_wiring():
    """get_sequence_output wires the three operators exactly like
    python/effective_transformer/__init__.py:42-82 and equals et_forward."""
    spec = W.tiny_spec(dtype="fp16", layers=3, batch=7, max_seq_len=20, seed=11)
    wl = W.make_workload(spec, random_gamma_beta=True)
    wl.mask[2, :] = 0                                         # an empty sequence
    wl.mask[4, :] = 1                                         # a full one
    eng = make_engine(spec, wl)
    x = torch.from_numpy(wl.from_tensor).half().cuda()
    m = torch.from_numpy(wl.mask).cuda()
    am = torch.from_numpy(W.attention_mask_from_input_mask(wl.mask)).half().cuda()
    cfg = et.BertConfig(spec.shape.hidden, spec.shape.num_layers, spec.shape.head_num, spec.shape.ffn_dim)
    y_ops = et.get_sequence_output(cfg, spec.batch, spec.max_seq_len, am, m, x, wl.weights, engine=eng)
    y_fwd = eng.forward(x, m)
    torch.cuda.synchronize()
    assert torch.equal(y_ops, y_fwd)
    # input op outputs
    packed, valid, bidx, widx = eng.effective_transformer_input(x, m)
    torch.cuda.synchronize()
    ref = P.padding_indices(wl.mask)
    t = int(ref["valid_word_num"][0])
    assert int(valid[0]) == t
    assert np.array_equal(bidx.cpu().numpy().ravel()[:t], ref["batch_idx"])
    assert np.array_equal(widx.cpu().numpy().ravel()[:t], ref["word_idx"])
    assert np.array_equal(packed.cpu().numpy().reshape(-1, spec.shape.hidden)[:t],
                          P.remove_padding(x.cpu().numpy(), wl.mask))
    assert_parity(y_fwd, oracle_valid(wl, spec, dtype64=True), wl.mask, fp16=True)
    eng.close()


def test_arbitrary_input_mask():
    """Non-prefix masks are legal for the input/output ops (word_idx keeps the
    true positions) and, with the key-only attention mask, for the layers."""
    spec = W.tiny_spec(dtype="fp32", batch=6, max_seq_len=17, seed=5)
    wl = W.make_workload(spec)
    rng = np.random.RandomState(9)
    wl.mask[:] = (rng.rand(*wl.mask.shape) < 0.55).astype(np.int32)
    eng = make_engine(spec, wl)
    y = run_forward(eng, wl)
    assert_parity(y, oracle_valid(wl, spec, dtype64=True), wl.mask, fp16=False)
    eng.close()


def test_forward_host_equals_device_forward():
    spec = W.tiny_spec(dtype="fp16", batch=9, max_seq_len=31, seed=21)
    wl = W.make_workload(spec)
    eng = make_engine(spec, wl)
    y_dev = run_forward(eng, wl).cpu().numpy()
    y_host, t = eng.forward_host(wl.from_tensor.astype(np.float16), wl.mask)
    assert t == wl.valid_tokens
    assert np.array_equal(y_host, y_dev)
    # a smaller run-time batch on the same handle (attr batch_size is only a maximum)
    y_small, t2 = eng.forward_host(wl.from_tensor[:4].astype(np.float16), wl.mask[:4])
    assert t2 == int(wl.mask[:4].sum())
    sel = wl.mask[:4].ravel() > 0
    a = y_small.reshape(-1, spec.shape.hidden)[sel].astype(np.float32)
    b = y_dev[:4].reshape(-1, spec.shape.hidden)[sel].astype(np.float32)
    assert np.abs(a - b).max() <= 2e-3       # sequences are independent of their batch mates
    eng.close()


def test_error_conventions():
    spec = W.tiny_spec(dtype="fp16")
    wl = W.make_workload(spec)
    sh = spec.shape
    with pytest.raises(et.EtError) as e:
        et.EffectiveTransformer(sh.num_layers, sh.head_num, 32, sh.ffn_dim, 4, 8)      # size_per_head != 64
    assert e.value.code == _capi.ET_INVALID_ARGUMENT
    eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, 64, sh.ffn_dim, spec.batch, spec.max_seq_len)
    x = torch.from_numpy(wl.from_tensor).half().cuda()
    m = torch.from_numpy(wl.mask).cuda()
    with pytest.raises(et.EtError) as e:
        eng.forward(x, m)                                                            # weights never set
    assert e.value.code == _capi.ET_NOT_READY
    eng.set_weights(wl.weights)
    big = torch.zeros(spec.batch + 1, spec.max_seq_len, sh.hidden, dtype=torch.float16, device="cuda")
    with pytest.raises(et.EtError) as e:
        eng.forward(big, torch.ones(spec.batch + 1, spec.max_seq_len, dtype=torch.int32, device="cuda"))
    assert e.value.code == _capi.ET_INVALID_ARGUMENT
    with pytest.raises(et.EtError):
        eng.set_layer_weights(99, wl.weights[:16])
    # all-padding batch: T = 0, output all zeros, no error
    y = eng.forward(x, torch.zeros_like(m))
    torch.cuda.synchronize()
    assert eng.device_status() == 0 and torch.all(y == 0)
    eng.close()


def test_cfg2_full_size_properties():
    """Headline workload (B=1000, S=64, 12 layers, fp16) at full size, checked
    through size-independent properties: a sub-batch against the oracle,
    independence of a sequence from its batch mates, invariance under a
    permutation of the sequences, zero padding rows."""
    spec = W.WORKLOADS[2]
    wl = W.make_workload(spec)
    eng = make_engine(spec, wl)
    y = run_forward(eng, wl)
    h = spec.shape.hidden
    # (1) all 1000 sequences against the CPU oracle (fp32, padded like the TF graph), in slices
    worst_max, total_abs, total_n = 0.0, 0.0, 0
    for b0 in range(0, spec.batch, 250):
        sl = slice(b0, b0 + 250)
        sub = W.Workload(spec, wl.lengths[sl], wl.mask[sl], wl.from_tensor[sl], wl.weights)
        ref = oracle_valid(sub, spec)
        got = O.valid_rows(y[sl].cpu().double(), sub.mask)
        diff = (got - ref.double()).abs()
        worst_max = max(worst_max, float(diff.max()))
        total_abs += float(diff.sum())
        total_n += diff.numel()
    assert total_n == wl.valid_tokens * h
    assert worst_max <= FP16_MAX_ABS and total_abs / total_n <= FP16_MEAN_ABS, (worst_max, total_abs / total_n)
    # (2) padding rows are zero everywhere
    pad = torch.from_numpy(wl.mask.ravel() == 0).cuda()
    assert torch.all(y.reshape(-1, h)[pad] == 0)
    # (3) permuting the sequences permutes the output
    perm = np.random.RandomState(0).permutation(spec.batch)
    wl_p = W.Workload(spec, wl.lengths[perm], wl.mask[perm], wl.from_tensor[perm], wl.weights)
    y_p = run_forward(eng, wl_p)
    # (a sequence's tile mates change with the order, so the fp32 summation order inside the
    # attention MMAs changes: equal up to a few fp16 roundings after 12 layers, not bit for bit)
    d = (y_p.float() - y[torch.from_numpy(perm).cuda()].float()).abs()
    assert float(d.max()) <= FP16_MAX_ABS and float(d.mean()) <= FP16_MEAN_ABS
    eng.close()


def test_cfg3_fp32_full_size_both_gemm_paths():
    """fp32 workload (B=500, S=64, 12 layers) at full size: a sub-batch against the float64
    oracle, and the tensor-core (tf32 split) and CUDA-core GEMM paths against each other."""
    spec = W.WORKLOADS[3]
    wl = W.make_workload(spec)
    eng = make_engine(spec, wl)
    y = run_forward(eng, wl)
    sub = W.Workload(spec, wl.lengths[:16], wl.mask[:16], wl.from_tensor[:16], wl.weights)
    ref = oracle_valid(sub, spec, dtype64=True)
    got = O.valid_rows(y[:16].cpu().double(), sub.mask)
    rms = float(ref.pow(2).mean().sqrt())
    assert float((got - ref).abs().max()) <= FP32_REL_RMS * rms
    eng.set_debug_simt(True)
    y_simt = run_forward(eng, wl)
    assert float((y - y_simt).abs().max()) <= FP32_REL_RMS * rms
    pad = torch.from_numpy(wl.mask.ravel() == 0).cuda()
    assert torch.all(y.reshape(-1, spec.shape.hidden)[pad] == 0)
    eng.close()


def test_cfg4_bert_large_skewed_lengths_full_size():
    """BERT-large, 24 layers, B=4096, S=128, 90 % short and 10 % long sequences (524 288
    positions, 82 348 valid): long sequences with their tile mates and short ones against the oracle."""
    spec = W.WORKLOADS[4]
    wl = W.make_workload(spec)
    assert wl.valid_tokens == 82348
    eng = make_engine(spec, wl)
    y = run_forward(eng, wl)
    # 16 long sequences (the 3 longest among them) with their neighbours in batch order, which are
    # the sequences an attention tile packs next to them, the shortest ones and a random draw: 72
    order = np.argsort(-wl.lengths, kind="stable")
    longs = np.concatenate([order[:3], np.flatnonzero(wl.lengths >= 100)[::31][:13]])
    near = np.concatenate([longs - 1, longs, longs + 1])
    rnd = np.random.RandomState(3).choice(spec.batch, 24, replace=False)
    pick = np.unique(np.clip(np.concatenate([near, order[-3:], [0, 1], rnd]), 0, spec.batch - 1))
    assert len(pick) >= 64
    sub = W.Workload(spec, wl.lengths[pick], wl.mask[pick], wl.from_tensor[pick], wl.weights)
    ref = oracle_valid(sub, spec)
    got = O.valid_rows(y[torch.from_numpy(pick).cuda()].cpu().double(), sub.mask)
    diff = (got - ref.double()).abs()
    assert float(diff.max()) <= FP16_MAX_ABS and float(diff.mean()) <= FP16_MEAN_ABS, \
        (float(diff.max()), float(diff.mean()))
    pad = torch.from_numpy(wl.mask.ravel() == 0).cuda()
    assert torch.all(y.reshape(-1, spec.shape.hidden)[pad] == 0)
    eng.close()


def test_two_handles_and_two_streams_do_not_share_state():
    """Two handles with different weights, driven alternately on two streams: each must
    reproduce what it computes alone (nothing of a pass lives in process-wide state)."""
    specs = [W.tiny_spec(dtype="fp16", seed=11), W.tiny_spec(dtype="fp16", layers=3, batch=7, max_seq_len=20, seed=12)]
    wls = [W.make_workload(s, random_gamma_beta=True) for s in specs]
    engs = [make_engine(s, w) for s, w in zip(specs, wls)]
    xs = [torch.from_numpy(w.from_tensor).half().cuda() for w in wls]
    ms = [torch.from_numpy(w.mask).cuda() for w in wls]
    alone = [e.forward(x, m).clone() for e, x, m in zip(engs, xs, ms)]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [[], []]
    for _ in range(4):
        for i in (0, 1):
            with torch.cuda.stream(streams[i]):
                outs[i].append(engs[i].forward(xs[i], ms[i]))
    torch.cuda.synchronize()
    for i in (0, 1):
        for y in outs[i]:
            assert torch.equal(y, alone[i])
        assert engs[i].device_status() == 0
        engs[i].close()


def test_layernorm_inside_the_gemm_equals_the_layernorm_kernel():
    """cfg1 (hidden 768, 12 layers): with a LayerNorm kernel behind each projection and
    with the LayerNorms inside the projection kernels the path launches 7 and 5 kernels per layer,
    computes the same arithmetic in the same order (a kernel-level test shows single last-place
    differences where the compiler contracts a multiply-add in one kernel and not in the other;
    twelve layers amplify them to a few fp16 roundings), and both meet the oracle gate."""
    spec = W.WORKLOADS[1]
    wl = W.make_workload(spec, random_gamma_beta=True)
    eng = make_engine(spec, wl)
    eng.set_deferred_layernorm(False)     # the default materialises no LayerNorm at all
    eng.get_profile(reset=True)
    y_split = run_forward(eng, wl).clone()
    prof = eng.get_profile(reset=True)
    assert prof["layernorm"][1] == 2 * spec.shape.num_layers
    assert sum(v[1] for v in prof.values()) == 5 + 7 * spec.shape.num_layers
    eng.set_fused_layernorm(True)
    y_fused = run_forward(eng, wl).clone()
    prof = eng.get_profile(reset=True)
    assert prof["layernorm"][1] == 0
    assert sum(v[1] for v in prof.values()) == 5 + 5 * spec.shape.num_layers
    d = (y_fused.float() - y_split.float()).abs()
    assert float(d.max()) <= FP16_MAX_ABS and float(d.mean()) <= 1e-3, (float(d.max()), float(d.mean()))
    ref = oracle_valid(wl, spec)
    assert_parity(y_fused, ref, wl.mask, fp16=True)
    assert_parity(y_split, ref, wl.mask, fp16=True)
    # ragged run-time batches on the same handle: T below one row tile
    for nb in (1, 3):
        sub = W.Workload(spec, wl.lengths[:nb], wl.mask[:nb], wl.from_tensor[:nb], wl.weights)
        eng.set_fused_layernorm(True)
        a = run_forward(eng, sub).clone()
        eng.set_fused_layernorm(False)
        d = (a.float() - run_forward(eng, sub).float()).abs()
        assert float(d.max()) <= FP16_MAX_ABS
    # a recorded pass with the LayerNorms inside the projections replays to the same values
    eng.set_fused_layernorm(True)
    x = torch.from_numpy(wl.from_tensor).half().cuda()
    m = torch.from_numpy(wl.mask).cuda()
    out = torch.empty_like(x)
    eng.capture(x, m, out)
    eng.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, y_fused)
    eng.close()


@pytest.mark.parametrize("cfg,ln_params", [(1, "benchmark"), (4, "benchmark"), (1, "random")])
def test_deferred_layernorm_meets_the_oracle_and_the_layernorm_kernels(cfg, ln_params):
    """et_set_deferred_layernorm: no LayerNorm between the projections is materialised (row statistics
    from the producers, gamma folded into the consumers' weights).  With the benchmark's LayerNorm
    parameters (gamma = 1, beta = 0): the gates of the header, as for the path with LayerNorm kernels.
    With gamma, beta drawn away from 1, 0 the activations grow heavy tails (|y| up to 20, where one fp16
    step is 0.016) and the path with LayerNorm kernels itself reaches 0.06: there the mean gate holds
    and the deferred path may not be worse than the other by more than a step of the largest value."""
    spec = W.WORKLOADS[cfg]
    wl = W.make_workload(spec, batch_override=72 if cfg == 4 else None)
    if ln_params == "random":
        rng = np.random.RandomState(5)
        for l in range(spec.shape.num_layers):        # beta, gamma of both LayerNorms: arrays 8, 9, 14, 15
            for i in (8, 14):
                wl.weights[16 * l + i] = (0.1 * rng.randn(spec.shape.hidden)).astype(np.float32)
            for i in (9, 15):
                wl.weights[16 * l + i] = (1 + 0.2 * rng.randn(spec.shape.hidden)).astype(np.float32)
    eng = make_engine(spec, wl)
    eng.set_deferred_layernorm(False)
    y_ln = run_forward(eng, wl).clone()
    eng.set_deferred_layernorm(True)
    eng.get_profile(reset=True)
    y_def = run_forward(eng, wl).clone()
    prof = eng.get_profile(reset=True)
    assert prof["layernorm"][1] == 1                      # the last layer's, behind the stack
    assert sum(v[1] for v in prof.values()) == 5 + 5 * spec.shape.num_layers + 1
    ref = oracle_valid(wl, spec).double()
    err_ln = (O.valid_rows(y_ln.cpu().double(), wl.mask) - ref).abs()
    err_def = (O.valid_rows(y_def.cpu().double(), wl.mask) - ref).abs()
    if ln_params == "benchmark":
        assert_parity(y_ln, ref, wl.mask, fp16=True)
        assert_parity(y_def, ref, wl.mask, fp16=True)
    else:
        assert float(err_ln.mean()) <= FP16_MEAN_ABS and float(err_def.mean()) <= FP16_MEAN_ABS
        assert float(err_def.max()) <= float(err_ln.max()) + 2e-2, (float(err_def.max()), float(err_ln.max()))
    # twice the same answer, and the replayed pass equals the eager one
    y_again = run_forward(eng, wl)
    assert torch.equal(y_again, y_def)
    x = torch.from_numpy(wl.from_tensor).to(eng.dtype).cuda()
    m = torch.from_numpy(wl.mask).cuda()
    out = torch.empty_like(x)
    eng.capture(x, m, out)
    eng.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, y_def)
    # back to the LayerNorm kernels
    eng.set_deferred_layernorm(False)
    assert torch.equal(run_forward(eng, wl), y_ln)
    eng.close()


def test_hidden_sizes_beyond_the_deferred_layernorm_run_the_layernorm_kernels():
    """hidden 1280 (a multiple of 256 above 1024): the handle falls back to LayerNorm kernels by itself,
    and asking for the deferred form is refused."""
    spec = W.tiny_spec(dtype="fp16", layers=2, heads=20, ffn=1280, batch=4, max_seq_len=24, seed=17)
    wl = W.make_workload(spec, random_gamma_beta=True)
    eng = make_engine(spec, wl)
    eng.get_profile(reset=True)
    y = run_forward(eng, wl)
    assert eng.get_profile(reset=True)["layernorm"][1] == 2 * spec.shape.num_layers
    assert_parity(y, oracle_valid(wl, spec), wl.mask, fp16=True)
    with pytest.raises(_capi.EtError):
        eng.set_deferred_layernorm(True)
    eng.close()


@pytest.mark.parametrize("heads,ffn,layers,batch,seq", [(4, 1024, 3, 9, 40), (8, 2048, 2, 33, 64), (4, 256, 4, 1, 7)])
def test_deferred_layernorm_other_widths(heads, ffn, layers, batch, seq):
    """Hidden sizes 256 and 512 (statistics of 2 and 4 vectors per row), ragged batches down to one
    short sequence: the default path (deferred LayerNorm) against the oracle and against the path
    with LayerNorm kernels."""
    spec = W.tiny_spec(dtype="fp16", layers=layers, heads=heads, ffn=ffn, batch=batch, max_seq_len=seq, seed=11)
    wl = W.make_workload(spec, random_gamma_beta=True)
    eng = make_engine(spec, wl)
    eng.get_profile(reset=True)
    y_def = run_forward(eng, wl).clone()
    prof = eng.get_profile(reset=True)
    assert prof["layernorm"][1] == 1, "the deferred path is the default for these widths"
    eng.set_deferred_layernorm(False)
    y_ln = run_forward(eng, wl).clone()
    ref = oracle_valid(wl, spec)
    assert_parity(y_def, ref, wl.mask, fp16=True)
    assert_parity(y_ln, ref, wl.mask, fp16=True)
    eng.close()


def test_sequences_longer_than_an_attention_tile():
    """max_seq_len 200 on an fp16 handle: the attention kernel for any length (sequences do not fit the
    128-row tiles) between the deferred-LayerNorm projections, and the same batch under a general mask
    (all-ones within the valid keys, so the same answer) through the CUDA-core masked attention."""
    spec = W.tiny_spec(dtype="fp16", layers=2, heads=4, ffn=1024, batch=5, max_seq_len=200, seed=13)
    wl = W.make_workload(spec, random_gamma_beta=True)
    wl.lengths[0] = 200
    wl.mask[:] = W.prefix_mask(wl.lengths, spec.max_seq_len)
    eng = make_engine(spec, wl)
    y = run_forward(eng, wl).clone()
    ref = oracle_valid(wl, spec)
    assert_parity(y, ref, wl.mask, fp16=True)
    am = torch.from_numpy(W.attention_mask_from_input_mask(wl.mask)).half().cuda()
    x = torch.from_numpy(wl.from_tensor).half().cuda()
    m = torch.from_numpy(wl.mask).cuda()
    y2 = eng.forward_general_mask(x, m, am)
    torch.cuda.synchronize()
    assert_parity(y2, ref, wl.mask, fp16=True)
    eng.close()


def test_failed_general_mask_call_does_not_poison_the_next_call():
    """et_layer in general-mask mode that returns early (weights of that layer missing) must leave
    the handle in key-only mode: the next plain call gives the plain result."""
    spec = W.tiny_spec(dtype="fp16", layers=2, batch=5, max_seq_len=16, seed=3)
    wl = W.make_workload(spec, random_gamma_beta=True)
    sh = spec.shape
    eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, sh.size_per_head, sh.ffn_dim, spec.batch,
                                  spec.max_seq_len)
    eng.set_layer_weights(0, wl.weights[:16])            # layer 1 has no weights
    x = torch.from_numpy(wl.from_tensor).half().cuda()
    m = torch.from_numpy(wl.mask).cuda()
    packed, valid, bidx, widx = eng.effective_transformer_input(x, m)
    want = eng.effective_transformer(0, packed, packed, None, valid, bidx, widx).clone()
    torch.cuda.synchronize()
    am = torch.tril(torch.ones(spec.max_seq_len, spec.max_seq_len)).expand(spec.batch, -1, -1).half().cuda().contiguous()
    eng.set_general_mask(True)
    with pytest.raises(et.EtError) as e:
        eng.effective_transformer(1, packed, packed, am, valid, bidx, widx)
    assert e.value.code == _capi.ET_NOT_READY
    eng.set_general_mask(False)
    got = eng.effective_transformer(0, packed, packed, None, valid, bidx, widx)
    torch.cuda.synchronize()
    t = int(valid[0])
    assert torch.equal(got.reshape(-1, sh.hidden)[:t], want.reshape(-1, sh.hidden)[:t])
    eng.close()


def test_workspace_query_matches_what_the_handle_allocated():
    for dtype in ("fp16", "fp32"):
        spec = W.tiny_spec(dtype=dtype, batch=9, max_seq_len=31)
        sh = spec.shape
        eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, sh.size_per_head, sh.ffn_dim, spec.batch,
                                      spec.max_seq_len, dtype=torch.float16 if dtype == "fp16" else torch.float32)
        assert eng.workspace_allocated_bytes() == eng.workspace_bytes(spec.batch, spec.max_seq_len) > 0
        assert eng.workspace_bytes(2, 8) < eng.workspace_bytes(spec.batch, spec.max_seq_len)
        eng.close()


def test_hidden_size_limits_are_checked_at_creation():
    with pytest.raises(et.EtError) as e:
        et.EffectiveTransformer(1, 20, 64, 1280, 2, 8, dtype=torch.float32)       # hidden 1280 > 1024 for fp32
    assert e.value.code == _capi.ET_INVALID_ARGUMENT
    with pytest.raises(et.EtError) as e:
        et.EffectiveTransformer(1, 34, 64, 4352, 2, 8, dtype=torch.float16)       # hidden 2176 > 2048 for fp16
    assert e.value.code == _capi.ET_INVALID_ARGUMENT


def test_bounded_wait_reports_through_the_status_word():
    """Failure detection without a fault: a kernel whose 2 ms wait runs out records its code and
    returns; the host reads and clears it, maps it to ET_DEVICE_TIMEOUT in the host-buffer call,
    and the handle keeps working."""
    spec = W.tiny_spec(dtype="fp16", batch=4, max_seq_len=16, seed=8)
    wl = W.make_workload(spec)
    eng = make_engine(spec, wl)
    want = run_forward(eng, wl).clone()
    eng.selftest_wait_timeout()
    torch.cuda.synchronize()
    assert eng.device_status() == (15 << 8) | 1          # kernel id 15 (self-test), site 1
    assert eng.device_status() == 0                      # reading clears it
    assert torch.equal(run_forward(eng, wl), want)
    # the first recorded code wins, and the host-buffer call turns it into ET_DEVICE_TIMEOUT
    eng.selftest_wait_timeout()
    torch.cuda.synchronize()                             # the host-buffer call runs on the handle's own stream
    with pytest.raises(et.EtError) as e:
        eng.forward_host(wl.from_tensor.astype(np.float16), wl.mask)
    assert e.value.code == _capi.ET_DEVICE_TIMEOUT and "0xf01" in str(e.value)
    y_host, t = eng.forward_host(wl.from_tensor.astype(np.float16), wl.mask)   # cleared: works again
    assert t == wl.valid_tokens and np.array_equal(y_host, want.cpu().numpy())
    eng.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_handles_on_two_devices_of_one_process():
    """Function attributes and the SM count are kept per device: a handle created on cuda:1
    after one on cuda:0 runs the same kernels (each touches only its own device's memory)."""
    spec = W.WORKLOADS[1]
    wl = W.make_workload(spec)
    sub = W.Workload(spec, wl.lengths[:24], wl.mask[:24], wl.from_tensor[:24], wl.weights)
    ref = oracle_valid(sub, spec)
    sh = spec.shape
    for dev_idx in (0, 1):
        with torch.cuda.device(dev_idx):
            eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, sh.size_per_head, sh.ffn_dim, 24,
                                          spec.max_seq_len, device=dev_idx)
            eng.set_weights(sub.weights)
            x = torch.from_numpy(sub.from_tensor).half().cuda(dev_idx)
            m = torch.from_numpy(sub.mask).cuda(dev_idx)
            y = eng.forward(x, m)
            torch.cuda.synchronize(dev_idx)
            assert eng.device_status() == 0
            assert_parity(y, ref, sub.mask, fp16=True)
            eng.close()
