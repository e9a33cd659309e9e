"""GPU tests of CUDA-graph replay of the forward pass.  The valid-token count
stays on the device, so a pass captured for given buffers and (B, S) must give
the eager result, bit for bit, for every batch later written into those
buffers - other lengths, other masks, no valid token at all."""
import numpy as np
import pytest
import torch

import effective_transformer_b200 as et
from effective_transformer_b200 import _capi
from effective_transformer_b200 import workloads as W

pytestmark = pytest.mark.gpu


def engine_for(spec, wl, heads=None):
    tdt = torch.float16 if spec.dtype == "fp16" else torch.float32
    sh = spec.shape
    eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, sh.size_per_head, sh.ffn_dim, spec.batch,
                                  spec.max_seq_len, dtype=tdt)
    eng.set_weights(wl.weights)
    if heads is not None:
        eng.set_embeddings(heads.word_table, heads.type_table, heads.position_table, heads.ln_gamma, heads.ln_beta)
        eng.set_pooler(heads.pooler_kernel, heads.pooler_bias)
    return eng, tdt


def other_batches(spec, rng):
    """(lengths, mask) variants for the same [B, S]: a new draw, a non-prefix mask, an empty batch."""
    b, s = spec.batch, spec.max_seq_len
    new_len = rng.randint(1, s + 1, size=b).astype(np.int32)
    yield W.prefix_mask(new_len, s)
    holes = (rng.rand(b, s) < 0.6).astype(np.int32)
    holes[0] = 0                                             # an empty sequence among them
    yield holes
    yield np.zeros((b, s), np.int32)


@pytest.mark.parametrize("spec", [W.tiny_spec(dtype="fp32"), W.WORKLOADS[1]], ids=["tiny_fp32", "cfg1_fp16"])
def test_replay_equals_eager_for_any_batch_in_the_same_buffers(spec):
    wl = W.make_workload(spec)
    eng, tdt = engine_for(spec, wl)
    x = torch.from_numpy(wl.from_tensor).to(tdt).cuda()
    mask = torch.from_numpy(wl.mask).cuda()
    out = torch.full_like(x, float("nan"))
    eng.capture(x, mask, out)
    eager = eng.forward(x, mask)
    out.fill_(float("nan"))
    eng.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    rng = np.random.RandomState(9)
    for m_np in other_batches(spec, rng):
        x.copy_(torch.from_numpy(rng.randn(*wl.from_tensor.shape).astype(np.float32)).to(tdt))
        mask.copy_(torch.from_numpy(m_np))
        eager = eng.forward(x, mask)
        out.fill_(float("nan"))
        eng.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)
        if m_np.sum() == 0:
            assert bool((out == 0).all())
    assert eng.device_status() == 0
    eng.close()


def test_replay_of_the_model_call_from_ids():
    spec = W.WORKLOADS[1]
    wl = W.make_workload(spec)
    heads = W.make_model_heads(spec, wl.lengths)
    eng, tdt = engine_for(spec, wl, heads)
    b, s, h = spec.batch, spec.max_seq_len, spec.shape.hidden
    ids = torch.from_numpy(heads.input_ids).cuda()
    types = torch.from_numpy(heads.token_type_ids).cuda()
    mask = torch.from_numpy(wl.mask).cuda()
    seq = torch.empty((b, s, h), dtype=tdt, device="cuda")
    pooled = torch.empty((b, h), dtype=tdt, device="cuda")
    eng.capture_ids(ids, mask, types, seq, pooled)
    rng = np.random.RandomState(10)
    for m_np in [wl.mask] + list(other_batches(spec, rng)):
        ids.copy_(torch.from_numpy(rng.randint(0, heads.word_table.shape[0], size=(b, s)).astype(np.int32)))
        mask.copy_(torch.from_numpy(m_np))
        seq_e, pooled_e = eng.forward_ids(ids, mask, types, True, True)
        seq.fill_(float("nan"))
        pooled.fill_(float("nan"))
        eng.replay()
        torch.cuda.synchronize()
        assert torch.equal(seq, seq_e) and torch.equal(pooled, pooled_e)
    # pooled-only capture: the padded tensor is never produced
    eng.capture_ids(ids, mask, types, None, pooled)
    pooled.fill_(float("nan"))
    eng.replay()
    torch.cuda.synchronize()
    assert torch.equal(pooled, pooled_e)
    assert eng.device_status() == 0
    eng.close()


def test_replay_counts_launches_and_needs_a_capture():
    spec = W.tiny_spec(dtype="fp16")
    wl = W.make_workload(spec)
    heads = W.make_model_heads(spec, wl.lengths, 1000, 2, 64)
    eng, tdt = engine_for(spec, wl)
    with pytest.raises(et.EtError) as e:
        eng.replay()
    assert e.value.code == _capi.ET_NOT_READY
    x = torch.from_numpy(wl.from_tensor).to(tdt).cuda()
    mask = torch.from_numpy(wl.mask).cuda()
    out = torch.empty_like(x)
    eng.get_profile(reset=True)
    eng.forward(x, mask, out)
    eager_counts = {k: v[1] for k, v in eng.get_profile(reset=True).items()}
    eng.capture(x, mask, out)
    eng.get_profile(reset=True)
    eng.replay()
    eng.replay()
    torch.cuda.synchronize()
    replay_counts = {k: v[1] for k, v in eng.get_profile(reset=True).items()}
    assert replay_counts == {k: 2 * v for k, v in eager_counts.items()}
    assert sum(eager_counts.values()) == 3 + 7 * spec.shape.num_layers + 1 + 1
    # new embedding tables free the old ones: a captured pass is dropped with them
    eng.set_embeddings(heads.word_table, heads.type_table, heads.position_table, heads.ln_gamma, heads.ln_beta)
    with pytest.raises(et.EtError):
        eng.replay()
    with pytest.raises(ValueError):
        eng.capture(x, mask.to(torch.int64), out)
    eng.close()


def test_host_buffer_call_replays_its_chunks_after_two_calls_of_one_shape(monkeypatch):
    """et_forward_host records one graph per chunk once a shape repeats and replays them from
    then on.  The result must not depend on which path ran: the first (eager) call on a batch
    and the replayed calls agree bit for bit, for every batch pushed through the same shape.
    (Chunk shares fixed: with other shares sequences share attention tiles differently.)"""
    monkeypatch.setenv("ETB_HOST_MID_SHARE", "6")
    spec = W.WORKLOADS[1]
    big = W.WorkloadSpec("cfg1_x8", spec.shape, "fp16", 800, 32, 8, 33, seed=5)   # 39 MB: cut into chunks
    wl = W.make_workload(big)
    rng = np.random.RandomState(12)
    batches = []
    for _ in range(3):
        lens = rng.randint(1, big.max_seq_len + 1, size=big.batch).astype(np.int32)
        batches.append((rng.randn(big.batch, big.max_seq_len, big.shape.hidden).astype(np.float16),
                        W.prefix_mask(lens, big.max_seq_len), int(lens.sum())))
    # eager results from a handle that never sees a shape twice in a row
    eng, tdt = engine_for(big, wl)
    small = wl.from_tensor[:100].astype(np.float16)
    eager = []
    for x, mask, t in batches:
        got, tt = eng.forward_host(x, mask)
        assert tt == t
        eager.append(got.copy())
        eng.forward_host(small, wl.mask[:100])               # another shape in between
    # chunked and whole-batch passes differ only in how sequences share attention tiles
    whole = eng.forward(torch.from_numpy(batches[0][0]).cuda(), torch.from_numpy(batches[0][1]).cuda())
    torch.cuda.synchronize()
    diff = np.abs(eager[0].astype(np.float32) - whole.cpu().numpy().astype(np.float32))
    assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3
    eng.close()
    # a fresh handle fed with the same shape every time: calls 3.. replay the recorded chunks
    eng, tdt = engine_for(big, wl)
    for rep in range(2):
        for (x, mask, t), want in zip(batches, eager):
            got, tt = eng.forward_host(x, mask)
            assert tt == t and np.array_equal(got, want), f"round {rep}"
    assert eng.device_status() == 0
    eng.close()


def test_host_buffer_call_settles_its_chunk_shares(monkeypatch):
    """Without a fixed share the handle tries the shares its model proposes against the default on
    replayed calls and settles within a dozen calls of one shape; every call along the way (eager,
    recording, replayed, with whichever shares) returns a result inside the gate of the whole-batch
    pass, and once settled the calls repeat bit for bit."""
    monkeypatch.delenv("ETB_HOST_MID_SHARE", raising=False)
    spec = W.WORKLOADS[1]
    big = W.WorkloadSpec("cfg1_x8", spec.shape, "fp16", 800, 32, 8, 33, seed=5)   # 39 MB: cut into chunks
    wl = W.make_workload(big)
    eng, tdt = engine_for(big, wl)
    x = wl.from_tensor.astype(np.float16)
    whole = eng.forward(torch.from_numpy(x).cuda(), torch.from_numpy(wl.mask).cuda())
    torch.cuda.synchronize()
    whole = whole.cpu().numpy().astype(np.float32)
    outs = []
    for call in range(14):
        got, tt = eng.forward_host(x, wl.mask)
        assert tt == wl.valid_tokens
        diff = np.abs(got.astype(np.float32) - whole)
        assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 2e-3, f"call {call}"
        outs.append(got.copy())
    chunks, share, measured = eng.host_chunk_shares()
    assert measured and chunks >= 1 and 0 <= share <= 8
    assert np.array_equal(outs[-1], outs[-2]) and np.array_equal(outs[-1], outs[-3])
    assert eng.device_status() == 0
    eng.close()
