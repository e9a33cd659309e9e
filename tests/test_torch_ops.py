"""The three operators as PyTorch custom ops (effective_transformer_b200/torch_ops.py):
the shape rules of the reference's TF op registrations
(tf_op/bert_transformer_op.cc:44-77, 249-274, 359-380) on CPU with fake tensors,
and the ops against the engine's own methods on the GPU."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import effective_transformer_b200.torch_ops as ops
from effective_transformer_b200 import workloads as W

NS = torch.ops.effective_transformer_b200


def test_ops_are_registered_with_the_reference_signatures():
    s_in = str(NS.effective_transformer_input.default._schema)
    s_layer = str(NS.effective_transformer.default._schema)
    s_out = str(NS.effective_transformer_output.default._schema)
    assert "Tensor from_tensor, Tensor mask" in s_in and "-> Tensor[]" in s_in
    assert "Tensor from_tensor, Tensor to_tensor, Tensor? attention_mask, Tensor valid_word_num, " \
           "Tensor batch_idx, Tensor word_idx" in s_layer and "-> Tensor" in s_layer
    assert "Tensor from_tensor, Tensor valid_word_num, Tensor batch_idx, Tensor word_idx" in s_out


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_shape_functions_with_fake_tensors(dtype):
    b, s, h = 7, 33, 768
    with FakeTensorMode():
        x = torch.empty((b, s, h), dtype=dtype, device="cuda")
        mask = torch.empty((b, s), dtype=torch.int32, device="cuda")
        to_tensor, valid, bidx, widx = NS.effective_transformer_input(0, x, mask)
        assert to_tensor.shape == (b, s, h) and to_tensor.dtype == dtype and to_tensor.device.type == "cuda"
        assert valid.shape == (1,) and valid.dtype == torch.int32
        assert bidx.shape == (b, s) and widx.shape == (b, s) and bidx.dtype == torch.int32
        am = torch.empty((b, s, s), dtype=dtype, device="cuda")
        y = NS.effective_transformer(0, 3, to_tensor, to_tensor, am, valid, bidx, widx)
        assert y.shape == (b, s, h) and y.dtype == dtype
        y = NS.effective_transformer(0, 3, to_tensor, to_tensor, None, valid, bidx, widx)
        out = NS.effective_transformer_output(0, y, valid, bidx, widx)
        assert out.shape == (b, s, h) and out.dtype == dtype
        # the checks of the TF shape functions / OP_REQUIRES
        with pytest.raises(Exception):
            NS.effective_transformer_input(0, x.reshape(b * s, h), mask)          # rank 2
        with pytest.raises(Exception):
            NS.effective_transformer_input(0, x, mask[:, :5])                     # mask shape
        with pytest.raises(Exception):
            NS.effective_transformer(0, 0, to_tensor, to_tensor[:, :8], None, valid, bidx, widx)   # seq lengths differ


def test_unknown_engine_id_is_an_error():
    with pytest.raises(RuntimeError):
        ops._engine(123456)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["fp16", "fp32"])
def test_ops_equal_the_engine_methods(dtype):
    import effective_transformer_b200 as et
    spec = W.tiny_spec(dtype=dtype)
    wl = W.make_workload(spec, random_gamma_beta=True)
    sh = spec.shape
    tdt = torch.float16 if dtype == "fp16" else torch.float32
    eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, sh.size_per_head, sh.ffn_dim, spec.batch,
                                  spec.max_seq_len, dtype=tdt)
    eng.set_weights(wl.weights)
    eid = ops.register_engine(eng)
    x = torch.from_numpy(wl.from_tensor).to(tdt).cuda()
    m = torch.from_numpy(wl.mask).cuda()
    want = eng.forward(x, m)
    got = ops.get_sequence_output(eid, sh.num_layers, None, m, x)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # traced: the ops stay opaque nodes with known shapes
    gm = torch.fx.experimental.proxy_tensor.make_fx(
        lambda a, b: ops.get_sequence_output(eid, sh.num_layers, None, b, a), tracing_mode="fake")(x, m)
    names = [n.target.__name__ if hasattr(n.target, "__name__") else str(n.target) for n in gm.graph.nodes
             if n.op == "call_function"]
    assert sum("effective_transformer" in str(n) for n in names) >= sh.num_layers + 2
    assert torch.equal(gm(x, m), want)
    torch.library.opcheck(NS.effective_transformer_input.default, (eid, x, m),
                          test_utils=("test_schema", "test_faketensor"))
    ops.unregister_engine(eid)
    with pytest.raises(RuntimeError):
        ops.get_sequence_output(eid, sh.num_layers, None, m, x)
    eng.close()
