"""CPU tests of the host-side logic: the C-ABI library loads and exports every
symbol the header declares, the synthetic workloads, the token-balanced shard
planner, and the multi-rank bookkeeping over gloo (world sizes 2 and 8)."""
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from effective_transformer_b200 import _capi
from effective_transformer_b200 import workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "et_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(et_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _capi.load()
    names = header_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/et_b200.h but not exported"
    assert sorted(_capi.SIGNATURES) == names, "ctypes prototypes and header are out of sync"


def test_handle_less_argument_checks_need_no_gpu():
    lib = _capi.load()
    # argument validation happens before any CUDA call
    assert lib.et_create(None, None) == _capi.ET_INVALID_ARGUMENT
    assert lib.et_padding_offsets(None, -1, 4, None, None, None, None, None, None, None, None, None) \
        == _capi.ET_INVALID_ARGUMENT
    assert lib.et_gemm(_capi.ET_FP16, None, None, None, None, None, None, 4, 128, 64, 0, 0, None, None) \
        == _capi.ET_INVALID_ARGUMENT
    assert lib.et_destroy(None) == _capi.ET_OK


def test_workload_recipe():
    spec = W.WORKLOADS[0]
    wl = W.make_workload(spec)
    assert wl.from_tensor.shape == (8, 32, 768) and wl.valid_tokens == 134
    assert len(wl.weights) == 16 * 12
    assert wl.weights[W.W_INTER_KERNEL].shape == (768, 3072) and wl.weights[W.W_OUT_KERNEL].shape == (3072, 768)
    assert np.all(wl.weights[W.W_ATT_LN_GAMMA] == 1) and np.all(wl.weights[W.W_OUT_LN_BETA] == 0)
    am = W.attention_mask_from_input_mask(wl.mask)
    assert am.shape == (8, 32, 32) and np.array_equal(am[3, 0], wl.mask[3]) and np.array_equal(am[3, 31], wl.mask[3])
    sub = W.make_workload(spec, batch_override=3)
    assert np.array_equal(sub.from_tensor, wl.from_tensor[:3]) and np.array_equal(sub.weights[5], wl.weights[5])
    # FLOP accounting of the headline configuration: 6.823e12 per batch
    lens = W.draw_lengths(W.WORKLOADS[2], np.random.RandomState(0))
    assert abs(W.algorithmic_flops(W.BERT_BASE, lens) / 6.823e12 - 1) < 1e-3


def test_balanced_shards():
    for cfg, tol in ((2, 0.002), (4, 0.002)):
        spec = W.WORKLOADS[cfg]
        lens = W.draw_lengths(spec, np.random.RandomState(spec.seed))
        for g in (1, 2, 4, 8):
            shards, loads = W.balanced_shards(lens, g)
            allidx = np.concatenate(shards)
            assert sorted(allidx.tolist()) == list(range(spec.batch))      # a partition
            assert int(loads.sum()) == int(lens.sum())
            assert (loads.max() - loads.min()) <= tol * loads.mean() + 128   # token-balanced
            for sh in shards:
                assert np.all(np.diff(sh) > 0)                               # batch order kept


RANK_SCRIPT = r'''
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from effective_transformer_b200 import workloads as W
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
spec = W.WORKLOADS[int(sys.argv[2])]
lens = W.draw_lengths(spec, np.random.RandomState(spec.seed))
shards, loads = W.balanced_shards(lens, world)
mine = lens[shards[rank]]
# the same reduction bench.py performs: MAX of times, SUM of tokens
stats = torch.tensor([10.0 + rank, float(mine.sum())], dtype=torch.float64)
mx, sm = stats.clone(), stats.clone()
dist.all_reduce(mx, op=dist.ReduceOp.MAX)
dist.all_reduce(sm, op=dist.ReduceOp.SUM)
assert float(mx[0]) == 10.0 + world - 1
assert int(sm[1]) == int(lens.sum()), (int(sm[1]), int(lens.sum()))
assert int(mine.sum()) == int(loads[rank])
# every rank owns a disjoint set of sequences
owned = torch.zeros(spec.batch, dtype=torch.int32)
owned[torch.from_numpy(shards[rank])] = 1
dist.all_reduce(owned)
assert bool(torch.all(owned == 1))
# the optional output gather: every rank's padded block goes to rank 0, which restores the batch order
from effective_transformer_b200.sharding import OutputGather, inverse_order
S, H = 4, 8
gather = OutputGather(shards, S, H, torch.float32, torch.device("cpu"), dst=0)
local = torch.from_numpy(shards[rank].astype(np.float32)).reshape(-1, 1, 1).expand(-1, S, H).contiguous()
for _ in range(2):                      # buffers are reused from call to call
    full = gather(local)
if rank == 0:
    want = torch.arange(spec.batch, dtype=torch.float32).reshape(-1, 1, 1).expand(-1, S, H)
    assert torch.equal(full, want)
    assert gather.bytes_received == (spec.batch - len(shards[0])) * S * H * 4
else:
    assert full is None
inv = inverse_order(shards)
assert np.array_equal(np.concatenate(shards)[inv], np.arange(spec.batch))
dist.destroy_process_group()
sys.stdout.write("rank%d-ok\n" % rank)
sys.stdout.flush()
'''


@pytest.mark.parametrize("world,cfg,port", [(2, 1, 29533), (8, 2, 29534)])
def test_sharding_over_gloo(tmp_path, world, cfg, port):
    """Two ranks on the small configuration, eight on the B=1000 benchmark batch."""
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=%d" % world,
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT, str(cfg)],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    for k in range(world):
        assert r.stdout.count("rank%d-ok" % k) == 1, r.stdout


def test_reference_arm_prints_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", "--workload", "0", "--cpu-sample", "2"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    import json
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "valid_tokens_per_sec"
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0
    assert line["value"] > 0
