#!/usr/bin/env python
"""Benchmark of the padding-free BERT encoder path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one forward pass of the whole path (input op, all encoder layers,
output op) over one batch of synthetic input with the shapes and value
distributions of the reference's benchmark script
(sample/tensorflow/benchmark.py:38-61): BERT-base, 12 layers, fp16, B=1000
sequences, Lmax=64, lengths randint(16, 65).  Metric: valid tokens/s over all
ranks.  Prints one JSON line (rank 0).

With N > 1 the ONE batch of 1000 sequences is sharded by sequence over the N
ranks, token-balanced, no collective in the forward pass ("scaling": "strong");
the figure with 1000 sequences per GPU is reported beside it under "weak".

  value     inputs resident in HBM, per-step CUDA-event time, max over ranks; a step is a replay of
            the pass recorded as a CUDA graph (--launch eager: one et_forward call per step)
  e2e       the same through et_forward_host with pinned HOST buffers: the
            host->device copy of the batch and the device->host copy of the
            [B,S,H] result are inside the timed region
  e2e_from_token_ids  (informational) the same batch given as token ids through
            et_forward_ids_host: embeddings of the valid tokens, the stack and the
            pooler; 12 bytes per position go up, the pooled [B,H] rows come back
  roofline  the tcgen05 GEMM (the dominant kernel): algorithmic FLOPs / CUDA-
            event time of its launches in an eager pass over the same steps.  On fp16
            handles those launches also carry the layers' LayerNorms (none runs as a
            kernel): `step_frac` = the same FLOPs over the whole step's time
  gather    N > 1: the optional gather of the shard outputs to rank 0 over NVLink
            (NCCL send/recv into a local buffer, then the batch order restored), timed
            separately and outside `value`
  other_workloads  N = 1: short passes over the fp32 workload (cfg3) and BERT-large with
            skewed lengths (cfg4)
  cpu_baseline  the CPU oracle (fp32 restatement of the reference's padded TF
            graph) timed on a bounded sample of the same batch, N=1 only
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from effective_transformer_b200 import workloads as W  # noqa: E402

METRIC = "valid_tokens_per_sec"
UNIT = "tokens/s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            with open(p) as f:
                d = json.load(f)
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def read_traffic(workload: str, tokens: int):
    """DRAM bytes per launch of the dominant kernel from the committed ncu capture, if one is on
    record for this workload (profiles/traffic.json; written when the capture is refreshed).  A pass
    over a shard of the workload gets the capture's bytes scaled by the rows it processes: operand
    and output rows grow with the tokens, only the weights (3-5 MB of the 190-255 MB) do not."""
    p = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(p) as f:
            rec = json.load(f).get(workload)
        if rec:
            full, note = float(rec["bytes_per_launch"]), rec.get("note")
            captured = int(rec.get("valid_tokens", tokens))
            if captured != tokens:
                return full * tokens / captured, (note or "") + "; scaled by %d / %d tokens for this shard" % (
                    tokens, captured)
            return full, note
    except Exception:
        pass
    return None, None


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "25"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples that arrived between t_begin and t_end (time.monotonic(); the
        sampler is started ahead of the timed region because nvidia-smi takes a while to come up)."""
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        rows = [r for t, r in self.rows if (t_begin is None or t >= t_begin) and (t_end is None or t <= t_end)]
        if not rows:
            rows = [r for _, r in self.rows]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def measure_matmul_tflops(dev, tf32: bool, n: int = 8192, iters: int = 8) -> float:
    """Rate of the library's fp32 GEMM on this GPU, measured in this run: with tf32=True on the
    tensor cores (kind tf32), with tf32=False on the CUDA cores (SGEMM)."""
    import torch
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = tf32
    try:
        a = torch.randn(n, n, device=dev, dtype=torch.float32)
        b = torch.randn(n, n, device=dev, dtype=torch.float32)
        for _ in range(2):
            torch.matmul(a, b)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(iters):
            torch.matmul(a, b)
        t1.record()
        t1.synchronize()
        return 2.0 * n ** 3 * iters / (t0.elapsed_time(t1) / 1000.0) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def bind_to_gpu_cpus(gpu_index: int):
    """Best effort: run this rank on the host cores next to its GPU (NVML's CPU affinity), so that
    the pinned host buffers it allocates are first touched on that NUMA node."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {i * 64 + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1}
        allowed = cpus & set(os.sched_getaffinity(0))
        if allowed:
            os.sched_setaffinity(0, allowed)
            return len(allowed)
    except Exception:
        pass
    return None


def cpu_oracle_throughput(spec: W.WorkloadSpec, sample_seqs: int):
    """Times the CPU oracle (padded encoder, fp32, all host threads) on the
    first `sample_seqs` sequences of the workload.  Returns (tokens/s, seconds,
    tokens, threads)."""
    import torch
    from oracle import bert_encoder as O
    # all host cores this process may use (torchrun presets OMP_NUM_THREADS=1 for its workers)
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    torch.set_num_threads(max(1, cores))
    wl = W.make_workload(spec, batch_override=sample_seqs)
    am = W.attention_mask_from_input_mask(wl.mask)
    warm = W.Workload(spec, wl.lengths[:4], wl.mask[:4], wl.from_tensor[:4], wl.weights)
    O.transformer_model(warm.from_tensor, am[:4], warm.weights, spec.shape.head_num, spec.shape.size_per_head,
                        round_to_fp16=(spec.dtype == "fp16"))
    t0 = time.perf_counter()
    O.transformer_model(wl.from_tensor, am, wl.weights, spec.shape.head_num, spec.shape.size_per_head,
                        round_to_fp16=(spec.dtype == "fp16"))
    dt = time.perf_counter() - t0
    return wl.valid_tokens / dt, dt, wl.valid_tokens, torch.get_num_threads()


def run_reference(args, spec):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    # a step of the reference arm is a bounded sample, so that K + W steps end within minutes
    sample = args.cpu_sample if args.cpu_sample > 0 else min(256, spec.batch)
    times, toks, threads = [], 0, 1
    for i in range(args.warmup + args.steps):
        tps, dt, toks, threads = cpu_oracle_throughput(spec, sample)
        if i >= args.warmup:
            times.append(dt)
    ms = 1000.0 * sum(times) / len(times)
    value = toks / (ms / 1000.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": spec.name, "note": "CPU port of the reference's padded TF-graph encoder "
                   "(TensorFlow is absent, the reference op cannot be built); each step = the first "
                   f"{sample} sequences of the batch, all layers; tokens/s does not depend on the sample size"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"first {sample} of {spec.batch} sequences, {toks} valid tokens, "
                                   f"{spec.shape.num_layers} layers, padded [B,S] fp32"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


class DevicePass:
    """An engine with one batch resident on the device, and the timing of its pass."""

    def __init__(self, et, torch, spec, lengths, x_np, weights, dev, local):
        self.torch, self.spec = torch, spec
        sh = spec.shape
        self.fp16 = spec.dtype == "fp16"
        self.tdt = torch.float16 if self.fp16 else torch.float32
        self.lengths = lengths.astype(np.int32)
        self.tokens = int(self.lengths.sum())
        self.b, self.s, self.h = len(lengths), spec.max_seq_len, sh.hidden
        self.mask_np = W.prefix_mask(self.lengths, self.s)
        self.eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, sh.size_per_head, sh.ffn_dim, max(self.b, 1),
                                           self.s, dtype=self.tdt, device=local)
        self.eng.set_weights(weights)
        if x_np is None:    # N(0,1) input drawn on the device (timing passes over the large workloads)
            gen = torch.Generator(device=dev).manual_seed(spec.seed)
            self.x = torch.randn((self.b, self.s, self.h), generator=gen, device=dev, dtype=torch.float32).to(self.tdt)
        else:
            self.x = torch.from_numpy(np.ascontiguousarray(x_np)).to(self.tdt).to(dev)
        self.mask = torch.from_numpy(self.mask_np).to(dev)
        self.out = torch.empty_like(self.x)

    def gemm_flops(self) -> float:
        sh = self.spec.shape
        return 2.0 * self.tokens * self.h * (3 * self.h + self.h + 2 * sh.ffn_dim) * sh.num_layers

    def time(self, steps, warmup, launch, flush, barrier, sampler=None):
        """Returns (sum of step ms, per-kernel profile of an eager pass over the same steps, clocks)."""
        torch, eng = self.torch, self.eng
        if sampler is not None:
            sampler.start()
        for _ in range(warmup):
            eng.forward(self.x, self.mask, self.out)
        torch.cuda.synchronize()
        assert eng.device_status() == 0, "a device-side wait expired during warm-up"
        graph = launch == "graph"
        if graph:
            eng.capture(self.x, self.mask, self.out)
            for _ in range(2):
                eng.replay()
            torch.cuda.synchronize()
        eng.get_profile(reset=True)
        eng.set_profiling(not graph)
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        barrier()
        t_begin = time.monotonic()
        for i in range(steps):
            flush.zero_()                         # evict the previous step's tensors from L2 (untimed)
            starts[i].record()
            if graph:
                eng.replay()
            else:
                eng.forward(self.x, self.mask, self.out)
            ends[i].record()
        barrier()
        clocks = sampler.stop(t_begin, time.monotonic()) if sampler is not None else None
        eng.set_profiling(False)
        total_ms = sum(a.elapsed_time(e) for a, e in zip(starts, ends))
        prof = eng.get_profile(reset=True)
        if graph:
            # replayed kernels cannot be bracketed by events: per-kernel times from an eager pass of the same steps
            replayed = {k: v[1] for k, v in prof.items()}
            eng.set_profiling(True)
            for i in range(steps):
                flush.zero_()
                eng.forward(self.x, self.mask, self.out)
            torch.cuda.synchronize()
            eng.set_profiling(False)
            prof = eng.get_profile(reset=True)
            assert {k: v[1] for k, v in prof.items()} == replayed
            eng.release_graph()
        assert eng.device_status() == 0, "a device-side wait expired during the timed steps"
        return total_ms, prof, clocks

    def close(self):
        self.eng.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", type=int, default=2, help="index into the five benchmark configurations")
    ap.add_argument("--scaling", default="auto", choices=["auto", "weak", "strong"],
                    help="N > 1: strong = the one batch sharded over the ranks (default), weak = a batch per rank")
    ap.add_argument("--launch", default="graph", choices=["graph", "eager"],
                    help="a timed step is a CUDA-graph replay of the pass (et_graph_launch) or one et_forward call")
    ap.add_argument("--cpu-sample", type=int, default=0,
                    help="sequences in the CPU sample; 0 = 512 for the cpu_baseline leg (about 5 s on 16 cores), "
                         "256 per step for --impl reference")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-other", action="store_true", help="skip the cfg3 / cfg4 passes (N = 1)")
    ap.add_argument("--no-gather", action="store_true", help="skip the output gather and the weak figure (N > 1)")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="one GPU only: time rank 0's shard of an N-way split of the batch (what one rank of "
                         "`--gpus N` runs), to study the small-batch regime without N GPUs")
    ap.add_argument("--deferred-layernorm", type=int, default=-1,
                    help="A/B: 1 / 0 = et_set_deferred_layernorm on / off (default: the library's default)")
    ap.add_argument("--fused-layernorm", action="store_true",
                    help="A/B: the LayerNorms inside the projection kernels (et_set_fused_layernorm) instead of a "
                         "LayerNorm kernel behind each projection")
    args = ap.parse_args()
    spec = W.WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, spec)
        return

    import torch
    import torch.distributed as dist
    import effective_transformer_b200 as et

    rank, world, local = dist_env()
    cpus_bound = bind_to_gpu_cpus(local) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    scaling = args.scaling if args.scaling != "auto" else ("strong" if world > 1 else "weak")

    # ---- workload: the one batch sharded over the ranks (strong) or a batch per rank (weak) -------
    base = W.make_workload(spec)                      # canonical draw: lengths, input, weights
    shards = None
    if world == 1 and args.shard_of > 1:
        one, _ = W.balanced_shards(base.lengths, args.shard_of)
        lengths, x_np = base.lengths[one[0]], base.from_tensor[one[0]]
    elif world == 1:
        lengths, x_np = base.lengths, base.from_tensor
    elif scaling == "strong":
        shards, _ = W.balanced_shards(base.lengths, world)
        lengths, x_np = base.lengths[shards[rank]], base.from_tensor[shards[rank]]
    else:
        g = np.random.RandomState(spec.seed + 101)
        all_len = np.concatenate([base.lengths] + [W.draw_lengths(spec, g) for _ in range(world - 1)])
        wshards, _ = W.balanced_shards(all_len, world)
        lengths = all_len[wshards[rank]].astype(np.int32)
        x_np = np.random.RandomState(spec.seed + 17 + rank).randn(
            len(lengths), spec.max_seq_len, spec.shape.hidden).astype(np.float32)
    sh = spec.shape
    fp16 = spec.dtype == "fp16"
    main_pass = DevicePass(et, torch, spec, lengths, x_np, base.weights, dev, local)
    if args.fused_layernorm:
        main_pass.eng.set_fused_layernorm(True)
    if args.deferred_layernorm >= 0:
        main_pass.eng.set_deferred_layernorm(bool(args.deferred_layernorm))
    eng, b, s, h = main_pass.eng, main_pass.b, main_pass.s, main_pass.h
    tokens_rank = main_pass.tokens
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > 126 MB L2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ------------------------------------------------
    total_ms, prof, clocks = main_pass.time(args.steps, args.warmup, args.launch, flush, barrier,
                                            ClockSampler(local) if rank == 0 else None)

    # ---- end to end through the host-buffer entry point -----------------------
    e2e_ms = None
    esz = main_pass.x.element_size()
    h2d = b * s * h * esz + b * s * 4
    d2h = b * s * h * esz + 8
    shares = None
    if not args.no_e2e:
        x_host = torch.from_numpy(np.ascontiguousarray(x_np)).to(main_pass.tdt).pin_memory()
        m_host = torch.from_numpy(main_pass.mask_np).pin_memory()
        o_host = torch.empty_like(x_host).pin_memory()
        xh, mh, oh = x_host.numpy(), m_host.numpy(), o_host.numpy()
        barrier()
        # calls of one shape until the handle has settled its chunk shares: eager, record, two replays
        # timed with the default shares; the same four with the shares its model proposes; and, if those
        # lose, two more to go back: from the 11th call on every call replays the final choice
        for _ in range(12):
            eng.forward_host(xh, mh, oh)
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            eng.forward_host(xh, mh, oh)
        torch.cuda.synchronize()
        e2e_ms = 1000.0 * (time.perf_counter() - t0)
        barrier()
        shares = eng.host_chunk_shares()

    # ---- the same batch as token ids: embeddings in front, pooler behind ------------
    # (not the headline: ids + mask go up, only the pooled [B,H] rows come back)
    ids_ms = None
    if not args.no_e2e:
        mh_ = W.make_model_heads(spec, lengths)
        eng.set_embeddings(mh_.word_table, mh_.type_table, mh_.position_table, mh_.ln_gamma, mh_.ln_beta)
        eng.set_pooler(mh_.pooler_kernel, mh_.pooler_bias)
        pin = lambda a: torch.from_numpy(a).pin_memory().numpy()
        ids_h, types_h, mask_h = pin(mh_.input_ids), pin(mh_.token_type_ids), pin(main_pass.mask_np)
        for _ in range(2):
            eng.forward_ids_host(ids_h, mask_h, types_h, sequence_output=False, pooled_output=True)
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            eng.forward_ids_host(ids_h, mask_h, types_h, sequence_output=False, pooled_output=True)
        torch.cuda.synchronize()
        ids_ms = 1000.0 * (time.perf_counter() - t0)
        barrier()

    # ---- N > 1: the optional output gather (timed separately) and the weak figure ----------------
    gather_info, weak_info = None, None
    if world > 1 and scaling == "strong" and not args.no_gather:
        from effective_transformer_b200.sharding import OutputGather
        eng.forward(main_pass.x, main_pass.mask, main_pass.out)
        torch.cuda.synchronize()
        gather = OutputGather(shards, s, h, main_pass.tdt, dev, dst=0)
        for _ in range(3):
            full = gather(main_pass.out)
        g0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        g1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        barrier()
        for i in range(args.steps):
            g0[i].record()
            full = gather(main_pass.out)
            g1[i].record()
        barrier()
        gather_ms = sum(a.elapsed_time(e) for a, e in zip(g0, g1)) / args.steps
        gm = torch.tensor([gather_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(gm, op=dist.ReduceOp.MAX)
        # transport check: an exact integer checksum of every rank's block, before and after
        mine = main_pass.out.view(torch.int16).to(torch.int64).sum().reshape(1)
        sums = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(sums, mine)
        # a batch per GPU (the weak-scaling figure); rank 0 runs the unsharded batch itself, which is
        # also what the gathered tensor is compared with
        if rank == 0:
            wl_len, wl_x = base.lengths, base.from_tensor
        else:
            rg = np.random.RandomState(spec.seed + 101 + rank)
            wl_len = W.draw_lengths(spec, rg)
            wl_x = rg.randn(len(wl_len), spec.max_seq_len, h).astype(np.float32)
        weak_pass = DevicePass(et, torch, spec, wl_len, wl_x, base.weights, dev, local)
        w_ms, _, _ = weak_pass.time(args.steps, args.warmup, args.launch, flush, barrier)
        wstats = torch.tensor([w_ms, float(weak_pass.tokens)], dtype=torch.float64, device=dev)
        wmx, wsm = wstats.clone(), wstats.clone()
        dist.all_reduce(wmx, op=dist.ReduceOp.MAX)
        dist.all_reduce(wsm, op=dist.ReduceOp.SUM)
        weak_info = {"value": float(wsm[1]) / (float(wmx[0]) / args.steps / 1000.0), "unit": UNIT,
                     "ms_per_step": float(wmx[0]) / args.steps, "sequences_per_gpu": spec.batch,
                     "valid_tokens_total": int(wsm[1])}
        if rank == 0:
            off = gather.offsets
            transport_ok = all(
                int(gather.recv[int(off[r]):int(off[r + 1])].view(torch.int16).to(torch.int64).sum()) == int(sums[r])
                for r in range(world))
            y_single = weak_pass.eng.forward(weak_pass.x, weak_pass.mask)
            torch.cuda.synchronize()
            valid = torch.from_numpy(base.mask.ravel() > 0).to(dev)
            d = (full.float() - y_single.float()).abs().reshape(-1, h)[valid]
            gather_info = {
                "ms": float(gm[0]), "bytes": gather.bytes_received,
                "gb_per_s": gather.bytes_received / (float(gm[0]) / 1000.0) / 1e9,
                "what": "padded [b_r,S,H] outputs of all ranks -> rank 0 (NCCL send/recv into a local buffer), "
                        "then the batch order restored by a row gather; outside `value`",
                "transport_bit_exact": bool(transport_ok),
                "vs_single_gpu_max_abs": float(d.max()), "vs_single_gpu_mean_abs": float(d.mean()),
                "padding_rows_zero": bool(torch.all(full.reshape(-1, h)[~valid] == 0))}
        weak_pass.close()

    # ---- reduce over ranks -------------------------------------------------------
    stats = torch.tensor([total_ms, e2e_ms or 0.0, float(tokens_rank), ids_ms or 0.0], dtype=torch.float64,
                         device=dev)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, e2e_total_ms, tokens_all, ids_total_ms = float(mx[0]), float(mx[1]), float(sm[2]), float(mx[3])
    else:
        e2e_total_ms, tokens_all, ids_total_ms = float(stats[1]), float(stats[2]), float(stats[3])

    if rank == 0:
        peaks, peak_src = read_peaks()
        ms_per_step = total_ms / args.steps
        value = tokens_all / (ms_per_step / 1000.0)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None,
            "dtype": "f16" if fp16 else "f32", "data": "synthetic",
            "config": {"workload": spec.name, "sequences_rank0": b, "max_seq_len": s,
                       "valid_tokens_rank0": tokens_rank, "valid_tokens_total": int(tokens_all),
                       "layers": sh.num_layers, "hidden": h,
                       "sharding": ("one batch of %d sequences split over %d ranks, token-balanced, no collective "
                                    "in the forward pass" % (spec.batch, world)) if scaling == "strong" and world > 1
                                   else "sequences, token-balanced, no collective",
                       "l2": "256 MB buffer written between timed steps (untimed)",
                       "layernorm": ("inside the projection kernels" if args.fused_layernorm
                                     else "LayerNorm kernels behind the projections" if args.deferred_layernorm == 0
                                     else "deferred: row statistics from the producing projection, gamma folded "
                                          "into the consuming one, one LayerNorm kernel behind the last layer"
                                     if fp16 else "LayerNorm kernels behind the projections"),
                       "launch": ("cuda-graph replay (et_graph_launch); per-kernel times from a second, eager pass"
                                  if args.launch == "graph"
                                  else "eager (et_forward), per-kernel events inside the timed steps")},
            "roofline": dict(roofline_of(main_pass, prof, args.steps, peaks, peak_src, dev, spec.name),
                             # the whole step against the same peak: projections' FLOPs / the step's time
                             step_frac=(main_pass.gemm_flops() / (ms_per_step / 1000.0) / 1e12 /
                                        peaks["bf16_tflops_sustained"]) if fp16 and ms_per_step > 0 else None),
            "kernels": {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[1] / args.steps}
                        for k, v in prof.items()},
            "gpu_launches": sum(v[1] for v in prof.values()),
            "clocks": clocks,
        }
        if cpus_bound:
            line["config"]["host_cores_bound_per_rank"] = cpus_bound
        if args.shard_of > 1:
            line["config"]["shard_of"] = args.shard_of
        if e2e_ms is not None:
            line["e2e"] = {"value": tokens_all / (e2e_total_ms / args.steps / 1000.0), "unit": UNIT,
                           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                           "ms_per_step": e2e_total_ms / args.steps,
                           "host_chunk_shares": None if shares is None else
                           {"chunks": shares[0] if shares[1] > 0 else 1,
                            "shares": ("1:%d:1" % shares[1]) if shares[1] > 0 else "one piece",
                            "measured_by_handle": shares[2]}}
        if ids_ms is not None:
            line["e2e_from_token_ids"] = {
                "value": tokens_all / (ids_total_ms / args.steps / 1000.0), "unit": UNIT,
                "ms_per_step": ids_total_ms / args.steps, "h2d_bytes_per_step": 3 * b * s * 4,
                "d2h_bytes_per_step": b * h * esz + 8,
                "call": "et_forward_ids_host: ids/types/mask up, embeddings for valid tokens only, "
                        "stack, pooler; pooled [B,H] down"}
        if gather_info is not None:
            line["gather"] = gather_info
        if weak_info is not None:
            line["weak"] = weak_info
    main_pass.close()

    # ---- N = 1: the other single-GPU workloads, short passes ---------------------------------------
    if rank == 0 and world == 1 and not args.no_other and args.workload == 2 and args.shard_of <= 1:
        del main_pass
        torch.cuda.empty_cache()
        other = {}
        for idx in (3, 4):
            ospec = W.WORKLOADS[idx]
            # canonical lengths (same valid-token count and tile packing); weights from the fast float32
            # generator and the N(0,1) input drawn on the device: same shapes and distributions
            owl = W.make_workload_fast(ospec, with_input=False)
            op = DevicePass(et, torch, ospec, owl.lengths, None, owl.weights, dev, local)
            o_steps = max(3, min(5, args.steps))
            o_ms, o_prof, _ = op.time(o_steps, 3, args.launch, flush, barrier)
            other[ospec.name] = {
                "ms_per_step": o_ms / o_steps, "value": op.tokens / (o_ms / o_steps / 1000.0), "unit": UNIT,
                "steps": o_steps, "valid_tokens": op.tokens, "dtype": "f16" if ospec.dtype == "fp16" else "f32",
                "roofline": roofline_of(op, o_prof, o_steps, peaks, peak_src, dev, ospec.name),
                "kernels_ms_per_step": {k: v[0] / o_steps for k, v in o_prof.items() if v[1]}}
            op.close()
            del op, owl
            torch.cuda.empty_cache()
        line["other_workloads"] = other

    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            n_cpu = args.cpu_sample if args.cpu_sample > 0 else min(512, spec.batch)
            tps, dt, toks, threads = cpu_oracle_throughput(spec, n_cpu)
            line["cpu_baseline"] = {
                "value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                "sample": f"first {n_cpu} of {spec.batch} sequences ({toks} valid tokens), "
                          f"{sh.num_layers} layers, padded [B,S] fp32 on the host, {dt:.1f} s"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def roofline_of(p: DevicePass, prof, steps, peaks, peak_src, dev, workload_name):
    """Roofline of the dominant kernel (the projections' GEMM) from the eager pass's events."""
    gemm_cats = ["gemm_qkv", "gemm_attn_out", "gemm_ffn1", "gemm_ffn2"]
    gemm_ms = sum(prof[c][0] for c in gemm_cats)
    gemm_launches = sum(prof[c][1] for c in gemm_cats)
    flops_step = p.gemm_flops()
    achieved = (flops_step * steps) / (gemm_ms / 1000.0) / 1e12 if gemm_ms > 0 else None
    out = {"bound": "tensor", "achieved": achieved, "unit": "TFLOP/s"}
    if p.fp16:
        peak_tf, note = peaks["bf16_tflops_sustained"], peak_src + " bf16_tflops_sustained"
        traffic, tnote = read_traffic(workload_name, p.tokens)
        out.update({"traffic": traffic, "traffic_note": tnote,
                    "kernel": "gemm_tcgen05_pair_kernel (bias / GELU / residual / LayerNorm epilogues)"})
    else:
        # every fp32 product is three tf32 tensor-core products, so the ceiling in fp32 FLOPs is the
        # tf32 rate / 3; the tf32 rate is the library's tf32 GEMM measured in this run on this GPU
        tf32 = measure_matmul_tflops(dev, tf32=True)
        peak_tf = tf32 / 3.0
        note = "tf32 matmul measured in this run (%.0f TFLOP/s) / 3 products per fp32 product" % tf32
        out.update({"traffic": None, "kernel": "gemm_tf32x3_pair_kernel (+ split_tf32_kernel)",
                    "tf32_matmul_tflops_measured_here": tf32,
                    "cublas_sgemm_tflops_measured_here": measure_matmul_tflops(dev, tf32=False, iters=3)})
    ln_launches = prof.get("layernorm", (0.0, 0))[1] / max(steps, 1)
    if p.fp16 and ln_launches <= 1.5:
        # the default of fp16 handles: the projections' epilogues also do the LayerNorms' work (row
        # statistics, normalised residuals), so the launches timed here are longer than a bare GEMM's
        out["note"] = ("no LayerNorm kernel between the projections: their work is inside these launches "
                       "(bench.py --deferred-layernorm 0 times the projections with LayerNorm kernels beside them)")
    out.update({"peak": peak_tf, "frac": (achieved / peak_tf) if (achieved and peak_tf) else None,
                "algorithmic_flops_per_launch": flops_step / max(gemm_launches / steps, 1),
                "launches_per_step": gemm_launches / steps,
                "avg_launch_ms": gemm_ms / max(gemm_launches, 1), "peak_source": note})
    return out


if __name__ == "__main__":
    main()
