#!/usr/bin/env python
"""Benchmark of the padding-free BERT encoder path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one forward pass of the whole path (input op, all encoder layers,
output op) over one batch of synthetic input with the shapes and value
distributions of the reference's benchmark script
(sample/tensorflow/benchmark.py:38-61): BERT-base, 12 layers, fp16, B=1000
sequences per GPU, Lmax=64, lengths randint(16, 65).  Metric: valid tokens/s
over all ranks.  Prints one JSON line (rank 0).

  value     inputs resident in HBM, per-step CUDA-event time, max over ranks
  e2e       the same through et_forward_host with pinned HOST buffers: the
            host->device copy of the batch and the device->host copy of the
            [B,S,H] result are inside the timed region
  e2e_from_token_ids  (informational) the same batch given as token ids through
            et_forward_ids_host: embeddings of the valid tokens, the stack and the
            pooler; 12 bytes per position go up, the pooled [B,H] rows come back
  roofline  the tcgen05 GEMM (the dominant kernel): algorithmic FLOPs / CUDA-
            event time of its launches inside the timed steps
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
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised in profiles/gemm_tcgen05_cfg2_ncu.md: mean of the FFN1 launch (66.1 + 189.2 MB)
# and the QKV launch (64.9 + 129.4 MB) of the headline workload.
NCU_GEMM_TRAFFIC = {"cfg2_base_fp16_b1000_s64": 224.8e6}
NCU_GEMM_TRAFFIC_NOTE = ("bytes per launch, ncu dram read+write, mean of the captured FFN1 and QKV launches; their "
                         "algorithmic bytes (A + W + C) are 310.2e6 and 247.9e6 (part of C is still in L2 at kernel end)")
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
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
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


def measure_fp32_gemm_tflops(dev, n: int = 8192, iters: int = 5) -> float:
    """FP32 rate of the CUDA cores as cuBLAS reaches it (TF32 disabled): the roofline
    denominator of the fp32 workloads, whose GEMMs do not use tensor cores."""
    import torch
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        a = torch.randn(n, n, device=dev, dtype=torch.float32)
        b = torch.randn(n, n, device=dev, dtype=torch.float32)
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
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": spec.name, "note": "CPU port of the reference's padded TF-graph encoder "
                   "(TensorFlow is absent, the reference op cannot be built); each step = the first "
                   f"{sample} sequences of the batch, all layers"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"first {sample} of {spec.batch} sequences, {toks} valid tokens, "
                                   f"{spec.shape.num_layers} layers, padded [B,S] fp32"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", type=int, default=2, help="index into the five benchmark configurations")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--cpu-sample", type=int, default=0,
                    help="sequences in the CPU sample; 0 = 512 for the cpu_baseline leg (about 5 s on 16 cores), "
                         "256 per step for --impl reference")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--graph", action="store_true",
                    help="time CUDA-graph replays of the pass (et_graph_capture); the per-kernel roofline then comes "
                         "from a second, eager pass of the same steps")
    args = ap.parse_args()
    spec = W.WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, spec)
        return

    import torch
    import torch.distributed as dist
    import effective_transformer_b200 as et

    rank, world, local = dist_env()
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    # Host-buffer path: chunk shares 1:6:1 are the measured best for one process per host; from
    # four ranks on, the ranks share PCIe switches and host memory, the middle chunk's upload no
    # longer hides behind the first chunk's pass, and the wider first chunk (1:2:1) is kept, the
    # setting the 4- and 8-GPU end-to-end figures were measured with.
    if world >= 4:
        os.environ.setdefault("ETB_HOST_MID_SHARE", "2")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)

    # ---- workload: B sequences per GPU (weak) or B in total (strong) ----------
    base = W.make_workload(spec)                      # canonical draw: lengths, input, weights
    if world == 1:
        lengths, x_np = base.lengths, base.from_tensor
    else:
        if args.scaling == "weak":
            g = np.random.RandomState(spec.seed + 101)
            all_len = np.concatenate([base.lengths] + [W.draw_lengths(spec, g) for _ in range(world - 1)])
        else:
            all_len = base.lengths
        shards, loads = W.balanced_shards(all_len, world)
        lengths = all_len[shards[rank]].astype(np.int32)
        x_np = np.random.RandomState(spec.seed + 17 + rank).randn(
            len(lengths), spec.max_seq_len, spec.shape.hidden).astype(np.float32)
    mask_np = W.prefix_mask(lengths, spec.max_seq_len)
    tokens_rank = int(lengths.sum())
    b, s, h = len(lengths), spec.max_seq_len, spec.shape.hidden
    fp16 = spec.dtype == "fp16"
    tdt, ndt = (torch.float16, np.float16) if fp16 else (torch.float32, np.float32)

    sh = spec.shape
    eng = et.EffectiveTransformer(sh.num_layers, sh.head_num, sh.size_per_head, sh.ffn_dim, b, s, dtype=tdt,
                                  device=local)
    eng.set_weights(base.weights)
    x = torch.from_numpy(x_np).to(tdt).to(dev)
    mask = torch.from_numpy(mask_np).to(dev)
    out = torch.empty_like(x)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > 126 MB L2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ------------------------------------------------
    for _ in range(args.warmup):
        eng.forward(x, mask, out)
    torch.cuda.synchronize()
    assert eng.device_status() == 0, "a device-side wait expired during warm-up"
    if args.graph:
        eng.capture(x, mask, out)
        for _ in range(2):
            eng.replay()
        torch.cuda.synchronize()
    eng.get_profile(reset=True)
    eng.set_profiling(not args.graph)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    for i in range(args.steps):
        flush.zero_()                         # evict the previous step's tensors from L2 (untimed)
        starts[i].record()
        if args.graph:
            eng.replay()
        else:
            eng.forward(x, mask, out)
        ends[i].record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    eng.set_profiling(False)
    step_ms = [a.elapsed_time(e) for a, e in zip(starts, ends)]
    total_ms = sum(step_ms)
    prof = eng.get_profile(reset=True)
    if args.graph:
        # replayed kernels cannot be bracketed by events: per-kernel times from an eager pass of the same steps
        launches_replayed = {k: v[1] for k, v in prof.items()}
        eng.set_profiling(True)
        for i in range(args.steps):
            flush.zero_()
            eng.forward(x, mask, out)
        torch.cuda.synchronize()
        eng.set_profiling(False)
        prof = eng.get_profile(reset=True)
        assert {k: v[1] for k, v in prof.items()} == launches_replayed
    assert eng.device_status() == 0, "a device-side wait expired during the timed steps"

    # ---- end to end through the host-buffer entry point -----------------------
    e2e_ms = None
    h2d = b * s * h * x.element_size() + b * s * 4
    d2h = b * s * h * x.element_size() + 8
    if not args.no_e2e:
        x_host = torch.from_numpy(x_np).to(tdt).pin_memory()
        m_host = torch.from_numpy(mask_np).pin_memory()
        o_host = torch.empty_like(x_host).pin_memory()
        xh, mh, oh = x_host.numpy(), m_host.numpy(), o_host.numpy()
        for _ in range(2):
            eng.forward_host(xh, mh, oh)
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            eng.forward_host(xh, mh, oh)
        torch.cuda.synchronize()
        e2e_ms = 1000.0 * (time.perf_counter() - t0)
        barrier()

    # ---- the same batch as token ids: embeddings in front, pooler behind ------------
    # (not the headline: ids + mask go up, only the pooled [B,H] rows come back)
    ids_ms = None
    if not args.no_e2e:
        mh_ = W.make_model_heads(spec, lengths)
        eng.set_embeddings(mh_.word_table, mh_.type_table, mh_.position_table, mh_.ln_gamma, mh_.ln_beta)
        eng.set_pooler(mh_.pooler_kernel, mh_.pooler_bias)
        pin = lambda a: torch.from_numpy(a).pin_memory().numpy()
        ids_h, types_h, mask_h = pin(mh_.input_ids), pin(mh_.token_type_ids), pin(mask_np)
        for _ in range(2):
            eng.forward_ids_host(ids_h, mask_h, types_h, sequence_output=False, pooled_output=True)
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            eng.forward_ids_host(ids_h, mask_h, types_h, sequence_output=False, pooled_output=True)
        torch.cuda.synchronize()
        ids_ms = 1000.0 * (time.perf_counter() - t0)
        barrier()

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
        # roofline of the dominant kernel (rank 0's launches)
        gemm_cats = ["gemm_qkv", "gemm_attn_out", "gemm_ffn1", "gemm_ffn2"]
        gemm_ms = sum(prof[c][0] for c in gemm_cats)
        gemm_launches = sum(prof[c][1] for c in gemm_cats)
        gemm_flops_step = 2.0 * tokens_rank * h * (3 * h + h + 2 * sh.ffn_dim) * sh.num_layers
        achieved = (gemm_flops_step * args.steps) / (gemm_ms / 1000.0) / 1e12 if gemm_ms > 0 else None
        if fp16:
            peak_tf, peak_note = peaks["bf16_tflops_sustained"], peak_src + " bf16_tflops_sustained"
        else:
            # the fp32 handle's GEMM takes every fp32 product as three tf32 tensor-core products
            # (tf32 runs at half the bf16 rate), so its ceiling in fp32 FLOPs is bf16 / 6; the FP32 FMA
            # rate of the CUDA cores, as cuBLAS SGEMM reaches it, is measured here for comparison
            peak_tf = peaks["bf16_tflops_sustained"] / 6.0
            peak_note = peak_src + " bf16_tflops_sustained / 6 (tf32 = bf16 / 2, three products per fp32 product)"
            sgemm_tf = measure_fp32_gemm_tflops(dev)
        kernels = {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[1] / args.steps}
                   for k, v in prof.items()}
        launches = sum(v[1] for v in prof.values())
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f16" if fp16 else "f32", "data": "synthetic",
            "config": {"workload": spec.name, "sequences_per_gpu": b, "max_seq_len": s,
                       "valid_tokens_rank0": tokens_rank, "valid_tokens_total": int(tokens_all),
                       "layers": sh.num_layers, "hidden": h, "sharding": "sequences, token-balanced, no collective",
                       "l2": "256 MB buffer written between timed steps (untimed)",
                       "host_chunk_shares": "1:%s:1" % os.environ.get("ETB_HOST_MID_SHARE", "6"),
                       "launch": ("cuda-graph replay (et_graph_launch); per-kernel times from a second, eager pass"
                                  if args.graph else "eager (et_forward), per-kernel events inside the timed steps")},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_tf,
                         "unit": "TFLOP/s",
                         "frac": (achieved / peak_tf) if (achieved and peak_tf) else None,
                         "traffic": NCU_GEMM_TRAFFIC.get(spec.name),
                         "traffic_note": NCU_GEMM_TRAFFIC_NOTE if spec.name in NCU_GEMM_TRAFFIC else None,
                         "kernel": "gemm_tcgen05_pair_kernel" if fp16 else "gemm_tf32x3_kernel (+ split_tf32_kernel)",
                         "algorithmic_flops_per_launch": gemm_flops_step / max(gemm_launches / args.steps, 1),
                         "launches_per_step": gemm_launches / args.steps,
                         "avg_launch_ms": gemm_ms / max(gemm_launches, 1),
                         "peak_source": peak_note},
            "kernels": kernels,
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if not fp16:
            line["roofline"]["cublas_sgemm_tflops_measured_here"] = sgemm_tf
        if e2e_ms is not None:
            line["e2e"] = {"value": tokens_all / (e2e_total_ms / args.steps / 1000.0), "unit": UNIT,
                           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                           "ms_per_step": e2e_total_ms / args.steps}
        if ids_ms is not None:
            line["e2e_from_token_ids"] = {
                "value": tokens_all / (ids_total_ms / args.steps / 1000.0), "unit": UNIT,
                "ms_per_step": ids_total_ms / args.steps, "h2d_bytes_per_step": 3 * b * s * 4,
                "d2h_bytes_per_step": b * h * x.element_size() + 8,
                "call": "et_forward_ids_host: ids/types/mask up, embeddings for valid tokens only, "
                        "stack, pooler; pooled [B,H] down"}
        if world == 1 and not args.no_cpu_baseline:
            n_cpu = args.cpu_sample if args.cpu_sample > 0 else min(512, spec.batch)
            tps, dt, toks, threads = cpu_oracle_throughput(spec, n_cpu)
            line["cpu_baseline"] = {
                "value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                "sample": f"first {n_cpu} of {spec.batch} sequences ({toks} valid tokens), "
                          f"{sh.num_layers} layers, padded [B,S] fp32 on the host, {dt:.1f} s"}
        print(json.dumps(line), flush=True)
    eng.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
