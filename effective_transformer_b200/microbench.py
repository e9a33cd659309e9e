"""Per-kernel micro-benchmark through the C ABI.

    python -m effective_transformer_b200.microbench [--kernel NAME|all] [--workload 2] [--iters 20]

Each kernel of the encoder path runs alone on tensors of a benchmark
configuration's shapes (default: BERT-base fp16, B=1000, S=64, T=39778), an
L2-sized buffer is overwritten between iterations, and every iteration is
timed with CUDA events on the launching stream.  One JSON line per kernel:
algorithmic bytes or FLOPs per launch, median time, achieved GB/s or TFLOP/s
and the fraction of the measured peak (MEASURED_PEAKS.json at the repository
root when present, else the stated fallback).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import numpy as np
import torch

from . import _capi
from . import workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"])}, "measured"
    return dict(FALLBACK), "fallback"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all")
    ap.add_argument("--workload", type=int, default=2)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    args = ap.parse_args()

    lib = _capi.load()
    spec = W.WORKLOADS[args.workload]
    lens = W.draw_lengths(spec, np.random.RandomState(spec.seed))
    b, s, h, f = spec.batch, spec.max_seq_len, spec.shape.hidden, spec.shape.ffn_dim
    heads = spec.shape.head_num
    t = int(lens.sum())
    fp16 = spec.dtype == "fp16"
    tdt = torch.float16 if fp16 else torch.float32
    dt = _capi.ET_FP16 if fp16 else _capi.ET_FP32
    e = 2 if fp16 else 4
    dev = torch.device("cuda", 0)
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g, dtype=torch.float32).to(tdt)

    mask = torch.from_numpy(W.prefix_mask(lens, s)).to(dev)
    i32 = dict(dtype=torch.int32, device=dev)
    tn = torch.tensor([t], **i32)
    n_pos = b * s
    prefix, bidx, widx, poff = [torch.zeros(n_pos, **i32) for _ in range(4)]
    slen, cu, scratch = torch.zeros(b, **i32), torch.zeros(b + 1, **i32), torch.zeros(b, **i32)
    valid = torch.zeros(1, **i32)
    status = torch.zeros(1, **i32)
    P = lambda x: None if x is None else x.data_ptr()

    def run_padding():
        return lib.et_padding_offsets(P(mask), b, s, P(prefix), P(valid), P(bidx), P(widx), P(slen), P(cu),
                                      P(poff), P(scratch), st)
    assert run_padding() == 0
    torch.cuda.synchronize()

    x_pad = rnd(b, s, h)
    x_packed = rnd(n_pos, h)
    out_pad = torch.empty_like(x_pad)
    res = rnd(n_pos, h)
    bias_h, gamma_h, beta_h = rnd(h), rnd(h), rnd(h)
    bias_f = rnd(f)
    qkv = rnd(n_pos, 3 * h)
    q, k, v = rnd(n_pos, h), rnd(n_pos, h), rnd(n_pos, h)
    qkv_t = rnd(3 * heads * n_pos * 64)
    ctx = torch.empty(n_pos, h, device=dev, dtype=tdt)
    ffn = rnd(n_pos, f)
    bias3 = rnd(3 * h)
    weights = {}
    for name, (kk, nn) in {"gemm_qkv": (h, 3 * h), "gemm_attn_out": (h, h), "gemm_ffn1": (h, f),
                           "gemm_ffn2": (f, h)}.items():
        w = (rnd(kk, nn) * 0.02).contiguous()
        wp = torch.empty(nn, kk, device=dev, dtype=tdt)
        assert lib.et_pack_weight(dt, P(w), P(wp), kk, nn, st) == 0
        weights[name] = (w, wp, kk, nn)
    gemm_out = torch.empty(n_pos, max(3 * h, f), device=dev, dtype=tdt)
    simt = 0 if fp16 else 1

    def gemm(name, a, bias, epi):
        w, wp, kk, nn = weights[name]
        return lambda: lib.et_gemm(dt, P(a), P(w), P(wp), P(bias), P(gemm_out), P(tn), n_pos, nn, kk, epi, simt,
                                   P(status), st)

    # embedding stage: ids drawn over the full BERT vocabulary, so word rows miss L2 as in production
    vocab = 30522
    ids = torch.randint(0, vocab, (b, s), device=dev, generator=g, dtype=torch.int32)
    types = torch.randint(0, 2, (b, s), device=dev, generator=g, dtype=torch.int32)
    word_t, type_t, pos_t = rnd(vocab, h), rnd(2, h), rnd(512, h)
    first_tok = torch.empty(b, h, device=dev, dtype=tdt)
    w_pool = (rnd(h, h) * 0.02).contiguous()
    wp_pool = torch.empty(h, h, device=dev, dtype=tdt)
    assert lib.et_pack_weight(dt, P(w_pool), P(wp_pool), h, h, st) == 0
    bn = torch.tensor([b], **i32)
    pooled = torch.empty(b, h, device=dev, dtype=tdt)

    plan = torch.zeros(int(lib.et_attention_plan_ints(b, n_pos)), **i32)
    if fp16 and s <= 128:
        assert lib.et_attention_plan(P(cu), b, n_pos, P(plan), st) == 0
    sum_len2 = float((lens.astype(np.int64) ** 2).sum())
    # name -> (callable, bound, algorithmic units per launch)
    kernels = {
        "padding_offsets": (run_padding, "hbm", 4.0 * n_pos + 12.0 * t + 8.0 * b),
        "remove_padding": (lambda: lib.et_remove_padding(dt, P(x_pad), P(bidx), P(widx), P(tn), P(x_packed), b, s, h, st),
                           "hbm", 2.0 * t * h * e),
        "restore_padding": (lambda: lib.et_restore_padding(dt, P(x_packed), P(bidx), P(widx), P(tn), P(out_pad), b, s, h, st),
                            "hbm", (t + n_pos) * h * e * 1.0),
        "qkv_bias_transpose": (lambda: lib.et_add_qkv_bias_transpose(dt, P(q), P(bias_h), P(k), P(bias_h), P(v), P(bias_h),
                                                                    P(qkv_t), P(tn), n_pos, heads, 64, st),
                               "hbm", 6.0 * t * h * e),
        "bias_gelu": (lambda: lib.et_add_bias_gelu(dt, P(ffn), P(bias_f), P(tn), n_pos, f, st), "hbm", 2.0 * t * f * e),
        "bias_residual_layernorm": (lambda: lib.et_add_bias_input_layernorm(dt, P(x_packed), P(res), P(bias_h), P(gamma_h),
                                                                            P(beta_h), P(tn), n_pos, h, 1e-6, st),
                                    "hbm", 3.0 * t * h * e),
        "attention": (lambda: lib.et_attention(dt, qkv.data_ptr(), qkv.data_ptr() + h * e, qkv.data_ptr() + 2 * h * e,
                                               3 * h, 64, P(ctx), P(cu), b, s, n_pos, heads, 64, simt, P(status), st),
                      "hbm", 4.0 * t * h * e),
        "attention_tiles": (lambda: lib.et_attention_tiles(qkv.data_ptr(), qkv.data_ptr() + h * e,
                                                           qkv.data_ptr() + 2 * h * e, 3 * h, 64, P(ctx), P(plan), b, s,
                                                           n_pos, heads, 64, P(status), st),
                            "hbm", 4.0 * t * h * e),
        # the same kernel reading the head-major [3, heads, positions, 64] layout of et_add_qkv_bias_transpose:
        # every TMA box is one contiguous 4 KB piece instead of 32 pieces of 128 bytes a row apart
        "attention_tiles_head_major": (lambda: lib.et_attention_tiles(
            qkv_t.data_ptr(), qkv_t.data_ptr() + heads * n_pos * 64 * e, qkv_t.data_ptr() + 2 * heads * n_pos * 64 * e,
            64, n_pos * 64, P(ctx), P(plan), b, s, n_pos, heads, 64, P(status), st), "hbm", 4.0 * t * h * e),
        "attention_plan": (lambda: lib.et_attention_plan(P(cu), b, n_pos, P(plan), st), "hbm", 4.0 * b + 8.0 * t),
        # per valid token: 12 B of ids/indices + one word row read + one packed row written
        "embedding_layernorm": (lambda: lib.et_embedding_layernorm(
            dt, P(ids), P(types), P(bidx), P(widx), P(tn), P(word_t), vocab, P(type_t), 2, P(pos_t), P(gamma_h),
            P(beta_h), 1e-12, P(x_packed), b, s, h, st), "hbm", t * (2.0 * h * e + 16.0)),
        "gather_first_tokens": (lambda: lib.et_gather_first_tokens(dt, P(x_packed), P(cu), P(first_tok), b, n_pos, h, st),
                                "hbm", 2.0 * b * h * e),
        "gemm_pooler": (lambda: lib.et_gemm(dt, P(first_tok), P(w_pool), P(wp_pool), P(bias_h), P(pooled), P(bn), b, h, h,
                                            3, simt, P(status), st), "tensor", 2.0 * b * h * h),
        "gemm_qkv": (gemm("gemm_qkv", x_packed, bias3, 1), "tensor", 2.0 * t * h * 3 * h),
        "gemm_attn_out": (gemm("gemm_attn_out", x_packed, None, 0), "tensor", 2.0 * t * h * h),
        "gemm_ffn1": (gemm("gemm_ffn1", x_packed, bias_f, 2), "tensor", 2.0 * t * h * f),
        "gemm_ffn2": (gemm("gemm_ffn2", ffn, None, 0), "tensor", 2.0 * t * h * f),
    }
    if fp16:
        # the projections that feed a LayerNorm, with the epilogues that take the residual: 4 = bias + residual,
        # 5 / 6 = the LayerNorm inside the GEMM kernel (bias + residual added in the epilogue / with the rows)
        counters = torch.zeros(8 * ((n_pos + 255) // 256) + 8, **i32)
        fused_out = torch.empty(n_pos, h, device=dev, dtype=tdt)

        def fused(name, a, epi):
            w, wp, kk, nn = weights[name]
            return lambda: lib.et_gemm_fused(P(a), P(wp), P(bias_h), P(res), P(gamma_h), P(beta_h), 1e-6, P(counters),
                                             P(fused_out), P(tn), n_pos, nn, kk, epi, P(status), st)
        # the projections with the LayerNorm deferred into them (et_gemm_deferred_norm): 7 / 8 consume
        # LN(A) from A's row statistics and folded weights, 9 adds LN(residual) on the fly and leaves
        # the statistics of its output rows
        rows_cap = (n_pos + 255) // 256 * 256
        stats_in = torch.rand(rows_cap, 2 * (h // 64), device=dev, dtype=torch.float32) + 64.0
        stats_out = torch.empty(rows_cap, 2 * (h // 64), device=dev, dtype=torch.float32)
        csum = rnd(max(3 * h, f))

        def deferred(name, a, epi, resid):
            w, wp, kk, nn = weights[name]
            bias_n = bias3 if nn == 3 * h else (bias_f if nn == f else bias_h)
            return lambda: lib.et_gemm_deferred_norm(P(a), P(wp), P(bias_n), P(csum), P(resid), P(gamma_h), P(beta_h),
                                                     1e-6, P(stats_in), P(stats_out), P(gemm_out), P(tn), n_pos, nn, kk,
                                                     epi, P(status), st)
        kernels["gemm_qkv_deferred_ln"] = (deferred("gemm_qkv", x_packed, 7, None), "tensor", 2.0 * t * h * 3 * h)
        kernels["gemm_ffn1_deferred_ln"] = (deferred("gemm_ffn1", x_packed, 8, None), "tensor", 2.0 * t * h * f)
        kernels["gemm_attn_out_deferred_ln"] = (deferred("gemm_attn_out", x_packed, 9, res), "tensor", 2.0 * t * h * h)
        kernels["gemm_ffn2_deferred_ln"] = (deferred("gemm_ffn2", ffn, 9, res), "tensor", 2.0 * t * h * f)
        kernels["gemm_ffn2_residual"] = (fused("gemm_ffn2", ffn, 4), "tensor", 2.0 * t * h * f)
        kernels["gemm_ffn2_layernorm"] = (fused("gemm_ffn2", ffn, 5), "tensor", 2.0 * t * h * f)
        kernels["gemm_attn_out_layernorm"] = (fused("gemm_attn_out", x_packed, 6), "tensor", 2.0 * t * h * h)
    # The library GEMM (cuBLAS through torch.matmul) on the same T x N x K, without bias or
    # activation: a comparison figure for the four projections, never part of the product path.
    lib_out = {name: torch.empty(t, w[3], device=dev, dtype=tdt) for name, w in weights.items()}

    def library_gemm(name, a):
        w = weights[name][0]
        rows, out = a[:t], lib_out[name]

        def run():
            torch.matmul(rows, w, out=out)
            return 0
        return run

    for name, a in (("gemm_qkv", x_packed), ("gemm_attn_out", x_packed), ("gemm_ffn1", x_packed), ("gemm_ffn2", ffn)):
        kernels["library_" + name] = (library_gemm(name, a), "tensor", kernels[name][2])
    if not (fp16 and s <= 128):
        kernels.pop("attention_tiles"), kernels.pop("attention_plan"), kernels.pop("attention_tiles_head_major")
    names = list(kernels) if args.kernel == "all" else args.kernel.split(",")
    pk, src = peaks()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    for name in names:
        fn, bound, units = kernels[name]
        for _ in range(args.warmup):
            assert fn() == 0, name
        torch.cuda.synchronize()
        times = []
        for _ in range(args.iters):
            if not args.no_flush:
                flush.zero_()
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            rc = fn()
            z.record()
            assert rc == 0, name
            z.synchronize()
            times.append(a.elapsed_time(z))
        assert int(status[0]) == 0, "a device-side wait expired"
        ms = statistics.median(times)
        if bound == "hbm":
            ach, peak, unit = units / (ms * 1e-3) / 1e9, pk["hbm_gbs"], "GB/s"
        else:
            ach, peak, unit = units / (ms * 1e-3) / 1e12, pk["bf16_tflops"], "TFLOP/s"
        print(json.dumps({"kernel": name, "workload": spec.name, "valid_tokens": t, "bound": bound,
                          "algorithmic_per_launch": units, "ms_median": ms, "ms_min": min(times),
                          "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                          "peak_source": src + (" hbm_gbs" if bound == "hbm" else " bf16_tflops (burst)")}),
              flush=True)


if __name__ == "__main__":
    main()
