#!/usr/bin/env python
"""bench.py -- Llama-3-8B Q8_0 single-stream decode (tg) on B200, the BASELINE.json headline.

A "step" is one single-token decode forward (all layers + lm_head + on-device argmax) at a
growing KV position, on the LlamaBench synthetic token stream (`new Random(42).nextInt(vocab)`,
LlamaBench.java:188-193) over a seeded synthetic GGUF-layout model of the real Llama-3-8B shape.

  value        tok/s with tokens already resident in HBM (device loop b200_decode_sequence,
               CUDA-event time on the plan's stream, max over ranks)
  e2e          tok/s through the reference-facing call b200_forward_decode with HOST buffers:
               every step copies the token/position H2D and the argmax D2H inside the timed region
  roofline     the WHOLE decode step (default: one CUDA graph of 227 kernels per token; --decode-mode persistent: one kernel):
               achieved = algorithmic bytes per token / device time per token, peak = MEASURED_PEAKS.json
               hbm_gbs; per launch = per token / kernels per token; the stand-alone streaming matvecs (the dominant
               kernels by bytes and time, timed live with CUDA events on the plan's stream) are listed under
               roofline.other_kernels; traffic = measured DRAM bytes per launch from the committed ncu capture
  cpu_baseline the oracle (CPU restatement of the reference's onGPU=false path) on this box's
               host cores, bounded sample
  parity       in the same run: greedy ids of the first steps GPU == oracle, max|dlogit| of step 0
               (BASELINE.md section 3); a mismatch exits non-zero
`--impl reference` times only that CPU restatement (the reference itself needs a JDK + TornadoVM,
neither is installable here).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

WORKLOAD = "llama-3-8b"
QUANT = "q8_0"
FALLBACK_HBM_GBS = 6650.0


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


FALLBACK_TENSOR_TFLOPS = 2250.0  # nominal dense bf16/fp16


def tensor_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            j = json.load(f)
        return float(j["bf16_tflops"]), float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), "measured (cuBLAS bf16 8192^3; fp16 shares the rate)"
    return FALLBACK_TENSOR_TFLOPS, FALLBACK_TENSOR_TFLOPS, "fallback (nominal)"


def prefill_leg(pkg, lb, local: int, n: int, reps: int):
    """BASELINE config 3: Llama-3-8B FP16, --batch-prefill-size 512, pp512 from depth 0 (LlamaBench `pp`
    semantics: forward only, no logits).  Tensor-core path: TMA + tcgen05 GEMMs, csrc/prefill*.cuh."""
    shape = pkg.synth.SHAPES[WORKLOAD]
    F16 = pkg.gguf.GGMLType.F16
    model = pkg.loader.model_from_tensors(shape, F16, pkg.synth.build_tensors_fast(shape, F16, seed=1234, device=f"cuda:{local}"), n + 8)
    plan = pkg.B200MasterPlan.initialize_plan(model, prefill_batch_size=n, device=local)
    toks = np.asarray(lb.synthetic_tokens(shape.vocab, n), dtype=np.int32)
    mode = plan.prefill_info()[0]
    dev, wall = [], []
    for r in range(3 + reps):  # 3 untimed warm-up chunks
        t0 = time.perf_counter()
        plan.forward_batch_prefill(toks, 0)  # host tokens in, synchronous: the e2e call
        t1 = time.perf_counter()
        if r >= 3:
            dev.append(plan.prefill_info()[2])
            wall.append((t1 - t0) * 1e3)
    launches = plan.prefill_info()[1]
    plan.free()
    d, w = float(np.mean(dev)), float(np.mean(wall))
    gemm = 2.0 * shape.matmul_elements_no_head() * n
    att = 4.0 * shape.q_dim * shape.n_layers * (n * (n + 1) / 2.0)
    burst, sustained, src = tensor_peak()
    tf = (gemm + att) / (d * 1e-3) / 1e12
    return {"metric": "prefill_tokens_per_s", "value": n / d * 1e3, "unit": "tok/s", "ms_per_chunk": d, "reps": reps, "dtype": "f16 operands, f32 accumulate (TMEM)",
            "e2e": {"value": n / w * 1e3, "unit": "tok/s", "h2d_bytes_per_step": 4 * n, "d2h_bytes_per_step": 0},
            "gpu_launches": launches, "mode": "tensor_core" if mode == 1 else "exact",
            "config": {"workload": f"Llama-3-8B-shaped synthetic GGUF, FP16, pp{n} in one chunk (--batch-prefill-size {n}) from depth 0, KV cache only (no logits)",
                       "l2": "inputs larger than L2 (15.0 GB of FP16 weights per chunk)"},
            "roofline": {"kernel": "whole prefill chunk (k_gemm_f16_tcgen05 = 85 % of it, profiles/)", "bound": "tensor", "achieved": tf, "peak": burst, "peak_sustained": sustained,
                         "peak_source": src, "unit": "TFLOP/s", "frac": tf / burst, "flop_per_chunk": {"gemm": gemm, "attention": att}, "traffic": None}}


# ---- --compare pibidra: the layered design beside the closest GGUF model at equal size -------------------------------------
# Sizes that resemble real layers (random weights, a few layers): the decode step is a weight stream (HBM roofline), the
# prefill chunk is GEMMs + window attention (tensor roofline).  The closest existing model is the FP16 Qwen3 plan (grouped
# key/value heads, q/k norm, FP32 residual, FP32 KV cache) with the same width, feed-forward width, heads and layer count.
COMPARE_SIZES = {
    # name: (width, ff, heads, kv_heads, head size, vocab, layers, window)
    "1b-like": (2048, 8192, 32, 8, 64, 32768, 4, 1024),
    "8b-like": (4096, 14336, 32, 8, 128, 32768, 2, 2048),
}


def compare_layered(pkg, lb, local: int, steps: int, warmup: int, sizes):
    hbm, hbm_src = peaks()
    burst, sustained, t_src = tensor_peak()
    S = pkg.synth
    out = {}
    for name in sizes:
        E, F, H, G, hs, V, NL, Wn = COMPARE_SIZES[name]
        depth, n_pp = 64, 512
        ctx = max(depth + steps + warmup + 8, n_pp + 8)
        toks = np.asarray(lb.synthetic_tokens(V, ctx), dtype=np.int32)
        row = {}
        # the new design: NL layers, the middle ones looped twice (so NL + (NL - 2) layer runs)
        cfg = S.pibidra_config(E, V, [S.pibidra_layer(H, G, hs, hs, Wn, F, bias_max=float(Wn)) for _ in range(NL)],
                               loop=(1, NL - 1, 2) if NL > 2 else None)
        runs = NL + (NL - 2 if NL > 2 else 0)
        w = S.pibidra_weights(cfg, 1234, bias_rows=32)
        per_run = (2 * H * hs + 2 * G * hs) * E + H * hs * E + 3 * F * E  # q, o, k, v, gate + feed-forward weights of one run
        for mode in ("bfloat16",):
            plan = pkg.B200MasterPlan.initialize_plan(S.pibidra_model(cfg, w, ctx), prefill_batch_size=n_pp, device=local, compute=mode)
            plan.decode_sequence(toks[:depth + warmup], depth + warmup, 0)
            _, ms = plan.decode_sequence(toks[depth + warmup:depth + warmup + steps], steps, depth + warmup)
            dbytes = 2 * (runs * per_run + V * E)
            pp = []
            for r in range(3 + 3):
                plan.forward_batch_prefill(toks[:n_pp], 0)
                if r >= 3:
                    pp.append(plan.prefill_info()[2])
            pp_ms = float(np.mean(pp))
            flop = 2.0 * runs * per_run * n_pp + 4.0 * runs * H * hs * sum(min(i + 1, Wn) for i in range(n_pp))
            kern = {}
            for which, kn in ((0, "gate_up"), (1, "down"), (2, "qkvg"), (3, "attn_out"), (4, "classifier")):
                kms, kb = plan.time_kernel(which, 5)
                kern[kn] = {"us": kms * 1e3, "GB/s": kb / kms / 1e6, "frac_hbm": kb / kms / 1e6 / hbm}
            row["pibidra_" + mode] = {
                "decode_tok_s": steps / ms * 1e3, "decode_ms": ms / steps, "decode_frac_hbm": dbytes / (ms / steps * 1e-3) / 1e9 / hbm,
                "launches_per_decode": plan.launches_per_decode, "layer_runs": runs,
                "prefill_tok_s": n_pp / pp_ms * 1e3, "prefill_ms": pp_ms, "prefill_tflops": flop / pp_ms / 1e9, "prefill_frac_tensor": flop / pp_ms / 1e9 / burst,
                "prefill_launches": plan.prefill_info()[1], "decode_kernels": kern}
            plan.free()
        # the closest existing model at equal size: Qwen3-shaped FP16 GGUF with `runs` layers
        shape = S.Shape("qwen3", E, F, runs, H, G, hs, V, False, 1000000.0, 1e-6, ctx)
        F16 = pkg.gguf.GGMLType.F16
        model = pkg.loader.model_from_tensors(shape, F16, S.build_tensors_fast(shape, F16, seed=1234, device=f"cuda:{local}"), ctx)
        plan = pkg.B200MasterPlan.initialize_plan(model, prefill_batch_size=n_pp, device=local)
        plan.decode_sequence(toks[:depth + warmup], depth + warmup, 0)
        _, ms = plan.decode_sequence(toks[depth + warmup:depth + warmup + steps], steps, depth + warmup)
        dbytes = 2 * shape.matmul_elements()
        pp = []
        for r in range(3 + 3):
            plan.forward_batch_prefill(toks[:n_pp], 0)
            if r >= 3:
                pp.append(plan.prefill_info()[2])
        pp_ms = float(np.mean(pp))
        flop = 2.0 * shape.matmul_elements_no_head() * n_pp + 4.0 * shape.q_dim * runs * (n_pp * (n_pp + 1) / 2.0)
        kern = {}
        for which, kn in ((0, "gate_up"), (1, "down"), (2, "qkv"), (3, "attn_out"), (4, "classifier")):
            kms, kb = plan.time_kernel(which, 5)
            kern[kn] = {"us": kms * 1e3, "GB/s": kb / kms / 1e6, "frac_hbm": kb / kms / 1e6 / hbm}
        row["qwen3_f16"] = {
            "decode_tok_s": steps / ms * 1e3, "decode_ms": ms / steps, "decode_frac_hbm": dbytes / (ms / steps * 1e-3) / 1e9 / hbm,
            "launches_per_decode": plan.launches_per_decode, "layers": runs,
            "prefill_tok_s": n_pp / pp_ms * 1e3, "prefill_ms": pp_ms, "prefill_tflops": flop / pp_ms / 1e9, "prefill_frac_tensor": flop / pp_ms / 1e9 / burst,
            "prefill_mode": "tensor_core" if plan.prefill_info()[0] == 1 else "exact", "prefill_launches": plan.prefill_info()[1], "decode_kernels": kern}
        plan.free()
        row["config"] = {"width": E, "ff": F, "heads": H, "kv_heads": G, "head_size": hs, "vocab": V, "layers": NL, "layer_runs": runs, "window": Wn,
                         "decode": f"tg{steps} from depth {depth + warmup}", "prefill": f"pp{n_pp} in one chunk from depth 0"}
        out[name] = row
    return {"metric": "layered_vs_closest_model", "unit": "tok/s", "data": "synthetic", "dtype": "bf16 weights (Pibidra) / f16 weights (Qwen3), f32 accumulate",
            "peaks": {"hbm_gbs": hbm, "hbm_source": hbm_src, "tensor_tflops": burst, "tensor_source": t_src}, "sizes": out}


# ---- --compare latusun: the parallel-block design beside the closest existing model (the Pibidra layered plan) at equal size -----
# Both are layered plans with BF16 weights and the same projection kernels.  Equal size = same width, heads, vocabulary and
# layer count; the Pibidra layers get the latent design's per-head query/key size (unrotated + rotated) and value size, one
# key/value head per four query heads, and a dense feed-forward as wide as the experts one token uses (top x expert width).
LATUSUN_SIZES = {
    # name: (width, heads, unrotated, rotated, value, latent, experts, top, expert ff, vocab, layers)
    # (key sizes unrotated + rotated = 64 / 192 with value sizes 64 / 128: instances of the tensor-core attention both designs run)
    "small": (1024, 8, 48, 16, 64, 256, 8, 2, 1024, 32768, 4),
    "lite-like": (2048, 16, 128, 64, 128, 512, 16, 4, 1408, 32768, 4),
}


def _layered_leg(plan, toks, depth, warmup, steps, n_pp, hbm, burst, dbytes, flop, kernel_names):
    plan.decode_sequence(toks[:depth + warmup], depth + warmup, 0)
    _, ms = plan.decode_sequence(toks[depth + warmup:depth + warmup + steps], steps, depth + warmup)
    pp = []
    for r in range(3 + 3):
        plan.forward_batch_prefill(toks[:n_pp], 0)
        if r >= 3:
            pp.append(plan.prefill_info()[2])
    pp_ms = float(np.mean(pp))
    kern = {}
    for which, kn in kernel_names:
        kms, kb = plan.time_kernel(which, 5)
        kern[kn] = {"us": kms * 1e3, "GB/s": kb / kms / 1e6, "frac_hbm": kb / kms / 1e6 / hbm}
    return {"decode_tok_s": steps / ms * 1e3, "decode_ms": ms / steps, "decode_frac_hbm": dbytes / (ms / steps * 1e-3) / 1e9 / hbm,
            "launches_per_decode": plan.launches_per_decode, "prefill_tok_s": n_pp / pp_ms * 1e3, "prefill_ms": pp_ms,
            "prefill_tflops": flop / pp_ms / 1e9, "prefill_frac_tensor": flop / pp_ms / 1e9 / burst, "prefill_launches": plan.prefill_info()[1],
            "decode_kernels": kern}


def compare_latusun(pkg, lb, local: int, steps: int, warmup: int, sizes):
    hbm, hbm_src = peaks()
    burst, sustained, t_src = tensor_peak()
    S = pkg.synth
    out = {}
    for name in sizes:
        E, H, dk, dr, dv, R, X, top, F, V, NL = LATUSUN_SIZES[name]
        depth, n_pp = 64, 512
        ctx = max(depth + steps + warmup + 8, n_pp + 8)
        toks = np.asarray(lb.synthetic_tokens(V, ctx), dtype=np.int32)
        A, B = "latent_attention", "latent_attention_2"
        blend = {"factor": 8.0, "original": 1024, "fast": 32.0, "slow": 1.0}
        layers = []
        for i in range(NL):  # gated / plain / plain reading the previous layer's cache / gated ...
            kind = (A, B, B, A)[i % 4]
            layers.append(S.latusun_layer(kind, H, dk, dr, dv, R, experts=X, top=top, ff=F, scaling=blend if kind == A else None,
                                          kv_from=i - 1 if i % 4 == 2 else None))
        cfg = S.latusun_config(E, V, layers)
        w = S.latusun_weights(cfg, 1234)
        streamed = 0  # weight elements one decode step reads
        mac = 0       # multiply-adds per prompt token outside the attention's score / value products
        for lc in layers:
            own = lc["mixer"].get("kv_from") is None
            gate = lc["type"] == A
            proj = H * (dk + dr) * E + (R + dr) * E * own + H * dv * E * gate
            mixer = proj + H * dk * R + H * dv * R + E * H * dv
            ff = X * E + top * 3 * F * E
            streamed += mixer + ff
            mac += mixer + ff
        att_mac = sum(NL * H * (2 * R + dr) * (i + 1) for i in range(n_pp))  # folded form: scores over R + dr, values over R
        plan = pkg.B200MasterPlan.initialize_plan(S.latusun_model(cfg, w, ctx), prefill_batch_size=n_pp, device=local, compute="bfloat16")
        row = {"latusun_bfloat16": _layered_leg(plan, toks, depth, warmup, steps, n_pp, hbm, burst, 2 * (streamed + V * E), 2.0 * mac * n_pp + 2.0 * att_mac,
                                                ((0, "expert_gate_up"), (1, "expert_down"), (2, "q_dkv_gate"), (3, "attn_out"), (4, "classifier")))}
        plan.free()
        del w
        # the closest existing model at equal size
        G = max(1, H // 4)
        Wn = ctx
        pcfg = S.pibidra_config(E, V, [S.pibidra_layer(H, G, dk + dr, dv, Wn, top * F, bias_max=float(Wn)) for _ in range(NL)])
        pw = S.pibidra_weights(pcfg, 1234, bias_rows=32)
        per = (H * (dk + dr) + G * (dk + dr) + G * dv + H * dv) * E + H * dv * E + 3 * top * F * E
        patt = sum(NL * H * (dk + dr + dv) * (i + 1) for i in range(n_pp))
        plan = pkg.B200MasterPlan.initialize_plan(S.pibidra_model(pcfg, pw, ctx), prefill_batch_size=n_pp, device=local, compute="bfloat16")
        row["pibidra_bfloat16"] = _layered_leg(plan, toks, depth, warmup, steps, n_pp, hbm, burst, 2 * (NL * per + V * E), 2.0 * NL * per * n_pp + 2.0 * patt,
                                               ((0, "gate_up"), (1, "down"), (2, "qkvg"), (3, "attn_out"), (4, "classifier")))
        plan.free()
        del pw
        row["config"] = {"width": E, "heads": H, "unrotated": dk, "rotated": dr, "value": dv, "latent": R, "experts": X, "top": top, "expert_ff": F, "vocab": V,
                         "layers": NL, "closest": f"Pibidra: {G} key/value heads of {dk + dr} / {dv}, dense feed-forward {top * F}, window = context",
                         "decode": f"tg{steps} from depth {depth + warmup}", "prefill": f"pp{n_pp} in one chunk from depth 0"}
        out[name] = row
    return {"metric": "latusun_vs_closest_model", "unit": "tok/s", "data": "synthetic", "dtype": "bf16 weights, f32 accumulate",
            "peaks": {"hbm_gbs": hbm, "hbm_source": hbm_src, "tensor_tflops": burst, "tensor_source": t_src}, "sizes": out}


# ---- --compare lerosun: the pre-norm hybrid (windowed attention + gated delta rule) beside the closest existing model (Pibidra) -----
# Both are layered plans with BF16 weights, an FP32 residual, window rings and the same projection kernels.  Equal size = same width,
# feed-forward width, heads, key/value heads, head size, window, vocabulary and number of layer runs; the Pibidra layers are all
# attention, the Lerosun layers alternate delta / attention / attention / delta with the two attention layers looped twice.
LEROSUN_SIZES = {
    # name: (width, ff, attention heads, key/value heads, head size, window, delta value heads, delta q/k heads, delta key size, delta value size, taps, vocab)
    # (the head-mixed attention reads key rows of key/value heads x head size = 128 / 256 with values of 64 / 128: instances of the tensor-core attention)
    "small": (1024, 4096, 16, 2, 64, 1024, 8, 4, 64, 128, 4, 32768),
    "1b-like": (2048, 8192, 16, 2, 128, 1024, 16, 8, 128, 128, 4, 32768),
}


def compare_lerosun(pkg, lb, local: int, steps: int, warmup: int, sizes):
    hbm, hbm_src = peaks()
    burst, sustained, t_src = tensor_peak()
    S = pkg.synth
    out = {}
    for name in sizes:
        E, F, H, G, hs, Wn, DH, DG, ddk, ddv, taps, V = LEROSUN_SIZES[name]
        depth, n_pp = 64, 512
        ctx = max(depth + steps + warmup + 8, n_pp + 8)
        toks = np.asarray(lb.synthetic_tokens(V, ctx), dtype=np.int32)
        att, dlt = S.lerosun_attention(H, G, hs, Wn, F, rot_dims=hs // 2), S.lerosun_delta(DH, DG, ddk, ddv, taps, F)
        cfg = S.lerosun_config(E, V, [dlt, att, att, dlt], loop=(1, 3, 2))
        order = [dlt, att, att, att, att, dlt]  # the six layer runs
        w = S.lerosun_weights(cfg, 1234)
        att_w = (H * hs + G * hs + H) * E + H * hs * E + 3 * F * E
        dlt_w = (2 * DG * ddk + 2 * DH * ddv + 2 * DH) * E + DH * ddv * E + 3 * F * E
        streamed = sum(att_w if lc["type"] == "attention" else dlt_w for lc in order)
        pairs = sum(min(i + 1, Wn) for i in range(n_pp))
        mix_mac = sum((H * 2 * hs * pairs) if lc["type"] == "attention" else (3 * DH * ddk * ddv * n_pp) for lc in order)  # scores + values | S^T k, k u^T, S^T q
        plan = pkg.B200MasterPlan.initialize_plan(S.lerosun_model(cfg, w, ctx), prefill_batch_size=n_pp, device=local, compute="bfloat16")
        row = {"lerosun_bfloat16": _layered_leg(plan, toks, depth, warmup, steps, n_pp, hbm, burst, 2 * (streamed + V * E), 2.0 * streamed * n_pp + 2.0 * mix_mac,
                                                ((0, "gate_up"), (1, "down"), (2, "fused_projection"), (3, "mixer_out"), (4, "classifier")))}
        plan.free()
        del w
        runs = len(order)
        pcfg = S.pibidra_config(E, V, [S.pibidra_layer(H, G, hs, hs, Wn, F, bias_max=float(Wn)) for _ in range(runs)])
        pw = S.pibidra_weights(pcfg, 1234, bias_rows=32)
        per = (2 * H * hs + 2 * G * hs) * E + H * hs * E + 3 * F * E
        plan = pkg.B200MasterPlan.initialize_plan(S.pibidra_model(pcfg, pw, ctx), prefill_batch_size=n_pp, device=local, compute="bfloat16")
        row["pibidra_bfloat16"] = _layered_leg(plan, toks, depth, warmup, steps, n_pp, hbm, burst, 2 * (runs * per + V * E), 2.0 * runs * per * n_pp + 2.0 * runs * H * 2 * hs * pairs,
                                               ((0, "gate_up"), (1, "down"), (2, "qkvg"), (3, "attn_out"), (4, "classifier")))
        plan.free()
        del pw
        row["config"] = {"width": E, "ff": F, "attention": f"{H} heads, {G} key/value heads of {hs}, window {Wn}", "delta": f"{DH} value heads of {ddv}, {DG} query/key heads of {ddk}, {taps} taps",
                         "vocab": V, "layer_runs": runs, "order": "delta, (attention, attention) x 2, delta", "closest": f"Pibidra: {runs} attention layers of the same heads and window",
                         "decode": f"tg{steps} from depth {depth + warmup}", "prefill": f"pp{n_pp} in one chunk from depth 0"}
        out[name] = row
    return {"metric": "lerosun_vs_closest_model", "unit": "tok/s", "data": "synthetic", "dtype": "bf16 weights, f32 accumulate",
            "peaks": {"hbm_gbs": hbm, "hbm_source": hbm_src, "tensor_tflops": burst, "tensor_source": t_src}, "sizes": out}


# ---- --compare dinuzen: the output-normed hybrid (differential attention, real-gated recurrent unit, state-space recurrence,
# softmax-routed experts) beside the closest existing model (Lerosun: the other hybrid of attention and a recurrence with a short
# convolution) -----
# Both are layered plans with BF16 weights, an FP32 residual, key rings, recurrent states with convolution rings and the same
# projection kernels.  Equal size = same width, vocabulary, number of layers and layer order (recurrent, attention, recurrent,
# attention), the same number of score maps per token (Dinuzen: heads x 2 maps; Lerosun: 2 x heads), the same key size, and a dense
# feed-forward as wide as what one Dinuzen token uses (chosen experts + shared expert).
DINUZEN_SIZES = {
    # name: (width, attention heads, key/value heads, key = value size per map, recurrent-unit blocks, state-space heads, value size, state size, taps,
    #        experts, identity experts, chosen, expert ff, shared ff, dense ff, vocab, Lerosun delta (value heads, q/k heads, key size, value size))
    "small": (1024, 8, 2, 64, 8, 32, 64, 128, 4, 8, 1, 2, 1024, 1024, 4096, 32768, (8, 4, 64, 128)),
    "1b-like": (2048, 8, 2, 128, 16, 64, 64, 128, 4, 16, 2, 4, 1408, 2816, 8192, 32768, (16, 8, 128, 128)),
}


def dinuzen_compare_models(S, name: str, ctx: int):
    """(Dinuzen config, Lerosun config, accounting) of one compare size."""
    E, H, G, dk, nb, SH, SP, SN, taps, X, I, top, F, SF, DF, V, (DH, DG, ddk, ddv) = DINUZEN_SIZES[name]
    moe = S.dinuzen_moe(X, top, F, identity=I, scale=2.0, shared=SF)
    layers = [S.dinuzen_mamba2(SH, SP, SN, 1, taps, moe), S.dinuzen_attention(H, G, dk, dk, S.dinuzen_dense(DF), scaling=(4.0, 4096, 32.0, 1.0)),
              S.dinuzen_rglru(E, nb, taps, moe), S.dinuzen_attention(H, G, dk, dk, moe, scaling=(4.0, 4096, 32.0, 1.0), kv_from=1)]
    cfg = S.dinuzen_config(E, V, layers, groups=4)
    real = top * X / (X + I)  # experts a token streams on average when every expert is equally likely
    moe_w = (X + I + 1) * E + 3 * SF * E + real * 3 * F * E
    inner = SH * SP
    w_ssd = (2 * inner + 2 * SN + SH) * E + inner * E + moe_w
    w_att = (H * 2 * dk + G * 2 * dk + G * dk) * E + H * dk * E + 2 * DF * E
    w_rg = 2 * E * E + 2 * E * (E // nb) + E * E + moe_w
    w_att2 = H * 2 * dk * E + H * dk * E + moe_w
    streamed = w_ssd + w_att + w_rg + w_att2
    FL = top * F + SF  # the closest model's dense feed-forward: as wide as what one token uses here
    att, dlt = S.lerosun_attention(2 * H, G, dk, ctx, FL, rot_dims=dk // 2), S.lerosun_delta(DH, DG, ddk, ddv, taps, FL)
    lcfg = S.lerosun_config(E, V, [dlt, att, dlt, att])
    l_att = (2 * H * dk + G * dk + 2 * H) * E + 2 * H * dk * E + 3 * FL * E
    l_dlt = (2 * DG * ddk + 2 * DH * ddv + 2 * DH) * E + DH * ddv * E + 3 * FL * E
    acct = {"streamed": streamed, "ssd_mac_per_token": 3 * SH * SN * SP, "att_mac_per_pair": H * 2 * (dk + dk), "l_streamed": 2 * (l_att + l_dlt),
            "l_att_mac_per_pair": 2 * H * 2 * dk, "l_delta_mac_per_token": 3 * DH * ddk * ddv}
    return cfg, lcfg, acct


def compare_dinuzen(pkg, lb, local: int, steps: int, warmup: int, sizes):
    hbm, hbm_src = peaks()
    burst, sustained, t_src = tensor_peak()
    S = pkg.synth
    out = {}
    for name in sizes:
        E, V = DINUZEN_SIZES[name][0], DINUZEN_SIZES[name][15]
        depth, n_pp = 64, 512
        ctx = max(depth + steps + warmup + 8, n_pp + 8)
        toks = np.asarray(lb.synthetic_tokens(V, ctx), dtype=np.int32)
        cfg, lcfg, a = dinuzen_compare_models(S, name, ctx)
        pairs = n_pp * (n_pp + 1) // 2
        w = S.dinuzen_weights(cfg, 1234)
        plan = pkg.B200MasterPlan.initialize_plan(S.dinuzen_model(cfg, w, ctx), prefill_batch_size=n_pp, device=local, compute="bfloat16")
        row = {"dinuzen_bfloat16": _layered_leg(plan, toks, depth, warmup, steps, n_pp, hbm, burst, 2 * (a["streamed"] + V * E),
                                                2.0 * a["streamed"] * n_pp + 2.0 * (2 * a["att_mac_per_pair"] * pairs + a["ssd_mac_per_token"] * n_pp),
                                                ((0, "up_or_gate_up"), (1, "down"), (2, "fused_projection"), (3, "mixer_out"), (4, "classifier")))}
        plan.free()
        del w
        lw = S.lerosun_weights(lcfg, 1234)
        plan = pkg.B200MasterPlan.initialize_plan(S.lerosun_model(lcfg, lw, ctx), prefill_batch_size=n_pp, device=local, compute="bfloat16")
        row["lerosun_bfloat16"] = _layered_leg(plan, toks, depth, warmup, steps, n_pp, hbm, burst, 2 * (a["l_streamed"] + V * E),
                                               2.0 * a["l_streamed"] * n_pp + 2.0 * (2 * a["l_att_mac_per_pair"] * pairs + 2 * a["l_delta_mac_per_token"] * n_pp),
                                               ((0, "gate_up"), (1, "down"), (2, "fused_projection"), (3, "mixer_out"), (4, "classifier")))
        plan.free()
        del lw
        row["config"] = {"width": E, "vocab": V, "layers": 4, "order": "state space, attention, recurrent unit, attention reading the first one's keys",
                         "sizes": dict(zip(("width", "attention_heads", "kv_heads", "key_value_size_per_map", "unit_blocks", "ssd_heads", "ssd_value", "ssd_state", "taps", "experts",
                                            "identity_experts", "chosen", "expert_ff", "shared_ff", "dense_ff", "vocab"), DINUZEN_SIZES[name][:16])),
                         "closest": "Lerosun: delta, attention, delta, attention with twice the heads of the same key size and a dense feed-forward of chosen x expert ff + shared ff",
                         "decode": f"tg{steps} from depth {depth + warmup}", "prefill": f"pp{n_pp} in one chunk from depth 0"}
        out[name] = row
    return {"metric": "dinuzen_vs_closest_model", "unit": "tok/s", "data": "synthetic", "dtype": "bf16 weights, f32 accumulate",
            "peaks": {"hbm_gbs": hbm, "hbm_source": hbm_src, "tensor_tflops": burst, "tensor_source": t_src}, "sizes": out}


class ClockSampler:
    """nvidia-smi clocks/throttle reasons sampled DURING the timed region."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "samples": len(sm), "reasons": sorted(reasons)}


def algorithmic_bytes_per_token(shape, quant_q8: bool, ctx_avg_pos: float) -> dict:
    """matmul weights read once + F32 norm weights + FP32 KV reads."""
    elems = shape.matmul_elements()
    w = elems // 32 * 34 if quant_q8 else elems * 2
    norms = (2 * shape.n_layers + 1) * shape.dim * 4
    kv = 2 * shape.n_layers * (ctx_avg_pos + 1) * shape.kv_dim * 4
    return {"weights": w, "norms": norms, "kv": kv, "total": w + norms + kv}


def build_model(pkg, ctx: int, device: str | None, tp_rank: int = 0, tp_size: int = 1):
    shape = pkg.synth.SHAPES[WORKLOAD]
    quant = pkg.gguf.GGMLType.Q8_0 if QUANT == "q8_0" else pkg.gguf.GGMLType.F16
    t0 = time.time()
    tensors = pkg.synth.build_tensors_fast(shape, quant, seed=1234, device=device, tp_rank=tp_rank, tp_size=tp_size)
    model = pkg.loader.model_from_tensors(shape, quant, tensors, ctx)
    return shape, model, time.time() - t0


def cpu_leg(orc, model, tokens, budget_s: float, max_tokens: int):
    """Times the CPU restatement (per-row activation quantisation exactly as the reference does,
    Q8_0FloatTensor.java:100-117; rows over all host cores like Parallel.parallelFor) on the bench's own
    token stream from position 0, and keeps what the parity gate needs: step 0's logits, every step's argmax."""
    cores = orc.use_all_cores()  # torchrun exports OMP_NUM_THREADS=1: set the thread count explicitly
    om = orc.OracleModel(model, per_row_quant=True)
    lg0 = om.forward(int(tokens[0]), 0).copy()  # untimed warm-up (page-in); position 0 of the stream
    ids = [orc.argmax(lg0)]
    n, t0 = 0, time.perf_counter()
    while n < max_tokens:
        ids.append(orc.argmax(om.forward(int(tokens[1 + n]), 1 + n)))
        n += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    om.close()
    return n / dt, n, dt, cores, {"logits0": lg0, "ids": ids}


def parity_gate(plan, tokens, ref, want_logits: bool):
    """the GPU path on the same tokens/positions the oracle just ran.  Teacher-forced (LlamaBench's
    token stream), so every step is an independent check of logits -> argmax at a growing KV depth."""
    plan.kv_reset()
    n = len(ref["ids"])
    got, dmax = [], None
    for i in range(n):
        lg, am = plan.forward_decode(int(tokens[i]), i, logits=want_logits and i == 0)
        got.append(int(am))
        if want_logits and i == 0:
            dmax = float(np.abs(lg - ref["logits0"]).max())
            bit_equal = bool(np.array_equal(lg.view(np.uint32), ref["logits0"].view(np.uint32)))
    out = {"steps": n, "ids_equal": got == [int(v) for v in ref["ids"]], "against": "oracle (CPU restatement of InferenceCore.forwardJava), same tokens and positions"}
    if dmax is not None:
        out["max_abs_dlogit"] = dmax
        out["logits_bit_equal"] = bit_equal
        out["tolerance"] = "0 (decode reproduces the CPU path's float order; FP16-scale 2^-8*max|logit| would be the north-star bound)"
    return out


def main():
    global WORKLOAD, QUANT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-budget", type=float, default=20.0, help="seconds of CPU-baseline work")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg (profiling runs)")
    ap.add_argument("--no-pp", action="store_true", help="skip the pp512 tensor-core prefill leg")
    ap.add_argument("--decode-mode", default="default", choices=["default", "persistent", "graph"],
                    help="decode implementation: one persistent kernel per token, or the round-1 CUDA graph of ~7 kernels per layer")
    ap.add_argument("--quant", default="q8_0", choices=["q8_0", "f16"], help="weight type of the synthetic model (f16: the exact lane-order FP16 matvec path, graph mode)")
    ap.add_argument("--depth", type=int, default=-1, help="LlamaBench -d: KV positions filled before the timed steps (default: the warm-up steps)")
    ap.add_argument("--workload", default=WORKLOAD, choices=["llama-3-8b", "llama-3-70b", "llama-3.2-1b", "qwen3-4b"],
                    help="shape of the synthetic model (default: the BASELINE headline, Llama-3-8B; 70B is BASELINE config 5, meant for --gpus 2/4/8)")
    ap.add_argument("--compare", default=None, choices=["pibidra", "latusun", "lerosun", "dinuzen"],
                    help="instead of the headline workload: decode and prefill throughput of a layered design beside its closest existing model "
                         "at equal sizes (pibidra: the FP16 Qwen3 plan; latusun, lerosun: the Pibidra plan; dinuzen: the Lerosun plan), with per-kernel rooflines; one JSON line")
    ap.add_argument("--compare-sizes", default=None, help="comma-separated size names (pibidra: 1b-like,8b-like; latusun: small,lite-like; lerosun, dinuzen: small,1b-like)")
    args = ap.parse_args()
    K, W = args.steps, max(args.warmup, 3)
    if args.compare:
        import torch

        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        pkg = ge.import_package()
        sampler = ClockSampler(local)
        sampler.start()
        if args.compare == "dinuzen":
            line = compare_dinuzen(pkg, pkg.llama_bench, local, min(K, 64), W, (args.compare_sizes or "small,1b-like").split(","))
        elif args.compare == "lerosun":
            line = compare_lerosun(pkg, pkg.llama_bench, local, min(K, 64), W, (args.compare_sizes or "small,1b-like").split(","))
        elif args.compare == "latusun":
            line = compare_latusun(pkg, pkg.llama_bench, local, min(K, 64), W, (args.compare_sizes or "small,lite-like").split(","))
        else:
            line = compare_layered(pkg, pkg.llama_bench, local, min(K, 64), W, (args.compare_sizes or "1b-like,8b-like").split(","))
        line["clocks"] = sampler.stop()
        print(json.dumps(line))
        return 0
    WORKLOAD = args.workload
    QUANT = args.quant
    pretty = {"llama-3-8b": "Llama-3-8B", "llama-3-70b": "Llama-3-70B", "llama-3.2-1b": "Llama-3.2-1B", "qwen3-4b": "Qwen3-4B"}[WORKLOAD]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    pkg = ge.import_package()
    lb = pkg.llama_bench
    shape = pkg.synth.SHAPES[WORKLOAD]
    D = max(W, args.depth)  # LlamaBench -d: positions filled before the timed steps; the fill doubles as the warm-up
    ctx = D + K + 8  # LlamaBench: depth + tokens + 8 (LlamaBench.java:174)
    tokens = np.asarray(lb.synthetic_tokens(shape.vocab, D + K), dtype=np.int32)
    qname = "Q8_0" if QUANT == "q8_0" else "FP16"
    config = {"workload": f"{pretty}-shaped synthetic GGUF, {qname}, tg{K} single-stream decode from depth {D}",
              "weights": "seeded N(0,1/sqrt(fan_in)) quantised with the ggml Q8_0 rule; tokens java.util.Random(42)",
              "context": ctx, "l2": f"inputs larger than L2 ({(shape.matmul_elements() // 32 * 34 if QUANT == 'q8_0' else shape.matmul_elements() * 2) / 1e9:.2f} GB of weights stream per step vs 126 MB L2)"}

    if args.impl == "reference":
        if world > 1 and rank != 0:
            return 0
        orc = ge.import_oracle()
        _, model, _ = build_model(pkg, ctx, None)
        budget = max(10.0, min(120.0, 8.0 * (K + W)))  # bounded sample: the whole run ends within minutes
        tps, n, dt, cores, _ = cpu_leg(orc, model, tokens, budget, max(1, min(K, D + K - 1)))
        line = {"metric": "decode_tokens_per_s", "value": tps, "unit": "tok/s", "n_gpus": args.gpus, "steps": K, "warmup": W,
                "ms_per_step": 1e3 / tps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "q8_0xq8_0->int32, f32 accumulate",
                "data": "synthetic", "impl": "reference", "config": config,
                "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": cores, "kind": "port",
                                 "sample": f"{n} decode steps of the same workload in {dt:.1f} s (C restatement of InferenceCore.forwardJava, -O2, OpenMP rows)"},
                "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    import torch
    import torch.distributed as dist

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    torch.cuda.set_device(local)
    # a rank that never runs the oracle keeps only the rows it uploads on the host (70B: ~10 GB instead of 74 GB per rank)
    shard_host = world > 1 and (rank != 0 or args.no_cpu)
    shape, model, gen_s = build_model(pkg, ctx, f"cuda:{local}", rank if shard_host else 0, world if shard_host else 1)
    t0 = time.time()
    plan = pkg.B200MasterPlan.initialize_plan(model, device=local, tp_rank=rank, tp_size=world)
    load_s = time.time() - t0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.decode_mode != "default":
        plan.set_decode_mode(args.decode_mode)
    dmode, launches_per_step, ring_stages, pd_smem = plan.decode_info()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # nvidia-smi forks BEFORE the barrier: no rank waits on it inside the timed region
    # ---- value: device loop, tokens resident in HBM ------------------------------------------
    plan.decode_sequence(tokens[:D], D, 0)  # D >= W untimed warm-up steps (positions 0..D-1)
    barrier()
    ids, ms = plan.decode_sequence(tokens[D:D + K], K, D)
    barrier()
    ms_rank = [ms]
    if world > 1:
        t = torch.tensor([ms], device=f"cuda:{local}")
        allt = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allt, t)
        ms_rank = [float(v.item()) for v in allt]
        ms = max(ms_rank)
    value = K / (ms / 1e3)  # one stream; under --gpus N the model is tensor-parallel over N ranks (strong scaling)

    # ---- e2e: reference-facing call, host token in / host argmax out every step ----------------
    plan.kv_reset()
    if D > W:
        plan.decode_sequence(tokens[:D - W], D - W, 0)
    for i in range(D - W, D):  # W untimed warm-up calls through the same entry point
        plan.forward_decode(int(tokens[i]), i, logits=False)
    barrier()
    t0 = time.perf_counter()
    e2e_ids = []
    for i in range(K):
        _, am = plan.forward_decode(int(tokens[D + i]), D + i, logits=False)
        e2e_ids.append(am)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    assert list(ids) == e2e_ids, "device loop and per-step API disagree"

    if rank != 0:
        if not args.no_cpu:  # tensor-parallel parity gate: rank 0 runs the oracle, every rank issues the same forwards
            box = [None]
            dist.broadcast_object_list(box, src=0)
            n_par = int(box[0])
            plan.kv_reset()
            for i in range(n_par):
                plan.forward_decode(int(tokens[i]), i, logits=False)
        plan.free()
        dist.barrier()
        dist.destroy_process_group()
        return 0

    # ---- roofline: the whole decode step (in persistent mode it is ONE kernel launch) ------------------
    peak, peak_src = peaks()
    ab = algorithmic_bytes_per_token(shape, QUANT == "q8_0", D + (K - 1) / 2.0)
    step_bytes = ab["total"] / world                 # algorithmic bytes one GPU must read per token
    step_gbs = step_bytes * value / 1e9              # ... x tok/s
    per_kernel = {}
    if world == 1:  # the stand-alone streaming matvecs of the graph path, for context (b200_time_kernel, PDL off)
        for which, name in ((0, "gate_up"), (1, "down_proj"), (2, "qkv"), (3, "attn_out"), (4, "lm_head")):
            m, b = plan.time_kernel(which, reps=3 if which != 4 else 1)
            per_kernel[name] = {"ms": m, "GB/s": b / (m / 1e3) / 1e9, "bytes": b, "frac": b / (m / 1e3) / 1e9 / peak}
    persistent = dmode == 1
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "r2_decode_traffic.json")  # dram bytes per launch from the committed ncu --set full capture
    if world == 1 and WORKLOAD == "llama-3-8b" and QUANT == "q8_0" and os.path.exists(tpath):
        with open(tpath) as f:
            traffic = json.load(f).get("persistent" if persistent else "graph")
    line = {
        "metric": "decode_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None,
        "dtype": "q8_0xq8_0->int32, f32 accumulate" if QUANT == "q8_0" else "f16 weights x f32 activations, f32 fma chains (16 lanes)", "data": "synthetic", "config": config,
        "parallelism": "single GPU" if world == 1 else f"tp{world}: row-sharded weights, in-kernel all-gather over NVLink peer memory (bit-exact with tp1)",
        "decode_mode": "persistent (1 kernel per token)" if persistent else f"graph ({launches_per_step} kernels per token)",
        "e2e": {"value": K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 32, "d2h_bytes_per_step": 4},
        "gpu_launches": launches_per_step * K,
        "clocks": clocks,
        "ms_per_step_by_rank": [m / K for m in ms_rank],
        "roofline": {"kernel": ("k_decode_persistent: the whole token (all layers + lm_head + argmax) in one launch; " if persistent else "whole decode step (CUDA graph); ")
                               + ("per GPU" if world > 1 else "single GPU"),
                     "bound": "hbm", "achieved": step_gbs, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": step_gbs / peak,
                     "bytes_per_launch": step_bytes if persistent else step_bytes / launches_per_step, "ms_per_launch": ms / K if persistent else ms / K / launches_per_step,
                     "algorithmic_bytes_per_token": ab, "traffic": traffic,
                     "persistent_kernel": {"ring_stages": ring_stages, "smem_bytes": pd_smem} if persistent else None,
                     "dominant_kernel": ({"name": ("k_stream_matvec_q8<GATEUP>" if QUANT == "q8_0" else "k_stream_matvec_f16<GATEUP>") + " (gate/up + SwiGLU: the largest share of the step's bytes and time), stand-alone, CUDA events on the plan's stream",
                                          "achieved": per_kernel["gate_up"]["GB/s"], "peak": peak, "unit": "GB/s", "frac": per_kernel["gate_up"]["frac"],
                                          "bytes_per_launch": per_kernel["gate_up"]["bytes"], "ms_per_launch": per_kernel["gate_up"]["ms"]} if "gate_up" in per_kernel else None),
                     "other_kernels": per_kernel},
        "load": {"synthesise_s": gen_s, "upload_repack_s": load_s, "device_bytes": plan.device_bytes, "pipeline": plan.upload_info()},
    }
    if not args.no_cpu:
        orc = ge.import_oracle()
        # N = 1: the reported CPU baseline (bounded sample).  N > 1: a short run, only to carry driver-visible TP parity.
        tps, n, dt, cores, ref = cpu_leg(orc, model, tokens, args.cpu_budget if world == 1 else 6.0, 16 if world == 1 else 4)
        if world == 1:
            line["cpu_baseline"] = {"value": tps, "unit": "tok/s", "cores": cores, "kind": "port",
                                    "sample": f"{n} decode steps of the same workload in {dt:.1f} s (C restatement of InferenceCore.forwardJava, -O2, OpenMP rows)"}
        if world > 1:  # the other ranks wait here, then run the same parity calls (TP: every rank issues the same forwards)
            dist.broadcast_object_list([len(ref["ids"])], src=0)
        line["parity"] = parity_gate(plan, tokens, ref, want_logits=world == 1)
    plan.free()
    if not args.no_pp and world == 1 and WORKLOAD == "llama-3-8b" and QUANT == "q8_0":  # BASELINE config 3 is the 8B FP16 model
        del model, plan
        line["pp512"] = prefill_leg(pkg, lb, local, 512, 5)
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if "parity" in line and not line["parity"]["ids_equal"]:
        sys.stderr.write("PARITY FAILURE: GPU greedy ids differ from the oracle\n")
        return 3
    return 0


if __name__ == "__main__":
    sys.exit(main())
