#!/usr/bin/env python
"""Benchmark: train tokens/s (forward + back-propagation + Adam) of the large encoder-decoder
Transformer (6+6 layers, d_model 1024, 16 heads, FFN 4096, vocabulary 32000, sequence 256,
GLOBAL batch 512) on 1/2/4/8 B200, data-parallel over NCCL.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Launched by torchrun for N > 1 (one rank per GPU).  Rank 0 prints ONE JSON line.

  value     whole-job decoder tokens per second with the batch already resident in HBM;
            strong scaling: the global batch of 512 is split over the ranks.
  e2e       the same step through the host-buffer entry point: pinned host ids are copied to
            the device inside the timed region and the loss statistics are read back each step.
  roofline  the dominant kernel (tcgen05 tf32 GEMM at the FFN shape of this workload), timed
            alone with CUDA events, against a TF32 tensor peak MEASURED in this run the way
            MEASURED_PEAKS.json measured bf16 (a library GEMM at 8192^3 as a peak probe: best of
            10 = burst, back to back for 4 s = sustained); the other GEMM layouts of the step
            (input gradient, weight gradient, vocabulary projection) and the HBM-bound kernels
            (LayerNorm, cross-entropy, Adam; against the measured copy bandwidth) beside it.
  cpu_baseline  the unmodified reference CPU library (oracle/_ref) on the box's host cores,
            on a bounded sample of the same workload (N = 1 only).

--impl reference times that CPU library alone (the reference has no multi-GPU path and its
own CUDA path needs cuDNN + its build system, which this benchmark does not run).
--workload config3 | config4 print a profiling line for BASELINE.json's configs 3 and 4
(tokens/s of the training step on one GPU, and the reference CPU library at full size).

Data are synthetic: token ids uniform in [1, 32000), row lengths ~U[64, 256], right-padded
with id 0, seed 3; parameters are the reference's default random initialisation.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(name="config5_large_encdec", S_in=256, S_dec=256, V_in=32000, V_out=32000, E=1024, H=16, F=4096, L=6,
                global_batch=512, micro_batch=64, seed=3, min_len=64, max_len=256)
# reference config 2 (1+1 layers, E 64): every kernel is tiny, the step is bound by launching ~190 of them; only
# reachable with --workload config2, which prints a profiling line (step time with and without CUDA-graph replay)
SMALL_WORKLOAD = dict(name="config2_small_encdec", S_in=32, S_dec=32, V_in=1000, V_out=1000, E=64, H=4, F=128, L=1,
                      global_batch=32, micro_batch=32, seed=3, min_len=8, max_len=32)
# reference configs 3 (mid encoder-decoder) and 4 (long-sequence decoder-only stack, no padding): profiling lines
MID_WORKLOAD = dict(name="config3_mid_encdec", S_in=128, S_dec=128, V_in=8000, V_out=8000, E=512, H=8, F=2048, L=6,
                    global_batch=64, micro_batch=64, seed=1, min_len=32, max_len=128)
LONG_WORKLOAD = dict(name="config4_long_decoder_only", decoder_only=True, S_in=0, S_dec=1024, V_in=0, V_out=8000, E=512, H=8, F=2048, L=2,
                     global_batch=16, micro_batch=16, seed=2, min_len=1024, max_len=1024)
CPU_SAMPLE_BATCH = 8          # samples of the 512-sample config-5 step the reference CPU library is timed on
METRIC = "train tokens/s (fwd+bwd+Adam)"
UNIT = "tokens/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peaks = json.load(f)
        return dict(hbm_gbs=peaks["hbm_gbs"], tflops=peaks["bf16_tflops"], tflops_sustained=peaks.get("bf16_tflops_sustained"),
                    source="measured (MEASURED_PEAKS.json)")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


def synthetic_batch(rng, batch, w):
    import numpy as np

    def ids(S, V):
        if S == 0:
            return None
        x = rng.integers(1, V, size=(batch, S)).astype(np.float32)
        lengths = rng.integers(w["min_len"], w["max_len"] + 1, size=batch)
        x[np.arange(S)[None, :] >= lengths[:, None]] = 0
        return x
    return ids(w["S_in"], w["V_in"]), ids(w["S_dec"], w["V_out"]), ids(w["S_dec"], w["V_out"])


# ---------------------------------------------------------------------------------------
# reference CPU library (oracle/_ref) on a bounded sample
# ---------------------------------------------------------------------------------------

def time_reference_cpu(w, batch, steps):
    """Runs the unmodified reference CPU path (Transformer + CrossEntropyError3d + Adam) on
    `batch` samples of the workload for `steps` steps; returns (tokens/s of the best step, cores)."""
    import numpy as np
    from oracle import ref_runner
    cores = os.cpu_count() or 1
    rng = np.random.default_rng(w["seed"])
    enc, dec, tgt = synthetic_batch(rng, batch, w)
    spec = dict(mode="decoder" if w.get("decoder_only") else "transformer", B=batch, S_in=w["S_in"], S_dec=w["S_dec"], V_in=w["V_in"],
                V_out=w["V_out"], E=w["E"], H=w["H"], F=w["F"], L=w["L"], steps=steps, lr=1e-3, dump=0, random_parameters=1)
    tensors = {"dec_ids": dec, "targets": tgt}
    if enc is not None:
        tensors["enc_ids"] = enc
    _, seconds = ref_runner.run(spec, tensors, [], threads=cores)
    best = min(seconds[1:]) if len(seconds) > 1 else seconds[0]
    return batch * w["S_dec"] / best, cores, seconds


def workload_config(w, world, micro):
    """The `config` object of the result line: the workload both arms run (the reference arm a bounded sample of it)."""
    return {"workload": w["name"], "global_batch": w["global_batch"], "seq_len": w["S_dec"], "parallelism": f"dp{world}",
            "micro_batch": micro, "layers": "6+6", "d_model": w["E"], "heads": w["H"], "ffn": w["F"], "vocab": w["V_out"],
            "l2": "per-step working set (tens of GB of activations) far exceeds the 126 MB L2; batches rotate"}


def time_reference_gpu_path(w, batch, steps):
    """The reference's OWN CUDA path (cuBLAS SGEMM + cuDNN + opennn/kernel.cu, the loop body of train_cuda) on the
    same configuration and synthetic batch: the existing GPU implementation, for comparison only.  Needs the binary
    `make -C oracle cuda` builds; returns None without it."""
    import numpy as np
    from oracle import ref_runner
    if not ref_runner.cuda_available():
        return None
    rng = np.random.default_rng(w["seed"])
    enc, dec, tgt = synthetic_batch(rng, batch, w)
    spec = dict(mode="decoder_cuda" if w.get("decoder_only") else "transformer_cuda", B=batch, S_in=w["S_in"], S_dec=w["S_dec"], V_in=w["V_in"],
                V_out=w["V_out"], E=w["E"], H=w["H"], F=w["F"], L=w["L"], steps=steps, lr=1e-3, random_parameters=1)
    tensors = {"dec_ids": dec, "targets": tgt}
    if enc is not None:
        tensors["enc_ids"] = enc
    out, seconds = ref_runner.run(spec, tensors, ["loss"], cuda=True)
    timed = seconds[2:] if len(seconds) > 3 else seconds[1:]
    best = min(timed)
    return {"what": "reference's own CUDA path (cuBLAS SGEMM, cuDNN, opennn/kernel.cu), fp32, one GPU, same configuration and batch",
            "ms_per_step": 1e3 * best, "tokens_per_s": batch * w["S_dec"] / best, "steps_timed": len(timed),
            "loss_first_last": [float(out["loss"][0]), float(out["loss"][-2])] if "loss" in out else None}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOAD
    from oracle import ref_runner
    if not ref_runner.available():
        emit({"impl": "reference", "unavailable": "oracle/_ref/onn_ref_harness is not built (make -C oracle)"})
        return
    sample_batch = CPU_SAMPLE_BATCH
    steps = max(2, min(args.steps + min(args.warmup, 1), 3))
    start = time.time()
    value, cores, seconds = time_reference_cpu(w, sample_batch, steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": len(seconds) - 1,
        "warmup": 1, "ms_per_step": 1e3 * min(seconds[1:]), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, args.gpus, min(w["micro_batch"], w["global_batch"] // max(args.gpus, 1))),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "reference",
                         "sample": f"batch {sample_batch} of the {w['global_batch']}-sample step (same S, E, H, F, V, L), "
                                   f"best of {len(seconds) - 1} steps after 1 warm-up, OpenMP/Eigen on {cores} threads, -O2"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.time() - start,
    }
    emit(line)


# ---------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------

class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(gpu_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, sm_max, reasons = [], [], set()
        for row in self.file.read().splitlines():
            cells = [c.strip() for c in row.split(",")]
            if len(cells) < 9:
                continue
            try:
                sm.append(float(cells[1]))
                sm_max.append(float(cells[2]))
            except ValueError:
                continue
            for label, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), cells[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(label)
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def measure_tf32_peak(torch, sustained_seconds=4.0):
    """Dense TF32 tensor peak of this GPU, measured the way MEASURED_PEAKS.json measured bf16: a library GEMM
    (torch.matmul with TF32 operands allowed) at 8192^3, best of 10 launches (burst) and back to back for
    `sustained_seconds` (sustained, under the power cap).  A peak probe only: no product path calls it."""
    n = 8192
    a, b = torch.randn(n, n, device="cuda"), torch.randn(n, n, device="cuda")
    c = torch.empty(n, n, device="cuda")
    previous = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    flops = 2.0 * n ** 3
    for _ in range(3):
        torch.matmul(a, b, out=c)
    torch.cuda.synchronize()
    best = float("inf")
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(10):
        start.record()
        torch.matmul(a, b, out=c)
        stop.record()
        torch.cuda.synchronize()
        best = min(best, start.elapsed_time(stop) * 1e-3)
    sustained = None
    if sustained_seconds > 0:
        launches = max(10, int(sustained_seconds / best))
        start.record()
        for _ in range(launches):
            torch.matmul(a, b, out=c)
        stop.record()
        torch.cuda.synchronize()
        sustained = flops * launches / (start.elapsed_time(stop) * 1e-3) / 1e12
    torch.backends.cuda.matmul.allow_tf32 = previous
    how = "torch.matmul fp32 with TF32 operands allowed, 8192^3: best of 10 (burst)"
    if sustained_seconds > 0:
        how += " and, after the kernel timings, back to back for %.0f s (sustained)" % sustained_seconds
    return {"tf32_tflops": flops / best / 1e12, "tf32_tflops_sustained": sustained, "how": how}


def weight_gradient_splits(M, N, K):
    """The reduction split the Dense layer picks for dW = X^T D (M = in, N = out, K = rows): the count, up to 16, whose
    last wave of 256 x 256 tiles on 74 CTA pairs is fullest, each extra split charged 0.4 % for its pass of reduce-adds
    (choose_split_k in opennn_b200/csrc/layers.cu; restated here so that the timed launch is the layer's own)."""
    tiles, units = ((M + 255) // 256) * ((N + 255) // 256), 74
    if tiles >= 4 * units or K < 1024:
        return 1
    best, best_score = 1, 0.0
    for s in range(1, min(K // 512, 16) + 1):
        work = tiles * s
        waves = (work + units - 1) // units
        score = work / (waves * units) - 0.004 * s
        if score > best_score + 1e-9:
            best, best_score = s, score
    return best


# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch, from ncu captures of `bench.py --profile-kernel ...`
# (--set full --clock-control none, one kernel, two launches); the summaries of those captures are committed.
NCU_DRAM_BYTES_PER_LAUNCH = {
    "gemm_tc2_kernel<0,1> M16384 N4096 K1024": {"read": 110.0e6, "write": 218.9e6, "algorithmic": 84e6 + 268e6},
}


def time_gemm(capi, torch, M, N, K, a_major, b_major, copies, launches, split_k=0, bias=False, relu=False):
    """One GEMM shape of the step through onn_gemm, launched back to back on `copies` operand sets that together exceed
    L2, timed with CUDA events.  Majors as the layers use them: (0,1) Y = X W, (0,0) dX = D W^T, (1,1) dW = X^T D."""
    A = [torch.randn((M, K) if a_major == 0 else (K, M), device="cuda") for _ in range(copies)]
    B = [torch.randn((K, N) if b_major == 1 else (N, K), device="cuda") * 0.05 for _ in range(copies)]
    Cm = [torch.zeros(M, N, device="cuda") for _ in range(copies)]
    lda, ldb = (K if a_major == 0 else M), (N if b_major == 1 else K)
    bias_t = torch.zeros(N, device="cuda") if bias else None

    def launch(i):
        capi.gemm(A[i], B[i], Cm[i], M, N, K, lda, ldb, N, a_major, b_major, bias=bias_t, relu=relu, split_k=split_k)
    for i in range(copies):
        launch(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(launches):
        launch(i % copies)
    stop.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(stop) * 1e-3 / launches
    return seconds, A, B, Cm


def time_dominant_kernel(capi, torch, w, peaks, copies=4, launches=24, with_cublas=True, tf32=None, other_layouts=True):
    """The tcgen05 GEMM at the FFN-up shape of one micro-batch (M = 64*256 tokens, K = 1024,
    N = 4096), launched back to back on fresh buffers larger than L2, timed with CUDA events."""
    M, K, N = w["micro_batch"] * w["S_dec"], w["E"], w["F"]
    # copies x (64 + 16 + 256) MiB of operands and outputs: every launch misses L2
    seconds, A, B, Cm = time_gemm(capi, torch, M, N, K, 0, 1, copies, launches, bias=True, relu=True)
    flops = 2.0 * M * N * K
    achieved = flops / seconds / 1e12

    # the same product by cuBLAS with TF32 operands, for orientation (not part of any product path)
    cublas_tf32 = None
    if with_cublas:
        torch.backends.cuda.matmul.allow_tf32 = True
        for i in range(copies):
            torch.matmul(A[i], B[i], out=Cm[i])
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(launches):
            j = i % copies
            torch.matmul(A[j], B[j], out=Cm[j])
        stop.record()
        torch.cuda.synchronize()
        cublas_tf32 = flops / (start.elapsed_time(stop) * 1e-3 / launches) / 1e12
        torch.backends.cuda.matmul.allow_tf32 = False
    del A, B, Cm

    # the kernel computes with tf32 operands, so its roofline is the TF32 tensor peak measured in this run (burst: the
    # kernel is timed alone); the fraction of the bf16 burst peak of MEASURED_PEAKS.json stays beside it
    if tf32:
        peak, peak_source = tf32["tf32_tflops"], "dense TF32 burst, measured in this run (" + tf32["how"] + ")"
    else:
        peak, peak_source = 0.5 * peaks["tflops"], "half the dense bf16 burst peak (" + peaks["source"] + "): no TF32 probe in this run"
    traffic = NCU_DRAM_BYTES_PER_LAUNCH["gemm_tc2_kernel<0,1> M16384 N4096 K1024"]
    line = {"bound": "tensor", "kernel": "gemm_tc2_kernel<0,1> (Dense forward with bias + ReLU, two-CTA tcgen05, tf32 operands, fp32 accumulate)",
            "shape": {"M": M, "N": N, "K": K}, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak, "frac_of_bf16_burst": achieved / peaks["tflops"], "bf16_burst_tflops": peaks["tflops"],
            "peak_source": peak_source, "us_per_launch": seconds * 1e6, "cublas_tf32_same_shape_tflops": cublas_tf32,
            "traffic": (traffic["read"] + traffic["write"]) if (M, N, K) == (16384, 4096, 1024) else None,
            "algorithmic_bytes": 4.0 * (M * K + K * N + M * N)}
    if tf32:
        line["tf32_peak"] = tf32
    if other_layouts:
        V = w["V_out"]
        shapes = [("input_gradient dX = D W^T, gemm_tc2_kernel<0,0>", M, K, N, 0, 0, 0),          # FFN-up layer: [M, F] x [E, F]^T
                  ("weight_gradient dW = X^T D, gemm_tc2_kernel<1,1>, split-K", K, N, M, 1, 1, weight_gradient_splits(K, N, M)),
                  ("ffn_down forward Y = X W, gemm_tc2_kernel<0,1>", M, K, N, 0, 1, 0),             # [M, F] x [F, E]
                  ("vocabulary_projection Y = X W, gemm_tc2_kernel<0,1>", M, V, K, 0, 1, 0)]
        layouts = {}
        for name, m, n, k, a_major, b_major, splits in shapes:
            sec, a, b, c = time_gemm(capi, torch, m, n, k, a_major, b_major, 2 if n >= 8192 else copies, 12, split_k=splits)
            del a, b, c
            tflops = 2.0 * m * n * k / sec / 1e12
            layouts[name] = {"shape": {"M": m, "N": n, "K": k}, "split_k": splits, "us_per_launch": sec * 1e6, "achieved": tflops,
                             "frac": tflops / peak, "frac_of_bf16_burst": tflops / peaks["tflops"]}
        line["other_layouts"] = layouts
    return line


def time_attention_core(capi, torch, w):
    """One MultiHeadAttention layer of the benchmark's shape on 32 samples (attention weights 134 MB: larger than
    L2), forward and backward, timed with CUDA events: the fused attention-core kernels with their projections."""
    B, S, E, H = 32, w["S_dec"], w["E"], w["H"]
    torch.manual_seed(0)
    p = {n: torch.randn(E, E, device="cuda") * 0.03 for n in ("Wq", "Wk", "Wv", "Wo")}
    p.update({n: torch.zeros(E, device="cuda") for n in ("bq", "bk", "bv", "bo")})
    x = torch.randn(B, S, E, device="cuda")
    dy = torch.randn(B, S, E, device="cuda")
    y, ws = capi.mha_fwd(x, x, p, H, True)
    capi.mha_bwd(x, x, p, H, True, ws, dy)
    torch.cuda.synchronize()
    start, middle, stop = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    start.record()
    y, ws = capi.mha_fwd(x, x, p, H, True)
    middle.record()
    capi.mha_bwd(x, x, p, H, True, ws, dy)
    stop.record()
    torch.cuda.synchronize()
    return {"kernel": "attention_core_kernel<64,false|true> inside onn_mha_fwd / onn_mha_bwd", "shape": {"B": B, "H": H, "Sq": S, "Sk": S, "E": E},
            "mha_fwd_us": start.elapsed_time(middle) * 1e3, "mha_bwd_us": middle.elapsed_time(stop) * 1e3}


def time_row_kernels(capi, torch, w, peaks=None, repeats=3):
    """The HBM-bound kernels of the step at the sizes of one micro-batch (and the whole parameter arena for Adam),
    on tensors larger than L2 with every row active, timed with CUDA events: one warm-up launch, then `repeats`
    groups of four back-to-back launches (the host runs ahead of the device, so the events bracket device time and not
    the time the host needs to issue a launch), best group; with `peaks`, each as a fraction of the measured copy bandwidth."""
    rows, E, V = w["micro_batch"] * w["S_dec"], w["E"], w["V_out"]
    out = {}

    def timed(name, fn, algorithmic_bytes):
        fn()
        torch.cuda.synchronize()
        best = float("inf")
        group = 4
        for _ in range(repeats):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(group):
                fn()
            stop.record()
            torch.cuda.synchronize()
            best = min(best, start.elapsed_time(stop) * 1e-3 / group)
        out[name] = {"us": best * 1e6, "algorithmic_MB": algorithmic_bytes / 1e6, "achieved_gbs": algorithmic_bytes / best / 1e9}
        if peaks:
            out[name]["frac"] = algorithmic_bytes / best / 1e9 / peaks["hbm_gbs"]

    # every kernel straight through the C ABI on buffers made once: a Python wrapper that allocates its outputs takes
    # longer than a 50 us kernel runs, and the events would then time the host
    import ctypes
    L, P, i64, stream = capi.lib(), capi.ptr, ctypes.c_int64, capi.stream_ptr()
    x, r, dy, y, total, dx = (torch.randn(rows, E, device="cuda") for _ in range(6))
    gamma, beta = torch.ones(E, device="cuda"), torch.zeros(E, device="cuda")
    mean, inv_std = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    dgamma, dbeta, sums = (torch.zeros(E, device="cuda") for _ in range(3))
    eps = ctypes.c_float(float(torch.finfo(torch.float32).eps))
    workspace = torch.empty(int(L.onn_layernorm_bwd_workspace_floats(i64(rows), i64(E))), device="cuda")

    def norm_forward():
        capi.check(L.onn_layernorm_fwd(P(x), P(r), P(gamma), P(beta), P(y), P(total), P(mean), P(inv_std), None, i64(rows), i64(E), eps,
                                       ctypes.c_uint32(0), stream), "onn_layernorm_fwd")

    def norm_backward():
        capi.check(L.onn_layernorm_bwd(P(dy), P(r), None, P(total), P(mean), P(inv_std), P(gamma), P(dx), P(dgamma), P(dbeta), P(sums),
                                       i64(rows), i64(E), P(workspace), ctypes.c_uint32(0), stream), "onn_layernorm_bwd")
    timed("layernorm_fwd_with_residual", norm_forward, 16 * rows * E)
    timed("layernorm_bwd_two_gradients", norm_backward, 16 * rows * E)
    del x, r, dy, y, total, dx
    logits = torch.randn(rows, V, device="cuda")
    targets = torch.randint(1, V, (rows,), device="cuda").float()
    # (the Python wrapper of the loss also reads the statistics back after every call)
    count, stats, scratch = torch.empty(1, device="cuda"), torch.empty(4, device="cuda"), torch.empty(2 * rows, device="cuda")
    capi.check(capi.lib().onn_ce3d_count_active(capi.ptr(targets), ctypes.c_int64(rows), ctypes.c_int64(V), capi.ptr(count), capi.stream_ptr()), "count")

    def loss_kernel(flags):
        capi.check(capi.lib().onn_ce3d_fwd_bwd(capi.ptr(logits), capi.ptr(targets), capi.ptr(count), None, capi.ptr(stats), capi.ptr(scratch),
                                               ctypes.c_int64(rows), ctypes.c_int64(V), 0, ctypes.c_uint32(flags), capi.stream_ptr()), "onn_ce3d_fwd_bwd")
    timed("ce3d_fwd_bwd", lambda: loss_kernel(0), 8 * rows * V)
    timed("ce3d_fwd_bwd_two_sweeps", lambda: loss_kernel(32), 8 * rows * V)
    del logits
    n = 274_700_000                                   # the parameter count of config 5, rounded
    p, m, v, g = (torch.zeros(n, device="cuda") for _ in range(4))
    g.fill_(1e-3)
    sq = capi.grad_sqnorm(g)
    timed("adam", lambda: capi.adam(p, m, v, g, 2, sqnorm=sq, zero_grad=False), 32 * n)
    norm_workspace = torch.empty(int(L.onn_grad_sqnorm_workspace_floats(i64(n))), device="cuda")
    timed("grad_sqnorm", lambda: capi.check(L.onn_grad_sqnorm(P(g), i64(n), P(sq), P(norm_workspace), stream), "onn_grad_sqnorm"), 4 * n)
    return {"kernel": "layernorm_fwd/bwd, ce3d_fwd_bwd, adam", "bound": "hbm", "peak_gbs": peaks["hbm_gbs"] if peaks else None,
            "peak_source": ("copy bandwidth, " + peaks["source"]) if peaks else None, "kernels": out}


def time_under_contention(capi, torch, w):
    """What a resident kernel of another library (NCCL's CTAs during a collective) costs the persistent kernels: the FFN
    GEMM, an attention layer and a LayerNorm pair of one micro-batch, timed alone and while `held` SMs are occupied by
    the library's bounded stand-in kernel on a second stream -- with a fixed share of the tiles per CTA and with tiles
    handed out by counter (onn_set_dynamic_work)."""
    import ctypes
    import numpy as np
    L = capi.lib()
    M, K, N = w["micro_batch"] * w["S_dec"], w["E"], w["F"]
    A, B, C = torch.randn(M, K, device="cuda"), torch.randn(N, K, device="cuda") / 32, torch.empty(M, N, device="cuda")
    Bt, H, S, E = 32, w["H"], w["S_dec"], w["E"]
    rng = np.random.default_rng(0)
    p = {n: torch.from_numpy((rng.standard_normal((E, E)) / 32).astype(np.float32)).cuda() for n in ("Wq", "Wk", "Wv", "Wo")}
    p.update({n: torch.zeros(E, device="cuda") for n in ("bq", "bk", "bv", "bo")})
    x, dy = torch.randn(Bt, S, E, device="cuda"), torch.randn(Bt, S, E, device="cuda")
    rows = torch.randn(M, E, device="cuda")
    gamma, beta = torch.ones(E, device="cuda"), torch.zeros(E, device="cuda")
    side = torch.cuda.Stream()

    def gemm():
        capi.gemm(A, B, C, M, N, K, K, K, N, 0, 0)

    def attention():
        y, ws = capi.mha_fwd(x, x, p, H, True)
        capi.mha_bwd(x, x, p, H, True, ws, dy)

    def norms():
        y, mean, inv_std, _ = capi.layernorm_fwd(rows, gamma, beta)
        capi.layernorm_bwd(rows, rows, mean, inv_std, gamma)

    def timed(fn, repeats, held):
        # the median of five: a stand-in that got its SMs late in one repeat must not decide the figure
        seen = []
        for _ in range(5):
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if held:
                capi.check(L.onn_selftest_hold_sms(held, ctypes.c_int64(12_000_000), ctypes.c_void_p(side.cuda_stream)), "onn_selftest_hold_sms")
                torch.cuda._sleep(1_000_000)               # ~0.5 ms: the stand-in has its SMs before the timed launches start
            start.record()
            for _ in range(repeats):
                fn()
            stop.record()
            torch.cuda.synchronize()
            seen.append(start.elapsed_time(stop) / repeats)
        return statistics.median(seen)

    out = {}
    for fn in (gemm, attention, norms):
        fn()
    for mode, label in ((0, "fixed_share"), (1, "by_counter")):
        previous = L.onn_set_dynamic_work(mode)
        try:
            for fn, name, repeats in ((gemm, "ffn_gemm", 20), (attention, "attention_layer_fwd_bwd", 4), (norms, "layernorm_fwd_bwd", 8)):
                fn()
                out[f"{name}_{label}_ms"] = {f"held_{held}": round(timed(fn, repeats, held), 4) for held in (0, 8, 16, 32)}
        finally:
            L.onn_set_dynamic_work(previous)
    if L.onn_gemm_device_status() != 0:
        raise SystemExit("a kernel gave up on a bounded wait: the numbers are void")
    return {"kernel": "two-CTA GEMM 16384 x 4096 x 1024, attention layer 32 x 16 heads x 256 x 256, LayerNorm 16384 x 1024: alone and with SMs held",
            "contention": out}


def time_greedy_decode(trainer, torch, w, rows, tokens):
    """Greedy decoding of `rows` source sequences with cached keys and values, `tokens` target positions each (the
    caller of the same layers on the inference side): one eager call, one that captures a graph per position, then timed
    replays.  Random parameters, no END token, so every row runs to the full length."""
    import time
    import numpy as np
    t = trainer.Trainer(trainer.TRANSFORMER, w["S_in"], tokens, w["V_in"], w["V_out"], w["E"], w["H"], w["F"], w["L"], rows)
    rng = np.random.default_rng(0)
    t.set_parameters((0.02 * rng.standard_normal(t.parameters_number)).astype(np.float32))
    source = rng.integers(1, w["V_in"], size=(rows, w["S_in"])).astype(np.float32)
    reference = t.greedy_decode(source, end_id=-1, cached=True)
    t.greedy_decode(source, end_id=-1, cached=True)
    best = float("inf")
    same = True
    for _ in range(2):
        torch.cuda.synchronize()
        start = time.perf_counter()
        out = t.greedy_decode(source, end_id=-1, cached=True)
        best = min(best, time.perf_counter() - start)
        same = same and bool((out == reference).all())
    t.close()
    return {"decode": "greedy, cached keys and values, one CUDA graph per position", "rows": rows, "tokens_per_row": tokens - 1,
            "seconds": best, "tokens_per_s": rows * (tokens - 1) / best, "replay_matches_eager": same}


def time_classifier_step(trainer, torch, w, rows, steps):
    """Training step of the text-classification network (Embedding -> self-attention -> max pooling -> Dense<2> head,
    CrossEntropyError2d, Adam) at the benchmark's layer sizes, `rows` samples per step, ids resident on the device."""
    import numpy as np
    classes = 8
    c = trainer.TextClassifier(w["V_in"], w["S_in"], w["E"], w["H"], [w["F"]], classes, rows)
    rng = np.random.default_rng(1)
    ids = torch.from_numpy(rng.integers(1, w["V_in"], size=(rows, w["S_in"])).astype(np.float32)).cuda()
    targets = torch.from_numpy(np.eye(classes, dtype=np.float32)[rng.integers(0, classes, rows)]).cuda()
    for _ in range(3):
        c.step_device(ids, targets, update=True)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        error, _ = c.step_device(ids, targets, update=True)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    parameters = c.parameters_number
    c.close()
    return {"classifier": "TextClassificationNetwork, one attention layer, hidden %d, %d classes" % (w["F"], classes), "rows": rows,
            "sequence": w["S_in"], "parameters": parameters, "ms_per_step": ms, "tokens_per_s": rows * w["S_in"] / (1e-3 * ms),
            "last_error": error}


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    w = WORKLOAD
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torchrun for --gpus > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local_rank)

    from opennn_b200 import build
    build(verbose=False)
    from opennn_b200 import capi, trainer

    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    if args.workload != "config5":
        w = {"config2": SMALL_WORKLOAD, "config3": MID_WORKLOAD, "config4": LONG_WORKLOAD}[args.workload]
    if args.micro_batch:
        w = dict(w, micro_batch=args.micro_batch)
    peaks = measured_peaks()
    if args.profile_kernel == "gemm":
        # small stand-alone case for an ncu capture of the dominant kernel: 2 warm-up + 2 timed launches, 0.7 GB on the device
        emit(dict(time_dominant_kernel(capi, torch, w, peaks, copies=2, launches=2, with_cublas=False, other_layouts=False), profiling_only=True))
        return
    if args.profile_kernel == "rowwise":
        emit(dict(time_row_kernels(capi, torch, w, peaks, repeats=1), profiling_only=True))
        return
    if args.profile_kernel == "attention":
        emit(dict(time_attention_core(capi, torch, w), profiling_only=True))
        return
    if args.profile_kernel == "contention":
        emit(dict(time_under_contention(capi, torch, w), profiling_only=True))
        return
    if args.profile_kernel == "classifier":
        emit(dict(time_classifier_step(trainer, torch, w, args.profile_batch or 64, max(args.steps, 5)), profiling_only=True))
        return
    if args.profile_kernel == "decode":
        rows = args.profile_batch or 8
        emit(dict(time_greedy_decode(trainer, torch, w, rows, args.decode_tokens or w["S_dec"]), profiling_only=True))
        return
    if args.profile_batch:
        w = dict(w, global_batch=args.profile_batch, name=w["name"] + f" (profiling batch {args.profile_batch})")
    local_batch = w["global_batch"] // world
    micro = min(w["micro_batch"], local_batch)
    kind = trainer.DECODER_ONLY if w.get("decoder_only") else trainer.TRANSFORMER
    t = trainer.Trainer(kind, w["S_in"], w["S_dec"], w["V_in"], w["V_out"], w["E"], w["H"], w["F"], w["L"], micro)
    if world > 1:
        # host-side check first: every rank present, same parameter arena and micro-batch on all of them
        comm = trainer.dp_init_from_torch(signature={"parameters": t.parameters_number, "micro_batch": micro, "workload": w["name"]})
        t.set_dp(comm, world)

    # synthetic batches: the same global stream on every rank, each rank keeps its contiguous slice
    rng = np.random.default_rng(w["seed"])
    pool = 3
    host_batches, device_batches = [], []
    for _ in range(pool):
        enc, dec, tgt = synthetic_batch(rng, w["global_batch"], w)
        pinned = [None if x is None else torch.from_numpy(np.ascontiguousarray(x)).pin_memory()
                  for x in trainer.shard_batch((dec, enc, tgt), rank, world)]
        host_batches.append(pinned)
        device_batches.append([None if x is None else x.cuda() for x in pinned])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = t.stream()
    tokens_per_step = w["global_batch"] * w["S_dec"]

    def timed(step_fn, steps):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            t.parameters_ready()                  # nothing of the warm-up's parameter gathers is carried in ...
            start.record(stream)
            for i in range(steps):
                step_fn(i)
            t.parameters_ready()                  # ... and the last step's are inside the timed region
            stop.record(stream)
        barrier()
        elapsed = torch.tensor([start.elapsed_time(stop)], device="cuda")
        if world > 1:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        return float(elapsed.item()) * 1e-3

    def device_step(i):
        d, e, g = device_batches[i % pool]
        t.step_device(d, e, g, update=True, want_statistics=False)

    last_stats = [None]

    def host_step(i):
        d, e, g = host_batches[i % pool]
        last_stats[0] = t.step_host(d, e, g, update=True, want_statistics=True)

    warmup = args.warmup if args.profile_batch else max(args.warmup, 3)
    for i in range(warmup):
        device_step(i)
    barrier()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches_before = capi.lib().onn_launch_count()
    seconds = timed(device_step, args.steps)
    launches = capi.lib().onn_launch_count() - launches_before
    clocks = sampler.stop() if sampler else None

    if args.profile_batch or args.workload != "config5":
        line = {"profiling_only": True, "workload": w["name"], "ms_per_step": 1e3 * seconds / args.steps, "gpu_launches": int(launches),
                "tokens_per_s": tokens_per_step * args.steps / seconds, "steps": args.steps, "clocks": clocks,
                "config": {k: w[k] for k in ("S_in", "S_dec", "V_out", "E", "H", "F", "L", "global_batch", "micro_batch")}}
        if args.workload != "config5":
            # the same steps launched kernel by kernel, to show what the graph replay of the micro-batch saves
            t.set_graph_capture(False)
            device_step(0)
            line["ms_per_step_without_graphs"] = 1e3 * timed(device_step, args.steps) / args.steps
            status = capi.lib().onn_gemm_device_status()
            if status != 0:
                raise SystemExit("a kernel gave up on a bounded wait: the numbers are void")
            if rank == 0 and args.workload in ("config3", "config4") and not args.no_cpu_baseline:
                t.close()
                gpu_reference = time_reference_gpu_path(w, w["global_batch"], 8)
                if gpu_reference:
                    line["reference_gpu_path"] = gpu_reference
            if rank == 0 and args.workload in ("config3", "config4") and not args.no_cpu_baseline:
                # the reference CPU library on the same configuration at full size (second of two steps)
                from oracle import ref_runner
                if ref_runner.available():
                    value, cores, step_seconds = time_reference_cpu(w, w["global_batch"], 2)
                    line["cpu_baseline"] = {"value": value, "unit": UNIT, "cores": cores, "kind": "reference", "seconds_per_step": step_seconds,
                                            "sample": "the whole configuration, second of 2 steps, unmodified reference CPU library, "
                                                      f"OpenMP/Eigen on {cores} threads, -O2"}
        if rank == 0:
            emit(line)
        t.close()
        return
    host_step(0)                                  # warm the host path (staging buffers)
    e2e_seconds = timed(host_step, args.steps)
    status = capi.lib().onn_gemm_device_status()
    if status != 0:
        raise SystemExit("a tcgen05 GEMM gave up on a bounded wait: the numbers are void")

    # Data-parallel runs: what the gradient exchange costs.  (a) the all-reduce of the whole gradient arena on its own,
    # through the library's communicator, as bus bandwidth 2(n-1)/n * bytes / time; (b) the same local batches stepped
    # without any exchange: the difference to the data-parallel step is the time the exchange is NOT hidden behind
    # back-propagation (replicas diverge from here on, which no longer matters: nothing is measured after it).
    # --trace-phases: where a step's time goes on each rank (events on the trainer's stream at the start of a step, after
    # the last micro-batch's forward pass, after its back-propagation, after the update), on untimed steps after the
    # timed ones; with it on the exchanging micro-batch runs kernel by kernel (a segment replay has no such events)
    phases = None
    if args.trace_phases:
        t.trace_phases(True)
        rows = []
        for i in range(6):
            device_step(i)
            rows.append(t.last_step_phases())
        t.trace_phases(False)
        mine = torch.tensor([statistics.median(r[k] for r in rows[1:]) for k in range(3)], device="cuda")
        if world > 1:
            gathered = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(gathered, mine)
        else:
            gathered = [mine]
        phases = {"unit": "ms, median of 5 steps, per rank", "forward_incl_earlier_micro_batches": [round(float(g[0]), 2) for g in gathered],
                  "back_propagation_last_micro_batch": [round(float(g[1]), 2) for g in gathered], "update": [round(float(g[2]), 2) for g in gathered]}

    allreduce = None
    if world > 1:
        import ctypes
        arena = torch.zeros(t.parameters_number, device="cuda")
        torch_stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

        def exchange(_):
            capi.check(capi.lib().onn_dp_allreduce(comm, capi.ptr(arena), ctypes.c_int64(arena.numel()), torch_stream), "onn_dp_allreduce")
            capi.check(capi.lib().onn_dp_wait(comm, torch_stream), "onn_dp_wait")

        def timed_on_current(fn, repeats):
            barrier()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(repeats):
                fn(i)
            stop.record()
            barrier()
            elapsed = torch.tensor([start.elapsed_time(stop)], device="cuda")
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
            return float(elapsed.item()) * 1e-3 / repeats

        sharded = os.environ.get("ONN_B200_DP_SHARDED", "1") != "0"
        exchange(0)
        exchange_seconds = timed_on_current(exchange, 5)
        t.set_dp(None, 1)
        device_step(0)
        local_seconds = timed(device_step, args.steps) / args.steps
        arena_bytes = 4 * t.parameters_number
        allreduce = {"update": "sharded: reduce-scatter by buckets, Adam on 1/world of the arena, all-gather" if sharded else
                               "all-reduce by buckets, the whole update on every rank",
                     "carve_sms": int(os.environ.get("ONN_B200_DP_CARVE_SMS", "0") or 0),
                     "bytes": arena_bytes, "alone_ms": 1e3 * exchange_seconds,
                     "bus_gbs": 2 * (world - 1) / world * arena_bytes / exchange_seconds / 1e9,
                     "step_ms_without_exchange": 1e3 * local_seconds,
                     "exposed_ms_per_step": 1e3 * (seconds / args.steps - local_seconds)}

    if rank == 0:
        t.close()                                     # the stand-alone kernel timings below want the trainer's memory
        # the kernel figures belong to the one-GPU line; data-parallel lines keep the dominant kernel and a burst probe only
        # burst against burst: the peak probe's best-of-10 first, the kernels next, the seconds-long sustained probe last
        # (it leaves the GPU at its power-capped clocks, which is not the state the burst figure was taken in)
        tf32 = measure_tf32_peak(torch, sustained_seconds=0.0)
        roofline = time_dominant_kernel(capi, torch, w, peaks, tf32=tf32, other_layouts=world == 1)
        if world == 1:
            roofline["hbm_kernels"] = time_row_kernels(capi, torch, w, peaks)
            sustained = measure_tf32_peak(torch, sustained_seconds=4.0)
            tf32["tf32_tflops_sustained"], tf32["how"] = sustained["tf32_tflops_sustained"], sustained["how"]
            tf32["tf32_tflops_second_burst"] = sustained["tf32_tflops"]
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            from oracle import ref_runner
            if ref_runner.available():
                value, cores, step_seconds = time_reference_cpu(w, CPU_SAMPLE_BATCH, 2)
                cpu = {"value": value, "unit": UNIT, "cores": cores, "kind": "reference",
                       "sample": f"batch {CPU_SAMPLE_BATCH} of the {w['global_batch']}-sample step (same S, E, H, F, V, L), second of 2 steps, "
                                 f"unmodified reference CPU library, OpenMP/Eigen on {cores} threads, -O2"}
        ids_bytes = 4 * w["global_batch"] * (2 * w["S_dec"] + w["S_in"])
        line = {
            "metric": METRIC, "value": tokens_per_step * args.steps / seconds, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": 1e3 * seconds / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "tf32 operands, f32 accumulate/storage", "data": "synthetic",
            "config": workload_config(w, world, micro),
            "e2e": {"value": tokens_per_step * args.steps / e2e_seconds, "unit": UNIT, "ms_per_step": 1e3 * e2e_seconds / args.steps,
                    "h2d_bytes_per_step": ids_bytes, "d2h_bytes_per_step": 4 * (4 * (local_batch // micro) + 3) * world,
                    "last_loss": last_stats[0][0] if last_stats[0] else None},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            # decoder tokens are the metric's unit; the encoder side of every sample is computed as well
            "encoder_plus_decoder_tokens_per_s": (w["global_batch"] * (w["S_dec"] + w["S_in"])) * args.steps / seconds,
        }
        if allreduce:
            line["allreduce"] = allreduce
        if phases:
            line["phases"] = phases
        emit(line)

    t.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--trace-phases", action="store_true",
                        help="add per-rank forward / back-propagation / update times of a step (untimed extra steps) to the line")
    parser.add_argument("--profile-batch", type=int, default=0,
                        help="profiling aid: run the device-resident loop only, on a global batch of this many samples "
                             "(the line it prints is not a benchmark result)")
    parser.add_argument("--micro-batch", type=int, default=0, help="samples per micro-batch (default: the workload's own)")
    parser.add_argument("--workload", default="config5", choices=["config5", "config2", "config3", "config4"],
                        help="config5 is the benchmark; config2 prints a profiling line for the launch-bound small network, config3 / config4 "
                             "one for the mid encoder-decoder and the long-sequence decoder-only stack (with the reference CPU library beside it)")
    parser.add_argument("--profile-kernel", nargs="?", const="gemm", default=None, choices=["gemm", "attention", "rowwise", "decode", "classifier", "contention"],
                        help="profiling aid: launch only the dominant GEMM (FFN-up shape) four times on buffers larger than L2, "
                             "or only one attention layer (forward and backward, 32 samples) twice, or only the HBM-bound kernels "
                             "(LayerNorm forward / backward, fused softmax-cross-entropy, Adam) at the benchmark's sizes; decode: greedy decoding "
                             "with cached keys and values of --profile-batch rows (default 8) over --decode-tokens positions; classifier: "
                             "training steps of the text-classification network at the benchmark's layer sizes")
    parser.add_argument("--decode-tokens", type=int, default=0, help="target positions for --profile-kernel decode (default: the workload's)")
    args = parser.parse_args()
    # Libraries (NCCL prints its version) write to file descriptor 1: keep it for the ONE JSON line by
    # pointing fd 1 at stderr while the benchmark runs and printing the line to the saved descriptor.
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    global _result_stream
    _result_stream = os.fdopen(saved_stdout, "w")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
    _result_stream.flush()


_result_stream = None


def emit(line):
    """Prints the result line on the process's original stdout."""
    stream = _result_stream or sys.stdout
    stream.write(json.dumps(line) + "\n")
    stream.flush()


if __name__ == "__main__":
    main()
