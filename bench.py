#!/usr/bin/env python3
"""Benchmark of the SmolLM2 training step (forward + backward + mixed-precision AdamW).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Own arm (default): SmolLM2-360M, bf16 mixed precision, 16 sequences x 2048 tokens per GPU, random-init
weights N(0, 0.02^2) (RMSNorm gains 1) from seed 42 and the reference's LCG token stream; one process per GPU
(torchrun for N > 1), data-parallel with a bucketed bf16 NCCL all-reduce overlapped with backward. Prints ONE
JSON line on rank 0:
  value  : training tokens/s over all N GPUs with the step's token batch already resident in HBM
           (CUDA events on the backend's stream, barrier + synchronize on both sides, max over ranks);
  e2e    : the same through the public API bm_train_step() with HOST int32 buffers — host->device copy of
           inputs/targets and device->host read of the loss inside the timed region, every step;
  roofline: the tcgen05 GEMM kernel, achieved TFLOP/s = algorithmic 2*M*N*K FLOPs / per-launch CUDA-event time
           collected live in two more steps of the same workload right after the timed ones (there the weight-gradient
           GEMMs run on the main stream; in the timed steps they overlap other kernels, which an event pair would
           also measure), against the measured bf16 peak (MEASURED_PEAKS.json);
  cpu_baseline: the reference's own host code + kernels running on this box's CPU cores (oracle/_ref), on a
           bounded sample of the same model (rank 0, N = 1 only).

Other workloads (--workload attention | gemm | decode): the isolated GQA flash attention, the linear-layer GEMMs per
shape, and Q8 prefill + greedy decode at batch 1 and 64; one JSON line per case.

Reference arm (--impl reference): times oracle/_ref (the reference's C11 host code and its Metal kernel sources
compiled for the CPU) on the host cores, same model, each step a bounded sample (1 sequence x 32 tokens).
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "bare.metal_b200"))
import bmapi  # noqa: E402

MODEL = "smollm2-360m"
PER_GPU_BATCH, SEQ_LEN = 16, 2048
METRIC = "train_tokens_per_sec"
UNIT = "tokens/s"
DATASHEET_BF16_TFLOPS = 2250.0


def flops_per_token(a, S):
    """Algorithmic training FLOPs per token: 6 x matmul parameters (tied head counted once) + causal attention
    6*S*NH*HD*L (half of the full S^2 work), no recompute credited."""
    HD = a.head_dim
    per_layer = a.n_heads * HD * a.dim * 2 + 2 * a.n_kv_heads * HD * a.dim + 3 * a.hidden_dim * a.dim
    p_mm = per_layer * a.n_layers + a.vocab_size * a.dim
    return 6.0 * p_mm + 6.0 * S * a.n_heads * HD * a.n_layers


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.lines:
            if ts < t0 or ts > t1 + 0.3:
                continue
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                smax = float(p[2])
            except ValueError:
                continue
            for name, val in zip(names, p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


def fill_weights(lib, model, a, seed=42, std=0.02):
    n = C.c_size_t()
    ptr = lib.bmx_model_weight_buffer(model, C.byref(n))
    buf = np.ctypeslib.as_array(ptr, (n.value,))
    rng = np.random.default_rng(seed)
    off = 0
    for name, shape in bmapi.weight_shapes(a):
        cnt = int(np.prod(shape))
        if name.startswith("ln"):
            buf[off:off + cnt] = 1.0
        else:
            # generate in slices to bound peak host memory
            step = 1 << 24
            for s in range(0, cnt, step):
                e = min(cnt, s + step)
                buf[off + s:off + e] = rng.standard_normal(e - s, dtype=np.float32) * np.float32(std)
        off += cnt


REF_ARM_MAX_THREADS = 16   # every box quotes the same baseline, whatever number of cores its lease exposes
REF_ARM_BUDGET_S = 200.0   # the timed steps of the reference arm stop after this much CPU wall time


def reference_tokens_per_sec(steps, warmup, S_ref=32, B_ref=1):
    """The reference's own training step on the host cores (oracle/_ref; the one place besides the parity checks where this
    file executes anything under oracle/). Returns (tokens/s, threads, sample text, ms per step).

    A launcher may export OMP_NUM_THREADS=1 for its workers (torch.distributed.run does): the thread count is therefore set
    explicitly, to the cores this process may run on, capped at REF_ARM_MAX_THREADS. Timed steps stop once REF_ARM_BUDGET_S is
    used up (at least two are always timed); the count actually timed is part of the sample text."""
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    threads = max(1, min(avail, REF_ARM_MAX_THREADS))
    os.environ["OMP_NUM_THREADS"] = str(threads)   # read by libgomp when the oracle library is the first to load it
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_check as oc
    ref = oc.load_reference()
    if ref is None:
        return None, 0, "oracle/_ref/libbm_ref.so not built", None
    try:   # libgomp may have been initialised already with the launcher's value
        gomp = C.CDLL("libgomp.so.1")
        gomp.omp_set_num_threads(C.c_int(threads))
        gomp.omp_get_max_threads.restype = C.c_int
        threads = int(gomp.omp_get_max_threads())
    except OSError:
        pass
    a = bmapi.make_arch(MODEL)
    a.precision = bmapi.BM_PRECISION_BF16
    ctx = ref.bm_create(bmapi.BM_DEVICE_METAL)
    model = ref.bm_create_model(ctx, C.byref(a))
    # the reference has no setter for weights either; write through its model struct's weight buffer via the .bin path
    w_path = "/tmp/bm_bench_ref_360m.bin"
    if not os.path.exists(w_path) or os.path.getsize(w_path) < 1000:
        w = bmapi.make_weights(a)
        bmapi.write_bin_checkpoint(w_path, a, w)
        del w
    ref.bm_load_weights(model, w_path.encode())
    ref.bmref_set_precision(model, bmapi.BM_PRECISION_BF16)
    cfg = bmapi.train_config(lr=3e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, seq_len=S_ref)
    tr = ref.bm_create_trainer(ctx, model, C.byref(cfg))
    x, y = bmapi.lcg_batch(B_ref * (steps + warmup), S_ref, a.vocab_size)
    times = []
    t_begin = time.perf_counter()
    for i in range(steps + warmup):
        if len(times) >= 2 and time.perf_counter() - t_begin > REF_ARM_BUDGET_S:
            break
        xs = np.ascontiguousarray(x[i * B_ref:(i + 1) * B_ref])
        ys = np.ascontiguousarray(y[i * B_ref:(i + 1) * B_ref])
        t0 = time.perf_counter()
        loss = ref.bm_train_step(tr, bmapi.as_int_ptr(xs), bmapi.as_int_ptr(ys), B_ref, S_ref)
        dt = time.perf_counter() - t0
        if i >= warmup or (i >= 1 and time.perf_counter() - t_begin > REF_ARM_BUDGET_S / 2):
            times.append(dt)
        if not np.isfinite(loss):
            raise RuntimeError("reference step returned a non-finite loss")
    ref.bm_destroy_trainer(tr)
    ref.bm_destroy_model(model)
    ref.bm_destroy(ctx)
    tps = B_ref * S_ref * len(times) / sum(times)
    sample = (f"{MODEL} bf16-weights, {B_ref} sequence x {S_ref} tokens per step, {len(times)} timed steps of the {steps} asked for "
              f"(time budget {REF_ARM_BUDGET_S:.0f} s), reference C11 host code + its kernel sources on {threads} host threads "
              f"(cap {REF_ARM_MAX_THREADS}; {avail} cores available)")
    return tps, threads, sample, sum(times) / len(times) * 1e3


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    out = reference_tokens_per_sec(args.steps, args.warmup)
    if out[0] is None:
        print(json.dumps({"impl": "reference", "unavailable": out[2]}))
        return 0
    tps, cores, sample, ms = out
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{MODEL} train step, bf16 weights / fp32 math (the reference's bf16 mode), CPU", "sample": sample},
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "reference", "sample": sample},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


def run_attention(args):
    """Isolated causal GQA flash attention forward + backward, bf16, 15 query / 5 KV heads, head_dim 64, batch 16
    (batch 4 at 8192 keeps the capture small); one JSON line per sequence length."""
    from bmcapi import BMC_BF16, Backend, Ptr
    lib = bmapi.load_product()
    be = Backend(lib)
    lib.bmc_timer_begin.argtypes = [C.c_void_p, C.c_int]
    lib.bmc_timer_end.argtypes = [C.c_void_p, C.c_int]
    lib.bmc_timer_end.restype = C.c_float
    NH, NKV, HD = 15, 5, 64
    QD, KV = NH * HD, NKV * HD
    ld = QD + 2 * KV
    peaks, src = measured_peaks()
    for S in ([args.seq_len] if args.seq_len != SEQ_LEN or "--seq-len" in sys.argv else [512, 2048, 8192]):
        B = 16 if S <= 2048 else 4
        M = B * S
        rng = np.random.default_rng(S)
        d = be.put(rng.standard_normal((M, ld)).astype(np.float32), BMC_BF16)
        dgo = be.put(rng.standard_normal((M, QD)).astype(np.float32), BMC_BF16)
        out, lse, dg = be.zeros(M * QD, BMC_BF16), be.zeros(B * NH * S), be.zeros(M * ld, BMC_BF16)

        def fwd():
            be.call("attention_forward", BMC_BF16, Ptr(out), QD, Ptr(lse), Ptr(d), ld, Ptr(d, QD * 2), Ptr(d, (QD + KV) * 2), ld, None, B, S, NH, NKV, HD, 0.125)

        def bwd():
            be.call("attention_backward", BMC_BF16, Ptr(dg), ld, Ptr(dg, QD * 2), Ptr(dg, (QD + KV) * 2), ld, Ptr(dgo), QD, Ptr(out), Ptr(lse), Ptr(d), ld,
                    Ptr(d, QD * 2), Ptr(d, (QD + KV) * 2), ld, None, B, S, NH, NKV, HD, 0.125)
        res = {}
        for name, fn in (("fwd", fwd), ("bwd", bwd)):
            for _ in range(max(args.warmup, 3)):
                fn()
            assert lib.bmc_sync(be.ctx) == 0
            lib.bmc_timer_begin(be.ctx, 0)
            for _ in range(args.steps):
                fn()
            res[name] = lib.bmc_timer_end(be.ctx, 0) / args.steps
        flops_fwd = 2.0 * B * NH * S * S * HD  # causal-counted: half of the full 4*S^2*HD; backward is twice the forward
        tf = (3 * flops_fwd) / ((res["fwd"] + res["bwd"]) * 1e-3) / 1e12
        print(json.dumps({"metric": "attention_fwd_bwd_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
                          "warmup": max(args.warmup, 3), "ms_per_step": res["fwd"] + res["bwd"], "higher_is_better": True, "dtype": "bf16",
                          "data": "synthetic", "config": {"workload": f"causal GQA flash attention fwd+bwd, NH {NH} NKV {NKV} HD {HD}, batch {B}, seq {S}"},
                          "fwd_ms": res["fwd"], "bwd_ms": res["bwd"], "fwd_tflops": flops_fwd / (res["fwd"] * 1e-3) / 1e12,
                          "bwd_tflops": 2 * flops_fwd / (res["bwd"] * 1e-3) / 1e12,
                          "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                       "frac": tf / peaks["bf16_tflops"], "traffic": None, "peak_source": f"bf16_tflops (burst) of {src}"}}), flush=True)
    be.close()
    return 0


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) and algorithmic bytes of ONE launch of every GEMM of the 360M training
# step, in MB, from ncu --set full captures at 32768 rows (the LM head at 8192 rows). (dram, algorithmic, launches per layer);
# the head runs once per step. The forward projections with a residual read 63 MB more in the step than in their capture.
GEMM_NCU_DRAM_MB = {
    "qkv forward": (122.9, 170.9, 1), "qkv input_grad": (142.5, 170.9, 1), "qkv weight_grad": (205.8, 173.9, 1),
    "o forward": (89.8, 127.7, 1), "o input_grad_rowdot": (165.4, 190.5, 1), "o weight_grad": (138.0, 129.5, 1),
    "gate_up forward_swiglu": (524.4, 576.0, 1), "gate_up input_grad": (426.9, 408.2, 1), "gate_up weight_grad": (557.9, 418.1, 1),
    "down forward": (216.0, 235.6, 1), "down input_grad_swiglu": (809.7, 738.8, 1), "down weight_grad": (298.0, 240.5, 1),
}
GEMM_NCU_HEAD_MB_8192_ROWS = {"head forward": (2455.5, 915.4), "head input_grad": (1034.1, 915.4), "head weight_grad": (1344.6, 1009.8)}


def gemm_step_traffic(model, rows):
    """DRAM and algorithmic bytes per average GEMM launch of the step. The table holds the 360M shapes at 32768 rows; for any other
    model or row count there is no capture and the traffic is reported as null."""
    if model != "smollm2-360m" or rows != 32768:
        return {"dram_bytes_per_launch": None, "case": "no ncu capture for this model / row count"}
    L = 32
    dram = L * sum(d * n for d, _, n in GEMM_NCU_DRAM_MB.values()) + 4.0 * sum(d for d, _ in GEMM_NCU_HEAD_MB_8192_ROWS.values())
    alg = L * sum(a * n for _, a, n in GEMM_NCU_DRAM_MB.values()) + 4.0 * sum(a for _, a in GEMM_NCU_HEAD_MB_8192_ROWS.values())
    launches = L * sum(n for _, _, n in GEMM_NCU_DRAM_MB.values()) + len(GEMM_NCU_HEAD_MB_8192_ROWS)
    return {"dram_bytes_per_launch": dram / launches * 1e6,
            "case": f"mean over the {launches} GEMM launches of a step from per-shape ncu captures (head scaled x4 from 8192 rows); "
                    f"algorithmic {alg / launches:.1f}e6 B per launch"}


def run_gemm(args):
    """The linear-layer GEMMs of the 360M step (forward, input gradient, weight gradient) in isolation, bf16 operands drawn
    from N(0,1), 16 x 2048 token rows; one JSON line per shape and kind. --shape picks one (e.g. gate_up)."""
    from bmcapi import BMC_BF16, Backend, Ptr
    lib = bmapi.load_product()
    be = Backend(lib)
    lib.bmc_timer_begin.argtypes = [C.c_void_p, C.c_int]
    lib.bmc_timer_end.argtypes = [C.c_void_p, C.c_int]
    lib.bmc_timer_end.restype = C.c_float
    a = bmapi.make_arch(args.model)
    BT = args.batch * args.seq_len
    D, H, QD, KV, V = a.dim, a.hidden_dim, a.n_heads * a.head_dim, a.n_kv_heads * a.head_dim, a.vocab_size
    shapes = [("qkv", D, QD + 2 * KV), ("o", QD, D), ("gate_up", D, 2 * H), ("down", H, D), ("head", D, V)]
    peaks, src = measured_peaks()
    rng = np.random.default_rng(3)

    def rand_bf16(n):
        # a 16 Mi-element random block tiled over the buffer keeps host time small and the values non-trivial
        blk = rng.standard_normal(min(n, 1 << 24)).astype(np.float32)
        return be.put(np.resize(blk, n), BMC_BF16)
    for name, Cc, OC in shapes:
        if args.shape and args.shape != name:
            continue
        inp, w, gout = rand_bf16(BT * Cc), rand_bf16(OC * Cc), rand_bf16(BT * OC)
        out, ginp, gw = be.zeros(BT * OC, BMC_BF16), be.zeros(BT * Cc, BMC_BF16), be.zeros(OC * Cc)
        kinds = {
            "forward": lambda: be.call("matmul_forward", BMC_BF16, Ptr(out), OC, Ptr(inp), Cc, Ptr(w), None, 0, BT, Cc, OC),
            "input_grad": lambda: be.call("matmul_backward_inp", BMC_BF16, Ptr(ginp), Cc, 0, Ptr(gout), OC, Ptr(w), BT, Cc, OC),
            "weight_grad": lambda: be.call("matmul_backward_w", BMC_BF16, Ptr(gw), Ptr(gout), OC, Ptr(inp), Cc, BT, Cc, OC),
        }
        # the same GEMMs with the memory-bound kernel next to them folded into the epilogue (the forms the training step uses)
        if name == "gate_up":
            act = be.zeros(BT * H, BMC_BF16)
            kinds["forward_swiglu"] = lambda: be.call("matmul_swiglu_forward", BMC_BF16, Ptr(out), OC, Ptr(act), H, Ptr(inp), Cc, Ptr(w), BT, Cc, H)
        if name == "down":
            gu, dgu = rand_bf16(BT * 2 * H), be.zeros(BT * 2 * H, BMC_BF16)
            kinds["input_grad_swiglu"] = lambda: be.call("matmul_backward_inp_swiglu", BMC_BF16, Ptr(dgu), 2 * H, Ptr(gout), OC, Ptr(w), Ptr(gu), 2 * H, BT, H, OC)
        if name == "o":
            rd = be.zeros(BT * a.n_heads)
            kinds["input_grad_rowdot"] = lambda: be.call("matmul_backward_inp_rowdot", BMC_BF16, Ptr(ginp), Cc, Ptr(rd), Ptr(gout), OC, Ptr(w), Ptr(inp), Cc,
                                                         BT, Cc, OC, args.seq_len, a.n_heads)
        for kind, fn in kinds.items():
            if args.kind and args.kind != kind:
                continue
            for _ in range(max(args.warmup, 1)):
                assert fn() == 0
            assert lib.bmc_sync(be.ctx) == 0
            lib.bmc_timer_begin(be.ctx, 0)
            for _ in range(max(args.steps, 1)):
                fn()
            ms = lib.bmc_timer_end(be.ctx, 0) / max(args.steps, 1)
            tf = 2.0 * BT * Cc * OC / (ms * 1e-3) / 1e12
            print(json.dumps({"metric": "gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": max(args.steps, 1),
                              "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                              "config": {"workload": f"{name} {kind}: rows {BT}, in {Cc}, out {OC}"},
                              "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                           "frac": tf / peaks["bf16_tflops"], "traffic": None, "peak_source": f"bf16_tflops (burst) of {src}"}}),
                  flush=True)
        for pbuf in (inp, w, gout, out, ginp, gw):
            lib.bmc_free(be.ctx, pbuf)
            be.bufs.remove(pbuf)
    be.close()
    return 0


def run_decode(args):
    """Q8 inference: prefill 512 uniform-random tokens, then greedy-decode 256, at batch 1 and 64; one JSON line per batch.
    Layer matrices are int8 blocks of 32 with one fp32 scale, the LM head is bf16, activations and the KV cache fp32.
    The timed regions are whole calls of the session API (host prompt in, host token ids out)."""
    import time
    lib = bmapi.load_product()
    a = bmapi.make_arch(args.model)
    a.precision = bmapi.BM_PRECISION_BF16
    w = bmapi.make_weights(a)
    path = f"/tmp/bm_bench_decode_{os.getpid()}.bin"
    bmapi.write_bin_checkpoint(path, a, w)
    del w
    peaks, src = measured_peaks()
    n_prompt, n_new = args.prompt_tokens, args.decode_tokens
    MS = n_prompt + n_new
    ctx = lib.bm_create(bmapi.BM_DEVICE_METAL)
    model = lib.bm_create_model(ctx, C.byref(a))
    lib.bm_load_weights(model, path.encode())
    os.unlink(path)
    assert lib.bmx_model_set_quant(model, 8) == 0
    L, KV, V = a.n_layers, a.n_kv_heads * a.head_dim, a.vocab_size
    for NB in [int(v) for v in args.decode_batches.split(",")]:
        sess = lib.bmx_create_session_batched(ctx, model, NB, MS)
        assert sess, "bmx_create_session_batched failed"
        wbytes = lib.bmx_session_weight_bytes(sess)                   # what this session streams per step
        wbytes_alg = lib.bmx_session_algorithmic_weight_bytes(sess)   # Q8 blocks at 1.125 B/weight + the bf16 head
        prompts = np.random.default_rng(7).integers(0, V, size=(NB, n_prompt), dtype=np.int32)
        first = np.zeros((NB, 1), np.int32)
        out = np.zeros((NB, n_new), np.int32)
        best = None
        best_pre = None
        for it in range(max(args.warmup, 1) + max(args.steps, 1)):
            lib.bm_reset_session(sess)
            t0 = time.perf_counter()
            assert lib.bmx_session_generate_greedy(sess, bmapi.as_int_ptr(prompts), n_prompt, 1, bmapi.as_int_ptr(first)) == 0
            t1 = time.perf_counter()
            # continues from position 512: feeds the first generated token, returns tokens 2..257; 256 decode steps
            assert lib.bmx_session_generate_greedy(sess, bmapi.as_int_ptr(first), 1, n_new, bmapi.as_int_ptr(out)) == 0
            t2 = time.perf_counter()
            if it >= max(args.warmup, 1):
                best_pre = t1 - t0 if best_pre is None else min(best_pre, t1 - t0)
                if best is None or t2 - t1 < best[1]:
                    best = (t1 - t0, t2 - t1)
        lib.bm_destroy_session(sess)
        t_pre, t_dec = best_pre, best[1]
        # algorithmic bytes of one decode step: every weight once (in the model's own precision) + the KV cache rows up to the
        # current position (fp32 cache, as the reference keeps it); `streamed` counts the layout this session really reads instead
        kv_avg = L * 2 * (n_prompt + n_new / 2.0) * KV * 4 * NB
        step_bytes = wbytes_alg + kv_avg
        gbs = step_bytes * n_new / t_dec / 1e9
        gbs_streamed = (wbytes + kv_avg) * n_new / t_dec / 1e9
        ref_bytes = wbytes_alg + L * 2 * KV * 4 * NB   # the reference's own accounting: weights + the KV rows of ONE token (bench/bench.c:339-348)
        print(json.dumps({"metric": "decode_tokens_per_sec", "value": NB * n_new / t_dec, "unit": "tokens/s", "n_gpus": 1,
                          "steps": max(args.steps, 1), "warmup": max(args.warmup, 1), "ms_per_step": t_dec / n_new * 1e3,
                          "higher_is_better": True, "dtype": "q8 weights / f32 activations", "data": "synthetic",
                          "config": {"workload": f"{args.model} Q8 inference: prefill {n_prompt} + greedy decode {n_new}, batch {NB}",
                                     "l2": "weights (>400 MB) exceed L2"},
                          "prefill_tokens_per_sec": NB * n_prompt / t_pre, "prefill_ms": t_pre * 1e3, "decode_ms": t_dec * 1e3,
                          "weight_bytes": wbytes_alg, "weight_bytes_streamed": wbytes,
                          "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                                       "traffic": None, "peak_source": f"hbm_gbs of {src}",
                                       "bytes_per_step": step_bytes, "streamed_gbs": gbs_streamed,
                                       "reference_accounting_gbs": ref_bytes * n_new / t_dec / 1e9}}), flush=True)
    lib.bm_destroy_model(model)
    lib.bm_destroy(ctx)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--batch", type=int, default=PER_GPU_BATCH)
    ap.add_argument("--seq-len", type=int, default=SEQ_LEN)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="train", choices=["train", "attention", "decode", "gemm"],
                    help="train (default, the contract line); attention: isolated GQA flash attention fwd+bwd; decode: Q8 prefill + greedy decode; gemm: the linear-layer GEMMs in isolation")
    ap.add_argument("--prompt-tokens", type=int, default=512, help="--workload decode: prompt length")
    ap.add_argument("--decode-tokens", type=int, default=256, help="--workload decode: generated tokens")
    ap.add_argument("--decode-batches", default="1,64", help="--workload decode: comma-separated sequence counts")
    ap.add_argument("--shape", default="", help="--workload gemm: qkv, o, gate_up, down or head (default all)")
    ap.add_argument("--kind", default="", help="--workload gemm: forward, input_grad, weight_grad or one of the fused forms (default all)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.workload == "attention":
        return run_attention(args)
    if args.workload == "decode":
        return run_decode(args)
    if args.workload == "gemm":
        return run_gemm(args)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        print(f"bench.py: WORLD_SIZE={world} but --gpus {args.gpus}", file=sys.stderr)
    B, S = args.batch, args.seq_len
    W = max(args.warmup, 3) if args.warmup >= 0 else 3
    K = max(args.steps, 1)

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local_rank))

    lib = bmapi.load_product()
    a = bmapi.make_arch(args.model)
    a.precision = bmapi.BM_PRECISION_BF16
    ctx = lib.bm_create(bmapi.BM_DEVICE_CUDA)
    if not ctx:
        raise SystemExit("bench.py: no CUDA context (the product has no CPU fallback)")
    model = lib.bm_create_model(ctx, C.byref(a))
    fill_weights(lib, model, a)
    cfg = bmapi.train_config(lr=3e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, seq_len=S)
    tr = lib.bm_create_trainer(ctx, model, C.byref(cfg))
    if not tr:
        raise SystemExit("bench.py: bm_create_trainer failed")

    if world > 1:
        import torch
        idbuf = (C.c_ubyte * 128)()
        if rank == 0 and lib.bmx_dp_unique_id(idbuf) != 0:
            raise SystemExit("bench.py: bmx_dp_unique_id failed")
        t_id = torch.tensor(list(bytes(idbuf)), dtype=torch.uint8, device="cuda")
        dist.broadcast(t_id, src=0)
        idbuf = (C.c_ubyte * 128)(*t_id.cpu().tolist())
        if lib.bmx_trainer_dp_init(tr, rank, world, idbuf) != 0:
            raise SystemExit("bench.py: bmx_trainer_dp_init failed")

    # rank r takes sequences r*B .. r*B+B-1 of every global batch
    n_steps_total = 2 * (W + K)
    x, y = bmapi.lcg_batch(B * world * n_steps_total, S, a.vocab_size)
    x = x.reshape(n_steps_total, world, B, S)[:, rank].copy()
    y = y.reshape(n_steps_total, world, B, S)[:, rank].copy()
    nbytes = B * S * 4
    d_x = [lib.bmx_device_alloc(ctx, nbytes) for _ in range(W + K)]
    d_y = [lib.bmx_device_alloc(ctx, nbytes) for _ in range(W + K)]
    for i in range(W + K):
        lib.bmx_device_upload(ctx, d_x[i], x[i].ctypes.data, nbytes)
        lib.bmx_device_upload(ctx, d_y[i], y[i].ctypes.data, nbytes)
    lib.bmx_device_sync(ctx)

    def barrier():
        lib.bmx_device_sync(ctx)
        if dist is not None:
            dist.barrier()
        lib.bmx_device_sync(ctx)

    def max_over_ranks(v):
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------- leg 1: inputs resident in HBM -----------------------------------------------------------
    for i in range(W):
        if lib.bmx_train_step_resident(tr, d_x[i], d_y[i], B, S) != 0:
            raise SystemExit("bench.py: warm-up step failed")
    loss_w = lib.bmx_train_last_loss(tr)
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    barrier()
    launches0 = lib.bmx_trainer_launch_count(tr)
    t_wall0 = time.time()
    lib.bmx_timer_begin(ctx, 7)
    for i in range(K):
        if lib.bmx_train_step_resident(tr, d_x[W + i], d_y[W + i], B, S) != 0:
            raise SystemExit("bench.py: timed step failed")
    ms_total = lib.bmx_timer_end(ctx, 7)
    barrier()
    t_wall1 = time.time()
    launches1 = lib.bmx_trainer_launch_count(tr)
    loss_t = lib.bmx_train_last_loss(tr)
    clocks = sampler.stop(t_wall0, t_wall1)
    # Roofline pass: per-launch CUDA events around every tensor-core GEMM, two more steps of the same workload. In the timed
    # region above the weight-gradient GEMMs run on a side stream and overlap memory-bound kernels, so an event pair around one
    # launch there also measures the kernels it shares the SMs with; for this pass they are serialised on the main stream.
    lib.bmx_trainer_set_option(tr, b"side_stream", 0)
    lib.bmx_train_step_resident(tr, d_x[W], d_y[W], B, S)
    barrier()
    lib.bmx_gemm_timing(ctx, 1)
    lib.bmx_timer_begin(ctx, 5)
    for i in range(2):
        lib.bmx_train_step_resident(tr, d_x[W + i % K], d_y[W + i % K], B, S)
    ms_roof = lib.bmx_timer_end(ctx, 5)
    gt = (C.c_double * 3)()
    lib.bmx_gemm_timing_collect(ctx, gt)
    lib.bmx_gemm_timing(ctx, 0)
    lib.bmx_trainer_set_option(tr, b"side_stream", 0 if os.environ.get("BM_NO_SIDE_STREAM") else 1)
    ms_total = max_over_ranks(ms_total)
    ms_per_step = ms_total / K
    tokens_per_step = B * S * world
    value = tokens_per_step / (ms_per_step * 1e-3)

    # ---------------- leg 2: end to end through bm_train_step with host buffers ----------------------------------
    for i in range(3):  # the third plain step captures the CUDA graph: keep that out of the timed region
        lib.bm_train_step(tr, bmapi.as_int_ptr(x[W + K + i]), bmapi.as_int_ptr(y[W + K + i]), B, S)
    barrier()
    lib.bmx_timer_begin(ctx, 6)
    t0 = time.perf_counter()
    loss_e = 0.0
    for i in range(K):
        j = W + K + 3 + i
        loss_e = lib.bm_train_step(tr, bmapi.as_int_ptr(x[j]), bmapi.as_int_ptr(y[j]), B, S)
    ms_e2e_dev = lib.bmx_timer_end(ctx, 6)
    barrier()
    ms_e2e_wall = (time.perf_counter() - t0) * 1e3
    ms_e2e = max_over_ranks(max(ms_e2e_dev, ms_e2e_wall)) / K
    e2e_value = tokens_per_step / (ms_e2e * 1e-3)

    if rank == 0:
        peaks, peak_src = measured_peaks()
        gemm_traffic = gemm_step_traffic(args.model, B * S)
        fpt = flops_per_token(a, S)
        tflops = value * fpt / 1e12
        n_l, g_ms, g_fl = gt[0], gt[1], gt[2]
        ach = (g_fl / (g_ms * 1e-3) / 1e12) if g_ms > 0 else None
        peak_tf = peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops"))
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.model} training step (fwd+bwd+AdamW), bf16 mixed precision, {B} seq x {S} tokens per GPU",
                       "global_batch": B * world, "seq_len": S, "parallelism": f"dp{world}",
                       "optimizer": "AdamW lr 3e-4 beta (0.9, 0.95) eps 1e-8 wd 0.1, fp32 master + moments",
                       "l2": "no explicit flush: each step streams tens of GB of activations and weights, far beyond the 126 MB L2"},
            "tflops_per_gpu": tflops / world, "flops_per_token": fpt,
            "mfu_vs_datasheet_2250": tflops / world / DATASHEET_BF16_TFLOPS,
            "mfu_vs_measured_sustained": tflops / world / peak_tf,
            "loss": {"after_warmup": loss_w, "after_timed": loss_t, "after_e2e": loss_e},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e, "h2d_bytes_per_step": 2 * nbytes * world,
                    "d2h_bytes_per_step": 4 * world},
            "gpu_launches": int(launches1 - launches0),
            "roofline": {"kernel": "gemm_bf16_umma_kernel (tcgen05)", "bound": "tensor", "achieved": ach, "peak": peak_tf,
                         "unit": "TFLOP/s", "frac": (ach / peak_tf) if ach else None,
                         # DRAM bytes of the step's average GEMM launch, from the ncu captures of every shape and kind
                         # (GEMM_NCU_DRAM_MB below; profiles/gemm_umma_step_shapes_ncu_full.md)
                         "traffic": gemm_traffic["dram_bytes_per_launch"], "traffic_case": gemm_traffic["case"],
                         "peak_source": f"bf16_tflops_sustained of {peak_src}", "launches": int(n_l),
                         "avg_launch_ms": (g_ms / n_l) if n_l else None, "avg_launch_flops": (g_fl / n_l) if n_l else None,
                         "share_of_step": (g_ms / ms_roof) if ms_roof else None,
                         "measured_in": "2 extra steps with the weight-gradient GEMMs serialised on the main stream "
                                        f"({ms_roof / 2:.1f} ms/step); in the timed region they overlap memory-bound kernels"},
        }
        if world == 1 and not args.no_cpu_baseline:
            try:
                tps, cores, sample, _ = reference_tokens_per_sec(1, 1)
                line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": cores, "kind": "reference", "sample": sample}
            except Exception as e:  # the checker is absent: report it, never substitute
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference", "sample": f"unavailable: {e}"}
        print(json.dumps(line), flush=True)

    lib.bm_destroy_trainer(tr)
    lib.bm_destroy_model(model)
    lib.bm_destroy(ctx)
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
