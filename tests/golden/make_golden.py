#!/usr/bin/env python3
"""Generates the committed golden fixtures. Needs a checkout of the reference (read-only) and, for part 2, the
reference-on-CPU build oracle/_ref/libbm_ref.so (oracle/build_ref.sh). Run from the repository root:

    python tests/golden/make_golden.py [/path/to/reference]

Part 1 — torch_kernel_goldens.npz: the reference's OWN PyTorch golden generators (test/grad/gen_*.py, the ones that
need no model download) are executed unmodified in a scratch directory; every tensor they dump (inputs and
autograd outputs) is stored under its file stem. These are the vectors the reference's kernel tests check against
(test/matmul_bwd_test.c, rmsnorm_bwd_test.c, rope_*_test.c, act_bwd_test.c, xent_bwd_test.c, embed_bwd_test.c,
adamw_test.c, attn_*_test.c, sched_bwd_test.c, layer_bwd_test.c).

Part 2 — ref_train_step_*.npz: the reference's training step (its C11 host code + its kernel sources on CPU) is run on
seeded random-init models and LCG tokens; losses, per-tensor gradient norms, sampled gradient / post-step weight
values are stored. Cases: scaled-down family members in fp32 and bf16-weight mode, batches of more than one sequence,
and the 135M-parameter single-step fp32 configuration (B=1, S=64, AdamW lr 3e-4, beta (0.9, 0.95), wd 0.1).

Part 2b (`--only TAG[,TAG...]` regenerates single files of parts 2, 2b and 3 by their tag) — the configurations that are
benchmarked: ref_train_step_360m_{f32,bf16}_b2.npz (SmolLM2-360M, two sequences of 128 tokens, two optimizer steps) and
ref_train_curve_135m_{f32,bf16}.npz (SmolLM2-135M, 50 optimizer steps on two sequences of 128 tokens each: the loss curve
and sampled final weights), ref_decode_360m_{f32,bf16}_q8.npz (SmolLM2-360M with Q8 layers: a 64-token prompt and 16 greedy tokens,
sampled logits only), oracle_attention_s8192_group.npz (the isolated-attention configuration at 8192 tokens, one KV group, from the
plain-C oracle).

Part 3 (`--only-decode` regenerates just this part) — ref_quantize_q8.npz / ref_quantize_q4.npz: the reference's Q8 and Q4 block
quantisers on seeded inputs with their edge cases (Q4 codes stored unpacked, one per byte); ref_decode_*.npz: logits of the
reference inference session after every prefix of a seeded prompt and a greedy continuation, fp32 / bf16 weights, plain, Q8 and Q4.
"""
import ctypes as C
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "bare.metal_b200"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import bmapi  # noqa: E402
import oracle_check as oc  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
GEN_SCRIPTS = ["gen_matmul_bwd", "gen_rmsnorm_bwd", "gen_rope_bwd", "gen_rope_seq", "gen_rope_real", "gen_act_bwd", "gen_xent_bwd",
               "gen_embed_bwd", "gen_adamw", "gen_attn_bwd", "gen_attn_real", "gen_sched_bwd", "gen_layer_bwd"]
INT_FILES = {"xent_targets", "embed_tokens"}
SAMPLE = 64  # sampled values per tensor
DECODE_LAYER_SCALE = 8.0


def torch_goldens(ref_dir):
    data = {}
    with tempfile.TemporaryDirectory() as td:
        os.makedirs(os.path.join(td, "test", "grad"))
        for s in GEN_SCRIPTS:
            subprocess.run([sys.executable, os.path.join(ref_dir, "test", "grad", s + ".py")], cwd=td, check=True,
                           stdout=subprocess.DEVNULL)
        for fn in sorted(os.listdir(os.path.join(td, "test", "grad"))):
            stem = fn[:-4]
            raw = np.fromfile(os.path.join(td, "test", "grad", fn), dtype=np.int32 if stem in INT_FILES else np.float32)
            data[stem] = raw
        # gen_adamw_wd0 writes the same file names with weight_decay 0: keep it under a prefix
        for fn in list(os.listdir(os.path.join(td, "test", "grad"))):
            if fn.startswith("adamw_"):
                os.unlink(os.path.join(td, "test", "grad", fn))
        subprocess.run([sys.executable, os.path.join(ref_dir, "test", "grad", "gen_adamw_wd0.py")], cwd=td, check=True,
                       stdout=subprocess.DEVNULL)
        for fn in sorted(os.listdir(os.path.join(td, "test", "grad"))):
            if fn.startswith("adamw_"):
                data["wd0_" + fn[:-4]] = np.fromfile(os.path.join(td, "test", "grad", fn), dtype=np.float32)
    np.savez_compressed(os.path.join(OUT, "torch_kernel_goldens.npz"), **data)
    print(f"torch_kernel_goldens.npz: {len(data)} tensors")


def sample_idx(n, seed):
    rng = np.random.default_rng(seed)
    return np.sort(rng.choice(n, size=min(SAMPLE, n), replace=False)).astype(np.int64)


def ref_train_case(ref, tag, arch_name, B, S, precision, steps, accum=1):
    a = bmapi.make_arch(arch_name)
    w = bmapi.make_weights(a)
    cfg = bmapi.train_config(seq_len=S, accum=accum)
    x, y = bmapi.lcg_batch(B * steps * accum, S, a.vocab_size)
    tr = oc.LibTrainer(ref, "reference", a, w, S, precision, cfg, tag=tag)
    n = tr.n_tensors()
    out = {"arch": np.array(arch_name), "B": B, "S": S, "precision": precision, "steps": steps, "accum": accum, "n_tensors": n}
    losses = []
    for st in range(steps * accum):
        xs = np.ascontiguousarray(x[st * B:(st + 1) * B])
        ys = np.ascontiguousarray(y[st * B:(st + 1) * B])
        losses.append(tr.step(xs, ys))
        if st == accum - 1:
            gn, gs, gi = [], [], []
            for i in range(n):
                g = tr.read(bmapi.BMX_GRAD, i)
                idx = sample_idx(g.size, 1000 + i)
                gn.append(np.linalg.norm(g.astype(np.float64)))
                gi.append(np.pad(idx, (0, SAMPLE - idx.size), constant_values=-1))
                gs.append(np.pad(g[idx], (0, SAMPLE - idx.size)))
            out["grad_norm"], out["grad_idx"], out["grad_val"] = np.array(gn), np.array(gi), np.array(gs, np.float32)
    wn, ws = [], []
    for i in range(n):
        t = tr.read(bmapi.BMX_WEIGHT, i)
        idx = out["grad_idx"][i]
        idx = idx[idx >= 0]
        wn.append(np.linalg.norm(t.astype(np.float64)))
        ws.append(np.pad(t[idx], (0, SAMPLE - idx.size)))
    out["weight_norm"], out["weight_val"] = np.array(wn), np.array(ws, np.float32)
    out["losses"] = np.array(losses, np.float32)
    tr.close()
    np.savez_compressed(os.path.join(OUT, f"ref_train_step_{tag}.npz"), **out)
    print(f"ref_train_step_{tag}.npz: losses {losses}")


def ref_curve_case(ref, tag, arch_name, B, S, precision, steps):
    """Loss after every optimizer step of a `steps`-step run of the reference, plus norms and sampled values of the final weights
    (the reference's own analogue runs 10 AdamW steps on real weights, test/g3_test.c:27)."""
    a = bmapi.make_arch(arch_name)
    w = bmapi.make_weights(a)
    cfg = bmapi.train_config(seq_len=S)
    x, y = bmapi.lcg_batch(B * steps, S, a.vocab_size)
    tr = oc.LibTrainer(ref, "reference", a, w, S, precision, cfg, tag=tag)
    n = tr.n_tensors()
    losses = []
    for st in range(steps):
        losses.append(tr.step(np.ascontiguousarray(x[st * B:(st + 1) * B]), np.ascontiguousarray(y[st * B:(st + 1) * B])))
        print(f"  {tag} step {st + 1}/{steps} loss {losses[-1]:.6f}", flush=True)
    wn, wi, ws = [], [], []
    for i in range(n):
        t = tr.read(bmapi.BMX_WEIGHT, i)
        idx = sample_idx(t.size, 1000 + i)
        wn.append(np.linalg.norm(t.astype(np.float64)))
        wi.append(np.pad(idx, (0, SAMPLE - idx.size), constant_values=-1))
        ws.append(np.pad(t[idx], (0, SAMPLE - idx.size)))
    tr.close()
    np.savez_compressed(os.path.join(OUT, f"ref_train_curve_{tag}.npz"), arch=np.array(arch_name), B=B, S=S, precision=precision,
                        steps=steps, n_tensors=n, losses=np.array(losses, np.float32), weight_norm=np.array(wn),
                        weight_idx=np.array(wi), weight_val=np.array(ws, np.float32))
    print(f"ref_train_curve_{tag}.npz: first {losses[0]:.5f} last {losses[-1]:.5f}")


def ref_decode_sampled_case(ref, tag, arch_name, precision, quant, n_prompt, n_new, n_sample=256, top=8):
    """Large-vocabulary variant of ref_decode_case: the logits of the full prompt and of every greedy step are stored only at
    `n_sample` seeded vocabulary indices and at the reference's `top` largest entries."""
    a = bmapi.make_arch(arch_name)
    w = bmapi.make_weights(a, layer_scale=DECODE_LAYER_SCALE)
    prompt = bmapi.lcg_tokens(n_prompt, a.vocab_size, seed=1234)
    s = oc.LibSession(ref, "reference", a, w, precision, quant, tag=tag)
    idx = np.sort(np.random.default_rng(99).choice(a.vocab_size, size=n_sample, replace=False)).astype(np.int64)
    seq = list(int(t) for t in prompt)
    greedy, margin, vals, top_ids, top_vals, amax = [], [], [], [], [], []
    for k in range(n_new):
        s.reset()
        lg = s.forward(np.array(seq, np.int32))
        order = np.argsort(lg)[::-1][:top]
        greedy.append(int(np.argmax(lg)))
        margin.append(float(lg[order[0]] - lg[order[1]]))
        vals.append(lg[idx])
        top_ids.append(order)
        top_vals.append(lg[order])
        amax.append(float(np.abs(lg).max()))
        seq.append(greedy[-1])
        print(f"  {tag} token {k + 1}/{n_new}: {greedy[-1]} margin {margin[-1]:.4g}", flush=True)
    s.close()
    np.savez_compressed(os.path.join(OUT, f"ref_decode_{tag}.npz"), arch=np.array(arch_name), precision=precision, quant=quant,
                        layer_scale=DECODE_LAYER_SCALE, prompt=np.asarray(prompt, np.int32), sample_idx=idx,
                        sample_logits=np.array(vals, np.float32), top_ids=np.array(top_ids, np.int32),
                        top_logits=np.array(top_vals, np.float32), logit_absmax=np.array(amax, np.float32),
                        greedy=np.array(greedy, np.int32), margin=np.array(margin, np.float32))
    print(f"ref_decode_{tag}.npz: greedy {greedy} min margin {min(margin):.3g}")


def c4_group_inputs(S, seed=8192):
    """Q (3 query heads), K, V (their one KV head) and dO for one KV group of the isolated-attention configuration, N(0,1) by seed,
    rounded to bf16. Shared by the generator below and by tests/test_gpu_attention_c4.py."""
    from bmcapi import bf16_round
    rng = np.random.default_rng(seed)
    q = bf16_round(rng.standard_normal((S, 3, 64)).astype(np.float32))
    k = bf16_round(rng.standard_normal((S, 1, 64)).astype(np.float32))
    v = bf16_round(rng.standard_normal((S, 1, 64)).astype(np.float32))
    go = bf16_round(rng.standard_normal((S, 3, 64)).astype(np.float32))
    return q, k, v, go


def c4_group_case(S=8192, every=32):
    """Isolated causal attention at S = 8192 for ONE KV group (one KV head and the three query heads that share it): O, dQ, dK, dV
    from the plain-C restatement of attention_forward_seq / attention_backward (src/kernels/forward.metal:1811,
    src/kernels/backward.metal:665, oracle/bm_oracle.c, pinned to the reference's own attention goldens by tests/test_oracle_pins.py).
    About 80 GFLOP of scalar work; every 32nd row and the tensor norms are stored."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import portk
    q, k, v, go = c4_group_inputs(S)
    o = portk.attention_forward(q, k, v, 0.125)
    gq, gk, gv = portk.attention_backward(go, q, k, v, 0.125)
    rows = np.arange(0, S, every)
    np.savez_compressed(os.path.join(OUT, f"oracle_attention_s{S}_group.npz"), S=S, rows=rows, checksum=float(np.float64(q.sum()) + k.sum() + v.sum() + go.sum()),
                        o=o[rows], gq=gq[rows], gk=gk[rows], gv=gv[rows],
                        norms=np.array([np.linalg.norm(t.astype(np.float64)) for t in (o, gq, gk, gv)]))
    print(f"oracle_attention_s{S}_group.npz: {rows.size} rows")


def q8_inputs():
    """Seeded quantiser inputs with the edge cases of the scheme: an all-zero block, a block whose extreme is negative,
    exact .5 ties after scaling, a huge dynamic range, denormal-sized values."""
    rng = np.random.default_rng(77)
    x = rng.standard_normal(64 * 32).astype(np.float32) * 0.02
    x[0:32] = 0.0
    x[32:64] = np.linspace(-1.0, 0.5, 32, dtype=np.float32)
    x[64:96] = (np.arange(32, dtype=np.float32) - 16.0) * 0.5 / 127.0 * 127.0   # scale 8/127 -> many x.5 quotients
    x[96:128] = np.float32(1e-30) * rng.standard_normal(32).astype(np.float32)
    x[128:160] = np.concatenate([[np.float32(1e4)], rng.standard_normal(31).astype(np.float32)])
    return x


def ref_q8_case(ref):
    x = q8_inputs()
    nb = x.size // 32
    blocks = np.zeros(nb, dtype=np.dtype([("scale", "<f4"), ("q", "i1", (32,))]))   # q8_block_t, src/baremetal/quant.h:19-22
    assert ref.bmt_quantize_q8(oc.fptr(x), blocks.ctypes.data, x.size) == nb
    np.savez_compressed(os.path.join(OUT, "ref_quantize_q8.npz"), x=x, scale=blocks["scale"].copy(), q=blocks["q"].copy())
    print(f"ref_quantize_q8.npz: {nb} blocks")


def ref_q4_case(ref):
    """Same inputs through bmt_quantize_q4; q4_block_t is {f32 scale; u8 qs[16]} with code 2j in the low and code 2j+1 in the high
    nibble of byte j (src/baremetal/quant.h:39-42, quant.c:44-50). Stored: the sign-extended codes, one per byte."""
    x = q8_inputs()
    x[64:96] = (np.arange(32, dtype=np.float32) - 16.0) * 0.5   # amax 8 -> scale 8/7: quotients on and next to .5
    nb = x.size // 32
    blocks = np.zeros(nb, dtype=np.dtype([("scale", "<f4"), ("qs", "u1", (16,))]))
    assert blocks.itemsize == 20
    assert ref.bmt_quantize_q4(oc.fptr(x), blocks.ctypes.data, x.size) == nb
    lo = (blocks["qs"] & 0x0F).astype(np.int8)
    hi = (blocks["qs"] >> 4).astype(np.int8)
    q = np.stack([lo, hi], axis=-1).reshape(nb, 32)
    q = np.where(q > 7, q - 16, q).astype(np.int8)
    np.savez_compressed(os.path.join(OUT, "ref_quantize_q4.npz"), x=x, scale=blocks["scale"].copy(), q=q)
    print(f"ref_quantize_q4.npz: {nb} blocks, codes {q.min()}..{q.max()}")


def ref_decode_case(ref, tag, arch_name, precision, quant, n_prompt, n_new):
    """Logits of the reference session after every prefix (2..n_prompt tokens) of a seeded prompt, then a greedy
    continuation, each token from a fresh prefill of the whole prefix (the barrier-free path of the CPU build)."""
    a = bmapi.make_arch(arch_name)
    w = bmapi.make_weights(a, layer_scale=DECODE_LAYER_SCALE)
    prompt = bmapi.lcg_tokens(n_prompt, a.vocab_size, seed=1234)
    s = oc.LibSession(ref, "reference", a, w, precision, quant, tag=tag)
    logits = []
    for n in range(2, n_prompt + 1):
        s.reset()
        logits.append(s.forward(prompt[:n]))
    seq = list(int(t) for t in prompt)
    greedy, margin = [], []
    for _ in range(n_new):
        s.reset()
        lg = s.forward(np.array(seq, np.int32))
        top = np.argsort(lg)[-2:]
        greedy.append(int(top[1]))
        margin.append(float(lg[top[1]] - lg[top[0]]))
        seq.append(int(top[1]))
    s.close()
    np.savez_compressed(os.path.join(OUT, f"ref_decode_{tag}.npz"), arch=np.array(arch_name), precision=precision, quant=quant, layer_scale=DECODE_LAYER_SCALE,
                        prompt=np.asarray(prompt, np.int32), logits=np.array(logits, np.float32), greedy=np.array(greedy, np.int32),
                        margin=np.array(margin, np.float32))
    print(f"ref_decode_{tag}.npz: greedy {greedy[:8]} min margin {min(margin):.3g}")


def main():
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    ref_dir = args[0] if args else (os.environ.get("BM_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference"))
    ref = oc.load_reference()
    if ref is None:
        raise SystemExit("oracle/_ref/libbm_ref.so missing: run oracle/build_ref.sh first")
    F32, BF16 = bmapi.BM_PRECISION_FP32, bmapi.BM_PRECISION_BF16
    decode_cases = (("gqa_f32", "gqa", F32, 0), ("gqa_f32_q8", "gqa", F32, 8), ("gqa_bf16", "gqa", BF16, 0),
                    ("gqa_bf16_q8", "gqa", BF16, 8), ("tiny_f32_q8", "tiny", F32, 8), ("gqa_f32_q4", "gqa", F32, 4),
                    ("gqa_bf16_q4", "gqa", BF16, 4))
    big = {
        "360m_bf16_b2": lambda: ref_train_case(ref, "360m_bf16_b2", "smollm2-360m", 2, 128, BF16, 2),
        "360m_f32_b2": lambda: ref_train_case(ref, "360m_f32_b2", "smollm2-360m", 2, 128, F32, 2),
        "135m_bf16_b2": lambda: ref_train_case(ref, "135m_bf16_b2", "smollm2-135m", 2, 128, BF16, 2),
        "curve_135m_bf16": lambda: ref_curve_case(ref, "135m_bf16", "smollm2-135m", 2, 128, BF16, 50),
        "curve_135m_f32": lambda: ref_curve_case(ref, "135m_f32", "smollm2-135m", 2, 128, F32, 50),
        "decode_360m_f32_q8": lambda: ref_decode_sampled_case(ref, "360m_f32_q8", "smollm2-360m", F32, 8, 64, 16),
        "decode_360m_bf16_q8": lambda: ref_decode_sampled_case(ref, "360m_bf16_q8", "smollm2-360m", BF16, 8, 64, 16),
        "c4_s8192_group": lambda: c4_group_case(8192),
    }
    small = {"quantize_q4": lambda: ref_q4_case(ref)}
    for tag, arch, prec, quant in decode_cases:
        small["decode_" + tag] = (lambda t=tag, a=arch, p=prec, q=quant: ref_decode_case(ref, t, a, p, q, 12, 12))
    for arg in sys.argv[1:]:
        if arg.startswith("--only="):
            for tag in arg[len("--only="):].split(","):
                (big | small)[tag]()
            return
    if "--only-decode" in sys.argv:
        ref_q8_case(ref)
        ref_q4_case(ref)
        for tag, arch, prec, quant in decode_cases:
            ref_decode_case(ref, tag, arch, prec, quant, 12, 12)
        return
    torch_goldens(ref_dir)
    ref_train_case(ref, "tiny_f32_b1", "tiny", 1, 16, F32, 3)
    ref_train_case(ref, "tiny_f32_b3", "tiny", 3, 32, F32, 2)
    ref_train_case(ref, "tiny_bf16_b2", "tiny", 2, 32, BF16, 3)
    ref_train_case(ref, "gqa_f32_b2", "gqa", 2, 128, F32, 2)
    ref_train_case(ref, "gqa_bf16_b2", "gqa", 2, 128, BF16, 2)
    ref_train_case(ref, "small_f32_accum2", "small", 2, 64, F32, 2, accum=2)
    ref_q8_case(ref)
    ref_q4_case(ref)
    for tag, arch, prec, quant in decode_cases:
        ref_decode_case(ref, tag, arch, prec, quant, 12, 12)
    if "--skip-135m" not in sys.argv:
        ref_train_case(ref, "135m_f32_c1", "smollm2-135m", 1, 64, F32, 1)
    if "--with-benchmarked-configs" in sys.argv:   # hours of CPU time: the 360M steps, the 135M 50-step curves, the 360M Q8 session
        for fn in big.values():
            fn()


if __name__ == "__main__":
    main()
