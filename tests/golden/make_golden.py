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


def main():
    ref_dir = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BM_REFERENCE", "/root/reference")
    torch_goldens(ref_dir)
    ref = bmapi.load_reference()
    if ref is None:
        raise SystemExit("oracle/_ref/libbm_ref.so missing: run oracle/build_ref.sh first")
    F32, BF16 = bmapi.BM_PRECISION_FP32, bmapi.BM_PRECISION_BF16
    ref_train_case(ref, "tiny_f32_b1", "tiny", 1, 16, F32, 3)
    ref_train_case(ref, "tiny_f32_b3", "tiny", 3, 32, F32, 2)
    ref_train_case(ref, "tiny_bf16_b2", "tiny", 2, 32, BF16, 3)
    ref_train_case(ref, "gqa_f32_b2", "gqa", 2, 128, F32, 2)
    ref_train_case(ref, "gqa_bf16_b2", "gqa", 2, 128, BF16, 2)
    ref_train_case(ref, "small_f32_accum2", "small", 2, 64, F32, 2, accum=2)
    if "--skip-135m" not in sys.argv:
        ref_train_case(ref, "135m_f32_c1", "smollm2-135m", 1, 64, F32, 1)


if __name__ == "__main__":
    main()
