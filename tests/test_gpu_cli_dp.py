"""The baremetal-train CLI end to end, and data-parallel training on two GPUs (skipped on a single-GPU box)."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

import bmapi
import oracle_check as oc

pytestmark = pytest.mark.gpu
CLI = os.path.join(bmapi.PKG_DIR, "baremetal-train")


def test_cli_train_prints_the_reference_format_and_resumes(tmp_path):
    a = bmapi.make_arch("tiny")
    model = str(tmp_path / "tiny.bin")
    bmapi.write_bin_checkpoint(model, a, bmapi.make_weights(a))
    toks = str(tmp_path / "data.bin")
    bmapi.lcg_tokens(5000, a.vocab_size).tofile(toks)
    cmd = [CLI, "train", model, toks, str(tmp_path), "--steps", "4", "--seq-len", "32", "--batch-size", "2", "--lr", "1e-3",
           "--save-every", "2", "--precision", "bf16"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.splitlines() if l.startswith("step ")]
    assert len(lines) == 4
    pat = re.compile(r"^step (\d+)/4: loss=(\d+\.\d{4})  step_ms=\d+  gpu_mem=\d+\.\dMB  rss=\d+MB$")  # tools/cli.c:777-778
    losses = [float(pat.match(l).group(2)) for l in lines]
    assert "Avg step time:" in out.stdout
    assert os.path.exists(tmp_path / "checkpoint_2.bin") and os.path.exists(tmp_path / "checkpoint_4.bin")
    step, tensors = bmapi.read_state_file(str(tmp_path / "checkpoint_2.bin"))
    assert step == 2 and len(tensors) == 9 * a.n_layers + 2
    # the same run through the library gives the same losses
    lib = bmapi.load_product()
    stream = bmapi.lcg_tokens(5000, a.vocab_size)
    tr = oc.LibTrainer(lib, "gpu", a, bmapi.make_weights(a), 32, bmapi.BM_PRECISION_BF16, bmapi.train_config(lr=1e-3, wd=0.0, seq_len=32), quirks=False)
    for st in range(4):
        x = stream[st * 64:(st + 1) * 64].reshape(2, 32).copy()
        y = stream[st * 64 + 1:(st + 1) * 64 + 1].reshape(2, 32).copy()
        assert abs(tr.step(x, y) - losses[st]) < 1e-4
    tr.close()
    # --resume continues from the saved optimizer step
    out2 = subprocess.run(cmd[:5] + ["--steps", "1", "--seq-len", "32", "--batch-size", "2", "--resume", str(tmp_path / "checkpoint_4.bin")],
                          capture_output=True, text=True, timeout=300)
    assert out2.returncode == 0 and "resumed from" in out2.stderr


def test_cli_lcg_stream_and_errors(tmp_path):
    a = bmapi.make_arch("tiny")
    model = str(tmp_path / "tiny.bin")
    bmapi.write_bin_checkpoint(model, a, bmapi.make_weights(a))
    out = subprocess.run([CLI, "train", model, "lcg:42", str(tmp_path), "--steps", "2", "--seq-len", "16", "--precision", "fp32"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and sum(l.startswith("step ") for l in out.stdout.splitlines()) == 2
    bad = subprocess.run([CLI, "train", model, "corpus.txt", str(tmp_path)], capture_output=True, text=True)
    assert bad.returncode != 0 and "tokenizer" in bad.stderr
    assert subprocess.run([CLI], capture_output=True).returncode != 0


def _dp_worker(rank, world, id_path, out_dir, B_per, S, precision, accum=1, micro_steps=2):
    os.environ["BM_CUDA_DEVICE"] = str(rank)
    lib = bmapi.load_product()
    a = bmapi.make_arch("gqa")
    w = bmapi.make_weights(a)
    cfg = bmapi.train_config(seq_len=S, accum=accum)
    tr = oc.LibTrainer(lib, "gpu", a, w, S, precision, cfg, quirks=False, tag=f"dp{rank}")
    idbuf = (C.c_ubyte * 128)()
    if rank == 0:
        assert lib.bmx_dp_unique_id(idbuf) == 0
        with open(id_path + ".tmp", "wb") as f:
            f.write(bytes(idbuf))
        os.rename(id_path + ".tmp", id_path)
    else:
        import time
        for _ in range(600):
            if os.path.exists(id_path):
                break
            time.sleep(0.1)
        idbuf = (C.c_ubyte * 128)(*open(id_path, "rb").read())
    assert lib.bmx_trainer_dp_init(tr.tr, rank, world, idbuf) == 0
    x, y = bmapi.lcg_batch(B_per * world * micro_steps, S, a.vocab_size)
    losses = []
    for st in range(micro_steps):
        g = x[st * B_per * world:(st + 1) * B_per * world]
        t = y[st * B_per * world:(st + 1) * B_per * world]
        losses.append(tr.step(np.ascontiguousarray(g[rank * B_per:(rank + 1) * B_per]), np.ascontiguousarray(t[rank * B_per:(rank + 1) * B_per])))
    lib.bm_train_flush(tr.tr)   # a no-op after a complete window; a collective exchange + AdamW after a partial one
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), losses=np.array(losses),
             **{f"w{i}": tr.read(bmapi.BMX_WEIGHT, i) for i in range(tr.n_tensors())},
             **{f"m{i}": tr.read(bmapi.BMX_ADAM_M, i) for i in range(tr.n_tensors())})
    tr.close()


def _gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for l in out.splitlines() if l.startswith("GPU "))
    except Exception:
        return 0


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("precision", [bmapi.BM_PRECISION_BF16, bmapi.BM_PRECISION_FP32])
def test_two_gpu_data_parallel_matches_single_gpu_full_batch(tmp_path, precision):
    """Two ranks with 2 sequences each == one GPU with the 4 sequences: replicas stay bit-identical, the returned loss is the
    global mean, and the averaged gradient (read back as Adam's first moment) agrees to bf16 all-reduce rounding."""
    import torch.multiprocessing as mp
    world, B_per, S = 2, 2, 64
    id_path = str(tmp_path / "nccl_id")
    mp.spawn(_dp_worker, args=(world, id_path, str(tmp_path), B_per, S, precision), nprocs=world, join=True)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    lib = bmapi.load_product()
    a = bmapi.make_arch("gqa")
    tr = oc.LibTrainer(lib, "gpu", a, bmapi.make_weights(a), S, precision, bmapi.train_config(seq_len=S), quirks=False)
    x, y = bmapi.lcg_batch(B_per * world * 2, S, a.vocab_size)
    losses = [tr.step(np.ascontiguousarray(x[st * 4:(st + 1) * 4]), np.ascontiguousarray(y[st * 4:(st + 1) * 4])) for st in range(2)]
    assert np.allclose(r0["losses"], r1["losses"]) and np.abs(r0["losses"] - np.array(losses)).max() < 2e-3
    for i in range(tr.n_tensors()):
        assert np.array_equal(r0[f"w{i}"], r1[f"w{i}"]), i          # replicas identical
        # bf16 trainers all-reduce bf16 gradients; fp32 trainers all-reduce fp32, so their parity bound holds across ranks too
        bound = 2e-2 if precision == bmapi.BM_PRECISION_BF16 else 1e-4
        assert oc.rel_err(r0[f"m{i}"], tr.read(bmapi.BMX_ADAM_M, i)) < bound, i
        assert oc.cosine(r0[f"m{i}"], tr.read(bmapi.BMX_ADAM_M, i)) > 0.999, i
    tr.close()


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_gpu_flush_of_a_partial_accumulation_window(tmp_path):
    """grad_accum_steps = 2 and three micro-steps: the third opens a window that bm_train_flush must close. Under data parallel the
    flush exchanges the whole gradient first; the result equals one GPU running the same three micro-steps on the full batches."""
    import torch.multiprocessing as mp
    world, B_per, S, prec = 2, 2, 64, bmapi.BM_PRECISION_FP32
    mp.spawn(_dp_worker, args=(world, str(tmp_path / "nccl_id"), str(tmp_path), B_per, S, prec, 2, 3), nprocs=world, join=True)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    lib = bmapi.load_product()
    a = bmapi.make_arch("gqa")
    tr = oc.LibTrainer(lib, "gpu", a, bmapi.make_weights(a), S, prec, bmapi.train_config(seq_len=S, accum=2), quirks=False)
    x, y = bmapi.lcg_batch(B_per * world * 3, S, a.vocab_size)
    for st in range(3):
        tr.step(np.ascontiguousarray(x[st * 4:(st + 1) * 4]), np.ascontiguousarray(y[st * 4:(st + 1) * 4]))
    lib.bm_train_flush(tr.tr)
    for i in range(tr.n_tensors()):
        assert np.array_equal(r0[f"w{i}"], r1[f"w{i}"]), i
        assert oc.rel_err(r0[f"w{i}"], tr.read(bmapi.BMX_WEIGHT, i)) < 1e-4, i
        assert oc.rel_err(r0[f"m{i}"], tr.read(bmapi.BMX_ADAM_M, i)) < 1e-4, i
    tr.close()


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_cli_data_parallel_two_ranks(tmp_path):
    """baremetal-train started once per GPU with RANK / WORLD_SIZE / LOCAL_RANK: rank 0 prints and saves, the losses are those of one
    process training on the same global batch (2 ranks x 2 sequences = 4 sequences per step)."""
    a = bmapi.make_arch("gqa")
    model = str(tmp_path / "gqa.bin")
    bmapi.write_bin_checkpoint(model, a, bmapi.make_weights(a))
    toks = str(tmp_path / "data.bin")
    bmapi.lcg_tokens(4000, a.vocab_size).tofile(toks)
    out_dir = tmp_path / "out"
    out_dir.mkdir()
    base = [CLI, "train", model, toks, str(out_dir), "--steps", "3", "--seq-len", "64", "--lr", "1e-3", "--save-every", "3", "--precision", "fp32"]
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT="29671",
                   NCCL_NVLS_ENABLE="0")
        env.pop("BM_CUDA_DEVICE", None)
        procs.append(subprocess.Popen(base + ["--batch-size", "2"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=600) for p in procs]
    assert all(p.returncode == 0 for p in procs), [o[1][-800:] for o in outs]
    pat = re.compile(r"^step (\d+)/3: loss=(\d+\.\d{4})")
    l0 = [float(pat.match(l).group(2)) for l in outs[0][0].splitlines() if l.startswith("step ")]
    assert len(l0) == 3 and not any(l.startswith("step ") for l in outs[1][0].splitlines())   # only rank 0 reports
    assert os.path.exists(out_dir / "checkpoint_3.bin") and not os.path.exists(out_dir / ".bm_nccl_id.29671")
    one = subprocess.run(base + ["--batch-size", "4"], env={k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")},
                         capture_output=True, text=True, timeout=600)
    assert one.returncode == 0, one.stderr[-800:]
    l1 = [float(pat.match(l).group(2)) for l in one.stdout.splitlines() if l.startswith("step ")]
    assert np.abs(np.array(l0) - np.array(l1)).max() < 2e-4, (l0, l1)
