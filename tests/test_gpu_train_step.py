"""The training step on the GPU against the reference: live against the reference build / plain-C oracle on scaled-down
members of the model family, and against committed golden outputs of the reference (tests/golden/ref_train_step_*.npz),
including the 135M-parameter single-step fp32 configuration.
Tolerances (as stated for this path): fp32 mode — per-tensor gradients and post-step weights within 1e-4 relative error,
loss within 1e-3; bf16 mode — within 2e-2 relative error and cosine similarity > 0.999."""
import ctypes as C
import glob
import os

import numpy as np
import pytest

import bmapi
import oracle_check as oc
from test_oracle_pins import GOLD_DIR

pytestmark = pytest.mark.gpu
F32, BF16 = bmapi.BM_PRECISION_FP32, bmapi.BM_PRECISION_BF16


def limits(precision):
    return (1e-4, 0.99999) if precision == F32 else (2e-2, 0.999)


@pytest.mark.parametrize("arch,B,S,precision", [("tiny", 1, 16, F32), ("tiny", 3, 32, F32), ("small", 2, 64, F32), ("gqa", 2, 128, F32),
                                                ("tiny", 2, 32, BF16), ("gqa", 2, 128, BF16), ("small", 3, 200, BF16), ("gqa", 1, 300, F32)])
def test_step_matches_reference(product, arch, B, S, precision):
    res = oc.compare_one_step(product, arch, B, S, precision, steps=2)
    rel, cos = limits(precision)
    assert np.abs(np.array(res["losses_gpu"]) - np.array(res["losses_oracle"])).max() < 1e-3, res
    assert res["worst_grad_rel"] < rel and res["min_grad_cos"] > cos, (res["worst_grad_rel"], res["min_grad_cos"], res["oracle_kind"])
    assert res["worst_weight_rel"] < rel and res["min_weight_cos"] > cos


def test_exact_gradient_mode_matches_oracle_without_quirks(product):
    """Default mode (no reference-compatibility switches) against the oracle with its three deviations switched off."""
    res = oc.compare_one_step(product, "tiny", 3, 32, F32, quirks=False, steps=2)
    assert res["oracle_kind"] == "port"
    assert res["worst_grad_rel"] < 1e-4 and res["worst_weight_rel"] < 1e-4
    assert np.abs(np.array(res["losses_gpu"]) - np.array(res["losses_oracle"])).max() < 1e-4


def test_gradient_accumulation_window(product):
    """Two micro-steps per optimizer step (test/grad_accum_test.c): gradients add up over the window, one AdamW update."""
    res = oc.compare_one_step(product, "small", 2, 64, F32, steps=2, accum=2)
    assert res["worst_grad_rel"] < 1e-4 and res["worst_weight_rel"] < 1e-4


def _run_gpu(lib, meta):
    arch = str(meta["arch"])
    B, S, prec, steps, accum = (int(meta[k]) for k in ("B", "S", "precision", "steps", "accum"))
    a = bmapi.make_arch(arch)
    w = bmapi.make_weights(a)
    cfg = bmapi.train_config(seq_len=S, accum=accum)
    x, y = bmapi.lcg_batch(B * steps * accum, S, a.vocab_size)
    tr = oc.LibTrainer(lib, "gpu", a, w, S, prec, cfg, quirks=True)
    losses, grads = [], None
    for st in range(steps * accum):
        losses.append(tr.step(np.ascontiguousarray(x[st * B:(st + 1) * B]), np.ascontiguousarray(y[st * B:(st + 1) * B])))
        if st == accum - 1:
            grads = [tr.read(bmapi.BMX_GRAD, i) for i in range(tr.n_tensors())]
    weights = [tr.read(bmapi.BMX_WEIGHT, i) for i in range(tr.n_tensors())]
    tr.close()
    return losses, grads, weights


CASES = sorted(os.path.basename(p)[len("ref_train_step_"):-4] for p in glob.glob(os.path.join(GOLD_DIR, "ref_train_step_*.npz")))


@pytest.mark.parametrize("case", CASES)
def test_step_matches_committed_reference_outputs(product, case):
    """Losses, per-tensor gradient norms and sampled gradient / post-step weight values recorded from the reference."""
    meta = np.load(os.path.join(GOLD_DIR, f"ref_train_step_{case}.npz"))
    losses, grads, weights = _run_gpu(product, meta)
    rel, _ = limits(int(meta["precision"]))
    assert np.abs(np.array(losses) - meta["losses"]).max() < 1e-3, (losses, meta["losses"])
    for i in range(int(meta["n_tensors"])):
        idx = meta["grad_idx"][i]
        idx = idx[idx >= 0]
        gn, wn = float(meta["grad_norm"][i]), float(meta["weight_norm"][i])
        assert abs(np.linalg.norm(grads[i].astype(np.float64)) - gn) <= rel * gn + 1e-12, (case, i)
        ref_s, got_s = meta["grad_val"][i][:idx.size].astype(np.float64), grads[i][idx].astype(np.float64)
        assert np.linalg.norm(got_s - ref_s) <= 3 * rel * max(np.linalg.norm(ref_s), gn * np.sqrt(idx.size / grads[i].size)) + 1e-12, (case, i)
        assert abs(np.linalg.norm(weights[i].astype(np.float64)) - wn) <= rel * wn, (case, i)
        ref_w, got_w = meta["weight_val"][i][:idx.size].astype(np.float64), weights[i][idx].astype(np.float64)
        assert np.linalg.norm(got_w - ref_w) <= 3 * rel * np.linalg.norm(ref_w) + 1e-9, (case, i)


CURVES = sorted(os.path.basename(p)[len("ref_train_curve_"):-4] for p in glob.glob(os.path.join(GOLD_DIR, "ref_train_curve_*.npz")))
# Loss-curve bounds. fp32 mode computes what the reference computes, in another summation order: 1e-3 on every step's loss. In bf16
# mode the reference keeps fp32 activations and only rounds the matrices, while this trainer also keeps activations in bf16
# (tensor-core operands). Training on uniformly random tokens at lr 3e-4 is sensitive to rounding: the reference's OWN two modes drift
# apart by up to 0.11 in loss over these 50 steps (both curves are committed). So in bf16 mode the curve must stay within 2e-3 of the
# reference's bf16 curve for the first ten steps, within 1e-2 at the median, and nowhere further from it than twice the distance
# between the reference's fp32 and bf16 curves.
def curve_bounds(case, prec, ref_losses):
    if prec == F32:
        return 1e-3, 1e-3, 1e-3
    other = np.load(os.path.join(GOLD_DIR, "ref_train_curve_" + case.replace("bf16", "f32") + ".npz"))["losses"]
    return 2e-3, 1e-2, 2.0 * float(np.abs(other - ref_losses).max())


@pytest.mark.parametrize("case", CURVES)
def test_loss_curve_over_50_steps_matches_reference(product, case):
    """SmolLM2-135M, 50 optimizer steps on fresh token windows (two sequences of 128 tokens per step, AdamW lr 3e-4): the loss after
    every step and the final weights against the reference's recorded run (its own analogue: test/g3_test.c, 10 steps)."""
    g = np.load(os.path.join(GOLD_DIR, f"ref_train_curve_{case}.npz"))
    B, S, prec, steps = (int(g[k]) for k in ("B", "S", "precision", "steps"))
    a = bmapi.make_arch(str(g["arch"]))
    w = bmapi.make_weights(a)
    x, y = bmapi.lcg_batch(B * steps, S, a.vocab_size)
    tr = oc.LibTrainer(product, "gpu", a, w, S, prec, bmapi.train_config(seq_len=S), quirks=True)
    losses = [tr.step(np.ascontiguousarray(x[st * B:(st + 1) * B]), np.ascontiguousarray(y[st * B:(st + 1) * B])) for st in range(steps)]
    diff = np.abs(np.array(losses) - g["losses"])
    print(f"curve {case}: max |loss - reference| {diff.max():.3e} at step {int(diff.argmax())}, final {losses[-1]:.5f} vs {float(g['losses'][-1]):.5f}")
    first10, median, anywhere = curve_bounds(case, prec, g["losses"])
    print(f"curve {case}: first ten {diff[:10].max():.2e} (bound {first10:.0e}), median {np.median(diff):.2e} (bound {median:.0e}), bound anywhere {anywhere:.3f}")
    assert diff[:10].max() < first10 and np.median(diff) < median and diff.max() < anywhere, (diff[:10].max(), np.median(diff), diff.max())
    # final weights: per-tensor norms within the step tolerance; the 64 sampled values per tensor within 3e-4 (fp32) / 1e-1 (bf16: fifty
    # AdamW updates of about lr each, whose direction for small gradients depends on rounding; measured 6e-2 worst)
    rel = 1e-4 if prec == F32 else 2e-2
    rel_sampled = 3e-4 if prec == F32 else 1e-1
    worst = 0.0
    for i in range(int(g["n_tensors"])):
        idx = g["weight_idx"][i]
        idx = idx[idx >= 0]
        t = tr.read(bmapi.BMX_WEIGHT, i)
        wn = float(g["weight_norm"][i])
        assert abs(np.linalg.norm(t.astype(np.float64)) - wn) <= rel * wn, (case, i)
        ref_w, got_w = g["weight_val"][i][:idx.size].astype(np.float64), t[idx].astype(np.float64)
        worst = max(worst, np.linalg.norm(got_w - ref_w) / (np.linalg.norm(ref_w) + 1e-30))
        assert np.linalg.norm(got_w - ref_w) <= rel_sampled * np.linalg.norm(ref_w) + 1e-9, (case, i)
    print(f"curve {case}: worst sampled final-weight error {worst:.3e}")
    tr.close()


@pytest.mark.parametrize("precision,use_attn_mask", [(F32, True), (F32, False), (BF16, True), (BF16, False)])
def test_masked_step_matches_reference(product, precision, use_attn_mask):
    """Completion-only loss with a padding mask (bm_train_step_masked; the reference's masked_sft_test.c): attn == 0 removes a
    position as key and as query, loss == 1 marks the rows that count, each sequence normalised by its own count; one
    sequence has no counted row at all."""
    ref = oc.load_reference()
    if ref is None:
        pytest.skip("reference build not present")
    a = bmapi.make_arch("gqa")
    w = bmapi.make_weights(a)
    B, S = 3, 48
    cfg = bmapi.train_config(seq_len=S)
    x, y = bmapi.lcg_batch(B, S, a.vocab_size)
    attn = np.ones((B, S), np.uint8)
    attn[0, 40:] = 0
    attn[1, 30:] = 0
    loss = np.zeros((B, S), np.uint8)
    loss[0, 10:40] = 1
    loss[1, 5:30] = 1  # sequence 2 keeps an all-zero loss mask
    am = attn if use_attn_mask else None
    g = oc.LibTrainer(product, "gpu", a, w, S, precision, cfg, quirks=True)
    r = oc.LibTrainer(ref, "reference", a, w, S, precision, cfg)
    le_g, le_r = g.step_masked(x, y, am, loss, evaluate=True), r.step_masked(x, y, am, loss, evaluate=True)
    lg, lr = g.step_masked(x, y, am, loss), r.step_masked(x, y, am, loss)
    assert abs(lg - lr) < 1e-3 and abs(le_g - le_r) < 1e-3 and abs(le_g - lg) < 1e-6
    rel, cos = limits(precision)
    for i in range(g.n_tensors()):
        gg, rg = g.read(bmapi.BMX_GRAD, i), r.read(bmapi.BMX_GRAD, i)
        if not rg.any():  # RMSNorm gains keep only the last sequence's gradient in the reference, and that sequence is fully masked
            assert not gg.any(), i
            continue
        assert oc.rel_err(gg, rg) < rel and oc.cosine(gg, rg) > cos, i
        assert oc.rel_err(g.read(bmapi.BMX_WEIGHT, i), r.read(bmapi.BMX_WEIGHT, i)) < rel, i
    g.close(); r.close()


def test_sequence_length_mismatch_is_an_error(product):
    a = bmapi.make_arch("tiny")
    tr = oc.LibTrainer(product, "gpu", a, bmapi.make_weights(a), 16, F32, bmapi.train_config(seq_len=16))
    x, y = bmapi.lcg_batch(1, 8, a.vocab_size)
    assert product.bm_train_step(tr.tr, bmapi.as_int_ptr(x), bmapi.as_int_ptr(y), 1, 8) == -1.0  # trainer.c:450-453
    tr.close()


def test_state_file_round_trip_and_layout(product, tmp_path):
    """bm_save_state writes the reference's layout; loading it into a fresh trainer resumes bit-identically."""
    a = bmapi.make_arch("tiny")
    w = bmapi.make_weights(a)
    cfg = bmapi.train_config(seq_len=32)
    x, y = bmapi.lcg_batch(6, 32, a.vocab_size)
    t1 = oc.LibTrainer(product, "gpu", a, w, 32, BF16, cfg, quirks=False)
    for st in range(2):
        t1.step(x[2 * st:2 * st + 2].copy(), y[2 * st:2 * st + 2].copy())
    path = str(tmp_path / "state.bin")
    product.bm_save_state(t1.tr, path.encode())
    step, tensors = bmapi.read_state_file(path)
    assert step == 2 and len(tensors) == 9 * a.n_layers + 2
    order = bmapi.state_tensor_order(a)
    shapes = dict(bmapi.weight_shapes(a))
    for (key, layer), (tw, tm, tv), i in zip(order, tensors, range(len(order))):
        n = int(np.prod(shapes[key][1:] if layer is not None else shapes[key]))
        assert tw.size == tm.size == tv.size == n
        assert np.array_equal(tw, t1.read(bmapi.BMX_WEIGHT, i)) and np.array_equal(tm, t1.read(bmapi.BMX_ADAM_M, i))
    l1 = t1.step(x[4:6].copy(), y[4:6].copy())
    t2 = oc.LibTrainer(product, "gpu", a, w, 32, BF16, cfg, quirks=False)
    product.bm_load_state(t2.tr, path.encode())
    l2 = t2.step(x[4:6].copy(), y[4:6].copy())
    assert l1 == l2
    for i in range(t1.n_tensors()):
        assert np.array_equal(t1.read(bmapi.BMX_WEIGHT, i), t2.read(bmapi.BMX_WEIGHT, i))
    t1.close(); t2.close()


def test_reference_can_load_our_state_file(product, tmp_path):
    """Cross-implementation check of the checkpoint layout: a state written by the GPU trainer is accepted by the
    reference's bm_load_state (its loader validates the tensor count and every size, trainer.c:213-226)."""
    ref = oc.load_reference()
    if ref is None:
        pytest.skip("reference build not present")
    a = bmapi.make_arch("tiny")
    w = bmapi.make_weights(a)
    cfg = bmapi.train_config(seq_len=16)
    x, y = bmapi.lcg_batch(2, 16, a.vocab_size)
    g = oc.LibTrainer(product, "gpu", a, w, 16, F32, cfg)
    g.step(x[:1].copy(), y[:1].copy())
    path = str(tmp_path / "s.bin")
    product.bm_save_state(g.tr, path.encode())
    r = oc.LibTrainer(ref, "reference", a, w, 16, F32, cfg)
    ref.bm_load_state(r.tr, path.encode())
    for i in range(g.n_tensors()):
        assert np.array_equal(r.read(bmapi.BMX_WEIGHT, i), g.read(bmapi.BMX_WEIGHT, i))
        assert np.array_equal(r.read(bmapi.BMX_ADAM_V, i), g.read(bmapi.BMX_ADAM_V, i))
    g.close(); r.close()


def test_loss_decreases_over_steps_bf16(product):
    """Repeatedly fitting one small batch drives the loss down (the reference's convergence smoke, test/g4_test.c)."""
    a = bmapi.make_arch("small")
    tr = oc.LibTrainer(product, "gpu", a, bmapi.make_weights(a), 64, BF16, bmapi.train_config(lr=1e-3, wd=0.0, seq_len=64), quirks=False)
    x, y = bmapi.lcg_batch(4, 64, a.vocab_size)
    losses = [tr.step(x, y) for _ in range(30)]
    tr.close()
    assert np.median(losses[-5:]) < np.median(losses[:5]) - 1.0, losses


def test_resident_step_equals_host_step(product):
    a = bmapi.make_arch("tiny")
    w = bmapi.make_weights(a)
    cfg = bmapi.train_config(seq_len=32)
    x, y = bmapi.lcg_batch(2, 32, a.vocab_size)
    t1 = oc.LibTrainer(product, "gpu", a, w, 32, BF16, cfg, quirks=False)
    t2 = oc.LibTrainer(product, "gpu", a, w, 32, BF16, cfg, quirks=False)
    l1 = t1.step(x, y)
    dx, dy = product.bmx_device_alloc(t2.ctx, x.nbytes), product.bmx_device_alloc(t2.ctx, y.nbytes)
    product.bmx_device_upload(t2.ctx, dx, x.ctypes.data, x.nbytes)
    product.bmx_device_upload(t2.ctx, dy, y.ctypes.data, y.nbytes)
    assert product.bmx_train_step_resident(t2.tr, dx, dy, 2, 32) == 0
    assert product.bmx_train_last_loss(t2.tr) == l1
    assert product.bmx_trainer_launch_count(t2.tr) > 0
    t1.close(); t2.close()


def test_graph_replay_matches_eager_steps_with_changing_batch(product):
    """From the third plain step on forward + backward are replayed as a CUDA graph; losses and weights must be the same as with
    the graph switched off, also when the batch size changes in between (the graph is dropped and re-made)."""
    a = bmapi.make_arch("small")
    w = bmapi.make_weights(a)
    S = 64
    plan = [2, 2, 2, 2, 3, 3, 3, 3, 2, 2, 2, 2]
    x, y = bmapi.lcg_batch(sum(plan), S, a.vocab_size)
    results = []
    for graph in (1, 0):
        tr = oc.LibTrainer(product, "gpu", a, w, S, BF16, bmapi.train_config(seq_len=S), quirks=False, tag=f"g{graph}")
        assert product.bmx_trainer_set_option(tr.tr, b"train_graph", graph) == 0
        assert product.bmx_trainer_set_option(tr.tr, b"side_stream", 0) == 0   # weight gradients in a fixed order on one stream
        losses, off = [], 0
        for B in plan:
            losses.append(tr.step(np.ascontiguousarray(x[off:off + B]), np.ascontiguousarray(y[off:off + B])))
            off += B
        weights = [tr.read(bmapi.BMX_WEIGHT, i) for i in range(tr.n_tensors())]
        tr.close()
        results.append((losses, weights))
    (l1, w1), (l0, w0) = results
    assert np.allclose(l1, l0, rtol=0, atol=2e-3), (l1, l0)
    for u, v in zip(w1, w0):
        assert oc.rel_err(u, v) < 1e-3
