"""Pins the CPU oracle (oracle/bm_oracle.c) before anything trusts it:
 1. against the golden vectors of the reference's own PyTorch generators (tests/golden/torch_kernel_goldens.npz, made by
    tests/golden/make_golden.py running test/grad/gen_*.py unmodified) — the same vectors and the same cosine > 0.9999
    criterion the reference's kernel tests use (e.g. test/matmul_bwd_test.c, test/attn_real_test.c), plus a tight max-abs bound;
 2. against golden outputs of the reference's training step executed on CPU (tests/golden/ref_train_step_*.npz);
 3. against that reference build itself when oracle/_ref/libbm_ref.so is present.
"""
import ctypes as C
import glob
import os

import numpy as np
import pytest

import bmapi
import oracle_check as oc
import portk

GOLD_DIR = os.path.join(bmapi.ROOT, "tests", "golden")


def close(a, b, tol=2e-5):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    cos = a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-30)
    assert cos > 0.9999, cos
    scale = max(1.0, np.abs(b).max())
    assert np.abs(a - b).max() <= tol * scale, np.abs(a - b).max()


def test_matmul_backward(goldens):
    g = goldens
    inp, w, gout = g["inp"].reshape(3, 16), g["w"].reshape(8, 16), g["gout"].reshape(3, 8)
    close(portk.matmul_backward_inp(gout, w), g["ginp"])
    close(portk.matmul_backward_w(gout, inp), g["gw"])


def test_rmsnorm_backward(goldens):
    g = goldens
    x, w, go = g["rms_x"].reshape(4, 24), g["rms_w"], g["rms_gout"].reshape(4, 24)
    close(portk.rmsnorm_backward_x(go, w, x), g["rms_gx"])
    close(portk.rmsnorm_backward_w(go, x), g["rms_gw"])


def test_rope_backward_single_position(goldens):
    g = goldens  # NH=6 NKV=2 HD=8 pos=3 theta=1e4: place the vectors at row 3 of a 4-row sequence
    gq, gk = np.zeros((4, 6, 8), np.float32), np.zeros((4, 2, 8), np.float32)
    gq[3], gk[3] = g["rope_gout_q"].reshape(6, 8), g["rope_gout_k"].reshape(2, 8)
    rq, rk = portk.rope_seq(gq, gk, 10000.0, -1)
    close(rq[3], g["rope_gq"])
    close(rk[3], g["rope_gk"])


@pytest.mark.parametrize("prefix,NH,NKV,HD,S,theta", [("roseq", 4, 2, 8, 5, 10000.0), ("roreal", 9, 3, 64, 4, 100000.0)])
def test_rope_seq_backward(goldens, prefix, NH, NKV, HD, S, theta):
    g = goldens
    rq, rk = portk.rope_seq(g[prefix + "_gout_q"].reshape(S, NH, HD), g[prefix + "_gout_k"].reshape(S, NKV, HD), theta, -1)
    close(rq, g[prefix + "_gQ"])
    close(rk, g[prefix + "_gK"])


def test_rope_forward_is_inverse_of_backward(goldens):
    g = goldens
    q, k = g["roreal_Q"].reshape(4, 9, 64), g["roreal_K"].reshape(4, 3, 64)
    fq, fk = portk.rope_seq(q, k, 100000.0, +1)
    bq, bk = portk.rope_seq(fq, fk, 100000.0, -1)
    close(bq, q)
    close(bk, k)


def test_swiglu_backward(goldens):
    g = goldens
    gg, gu = portk.swiglu_backward(g["swiglu_gate"], g["swiglu_up"], g["swiglu_gout"])
    close(gg, g["swiglu_ggate"])
    close(gu, g["swiglu_gup"])


def test_xent_backward(goldens):
    g = goldens
    loss, grad = portk.xent(g["xent_logits"].reshape(3, 10), g["xent_targets"])
    close(grad, g["xent_glogits"])
    lg = g["xent_logits"].reshape(3, 10).astype(np.float64)
    ref_loss = np.mean([-(lg[n, t] - np.log(np.exp(lg[n]).sum())) for n, t in enumerate(g["xent_targets"])])
    assert abs(loss - ref_loss) < 1e-5


def test_embedding_backward_with_repeated_tokens(goldens):
    g = goldens
    out = portk.embedding_backward(np.zeros((8, 5), np.float32), g["embed_gout"].reshape(6, 5), g["embed_tokens"])
    close(out, g["embed_gwte"])
    assert len(set(g["embed_tokens"].tolist())) < 6  # the fixture does repeat tokens


@pytest.mark.parametrize("prefix,lr,wd", [("", 1e-2, 0.1), ("wd0_", 1e-3, 0.0)])
def test_adamw_step(goldens, prefix, lr, wd):
    g = goldens  # betas (0.9, 0.999), eps 1e-8, t = 1; (lr 1e-2, wd 0.1) from gen_adamw.py, (lr 1e-3, wd 0) from gen_adamw_wd0.py / test/adamw_test.c:49
    b1, b2 = 0.9, 0.999
    hp = [lr, b1, b2, 1e-8, wd, 1 - b1, 1 - b2, 1.0]
    w, m, v = portk.adamw(g[prefix + "adamw_w0"], g[prefix + "adamw_g"], np.zeros(64, np.float32), np.zeros(64, np.float32), hp)
    close(w, g[prefix + "adamw_w"], 1e-6)
    close(m, g[prefix + "adamw_m"], 1e-6)
    close(v, g[prefix + "adamw_v"], 1e-6)


@pytest.mark.parametrize("prefix,NH,NKV,HD,S", [("attn", 4, 2, 4, 3), ("attn_real", 9, 3, 64, 4)])
def test_attention_forward_backward(goldens, prefix, NH, NKV, HD, S):
    g = goldens
    Q, K, V = (g[f"{prefix}_{n}"].reshape(S, h, HD) for n, h in (("Q", NH), ("K", NKV), ("V", NKV)))
    scale = 1.0 / np.sqrt(HD)
    close(portk.attention_forward(Q, K, V, scale), g[prefix + "_out"])
    gq, gk, gv = portk.attention_backward(g[prefix + "_gout"].reshape(S, NH, HD), Q, K, V, scale)
    close(gq, g[prefix + "_gQ"])
    close(gk, g[prefix + "_gK"])
    close(gv, g[prefix + "_gV"])


def test_matmul_rmsnorm_matmul_chain(goldens):
    g = goldens  # test/sched_bwd_test.c: matmul -> rmsnorm -> matmul, BT4 C16 OC8 OC5
    inp, w1, rw, w2, gout = g["sb_inp"].reshape(4, 16), g["sb_w1"].reshape(8, 16), g["sb_rmsw"], g["sb_w2"].reshape(5, 8), g["sb_gout"].reshape(4, 5)
    h = portk.matmul_forward(inp, w1)
    hn = portk.rmsnorm_forward(h, rw)
    out = portk.matmul_forward(hn, w2)
    close(h, g["sb_h"]); close(hn, g["sb_hn"]); close(out, g["sb_out"])
    ghn = portk.matmul_backward_inp(gout, w2)
    close(portk.matmul_backward_w(gout, hn), g["sb_gw2"])
    close(portk.rmsnorm_backward_w(ghn, h), g["sb_grmsw"])
    gh = portk.rmsnorm_backward_x(ghn, rw, h)
    close(portk.matmul_backward_w(gh, inp), g["sb_gw1"])
    close(portk.matmul_backward_inp(gh, w1), g["sb_ginp"])


def test_full_decoder_layer(goldens):
    """One decoder layer, forward intermediates and all ten gradients (test/layer_bwd_test.c; S8 D64 NH4 NKV1 HD16 HID128)."""
    g = goldens
    S, D, NH, NKV, HD, HID, theta = 8, 64, 4, 1, 16, 128, 10000.0
    KV = NKV * HD
    inp, rw1, rw2 = g["layer_inp"].reshape(S, D), g["layer_rmsw1"], g["layer_rmsw2"]
    wq, wk, wv = g["layer_wq"].reshape(D, D), g["layer_wk"].reshape(KV, D), g["layer_wv"].reshape(KV, D)
    wo, wg, wu, wd = g["layer_wproj"].reshape(D, D), g["layer_wgate"].reshape(HID, D), g["layer_wup"].reshape(HID, D), g["layer_wdown"].reshape(D, HID)
    scale = 1.0 / np.sqrt(HD)
    n1 = portk.rmsnorm_forward(inp, rw1)
    q, k, v = portk.matmul_forward(n1, wq), portk.matmul_forward(n1, wk), portk.matmul_forward(n1, wv)
    qr, kr = portk.rope_seq(q.reshape(S, NH, HD), k.reshape(S, NKV, HD), theta, +1)
    att = portk.attention_forward(qr, kr, v.reshape(S, NKV, HD), scale).reshape(S, D)
    res1 = inp + portk.matmul_forward(att, wo)
    n2 = portk.rmsnorm_forward(res1, rw2)
    gate, up = portk.matmul_forward(n2, wg), portk.matmul_forward(n2, wu)
    act = portk.swiglu_forward(gate, up)
    res2 = res1 + portk.matmul_forward(act, wd)
    for name, val in (("n1", n1), ("q", qr), ("k", kr), ("attn_out", att), ("res1", res1), ("n2", n2), ("res2", res2)):
        close(val, g["layer_" + name], 1e-4)
    gres = g["layer_gout"].reshape(S, D).copy()
    close(portk.matmul_backward_w(gres, act), g["layer_gwdown"], 1e-4)
    gact = portk.matmul_backward_inp(gres, wd)
    gg, gu = portk.swiglu_backward(gate, up, gact)
    close(portk.matmul_backward_w(gg, n2), g["layer_gwgate"], 1e-4)
    close(portk.matmul_backward_w(gu, n2), g["layer_gwup"], 1e-4)
    gn2 = portk.matmul_backward_inp(gu, wu, portk.matmul_backward_inp(gg, wg))
    close(portk.rmsnorm_backward_w(gn2, res1), g["layer_grmsw2"], 1e-4)
    gres = portk.rmsnorm_backward_x(gn2, rw2, res1, gres)
    close(portk.matmul_backward_w(gres, att), g["layer_gwproj"], 1e-4)
    gatt = portk.matmul_backward_inp(gres, wo)
    gq, gk, gv = portk.attention_backward(gatt.reshape(S, NH, HD), qr, kr, v.reshape(S, NKV, HD), scale)
    gq, gk = portk.rope_seq(gq, gk, theta, -1)
    gq, gk, gv = gq.reshape(S, D), gk.reshape(S, KV), gv.reshape(S, KV)
    close(portk.matmul_backward_w(gq, n1), g["layer_gwq"], 1e-4)
    close(portk.matmul_backward_w(gk, n1), g["layer_gwk"], 1e-4)
    close(portk.matmul_backward_w(gv, n1), g["layer_gwv"], 1e-4)
    gn1 = portk.matmul_backward_inp(gv, wv, portk.matmul_backward_inp(gk, wk, portk.matmul_backward_inp(gq, wq)))
    close(portk.rmsnorm_backward_w(gn1, inp), g["layer_grmsw1"], 1e-4)
    close(portk.rmsnorm_backward_x(gn1, rw1, inp, gres), g["layer_ginp"], 1e-4)


def test_argmax_takes_the_lowest_index_among_maxima():
    x = np.array([0.5, 2.0, -1.0, 2.0, 2.0, 1.0], np.float32)
    assert portk.argmax(x) == 1  # strict '>' scan, src/baremetal/sampler.c:36-40
    assert portk.argmax(np.zeros(7, np.float32)) == 0


# ---- the training step as a whole ------------------------------------------------------------------------------
def _run_port(meta, quirks=oc.Q_ALL):
    arch = str(meta["arch"])
    B, S, prec, steps, accum = (int(meta[k]) for k in ("B", "S", "precision", "steps", "accum"))
    a = bmapi.make_arch(arch)
    w = bmapi.make_weights(a)
    cfg = bmapi.train_config(seq_len=S, accum=accum)
    x, y = bmapi.lcg_batch(B * steps * accum, S, a.vocab_size)
    tr = oc.PortTrainer(a, w, S, prec, cfg, quirks=quirks)
    losses, grads = [], None
    for st in range(steps * accum):
        losses.append(tr.step(np.ascontiguousarray(x[st * B:(st + 1) * B]), np.ascontiguousarray(y[st * B:(st + 1) * B])))
        if st == accum - 1:
            grads = [tr.read(bmapi.BMX_GRAD, i) for i in range(tr.n_tensors())]
    weights = [tr.read(bmapi.BMX_WEIGHT, i) for i in range(tr.n_tensors())]
    tr.close()
    return losses, grads, weights


def check_against_train_golden(meta, losses, grads, weights, rel_tol, loss_tol):
    assert np.abs(np.array(losses) - meta["losses"]).max() < loss_tol, (losses, meta["losses"])
    for i in range(int(meta["n_tensors"])):
        idx = meta["grad_idx"][i]
        idx = idx[idx >= 0]
        gn = float(meta["grad_norm"][i])
        assert abs(np.linalg.norm(grads[i].astype(np.float64)) - gn) <= rel_tol * gn + 1e-12, i
        assert np.abs(grads[i][idx] - meta["grad_val"][i][:idx.size]).max() <= rel_tol * max(np.abs(meta["grad_val"][i]).max(), gn / np.sqrt(grads[i].size)) * 10 + 1e-12, i
        wn = float(meta["weight_norm"][i])
        assert abs(np.linalg.norm(weights[i].astype(np.float64)) - wn) <= rel_tol * wn, i
        assert np.abs(weights[i][idx] - meta["weight_val"][i][:idx.size]).max() <= 10 * rel_tol * max(1e-3, np.abs(meta["weight_val"][i]).max()), i


SMALL_CASES = sorted(os.path.basename(p)[len("ref_train_step_"):-4] for p in glob.glob(os.path.join(GOLD_DIR, "ref_train_step_*.npz"))
                     if "135m" not in p)
# The 360M cases take the plain-C port 3.5 minutes each on eight cores: they run when BM_SLOW_PINS=1 (the GPU tests compare the product
# with the same recorded reference outputs directly, tests/test_gpu_train_step.py).
SLOW_CASES = {c for c in SMALL_CASES if "360m" in c}


@pytest.mark.parametrize("case", SMALL_CASES)
def test_port_matches_reference_train_step_golden(case):
    if case in SLOW_CASES and not os.environ.get("BM_SLOW_PINS"):
        pytest.skip("360M on the CPU port: set BM_SLOW_PINS=1")
    meta = np.load(os.path.join(GOLD_DIR, f"ref_train_step_{case}.npz"))
    losses, grads, weights = _run_port(meta)
    check_against_train_golden(meta, losses, grads, weights, rel_tol=2e-5, loss_tol=2e-5)


def test_goldens_exist():
    assert len(SMALL_CASES) >= 5
    assert os.path.exists(os.path.join(GOLD_DIR, "ref_train_step_135m_f32_c1.npz"))


@pytest.mark.skipif(oc.load_reference() is None, reason="reference build oracle/_ref/libbm_ref.so not present")
@pytest.mark.parametrize("arch,B,S,prec", [("tiny", 2, 16, 0), ("tiny", 1, 24, 2), ("small", 3, 24, 0)])
def test_port_matches_live_reference_build(arch, B, S, prec):
    a = bmapi.make_arch(arch)
    w = bmapi.make_weights(a, seed=7)
    cfg = bmapi.train_config(seq_len=S)
    x, y = bmapi.lcg_batch(B * 2, S, a.vocab_size, seed=9)
    r = oc.LibTrainer(oc.load_reference(), "reference", a, w, S, prec, cfg)
    p = oc.PortTrainer(a, w, S, prec, cfg)
    for st in range(2):
        xs, ys = np.ascontiguousarray(x[st * B:(st + 1) * B]), np.ascontiguousarray(y[st * B:(st + 1) * B])
        assert abs(r.step(xs, ys) - p.step(xs, ys)) < 2e-6
        for i in range(p.n_tensors()):
            assert oc.rel_err(p.read(bmapi.BMX_GRAD, i), r.read(bmapi.BMX_GRAD, i)) < 1e-5, (st, i)
    for i in range(p.n_tensors()):
        assert oc.rel_err(p.read(bmapi.BMX_WEIGHT, i), r.read(bmapi.BMX_WEIGHT, i)) < 1e-5
    r.close(); p.close()


@pytest.mark.skipif(oc.load_reference() is None, reason="reference build oracle/_ref/libbm_ref.so not present")
def test_adapter_merge_matches_live_reference_build(tmp_path):
    """bm_load_adapter of the product and of the reference build, given the same base weights and adapter file, leave the same
    merged weights: the reference's are read back through a trainer created after the merge (fp32 working copies)."""
    ref, prod = oc.load_reference(), bmapi.load_product()
    a = bmapi.make_arch("gqa")
    w = bmapi.make_weights(a, seed=5)
    rank, alpha = 4, 6.0
    rng = np.random.default_rng(3)
    shapes = dict(bmapi.weight_shapes(a))
    entries = []
    for layer, tgt in [(0, "q"), (0, "down"), (1, "k"), (1, "v"), (1, "o"), (0, "gate"), (1, "up")]:
        oc_, c = shapes[bmapi.ADAPTER_WEIGHT_KEY[tgt]][1:]
        entries.append((layer, tgt, rng.standard_normal((rank, c), dtype=np.float32) * np.float32(0.1),
                        rng.standard_normal((oc_, rank), dtype=np.float32) * np.float32(0.1)))
    base, adp = str(tmp_path / "base.bin"), str(tmp_path / "a.bmlora")
    bmapi.write_bin_checkpoint(base, a, w)
    bmapi.write_adapter_file(adp, a, rank, alpha, entries)

    pm = prod.bm_create_model(None, C.byref(a))
    prod.bm_load_weights(pm, base.encode())
    assert prod.bm_load_adapter(pm, adp.encode()) == 0
    n = C.c_size_t()
    flat = np.ctypeslib.as_array(prod.bmx_model_weight_buffer(pm, C.byref(n)), (n.value,)).copy()
    prod.bm_destroy_model(pm)
    got, off = {}, 0
    for k, shp in bmapi.weight_shapes(a):
        got[k] = flat[off:off + int(np.prod(shp))].reshape(shp)
        off += int(np.prod(shp))

    ctx = ref.bm_create(bmapi.BM_DEVICE_METAL)
    rm = ref.bm_create_model(ctx, C.byref(a))
    ref.bm_load_weights(rm, base.encode())
    assert ref.bm_load_adapter(rm, adp.encode()) == 0
    cfg = bmapi.train_config(seq_len=16)
    tr = ref.bm_create_trainer(ctx, rm, C.byref(cfg))
    assert tr
    changed = 0
    for i, (k, l) in enumerate(bmapi.state_tensor_order(a)):
        r = oc.reference_read(ref, tr, bmapi.BMX_WEIGHT, i)
        mine = (got[k] if l is None else got[k][l]).ravel()
        assert np.array_equal(r, mine), (k, l)
        changed += int(not np.array_equal(mine, (w[k] if l is None else w[k][l]).ravel()))
    assert changed == len(entries)
    ref.bm_destroy_trainer(tr)
    ref.bm_destroy_model(rm)
    ref.bm_destroy(ctx)


def test_quirk_flags_change_only_what_they_name():
    """With a single sequence per window the three reference deviations vanish: flags on == flags off."""
    a = bmapi.make_arch("tiny")
    w = bmapi.make_weights(a)
    cfg = bmapi.train_config(seq_len=16)
    x, y = bmapi.lcg_batch(1, 16, a.vocab_size)
    t1, t0 = oc.PortTrainer(a, w, 16, 0, cfg, quirks=oc.Q_ALL), oc.PortTrainer(a, w, 16, 0, cfg, quirks=0)
    assert t1.step(x, y) == t0.step(x, y)
    for i in range(t1.n_tensors()):
        assert np.array_equal(t1.read(bmapi.BMX_GRAD, i), t0.read(bmapi.BMX_GRAD, i))
    t1.close(); t0.close()


# ---- inference: Q8 quantiser and decode with a KV cache ---------------------------------------------------------------
# full-logit fixtures of the scaled-down models; the SmolLM2-360M fixtures (ref_decode_360m_*) store sampled logits only
DECODE_GOLDENS = sorted(p for p in glob.glob(os.path.join(GOLD_DIR, "ref_decode_*.npz")) if "_360m_" not in os.path.basename(p))
DECODE_GOLDENS_SAMPLED = sorted(glob.glob(os.path.join(GOLD_DIR, "ref_decode_360m_*.npz")))


def _quantize(fn, x):
    q = np.zeros(x.size, np.int8)
    sc = np.zeros(x.size // 32, np.float32)
    assert fn(oc.fptr(x), q.ctypes.data, oc.fptr(sc), x.size) == x.size // 32
    return q.reshape(-1, 32), sc


def test_quantize_q8_port_is_bit_exact_with_the_reference(port):
    """Reference quantiser output on seeded inputs with the scheme's edge cases (all-zero block, negative extreme,
    .5 ties, tiny values, one huge outlier): int8 values and fp32 scales must be identical."""
    g = np.load(os.path.join(GOLD_DIR, "ref_quantize_q8.npz"))
    q, sc = _quantize(port.orc_quantize_q8, np.ascontiguousarray(g["x"]))
    assert np.array_equal(q, g["q"]) and np.array_equal(sc.view(np.uint32), g["scale"].view(np.uint32))


def test_quantize_q8_rejects_ragged_input(port):
    x = np.ones(33, np.float32)
    q = np.zeros(64, np.int8)
    sc = np.zeros(2, np.float32)
    assert port.orc_quantize_q8(oc.fptr(x), q.ctypes.data, oc.fptr(sc), 33) == 0   # src/baremetal/quant.c:55
    assert port.orc_quantize_q8(oc.fptr(x), q.ctypes.data, oc.fptr(sc), 0) == 0


def test_product_host_quantiser_is_bit_exact_with_the_reference():
    """The product quantises on the host at session creation; same fixture, same bits."""
    lib = bmapi.load_product()
    g = np.load(os.path.join(GOLD_DIR, "ref_quantize_q8.npz"))
    q, sc = _quantize(lib.bmx_quantize_q8, np.ascontiguousarray(g["x"]))
    assert np.array_equal(q, g["q"]) and np.array_equal(sc.view(np.uint32), g["scale"].view(np.uint32))


def test_quantize_q4_port_and_product_are_bit_exact_with_the_reference(port):
    """bmt_quantize_q4 on the same seeded blocks (scale = amax / 7, codes in [-8, 7], src/baremetal/quant.c:31-52): the fixture holds the
    reference's codes sign-extended and unpacked; the port's and the product's host quantiser give the same codes and scales."""
    g = np.load(os.path.join(GOLD_DIR, "ref_quantize_q4.npz"))
    x = np.ascontiguousarray(g["x"])
    for fn in (port.orc_quantize_q4, bmapi.load_product().bmx_quantize_q4):
        q, sc = _quantize(fn, x)
        assert np.array_equal(q, g["q"]) and np.array_equal(sc.view(np.uint32), g["scale"].view(np.uint32))
        assert q.min() >= -8 and q.max() <= 7
        one = np.ones(33, np.float32)
        assert fn(oc.fptr(one), q.ctypes.data, oc.fptr(sc), 33) == 0 and fn(oc.fptr(one), q.ctypes.data, oc.fptr(sc), 0) == 0


def test_live_reference_q4_quantiser_matches_port_on_random_blocks(port):
    ref = oc.load_reference()
    if ref is None:
        pytest.skip("reference build absent")
    x = (np.random.default_rng(6).standard_normal(32 * 257) * 0.3).astype(np.float32)
    blocks = np.zeros(x.size // 32, dtype=np.dtype([("scale", "<f4"), ("qs", "u1", (16,))]))   # q4_block_t, src/baremetal/quant.h:39-42
    assert ref.bmt_quantize_q4(oc.fptr(x), blocks.ctypes.data, x.size) == x.size // 32
    codes = np.stack([blocks["qs"] & 0x0F, blocks["qs"] >> 4], axis=-1).reshape(-1, 32).astype(np.int8)
    codes = np.where(codes > 7, codes - 16, codes).astype(np.int8)
    q, sc = _quantize(port.orc_quantize_q4, x)
    assert np.array_equal(q, codes) and np.array_equal(sc, blocks["scale"])


def test_live_reference_quantiser_matches_port_on_random_blocks(port):
    ref = oc.load_reference()
    if ref is None:
        pytest.skip("reference build absent")
    x = (np.random.default_rng(5).standard_normal(32 * 257) * 0.3).astype(np.float32)
    blocks = np.zeros(x.size // 32, dtype=np.dtype([("scale", "<f4"), ("q", "i1", (32,))]))
    assert ref.bmt_quantize_q8(oc.fptr(x), blocks.ctypes.data, x.size) == x.size // 32
    q, sc = _quantize(port.orc_quantize_q8, x)
    assert np.array_equal(q, blocks["q"]) and np.array_equal(sc, blocks["scale"])


def decode_case(path):
    g = np.load(path)
    a = bmapi.make_arch(str(g["arch"]))
    w = bmapi.make_weights(a, layer_scale=float(g["layer_scale"]))
    return g, a, w


@pytest.mark.parametrize("path", DECODE_GOLDENS, ids=[os.path.basename(p)[11:-4] for p in DECODE_GOLDENS])
def test_decode_port_matches_reference_session(path):
    """Token-by-token decode of the plain-C oracle against logits of the reference session after every prompt prefix, and
    the reference's greedy continuation; fp32 and bf16 weights, plain and Q8."""
    g, a, w = decode_case(path)
    dec = oc.PortDecoder(a, w, int(g["precision"]), int(g["quant"]), 64)
    prompt = g["prompt"]
    for i, t in enumerate(prompt):
        lg = dec.step(t)
        if i >= 1:
            ref = g["logits"][i - 1]
            assert np.abs(lg - ref).max() <= 1e-5 * np.abs(ref).max(), (i, np.abs(lg - ref).max())
    out = []
    for _ in range(len(g["greedy"])):
        out.append(int(np.argmax(lg)))
        lg = dec.step(out[-1])
    dec.close()
    assert out == list(g["greedy"])
