"""Per-kernel parity on the GPU, called through the extern "C" backend ABI (include/bm_cuda_backend.h) and checked
against the CPU oracle on the same seeded inputs and against the reference's own golden vectors.
fp32 activations: relative error <= 1e-5 (exact arithmetic up to summation order).
bf16 activations: inputs are rounded to bf16 first, the oracle runs on those rounded values in fp32, and the result may
differ by bf16 output rounding plus bf16 rounding of intermediates: relative error <= 2e-2, cosine > 0.999."""
import numpy as np
import pytest

import oracle_check as oc
import portk
from bmcapi import BMC_BF16, BMC_F32, Backend, Ptr, bf16_round

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(1234)


@pytest.fixture(scope="module")
def be(product):
    b = Backend(product)
    yield b
    b.close()


def tol(dtype):
    return (1e-5, 0.999999) if dtype == BMC_F32 else (2e-2, 0.999)


def check(got, ref, dtype, scale_rel=1.0):
    r, c = tol(dtype)
    assert oc.rel_err(got, ref) <= r * scale_rel, oc.rel_err(got, ref)
    if np.linalg.norm(ref) > 0:
        assert oc.cosine(got.ravel(), ref.ravel()) >= c


def rnd(*shape, scale=1.0, dtype=BMC_F32):
    x = (RNG.standard_normal(shape) * scale).astype(np.float32)
    return bf16_round(x) if dtype == BMC_BF16 else x


DTYPES = [BMC_F32, BMC_BF16]

# (BT, C, OC): SmolLM2 projection shapes at small BT, tile-edge cases, and the reference's odd test shape scaled to the
# 8-element granularity TMA needs (test/simd_matmul_test.c:30 uses BT37 C53 OC70)
GEMM_SHAPES = [(64, 576, 576), (64, 576, 192), (37, 56, 72), (200, 960, 1600), (130, 2560, 960), (256, 960, 5120), (3, 16, 8),
               (129, 64, 200), (300, 72, 160), (700, 960, 1600), (513, 192, 960), (1024, 320, 136)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("BT,C,OC", GEMM_SHAPES)
def test_matmul_forward_backward(be, dtype, BT, C, OC):
    x, w, go = rnd(BT, C, dtype=dtype), rnd(OC, C, scale=C ** -0.5, dtype=dtype), rnd(BT, OC, dtype=dtype)
    res = rnd(BT, OC, dtype=dtype)
    dx, dw, dgo, dres = be.put(x, dtype), be.put(w, dtype), be.put(go, dtype), be.put(res, dtype)
    out = be.zeros(BT * OC, dtype)
    be.ok("matmul_forward", dtype, Ptr(out), OC, Ptr(dx), C, Ptr(dw), None, 0, BT, C, OC)
    check(be.get(out, (BT, OC), dtype), portk.matmul_forward(x, w), dtype)
    be.ok("matmul_forward", dtype, Ptr(out), OC, Ptr(dx), C, Ptr(dw), Ptr(dres), OC, BT, C, OC)  # fused residual add
    check(be.get(out, (BT, OC), dtype), portk.matmul_forward(x, w) + res, dtype)
    gin = be.zeros(BT * C, dtype)
    be.ok("matmul_backward_inp", dtype, Ptr(gin), C, 0, Ptr(dgo), OC, Ptr(dw), BT, C, OC)
    ref_gin = portk.matmul_backward_inp(go, w)
    check(be.get(gin, (BT, C), dtype), ref_gin, dtype)
    be.ok("matmul_backward_inp", dtype, Ptr(gin), C, 1, Ptr(dgo), OC, Ptr(dw), BT, C, OC)  # the reference's '+=' form
    check(be.get(gin, (BT, C), dtype), 2 * ref_gin, dtype, 1.5)
    gw0 = rnd(OC, C)
    gw = be.put(gw0)  # weight gradients are fp32 and accumulate (backward.metal:277)
    be.ok("matmul_backward_w", dtype, Ptr(gw), Ptr(dgo), OC, Ptr(dx), C, BT, C, OC)
    check(be.get(gw, (OC, C)), portk.matmul_backward_w(go, x, gw0), BMC_F32 if dtype == BMC_F32 else BMC_BF16)


@pytest.mark.parametrize("dtype", DTYPES)
def test_matmul_golden_vectors(be, goldens, dtype):
    g = goldens  # test/matmul_bwd_test.c: BT3 C16 OC8
    inp, w, gout = (bf16_round(a) if dtype == BMC_BF16 else a for a in (g["inp"].reshape(3, 16), g["w"].reshape(8, 16), g["gout"].reshape(3, 8)))
    gin, gw = be.zeros(48, dtype), be.zeros(128)
    be.ok("matmul_backward_inp", dtype, Ptr(gin), 16, 0, Ptr(be.put(gout, dtype)), 8, Ptr(be.put(w, dtype)), 3, 16, 8)
    be.ok("matmul_backward_w", dtype, Ptr(gw), Ptr(be.put(gout, dtype)), 8, Ptr(be.put(inp, dtype)), 16, 3, 16, 8)
    ref_gi, ref_gw = (g["ginp"].reshape(3, 16), g["gw"].reshape(8, 16)) if dtype == BMC_F32 else (portk.matmul_backward_inp(gout, w), portk.matmul_backward_w(gout, inp))
    check(be.get(gin, (3, 16), dtype), ref_gi, dtype)
    check(be.get(gw, (8, 16)), ref_gw, dtype)


FUSED_MLP_SHAPES = [(64, 128, 128), (300, 192, 256), (1000, 960, 2560), (513, 576, 1536), (256, 64, 384)]


@pytest.mark.parametrize("BT,C,H", FUSED_MLP_SHAPES)
def test_gate_up_projection_with_swiglu_in_the_epilogue(be, BT, C, H):
    """One launch = matmul_forward over [gate; up] followed by swiglu_forward: gate | up against the oracle GEMM, act against the
    oracle activation of the stored (bf16) gate and up, and everything against the two-launch path."""
    dt = BMC_BF16
    x, w = rnd(BT, C, dtype=dt), rnd(2 * H, C, scale=2.0 * C ** -0.5, dtype=dt)
    dx, dw = be.put(x, dt), be.put(w, dt)
    gu, act = be.zeros(BT * 2 * H, dt), be.zeros(BT * H, dt)
    be.ok("matmul_swiglu_forward", dt, Ptr(gu), 2 * H, Ptr(act), H, Ptr(dx), C, Ptr(dw), BT, C, H)
    got_gu, got_act = be.get(gu, (BT, 2 * H), dt), be.get(act, (BT, H), dt)
    check(got_gu, portk.matmul_forward(x, w), dt)
    check(got_act, portk.swiglu_forward(got_gu[:, :H], got_gu[:, H:]), dt)
    gu2, act2 = be.zeros(BT * 2 * H, dt), be.zeros(BT * H, dt)
    be.ok("matmul_forward", dt, Ptr(gu2), 2 * H, Ptr(dx), C, Ptr(dw), None, 0, BT, C, 2 * H)
    be.ok("swiglu_forward", dt, Ptr(act2), H, Ptr(gu2), Ptr(gu2, H * 2), 2 * H, BT, H)
    assert np.array_equal(got_gu, be.get(gu2, (BT, 2 * H), dt))
    assert oc.rel_err(got_act, be.get(act2, (BT, H), dt)) < 1e-2


@pytest.mark.parametrize("BT,D,H", FUSED_MLP_SHAPES)
def test_down_projection_input_gradient_with_swiglu_backward_in_the_epilogue(be, BT, D, H):
    dt = BMC_BF16
    go, w, gu = rnd(BT, D, dtype=dt), rnd(D, H, scale=H ** -0.5, dtype=dt), rnd(BT, 2 * H, scale=2.0, dtype=dt)
    dgo, dw, dgu = be.put(go, dt), be.put(w, dt), be.put(gu, dt)
    out = be.zeros(BT * 2 * H, dt)
    be.ok("matmul_backward_inp_swiglu", dt, Ptr(out), 2 * H, Ptr(dgo), D, Ptr(dw), Ptr(dgu), 2 * H, BT, H, D)
    dact = portk.matmul_backward_inp(go, w)
    rg, ru = portk.swiglu_backward(gu[:, :H], gu[:, H:], dact)
    got = be.get(out, (BT, 2 * H), dt)
    check(got[:, :H], rg, dt)
    check(got[:, H:], ru, dt)


def test_fused_mlp_entry_points_decline_what_they_cannot_fuse(be):
    z = be.zeros(64 * 512, BMC_F32)
    assert be.call("matmul_swiglu_forward", BMC_F32, Ptr(z), 256, Ptr(z), 128, Ptr(z), 64, Ptr(z), 64, 64, 128) == -70   # fp32
    assert be.call("matmul_swiglu_forward", BMC_BF16, Ptr(z), 272, Ptr(z), 136, Ptr(z), 64, Ptr(z), 64, 64, 136) == -70  # H % 128
    assert be.call("matmul_backward_inp_swiglu", BMC_BF16, Ptr(z), 272, Ptr(z), 64, Ptr(z), Ptr(z), 272, 64, 136, 64) == -70
    assert be.call("matmul_backward_inp_rowdot", BMC_BF16, Ptr(z), 96, Ptr(z), Ptr(z), 64, Ptr(z), Ptr(z), 96, 64, 96, 64, 32, 2) == -70
    assert product_status(be) == 0


def product_status(be):
    return be.lib.bmc_sync(be.ctx)


@pytest.mark.parametrize("B,S,NH,D", [(1, 64, 2, 128), (2, 160, 6, 384), (1, 512, 15, 960)])
def test_o_projection_input_gradient_with_row_sums_in_the_epilogue(be, B, S, NH, D):
    """ginp = gout * W and, per (row, head), the dot product of the stored ginp with another tensor of the same shape."""
    dt = BMC_BF16
    BT, QD = B * S, NH * 64
    go, w, other = rnd(BT, D, dtype=dt), rnd(D, QD, scale=D ** -0.5, dtype=dt), rnd(BT, QD, dtype=dt)
    gin, rd = be.zeros(BT * QD, dt), be.zeros(B * NH * S)
    be.ok("matmul_backward_inp_rowdot", dt, Ptr(gin), QD, Ptr(rd), Ptr(be.put(go, dt)), D, Ptr(be.put(w, dt)), Ptr(be.put(other, dt)), QD, BT, QD, D, S, NH)
    got = be.get(gin, (BT, QD), dt)
    check(got, portk.matmul_backward_inp(go, w), dt)
    ref = (got.reshape(B, S, NH, 64).astype(np.float64) * other.reshape(B, S, NH, 64)).sum(-1).transpose(0, 2, 1)
    assert np.abs(be.get(rd, (B, NH, S)) - ref).max() <= 1e-4 * max(1.0, np.abs(ref).max())


def test_matmul_rejects_misaligned_leading_dimension_in_bf16(be):
    x, w = be.put(rnd(8, 53), BMC_BF16), be.put(rnd(70, 53), BMC_BF16)
    assert be.call("matmul_forward", BMC_BF16, Ptr(be.zeros(8 * 70, BMC_BF16)), 70, Ptr(x), 53, Ptr(w), None, 0, 8, 53, 70) != 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,C", [(4, 24), (70, 576), (33, 960), (17, 128), (5, 1024)])
def test_rmsnorm_forward_backward(be, dtype, N, C):
    x, w, go, gx0 = rnd(N, C, dtype=dtype), rnd(C), rnd(N, C, dtype=dtype), rnd(N, C, dtype=dtype)
    dx, dw = be.put(x, dtype), be.put(w)
    out, rstd = be.zeros(N * C, dtype), be.zeros(N)
    be.ok("rmsnorm_forward", dtype, Ptr(out), Ptr(rstd), Ptr(dx), Ptr(dw), N, C, 1e-5)
    check(be.get(out, (N, C), dtype), portk.rmsnorm_forward(x, w), dtype)
    gx, gw = be.put(gx0, dtype), be.put(np.full(C, 3.0, np.float32))
    be.ok("rmsnorm_backward", dtype, Ptr(gx), Ptr(gw), 0, Ptr(be.put(go, dtype)), Ptr(dx), Ptr(dw), Ptr(rstd), N, C, 0, N)
    check(be.get(gx, (N, C), dtype), portk.rmsnorm_backward_x(go, w, x, gx0), dtype)  # accumulates into gx
    check(be.get(gw, (C,)), portk.rmsnorm_backward_w(go, x), BMC_F32 if dtype == BMC_F32 else BMC_BF16)  # overwrite form
    # row window + accumulate: gw += sum over the last two rows only
    lo = max(0, N - 2)
    be.ok("rmsnorm_backward", dtype, Ptr(gx), Ptr(gw), 1, Ptr(be.put(go, dtype)), Ptr(dx), Ptr(dw), Ptr(rstd), N, C, lo, N)
    check(be.get(gw, (C,)), portk.rmsnorm_backward_w(go, x) + portk.rmsnorm_backward_w(go[lo:], x[lo:]), dtype if dtype == BMC_BF16 else BMC_F32, 2.0)


def test_rmsnorm_golden_vectors(be, goldens):
    g = goldens  # test/rmsnorm_bwd_test.c: N4 C24
    x, w, go = g["rms_x"].reshape(4, 24), g["rms_w"], g["rms_gout"].reshape(4, 24)
    out, rstd, gx, gw = be.zeros(96), be.zeros(4), be.zeros(96), be.zeros(24)
    be.ok("rmsnorm_forward", BMC_F32, Ptr(out), Ptr(rstd), Ptr(be.put(x)), Ptr(be.put(w)), 4, 24, 1e-5)
    be.ok("rmsnorm_backward", BMC_F32, Ptr(gx), Ptr(gw), 0, Ptr(be.put(go)), Ptr(be.put(x)), Ptr(be.put(w)), Ptr(rstd), 4, 24, 0, 4)
    check(be.get(gx, (4, 24)), g["rms_gx"].reshape(4, 24), BMC_F32, 3)
    check(be.get(gw, (24,)), g["rms_gw"], BMC_F32, 3)


def rope_table(S, HD, theta):
    hd2 = HD // 2
    inv = (np.float32(1.0) / np.power(np.float32(theta), (2 * np.arange(hd2, dtype=np.float32)) / np.float32(HD))).astype(np.float32)
    ang = (np.arange(S, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    return np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,S,NH,NKV,HD,theta", [(1, 5, 4, 2, 8, 1e4), (2, 33, 9, 3, 64, 1e5), (1, 4, 6, 2, 16, 1e4)])
def test_rope_forward_backward_packed_rows(be, dtype, B, S, NH, NKV, HD, theta):
    """Q and K live in one packed row [q heads | k heads | v heads] exactly as the trainer lays them out."""
    ld = (NH + 2 * NKV) * HD
    qkv = rnd(B * S, ld, dtype=dtype)
    es = 2 if dtype == BMC_BF16 else 4
    cs = be.put(rope_table(S, HD, theta))
    for direction in (+1, -1):
        d = be.put(qkv, dtype)
        be.ok("rope", dtype, Ptr(d), ld, Ptr(d, NH * HD * es), ld, Ptr(cs), B * S, S, NH, NKV, HD, direction)
        got = be.get(d, (B, S, ld), dtype)
        for b in range(B):
            q = qkv.reshape(B, S, ld)[b, :, :NH * HD].reshape(S, NH, HD)
            k = qkv.reshape(B, S, ld)[b, :, NH * HD:(NH + NKV) * HD].reshape(S, NKV, HD)
            rq, rk = portk.rope_seq(q, k, theta, direction)
            check(got[b, :, :NH * HD].reshape(S, NH, HD), rq, dtype, 3)
            check(got[b, :, NH * HD:(NH + NKV) * HD].reshape(S, NKV, HD), rk, dtype, 3)
            assert np.array_equal(got[b, :, (NH + NKV) * HD:], qkv.reshape(B, S, ld)[b, :, (NH + NKV) * HD:])  # V untouched


def test_rope_golden_vectors(be, goldens):
    g = goldens  # test/rope_real_test.c: NH9 NKV3 HD64 S4 theta 1e5, backward of random upstream gradients
    S, NH, NKV, HD = 4, 9, 3, 64
    gq, gk = be.put(g["roreal_gout_q"]), be.put(g["roreal_gout_k"])
    be.ok("rope", BMC_F32, Ptr(gq), NH * HD, Ptr(gk), NKV * HD, Ptr(be.put(rope_table(S, HD, 1e5))), S, S, NH, NKV, HD, -1)
    check(be.get(gq, (S * NH * HD,)), g["roreal_gQ"], BMC_F32, 3)
    check(be.get(gk, (S * NKV * HD,)), g["roreal_gK"], BMC_F32, 3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_forward_backward_packed(be, dtype, goldens):
    rows, H = 19, 136
    gu, go = rnd(rows, 2 * H, scale=2.0, dtype=dtype), rnd(rows, H, dtype=dtype)
    es = 2 if dtype == BMC_BF16 else 4
    dgu = be.put(gu, dtype)
    out = be.zeros(rows * H, dtype)
    be.ok("swiglu_forward", dtype, Ptr(out), H, Ptr(dgu), Ptr(dgu, H * es), 2 * H, rows, H)
    check(be.get(out, (rows, H), dtype), portk.swiglu_forward(gu[:, :H], gu[:, H:]), dtype)
    dg = be.zeros(rows * 2 * H, dtype)
    be.ok("swiglu_backward", dtype, Ptr(dg), Ptr(dg, H * es), 2 * H, Ptr(dgu), Ptr(dgu, H * es), 2 * H, Ptr(be.put(go, dtype)), H, rows, H)
    rg, ru = portk.swiglu_backward(gu[:, :H], gu[:, H:], go)
    got = be.get(dg, (rows, 2 * H), dtype)
    check(got[:, :H], rg, dtype)
    check(got[:, H:], ru, dtype)
    if dtype == BMC_F32:  # test/act_bwd_test.c vectors, N=32
        g = goldens
        a, b = be.zeros(32), be.zeros(32)
        be.ok("swiglu_backward", BMC_F32, Ptr(a), Ptr(b), 32, Ptr(be.put(g["swiglu_gate"])), Ptr(be.put(g["swiglu_up"])), 32, Ptr(be.put(g["swiglu_gout"])), 32, 1, 32)
        check(be.get(a, (32,)), g["swiglu_ggate"], BMC_F32, 3)
        check(be.get(b, (32,)), g["swiglu_gup"], BMC_F32, 3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,S,V", [(1, 3, 16), (2, 5, 2048), (1, 2, 49152)])
def test_softmax_cross_entropy(be, dtype, B, S, V):
    logits = rnd(B * S, V, scale=3.0, dtype=dtype)
    targets = RNG.integers(0, V, B * S).astype(np.int32)
    dl, rl, loss = be.put(logits, dtype), be.zeros(B * S), be.zeros(4)
    be.ok("xent", dtype, Ptr(dl), V, Ptr(rl), Ptr(loss), Ptr(be.put(targets)), None, B, S, V, 1.0 / S)
    ref_loss, ref_g = 0.0, []
    for b in range(B):  # per-sequence mean, then batch mean (scheduler.c:1634, trainer.c:528)
        l, g = portk.xent(logits[b * S:(b + 1) * S], targets[b * S:(b + 1) * S])
        ref_loss += l / B
        ref_g.append(g)
    assert abs(float(be.get(loss, (1,))[0]) - ref_loss) < (1e-5 if dtype == BMC_F32 else 1e-4) * max(1.0, ref_loss)
    check(be.get(dl, (B * S, V), dtype), np.concatenate(ref_g), dtype)


def test_xent_golden_vectors(be, goldens):
    g = goldens  # test/xent_bwd_test.c: N3 V10 — V is padded to the 4-float vector width with very negative logits
    lg = np.full((3, 12), -1e30, np.float32)
    lg[:, :10] = g["xent_logits"].reshape(3, 10)
    dl = be.put(lg)
    be.ok("xent", BMC_F32, Ptr(dl), 12, Ptr(be.zeros(3)), Ptr(be.zeros(4)), Ptr(be.put(g["xent_targets"])), None, 1, 3, 12, 1.0 / 3)
    check(be.get(dl, (3, 12))[:, :10], g["xent_glogits"].reshape(3, 10), BMC_F32, 3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_gather_and_scatter(be, dtype, goldens):
    V, D, T = 50, 64, 40
    table, go = rnd(V, D), rnd(T, D, dtype=dtype)
    tokens = RNG.integers(0, 6, T).astype(np.int32)  # heavy repetition: atomics must accumulate
    dtok = be.put(tokens)
    out = be.zeros(T * D, dtype)
    be.ok("embedding_forward", dtype, Ptr(out), Ptr(be.put(table)), Ptr(dtok), T, D, V)
    ref = table[tokens]
    assert np.array_equal(be.get(out, (T, D), dtype), bf16_round(ref) if dtype == BMC_BF16 else ref)
    g0 = rnd(V, D)
    gw = be.put(g0)
    be.ok("embedding_backward", dtype, Ptr(gw), Ptr(be.put(go, dtype)), Ptr(dtok), T, D, V)
    check(be.get(gw, (V, D)), portk.embedding_backward(g0, go, tokens), BMC_F32, 3)
    g = goldens  # test/embed_bwd_test.c: V8 D5 T6 -> D padded to 8 for the 4-float vector width
    gout = np.zeros((6, 8), np.float32)
    gout[:, :5] = g["embed_gout"].reshape(6, 5)
    gw = be.zeros(64)
    be.ok("embedding_backward", BMC_F32, Ptr(gw), Ptr(be.put(gout)), Ptr(be.put(g["embed_tokens"])), 6, 8, 8)
    check(be.get(gw, (8, 8))[:, :5], g["embed_gwte"].reshape(8, 5), BMC_F32, 3)


@pytest.mark.parametrize("grad_dtype", DTYPES)
def test_adamw(be, goldens, grad_dtype):
    import ctypes as C
    n = 4096 + 64
    w, g, m, v = rnd(n), rnd(n, scale=1e-2, dtype=grad_dtype), np.abs(rnd(n, scale=1e-3)), np.abs(rnd(n, scale=1e-5))
    hp = [3e-4, 0.9, 0.95, 1e-8, 0.1, 1 - 0.9 ** 3, 1 - 0.95 ** 3, 1.0 / 16]
    dw, dm, dv, dwb = be.put(w), be.put(m), be.put(v), be.zeros(n, BMC_BF16)
    assert be.lib.bmc_adamw(be.ctx, dw, dwb, be.put(g, grad_dtype), grad_dtype, dm, dv, n, (C.c_float * 8)(*hp)) == 0
    rw, rm, rv = portk.adamw(w, g, m, v, hp)
    check(be.get(dw, (n,)), rw, BMC_F32)
    check(be.get(dm, (n,)), rm, BMC_F32)
    check(be.get(dv, (n,)), rv, BMC_F32)
    assert np.array_equal(be.get(dwb, (n,), BMC_BF16), bf16_round(be.get(dw, (n,))))  # working copy = RNE(master)
    if grad_dtype == BMC_F32:  # test/adamw_test.c vectors (gen_adamw.py: lr 1e-2, wd 0.1, t = 1)
        gd = goldens
        dw, dm, dv = be.put(gd["adamw_w0"]), be.zeros(64), be.zeros(64)
        hp = [1e-2, 0.9, 0.999, 1e-8, 0.1, 0.1, 0.001, 1.0]
        assert be.lib.bmc_adamw(be.ctx, dw, None, be.put(gd["adamw_g"]), BMC_F32, dm, dv, 64, (C.c_float * 8)(*hp)) == 0
        check(be.get(dw, (64,)), gd["adamw_w"], BMC_F32, 3)
        check(be.get(dm, (64,)), gd["adamw_m"], BMC_F32, 3)
        check(be.get(dv, (64,)), gd["adamw_v"], BMC_F32, 3)


# (B, S, NH, NKV, HD): golden shapes, GQA 9/3 and 15/5 at HD 64 (tensor-core kernel in bf16), ragged S, other head dims
ATTN_SHAPES = [(1, 3, 4, 2, 4), (1, 4, 9, 3, 64), (2, 64, 9, 3, 64), (1, 200, 15, 5, 64), (2, 129, 6, 2, 64), (1, 70, 4, 1, 16), (1, 33, 2, 2, 32)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,S,NH,NKV,HD", ATTN_SHAPES)
def test_attention_forward_backward(be, dtype, B, S, NH, NKV, HD):
    if dtype == BMC_BF16 and HD % 8:
        pytest.skip("bf16 rows need 16-byte alignment")
    QD, KV = NH * HD, NKV * HD
    ld = QD + 2 * KV
    es = 2 if dtype == BMC_BF16 else 4
    qkv, go = rnd(B * S, ld, dtype=dtype), rnd(B * S, QD, dtype=dtype)
    scale = 1.0 / np.sqrt(HD)
    d = be.put(qkv, dtype)
    out, lse = be.zeros(B * S * QD, dtype), be.zeros(B * NH * S)
    be.ok("attention_forward", dtype, Ptr(out), QD, Ptr(lse), Ptr(d), ld, Ptr(d, QD * es), Ptr(d, (QD + KV) * es), ld, None, B, S, NH, NKV, HD, float(scale))
    got_o = be.get(out, (B, S, QD), dtype)
    dg = be.zeros(B * S * ld, dtype)
    be.ok("attention_backward", dtype, Ptr(dg), ld, Ptr(dg, QD * es), Ptr(dg, (QD + KV) * es), ld, Ptr(be.put(go, dtype)), QD, Ptr(out), Ptr(lse),
          Ptr(d), ld, Ptr(d, QD * es), Ptr(d, (QD + KV) * es), ld, None, B, S, NH, NKV, HD, float(scale))
    got_g = be.get(dg, (B, S, ld), dtype)
    x = qkv.reshape(B, S, ld)
    for b in range(B):
        Q, K, V = x[b, :, :QD].reshape(S, NH, HD), x[b, :, QD:QD + KV].reshape(S, NKV, HD), x[b, :, QD + KV:].reshape(S, NKV, HD)
        ro = portk.attention_forward(Q, K, V, scale)
        check(got_o[b].reshape(S, NH, HD), ro, dtype)
        rq, rk, rv = portk.attention_backward(go.reshape(B, S, NH, HD)[b], Q, K, V, scale)
        check(got_g[b, :, :QD].reshape(S, NH, HD), rq, dtype, 1.5)
        check(got_g[b, :, QD:QD + KV].reshape(S, NKV, HD), rk, dtype, 1.5)
        check(got_g[b, :, QD + KV:].reshape(S, NKV, HD), rv, dtype, 1.5)


@pytest.mark.parametrize("prefix,NH,NKV,HD,S", [("attn", 4, 2, 4, 3), ("attn_real", 9, 3, 64, 4)])
def test_attention_golden_vectors(be, goldens, prefix, NH, NKV, HD, S):
    g = goldens  # test/attn_fwd_test.c, attn_bwd_test.c, attn_real_test.c
    QD, KV = NH * HD, NKV * HD
    scale = 1.0 / np.sqrt(HD)
    q, k, v = be.put(g[prefix + "_Q"]), be.put(g[prefix + "_K"]), be.put(g[prefix + "_V"])
    out, lse = be.zeros(S * QD), be.zeros(NH * S)
    be.ok("attention_forward", BMC_F32, Ptr(out), QD, Ptr(lse), Ptr(q), QD, Ptr(k), Ptr(v), KV, None, 1, S, NH, NKV, HD, float(scale))
    check(be.get(out, (S * QD,)), g[prefix + "_out"], BMC_F32, 5)
    gq, gk, gv = be.zeros(S * QD), be.zeros(S * KV), be.zeros(S * KV)
    be.ok("attention_backward", BMC_F32, Ptr(gq), QD, Ptr(gk), Ptr(gv), KV, Ptr(be.put(g[prefix + "_gout"])), QD, Ptr(out), Ptr(lse), Ptr(q), QD,
          Ptr(k), Ptr(v), KV, None, 1, S, NH, NKV, HD, float(scale))
    check(be.get(gq, (S * QD,)), g[prefix + "_gQ"], BMC_F32, 5)
    check(be.get(gk, (S * KV,)), g[prefix + "_gK"], BMC_F32, 5)
    check(be.get(gv, (S * KV,)), g[prefix + "_gV"], BMC_F32, 5)


def test_attention_key_query_mask_fp32(be):
    """mask == 0 removes a position both as key and as query (attention_forward_seq_masked, forward.metal:1853)."""
    S, NH, NKV, HD = 24, 4, 2, 16
    QD, KV = NH * HD, NKV * HD
    Q, K, V = rnd(S, NH, HD), rnd(S, NKV, HD), rnd(S, NKV, HD)
    mask = np.ones(S, np.uint8)
    mask[[0, 5, 6, 23]] = 0
    out, lse = be.zeros(S * QD), be.zeros(NH * S)
    be.ok("attention_forward", BMC_F32, Ptr(out), QD, Ptr(lse), Ptr(be.put(Q)), QD, Ptr(be.put(K)), Ptr(be.put(V)), KV, Ptr(be.put(mask)), 1, S, NH, NKV, HD, 0.25)
    got = be.get(out, (S, NH, HD))
    keep = np.flatnonzero(mask)
    ref = portk.attention_forward(Q[keep], K[keep], V[keep], 0.25)  # dropping the masked positions is the same thing
    check(got[keep], ref, BMC_F32, 3)
    assert np.all(got[mask == 0] == 0)


def test_argmax_first_maximum(be):
    for V in (7, 1000, 49152):
        x = RNG.standard_normal(V).astype(np.float32)
        x[RNG.integers(0, V, 3)] = 9.0
        idx = be.zeros(1)
        be.ok("argmax", Ptr(idx), Ptr(be.put(x)), V)
        assert int(be.get(idx, (1,), np_dtype=np.int32)[0]) == portk.argmax(x) == int(np.argmax(x))


def test_seq_prefix_accumulate(be):
    B, n = 3, 1000
    x, carry = rnd(B, n), rnd(n)
    dx, dc = be.put(x), be.put(carry)
    assert be.lib.bmc_seq_prefix_accumulate(be.ctx, BMC_F32, dx, dc, B, n) == 0
    ref = carry[None, :] + np.cumsum(x, axis=0)
    check(be.get(dx, (B, n)), ref, BMC_F32)
    check(be.get(dc, (n,)), ref[-1], BMC_F32)


def test_bounded_wait_reports_instead_of_hanging(be):
    """A wait that cannot complete ends with a status code, not with a hang: bmc_selftest_bounded_wait runs the kernels' own wait
    primitive (2 ms limit in that translation unit) on a barrier nothing arrives at. The status is reported once, then cleared, and
    the context goes on to run a tensor-core GEMM whose result is right and whose own waits all completed (status 0)."""
    assert be.lib.bmc_status(be.ctx) == 0
    assert be.call("selftest_bounded_wait") == 0
    assert be.lib.bmc_sync(be.ctx) == 1999          # the wait ran out and said so
    assert be.lib.bmc_status(be.ctx) == 0           # reported once
    x, w = rnd(128, 64, dtype=BMC_BF16), rnd(64, 64, dtype=BMC_BF16)
    out = be.zeros(128 * 64, BMC_BF16)
    be.ok("matmul_forward", BMC_BF16, Ptr(out), 64, Ptr(be.put(x, BMC_BF16)), 64, Ptr(be.put(w, BMC_BF16)), None, 0, 128, 64, 64)
    check(be.get(out, (128, 64), BMC_BF16), portk.matmul_forward(x, w), BMC_BF16)
    assert be.lib.bmc_status(be.ctx) == 0
