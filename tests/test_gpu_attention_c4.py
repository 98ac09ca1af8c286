"""Isolated causal GQA flash attention, forward + backward, bf16, 15 query heads / 5 KV heads, head_dim 64, at
seq in {512, 2048, 8192}: O, dQ, dK, dV against the reference's attention arithmetic
(attention_forward_seq / attention_backward, src/kernels/forward.metal:1811, src/kernels/backward.metal:665, restated in
oracle/bm_oracle.c with the per-thread array bound lifted). Q, K, V, dO ~ N(0, 1) by seed, rounded to bf16 for both sides.
S = 512 (batch 2 and the full batch 16, three entries checked) and 2048: the CPU oracle on whole sequences. S = 8192: committed
outputs of the CPU oracle for one KV group (O, dQ, dK, dV at every 32nd row plus tensor norms), a forward prefix computed live, and
the whole problem against the exact-softmax fp32 GPU kernel, which the smaller cases tie to the oracle. Tolerance: 2e-2 relative,
cosine > 0.999."""
import numpy as np
import pytest

import oracle_check as oc
import portk
from bmcapi import BMC_BF16, BMC_F32, Backend, Ptr, bf16_round

pytestmark = pytest.mark.gpu
NH, NKV, HD = 15, 5, 64
QD, KV = NH * HD, NKV * HD
LD = QD + 2 * KV
SCALE = 1.0 / np.sqrt(HD)


@pytest.fixture(scope="module")
def be(product):
    b = Backend(product)
    yield b
    b.close()


def run_gpu(be, dtype, qkv, go, B, S):
    es = 2 if dtype == BMC_BF16 else 4
    d, dgo = be.put(qkv, dtype), be.put(go, dtype)
    out, lse, dg = be.zeros(B * S * QD, dtype), be.zeros(B * NH * S), be.zeros(B * S * LD, dtype)
    be.ok("attention_forward", dtype, Ptr(out), QD, Ptr(lse), Ptr(d), LD, Ptr(d, QD * es), Ptr(d, (QD + KV) * es), LD, None, B, S, NH, NKV, HD, float(SCALE))
    be.ok("attention_backward", dtype, Ptr(dg), LD, Ptr(dg, QD * es), Ptr(dg, (QD + KV) * es), LD, Ptr(dgo), QD, Ptr(out), Ptr(lse), Ptr(d), LD,
          Ptr(d, QD * es), Ptr(d, (QD + KV) * es), LD, None, B, S, NH, NKV, HD, float(SCALE))
    return be.get(out, (B, S, QD), dtype), be.get(dg, (B, S, LD), dtype)


def rope_table(S):
    inv = (np.float32(1.0) / np.power(np.float32(1e5), (2 * np.arange(HD // 2, dtype=np.float32)) / np.float32(HD))).astype(np.float32)
    ang = (np.arange(S, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    return np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)


def close(got, ref, what):
    assert oc.rel_err(got, ref) < 2e-2, (what, oc.rel_err(got, ref))
    assert oc.cosine(got.ravel(), ref.ravel()) > 0.999, what


@pytest.mark.parametrize("S,B", [(512, 2), (2048, 1), (512, 16)])
def test_flash_attention_against_the_oracle(be, S, B):
    rng = np.random.default_rng(S)
    qkv = bf16_round(rng.standard_normal((B * S, LD)).astype(np.float32))
    go = bf16_round(rng.standard_normal((B * S, QD)).astype(np.float32))
    out, dg = run_gpu(be, BMC_BF16, qkv, go, B, S)
    x = qkv.reshape(B, S, LD)
    for b in (range(B) if B <= 2 else (0, B // 2, B - 1)):   # the full batch of 16 runs on the GPU; the CPU oracle checks three entries
        Q, K, V = x[b, :, :QD].reshape(S, NH, HD), x[b, :, QD:QD + KV].reshape(S, NKV, HD), x[b, :, QD + KV:].reshape(S, NKV, HD)
        close(out[b].reshape(S, NH, HD), portk.attention_forward(Q, K, V, SCALE), "O")
        gq, gk, gv = portk.attention_backward(go.reshape(B, S, NH, HD)[b], Q, K, V, SCALE)
        close(dg[b, :, :QD].reshape(S, NH, HD), gq, "dQ")
        close(dg[b, :, QD:QD + KV].reshape(S, NKV, HD), gk, "dK")
        close(dg[b, :, QD + KV:].reshape(S, NKV, HD), gv, "dV")


def test_flash_attention_8192(be):
    S, B = 8192, 1
    rng = np.random.default_rng(8192)
    qkv = bf16_round(rng.standard_normal((B * S, LD)).astype(np.float32))
    go = bf16_round(rng.standard_normal((B * S, QD)).astype(np.float32))
    out, dg = run_gpu(be, BMC_BF16, qkv, go, B, S)
    # forward prefix against the CPU oracle
    n = 768
    x = qkv.reshape(S, LD)
    Q, K, V = x[:n, :QD].reshape(n, NH, HD), x[:n, QD:QD + KV].reshape(n, NKV, HD), x[:n, QD + KV:].reshape(n, NKV, HD)
    close(out[0, :n].reshape(n, NH, HD), portk.attention_forward(Q, K, V, SCALE), "O prefix")
    # whole problem against the exact fp32 kernel on the same (bf16-rounded) inputs
    out32, dg32 = run_gpu(be, BMC_F32, qkv, go, B, S)
    close(out, out32, "O")
    close(dg[..., :QD], dg32[..., :QD], "dQ")
    close(dg[..., QD:QD + KV], dg32[..., QD:QD + KV], "dK")
    close(dg[..., QD + KV:], dg32[..., QD + KV:], "dV")
    assert np.isfinite(dg).all()


def test_flash_attention_8192_against_the_committed_oracle_outputs(be):
    """S = 8192 against the CPU oracle itself: tests/golden/oracle_attention_s8192_group.npz holds O, dQ, dK, dV of ONE KV group (KV
    head 0 and query heads 0-2 of one sequence) computed by the plain-C restatement of the reference kernels on seeded inputs
    (tests/golden/make_golden.py, c4_group_case). The GPU runs the whole 15 / 5-head problem with that group embedded."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    from make_golden import c4_group_inputs
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_attention_s8192_group.npz"))
    S = int(g["S"])
    q, k, v, go3 = c4_group_inputs(S)
    assert abs(float(np.float64(q.sum()) + k.sum() + v.sum() + go3.sum()) - float(g["checksum"])) < 1e-6   # same seeded inputs as the fixture
    rng = np.random.default_rng(1)
    qkv = bf16_round(rng.standard_normal((S, LD)).astype(np.float32))
    go = bf16_round(rng.standard_normal((S, QD)).astype(np.float32))
    qkv[:, :3 * HD], qkv[:, QD:QD + HD], qkv[:, QD + KV:QD + KV + HD] = q.reshape(S, -1), k.reshape(S, -1), v.reshape(S, -1)
    go[:, :3 * HD] = go3.reshape(S, -1)
    out, dg = run_gpu(be, BMC_BF16, qkv, go, 1, S)
    rows = g["rows"]
    close(out[0][rows, :3 * HD].reshape(-1, 3, HD), g["o"], "O")
    close(dg[0][rows, :3 * HD].reshape(-1, 3, HD), g["gq"], "dQ")
    close(dg[0][rows, QD:QD + HD].reshape(-1, 1, HD), g["gk"], "dK")
    close(dg[0][rows, QD + KV:QD + KV + HD].reshape(-1, 1, HD), g["gv"], "dV")
    got_norms = [np.linalg.norm(t.astype(np.float64)) for t in (out[0][:, :3 * HD], dg[0][:, :3 * HD], dg[0][:, QD:QD + HD], dg[0][:, QD + KV:QD + KV + HD])]
    assert np.allclose(got_norms, g["norms"], rtol=2e-2)


def test_exact_kernel_matches_oracle_at_2048(be):
    """Ties the fp32 GPU kernel used as the 8192 cross-check to the CPU oracle (one KV group, S = 2048)."""
    S = 2048
    rng = np.random.default_rng(5)
    qkv = rng.standard_normal((S, LD)).astype(np.float32)
    go = rng.standard_normal((S, QD)).astype(np.float32)
    out, dg = run_gpu(be, BMC_F32, qkv, go, 1, S)
    Q, K, V = qkv[:, :QD].reshape(S, NH, HD), qkv[:, QD:QD + KV].reshape(S, NKV, HD), qkv[:, QD + KV:].reshape(S, NKV, HD)
    ref_o = portk.attention_forward(Q, K, V, SCALE)
    assert oc.rel_err(out[0].reshape(S, NH, HD), ref_o) < 1e-5
    gq, gk, gv = portk.attention_backward(go.reshape(S, NH, HD), Q, K, V, SCALE)
    assert oc.rel_err(dg[0, :, :QD].reshape(S, NH, HD), gq) < 2e-5
    assert oc.rel_err(dg[0, :, QD:QD + KV].reshape(S, NKV, HD), gk) < 2e-5
    assert oc.rel_err(dg[0, :, QD + KV:].reshape(S, NKV, HD), gv) < 2e-5


@pytest.mark.parametrize("S,B", [(384, 2), (200, 2), (2048, 1)])
def test_backward_with_row_sums_supplied_and_rope_backward_folded_in(be, S, B):
    """bmc_attention_backward_fused with delta from outside and the rotation table = bmc_attention_backward followed by the
    backward rotation of dQ and dK; V's gradient is the same in both."""
    rng = np.random.default_rng(S + 1)
    dt, es = BMC_BF16, 2
    qkv = bf16_round(rng.standard_normal((B * S, LD)).astype(np.float32))
    go = bf16_round(rng.standard_normal((B * S, QD)).astype(np.float32))
    d, dgo = be.put(qkv, dt), be.put(go, dt)
    out, lse = be.zeros(B * S * QD, dt), be.zeros(B * NH * S)
    args_f = (Ptr(out), QD, Ptr(lse), Ptr(d), LD, Ptr(d, QD * es), Ptr(d, (QD + KV) * es), LD, None, B, S, NH, NKV, HD, float(SCALE))
    be.ok("attention_forward", dt, *args_f)
    o = be.get(out, (B, S, NH, HD), dt)
    delta = (o.astype(np.float64) * go.reshape(B, S, NH, HD)).sum(-1).transpose(0, 2, 1).astype(np.float32)
    cs = be.put(rope_table(S))
    ref, got = be.zeros(B * S * LD, dt), be.zeros(B * S * LD, dt)
    tail = (Ptr(dgo), QD, Ptr(out), Ptr(lse), Ptr(d), LD, Ptr(d, QD * es), Ptr(d, (QD + KV) * es), LD, None)
    be.ok("attention_backward", dt, Ptr(ref), LD, Ptr(ref, QD * es), Ptr(ref, (QD + KV) * es), LD, *tail, B, S, NH, NKV, HD, float(SCALE))
    unrotated = be.get(ref, (B, S, LD), dt)
    be.ok("attention_backward_fused", dt, Ptr(got), LD, Ptr(got, QD * es), Ptr(got, (QD + KV) * es), LD, *tail, Ptr(be.put(delta)), Ptr(cs),
          B, S, NH, NKV, HD, float(SCALE))
    g = be.get(got, (B, S, LD), dt)
    for b in range(B):
        rq, rk = portk.rope_seq(unrotated[b, :, :QD].reshape(S, NH, HD), unrotated[b, :, QD:QD + KV].reshape(S, NKV, HD), 1e5, -1)
        # the unrotated reference was rounded to bf16 before the rotation, the fused path rotates fp32 values: two roundings apart
        assert oc.rel_err(g[b, :, :QD].reshape(S, NH, HD), rq) < 1e-2
        assert oc.rel_err(g[b, :, QD:QD + KV].reshape(S, NKV, HD), rk) < 1e-2
    assert oc.rel_err(g[..., QD + KV:], unrotated[..., QD + KV:]) < 1e-3


@pytest.mark.parametrize("S,B", [(300, 2), (1024, 1)])
def test_padding_mask_on_the_tensor_core_kernels(be, S, B):
    """A position whose mask byte is 0 is neither key nor query (attention_forward_seq_masked, src/kernels/forward.metal:1853;
    attention_backward_masked, src/kernels/backward.metal:738): the bf16 tensor-core kernels against the exact fp32 kernel, which
    the masked training-step tests tie to the reference. Padding at the end of one sequence, a hole inside another."""
    rng = np.random.default_rng(S)
    qkv = bf16_round(rng.standard_normal((B * S, LD)).astype(np.float32))
    go = bf16_round(rng.standard_normal((B * S, QD)).astype(np.float32))
    mask = np.ones((B, S), np.uint8)
    mask[0, S - 70:] = 0
    mask[B - 1, 40:170] = 0
    mask[B - 1, 5] = 0
    dm = be.put(mask.reshape(-1))
    res = {}
    for dtype in (BMC_BF16, BMC_F32):
        es = 2 if dtype == BMC_BF16 else 4
        d, dgo = be.put(qkv, dtype), be.put(go, dtype)
        out, lse, dg = be.zeros(B * S * QD, dtype), be.zeros(B * NH * S), be.zeros(B * S * LD, dtype)
        be.ok("attention_forward", dtype, Ptr(out), QD, Ptr(lse), Ptr(d), LD, Ptr(d, QD * es), Ptr(d, (QD + KV) * es), LD, Ptr(dm), B, S, NH, NKV, HD, float(SCALE))
        be.ok("attention_backward", dtype, Ptr(dg), LD, Ptr(dg, QD * es), Ptr(dg, (QD + KV) * es), LD, Ptr(dgo), QD, Ptr(out), Ptr(lse), Ptr(d), LD,
              Ptr(d, QD * es), Ptr(d, (QD + KV) * es), LD, Ptr(dm), B, S, NH, NKV, HD, float(SCALE))
        res[dtype] = (be.get(out, (B, S, QD), dtype), be.get(dg, (B, S, LD), dtype))
    (o16, g16), (o32, g32) = res[BMC_BF16], res[BMC_F32]
    off = mask == 0
    assert not o16[off].any() and not g16[off][:, :QD].any()            # masked queries: zero output, zero dQ
    assert not g16[off][:, QD:].any()                                   # masked keys: zero dK and dV
    close(o16, o32, "O")
    close(g16[..., :QD], g32[..., :QD], "dQ")
    close(g16[..., QD:QD + KV], g32[..., QD:QD + KV], "dK")
    close(g16[..., QD + KV:], g32[..., QD + KV:], "dV")
