"""Inference session on the GPU (prefill + token-by-token decode with a KV cache; fp32 / bf16 / Q8 weights) against the
reference session's committed logits and greedy continuations (tests/golden/ref_decode_*.npz) and, live, against the
plain-C oracle. Activations are fp32 in every mode, so logits must agree within 1e-4 of the largest logit (summation order
is the only difference); greedy token ids must be identical wherever the reference's top-2 margin exceeds that bound."""
import ctypes as C
import os

import numpy as np
import pytest

import bmapi
import oracle_check as oc
from test_oracle_pins import DECODE_GOLDENS, DECODE_GOLDENS_SAMPLED, decode_case

pytestmark = pytest.mark.gpu
F32, BF16 = bmapi.BM_PRECISION_FP32, bmapi.BM_PRECISION_BF16
IDS = [os.path.basename(p)[11:-4] for p in DECODE_GOLDENS]
TOL = 1e-4


def close(x, ref):
    return np.abs(x - ref).max() <= TOL * np.abs(ref).max()


@pytest.mark.parametrize("path", DECODE_GOLDENS, ids=IDS)
def test_step_logits_match_reference_session(product, path):
    g, a, w = decode_case(path)
    s = oc.LibSession(product, "gpu", a, w, int(g["precision"]), int(g["quant"]))
    for i, t in enumerate(g["prompt"]):
        lg = s.step(t)
        if i >= 1:
            assert close(lg, g["logits"][i - 1]), (i, np.abs(lg - g["logits"][i - 1]).max())
    # the prompt in one pass (tensor-core prefill, test/prefill_test.c): same logits within the bound
    s.reset()
    lf = s.forward(g["prompt"])
    assert close(lf, g["logits"][-1]) and close(lf, lg), np.abs(lf - lg).max()
    # and token by token through bm_forward (steps after the first replay a captured graph): the same bits as bm_step
    os.environ["BM_NO_PREFILL"] = "1"
    try:
        s.reset()
        lf = s.forward(g["prompt"])
    finally:
        del os.environ["BM_NO_PREFILL"]
    assert np.array_equal(lf, lg)
    # greedy continuation through the public API
    out = []
    for _ in range(len(g["greedy"])):
        out.append(int(np.argmax(lg)))
        lg = s.step(out[-1])
    s.close()
    safe = g["margin"] > 10 * TOL * np.abs(g["logits"]).max()
    n = len(out) if safe.all() else int(np.argmin(safe)) + 1
    assert out[:n] == list(g["greedy"][:n])


# Logit bounds for the 32-layer model, as a fraction of the largest logit. Token-by-token decode does fp32 arithmetic in another
# summation order. The one-pass prefill runs its GEMMs on the tensor cores with operands split into two bf16 terms (16 mantissa
# bits, about 2^-17 per product), in the projections and in the attention, and 32 layers whose matrices were scaled up by 8 for the
# fixture amplify that; the split-K partial sums of those GEMMs also land in an order that changes from run to run. Measured
# 0.7e-3 to 1.1e-3 over repeated runs: 1.5e-3 there.
TOL_360M = {"steps": 3e-4, "prefill": 1.5e-3}


@pytest.mark.parametrize("mode", ["steps", "prefill"])
@pytest.mark.parametrize("path", DECODE_GOLDENS_SAMPLED, ids=[os.path.basename(p)[11:-4] for p in DECODE_GOLDENS_SAMPLED])
def test_smollm2_360m_q8_session_matches_reference_session(product, path, mode):
    """The benchmarked inference model: SmolLM2-360M with Q8 layer matrices, a 64-token prompt (token by token, or in one prefill
    pass) and 16 greedy tokens, against the reference session's recorded outputs (sampled logits, its eight largest logits and its
    greedy ids)."""
    g, a, w = decode_case(path)
    s = oc.LibSession(product, "gpu", a, w, int(g["precision"]), int(g["quant"]))
    idx, top_ids = g["sample_idx"], g["top_ids"]
    if mode == "steps":
        os.environ["BM_NO_PREFILL"] = "1"
    try:
        lg = s.forward(g["prompt"])
    finally:
        os.environ.pop("BM_NO_PREFILL", None)
    out, worst = [], 0.0
    for k in range(len(g["greedy"])):
        bound = TOL_360M[mode] * float(g["logit_absmax"][k])
        err = max(np.abs(lg[idx] - g["sample_logits"][k]).max(), np.abs(lg[top_ids[k]] - g["top_logits"][k]).max())
        worst = max(worst, err / float(g["logit_absmax"][k]))
        assert err <= bound, (k, err, bound)
        out.append(int(np.argmax(lg)))
        if float(g["margin"][k]) > 10 * bound:   # else a near-tie in the reference: either id is right
            assert out[-1] == int(g["greedy"][k]), (k, out, g["greedy"])
        lg = s.step(int(g["greedy"][k]))   # continue on the reference's own sequence, so that every later step stays comparable
    s.close()
    print(f"360m decode {os.path.basename(path)} {mode}: worst logit error {worst:.2e} of the largest logit")
    assert sum(float(m) > 10 * TOL_360M[mode] * float(x) for m, x in zip(g["margin"], g["logit_absmax"])) >= 10   # most of the 16 steps are unambiguous


@pytest.mark.parametrize("path", DECODE_GOLDENS, ids=IDS)
def test_device_side_greedy_loop_matches_reference(product, path):
    """bmx_session_generate_greedy never returns to the host between tokens; ids must equal the reference's."""
    g, a, w = decode_case(path)
    s = oc.LibSession(product, "gpu", a, w, int(g["precision"]), int(g["quant"]))
    prompt = np.ascontiguousarray(g["prompt"], np.int32)
    n_new = len(g["greedy"])
    out = np.zeros(n_new, np.int32)
    assert product.bmx_session_generate_greedy(s.sess, bmapi.as_int_ptr(prompt), len(prompt), n_new, bmapi.as_int_ptr(out)) == 0
    assert product.bmx_session_position(s.sess) == len(prompt) + n_new - 1
    s.close()
    assert list(out) == list(g["greedy"])


def _batched(product, a, w, precision, quant, NB, MS):
    sa = bmapi.make_arch({k: getattr(a, k) for k in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size")} | {"head_dim": a.head_dim})
    sa.precision = precision
    path = f"/tmp/bm_dec_{os.getpid()}.bin"
    bmapi.write_bin_checkpoint(path, sa, w)
    ctx = product.bm_create(bmapi.BM_DEVICE_METAL)
    model = product.bm_create_model(ctx, C.byref(sa))
    product.bm_load_weights(model, path.encode())
    os.unlink(path)
    assert product.bmx_model_set_quant(model, quant) == 0
    sess = product.bmx_create_session_batched(ctx, model, NB, MS)
    assert sess
    return ctx, model, sess


@pytest.mark.parametrize("precision,quant,NB", [(F32, 0, 3), (BF16, 8, 11), (BF16, 0, 8), (F32, 8, 1), (F32, 8, 5), (F32, 0, 16), (BF16, 8, 64), (BF16, 4, 11)])
def test_batched_sequences_equal_single_sequences(product, precision, quant, NB):
    """NB sequences decoded in lock step give, per sequence, exactly the ids and logits of that sequence decoded alone."""
    a = bmapi.make_arch("gqa")
    w = bmapi.make_weights(a, layer_scale=8.0)
    n_prompt, n_new = 9, 7
    prompts = np.stack([bmapi.lcg_tokens(n_prompt, a.vocab_size, seed=100 + b) for b in range(NB)]).astype(np.int32)
    ctx, model, sess = _batched(product, a, w, precision, quant, NB, 32)
    out = np.zeros((NB, n_new), np.int32)
    assert product.bmx_session_generate_greedy(sess, bmapi.as_int_ptr(prompts), n_prompt, n_new, bmapi.as_int_ptr(out)) == 0
    lg = np.ctypeslib.as_array(product.bmx_session_logits(sess), shape=(NB, a.vocab_size)).copy()
    product.bm_destroy_session(sess)
    product.bm_destroy_model(model)
    product.bm_destroy(ctx)
    bound = 10 * TOL
    for b in range(NB):
        dec = oc.PortDecoder(a, w, precision, quant, 32)
        l1 = dec.forward(prompts[b])
        for i in range(n_new):
            top = np.argsort(l1)[-2:]
            if l1[top[1]] - l1[top[0]] <= bound * np.abs(l1).max():
                break                                   # a near-tie: either choice is right, and the sequences part ways
            assert int(top[1]) == int(out[b, i]), (b, i)
            if i + 1 < n_new:
                l1 = dec.step(int(out[b, i]))
        else:
            assert close(lg[b], l1), b
        dec.close()


@pytest.mark.parametrize("NB", [1, 16])
def test_bf16_kv_cache_session_tracks_the_fp32_one(product, NB):
    """bmx_create_session_kv(..., kv_bf16=1): keys and values are rounded to bf16 on their way into the cache (prefill scatter and
    decode store). Logits stay within 2e-2 of the largest logit of the fp32-cache session on the same prompts, and the session
    reports two bytes per cache element."""
    a = bmapi.make_arch("gqa")
    w = bmapi.make_weights(a, layer_scale=8.0)
    n_prompt, n_new = 12, 6
    prompts = np.stack([bmapi.lcg_tokens(n_prompt, a.vocab_size, seed=300 + b) for b in range(NB)]).astype(np.int32)
    res = {}
    for kv in (0, 1):
        ctx, model, sess = _batched(product, a, w, F32, 0, NB, 32)
        product.bm_destroy_session(sess)
        sess = product.bmx_create_session_kv(ctx, model, NB, 32, kv)
        assert sess and product.bmx_session_kv_bytes_per_element(sess) == (2 if kv else 4)
        out = np.zeros((NB, 1), np.int32)
        assert product.bmx_session_generate_greedy(sess, bmapi.as_int_ptr(prompts), n_prompt, 1, bmapi.as_int_ptr(out)) == 0
        steps = [np.ctypeslib.as_array(product.bmx_session_logits(sess), shape=(NB, a.vocab_size)).copy()]
        tok = prompts[:, :1].copy()
        for i in range(n_new):   # the same forced tokens in both sessions, so that the logits stay comparable
            tok = np.ascontiguousarray(prompts[:, i + 1:i + 2])
            assert product.bmx_session_generate_greedy(sess, bmapi.as_int_ptr(tok), 1, 1, bmapi.as_int_ptr(out)) == 0
            steps.append(np.ctypeslib.as_array(product.bmx_session_logits(sess), shape=(NB, a.vocab_size)).copy())
        res[kv] = np.stack(steps)
        product.bm_destroy_session(sess)
        product.bm_destroy_model(model)
        product.bm_destroy(ctx)
    err = np.abs(res[1] - res[0]).max() / np.abs(res[0]).max()
    assert 0 < err < 2e-2, err   # not identical (the cache really is bf16), and close


def test_reset_replays_and_cache_overflow_is_refused(product):
    a = bmapi.make_arch("tiny")
    w = bmapi.make_weights(a, layer_scale=8.0)
    ctx, model, sess = _batched(product, a, w, F32, 8, 1, 8)
    V = a.vocab_size
    toks = bmapi.lcg_tokens(8, V, seed=9)
    first = [np.ctypeslib.as_array(product.bm_step(sess, int(t)), shape=(V,)).copy() for t in toks]
    assert not product.bm_step(sess, 1)          # position 8 does not fit a cache of 8
    assert not product.bm_step(sess, V)          # token id out of range
    product.bm_reset_session(sess)
    again = [np.ctypeslib.as_array(product.bm_step(sess, int(t)), shape=(V,)).copy() for t in toks]
    assert all(np.array_equal(x, y) for x, y in zip(first, again))
    product.bm_destroy_session(sess)
    product.bm_destroy_model(model)
    product.bm_destroy(ctx)


def test_135m_q8_decode_against_oracle(product):
    """The 135M-parameter family member, bf16 head + Q8 layers (the decode configuration), a few tokens against the plain-C oracle."""
    a = bmapi.make_arch("smollm2-135m")
    w = bmapi.make_weights(a, layer_scale=2.0)
    toks = bmapi.lcg_tokens(5, a.vocab_size, seed=3)
    s = oc.LibSession(product, "gpu", a, w, BF16, 8)
    dec = oc.PortDecoder(a, w, BF16, 8, 16)
    for t in toks:
        lg, lo = s.step(t), dec.step(t)
        assert close(lg, lo), np.abs(lg - lo).max()
    assert int(np.argmax(lg)) == int(np.argmax(lo))
    s.close()
    dec.close()


@pytest.mark.parametrize("quant", [0, 4])
def test_session_after_adapter_merge_against_oracle(product, quant, tmp_path):
    """bm_load_weights -> bm_load_adapter -> session: the logits are those of the plain-C oracle on base weights + (alpha / rank) * B * A
    (merged here with numpy in the reference's summation order), and differ from the base model's."""
    a = bmapi.make_arch("gqa")
    w = bmapi.make_weights(a, layer_scale=8.0)
    rank, alpha = 4, 8.0
    rng = np.random.default_rng(31)
    shapes = dict(bmapi.weight_shapes(a))
    entries, merged = [], {k: v.copy() for k, v in w.items()}
    for layer, tgt in [(0, "q"), (0, "v"), (1, "o"), (1, "gate"), (0, "down")]:
        key = bmapi.ADAPTER_WEIGHT_KEY[tgt]
        oc_, c = shapes[key][1:]
        A = rng.standard_normal((rank, c), dtype=np.float32) * np.float32(0.1)
        B = rng.standard_normal((oc_, rank), dtype=np.float32) * np.float32(0.1)
        entries.append((layer, tgt, A, B))
        acc = np.zeros((oc_, c), np.float32)
        for k in range(rank):
            acc += B[:, k:k + 1] * A[k:k + 1, :]
        merged[key][layer] += (np.float32(alpha) / np.float32(rank)) * acc
    base, adp = str(tmp_path / "base.bin"), str(tmp_path / "a.bmlora")
    bmapi.write_bin_checkpoint(base, a, w)
    bmapi.write_adapter_file(adp, a, rank, alpha, entries)
    ctx = product.bm_create(bmapi.BM_DEVICE_METAL)
    model = product.bm_create_model(ctx, C.byref(a))
    product.bm_load_weights(model, base.encode())
    assert product.bm_load_adapter(model, adp.encode()) == 0
    assert product.bmx_model_set_quant(model, quant) == 0
    sess = product.bm_create_session(ctx, model)
    assert sess
    dec, plain = oc.PortDecoder(a, merged, F32, quant, 16), oc.PortDecoder(a, w, F32, quant, 16)
    V = a.vocab_size
    for t in bmapi.lcg_tokens(6, V, seed=5):
        lg = np.ctypeslib.as_array(product.bm_step(sess, int(t)), shape=(V,)).copy()
        lo, lb = dec.step(t), plain.step(t)
        assert close(lg, lo), np.abs(lg - lo).max()
    assert np.abs(lo - lb).max() > 100 * TOL * np.abs(lo).max()   # the adapter changed the model
    dec.close(); plain.close()
    product.bm_destroy_session(sess)
    product.bm_destroy_model(model)
    product.bm_destroy(ctx)


# ---- kernels of the inference path through the extern "C" backend ABI ----------------------------------------------------
import portk  # noqa: E402
from bmcapi import BMC_BF16, BMC_F32, Backend, Ptr, bf16_round, f32_to_bf16_bits  # noqa: E402

RNG = np.random.default_rng(77)


@pytest.fixture(scope="module")
def be(product):
    b = Backend(product)
    yield b
    b.close()


def rndf(*shape, scale=1.0):
    return (RNG.standard_normal(shape) * scale).astype(np.float32)


@pytest.mark.parametrize("NB,T,NH,NKV", [(2, 200, 6, 2), (1, 64, 3, 1), (3, 65, 2, 2), (1, 513, 15, 5)])
def test_prefill_attention_fp32(be, NB, T, NH, NKV):
    HD = 64
    QD, KV = NH * HD, NKV * HD
    ld = QD + 2 * KV
    qkv = rndf(NB * T, ld)
    d = be.put(qkv)
    out = be.zeros(NB * T * QD)
    be.ok("prefill_attention", Ptr(out), QD, Ptr(d), ld, Ptr(d, QD * 4), Ptr(d, (QD + KV) * 4), ld, NB, T, NH, NKV, HD, 0.125)
    got = be.get(out, (NB, T, NH, HD))
    x = qkv.reshape(NB, T, ld)
    for b in range(NB):
        ref = portk.attention_forward(x[b, :, :QD].reshape(T, NH, HD), x[b, :, QD:QD + KV].reshape(T, NKV, HD),
                                      x[b, :, QD + KV:].reshape(T, NKV, HD), 0.125)
        assert oc.rel_err(got[b], ref) < 1e-5


def _q8(w):
    q = np.zeros(w.size, np.int8)
    sc = np.zeros(w.size // 32, np.float32)
    lib = oc.load_port()
    assert lib.orc_quantize_q8(oc.fptr(np.ascontiguousarray(w)), q.ctypes.data, oc.fptr(sc), w.size) == w.size // 32
    return q.reshape(w.shape), sc.reshape(w.shape[0], -1)


def _q4(w):
    """Q4 codes from the oracle's quantiser, packed as the reference packs them: element 2j low, 2j+1 high nibble of byte j. The
    quantiser never produces -8 (|w| / scale <= 7), the format holds it: a few codes are set to the extremes by hand."""
    q = np.zeros(w.size, np.int8)
    sc = np.zeros(w.size // 32, np.float32)
    assert oc.load_port().orc_quantize_q4(oc.fptr(np.ascontiguousarray(w)), q.ctypes.data, oc.fptr(sc), w.size) == w.size // 32
    q[:8] = [-8, 7, -1, 0, 1, -8, -7, 7]
    q[-3:] = [-8, 7, -8]
    u = q.view(np.uint8).reshape(w.shape[0], -1, 2) & 0x0F
    packed = np.ascontiguousarray((u[:, :, 0] | (u[:, :, 1] << 4)).astype(np.uint8))
    return q.reshape(w.shape), sc.reshape(w.shape[0], -1), packed


@pytest.mark.parametrize("wtype", [0, 1, 2, 3])
@pytest.mark.parametrize("NB,C,OC,prologue", [(1, 960, 1600, 0), (1, 960, 5120, 1), (2, 2560, 960, 2), (3, 576, 77, 1), (5, 384, 200, 0), (17, 1024, 130, 0)])
def test_decode_gemv_all_weight_types(be, wtype, NB, C, OC, prologue):
    """out = operand(x) W^T + residual, Q8 / bf16 / fp32 / packed Q4 weights, plain / RMSNorm / SwiGLU operand, single-sequence and
    batched kernels."""
    if prologue and NB >= 4:
        pytest.skip("prologues exist in the single-sequence kernel only")
    w = rndf(OC, C, scale=0.05)
    x = rndf(NB, 2 * C if prologue == 2 else C)
    res = rndf(NB, OC)
    lnw = (1.0 + 0.1 * rndf(C)).astype(np.float32)
    if wtype == 0:
        q, sc = _q8(w)
        weff = q.astype(np.float32) * np.repeat(sc, 32, axis=1)
        dw, dsc = be.put(q.view(np.uint8)), be.put(sc)
    elif wtype == 1:
        weff = bf16_round(w)
        hb = f32_to_bf16_bits(w)
        dw = be.alloc(hb.nbytes)
        assert be.lib.bmc_upload(be.ctx, dw, hb.ctypes.data, hb.nbytes) == 0
        dsc = None
    elif wtype == 3:
        q, sc, packed = _q4(w)
        assert q.min() == -8 and q.max() == 7 and packed.shape == (OC, C // 2)
        weff = q.astype(np.float32) * np.repeat(sc, 32, axis=1)
        dw, dsc = be.put(packed), be.put(sc)
    else:
        weff, dw, dsc = w, be.put(w), None
    if prologue == 1:
        op = x / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5).astype(np.float32) * lnw
    elif prologue == 2:
        g, u = x[:, :C], x[:, C:]
        op = g / (1.0 + np.exp(-g)) * u
    else:
        op = x
    ref = (op.astype(np.float64) @ weff.astype(np.float64).T + res).astype(np.float32)
    out = be.zeros(NB * OC)
    be.ok("decode_gemv_fused", Ptr(out), OC, Ptr(be.put(x)), x.shape[1], wtype, Ptr(dw), Ptr(dsc) if dsc else None, Ptr(be.put(res)), OC,
          prologue, Ptr(be.put(lnw)), 1e-5, NB, C, OC)
    assert oc.rel_err(be.get(out, (NB, OC)), ref) < 1e-5


@pytest.mark.parametrize("rows,C,OC,parts,mode", [(64, 960, 1600, 3, 1), (8, 960, 960, 2, 0), (300, 2560, 960, 3, 2), (33, 384, 2048, 2, 1)])
def test_split_bf16_gemm_matches_fp32_product(be, rows, C, OC, parts, mode):
    """bmc_decode_prep + bmc_decode_gemm: the tensor-core product of the bf16 hi/lo split operands reproduces the fp32 product."""
    w = rndf(OC, C, scale=0.05)
    if parts == 2:
        w = bf16_round(w)
    hi = bf16_round(w)
    lo = bf16_round(w - hi)
    wx = np.concatenate([hi, hi, lo] if parts == 3 else [hi, hi], axis=1)
    hb = f32_to_bf16_bits(wx)
    dwx = be.alloc(hb.nbytes)
    assert be.lib.bmc_upload(be.ctx, dwx, hb.ctypes.data, hb.nbytes) == 0
    x = rndf(rows, 2 * C if mode == 2 else C)
    res = rndf(rows, OC)
    lnw = (1.0 + 0.1 * rndf(C)).astype(np.float32)
    if mode == 1:
        op = x / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-5).astype(np.float32) * lnw
    elif mode == 2:
        op = x[:, :C] / (1.0 + np.exp(-x[:, :C])) * x[:, C:]
    else:
        op = x
    ref = (op.astype(np.float64) @ w.astype(np.float64).T + res).astype(np.float32)
    a = be.alloc(rows * parts * C * 2)
    out = be.zeros(rows * OC)
    be.ok("decode_prep", Ptr(a), parts, Ptr(be.put(x)), x.shape[1], mode, Ptr(be.put(lnw)), 1e-5, Ptr(out), OC, Ptr(be.put(res)), OC, OC, rows, C)
    be.ok("decode_gemm", Ptr(out), OC, Ptr(a), Ptr(dwx), parts, rows, C, OC)
    assert oc.rel_err(be.get(out, (rows, OC)), ref) < 2e-5


@pytest.mark.parametrize("kv", [BMC_F32, BMC_BF16])
@pytest.mark.parametrize("NB,NH,NKV,MS,pos", [(1, 15, 5, 768, 700), (2, 6, 2, 96, 95), (70, 3, 1, 64, 10), (1, 4, 4, 2048, 1500)])
def test_decode_attention_split_positions(be, NB, NH, NKV, MS, pos, kv):
    """One query against a cache of pos + 1 rows, with RoPE and the cache store inside the kernel, positions split over blocks.
    With a bf16 cache the expected result is that of the same arithmetic on keys and values rounded to bf16 when stored."""
    HD, L = 64, 2
    QD, KV = NH * HD, NKV * HD
    W = QD + 2 * KV
    layer = 1
    cache = np.zeros((L, 2, NB, MS, KV), np.float32)
    cache[layer, :, :, :pos] = rndf(2, NB, pos, KV)
    if kv == BMC_BF16:
        cache = bf16_round(cache)
    qkv = rndf(NB, W)
    hd2 = HD // 2
    inv = (1.0 / np.power(np.float32(100000.0), (2 * np.arange(hd2, dtype=np.float32)) / np.float32(HD))).astype(np.float32)
    ang = np.arange(MS, dtype=np.float32)[:, None] * inv[None, :]
    cs = np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)

    def rot(xh):  # [..., HD] at position pos
        c, s = cs[pos, :, 0], cs[pos, :, 1]
        x0, x1 = xh[..., :hd2], xh[..., hd2:]
        return np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c], axis=-1)
    qr = rot(qkv[:, :QD].reshape(NB, NH, HD))
    kr = rot(qkv[:, QD:QD + KV].reshape(NB, NKV, HD)).reshape(NB, KV)
    full = cache.copy()
    full[layer, 0, :, pos] = kr
    full[layer, 1, :, pos] = qkv[:, QD + KV:]
    if kv == BMC_BF16:
        full = bf16_round(full)
    mul = NH // NKV
    ref = np.zeros((NB, NH, HD), np.float32)
    for b in range(NB):
        for h in range(NH):
            kh = h // mul
            K = full[layer, 0, b, :pos + 1, kh * HD:(kh + 1) * HD].astype(np.float64)
            V = full[layer, 1, b, :pos + 1, kh * HD:(kh + 1) * HD].astype(np.float64)
            sc = K @ qr[b, h].astype(np.float64) * 0.125
            p = np.exp(sc - sc.max())
            ref[b, h] = (p / p.sum()) @ V
    dcache = be.put(cache, kv)
    dpos = be.put(np.array([pos], np.int32))
    be.lib.bmc_decode_attention_scratch_bytes.restype = C.c_size_t
    nbytes = be.lib.bmc_decode_attention_scratch_bytes(NB, MS, NH, NKV, HD)
    scratch = be.zeros((nbytes + 3) // 4)
    out = be.zeros(NB * QD)
    for _ in range(2):  # twice: the tickets must return to zero
        be.ok("decode_attention_fused", Ptr(out), Ptr(be.put(qkv)), Ptr(dcache), kv, Ptr(be.put(cs)), Ptr(dpos), Ptr(scratch), layer, NB, MS, NH, NKV, HD, 0.125)
        assert oc.rel_err(be.get(out, (NB, NH, HD)), ref) < (1e-5 if kv == BMC_F32 else 2e-3)   # a rotated key may round to the neighbouring bf16 value
    got_cache = be.get(dcache, cache.shape, kv)
    assert oc.rel_err(got_cache[layer, :, :, pos], full[layer, :, :, pos]) < (1e-6 if kv == BMC_F32 else 4e-3)
    assert np.array_equal(got_cache[layer, :, :, :pos], cache[layer, :, :, :pos]) and not got_cache[0].any()
