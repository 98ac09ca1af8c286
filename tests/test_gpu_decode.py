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
from test_oracle_pins import DECODE_GOLDENS, decode_case

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
    # the step after the first is replayed from a captured graph; prefill must give the same bits as stepping
    s.reset()
    lf = s.forward(g["prompt"])
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


@pytest.mark.parametrize("precision,quant,NB", [(F32, 0, 3), (BF16, 8, 11), (BF16, 0, 8), (F32, 8, 1), (F32, 8, 5), (F32, 0, 16), (BF16, 8, 64)])
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
    for b in range(NB):
        dec = oc.PortDecoder(a, w, precision, quant, 32)
        l1 = dec.forward(prompts[b])
        ids = []
        for i in range(n_new):
            ids.append(int(np.argmax(l1)))
            if i + 1 < n_new:
                l1 = dec.step(ids[-1])
        dec.close()
        assert ids == list(out[b]), b
        assert close(lg[b], l1), b


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
