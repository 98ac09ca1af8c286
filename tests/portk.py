"""numpy-in / numpy-out wrappers over the single-kernel entry points of the plain-C oracle (oracle/bm_oracle.c)."""
import ctypes as C

import numpy as np

import oracle_check as oc

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = oc.load_port()
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def _i(a):
    a = np.ascontiguousarray(a, np.int32)
    return a, a.ctypes.data_as(C.POINTER(C.c_int))


def matmul_forward(inp, w):
    BT, Cc = inp.shape
    OC = w.shape[0]
    out = np.zeros((BT, OC), np.float32)
    (i, ip), (ww, wp), (o, op) = _f(inp), _f(w), _f(out)
    lib().orc_matmul_forward(op, ip, wp, BT, Cc, OC)
    return o


def matmul_backward_inp(gout, w, ginp0=None):
    BT, OC = gout.shape
    Cc = w.shape[1]
    g = np.zeros((BT, Cc), np.float32) if ginp0 is None else ginp0.astype(np.float32).copy()
    (go, gop), (ww, wp), (gi, gip) = _f(gout), _f(w), _f(g)
    lib().orc_matmul_backward_inp(gip, gop, wp, BT, Cc, OC)
    return gi


def matmul_backward_w(gout, inp, gw0=None):
    BT, OC = gout.shape
    Cc = inp.shape[1]
    g = np.zeros((OC, Cc), np.float32) if gw0 is None else gw0.astype(np.float32).copy()
    (go, gop), (ii, ip), (gw, gwp) = _f(gout), _f(inp), _f(g)
    lib().orc_matmul_backward_w(gwp, gop, ip, BT, Cc, OC)
    return gw


def rmsnorm_forward(x, w, eps=1e-5):
    N, Cc = x.shape
    out = np.zeros_like(x, dtype=np.float32)
    (xx, xp), (ww, wp), (o, op) = _f(x), _f(w), _f(out)
    lib().orc_rmsnorm_forward(op, xp, wp, N, Cc, C.c_float(eps))
    return o


def rmsnorm_backward_x(gout, w, x, gx0=None, eps=1e-5):
    N, Cc = x.shape
    g = np.zeros((N, Cc), np.float32) if gx0 is None else gx0.astype(np.float32).copy()
    (go, gop), (ww, wp), (xx, xp), (gx, gxp) = _f(gout), _f(w), _f(x), _f(g)
    lib().orc_rmsnorm_backward_x(gxp, gop, wp, xp, N, Cc, C.c_float(eps))
    return gx


def rmsnorm_backward_w(gout, x, eps=1e-5):
    N, Cc = x.shape
    (go, gop), (xx, xp), (gw, gwp) = _f(gout), _f(x), _f(np.zeros(Cc, np.float32))
    lib().orc_rmsnorm_backward_w(gwp, gop, xp, N, Cc, C.c_float(eps))
    return gw


def rope_seq(q, k, theta, direction=1):
    """q [S,NH,HD], k [S,NKV,HD]; returns rotated copies."""
    S, NH, HD = q.shape
    NKV = k.shape[1]
    (qq, qp), (kk, kp) = _f(q.copy()), _f(k.copy())
    lib().orc_rope_seq(qp, kp, S, NH, NKV, HD, C.c_float(theta), direction)
    return qq, kk


def attention_forward(Q, K, V, scale):
    S, NH, HD = Q.shape
    NKV = K.shape[1]
    (q, qp), (k, kp), (v, vp), (o, op) = _f(Q), _f(K), _f(V), _f(np.zeros_like(Q, dtype=np.float32))
    lib().orc_attention_forward(op, qp, kp, vp, S, NH, NKV, HD, C.c_float(scale))
    return o


def attention_backward(gout, Q, K, V, scale):
    S, NH, HD = Q.shape
    NKV = K.shape[1]
    (g, gp), (q, qp), (k, kp), (v, vp) = _f(gout), _f(Q), _f(K), _f(V)
    (gq, gqp), (gk, gkp), (gv, gvp) = _f(np.zeros_like(q)), _f(np.zeros_like(k)), _f(np.zeros_like(v))
    lib().orc_attention_backward(gqp, gkp, gvp, gp, qp, kp, vp, S, NH, NKV, HD, C.c_float(scale))
    return gq, gk, gv


def swiglu_forward(gate, up):
    (g, gp), (u, up_), (o, op) = _f(gate), _f(up), _f(np.zeros_like(gate, dtype=np.float32))
    lib().orc_swiglu_forward(op, gp, up_, C.c_size_t(g.size))
    return o


def swiglu_backward(gate, up, gout):
    (g, gp), (u, up_), (go, gop) = _f(gate), _f(up), _f(gout)
    (gg, ggp), (gu, gup) = _f(np.zeros_like(g)), _f(np.zeros_like(g))
    lib().orc_swiglu_backward(ggp, gup, gp, up_, gop, C.c_size_t(g.size))
    return gg, gu


def xent(logits, targets):
    N, V = logits.shape
    (l, lp), (t, tp), (g, gp) = _f(logits), _i(targets), _f(np.zeros_like(logits, dtype=np.float32))
    loss = lib().orc_xent(gp, lp, tp, N, V)
    return float(loss), g


def adamw(w, g, m, v, hp8):
    (ww, wp), (gg, gp), (mm, mp), (vv, vp) = _f(w.copy()), _f(g), _f(m.copy()), _f(v.copy())
    hp = (C.c_float * 8)(*hp8)
    lib().orc_adamw(wp, gp, mp, vp, C.c_size_t(ww.size), hp)
    return ww, mm, vv


def embedding_backward(gwte0, gout, tokens):
    T, D = gout.shape
    (gw, gwp), (go, gop), (t, tp) = _f(gwte0.copy()), _f(gout), _i(tokens)
    lib().orc_embedding_backward(gwp, gop, tp, T, D)
    return gw


def argmax(logits):
    l, lp = _f(logits)
    return int(lib().orc_argmax(lp, l.size))
