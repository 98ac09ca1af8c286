"""TEST INFRASTRUCTURE — Python access to the two CPU oracles and the comparison helpers the tests,
smoke() and bench.py's cpu_baseline leg use. Nothing in the product imports this module.

Two checkers, same inputs, same outputs:
  * "reference": oracle/_ref/libbm_ref.so — the reference's own C11 host code + Metal kernel sources on CPU
    (built by oracle/build_ref.sh from a reference checkout; travels as a built file);
  * "port": oracle/liboracle.so — the plain-C restatement in oracle/bm_oracle.c (always buildable).
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, os.path.join(ROOT, "bare.metal_b200"))
import bmapi  # noqa: E402

PORT_PATH = os.path.join(HERE, "liboracle.so")
Q_NORM_GRAD, Q_GX_CARRY, Q_STALE_EMBED = 1, 2, 4
Q_ALL = 7


REF_LIB_PATH = os.path.join(HERE, "_ref", "libbm_ref.so")


def reference_read(lib, trainer, what, i):
    n = lib.bmref_state_size(trainer, i)
    fn = {bmapi.BMX_WEIGHT: lib.bmref_weight, bmapi.BMX_GRAD: lib.bmref_grad, bmapi.BMX_ADAM_M: lib.bmref_m, bmapi.BMX_ADAM_V: lib.bmref_v}[what]
    return np.ctypeslib.as_array(fn(trainer, i), (n,)).copy()


REF_CUDA_LIB_PATH = os.path.join(HERE, "_ref", "libbm_ref_cuda.so")
KERNEL_TESTS_DIR = os.path.join(HERE, "_ref", "kernel_tests")


def load_reference(path=REF_LIB_PATH):
    """The reference's own host code + kernels on CPU (built by oracle/build_ref.sh). None if absent.
    With path=REF_CUDA_LIB_PATH: the same host code linked against the product's CUDA backend (needs a GPU)."""
    if not os.path.exists(path):
        return None
    lib = bmapi.bind_public_api(C.CDLL(path))
    vp, fp = C.c_void_p, C.POINTER(C.c_float)
    lib.bmref_set_precision.argtypes = [vp, C.c_int]
    lib.bmref_set_quant.argtypes = [vp, C.c_int]
    lib.bmt_quantize_q8.restype, lib.bmt_quantize_q8.argtypes = C.c_size_t, [fp, vp, C.c_size_t]
    lib.bmt_quantize_q4.restype, lib.bmt_quantize_q4.argtypes = C.c_size_t, [fp, vp, C.c_size_t]
    lib.bmref_n_states.restype, lib.bmref_n_states.argtypes = C.c_int, [vp]
    lib.bmref_state_size.restype, lib.bmref_state_size.argtypes = C.c_size_t, [vp, C.c_int]
    for n in ("bmref_grad", "bmref_weight", "bmref_m", "bmref_v"):
        getattr(lib, n).restype, getattr(lib, n).argtypes = fp, [vp, C.c_int]
    lib.bmref_logits.restype, lib.bmref_logits.argtypes = fp, [vp]
    return lib


def load_port():
    if not os.path.exists(PORT_PATH):
        raise RuntimeError(f"{PORT_PATH} missing: run `make -C oracle`")
    lib = C.CDLL(PORT_PATH)
    fp, ip, vp = C.POINTER(C.c_float), C.POINTER(C.c_int), C.c_void_p
    lib.orc_create.restype = vp
    lib.orc_create.argtypes = [C.c_int] * 10 + [C.c_float] * 6 + [C.c_int, fp]
    lib.orc_destroy.argtypes = [vp]
    lib.orc_step.restype, lib.orc_step.argtypes = C.c_float, [vp, ip, ip, C.c_int]
    lib.orc_num_tensors.restype, lib.orc_num_tensors.argtypes = C.c_int, [vp]
    lib.orc_tensor_size.restype, lib.orc_tensor_size.argtypes = C.c_size_t, [vp, C.c_int]
    lib.orc_read.argtypes = [vp, C.c_int, C.c_int, fp]
    lib.orc_xent.restype = C.c_float
    lib.orc_argmax.restype = C.c_int
    lib.orc_quantize_q8.restype, lib.orc_quantize_q8.argtypes = C.c_size_t, [fp, vp, fp, C.c_size_t]
    lib.orc_quantize_q4.restype, lib.orc_quantize_q4.argtypes = C.c_size_t, [fp, vp, fp, C.c_size_t]
    lib.orc_dec_create.restype = vp
    lib.orc_dec_create.argtypes = [C.c_int] * 10 + [C.c_float, fp]
    lib.orc_dec_destroy.argtypes = [vp]
    lib.orc_dec_reset.argtypes = [vp]
    lib.orc_dec_step.restype, lib.orc_dec_step.argtypes = fp, [vp, C.c_int]
    return lib


def fptr(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def flat_model_weights(a, w):
    return np.concatenate([np.ascontiguousarray(w[name], np.float32).ravel() for name, _ in bmapi.weight_shapes(a)])


class PortTrainer:
    """The plain-C oracle behind the same small interface as the library-backed runners below."""
    kind = "port"

    def __init__(self, a, w, S, precision, cfg, quirks=Q_ALL):
        self.lib = load_port()
        flat = flat_model_weights(a, w)
        self.h = self.lib.orc_create(a.dim, a.hidden_dim, a.n_layers, a.n_heads, a.n_kv_heads, a.vocab_size, a.head_dim, S,
                                     precision, quirks, cfg.learning_rate, cfg.beta1, cfg.beta2, cfg.epsilon,
                                     cfg.weight_decay, a.rope_theta, cfg.grad_accum_steps, fptr(flat))
        self.S = S

    def step(self, x, y):
        B = x.shape[0]
        return float(self.lib.orc_step(self.h, bmapi.as_int_ptr(x), bmapi.as_int_ptr(y), B))

    def n_tensors(self):
        return self.lib.orc_num_tensors(self.h)

    def read(self, what, i):
        out = np.empty(self.lib.orc_tensor_size(self.h, i), np.float32)
        self.lib.orc_read(self.h, what, i, fptr(out))
        return out

    def close(self):
        self.lib.orc_destroy(self.h)


class LibTrainer:
    """A trainer behind the public C API: the product (kind 'gpu') or the reference build (kind 'reference')."""

    def __init__(self, lib, kind, a, w, S, precision, cfg, quirks=True, tag="t"):
        self.lib, self.kind, self.S = lib, kind, S
        a = bmapi.make_arch({k: getattr(a, k) for k in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size")} |
                            {"head_dim": a.head_dim})
        a.precision = precision
        path = f"/tmp/bm_{tag}_{os.getpid()}_{kind}.bin"
        bmapi.write_bin_checkpoint(path, a, w)
        self.ctx = lib.bm_create(bmapi.BM_DEVICE_METAL)
        if not self.ctx:
            raise RuntimeError("bm_create failed (no GPU for the product / no backend)")
        self.model = lib.bm_create_model(self.ctx, C.byref(a))
        lib.bm_load_weights(self.model, path.encode())
        os.unlink(path)
        if kind == "reference":
            lib.bmref_set_precision(self.model, precision)
        self.tr = lib.bm_create_trainer(self.ctx, self.model, C.byref(cfg))
        if not self.tr:
            raise RuntimeError("bm_create_trainer failed")
        if kind == "gpu" and quirks:
            assert lib.bmx_trainer_set_option(self.tr, b"ref_quirks", 1) == 0

    def step(self, x, y):
        B = x.shape[0]
        return float(self.lib.bm_train_step(self.tr, bmapi.as_int_ptr(x), bmapi.as_int_ptr(y), B, self.S))

    def step_masked(self, x, y, attn_mask, loss_mask, evaluate=False):
        B = x.shape[0]
        am = None if attn_mask is None else np.ascontiguousarray(attn_mask, np.uint8).ctypes.data
        lm = None if loss_mask is None else np.ascontiguousarray(loss_mask, np.uint8).ctypes.data
        fn = self.lib.bm_train_eval_masked if evaluate else self.lib.bm_train_step_masked
        return float(fn(self.tr, bmapi.as_int_ptr(x), bmapi.as_int_ptr(y), am, lm, B, self.S))

    def n_tensors(self):
        return self.lib.bmref_n_states(self.tr) if self.kind == "reference" else self.lib.bmx_trainer_num_tensors(self.tr)

    def read(self, what, i):
        if self.kind == "reference":
            return reference_read(self.lib, self.tr, what, i)
        return bmapi.product_read(self.lib, self.tr, what, i)

    def close(self):
        self.lib.bm_destroy_trainer(self.tr)
        self.lib.bm_destroy_model(self.model)
        self.lib.bm_destroy(self.ctx)


class PortDecoder:
    """Decode with a KV cache in the plain-C oracle: one sequence, one token per step."""
    kind = "port"

    def __init__(self, a, w, precision, quant, max_positions):
        self.lib = load_port()
        flat = flat_model_weights(a, w)
        self.V = a.vocab_size
        self.h = self.lib.orc_dec_create(a.dim, a.hidden_dim, a.n_layers, a.n_heads, a.n_kv_heads, a.vocab_size, a.head_dim,
                                         max_positions, quant, 1 if precision == bmapi.BM_PRECISION_BF16 else 0, a.rope_theta,
                                         fptr(flat))

    def step(self, token):
        p = self.lib.orc_dec_step(self.h, int(token))
        return np.ctypeslib.as_array(p, shape=(self.V,)).copy()

    def forward(self, tokens):
        for t in tokens:
            out = self.step(t)
        return out

    def reset(self):
        self.lib.orc_dec_reset(self.h)

    def close(self):
        self.lib.orc_dec_destroy(self.h)


class LibSession:
    """An inference session behind the public C API: the product (kind 'gpu') or the reference build (kind 'reference')."""

    def __init__(self, lib, kind, a, w, precision, quant, tag="s"):
        self.lib, self.kind = lib, kind
        a = bmapi.make_arch({k: getattr(a, k) for k in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size")} |
                            {"head_dim": a.head_dim})
        a.precision = precision
        self.V = a.vocab_size
        path = f"/tmp/bm_{tag}_{os.getpid()}_{kind}.bin"
        bmapi.write_bin_checkpoint(path, a, w)
        self.ctx = lib.bm_create(bmapi.BM_DEVICE_METAL)
        if not self.ctx:
            raise RuntimeError("bm_create failed (no GPU for the product / no backend)")
        self.model = lib.bm_create_model(self.ctx, C.byref(a))
        lib.bm_load_weights(self.model, path.encode())
        os.unlink(path)
        if kind == "reference":
            lib.bmref_set_precision(self.model, precision)
            lib.bmref_set_quant(self.model, quant)
        else:
            assert lib.bmx_model_set_quant(self.model, quant) == 0
        lib.bm_compile(self.model)
        self.sess = lib.bm_create_session(self.ctx, self.model)
        if not self.sess:
            raise RuntimeError("bm_create_session failed")

    def step(self, token):
        p = self.lib.bm_step(self.sess, int(token))
        if not p:
            raise RuntimeError("bm_step failed")
        return np.ctypeslib.as_array(p, shape=(self.V,)).copy()

    def forward(self, tokens):
        t = np.ascontiguousarray(tokens, np.int32)
        p = self.lib.bm_forward(self.sess, bmapi.as_int_ptr(t), len(t))
        if not p:
            raise RuntimeError("bm_forward failed")
        return np.ctypeslib.as_array(p, shape=(self.V,)).copy()

    def reset(self):
        self.lib.bm_reset_session(self.sess)

    def close(self):
        self.lib.bm_destroy_session(self.sess)
        self.lib.bm_destroy_model(self.model)
        self.lib.bm_destroy(self.ctx)


def make_oracle(a, w, S, precision, cfg, prefer="reference", quirks=True):
    """The strongest checker available: the reference build when present, else the plain-C port."""
    ref = load_reference() if prefer == "reference" and quirks else None
    if ref is not None:
        return LibTrainer(ref, "reference", a, w, S, precision, cfg)
    return PortTrainer(a, w, S, precision, cfg, quirks=Q_ALL if quirks else 0)


def rel_err(x, ref):
    x = x.astype(np.float64)
    ref = ref.astype(np.float64)
    return float(np.linalg.norm(x - ref) / (np.linalg.norm(ref) + 1e-30))


def cosine(x, ref):
    x = x.astype(np.float64)
    ref = ref.astype(np.float64)
    return float(x @ ref / (np.linalg.norm(x) * np.linalg.norm(ref) + 1e-30))


def compare_one_step(lib, arch_name, B, S, precision, quirks=True, prefer="reference", steps=1, accum=1):
    """Run `steps` optimizer steps on the product (GPU) and on the oracle from identical weights and tokens; compare
    the first step's per-tensor gradients and the final weights."""
    a = bmapi.make_arch(arch_name)
    w = bmapi.make_weights(a)
    cfg = bmapi.train_config(seq_len=S, accum=accum)
    x, y = bmapi.lcg_batch(B * steps * accum, S, a.vocab_size)
    gpu = LibTrainer(lib, "gpu", a, w, S, precision, cfg, quirks=quirks)
    orc = make_oracle(a, w, S, precision, cfg, prefer=prefer, quirks=quirks)
    out = {"oracle_kind": orc.kind, "losses_gpu": [], "losses_oracle": []}
    n = gpu.n_tensors()
    assert n == orc.n_tensors()
    for st in range(steps * accum):
        xs = np.ascontiguousarray(x[st * B:(st + 1) * B])
        ys = np.ascontiguousarray(y[st * B:(st + 1) * B])
        out["losses_gpu"].append(gpu.step(xs, ys))
        out["losses_oracle"].append(orc.step(xs, ys))
        if st == accum - 1:
            rels = [rel_err(gpu.read(bmapi.BMX_GRAD, i), orc.read(bmapi.BMX_GRAD, i)) for i in range(n)]
            coss = [cosine(gpu.read(bmapi.BMX_GRAD, i), orc.read(bmapi.BMX_GRAD, i)) for i in range(n)]
            out["grad_rel"], out["grad_cos"] = rels, coss
            out["worst_grad_rel"], out["min_grad_cos"] = max(rels), min(coss)
    wrel = [rel_err(gpu.read(bmapi.BMX_WEIGHT, i), orc.read(bmapi.BMX_WEIGHT, i)) for i in range(n)]
    wcos = [cosine(gpu.read(bmapi.BMX_WEIGHT, i), orc.read(bmapi.BMX_WEIGHT, i)) for i in range(n)]
    out["weight_rel"], out["worst_weight_rel"], out["min_weight_cos"] = wrel, max(wrel), min(wcos)
    out["loss_gpu"], out["loss_oracle"] = out["losses_gpu"][0], out["losses_oracle"][0]
    gpu.close()
    orc.close()
    return out
