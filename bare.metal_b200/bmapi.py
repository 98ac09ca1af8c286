"""ctypes bindings and synthetic-input helpers shared by the tests, bench.py and smoke().

The public C API is the reference's `include/baremetal.h` (functions at baremetal.h:120-206), so `bind_public_api`
binds any library that exports it: the product library (libbaremetal_b200.so) here, and the reference build that the
tests use as their parity oracle (loaded by oracle/oracle_check.py, not by this package).
"""
import ctypes as C
import os
import struct

import numpy as np

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)

BM_PRECISION_FP32, BM_PRECISION_FP16, BM_PRECISION_BF16 = 0, 1, 2
BM_DEVICE_CPU, BM_DEVICE_METAL, BM_DEVICE_CUDA = 0, 1, 2
BM_NORM_RMSNORM, BM_ACT_SWIGLU, BM_POS_ROPE, BM_ATTN_GQA = 1, 1, 1, 1
CHECKPOINT_MAGIC = 20250718  # src/baremetal/checkpoint.h:11


class BmArch(C.Structure):
    """bm_arch_t, include/baremetal.h:54-87."""
    _fields_ = [(n, C.c_int) for n in (
        "dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size", "padded_vocab_size",
        "max_seq_len", "norm", "activation", "pos_enc", "attention", "precision", "bias", "weight_tie",
        "has_qk_norm", "has_ffn_post_norm", "head_dim", "gated_mlp", "gemma_norm", "embed_scale",
        "weight_layout")] + [("rope_theta", C.c_float), ("rope_scaling", C.c_int),
                             ("rope_factor", C.c_float), ("rope_low_freq_factor", C.c_float),
                             ("rope_high_freq_factor", C.c_float), ("rope_original_max", C.c_float)]


class BmTrainConfig(C.Structure):
    """bm_train_config_t, include/baremetal.h:91-107."""
    _fields_ = [("learning_rate", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float),
                ("epsilon", C.c_float), ("weight_decay", C.c_float), ("grad_clip", C.c_float),
                ("grad_accum_steps", C.c_int), ("warmup_steps", C.c_int), ("max_steps", C.c_int),
                ("use_master_weights", C.c_int), ("seq_len", C.c_int), ("lora_rank", C.c_int),
                ("lora_alpha", C.c_float), ("lora_targets", C.c_int), ("lora_seed", C.c_int)]


ARCHS = {
    # name: D, H, L, NH, NKV, V
    "smollm2-135m": dict(dim=576, hidden_dim=1536, n_layers=30, n_heads=9, n_kv_heads=3, vocab_size=49152),
    "smollm2-360m": dict(dim=960, hidden_dim=2560, n_layers=32, n_heads=15, n_kv_heads=5, vocab_size=49152),
    # scaled-down members of the same family for fast CPU-oracle comparisons (head_dim stays 64)
    "tiny": dict(dim=128, hidden_dim=256, n_layers=2, n_heads=2, n_kv_heads=1, vocab_size=512),
    "small": dict(dim=192, hidden_dim=512, n_layers=3, n_heads=3, n_kv_heads=1, vocab_size=1024),
    "gqa": dict(dim=384, hidden_dim=1024, n_layers=2, n_heads=6, n_kv_heads=2, vocab_size=2048),
}


def make_arch(name_or_dict, max_seq_len=8192):
    d = ARCHS[name_or_dict] if isinstance(name_or_dict, str) else dict(name_or_dict)
    a = BmArch()
    for k, v in d.items():
        setattr(a, k, v)
    a.padded_vocab_size = a.vocab_size
    a.max_seq_len = max_seq_len
    a.norm, a.activation, a.pos_enc, a.attention = BM_NORM_RMSNORM, BM_ACT_SWIGLU, BM_POS_ROPE, BM_ATTN_GQA
    a.precision = BM_PRECISION_FP32
    a.weight_tie = 1
    a.head_dim = d.get("head_dim", 64)
    a.gated_mlp = 1
    a.rope_theta = 100000.0
    return a


def weight_shapes(a):
    """Flat fp32 order of the reference's model buffer and .bin payload (src/baremetal/model.c:140-172)."""
    L, D, H = a.n_layers, a.dim, a.hidden_dim
    QD, KV = a.n_heads * a.head_dim, a.n_kv_heads * a.head_dim
    return [("embed", (a.vocab_size, D)), ("ln1w", (L, D)), ("qw", (L, QD, D)), ("kw", (L, KV, D)),
            ("vw", (L, KV, D)), ("ow", (L, D, QD)), ("ln2w", (L, D)), ("gate", (L, H, D)),
            ("up", (L, H, D)), ("down", (L, D, H)), ("lnfw", (D,))]


def make_weights(a, seed=42, std=0.02, layer_scale=1.0):
    """Random-init weights: every matrix N(0, std^2) from `seed`; RMSNorm gains are 1. layer_scale multiplies the
    per-layer matrices (not the embedding): with tied embeddings a larger value lets the layers, rather than the input
    token's own embedding row, decide the next token, which makes greedy continuations non-trivial."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in weight_shapes(a):
        if name.startswith("ln"):
            w[name] = np.ones(shape, np.float32)
        else:
            w[name] = (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)
            if name != "embed" and layer_scale != 1.0:
                w[name] *= np.float32(layer_scale)
    return w


def write_bin_checkpoint(path, a, w):
    """Legacy .bin checkpoint: 256 x int32 header then the flat fp32 payload
    (src/baremetal/checkpoint.c:19-57 header fields, :69-72 payload)."""
    hdr = [0] * 256
    hdr[0] = CHECKPOINT_MAGIC
    hdr[1] = 1
    hdr[2:24] = [a.precision, a.dim, a.hidden_dim, a.n_layers, a.n_heads, a.n_kv_heads, a.vocab_size,
                 a.max_seq_len, a.norm, a.activation, a.pos_enc, a.attention, a.bias, a.weight_tie,
                 a.has_qk_norm, a.has_ffn_post_norm, a.head_dim, a.gated_mlp, a.embed_scale,
                 a.weight_layout, a.gemma_norm, int(a.rope_theta)]
    with open(path, "wb") as f:
        f.write(struct.pack("<256i", *hdr))
        for name, _ in weight_shapes(a):
            f.write(np.ascontiguousarray(w[name], np.float32).tobytes())


ADAPTER_MAGIC = 0x424D4C52
ADAPTER_TARGETS = {"q": 1, "k": 2, "v": 4, "o": 8, "gate": 16, "up": 32, "down": 64}   # src/baremetal/lora.h:13-21
ADAPTER_WEIGHT_KEY = {"q": "qw", "k": "kw", "v": "vw", "o": "ow", "gate": "gate", "up": "up", "down": "down"}


def write_adapter_file(path, a, rank, alpha, entries, header_overrides=None):
    """Adapter file as bm_save_adapter writes it and bm_load_adapter reads it (src/baremetal/adapter.c:20-40, :85-147):
    an 11-word header, then per entry five int32 {layer, target bit, r, c, oc} followed by A[r][c] and B[oc][r] as fp32.
    `entries` is a list of (layer, target name, A, B); `header_overrides` replaces header fields by name (for tests)."""
    h = dict(magic=ADAPTER_MAGIC, version=1, dim=a.dim, layers=a.n_layers, n_heads=a.n_heads, n_kv_heads=a.n_kv_heads,
             vocab=a.vocab_size, head_size=a.head_dim, rank=rank, alpha=float(alpha), n_adapters=len(entries))
    h.update(header_overrides or {})
    with open(path, "wb") as f:
        f.write(struct.pack("<II7ifi", h["magic"], h["version"], h["dim"], h["layers"], h["n_heads"], h["n_kv_heads"],
                            h["vocab"], h["head_size"], h["rank"], h["alpha"], h["n_adapters"]))
        for layer, target, A, B in entries:
            A, B = np.ascontiguousarray(A, np.float32), np.ascontiguousarray(B, np.float32)
            tbit = ADAPTER_TARGETS[target] if isinstance(target, str) else int(target)
            f.write(struct.pack("<5i", layer, tbit, A.shape[0], A.shape[1], B.shape[0]))
            f.write(A.tobytes())
            f.write(B.tobytes())


def state_tensor_order(a):
    """Tensor order of the trainer-state file and of the optimizer-state list: per layer ln1w, qw, kw,
    vw, ow, ln2w, gate, up, down; then lnfw; then the tied embedding (src/baremetal/graph.c:288-369,
    src/baremetal/trainer.c:86-111). Yields (key, layer or None)."""
    out = []
    for l in range(a.n_layers):
        for k in ("ln1w", "qw", "kw", "vw", "ow", "ln2w", "gate", "up", "down"):
            out.append((k, l))
    out.append(("lnfw", None))
    out.append(("embed", None))
    return out


def lcg_tokens(n, vocab, seed=42):
    """The reference's synthetic token stream: s = s*1664525 + 1013904223 (mod 2^32), tok = s % V
    (bench/train_bench.c:286-290)."""
    # closed form of the recurrence, evaluated with wrapping uint32 arithmetic:
    # s_i = a^i * s_0 + c * (1 + a + ... + a^(i-1))  (mod 2^32)
    if n <= 0:
        return np.empty(0, np.int32)
    with np.errstate(over="ignore"):
        a_pow = np.cumprod(np.full(n, 1664525, dtype=np.uint32), dtype=np.uint32)           # a^1 .. a^n
        geo = np.cumsum(np.concatenate((np.ones(1, np.uint32), a_pow[:-1])), dtype=np.uint32)  # sum_{j<i} a^j
        s = a_pow * np.uint32(seed & 0xFFFFFFFF) + np.uint32(1013904223) * geo
    return (s % np.uint32(vocab)).astype(np.int32)


def lcg_batch(B, S, vocab, seed=42):
    """B contiguous windows of S tokens from one LCG stream; targets are the inputs shifted by one
    (the next stream value for the last position, as tools/cli.c:762-768 does)."""
    stream = lcg_tokens(B * S + 1, vocab, seed)
    inputs = stream[:B * S].reshape(B, S).copy()
    targets = stream[1:B * S + 1].reshape(B, S).copy()
    return inputs, targets


def train_config(lr=3e-4, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, accum=1, seq_len=64):
    c = BmTrainConfig()
    c.learning_rate, c.beta1, c.beta2, c.epsilon, c.weight_decay = lr, b1, b2, eps, wd
    c.grad_clip, c.grad_accum_steps, c.warmup_steps, c.max_steps = 1.0, accum, 0, 0
    c.use_master_weights, c.seq_len = 1, seq_len
    return c


def bind_public_api(lib):
    vp, ip, fp = C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_float)
    sig = {
        "bm_create": (vp, [C.c_int]), "bm_destroy": (None, [vp]),
        "bm_get_supported_precision": (C.c_int, [vp]),
        "bm_create_model": (vp, [vp, C.POINTER(BmArch)]), "bm_load_weights": (None, [vp, C.c_char_p]),
        "bm_destroy_model": (None, [vp]), "bm_get_num_parameters": (C.c_int, [vp]),
        "bm_load_adapter": (C.c_int, [vp, C.c_char_p]),
        "bm_create_trainer": (vp, [vp, vp, C.POINTER(BmTrainConfig)]),
        "bm_train_step": (C.c_float, [vp, ip, ip, C.c_int, C.c_int]),
        "bm_train_step_masked": (C.c_float, [vp, ip, ip, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
        "bm_train_eval_masked": (C.c_float, [vp, ip, ip, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
        "bm_train_flush": (None, [vp]),
        "bm_save_state": (None, [vp, C.c_char_p]), "bm_load_state": (None, [vp, C.c_char_p]),
        "bm_destroy_trainer": (None, [vp]),
        "bm_create_session": (vp, [vp, vp]), "bm_forward": (fp, [vp, ip, C.c_int]), "bm_step": (fp, [vp, C.c_int]),
        "bm_reset_session": (None, [vp]), "bm_destroy_session": (None, [vp]),
        "bm_create_sampler": (vp, [C.c_int, C.c_float, C.c_float, C.c_uint64]),
        "bm_sample": (C.c_int, [vp, fp]), "bm_destroy_sampler": (None, [vp]),
    }
    for name, (res, args) in sig.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
    return lib


LIB_PATH = os.path.join(PKG_DIR, "libbaremetal_b200.so")

BMX_WEIGHT, BMX_GRAD, BMX_ADAM_M, BMX_ADAM_V = 0, 1, 2, 3


def load_product():
    """The product library. Raises if it has not been built: there is no fallback."""
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `make -C bare.metal_b200` "
                           "(or __graft_entry__.build())")
    lib = bind_public_api(C.CDLL(LIB_PATH))
    vp, fp, ip = C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_int)
    ext = {
        "bmx_trainer_num_tensors": (C.c_int, [vp]), "bmx_trainer_tensor_size": (C.c_size_t, [vp, C.c_int]),
        "bmx_trainer_read": (C.c_int, [vp, C.c_int, C.c_int, fp]),
        "bmx_trainer_set_option": (C.c_int, [vp, C.c_char_p, C.c_int]),
        "bmx_trainer_launch_count": (C.c_long, [vp]), "bmx_trainer_device_bytes": (C.c_size_t, [vp]),
        "bmx_train_step_resident": (C.c_int, [vp, vp, vp, C.c_int, C.c_int]),
        "bmx_train_last_loss": (C.c_float, [vp]),
        "bmx_device_alloc": (vp, [vp, C.c_size_t]), "bmx_device_free": (None, [vp, vp]),
        "bmx_device_upload": (C.c_int, [vp, vp, vp, C.c_size_t]), "bmx_device_sync": (C.c_int, [vp]),
        "bmx_timer_begin": (C.c_int, [vp, C.c_int]), "bmx_timer_end": (C.c_float, [vp, C.c_int]),
        "bmx_model_weight_buffer": (fp, [vp, C.POINTER(C.c_size_t)]),
        "bmx_gemm_timing": (C.c_int, [vp, C.c_int]), "bmx_gemm_timing_collect": (C.c_int, [vp, C.POINTER(C.c_double)]),
        "bmx_model_set_quant": (C.c_int, [vp, C.c_int]), "bmx_model_vocab_size": (C.c_int, [vp]),
        "bmx_quantize_q8": (C.c_size_t, [fp, vp, fp, C.c_size_t]),
        "bmx_quantize_q4": (C.c_size_t, [fp, vp, fp, C.c_size_t]),
        "bmx_create_session_batched": (vp, [vp, vp, C.c_int, C.c_int]), "bmx_create_session_kv": (vp, [vp, vp, C.c_int, C.c_int, C.c_int]),
        "bmx_session_kv_bytes_per_element": (C.c_int, [vp]),
        "bmx_session_generate_greedy": (C.c_int, [vp, ip, C.c_int, C.c_int, ip]),
        "bmx_session_logits": (fp, [vp]), "bmx_session_position": (C.c_int, [vp]), "bmx_session_weight_bytes": (C.c_size_t, [vp]), "bmx_session_algorithmic_weight_bytes": (C.c_size_t, [vp]),
        "bmx_trainer_sync_model": (C.c_int, [vp]), "bmx_model_arch_field": (C.c_double, [vp, C.c_char_p]),
        "bmx_dp_unique_id": (C.c_int, [vp]), "bmx_trainer_dp_init": (C.c_int, [vp, C.c_int, C.c_int, vp]),
    }
    for name, (res, args) in ext.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


def product_read(lib, trainer, what, i):
    n = lib.bmx_trainer_tensor_size(trainer, i)
    out = np.empty(n, np.float32)
    rc = lib.bmx_trainer_read(trainer, what, i, out.ctypes.data_as(C.POINTER(C.c_float)))
    if rc != 0:
        raise RuntimeError(f"bmx_trainer_read failed: {rc}")
    return out


def read_state_file(path):
    """Trainer-state layout: int32 step, int32 n_states, then per tensor size_t n, float w[n], m[n], v[n]
    (src/baremetal/trainer.c:144-191)."""
    with open(path, "rb") as f:
        step, n_states = struct.unpack("<ii", f.read(8))
        tensors = []
        for _ in range(n_states):
            (n,) = struct.unpack("<Q", f.read(8))
            w = np.frombuffer(f.read(4 * n), np.float32)
            m = np.frombuffer(f.read(4 * n), np.float32)
            v = np.frombuffer(f.read(4 * n), np.float32)
            tensors.append((w, m, v))
    return step, tensors


def as_int_ptr(a):
    return a.ctypes.data_as(C.POINTER(C.c_int))
