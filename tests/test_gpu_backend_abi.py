"""The reference's backend ABI (include/backend.h = src/backend/backend.h:17-67 of the reference) served by the CUDA backend.

Two checkers, both built by oracle/build_ref.sh where a reference checkout is present and shipped as built files:
  * oracle/_ref/libbm_ref_cuda.so — the reference's unmodified C11 host code (graph, scheduler, trainer, AdamW driver) linked against
    libbaremetal_b200.so's backend_* functions. Its training step must agree with the same host code on the CPU backend
    (oracle/_ref/libbm_ref.so) within 1e-4: both dispatch the same kernels by name, one on the GPU and one on the host.
  * oracle/_ref/kernel_tests/* — the reference's own kernel test programs (test/*_test.c), compiled unchanged against the same
    backend_* functions. They load the reference's golden vectors from test/grad/*.bin (regenerated here from the committed
    torch_kernel_goldens.npz) and exit 0 when their own cosine criterion (> 0.9999) holds.
A third group drives backend_* directly through ctypes for the contract points the programs above do not reach: byte offsets,
missing names, size-0 buffers, host visibility without unmap, encoder timing."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import bmapi
import oracle_check as oc
from test_oracle_pins import GOLD_DIR

pytestmark = pytest.mark.gpu
F32, BF16 = bmapi.BM_PRECISION_FP32, bmapi.BM_PRECISION_BF16
INT_FILES = {"xent_targets", "embed_tokens"}


@pytest.mark.parametrize("precision,B,S", [(F32, 2, 32), (BF16, 2, 32), (F32, 1, 300)])
def test_reference_host_code_trains_on_the_cuda_backend(precision, B, S):
    cpu, gpu = oc.load_reference(), oc.load_reference(oc.REF_CUDA_LIB_PATH)
    if cpu is None or gpu is None:
        pytest.skip("reference builds not present (oracle/build_ref.sh needs a reference checkout)")
    a = bmapi.make_arch("tiny")
    w = bmapi.make_weights(a)
    cfg = bmapi.train_config(seq_len=S)
    x, y = bmapi.lcg_batch(2 * B, S, a.vocab_size)
    r = oc.LibTrainer(cpu, "reference", a, w, S, precision, cfg, tag="abi_cpu")
    g = oc.LibTrainer(gpu, "reference", a, w, S, precision, cfg, tag="abi_gpu")
    for st in range(2):
        xs, ys = np.ascontiguousarray(x[st * B:(st + 1) * B]), np.ascontiguousarray(y[st * B:(st + 1) * B])
        lr, lg = r.step(xs, ys), g.step(xs, ys)
        assert abs(lr - lg) < 1e-4, (st, lr, lg)
        if st == 0:
            for i in range(r.n_tensors()):
                assert oc.rel_err(g.read(bmapi.BMX_GRAD, i), r.read(bmapi.BMX_GRAD, i)) < 1e-4, i
    for i in range(r.n_tensors()):
        assert oc.rel_err(g.read(bmapi.BMX_WEIGHT, i), r.read(bmapi.BMX_WEIGHT, i)) < 1e-4, i
    r.close(); g.close()


KERNEL_TESTS = ["matmul_bwd_test", "rmsnorm_bwd_test", "rope_seq_bwd_test", "rope_real_test", "xent_bwd_test", "embed_bwd_test",
                "adamw_test", "attn_bwd_test", "attn_fwd_test", "attn_real_test", "train_attn_tiled_test"]


@pytest.fixture(scope="module")
def golden_bin_dir(tmp_path_factory):
    """test/grad/<name>.bin as the reference's generators write them, from the committed npz."""
    root = tmp_path_factory.mktemp("refcwd")
    d = root / "test" / "grad"
    d.mkdir(parents=True)
    g = np.load(os.path.join(GOLD_DIR, "torch_kernel_goldens.npz"))
    for k in g.files:
        if not k.startswith("wd0_"):
            g[k].astype(np.int32 if k in INT_FILES else np.float32).tofile(str(d / (k + ".bin")))
    return str(root)


@pytest.mark.parametrize("name", KERNEL_TESTS)
def test_reference_kernel_test_program_passes_on_the_cuda_backend(golden_bin_dir, name):
    exe = os.path.join(oc.KERNEL_TESTS_DIR, name)
    if not os.path.exists(exe):
        pytest.skip("reference kernel tests not built (oracle/build_ref.sh needs a reference checkout)")
    res = subprocess.run([exe], cwd=golden_bin_dir, capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, (name, res.stdout[-1500:], res.stderr[-500:])
    assert "FAIL" not in res.stdout, res.stdout[-1500:]


class Abi:
    def __init__(self, lib):
        vp, sz, ci = C.c_void_p, C.c_size_t, C.c_int
        self.lib = lib
        for name, res, args in [("backend_create", vp, []), ("backend_destroy", None, [vp]), ("backend_buffer_alloc", vp, [vp, sz]),
                                ("backend_buffer_free", None, [vp]), ("backend_buffer_map", vp, [vp]), ("backend_buffer_unmap", None, [vp]),
                                ("backend_buffer_size", sz, [vp]), ("backend_kernel_create", vp, [vp, C.c_char_p]),
                                ("backend_kernel_destroy", None, [vp]), ("backend_encode_begin", vp, [vp]),
                                ("backend_encode_dispatch", ci, [vp, vp, C.POINTER(vp), C.POINTER(sz), ci] + [ci] * 6),
                                ("backend_kernel_dispatch", ci, [vp, vp, C.POINTER(vp), C.POINTER(sz), ci] + [ci] * 6),
                                ("backend_encode_commit", None, [vp]), ("backend_encode_wait", None, [vp]),
                                ("backend_encode_wait_timed", C.c_double, [vp]), ("backend_get_allocated_memory", sz, [vp]),
                                ("backend_get_peak_allocated_memory", sz, [vp]), ("backend_get_gpu_busy_ms", C.c_double, [vp]),
                                ("backend_get_command_buffers", C.c_uint64, [vp]), ("backend_reset_gpu_timing", None, [vp]),
                                ("backend_synchronize", None, [vp])]:
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        self.ctx = lib.backend_create()
        assert self.ctx

    def buf(self, arr):
        arr = np.ascontiguousarray(arr)
        b = self.lib.backend_buffer_alloc(self.ctx, arr.nbytes)
        assert b
        C.memmove(self.lib.backend_buffer_map(b), arr.ctypes.data, arr.nbytes)   # no unmap: callers may omit it (tools/cli.c:115-121)
        return b

    def read(self, b, dtype, n):
        p = self.lib.backend_buffer_map(b)
        return np.frombuffer((C.c_char * (n * np.dtype(dtype).itemsize)).from_address(p), dtype).copy()

    def run(self, name, bufs, offsets=None, grid=1, timed=False):
        k = self.lib.backend_kernel_create(self.ctx, name.encode())
        assert k, name
        arr = (C.c_void_p * len(bufs))(*bufs)
        offs = (C.c_size_t * len(bufs))(*offsets) if offsets else None
        enc = self.lib.backend_encode_begin(self.ctx)
        assert self.lib.backend_encode_dispatch(enc, k, arr, offs, len(bufs), grid, 1, 1, 32, 1, 1) == 0
        self.lib.backend_encode_commit(enc)
        ms = self.lib.backend_encode_wait_timed(enc) if timed else self.lib.backend_encode_wait(enc)
        self.lib.backend_kernel_destroy(k)
        return ms


@pytest.fixture()
def abi(product):
    a = Abi(product)
    yield a
    product.backend_destroy(a.ctx)


def test_buffers_names_offsets_and_counters(abi, product):
    lib = abi.lib
    assert not lib.backend_buffer_alloc(abi.ctx, 0)                         # size 0 -> NULL (src/backend/metal/device.m:117)
    assert not lib.backend_kernel_create(abi.ctx, b"no_such_kernel")        # unknown name -> NULL, callers degrade
    assert not lib.backend_kernel_create(abi.ctx, b"residual_rmsnorm_forward")
    b = lib.backend_buffer_alloc(abi.ctx, 4096)
    assert lib.backend_buffer_size(b) == 4096 and lib.backend_get_allocated_memory(abi.ctx) >= 4096
    assert not abi.read(b, np.float32, 1024).any()                          # fresh buffers read as zero
    # zero_buffer with a byte offset into the data buffer AND into a shared int array (src/baremetal/scheduler.c:1378-1381)
    data = abi.buf(np.arange(64, dtype=np.float32) + 1)
    counts = abi.buf(np.array([0, 0, 16, 0], np.int32))
    abi.run("zero_buffer", [data, counts], offsets=[8 * 4, 2 * 4])
    got = abi.read(data, np.float32, 64)
    assert not got[8:24].any() and got[:8].all() and got[24:].all()
    # add_forward twice through one encoder: in-order execution with visibility between dispatches
    x, y, n = abi.buf(np.full(100, 1.5, np.float32)), abi.buf(np.full(100, 2.0, np.float32)), abi.buf(np.array([100], np.int32))
    k = lib.backend_kernel_create(abi.ctx, b"add_forward")
    enc = lib.backend_encode_begin(abi.ctx)
    for _ in range(3):   # y = x + y, three times
        arr = (C.c_void_p * 4)(x, y, y, n)
        assert lib.backend_encode_dispatch(enc, k, arr, None, 4, 100, 1, 1, 32, 1, 1) == 0
    lib.backend_encode_commit(enc)
    before = lib.backend_get_command_buffers(abi.ctx)
    assert lib.backend_encode_wait_timed(enc) >= 0.0
    assert lib.backend_get_command_buffers(abi.ctx) == before + 1 and lib.backend_get_gpu_busy_ms(abi.ctx) >= 0.0
    assert np.array_equal(abi.read(y, np.float32, 100), np.full(100, 6.5, np.float32))
    # a host write through a pointer obtained earlier is seen by the next (blocking) dispatch
    px = lib.backend_buffer_map(x)
    np.frombuffer((C.c_char * 400).from_address(px), np.float32)[:] = -6.5
    arr = (C.c_void_p * 4)(x, y, y, n)
    assert lib.backend_kernel_dispatch(abi.ctx, k, arr, None, 4, 100, 1, 1, 32, 1, 1) == 0
    assert not abi.read(y, np.float32, 100).any()
    lib.backend_kernel_destroy(k)
    for h in (b, data, counts, x, y, n):
        lib.backend_buffer_free(h)
    assert lib.backend_get_peak_allocated_memory(abi.ctx) >= 4096


def test_slot_order_of_the_matmul_and_attention_backward_kernels(abi, goldens):
    """The cases of test/matmul_bwd_test.c and test/attn_bwd_test.c dispatched through backend_encode_dispatch from Python."""
    g = goldens
    par = abi.buf(np.array([3, 16, 8, 0], np.int32))   # {BT, C, OC}
    gout, w, inp = abi.buf(g["gout"]), abi.buf(g["w"]), abi.buf(g["inp"])
    ginp, gw = abi.buf(np.zeros(48, np.float32)), abi.buf(np.zeros(128, np.float32))
    abi.run("matmul_backward_inp", [gout, w, ginp, par], grid=48)
    abi.run("matmul_backward_w", [gout, inp, gw, par], grid=128)
    abi.run("matmul_backward_w_tiled", [gout, inp, gw, par], grid=128)   # '+=': a second pass doubles the gradient
    assert oc.rel_err(abi.read(ginp, np.float32, 48), g["ginp"]) < 1e-5
    assert oc.rel_err(abi.read(gw, np.float32, 128), 2 * g["gw"]) < 1e-5
    NH, NKV, HD, S = 4, 2, 4, 3
    par = abi.buf(np.array([NH, S, HD, NKV, 2] + [0] * 11, np.int32))
    sc = abi.buf(np.array([0.5], np.float32))
    q, k, v, go = abi.buf(g["attn_Q"]), abi.buf(g["attn_K"]), abi.buf(g["attn_V"]), abi.buf(g["attn_gout"])
    gq, gk, gv = abi.buf(np.zeros(48, np.float32)), abi.buf(np.zeros(24, np.float32)), abi.buf(np.zeros(24, np.float32))
    ms = abi.run("attention_backward", [go, q, k, v, gq, gk, gv, par, sc], grid=NH * S, timed=True)
    assert ms >= 0.0
    for got, ref in ((gq, "attn_gQ"), (gk, "attn_gK"), (gv, "attn_gV")):
        assert oc.cosine(abi.read(got, np.float32, g[ref].size), g[ref]) > 0.9999
