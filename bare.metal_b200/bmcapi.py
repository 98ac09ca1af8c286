"""ctypes access to the backend C ABI (include/bm_cuda_backend.h): a context, device buffers and typed calls of the bmc_* entry
points, plus the bf16 bit conversions their callers need. Used by the kernel workloads of bench.py and by the GPU tests."""
import ctypes as C

import numpy as np

BMC_F32, BMC_BF16 = 0, 1


def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return u.astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_round(x):
    return bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(np.shape(x))


class Backend:
    """A backend context plus typed wrappers; every call goes through the extern "C" entry points."""

    def __init__(self, lib):
        self.lib = lib
        lib.bmc_create.restype = C.c_void_p
        lib.bmc_alloc.restype = C.c_void_p
        lib.bmc_alloc.argtypes = [C.c_void_p, C.c_size_t]
        lib.bmc_free.argtypes = [C.c_void_p, C.c_void_p]
        lib.bmc_upload.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        lib.bmc_download.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        lib.bmc_memset.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t]
        lib.bmc_sync.argtypes = [C.c_void_p]
        lib.bmc_status.argtypes = [C.c_void_p]
        lib.bmc_destroy.argtypes = [C.c_void_p]
        lib.bmc_launch_count.restype = C.c_long
        lib.bmc_launch_count.argtypes = [C.c_void_p]
        vp, sz, ci, cf = C.c_void_p, C.c_size_t, C.c_int, C.c_float
        lib.bmc_adamw.argtypes = [vp, vp, vp, vp, ci, vp, vp, sz, C.POINTER(cf)]
        lib.bmc_add_forward.argtypes = [vp, ci, vp, vp, vp, sz]
        lib.bmc_cast_f32_to_bf16.argtypes = [vp, vp, vp, sz]
        lib.bmc_cast_bf16_to_f32.argtypes = [vp, vp, vp, sz]
        lib.bmc_seq_prefix_accumulate.argtypes = [vp, ci, vp, vp, ci, sz]
        self.ctx = lib.bmc_create(0)
        if not self.ctx:
            raise RuntimeError("bmc_create(0) failed: no sm_100 GPU (the backend has no CPU fallback)")
        self.bufs = []

    def close(self):
        for b in self.bufs:
            self.lib.bmc_free(self.ctx, b)
        self.lib.bmc_destroy(self.ctx)

    def alloc(self, nbytes):
        p = self.lib.bmc_alloc(self.ctx, max(int(nbytes), 16))
        assert p, "bmc_alloc failed"
        self.bufs.append(p)
        return p

    def put(self, arr, dtype=BMC_F32):
        """Upload a numpy array; float arrays are stored as fp32 or bf16 according to dtype."""
        if arr.dtype in (np.int32, np.uint8):
            host = np.ascontiguousarray(arr)
        elif dtype == BMC_BF16:
            host = f32_to_bf16_bits(arr)
        else:
            host = np.ascontiguousarray(arr, np.float32)
        p = self.alloc(host.nbytes)
        assert self.lib.bmc_upload(self.ctx, p, host.ctypes.data, host.nbytes) == 0
        assert self.lib.bmc_sync(self.ctx) == 0
        return p

    def zeros(self, n, dtype=BMC_F32):
        nbytes = n * (2 if dtype == BMC_BF16 else 4)
        p = self.alloc(nbytes)
        assert self.lib.bmc_memset(self.ctx, p, 0, nbytes) == 0
        return p

    def get(self, p, shape, dtype=BMC_F32, np_dtype=None):
        n = int(np.prod(shape))
        if np_dtype is not None:
            host = np.empty(n, np_dtype)
        elif dtype == BMC_BF16:
            host = np.empty(n, np.uint16)
        else:
            host = np.empty(n, np.float32)
        assert self.lib.bmc_download(self.ctx, host.ctypes.data, p, host.nbytes) == 0
        if np_dtype is None and dtype == BMC_BF16:
            host = bf16_bits_to_f32(host)
        return host.reshape(shape)

    def call(self, name, *args):
        """Call bmc_<name>(ctx, ...) converting ints -> c_int, floats -> c_float, None / addresses -> c_void_p."""
        fn = getattr(self.lib, "bmc_" + name)
        if fn.argtypes:
            rc = fn(self.ctx, *args)
        else:
            conv = []
            for a in args:
                if a is None:
                    conv.append(C.c_void_p(None))
                elif isinstance(a, Ptr):
                    conv.append(C.c_void_p(a.addr))
                elif isinstance(a, float):
                    conv.append(C.c_float(a))
                elif isinstance(a, (int, np.integer)):
                    conv.append(C.c_int(int(a)))
                else:
                    conv.append(a)
            rc = fn(C.c_void_p(self.ctx), *conv)
        return rc

    def ok(self, name, *args):
        rc = self.call(name, *args)
        assert rc == 0, f"bmc_{name} returned {rc}"
        st = self.lib.bmc_sync(self.ctx)
        assert st == 0, f"backend status {st} after bmc_{name}"


class Ptr:
    """A device address (with optional element offset) — distinguishes pointers from plain ints in Backend.call."""

    def __init__(self, addr, offset_bytes=0):
        self.addr = int(addr) + int(offset_bytes)
