"""The shared library loads on a machine without a GPU and exports every function the public headers declare.
No compute entry point is called here."""
import ctypes as C
import os
import re

import bmapi

ROOT = bmapi.ROOT
DECL = re.compile(r"^\s*(?:[A-Za-z_][\w\s\*]*?)\b((?:bm|bmc|bmx|backend)_[a-z0-9_]+)\s*\(", re.M)


def declared_functions(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    names = set(DECL.findall(text))
    # typedef'd callback and static inline helpers are not exports
    return {n for n in names if n not in ("bm_token_cb_t",) and not re.search(r"static\s+inline[^;{]*\b" + n + r"\b", text)}


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(bmapi.LIB_PATH)
    total = 0
    for header in ("baremetal.h", "baremetal_ext.h", "bm_cuda_backend.h", "backend.h"):
        names = declared_functions(header)
        assert len(names) > 10, header
        missing = [n for n in sorted(names) if not hasattr(lib, n)]
        assert not missing, f"{header}: not exported: {missing}"
        total += len(names)
    assert total > 80


def test_reference_api_surface_is_complete():
    """Every function of the reference's public header is present with the same name (baremetal.h:120-206)."""
    expected = """bm_create bm_destroy bm_get_supported_precision bm_create_model bm_load_weights bm_save_weights bm_destroy_model
    bm_compile bm_autotune bm_load_adapter bm_create_session bm_forward bm_step bm_reset_session bm_destroy_session
    bm_profile_begin bm_profile_end bm_run_tokens bm_create_sampler bm_sample bm_destroy_sampler bm_create_tokenizer bm_encode
    bm_decode bm_destroy_tokenizer bm_create_trainer bm_train_step bm_train_step_masked bm_train_eval_masked bm_load_state
    bm_save_state bm_train_flush bm_save_adapter bm_train_profile_begin bm_train_profile_end bm_destroy_trainer
    bm_get_num_parameters bm_get_arch_name bm_print_model_info""".split()
    lib = C.CDLL(bmapi.LIB_PATH)
    assert len(expected) == 39
    for n in expected:
        assert hasattr(lib, n), n


def test_reference_backend_abi_is_complete():
    """The 22 functions of the reference's internal backend interface (src/backend/backend.h:17-67), by name."""
    expected = """backend_create backend_destroy backend_get_allocated_memory backend_get_peak_allocated_memory backend_get_device_info
    backend_get_gpu_busy_ms backend_get_command_buffers backend_reset_gpu_timing backend_encode_wait_timed backend_buffer_alloc
    backend_buffer_free backend_buffer_map backend_buffer_unmap backend_buffer_size backend_kernel_create backend_kernel_destroy
    backend_kernel_dispatch backend_synchronize backend_encode_begin backend_encode_dispatch backend_encode_commit
    backend_encode_wait""".split()
    lib = C.CDLL(bmapi.LIB_PATH)
    assert len(expected) == 22
    assert set(expected) == declared_functions("backend.h")
    for n in expected:
        assert hasattr(lib, n), n


def test_struct_layouts_match_the_reference_header():
    # bm_arch_t: 22 ints/enums, float, enum, 4 floats = 112 bytes; bm_train_config_t: 6 floats + 6 ints + float + 2 ints = 60 bytes
    assert C.sizeof(bmapi.BmArch) == 112
    assert C.sizeof(bmapi.BmTrainConfig) == 60
