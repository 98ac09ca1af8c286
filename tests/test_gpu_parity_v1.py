"""The reference's architecture parity harness (test/parity/parity.c) as the CLI's `parity` sub-command, run on a committed
`baremetal.parity/v1` fixture whose ground truth is Hugging Face's LlamaForCausalLM in float32 (tests/golden/make_parity_fixture.py).
The model is rebuilt from its seed and exported with bm_save_weights, so the test also covers the safetensors round trip."""
import json
import os
import subprocess

import pytest

import bmapi

ROOT = bmapi.ROOT
CLI = os.path.join(ROOT, "bare.metal_b200", "baremetal-train")
FIXTURE = os.path.join(ROOT, "tests", "golden", "parity_v1", "tiny.json")


def _export_fixture_model(tmp_path):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_parity_fixture", os.path.join(ROOT, "tests", "golden", "make_parity_fixture.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = str(tmp_path / "model")
    mod.export_model(out)
    return out


def test_fixture_is_in_the_reference_format():
    fx = json.load(open(FIXTURE))
    assert fx["format"] == "baremetal.parity/v1" and fx["precision"] == "fp32"
    assert len(fx["prompt_token_ids"]) == 88 and len(fx["generated_token_ids"]) == 48
    assert os.path.getsize(os.path.join(os.path.dirname(FIXTURE), fx["logits_file"])) == 4 * fx["vocab_size"]


def test_parity_subcommand_reports_usage_and_missing_files():
    r = subprocess.run([CLI, "parity"], capture_output=True, text=True)
    assert r.returncode == 2 and "--fixture" in r.stderr
    r = subprocess.run([CLI, "parity", "--model", "/nonexistent", "--fixture", "/nonexistent.json"], capture_output=True, text=True)
    assert r.returncode == 1 and "cannot read fixture" in r.stderr


@pytest.mark.gpu
def test_session_passes_the_parity_harness_against_transformers(tmp_path):
    model_dir = _export_fixture_model(tmp_path)
    r = subprocess.run([CLI, "parity", "--model", model_dir, "--fixture", FIXTURE], capture_output=True, text=True, timeout=300)
    print(r.stdout, r.stderr)
    assert r.returncode == 0 and "PARITY PASS" in r.stdout
    assert "tokens: match (48/48)" in r.stdout
    cos = float(r.stdout.split("logits cos:")[1].split()[0])
    assert cos > 0.999999


@pytest.mark.gpu
def test_parity_harness_fails_on_a_wrong_model(tmp_path):
    """A different seed must not pass: the harness really compares."""
    import ctypes as C
    lib = bmapi.load_product()
    lib.bm_save_weights.argtypes = [C.c_void_p, C.c_char_p]
    a = bmapi.make_arch("tiny")
    src = str(tmp_path / "other.bin")
    bmapi.write_bin_checkpoint(src, a, bmapi.make_weights(a, seed=8, layer_scale=8.0))
    model = lib.bm_create_model(None, C.byref(a))
    lib.bm_load_weights(model, src.encode())
    out = str(tmp_path / "other")
    lib.bm_save_weights(model, out.encode())
    lib.bm_destroy_model(model)
    r = subprocess.run([CLI, "parity", "--model", out, "--fixture", FIXTURE], capture_output=True, text=True, timeout=300)
    assert r.returncode == 1 and "PARITY FAIL" in r.stdout
