"""Writes a `baremetal.parity/v1` fixture (the format of the reference's test/parity/make_fixture.py and test/parity/parity.c)
for a random-init model of the family, with Hugging Face's LlamaForCausalLM in float32 as the ground truth — the same ground
truth the reference's own fixtures use, which need the real SmolLM2 weights and are therefore not replayable here.

The model is exported by the product's own bm_save_weights (a safetensors directory + config.json), loaded by transformers
from that directory, and the fixture holds the prompt, the greedy continuation and the full-vocabulary logits after the prompt.
The weights are not committed: tests rebuild them from the seed below.

    python tests/golden/make_parity_fixture.py        # CPU only; needs torch + transformers
"""
import ctypes as C
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "bare.metal_b200"))
import bmapi  # noqa: E402

ARCH, SEED, LAYER_SCALE, N_PROMPT, N_GEN = "tiny", 7, 8.0, 88, 48
OUT = os.path.join(HERE, "parity_v1")


def export_model(out_dir):
    """The fixture's model as a safetensors directory, written by bm_save_weights."""
    lib = bmapi.load_product()
    lib.bm_save_weights.argtypes = [C.c_void_p, C.c_char_p]
    a = bmapi.make_arch(ARCH)
    w = bmapi.make_weights(a, seed=SEED, layer_scale=LAYER_SCALE)
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "src.bin")
        bmapi.write_bin_checkpoint(src, a, w)
        model = lib.bm_create_model(None, C.byref(a))
        lib.bm_load_weights(model, src.encode())
        lib.bm_save_weights(model, out_dir.encode())
        lib.bm_destroy_model(model)
    return a


def main():
    import torch
    from transformers import AutoModelForCausalLM
    os.makedirs(OUT, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        model_dir = os.path.join(tmp, "model")
        a = export_model(model_dir)
        prompt = [int(t) for t in np.random.default_rng(SEED).integers(0, a.vocab_size, N_PROMPT)]
        model = AutoModelForCausalLM.from_pretrained(model_dir, dtype=torch.float32)
        model.eval()
        with torch.no_grad():
            out = model(input_ids=torch.tensor([prompt]), use_cache=True)
            past = out.past_key_values
            logits = out.logits[0, -1].float().numpy()
            nxt = int(np.argmax(logits))
            generated = [nxt]
            margins = [float(np.sort(logits)[-1] - np.sort(logits)[-2])]
            for _ in range(N_GEN - 1):
                out = model(input_ids=torch.tensor([[nxt]]), past_key_values=past, use_cache=True)
                past = out.past_key_values
                step = out.logits[0, -1].float().numpy()
                margins.append(float(np.sort(step)[-1] - np.sort(step)[-2]))
                nxt = int(np.argmax(step))
                generated.append(nxt)
    logits.astype("<f4").tofile(os.path.join(OUT, f"{ARCH}.logits.f32"))
    fixture = {"format": "baremetal.parity/v1", "model": f"random-init {ARCH} (seed {SEED}, layer scale {LAYER_SCALE})", "precision": "fp32",
               "prompt_token_ids": prompt, "generated_token_ids": generated, "vocab_size": int(a.vocab_size),
               "logits_file": f"{ARCH}.logits.f32", "min_top2_margin": min(margins)}
    json.dump(fixture, open(os.path.join(OUT, f"{ARCH}.json"), "w"), indent=1)
    print("wrote", OUT, "distinct generated ids:", len(set(generated)), "smallest top-2 margin:", min(margins))


if __name__ == "__main__":
    main()
