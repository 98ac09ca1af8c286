"""Host-side behaviour that needs no GPU: synthetic inputs, file formats, model layout, loud failure without a device,
the greedy sampler, and the data-parallel bucket plan."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

import bmapi
import portk


def test_lcg_stream_matches_the_scalar_recurrence():
    s, out = 42, []
    for _ in range(200):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF  # bench/train_bench.c:286-290
        out.append(s % 49152)
    assert bmapi.lcg_tokens(200, 49152).tolist() == out
    x, y = bmapi.lcg_batch(3, 8, 1000)
    flat = bmapi.lcg_tokens(25, 1000)
    assert x.ravel().tolist() == flat[:24].tolist() and y.ravel().tolist() == flat[1:25].tolist()


def test_parameter_counts_of_the_named_models():
    for name, n in (("smollm2-135m", 134515008), ("smollm2-360m", 361821120)):
        a = bmapi.make_arch(name)
        total = sum(int(np.prod(shape)) for _, shape in bmapi.weight_shapes(a))
        assert total == n


def test_bin_checkpoint_round_trip_through_the_host_layer(product, tmp_path):
    lib = product
    a = bmapi.make_arch("tiny")
    w = bmapi.make_weights(a, seed=3)
    path = str(tmp_path / "tiny.bin")
    bmapi.write_bin_checkpoint(path, a, w)
    with open(path, "rb") as f:
        hdr = struct.unpack("<256i", f.read(1024))
    assert hdr[0] == 20250718 and hdr[3] == a.dim and hdr[8] == a.vocab_size and hdr[23] == 100000
    # bm_create_model / bm_load_weights are host-only and work without a GPU
    model = lib.bm_create_model(None, C.byref(a))
    assert model
    lib.bm_load_weights(model, path.encode())
    n = C.c_size_t()
    ptr = lib.bmx_model_weight_buffer(model, C.byref(n))
    flat = np.ctypeslib.as_array(ptr, (n.value,))
    expect = np.concatenate([w[k].ravel() for k, _ in bmapi.weight_shapes(a)])
    assert n.value == expect.size == lib.bm_get_num_parameters(model)
    assert np.array_equal(flat, expect)
    lib.bm_destroy_model(model)


def test_save_weights_round_trip_safetensors_and_bin(product, tmp_path):
    """bm_save_weights writes a Hugging Face safetensors directory (or the legacy .bin): an independent reader sees the Llama tensor
    names, shapes and values, and loading the export back gives the same buffer bit for bit."""
    from safetensors.numpy import load_file
    lib = product
    lib.bm_save_weights.argtypes = [C.c_void_p, C.c_char_p]
    a = bmapi.make_arch("gqa")
    w = bmapi.make_weights(a, seed=11)
    src = str(tmp_path / "src.bin")
    bmapi.write_bin_checkpoint(src, a, w)
    model = lib.bm_create_model(None, C.byref(a))
    lib.bm_load_weights(model, src.encode())
    out_dir, out_bin = str(tmp_path / "export"), str(tmp_path / "export.bin")
    lib.bm_save_weights(model, out_dir.encode())
    lib.bm_save_weights(model, out_bin.encode())
    assert open(out_bin, "rb").read() == open(src, "rb").read()
    t = load_file(os.path.join(out_dir, "model.safetensors"))
    assert len(t) == 9 * a.n_layers + 2 and "lm_head.weight" not in t
    assert np.array_equal(t["model.embed_tokens.weight"], w["embed"]) and np.array_equal(t["model.norm.weight"], w["lnfw"])
    for l in range(a.n_layers):
        for name, key in (("input_layernorm", "ln1w"), ("self_attn.q_proj", "qw"), ("self_attn.k_proj", "kw"), ("self_attn.v_proj", "vw"),
                          ("self_attn.o_proj", "ow"), ("post_attention_layernorm", "ln2w"), ("mlp.gate_proj", "gate"), ("mlp.up_proj", "up"),
                          ("mlp.down_proj", "down")):
            assert np.array_equal(t[f"model.layers.{l}.{name}.weight"], w[key][l]), (l, name)
    import json
    cfg = json.load(open(os.path.join(out_dir, "config.json")))
    assert cfg["hidden_size"] == a.dim and cfg["num_key_value_heads"] == a.n_kv_heads and cfg["tie_word_embeddings"] is True
    assert cfg["rope_theta"] == 100000.0 and cfg["rope_scaling"] is None
    back = lib.bm_create_model(None, C.byref(bmapi.make_arch("tiny")))   # the loader re-creates the buffers from config.json
    lib.bm_load_weights(back, out_dir.encode())
    n = C.c_size_t()
    flat = np.ctypeslib.as_array(lib.bmx_model_weight_buffer(back, C.byref(n)), (lib.bm_get_num_parameters(back),))
    assert np.array_equal(flat, np.concatenate([w[k].ravel() for k, _ in bmapi.weight_shapes(a)]))
    lib.bm_destroy_model(model)
    lib.bm_destroy_model(back)


def test_config_json_rope_scaling_is_parsed_or_refused(product, tmp_path):
    """rope_scaling of type llama3 reaches the architecture (src/baremetal/config.c:192-211); any other rule is refused, because the
    engine would otherwise rotate by the wrong frequencies without saying so; a key inside a nested object never shadows a
    top-level one."""
    from safetensors.numpy import save_file
    import json
    lib = product
    a = bmapi.make_arch("tiny")
    w = bmapi.make_weights(a)
    names = {"model.embed_tokens.weight": w["embed"], "model.norm.weight": w["lnfw"]}
    for l in range(a.n_layers):
        for name, key in (("input_layernorm", "ln1w"), ("self_attn.q_proj", "qw"), ("self_attn.k_proj", "kw"), ("self_attn.v_proj", "vw"),
                          ("self_attn.o_proj", "ow"), ("post_attention_layernorm", "ln2w"), ("mlp.gate_proj", "gate"), ("mlp.up_proj", "up"),
                          ("mlp.down_proj", "down")):
            names[f"model.layers.{l}.{name}.weight"] = np.ascontiguousarray(w[key][l])
    base = {"model_type": "llama", "text_config": {"hidden_size": 9999}, "hidden_size": a.dim, "intermediate_size": a.hidden_dim,
            "num_hidden_layers": a.n_layers, "num_attention_heads": a.n_heads, "num_key_value_heads": a.n_kv_heads,
            "vocab_size": a.vocab_size, "max_position_embeddings": 4096, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
            "tie_word_embeddings": True}
    lib.bmx_model_arch_field.restype = C.c_double
    lib.bmx_model_arch_field.argtypes = [C.c_void_p, C.c_char_p]
    for scaling, ok in (({"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                          "original_max_position_embeddings": 8192}, True), ({"type": "yarn", "factor": 4.0}, False), (None, True)):
        d = tmp_path / f"m_{'none' if scaling is None else scaling.get('rope_type', scaling.get('type'))}"
        d.mkdir()
        json.dump(dict(base, rope_scaling=scaling), open(d / "config.json", "w"))
        save_file(names, str(d / "model.safetensors"))
        m = lib.bm_create_model(None, C.byref(bmapi.make_arch("tiny")))
        lib.bm_load_weights(m, str(d).encode())
        loaded = lib.bm_get_num_parameters(m) > 0 and abs(lib.bmx_model_arch_field(m, b"rope_theta") - 500000.0) < 1
        assert loaded == ok, scaling
        if ok:
            assert lib.bmx_model_arch_field(m, b"dim") == a.dim   # not the 9999 of the nested object
            assert lib.bmx_model_arch_field(m, b"rope_scaling") == (1 if scaling else 0)
            if scaling:
                assert lib.bmx_model_arch_field(m, b"rope_factor") == 32.0 and lib.bmx_model_arch_field(m, b"rope_original_max") == 8192.0
        lib.bm_destroy_model(m)


def test_unsupported_architectures_are_rejected(product):
    lib = product
    for field in ("bias", "has_qk_norm", "has_ffn_post_norm", "gemma_norm", "embed_scale"):
        a = bmapi.make_arch("tiny")
        setattr(a, field, 1)
        assert not lib.bm_create_model(None, C.byref(a)), field  # bmt_arch_validate, src/baremetal/model.c:14-40
    a = bmapi.make_arch("tiny")
    a.weight_tie = 0
    assert not lib.bm_create_model(None, C.byref(a))


def test_no_gpu_means_no_context_not_a_fallback(product):
    """On a machine without an sm_100 GPU bm_create returns NULL; BM_DEVICE_CPU never yields a context."""
    lib = product
    assert not lib.bm_create(bmapi.BM_DEVICE_CPU)
    ctx = lib.bm_create(bmapi.BM_DEVICE_CUDA)
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = os.path.exists("/dev/nvidia0")
    if not has_gpu:
        assert not ctx
    elif ctx:
        lib.bm_destroy(ctx)


def test_out_of_scope_entry_points_return_their_failure_values(product):
    lib = product
    lib.bm_create_tokenizer.restype = C.c_void_p
    assert not lib.bm_create_session(None, None)  # no context: no session
    assert not lib.bm_create_tokenizer(b"/nonexistent")
    assert lib.bm_save_adapter(None, b"x") == -1


def _adapter_case(a, rank, seed, targets):
    """Random A [r][c] and B [oc][r] for every (layer, target) asked for."""
    rng = np.random.default_rng(seed)
    shapes = dict(bmapi.weight_shapes(a))
    entries = []
    for layer, tgt in targets:
        oc, c = shapes[bmapi.ADAPTER_WEIGHT_KEY[tgt]][1:]
        entries.append((layer, tgt, rng.standard_normal((rank, c), dtype=np.float32) * np.float32(0.1),
                        rng.standard_normal((oc, rank), dtype=np.float32) * np.float32(0.1)))
    return entries


def _merged(w, entries, rank, alpha):
    """The reference's merge (src/baremetal/adapter.c:201-208): fp32 sum over k in increasing order, then w += scale * sum."""
    out = {k: v.copy() for k, v in w.items()}
    scale = np.float32(alpha) / np.float32(rank)
    for layer, tgt, A, B in entries:
        acc = np.zeros((B.shape[0], A.shape[1]), np.float32)
        for k in range(rank):
            acc += B[:, k:k + 1] * A[k:k + 1, :]
        out[bmapi.ADAPTER_WEIGHT_KEY[tgt]][layer] += scale * acc
    return out


def _model_with_weights(lib, a, w, tmp_path):
    path = str(tmp_path / "base.bin")
    bmapi.write_bin_checkpoint(path, a, w)
    model = lib.bm_create_model(None, C.byref(a))
    lib.bm_load_weights(model, path.encode())
    n = C.c_size_t()
    flat = np.ctypeslib.as_array(lib.bmx_model_weight_buffer(model, C.byref(n)), (n.value,))
    return model, flat


def test_load_adapter_merges_every_target_into_the_host_weights(product, tmp_path):
    """bm_load_adapter adds (alpha / rank) * B * A to the projection each entry names and leaves everything else alone; the
    merged buffer equals the reference's arithmetic float for float."""
    lib = product
    a = bmapi.make_arch("gqa")
    w = bmapi.make_weights(a, seed=5)
    rank, alpha = 4, 12.0
    targets = [(l, t) for l in range(a.n_layers) for t in ("q", "k", "v", "o", "gate", "up", "down")][::-1]  # any order
    entries = _adapter_case(a, rank, 17, targets)
    path = str(tmp_path / "all.bmlora")
    bmapi.write_adapter_file(path, a, rank, alpha, entries)
    model, flat = _model_with_weights(lib, a, w, tmp_path)
    assert lib.bm_load_adapter(model, path.encode()) == 0
    want = _merged(w, entries, rank, alpha)
    expect = np.concatenate([want[k].ravel() for k, _ in bmapi.weight_shapes(a)])
    assert np.array_equal(flat, expect)
    for k in ("embed", "ln1w", "ln2w", "lnfw"):
        assert np.array_equal(want[k], w[k])
    # a second adapter on one projection of one layer stacks on the first
    one = _adapter_case(a, 2, 23, [(1, "down")])
    path2 = str(tmp_path / "one.bmlora")
    bmapi.write_adapter_file(path2, a, 2, 1.0, one)
    assert lib.bm_load_adapter(model, path2.encode()) == 0
    want2 = _merged(want, one, 2, 1.0)
    assert np.array_equal(flat, np.concatenate([want2[k].ravel() for k, _ in bmapi.weight_shapes(a)]))
    lib.bm_destroy_model(model)


def test_load_adapter_refuses_what_does_not_fit_the_model(product, tmp_path):
    """Failure values of src/baremetal/adapter.c:151-196: unreadable file, bad magic / version, another architecture, an entry of
    another rank, shape or target, a truncated payload; plus a layer index outside the model, which this build refuses."""
    lib = product
    a = bmapi.make_arch("gqa")
    w = bmapi.make_weights(a, seed=5)
    model, flat = _model_with_weights(lib, a, w, tmp_path)
    before = flat.copy()
    good = _adapter_case(a, 2, 1, [(0, "q")])
    p = str(tmp_path / "bad.bmlora")
    assert lib.bm_load_adapter(None, p.encode()) == -1
    assert lib.bm_load_adapter(model, None) == -1
    assert lib.bm_load_adapter(model, str(tmp_path / "missing").encode()) == -1
    for over in ({"magic": 0x12345678}, {"version": 2}, {"dim": a.dim + 1}, {"layers": a.n_layers + 1}, {"n_heads": a.n_heads * 2},
                 {"n_kv_heads": a.n_kv_heads + 1}, {"vocab": a.vocab_size - 1}, {"head_size": a.head_dim * 2}, {"rank": 0},
                 {"n_adapters": 0}, {"rank": 3}):
        bmapi.write_adapter_file(p, a, 2, 4.0, good, header_overrides=over)
        assert lib.bm_load_adapter(model, p.encode()) == -1, over
    _, _, A, B = good[0]
    for bad in ((0, "k", A, B),                       # q-sized B on the k projection: oc mismatch
                (0, 128, A, B),                       # not a target bit
                (0, 3, A, B),                         # two bits at once
                (a.n_layers, "q", A, B), (-1, "q", A, B),
                (0, "q", A[:, :-1], B)):              # c mismatch
        bmapi.write_adapter_file(p, a, 2, 4.0, [bad])
        assert lib.bm_load_adapter(model, p.encode()) == -1, bad[:2]
    bmapi.write_adapter_file(p, a, 2, 4.0, good)
    blob = open(p, "rb").read()
    for cut in (10, 44, 44 + 12, len(blob) - 4):
        open(p, "wb").write(blob[:cut])
        assert lib.bm_load_adapter(model, p.encode()) == -1, cut
    assert np.array_equal(flat, before)               # none of the refused files touched the weights
    open(p, "wb").write(blob)
    assert lib.bm_load_adapter(model, p.encode()) == 0
    assert not np.array_equal(flat, before)
    lib.bm_destroy_model(model)


def test_greedy_sampler_takes_the_first_maximum(product):
    lib = product
    rng = np.random.default_rng(0)
    for trial in range(20):
        V = int(rng.integers(5, 3000))
        logits = rng.standard_normal(V).astype(np.float32)
        if trial % 2:  # plant ties
            logits[rng.integers(0, V, 4)] = logits.max() + 1.0
        s = lib.bm_create_sampler(V, 0.0, 0.9, 1)
        got = lib.bm_sample(s, logits.ctypes.data_as(C.POINTER(C.c_float)))
        lib.bm_destroy_sampler(s)
        assert got == int(np.argmax(logits)) == portk.argmax(logits)


def test_state_file_reader_matches_the_documented_layout(tmp_path):
    path = tmp_path / "state.bin"
    with open(path, "wb") as f:
        f.write(struct.pack("<ii", 7, 2))
        for n in (3, 5):
            f.write(struct.pack("<Q", n))
            for k in range(3):
                f.write((np.arange(n, dtype=np.float32) + k).tobytes())
    step, tensors = bmapi.read_state_file(str(path))
    assert step == 7 and len(tensors) == 2
    assert tensors[1][2].tolist() == [2, 3, 4, 5, 6]


def test_dp_bucket_plan_partitions_the_parameters(product):
    lib = product
    lib.bmx_dp_plan_buckets.restype = C.c_int
    for L, per in ((32, 4), (30, 4), (2, 4), (7, 3), (5, 1)):
        layer_begin = (C.c_size_t * (L + 1))(*[100 * l for l in range(L + 1)])
        P = 100 * L + 50 + 7777
        n = lib.bmx_dp_plan_buckets(L, layer_begin, C.c_size_t(P), per, None, None, None, 0)
        b, e, r = (C.c_size_t * n)(), (C.c_size_t * n)(), (C.c_int * n)()
        assert lib.bmx_dp_plan_buckets(L, layer_begin, C.c_size_t(P), per, b, e, r, n) == n
        spans = sorted(zip(list(b), list(e)))
        assert spans[0][0] == 0 and spans[-1][1] == P
        assert all(spans[i][1] == spans[i + 1][0] for i in range(n - 1))  # exact partition, no overlap
        assert list(r)[-1] == -1 and list(r)[:-1] == sorted(list(r)[:-1], reverse=True)  # completion order of backward
        for bi, ri in zip(list(b)[:-1], list(r)[:-1]):
            assert bi == 100 * ri  # a bucket is complete when its lowest layer is
        if L > 1:
            # what is exchanged after backward has ended is exposed: layer 0 travels alone, and the embedding bucket is the last
            assert (b[n - 2], e[n - 2], r[n - 2]) == (0, 100, 0) and (b[n - 1], e[n - 1]) == (100 * L, P)


def _write_safetensors(path, tensors, dtype="F32"):
    import json
    header, blobs, off = {}, [], 0
    for name, arr in tensors.items():
        if dtype == "BF16":
            from bmcapi import f32_to_bf16_bits
            raw = f32_to_bf16_bits(arr).tobytes()
        else:
            raw = np.ascontiguousarray(arr, np.float32).tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


@pytest.mark.parametrize("dtype,sharded", [("F32", False), ("BF16", False), ("F32", True)])
def test_safetensors_directory_loader(product, tmp_path, dtype, sharded):
    """HF-style directory (config.json + *.safetensors with Llama tensor names) into the flat model buffer
    (the reference's loader: src/baremetal/checkpoint_st.c:430-671; its synthetic-shard test: test/sharded_load_test.c)."""
    import json
    lib = product
    a = bmapi.make_arch("tiny")
    w = bmapi.make_weights(a, seed=11)
    w["ln1w"] = np.random.default_rng(1).standard_normal(w["ln1w"].shape).astype(np.float32)
    cfg = {"model_type": "llama", "hidden_size": a.dim, "intermediate_size": a.hidden_dim, "num_hidden_layers": a.n_layers,
           "num_attention_heads": a.n_heads, "num_key_value_heads": a.n_kv_heads, "vocab_size": a.vocab_size, "head_dim": a.head_dim,
           "max_position_embeddings": 2048, "rms_norm_eps": 1e-5, "rope_theta": 100000.0, "tie_word_embeddings": True, "hidden_act": "silu"}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    names = {"ln1w": "input_layernorm.weight", "qw": "self_attn.q_proj.weight", "kw": "self_attn.k_proj.weight",
             "vw": "self_attn.v_proj.weight", "ow": "self_attn.o_proj.weight", "ln2w": "post_attention_layernorm.weight",
             "gate": "mlp.gate_proj.weight", "up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight"}
    tensors = {"model.embed_tokens.weight": w["embed"], "model.norm.weight": w["lnfw"]}
    for l in range(a.n_layers):
        for k, suffix in names.items():
            tensors[f"model.layers.{l}.{suffix}"] = w[k][l]
    if sharded:
        items = list(tensors.items())
        _write_safetensors(tmp_path / "model-00001-of-00002.safetensors", dict(items[:7]), dtype)
        _write_safetensors(tmp_path / "model-00002-of-00002.safetensors", dict(items[7:]), dtype)
        wm = {k: ("model-00001-of-00002.safetensors" if i < 7 else "model-00002-of-00002.safetensors") for i, (k, _) in enumerate(items)}
        (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": wm}))
    else:
        _write_safetensors(tmp_path / "model.safetensors", tensors, dtype)
    seed = bmapi.make_arch("tiny")
    seed.dim, seed.n_layers = 64, 1  # deliberately different: the directory's config.json decides
    model = lib.bm_create_model(None, C.byref(seed))
    lib.bm_load_weights(model, str(tmp_path).encode())
    n = C.c_size_t()
    flat = np.ctypeslib.as_array(lib.bmx_model_weight_buffer(model, C.byref(n)), (n.value,))
    expect = np.concatenate([w[k].ravel() for k, _ in bmapi.weight_shapes(a)])
    assert n.value == expect.size
    if dtype == "BF16":
        from bmcapi import bf16_round
        expect = bf16_round(expect)
    assert np.array_equal(flat, expect)
    assert lib.bmx_model_vocab_size(model) == a.vocab_size
    lib.bm_destroy_model(model)
