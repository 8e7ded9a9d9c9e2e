"""Weights by tensor name: dtype policy, the one error that lists everything, hostile files, random weights."""
import json
import os
import struct

import pytest
import torch

from conftest import TINY_A, TINY_B


def _specs(d):
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    return config_from_dict(d), build_model_specs(config_from_dict(d))


def test_names_and_shapes_of_the_checkpoint():
    _, specs = _specs(TINY_B)
    by = {s.name: s.shape for s in specs}
    assert by["model.embed_tokens.weight"] == (1000, 192) and by["lm_head.weight"] == (1000, 192)
    assert by["model.layers.2.self_attn.q_proj.weight"] == (192, 192) and by["model.layers.2.self_attn.k_proj.bias"] == (96,)
    assert by["model.layers.0.mlp.gate_proj.weight"] == (320, 192) and by["model.layers.0.mlp.down_proj.weight"] == (192, 320)
    assert by["model.norm.weight"] == (192,) and len(by) == 3 + 3 * 12
    _, tied = _specs(TINY_A)
    head = [s for s in tied if s.name == "lm_head.weight"]
    assert head and head[0].optional                           # a tied head reads the embedding (src/model.c:156-158)


def test_random_model_round_trip_and_dtype_policy(tmp_path):
    import hfcpu_b200
    from hfcpu_b200.weights import load_tensors
    cfg, specs = _specs(TINY_A)
    hfcpu_b200.write_random_model(cfg, str(tmp_path / "bf"), seed=1, dtype=torch.bfloat16)
    hfcpu_b200.write_random_model(cfg, str(tmp_path / "f32"), seed=1, dtype=torch.float32)
    again = str(tmp_path / "again")
    hfcpu_b200.write_random_model(cfg, again, seed=1, dtype=torch.float32)
    cpu = torch.device("cpu")
    bf_bf = load_tensors(str(tmp_path / "bf"), specs, torch.bfloat16, cpu)
    bf_32 = load_tensors(str(tmp_path / "bf"), specs, torch.float32, cpu)
    f32_bf = load_tensors(str(tmp_path / "f32"), specs, torch.bfloat16, cpu)
    f32_again = load_tensors(again, specs, torch.float32, cpu)
    name = "model.layers.1.mlp.up_proj.weight"
    assert bf_bf[name].dtype == torch.bfloat16                 # 16-bit stays 16-bit in a bfloat16 run
    assert bf_32[name].dtype == torch.float32 and torch.equal(bf_32[name], bf_bf[name].float())   # widening is exact
    assert f32_bf[name].dtype == torch.float32                 # a tensor stored in 32-bit stays so
    assert torch.equal(f32_bf[name], f32_again[name])          # same seed, same values, whatever the order
    w = f32_again["model.layers.0.input_layernorm.weight"]
    assert abs(float(w.mean()) - 1) < 0.02 and 0.001 < float(f32_again[name].std()) < 0.05
    other = str(tmp_path / "other")
    hfcpu_b200.write_random_model(cfg, other, seed=2, dtype=torch.float32)
    assert not torch.equal(load_tensors(other, specs, torch.float32, cpu)[name], f32_again[name])


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    from hfcpu_b200.weights import WeightError, load_tensors, random_tensors, weights_path, write_safetensors
    cfg, specs = _specs(TINY_A)
    t = random_tensors(specs, 0, torch.float32)
    del t["model.norm.weight"], t["model.layers.1.self_attn.v_proj.bias"]
    t["model.layers.0.mlp.up_proj.weight"] = torch.zeros(176, 63)
    t["model.layers.9.extra"] = torch.zeros(3)
    t["lm_head.weight"] = torch.zeros(512, 64)                 # a copy of the tied head is tolerated
    cfg.save(str(tmp_path))
    write_safetensors(weights_path(str(tmp_path)), t)
    with pytest.raises(WeightError) as e:
        load_tensors(str(tmp_path), specs, torch.float32, torch.device("cpu"))
    msg = str(e.value)
    assert "missing (2): " in msg and "model.norm.weight" in msg and "model.layers.1.self_attn.v_proj.bias" in msg
    assert "unexpected (1): model.layers.9.extra" in msg
    assert "tensor 'model.layers.0.mlp.up_proj.weight' has shape 176x63, expected 176x64" in msg
    assert e.value.missing and e.value.unexpected and e.value.misshapen


def test_integer_tables_become_int32(tmp_path):
    from hfcpu_b200.weights import TensorSpec, load_tensors, weights_path, write_safetensors
    write_safetensors(weights_path(str(tmp_path)), {"table": torch.arange(6, dtype=torch.int64).view(2, 3),
                                                    "w": torch.ones(2, dtype=torch.float16)})
    t = load_tensors(str(tmp_path), [TensorSpec("table", (2, 3), init="int"), TensorSpec("w", (2,))], torch.bfloat16,
                     torch.device("cpu"))
    assert t["table"].dtype == torch.int32 and t["table"].tolist() == [[0, 1, 2], [3, 4, 5]] and t["w"].dtype == torch.bfloat16


def test_hostile_files_are_refused(tmp_path):
    from hfcpu_b200.weights import SafetensorsFile, WeightFormatError
    p = str(tmp_path / "model.safetensors")

    def expect(data, what):
        open(p, "wb").write(data)
        with pytest.raises(WeightFormatError, match=what):
            SafetensorsFile(p)
    expect(b"abc", "too short")
    expect(struct.pack("<Q", 1 << 40) + b"{}", "header length")
    expect(struct.pack("<Q", 4) + b"nope", "not valid JSON")
    expect(struct.pack("<Q", 2) + b"[]", "JSON object")
    h = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    expect(struct.pack("<Q", len(h)) + h + b"\0" * 8, "does not match")           # data runs past the file
    h = json.dumps({"t": {"dtype": "F32", "shape": [5], "data_offsets": [0, 16]}}).encode()
    expect(struct.pack("<Q", len(h)) + h + b"\0" * 16, "does not match")          # shape and extent disagree
    h = json.dumps({"t": {"dtype": "Q4_K", "shape": [4], "data_offsets": [0, 16]}}).encode()
    expect(struct.pack("<Q", len(h)) + h + b"\0" * 16, "unsupported dtype")
    h = json.dumps({"t": {"dtype": "F32"}}).encode()
    expect(struct.pack("<Q", len(h)) + h, "malformed entry")
    with pytest.raises(WeightFormatError, match="no such file"):
        SafetensorsFile(str(tmp_path / "absent"))
    # truncation at every length of a good file is refused or leaves every tensor inside the file
    from hfcpu_b200.weights import write_safetensors
    write_safetensors(p, {"a": torch.ones(3, 5), "b": torch.zeros(7, dtype=torch.bfloat16)})
    good = open(p, "rb").read()
    for n in range(len(good)):
        open(p, "wb").write(good[:n])
        try:
            f = SafetensorsFile(p)
        except WeightFormatError:
            continue
        for name in f.names():
            f.tensor(name)
        f.close()


def _shard(folder, tensors, n_shards, with_index, cfg):
    """Write ``tensors`` as ``n_shards`` files named like a published checkpoint's, optionally with an index."""
    from hfcpu_b200.weights import write_safetensors
    os.makedirs(folder, exist_ok=True)
    cfg.save(folder)
    names = sorted(tensors)
    parts = [names[i::n_shards] for i in range(n_shards)]
    wmap = {}
    for i, part in enumerate(parts):
        fn = f"model-{i + 1:05d}-of-{n_shards:05d}.safetensors"
        write_safetensors(os.path.join(folder, fn), {n: tensors[n] for n in part})
        wmap.update({n: fn for n in part})
    if with_index:
        with open(os.path.join(folder, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": 0}, "weight_map": wmap}, f)
    return wmap


@pytest.mark.parametrize("with_index", [True, False])
def test_sharded_folders_load_like_a_single_file(tmp_path, with_index):
    from hfcpu_b200.weights import find_weight_files, load_tensors, random_tensors, weights_path, write_safetensors
    cfg, specs = _specs(TINY_B)
    t = random_tensors(specs, 3, torch.bfloat16)
    one, many = str(tmp_path / "one"), str(tmp_path / "many")
    cfg.save(one)
    write_safetensors(weights_path(one), t)
    _shard(many, t, 3, with_index, cfg)
    files, index = find_weight_files(many)
    assert len(files) == 3 and (index is not None) == with_index
    a = load_tensors(one, specs, torch.bfloat16, torch.device("cpu"))
    b = load_tensors(many, specs, torch.bfloat16, torch.device("cpu"))
    assert set(a.keys()) == set(b.keys()) == set(t)
    assert all(torch.equal(a[n], b[n]) and torch.equal(a[n], t[n]) for n in t)
    assert b.meta("model.layers.1.mlp.up_proj.weight") == (torch.bfloat16, (320, 192))
    assert len(b.paths()) == 3


def test_sharded_folder_errors(tmp_path):
    from hfcpu_b200.weights import WeightError, WeightFormatError, load_tensors, random_tensors, write_safetensors
    cfg, specs = _specs(TINY_A)
    cpu = torch.device("cpu")
    t = random_tensors(specs, 3, torch.float32)
    # a tensor missing from its shard, one unexpected, one misshapen: one error over all shards
    bad = dict(t)
    del bad["model.layers.1.mlp.down_proj.weight"]
    bad["model.layers.0.self_attn.k_proj.bias"] = torch.zeros(31)
    bad["stray.weight"] = torch.zeros(2)
    folder = str(tmp_path / "bad")
    wmap = _shard(folder, bad, 3, True, cfg)
    with pytest.raises(WeightError) as e:
        load_tensors(folder, specs, torch.float32, cpu)
    msg = str(e.value)
    assert "missing (1): model.layers.1.mlp.down_proj.weight" in msg and "unexpected (1): stray.weight" in msg
    assert "tensor 'model.layers.0.self_attn.k_proj.bias' has shape 31, expected 32" in msg
    # the index names a tensor that its file does not hold
    folder = str(tmp_path / "moved")
    wmap = _shard(folder, t, 3, True, cfg)
    wmap["model.norm.weight"] = [f for f in set(wmap.values()) if f != wmap["model.norm.weight"]][0]
    json.dump({"weight_map": wmap}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    with pytest.raises(WeightError, match="tensor 'model.norm.weight' is not in the file the index names"):
        load_tensors(folder, specs, torch.float32, cpu)
    # a name in two shards
    folder = str(tmp_path / "twice")
    _shard(folder, t, 2, False, cfg)
    write_safetensors(os.path.join(folder, "extra.safetensors"), {"model.norm.weight": t["model.norm.weight"]})
    with pytest.raises(WeightFormatError, match="tensor 'model.norm.weight' is in extra.safetensors and model-0000"):
        load_tensors(folder, specs, torch.float32, cpu)
    # an index that names a file that is not there; an index that leaves the folder; no weights at all
    folder = str(tmp_path / "gone")
    wmap = _shard(folder, t, 3, True, cfg)
    os.remove(os.path.join(folder, "model-00002-of-00003.safetensors"))
    with pytest.raises(WeightFormatError, match="names model-00002-of-00003.safetensors, which is not in the folder"):
        load_tensors(folder, specs, torch.float32, cpu)
    json.dump({"weight_map": {"a": "../x.safetensors"}}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    with pytest.raises(WeightFormatError, match="leaves the model folder"):
        load_tensors(folder, specs, torch.float32, cpu)
    json.dump([1], open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    with pytest.raises(WeightFormatError, match="not an index"):
        load_tensors(folder, specs, torch.float32, cpu)
    empty = str(tmp_path / "empty")
    os.makedirs(empty)
    with pytest.raises(WeightFormatError, match="no such file"):
        load_tensors(empty, specs, torch.float32, cpu)


def test_tensors_are_made_one_at_a_time_and_shared_ones_once(tmp_path, emu):
    """Binding asks the source for each tensor when its part needs it; the embedding of a tied head is made once."""
    import hfcpu_b200
    from hfcpu_b200.weights import CheckpointSource
    cfg, specs = _specs(TINY_A)
    folder = hfcpu_b200.write_random_model(cfg, str(tmp_path / "m"), seed=1, dtype=torch.float32)
    made = []
    orig = CheckpointSource._make

    def spy(self, name):
        made.append(name)
        return orig(self, name)
    CheckpointSource._make = spy
    try:
        model = hfcpu_b200.load_model(folder, torch.float32, "cpu")
    finally:
        CheckpointSource._make = orig
    assert sorted(made) == sorted(s.name for s in specs if s.name != "lm_head.weight")        # each exactly once
    assert model.head.weight.data_ptr() == model.embedding.table.data_ptr()
    assert model.files == [os.path.join(folder, "model.safetensors")]
    att = model.layers[0].mixer
    assert att.w_qkv.shape == (4 * 16 + 2 * 2 * 16, 64) and model.layers[0].ffn.w_gate_up.shape == (2 * 176, 64)
    # the fused buffers hold what stacking the loaded tensors would give
    src = hfcpu_b200.weights.load_tensors(folder, specs, torch.float32, torch.device("cpu"))
    p = "model.layers.0."
    assert torch.equal(att.w_qkv, torch.cat([src[p + f"self_attn.{x}_proj.weight"] for x in "qkv"]))
    g, u = src[p + "mlp.gate_proj.weight"], src[p + "mlp.up_proj.weight"]
    assert torch.equal(model.layers[0].ffn.w_gate_up, torch.stack([g, u], 1).reshape(352, 64))


def test_tensor_core_product_refuses_a_misaligned_bias_before_launching():
    """The many-token epilogue reads the bias sixteen bytes at a time: a bias (or operand) that is not 16-byte aligned is
    answered HFB_ENOTSUP from the argument check, before anything touches a GPU (none is needed for this test)."""
    import ctypes
    from ctypes import c_int, c_size_t, c_void_p
    from hfcpu_b200.kernels import build
    lib = ctypes.CDLL(build.build())
    lib.hfb_last_error.restype = ctypes.c_char_p
    args = lambda bias, a=4096: (c_void_p(a), c_void_p(8192), c_void_p(bias), c_int(1), c_void_p(16384), c_int(1), c_int(0),
                                 c_int(256), c_int(64), c_int(64), c_void_p(0), c_size_t(0), c_void_p(0))
    for bias in (2, 4, 8):
        assert lib.hfb_linear_tc(*args(bias)) == 2 and b"aligned" in lib.hfb_last_error()
        assert lib.hfb_linear_tc_noalloc(*args(bias)[:10], c_void_p(0)) == 2
    assert lib.hfb_linear_tc(*args(32, a=4098)) == 2
