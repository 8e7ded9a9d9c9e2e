import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


# Two tiny configurations that differ in every size and option.
TINY_A = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, intermediate_size=176, vocab_size=512,
              max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True,
              use_sliding_window=False, hidden_act="silu")
TINY_B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=3, hidden_size=192,
              num_attention_heads=6, num_key_value_heads=3, head_dim=32, intermediate_size=320, vocab_size=1000,
              max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=1e6, tie_word_embeddings=False,
              use_sliding_window=True, sliding_window=64, max_window_layers=1, hidden_act="silu")
# A third one whose sizes the tensor-core kernels take (head_dim 128, widths that are multiples of 8), so that the
# replay tests drive those kernels too, with a window on its second layer.
TINY_C = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=2, hidden_size=256,
              num_attention_heads=6, num_key_value_heads=2, head_dim=128, intermediate_size=456, vocab_size=1032,
              max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=50000.0, tie_word_embeddings=False,
              use_sliding_window=True, sliding_window=96, max_window_layers=1, hidden_act="silu")
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
BLOCK = {"A": 16, "B": 8, "C": 16}


def make_folder(cfg_dict, folder, seed, dtype, sharp=4.0, std=0.05):
    """Write a model folder with random weights whose attention is far from uniform: the query and key
    projections are scaled up so that single scores stand out and a wrong or missing key shows."""
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    from hfcpu_b200.weights import random_tensors, write_safetensors, weights_path
    cfg = config_from_dict(cfg_dict)
    cfg.save(folder)
    tensors = random_tensors(build_model_specs(cfg), seed, torch.float32, std=std)
    for name in tensors:
        if ".q_proj." in name or ".k_proj." in name:
            tensors[name] = tensors[name] * sharp
    write_safetensors(weights_path(folder), {k: v.to(dtype) for k, v in tensors.items()})
    return folder


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """Model folders for both tiny configurations, stored in float32 ("A", "B") and bfloat16 ("A16", "B16")."""
    out = {}
    for i, (name, d) in enumerate(TINY.items()):
        out[name] = make_folder(d, str(tmp_path_factory.mktemp(f"tiny_{name}")), 11 + i, torch.float32)
        # bfloat16 storage: smaller weights, so that rounding of sharp scores does not swamp the comparison
        out[name + "16"] = make_folder(d, str(tmp_path_factory.mktemp(f"tiny_{name}16")), 11 + i, torch.bfloat16,
                                       std=0.02)
    return out


_PLAIN_CACHE = {}


def plain_logits(folder, ids):
    """Logits of the plain implementation (float64) for every position of ``ids``, cached per (folder, ids)."""
    import plain_qwen2 as plain
    key = (folder, tuple(ids))
    if key not in _PLAIN_CACHE:
        cfg, W = plain.read_folder(folder)
        _PLAIN_CACHE[key] = plain.forward(cfg, W, list(ids))
    return _PLAIN_CACHE[key]


def make_requests(name, lengths, seed=0):
    g = torch.Generator().manual_seed(seed)
    V = TINY[name]["vocab_size"]
    return {f"r{i}": torch.randint(0, V, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


SAMPLER_VOCAB, SAMPLER_ROWS = 1000, 6


def sampler_logits():
    """Rows of synthetic logits made from integer arithmetic only (the same on every machine): values in
    [-8, 8) on a grid of 2^-20, with ties at the top of some rows (lowest id wins) and one row that is nearly flat."""
    import numpy as np
    i = np.arange(SAMPLER_VOCAB, dtype=np.uint64)[None, :]
    r = np.arange(SAMPLER_ROWS, dtype=np.uint64)[:, None]
    x = (i * np.uint64(2654435761) + r * np.uint64(40503) + np.uint64(12345)) & np.uint64(0xFFFFFFFF)
    x ^= (x << np.uint64(13)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(17)
    x ^= (x << np.uint64(5)) & np.uint64(0xFFFFFFFF)
    L = ((x >> np.uint64(8)).astype(np.float32) / np.float32(1 << 24) * np.float32(16) - np.float32(8)).astype(np.float32)
    L[1, 900] = L[1, 17] = L[1].max()                      # a tie at the top: the lower id comes first
    L[2, 5] = L[2, 3] = L[2, 600] = np.float32(9.5)
    L[3] = (L[3] * np.float32(1 / 64)).astype(np.float32)  # nearly flat: thousands of candidates survive
    L[4, 123] = np.float32(30.0)                           # one token dominates
    return np.ascontiguousarray(L)


# Tolerances: max|a-b| / max|b| per logits row against the float64 plain implementation.
TOL = {"float32": 1e-4, "bfloat16": 3e-2}


@pytest.fixture
def emu():
    """Install the torch stand-in for the CUDA library for the duration of a test."""
    from hfcpu_b200 import kernels
    from emu_backend import EmuBackend
    old = kernels._backend
    kernels.set_backend(EmuBackend())
    yield
    kernels.set_backend(old)
