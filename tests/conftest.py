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
TINY = {"A": TINY_A, "B": TINY_B}
BLOCK = {"A": 16, "B": 8}


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """Model folders (config.json + model.safetensors, float32 random weights) for both tiny configurations."""
    import hfcpu_b200
    from hfcpu_b200.config import config_from_dict
    out = {}
    for name, d in TINY.items():
        folder = str(tmp_path_factory.mktemp(f"tiny_{name}"))
        hfcpu_b200.write_random_model(config_from_dict(d), folder, seed=11 + len(out), dtype=torch.float32)
        out[name] = folder
    return out


@pytest.fixture
def emu():
    """Install the torch stand-in for the CUDA library for the duration of a test."""
    from hfcpu_b200 import kernels
    from emu_backend import EmuBackend
    old = kernels._backend
    kernels.set_backend(EmuBackend())
    yield
    kernels.set_backend(old)
