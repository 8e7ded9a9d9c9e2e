"""The tensor-core kernels at the layer sizes of the benchmark configurations (two layers each): a prompt in portions,
then decode steps at batch 1, 5 and 64, against the plain implementation (tests/plain_qwen2.py, evaluated in float32 by
torch on the GPU on the same bfloat16 weights) at the end of every portion, and against the engine's plain kernels
everywhere."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = {
    # Qwen2.5-0.5B: 14 heads over 2 key/value heads of 64, tied head
    "0.5B": dict(hidden_size=896, num_attention_heads=14, num_key_value_heads=2, intermediate_size=4864, vocab_size=151936,
                 tie_word_embeddings=True, rms_norm_eps=1e-6),
    # Qwen2.5-7B: 28 heads over 4 of 128
    "7B": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944, vocab_size=152064,
               tie_word_embeddings=False, rms_norm_eps=1e-6),
    # Qwen2.5-32B: 40 heads over 8 of 128
    "32B": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=27648, vocab_size=152064,
                tie_word_embeddings=False, rms_norm_eps=1e-5),
}


@pytest.mark.parametrize("name", list(SHAPES))
def test_fast_kernels_agree_with_plain_kernels(name):
    import hfcpu_b200
    from hfcpu_b200 import StepEntry, kernels
    from hfcpu_b200.config import config_from_dict
    cfg = config_from_dict(dict(architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, max_position_embeddings=32768,
                                rope_theta=1e6, **SHAPES[name]))
    model = hfcpu_b200.random_model(cfg, seed=1, dtype=torch.bfloat16, device="cuda:0", std=0.02)
    b = kernels.backend()
    g = torch.Generator().manual_seed(3)
    V = cfg.vocab_size
    prompts = {i: torch.randint(0, V, (n,), generator=g).tolist() for i, n in enumerate([700, 33, 129, 64, 300])}
    filler = {i: torch.randint(0, V, (40,), generator=g).tolist() for i in range(5, 64)}

    def run(fast):
        b.gemm, b.attention = ("tc", "fast") if fast else ("plain", "plain")
        try:
            eng = hfcpu_b200.Engine(model, block_size=16, num_pages=400, max_requests=64, ctx_max=2048)
            eng.use_graphs = eng.use_graphs and fast
            rows = []
            for r, ids in prompts.items():                       # prompts in portions of changing size
                eng.add_request(r)
                a = 0
                for n in (300, 17, 128, 255):
                    if a >= len(ids):
                        break
                    part = ids[a:a + n]
                    rows.append(eng.step([StepEntry(r, part, [len(part) - 1])])[0].float().cpu())
                    a += len(part)
            toks = {r: ids[-1] for r, ids in prompts.items()}      # given, not sampled: a near-tie of two logits must not make the runs diverge
            for batch in ([0], list(prompts), None):
                if batch is None:                                 # 64 requests decoding together
                    for r, ids in filler.items():
                        eng.add_request(r)
                        eng.step([StepEntry(r, ids, [])])
                        toks[r] = ids[0]
                    batch = list(prompts) + list(filler)
                for _ in range(3):                                # the third step of a kind replays its CUDA graph
                    out = eng.step([StepEntry(r, [toks[r]], [0]) for r in batch])
                    rows.append(out.float().cpu().clone())
            kernels.check_device_errors()
            return rows
        finally:
            b.gemm, b.attention = "tc", "fast"
    fast, plain = run(True), run(False)
    assert len(fast) == len(plain)
    for i, (x, y) in enumerate(zip(fast, plain)):
        err = float((x - y).abs().max() / y.abs().max())
        assert err < 3e-2, f"{name}: output {i} differs by {err:.3g}"
    # the plain implementation, which shares nothing with the engine, at the end of every portion of every prompt
    import plain_qwen2
    from hfcpu_b200.weights import RandomSource
    src = RandomSource(model.tensor_specs(), 1, torch.bfloat16, torch.device("cuda:0"), std=0.02)
    W = {n: src[n].float() for n in src.names()}
    old_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        at = 0
        for r, ids in prompts.items():
            ref = plain_qwen2.forward(cfg.to_dict(), W, ids, dtype=torch.float32)
            a = 0
            for n in (300, 17, 128, 255):
                if a >= len(ids):
                    break
                a = min(a + n, len(ids))
                want = ref[a - 1].cpu()
                err = float((fast[at] - want).abs().max() / want.abs().max())
                assert err < 3e-2, f"{name}: request {r} position {a - 1} differs from the plain implementation by {err:.3g}"
                at += 1
            del ref
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old_tf32
