"""Shared fixtures: tiny configurations of the architecture that differ in every size and
option, written as real model folders (config.json + model.safetensors) with seeded random
weights in a temporary folder."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_cuda = torch.cuda.is_available()
    except Exception:
        has_cuda = False
    if has_cuda:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def tiny_configs():
    from gophonic_b200.config import Qwen3Config
    return {
        # layers / hidden / heads / kv heads / head_dim / inter / vocab / theta / eps / tied: all differ
        "A": Qwen3Config(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         head_dim=16, intermediate_size=160, vocab_size=512, max_position_embeddings=512,
                         rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True),
        "B": Qwen3Config(hidden_size=96, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3,
                         head_dim=32, intermediate_size=256, vocab_size=1000, max_position_embeddings=1024,
                         rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False),
        # one kv head for five heads, head_dim 48, nothing a power of two
        "C": Qwen3Config(hidden_size=80, num_hidden_layers=1, num_attention_heads=5, num_key_value_heads=1,
                         head_dim=48, intermediate_size=136, vocab_size=333, max_position_embeddings=768,
                         rms_norm_eps=3e-6, rope_theta=50000.0, tie_word_embeddings=False),
        # head_dim 128 and widths that reach the kernels the full-size model runs on: the tcgen05
        # attention (prompts of 65 rows and more), the head_dim-128 rotation kernel, the tiled
        # tcgen05 GEMMs (128 rows and more) and the tcgen05 decode GEMM (9 to 64 rows)
        "D": Qwen3Config(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         head_dim=128, intermediate_size=520, vocab_size=2000, max_position_embeddings=1024,
                         rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False),
        # widths whose bfloat16 rows are not 16-byte aligned (84, 100): the tensor-core kernels refuse
        # them and every product of the bfloat16 model runs on the CUDA-core kernel instead
        "E": Qwen3Config(hidden_size=84, num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=3,
                         head_dim=16, intermediate_size=100, vocab_size=257, max_position_embeddings=600,
                         rms_norm_eps=1e-5, rope_theta=20000.0, tie_word_embeddings=True),
        # the reference's own small test geometry (internal/qwen3lm/lmtest/lmtest.go:27-30): a head
        # size that is no multiple of 16, attention wider than the hidden state, a vocabulary of 23
        "F": Qwen3Config(hidden_size=96, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
                         head_dim=24, intermediate_size=136, vocab_size=23, max_position_embeddings=320,
                         rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False),
    }


TEST_SCALES = dict(matrix=0.1, embedding=1.0, head=0.1, norm=0.1)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> folder of a random model with bfloat16 weights (A, B, C) or float32 weights (A32)."""
    from gophonic_b200.weights import InitScales, write_random_model
    out = {}
    scales = InitScales(**TEST_SCALES)
    for i, (name, cfg) in enumerate(tiny_configs().items()):
        d = str(tmp_path_factory.mktemp(f"model_{name}"))
        write_random_model(cfg, seed=100 + i, out_dir=d, weight_dtype="bfloat16", scales=scales)
        out[name] = d
    d = str(tmp_path_factory.mktemp("model_A32"))
    write_random_model(tiny_configs()["A"], seed=7, out_dir=d, weight_dtype="float32", scales=scales)
    out["A32"] = d
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    """name -> (config dict, float64 weights) read by the plain implementation's own reader."""
    from tests.plain.qwen3_plain import read_model
    return {name: read_model(d) for name, d in model_dirs.items()}
