"""Shared fixtures: tiny configurations, model folders with seeded random weights, and the
plain implementation's logits for given token sequences."""
import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on the GPU box)")


# Two tiny GPT-2 configurations that differ in every size and option.
TINY_A = dict(architectures=["GPT2LMHeadModel"], vocab_size=512, n_positions=128, n_embd=64, n_layer=2, n_head=4,
              n_inner=256, layer_norm_epsilon=1e-5, activation_function="gelu_new", tie_word_embeddings=True,
              scale_attn_by_inverse_layer_idx=False)
TINY_B = dict(architectures=["GPT2LMHeadModel"], vocab_size=1000, n_positions=64, n_embd=120, n_layer=3, n_head=5,
              n_inner=200, layer_norm_epsilon=1e-6, activation_function="gelu", tie_word_embeddings=False,
              scale_attn_by_inverse_layer_idx=True)
# A longer context for the long-decoding tests: hundreds of keys, pages far apart.
TINY_LONG = dict(architectures=["GPT2LMHeadModel"], vocab_size=320, n_positions=640, n_embd=96, n_layer=2, n_head=3,
                 n_inner=160, layer_norm_epsilon=1e-5, activation_function="gelu_new", tie_word_embeddings=True,
                 scale_attn_by_inverse_layer_idx=False)
# GPT-2 small's layer sizes (width 768, 12 heads of 64, inner 3072, 1024 positions) with two layers and a
# small vocabulary: the sizes at which the engine picks its tensor-memory kernels.
WIDE = dict(architectures=["GPT2LMHeadModel"], vocab_size=2003, n_positions=1024, n_embd=768, n_layer=2, n_head=12,
            n_inner=3072, layer_norm_epsilon=1e-5, activation_function="gelu_new", tie_word_embeddings=True,
            scale_attn_by_inverse_layer_idx=False)
# GPT-2 XL's layer sizes (width 1600, 25 heads of 64, inner 6400) with one layer: a width that is no
# multiple of 128 or 256, an odd number of heads, rows too wide for the norm folded into the few-row product.
XLW = dict(architectures=["GPT2LMHeadModel"], vocab_size=1501, n_positions=512, n_embd=1600, n_layer=1, n_head=25,
           n_inner=6400, layer_norm_epsilon=1e-5, activation_function="gelu_new", tie_word_embeddings=True,
           scale_attn_by_inverse_layer_idx=False)
# GPT-2 medium's layer sizes (width 1024, 16 heads of 64, inner 4096) with two layers.
MEDW = dict(architectures=["GPT2LMHeadModel"], vocab_size=1777, n_positions=1024, n_embd=1024, n_layer=2, n_head=16,
            n_inner=4096, layer_norm_epsilon=1e-5, activation_function="gelu_new", tie_word_embeddings=True,
            scale_attn_by_inverse_layer_idx=False)
# One layer of GPT-2 small's sizes with the real vocabulary: 50257 is no multiple of anything a tile likes.
V50K = dict(architectures=["GPT2LMHeadModel"], vocab_size=50257, n_positions=256, n_embd=768, n_layer=1, n_head=12,
            n_inner=3072, layer_norm_epsilon=1e-5, activation_function="gelu_new", tie_word_embeddings=True,
            scale_attn_by_inverse_layer_idx=False)
# GPT-2 small whole: twelve layers, the real vocabulary, 1024 positions (the sizes the benchmark runs).
SMALL = dict(architectures=["GPT2LMHeadModel"], vocab_size=50257, n_positions=1024, n_embd=768, n_layer=12, n_head=12,
             n_inner=3072, layer_norm_epsilon=1e-5, activation_function="gelu_new", tie_word_embeddings=True,
             scale_attn_by_inverse_layer_idx=False)
# a context of thousands of positions, heads of 64 (the tensor-core decode attention): a decoded token's keys
# are then cut into more splits than one cluster holds
FAR = dict(architectures=["GPT2LMHeadModel"], vocab_size=300, n_positions=4608, n_embd=128, n_layer=2, n_head=2,
           n_inner=192, layer_norm_epsilon=1e-5, activation_function="gelu_new", tie_word_embeddings=True,
           scale_attn_by_inverse_layer_idx=False)
TINY = {"FAR": FAR, "A": TINY_A, "B": TINY_B, "LONG": TINY_LONG, "WIDE": WIDE, "XLW": XLW, "MEDW": MEDW, "V50K": V50K,
        "SMALL": SMALL}


def sharpen_attention(tensors, factor):
    """Scale the query and key columns of every c_attn so that scores spread over several units:
    the softmax then leans on single keys, and a wrong key, page or position shows in the logits
    (with N(0, 0.02) weights attention is nearly uniform and would hide it)."""
    for name, t in tensors.items():
        if name.endswith("attn.c_attn.weight"):
            c = t.shape[0]
            t[:, :2 * c] *= factor
    return tensors


def write_tiny(name, out_dir, dtype, seed=7, sharpen=6.0):
    from nanoinfer_b200.config import GPT2Config
    from nanoinfer_b200.models.model import Model
    from nanoinfer_b200.registry import get_architecture
    from nanoinfer_b200.weights import random_tensors, write_safetensors

    cfg = GPT2Config.from_dict(TINY[name])
    model = Model(get_architecture(cfg.architecture).build_spec(cfg), cfg)
    tensors = random_tensors(model, seed, 0.02, torch.float32)
    if sharpen:
        sharpen_attention(tensors, sharpen)
    tensors = {k: v.to(dtype) for k, v in tensors.items()}
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors)
    return out_dir


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders, made on demand in a temporary folder: model_dirs(name, dtype) -> path."""
    made = {}

    def get(name, dtype=torch.float32, sharpen=6.0, seed=7):
        key = (name, dtype, sharpen, seed)
        if key not in made:
            d = tmp_path_factory.mktemp(f"tiny_{name}_{str(dtype).split('.')[-1]}")
            made[key] = write_tiny(name, str(d), dtype, seed, sharpen)
        return made[key]

    return get


@pytest.fixture(scope="session")
def plain_logits():
    """plain_logits(model_dir, tokens) -> float32 [n, vocab] from the plain implementation (float64 inside)."""
    from plain_gpt2 import PlainGPT2

    models, cache = {}, {}

    def get(model_dir, tokens, device="cpu"):
        key = (model_dir, tuple(tokens))
        if key not in cache:
            if model_dir not in models:
                models.clear()             # one plain model at a time: the large ones take gigabytes
                models[model_dir] = PlainGPT2(model_dir, device=device)
            cache[key] = models[model_dir].logits(list(tokens)).to(torch.float32).cpu()
        return cache[key]

    return get


def random_tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
