"""The plain implementation's own checks (no GPU): the formula-level examples of the reference's
unit tests (crates/core/src/kernels/reference.rs:155-200, crates/core/src/sampler.rs:81-92) and the
properties the engine is later compared on."""
import math

import torch

from conftest import random_tokens
import plain_gpt2 as P


def test_matmul_small():
    # reference.rs:159-168: x [2,3] . w[2,3]^T + b
    x = torch.tensor([[1., 2., 3.], [4., 5., 6.]], dtype=torch.float64)
    w_out_in = torch.tensor([[1., 0., -1.], [2., 1., 0.]], dtype=torch.float64)
    b = torch.tensor([0.5, -0.5], dtype=torch.float64)
    y = P.linear_in_out(x, w_out_in.T.contiguous(), b)
    assert torch.allclose(y, torch.tensor([[-1.5, 3.5], [-1.5, 12.5]], dtype=torch.float64))


def test_softmax_sums_to_one_with_an_outlier():
    s = P.softmax(torch.tensor([1000.0, 1.0, 2.0, 3.0], dtype=torch.float64))
    assert abs(float(s.sum()) - 1.0) < 1e-12 and float(s[0]) > 0.999 and torch.isfinite(s).all()


def test_layernorm_normalises():
    x = torch.randn(3, 50, dtype=torch.float64, generator=torch.Generator().manual_seed(0)) * 3 + 2
    y = P.layernorm(x, torch.ones(50, dtype=torch.float64), torch.zeros(50, dtype=torch.float64), 1e-5)
    assert y.mean(-1).abs().max() < 1e-9 and (y.var(-1, unbiased=False) - 1).abs().max() < 1e-4


def test_attention_single_key_copies_value():
    q, k, v = torch.randn(1, 8, dtype=torch.float64), torch.randn(1, 8, dtype=torch.float64), torch.randn(1, 8, dtype=torch.float64)
    assert torch.allclose(P.causal_attention(q, k, v, n_head=2), v)


def test_attention_is_causal_and_windowed():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(9, 12, dtype=torch.float64, generator=g) for _ in range(3))
    full = P.causal_attention(q, k, v, n_head=3)
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 99.0, 99.0
    assert torch.allclose(P.causal_attention(q, k2, v2, n_head=3)[:5], full[:5])     # the future is not read
    win = P.causal_attention(q, k, v, n_head=3, window=4)
    assert torch.allclose(win[:4], full[:4]) and not torch.allclose(win[6], full[6])
    k3 = k.clone(); k3[0] = 50.0
    assert torch.allclose(P.causal_attention(q, k3, v, n_head=3, window=4)[6], win[6])  # key 0 is outside
    # grouped key/value heads: query heads 0,1 read key head 0
    g1 = P.causal_attention(q, k[:, :4], v[:, :4], n_head=3, n_kv_head=1)
    assert torch.allclose(g1[:, :4], P.causal_attention(q[:, :4], k[:, :4], v[:, :4], n_head=1))


def test_gelu_forms():
    u = torch.linspace(-4, 4, 41, dtype=torch.float64)
    assert torch.allclose(P.gelu_erf(u), torch.nn.functional.gelu(u), atol=1e-12)
    assert torch.allclose(P.gelu_tanh(u), torch.nn.functional.gelu(u, approximate="tanh"), atol=1e-12)
    assert (P.gelu_erf(u) - P.gelu_tanh(u)).abs().max() > 1e-4


def test_argmax_ties_go_to_the_lowest_index_and_topk_orders():
    assert P.argmax(torch.tensor([1.0, 3.0, 3.0, 2.0])) == 1
    lg = torch.tensor([0.0, 3.0, 1.0, 2.0])
    assert [t for t, _ in P.top_k_probs(lg, 2)] == [1, 3]                       # sampler.rs:85-91
    assert abs(sum(p for _, p in P.top_k_probs(lg, 4)) - 1.0) < 1e-6


def test_sampler_matches_its_generator_and_is_greedy_at_zero():
    s = P.XorShiftSampler(0.0, 40, 42)
    assert s.sample(torch.tensor([0.1, 0.9, 0.3])) == 1
    a, b = P.XorShiftSampler(0.8, 3, 42), P.XorShiftSampler(0.8, 3, 42)
    lg = torch.randn(50, generator=torch.Generator().manual_seed(3))
    draws = [a.sample(lg) for _ in range(20)]
    assert draws == [b.sample(lg) for _ in range(20)] and len(set(draws)) > 1
    top3 = {t for t, _ in P.top_k_probs(lg, 3)}
    assert set(draws) <= top3
    u = [P.XorShiftSampler(1.0, 0, 7).next_f32() for _ in range(1)]
    assert 0.0 <= u[0] < 1.0


def test_whole_model_prefix_property(model_dirs):
    """Logits at position t depend on tokens 0..t only: the property every way of cutting rests on."""
    d = model_dirs("B")
    m = P.PlainGPT2(d)
    toks = random_tokens(1000, 30, 5)
    full = m.logits(toks)
    assert torch.allclose(m.logits(toks[:17]), full[:17], atol=1e-10)
    assert full.shape == (30, 1000) and m.greedy(toks[:4], 3) == m.greedy(toks[:4], 3)


def test_options_change_the_result(model_dirs):
    d = model_dirs("B")
    m = P.PlainGPT2(d)
    toks = random_tokens(1000, 12, 6)
    base = m.logits(toks)
    m.scale_by_layer = False
    assert (m.logits(toks) - base).abs().max() > 1e-4
    m.scale_by_layer = True
    m.act = P.gelu_tanh
    assert (m.logits(toks) - base).abs().max() > 1e-7
    m.act = P.gelu_erf
    m.eps = 1e-2
    assert (m.logits(toks) - base).abs().max() > 1e-5
