"""A plain, slow GPT-2 for the tests: whole sequences, no cache, one function a part.

It shares no code with ``nanoinfer_b200``: it reads the model folder with the
``safetensors`` package and ``json``, and computes in torch on the CPU (float64
by default, so that it can judge a 32-bit engine).  Every function restates a
formula of the reference and cites it by the file's path inside the reference
project.  Options the reference fixes in code (exact-erf GELU, an untied head,
the 1/(l+1) score factor, an inner width other than 4C, a head size other than
64, fewer key/value heads than query heads, a window) are parameters here and
marked "not in the reference".

The reference's own model code is Rust and no Rust toolchain exists where this
was written, so this file rests on the reference's formulas, not on its output.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- parts
def embed(wte: torch.Tensor, wpe: Optional[torch.Tensor], tokens: Sequence[int], pos0: int = 0) -> torch.Tensor:
    """x[t] = wte[tok_t] + wpe[pos0 + t]  (crates/core/src/kernels/reference.rs:86-94)."""
    tok = torch.as_tensor(list(tokens), dtype=torch.long, device=wte.device)
    x = wte[tok]
    if wpe is not None:
        pos = torch.arange(pos0, pos0 + len(tok), device=wte.device)
        x = x + wpe[pos]
    return x


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    """Two-pass LayerNorm with biased variance (crates/core/src/kernels/reference.rs:42-51)."""
    mean = x.sum(dim=-1, keepdim=True) / x.shape[-1]
    var = ((x - mean) ** 2).sum(dim=-1, keepdim=True) / x.shape[-1]
    rstd = 1.0 / torch.sqrt(var + eps)
    return (x - mean) * rstd * weight + bias


def linear_in_out(x: torch.Tensor, w_in_out: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """out = x . W + b with W stored [in, out] as in the checkpoint.  The reference
    transposes to [out, in] at load and computes x . W^T (crates/core/src/weights.rs:48-57,
    kernels/reference.rs:26-37); the product is the same."""
    y = x @ w_in_out
    return y if bias is None else y + bias


def gelu_tanh(u: torch.Tensor) -> torch.Tensor:
    """0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3)))  (crates/core/src/kernels/reference.rs:53-61)."""
    return 0.5 * u * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (u + 0.044715 * u * u * u)))


def gelu_erf(u: torch.Tensor) -> torch.Tensor:
    """0.5 u (1 + erf(u / sqrt 2)): the exact form; not in the reference."""
    return 0.5 * u * (1.0 + torch.erf(u / math.sqrt(2.0)))


def softmax(s: torch.Tensor) -> torch.Tensor:
    """Subtract the max, exp, divide by the sum (crates/core/src/kernels/reference.rs:63-76)."""
    e = torch.exp(s - s.max())
    return e / e.sum()


def causal_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    n_head: int,
    n_kv_head: Optional[int] = None,
    scale: Optional[float] = None,
    window: int = 0,
    q_pos0: int = 0,
) -> torch.Tensor:
    """Causal multi-head attention, one (query, head) at a time
    (crates/core/src/kernels/reference.rs:109-142): s_j = (q_i . k_j) * scale for
    j <= p, softmax, o_i = sum_j p_j v_j, heads concatenated.

    q is [n_q, n_head * hd]; k, v are [n_kv, n_kv_head * hd] for positions 0..n_kv;
    query i stands at position q_pos0 + i.  Not in the reference: ``n_kv_head``
    (query head h reads key head h // (n_head / n_kv_head)), ``scale`` other than
    1/sqrt(hd), and ``window`` (> 0: only the last ``window`` keys, the query's
    own position included).
    """
    n_q = q.shape[0]
    hd = q.shape[1] // n_head
    n_kv_head = n_kv_head or n_head
    group = n_head // n_kv_head
    if scale is None:
        scale = 1.0 / math.sqrt(hd)
    out = torch.zeros(n_q, n_head * hd, dtype=q.dtype, device=q.device)
    for i in range(n_q):
        p = q_pos0 + i
        lo = max(0, p - window + 1) if window > 0 else 0
        for h in range(n_head):
            hk = h // group
            qh = q[i, h * hd:(h + 1) * hd]
            kh = k[lo:p + 1, hk * hd:(hk + 1) * hd]
            vh = v[lo:p + 1, hk * hd:(hk + 1) * hd]
            s = (kh @ qh) * scale
            out[i, h * hd:(h + 1) * hd] = softmax(s) @ vh
    return out


# --------------------------------------------------------------------------- model
class PlainGPT2:
    """Whole-sequence GPT-2 forward (crates/core/src/stages/naive.rs:21-45 with the
    block of stages/blocks.rs:4-8), returning the logits of every position."""

    def __init__(self, model_dir: str, dtype: torch.dtype = torch.float64, device: str = "cpu"):
        """``device``: where the same torch formulas run; the tests use the CPU except for models of
        full size, whose float64 products take minutes there."""
        from safetensors.torch import load_file

        with open(os.path.join(model_dir, "config.json")) as fh:
            self.cfg = json.load(fh)
        raw = load_file(os.path.join(model_dir, "model.safetensors"))
        self.w: Dict[str, torch.Tensor] = {}
        for name, t in raw.items():
            if name.startswith("transformer."):
                name = name[len("transformer."):]
            self.w[name] = t.to(device=device, dtype=dtype)
        self.dtype = dtype
        c = self.cfg
        self.n_layer = c["n_layer"]
        self.n_head = c["n_head"]
        self.n_embd = c["n_embd"]
        self.eps = c["layer_norm_epsilon"]
        act = c["activation_function"]
        self.act = gelu_erf if act == "gelu" else gelu_tanh
        self.tied = c.get("tie_word_embeddings", True)
        self.scale_by_sqrt = c.get("scale_attn_weights", True)
        self.scale_by_layer = c.get("scale_attn_by_inverse_layer_idx", False)

    def score_scale(self, layer: int) -> float:
        hd = self.n_embd // self.n_head
        s = 1.0 / math.sqrt(hd) if self.scale_by_sqrt else 1.0
        if self.scale_by_layer:
            s = s / float(layer + 1)  # not in the reference
        return s

    def block(self, l: int, x: torch.Tensor) -> torch.Tensor:
        """x += c_proj(attn(c_attn(ln_1 x))); x += c_proj(gelu(c_fc(ln_2 x)))
        (crates/core/src/stages/blocks.rs:31-50, 93-138)."""
        w, p, c = self.w, f"h.{l}.", self.n_embd
        xn = layernorm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], self.eps)
        qkv = linear_in_out(xn, w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"])
        q, k, v = qkv[:, :c], qkv[:, c:2 * c], qkv[:, 2 * c:]
        att = causal_attention(q, k, v, self.n_head, scale=self.score_scale(l))
        x = x + linear_in_out(att, w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"])
        xn = layernorm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], self.eps)
        fc = self.act(linear_in_out(xn, w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"]))
        x = x + linear_in_out(fc, w[p + "mlp.c_proj.weight"], w[p + "mlp.c_proj.bias"])
        return x

    def logits(self, tokens: Sequence[int], schedule: Optional[List[int]] = None) -> torch.Tensor:
        """Logits [n, vocab] after every token.  The reference computes the last row
        only (stages/blocks.rs:143-158); all rows are the same formula per row."""
        w = self.w
        x = embed(w["wte.weight"], w["wpe.weight"], tokens, 0)
        for l in (schedule if schedule is not None else range(self.n_layer)):
            x = self.block(l, x)
        h = layernorm(x, w["ln_f.weight"], w["ln_f.bias"], self.eps)
        head = w["wte.weight"] if self.tied else w["lm_head.weight"]
        return h @ head.T

    def greedy(self, prompt: Sequence[int], n_new: int) -> List[int]:
        """Recompute the whole sequence for every token (stages/naive.rs) and take
        the argmax with ties to the lowest index (crates/core/src/sampler.rs:4-12)."""
        toks = list(prompt)
        out = []
        for _ in range(n_new):
            nxt = argmax(self.logits(toks)[-1].to(torch.float32))
            out.append(nxt)
            toks.append(nxt)
        return out


# --------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor) -> int:
    """First maximum wins (crates/core/src/sampler.rs:4-12)."""
    best = 0
    vals = logits.tolist()
    for i, v in enumerate(vals):
        if v > vals[best]:
            best = i
    return best


def top_k_probs(logits: torch.Tensor, k: int):
    """The k most likely tokens with their full-vocabulary softmax probabilities,
    highest first (crates/core/src/sampler.rs:15-30)."""
    lg = logits.to(torch.float32)
    mx = lg.max()
    total = torch.exp(lg - mx).sum()
    k = min(k, lg.numel())
    if k == 0:
        return []
    order = sorted(range(lg.numel()), key=lambda i: (-float(lg[i]), i))[:k]
    return [(i, float(torch.exp(lg[i] - mx) / total)) for i in order]


class XorShiftSampler:
    """Greedy for temperature <= 0, else temperature and top-k sampling with the
    xorshift64* generator (crates/core/src/sampler.rs:46-78)."""

    MASK = (1 << 64) - 1

    def __init__(self, temperature: float, top_k: int, seed: int):
        self.temperature, self.top_k = temperature, top_k
        self.rng = max(seed, 1)

    def next_f32(self) -> float:
        self.rng ^= self.rng >> 12
        self.rng ^= (self.rng << 25) & self.MASK
        self.rng ^= self.rng >> 27
        r = (self.rng * 0x2545F4914F6CDD1D) & self.MASK
        return (r >> 40) / float(1 << 24)

    def sample(self, logits: torch.Tensor) -> int:
        if self.temperature <= 0.0:
            return argmax(logits)
        k = logits.numel() if self.top_k == 0 else self.top_k
        cands = top_k_probs(logits.to(torch.float32) / self.temperature, k)
        total = sum(p for _, p in cands)
        r = self.next_f32() * total
        for tok, p in cands:
            r -= p
            if r <= 0.0:
                return tok
        return cands[-1][0] if cands else 0
