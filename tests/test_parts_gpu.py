"""The parts alone and put together in ways GPT-2 does not use, without a change to the
framework's files: a toy architecture is registered here whose layers differ from one another
(grouped key/value heads with a window, a mixer with per-request state of its own, a feed-forward
with routing, a position encoding inside the mixer) and whose run order names a layer twice and
lets a run read another run's cache.  Everything is compared with a plain whole-sequence
computation written in this file."""
import dataclasses
import json
import math
import os
from typing import ClassVar, List, Tuple

import pytest
import torch

from conftest import random_tokens

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------------------- toy parts (torch, test only)
def register_toys():
    from nanoinfer_b200 import parts as P
    from nanoinfer_b200.config.base import ModelConfig, field
    from nanoinfer_b200.models.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from nanoinfer_b200.parts.base import MATRIX, VECTOR, ParamSpec, StateSpec, TensorRef
    from nanoinfer_b200.registry import architectures, register_architecture

    if "ToyMixLM" in architectures():
        return

    @P.register_mixer("toy_decay_mixer")
    class DecayMixer(P.Mixer):
        """s <- decay * s + (1 - decay) * (W xn_t);  x_t += s.  The state s is per request."""

        def __init__(self, width, decay):
            self.width, self.decay = width, decay

        def param_specs(self):
            return [ParamSpec("weight", (self.width, self.width), MATRIX)]

        def state_spec(self):
            return StateSpec((self.width,), torch.float32)

        def forward(self, xn, x, ctx, cache, state, writes_cache=True):
            assert cache is None and state is not None
            u = xn[:ctx.n_rows].float() @ self.params["weight"].float().T
            for e in range(ctx.n_entries):
                a, b, slot = ctx.host_entry_start[e], ctx.host_entry_start[e + 1], ctx.host_entry_slot[e]
                s = state[slot]
                for t in range(a, b):
                    s = self.decay * s + (1.0 - self.decay) * u[t]
                    x[t] += s
                state[slot] = s

    @P.register_feed_forward("toy_routed_ffn")
    class RoutedFFN(P.FeedForward):
        """Router logits in 32-bit, the best expert per row, x += gate * relu(xn W1_e^T) W2_e^T."""

        def __init__(self, width, inner, n_expert):
            self.width, self.inner, self.n_expert = width, inner, n_expert

        def param_specs(self):
            return [ParamSpec("router", (self.n_expert, self.width), MATRIX),
                    ParamSpec("up", (self.n_expert * self.inner, self.width), MATRIX),
                    ParamSpec("down", (self.n_expert * self.width, self.inner), MATRIX)]

        def forward(self, xn, x, ctx):
            T = ctx.n_rows
            h = xn[:T].float()
            probs = torch.softmax(h @ self.params["router"].float().T, dim=-1)
            gate, idx = probs.max(dim=-1)
            up = self.params["up"].float().view(self.n_expert, self.inner, self.width)
            down = self.params["down"].float().view(self.n_expert, self.width, self.inner)
            for e in range(self.n_expert):
                rows = (idx == e).nonzero().flatten()
                if rows.numel():
                    y = torch.relu(h[rows] @ up[e].T) @ down[e].T
                    x[rows] += gate[rows, None] * y

    @P.register_position("toy_phase")
    class Phase(P.PositionEncoding):
        """q and k are multiplied by cos(pos * w_d): a position encoding that acts inside the mixer."""

        def __init__(self, head_dim, base):
            self.head_dim, self.base = head_dim, base

        def _factor(self, ctx, width, dtype):
            d = torch.arange(width, device=ctx.positions.device) % self.head_dim
            w = self.base ** (-d.float() / self.head_dim)
            return torch.cos(ctx.positions[:ctx.n_rows, None].float() * w[None, :]).to(dtype)

        def on_qk(self, q, k, ctx):
            q.mul_(self._factor(ctx, q.shape[1], q.dtype))
            if k is not None:
                k.mul_(self._factor(ctx, k.shape[1], k.dtype))

    @dataclasses.dataclass
    class ToyConfig(ModelConfig):
        architecture_names: ClassVar[Tuple[str, ...]] = ("ToyMixLM",)
        vocab_size: int = field()
        width: int = field()
        n_positions: int = field()
        eps: float = field()
        window: int = field()
        decay: float = field()
        n_expert: int = field()

        def to_dict(self):
            return dict(architectures=["ToyMixLM"], **super().to_dict())

    def build(cfg):
        c = cfg.width

        def norm(name):
            return PartSpec("layernorm", dict(width=c, eps=cfg.eps),
                            {"weight": TensorRef(name + ".g"), "bias": TensorRef(name + ".b")})

        def attn(name, n_head, n_kv_head, hd, window, scale):
            return PartSpec("causal_attention",
                            dict(width=c, n_head=n_head, n_kv_head=n_kv_head, head_dim=hd, scale=scale, window=window,
                                 bias=False),
                            {"qkv_weight": TensorRef(name + ".qkv"), "out_weight": TensorRef(name + ".out")})

        def mlp(name, inner, act):
            return PartSpec("dense_mlp", dict(width=c, inner=inner, activation=act, bias=True),
                            {"fc_weight": TensorRef(name + ".fc.w"), "fc_bias": TensorRef(name + ".fc.b"),
                             "proj_weight": TensorRef(name + ".proj.w"), "proj_bias": TensorRef(name + ".proj.b")})

        layers = [
            LayerSpec("pre_norm", norm_1=norm("l0.n1"), mixer=attn("l0.att", 4, 2, 16, cfg.window, 0.3),
                      norm_2=norm("l0.n2"), feed_forward=mlp("l0.mlp", 96, "tanh")),
            LayerSpec("pre_norm", norm_1=norm("l1.n1"),
                      mixer=PartSpec("toy_decay_mixer", dict(width=c, decay=cfg.decay), {"weight": TensorRef("l1.mix.w")}),
                      norm_2=norm("l1.n2"),
                      feed_forward=PartSpec("toy_routed_ffn", dict(width=c, inner=40, n_expert=cfg.n_expert),
                                            {"router": TensorRef("l1.moe.router"), "up": TensorRef("l1.moe.up"),
                                             "down": TensorRef("l1.moe.down")})),
            LayerSpec("pre_norm", norm_1=norm("l2.n1"), mixer=attn("l2.att", 2, 2, 32, 0, 0.25),
                      norm_2=norm("l2.n2"), feed_forward=mlp("l2.mlp", 80, "erf"),
                      mixer_position=PartSpec("toy_phase", dict(head_dim=32, base=50.0))),
        ]
        return ModelSpec(
            width=c,
            embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, width=c), {"table": TensorRef("emb")}),
            position=None, layers=layers,
            schedule=[ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(0), ScheduleEntry(2, cache_of=2)],
            final_norm=norm("final"),
            head=PartSpec("linear_head", dict(vocab_size=cfg.vocab_size, width=c), {"weight": TensorRef("head")}),
            max_positions=cfg.n_positions)

    register_architecture("ToyMixLM", ToyConfig, build)


TOY = dict(architectures=["ToyMixLM"], vocab_size=200, width=64, n_positions=96, eps=1e-5, window=20, decay=0.7,
           n_expert=3)


# ----------------------------------------------------------------------------- the plain toy model
def plain_toy_logits(folder, tokens):
    import plain_gpt2 as P
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    cfg = json.load(open(os.path.join(folder, "config.json")))
    n = len(tokens)
    pos = torch.arange(n, dtype=torch.float64)
    x = w["emb"][torch.tensor(tokens)]

    def ln(name, x):
        return P.layernorm(x, w[name + ".g"], w[name + ".b"], cfg["eps"])

    def phase(t, hd, base):
        d = torch.arange(t.shape[1]) % hd
        return t * torch.cos(pos[:, None] * (base ** (-d.double() / hd))[None, :])

    def att(name, x, n_head, n_kv_head, hd, window, scale, kv=None, rotate=False):
        qkv = x @ w[name + ".qkv"].T
        q, k, v = qkv[:, :n_head * hd], qkv[:, n_head * hd:(n_head + n_kv_head) * hd], qkv[:, (n_head + n_kv_head) * hd:]
        if rotate:
            q, k = phase(q, hd, 50.0), phase(k, hd, 50.0)
        if kv is not None:
            k, v = kv
        o = P.causal_attention(q, k, v, n_head, n_kv_head, scale=scale, window=window)
        return o @ w[name + ".out"].T, (k, v)

    def mlp(name, x, act):
        return act(x @ w[name + ".fc.w"].T + w[name + ".fc.b"]) @ w[name + ".proj.w"].T + w[name + ".proj.b"]

    def layer0(x):
        x = x + att("l0.att", ln("l0.n1", x), 4, 2, 16, cfg["window"], 0.3)[0]
        return x + mlp("l0.mlp", ln("l0.n2", x), P.gelu_tanh)

    def layer1(x):
        u = ln("l1.n1", x) @ w["l1.mix.w"].T
        s = torch.zeros(x.shape[1], dtype=torch.float64)
        out = []
        for t in range(n):
            s = cfg["decay"] * s + (1 - cfg["decay"]) * u[t]
            out.append(s)
        x = x + torch.stack(out)
        h = ln("l1.n2", x)
        probs = torch.softmax(h @ w["l1.moe.router"].T, dim=-1)
        gate, idx = probs.max(-1)
        up, down = w["l1.moe.up"].view(3, 40, -1), w["l1.moe.down"].view(3, -1, 40)
        y = torch.stack([torch.relu(h[t] @ up[idx[t]].T) @ down[idx[t]].T for t in range(n)])
        return x + gate[:, None] * y

    def layer2(x, kv=None):
        a, kv_out = att("l2.att", ln("l2.n1", x), 2, 2, 32, 0, 0.25, kv=kv, rotate=True)
        x = x + a
        return x + mlp("l2.mlp", ln("l2.n2", x), P.gelu_erf), kv_out

    x = layer0(x)
    x = layer1(x)
    x, kv2 = layer2(x)
    x = layer0(x)                 # the same weights a second time, with keys and values of its own
    x, _ = layer2(x, kv=kv2)      # reads the keys and values of the first run of layer 2
    return (ln("final", x) @ w["head"].T).float()


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    register_toys()
    from nanoinfer_b200.registry import get_architecture
    from nanoinfer_b200.weights import write_random_model
    cfg = get_architecture("ToyMixLM").config_cls.from_dict(TOY)
    d = str(tmp_path_factory.mktemp("toy"))
    write_random_model(cfg, d, seed=21, dtype=torch.float32, std=0.08)
    return d


def test_toy_architecture_is_registered_built_and_stepped(toy_folder):
    """A mixer with state of its own, a routed feed-forward and an in-mixer position encoding are
    registered from this file; the model is built from config.json, cut into steps every way, and
    agrees with the plain computation."""
    from nanoinfer_b200 import load_model
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.engine import ModelRunner, StepItem
    m = load_model(toy_folder, torch.float32, "cuda")
    kinds = [type(l.mixer).__name__ for l in m.layers]
    assert kinds == ["CausalSelfAttention", "DecayMixer", "CausalSelfAttention"]
    assert [i for i, _ in m.kv_needs()] == [0, 2, 3] and [i for i, _ in m.state_needs()] == [1]
    cache = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=256, max_requests=3, page_size=16,
                         dtype=torch.float32, device=torch.device("cuda"), max_positions=m.max_positions)
    # the windowed runs (0 and 3) share one group, the run that keeps all keys has another
    assert sorted(g.owners for g in cache.groups) == [[0, 3], [2]]
    runner = ModelRunner(m, cache, max_rows=96, max_entries=3)
    seqs = [random_tokens(200, n, 300 + i) for i, n in enumerate([96, 61, 40])]
    want = [plain_toy_logits(toy_folder, s) for s in seqs]

    # whole
    for s, w in zip(seqs, want):
        r = cache.open_request()
        got = runner.step([StepItem(r, s, range(len(s)))]).cpu()
        assert (got - w).abs().max() < 2e-4
        cache.close_request(r)
    # portions of changing size, three requests side by side, state carried from step to step
    reqs = [cache.open_request() for _ in seqs]
    prog = [0, 0, 0]
    got = [[] for _ in seqs]
    sizes = [[7, 1, 2, 30, 1], [2, 2, 19, 1], [1, 1, 1, 5]]
    k = 0
    while any(p < len(s) for p, s in zip(prog, seqs)):
        items, idx = [], []
        for i, s in enumerate(seqs):
            if prog[i] < len(s) and (k + i) % 4 != 3:
                n = min(sizes[i][k % len(sizes[i])], len(s) - prog[i])
                items.append(StepItem(reqs[i], s[prog[i]:prog[i] + n], range(n)))
                idx.append((i, n))
                prog[i] += n
        k += 1
        if not items:
            continue
        lg = runner.step(items).cpu()
        o = 0
        for i, n in idx:
            got[i].append(lg[o:o + n].clone())
            o += n
    for g, w in zip(got, want):
        assert (torch.cat(g) - w).abs().max() < 2e-4
    # the windowed group gave pages back while the other kept all of them
    win = next(i for i, g in enumerate(cache.groups) if g.spec.window)
    assert reqs[0].blocks[win][0] == -1 and all(p >= 0 for p in reqs[0].blocks[1 - win])
    for r in reqs:
        cache.close_request(r)
    cache.check()
    assert cache.pages_used() == [0, 0]


def test_state_slot_is_zeroed_for_a_new_request(toy_folder):
    from nanoinfer_b200 import load_model
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.engine import ModelRunner, StepItem
    m = load_model(toy_folder, torch.float32, "cuda")
    cache = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=128, max_requests=1, page_size=16,
                         dtype=torch.float32, device=torch.device("cuda"), max_positions=m.max_positions)
    runner = ModelRunner(m, cache, max_rows=64, max_entries=1)
    s = random_tokens(200, 20, 9)
    r = cache.open_request()
    first = runner.step([StepItem(r, s, [19])]).cpu().clone()
    cache.close_request(r)
    r = cache.open_request()                      # the same slot again
    again = runner.step([StepItem(r, s, [19])]).cpu()
    assert torch.equal(first, again)


# ----------------------------------------------------------------------------- a second toy: another arrangement
def register_parallel_toy():
    """A block arrangement of its own (ONE norm; mixer and feed-forward both read it and both add to
    the stream), a layer without any mixer, and a mixer with per-request state whose work is all
    on the device, so that steps of the model are captured in graphs like any other."""
    from nanoinfer_b200 import parts as P
    from nanoinfer_b200.config.base import ModelConfig, field
    from nanoinfer_b200.models.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from nanoinfer_b200.parts.base import FEED_FORWARDS, MATRIX, MIXERS, NORMS, ParamSpec, StateSpec, TensorRef
    from nanoinfer_b200.parts.block import Block, register_block
    from nanoinfer_b200.registry import architectures, register_architecture

    if "ToyParallelLM" in architectures():
        return

    @P.register_mixer("toy_running_sum")
    class RunningSum(P.Mixer):
        """x_t += rate * sum_{j <= t} (W xn_j): the sum over the request's earlier steps is its state.
        Everything runs on the device from the step's tables; only shapes are read on the host."""

        capture_safe = True

        def __init__(self, width, rate):
            self.width, self.rate = width, rate

        def param_specs(self):
            return [ParamSpec("weight", (self.width, self.width), MATRIX)]

        def state_spec(self):
            return StateSpec((self.width,), torch.float32)

        def forward(self, xn, x, ctx, cache, state, writes_cache=True):
            T = ctx.n_rows
            u = xn[:T].float() @ self.params["weight"].float().T
            c = torch.cumsum(u, 0)
            first = ctx.entry_start[:-1].long()                 # [entries], on the device
            last = ctx.entry_start[1:].long() - 1
            ent, slots = ctx.row_entry.long(), ctx.entry_slot.long()
            before = (c[first] - u[first])                       # the running sum ahead of each entry's rows
            within = c - before[ent]
            x[:T] += self.rate * (state[slots][ent] + within)
            state.index_add_(0, slots, within[last])

    @register_block("toy_parallel")
    class ParallelBlock(Block):
        slots = {"norm": NORMS, "mixer": MIXERS, "feed_forward": FEED_FORWARDS}

        def forward(self, x, ctx, cache, state, writes_cache, dtype):
            xn = ctx.workspace.get("toy_parallel.normed", (ctx.max_rows, self.width), dtype)
            self.norm.forward(x, xn, ctx.n_rows)
            self.mixer.forward(xn, x, ctx, cache, state, writes_cache)
            self.feed_forward.forward(xn, x, ctx)

    @register_block("toy_ffn_only")
    class FFNOnly(Block):
        slots = {"norm": NORMS, "feed_forward": FEED_FORWARDS}

        def forward(self, x, ctx, cache, state, writes_cache, dtype):
            xn = ctx.workspace.get("toy_parallel.normed", (ctx.max_rows, self.width), dtype)
            self.norm.forward(x, xn, ctx.n_rows)
            self.feed_forward.forward(xn, x, ctx)

    @dataclasses.dataclass
    class ParallelConfig(ModelConfig):
        architecture_names: ClassVar[Tuple[str, ...]] = ("ToyParallelLM",)
        vocab_size: int = field()
        width: int = field()
        inner: int = field()
        eps: float = field()
        rate: float = field()

        def to_dict(self):
            return dict(architectures=["ToyParallelLM"], **super().to_dict())

    def build(cfg):
        c = cfg.width

        def norm(name):
            return PartSpec("layernorm", dict(width=c, eps=cfg.eps),
                            {"weight": TensorRef(name + ".g"), "bias": TensorRef(name + ".b")})

        def mlp(name):
            return PartSpec("dense_mlp", dict(width=c, inner=cfg.inner, activation="tanh", bias=True),
                            {"fc_weight": TensorRef(name + ".fc.w"), "fc_bias": TensorRef(name + ".fc.b"),
                             "proj_weight": TensorRef(name + ".proj.w"), "proj_bias": TensorRef(name + ".proj.b")})

        layers = [
            LayerSpec("toy_parallel", norm=norm("l0.n"), feed_forward=mlp("l0.mlp"),
                      mixer=PartSpec("toy_running_sum", dict(width=c, rate=cfg.rate), {"weight": TensorRef("l0.mix")})),
            LayerSpec("toy_ffn_only", parts={"norm": norm("l1.n"), "feed_forward": mlp("l1.mlp")}),
        ]
        return ModelSpec(
            width=c,
            embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, width=c), {"table": TensorRef("emb")}),
            position=None, layers=layers, schedule=[ScheduleEntry(0), ScheduleEntry(1)], final_norm=norm("final"),
            head=PartSpec("linear_head", dict(vocab_size=cfg.vocab_size, width=c), {"weight": TensorRef("emb")}),
            max_positions=None)

    register_architecture("ToyParallelLM", ParallelConfig, build)


PARALLEL = dict(architectures=["ToyParallelLM"], vocab_size=150, width=48, inner=72, eps=1e-5, rate=0.05)


def plain_parallel_logits(folder, tokens):
    import plain_gpt2 as P
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    x = w["emb"][torch.tensor(tokens)]

    def ln(name, x):
        return P.layernorm(x, w[name + ".g"], w[name + ".b"], PARALLEL["eps"])

    def mlp(name, h):
        return P.gelu_tanh(h @ w[name + ".fc.w"].T + w[name + ".fc.b"]) @ w[name + ".proj.w"].T + w[name + ".proj.b"]

    h = ln("l0.n", x)
    x = x + PARALLEL["rate"] * torch.cumsum(h @ w["l0.mix"].T, 0) + mlp("l0.mlp", h)
    x = x + mlp("l1.mlp", ln("l1.n", x))
    return (ln("final", x) @ w["emb"].T).float()


def test_another_arrangement_with_a_stateful_mixer_runs_in_graphs_and_is_measured(tmp_path):
    """A block arrangement with one norm, a layer without a mixer and a mixer with per-request state
    that declares itself safe to capture are registered from this file: the step function captures
    its decode steps in graphs as for any model (the state lives in the request's slot, the graph
    bakes in the step's shape only), the results agree with the plain computation, and the byte
    and FLOP counts of the measurement come from the built model, not from a configuration's field
    names."""
    register_parallel_toy()
    from nanoinfer_b200 import load_model, measure
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.engine import ModelRunner, StepItem
    from nanoinfer_b200.registry import get_architecture
    from nanoinfer_b200.weights import write_random_model
    cfg = get_architecture("ToyParallelLM").config_cls.from_dict(PARALLEL)
    d = write_random_model(cfg, str(tmp_path / "par"), seed=5, dtype=torch.float32, std=0.1)
    m = load_model(d, torch.float32, "cuda")
    assert [type(b).__name__ for b in m.layers] == ["ParallelBlock", "FFNOnly"] and m.layers[1].mixer is None
    assert m.kv_needs() == [] and [i for i, _ in m.state_needs()] == [0] and m.capture_safe()
    cache = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=512, max_requests=3, page_size=16,
                         dtype=torch.float32, device=torch.device("cuda"), max_positions=None, padding=True)
    runner = ModelRunner(m, cache, max_rows=96, max_entries=3)
    assert runner.use_graphs
    seqs = [random_tokens(150, n, 40 + i) for i, n in enumerate([50, 33, 41])]
    want = [plain_parallel_logits(d, s) for s in seqs]
    reqs = [cache.open_request() for _ in seqs]
    got = [[] for _ in seqs]
    # a portion of each prompt in one step, then single tokens side by side (the same shape step after
    # step: captured the second time and replayed from then on; requests drop out as they end)
    lg = runner.step([StepItem(r, s[:20 + 3 * i], range(20 + 3 * i)) for i, (r, s) in enumerate(zip(reqs, seqs))]).cpu()
    at, prog = 0, []
    for i in range(3):
        n = 20 + 3 * i
        got[i].append(lg[at:at + n].clone())
        at, prog = at + n, prog + [n]
    while any(p < len(s) for p, s in zip(prog, seqs)):
        live = [i for i, s in enumerate(seqs) if prog[i] < len(s)]
        lg = runner.step([StepItem(reqs[i], [seqs[i][prog[i]]], [0]) for i in live]).cpu()
        for row, i in enumerate(live):
            got[i].append(lg[row:row + 1].clone())
            prog[i] += 1
    assert runner.graph_replays > 20 and runner.graph_drops == 0
    for g, w in zip(got, want):
        assert (torch.cat(g) - w).abs().max() < 2e-4
    # measurement from the built model: the tied table is one tensor and is streamed (it is the head),
    # FLOPs are 2 per matrix element and row for each run, plus the head per logits row
    c, i, v = PARALLEL["width"], PARALLEL["inner"], PARALLEL["vocab_size"]
    n_params = v * c + c * c + 2 * (2 * c * i + i + c) + 3 * 2 * c
    assert measure.parameter_count(m) == n_params == measure.parameter_count_of_spec(m)
    assert measure.weight_bytes_per_step(m) == 4 * n_params
    assert measure.kv_bytes(cache, [100, 7]) == 0
    assert measure.step_flops(m, [5, 9, 2], 2) == 3 * 2.0 * (c * c + 4 * c * i) + 2 * 2.0 * v * c


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_embedding_mlp_and_head_parts_alone(dtype):
    """Each built-in part alone, built through its registry with sizes of its own."""
    import plain_gpt2 as P
    from nanoinfer_b200 import parts as NP
    from nanoinfer_b200.parts.base import StepContext, Workspace
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(4)
    T, C, I, V = 23, 72, 136, 333
    tol = 3e-5 if dtype == torch.float32 else 4e-2

    def bind(part, **tensors):
        part.bind({k: v.to(dev) for k, v in tensors.items()})
        part.prepare(dtype, dev)
        return part

    tokens = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    positions = torch.arange(5, 5 + T, dtype=torch.int32)
    ctx = StepContext(n_rows=T, n_entries=1, max_rows=T, tokens=tokens.to(dev), positions=positions.to(dev),
                      row_entry=torch.zeros(T, dtype=torch.int32, device=dev),
                      entry_start=torch.tensor([0, T], dtype=torch.int32, device=dev),
                      entry_pos0=torch.tensor([5], dtype=torch.int32, device=dev),
                      entry_slot=torch.zeros(1, dtype=torch.int32, device=dev),
                      status=torch.zeros(1, dtype=torch.int32, device=dev), workspace=Workspace(dev),
                      host_entry_start=[0, T], host_entry_pos0=[5], host_entry_slot=[0], max_q_len=T, max_kv_len=5 + T)
    wte, wpe = torch.randn(V, C, generator=g).to(dtype), torch.randn(64, C, generator=g).to(dtype)
    emb = bind(NP.EMBEDDINGS.build("token_embedding", vocab_size=V, width=C), table=wte)
    pos = bind(NP.POSITIONS.build("learned_absolute", n_positions=64, width=C), table=wpe)
    x = torch.zeros(T, C, device=dev)
    emb.forward(ctx, x, pos)
    want_x = P.embed(wte.double(), wpe.double(), tokens.tolist(), 5)
    assert (x.cpu().double() - want_x).abs().max() < 1e-6

    gamma, beta = 1 + 0.1 * torch.randn(C, generator=g), 0.1 * torch.randn(C, generator=g)
    norm = bind(NP.NORMS.build("layernorm", width=C, eps=3e-4), weight=gamma, bias=beta)
    xn = torch.zeros(T, C, dtype=dtype, device=dev)
    norm.forward(x, xn, T)
    want_n = P.layernorm(x.cpu().double(), gamma.double(), beta.double(), 3e-4)
    assert (xn.cpu().double() - want_n).abs().max() < tol

    for act, fn in (("tanh", P.gelu_tanh), ("erf", P.gelu_erf)):
        w1, b1 = (torch.randn(I, C, generator=g) * 0.1).to(dtype), torch.randn(I, generator=g) * 0.1
        w2, b2 = (torch.randn(C, I, generator=g) * 0.1).to(dtype), torch.randn(C, generator=g) * 0.1
        mlp = bind(NP.FEED_FORWARDS.build("dense_mlp", width=C, inner=I, activation=act),
                   fc_weight=w1, fc_bias=b1, proj_weight=w2, proj_bias=b2)
        x2 = x.clone()
        mlp.forward(xn, x2, ctx)
        h = xn.cpu().double()
        want = x.cpu().double() + fn(h @ w1.double().T + b1.double()) @ w2.double().T + b2.double()
        assert (x2.cpu().double() - want).abs().max() < tol

    head = bind(NP.HEADS.build("linear_head", vocab_size=V, width=C), weight=wte)
    logits = torch.zeros(T, V + 3, device=dev)[:, :V]
    head.forward(xn, logits, T, ctx)
    assert (logits.cpu().double() - xn.cpu().double() @ wte.double().T).abs().max() < tol * 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_head, n_kv_head, hd, window", [(5, 5, 16, 0), (6, 2, 48, 0), (4, 1, 32, 20)])
def test_attention_mixer_and_block_alone(dtype, n_head, n_kv_head, hd, window):
    """The attention mixer alone, built through its registry with sizes of its own (grouped key/value
    heads, a window): two steps over a hand-made cache, a prompt portion beside another request's single
    token, then single tokens; and the pre-norm block around it and a feed-forward.  Against the plain
    formulas on whole sequences."""
    import plain_gpt2 as P
    from nanoinfer_b200 import parts as NP
    from nanoinfer_b200.parts.base import KVCacheView, StepContext, Workspace
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(n_head + hd)
    C, ps, scale = 56, 16, 0.9 / math.sqrt(hd)
    q_dim, kv_dim = n_head * hd, n_kv_head * hd
    w_qkv = (torch.randn(q_dim + 2 * kv_dim, C, generator=g) * 0.2).to(dtype)
    b_qkv = torch.randn(q_dim + 2 * kv_dim, generator=g) * 0.1
    w_out = (torch.randn(C, q_dim, generator=g) * 0.2).to(dtype)
    b_out = torch.randn(C, generator=g) * 0.1
    mixer = NP.MIXERS.build("causal_attention", width=C, n_head=n_head, n_kv_head=n_kv_head, head_dim=hd, scale=scale,
                            window=window)
    mixer.bind({"qkv_weight": w_qkv.to(dev), "qkv_bias": b_qkv.to(dev), "out_weight": w_out.to(dev),
                "out_bias": b_out.to(dev)})
    mixer.prepare(dtype, dev)
    lens = [37, 9]                                       # two requests
    xn_all = [(torch.randn(n, C, generator=g)).to(dtype) for n in lens]
    x0_all = [torch.randn(n, C, generator=g) for n in lens]
    # the plain result on whole sequences
    want = []
    for xn, x0 in zip(xn_all, x0_all):
        qkv = xn.double() @ w_qkv.double().T + b_qkv.double()
        att = P.causal_attention(qkv[:, :q_dim], qkv[:, q_dim:q_dim + kv_dim], qkv[:, q_dim + kv_dim:], n_head, n_kv_head,
                                 scale=scale, window=window)
        want.append(x0.double() + att @ w_out.double().T + b_out.double())
    # the pre-norm block around the same mixer and a feed-forward: x += mixer(norm_1(x)); x += mlp(norm_2(x))
    I = 88
    g1, be1 = 1 + 0.1 * torch.randn(C, generator=g), 0.1 * torch.randn(C, generator=g)
    g2, be2 = 1 + 0.1 * torch.randn(C, generator=g), 0.1 * torch.randn(C, generator=g)
    w1, b1 = (torch.randn(I, C, generator=g) * 0.1).to(dtype), torch.randn(I, generator=g) * 0.1
    w2, b2 = (torch.randn(C, I, generator=g) * 0.1).to(dtype), torch.randn(C, generator=g) * 0.1

    def bind(part, **tensors):
        part.bind({k: v.to(dev) for k, v in tensors.items()})
        part.prepare(dtype, dev)
        return part

    def attention_part():
        return bind(NP.MIXERS.build("causal_attention", width=C, n_head=n_head, n_kv_head=n_kv_head, head_dim=hd,
                                    scale=scale, window=window),
                    qkv_weight=w_qkv, qkv_bias=b_qkv, out_weight=w_out, out_bias=b_out)

    block = NP.BLOCKS["pre_norm"](C, dict(
        norm_1=bind(NP.NORMS.build("layernorm", width=C, eps=2e-5), weight=g1, bias=be1), mixer=attention_part(),
        norm_2=bind(NP.NORMS.build("layernorm", width=C, eps=2e-5), weight=g2, bias=be2),
        feed_forward=bind(NP.FEED_FORWARDS.build("dense_mlp", width=C, inner=I, activation="tanh"),
                          fc_weight=w1, fc_bias=b1, proj_weight=w2, proj_bias=b2)))
    want_block = []
    for x0 in x0_all:
        x = x0.double()
        xn = P.layernorm(x, g1.double(), be1.double(), 2e-5)
        qkv = xn @ w_qkv.double().T + b_qkv.double()
        att = P.causal_attention(qkv[:, :q_dim], qkv[:, q_dim:q_dim + kv_dim], qkv[:, q_dim + kv_dim:], n_head, n_kv_head,
                                 scale=scale, window=window)
        x = x + att @ w_out.double().T + b_out.double()
        h = P.layernorm(x, g2.double(), be2.double(), 2e-5)
        want_block.append(x + P.gelu_tanh(h @ w1.double().T + b1.double()) @ w2.double().T + b2.double())

    ws = Workspace(dev)
    table = torch.tensor([[5, 2, 7, -1], [3, 0, -1, -1]], dtype=torch.int32, device=dev)

    def run(apply, want, tol, cuts):
        layer = torch.zeros(8, 2, n_kv_head, ps, hd, dtype=dtype, device=dev)
        for entries in cuts:                        # entries: (request, first row, rows)
            rows = sum(n for _, _, n in entries)
            starts = [0]
            for _, _, n in entries:
                starts.append(starts[-1] + n)
            pos0 = [a for _, a, _ in entries]
            ctx = StepContext(
                n_rows=rows, n_entries=len(entries), max_rows=64,
                tokens=torch.zeros(rows, dtype=torch.int32, device=dev),
                positions=torch.tensor([a + i for _, a, n in entries for i in range(n)], dtype=torch.int32, device=dev),
                row_entry=torch.tensor([e for e, (_, _, n) in enumerate(entries) for _ in range(n)], dtype=torch.int32,
                                       device=dev),
                entry_start=torch.tensor(starts, dtype=torch.int32, device=dev),
                entry_pos0=torch.tensor(pos0, dtype=torch.int32, device=dev),
                entry_slot=torch.arange(len(entries), dtype=torch.int32, device=dev),
                status=torch.zeros(1, dtype=torch.int32, device=dev), workspace=ws,
                host_entry_start=starts, host_entry_pos0=pos0, host_entry_slot=list(range(len(entries))),
                max_q_len=max(n for _, _, n in entries), max_kv_len=max(a + n for _, a, n in entries))
            x = torch.zeros(64, C, device=dev)
            x[:rows] = torch.cat([x0_all[r][a:a + n] for r, a, n in entries]).to(dev)
            view = KVCacheView(layer, torch.stack([table[r] for r, _, _ in entries]).contiguous(), ps, window)
            apply(x, ctx, view, entries)
            assert int(ctx.status.item()) == 0
            at = 0
            for r, a, n in entries:
                assert (x[at:at + n].cpu().double() - want[r][a:a + n]).abs().max() < tol, (r, a, n)
                at += n

    # a prompt portion beside another request's single token; the other way round; then single tokens
    cuts = [[(0, 0, 30), (1, 0, 1)], [(1, 1, 7), (0, 30, 1)], [(0, 31, 1), (1, 8, 1)]] + [[(0, i, 1)] for i in range(32, 37)]

    def apply_mixer(x, ctx, view, entries):
        xn = torch.zeros(64, C, dtype=dtype, device=dev)
        xn[:ctx.n_rows] = torch.cat([xn_all[r][a:a + n] for r, a, n in entries]).to(dev)
        mixer.forward(xn, x, ctx, view, None)

    run(apply_mixer, want, 5e-5 if dtype == torch.float32 else 6e-2, cuts)
    run(lambda x, ctx, view, entries: block.forward(x, ctx, view, None, True, dtype), want_block,
        1e-4 if dtype == torch.float32 else 1e-1, cuts)


def test_unsupported_sizes_are_refused_with_a_clear_error():
    from nanoinfer_b200 import parts as NP
    with pytest.raises(ValueError, match="head_dim"):
        NP.MIXERS.build("causal_attention", width=60, n_head=5, n_kv_head=5, head_dim=12, scale=1.0)
    with pytest.raises(ValueError, match="multiple"):
        NP.MIXERS.build("causal_attention", width=64, n_head=4, n_kv_head=3, head_dim=16, scale=1.0)
    with pytest.raises(ValueError, match="activation"):
        NP.FEED_FORWARDS.build("dense_mlp", width=8, inner=8, activation="relu")
    with pytest.raises(KeyError, match="unknown mixer"):
        NP.MIXERS.build("no_such_mixer")
