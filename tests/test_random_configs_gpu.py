"""Random configurations of the architecture and random ways of cutting requests into steps: the step
function against the plain implementation, in 32-bit and in bfloat16.

Every size is drawn anew per case (head sizes in steps of 16 up to 128, one to seven heads, one to
three layers, an inner width that is no multiple of the width, vocabularies that are no power of two,
the norm's eps, the activation, tied or untied head, the per-layer score scale, pages of 16 to 64
positions), the pool holds about
60 % of the pages that all requests of a case would need at once, and each step takes a random
portion (1 to 400 tokens) of a random subset of the live requests and asks for the logits at random
places.  The seeds are fixed; a failure names the case."""
import json
import os
import random

import pytest
import torch

from conftest import sharpen_attention

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 6e-2}


def write_model(cfg_dict, out_dir, dtype, seed, sharpen):
    from nanoinfer_b200.config import GPT2Config
    from nanoinfer_b200.models.model import Model
    from nanoinfer_b200.registry import get_architecture
    from nanoinfer_b200.weights import random_tensors, write_safetensors

    cfg = GPT2Config.from_dict(cfg_dict)
    model = Model(get_architecture(cfg.architecture).build_spec(cfg), cfg)
    tensors = sharpen_attention(random_tensors(model, seed, 0.02, torch.float32), sharpen)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), {k: v.to(dtype) for k, v in tensors.items()})


def random_config(rnd):
    hd, n_head = rnd.choice([16, 32, 48, 64, 80, 96, 112, 128]), rnd.choice([1, 2, 3, 4, 5, 7])
    width = hd * n_head
    return dict(architectures=["GPT2LMHeadModel"], vocab_size=rnd.choice([97, 256, 1000, 1533, 2048, 3001]),
                n_positions=rnd.choice([96, 160, 272, 400]), n_embd=width, n_layer=rnd.choice([1, 2, 3]), n_head=n_head,
                n_inner=rnd.choice([None, 8 * rnd.randint(4, 80), 4 * width, 24 * rnd.randint(3, 40)]),
                layer_norm_epsilon=rnd.choice([1e-5, 1e-6, 3e-4]), activation_function=rnd.choice(["gelu_new", "gelu"]),
                tie_word_embeddings=rnd.choice([True, False]),
                scale_attn_by_inverse_layer_idx=rnd.choice([True, False]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", range(16))
def test_random_configuration_cut_at_random(case, dtype, tmp_path):
    from plain_gpt2 import PlainGPT2
    from nanoinfer_b200 import load_model
    from nanoinfer_b200.cache import CacheManager
    from nanoinfer_b200.engine import ModelRunner, StepItem

    rnd = random.Random(7000 + case)
    cfg = random_config(rnd)
    torch_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
    write_model(cfg, str(tmp_path), torch_dtype, seed=case + 1, sharpen=rnd.choice([2.0, 4.0]))
    plain = PlainGPT2(str(tmp_path))
    model = load_model(str(tmp_path), torch_dtype, "cuda")
    limit, vocab = cfg["n_positions"], cfg["vocab_size"]
    lens = [rnd.randint(2, limit) for _ in range(rnd.randint(2, 6))]
    toks = [[rnd.randrange(vocab) for _ in range(n)] for n in lens]
    want = [plain.logits(t).float() for t in toks]
    page = rnd.choice([16, 32, 48, 64])
    pages_of = lambda n: -(-n // page)
    pages = max(max(pages_of(n) for n in lens) + 2, int(0.6 * sum(pages_of(n) for n in lens)))
    cache = CacheManager(model.kv_needs(), model.state_needs(), max_tokens=pages * page, max_requests=4, page_size=page,
                         dtype=torch_dtype, device=torch.device("cuda"), max_positions=model.max_positions)
    runner = ModelRunner(model, cache, max_rows=rnd.choice([64, 200, 512]), max_entries=4)
    pending, live, checked = list(range(len(lens))), {}, 0
    while pending or live:
        while pending and len(live) < 4:
            i = pending[0]
            still = sum(pages_of(lens[j]) - pages_of(at) for j, (_, at) in live.items())
            if cache.pages_free()[0] < pages_of(lens[i]) + still:
                break
            pending.pop(0)
            live[i] = (cache.open_request(), 0)
        assert live, f"case {case}: no request fits the pool"
        items, meta, rows = [], [], 0
        for i, (req, at) in list(live.items()):
            if rnd.random() < 0.2 and len(live) > 1:
                continue                                   # this request sits the step out
            n = min(lens[i] - at, rnd.choice([1, 1, 2, 3, 7, 16, 17, 33, 64, 100, 400]), runner.max_rows - rows)
            if n <= 0:
                continue
            places = sorted(rnd.sample(range(n), min(n, rnd.randint(0, 3))))
            items.append(StepItem(req, toks[i][at:at + n], places))
            meta.append((i, at, n, places))
            rows += n
        if not items:
            continue
        out = runner.step(items)
        k = 0
        for i, at, n, places in meta:
            for j in places:
                diff = float((out[k].float().cpu() - want[i][at + j]).abs().max())
                assert diff <= TOL[dtype], f"case {case} {cfg}: request {i}, position {at + j}: {diff:.3e}"
                k += 1
                checked += 1
            if at + n == lens[i]:
                cache.close_request(live[i][0])
                del live[i]
            else:
                live[i] = (live[i][0], at + n)
    cache.check()
    assert cache.pages_used() == [0] and checked > 0
