"""The byte and FLOP counts of a step, taken from the built model and its cache (no GPU): they must
give the reference's closed forms for GPT-2 (crates/core/src/config.rs:29-48,
crates/cli/src/bench.rs:261-271) without reading a single field of the configuration."""
import torch

from conftest import TINY, write_tiny
from nanoinfer_b200 import load_model, measure
from nanoinfer_b200.cache import CacheManager


def test_counts_of_a_gpt2_follow_the_closed_forms(tmp_path):
    for name in ("A", "B"):
        raw = TINY[name]
        d = write_tiny(name, str(tmp_path / name), torch.float32)
        for dtype, size in ((torch.float32, 4), (torch.bfloat16, 2)):
            m = load_model(d, dtype, "cpu")
            c, i, L, v, p = raw["n_embd"], raw["n_inner"], raw["n_layer"], raw["vocab_size"], raw["n_positions"]
            tied = raw["tie_word_embeddings"]
            per_layer = (c * 3 * c + 3 * c) + (c * c + c) + (c * i + i) + (i * c + c) + 4 * c
            n_params = L * per_layer + v * c + p * c + 2 * c + (0 if tied else v * c)
            assert measure.parameter_count(m) == n_params == measure.parameter_count_of_spec(m) == m.config.n_params()
            # a step streams the layers' matrices and the head's (in the engine's dtype) and every vector (32-bit);
            # the token and position tables are touched a row per token and left out unless the head is the table
            matrices = L * (4 * c * c + 2 * c * i) + v * c
            vectors = L * (3 * c + c + i + c + 4 * c) + 2 * c
            assert measure.weight_bytes_per_step(m) == matrices * size + vectors * 4
            cache = CacheManager(m.kv_needs(), m.state_needs(), max_tokens=256, max_requests=2, page_size=16,
                                 dtype=dtype, device=None, max_positions=m.max_positions)
            assert measure.kv_bytes(cache, [10, 33]) == 43 * 2 * L * c * size
            rows = [5, 9, 2]
            want = 2.0 * L * (4 * c * c + 2 * c * i) * 3 + 2.0 * v * c * 2 + 4.0 * c * L * sum(rows)
            assert measure.step_flops(m, rows, 2) == want
