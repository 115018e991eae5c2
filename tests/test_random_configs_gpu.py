"""Configurations drawn at random - head sizes in steps of 16, any number of
heads and groups, widths, intermediate sizes and vocabularies that are no power
of two, pages of several sizes - through the engine against the plain
implementation: a prompt long enough for the kernels that work on tiles of 256
tokens, cut in two uneven portions, then tokens decoded one by one beside a
second request.  Sizes that a fast kernel cannot take must end up on a slower
one, never in a wrong result."""
import random

import pytest

from helpers import TOL, Plain, compare_trace, make_model_folder, peak_tokens, random_tokens, \
    run_trace_inprocess

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    rng = random.Random(seed)
    head_dim = rng.choice([16, 32, 48, 64, 80, 96, 112, 128])
    kv_heads = rng.choice([1, 2, 3])
    group = rng.choice([1, 2, 3, 4, 5, 8])
    cfg = {
        "model_type": "llama", "num_hidden_layers": rng.choice([1, 2, 3]),
        "hidden_size": 8 * rng.randint(6, 40), "num_attention_heads": kv_heads * group,
        "num_key_value_heads": kv_heads, "head_dim": head_dim,
        "intermediate_size": rng.choice([64 * rng.randint(1, 6), 8 * rng.randint(5, 50), rng.randint(30, 300)]),
        "vocab_size": rng.randint(90, 700), "rope_theta": rng.choice([10000.0, 500000.0, 1234.5]),
        "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-4]), "tie_word_embeddings": rng.random() < 0.5,
        "max_position_embeddings": 512,
    }
    if rng.random() < 0.5:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": rng.choice([2.0, 8.0, 32.0]),
                               "low_freq_factor": 1.0, "high_freq_factor": rng.choice([2.0, 4.0]),
                               "original_max_position_embeddings": rng.choice([64, 256])}
    return cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(8))
def test_random_configuration(seed, dtype, tmp_path):
    cfg = draw_config(seed)
    rng = random.Random(1000 + seed)
    page_size = rng.choice([4, 8, 16, 32])
    folder = make_model_folder(str(tmp_path / "model"), cfg, seed=seed)
    plain = Plain(folder)
    n = rng.randint(290, 330)
    seqs = {"long": random_tokens(n + 6, cfg["vocab_size"], seed), "short": random_tokens(23, cfg["vocab_size"], seed + 1)}
    first = rng.choice([256, 257, 270])
    steps = [
        {"step": 0, "entries": [{"id": "long", "tokens": seqs["long"][:first], "want": [0, 63, 64, first - 1]}], "end": []},
        {"step": 1, "entries": [{"id": "long", "tokens": seqs["long"][first:n], "want": [0, n - first - 1]},
                                {"id": "short", "tokens": seqs["short"][:20], "want": [19]}], "end": []},
    ]
    for i in range(3):  # both decode; then the long one alone
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": "long", "tokens": [seqs["long"][n + 2 * i]], "want": [0]},
                                  {"id": "short", "tokens": [seqs["short"][20 + i]], "want": [0]}]})
        steps.append({"step": len(steps), "end": [],
                      "entries": [{"id": "long", "tokens": [seqs["long"][n + 2 * i + 1]], "want": [0]}]})
    steps[-1]["end"] = ["long", "short"]
    outputs = run_trace_inprocess(folder, dtype, steps, str(tmp_path / "out"), peak_tokens(steps), page_size)
    compare_trace(steps, outputs, seqs, plain, TOL[dtype])
