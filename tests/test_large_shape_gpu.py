"""The engine at layer sizes of the 8B class (hidden 4096, 32 heads over 8 kv
heads of size 128, intermediate 14336, llama3 rope scaling; two layers and a
32k vocabulary to keep it quick) and of the 1B class (hidden 2048, 32 heads
over 8 kv heads of size 64, intermediate 8192, tied embeddings, three layers)
against the plain implementation, in float32
and in bfloat16, under every way of cutting the work: whole prompts, portions
of 512 and less, most of a prompt in one step and its last 32 tokens one by
one, and four requests mixed.  This is where the tensor-core products, the
prompt and the decode attention kernels and the fused epilogues run at their
real tile counts (K = 4096 and 14336, 32 heads of 128) inside the engine, and
the yardstick shares nothing with them: the plain implementation runs on the
CPU in float64 over the same random tensors."""
import pytest
import torch

import plain_llama as pl
from helpers import TOL, random_tokens

pytestmark = pytest.mark.gpu

CFGS = {
    "8b": {
        "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 32000,
        "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192,
    },
    "1b": {
        "model_type": "llama", "num_hidden_layers": 3, "hidden_size": 2048, "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 32000,
        "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192,
    },
}
SEED = 7
SEQS = {"a": random_tokens(700, 32000, 1), "b": random_tokens(130, 32000, 2),
        "c": random_tokens(300, 32000, 3), "d": random_tokens(40, 32000, 4)}
PICKS = {"a": [0, 1, 63, 64, 511, 512] + list(range(667, 700)), "b": [0, 129], "c": [5, 299], "d": [39]}


def run(model, seqs, plan, page_size=16):
    """plan: list of steps, each a list of (request, n tokens, wanted places)."""
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.step import ModelRunner, StepEntry
    cache = CacheManager(model.cache_needs(), page_size=page_size, num_pages=1024, max_requests=8,
                         dtype=model.rt.dtype, device=model.rt.device)
    runner = ModelRunner(model, cache, max_rows=4096)
    rcs = {k: cache.admit(k) for k in seqs}
    fed = {k: 0 for k in seqs}
    rows = {}
    for step in plan:
        entries, who = [], []
        for rid, n, want in step:
            entries.append(StepEntry(rcs[rid], seqs[rid][fed[rid]: fed[rid] + n], want))
            who.append((rid, fed[rid], want))
            fed[rid] += n
        logits = runner.step(entries)
        runner.check_errors()
        r = 0
        for rid, start, want in who:
            for w in want:
                rows[(rid, start + w)] = logits[r].double().cpu()
                r += 1
    return rows


@pytest.fixture(scope="module", params=["8b", "1b"])
def world(request):
    """For one of the shapes: the plain implementation's logits at the picked
    places, over the very tensors the engine's models are made of (drawn once
    on the device; the random generator is all that is shared), and the
    engine's models in both precisions."""
    import infernum_b200 as ib
    from infernum_b200.weights.random_init import model_specs_for, random_tensors
    config = CFGS[request.param]
    _, _, specs = model_specs_for(config)
    weights = {k: v.cpu() for k, v in random_tensors(specs, SEED, "cuda:0", torch.bfloat16).items()}
    cfg = pl.read_config(config)
    rows = {}
    for rid, seq in SEQS.items():
        logits = pl.forward(cfg, weights, seq)
        for pos in PICKS[rid]:
            rows[(rid, pos)] = logits[pos].clone()
    models = {d: ib.random_model(config, seed=SEED, dtype=d) for d in ("float32", "bfloat16")}
    yield request.param, models, rows
    del models
    torch.cuda.empty_cache()


def plans():
    whole = [[(rid, len(s), PICKS[rid])] for rid, s in SEQS.items()]
    chunks, pos = [], 0
    while pos < 700:
        n = min(512 if pos == 0 else 97, 700 - pos)
        chunks.append([("a", n, [w - pos for w in PICKS["a"] if pos <= w < pos + n])])
        pos += n
    tail = [[("a", 668, [0, 1, 63, 64, 511, 512, 667])]] + [[("a", 1, [0])] for _ in range(32)]
    # a prompt in portions, its tail one token at a time, beside portions and single tokens of the others
    mixed = [[("a", 512, [0, 1, 63, 64, 511]), ("b", 100, [0]), ("d", 39, [])],
             [("a", 150, [0]), ("b", 29, []), ("c", 250, [5]), ("d", 1, [0])],
             [("a", 2, []), ("b", 1, [0]), ("c", 49, [])]]
    # after these three steps a has 664 of its 700 tokens, c 299 of 300, b and d are done:
    # c's last token rides with a's next one, then a decodes alone
    mixed.append([("a", 1, []), ("c", 1, [0])])
    mixed += [[("a", 1, [0] if 665 + i >= 667 else [])] for i in range(35)]
    return {"whole": whole, "portions": chunks, "tail": tail, "mixed": mixed}


@pytest.mark.parametrize("cut", ["whole", "portions", "tail", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_layer_sizes_against_plain(world, dtype, cut):
    shape, models, plain_rows = world
    plan = plans()[cut]
    seqs = SEQS if cut in ("whole", "mixed") else {"a": SEQS["a"]}
    rows = run(models[dtype], seqs, plan)
    compared = 0
    for key, row in rows.items():
        ref = plain_rows[key]
        assert torch.isfinite(row).all(), f"{cut}: request {key[0]} position {key[1]}: not finite"
        err = float((row - ref).abs().max() / ref.abs().max())
        assert err < TOL[dtype], f"{shape} {dtype} {cut}: request {key[0]} position {key[1]}: relative error {err:.3e}"
        compared += 1
    assert compared >= {"whole": 44, "portions": 39, "tail": 39, "mixed": 40}[cut]
    if cut in ("tail", "mixed"):
        assert ("a", 699) in rows
