"""The engine at layer sizes of the 8B class (hidden 4096, 32 heads over 8 kv
heads of size 128, intermediate 14336, llama3 rope scaling; two layers and a
32k vocabulary to keep it quick): bfloat16 against the float32 engine under
different ways of cutting the work.  The float32 engine itself is checked
against the plain implementation at small sizes; here it is the yardstick,
because a float64 CPU pass over these sizes would take minutes.  This is where
the tensor-core product, the tile-mode and split-mode attention and the fused
epilogues run at their real tile counts inside the engine."""
import pytest
import torch

from helpers import random_tokens

pytestmark = pytest.mark.gpu

CFG = {
    "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 32000,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 8192,
}


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
                rows[(rid, start + w)] = logits[r].float().cpu()
                r += 1
    return rows


@pytest.fixture(scope="module")
def models():
    import infernum_b200 as ib
    return {d: ib.random_model(CFG, seed=7, dtype=d) for d in ("float32", "bfloat16")}


def test_8b_class_layers_under_every_cut(models):
    seqs = {"a": random_tokens(700, 32000, 1), "b": random_tokens(130, 32000, 2),
            "c": random_tokens(300, 32000, 3), "d": random_tokens(40, 32000, 4)}
    picks = {"a": [0, 1, 63, 64, 511, 512, 699], "b": [0, 129], "c": [5, 299], "d": [39]}
    whole = [[(rid, len(s), picks[rid])] for rid, s in seqs.items()]
    ref = run(models["float32"], seqs, whole)
    scale = max(v.abs().max().item() for v in ref.values())

    def check(rows, tol, what):
        for key, row in rows.items():
            if key in ref:
                err = (row - ref[key]).abs().max().item() / scale
                assert err < tol, f"{what}: request {key[0]} position {key[1]}: {err:.3e}"

    # float32: portions and a mixed batch equal whole prompts to rounding
    chunks = []
    pos = 0
    while pos < 700:
        n = min(512 if pos == 0 else 97, 700 - pos)
        chunks.append([("a", n, [w - pos for w in picks["a"] if pos <= w < pos + n])])
        pos += n
    check(run(models["float32"], {"a": seqs["a"]}, chunks), 2e-5, "float32 in portions")
    # bfloat16: whole prompts (tile-mode attention, library product above 64 tokens)
    check(run(models["bfloat16"], seqs, whole), 4e-2, "bfloat16 whole")
    # bfloat16: a prompt in portions, its tail one token at a time (tcgen05 product,
    # split-mode attention), beside portions and single tokens of the others
    plan = [[("a", 512, [0, 1, 63, 64, 511]), ("b", 100, [0]), ("d", 39, [])],
            [("a", 150, [0]), ("b", 29, []), ("c", 250, [5]), ("d", 1, [0])],
            [("a", 2, []), ("b", 1, [0]), ("c", 49, [])]]
    # after these three steps a has 664 of its 700 tokens, c 299 of 300, b and d are done:
    # c's last token rides with a's next one, then a decodes alone; the last row of each is wanted
    plan.append([("a", 1, []), ("c", 1, [0])])
    plan += [[("a", 1, [0] if 665 + i == 699 else [])] for i in range(35)]
    rows = run(models["bfloat16"], seqs, plan)
    assert ("a", 699) in rows and ("b", 129) in rows and ("c", 299) in rows and ("d", 39) in rows
    check(rows, 4e-2, "bfloat16 mixed")
