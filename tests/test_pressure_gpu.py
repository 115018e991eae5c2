"""Pages run out at the layer sizes of the 13B class (hidden 5120, 40 heads of
128 that are their own key/value heads, intermediate 13824; two layers and a
small vocabulary to keep it quick): with a pool of 0.8 of what the requests
need together, requests are preempted, give their pages back and are computed
again from their tokens so far, and every request still gets the tokens it
gets alone in an engine with room.  The reference has no such behaviour to
compare with: when its pool is exhausted a request waits
(infernum-cuda/tests/batching_integration.rs:261-298)."""
import pytest
import torch

from helpers import Plain, assert_same_up_to_ties, random_tokens

pytestmark = pytest.mark.gpu

CFG = {
    "model_type": "llama", "num_hidden_layers": 2, "hidden_size": 5120, "num_attention_heads": 40,
    "num_key_value_heads": 40, "head_dim": 128, "intermediate_size": 13824, "vocab_size": 2048,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 4096,
}
SEED = 13


@pytest.fixture(scope="module")
def plain():
    from infernum_b200.weights.random_init import model_specs_for, random_tensors
    _, _, specs = model_specs_for(CFG)
    return Plain(None, CFG, {k: v.cpu() for k, v in random_tensors(specs, SEED, "cuda:0", torch.bfloat16).items()})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_13b_class_layers_under_page_pressure_equal_solo_runs(plain, dtype):
    import infernum_b200 as ib
    model = ib.random_model(CFG, seed=SEED, dtype=dtype)
    n_req, prompt_len, new_tokens, block = 8, 160, 64, 16
    prompts = [random_tokens(prompt_len - 7 * i, CFG["vocab_size"], 300 + i) for i in range(n_req)]
    sampled = ib.SamplingParams(temperature=0.8, top_p=0.95, seed=17)
    opts = [ib.GenerateOptions(max_new_tokens=new_tokens, ignore_eos=True, sampling=sampled if i == 3 else None)
            for i in range(n_req)]
    per_req = -(-(prompt_len + new_tokens) // block)
    base = dict(max_prefill_tokens=128, block_size=block, max_tokens_per_step=128 + n_req,
                max_model_len=prompt_len + new_tokens + 1)
    tight = ib.Engine(model, ib.BatchConfig(max_batch_size=n_req, num_blocks=int(0.8 * n_req * per_req), **base))
    got = tight.generate_batch(prompts, opts)
    assert tight.stats.preemptions > 0
    assert tight.cache.free_pages() == [int(0.8 * n_req * per_req)] and tight.cache.num_free_slots == n_req
    solo = ib.Engine(model, ib.BatchConfig(max_batch_size=1, num_blocks=per_req + 2, **base))
    compared = 0
    for p, o, g in zip(prompts, opts, got):
        want = solo.generate(p, o)
        assert len(g) == len(want) == new_tokens
        compared += assert_same_up_to_ties(plain, p, g, want, dtype, sampling=o.sampling)
    assert solo.stats.preemptions == 0
    if dtype == "float32":
        assert compared == n_req * new_tokens
