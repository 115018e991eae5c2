"""Whole prompts of 2,048 tokens at a width of 5120 with 40 heads and as many
key/value heads (intermediate 13824), step after step.

At these sizes every product of a layer runs on pairs of SMs in 216 to 864
tiles, and the prompt attention in 640 CTAs.  With the product on pairs of SMs
launched as a programmatic dependent (its CTAs, each filling an SM, arriving
under the tail of the kernels before it), such steps now and then never ended:
the product's MMA issuer reported its time-out and the rest of the kernel stayed
in its wait for the grid before.  The steps run in a child process with a time
limit, so that a step that does not end fails this test instead of holding the
whole run."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

CHILD = textwrap.dedent("""
    import torch
    import infernum_b200 as ib
    from infernum_b200.cache import CacheManager
    from infernum_b200.engine.step import ModelRunner, StepEntry

    cfg = {"model_type": "llama", "num_hidden_layers": 6, "hidden_size": 5120, "num_attention_heads": 40,
           "num_key_value_heads": 40, "head_dim": 128, "intermediate_size": 13824, "vocab_size": 32000,
           "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
           "max_position_embeddings": 4096}
    model = ib.random_model(cfg, seed=3, dtype="bfloat16", device="cuda:0")
    T = 2048
    cache = CacheManager(model.cache_needs(), page_size=16, num_pages=T // 16 + 2, max_requests=1,
                         dtype=model.rt.dtype, device=model.rt.device)
    runner = ModelRunner(model, cache, max_rows=T, max_entries=1)
    prompt = torch.randint(0, 32000, (T,), generator=torch.Generator().manual_seed(5)).tolist()
    first = None
    for i in range(40):
        rc = cache.admit(("prompt", i))
        cache.extend(rc, T)
        logits = runner.step([StepEntry(rc, prompt, [T - 1])]).float()
        runner.check_errors()
        cache.release(rc)
        assert torch.isfinite(logits).all()
        if first is None:
            first = logits
        else:
            assert (logits - first).abs().max().item() <= 1e-3 * first.abs().max().item(), i
    print("steps done", flush=True)
""")


def test_whole_prompts_at_width_5120_with_40_heads_run_to_the_end():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    try:
        done = subprocess.run([sys.executable, "-c", CHILD], cwd=root, env=env, capture_output=True, text=True,
                              timeout=240)
    except subprocess.TimeoutExpired as exc:
        pytest.fail("the steps did not end within the time limit; output so far: %s" % ((exc.stdout or b"")[-2000:],))
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    assert "steps done" in done.stdout
