"""``generate``: a prompt in, tokens out, with the option names, meanings and
defaults of the reference's example (infernum-examples/examples/generate.rs:37-86):

    generate -m DIR [PROMPT] [-n 100] [--greedy] [-t 0.7] [-p 0.9] [-s 42]
             [-r 1.1] [--repetition-penalty-window 64] [--max-seq-len N]

The model folder defaults to $LLAMA_MODEL_PATH.  The architecture is chosen by
``model_type`` in config.json.  The prompt is text when the folder holds a
``tokenizer.json`` and the ``tokenizers`` package is importable; otherwise
(and always with ``--prompt-ids``) it is a list of token ids such as
"1,15043,3186".  Like the reference it prints the decoding mode, the output as
it is produced and "Generated N tokens in S s (R tokens/sec)" (generate.rs:180-240).
Beyond the reference: ``--dtype`` (bfloat16 or float32), the engine limits
``--block-size``, ``--num-blocks``, ``--max-batch-size``, ``--max-prefill-tokens``,
``--allow-unused-tensors``, and a random-weights mode that needs no checkpoint:

    generate --config config.json --random-weights [--weights-seed 0] "5,6,7,8" -n 16 --greedy

draws the weights on the GPU from the configuration file and a seed (the values
``write_random_model`` would write to a folder for the same two).
"""

from __future__ import annotations

import argparse
import os
import sys
import time
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="generate", description=__doc__,
                                 formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("-m", "--model", default=os.environ.get("LLAMA_MODEL_PATH", "models/llama-3.2-1b"),
                    help="path to the model folder (env LLAMA_MODEL_PATH)")
    ap.add_argument("prompt", nargs="?", default="Hello", help="text prompt, or token ids")
    ap.add_argument("-n", "--max-tokens", type=int, default=100, help="maximum tokens to generate")
    ap.add_argument("--greedy", action="store_true", help="greedy (argmax) decoding instead of sampling")
    ap.add_argument("--no-kv-cache", action="store_true",
                    help="accepted for the reference's option set; this engine always uses its cache")
    ap.add_argument("-t", "--temperature", type=float, default=0.7, help="sampling temperature")
    ap.add_argument("-p", "--top-p", type=float, default=0.9, help="nucleus sampling threshold")
    ap.add_argument("-s", "--seed", type=int, default=42, help="seed of the sampling random numbers")
    ap.add_argument("-r", "--repetition-penalty", type=float, default=1.1,
                    help="repetition penalty (1.0 = off, > 1.0 penalises repeated tokens)")
    ap.add_argument("--repetition-penalty-window", type=int, default=64,
                    help="number of recent tokens the penalty looks at")
    ap.add_argument("--max-seq-len", type=int, default=None,
                    help="longest sequence held in the cache (default: min(model max, 4096))")
    ap.add_argument("--prompt-ids", action="store_true", help="the prompt is a list of token ids")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "f32"])
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--num-blocks", type=int, default=None)
    ap.add_argument("--max-batch-size", type=int, default=32)
    ap.add_argument("--max-prefill-tokens", type=int, default=512)
    ap.add_argument("--config", default=None, metavar="FILE",
                    help="a config.json to build the model from (with --random-weights)")
    ap.add_argument("--random-weights", action="store_true",
                    help="no checkpoint: draw the weights from --config and --weights-seed")
    ap.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights")
    ap.add_argument("--allow-unused-tensors", action="store_true",
                    help="warn about tensors in the checkpoint that the model does not use instead of refusing")
    return ap


def _load_tokenizer(folder: str):
    path = os.path.join(folder, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(path)


def _parse_ids(text: str) -> List[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    from .. import BatchConfig, Engine, GenerateOptions, SamplingParams, load_model, random_model

    if args.random_weights != (args.config is not None):
        print("--config FILE and --random-weights go together", file=sys.stderr)
        return 2
    if args.random_weights:
        import json

        with open(args.config, encoding="utf-8") as fh:
            model = random_model(json.load(fh), seed=args.weights_seed, dtype=args.dtype)
        tokenizer = None
    else:
        model = load_model(args.model, dtype=args.dtype, strict=not args.allow_unused_tensors)
        tokenizer = None if args.prompt_ids else _load_tokenizer(args.model)
    if tokenizer is not None:
        ids = tokenizer.encode(args.prompt, add_special_tokens=False).ids
        if model.spec.bos_token_id is not None:
            ids = [model.spec.bos_token_id] + ids  # the reference encodes with BOS (runtime.rs:99-101)
    else:
        try:
            ids = _parse_ids(args.prompt)
        except ValueError:
            print("no tokenizer.json in the model folder: give the prompt as token ids, "
                  "e.g. \"1,15043,3186\"", file=sys.stderr)
            return 2
    sampling = None if args.greedy else SamplingParams(
        temperature=args.temperature, top_p=args.top_p, seed=args.seed,
        repetition_penalty=args.repetition_penalty,
        repetition_penalty_window=args.repetition_penalty_window)
    options = GenerateOptions(max_new_tokens=args.max_tokens, eos_token_id=model.spec.eos_token_id,
                              sampling=sampling, use_kv_cache=not args.no_kv_cache)
    max_len = args.max_seq_len or min(model.spec.max_position, 4096)
    max_len = max(max_len, len(ids) + args.max_tokens)
    num_blocks = args.num_blocks or (max_len + args.block_size - 1) // args.block_size + 1
    engine = Engine(model, BatchConfig(max_batch_size=args.max_batch_size,
                                       max_prefill_tokens=args.max_prefill_tokens,
                                       block_size=args.block_size, num_blocks=num_blocks,
                                       max_model_len=max_len))
    if sampling:
        print(f"Sampling: temperature={sampling.temperature}, top_p={sampling.top_p}, "
              f"seed={sampling.seed}, repetition_penalty={sampling.repetition_penalty} "
              f"(window={sampling.repetition_penalty_window})")
    else:
        print("Decoding: greedy (argmax)")
    print(f"KV cache: {'enabled' if options.use_kv_cache else 'enabled (always)'}")
    print(args.prompt, end="", flush=True)
    start = time.perf_counter()
    out: List[int] = []
    for tok in engine.generate_stream(ids, options):
        out.append(tok)
        if tokenizer is not None:
            print(tokenizer.decode([tok]), end="", flush=True)
        else:
            print(f" {tok}", end="", flush=True)
    elapsed = time.perf_counter() - start
    print()
    print(f"Generated {len(out)} tokens in {elapsed:.2f}s ({len(out) / max(elapsed, 1e-9):.1f} tokens/sec)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
