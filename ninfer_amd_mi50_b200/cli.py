"""The ``ninfer`` command line, with the reference's flags where it has them.

Reference: src/apps/ninfer.cpp:55-119.  Kept with their meanings and defaults:
``<model_dir>``, ``--prompt``, ``--raw``, ``--system``, ``--max-context`` (32768),
``--prefill-chunk`` (512), ``--max-new`` (512), ``--temperature`` (0.7; 0 = greedy),
``--top-k`` (50), ``--top-p`` (0.95), ``--repeat-penalty`` (1.05), ``--seed`` (0 -> 1234 for a
one-shot run, ninfer.cpp:205), ``--graph``, ``--log-level``.  Dropped: ``--gpus``, ``--quant``,
``--parallel``, ``--verify`` (one GPU, no quantisation), ``--no-thinking`` (Qwen3 only).
Added: ``--prompt-ids`` / ``--prompt-ids-file`` (token ids in, for models without a
tokenizer.json), ``--print-ids``, ``--dtype``, ``--random-weights SEED`` (a folder with only
config.json), ``--page-size``, ``--cache-tokens``, ``--num-sequences``, ``--max-batched-tokens``.
The answer goes to stdout, diagnostics to stderr (ninfer.cpp:2).
"""

from __future__ import annotations

import argparse
import sys
from typing import List


def parse_ids(text: str) -> List[int]:
    return [int(x) for x in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="ninfer", description="Qwen2-MoE generation on one B200")
    ap.add_argument("model_dir")
    ap.add_argument("--prompt", help="one-shot generation from text (needs tokenizer.json)")
    ap.add_argument("--system", default="", help="system message")
    ap.add_argument("--raw", action="store_true", help="treat the prompt as raw text (no template)")
    ap.add_argument("--prompt-ids", action="append", default=[], help="token ids, e.g. 1,2,3 (repeatable)")
    ap.add_argument("--prompt-ids-file", help="file with one prompt of token ids per line")
    ap.add_argument("--print-ids", action="store_true", help="print generated token ids, not text")
    ap.add_argument("--max-context", type=int, default=32768, help="KV capacity in tokens per request")
    ap.add_argument("--prefill-chunk", type=int, default=512, help="prefill chunk size")
    ap.add_argument("--max-new", type=int, default=512, help="new tokens per generation")
    ap.add_argument("--temperature", type=float, default=0.7, help="sampling temperature (0 = greedy)")
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.95, help="nucleus probability")
    ap.add_argument("--repeat-penalty", type=float, default=1.05, help="repetition penalty")
    ap.add_argument("--seed", type=int, default=0, help="sampling seed (0 = 1234 for a one-shot run)")
    ap.add_argument("--graph", action="store_true", default=True, help="CUDA-graph decode (default on)")
    ap.add_argument("--no-graph", dest="graph", action="store_false")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32", "bfloat16", "float32"])
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--cache-tokens", type=int, default=None)
    ap.add_argument("--num-sequences", type=int, default=None)
    ap.add_argument("--max-batched-tokens", type=int, default=None)
    ap.add_argument("--log-level", default="warn", choices=["debug", "info", "warn", "error"])
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from . import log
    log.set_level(args.log_level)
    prompts: List[List[int]] = [parse_ids(p) for p in args.prompt_ids]
    if args.prompt_ids_file:
        with open(args.prompt_ids_file) as fh:
            prompts += [parse_ids(line) for line in fh if line.strip()]
    if not prompts and args.prompt is None:
        sys.stderr.write("ninfer: give --prompt, --prompt-ids or --prompt-ids-file\n")
        return 2
    from .api import Ninfer
    n_seq = args.num_sequences or max(1, len(prompts))
    total = max(len(p) for p in prompts) + args.max_new if prompts else args.max_context
    eng = Ninfer(args.model_dir, max_context=min(args.max_context, max(total, 64)) if prompts else args.max_context,
                 prefill_chunk=args.prefill_chunk, num_sequences=n_seq, dtype=args.dtype,
                 page_size=args.page_size, cache_tokens=args.cache_tokens,
                 max_batched_tokens=args.max_batched_tokens, use_graph=args.graph,
                 random_weights=args.random_weights)
    text_mode = args.prompt is not None
    if text_mode:
        from .frontend.chat import render_chatml
        text = args.prompt if args.raw else render_chatml(args.system, args.prompt)
        prompts.append(eng.tokenize(text))
    seed = args.seed or 1234
    outs = eng.generate(prompts, max_new_tokens=args.max_new, temperature=args.temperature,
                        top_k=args.top_k, top_p=args.top_p, repetition_penalty=args.repeat_penalty,
                        seed=seed, stop_ids=eng._tok().stop_ids() if text_mode else ())
    for ids in outs:
        if args.print_ids or not text_mode:
            sys.stdout.write(" ".join(str(i) for i in ids) + "\n")
        else:
            sys.stdout.write(eng.detokenize(ids) + "\n")
    sys.stdout.flush()
    st = eng.stats()
    log.info(f"steps={st['steps']} prompt_tokens={st['prompt_tokens']} decode_tokens={st['decode_tokens']} "
             f"preemptions={st['preemptions']}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
