"""The ``ninfer`` command line, with the reference's flags where it has them.

Reference: src/apps/ninfer.cpp:55-119.  Kept with their meanings and defaults:
``<model_dir>``, ``--prompt``, ``--raw``, ``--system``, ``--max-context`` (32768),
``--prefill-chunk`` (2048; the reference's 512 suits its GPU, not this one), ``--max-new`` (512),
``--temperature`` (0.7; 0 = greedy),
``--top-k`` (50), ``--top-p`` (0.95), ``--repeat-penalty`` (1.05), ``--seed`` (0 -> 1234 for a
one-shot run, ninfer.cpp:205), ``--graph``, ``--log-level``.  Dropped: ``--gpus``, ``--quant``,
``--parallel``, ``--verify`` (one GPU, no quantisation), ``--no-thinking`` (Qwen3 only).
Added: ``--prompt-ids`` / ``--prompt-ids-file`` (token ids in, for models without a
tokenizer.json), ``--print-ids``, ``--dtype``, ``--random-weights SEED`` (a folder with only
config.json), ``--page-size``, ``--cache-tokens``, ``--num-sequences``, ``--max-batched-tokens``, ``--device``.
The answer goes to stdout, diagnostics to stderr (ninfer.cpp:2).

A templated prompt is tokenized with the chat markers as tokens of their own
(``encode_with_special``, src/runtime/engine.cpp:115-120); ``--raw`` text is encoded as it
stands (engine.cpp:108-112).  One prompt is printed as it is generated, piece by piece
(ninfer.cpp:121-138); several ``--prompt-ids`` run together as one batch and are printed when
all are done.  Without any prompt the program is the reference's chat loop (ninfer.cpp:222-238):
a line from standard input is a user turn, the conversation so far is the prompt of the next.
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
    ap.add_argument("--prefill-chunk", type=int, default=2048, help="prefill chunk size")
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
    ap.add_argument("--device", default="cuda:0", help="torch device of the engine (the kernels are CUDA only)")
    ap.add_argument("--log-level", default="warn", choices=["debug", "info", "warn", "error"])
    return ap


class TextPrinter:
    """Prints a generation's text as its tokens arrive: the bytes of all tokens so far, up to the
    last complete UTF-8 character, minus what was printed already (a character may be split
    between two tokens).  Special tokens are not printed (src/runtime/engine.cpp:173)."""

    def __init__(self, tokenizer, out):
        self.tok, self.out, self.ids, self.sent = tokenizer, out, [], 0

    def push(self, token_id: int) -> None:
        if self.tok.is_special(token_id):
            return
        self.ids.append(token_id)
        data = self.tok.decode_bytes(self.ids)
        end = len(data)
        # step back over an unfinished multi-byte character at the end
        k = 1
        while k <= 3 and end - k >= 0 and (data[end - k] & 0xC0) == 0x80:
            k += 1
        if end - k >= 0 and k <= 4:
            lead = data[end - k]
            need = 2 if lead >> 5 == 0b110 else 3 if lead >> 4 == 0b1110 else 4 if lead >> 3 == 0b11110 else 1
            if need > k:
                end -= k
        if end > self.sent:
            self.out.write(data[self.sent:end].decode("utf-8", errors="replace"))
            self.out.flush()
            self.sent = end

    def finish(self) -> str:
        data = self.tok.decode_bytes(self.ids)
        if len(data) > self.sent:
            self.out.write(data[self.sent:].decode("utf-8", errors="replace"))
            self.sent = len(data)
        self.out.write("\n")
        self.out.flush()
        return data.decode("utf-8", errors="replace")


def main(argv=None, stdin=None, stdout=None) -> int:
    args = build_parser().parse_args(argv)
    stdin, stdout = stdin or sys.stdin, stdout or sys.stdout
    from . import log
    log.set_level(args.log_level)
    prompts: List[List[int]] = [parse_ids(p) for p in args.prompt_ids]
    if args.prompt_ids_file:
        with open(args.prompt_ids_file) as fh:
            prompts += [parse_ids(line) for line in fh if line.strip()]
    if prompts and args.prompt is not None:
        sys.stderr.write("ninfer: give either --prompt or token ids, not both\n")
        return 2
    from .api import Ninfer
    from .frontend.chat import render_chatml_messages
    n_seq = args.num_sequences or max(1, len(prompts))
    total = max(len(p) for p in prompts) + args.max_new if prompts else args.max_context
    eng = Ninfer(args.model_dir, max_context=min(args.max_context, max(total, 64)) if prompts else args.max_context,
                 prefill_chunk=args.prefill_chunk, num_sequences=n_seq, dtype=args.dtype,
                 page_size=args.page_size, cache_tokens=args.cache_tokens,
                 max_batched_tokens=args.max_batched_tokens, use_graph=args.graph,
                 random_weights=args.random_weights, device=args.device)
    sampling = dict(max_new_tokens=args.max_new, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                    repetition_penalty=args.repeat_penalty)

    def say(ids: List[int], seed: int) -> str:
        """One generation from text-derived ids, printed as it comes; returns the answer."""
        tok = eng._tok()
        room = eng.max_context - len(ids)
        if room < 1:
            raise ValueError(f"the prompt has {len(ids)} tokens; --max-context is {eng.max_context}")
        printer = TextPrinter(tok, stdout)
        for t in eng.stream(ids, **dict(sampling, max_new_tokens=min(args.max_new, room)), seed=seed,
                            stop_ids=tok.stop_ids()):
            if args.print_ids:
                stdout.write(f"{t} ")
                stdout.flush()
            else:
                printer.push(t)
        if args.print_ids:
            stdout.write("\n")
            stdout.flush()
            return ""
        return printer.finish()

    system = [("system", args.system)] if args.system else []
    if args.prompt is not None:
        if args.raw:
            ids = eng.tokenize(args.prompt)                                    # the text as it stands
        else:
            ids = eng.tokenize(render_chatml_messages(system + [("user", args.prompt)]), special=True)
        say(ids, args.seed or 1234)
    elif prompts:
        if len(prompts) == 1:
            for t in eng.stream(prompts[0], **sampling, seed=args.seed or 1234):
                stdout.write(f"{t} ")
                stdout.flush()
            stdout.write("\n")
        else:
            for ids in eng.generate(prompts, **sampling, seed=args.seed or 1234):
                stdout.write(" ".join(str(i) for i in ids) + "\n")
        stdout.flush()
    else:
        # the chat loop: every turn's prompt is the whole conversation so far
        eng._tok()                      # fail now, not at the first turn, if there is no tokenizer.json
        sys.stderr.write("ninfer chat ready. Ctrl-D to exit.\n")
        messages = list(system)
        turn = 0
        while True:
            sys.stderr.write("\n> ")
            sys.stderr.flush()
            line = stdin.readline()
            if not line:
                break
            line = line.rstrip("\r\n")
            if not line:
                continue
            messages.append(("user", line))
            ids = eng.tokenize(render_chatml_messages(messages), special=True)
            answer = say(ids, (args.seed + turn) if args.seed else 0)
            messages.append(("assistant", answer))
            turn += 1
    st = eng.stats()
    log.info(f"steps={st['steps']} prompt_tokens={st['prompt_tokens']} decode_tokens={st['decode_tokens']} "
             f"preemptions={st['preemptions']}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
