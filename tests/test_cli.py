"""The ``ninfer`` command line: token ids in and out against the plain model, text prompts
through a made-up tokenizer.json (chat markers must arrive as their own ids), text printed
piece by piece, the chat loop; on the CPU with the kernels' plain twins, and on the GPU as
the program itself."""

import io
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_kernels
import plain_model
from tiny_configs import TINY_A, TINY_B, random_tokens

from ninfer_amd_mi50_b200 import cli
from ninfer_amd_mi50_b200.frontend.tokenizer import Tokenizer, _byte_alphabet
from ninfer_amd_mi50_b200.weights import write_random_model

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def write_tokenizer(folder):
    """Bytes as tokens 0..255, a few merges, chat markers at 1000..1002 (inside tiny A's vocabulary)."""
    alpha = _byte_alphabet()
    vocab = {alpha[b]: b for b in range(256)}
    merges = []
    for a, b in (("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o")):
        merges.append(f"{a} {b}")
        vocab[a + b] = len(vocab)
    added = [{"id": 1000, "content": "<|im_start|>", "special": True},
             {"id": 1001, "content": "<|im_end|>", "special": True},
             {"id": 1002, "content": "<|endoftext|>", "special": True}]
    with open(os.path.join(folder, "tokenizer.json"), "w") as fh:
        json.dump({"model": {"vocab": vocab, "merges": merges}, "added_tokens": added}, fh)
    return Tokenizer(os.path.join(folder, "tokenizer.json"))


@pytest.fixture
def folder(tmp_path, monkeypatch):
    d = str(tmp_path / "a")
    write_random_model(TINY_A, 0, d)
    plain_kernels.install(monkeypatch)
    return d


def run_cli(argv, stdin_text=""):
    out = io.StringIO()
    rc = cli.main(argv + ["--device", "cpu", "--dtype", "fp32", "--no-graph", "--repeat-penalty", "1"], stdin=io.StringIO(stdin_text), stdout=out)
    return rc, out.getvalue()


def test_token_ids_in_and_out_equal_the_plain_model(folder):
    pcfg, weights = plain_model.read_model_folder(folder)
    prompts = [random_tokens(n, 1024, 600 + n) for n in (5, 12)]
    want = [plain_model.plain_greedy(pcfg, weights, p, 5) for p in prompts]
    # one prompt: printed token by token
    rc, out = run_cli([folder, "--prompt-ids", ",".join(map(str, prompts[0])), "--temperature", "0", "--max-new", "5"])
    assert rc == 0 and [int(x) for x in out.split()] == want[0]
    # two prompts: one batch, one line each
    rc, out = run_cli([folder, "--prompt-ids", " ".join(map(str, prompts[0])), "--prompt-ids",
                       ",".join(map(str, prompts[1])), "--temperature", "0", "--max-new", "5", "--prefill-chunk", "4"])
    assert rc == 0 and [[int(x) for x in line.split()] for line in out.strip().split("\n")] == want


def test_a_text_prompt_reaches_the_model_with_the_chat_markers_as_tokens(folder, monkeypatch):
    from ninfer_amd_mi50_b200.engine.engine import Engine
    tok = write_tokenizer(folder)
    seen = []
    submit = Engine.submit

    def spy(self, prompt, *a, **k):
        seen.append(list(prompt))
        return submit(self, prompt, *a, **k)

    monkeypatch.setattr(Engine, "submit", spy)
    rc, out = run_cli([folder, "--prompt", "hello", "--system", "be brief", "--temperature", "0", "--max-new", "6"])
    assert rc == 0
    ids = seen[0]
    assert ids.count(1000) == 3 and ids.count(1001) == 2            # the markers, not their spelling
    assert tok.decode(ids) == ("<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhello<|im_end|>\n"
                               "<|im_start|>assistant\n")
    # what was printed is the text of the greedy continuation, up to a special token
    pcfg, weights = plain_model.read_model_folder(folder)
    gen = plain_model.plain_greedy(pcfg, weights, ids, 6)
    cut = next((i for i, t in enumerate(gen) if tok.is_special(t)), len(gen))
    assert out == tok.decode(gen[:cut]) + "\n"
    # --raw: the text as it stands, no template, no markers
    seen.clear()
    rc, _ = run_cli([folder, "--prompt", "<|im_start|>hello", "--raw", "--temperature", "0", "--max-new", "2"])
    assert rc == 0 and 1000 not in seen[0] and tok.decode(seen[0]) == "<|im_start|>hello"


def test_chat_loop_carries_the_conversation(folder, monkeypatch):
    from ninfer_amd_mi50_b200.engine.engine import Engine
    tok = write_tokenizer(folder)
    seen = []
    submit = Engine.submit
    monkeypatch.setattr(Engine, "submit", lambda self, prompt, *a, **k: (seen.append(list(prompt)), submit(self, prompt, *a, **k))[1])
    rc, out = run_cli([folder, "--temperature", "0", "--max-new", "4", "--max-context", "256"], "hello\n\nagain\n")
    assert rc == 0 and len(seen) == 2
    first_answer = out.split("\n")[0]
    text = tok.decode(seen[1])
    assert text.startswith("<|im_start|>user\nhello<|im_end|>\n<|im_start|>assistant\n" + first_answer + "<|im_end|>\n")
    assert text.endswith("<|im_start|>user\nagain<|im_end|>\n<|im_start|>assistant\n")


def test_text_is_printed_at_character_boundaries(tmp_path):
    """A character of three bytes split over two tokens appears when its last byte has come."""
    os.makedirs(tmp_path / "t")
    tok = write_tokenizer(str(tmp_path / "t"))
    out = io.StringIO()
    p = cli.TextPrinter(tok, out)
    data = "a日b".encode()
    shown = []
    for b in data:
        p.push(b)                      # byte tokens have their byte's value as id
        shown.append(out.getvalue())
    assert shown == ["a", "a", "a", "a日", "a日b"]
    p.push(1001)                       # a special token prints nothing
    assert p.finish() == "a日b" and out.getvalue() == "a日b\n"


def test_no_prompt_and_no_tokenizer_is_an_error(folder):
    from ninfer_amd_mi50_b200.api import NinferError
    with pytest.raises(NinferError, match="tokenizer.json"):
        run_cli([folder], "hello\n")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_the_program_on_the_gpu(tmp_path, dtype):
    d = str(tmp_path / "b")
    write_random_model(TINY_B, 1, d)
    pcfg, weights = plain_model.read_model_folder(d)
    prompt = random_tokens(40, TINY_B["vocab_size"], 77)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ninfer"), d, "--prompt-ids",
                        ",".join(map(str, prompt)), "--temperature", "0", "--max-new", "8", "--dtype", dtype,
                        "--prefill-chunk", "16", "--repeat-penalty", "1"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    got = [int(x) for x in p.stdout.split()]
    assert len(got) == 8
    if dtype == "fp32":
        assert got == plain_model.plain_greedy(pcfg, weights, prompt, 8)
    else:
        logits = plain_model.plain_forward(pcfg, weights, prompt + got)[len(prompt) - 1:-1]
        scale = logits.abs().max().item()
        for i, t in enumerate(got):
            assert logits[i, t].item() >= logits[i].max().item() - 3e-2 * scale
