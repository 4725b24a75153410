"""Tokenizer and chat template on a small made-up tokenizer.json."""

import json

import pytest

from ninfer_amd_mi50_b200.frontend.chat import render_chatml
from ninfer_amd_mi50_b200.frontend.tokenizer import Tokenizer, _byte_alphabet


@pytest.fixture
def tok(tmp_path):
    alpha = _byte_alphabet()
    vocab = {alpha[b]: b for b in range(256)}
    merges = []

    def merge(a, b):
        merges.append(f"{a} {b}")
        vocab[a + b] = len(vocab)

    sp = alpha[ord(" ")]
    merge("h", "e"); merge("l", "l"); merge("he", "ll"); merge("hell", "o"); merge(sp, "w"); merge("1", "2")
    added = [{"id": 1000, "content": "<|im_start|>", "special": True},
             {"id": 1001, "content": "<|im_end|>", "special": True},
             {"id": 1002, "content": "<|endoftext|>", "special": True},
             {"id": 1003, "content": "<tool>", "special": False}]
    p = tmp_path / "tokenizer.json"
    p.write_text(json.dumps({"model": {"vocab": vocab, "merges": merges}, "added_tokens": added}))
    return Tokenizer(str(p))


def test_merges_by_rank_and_round_trip(tok):
    ids = tok.encode("hello world 123")
    assert ids[0] == tok.token_to_id["hello"]
    assert tok.token_to_id[_byte_alphabet()[ord(" ")] + "w"] in ids
    assert tok.token_to_id["12"] in ids
    for text in ["hello world 123", "naïve café\n\n  x", "日本語 text's", "tabs\tand\r\nlines"]:
        assert tok.decode(tok.encode(text)) == text


def test_special_tokens(tok):
    text = render_chatml("be brief", "hello")
    assert text == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhello<|im_end|>\n<|im_start|>assistant\n"
    ids = tok.encode_with_special(text)
    assert ids.count(1000) == 3 and ids.count(1001) == 2
    assert 1000 not in tok.encode(text)                 # raw encoding spells the markers out
    assert tok.decode(ids) == text and "<|im_start|>" not in tok.decode(ids, skip_special=True)
    assert tok.eos_id == 1001 and tok.stop_ids() == [1000, 1001, 1002]
    assert tok.is_special(1002) and not tok.is_special(1003)


def test_missing_vocab(tmp_path):
    p = tmp_path / "tokenizer.json"
    p.write_text(json.dumps({"model": {}}))
    with pytest.raises(ValueError, match="vocab"):
        Tokenizer(str(p))
