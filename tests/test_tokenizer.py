"""The host-side tokenizers (tokenizer.js) on a toy merge list written by the test; the published GPT-2 merge list is
used as well when a copy sits where the reference keeps it (it is not part of this repository)."""
import os

import pytest

from webgpt_b200.tokenizer import GPT2Tokenizer, SimpleTokenizer, bytes_to_unicode


def test_simple_tokenizer_round_trip():
    table = {c: i for i, c in enumerate("\n !abcdehlorw")}
    t = SimpleTokenizer().load(table=table)
    ids = t.encode("hello world!")
    assert ids == [table[c] for c in "hello world!"]
    assert t.decode(ids) == "hello world!"
    assert t.getVocabSize() == len(table)


def test_bytes_to_unicode_is_a_bijection_on_printable_stand_ins():
    m = bytes_to_unicode()
    assert len(m) == 256 and len(set(m.values())) == 256
    assert m[ord("A")] == "A" and m[ord(" ")] == "Ġ" and m[0] == "Ā"


def toy():
    bpe = "#version: toy\nh e\nl l\nhe ll\nhell o\nĠ w\nĠw o\no r\n"
    return GPT2Tokenizer().load(bpe_text=bpe)


def test_bpe_merges_in_rank_order_and_round_trips():
    t = toy()
    assert t.bpe("hello") == "hello"            # h e -> he, l l -> ll, he ll -> hell, hell o -> hello
    assert t.bpe("help") == "he l p"
    assert t.bpe("Ġworld") == "Ġwo r l d"   # " w" + "o" merges before "o r" can (rank 5 < 6)
    ids = t.encode("hello world")
    assert [t.decoder[i] for i in ids] == ["hello", "Ġwo", "r", "l", "d"]
    assert t.decode(ids) == "hello world"
    # bytes outside ASCII go through the byte table and come back
    s = "naïve ☃ café"
    assert t.decode(t.encode(s)) == s
    assert t.getVocabSize() == 256 + 7 + 1
    # contractions and digit runs split as the reference's pattern splits them
    assert t.pat.findall("it's 42 days!") == ["it", "'s", " 42", " days", "!"]


def test_published_gpt2_merges_when_available():
    # a checkout of the reference beside this repository, if there is one
    here = os.path.dirname(os.path.abspath(__file__))
    folder = os.path.join(os.path.dirname(os.path.dirname(here)), "reference", "weights", "tokenization")
    if not os.path.exists(os.path.join(folder, "vocab.bpe")):
        pytest.skip("no GPT-2 merge list on this machine")
    t = GPT2Tokenizer().load(folder)
    assert t.getVocabSize() == 50257
    assert t.encode("Hello world") == [15496, 995]
    text = "WebGPT runs GPT-2 in the browser, 117M parameters; café ☃."
    assert t.decode(t.encode(text)) == text
