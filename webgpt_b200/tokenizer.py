"""The reference's two tokenizers (tokenizer.js) for the host side of GPT.generate: strings in, token ids out.

SimpleTokenizer (tokenizer.js:25-45) maps single characters through a JSON table. GPT2Tokenizer
(tokenizer.js:50-160) is byte-level BPE over a merge list ("vocab.bpe") and a token table ("gpt_tokens.json").
Both read their files from a directory the caller names; none is shipped here. When the token table is absent the
GPT-2 table is rebuilt from the merge list the way the published GPT-2 vocabulary is laid out: the 256 byte
symbols in bytes_to_unicode order, then one token per merge in file order, then "<|endoftext|>".
"""
import json
import os

import regex


class Tokenizer:
    """tokenizer.js:1-23."""

    def __init__(self):
        self.encoder = None
        self.decoder = None
        self.vocab_size = None

    def load(self, folder):
        raise NotImplementedError("Not implemented.")

    def getVocabSize(self):
        return self.vocab_size

    def encode(self, text):
        raise NotImplementedError("Not implemented.")

    def decode(self, arr):
        raise NotImplementedError("Not implemented.")


class SimpleTokenizer(Tokenizer):
    """tokenizer.js:25-45: one token per character."""

    def load(self, folder=None, table=None):
        if table is None:
            with open(os.path.join(folder, "simple_tokens.json"), encoding="utf-8") as f:
                table = json.load(f)
        self.encoder = dict(table)
        self.decoder = {v: k for k, v in self.encoder.items()}
        self.vocab_size = len(self.encoder)
        return self

    def encode(self, text):
        return [self.encoder[c] for c in text]

    def decode(self, arr):
        return "".join(self.decoder[int(t)] for t in arr)


def bytes_to_unicode():
    """tokenizer.js:190-207: a printable stand-in character for each of the 256 byte values."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + \
        list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


def get_pairs(word):
    """tokenizer.js:209-218, as an ordered list without repeats (a JS Set keeps insertion order)."""
    pairs = []
    for a, b in zip(word, word[1:]):
        if (a, b) not in pairs:
            pairs.append((a, b))
    return pairs


class GPT2Tokenizer(Tokenizer):
    """tokenizer.js:50-160."""

    PAT = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""

    def __init__(self):
        super().__init__()
        self.pat = regex.compile(self.PAT)
        self.byte_encoder = None

    def load(self, folder=None, bpe_text=None, encoder=None):
        if bpe_text is None:
            with open(os.path.join(folder, "vocab.bpe"), encoding="utf-8") as f:
                bpe_text = f.read()
        lines = bpe_text.split("\n")
        merges = [tuple(x.split()) for x in lines[1:len(lines) - 1]]  # first line is a header, last is empty
        merges = [m for m in merges if len(m) == 2]
        self.byte_encoder = bytes_to_unicode()
        self.byte_decoder = {v: k for k, v in self.byte_encoder.items()}
        if encoder is None and folder is not None:
            path = os.path.join(folder, "gpt_tokens.json")
            try:
                with open(path, encoding="utf-8") as f:
                    encoder = json.load(f)
            except (OSError, ValueError):
                encoder = None  # absent, or a placeholder that is not JSON
        if encoder is None:
            symbols = list(self.byte_encoder.values())
            encoder = {s: i for i, s in enumerate(symbols)}
            for a, b in merges:
                encoder.setdefault(a + b, len(encoder))
            encoder.setdefault("<|endoftext|>", len(encoder))
        self.encoder = encoder
        self.decoder = {v: k for k, v in encoder.items()}
        # the reference keys its rank table by the pair's array-to-string form "first,second" (dictZip over
        # arrays, tokenizer.js:85,180-186); the same key is used here so that look-ups behave identically
        self.bpe_ranks = {",".join(m): i for i, m in enumerate(merges)}
        self.cache = {}
        self.vocab_size = len(encoder)
        return self

    def encode(self, text):
        if self.byte_encoder is None:
            raise RuntimeError("Tokenizer not loaded.")
        out = []
        for token in self.pat.findall(text):
            token = "".join(self.byte_encoder[b] for b in token.encode("utf-8"))
            out.extend(self.encoder[x] for x in self.bpe(token).split(" "))
        return out

    def decode(self, tokens):
        if self.byte_encoder is None:
            raise RuntimeError("Tokenizer not loaded.")
        text = "".join(self.decoder[int(t)] for t in tokens)
        return bytes(self.byte_decoder[c] for c in text).decode("utf-8", errors="replace")

    def bpe(self, token):
        if token in self.cache:
            return self.cache[token]
        word = list(token)
        pairs = get_pairs(word)
        if not pairs:
            return token
        while True:
            # lowest-ranked pair; pairs without a rank all share the sentinel 10e10 and the last one stays
            best = {}
            for p in pairs:
                best[self.bpe_ranks.get(",".join(p), 10e10)] = p
            bigram = best[min(best)]
            if ",".join(bigram) not in self.bpe_ranks:
                break
            first, second = bigram
            new_word = []
            i = 0
            while i < len(word):
                try:
                    j = word.index(first, i)
                except ValueError:
                    new_word.extend(word[i:])
                    break
                new_word.extend(word[i:j])
                i = j
                if word[i] == first and i < len(word) - 1 and word[i + 1] == second:
                    new_word.append(first + second)
                    i += 2
                else:
                    new_word.append(word[i])
                    i += 1
            word = new_word
            if len(word) == 1:
                break
            pairs = get_pairs(word)
        out = " ".join(word)
        self.cache[token] = out
        return out
