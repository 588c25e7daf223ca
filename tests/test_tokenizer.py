"""The byte-level BPE tokenizer (no GPU): the reference's own unit tests
(crates/core/src/tokenizer.rs:229-252) and a small hand-made vocabulary."""
import json

import pytest

from nanoinfer_b200.tokenizer import (END_OF_TEXT, Tokenizer, TokenizerError, bytes_to_unicode, pre_tokenize,
                                      write_byte_tokenizer)


def test_pre_tokenize_follows_the_pattern():
    assert pre_tokenize("Hello world") == ["Hello", " world"]
    assert pre_tokenize("I'll don't") == ["I", "'ll", " don", "'t"]
    assert pre_tokenize("a  b") == ["a", " ", " b"]
    assert pre_tokenize("x\n\ny ") == ["x", "\n", "\n", "y", " "]
    assert pre_tokenize("pi=3.14!") == ["pi", "=", "3", ".", "14", "!"]
    assert pre_tokenize("") == [] and "".join(pre_tokenize(" déjà vu,  2x\t")) == " déjà vu,  2x\t"


def test_byte_table_is_a_bijection():
    t = bytes_to_unicode()
    assert len(set(t)) == 256 and t[ord(" ")] == "Ġ" and t[ord("A")] == "A" and t[0] == chr(256)


def small_tokenizer():
    b2u = bytes_to_unicode()
    vocab = {c: i for i, c in enumerate(b2u)}
    sp = b2u[ord(" ")]
    merges = [("t", "h"), ("th", "e"), (sp, "the"), ("a", "n"), (sp, "an"), ("é"[0:0] + b2u[0xC3], b2u[0xA9])]
    for a, b in merges:
        vocab[a + b] = len(vocab)
    vocab[END_OF_TEXT] = len(vocab)
    return Tokenizer(vocab, "#version: 0.2\n" + "\n".join(f"{a} {b}" for a, b in merges) + "\n"), vocab


def test_merges_by_rank_and_round_trip():
    tok, vocab = small_tokenizer()
    sp = bytes_to_unicode()[ord(" ")]
    ids = tok.encode("the then an")
    # "the" | " then" -> " the" + "n" | " an"
    assert ids == [vocab["the"], vocab[sp + "the"], vocab["n"], vocab[sp + "an"]]
    for text in ["the then an", "café au lait\n\n  x", "I'll  be there", "日本語 42"]:
        assert tok.decode(tok.encode(text)) == text
    assert tok.encode("a" + END_OF_TEXT + "the") == [vocab["a"], vocab[END_OF_TEXT], vocab["the"]]
    assert tok.decode([vocab[bytes_to_unicode()[0xC3]]]) == "�"        # half of a two-byte character
    assert tok.token_bytes(10 ** 6) == b""


def test_errors_name_the_problem(tmp_path):
    with pytest.raises(TokenizerError, match="vocab.json"):
        Tokenizer.from_folder(str(tmp_path))
    vocab = {c: i for i, c in enumerate(bytes_to_unicode())}
    with pytest.raises(TokenizerError, match="not in the vocabulary"):
        Tokenizer(vocab, "t h\n")
    with pytest.raises(TokenizerError, match="bad merge line"):
        Tokenizer(vocab, "t h e\n")
    del vocab["A"]
    with pytest.raises(TokenizerError, match="no token for the byte"):
        Tokenizer(vocab, "")


def test_byte_tokenizer_for_random_models(tmp_path):
    write_byte_tokenizer(str(tmp_path), 300)
    tok = Tokenizer.from_folder(str(tmp_path))
    assert tok.vocab_size == 257 and tok.end_of_text == 256
    assert tok.encode("Hi é") == list("Hi é".encode()) and tok.decode(tok.encode("Hi é")) == "Hi é"
    assert json.load(open(tmp_path / "vocab.json", encoding="utf-8"))["Ġ"] == 32
    with pytest.raises(TokenizerError, match="at least 257"):
        write_byte_tokenizer(str(tmp_path), 200)


def test_command_line_tokenize_prints_ids_and_pieces(tmp_path, capsys):
    """``tokenize TEXT`` as the reference prints it: an id and its piece per line, then the count."""
    from nanoinfer_b200.cli import main
    from nanoinfer_b200.tokenizer import write_byte_tokenizer
    write_byte_tokenizer(str(tmp_path), 300)
    assert main(["--weights", str(tmp_path), "tokenize", "Hi!"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert lines[-1] == "3 tokens" and len(lines) == 4
    assert [line.split()[1] for line in lines[:3]] == ["'H'", "'i'", "'!'"]
    assert main(["--weights", str(tmp_path / "nothing"), "tokenize", "Hi"]) == 2
