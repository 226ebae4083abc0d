"""The optional text side: the byte-level BPE used by the command line (no GPU)."""
import json

from cretif_b200.text import ByteLevelBPE, load_tokenizer


def _toy(tmp_path):
    from cretif_b200.text import _byte_table
    b2u = _byte_table()
    sp = b2u[ord(" ")]
    vocab = {b2u[i]: i for i in range(256)}
    merges = [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), (sp, "w")]
    for a, b in merges:
        vocab[a + b] = len(vocab)
    doc = {"model": {"type": "BPE", "vocab": vocab, "merges": [f"{a} {b}" for a, b in merges]},
           "added_tokens": [{"id": 900, "content": "<|end|>", "special": True}]}
    (tmp_path / "tokenizer.json").write_text(json.dumps(doc))
    (tmp_path / "config.json").write_text(json.dumps({"bos_token_id": 900}))
    return vocab, sp


def test_bpe_round_trip_merges_and_specials(tmp_path):
    vocab, sp = _toy(tmp_path)
    tok = load_tokenizer(str(tmp_path))
    assert isinstance(tok, ByteLevelBPE)
    ids = tok.encode("hello world")
    assert ids[0] == vocab["hello"]                       # merged down to one token
    assert vocab[sp + "w"] in ids                         # the space travels with its word
    assert tok.decode(ids) == "hello world"
    assert tok.encode("hello", add_special=True)[0] == 900
    assert tok.decode([900] + ids) == "hello world"       # control tokens are not shown
    text = "naïve café ☕"
    assert tok.decode(tok.encode(text)) == text            # bytes outside the merges survive


def test_no_tokenizer_file_means_token_ids_only(tmp_path):
    assert load_tokenizer(str(tmp_path)) is None
    (tmp_path / "tokenizer.json").write_text(json.dumps({"model": {"type": "Unigram"}}))
    assert load_tokenizer(str(tmp_path)) is None
