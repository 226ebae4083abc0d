"""Optional text in and out.  Token ids are the library's interface; a tokenizer is
only used by the command line when the model folder carries a ``tokenizer.json``
with a byte-level BPE model (the kind the reference builds from its file's metadata
in "gpt2" mode, src/tokenizer.cpp:341-496: byte→unicode table, greedy lowest-rank
merges, special tokens matched whole; decode at :500-569)."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Tuple


def _byte_table() -> Dict[int, str]:
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    table, n = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + n)
            n += 1
    return table


class ByteLevelBPE:
    def __init__(self, vocab: Dict[str, int], merges: List[Tuple[str, str]],
                 special: Dict[str, int], bos: Optional[int]):
        self.vocab, self.special, self.bos = vocab, special, bos
        self.rank = {pair: i for i, pair in enumerate(merges)}
        self.inv = {i: t for t, i in vocab.items()}
        self.inv.update({i: t for t, i in special.items()})
        self.b2u = _byte_table()
        self.u2b = {u: b for b, u in self.b2u.items()}

    def _bpe(self, word: List[str]) -> List[str]:
        while len(word) > 1:
            best, at = None, -1
            for i in range(len(word) - 1):
                r = self.rank.get((word[i], word[i + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            word[at:at + 2] = [word[at] + word[at + 1]]
        return word

    def encode(self, text: str, add_special: bool = False) -> List[int]:
        ids: List[int] = [self.bos] if add_special and self.bos is not None else []
        # split on spaces, keeping each space with the word that follows it
        pieces, cur = [], ""
        for ch in text:
            if ch == " " and cur and not cur.endswith(" "):
                pieces.append(cur)
                cur = ch
            else:
                cur += ch
        if cur:
            pieces.append(cur)
        for piece in pieces:
            if piece in self.special:
                ids.append(self.special[piece])
                continue
            word = [self.b2u[b] for b in piece.encode("utf-8")]
            for tok in self._bpe(word):
                if tok in self.vocab:
                    ids.append(self.vocab[tok])
                else:
                    ids.extend(self.vocab[c] for c in tok if c in self.vocab)
        return ids

    def decode(self, ids: List[int]) -> str:
        data = bytearray()
        for i in ids:
            tok = self.inv.get(int(i), "")
            if tok in self.special:
                continue                      # control tokens are not shown
            data.extend(self.u2b.get(c, ord("?")) for c in tok)
        return data.decode("utf-8", errors="replace")


def load_tokenizer(model_dir: str) -> Optional[ByteLevelBPE]:
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    with open(path, "r", encoding="utf-8") as f:
        doc = json.load(f)
    model = doc.get("model", {})
    if model.get("type") != "BPE":
        return None
    merges = [tuple(m.split(" ", 1)) if isinstance(m, str) else tuple(m)
              for m in model.get("merges", [])]
    special = {t["content"]: t["id"] for t in doc.get("added_tokens", []) if t.get("special")}
    bos = None
    cfg = os.path.join(model_dir, "config.json")
    if os.path.isfile(cfg):
        with open(cfg, "r", encoding="utf-8") as f:
            bos = json.load(f).get("bos_token_id")
    return ByteLevelBPE(model.get("vocab", {}), merges, special, bos)
