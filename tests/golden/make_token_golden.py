"""Makes tests/golden/token/: the tokenizer fixtures.

    python tests/golden/make_token_golden.py /path/to/reference

* toy.json, strings.jsonl, toy.ids: the reference's own fixture (crates/tachyon/tests/fixtures/: a small tokenizer shaped like
  Gemma's, the strings its tests encode, and per string the number of tokens and the FNV-1a 64 of their ids as Hugging Face
  `tokenizers` gives them), every tenth string, so that the files stay small.
* metaspace.json, metaspace.ids: the same vocabulary behind a Metaspace pre-tokenizer that splits at every space and prepends
  one (mmBERT's kind), the ids computed here by Hugging Face `tokenizers`.
* chat.json, chat.jsonl: the toy tokenizer with Gemma 4's chat marks added as special tokens, and the conversations of the
  reference's gemma-4.chat with the text its template renders (the ids there are the real model's and are left out).
"""
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent / "token"
STEP = 10


def fnv(ids):
    h = 0xCBF29CE484222325
    for i in ids:
        for b in int(i).to_bytes(4, "little"):
            h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def main(reference: str) -> None:
    from tokenizers import Tokenizer

    src = Path(reference) / "crates/tachyon/tests/fixtures"
    HERE.mkdir(parents=True, exist_ok=True)
    lines = (src / "strings.jsonl").read_text(encoding="utf-8").splitlines()[::STEP]
    ids = (src / "toy.ids").read_text().splitlines()[::STEP]
    (HERE / "strings.jsonl").write_text("\n".join(lines) + "\n", encoding="utf-8")
    (HERE / "toy.ids").write_text("\n".join(ids) + "\n")
    toy = json.loads((src / "toy.json").read_text(encoding="utf-8"))
    (HERE / "toy.json").write_text(json.dumps(toy, ensure_ascii=False), encoding="utf-8")
    strings = [json.loads(l) for l in lines]

    # the toy tokenizer itself, through Hugging Face here: the reference's ids must come out again
    hf = Tokenizer.from_file(str(HERE / "toy.json"))
    hf.encode_special_tokens = True  # a special token's text in a text stays text, as the reference encodes
    for s, line in zip(strings, ids):
        got = hf.encode(s, add_special_tokens=False).ids
        assert f"{len(got)} {fnv(got):016x}" == line, s

    meta = json.loads(json.dumps(toy))
    meta["normalizer"] = None
    meta["pre_tokenizer"] = {"type": "Metaspace", "replacement": "▁", "prepend_scheme": "always", "split": True}
    meta["decoder"] = {"type": "Metaspace", "replacement": "▁", "prepend_scheme": "always", "split": True}
    (HERE / "metaspace.json").write_text(json.dumps(meta, ensure_ascii=False), encoding="utf-8")
    hf = Tokenizer.from_file(str(HERE / "metaspace.json"))
    hf.encode_special_tokens = True
    out = []
    for s in strings:
        got = hf.encode(s, add_special_tokens=False).ids
        out.append(f"{len(got)} {fnv(got):016x}")
    (HERE / "metaspace.ids").write_text("\n".join(out) + "\n")

    chat = json.loads(json.dumps(toy))
    n = max(max(chat["model"]["vocab"].values()), max(t["id"] for t in chat["added_tokens"])) + 1
    for k, mark in enumerate(["<|turn>", "<turn|>", "<|think|>", "<|channel>", "<channel|>"]):
        chat["added_tokens"].append({"id": n + k, "content": mark, "single_word": False, "lstrip": False, "rstrip": False, "normalized": False, "special": True})
    (HERE / "chat.json").write_text(json.dumps(chat, ensure_ascii=False), encoding="utf-8")
    rows = []
    for line in (src / "gemma-4.chat").read_text(encoding="utf-8").splitlines():
        row = json.loads(line)
        rows.append(json.dumps({"messages": row["messages"], "think": row["think"], "text": row["text"]}, ensure_ascii=False))
    (HERE / "chat.jsonl").write_text("\n".join(rows) + "\n", encoding="utf-8")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
