"""Makes tests/golden/token/: the tokenizer fixtures.

    python tests/golden/make_token_golden.py /path/to/reference

* toy.json, strings.jsonl, toy.ids: the reference's own fixture (crates/tachyon/tests/fixtures/: a small tokenizer shaped like
  Gemma's, the strings its tests encode, and per string the number of tokens and the FNV-1a 64 of their ids as Hugging Face
  `tokenizers` gives them), every tenth string, so that the files stay small.
* metaspace.json, metaspace.ids: the same vocabulary behind a Metaspace pre-tokenizer that splits at every space and prepends
  one (mmBERT's kind), the ids computed here by Hugging Face `tokenizers`.
* bytes_gpt2_nfc.json, bytes_cl100k.json, bytes_o200k.json and their .ids: byte-level tokenizers trained here on the strings
  (1,200 tokens each): GPT-2's pattern behind an NFC normalizer (ModernBERT's kind), the cl100k pattern with `ignore_merges`
  (Llama 3's kind), the o200k pattern (Granite Embedding 97M's kind); the ids by Hugging Face `tokenizers`.  nfc.jsonl:
  strings of letters and combining marks (composites, Hangul, excluded compositions), with Python's NFC of each and the
  first tokenizer's ids.
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


PATTERNS = {
    "cl100k": r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+",
    "o200k": r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]*[\p{Ll}\p{Lm}\p{Lo}\p{M}]+(?i:'s|'t|'re|'ve|'m|'ll|'d)?|[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]+[\p{Ll}\p{Lm}\p{Lo}\p{M}]*(?i:'s|'t|'re|'ve|'m|'ll|'d)?|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+",
}


def byte_level(strings) -> None:
    import random
    import unicodedata

    from tokenizers import Regex, Tokenizer, decoders, models, normalizers, pre_tokenizers, trainers

    def make(kind: str):
        tok = Tokenizer(models.BPE(ignore_merges=kind == "cl100k"))
        if kind == "gpt2_nfc":
            tok.normalizer = normalizers.NFC()
            tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=True, use_regex=True)
        else:
            tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(PATTERNS[kind]), behavior="isolated", invert=False),
                                                         pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
        tok.decoder = decoders.ByteLevel()
        trainer = trainers.BpeTrainer(vocab_size=1200, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), special_tokens=["<|endoftext|>"], show_progress=False)
        tok.train_from_iterator(strings, trainer)
        tok.add_tokens(["<body>"])
        tok.encode_special_tokens = True
        return tok

    for kind in ("gpt2_nfc", "cl100k", "o200k"):
        tok = make(kind)
        (HERE / f"bytes_{kind}.json").write_text(tok.to_str(), encoding="utf-8")
        lines = []
        for s in strings:
            got = tok.encode(s, add_special_tokens=False).ids
            lines.append(f"{len(got)} {fnv(got):016x}")
        (HERE / f"bytes_{kind}.ids").write_text("\n".join(lines) + "\n")
        if kind == "gpt2_nfc":
            rng = random.Random(3)
            marks = list(range(0x300, 0x370)) + [0x5B0, 0x5BC, 0x64B, 0x651, 0x93C, 0x9BC, 0x9BE, 0x9D7, 0xB3E, 0xB56, 0xB57, 0xBBE, 0xBD7, 0xC56, 0xCC2, 0xCD5, 0xD3E, 0xD57, 0xDCA, 0xDCF,
                                                 0xDDF, 0xF71, 0xF72, 0xF74, 0xF80, 0x102E, 0x1161, 0x1175, 0x11A8, 0x11C2, 0x1B35, 0x3099, 0x309A, 0x1D165, 0x11127, 0x1133E, 0x114BA, 0x115AF]
            bases = list("aeiounAEIOUcsz") + [chr(c) for c in (0x3B1, 0x3C9, 0x415, 0x438, 0x5D0, 0x5E9, 0x627, 0x64A, 0x915, 0x928, 0x9A1, 0x9C7, 0xB47, 0xB92, 0xBC6, 0xBC7, 0xC46, 0xCBF,
                                                                     0xCC6, 0xD46, 0xD47, 0xDD9, 0xF40, 0x1025, 0x1100, 0x1112, 0xAC00, 0xAC1C, 0xD788, 0x1B05, 0x304B, 0x30AB, 0x212B,
                                                                     0x2126, 0xF900, 0xFB1D, 0x11131, 0x11347, 0x114B9, 0x115B8, 0x1D157)]
            rows = []
            for _ in range(400):
                s = "".join(rng.choice(bases) + "".join(chr(rng.choice(marks)) for _ in range(rng.randrange(0, 4))) for _ in range(rng.randrange(1, 8)))
                rows.append(json.dumps({"text": s, "nfc": unicodedata.normalize("NFC", s), "ids": tok.encode(s, add_special_tokens=False).ids}, ensure_ascii=True))
            (HERE / "nfc.jsonl").write_text("\n".join(rows) + "\n")


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

    byte_level(strings)

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
