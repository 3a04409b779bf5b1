"""Golden vectors for the native tokenizer, made by the REAL reference code.

Run where a checkout of the reference is present (``--reference``)::

    python tests/golden/make_tokenizer_golden.py --reference /path/to/cudaBERT

It imports the reference's tokenizer unmodified (apps/pytorch_pretrained_bert/tokenization.py) and
its per-line feature function (apps/tokenlizer.py:122-147), builds a seeded synthetic vocabulary
and corpus (hand-made sentences in several scripts plus random strings over many Unicode blocks),
and stores what the reference returns for them in ``tokenizer_golden.json``:

  vocab      the vocabulary file, one token per line
  tokenize   [text, ids] pairs of BertTokenizer.tokenize + convert_tokens_to_ids
  features   [max_seq_length, line, ids of the real tokens, number of entries in segment 0] of
             tokenlizer_line (mask and segment ids follow from the two counts and are checked to)
  ...        all of it once lower-cased and once cased
"""
import argparse
import json
import os
import random
import sys
import tempfile

SENTENCES = [
    "The quick brown fox, aged 7, jumped over 13 lazy dogs -- twice!",
    "Hello   world\tthis is\ta TAB separated\nline with\r\nodd  spacing.",
    "E-mail me at someone@example.org (or call +1-555-0100) before 5:30pm; thanks...",
    "Crème brûlée, jalapeño, naïve façade, Ångström, Zürich, Łódź, Dvořák, Ğ İstanbul ılık.",
    "ΟΔΥΣΣΕΥΣ ΚΑΙ ΟΙ ΣΥΝΤΡΟΦΟΙ ΤΟΥ. Σ ΑΣ Σα ΑΣ. άέήίόύώ ΐΰ",
    "Съешь ещё этих мягких французских булок, да выпей чаю. ЁЖИК Й",
    "שלום עולם! مرحبا بالعالم، كيف حالك؟ नमस्ते दुनिया। สวัสดีชาวโลก",
    "今天天气很好,我们去公园散步吧。東京タワーは高いです。カタカナとひらがな",
    "한국어 문장도 잘 처리되어야 합니다. 값 닭 꿩",
    "Mixed中文and English混在一起without spaces再加上123数字.",
    "Symbols: $100 ^caret` ~tilde| <tag> {brace} [bracket] =equals= \\backslash/",
    "Quotes “curly” ‘single’ «guillemets» „low“ – en — em … ellipsis • bullet ‰ ¿qué? ¡sí!",
    "Zero\u200bwidth\u200cjoiners\u200dand\ufeffBOM and soft\u00adhyphen and NBSP\u00a0here\u2003em\u2009thin\u3000ideographic.",
    "Line\u2028separator and paragraph\u2029separator and NEL\u0085inside and FF\x0cVT\x0bBEL\x07done.",
    "Combining: a\u0301 e\u0302\u0323 o\u0308\u0304 n\u0303 Å\u030a \u0301leading, Vietnamese: Tiếng Việt đẹp lắm.",
    "Special tokens [CLS] [SEP] [MASK] [UNK] [PAD] in text, and [cls] [Sep] lowercase ones.",
    "A" + "b" * 120 + " short " + "x" * 100 + " " + "y" * 101 + ".",
    "Emoji 😀 and 👩‍👩‍👧 and flags 🇯🇵 stay, math ∑∫√∞ ≈ ≠ ≤, arrows → ⇒, currency € £ ¥ ₹.",
    "ǅ ǈ ǋ ǲ titlecase digraphs, ß ẞ sharp s, ﬁ ﬂ ligatures, ＦＵＬＬＷＩＤＴＨ ｆｏｒｍｓ １２３.",
    "",
    "   ",
    "\u0301\u0302",
    "unaffable unbelievably unaffordable restructuring misunderstandings",
]

BLOCKS = [(0x20, 0x7F), (0xA0, 0x17F), (0x180, 0x24F), (0x2B0, 0x36F), (0x370, 0x3FF), (0x400, 0x4FF),
          (0x530, 0x5FF), (0x600, 0x6FF), (0x900, 0x97F), (0xE00, 0xE7F), (0x10A0, 0x10FF), (0x1100, 0x11FF),
          (0x1E00, 0x1FFF), (0x2000, 0x206F), (0x20A0, 0x20CF), (0x2100, 0x214F), (0x2190, 0x21FF),
          (0x2460, 0x24FF), (0x2C00, 0x2C5F), (0x3000, 0x30FF), (0x3400, 0x3420), (0x4E00, 0x4E80),
          (0xA720, 0xA7FF), (0xAC00, 0xAC80), (0xD7A0, 0xD7FF), (0xE000, 0xE010), (0xF900, 0xF940),
          (0xFB00, 0xFB4F), (0xFE30, 0xFE6F), (0xFF00, 0xFFEF), (0x10400, 0x1044F), (0x1D400, 0x1D440),
          (0x1F600, 0x1F640), (0x20000, 0x20010), (0x2F800, 0x2F810), (0xE0000, 0xE0080), (0x0, 0x1F)]


def random_text(rng):
    n = rng.randint(1, 40)
    out = []
    for _ in range(n):
        if rng.random() < 0.25:
            out.append(" ")
            continue
        lo, hi = rng.choice(BLOCKS)
        cp = rng.randint(lo, hi)
        if 0xD800 <= cp <= 0xDFFF or cp == 0:
            cp = 0x41
        out.append(chr(cp))
    return "".join(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "tokenizer_golden.json"))
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "apps"))
    from pytorch_pretrained_bert.tokenization import BasicTokenizer, BertTokenizer
    import tokenlizer as ref_app

    rng = random.Random(20240607)
    texts = list(SENTENCES) + [random_text(rng) for _ in range(250)]

    # vocabulary: specials, then pieces cut from the words the reference's basic tokenizer sees
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"]
    seen = set(vocab)

    def add(tok):
        if tok and tok not in seen and len(seen) < 6000:
            seen.add(tok)
            vocab.append(tok)

    for lower in (True, False):
        basic = BasicTokenizer(do_lower_case=lower)
        for t in texts:
            for word in basic.tokenize(t):
                r = rng.random()
                if r < 0.15:
                    continue                      # stays out of the vocabulary: [UNK] unless pieces cover it
                if r < 0.5 or len(word) == 1:
                    add(word)
                    continue
                cut = sorted(rng.sample(range(1, len(word)), min(len(word) - 1, rng.randint(1, 3))))
                pieces = [word[i:j] for i, j in zip([0] + cut, cut + [len(word)])]
                add(pieces[0])
                for p in pieces[1:]:
                    add("##" + p)
                if rng.random() < 0.3:
                    for ch in word:
                        add("##" + ch)
    rng.shuffle(vocab)

    result = {"vocab": vocab, "cases": {}}
    with tempfile.TemporaryDirectory() as d:
        vf = os.path.join(d, "vocab.txt")
        with open(vf, "w", encoding="utf-8") as f:
            f.write("\n".join(vocab) + "\n")
        for lower in (True, False):
            tok = BertTokenizer(vf, do_lower_case=lower)
            ref_app.tokenizer = tok
            toks = [[t, tok.convert_tokens_to_ids(tok.tokenize(t))] for t in texts]
            feats = []
            lines = []
            for i in range(0, len(texts) - 1, 2):
                a = texts[i].replace("\t", " ").replace("\n", " ").replace("\r", " ")
                b = texts[i + 1].replace("\t", " ").replace("\n", " ").replace("\r", " ")
                lines.append(a + "\t" + b)
                lines.append(a + "\t")
            for k, line in enumerate(lines):
                for max_seq in ((8, 32, 128) if k % 4 == 0 else (32,)):
                    try:
                        idx, raw, ids, mask, seg = ref_app.tokenlizer_line(max_seq, line, k)
                    except Exception:      # the reference fails on some degenerate lines: not part of the contract
                        continue
                    n = sum(mask)
                    n0 = n - sum(seg)
                    assert mask == [1] * n + [0] * (max_seq - n) and ids[n:] == [0] * (max_seq - n)
                    assert seg == [0] * n0 + [1] * (n - n0) + [0] * (max_seq - n)
                    assert raw == "\t".join(line.replace("\0", "").rstrip().split("\t"))
                    feats.append([max_seq, line, ids[:n], n0])
            result["cases"]["lower" if lower else "cased"] = {"tokenize": toks, "features": feats}
    with open(args.out, "w", encoding="utf-8") as f:
        json.dump(result, f, ensure_ascii=True, separators=(",", ":"))
    print("wrote", args.out, os.path.getsize(args.out), "bytes;", len(vocab), "vocabulary entries;",
          {k: (len(v["tokenize"]), len(v["features"])) for k, v in result["cases"].items()})


if __name__ == "__main__":
    main()
