"""Generates tokenizer fixtures with the Hugging Face `tokenizers` library (needs that Python package; no GPU).

    python tests/golden/make_golden_tokenizer.py

The reference does not carry a tokenizer of its own: rust/crates/quintrit-runtime/src/tokenizer.rs configures the Hugging
Face `tokenizers` crate (0.21, pinned in rust/Cargo.lock, not part of the reference tree). The Python package of the same
library is configured here exactly as tokenizer.rs:82-146 and :215-293 configure the crate - a BPE model over the GGUF token
and merge lists (ignore_merges for the LLaMA 3 kind), a Sequence of Split(regex, Isolated) pre-tokenizers followed by
ByteLevel(add_prefix_space = false, use_regex = false), a ByteLevel decoder, control tokens (token type 3) as special
tokens, user-defined tokens (type 4) as added tokens, decoding with skip_special_tokens and the final replacement of the
byte-level space and line feed characters (tokenizer.rs:158-161) - and its answers are stored:

  tokenizer_vectors.json.gz   a byte-level vocabulary of 1100 entries trained here on seeded synthetic text (Latin with
                              accents, Greek, Cyrillic, CJK, digits, punctuation, emoji), its merges and token types;
                              260 texts; for each of the pre-tokenizer kinds default, gpt2, llama3, qwen2 the ids of every
                              text and the text the ids decode to.

The splitting expressions are quoted from the reference (tokenizer.rs:215-226); they are data of the fixture.
"""
import gzip
import json
import os
import random

from tokenizers import AddedToken, Regex, Tokenizer, decoders, models, pre_tokenizers, trainers

HERE = os.path.dirname(os.path.abspath(__file__))

GPT2 = r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"
LLAMA3 = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
QWEN2 = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
DEFAULT = [r"[\p{P}\$\+<=>\^~\|]+", r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)", r"\p{N}+", r"[0-9][0-9][0-9]"]
KINDS = {"default": DEFAULT, "gpt2": [GPT2], "llama3": [LLAMA3], "qwen2": [QWEN2]}
PRE_VALUE = {"default": None, "gpt2": "gpt2", "llama3": "llama3", "qwen2": "qwen2"}  # tokenizer.ggml.pre of a file of that kind

WORDS = ("the of and to in is that it was for on are as with his they at be this from have or by one had not but what all were when we there can an your "
         "which their said if do will each about how up out them then she many some so these would other into has more her two like him see time could no "
         "make than first been its who now people my made over did down only way find use may water long little very after words called just where most "
         "über straße naïve café señor niño façade crème brûlée São Paulo Ångström "
         "λόγος και το είναι πολύ καλημέρα σας привет мир это очень хорошо спасибо большое "
         "東京 日本語 こんにちは 世界 你好 谢谢 再见 한국어 감사합니다").split()
PUNCT = [".", ",", "!", "?", ";", ":", "...", " - ", " — ", "(", ")", "\"", "'", "«", "»", "¿", "¡", "、", "。", "$", "+", "<", "=", ">", "^", "~", "|", "%", "#", "@", "&", "*", "/"]
EMOJI = ["🙂", "🚀", "☃", "❤️", "👍🏽", "é", "é", "①", "½", "²"]
SPACES = [" ", "  ", "   ", "\n", "\n\n", " \n", "\t", "\r\n", " \n ", " ", "　"]


def sentence(rng: random.Random) -> str:
    out = []
    for _ in range(rng.randint(1, 14)):
        r = rng.random()
        if r < 0.62:
            w = rng.choice(WORDS)
            if rng.random() < 0.15:
                w = w.capitalize()
            if rng.random() < 0.05:
                w = w.upper()
            if rng.random() < 0.08:
                w += rng.choice(["'s", "'t", "'re", "'ve", "'m", "'ll", "'d", "'S", "'LL", "'x"])
            out.append(w)
        elif r < 0.74:
            out.append(str(rng.randint(0, 10 ** rng.randint(1, 8))))
        elif r < 0.86:
            out.append(rng.choice(PUNCT) * rng.randint(1, 3))
        elif r < 0.92:
            out.append(rng.choice(EMOJI))
        else:
            out.append("")
        out.append(rng.choice(SPACES) if rng.random() < 0.85 else "")
    return "".join(out)


HANDMADE = [
    "", " ", "  ", "\n", "a", "Hello", "Hello there", "the cat sat on the mat", " the", "the", "I'm sure they'll say it's what we'd've done, DON'T you?",
    "1234567 12 3.14159 1,000,000 2024-11-25", "x=1+2<3>>4^5~6|7$8", "tabs\tand\nnewlines\r\nand   runs   of   spaces   ", "trailing space ", " leading",
    "multiple\n\n\nblank lines\n", "   \n   indented", "end with newline\n", "ünïcödé çhârs — and “quotes” … done", "日本語のテキストと English mixed 123",
    "emoji 🙂🚀 at ☃☃ end", "<|endoftext|>", "a<|endoftext|>b", "say <think>hmm</think> ok", "<s>not special</s>", "<|user|>\nHello there\n<|assistant|>\n",
    "### System:\nbe brief\n\n### User:\nhi\n\n### Assistant:\n", "CamelCaseWordsAndSHOUTING", "é combining and  nbsp　ideographic", "١٢٣ ४५६ ①②③ ½",
    "'s 't 're 've 'm 'll 'd", "'S 'T 'RE", "don't won't can't", "http://example.com/path?q=1&r=2#frag", "a.b,c;d:e!f?g", "((nested)) [brackets] {braces}",
    "snake_case and kebab-case", "100%", "$100.00", "C++ > C#", " line sep para sep", "\x00nul and \x7f del", "� replacement",
]


def build(tokens, merges, types, kind):
    vocab = {}
    for i, t in enumerate(tokens):
        key = t.replace("\n", "Ċ").replace("\r", "č").replace("\t", "ċ")
        if key != t:
            vocab.setdefault(t, i)
        vocab[key] = i
    pairs = [tuple(m.split()) for m in merges if len(m.split()) == 2]
    tok = Tokenizer(models.BPE(vocab=vocab, merges=pairs, ignore_merges=(kind == "llama3")))
    parts = [pre_tokenizers.Split(Regex(r), behavior="isolated", invert=False) for r in KINDS[kind]]
    parts.append(pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False))
    tok.pre_tokenizer = pre_tokenizers.Sequence(parts)
    tok.decoder = decoders.ByteLevel()
    tok.add_special_tokens([AddedToken(t, special=True) for t, ty in zip(tokens, types) if ty == 3 and t])
    tok.add_tokens([AddedToken(t, special=False) for t, ty in zip(tokens, types) if ty == 4 and t])
    return tok


def main() -> None:
    rng = random.Random(20240611)
    corpus = [sentence(rng) for _ in range(6000)]
    trainer_tok = Tokenizer(models.BPE())
    trainer_tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(GPT2), behavior="isolated"), pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    trainer = trainers.BpeTrainer(vocab_size=1092, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    trainer_tok.train_from_iterator(corpus, trainer)
    model = json.loads(trainer_tok.to_str())["model"]
    tokens = [t for t, _ in sorted(model["vocab"].items(), key=lambda kv: kv[1])]
    merges = [m if isinstance(m, str) else " ".join(m) for m in model["merges"]]
    types = [1] * len(tokens)
    for text, ty in (("<s>", 3), ("</s>", 3), ("<|endoftext|>", 3), ("<|user|>", 3), ("<|assistant|>", 3), ("<think>", 4), ("</think>", 4), ("\n", 4)):
        tokens.append(text)
        types.append(ty)
    bos, eos = tokens.index("<s>"), tokens.index("</s>")
    texts = HANDMADE + [sentence(rng) for _ in range(260 - len(HANDMADE))]
    out = {"tokens": tokens, "merges": merges, "types": types, "bos": bos, "eos": eos, "texts": texts, "pre": PRE_VALUE, "kinds": {}}
    for kind in KINDS:
        tok = build(tokens, merges, types, kind)
        ids = [tok.encode(t, add_special_tokens=False).ids for t in texts]
        dec = [tok.decode(i, skip_special_tokens=True).replace("Ġ", " ").replace("Ċ", "\n") for i in ids]
        out["kinds"][kind] = {"ids": ids, "decoded": dec}
        print(kind, sum(len(i) for i in ids), "ids;", sum(d == t for d, t in zip(dec, texts)), "of", len(texts), "texts decode to themselves")
    with gzip.open(os.path.join(HERE, "tokenizer_vectors.json.gz"), "wt", encoding="utf-8") as f:
        json.dump(out, f, ensure_ascii=False)
    print(len(tokens), "tokens,", len(merges), "merges")


if __name__ == "__main__":
    main()
