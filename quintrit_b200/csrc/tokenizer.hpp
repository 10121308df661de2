// Byte-level BPE tokenizer built from GGUF metadata, host side of the text entry points of the runtime ABI.
//
// Plays the part of rust/crates/quintrit-runtime/src/tokenizer.rs, which configures the Hugging Face `tokenizers` crate
// (not part of the reference tree) as: a BPE model over `tokenizer.ggml.tokens` / `tokenizer.ggml.merges` (tokenizer.rs:
// 96-124), a pre-tokenizer chosen by `tokenizer.ggml.pre` that splits the text by regular expressions and then maps every
// byte to a printable character (tokenizer.rs:215-293), control tokens (`tokenizer.ggml.token_type` 3) as special tokens that
// match as a whole and are skipped when decoding, user-defined tokens (type 4) that match as a whole and decode to their
// text (tokenizer.rs:126-146), and the streaming decoder that never hands out half a UTF-8 character (tokenizer.rs:295-337).
// This file restates that behaviour in plain C++: the published byte-level BPE algorithm (bytes -> 256 printable characters,
// lowest-rank merge first), hand-written matchers for the splitting expressions, leftmost-longest matching of added tokens.
//
// The expressions use the Unicode classes \p{L}, \p{N}, \p{P} and \s: the general categories come from generated tables
// (unicode_tables.hpp), \s is the White_Space property. The Tekken, Qwen3.5 and Falcon-E pre-tokenizers are not built.
#pragma once
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "unicode_tables.hpp"

namespace qtb {

// ---- UTF-8 and character classes ---------------------------------------------------------------------------------------
inline void utf8_append(std::string& out, uint32_t cp) {
    if (cp < 0x80) {
        out.push_back(static_cast<char>(cp));
    } else if (cp < 0x800) {
        out.push_back(static_cast<char>(0xC0 | (cp >> 6)));
        out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
        out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
        out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
        out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
        out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
        out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
        out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
        out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
}

// Length of the well-formed UTF-8 sequence at s[i] (1..4), 0 if the bytes there are not one (truncated, overlong, surrogate).
inline size_t utf8_sequence(const unsigned char* s, size_t n, size_t i, uint32_t* cp = nullptr) {
    const unsigned char b = s[i];
    size_t len = 0;
    uint32_t c = 0;
    if (b < 0x80) {
        len = 1, c = b;
    } else if (b >= 0xC2 && b <= 0xDF) {
        len = 2, c = b & 0x1F;
    } else if (b >= 0xE0 && b <= 0xEF) {
        len = 3, c = b & 0x0F;
    } else if (b >= 0xF0 && b <= 0xF4) {
        len = 4, c = b & 0x07;
    } else {
        return 0;
    }
    if (i + len > n) return 0;
    for (size_t k = 1; k < len; ++k) {
        if ((s[i + k] & 0xC0) != 0x80) return 0;
        c = (c << 6) | (s[i + k] & 0x3F);
    }
    if ((len == 3 && (c < 0x800 || (c >= 0xD800 && c <= 0xDFFF))) || (len == 4 && (c < 0x10000 || c > 0x10FFFF))) return 0;
    if (cp) *cp = c;
    return len;
}

inline bool utf8_valid(const std::string& s) {
    const unsigned char* p = reinterpret_cast<const unsigned char*>(s.data());
    for (size_t i = 0; i < s.size();) {
        const size_t l = utf8_sequence(p, s.size(), i);
        if (l == 0) return false;
        i += l;
    }
    return true;
}

// Bytes as text: every maximal ill-formed part becomes U+FFFD (what String::from_utf8_lossy does).
inline std::string utf8_lossy(const std::string& s) {
    const unsigned char* p = reinterpret_cast<const unsigned char*>(s.data());
    std::string out;
    out.reserve(s.size());
    for (size_t i = 0; i < s.size();) {
        const size_t l = utf8_sequence(p, s.size(), i);
        if (l != 0) {
            out.append(s, i, l);
            i += l;
            continue;
        }
        // skip the lead byte and the continuation bytes that could have belonged to it
        const unsigned char b = p[i];
        size_t want = b >= 0xF0 ? 3 : (b >= 0xE0 ? 2 : (b >= 0xC2 ? 1 : 0));
        ++i;
        while (want > 0 && i < s.size() && (p[i] & 0xC0) == 0x80 && utf8_sequence(p, s.size(), i) == 0) {
            // a continuation byte that is acceptable as the next byte of the truncated sequence
            ++i;
            --want;
            if (i < s.size() && (p[i] & 0xC0) != 0x80) break;
        }
        out += "\xEF\xBF\xBD";
    }
    return out;
}

inline std::vector<uint32_t> utf8_decode(const std::string& s) {
    std::vector<uint32_t> cps;
    const unsigned char* p = reinterpret_cast<const unsigned char*>(s.data());
    for (size_t i = 0; i < s.size();) {
        uint32_t cp = 0xFFFD;
        const size_t l = utf8_sequence(p, s.size(), i, &cp);
        cps.push_back(l ? cp : 0xFFFD);
        i += l ? l : 1;
    }
    return cps;
}

inline bool cp_in(uint32_t c, uint32_t lo, uint32_t hi) { return c >= lo && c <= hi; }
inline bool cp_space(uint32_t c) {
    return c == ' ' || cp_in(c, 9, 13) || c == 0x85 || c == 0xA0 || c == 0x1680 || cp_in(c, 0x2000, 0x200A) || c == 0x2028 || c == 0x2029 ||
           c == 0x202F || c == 0x205F || c == 0x3000;
}
template <size_t N>
inline bool cp_in_table(const CpRange (&table)[N], uint32_t c) {
    size_t lo = 0, hi = N;
    while (lo < hi) {
        const size_t mid = (lo + hi) / 2;
        if (c > table[mid].last) lo = mid + 1;
        else hi = mid;
    }
    return lo < N && c >= table[lo].first;
}
inline bool cp_number(uint32_t c) { return c < 0x80 ? cp_in(c, '0', '9') : cp_in_table(kUnicodeNumber, c); }  // \p{N}
inline bool cp_punct(uint32_t c) { return cp_in_table(kUnicodePunct, c); }                                     // \p{P}
inline bool cp_letter(uint32_t c) {                                                                           // \p{L}
    if (c < 0x80) return cp_in(c, 'a', 'z') || cp_in(c, 'A', 'Z');
    return cp_in_table(kUnicodeLetter, c);
}

// ---- the splitting expressions --------------------------------------------------------------------------------------------
enum class PreKind { Gpt2, Default, Llama3, Qwen2 };

struct PreSplitter {
    using Text = std::vector<uint32_t>;

    // 's 't 're 've 'm 'll 'd
    static size_t contraction(const Text& t, size_t i, bool fold) {
        if (t[i] != '\'' || i + 1 >= t.size()) return 0;
        auto low = [&](uint32_t c) { return fold && cp_in(c, 'A', 'Z') ? c + 32 : c; };
        const uint32_t a = low(t[i + 1]), b = i + 2 < t.size() ? low(t[i + 2]) : 0;
        if (a == 's' || a == 't' || a == 'm' || a == 'd') return 2;
        if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) return 3;
        return 0;
    }
    template <typename Pred>
    static size_t run(const Text& t, size_t i, Pred pred) {
        size_t n = 0;
        while (i + n < t.size() && pred(t[i + n])) ++n;
        return n;
    }
    static bool other(uint32_t c) { return !cp_space(c) && !cp_letter(c) && !cp_number(c); }

    // Length of the match of the GPT-2 expression at i (tokenizer.rs:215; `with_trailing_space` adds the final \s+), 0 if none.
    static size_t gpt2(const Text& t, size_t i, bool with_trailing_space) {
        if (size_t n = contraction(t, i, false)) return n;
        const size_t sp = t[i] == ' ' ? 1 : 0;
        if (i + sp < t.size()) {
            if (size_t n = run(t, i + sp, cp_letter)) return sp + n;
            if (size_t n = run(t, i + sp, cp_number)) return sp + n;
            if (size_t n = run(t, i + sp, other)) return sp + n;
        }
        if (size_t n = run(t, i, cp_space)) {
            if (i + n == t.size()) return n;  // \s+(?!\S) at the end of the text
            if (n > 1) return n - 1;          // ... or leaving the last white space to the next piece
            return with_trailing_space ? 1 : 0;
        }
        return 0;
    }
    // The LLaMA 3 expression (tokenizer.rs:216); `digits` is 3 for it and 1 for the Qwen2 one (:217).
    static size_t llama3(const Text& t, size_t i, size_t digits) {
        if (size_t n = contraction(t, i, true)) return n;
        {
            const uint32_t c = t[i];
            const size_t lead = (c != '\r' && c != '\n' && !cp_letter(c) && !cp_number(c)) ? 1 : 0;
            if (lead && i + 1 < t.size()) {
                if (size_t n = run(t, i + 1, cp_letter)) return 1 + n;
            }
            if (size_t n = run(t, i, cp_letter)) return n;
        }
        if (size_t n = run(t, i, cp_number)) return std::min(n, digits);
        {
            const size_t sp = t[i] == ' ' ? 1 : 0;
            if (i + sp < t.size()) {
                if (size_t n = run(t, i + sp, other)) {
                    const size_t nl = run(t, i + sp + n, [](uint32_t c) { return c == '\r' || c == '\n'; });
                    return sp + n + nl;
                }
            }
        }
        if (size_t n = run(t, i, cp_space)) {
            size_t last_nl = 0;  // \s*[\r\n]+: up to the last line break of the white space
            for (size_t k = 0; k < n; ++k)
                if (t[i + k] == '\r' || t[i + k] == '\n') last_nl = k + 1;
            if (last_nl) return last_nl;
            if (i + n == t.size()) return n;
            if (n > 1) return n - 1;
            return 1;
        }
        return 0;
    }

    // Splits `t` at the matches of `match` (a piece per match, a piece per gap: SplitDelimiterBehavior::Isolated).
    template <typename Match>
    static void split(const Text& t, Match match, std::vector<Text>& out) {
        size_t gap = 0, i = 0;
        while (i < t.size()) {
            const size_t n = match(t, i);
            if (n == 0) {
                ++i;
                continue;
            }
            if (i > gap) out.emplace_back(t.begin() + gap, t.begin() + i);
            out.emplace_back(t.begin() + i, t.begin() + i + n);
            i += n;
            gap = i;
        }
        if (t.size() > gap) out.emplace_back(t.begin() + gap, t.end());
    }

    static std::vector<Text> apply(PreKind kind, const Text& text) {
        std::vector<Text> pieces;
        switch (kind) {
            case PreKind::Gpt2: split(text, [](const Text& t, size_t i) { return gpt2(t, i, true); }, pieces); break;
            case PreKind::Llama3: split(text, [](const Text& t, size_t i) { return llama3(t, i, 3); }, pieces); break;
            case PreKind::Qwen2: split(text, [](const Text& t, size_t i) { return llama3(t, i, 1); }, pieces); break;
            case PreKind::Default: {
                // four expressions one after the other (tokenizer.rs:221-226): punctuation runs, the GPT-2 expression without
                // its final \s+, digit runs, groups of three ASCII digits
                auto stage = [](const std::vector<Text>& in, auto match) {
                    std::vector<Text> out;
                    for (const Text& p : in) split(p, match, out);
                    return out;
                };
                std::vector<Text> cur{text};
                cur = stage(cur, [](const Text& t, size_t i) {
                    return run(t, i, [](uint32_t c) { return cp_punct(c) || c == '$' || c == '+' || c == '<' || c == '=' || c == '>' || c == '^' || c == '~' || c == '|'; });
                });
                cur = stage(cur, [](const Text& t, size_t i) { return gpt2(t, i, false); });
                cur = stage(cur, [](const Text& t, size_t i) { return run(t, i, cp_number); });
                cur = stage(cur, [](const Text& t, size_t i) {
                    return i + 2 < t.size() && cp_in(t[i], '0', '9') && cp_in(t[i + 1], '0', '9') && cp_in(t[i + 2], '0', '9') ? size_t(3) : size_t(0);
                });
                pieces = std::move(cur);
                break;
            }
        }
        return pieces;
    }
};

// ---- the tokenizer --------------------------------------------------------------------------------------------------------
class BpeTokenizer {
  public:
    static constexpr int kTypeControl = 3, kTypeUserDefined = 4;  // tokenizer.rs:8-14

    // Returns an empty string, or why the tokenizer cannot be built. `pre` is tokenizer.ggml.pre (nullptr = absent).
    std::string build(const std::vector<std::string>& tokens, const std::vector<std::string>& merges, const std::vector<int64_t>& types, const char* pre,
                      int64_t bos, int64_t eos) {
        if (pre == nullptr || std::strcmp(pre, "default") == 0) {
            kind_ = PreKind::Default;
        } else {
            const std::string p(pre);
            static const char* const l3[] = {"llama3", "llama-v3", "llama-bpe", "falcon3", "falcon-h1", "midm-2.0", "jina-v5-nano", "lfm2"};
            static const char* const q2[] = {"qwen2", "deepseek-r1-qwen", "kormo", "f2llmv2"};
            static const char* const g2[] = {"gpt-2", "phi-2", "gpt2"};
            bool found = false;
            for (const char* n : l3) found |= p == n;
            if (found) {
                kind_ = PreKind::Llama3;
            } else {
                for (const char* n : q2) found |= p == n;
                if (found) {
                    kind_ = PreKind::Qwen2;
                } else {
                    for (const char* n : g2) found |= p == n;
                    if (!found) return "pre-tokenizer type '" + p + "' (tokenizer.ggml.pre) is not supported by this library";
                    kind_ = PreKind::Gpt2;
                }
            }
        }
        ignore_merges_ = kind_ == PreKind::Llama3;  // tokenizer.rs:246-248
        bos_ = bos, eos_ = eos;
        // bytes <-> printable characters (the published GPT-2 table: printable Latin-1 keeps its code, the rest moves to 256 + n)
        {
            int n = 0;
            for (int b = 0; b < 256; ++b) {
                const bool keep = (b >= '!' && b <= '~') || (b >= 0xA1 && b <= 0xAC) || (b >= 0xAE && b <= 0xFF);
                byte_to_cp_[b] = keep ? static_cast<uint32_t>(b) : static_cast<uint32_t>(256 + n++);
                cp_to_byte_[byte_to_cp_[b]] = b;
            }
        }
        tokens_ = tokens;
        vocab_.clear();
        vocab_.reserve(tokens.size() * 2);
        for (size_t i = 0; i < tokens.size(); ++i) {
            // tokenizer.rs:99-107: raw control characters inside a stored token stand for their byte-level characters
            std::string key;
            for (char ch : tokens[i]) {
                if (ch == '\n') key += "\xC4\x8A";       // U+010A
                else if (ch == '\r') key += "\xC4\x8D";  // U+010D
                else if (ch == '\t') key += "\xC4\x8B";  // U+010B
                else key.push_back(ch);
            }
            if (key != tokens[i]) vocab_.emplace(tokens[i], static_cast<uint32_t>(i));
            vocab_[key] = static_cast<uint32_t>(i);
        }
        ranks_.clear();
        ranks_.reserve(merges.size() * 2);
        uint32_t rank = 0;
        for (const std::string& m : merges) {
            // two parts separated by white space (tokenizer.rs:112-117); other lines are ignored
            std::vector<std::string> parts;
            size_t i = 0;
            while (i < m.size()) {
                while (i < m.size() && (m[i] == ' ' || m[i] == '\t' || m[i] == '\n' || m[i] == '\r')) ++i;
                size_t j = i;
                while (j < m.size() && !(m[j] == ' ' || m[j] == '\t' || m[j] == '\n' || m[j] == '\r')) ++j;
                if (j > i) parts.emplace_back(m, i, j - i);
                i = j;
            }
            if (parts.size() == 2) ranks_.emplace(parts[0] + '\x01' + parts[1], rank++);
        }
        added_.clear();
        special_.assign(tokens.size(), 0);
        if (!types.empty()) {
            for (size_t i = 0; i < tokens.size() && i < types.size(); ++i) {
                if (tokens[i].empty() || (types[i] != kTypeControl && types[i] != kTypeUserDefined)) continue;
                auto it = vocab_.find(tokens[i]);  // an added token whose text is in the vocabulary keeps that id
                const uint32_t id = it != vocab_.end() ? it->second : static_cast<uint32_t>(i);
                added_.push_back({tokens[i], id, types[i] == kTypeControl});
                if (id < special_.size()) special_[id] = types[i] == kTypeControl ? 1 : 2;
            }
            std::sort(added_.begin(), added_.end(), [](const Added& a, const Added& b) { return a.text.size() > b.text.size(); });
        }
        return std::string();
    }

    size_t vocab_size() const { return tokens_.size(); }
    int64_t bos() const { return bos_; }
    int64_t eos() const { return eos_; }

    std::vector<uint32_t> encode(const std::string& text) const {
        std::vector<uint32_t> ids;
        // split at added tokens first: leftmost match, the longest of those that start there
        size_t start = 0, i = 0;
        while (i < text.size()) {
            const Added* hit = nullptr;
            if (!added_.empty())
                for (const Added& a : added_)  // sorted by length, longest first
                    if (text.compare(i, a.text.size(), a.text) == 0) {
                        hit = &a;
                        break;
                    }
            if (hit == nullptr) {
                ++i;
                continue;
            }
            if (i > start) encode_plain(text.substr(start, i - start), ids);
            ids.push_back(hit->id);
            i += hit->text.size();
            start = i;
        }
        if (text.size() > start) encode_plain(text.substr(start), ids);
        return ids;
    }

    // The bytes the tokens stand for; control tokens are skipped, user-defined tokens give their text (tokenizer.rs:157-160).
    std::string decode_bytes(const uint32_t* ids, size_t n) const {
        std::string out;
        for (size_t k = 0; k < n; ++k) {
            const uint32_t id = ids[k];
            if (id >= tokens_.size() || special_[id] == 1) continue;
            const std::string& tok = tokens_[id];
            if (special_[id] == 2) {  // its text, with the byte-level space and line feed read as such
                for (uint32_t cp : utf8_decode(tok)) {
                    if (cp == 0x120) out.push_back(' ');
                    else if (cp == 0x10A) out.push_back('\n');
                    else utf8_append(out, cp);
                }
                continue;
            }
            for (uint32_t cp : utf8_decode(tok)) {
                auto it = cp_to_byte_.find(cp);
                if (it != cp_to_byte_.end()) out.push_back(static_cast<char>(it->second));
                else utf8_append(out, cp);
            }
        }
        return out;
    }
    std::string decode(const uint32_t* ids, size_t n) const { return utf8_lossy(decode_bytes(ids, n)); }

  private:
    struct Added {
        std::string text;
        uint32_t id;
        bool special;
    };

    void encode_plain(const std::string& text, std::vector<uint32_t>& ids) const {
        const std::vector<uint32_t> cps = utf8_decode(text);
        for (const auto& piece : PreSplitter::apply(kind_, cps)) {
            // byte level: the UTF-8 bytes of the piece as printable characters
            std::string bytes;
            for (uint32_t cp : piece) utf8_append(bytes, cp);
            std::vector<std::string> sym;
            std::string whole;
            for (unsigned char b : bytes) {
                std::string ch;
                utf8_append(ch, byte_to_cp_[b]);
                whole += ch;
                sym.push_back(std::move(ch));
            }
            if (ignore_merges_) {
                auto it = vocab_.find(whole);
                if (it != vocab_.end()) {
                    ids.push_back(it->second);
                    continue;
                }
            }
            // merge the neighbouring pair of lowest rank until none is left
            while (sym.size() > 1) {
                uint32_t best = UINT32_MAX;
                size_t at = 0;
                for (size_t k = 0; k + 1 < sym.size(); ++k) {
                    auto it = ranks_.find(sym[k] + '\x01' + sym[k + 1]);
                    if (it != ranks_.end() && it->second < best) best = it->second, at = k;
                }
                if (best == UINT32_MAX) break;
                sym[at] += sym[at + 1];
                sym.erase(sym.begin() + static_cast<long>(at) + 1);
            }
            for (const std::string& s : sym) {
                auto it = vocab_.find(s);
                if (it != vocab_.end()) ids.push_back(it->second);  // a symbol outside the vocabulary has no id (no unknown token is configured)
            }
        }
    }

    PreKind kind_ = PreKind::Default;
    bool ignore_merges_ = false;
    int64_t bos_ = -1, eos_ = -1;
    uint32_t byte_to_cp_[256] = {};
    std::unordered_map<uint32_t, int> cp_to_byte_;
    std::vector<std::string> tokens_;
    std::unordered_map<std::string, uint32_t> vocab_;
    std::unordered_map<std::string, uint32_t> ranks_;
    std::vector<Added> added_;
    std::vector<unsigned char> special_;  // 0 = ordinary, 1 = control (special), 2 = user-defined
};

// Token ids to text, piece by piece, never ending inside a UTF-8 character (tokenizer.rs:295-337): the pending tokens are
// decoded together with the window already handed out, and text that ends in an incomplete character is held back.
class StreamDecoder {
  public:
    std::string push(const BpeTokenizer& tok, uint32_t id) {
        ids_.push_back(id);
        const std::string prefix = tok.decode(ids_.data() + prefix_, read_ - prefix_);
        const std::string all = tok.decode(ids_.data() + prefix_, ids_.size() - prefix_);
        const bool ends_bad = all.size() >= 3 && all.compare(all.size() - 3, 3, "\xEF\xBF\xBD") == 0;
        if (all.size() > prefix.size() && !ends_bad) {
            prefix_ = read_;
            read_ = ids_.size();
            return all.substr(prefix.size());
        }
        return std::string();
    }
    std::string finish(const BpeTokenizer& tok) {
        const std::string prefix = tok.decode(ids_.data() + prefix_, read_ - prefix_);
        const std::string all = tok.decode(ids_.data() + prefix_, ids_.size() - prefix_);
        prefix_ = read_ = ids_.size();
        return all.size() > prefix.size() ? all.substr(prefix.size()) : std::string();
    }

  private:
    std::vector<uint32_t> ids_;
    size_t prefix_ = 0, read_ = 0;
};

}  // namespace qtb
