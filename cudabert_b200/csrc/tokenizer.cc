// BERT tokenisation as native host code: basic tokenisation (text clean-up, CJK spacing,
// lower-casing + accent stripping, punctuation splitting) followed by greedy longest-match-first
// WordPiece, and the packing of one or two texts into ids / mask / segment ids of a fixed length.
// It restates, for the engine's reader stage, what the reference's sample application does in
// Python (apps/tokenlizer.py:45-147 on top of apps/pytorch_pretrained_bert/tokenization.py:51-372)
// and has to produce the same ids; character classes and case/accent folding come from tables
// generated from Python's own Unicode database (unicode_tables.h, make_unicode_tables.py).
//
// Known differences from the Python code, all outside ordinary text: invalid UTF-8 bytes become
// U+FFFD and are then dropped like any U+FFFD (Python refuses to read such a file); combining marks
// that survive accent stripping (categories Mc, Me) keep their input order (NFD may reorder them);
// in the final-sigma rule of lower-casing, case-ignorable characters between sigma and its
// neighbours are not skipped.
#include "../../include/cudabert.h"
#include "unicode_tables.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

typedef std::vector<uint32_t> U32;

bool in_ranges(const uint32_t (*table)[2], int count, uint32_t cp) {
  int lo = 0, hi = count - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) >> 1;
    if (cp < table[mid][0]) hi = mid - 1;
    else if (cp > table[mid][1]) lo = mid + 1;
    else return true;
  }
  return false;
}

// tokenization.py:334-372
bool is_whitespace(uint32_t cp) {
  return cp == ' ' || cp == '\t' || cp == '\n' || cp == '\r' || (cp >= 0x80 && in_ranges(kSpaceZs, kSpaceZsCount, cp));
}
bool is_control(uint32_t cp) {
  if (cp < 0x80) return (cp < 32 && cp != '\t' && cp != '\n' && cp != '\r') || cp == 127;
  return in_ranges(kControl, kControlCount, cp);
}
bool is_punctuation(uint32_t cp) {
  if ((cp >= 33 && cp <= 47) || (cp >= 58 && cp <= 64) || (cp >= 91 && cp <= 96) || (cp >= 123 && cp <= 126)) return true;
  return cp >= 0x80 && in_ranges(kPunct, kPunctCount, cp);
}
// what str.split() splits on
bool is_py_space(uint32_t cp) {
  if (cp < 0x80) return cp == ' ' || (cp >= 9 && cp <= 13) || (cp >= 28 && cp <= 31);
  return in_ranges(kPySpace, kPySpaceCount, cp);
}
// tokenization.py:239-255
bool is_cjk(uint32_t cp) {
  return (cp >= 0x4E00 && cp <= 0x9FFF) || (cp >= 0x3400 && cp <= 0x4DBF) || (cp >= 0x20000 && cp <= 0x2A6DF) ||
         (cp >= 0x2A700 && cp <= 0x2B73F) || (cp >= 0x2B740 && cp <= 0x2B81F) || (cp >= 0x2B820 && cp <= 0x2CEAF) ||
         (cp >= 0xF900 && cp <= 0xFAFF) || (cp >= 0x2F800 && cp <= 0x2FA1F);
}

void decode_utf8(const char* s, U32* out) {
  const unsigned char* p = reinterpret_cast<const unsigned char*>(s);
  while (*p) {
    uint32_t cp = 0xFFFD;
    int extra = 0;
    const unsigned char c = *p++;
    if (c < 0x80) { out->push_back(c); continue; }
    if (c >= 0xC2 && c <= 0xDF) { cp = c & 0x1F; extra = 1; }
    else if (c >= 0xE0 && c <= 0xEF) { cp = c & 0x0F; extra = 2; }
    else if (c >= 0xF0 && c <= 0xF4) { cp = c & 0x07; extra = 3; }
    else { out->push_back(0xFFFD); continue; }
    bool ok = true;
    for (int i = 0; i < extra; ++i) {
      if ((p[i] & 0xC0) != 0x80) { ok = false; break; }  // also stops at the terminating 0
      cp = (cp << 6) | (p[i] & 0x3F);
    }
    if (!ok || (extra == 2 && (cp < 0x800 || (cp >= 0xD800 && cp <= 0xDFFF))) ||
        (extra == 3 && (cp < 0x10000 || cp > 0x10FFFF))) {
      out->push_back(0xFFFD);
      continue;
    }
    p += extra;
    out->push_back(cp);
  }
}

void append_utf8(uint32_t cp, std::string* out) {
  if (cp < 0x80) out->push_back(static_cast<char>(cp));
  else if (cp < 0x800) {
    out->push_back(static_cast<char>(0xC0 | (cp >> 6)));
    out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
  } else if (cp < 0x10000) {
    out->push_back(static_cast<char>(0xE0 | (cp >> 12)));
    out->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
    out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
  } else {
    out->push_back(static_cast<char>(0xF0 | (cp >> 18)));
    out->push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
    out->push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
    out->push_back(static_cast<char>(0x80 | (cp & 0x3F)));
  }
}

// strip_accents(lower(c)) appended to `out` (tokenization.py:187-201)
void fold_append(uint32_t cp, U32* out) {
  if (cp < 0x80) {
    out->push_back((cp >= 'A' && cp <= 'Z') ? cp + 32 : cp);
    return;
  }
  if (cp >= 0xAC00 && cp <= 0xD7A3) {  // Hangul syllable: canonical decomposition into jamo
    const uint32_t s = cp - 0xAC00;
    out->push_back(0x1100 + s / 588);
    out->push_back(0x1161 + (s % 588) / 28);
    if (s % 28) out->push_back(0x11A7 + s % 28);
    return;
  }
  const uint32_t* end = kFoldKey + kFoldCount;
  const uint32_t* it = std::lower_bound(kFoldKey, end, cp);
  if (it == end || *it != cp) {
    out->push_back(cp);
    return;
  }
  const size_t i = static_cast<size_t>(it - kFoldKey);
  for (int j = 0; j < kFoldLen[i]; ++j) out->push_back(kFoldData[kFoldOff[i] + j]);
}

struct Tokenizer {
  std::unordered_map<std::string, int> vocab;
  bool lower = true;
  int unk = -1, cls = -1, sep = -1;
  std::vector<U32> never_split;  // [UNK] [SEP] [PAD] [CLS] [MASK]
  static constexpr size_t MAX_WORD_CHARS = 100;
  size_t max_piece_chars = 1;  // characters of the longest vocabulary entry, its "##" not counted

  bool is_never_split(const U32& tok) const {
    for (const U32& n : never_split)
      if (n == tok) return true;
    return false;
  }

  // greedy longest-match-first (tokenization.py:278-331)
  void wordpiece(const U32& word, std::vector<int>* ids) const {
    if (word.size() > MAX_WORD_CHARS) {
      ids->push_back(unk);
      return;
    }
    std::string bytes;
    std::vector<size_t> off(word.size() + 1);
    for (size_t i = 0; i < word.size(); ++i) {
      off[i] = bytes.size();
      append_utf8(word[i], &bytes);
    }
    off[word.size()] = bytes.size();
    const size_t first = ids->size();
    std::string key;
    size_t start = 0;
    while (start < word.size()) {
      // no vocabulary entry is longer than max_piece_chars, so longer candidates need no lookup
      size_t end = std::min(word.size(), start + max_piece_chars);
      int found = -1;
      const size_t prefix = start > 0 ? 2 : 0;
      key.assign(start > 0 ? "##" : "");
      key.append(bytes, off[start], off[end] - off[start]);
      for (; start < end; --end) {
        key.resize(prefix + off[end] - off[start]);  // the candidate shrinks from its end
        const auto it = vocab.find(key);
        if (it != vocab.end()) {
          found = it->second;
          break;
        }
      }
      if (found < 0) {  // the whole word becomes the unknown token
        ids->resize(first);
        ids->push_back(unk);
        return;
      }
      ids->push_back(found);
      start = end;
    }
  }

  // split one whitespace-delimited token on punctuation and emit the pieces' word pieces
  void emit_token(const U32& tok, std::vector<int>* ids) const {
    if (is_never_split(tok)) {
      wordpiece(tok, ids);
      return;
    }
    U32 folded;
    const U32* text = &tok;
    if (lower) {
      for (size_t i = 0; i < tok.size(); ++i) {
        if (tok[i] == 0x3A3) {  // capital sigma: final form after a cased letter at the end of a word
          const bool before = i > 0 && in_ranges(kCased, kCasedCount, tok[i - 1]);
          const bool after = i + 1 < tok.size() && in_ranges(kCased, kCasedCount, tok[i + 1]);
          folded.push_back(before && !after ? 0x3C2 : 0x3C3);
        } else {
          fold_append(tok[i], &folded);
        }
      }
      text = &folded;
    }
    U32 word;
    auto flush = [&]() {
      if (!word.empty()) wordpiece(word, ids);
      word.clear();
    };
    for (uint32_t cp : *text) {
      if (is_punctuation(cp)) {
        flush();
        word.push_back(cp);
        flush();
      } else if (is_py_space(cp)) {  // the pieces are joined and split on whitespace once more
        flush();
      } else {
        word.push_back(cp);
      }
    }
    flush();
  }

  // BasicTokenizer.tokenize + WordpieceTokenizer.tokenize (tokenization.py:92-99, 163-185)
  void tokenize(const char* utf8, std::vector<int>* ids) const {
    U32 raw;
    decode_utf8(utf8, &raw);
    U32 tok;
    auto flush = [&]() {
      if (!tok.empty()) emit_token(tok, ids);
      tok.clear();
    };
    for (uint32_t cp : raw) {
      if (cp == 0 || cp == 0xFFFD || is_control(cp)) continue;  // _clean_text
      if (is_whitespace(cp) || is_py_space(cp)) {
        flush();
      } else if (is_cjk(cp)) {  // _tokenize_chinese_chars: a CJK character is a token of its own
        flush();
        tok.push_back(cp);
        flush();
      } else {
        tok.push_back(cp);
      }
    }
    flush();
  }
};

U32 ascii_u32(const char* s) {
  U32 v;
  for (; *s; ++s) v.push_back(static_cast<unsigned char>(*s));
  return v;
}

}  // namespace

extern "C" {

void* cudabert_tokenizer_create(const char* vocab_path, int do_lower_case) {
  if (!vocab_path) return nullptr;
  std::FILE* f = std::fopen(vocab_path, "rb");
  if (!f) return nullptr;
  std::unique_ptr<Tokenizer> t(new Tokenizer);
  t->lower = do_lower_case != 0;
  std::string line;
  int index = 0;
  int c;
  auto take_line = [&]() {
    // load_vocab (tokenization.py:51-63): one token per line, stripped, numbered by line
    U32 cps;
    decode_utf8(line.c_str(), &cps);
    size_t b = 0, e = cps.size();
    while (b < e && is_py_space(cps[b])) ++b;
    while (e > b && is_py_space(cps[e - 1])) --e;
    std::string tok;
    for (size_t i = b; i < e; ++i) append_utf8(cps[i], &tok);
    t->vocab[tok] = index++;
    const size_t chars = (e - b >= 2 && cps[b] == '#' && cps[b + 1] == '#') ? e - b - 2 : e - b;
    t->max_piece_chars = std::max(t->max_piece_chars, chars);
    line.clear();
  };
  while ((c = std::fgetc(f)) != EOF) {
    if (c == '\n') take_line();
    else if (c != 0) line.push_back(static_cast<char>(c));
  }
  if (!line.empty()) take_line();
  std::fclose(f);
  auto id_of = [&](const char* s) {
    const auto it = t->vocab.find(s);
    return it == t->vocab.end() ? -1 : it->second;
  };
  t->unk = id_of("[UNK]");
  t->cls = id_of("[CLS]");
  t->sep = id_of("[SEP]");
  if (t->unk < 0 || t->cls < 0 || t->sep < 0) return nullptr;  // the Python code would raise KeyError at first use
  for (const char* s : {"[UNK]", "[SEP]", "[PAD]", "[CLS]", "[MASK]"}) t->never_split.push_back(ascii_u32(s));
  return t.release();
}

void cudabert_tokenizer_destroy(void* tokenizer) { delete static_cast<Tokenizer*>(tokenizer); }

int cudabert_tokenizer_vocab_size(void* tokenizer) {
  return tokenizer ? static_cast<int>(static_cast<Tokenizer*>(tokenizer)->vocab.size()) : -1;
}

int cudabert_tokenizer_tokenize(void* tokenizer, const char* text_utf8, int* ids_out, int capacity) {
  const Tokenizer* t = static_cast<const Tokenizer*>(tokenizer);
  if (!t || !text_utf8 || capacity < 0 || (capacity > 0 && !ids_out)) return -1;
  std::vector<int> ids;
  t->tokenize(text_utf8, &ids);
  const int n = static_cast<int>(ids.size());
  if (n > 0 && capacity > 0) std::memcpy(ids_out, ids.data(), sizeof(int) * std::min(n, capacity));
  return n;
}

int cudabert_tokenizer_encode_pair(void* tokenizer, const char* text_a, const char* text_b, int max_seq_length, int* ids,
                                   int* mask, int* seg) {
  const Tokenizer* t = static_cast<const Tokenizer*>(tokenizer);
  if (!t || !text_a || !ids || !mask || !seg || max_seq_length < 3) return -1;
  std::vector<int> a, b;
  t->tokenize(text_a, &a);
  if (text_b && *text_b) t->tokenize(text_b, &b);
  if (!b.empty()) {
    // _truncate_seq_pair (apps/tokenlizer.py:45-57): drop from the end of the longer list, of the
    // second one on a tie, until both fit beside [CLS] [SEP] [SEP]
    const size_t room = static_cast<size_t>(max_seq_length - 3);
    while (a.size() + b.size() > room) {
      if (a.size() > b.size()) a.pop_back();
      else b.pop_back();
    }
  } else if (a.size() > static_cast<size_t>(max_seq_length - 2)) {
    a.resize(max_seq_length - 2);
  }
  int n = 0;
  auto put = [&](int id, int segment) {
    ids[n] = id;
    mask[n] = 1;
    seg[n] = segment;
    ++n;
  };
  put(t->cls, 0);
  for (int id : a) put(id, 0);
  put(t->sep, 0);
  if (!b.empty()) {
    for (int id : b) put(id, 1);
    put(t->sep, 1);
  }
  for (int i = n; i < max_seq_length; ++i) ids[i] = mask[i] = seg[i] = 0;
  return n;
}

}  // extern "C"
