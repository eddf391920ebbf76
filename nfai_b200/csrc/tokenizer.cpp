// Byte-pair tokenizer with the behaviour of the reference's NFAI.Models.Llama3/Tokenizer.cs, host side only.
//
// The reference finds the next merge by comparing every adjacent pair of a word against every entry of the merges
// list (Tokenizer.cs:130-166: O(parts x merges) byte comparisons per merge round, ~280 000 merges for Llama-3).
// Here the merges sit in a hash map (left, right) -> rank, so a round costs one lookup per adjacent pair. Everything
// observable is kept: the chat template (Tokenizer.cs:70-91), the special-token split that drops text in front of
// the first special token (:93-107), the pre-tokenisation pattern (:109-111) evaluated on UTF-16 code units, the
// initial units (one per UTF-16 code unit; ' ' and '\n' become C4 A0 / C4 8A, :242-267), lowest rank first and the
// leftmost pair among equal ranks (:137-157), last-one-wins for duplicate vocabulary entries (:50-57), first-one-wins
// for duplicate merges (:142-155), and the errors (unknown special token, part without a vocabulary entry).
#include <stdint.h>
#include <string.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/nfai_cuda.h"
#include "unicode_tables.h"

namespace {

bool in_ranges(const uint16_t (*r)[2], int n, uint16_t c) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) / 2;
    if (c < r[mid][0]) hi = mid - 1;
    else if (c > r[mid][1]) lo = mid + 1;
    else return true;
  }
  return false;
}
bool is_letter(uint16_t c) { return in_ranges(kUnicodeLetter, kUnicodeLetter_count, c); }
bool is_number(uint16_t c) { return in_ranges(kUnicodeNumber, kUnicodeNumber_count, c); }
// .NET \s: [\f\n\r\t\v\x85\p{Z}]
bool is_space(uint16_t c) {
  return (c >= 0x09 && c <= 0x0D) || c == 0x85 || in_ranges(kUnicodeSeparator, kUnicodeSeparator_count, c);
}
bool is_crlf(uint16_t c) { return c == '\r' || c == '\n'; }
bool is_other(uint16_t c) { return !is_space(c) && !is_letter(c) && !is_number(c); }

// UTF-8 -> UTF-16 code units (invalid bytes become U+FFFD, as Encoding.UTF8 does when the C# string is built)
std::vector<uint16_t> to_utf16(const char* s, size_t n) {
  std::vector<uint16_t> out;
  out.reserve(n);
  size_t i = 0;
  while (i < n) {
    const unsigned char b = (unsigned char)s[i];
    uint32_t cp = 0xFFFD;
    size_t len = 1;
    if (b < 0x80) cp = b;
    else if ((b & 0xE0) == 0xC0 && i + 1 < n && ((unsigned char)s[i + 1] & 0xC0) == 0x80) {
      cp = ((b & 0x1Fu) << 6) | ((unsigned char)s[i + 1] & 0x3Fu);
      len = 2;
      if (cp < 0x80) cp = 0xFFFD;
    } else if ((b & 0xF0) == 0xE0 && i + 2 < n && ((unsigned char)s[i + 1] & 0xC0) == 0x80 && ((unsigned char)s[i + 2] & 0xC0) == 0x80) {
      cp = ((b & 0x0Fu) << 12) | (((unsigned char)s[i + 1] & 0x3Fu) << 6) | ((unsigned char)s[i + 2] & 0x3Fu);
      len = 3;
      if (cp < 0x800 || (cp >= 0xD800 && cp <= 0xDFFF)) cp = 0xFFFD;
    } else if ((b & 0xF8) == 0xF0 && i + 3 < n && ((unsigned char)s[i + 1] & 0xC0) == 0x80 && ((unsigned char)s[i + 2] & 0xC0) == 0x80 &&
               ((unsigned char)s[i + 3] & 0xC0) == 0x80) {
      cp = ((b & 0x07u) << 18) | (((unsigned char)s[i + 1] & 0x3Fu) << 12) | (((unsigned char)s[i + 2] & 0x3Fu) << 6) |
           ((unsigned char)s[i + 3] & 0x3Fu);
      len = 4;
      if (cp < 0x10000 || cp > 0x10FFFF) cp = 0xFFFD;
    }
    i += len;
    if (cp >= 0x10000) {
      cp -= 0x10000;
      out.push_back((uint16_t)(0xD800 + (cp >> 10)));
      out.push_back((uint16_t)(0xDC00 + (cp & 0x3FF)));
    } else {
      out.push_back((uint16_t)cp);
    }
  }
  return out;
}

// One UTF-16 code unit as the bytes Encoding.UTF8.GetBytes(ch.ToString()) yields (a lone surrogate is U+FFFD)
void unit_bytes(uint16_t c, std::string& out) {
  out.clear();
  if (c >= 0xD800 && c <= 0xDFFF) c = 0xFFFD;
  if (c < 0x80) out.push_back((char)c);
  else if (c < 0x800) {
    out.push_back((char)(0xC0 | (c >> 6)));
    out.push_back((char)(0x80 | (c & 0x3F)));
  } else {
    out.push_back((char)(0xE0 | (c >> 12)));
    out.push_back((char)(0x80 | ((c >> 6) & 0x3F)));
    out.push_back((char)(0x80 | (c & 0x3F)));
  }
}

bool ieq(uint16_t c, char lower) { return c == (uint16_t)lower || c == (uint16_t)(lower - 32); }

// Length of the match of the pre-tokenisation pattern at position i (always >= 1):
// (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
size_t match_at(const std::vector<uint16_t>& t, size_t i) {
  const size_t n = t.size();
  const uint16_t c = t[i];
  // 1. contractions
  if (c == '\'' && i + 1 < n) {
    const uint16_t d = t[i + 1];
    if (ieq(d, 's') || ieq(d, 't') || ieq(d, 'm') || ieq(d, 'd')) return 2;
    if (i + 2 < n) {
      const uint16_t e = t[i + 2];
      if ((ieq(d, 'r') && ieq(e, 'e')) || (ieq(d, 'v') && ieq(e, 'e')) || (ieq(d, 'l') && ieq(e, 'l'))) return 3;
    }
  }
  // 2. optional non-letter/number/CR/LF prefix, then letters
  {
    size_t j = i;
    if (!is_letter(c)) {
      if (!is_crlf(c) && !is_number(c) && i + 1 < n && is_letter(t[i + 1])) j = i + 1;
      else j = n + 1;  // no match
    }
    if (j <= n && j < n && is_letter(t[j])) {
      while (j < n && is_letter(t[j])) ++j;
      return j - i;
    }
  }
  // 3. one to three numbers
  if (is_number(c)) {
    size_t j = i;
    while (j < n && j - i < 3 && is_number(t[j])) ++j;
    return j - i;
  }
  // 4. optional space, other characters, trailing CR/LF
  {
    size_t j = i;
    if (c == ' ' && i + 1 < n && is_other(t[i + 1])) j = i + 1;
    if (is_other(t[j])) {
      while (j < n && is_other(t[j])) ++j;
      while (j < n && is_crlf(t[j])) ++j;
      return j - i;
    }
  }
  // 5.-7. whitespace runs
  size_t end = i;
  while (end < n && is_space(t[end])) ++end;
  if (end > i) {
    size_t last = n;  // last CR/LF inside the run
    for (size_t k = i; k < end; ++k)
      if (is_crlf(t[k])) last = k;
    if (last != n) return last + 1 - i;       // \s*[\r\n]+
    if (end == n) return end - i;             // \s+(?!\S) at the end of the text
    if (end - i >= 2) return end - i - 1;     // \s+(?!\S): leaves the last space to the next word
    return end - i;                           // \s+
  }
  return 1;  // unreachable: every code unit is a space, a letter, a number or "other"
}

struct PairHash {
  size_t operator()(const std::pair<std::string, std::string>& p) const {
    return std::hash<std::string>()(p.first) * 1000003u ^ std::hash<std::string>()(p.second);
  }
};

}  // namespace

struct nfai_tokenizer {
  std::vector<std::string> id_to_bytes;
  std::unordered_map<std::string, uint32_t> bytes_to_id;
  std::unordered_map<std::pair<std::string, std::string>, uint32_t, PairHash> rank;
  uint32_t bos = 0, eos = 0;
  std::string error;
};

namespace {

int tk_fail(nfai_tokenizer* t, int code, const std::string& msg) {
  if (t) t->error = msg;
  return code;
}

// Tokenizer.cs:115-180 for one stretch of text between special tokens
int encode_plain(nfai_tokenizer* t, const std::vector<uint16_t>& text, std::vector<uint32_t>& ids) {
  std::vector<std::string> parts;
  std::string unit;
  size_t i = 0;
  while (i < text.size()) {
    const size_t len = match_at(text, i);
    parts.clear();
    for (size_t k = i; k < i + len; ++k) {
      const uint16_t c = text[k];
      if (c == ' ' || c == '\n') {  // byte-level alphabet of the vocabulary: U+0120 / U+010A
        const char b[2] = {(char)0xC4, (char)(c + 0x80)};
        parts.emplace_back(b, 2);
      } else {
        unit_bytes(c, unit);
        parts.push_back(unit);
      }
    }
    i += len;
    while (parts.size() > 1) {
      uint32_t best_rank = 0xffffffffu;
      size_t best_j = 0;
      for (size_t j = 0; j + 1 < parts.size(); ++j) {
        auto it = t->rank.find(std::make_pair(parts[j], parts[j + 1]));
        if (it != t->rank.end() && it->second < best_rank) {
          best_rank = it->second;
          best_j = j;
        }
      }
      if (best_rank == 0xffffffffu) break;
      parts[best_j] += parts[best_j + 1];
      parts.erase(parts.begin() + (long)best_j + 1);
    }
    for (const std::string& p : parts) {
      auto it = t->bytes_to_id.find(p);
      if (it == t->bytes_to_id.end()) return tk_fail(t, NFAI_ERR_ARG, "Token not found: " + p);
      ids.push_back(it->second);
    }
  }
  return NFAI_OK;
}

// Tokenizer.cs:93-180: special tokens <|...|> and the text behind each; text in front of the first one is dropped
int encode_with_specials(nfai_tokenizer* t, const std::string& templ, std::vector<uint32_t>& ids) {
  struct Span { size_t b, e; };
  std::vector<Span> specials;
  size_t i = 0;
  while (i + 1 < templ.size()) {
    if (templ[i] == '<' && templ[i + 1] == '|') {
      size_t j = i + 2;
      while (j < templ.size() && templ[j] != '|' && templ[j] != '>') ++j;
      if (j > i + 2 && j + 1 < templ.size() && templ[j] == '|' && templ[j + 1] == '>') {
        specials.push_back({i, j + 2});
        i = j + 2;
        continue;
      }
    }
    ++i;
  }
  for (size_t k = 0; k < specials.size(); ++k) {
    const std::string sp = templ.substr(specials[k].b, specials[k].e - specials[k].b);
    auto it = t->bytes_to_id.find(sp);
    if (it == t->bytes_to_id.end()) return tk_fail(t, NFAI_ERR_ARG, "special token not in the vocabulary: " + sp);
    ids.push_back(it->second);
    const size_t tb = specials[k].e, te = k + 1 < specials.size() ? specials[k + 1].b : templ.size();
    const std::vector<uint16_t> text = to_utf16(templ.data() + tb, te - tb);
    const int rc = encode_plain(t, text, ids);
    if (rc) return rc;
  }
  return NFAI_OK;
}

int copy_out(nfai_tokenizer* t, const std::vector<uint32_t>& ids, uint32_t* out, size_t cap, size_t* n_out) {
  if (n_out) *n_out = ids.size();
  if (ids.size() > cap) return tk_fail(t, NFAI_ERR_ARG, "output buffer too small");
  if (out && !ids.empty()) memcpy(out, ids.data(), ids.size() * sizeof(uint32_t));
  return NFAI_OK;
}

}  // namespace

extern "C" {

int nfai_tokenizer_create(const char* const* tokens, const uint32_t* token_lens, uint32_t n_tokens, const char* const* merges,
                          const uint32_t* merge_lens, uint32_t n_merges, uint32_t bos_id, uint32_t eos_id,
                          nfai_tokenizer** out) {
  if (!out || (!tokens && n_tokens) || (!merges && n_merges) || (n_tokens && !token_lens) || (n_merges && !merge_lens)) return NFAI_ERR_ARG;
  nfai_tokenizer* t = new nfai_tokenizer();
  t->bos = bos_id;
  t->eos = eos_id;
  t->id_to_bytes.reserve(n_tokens);
  t->bytes_to_id.reserve(n_tokens * 2);
  for (uint32_t i = 0; i < n_tokens; ++i) {
    t->id_to_bytes.emplace_back(tokens[i], token_lens[i]);
    t->bytes_to_id[t->id_to_bytes.back()] = i;  // a repeated byte string keeps the last id (Tokenizer.cs:55)
  }
  t->rank.reserve(n_merges * 2);
  for (uint32_t k = 0; k < n_merges; ++k) {
    const std::string m(merges[k], merge_lens[k]);
    const size_t sp = m.find(' ');  // "left right": split at the first space (Tokenizer.cs:33-35)
    if (sp == std::string::npos) {
      delete t;
      return NFAI_ERR_ARG;
    }
    t->rank.emplace(std::make_pair(m.substr(0, sp), m.substr(sp + 1)), k);  // a repeated pair keeps the first rank
  }
  *out = t;
  return NFAI_OK;
}

void nfai_tokenizer_destroy(nfai_tokenizer* t) { delete t; }

const char* nfai_tokenizer_last_error(const nfai_tokenizer* t) { return t ? t->error.c_str() : "null tokenizer"; }

int nfai_tokenizer_encode(nfai_tokenizer* t, const char* text, size_t text_len, uint32_t* ids_out, size_t cap, size_t* n_out) {
  if (!t || (!text && text_len) || !n_out) return NFAI_ERR_ARG;
  std::vector<uint32_t> ids;
  const int rc = encode_with_specials(t, std::string(text ? text : "", text_len), ids);
  if (rc) return rc;
  return copy_out(t, ids, ids_out, cap, n_out);
}

int nfai_tokenizer_encode_chat(nfai_tokenizer* t, const char* prompt, size_t prompt_len, int add_bos, uint32_t* ids_out, size_t cap,
                               size_t* n_out) {
  if (!t || (!prompt && prompt_len) || !n_out) return NFAI_ERR_ARG;
  const std::string user(prompt ? prompt : "", prompt_len);
  std::string templ;
  if (add_bos)
    templ = "<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\nYou are a helpful assistant.<|eot_id|>"
            "<|start_header_id|>user<|end_header_id|>\n\n" + user + "<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n";
  else
    templ = "\n\n<|start_header_id|>user<|end_header_id|>\n\n" + user + "<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n";
  std::string clean;  // .Replace("\r", "")
  clean.reserve(templ.size());
  for (char ch : templ)
    if (ch != '\r') clean.push_back(ch);
  std::vector<uint32_t> ids;
  const int rc = encode_with_specials(t, clean, ids);
  if (rc) return rc;
  return copy_out(t, ids, ids_out, cap, n_out);
}

int nfai_tokenizer_pretokenize(nfai_tokenizer* t, const char* text, size_t text_len, uint32_t* ends_out, size_t cap, size_t* n_out) {
  if (!t || (!text && text_len) || !n_out) return NFAI_ERR_ARG;
  const std::vector<uint16_t> units = to_utf16(text ? text : "", text_len);
  std::vector<uint32_t> ends;
  size_t i = 0;
  while (i < units.size()) {
    i += match_at(units, i);
    ends.push_back((uint32_t)i);
  }
  return copy_out(t, ends, ends_out, cap, n_out);
}

int nfai_tokenizer_decode(nfai_tokenizer* t, const uint32_t* ids, size_t n, char* text_out, size_t cap, size_t* n_out) {
  if (!t || (!ids && n) || !n_out) return NFAI_ERR_ARG;
  std::string bytes;
  for (size_t i = 0; i < n; ++i) {
    if (ids[i] >= t->id_to_bytes.size()) return tk_fail(t, NFAI_ERR_ARG, "Token ID " + std::to_string(ids[i]) + " not found in vocabulary.");
    bytes += t->id_to_bytes[ids[i]];
  }
  // U+0120 -> ' ', U+010A -> '\n' (Tokenizer.cs:457-459); other bytes pass through
  std::string out;
  out.reserve(bytes.size());
  for (size_t i = 0; i < bytes.size(); ++i) {
    if ((unsigned char)bytes[i] == 0xC4 && i + 1 < bytes.size() && ((unsigned char)bytes[i + 1] == 0xA0 || (unsigned char)bytes[i + 1] == 0x8A)) {
      out.push_back((unsigned char)bytes[i + 1] == 0xA0 ? ' ' : '\n');
      ++i;
    } else {
      out.push_back(bytes[i]);
    }
  }
  *n_out = out.size();
  if (out.size() > cap) return tk_fail(t, NFAI_ERR_ARG, "output buffer too small");
  if (text_out && !out.empty()) memcpy(text_out, out.data(), out.size());
  return NFAI_OK;
}

}  // extern "C"
