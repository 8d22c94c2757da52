// Hand-written scanner for the GPT-4-style split pattern
//
//   '(?i:[sdmt]|ll|ve|re) | [^\r\n\p{L}\p{N}]?+\p{L}+ | \p{N}{1,2} | ?[^\s\p{L}\p{N}]++[\r\n]* |
//   \s*[\r\n] | \s+(?!\S) | \s+
//
// over UTF-8 text. It yields the same pieces a backtracking regex engine produces for that
// pattern (alternatives tried in order at each position, possessive quantifiers never give
// back, the look-ahead alternative gives back exactly one code point). Invalid UTF-8 bytes
// are treated as single "other" code points so the pieces always tile the input.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string_view>
#include <vector>

namespace tok {

enum CharClass : uint8_t { C_OTHER = 0, C_LETTER = 1, C_NUMBER = 2, C_SPACE = 3 };

CharClass classify(uint32_t cp);

// Decodes one code point starting at s[i] (i < n); returns its byte length (>= 1).
inline int decode_utf8(const unsigned char* s, size_t i, size_t n, uint32_t& cp) {
  const unsigned char c = s[i];
  if (c < 0x80) { cp = c; return 1; }
  int len = (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 0;
  if (len == 0 || i + len > n) { cp = 0xFFFD; return 1; }
  uint32_t v = c & (0xFF >> (len + 1));
  for (int k = 1; k < len; ++k) {
    const unsigned char d = s[i + k];
    if ((d & 0xC0) != 0x80) { cp = 0xFFFD; return 1; }
    v = (v << 6) | (d & 0x3F);
  }
  cp = v;
  return len;
}

// Appends [start, end) byte offsets of the pieces of `text` to `out`.
void split(std::string_view text, std::vector<std::pair<uint32_t, uint32_t>>& out);

}  // namespace tok
