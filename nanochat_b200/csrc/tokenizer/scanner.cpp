#include "scanner.h"

#include <algorithm>

namespace tok {

#include "unicode_tables.inc"

static uint8_t g_ascii[128];
static bool g_ascii_ready = false;

static bool in_ranges(const uint32_t (*r)[2], int n, uint32_t cp) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) >> 1;
    if (cp < r[mid][0]) hi = mid - 1;
    else if (cp > r[mid][1]) lo = mid + 1;
    else return true;
  }
  return false;
}

static CharClass classify_slow(uint32_t cp) {
  if (in_ranges(UNI_SPACE, UNI_SPACE_N, cp)) return C_SPACE;
  if (in_ranges(UNI_LETTER, UNI_LETTER_N, cp)) return C_LETTER;
  if (in_ranges(UNI_NUMBER, UNI_NUMBER_N, cp)) return C_NUMBER;
  return C_OTHER;
}

CharClass classify(uint32_t cp) {
  if (cp < 128) {
    if (!g_ascii_ready) {
      for (uint32_t c = 0; c < 128; ++c) g_ascii[c] = classify_slow(c);
      g_ascii_ready = true;
    }
    return static_cast<CharClass>(g_ascii[cp]);
  }
  return classify_slow(cp);
}

namespace {
struct Cursor {
  const unsigned char* s;
  size_t n;
  // code point at byte offset i (i < n)
  inline int at(size_t i, uint32_t& cp) const { return decode_utf8(s, i, n, cp); }
};

inline bool is_newline(uint32_t cp) { return cp == '\r' || cp == '\n'; }

// contraction suffix after an apostrophe at i: returns byte length of the suffix or 0
inline size_t contraction(const Cursor& c, size_t i) {
  if (i >= c.n) return 0;
  uint32_t a; const int la = c.at(i, a);
  auto lower = [](uint32_t x) { return (x >= 'A' && x <= 'Z') ? x + 32 : x; };
  const uint32_t al = lower(a);
  if (al == 's' || al == 'd' || al == 'm' || al == 't' || a == 0x17F /* long s folds to s */) return la;
  if (i + la >= c.n) return 0;
  uint32_t b; const int lb = c.at(i + la, b);
  const uint32_t bl = lower(b);
  if ((al == 'l' && bl == 'l') || (al == 'v' && bl == 'e') || (al == 'r' && bl == 'e')) return la + lb;
  return 0;
}
}  // namespace

void split(std::string_view text, std::vector<std::pair<uint32_t, uint32_t>>& out) {
  classify(0);  // make sure the ASCII table exists before worker threads race on it
  const Cursor c{reinterpret_cast<const unsigned char*>(text.data()), text.size()};
  const size_t n = c.n;
  size_t i = 0;
  while (i < n) {
    uint32_t cp; const int len = c.at(i, cp);
    const CharClass cls = classify(cp);
    size_t end = 0;
    // 1) contractions
    if (cp == '\'') {
      const size_t k = contraction(c, i + len);
      if (k) end = i + len + k;
    }
    // 2) optional non-letter/number/newline prefix + letters
    if (!end) {
      size_t j = i;
      bool ok = false;
      if (cls == C_LETTER) {
        ok = true;
      } else if (cls != C_NUMBER && !is_newline(cp) && i + len < n) {
        uint32_t nx; c.at(i + len, nx);
        if (classify(nx) == C_LETTER) { ok = true; j = i + len; }
      }
      if (ok) {
        while (j < n) {
          uint32_t x; const int lx = c.at(j, x);
          if (classify(x) != C_LETTER) break;
          j += lx;
        }
        end = j;
      }
    }
    // 3) one or two numbers
    if (!end && cls == C_NUMBER) {
      size_t j = i + len;
      if (j < n) {
        uint32_t x; const int lx = c.at(j, x);
        if (classify(x) == C_NUMBER) j += lx;
      }
      end = j;
    }
    // 4) optional space + run of "other" + trailing newlines
    if (!end) {
      size_t j = i;
      bool ok = false;
      if (cls == C_OTHER) {
        ok = true;
      } else if (cp == ' ' && i + len < n) {
        uint32_t nx; c.at(i + len, nx);
        if (classify(nx) == C_OTHER) { ok = true; j = i + len; }
      }
      if (ok) {
        while (j < n) {
          uint32_t x; const int lx = c.at(j, x);
          if (classify(x) != C_OTHER) break;
          j += lx;
        }
        while (j < n && (c.s[j] == '\r' || c.s[j] == '\n')) ++j;
        end = j;
      }
    }
    // 5-7) whitespace runs
    if (!end) {
      // here cls == C_SPACE necessarily
      size_t j = i, last_nl_end = 0, last_cp_start = i;
      while (j < n) {
        uint32_t x; const int lx = c.at(j, x);
        if (classify(x) != C_SPACE) break;
        if (is_newline(x)) last_nl_end = j + lx;
        last_cp_start = j;
        j += lx;
      }
      if (last_nl_end) end = last_nl_end;                 // \s*[\r\n]
      else if (j == n) end = j;                           // \s+(?!\S) at end of text
      else if (last_cp_start > i) end = last_cp_start;    // \s+(?!\S): give back one code point
      else end = j;                                       // \s+
    }
    out.emplace_back(static_cast<uint32_t>(i), static_cast<uint32_t>(end));
    i = end;
  }
}

}  // namespace tok
