// Token byte table shared by the grammar matchers: token t is bytes[offsets[t] .. offsets[t + 1]).
#pragma once
#include <cstdint>
#include <vector>

struct MrtVocab {
  std::vector<uint8_t> bytes;
  std::vector<int64_t> offsets;     // n + 1 entries
  int32_t n = 0;
  // tokens in byte-lexicographic order and the common-prefix length of each with its predecessor
  // (filled on first use by the pushdown matcher's mask fill)
  std::vector<int32_t> sorted;
  std::vector<int32_t> lcp;
};
