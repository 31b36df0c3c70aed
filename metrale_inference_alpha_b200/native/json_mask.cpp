// Host runtime, part 2: constrained decoding for JSON. A byte-level pushdown recogniser that
// accepts exactly the prefixes of a JSON value (optionally: top level must be an object), and the
// token-mask fill that lifts it to a vocabulary: for every token, simulate its bytes from the
// current state and mark it legal if no byte is refused. A first-byte filter (256 one-step
// simulations) skips most of the vocabulary before any token is walked, so a fill over ~150k
// tokens costs well under a millisecond. Role of the reference's crates/grammar matcher +
// token bitmask fill for the `json_object` / `json_schema` response formats.
#include <cstdint>
#include <cstring>
#include <vector>

#include "vocab.h"

namespace {

enum State : uint8_t {
  VALUE, KEY, STRING, ESCAPE, UNICODE, LITERAL, BETWEEN, DONE,
  N_MINUS, N_ZERO, N_INT, N_DOT, N_FRAC, N_E, N_ESIGN, N_EXP
};
enum Frame : uint8_t { OBJ_KEY_FIRST, OBJ_KEY, OBJ_COLON, OBJ_VAL, OBJ_NEXT, ARR_FIRST, ARR_VAL, ARR_NEXT };

inline bool is_ws(uint8_t c) { return c == ' ' || c == '\t' || c == '\n' || c == '\r'; }
inline bool is_digit(uint8_t c) { return c >= '0' && c <= '9'; }
inline bool is_hex(uint8_t c) { return is_digit(c) || (c >= 'a' && c <= 'f') || (c >= 'A' && c <= 'F'); }

struct Json {
  std::vector<uint8_t> stack;
  State state = VALUE;
  const char* lit = nullptr;
  uint8_t lit_pos = 0, uni = 0;
  bool string_is_key = false, require_object = false, started = false;
  int32_t max_depth = 64;

  void end_value() {
    if (stack.empty()) { state = DONE; return; }
    if (stack.back() == OBJ_VAL) stack.back() = OBJ_NEXT;
    else if (stack.back() == ARR_VAL) stack.back() = ARR_NEXT;
    state = BETWEEN;
  }
  bool number_complete() const { return state == N_ZERO || state == N_INT || state == N_FRAC || state == N_EXP; }
  bool complete() const { return state == DONE || (stack.empty() && number_complete()); }

  bool feed(uint8_t c) {
    switch (state) {
      case DONE: return is_ws(c);
      case STRING:
        if (c == '"') {
          if (string_is_key) { stack.back() = OBJ_COLON; state = BETWEEN; }
          else end_value();
          return true;
        }
        if (c == '\\') { state = ESCAPE; return true; }
        return c >= 0x20;
      case ESCAPE:
        if (c == 'u') { state = UNICODE; uni = 0; return true; }
        if (std::strchr("\"\\/bfnrt", c) && c) { state = STRING; return true; }
        return false;
      case UNICODE:
        if (!is_hex(c)) return false;
        if (++uni == 4) state = STRING;
        return true;
      case LITERAL:
        if (static_cast<uint8_t>(lit[lit_pos]) != c) return false;
        if (lit[++lit_pos] == 0) end_value();
        return true;
      case N_MINUS:
        if (c == '0') { state = N_ZERO; return true; }
        if (is_digit(c)) { state = N_INT; return true; }
        return false;
      case N_ZERO: case N_INT:
        if (state == N_INT && is_digit(c)) return true;
        if (c == '.') { state = N_DOT; return true; }
        if (c == 'e' || c == 'E') { state = N_E; return true; }
        if (is_digit(c)) return false;                      // leading zero followed by a digit
        end_value();
        return feed(c);                                      // the delimiter belongs to the parent
      case N_DOT:
        if (is_digit(c)) { state = N_FRAC; return true; }
        return false;
      case N_FRAC:
        if (is_digit(c)) return true;
        if (c == 'e' || c == 'E') { state = N_E; return true; }
        end_value();
        return feed(c);
      case N_E:
        if (c == '+' || c == '-') { state = N_ESIGN; return true; }
        if (is_digit(c)) { state = N_EXP; return true; }
        return false;
      case N_ESIGN:
        if (is_digit(c)) { state = N_EXP; return true; }
        return false;
      case N_EXP:
        if (is_digit(c)) return true;
        end_value();
        return feed(c);
      case BETWEEN: {
        if (is_ws(c)) return true;
        if (stack.empty()) return false;
        uint8_t& top = stack.back();
        if (top == OBJ_COLON && c == ':') { top = OBJ_VAL; state = VALUE; return true; }
        if (top == OBJ_NEXT) {
          if (c == ',') { top = OBJ_KEY; state = KEY; return true; }
          if (c == '}') { stack.pop_back(); end_value(); return true; }
        }
        if (top == ARR_NEXT) {
          if (c == ',') { top = ARR_VAL; state = VALUE; return true; }
          if (c == ']') { stack.pop_back(); end_value(); return true; }
        }
        return false;
      }
      case KEY:
        if (is_ws(c)) return true;
        if (c == '"') { stack.back() = OBJ_KEY; state = STRING; string_is_key = true; return true; }
        if (c == '}' && stack.back() == OBJ_KEY_FIRST) { stack.pop_back(); end_value(); return true; }
        return false;
      case VALUE:
        if (is_ws(c)) return true;
        if (require_object && !started && c != '{') return false;
        if (c == ']' && !stack.empty() && stack.back() == ARR_FIRST) { stack.pop_back(); end_value(); return true; }
        if ((c == '{' || c == '[') && static_cast<int32_t>(stack.size()) >= max_depth) return false;
        if (c == '{' || c == '[' || c == '"' || c == '-' || is_digit(c) || c == 't' || c == 'f' || c == 'n') {
          started = true;
          if (!stack.empty() && stack.back() == ARR_FIRST) stack.back() = ARR_VAL;
        }
        if (c == '{') { stack.push_back(OBJ_KEY_FIRST); state = KEY; return true; }
        if (c == '[') { stack.push_back(ARR_FIRST); state = VALUE; return true; }
        if (c == '"') { state = STRING; string_is_key = false; return true; }
        if (c == '-') { state = N_MINUS; return true; }
        if (c == '0') { state = N_ZERO; return true; }
        if (is_digit(c)) { state = N_INT; return true; }
        if (c == 't') { state = LITERAL; lit = "true"; lit_pos = 1; return true; }
        if (c == 'f') { state = LITERAL; lit = "false"; lit_pos = 1; return true; }
        if (c == 'n') { state = LITERAL; lit = "null"; lit_pos = 1; return true; }
        return false;
    }
    return false;
  }
};

using Vocab = MrtVocab;

}  // namespace

extern "C" {

void* mrt_vocab_create(int32_t n, const uint8_t* blob, const int64_t* offsets) {
  auto* v = new Vocab();
  v->n = n;
  v->offsets.assign(offsets, offsets + n + 1);
  v->bytes.assign(blob, blob + offsets[n]);
  return v;
}
void mrt_vocab_destroy(void* v) { delete static_cast<Vocab*>(v); }

void* mrt_json_create(int32_t require_object) {
  auto* j = new Json();
  j->require_object = require_object != 0;
  return j;
}
void* mrt_json_clone(void* h) { return new Json(*static_cast<Json*>(h)); }
void mrt_json_destroy(void* h) { delete static_cast<Json*>(h); }
int32_t mrt_json_complete(void* h) { return static_cast<Json*>(h)->complete() ? 1 : 0; }

// feeds bytes until one is refused; returns the number accepted (== n when all were legal)
int32_t mrt_json_feed(void* h, const uint8_t* b, int32_t n) {
  auto* j = static_cast<Json*>(h);
  for (int32_t i = 0; i < n; ++i)
    if (!j->feed(b[i])) return i;
  return n;
}

// mask[t] = 1 when token t may come next. eos (>= 0) is legal exactly when the document is complete.
// Tokens with no bytes (special tokens) are never legal. Returns the number of legal tokens.
int32_t mrt_json_fill_mask(void* h, void* vocab, int32_t eos, uint8_t* mask, int32_t mask_len) {
  const auto* j = static_cast<const Json*>(h);
  const auto* v = static_cast<const Vocab*>(vocab);
  bool first_ok[256];
  for (int c = 0; c < 256; ++c) {
    Json t = *j;
    first_ok[c] = t.feed(static_cast<uint8_t>(c));
  }
  const int32_t n = v->n < mask_len ? v->n : mask_len;
  std::memset(mask, 0, mask_len);
  int32_t legal = 0;
  Json t;
  for (int32_t tok = 0; tok < n; ++tok) {
    const int64_t a = v->offsets[tok], b = v->offsets[tok + 1];
    if (tok == eos || a == b || !first_ok[v->bytes[a]]) continue;
    bool ok = true;
    if (b - a > 1) {
      t = *j;
      for (int64_t i = a; i < b && ok; ++i) ok = t.feed(v->bytes[i]);
    }
    if (ok) { mask[tok] = 1; ++legal; }
  }
  if (eos >= 0 && eos < mask_len && j->complete()) { mask[eos] = 1; ++legal; }
  return legal;
}

// advance by one token; returns 1 when every byte was legal, 0 otherwise (state is then undefined)
int32_t mrt_json_advance(void* h, void* vocab, int32_t tok) {
  auto* j = static_cast<Json*>(h);
  const auto* v = static_cast<const Vocab*>(vocab);
  if (tok < 0 || tok >= v->n) return 0;
  for (int64_t i = v->offsets[tok]; i < v->offsets[tok + 1]; ++i)
    if (!j->feed(v->bytes[i])) return 0;
  return 1;
}

}  // extern "C"
