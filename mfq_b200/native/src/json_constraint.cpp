// Token constraints for structured output: which tokens of the vocabulary keep the generated text a prefix of a
// valid JSON document.
//
//   * a byte-level pushdown automaton for JSON (RFC 8259): containers on a bit stack (1 = object, 0 = array, depth
//     <= 64), scalar sub-states for strings (escapes, \uXXXX), numbers and the three literals; the whole state is a
//     16-byte value, so trying a token is copy + a few byte steps, no allocation;
//   * the vocabulary as a byte trie built once per tokenizer; the mask of a state is one depth-first walk that steps
//     the automaton along trie edges and abandons a subtree at the first byte the grammar refuses, so the cost is the
//     number of reachable trie nodes, not vocabulary size x token length.
//
// Bytes >= 0x80 (UTF-8 continuation and lead bytes, and the 0xFF placeholder the Python side uses for tokens whose
// bytes it cannot recover) are accepted inside strings only.  Runs of insignificant whitespace are capped, otherwise
// a model can satisfy the grammar forever without making progress.
//
// The reference constrains sampling with the grammar machinery of its tokenizer component
// (cpp_runtime/components/tokenizer: grammar; engine token constraints, cpp_runtime/engine/include).
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "common.h"
#include "mfq_core.h"

namespace {

enum Mode : uint8_t {
  kValue,        // expect the first byte of a value
  kAfterValue,   // a value just ended: , } ] or (at depth 0) the end
  kObjFirst,     // after '{': '"' or '}'
  kObjKey,       // after ',' inside an object: '"'
  kObjColon,     // after a key: ':'
  kArrFirst,     // after '[': a value or ']'
  kString,       // inside a string (key or value, see in_key)
  kStrEsc,       // after a backslash
  kStrHex,       // inside \uXXXX, sub = digits still expected
  kNumSign,      // after '-'
  kNumZero,      // after a leading 0
  kNumInt,       // inside the integer digits
  kNumFracFirst, // after '.'
  kNumFrac,      // inside the fraction digits
  kNumExpSign,   // after e / E
  kNumExpFirst,  // after the exponent's sign
  kNumExp,       // inside the exponent digits
  kLiteral,      // inside true / false / null: lit = which, sub = next index
  kDone,         // the top-level value is complete
};

struct State {
  uint64_t stack = 0;  // bit i = container at depth i + 1 is an object
  uint8_t depth = 0;
  uint8_t mode = kValue;
  uint8_t sub = 0;
  uint8_t lit = 0;
  uint8_t in_key = 0;
  uint8_t ws = 0;           // whitespace bytes in a row
  uint8_t need_object = 0;  // the top-level value has to be an object
  uint8_t pad = 0;
};
static_assert(sizeof(State) == 16, "the state travels to Python as 16 opaque bytes");

constexpr int kMaxDepth = 64;
constexpr int kMaxWhitespace = 8;
const char* const kLiterals[3] = {"true", "false", "null"};

inline bool is_ws(uint8_t c) { return c == ' ' || c == '\n' || c == '\t' || c == '\r'; }
inline bool is_digit(uint8_t c) { return c >= '0' && c <= '9'; }
inline bool is_hex(uint8_t c) { return is_digit(c) || (c >= 'a' && c <= 'f') || (c >= 'A' && c <= 'F'); }

inline void value_ended(State& s) { s.mode = s.depth == 0 ? kDone : kAfterValue; }

inline bool number_can_end(const State& s) {
  return s.mode == kNumZero || s.mode == kNumInt || s.mode == kNumFrac || s.mode == kNumExp;
}

// Consume one byte; false if the grammar refuses it (the state is then unspecified).
bool step(State& s, uint8_t c) {
  for (;;) {  // at most two rounds: a number ends ON the byte after it, which is then read again
    switch (s.mode) {
      case kString:
        if (c == '"') {
          if (s.in_key) { s.in_key = 0; s.mode = kObjColon; } else value_ended(s);
          s.ws = 0;
          return true;
        }
        if (c == '\\') { s.mode = kStrEsc; return true; }
        return c >= 0x20;  // control characters must be escaped
      case kStrEsc:
        if (c == 'u') { s.mode = kStrHex; s.sub = 4; return true; }
        if (std::strchr("\"\\/bfnrt", c) == nullptr || c == 0) return false;
        s.mode = kString;
        return true;
      case kStrHex:
        if (!is_hex(c)) return false;
        if (--s.sub == 0) s.mode = kString;
        return true;
      case kLiteral: {
        const char* word = kLiterals[s.lit];
        if (c != uint8_t(word[s.sub])) return false;
        if (word[++s.sub] == 0) value_ended(s);
        return true;
      }
      case kNumSign:
        if (c == '0') { s.mode = kNumZero; return true; }
        if (is_digit(c)) { s.mode = kNumInt; return true; }
        return false;
      case kNumZero:
      case kNumInt:
        if (s.mode == kNumInt && is_digit(c)) return true;
        if (c == '.') { s.mode = kNumFracFirst; return true; }
        if (c == 'e' || c == 'E') { s.mode = kNumExpSign; return true; }
        if (is_digit(c)) return false;  // no digit after a leading zero
        value_ended(s);
        continue;
      case kNumFracFirst:
        if (!is_digit(c)) return false;
        s.mode = kNumFrac;
        return true;
      case kNumFrac:
        if (is_digit(c)) return true;
        if (c == 'e' || c == 'E') { s.mode = kNumExpSign; return true; }
        value_ended(s);
        continue;
      case kNumExpSign:
        if (c == '+' || c == '-') { s.mode = kNumExpFirst; return true; }
        if (is_digit(c)) { s.mode = kNumExp; return true; }
        return false;
      case kNumExpFirst:
        if (!is_digit(c)) return false;
        s.mode = kNumExp;
        return true;
      case kNumExp:
        if (is_digit(c)) return true;
        value_ended(s);
        continue;
      default:
        break;
    }
    break;
  }
  // structural positions: whitespace is insignificant but bounded
  if (is_ws(c)) {
    if (s.mode == kDone && s.depth == 0 && s.ws >= 1) return false;  // one trailing newline at most
    if (++s.ws > kMaxWhitespace) return false;
    return true;
  }
  s.ws = 0;
  switch (s.mode) {
    case kArrFirst:
      if (c == ']') {
        --s.depth;
        value_ended(s);
        return true;
      }
      [[fallthrough]];
    case kValue:
      if (s.need_object && s.depth == 0 && c != '{') return false;
      if (c == '{' || c == '[') {
        if (s.depth >= kMaxDepth) return false;
        if (c == '{') s.stack |= uint64_t(1) << s.depth; else s.stack &= ~(uint64_t(1) << s.depth);
        ++s.depth;
        s.mode = c == '{' ? kObjFirst : kArrFirst;
        return true;
      }
      if (c == '"') { s.mode = kString; s.in_key = 0; return true; }
      if (c == '-') { s.mode = kNumSign; return true; }
      if (c == '0') { s.mode = kNumZero; return true; }
      if (is_digit(c)) { s.mode = kNumInt; return true; }
      if (c == 't' || c == 'f' || c == 'n') {
        s.mode = kLiteral;
        s.lit = c == 't' ? 0 : (c == 'f' ? 1 : 2);
        s.sub = 1;
        return true;
      }
      return false;
    case kObjFirst:
      if (c == '}') {
        --s.depth;
        value_ended(s);
        return true;
      }
      [[fallthrough]];
    case kObjKey:
      if (c != '"') return false;
      s.mode = kString;
      s.in_key = 1;
      return true;
    case kObjColon:
      if (c != ':') return false;
      s.mode = kValue;
      return true;
    case kAfterValue: {
      const bool in_object = (s.stack >> (s.depth - 1)) & 1;
      if (c == ',') { s.mode = in_object ? kObjKey : kValue; return true; }
      if (c == (in_object ? '}' : ']')) {
        --s.depth;
        value_ended(s);
        return true;
      }
      return false;
    }
    default:  // kDone: nothing but (bounded) whitespace may follow
      return false;
  }
}

inline bool complete(const State& s) {
  return s.mode == kDone || (s.depth == 0 && !s.need_object && number_can_end(s));
}

struct Trie {
  struct Node {
    int32_t first_child = -1, next_sibling = -1;
    int32_t first_token = -1;  // head of the list of tokens that end here
    uint8_t byte = 0;
  };
  std::vector<Node> nodes;
  std::vector<int32_t> next_token;  // token -> next token ending at the same node
  int64_t vocab = 0;

  int child(int node, uint8_t b) {
    for (int c = nodes[node].first_child; c >= 0; c = nodes[c].next_sibling)
      if (nodes[c].byte == b) return c;
    Node n;
    n.byte = b;
    n.next_sibling = nodes[node].first_child;
    nodes.push_back(n);
    nodes[node].first_child = int(nodes.size()) - 1;
    return int(nodes.size()) - 1;
  }
};

void walk(const Trie& t, int node, const State& s, uint32_t* bits, int64_t& count) {
  for (int c = t.nodes[node].first_child; c >= 0; c = t.nodes[c].next_sibling) {
    State next = s;
    if (!step(next, t.nodes[c].byte)) continue;
    for (int tok = t.nodes[c].first_token; tok >= 0; tok = t.next_token[tok]) {
      bits[tok >> 5] |= 1u << (tok & 31);
      ++count;
    }
    walk(t, c, next, bits, count);
  }
}

}  // namespace

extern "C" {

// bytes: the concatenated byte strings of all tokens; offsets [vocab + 1].  Tokens with an empty string (special
// tokens) never match.
void* mfq_json_vocab_open(const uint8_t* bytes, const int64_t* offsets, int64_t vocab) {
  if (!bytes || !offsets || vocab <= 0) {
    mfqn::fail(-1, "json vocabulary: empty input");
    return nullptr;
  }
  auto* t = new Trie();
  t->vocab = vocab;
  t->nodes.emplace_back();
  t->next_token.assign(size_t(vocab), -1);
  for (int64_t tok = 0; tok < vocab; ++tok) {
    const int64_t lo = offsets[tok], hi = offsets[tok + 1];
    if (hi <= lo) continue;
    int node = 0;
    for (int64_t i = lo; i < hi; ++i) node = t->child(node, bytes[i]);
    t->next_token[size_t(tok)] = t->nodes[size_t(node)].first_token;
    t->nodes[size_t(node)].first_token = int32_t(tok);
  }
  return t;
}

void mfq_json_vocab_close(void* vocab) { delete static_cast<Trie*>(vocab); }

int64_t mfq_json_vocab_nodes(void* vocab) { return vocab ? int64_t(static_cast<Trie*>(vocab)->nodes.size()) : -1; }

// state: 16 opaque bytes
void mfq_json_state_init(void* state, int need_object) {
  State s;
  s.need_object = need_object ? 1 : 0;
  std::memcpy(state, &s, sizeof s);
}

// Feed bytes; returns 0, or -1 at the first refused byte (the state is left as it was before the call).
int mfq_json_state_feed(void* state, const uint8_t* bytes, int64_t n) {
  State s;
  std::memcpy(&s, state, sizeof s);
  for (int64_t i = 0; i < n; ++i)
    if (!step(s, bytes[i])) return -1;
  std::memcpy(state, &s, sizeof s);
  return 0;
}

// 1 when the text so far is a complete document (the end-of-sequence token may follow)
int mfq_json_state_complete(const void* state) {
  State s;
  std::memcpy(&s, state, sizeof s);
  return complete(s) ? 1 : 0;
}

// bits_out [ceil(vocab / 32)] words: bit t set = token t may come next.  Returns the number of set bits.
int64_t mfq_json_mask(void* vocab, const void* state, uint32_t* bits_out) {
  if (!vocab || !state || !bits_out) {
    mfqn::fail(-1, "json mask: null argument");
    return -1;
  }
  const Trie& t = *static_cast<Trie*>(vocab);
  State s;
  std::memcpy(&s, state, sizeof s);
  std::memset(bits_out, 0, size_t((t.vocab + 31) / 32) * sizeof(uint32_t));
  int64_t count = 0;
  walk(t, 0, s, bits_out, count);
  return count;
}
}
