// A small backtracking regular-expression matcher for the pre-tokenisation patterns of byte-level
// BPE tokenizers (the `Split` and `ByteLevel` pre-tokenisers of a tokenizer.json, which the
// reference runs through its tokenizer dependency's regular-expression engine).  It takes the
// constructs those patterns are written in:
//
//   alternation, groups ( ) (?: ) (?i: ) (?i) (?> ), look-ahead (?= ) (?! ), classes [ ] [^ ] with
//   ranges and escapes, . ^ $ (line anchors) \A \z \b \B, \s \S \d \D \w \W, \p{..} \P{..} with
//   general categories (one- and two-letter names) and a few scripts, \r \n \t \f \v \xHH \uHHHH
//   \x{H..}, quantifiers ? * + {m} {m,} {m,n}, greedy, lazy (?) or, for ? * +, possessive (+); X{m}?
//   is (?:X{m})? as in the engine this follows.
//
// Anything else (look-behind, back-references, named groups, class intersections, case-insensitive
// matching of non-ASCII text, unknown property names) is refused when the pattern is compiled, with
// a message: nothing is approximated.  Matching is leftmost with the alternatives tried in
// order, as in the engines tokenizers use; character classes follow the tables of unicode_tables.h.
// Host-only C++.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace llmcp_b200 {
namespace detail {

class Regex {
public:
  // "" or the reason the pattern is not taken.
  std::string compile(const std::string &pattern_utf8);
  // Leftmost match at or after code point `from` of `text`.  Returns 1 with [*begin, *end), 0 when
  // there is none, -1 when the step budget ran out (a pattern that backtracks without end).
  int search(const std::vector<uint32_t> &text, size_t from, size_t *begin, size_t *end) const;

private:
  struct Range {
    uint32_t first, last;
  };
  using Set = std::vector<Range>; // sorted, disjoint
  enum Op { kSet, kSpan, kSplit, kJump, kMatch, kLook, kAtomic, kBol, kEol, kTextBegin, kTextFinish, kWordBoundary, kNotWordBoundary };
  struct Inst {
    Op op;
    int x = 0, y = 0; // kSplit: first and second continuation; kJump: x; kLook / kAtomic: y = continuation, body at pc + 1
    int set = -1;
    int min = 0, max = -1, mode = 0; // kSpan: counts (-1: unbounded) and 0 greedy, 1 lazy, 2 possessive
    bool negate = false;             // kLook
  };
  struct Node;
  struct Parser;

  size_t run(int pc, size_t pos, const std::vector<uint32_t> &text, int64_t *budget) const;
  static bool in_set(const Set &set, uint32_t cp);
  int emit(const Node &node, std::string *error);

  std::vector<Set> sets_;
  std::vector<Inst> program_;
};

// How a `Split` pre-tokeniser treats its matches (SplitDelimiterBehavior of the tokenizers library).
enum class SplitBehavior { kRemoved, kIsolated, kMergedWithPrevious, kMergedWithNext, kContiguous };

// "" and the behaviour, or an error for an unknown name ("Isolated", "isolated", "merged_with_previous", ...).
std::string parse_split_behavior(const std::string &name, SplitBehavior *behavior);

// The pieces of `text` (UTF-8) under a Split with this pattern; empty pieces are dropped.  Returns ""
// or an error (step budget, or a match of the empty string, which no pre-tokenisation pattern has).
std::string regex_split(const Regex &regex, const std::string &text, SplitBehavior behavior, bool invert,
                        std::vector<std::string> *pieces);

} // namespace detail
} // namespace llmcp_b200
