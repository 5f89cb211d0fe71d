#include "text_regex.h"

#include <algorithm>
#include <cstring>

#include "unicode_tables.h"

namespace llmcp_b200 {
namespace detail {

void utf8_points(const std::string &text, std::vector<uint32_t> *points, std::vector<size_t> *offsets); // text.cpp

namespace {

constexpr uint32_t kMaxPoint = 0x10ffff;
constexpr int kMaxCopies = 64;           // of a repeated group that is not a single character
constexpr int64_t kStepBudget = 200000000; // instructions per search

struct R {
  uint32_t first, last;
};

void normalise(std::vector<R> *set) {
  std::sort(set->begin(), set->end(), [](const R &a, const R &b) { return a.first < b.first; });
  std::vector<R> out;
  for (const R &r : *set) {
    if (!out.empty() && r.first <= out.back().last + 1)
      out.back().last = std::max(out.back().last, r.last);
    else
      out.push_back(r);
  }
  set->swap(out);
}

void complement(std::vector<R> *set) {
  normalise(set);
  std::vector<R> out;
  uint32_t next = 0;
  bool open = true;
  for (const R &r : *set) {
    if (r.first > next)
      out.push_back({next, r.first - 1});
    if (r.last == kMaxPoint) {
      open = false;
      break;
    }
    next = r.last + 1;
  }
  if (open)
    out.push_back({next, kMaxPoint});
  set->swap(out);
}

template <typename T, size_t N>
void add_table(const T (&table)[N], std::vector<R> *set) {
  for (const T &r : table)
    set->push_back({r.first, r.last});
}

// \p{name}: a general category (one letter: all categories that start with it; two letters; Cn and
// C take the unlisted code points), a long category name, or one of the listed scripts.
bool add_property(const std::string &name, std::vector<R> *set) {
  static const struct {
    const char *longer, *shorter;
  } aliases[] = {{"Letter", "L"}, {"Mark", "M"}, {"Number", "N"}, {"Punctuation", "P"}, {"Symbol", "S"}, {"Separator", "Z"},
                 {"Other", "C"}, {"Uppercase_Letter", "Lu"}, {"Lowercase_Letter", "Ll"}, {"Titlecase_Letter", "Lt"},
                 {"Modifier_Letter", "Lm"}, {"Other_Letter", "Lo"}, {"Decimal_Number", "Nd"}, {"Nonspacing_Mark", "Mn"},
                 {"Spacing_Mark", "Mc"}, {"Space_Separator", "Zs"}};
  std::string key = name;
  for (const auto &alias : aliases)
    if (name == alias.longer)
      key = alias.shorter;
  constexpr size_t categories = sizeof(kCategoryNames) / sizeof(kCategoryNames[0]);
  bool wanted[categories] = {};
  bool any = false, unassigned = false;
  if (key.size() == 1 || key.size() == 2)
    for (size_t i = 0; i < categories; ++i)
      if (std::strncmp(kCategoryNames[i], key.c_str(), key.size()) == 0)
        wanted[i] = any = true;
  if (key == "Cn" || key == "C")
    unassigned = true;
  if (key == "Cs")
    return true; // surrogates do not occur in UTF-8 text
  if (any || unassigned) {
    std::vector<R> listed;
    for (const CategoryRange &r : kCategoryRanges) {
      if (wanted[r.category])
        set->push_back({r.first, r.last});
      listed.push_back({r.first, r.last});
    }
    if (unassigned) {
      listed.push_back({0xd800, 0xdfff});
      complement(&listed);
      set->insert(set->end(), listed.begin(), listed.end());
    }
    return true;
  }
  constexpr size_t scripts = sizeof(kScriptNames) / sizeof(kScriptNames[0]);
  for (size_t i = 0; i < scripts; ++i)
    if (key == kScriptNames[i]) {
      for (const ScriptRange &r : kScriptRanges)
        if (r.script == i)
          set->push_back({r.first, r.last});
      return true;
    }
  return false;
}

void add_digits(std::vector<R> *set) { add_property("Nd", set); }

} // namespace

// ---- syntax tree ---------------------------------------------------------------------------------
struct Regex::Node {
  enum Kind { kEmpty, kChar, kSeq, kAlt, kRepeat, kLookahead, kAtomicGroup, kStart, kEnd, kTextStart, kTextEnd, kBoundary, kNotBoundary } kind = kEmpty;
  int set = -1;
  std::vector<Node> kids;
  int min = 0, max = -1, mode = 0;
  bool negate = false;

  bool nullable() const {
    switch (kind) {
    case kChar:
      return false;
    case kSeq:
      for (const Node &k : kids)
        if (!k.nullable())
          return false;
      return true;
    case kAlt:
      for (const Node &k : kids)
        if (k.nullable())
          return true;
      return false;
    case kRepeat:
      return min == 0 || kids[0].nullable();
    case kAtomicGroup:
      return kids[0].nullable();
    default:
      return true;
    }
  }
};

struct Regex::Parser {
  const std::vector<uint32_t> &p;
  size_t at = 0;
  std::vector<Set> *sets;
  std::string error;
  int depth = 0; // of nested groups

  bool done() const { return at >= p.size(); }
  uint32_t peek(size_t ahead = 0) const { return at + ahead < p.size() ? p[at + ahead] : 0; }
  bool take(uint32_t c) {
    if (!done() && p[at] == c) {
      ++at;
      return true;
    }
    return false;
  }
  bool fail(const std::string &why) {
    if (error.empty())
      error = why + " (at character " + std::to_string(at) + " of the pattern)";
    return false;
  }

  int new_set(std::vector<R> ranges, bool negated, bool fold) {
    if (fold) {
      std::vector<R> extra;
      for (const R &r : ranges) {
        if (r.last > 0x7f)
          return fail("case-insensitive matching of non-ASCII characters is not supported"), -1;
        for (uint32_t c = r.first; c <= r.last; ++c) {
          if (c >= 'a' && c <= 'z')
            extra.push_back({c - 32, c - 32});
          if (c >= 'A' && c <= 'Z')
            extra.push_back({c + 32, c + 32});
          if (c == 's' || c == 'S')
            extra.push_back({0x17f, 0x17f}); // LATIN SMALL LETTER LONG S folds to s
          if (c == 'k' || c == 'K')
            extra.push_back({0x212a, 0x212a}); // KELVIN SIGN folds to k
        }
      }
      ranges.insert(ranges.end(), extra.begin(), extra.end());
    }
    if (negated)
      complement(&ranges);
    else
      normalise(&ranges);
    Set set;
    for (const R &r : ranges)
      set.push_back({r.first, r.last});
    sets->push_back(set);
    return static_cast<int>(sets->size()) - 1;
  }

  bool hex(int digits, uint32_t *value) {
    *value = 0;
    for (int i = 0; i < digits; ++i) {
      const uint32_t c = peek();
      int v = c >= '0' && c <= '9' ? int(c - '0') : c >= 'a' && c <= 'f' ? int(c - 'a' + 10) : c >= 'A' && c <= 'F' ? int(c - 'A' + 10) : -1;
      if (v < 0)
        return fail("malformed hexadecimal escape");
      *value = *value * 16 + static_cast<uint32_t>(v);
      ++at;
    }
    return true;
  }

  // After a backslash.  Either a single character (*single) or a class added to `ranges`.
  bool escape(std::vector<R> *ranges, bool *is_single, uint32_t *single, bool in_class) {
    if (done())
      return fail("pattern ends in a backslash");
    const uint32_t c = p[at++];
    *is_single = false;
    std::vector<R> cls;
    switch (c) {
    case 'r': *is_single = true, *single = '\r'; return true;
    case 'n': *is_single = true, *single = '\n'; return true;
    case 't': *is_single = true, *single = '\t'; return true;
    case 'f': *is_single = true, *single = '\f'; return true;
    case 'v': *is_single = true, *single = '\v'; return true;
    case '0': *is_single = true, *single = 0; return true;
    case 's': add_table(kSpaceRanges, ranges); return true;
    case 'S': add_table(kSpaceRanges, &cls); complement(&cls); ranges->insert(ranges->end(), cls.begin(), cls.end()); return true;
    case 'd': add_digits(ranges); return true;
    case 'D': add_digits(&cls); complement(&cls); ranges->insert(ranges->end(), cls.begin(), cls.end()); return true;
    case 'w':
    case 'W': // the engine this follows has a slightly smaller \w inside brackets
      if (in_class)
        add_table(kWordClassRanges, &cls);
      else
        add_table(kWordRanges, &cls);
      if (c == 'W')
        complement(&cls);
      ranges->insert(ranges->end(), cls.begin(), cls.end());
      return true;
    case 'p':
    case 'P': {
      std::string name;
      bool inverted = c == 'P';
      if (take('{')) {
        if (take('^'))
          inverted = !inverted;
        while (!done() && peek() != '}')
          name += static_cast<char>(p[at++] < 0x80 ? p[at - 1] : '?');
        if (!take('}'))
          return fail("unterminated \\p{");
      } else if (!done()) {
        name = static_cast<char>(p[at++]);
      }
      if (!add_property(name, &cls))
        return fail("unknown property \\p{" + name + "}");
      if (inverted)
        complement(&cls);
      ranges->insert(ranges->end(), cls.begin(), cls.end());
      return true;
    }
    case 'x':
      *is_single = true;
      if (take('{')) {
        *single = 0;
        int digits = 0;
        while (!done() && peek() != '}' && digits < 8) {
          uint32_t v;
          if (!hex(1, &v))
            return false;
          *single = *single * 16 + v;
          ++digits;
        }
        if (!take('}') || *single > kMaxPoint)
          return fail("malformed \\x{ } escape");
        return true;
      }
      return hex(2, single);
    case 'u':
      *is_single = true;
      return hex(4, single);
    default:
      break;
    }
    if ((c >= '1' && c <= '9') || c == 'k' || c == 'g')
      return fail("back-references are not supported");
    if ((c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z'))
      return fail(std::string("the escape \\") + static_cast<char>(c) + (in_class ? " is not supported in a class" : " is not supported"));
    *is_single = true, *single = c; // an escaped punctuation character
    return true;
  }

  bool char_class(bool fold, Node *out) {
    const bool negated = take('^');
    std::vector<R> ranges;
    bool first = true;
    while (true) {
      if (done())
        return fail("unterminated character class");
      uint32_t c = p[at];
      if (c == ']' && !first) {
        ++at;
        break;
      }
      first = false;
      if (c == '[' )
        return fail("nested classes and POSIX brackets are not supported");
      if (c == '&' && peek(1) == '&')
        return fail("class intersections are not supported");
      ++at;
      bool is_single = true;
      uint32_t low = c;
      if (c == '\\') {
        if (!escape(&ranges, &is_single, &low, true))
          return false;
        if (!is_single)
          continue;
      }
      if (peek() == '-' && peek(1) != ']' && at + 1 < p.size()) {
        ++at; // the dash
        uint32_t high = p[at++];
        if (high == '\\') {
          bool high_single = true;
          std::vector<R> ignored;
          if (!escape(&ignored, &high_single, &high, true))
            return false;
          if (!high_single)
            return fail("a class cannot end a range");
        }
        if (high < low)
          return fail("range out of order in a character class");
        ranges.push_back({low, high});
      } else {
        ranges.push_back({low, low});
      }
    }
    out->kind = Node::kChar;
    out->set = new_set(ranges, negated, fold);
    return out->set >= 0;
  }

  bool quantifier(Node *atom) {
    int min = 0, max = -1;
    bool braces = false, exact = false;
    if (take('?'))
      min = 0, max = 1;
    else if (take('*'))
      min = 0, max = -1;
    else if (take('+'))
      min = 1, max = -1;
    else if (peek() == '{' && peek(1) >= '0' && peek(1) <= '9') {
      ++at;
      auto number = [&](int *value) {
        *value = 0;
        int digits = 0;
        while (peek() >= '0' && peek() <= '9' && digits < 6)
          *value = *value * 10 + static_cast<int>(p[at++] - '0'), ++digits;
        return digits > 0;
      };
      if (!number(&min))
        return fail("malformed { } quantifier");
      max = min;
      braces = exact = true;
      if (take(',')) {
        exact = false;
        max = -1;
        if (peek() != '}' && !number(&max))
          return fail("malformed { } quantifier");
      }
      if (!take('}') || (max >= 0 && max < min))
        return fail("malformed { } quantifier");
    } else {
      return true; // no quantifier
    }
    int mode = 0;
    bool optional_group = false;
    if (braces) { // in this syntax X{n}? is (?:X{n})? and X{n,m}+ repeats the repetition
      if (exact && take('?'))
        optional_group = true;
      else if (take('?'))
        mode = 1;
      else if (peek() == '+')
        return fail("a + behind a { } quantifier is not supported");
    } else if (take('?')) {
      mode = 1;
    } else if (take('+')) {
      mode = 2;
    }
    if (atom->kind == Node::kStart || atom->kind == Node::kEnd || atom->kind == Node::kTextStart || atom->kind == Node::kTextEnd ||
        atom->kind == Node::kLookahead || atom->kind == Node::kBoundary || atom->kind == Node::kNotBoundary)
      return fail("a quantifier on an anchor or a look-ahead is not supported");
    if (max == -1 && atom->nullable())
      return fail("an unbounded repetition of something that can be empty is not supported");
    Node repeat;
    repeat.kind = Node::kRepeat;
    repeat.min = min, repeat.max = max, repeat.mode = mode;
    repeat.kids.push_back(*atom);
    *atom = repeat;
    if (optional_group) {
      Node outer;
      outer.kind = Node::kRepeat;
      outer.min = 0, outer.max = 1, outer.mode = 0;
      outer.kids.push_back(*atom);
      *atom = outer;
    }
    if (peek() == '?' || peek() == '*' || peek() == '+' || (peek() == '{' && peek(1) >= '0' && peek(1) <= '9'))
      return fail("a quantifier on a quantifier is not supported");
    return true;
  }

  bool atom(bool *fold, Node *out, bool *is_atom) {
    *is_atom = true;
    const uint32_t c = p[at++];
    switch (c) {
    case '(': {
      bool inner_fold = *fold;
      Node::Kind kind = Node::kSeq;
      bool negate = false;
      if (take('?')) {
        if (take(':')) {
        } else if (take('=')) {
          kind = Node::kLookahead;
        } else if (take('!')) {
          kind = Node::kLookahead, negate = true;
        } else if (take('>')) {
          kind = Node::kAtomicGroup;
        } else if (peek() == '<' || peek() == 'P' || peek() == '\'') {
          return fail("look-behind and named groups are not supported");
        } else {
          // inline flags: (?i) for the rest of the enclosing group, (?i: ... ) for a group; -i turns it off
          bool on = true, value = inner_fold, seen = false;
          while (!done() && peek() != ':' && peek() != ')') {
            const uint32_t f = p[at++];
            if (f == '-')
              on = false;
            else if (f == 'i')
              value = on, seen = true;
            else
              return fail("only the flag i is supported in (? )");
          }
          if (!seen)
            return fail("malformed (? ) group");
          if (take(')')) {
            // (?i) takes the rest of the enclosing group, its later alternatives included, as one group
            *fold = value;
            return alternation(value, out);
          }
          if (!take(':'))
            return fail("malformed (? ) group");
          inner_fold = value;
        }
      }
      Node inner;
      if (++depth > 100)
        return fail("groups nested more than 100 deep");
      if (!alternation(inner_fold, &inner))
        return false;
      --depth;
      if (!take(')'))
        return fail("missing )");
      if (kind == Node::kSeq) {
        *out = inner;
      } else {
        out->kind = kind;
        out->negate = negate;
        out->kids.push_back(inner);
      }
      return true;
    }
    case '[':
      return char_class(*fold, out);
    case '.':
      out->kind = Node::kChar;
      out->set = new_set({{'\n', '\n'}}, true, false);
      return out->set >= 0;
    case '^':
      out->kind = Node::kStart;
      return true;
    case '$':
      out->kind = Node::kEnd;
      return true;
    case '\\': {
      if (peek() == 'b' || peek() == 'B') {
        out->kind = p[at++] == 'b' ? Node::kBoundary : Node::kNotBoundary;
        return true;
      }
      if (peek() == 'A') {
        ++at, out->kind = Node::kTextStart;
        return true;
      }
      if (peek() == 'z') {
        ++at, out->kind = Node::kTextEnd;
        return true;
      }
      std::vector<R> ranges;
      bool is_single = false;
      uint32_t single = 0;
      if (!escape(&ranges, &is_single, &single, false))
        return false;
      out->kind = Node::kChar;
      if (is_single)
        out->set = new_set({{single, single}}, false, *fold);
      else
        out->set = new_set(ranges, false, false);
      return out->set >= 0;
    }
    case '*':
    case '+':
    case '?':
      return fail("a quantifier without anything to repeat");
    case ')':
      return fail("unmatched )");
    default:
      out->kind = Node::kChar;
      out->set = new_set({{c, c}}, false, *fold);
      return out->set >= 0;
    }
  }

  bool sequence(bool fold, Node *out) {
    out->kind = Node::kSeq;
    while (!done() && peek() != '|' && peek() != ')') {
      Node item;
      bool is_atom = true;
      if (!atom(&fold, &item, &is_atom))
        return false;
      if (!is_atom)
        continue;
      if (!quantifier(&item))
        return false;
      out->kids.push_back(item);
    }
    return true;
  }

  bool alternation(bool fold, Node *out) {
    Node first;
    if (!sequence(fold, &first))
      return false;
    if (peek() != '|' || done()) {
      *out = first;
      return true;
    }
    out->kind = Node::kAlt;
    out->kids.push_back(first);
    while (take('|')) {
      Node next;
      if (!sequence(fold, &next))
        return false;
      out->kids.push_back(next);
    }
    return true;
  }
};

// ---- program -------------------------------------------------------------------------------------
int Regex::emit(const Node &node, std::string *error) {
  auto add = [&](Inst inst) {
    program_.push_back(inst);
    return static_cast<int>(program_.size()) - 1;
  };
  switch (node.kind) {
  case Node::kEmpty:
    return 0;
  case Node::kChar: {
    Inst inst{kSet};
    inst.set = node.set;
    add(inst);
    return 0;
  }
  case Node::kSeq:
    for (const Node &k : node.kids)
      if (emit(k, error) < 0)
        return -1;
    return 0;
  case Node::kAlt: {
    std::vector<int> jumps;
    for (size_t i = 0; i < node.kids.size(); ++i) {
      int split = -1;
      if (i + 1 < node.kids.size())
        split = add(Inst{kSplit});
      if (split >= 0)
        program_[static_cast<size_t>(split)].x = static_cast<int>(program_.size());
      if (emit(node.kids[i], error) < 0)
        return -1;
      if (i + 1 < node.kids.size()) {
        jumps.push_back(add(Inst{kJump}));
        program_[static_cast<size_t>(split)].y = static_cast<int>(program_.size());
      }
    }
    for (int j : jumps)
      program_[static_cast<size_t>(j)].x = static_cast<int>(program_.size());
    return 0;
  }
  case Node::kRepeat: {
    const Node &body = node.kids[0];
    if (body.kind == Node::kChar) {
      Inst inst{kSpan};
      inst.set = body.set;
      inst.min = node.min, inst.max = node.max, inst.mode = node.mode;
      add(inst);
      return 0;
    }
    if (node.min > kMaxCopies || node.max > kMaxCopies) {
      *error = "a group is repeated more than " + std::to_string(kMaxCopies) + " times";
      return -1;
    }
    int atomic = -1;
    if (node.mode == 2)
      atomic = add(Inst{kAtomic});
    const bool lazy = node.mode == 1;
    for (int i = 0; i < node.min; ++i)
      if (emit(body, error) < 0)
        return -1;
    if (node.max < 0) {
      const int loop = add(Inst{kSplit});
      const int start = static_cast<int>(program_.size());
      if (emit(body, error) < 0)
        return -1;
      Inst back{kJump};
      back.x = loop;
      add(back);
      const int out = static_cast<int>(program_.size());
      program_[static_cast<size_t>(loop)].x = lazy ? out : start;
      program_[static_cast<size_t>(loop)].y = lazy ? start : out;
    } else {
      std::vector<int> splits;
      for (int i = node.min; i < node.max; ++i) {
        splits.push_back(add(Inst{kSplit}));
        const int start = static_cast<int>(program_.size());
        program_[static_cast<size_t>(splits.back())].x = start; // patched below for lazy
        if (emit(body, error) < 0)
          return -1;
      }
      const int out = static_cast<int>(program_.size());
      for (int s : splits) {
        Inst &split = program_[static_cast<size_t>(s)];
        const int start = split.x;
        split.x = lazy ? out : start;
        split.y = lazy ? start : out;
      }
    }
    if (atomic >= 0) {
      add(Inst{kMatch});
      program_[static_cast<size_t>(atomic)].y = static_cast<int>(program_.size());
    }
    return 0;
  }
  case Node::kLookahead:
  case Node::kAtomicGroup: {
    Inst inst{node.kind == Node::kLookahead ? kLook : kAtomic};
    inst.negate = node.negate;
    const int at = add(inst);
    if (emit(node.kids[0], error) < 0)
      return -1;
    add(Inst{kMatch});
    program_[static_cast<size_t>(at)].y = static_cast<int>(program_.size());
    return 0;
  }
  case Node::kStart:
    add(Inst{kBol});
    return 0;
  case Node::kEnd:
    add(Inst{kEol});
    return 0;
  case Node::kTextStart:
    add(Inst{kTextBegin});
    return 0;
  case Node::kTextEnd:
    add(Inst{kTextFinish});
    return 0;
  case Node::kBoundary:
    add(Inst{kWordBoundary});
    return 0;
  case Node::kNotBoundary:
    add(Inst{kNotWordBoundary});
    return 0;
  }
  return 0;
}

std::string Regex::compile(const std::string &pattern) {
  sets_.clear();
  program_.clear();
  std::vector<uint32_t> points;
  std::vector<size_t> offsets;
  utf8_points(pattern, &points, &offsets);
  Parser parser{points, 0, &sets_, "", 0};
  Node root;
  if (!parser.alternation(false, &root))
    return "regular expression: " + parser.error;
  if (!parser.done())
    return "regular expression: unmatched ) (at character " + std::to_string(parser.at) + " of the pattern)";
  std::string error;
  if (emit(root, &error) < 0)
    return "regular expression: " + error;
  program_.push_back(Inst{kMatch});
  return "";
}

bool Regex::in_set(const Set &set, uint32_t cp) {
  size_t lo = 0, hi = set.size();
  while (lo < hi) {
    const size_t mid = (lo + hi) / 2;
    if (cp < set[mid].first)
      hi = mid;
    else if (cp > set[mid].last)
      lo = mid + 1;
    else
      return true;
  }
  return false;
}

// Runs the program from pc at pos; the end of the first match in backtracking order, or npos.
size_t Regex::run(int pc, size_t pos, const std::vector<uint32_t> &text, int64_t *budget) const {
  constexpr size_t npos = static_cast<size_t>(-1);
  struct Entry {
    int pc, kind; // kind 0: resume at (pc, pos); 1: greedy span gives one back; 2: lazy span takes one more
    size_t pos, bound;
  };
  std::vector<Entry> stack;
  const size_t n = text.size();
  auto is_word = [&](size_t i) {
    if (i >= n)
      return false;
    static const Set word = [] {
      Set s;
      for (const CodeRange &r : kWordRanges)
        s.push_back({r.first, r.last});
      return s;
    }();
    return in_set(word, text[i]);
  };
  while (true) {
    bool failed = false;
    while (!failed) {
      if (--*budget < 0)
        return npos;
      const Inst &inst = program_[static_cast<size_t>(pc)];
      switch (inst.op) {
      case kSet:
        if (pos < n && in_set(sets_[static_cast<size_t>(inst.set)], text[pos]))
          ++pc, ++pos;
        else
          failed = true;
        break;
      case kSpan: {
        const Set &set = sets_[static_cast<size_t>(inst.set)];
        const size_t most = inst.max < 0 ? n : std::min(n, pos + static_cast<size_t>(inst.max));
        size_t end = pos;
        const size_t least = pos + static_cast<size_t>(inst.min);
        if (inst.mode == 1) { // lazy: the fewest first
          while (end < least && end < n && in_set(set, text[end]))
            ++end;
          if (end < least) {
            failed = true;
            break;
          }
          if (end < most)
            stack.push_back({pc, 2, end, most});
        } else {
          while (end < most && in_set(set, text[end]))
            ++end;
          *budget -= static_cast<int64_t>(end - pos);
          if (end < least) {
            failed = true;
            break;
          }
          if (inst.mode == 0 && end > least)
            stack.push_back({pc, 1, end - 1, least});
        }
        pos = end;
        ++pc;
        break;
      }
      case kSplit:
        stack.push_back({inst.y, 0, pos, 0});
        pc = inst.x;
        break;
      case kJump:
        pc = inst.x;
        break;
      case kMatch:
        return pos;
      case kLook: {
        const size_t end = run(pc + 1, pos, text, budget);
        if (*budget < 0)
          return npos;
        if ((end != npos) != inst.negate)
          pc = inst.y;
        else
          failed = true;
        break;
      }
      case kAtomic: {
        const size_t end = run(pc + 1, pos, text, budget);
        if (*budget < 0)
          return npos;
        if (end != npos)
          pos = end, pc = inst.y;
        else
          failed = true;
        break;
      }
      case kBol: // ^ and $ are line anchors in the syntax the tokenizers' engine reads
        if (pos == 0 || (text[pos - 1] == '\n' && pos < n)) // not behind a newline that ends the text
          ++pc;
        else
          failed = true;
        break;
      case kEol:
        if (pos == n || text[pos] == '\n')
          ++pc;
        else
          failed = true;
        break;
      case kTextBegin:
        if (pos == 0)
          ++pc;
        else
          failed = true;
        break;
      case kTextFinish:
        if (pos == n)
          ++pc;
        else
          failed = true;
        break;
      case kWordBoundary:
      case kNotWordBoundary: {
        const bool boundary = (pos > 0 && is_word(pos - 1)) != is_word(pos);
        if (boundary == (inst.op == kWordBoundary))
          ++pc;
        else
          failed = true;
        break;
      }
      }
    }
    // backtrack
    if (stack.empty())
      return npos;
    Entry e = stack.back();
    stack.pop_back();
    if (e.kind == 0) {
      pc = e.pc, pos = e.pos;
    } else if (e.kind == 1) {
      if (e.pos > e.bound)
        stack.push_back({e.pc, 1, e.pos - 1, e.bound});
      pc = e.pc + 1, pos = e.pos;
    } else {
      const Inst &inst = program_[static_cast<size_t>(e.pc)];
      if (e.pos < e.bound && in_set(sets_[static_cast<size_t>(inst.set)], text[e.pos])) {
        if (e.pos + 1 < e.bound)
          stack.push_back({e.pc, 2, e.pos + 1, e.bound});
        pc = e.pc + 1, pos = e.pos + 1;
      } else {
        continue; // nothing more to take: keep backtracking
      }
    }
  }
}

int Regex::search(const std::vector<uint32_t> &text, size_t from, size_t *begin, size_t *end) const {
  int64_t budget = kStepBudget;
  for (size_t start = from; start <= text.size(); ++start) {
    const size_t stop = run(0, start, text, &budget);
    if (budget < 0)
      return -1;
    if (stop != static_cast<size_t>(-1)) {
      *begin = start, *end = stop;
      return 1;
    }
  }
  return 0;
}

std::string parse_split_behavior(const std::string &name, SplitBehavior *behavior) {
  std::string key;
  for (char c : name)
    if (c != '_')
      key += static_cast<char>(c >= 'A' && c <= 'Z' ? c + 32 : c);
  if (key == "removed")
    *behavior = SplitBehavior::kRemoved;
  else if (key == "isolated")
    *behavior = SplitBehavior::kIsolated;
  else if (key == "mergedwithprevious")
    *behavior = SplitBehavior::kMergedWithPrevious;
  else if (key == "mergedwithnext")
    *behavior = SplitBehavior::kMergedWithNext;
  else if (key == "contiguous")
    *behavior = SplitBehavior::kContiguous;
  else
    return "unknown split behaviour '" + name + "'";
  return "";
}

std::string regex_split(const Regex &regex, const std::string &text, SplitBehavior behavior, bool invert,
                        std::vector<std::string> *pieces) {
  std::vector<uint32_t> points;
  std::vector<size_t> offsets;
  utf8_points(text, &points, &offsets);
  struct Span {
    size_t begin, end; // code points
    bool match;
  };
  std::vector<Span> spans; // matches and the gaps between them, in order, covering the text
  size_t at = 0;
  while (at <= points.size()) {
    size_t begin = 0, end = 0;
    const int found = regex.search(points, at, &begin, &end);
    if (found < 0)
      return "regular expression: step budget exhausted";
    if (found == 0)
      break;
    if (end == begin)
      return "regular expression: the pattern matched the empty string";
    if (begin > at)
      spans.push_back({at, begin, invert});
    spans.push_back({begin, end, !invert});
    at = end;
  }
  if (at < points.size())
    spans.push_back({at, points.size(), invert});
  // SplitDelimiterBehavior of the tokenizers library (NormalizedString::split)
  std::vector<Span> out;
  switch (behavior) {
  case SplitBehavior::kRemoved:
    for (const Span &s : spans)
      if (!s.match)
        out.push_back(s);
    break;
  case SplitBehavior::kIsolated:
    out = spans;
    break;
  case SplitBehavior::kContiguous: {
    bool previous = false;
    for (const Span &s : spans) {
      if (s.match == previous && !out.empty())
        out.back().end = s.end;
      else
        out.push_back(s);
      previous = s.match;
    }
    break;
  }
  case SplitBehavior::kMergedWithPrevious: {
    bool previous = false;
    for (const Span &s : spans) {
      if (s.match && !previous && !out.empty())
        out.back().end = s.end;
      else
        out.push_back(s);
      previous = s.match;
    }
    break;
  }
  case SplitBehavior::kMergedWithNext: {
    bool previous = false;
    for (size_t i = spans.size(); i-- > 0;) {
      const Span &s = spans[i];
      if (s.match && !previous && !out.empty())
        out.back().begin = s.begin;
      else
        out.push_back(s);
      previous = s.match;
    }
    std::reverse(out.begin(), out.end());
    break;
  }
  }
  for (const Span &s : out)
    if (s.end > s.begin)
      pieces->emplace_back(text, offsets[s.begin], offsets[s.end] - offsets[s.begin]);
  return "";
}

} // namespace detail
} // namespace llmcp_b200
