"""Writes llmcp_b200/csrc/unicode_tables.h: the code-point ranges of the Unicode general categories
L (letters) and N (numbers) that the tokenizer's pre-tokenisation pattern names (\\p{L}, \\p{N}),
as the regular-expression engine inside the Hugging Face `tokenizers` package classifies them (the
engine the reference's tokenizer runs the pattern on, so a code point assigned in a recent Unicode
version is split the way that package splits it); without the package, from this interpreter's
`unicodedata`.  Run it again to move to a newer Unicode version:

    python llmcp_b200/csrc/tools/make_unicode_tables.py
"""
import pathlib
import sys
import unicodedata


def engine_ranges(prefix):
    """Ranges of \\p{prefix} according to the tokenizers package: everything its Split removes."""
    from tokenizers import Regex, pre_tokenizers

    points = [cp for cp in range(sys.maxunicode + 1) if not 0xD800 <= cp <= 0xDFFF]
    text = "".join(map(chr, points))
    split = pre_tokenizers.Split(Regex("\\p{%s}+" % prefix), behavior="removed", invert=False)
    kept = [span for _, span in split.pre_tokenize_str(text)]  # character offsets of what is NOT in the class
    out, at = [], 0
    for start, end in kept + [(len(points), len(points))]:
        if start > at:
            out.append((points[at], points[start - 1]))
        at = end
    return out


CATEGORIES = "Lu Ll Lt Lm Lo Mn Mc Me Nd Nl No Pc Pd Ps Pe Pi Pf Po Sm Sc Sk So Zs Zl Zp Cc Cf Co".split()  # Cn, Cs: the rest
SCRIPTS = "Han Hiragana Katakana Hangul Latin Cyrillic Greek Arabic Hebrew Thai Devanagari".split()


def engine_class_ranges(pattern):
    """Ranges of a one-character pattern (\\w, \\p{Han}, ...) according to the tokenizers package."""
    from tokenizers import Regex, pre_tokenizers

    points = [cp for cp in range(sys.maxunicode + 1) if not 0xD800 <= cp <= 0xDFFF]
    text = "".join(map(chr, points))
    split = pre_tokenizers.Split(Regex("(?:%s)+" % pattern), behavior="removed", invert=False)
    kept = [span for _, span in split.pre_tokenize_str(text)]
    out, at = [], 0
    for start, end in kept + [(len(points), len(points))]:
        if start > at:
            out.append((points[at], points[start - 1]))
        at = end
    return out


def category_rows():
    """(first, last, index into CATEGORIES) over all code points that have one of those categories."""
    try:
        import tokenizers  # noqa: F401

        found = [(a, b, i) for i, name in enumerate(CATEGORIES) for a, b in engine_class_ranges("\\p{%s}" % name)]
    except ImportError:
        found = [(a, b, i) for i, name in enumerate(CATEGORIES) for a, b in unicodedata_ranges(name)]
    return sorted(found)


def class_ranges(pattern, fallback):
    try:
        import tokenizers  # noqa: F401

        return engine_class_ranges(pattern)
    except ImportError:
        return fallback()


def unicodedata_ranges(prefix):
    out, start = [], None
    for cp in range(sys.maxunicode + 1):
        inside = unicodedata.category(chr(cp)).startswith(prefix)
        if inside and start is None:
            start = cp
        elif not inside and start is not None:
            out.append((start, cp - 1))
            start = None
    if start is not None:
        out.append((start, sys.maxunicode))
    return out


def ranges(prefix):
    try:
        import tokenizers

        return engine_ranges(prefix), f"the regular-expression engine of tokenizers {tokenizers.__version__}"
    except ImportError:
        return unicodedata_ranges(prefix), f"Unicode {unicodedata.unidata_version}"


def package_normalizers():
    """(NFD, NFC) of the `tokenizers` package, or None.  Its normalisation tables are older than this
    interpreter's (combining marks added since Unicode 10 are starters to it), and the encoder has to
    normalise as that package does, so the tables below keep only what the package knows."""
    try:
        from tokenizers import normalizers

        return normalizers.NFD().normalize_str, normalizers.NFC().normalize_str
    except ImportError:
        return None


def combining_classes():
    """(first, last, canonical combining class) for every run of code points with a non-zero class."""
    package = package_normalizers()
    out = []
    for cp in range(sys.maxunicode + 1):
        c = chr(cp)
        cc = unicodedata.combining(c)
        if cc and cc < 240 and package:  # known to the package: it moves the mark in front of U+0345 (class 240)
            nfd = package[0]
            if nfd("a\u0345" + c) != "a" + nfd(c) + "\u0345":
                cc = 0
        if cc:
            if out and out[-1][1] == cp - 1 and out[-1][2] == cc:
                out[-1][1] = cp
            else:
                out.append([cp, cp, cc])
    return out


def decompositions():
    """(code point, first, second or 0, 1 if NFC composes the pair back) for every canonical
    decomposition mapping (one level; Hangul syllables are algorithmic and not listed)."""
    package = package_normalizers()
    out = []
    for cp in range(sys.maxunicode + 1):
        parts = unicodedata.decomposition(chr(cp)).split()
        if not parts or parts[0].startswith("<"):
            continue
        a, b = int(parts[0], 16), int(parts[1], 16) if len(parts) == 2 else 0
        if package and package[0](chr(cp)) == chr(cp):
            continue  # the package leaves it alone
        nfc = package[1] if package else (lambda t: unicodedata.normalize("NFC", t))
        composes = int(b != 0 and nfc(chr(a) + chr(b)) == chr(cp))
        out.append((cp, a, b, composes))
    return out


def rows(name, kind, items, fmt):
    lines = [f"constexpr {kind} {name}[] = {{"]
    row = "   "
    for item in items:
        cell = " " + fmt(item) + ","
        if len(row) + len(cell) > 118:
            lines.append(row)
            row = "   "
        row += cell
    lines.append(row)
    lines.append("};")
    return "\n".join(lines)


def table(name, items):
    lines = [f"constexpr CodeRange {name}[] = {{"]
    row = "   "
    for a, b in items:
        cell = f" {{0x{a:X}, 0x{b:X}}},"
        if len(row) + len(cell) > 118:
            lines.append(row)
            row = "   "
        row += cell
    lines.append(row)
    lines.append("};")
    return "\n".join(lines)


def main():
    target = pathlib.Path(__file__).resolve().parents[1] / "unicode_tables.h"
    (letters, source), (numbers, _) = ranges("L"), ranges("N")
    text = f"""// Code-point ranges of the Unicode general categories L and N ({source}).
// Generated by tools/make_unicode_tables.py; do not edit by hand.
#pragma once

#include <cstdint>

namespace llmcp_b200 {{
namespace detail {{

struct CodeRange {{
  uint32_t first, last;
}};

{table("kLetterRanges", letters)}

{table("kNumberRanges", numbers)}

// General category of every assigned code point (what is not listed is Cn, or a surrogate), for
// the \\p{{..}} classes of a tokenizer's pre-tokenisation patterns.  Sorted by first code point.
constexpr const char *kCategoryNames[] = {{{", ".join('"%s"' % c for c in CATEGORIES)}}};

struct CategoryRange {{
  uint32_t first, last, category; // index into kCategoryNames
}};

{rows("kCategoryRanges", "CategoryRange", category_rows(), lambda r: "{0x%X, 0x%X, %d}" % r)}

// \\w and \\s of that engine; \\w inside a bracketed class is a slightly smaller set there.
{table("kWordRanges", class_ranges("\\w", lambda: []))}

{table("kWordClassRanges", class_ranges("[\\w]", lambda: []))}

{table("kSpaceRanges", class_ranges("\\s", lambda: []))}

// Scripts that pre-tokenisation patterns name.
constexpr const char *kScriptNames[] = {{{", ".join('"%s"' % c for c in SCRIPTS)}}};

struct ScriptRange {{
  uint32_t first, last, script; // index into kScriptNames
}};

{rows("kScriptRanges", "ScriptRange", sorted((a, b, i) for i, name in enumerate(SCRIPTS) for a, b in class_ranges("\\p{%s}" % name, lambda: [])), lambda r: "{0x%X, 0x%X, %d}" % r)}

// Normalisation data: Unicode {unicodedata.unidata_version} (this interpreter's `unicodedata`), less what the NFC
// normaliser of {source.split(" of ")[-1]} does not know (it treats those code points as inert).
struct CombiningClass {{
  uint32_t first, last, value;
}};

{rows("kCombiningClasses", "CombiningClass", combining_classes(), lambda r: "{0x%X, 0x%X, %d}" % tuple(r))}

// One level of canonical decomposition: code point -> first, second (0: none); composes = 1 where
// NFC puts the pair together again (no composition exclusion).  Sorted by code point.
struct Decomposition {{
  uint32_t point, first, second, composes;
}};

{rows("kDecompositions", "Decomposition", decompositions(), lambda r: "{0x%X, 0x%X, 0x%X, %d}" % r)}

}} // namespace detail
}} // namespace llmcp_b200
"""
    target.write_text(text)
    print(target, len(text), "bytes")


if __name__ == "__main__":
    main()
