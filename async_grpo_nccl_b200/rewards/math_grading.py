"""Math answer grading: ``\\boxed{}`` extraction, MATH-style string normalisation and a sympy
equivalence check with guards against pathological inputs.

It covers the role of the reference's vendored deepscaler_math_utils.py (extract_answer :478,
grade_answer_mathd :469, grade_answer_sympy :430): the "mathd" grader compares normalised strings, the
"sympy" grader additionally accepts answers whose difference simplifies to zero, handling tuples /
intervals element-wise.
"""
from __future__ import annotations

import re
from typing import List, Optional

_BAD_SUBSTRINGS = ("^{", "^(")
_BAD_REGEXES = (r"\^[0-9]+\^", r"\^[0-9][0-9]+")
_UNITS = ("degree", "cm", "centimeter", "meter", "mile", "second", "minute", "hour", "day", "week", "month", "year",
          "foot", "feet", "inch", "yard", "unit", "dollar", "cent", "mph", "km", "kg", "gram", "liter", "point")


def last_boxed_only_string(text: str) -> Optional[str]:
    idx = max(text.rfind("\\boxed"), text.rfind("\\fbox"))
    if idx < 0:
        return None
    depth = 0
    start = text.find("{", idx)
    if start < 0:
        # "\boxed 5" form
        m = re.match(r"\\boxed\s+([^\s$]+)", text[idx:])
        return "\\boxed{" + m.group(1) + "}" if m else None
    for j in range(start, len(text)):
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            depth -= 1
            if depth == 0:
                return text[idx:j + 1]
    return None


def remove_boxed(s: Optional[str]) -> Optional[str]:
    if s is None:
        return None
    m = re.match(r"\\(?:boxed|fbox)\{(.*)\}$", s, re.DOTALL)
    return m.group(1) if m else None


def extract_answer(text: str) -> Optional[str]:
    """Content of the last \\boxed{...} in ``text`` (None when there is none)."""
    return remove_boxed(last_boxed_only_string(text))


def _fix_fracs(s: str) -> str:
    # \frac12 -> \frac{1}{2}, \frac1{2} -> \frac{1}{2}
    out = []
    parts = s.split("\\frac")
    out.append(parts[0])
    for p in parts[1:]:
        out.append("\\frac")
        if p.startswith("{"):
            out.append(p)
            continue
        if len(p) < 2:
            return s
        a, rest = p[0], p[1:]
        if rest.startswith("{"):
            out.append("{" + a + "}" + rest)
        else:
            out.append("{" + a + "}{" + rest[0] + "}" + rest[1:])
    return "".join(out)


def _fix_a_slash_b(s: str) -> str:
    m = re.fullmatch(r"(-?\d+)/(\d+)", s)
    return f"\\frac{{{m.group(1)}}}{{{m.group(2)}}}" if m else s


def _fix_sqrt(s: str) -> str:
    return re.sub(r"\\sqrt(\w)", r"\\sqrt{\1}", s)


def _drop_units(text: str) -> str:
    out = text
    for u in _UNITS:
        out = re.sub(rf"\b{u}(es|s)?\b", "", out, flags=re.IGNORECASE)
    return out.strip()


def strip_string(s: str) -> str:
    s = str(s).replace("\n", "").replace("\\!", "")
    s = s.replace("\\\\", "\\").replace("tfrac", "frac").replace("dfrac", "frac")
    s = s.replace("\\left", "").replace("\\right", "")
    s = s.replace("^{\\circ}", "").replace("^\\circ", "")
    s = s.replace("\\$", "").replace("$", "")
    s = re.sub(r"\\text\{\s*([^}]*)\}", lambda m: _drop_units(m.group(1)), s)
    s = s.replace("\\%", "").replace("%", "")
    s = s.replace(" .", " 0.").replace("{.", "{0.")
    if not s:
        return s
    if s[0] == ".":
        s = "0" + s
    if len(s.split("=")) == 2 and len(s.split("=")[0]) <= 2:
        s = s.split("=")[1]
    s = _fix_sqrt(s)
    s = s.replace(" ", "")
    s = _fix_fracs(s)
    if s == "0.5":
        s = "\\frac{1}{2}"
    s = _fix_a_slash_b(s)
    return s.rstrip(".")


def grade_answer_mathd(given: Optional[str], truth: Optional[str]) -> bool:
    if given is None or truth is None:
        return False
    try:
        return strip_string(given) == strip_string(truth)
    except Exception:
        return given == truth


# ---- sympy path -----------------------------------------------------------------------------------
def _latex_to_plain(s: str) -> str:
    s = s.replace("\\cdot", "*").replace("\\times", "*").replace("\\div", "/").replace("\\pi", "pi")
    for _ in range(8):
        new = re.sub(r"\\frac\{([^{}]*)\}\{([^{}]*)\}", r"((\1)/(\2))", s)
        new = re.sub(r"\\sqrt\{([^{}]*)\}", r"sqrt(\1)", new)
        if new == s:
            break
        s = new
    s = s.replace("{", "(").replace("}", ")").replace("^", "**").replace("\\", "")
    s = re.sub(r"(\d)\s*\(", r"\1*(", s)
    s = re.sub(r"\)\s*\(", r")*(", s)
    s = re.sub(r"(\d)([a-zA-Z])", r"\1*\2", s)
    return s


def normalize_for_sympy(expr: Optional[str]) -> Optional[str]:
    if expr is None:
        return None
    s = expr.strip().replace("\\dfrac", "\\frac").replace("\\tfrac", "\\frac").replace("\\left", "").replace("\\right", "")
    s = _fix_fracs(s.replace("\\!", ""))
    m = re.search(r"^\\text\{(?P<t>.+?)\}$", s)
    if m:
        s = m.group("t")
    s = s.replace("\\%", "%").replace("\\$", "$").replace("$", "").replace("%", "")
    s = s.replace(" or ", " , ").replace(" and ", " , ")
    for word, mult in (("million", "*10^6"), ("billion", "*10^9"), ("trillion", "*10^12")):
        s = s.replace(word, mult)
    for u in _UNITS:
        s = re.sub(rf"{u}(es)?(s)? *(\^[0-9]+)?", "", s)
    s = re.sub(r"\^ *\\circ", "", s)
    if s and s[0] == "{" and s[-1] == "}":
        s = s[1:-1]
    s = re.sub(r",\\! *", "", s)
    try:
        f = float(s.replace(",", ""))
        if abs(f - round(f)) <= 1e-7:
            s = str(int(round(f)))
    except ValueError:
        pass
    s = s.replace("- ", "-")
    return s.replace(" ", "").lower() if "\\" not in s else s.replace(" ", "")


def _should_allow_eval(expr: str) -> bool:
    if len(set(c for c in expr.replace("sqrt", "").replace("pi", "") if c.isalpha())) > 2:
        return False
    if any(b in expr for b in _BAD_SUBSTRINGS):
        return False
    return not any(re.search(r, expr) for r in _BAD_REGEXES)


def _sympy_equal(a: str, b: str) -> bool:
    import sympy
    from sympy.parsing.sympy_parser import parse_expr

    try:
        expr = f"({_latex_to_plain(a)})-({_latex_to_plain(b)})"
        if not _should_allow_eval(expr):
            return False
        return sympy.simplify(parse_expr(expr, evaluate=True)) == 0
    except Exception:
        return False


def _split_tuple(s: str) -> List[str]:
    s = s.strip()
    if len(s) > 2 and s[0] in "([" and s[-1] in ")]" and all(ch not in s[1:-1] for ch in "()[]"):
        return [x.strip() for x in s[1:-1].split(",")]
    return [s]


def grade_answer_sympy(given: Optional[str], truth: Optional[str]) -> bool:
    t = normalize_for_sympy(truth)
    g = normalize_for_sympy(given)
    if t is None or g is None or len(g) == 0:
        return False
    if g == t:
        return True
    te, ge = _split_tuple(t), _split_tuple(g)
    if len(te) > 1 and (t[0] != g[0] or t[-1] != g[-1]):
        return False
    if len(te) != len(ge):
        return False
    for a, b in zip(te, ge):
        if a == b:
            continue
        # fractions must match in reduced form; integers must match exactly
        is_int = lambda x: re.fullmatch(r"-?\d+", x) is not None
        if is_int(a) or is_int(b):
            if is_int(a) and is_int(b):
                return False
        if not _sympy_equal(a, b):
            return False
    return True


def grade_answer(given: Optional[str], truth: Optional[str]) -> bool:
    """String grader first, sympy grader second (the reference's grade_answer_verl :483 ordering)."""
    return grade_answer_mathd(given, truth) or grade_answer_sympy(given, truth)
