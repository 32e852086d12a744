"""Answer extraction and grading for MATH / AIME style problems.

Two graders, as in tunix/utils/math_utils.py: a string grader after the MATH dataset's answer
normalisation (`grade_answer_mathd`) and a symbolic grader (`grade_answer_sympy`) that accepts
answers sympy proves equal (fractions vs decimals, reordered sums, tuples and intervals
element by element). `grade_answer_special_handling` covers recurring decimals, unions of
intervals and malformed `\\sqrt` that neither grader parses. `extract_answer` returns the
content of the last `\\boxed{...}` of a solution.
"""
from __future__ import annotations

import re
from typing import List, Optional

try:
  import sympy
  from sympy.parsing import sympy_parser
except ImportError:   # pragma: no cover - sympy ships with torch
  sympy = None

BAD_SUBSTRINGS = ["^{", "^("]
BAD_REGEXES = [r"\^[0-9]+\^", r"\^[0-9][0-9]+"]
TUPLE_CHARS = "()[]"
_UNIT_WORDS = ["degree", "cm", "centimeter", "meter", "mile", "second", "minute", "hour", "day", "week", "month",
               "year", "foot", "feet", "inch", "yard", "unit", "square", "cent", "dollar", "point", "percent"]


# ---------------------------------------------------------------------------------------------
# boxed answers
# ---------------------------------------------------------------------------------------------
def last_boxed_only_string(string: str) -> Optional[str]:
  """The last `\\boxed{...}` / `\\fbox{...}` (braces balanced) or `\\boxed x` of `string`."""
  idx = string.rfind("\\boxed")
  if idx < 0:
    idx = string.rfind("\\fbox")
    if idx < 0:
      return None
  if string[idx:].startswith("\\boxed "):
    return "\\boxed " + string[idx + len("\\boxed "):].split("$")[0]
  depth = 0
  for i in range(idx, len(string)):
    if string[i] == "{":
      depth += 1
    elif string[i] == "}":
      depth -= 1
      if depth == 0:
        return string[idx:i + 1]
  return None


def remove_boxed(s: Optional[str]) -> Optional[str]:
  if s is None:
    return None
  for left in ("\\boxed ", "\\boxed{", "\\fbox{"):
    if s.startswith(left):
      body = s[len(left):]
      if left.endswith("{"):
        if not body.endswith("}"):
          return None
        body = body[:-1]
      return body
  return None


def extract_boxed_answer(solution: str) -> Optional[str]:
  return remove_boxed(last_boxed_only_string(solution))


def extract_answer(passage: str) -> Optional[str]:
  if "\\boxed" in passage or "\\fbox" in passage:
    return extract_boxed_answer(passage)
  return None


# ---------------------------------------------------------------------------------------------
# MATH-dataset string normalisation
# ---------------------------------------------------------------------------------------------
def _fix_fracs(s: str) -> str:
  """\\frac12 -> \\frac{1}{2}, \\frac1{72} -> \\frac{1}{72}."""
  parts = s.split("\\frac")
  out = parts[0]
  for p in parts[1:]:
    out += "\\frac"
    if p.startswith("{") or len(p) < 2:
      out += p
      continue
    a, b, rest = p[0], p[1], p[2:]
    out += "{" + a + "}" + (b + rest if b == "{" else "{" + b + "}" + rest)
  return out


def _fix_a_slash_b(s: str) -> str:
  m = re.fullmatch(r"(-?\d+)/(-?\d+)", s)
  return f"\\frac{{{m.group(1)}}}{{{m.group(2)}}}" if m else s


def _fix_sqrt(s: str) -> str:
  return re.sub(r"\\sqrt(\w)", r"\\sqrt{\1}", s)


def _remove_right_units(s: str) -> str:
  if "\\text{ " in s:
    head = s.split("\\text{ ")
    if len(head) == 2:
      return head[0]
  return s


def _strip_string(s: str) -> str:
  s = str(s).replace("\n", "").replace("\\!", "")
  s = s.replace("\\\\", "\\").replace("tfrac", "frac").replace("dfrac", "frac")
  s = s.replace("\\left", "").replace("\\right", "")
  s = s.replace("^{\\circ}", "").replace("^\\circ", "").replace("\\$", "")
  s = _remove_right_units(s)
  s = s.replace("\\%", "").replace("%", "")
  s = s.replace(" .", " 0.").replace("{.", "{0.")
  if not s:
    return s
  if s[0] == ".":
    s = "0" + s
  if len(s.split("=")) == 2 and len(s.split("=")[0]) <= 2:   # "k = 5" -> "5"
    s = s.split("=")[1]
  s = _fix_sqrt(s).replace(" ", "")
  s = _fix_fracs(s)
  if s == "0.5":
    s = "\\frac{1}{2}"
  return _fix_a_slash_b(s)


def mathd_normalize_answer(answer: Optional[str]) -> Optional[str]:
  if answer is None:
    return None
  answer = answer.strip()
  m = re.search(r"^\\text\{(?P<text>.+?)\}$", answer)
  if m is not None:
    answer = m.group("text").strip()
  try:
    return _strip_string(answer)
  except Exception:  # pylint: disable=broad-exception-caught
    return answer


def grade_answer_mathd(given_answer: str, ground_truth: str) -> bool:
  gt = mathd_normalize_answer(str(ground_truth))
  given = mathd_normalize_answer(str(given_answer))
  return gt is not None and gt == given


# ---------------------------------------------------------------------------------------------
# symbolic normalisation and grading
# ---------------------------------------------------------------------------------------------
def _sympy_parse(expr: str):
  py = expr.replace("^", "**")
  return sympy_parser.parse_expr(
      py, transformations=(sympy_parser.standard_transformations
                           + (sympy_parser.implicit_multiplication_application,)))


def _latex_to_text(expr: str) -> str:
  """A small LaTeX-to-plain converter for the constructs answers use (no external package)."""
  expr = expr.replace("\\tfrac", "\\frac").replace("\\dfrac", "\\frac")
  expr = re.sub(r"\\frac\{(-?\d+)\}\{(-?\d+)\}", r"\1/\2", expr)      # plain numeric fractions stay a/b
  for _ in range(8):    # nested fractions, innermost first
    new = re.sub(r"\\frac\{([^{}]*)\}\{([^{}]*)\}", r"((\1)/(\2))", expr)
    if new == expr:
      break
    expr = new
  for _ in range(4):
    new = re.sub(r"\\sqrt\{([^{}]*)\}", r"sqrt(\1)", expr)
    if new == expr:
      break
    expr = new
  expr = re.sub(r"\\sqrt\s*(\w)", r"sqrt(\1)", expr)
  expr = re.sub(r"\\text\{([^{}]*)\}", r"\1", expr)
  expr = re.sub(r"\\(?:mathrm|mathbf|textbf)\{([^{}]*)\}", r"\1", expr)
  rep = {"\\pi": "pi", "\\infty": "oo", "\\cup": "U", "\\cdot": "*", "\\times": "*", "\\div": "/", "\\le": "<=",
         "\\ge": ">=", "\\leq": "<=", "\\geq": ">=", "\\%": "%", "\\$": "$", "\\,": "", "\\;": "", "\\ ": " ",
         "\\!": "", "\\left": "", "\\right": "", "√": "sqrt", "π": "pi", "∞": "oo", "∪": "U", "·": "*", "×": "*"}
  for k in sorted(rep, key=len, reverse=True):
    expr = expr.replace(k, rep[k])
  expr = expr.replace("{", "(").replace("}", ")")
  return expr.strip()


def _is_float(x: str) -> bool:
  try:
    float(x)
    return True
  except ValueError:
    return False


def _str_is_int(x: str) -> bool:
  try:
    x = x.replace(",", "")
    return abs(float(x) - int(round(float(x)))) <= 1e-7
  except (ValueError, OverflowError):
    return False


def _strip_thousands_commas(expr: str) -> str:
  pat = re.compile(r"(\d)(,)(\d\d\d)($|\D)")
  while True:
    new = pat.sub(r"\1\3\4", expr)
    if new == expr:
      return new
    expr = new


def _normalize(expr: Optional[str]) -> Optional[str]:
  """Plain-text canonical form: no units, no thousands commas, LaTeX flattened, lower case."""
  if expr is None:
    return None
  m = re.search(r"^\\text\{(?P<text>.+?)\}$", expr)
  if m is not None:
    expr = m.group("text")
  expr = expr.replace("\\%", "%").replace("\\$", "$").replace("$", "").replace("%", "")
  expr = expr.replace(" or ", " , ").replace(" and ", " , ")
  expr = expr.replace("million", "*10^6").replace("billion", "*10^9").replace("trillion", "*10^12")
  for unit in _UNIT_WORDS:
    expr = re.sub(rf"{unit}(es)?(s)? *(\^[0-9]+)?", "", expr)
  expr = re.sub(r"\^ *\\circ", "", expr)
  if expr and expr[0] == "{" and expr[-1] == "}":
    expr = expr[1:-1]
  expr = re.sub(r",\\! *", "", expr)
  if _is_float(expr) and _str_is_int(expr):
    expr = str(int(round(float(expr))))
  if "\\" in expr:
    try:
      expr = _latex_to_text(expr)
    except Exception:  # pylint: disable=broad-exception-caught
      pass
  expr = re.sub(r"- *", "-", expr)
  expr = re.sub(r"([0-9]) +([0-9])", r"\1+\2", expr)    # mixed numbers: 7 3/4 -> 7+3/4
  expr = expr.replace(" ", "").replace("{", "").replace("}", "").lower()
  if _str_is_int(expr):
    expr = str(int(round(float(expr.replace(",", "")))))
  return expr


def count_unknown_letters_in_expr(expr: str) -> int:
  expr = expr.replace("sqrt", "").replace("frac", "").replace("pi", "").replace("oo", "")
  return len({c for c in expr if c.isalpha()})


def should_allow_eval(expr: str) -> bool:
  """Refuses expressions that would make sympy slow or that are not arithmetic."""
  if count_unknown_letters_in_expr(expr) > 2:
    return False
  if any(b in expr for b in BAD_SUBSTRINGS):
    return False
  return not any(re.search(r, expr) for r in BAD_REGEXES)


def are_equal_under_sympy(ground_truth_normalized: str, given_normalized: str) -> bool:
  if sympy is None:
    return False
  try:
    expr = f"({ground_truth_normalized})-({given_normalized})"
    if should_allow_eval(expr):
      return sympy.simplify(_sympy_parse(expr)) == 0
  except Exception:  # pylint: disable=broad-exception-caught
    pass
  return False


def split_tuple(expr: str) -> List[str]:
  """"(1,2)" -> ["1", "2"]; anything that is not a bracketed list stays one element."""
  expr = _strip_thousands_commas(expr)
  if not expr:
    return []
  if (len(expr) > 2 and expr[0] in TUPLE_CHARS and expr[-1] in TUPLE_CHARS
      and all(c not in expr[1:-1] for c in TUPLE_CHARS)):
    return [e.strip() for e in expr[1:-1].split(",")]
  return [expr]


def _is_frac(expr: str) -> bool:
  return bool(re.search(r"^-?[0-9]+.?/0*[1-9][0-9]*.?$", expr))


def grade_answer_sympy(given_answer: str, ground_truth: str) -> bool:
  gt = _normalize(str(ground_truth))
  given = _normalize(str(given_answer))
  if gt is None or given is None:
    return False
  if gt == given:
    return True
  if not given:
    return False
  gt_el, given_el = split_tuple(gt), split_tuple(given)
  if len(gt_el) > 1 and (gt[0] != given[0] or gt[-1] != given[-1]):
    return False          # (1,2) vs [1,2]: open and closed intervals differ
  if len(gt_el) != len(given_el):
    return False
  for a, b in zip(gt_el, given_el):
    if _is_frac(a) and _is_frac(b):
      ok = a == b          # fractions must be given reduced, as the reference grader requires
    elif _str_is_int(a) != _str_is_int(b):
      ok = False           # 3 vs 3.0001, or an unevaluated expression given for an integer answer
    else:
      ok = are_equal_under_sympy(a, b)
    if not ok:
      return False
  return True


# ---------------------------------------------------------------------------------------------
# special cases
# ---------------------------------------------------------------------------------------------
def _recurring_value(expr: str):
  """0.\\overline{3} / 0.1\\overline{6} -> exact Rational."""
  m = re.fullmatch(r"(-?)(\d*)\.(\d*)\\overline\{(\d+)\}", expr.replace(" ", ""))
  if not m or sympy is None:
    return None
  sign, whole, fixed, rep = m.groups()
  base = sympy.Rational(int((whole or "0") + fixed), 10 ** len(fixed)) if (whole or fixed) else sympy.Integer(0)
  val = base + sympy.Rational(int(rep), (10 ** len(rep) - 1) * 10 ** len(fixed))
  return -val if sign else val


def _parse_interval_set(expr: str):
  """"(-oo,1]U[2,3)" -> sorted list of (lo, hi, closed_lo, closed_hi), or None."""
  if sympy is None:
    return None
  text = _latex_to_text(expr).replace(" ", "")
  pieces = [p for p in re.split(r"U|\\cup", text) if p]
  out = []
  for p in pieces:
    m = re.fullmatch(r"([\(\[])(.+),(.+)([\)\]])", p)
    if not m:
      return None
    try:
      lo, hi = _sympy_parse(m.group(2)), _sympy_parse(m.group(3))
    except Exception:  # pylint: disable=broad-exception-caught
      return None
    out.append((lo, hi, m.group(1) == "[", m.group(4) == "]"))
  try:
    return sorted(out, key=lambda t: float(t[0]) if t[0].is_finite else float("-inf"))
  except Exception:  # pylint: disable=broad-exception-caught
    return out


def grade_answer_special_handling(given_answer: str, ground_truth: str) -> bool:
  given, gt = str(given_answer), str(ground_truth)
  # recurring decimals against fractions or other recurring decimals
  a, b = _recurring_value(given), _recurring_value(gt)
  if a is not None or b is not None:
    try:
      a = a if a is not None else sympy.nsimplify(_sympy_parse(_normalize(given)))
      b = b if b is not None else sympy.nsimplify(_sympy_parse(_normalize(gt)))
      return sympy.simplify(a - b) == 0
    except Exception:  # pylint: disable=broad-exception-caught
      return False
  # unions of intervals, order-insensitive
  if ("\\cup" in given or "U" in given or "∪" in given) and ("\\cup" in gt or "U" in gt or "∪" in gt):
    sa, sb = _parse_interval_set(given), _parse_interval_set(gt)
    if sa is not None and sb is not None and len(sa) == len(sb):
      try:
        same = lambda u, v: u == v or sympy.simplify(u - v) == 0
        return all(x[2:] == y[2:] and same(x[0], y[0]) and same(x[1], y[1]) for x, y in zip(sa, sb))
      except Exception:  # pylint: disable=broad-exception-caught
        return False
  # "\\sqrt{}3"-style malformed roots: compare with the empty braces removed
  if "\\sqrt{}" in given or "\\sqrt{}" in gt:
    return grade_answer_sympy(given.replace("\\sqrt{}", "\\sqrt"), gt.replace("\\sqrt{}", "\\sqrt")) or \
        grade_answer_mathd(given.replace("\\sqrt{}", "\\sqrt"), gt.replace("\\sqrt{}", "\\sqrt"))
  return False
