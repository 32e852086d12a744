"""Span trees: `Span` (a named interval) and `SpanGroup` (a named interval containing spans and
groups), with the lookups the metric exporters use (tunix/perf/span.py:28-320)."""
from __future__ import annotations

import copy
from typing import List, Optional, Union


class Span:

  def __init__(self, name: str, begin: float):
    self.name = name
    self.begin = begin
    self.end = float("inf")

  def __repr__(self) -> str:
    return f"Span({self.name}, {self.begin:.6f}, {self.end:.6f})"

  @property
  def ended(self) -> bool:
    return self.end != float("inf")

  @property
  def duration(self) -> float:
    return self.end - self.begin


class SpanGroup:

  def __init__(self, name: str, outer: Optional["SpanGroup"] = None):
    self.name = name
    self.begin = 0.0
    self.end = float("inf")
    self.outer = outer
    self.inner: List[Union[Span, "SpanGroup"]] = []
    if outer is not None:
      outer.inner.append(self)

  def __repr__(self) -> str:
    return f"SpanGroup({self.name}, {self.begin:.6f}, {self.end:.6f}, inner={len(self.inner)})"

  @property
  def ended(self) -> bool:
    return self.end != float("inf")

  @property
  def duration(self) -> float:
    return self.end - self.begin

  def _groups(self):
    return [x for x in self.inner if isinstance(x, SpanGroup)]

  def find_first_inner_group(self, name: str) -> Optional["SpanGroup"]:
    return next((g for g in self._groups() if g.name == name), None)

  def find_last_inner_group(self, name: str) -> Optional["SpanGroup"]:
    return next((g for g in reversed(self._groups()) if g.name == name), None)

  def find_all_inner_groups(self, name: str) -> List["SpanGroup"]:
    return [g for g in self._groups() if g.name == name]

  def find_last_inner_span(self, name: str) -> Optional[Span]:
    return next((s for s in reversed(self.inner) if isinstance(s, Span) and s.name == name), None)

  def find_all_inner_spans(self, name: str) -> List[Span]:
    return [s for s in self.inner if isinstance(s, Span) and s.name == name]

  def find_all_spans_recursive(self, name: str) -> List[Span]:
    out: List[Span] = []
    for x in self.inner:
      if isinstance(x, Span):
        if x.name == name:
          out.append(x)
      else:
        out.extend(x.find_all_spans_recursive(name))
    return out

  def find_all_groups_recursive(self, name: str) -> List["SpanGroup"]:
    out: List[SpanGroup] = []
    for g in self._groups():
      if g.name == name:
        out.append(g)
      out.extend(g.find_all_groups_recursive(name))
    return out


def span_group_tostring(group: SpanGroup, born: float = 0.0) -> str:
  def rec(out: str, g: SpanGroup, indent: int) -> str:
    out += " " * indent + f"[{g.name}] {g.begin - born:.6f} -> {g.end - born:.6f}\n"
    for x in g.inner:
      if isinstance(x, SpanGroup):
        out = rec(out, x, indent + 2)
      else:
        out += " " * (indent + 2) + f"{x.name}: {x.begin - born:.6f} -> {x.end - born:.6f}\n"
    return out
  return rec("", group, 0)


def span_group_print(group: SpanGroup, born: float = 0.0) -> None:
  print(span_group_tostring(group, born))


def span_group_batch_query_first(groups: List[SpanGroup], name: str) -> List[SpanGroup]:
  return [g2 for g in groups if (g2 := g.find_first_inner_group(name)) is not None]


def span_group_batch_query_last(groups: List[SpanGroup], name: str) -> List[SpanGroup]:
  return [g2 for g in groups if (g2 := g.find_last_inner_group(name)) is not None]


def span_group_batch_query_nth(groups: List[SpanGroup], name: str, index: int) -> List[SpanGroup]:
  out = []
  for g in groups:
    all_ = g.find_all_inner_groups(name)
    if -len(all_) <= index < len(all_):
      out.append(all_[index])
  return out


def span_group_batch_query_all(groups: List[SpanGroup], name: str) -> List[SpanGroup]:
  return [g2 for g in groups for g2 in g.find_all_inner_groups(name)]


def clone_span_or_group(node, outer: Optional[SpanGroup] = None):
  if isinstance(node, Span):
    s = Span(node.name, node.begin)
    s.end = node.end
    if outer is not None:
      outer.inner.append(s)
    return s
  g = SpanGroup(node.name, outer)
  g.begin, g.end = node.begin, node.end
  for x in node.inner:
    clone_span_or_group(x, g)
  return g
