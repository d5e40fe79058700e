"""Name predicates used to pick modules out of a model tree (counterpart of the reference's
src/sparse_llm_cache/utils/filter.py: Filter, RegexFilter, reverse())."""
from __future__ import annotations

import re


class Filter:
    """Accepts every name."""

    def __call__(self, name: str) -> bool:
        return True

    def reverse(self) -> "Filter":
        return _Negated(self)


class _Negated(Filter):
    def __init__(self, inner: Filter):
        self.inner = inner

    def __call__(self, name: str) -> bool:
        return not self.inner(name)

    def reverse(self) -> Filter:
        return self.inner


class RegexFilter(Filter):
    """Accepts names that match the pattern from their first character (re.match)."""

    def __init__(self, pattern: str):
        self.pattern = re.compile(pattern)

    def __call__(self, name: str) -> bool:
        return self.pattern.match(name) is not None
