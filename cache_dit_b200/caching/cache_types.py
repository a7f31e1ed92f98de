"""Cache type names accepted by the public API (mirrors src/cache_dit/caching/cache_types.py:5-51)."""
from enum import Enum

_ALIASES = {
  "DBCache": ("DUAL_BLOCK_CACHE", "DB_CACHE", "DBCACHE", "DB"),
  "DBPrune": ("DYNAMIC_BLOCK_PRUNE", "DB_PRUNE", "DBPRUNE", "DBP"),
  "NONE": ("NONE", "NO_CACHE", "NOCACHE", "NC"),
}


class CacheType(Enum):
  NONE = "NONE"
  DBCache = "DBCache"
  DBPrune = "DBPrune"  # accepted as a name; the pruning algorithm itself is outside this package

  @staticmethod
  def type(type_hint: "CacheType | str | None") -> "CacheType":
    return cache_type(type_hint)

  def __str__(self) -> str:
    return self.value


def cache_type(type_hint: "CacheType | str | None") -> CacheType:
  if type_hint is None:
    return CacheType.NONE
  if isinstance(type_hint, CacheType):
    return type_hint
  upper = type_hint.upper()
  for name, aliases in _ALIASES.items():
    if upper in aliases:
      return CacheType[name]
  return CacheType.NONE


def block_range(start: int, end: int, step: int = 1) -> list:
  """Block ids that always run: 0, every `step`-th from `start`, and the last one."""
  if start > end or end <= 0 or step <= 1:
    return []
  return sorted(set([0] + list(range(start, end, step)) + [end - 1]))
