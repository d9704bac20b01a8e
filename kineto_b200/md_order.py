"""Visit order of GenericTraceActivity metadata.

The reference keeps per-activity metadata in a `std::unordered_map<std::string, TypedValue>` and
serialises it in that container's iteration order (libkineto/include/GenericTraceActivity.h:160-170,
:195).  A host that flattens activities into columns captures that order by visiting the real
object; synthetic generators have no object to visit, so this module reproduces the order for the
GNU libstdc++ container: 64-bit murmur-style `std::hash<std::string>` (seed 0xc70f6907), 13 buckets
up to 13 elements (then 29, 59, ...), a new node going to the front of its bucket's run or, for an empty bucket, to
the front of the whole list.
"""
from __future__ import annotations

from functools import lru_cache

_M = 0xFFFFFFFFFFFFFFFF
_MUL = (0xC6A4A793 << 32) + 0x5BD1E995


def _shift_mix(v: int) -> int:
    return v ^ (v >> 47)


def hash_bytes(data: bytes, seed: int = 0xC70F6907) -> int:
    n = len(data)
    h = (seed ^ (n * _MUL)) & _M
    aligned = n & ~7
    for i in range(0, aligned, 8):
        d = int.from_bytes(data[i:i + 8], "little")
        d = (_shift_mix((d * _MUL) & _M) * _MUL) & _M
        h ^= d
        h = (h * _MUL) & _M
    if n & 7:
        d = int.from_bytes(data[aligned:], "little")
        h ^= d
        h = (h * _MUL) & _M
    h = (_shift_mix(h) * _MUL) & _M
    return _shift_mix(h)


_BUCKETS = (13, 29, 59, 127, 257)  # the container's bucket counts as it grows (load factor 1, growth factor 2)


def _insert(order: list, key: str, nb: int) -> None:
    """A node goes to the front of its bucket's run or, when the bucket is empty, to the front of the list."""
    b = hash_bytes(key.encode()) % nb
    pos = next((i for i, o in enumerate(order) if hash_bytes(o.encode()) % nb == b), None)
    order.insert(0 if pos is None else pos, key)


@lru_cache(maxsize=None)
def md_visit_order(keys: tuple) -> tuple:
    """Order in which a GenericTraceActivity that received `keys` in this insertion order visits
    them.  Duplicate keys keep the first insertion (emplace semantics).  When an insertion would exceed
    one element per bucket the container first moves to the next bucket count, re-linking its nodes in
    their current order by the same rule as an insertion."""
    level = 0
    order: list[str] = []
    for k in keys:
        if k in order:
            continue
        if len(order) + 1 > _BUCKETS[level]:
            level += 1
            if level >= len(_BUCKETS):
                raise ValueError("more than %d metadata keys per activity is not modelled" % _BUCKETS[-1])
            old, order = order, []
            for o in old:
                _insert(order, o, _BUCKETS[level])
        _insert(order, k, _BUCKETS[level])
    return tuple(order)
