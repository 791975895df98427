"""The C++ host library (csrc/host/host_runtime.cpp) as seen from Python: loading, signatures, errors.

Requests and holders have any hashable name in Python and a 64-bit handle in the library; `Names` keeps
the two apart and puts the names back into the library's error texts.
"""
from __future__ import annotations

import ctypes
import re
from ctypes import POINTER, c_char_p, c_int, c_longlong, c_void_p
from typing import Dict, Hashable

_lib = None
NOBODY = -(1 << 63)


class PoolExhausted(RuntimeError):
    """No free page (the reference's KvPoolExhausted, src/main/java/org/robomiri/jllm/kv/KvPoolExhausted.java:4)."""


class PageBookkeepingError(AssertionError):
    """A page was freed twice, freed by someone who does not hold it, or handed out twice: a bug."""


def lib():
    """The loaded host library; compiled at the first call if need be."""
    global _lib
    if _lib is None:
        from ..csrc.build import ensure_host_built
        L = ctypes.CDLL(str(ensure_host_built()))
        P, I, LL, PI, PLL = c_void_p, c_int, c_longlong, POINTER(c_int), POINTER(c_longlong)
        sig = {
            "jh_last_error": ([], c_char_p),
            "jh_pool_new": ([I, c_char_p], P), "jh_pool_delete": ([P], None), "jh_pool_alloc": ([P, LL, PI], I),
            "jh_pool_free": ([P, I, LL], I), "jh_pool_check": ([P], I), "jh_pool_num_free": ([P], I),
            "jh_pool_holder": ([P, I], LL), "jh_pool_stats": ([P, PLL, PLL], None),
            "jh_cache_new": ([I, PI, I, I, I], P), "jh_cache_delete": ([P], None), "jh_cache_open": ([P, LL, PI], I),
            "jh_cache_close": ([P, LL], I), "jh_cache_is_open": ([P, LL], I), "jh_cache_num_requests": ([P], I),
            "jh_cache_request_ids": ([P, PLL, I], I), "jh_cache_request": ([P, LL, PI, PI, PLL, PI], I),
            "jh_cache_table": ([P, LL, I, PI, I], I), "jh_cache_pages_missing": ([P, LL, I, I, PI], I),
            "jh_cache_can_reserve": ([P, LL, I, I], I), "jh_cache_reserve": ([P, LL, I, I], I),
            "jh_cache_commit": ([P, LL, I, PI, I, PI], I), "jh_cache_truncate": ([P, LL, I], I),
            "jh_cache_trim": ([P, LL], I), "jh_cache_check": ([P], I), "jh_cache_free_pages": ([P, PI], I),
            "jh_cache_pool": ([P, I], P),
            "jh_step_reserve": ([P, I, P, P, P], I), "jh_step_commit": ([P, I, P, P, P, I, P], I),
            "jh_builder_new": ([I, I, I, I, I], P), "jh_builder_delete": ([P], None),
            "jh_builder_build": ([P, P, I, P, P, P, P, P, P, I, P, P, P], I),
        }
        for name, (args, res) in sig.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, res
        _lib = L
    return _lib


class Names:
    """Hashable names <-> handles, for one pool or one cache."""

    def __init__(self):
        self._handle: Dict[Hashable, int] = {}
        self._name: Dict[int, Hashable] = {}
        self._next = 0

    def handle(self, name: Hashable, make: bool = False) -> int:
        h = self._handle.get(name)
        if h is None:
            if not make:
                return -1 - hash(name) % (1 << 40)      # a handle no request has: the library answers "not open"
            h = self._next
            self._next += 1
            self._handle[name] = h
            self._name[h] = name
        return h

    def name(self, handle: int):
        return self._name.get(handle)

    def forget(self, name: Hashable) -> None:
        h = self._handle.pop(name, None)
        if h is not None:
            self._name.pop(h, None)

    def text(self, message: str) -> str:
        return re.sub(r"#(-?\d+)", lambda m: repr(self._name.get(int(m.group(1)), "?")), message)


def check(code: int, names: Names | None = None) -> None:
    """Raises what the library's error code stands for, with the names of the requests back in the text."""
    if code == 0:
        return
    text = lib().jh_last_error().decode(errors="replace")
    if names is not None:
        text = names.text(text)
    if code == 2:
        raise PoolExhausted(text)
    if code == 3:
        raise PageBookkeepingError(text)
    if code == 4:
        raise KeyError(text)
    raise ValueError(text)
