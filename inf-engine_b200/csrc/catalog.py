"""Which libraries exist and with which compile-time sizes they can be asked for."""

from __future__ import annotations

from .build import LIBRARIES


def all_build_requests():
    """(name, sources, defines, extra headers) of everything worth pre-building."""
    reqs = [("core", LIBRARIES["core"], {}, [])]
    return reqs
