"""Paged key/value cache, block tables and per-request state slots."""
from .paged import Group, PagedCache

__all__ = ["Group", "PagedCache"]
