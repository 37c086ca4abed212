"""The cache manager: pages, block tables, layer groups and per-request state slots."""

from .manager import PagedCache

__all__ = ["PagedCache"]
