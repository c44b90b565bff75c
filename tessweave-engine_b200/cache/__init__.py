"""Cache manager: paged keys/values per group of layers, block tables, prefix index, state slots."""
from .manager import CacheManager, CapacityError, Lease, PageGroup

__all__ = ["CacheManager", "CapacityError", "Lease", "PageGroup"]
