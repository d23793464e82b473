from .allocator import PageAllocator, PageError, pages_for, prefix_hash
from .manager import CachePlan, GroupLayout, OutOfPages, RequestCache, plan_groups

__all__ = ["CachePlan", "GroupLayout", "OutOfPages", "PageAllocator", "PageError", "RequestCache",
           "pages_for", "plan_groups", "prefix_hash"]
