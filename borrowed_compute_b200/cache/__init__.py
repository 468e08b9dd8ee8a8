from .paged import PagedCache
from .slots import PAGE, GroupPlan, PagePool, SlotTable, pages_for

__all__ = ["PAGE", "GroupPlan", "PagePool", "PagedCache", "SlotTable", "pages_for"]
