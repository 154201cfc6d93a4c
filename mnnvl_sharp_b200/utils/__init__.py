"""Host-side utilities: numerics and oracle, rack inventory and rank plan, reports."""
from . import numerics, rack  # noqa: F401
