"""Op families: `gla` (per-channel gates), `simple_gla` (scalar gates),
`common` (cumsum and the two state scans)."""
from . import common, gla, simple_gla  # noqa: F401
from .gla import chunk_gla, fused_chunk_gla, fused_recurrent_gla  # noqa: F401
from .simple_gla import chunk_simple_gla, simple_gla  # noqa: F401
