"""Op families: `gla` (per-channel gates), `simple_gla` (scalar gates),
`common` (cumsum and the two state scans).  Import the functions from the
family modules, e.g. `from tops_b200.ops.gla import chunk_gla`."""
from . import common, gla, simple_gla  # noqa: F401
