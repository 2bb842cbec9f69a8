"""Op families: `gla` (per-channel gates), `simple_gla` (scalar gates),
`kda` (gated delta rule),
`common` (cumsum and the two state scans).  Import the functions from the
family modules, e.g. `from tops_b200.ops.gla import chunk_gla`."""
from . import common, gla, kda, simple_gla  # noqa: F401
