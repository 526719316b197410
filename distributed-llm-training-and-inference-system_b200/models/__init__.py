"""Model families.  Importing the package registers every architecture (``models/registry.py``)."""
from . import nafazen as _nafazen  # noqa: F401  (registers "Nafazen")
from . import namisun as _namisun  # noqa: F401  (registers "Namisun")
from . import teluzen as _teluzen  # noqa: F401  (registers "Teluzen")
from . import tupidra as _tupidra  # noqa: F401  (registers "Tupidra")
