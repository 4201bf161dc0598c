"""Architectures.  Importing this package registers them by name."""
from . import fozedra, lfm3, maferax, narasun, relilix  # noqa: F401
