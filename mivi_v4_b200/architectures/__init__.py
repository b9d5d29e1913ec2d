"""One file per architecture; importing this package registers them all."""
from . import lfm2  # noqa: F401
