"""One file per architecture; importing this package registers them all."""
from . import lfm2, puzorax, tevirax, votavik  # noqa: F401
