"""Architecture builders.  Importing this package registers them."""
from . import minimax_m2  # noqa: F401
