"""Stand-in for NVIDIA apex (not installable offline): only ``apex.optimizers`` is provided."""
from . import optimizers  # noqa: F401
