"""Drop-in import name of the reference package (`mapped_convolution`, package/setup.py:96-109)."""
from . import nn, util  # noqa: F401
