"""Plural spelling used by the reference's README usage text; same objects as `mapped_convolution`."""
from . import nn, util  # noqa: F401
