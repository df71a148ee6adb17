"""B200-native (sm_100a) mapped convolution hot path behind the reference's layer API."""
from . import nn, ops, util  # noqa: F401

__version__ = "0.1.0"
