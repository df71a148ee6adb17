from .layers import (MappedAvgPool, MappedAvgUnpool, MappedConvolution, MappedMaxPool,
                     MappedTransposedConvolution, Resample, Unresample)

__all__ = ["MappedConvolution", "MappedTransposedConvolution", "MappedMaxPool", "MappedAvgPool",
           "MappedAvgUnpool", "Resample", "Unresample"]
