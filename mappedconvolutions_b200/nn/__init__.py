from .layers import (Convolution, MappedAvgPool, MappedAvgUnpool, MappedConvolution, MappedMaxPool,
                     MappedTransposedConvolution, Resample, TransposedConvolution, Unresample)

__all__ = ["Convolution", "TransposedConvolution", "MappedConvolution", "MappedTransposedConvolution",
           "MappedMaxPool", "MappedAvgPool", "MappedAvgUnpool", "Resample", "Unresample"]
