"""B200-native dequantize-fused low-bit linear kernels behind NNFusion's operator interface."""
__version__ = "0.1.0"
