"""B200-native wave-index decode attention (RetroInfer-compatible hot path).

The CUDA library is loaded on first use of a kernel-backed module; the package itself
(configuration, synthetic inputs) imports without it.
"""
from .config import GEOMETRIES, Geometry, WaveIndexConfig, generate_config  # noqa: F401

__version__ = "0.1.0"
