"""B200-native (sm_100a) fused neighbourhood kernels for gauge-equivariant
attention on the sphere: hand-written CUDA behind a C-ABI shared library
(``libgmb200.so``), with a Python host layer that mirrors the operator
interface of masonfaldet/gm-attention's ``gm_attention.nn.fused_*`` drivers.

There is no CPU path: every operator raises if the CUDA library is missing.
"""

__all__ = ["__version__"]
__version__ = "0.1.0"
