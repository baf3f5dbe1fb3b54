"""flashgs_b200: a forward 3D Gaussian Splatting rasterizer written for NVIDIA B200 (sm_100a).

``flashgs_b200.ops`` mirrors the operator API of InternLandMark/FlashGS
(``flash_gaussian_splatting.ops``); the kernels live in ``csrc/`` behind the C ABI
declared in ``include/flashgs_b200.h``.
"""
__version__ = "0.1.0"
