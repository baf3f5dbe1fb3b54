"""Drop-in module name of the reference extension (setup.py:34, csrc/pybind.cpp:233-235).

``import flash_gaussian_splatting`` followed by ``flash_gaussian_splatting.ops.<op>(...)``
works exactly as with the reference build, so the reference's example.py runs unchanged
against the sm_100a kernels of ``flashgs_b200``.
"""
from flashgs_b200 import ops  # noqa: F401
