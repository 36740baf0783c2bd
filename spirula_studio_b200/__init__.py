"""B200-native training hot path of a 3D Gaussian splatting trainer.

`lib` binds the C ABI of libssb_b200.so (include/ssb.h); `scenes` generates the
seeded benchmark scenes; `trainer.Trainer` drives one iteration per call.
Importing the package does not need a GPU; calling into the library does, and
fails loudly if libssb_b200.so has not been built.
"""
from . import lib, scenes  # noqa: F401

__all__ = ["lib", "scenes"]
