"""kiln_b200: a B200-native (sm_100a) replacement for Kiln's ``kiln.gpu`` package.

    import kiln_b200
    kiln_b200.build()          # once: nvcc -> kiln_b200/_lib/libkb200.so
    kiln = kiln_b200.install() # kiln.compile(..., device="cuda") now runs on this backend
"""

from kiln_b200._cabi import build
from kiln_b200.install import install

__version__ = "0.1.0"
__all__ = ["build", "install"]
