"""kiln_b200: a B200-native (sm_100a) replacement for Kiln's ``kiln.gpu`` package."""

__version__ = "0.1.0"
