"""Drop-in for the reference project's `kernels` package, EMA path only.

Put this directory's parent on sys.path ahead of the reference checkout and
`from kernels.ema_kernels.ema_combined_fwd import ema_matmul_scan_combined` (and every other EMA
entry point of the reference) resolves to the B200 implementation: same names, same argument
meaning, same return layouts and dtypes, same assertion behaviour.
"""
import os
import sys

_parent = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if _parent not in sys.path:
    sys.path.insert(0, _parent)
