"""The parity tests' checker helpers live beside the oracle they drive (``oracle/check.py``)."""
from oracle.check import *  # noqa: F401,F403
from oracle.check import MAX_ABS_TOL, REL_L2_TOL  # noqa: F401
