"""Single-tile n-D DWM with the reference's signature (``dwm_convnd.py:7-40``): input
``[B, C, (k+1)^n]``, kernel ``[K, C, k^n]`` -> ``[B, K, 2^n]``.  The reference loops over the
<=3-wide pieces in Python and sums ``matrix_convnd.conv32`` of each; here the decomposition
happens inside the engine's kernels (one call)."""
from . import matrix_convnd


def conv32(input, kernel, n):
    return matrix_convnd.conv32(input, kernel, n)
