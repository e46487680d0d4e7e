"""B200-native Winograd / DWM forward convolution behind the operator surface of
huangdi95/pytorch_winoconv.  See DESIGN.md for the layout of this package."""
__version__ = "0.1.0"
