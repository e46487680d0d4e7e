"""B200-native Winograd / DWM forward convolution behind the operator surface of
huangdi95/pytorch_winoconv: the C-ABI loader (capi), the planned-convolution objects (engine), torch.nn
modules (conv) and the reference-named operator modules (dwm, matrix_conv*, Split_and_Concat, Add, WinoConv)."""
__version__ = "0.1.0"
