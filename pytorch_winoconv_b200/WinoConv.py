"""``Wino`` with the method names of the reference's class (``WinoConv.py:8-228``).  The
reference's body is unrunnable TF-era code (``tf.convert_to_tensor`` at ``:21``, undefined
globals at ``:20,45``); its intended semantics are those of ``matrix_conv``, which this class
delegates to."""
from . import matrix_conv


class Wino:
    def matrix_alloc(self, m, r):
        return matrix_conv.matrix_alloc(m, r)

    def conv16(self, input, kernel, bias=None, stride=(1, 1), padding=0, groups=1, output_block=2):
        return matrix_conv.conv16(input, kernel, bias, stride, padding, groups, output_block)

    def conv32(self, input, kernel, bias=None, stride=(1, 1), padding=0, groups=1, output_block=2):
        return matrix_conv.conv32(input, kernel, bias, stride, padding, groups, output_block)

    def conv(self, input, kernel, output_block, stride, fp16=False):
        return matrix_conv.conv(input, kernel, output_block, stride, fp16)

    def base_conv32(self, input, kernel, fp16, m, r):
        return matrix_conv.base_conv32(input, kernel, fp16, m, r)
