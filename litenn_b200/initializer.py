"""Initializers.  Scalar and NumpyArray fill device buffers through the C ABI
(litenn/core/initializer/Scalar.py, NumpyArray.py).  The random ones draw on the HOST with
numpy and upload -- the reference generates them on the device with a PCG hash
(initializer/RandomUniform.py:12-28), whose bit stream is not reproduced here; the
distributions (uniform range, normal mean/std, He/Glorot fans) are the same."""
import numpy as np


class Initializer:
    def initialize_buffer(self, buf, shape):
        raise NotImplementedError()


class Scalar(Initializer):
    def __init__(self, value=0.0):
        self.value = float(value)

    def initialize_buffer(self, buf, shape):
        buf.fill(np.float32(self.value))

    def __str__(self): return f"Scalar ({self.value})"


class Uninitialized(Initializer):
    """Leaves the buffer as allocated: for tensors every element of which the producing kernel
    overwrites (op outputs), so the zero fill of the default initializer would be wasted."""

    def initialize_buffer(self, buf, shape):
        pass


class NumpyArray(Initializer):
    def __init__(self, np_value):
        self.np_value = np.asarray(np_value, dtype=np.float32)

    def initialize_buffer(self, buf, shape):
        if self.np_value.size != shape.size:
            raise ValueError(f"NumpyArray of size {self.np_value.size} cannot initialize shape {shape}")
        buf.set(self.np_value.reshape(shape.shape))


def _rng():
    return np.random.default_rng(np.random.randint(2**31))


class RandomUniform(Initializer):
    def __init__(self, low=0.0, high=1.0):
        self.low, self.high = low, high

    def initialize_buffer(self, buf, shape):
        buf.set(_rng().uniform(self.low, self.high, shape.shape).astype(np.float32))


class RandomNormal(Initializer):
    def __init__(self, mean=0.0, stddev=1.0):
        self.mean, self.stddev = mean, stddev

    def initialize_buffer(self, buf, shape):
        buf.set(_rng().normal(self.mean, self.stddev, shape.shape).astype(np.float32))


def _fans(shape, fan_in, fan_out):
    """Fans as initializer/He.py:18-31 / Glorot.py derive them: conv kernels (OC,IC,KH,KW)
    use IC*KH*KW / OC*KH*KW, matrices (in,out) use the two extents."""
    if fan_in is not None and fan_out is not None:
        return fan_in, fan_out
    s = shape.shape
    if len(s) == 4:
        rf = s[2] * s[3]
        return s[1] * rf, s[0] * rf
    if len(s) >= 2:
        return s[0], s[1]
    return s[0], s[0]


class HeNormal(Initializer):
    def __init__(self, fan_in=None, fan_out=None, gain=1.0):
        self.fan_in, self.fan_out, self.gain = fan_in, fan_out, gain

    def initialize_buffer(self, buf, shape):
        fi, _ = _fans(shape, self.fan_in, self.fan_out)
        buf.set(_rng().normal(0.0, self.gain * np.sqrt(2.0 / fi), shape.shape).astype(np.float32))


class HeUniform(Initializer):
    def __init__(self, fan_in=None, fan_out=None, gain=1.0):
        self.fan_in, self.fan_out, self.gain = fan_in, fan_out, gain

    def initialize_buffer(self, buf, shape):
        fi, _ = _fans(shape, self.fan_in, self.fan_out)
        lim = self.gain * np.sqrt(6.0 / fi)
        buf.set(_rng().uniform(-lim, lim, shape.shape).astype(np.float32))


class GlorotNormal(Initializer):
    def __init__(self, fan_in=None, fan_out=None, gain=1.0):
        self.fan_in, self.fan_out, self.gain = fan_in, fan_out, gain

    def initialize_buffer(self, buf, shape):
        fi, fo = _fans(shape, self.fan_in, self.fan_out)
        buf.set(_rng().normal(0.0, self.gain * np.sqrt(2.0 / (fi + fo)), shape.shape).astype(np.float32))


class GlorotUniform(Initializer):
    def __init__(self, fan_in=None, fan_out=None, gain=1.0):
        self.fan_in, self.fan_out, self.gain = fan_in, fan_out, gain

    def initialize_buffer(self, buf, shape):
        fi, fo = _fans(shape, self.fan_in, self.fan_out)
        lim = self.gain * np.sqrt(6.0 / (fi + fo))
        buf.set(_rng().uniform(-lim, lim, shape.shape).astype(np.float32))
