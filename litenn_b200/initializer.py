"""Initializers (litenn/core/initializer/*.py).  Scalar and NumpyArray fill device buffers
through the C ABI; the random ones run on the device with the reference's counter-based PCG
hash (RandomUniform.py:12-28, RandomNormal.py:10-30) and draw the hash seed the way it does,
np.random.randint(2**31) at initialisation time, so after the same np.random.seed(...) a
uniform tensor has the reference's bits and a normal one differs only by the device's log / cos
rounding.  HeUniform / HeNormal / GlorotUniform / GlorotNormal take (gain, fan_in[, fan_out]) in
the reference's order; Conv2D / Dense fill in missing fans (Conv2D.py:41-44, Dense.py:28-31)."""
import numpy as np

from . import _lib


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


def _draw_seed():
    return int(np.random.randint(2147483648))


def _each_device_buffer(buf):
    from .devices import devices
    if devices._shallow > 0:
        return None
    return buf.device.index, buf.ptr(), buf.size // 4


class RandomUniform(Initializer):
    def __init__(self, low=0.0, high=1.0):
        self.low, self.high = low, high

    def initialize_buffer(self, buf, shape):
        seed = _draw_seed()
        tgt = _each_device_buffer(buf)
        if tgt is not None:
            _lib.get_lib().lnn_init_uniform(tgt[0], tgt[1], tgt[2], seed, float(np.float32(self.low)), float(np.float32(self.high)))

    def __str__(self): return f"RandomUniform low={self.low}, high={self.high}"


class RandomNormal(Initializer):
    def __init__(self, mean=0.0, stddev=1.0):
        self.mean, self.stddev = mean, stddev

    def initialize_buffer(self, buf, shape):
        seed = _draw_seed()
        tgt = _each_device_buffer(buf)
        if tgt is not None:
            _lib.get_lib().lnn_init_normal(tgt[0], tgt[1], tgt[2], seed, float(np.float32(self.mean)), float(np.float32(self.stddev)))

    def __str__(self): return f"RandomNormal mean={self.mean}, stddev={self.stddev}"


def _fans(shape, fan_in, fan_out):
    """Fans when the layer did not set them: conv kernels (OC,IC,KH,KW) use IC*KH*KW /
    OC*KH*KW (Conv2D.py:41-44), matrices (in,out) the two extents (Dense.py:28-31)."""
    s = shape.shape
    if len(s) == 4:
        rf = s[2] * s[3]
        fi, fo = s[1] * rf, s[0] * rf
    elif len(s) >= 2:
        fi, fo = s[0], s[1]
    else:
        fi = fo = s[0]
    return (fan_in if fan_in is not None else fi), (fan_out if fan_out is not None else fo)


class _InitHe(Initializer):
    """std = gain * sqrt(2 / fan_in); uniform uses +-sqrt(3) * std  (He.py:18-31)."""

    def __init__(self, type, gain, fan_in):
        self.type, self.gain, self.fan_in = type, gain, fan_in

    def has_fan_in(self): return True
    def has_fan_out(self): return False

    def initialize_buffer(self, buf, shape):
        fi, _ = _fans(shape, self.fan_in, None)
        std = self.gain * np.sqrt(2.0 / fi)
        if self.type == "uniform":
            a = np.sqrt(3.0) * std
            RandomUniform(-a, a).initialize_buffer(buf, shape)
        else:
            RandomNormal(0.0, std).initialize_buffer(buf, shape)

    def __str__(self): return f"InitHe type={self.type}, gain={self.gain}, fan_in={self.fan_in}"


class _InitGlorot(Initializer):
    """std = gain * sqrt(2 / (fan_in + fan_out)); uniform uses +-sqrt(3) * std  (Glorot.py:18-33)."""

    def __init__(self, type, gain, fan_in, fan_out):
        self.type, self.gain, self.fan_in, self.fan_out = type, gain, fan_in, fan_out

    def has_fan_in(self): return True
    def has_fan_out(self): return True

    def initialize_buffer(self, buf, shape):
        fi, fo = _fans(shape, self.fan_in, self.fan_out)
        std = self.gain * np.sqrt(2.0 / (fi + fo))
        if self.type == "uniform":
            a = np.sqrt(3.0) * std
            RandomUniform(-a, a).initialize_buffer(buf, shape)
        else:
            RandomNormal(0.0, std).initialize_buffer(buf, shape)

    def __str__(self):
        return f"InitGlorot type={self.type}, gain={self.gain}, fan_in={self.fan_in}, fan_out={self.fan_out}"


def HeUniform(gain=2.0, fan_in=None): return _InitHe("uniform", gain, fan_in)
def HeNormal(gain=1.0, fan_in=None): return _InitHe("normal", gain, fan_in)
def GlorotUniform(gain=1.0, fan_in=None, fan_out=None): return _InitGlorot("uniform", gain, fan_in, fan_out)
def GlorotNormal(gain=1.0, fan_in=None, fan_out=None): return _InitGlorot("normal", gain, fan_in, fan_out)
