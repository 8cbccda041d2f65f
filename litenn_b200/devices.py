"""Device registry and device buffers.

Same public surface as the reference's `nn.devices` (litenn/core/minicl/devices.py:
get_all, get_best, get_by_idx, set_current, get_current, wait, cleanup) and CLBuffer
(litenn/core/minicl/CLBuffer.py: lazy physical allocation with an initializer run on
first touch, set / fill / np), over the C-ABI runtime instead of OpenCL.
"""
import ctypes
from collections.abc import Iterable

import numpy as np

from . import _lib


class Device:
    """One B200.  `.index` is the CUDA ordinal and the slot used in every C-ABI call."""

    def __init__(self, index, name, global_mem_size, sm_count, cc):
        self.index = index
        self.name = name
        self.global_mem_size = global_mem_size
        self.sm_count = sm_count
        self.cc = cc
        self.is_cpu = False
        self._inited = False

    def _ensure(self):
        if not self._inited:
            _lib.get_lib().lnn_init(self.index)
            self._inited = True

    def get_used_memory(self):
        a, p = self._mem_stats()
        return a - p

    def get_total_allocated_memory(self):
        return self._mem_stats()[0]

    def get_total_pooled_memory(self):
        return self._mem_stats()[1]

    def _mem_stats(self):
        if not self._inited:
            return 0, 0
        a, p = ctypes.c_uint64(), ctypes.c_uint64()
        _lib.get_lib().lnn_mem_stats(self.index, ctypes.byref(a), ctypes.byref(p))
        return a.value, p.value

    def wait(self):
        if self._inited:
            _lib.get_lib().lnn_sync(self.index)

    def launch_count(self):
        if not self._inited:
            return 0
        c = ctypes.c_uint64()
        _lib.get_lib().lnn_launch_count(self.index, ctypes.byref(c))
        return c.value

    def check_status(self):
        """Raise LnnError if a bounded device-side wait gave up since the last check."""
        if not self._inited:
            return
        st = ctypes.c_int()
        lib = _lib.get_lib()
        lib.lnn_device_status(self.index, ctypes.byref(st))
        if st.value != 0:
            raise _lib.LnnError(st.value, lib.lnn_last_error().decode(), "device_status")

    def _cleanup(self):
        if self._inited:
            _lib.get_lib().lnn_shutdown(self.index)
            self._inited = False

    def __str__(self):
        return f"[{self.index}]:[{self.name}][{self.global_mem_size / 1024**3:.3} GB]"

    __repr__ = __str__


class DeviceBuffer:
    """Device memory of `size` bytes, physically allocated on first use (CLBuffer.py:36-42)."""

    __slots__ = ["device", "size", "init_func", "_ptr"]
    _object_count = 0

    def __init__(self, device, size, init_func=None):
        if size <= 0:
            raise ValueError(f"Create DeviceBuffer with {size} size.")
        DeviceBuffer._object_count += 1
        self._ptr = None
        self.device = device
        self.size = int(size)
        self.init_func = init_func

    def __del__(self):
        DeviceBuffer._object_count -= 1
        try:
            self.free()
        except Exception:
            pass

    def has_mem(self):
        return self._ptr is not None

    def ptr(self):
        if self._ptr is None:
            self.device._ensure()
            p = ctypes.c_uint64()
            _lib.get_lib().lnn_alloc(self.device.index, self.size, ctypes.byref(p))
            self._ptr = p.value
            if self.init_func is not None:
                self.init_func(self)
        return self._ptr

    def free(self):
        if self._ptr is not None:
            _lib.get_lib().lnn_free(self.device.index, self._ptr, self.size)
            self._ptr = None

    def set(self, value):
        if isinstance(value, DeviceBuffer):
            if value is self:
                return
            if self.size != value.size:
                raise Exception(f"Unable to copy from buffer with {value.size} size to buffer with {self.size} size.")
            if devices._shallow > 0:
                return
            if self.device is value.device:
                _lib.get_lib().lnn_d2d(self.device.index, self.ptr(), value.ptr(), self.size)
            else:
                self.set(value.np())    # staged through the host, as CLBuffer.py:68-70
            return
        if not isinstance(value, np.ndarray):
            raise ValueError(f"Invalid type {value.__class__}. Must be np.ndarray.")
        if value.nbytes != self.size:
            raise ValueError(f"Value size {value.nbytes} does not match buffer size {self.size}.")
        if devices._shallow > 0:
            return
        value = np.ascontiguousarray(value)
        _lib.get_lib().lnn_h2d(self.device.index, self.ptr(), value.ctypes.data_as(ctypes.c_void_p), self.size)

    def fill(self, value):
        if devices._shallow > 0:
            return
        _lib.get_lib().lnn_fill_f32(self.device.index, self.ptr(), self.size // 4, float(value))

    def np(self, shape=None, dtype=np.float32):
        if shape is None or len(shape) == 0:
            shape = (self.size // 4,)
        out = np.empty(tuple(shape), dtype)
        if out.nbytes != self.size:
            raise ValueError(f"Unable to represent buffer with size {self.size} as shape {shape} with dtype {dtype}")
        if devices._shallow == 0:
            _lib.get_lib().lnn_d2h(self.device.index, out.ctypes.data_as(ctypes.c_void_p), self.ptr(), self.size)
        return out

    def __str__(self):
        return f"DeviceBuffer [{self.size} bytes] on {self.device}"

    __repr__ = __str__


class _ShallowMode:
    def __enter__(self):
        devices._shallow += 1
        return self

    def __exit__(self, *exc):
        devices._shallow -= 1


class devices:
    """Static registry, like `nn.devices` in the reference."""

    _all_devices = None
    _current_devices = None
    _shallow = 0

    @staticmethod
    def _shallow_mode():
        """Inside this context no kernel is launched and no memory is touched
        (shape inference only; CLShallowMode.py, CLDevice.py:84-85)."""
        return _ShallowMode()

    @staticmethod
    def get_all():
        if devices._all_devices is None:
            lib = _lib.get_lib()
            n = ctypes.c_int()
            try:
                lib.lnn_device_count(ctypes.byref(n))
            except _lib.LnnError:
                n = ctypes.c_int(0)
            ar = []
            for i in range(n.value):
                name = ctypes.create_string_buffer(256)
                mem, sms, mj, mn = ctypes.c_uint64(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
                lib.lnn_device_info(i, name, 256, ctypes.byref(mem), ctypes.byref(sms), ctypes.byref(mj), ctypes.byref(mn))
                ar.append(Device(i, name.value.decode(), mem.value, sms.value, (mj.value, mn.value)))
            devices._all_devices = ar
        return devices._all_devices

    @staticmethod
    def get_by_idx(index):
        return devices.get_all()[index]

    @staticmethod
    def get_best():
        best, best_mem = None, 0
        for d in devices.get_all():
            if d.global_mem_size > best_mem:
                best, best_mem = d, d.global_mem_size
        return best

    @staticmethod
    def get_current():
        if devices._current_devices is None:
            best = devices.get_best()
            if best is None:
                raise Exception("No CUDA device found (this backend has no CPU fallback).")
            devices.set_current(best)
        return devices._current_devices

    @staticmethod
    def set_current(device_or_list, verbose=False):
        if DeviceBuffer._object_count != 0:
            raise Exception("You cannot set current devices while any DeviceBuffer objects exists.")
        devices.cleanup()
        if isinstance(device_or_list, Iterable):
            device_or_list = tuple(device_or_list)
        if not isinstance(device_or_list, tuple):
            device_or_list = (device_or_list,)
        if len(device_or_list) == 0:
            raise ValueError("device_or_list cannot be empty")
        if not all(isinstance(d, Device) for d in device_or_list):
            raise ValueError("argument should be Device")
        if verbose:
            print(f'Using {", ".join(d.name for d in device_or_list)}')
        devices._current_devices = device_or_list

    @staticmethod
    def cleanup():
        if DeviceBuffer._object_count != 0:
            raise Exception(f"Unable to cleanup while {DeviceBuffer._object_count} DeviceBuffer objects exist.")
        if devices._current_devices is not None:
            for d in devices._current_devices:
                d._cleanup()

    @staticmethod
    def wait():
        for d in devices.get_current():
            d.wait()

    @staticmethod
    def check_status():
        for d in devices.get_current():
            d.check_status()


class DevicesBuffers:
    """One DeviceBuffer per current device (CLDevicesBuffers.py:4-23)."""

    def __init__(self, size, init_func=None):
        self._buffers = [DeviceBuffer(d, size, init_func=init_func) for d in devices.get_current()]

    def _get_buffers(self):
        return self._buffers
