"""Host-C execution of the reference's OpenCL kernel text, used ONLY to generate golden
vectors (make_golden.py) in a container that has the reference checkout but no OpenCL
device.  It is a module with the surface of `litenn.core.minicl.api.OpenCL` (the 22 names
listed in that package's __init__): buffers are numpy arrays, a "program" is the kernel
text compiled by gcc as C (`-std=gnu11 -O2 -ffp-contract=off -fsingle-precision-constant`,
matching the reference's `-cl-single-precision-constant`), and an NDRange launch is a
serial loop over work-items, so atomics resolve in work-item order.

Install with `install()` BEFORE importing litenn; nothing in the reference tree is edited.
"""
import collections
import collections.abc
import ctypes
import hashlib
import os
import re
import subprocess
import sys
import tempfile
import types

import numpy as np

PRELUDE = r"""
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#define __kernel
#define __global
#define __constant const
#define __local
#define restrict __restrict__
typedef unsigned int uint;
typedef unsigned long ulong;
typedef float float2  __attribute__((vector_size(8),  aligned(4)));
typedef float float4  __attribute__((vector_size(16), aligned(4)));
typedef float float8  __attribute__((vector_size(32), aligned(4)));
typedef float float16 __attribute__((vector_size(64), aligned(4)));
static size_t lnn_gid[3];
#define get_global_id(d) (lnn_gid[d])
static inline int atomic_inc(volatile int* p) { int old = *p; *p = old + 1; return old; }
/* OpenCL's float overloads: evaluate in double, round once */
#define exp(x)  ((float)exp((double)(x)))
#define log(x)  ((float)log((double)(x)))
#define sin(x)  ((float)sin((double)(x)))
#define cos(x)  ((float)cos((double)(x)))
#define sqrt(x) (sqrtf((float)(x)))
#define fabs(x) (fabsf((float)(x)))
#define fmax(a,b) (fmaxf((float)(a),(float)(b)))
#define fmin(a,b) (fminf((float)(a),(float)(b)))
"""

_CACHE_DIR = os.path.join(tempfile.gettempdir(), "lnn_cl_on_cpu")


class CLException(Exception):
    def __init__(self, error, message=None):
        self.error = error
        super().__init__(f"{error} {message or ''}")


class _Enum:
    def __init__(self, value):
        self.value = value


class ERROR:
    SUCCESS = 0
    MEM_OBJECT_ALLOCATION_FAILURE = -4
    BUILD_PROGRAM_FAILURE = -11


class DEVICE_TYPE(int):
    GPU = 4
    ACCELERATOR = 8
    CPU = 2
    ALL = 0xFFFFFFFF


class PROGRAM_INFO:
    BINARY_SIZES = 0x1165
    BINARIES = 0x1166


class PROGRAM_BUILD_INFO:
    BUILD_STATUS = 0x1181
    BUILD_LOG = 0x1183


class BUILD_STATUS:
    SUCCESS = 0


class _Event:
    def wait(self):
        pass


class _Device:
    name = "host-C execution of OpenCL kernel text"
    global_mem_size = 8 * 1024**3
    max_mem_alloc_size = 8 * 1024**3
    device_version = "OpenCL 1.2 (gcc)"


class _Mem:
    def __init__(self, size):
        raw = np.zeros(size + 64, dtype=np.uint8)
        off = (-raw.ctypes.data) % 64
        self.raw = raw
        self.view = raw[off:off + size]     # 64-byte aligned for the vector loads
        self.size = size

    @property
    def addr(self):
        return self.view.ctypes.data


class _Program:
    def __init__(self, source):
        self.source = source
        self.lib = None
        self.log = ""
        self.kernels = []


class _Kernel:
    def __init__(self, program, name, params):
        self.program, self.name, self.params = program, name, params
        self.fn = getattr(program.lib, "lnn_run_" + name)
        self.fn.restype = None

    def __call__(self, queue, global_shape, local_shape=None, shape_offsets=None, *args):
        if len(args) != len(self.params):
            raise CLException(-52, f"kernel {self.name} takes {len(self.params)} args, got {len(args)}")
        g = list(global_shape) + [1] * (3 - len(global_shape))
        holders, ptrs = [], (ctypes.c_void_p * len(args))()
        for i, (arg, (is_ptr, ctype)) in enumerate(zip(args, self.params)):
            if is_ptr:
                if not isinstance(arg, _Mem):
                    raise CLException(-50, f"arg {i} of {self.name} must be a buffer")
                ptrs[i] = arg.addr
            else:
                cval = {"long": ctypes.c_int64, "ulong": ctypes.c_uint64, "int": ctypes.c_int32,
                        "uint": ctypes.c_uint32, "float": ctypes.c_float, "size_t": ctypes.c_uint64}[ctype](arg)
                holders.append(cval)
                ptrs[i] = ctypes.addressof(cval)
        self.fn(ctypes.c_size_t(g[0]), ctypes.c_size_t(g[1]), ctypes.c_size_t(g[2]), ptrs)
        return _Event()


def GetPlatforms():
    return ["host"]


def GetDeviceIDs(platform, DEVICE_TYPE=DEVICE_TYPE.ALL):
    # report one "GPU-class" device so the reference's device enumeration picks it
    return [_Device()] if (int(DEVICE_TYPE) & 4) else []


def CreateContext(devices):
    return object()


def CreateCommandQueue(context, device):
    return object()


def Finish(queue):
    pass


def CreateBuffer(context, size):
    return _Mem(size)


def EnqueueCopyBuffer(queue, src, dst, src_offset, dst_offset, size):
    dst.view[dst_offset:dst_offset + size] = src.view[src_offset:src_offset + size]
    return _Event()


def EnqueueFillBuffer(queue, mem, pattern, size, offset=0):
    pat = np.array([pattern]).view(np.uint8)
    n = max(len(pat), size) // len(pat)
    mem.view[offset:offset + n * len(pat)] = np.tile(pat, n)
    return _Event()


def EnqueueWriteBuffer(queue, mem, pointer, size, offset=0):
    ctypes.memmove(mem.addr + offset, pointer, size)
    return _Event()


def ndarray_to_buffer(queue, buf, np_ar):
    np_ar = np.ascontiguousarray(np_ar)
    ctypes.memmove(buf.addr, np_ar.ctypes.data, np_ar.nbytes)
    return _Event()


def buffer_to_ndarray(queue, buf, np_ar):
    ctypes.memmove(np_ar.ctypes.data, buf.addr, np_ar.nbytes)
    return _Event()


def CreateProgramWithSource(context, source):
    return _Program(source)


_PARAM_RE = re.compile(r"__kernel\s+void\s+(\w+)\s*\(([^)]*)\)", re.S)


def _parse_params(plist):
    params = []
    for p in [x.strip() for x in plist.split(",") if x.strip()]:
        if "*" in p:
            params.append((True, None))
        else:
            toks = p.replace("const", " ").split()
            params.append((False, toks[-2]))
    return params


def _strip_hash_helpers(source):
    """The optimizer kernels prepend hash helpers written with OpenCL-only vector literals
    (CLKernelHelper.py:208-273).  They are referenced only when lr_dropout is enabled, which
    no golden case uses, so the block is cut out before compiling as C."""
    start = source.find("//---------- PCG hashes")
    if start < 0:
        return source
    tail = source.find("float hash_float_float2(float2 p)", start)
    end = source.find("}", tail) + 1
    return source[:start] + source[end:]


_VEC_CAST_RE = re.compile(r"\((uint2|uint3|float2|float3)\)\s*\(([^()]*)\)")
_VEC_FIELD_RE = re.compile(r"\b([A-Za-z_]\w*)\.([xyz])\b")


def _uses_hash(source):
    """True when the kernel itself calls one of the PCG hash helpers (the random initializers,
    initializer/RandomUniform.py:12-20, RandomNormal.py:10-24)."""
    start = source.find("//---------- PCG hashes")
    if start < 0:
        return False
    tail = source.find("float hash_float_float2(float2 p)", start)
    end = source.find("}", tail) + 1
    return "hash_" in source[end:]


def _hash_dialect_to_gnu_c(source):
    """OpenCL vector syntax of the hash helpers -> GNU C vector extensions, nothing else:
    (uint2)(a, b) becomes the compound literal (uint2){a, b} and v.x / v.y / v.z become
    v[0] / v[1] / v[2].  The arithmetic text is left as the reference wrote it."""
    source = _VEC_CAST_RE.sub(lambda m: "(%s){%s}" % (m.group(1), m.group(2)), source)
    return _VEC_FIELD_RE.sub(lambda m: "%s[%d]" % (m.group(1), "xyz".index(m.group(2))), source)


HASH_PRELUDE = r"""
typedef unsigned int uint2 __attribute__((vector_size(8),  aligned(4)));
typedef unsigned int uint3 __attribute__((vector_size(16), aligned(4)));
typedef float float3 __attribute__((vector_size(16), aligned(4)));
static inline float dot(float2 a, float2 b) { return a[0] * b[0] + a[1] * b[1]; }
"""


def BuildProgram(program, devices, options=None):
    if _uses_hash(program.source):
        program.source = HASH_PRELUDE + _hash_dialect_to_gnu_c(program.source)
    else:
        program.source = _strip_hash_helpers(program.source)
    m = _PARAM_RE.search(program.source)
    if not m:
        raise CLException(_Enum(ERROR.BUILD_PROGRAM_FAILURE), "no __kernel found")
    name, plist = m.group(1), m.group(2)
    params = _parse_params(plist)
    call_args = []
    decl = [x.strip() for x in plist.split(",") if x.strip()]
    for i, ((is_ptr, ctype), d) in enumerate(zip(params, decl)):
        if is_ptr:
            ptype = d[:d.rindex("*") + 1]
            call_args.append(f"({ptype})args[{i}]")
        else:
            call_args.append(f"*({ctype}*)args[{i}]")
    driver = f"""
void lnn_run_{name}(size_t g0, size_t g1, size_t g2, void** args) {{
  for (size_t z = 0; z < g2; ++z) for (size_t y = 0; y < g1; ++y) for (size_t x = 0; x < g0; ++x) {{
    lnn_gid[0] = x; lnn_gid[1] = y; lnn_gid[2] = z;
    {name}({", ".join(call_args)});
  }}
}}
"""
    text = PRELUDE + program.source + driver
    os.makedirs(_CACHE_DIR, exist_ok=True)
    key = hashlib.sha1(text.encode()).hexdigest()
    so = os.path.join(_CACHE_DIR, key + ".so")
    if not os.path.exists(so):
        src = os.path.join(_CACHE_DIR, key + ".c")
        with open(src, "w") as f:
            f.write(text)
        cmd = ["gcc", "-x", "c", "-std=gnu11", "-O2", "-ffp-contract=off", "-fsingle-precision-constant",
               "-fno-strict-aliasing", "-w", "-shared", "-fPIC", src, "-o", so + ".tmp", "-lm"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        program.log = r.stdout + r.stderr
        if r.returncode != 0:
            raise CLException(_Enum(ERROR.BUILD_PROGRAM_FAILURE), program.log)
        os.replace(so + ".tmp", so)
    program.lib = ctypes.CDLL(so)
    program.kernels = [_Kernel(program, name, params)]


def CreateKernelsInProgram(program):
    return program.kernels


def GetProgramInfo(program, param_name):
    return None


def GetProgramBuildInfo(program, param_name, device):
    return program.log


Exception_ = CLException


def install():
    """Register this module as litenn.core.minicl.api.OpenCL and patch the removed
    `collections.Iterable` alias the reference still imports (Python >= 3.10)."""
    if not hasattr(collections, "Iterable"):
        collections.Iterable = collections.abc.Iterable
    mod = types.ModuleType("litenn.core.minicl.api.OpenCL")
    this = sys.modules[__name__]
    for k in ("BuildProgram", "BUILD_STATUS", "DEVICE_TYPE", "CreateBuffer", "CreateContext",
              "CreateCommandQueue", "CreateKernelsInProgram", "CreateProgramWithSource",
              "EnqueueCopyBuffer", "EnqueueFillBuffer", "EnqueueWriteBuffer", "Finish", "GetPlatforms",
              "GetProgramInfo", "GetProgramBuildInfo", "GetDeviceIDs", "PROGRAM_INFO",
              "PROGRAM_BUILD_INFO", "ERROR", "buffer_to_ndarray", "ndarray_to_buffer", "CLException"):
        setattr(mod, k, getattr(this, k))
    mod.Exception = CLException
    sys.modules["litenn.core.minicl.api.OpenCL"] = mod
