"""ctypes binding of the b2vx C ABI (include/b2vx.h) for tests and benchmarks.

The binding drives any library that exports the ABI: ``tim-vx_b200/csrc/libb2vx.so``
(the CUDA product, PRODUCT_LIB) and, from the tests, the CPU oracle's library.
Nothing here computes anything: tensors go in and out as numpy arrays in
tim::vx order (shape listed fastest dimension first, i.e. the reversed numpy
shape of a C-contiguous array).
"""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PRODUCT_LIB = os.path.join(ROOT, "tim-vx_b200", "csrc", "libb2vx.so")

NO_TENSOR = 0xFFFFFFFF
DT_INT8, DT_UINT8, DT_INT32, DT_FLOAT32 = 1, 2, 5, 9
NP_DTYPE = {DT_INT8: np.int8, DT_UINT8: np.uint8, DT_INT32: np.int32, DT_FLOAT32: np.float32}
Q_NONE, Q_ASYM, Q_PER_CHANNEL = 0, 1, 2
ATTR_CONSTANT, ATTR_TRANSIENT, ATTR_VARIABLE, ATTR_INPUT, ATTR_OUTPUT = 1, 2, 4, 8, 16
PAD_NONE, PAD_AUTO, PAD_VALID, PAD_SAME = -1, 0, 1, 2
POOL_MAX, POOL_AVG, POOL_L2, POOL_AVG_ANDROID = 0, 1, 2, 3
ROUND_CEILING, ROUND_FLOOR = 0, 1
NODE_CONV2D, NODE_FC, NODE_POOL2D, NODE_ADD, NODE_RELU, NODE_RELU6, NODE_SOFTMAX = 1, 2, 3, 4, 5, 6, 7
NODE_RESHAPE, NODE_TRANSPOSE, NODE_CONCAT, NODE_DATACONVERT, NODE_ADDN = 8, 9, 10, 11, 12
STATUS_NAMES = ["OK", "INVALID_ARG", "UNSUPPORTED", "SHAPE_MISMATCH", "QUANT_MISMATCH", "OOM", "CUDA_ERROR",
                "DEVICE_TIMEOUT", "BAD_STATE"]


class TensorDesc(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("rank", C.c_uint32), ("dims", C.c_uint32 * 8), ("attr", C.c_int32),
                ("quant_type", C.c_int32), ("scale", C.c_float), ("zero_point", C.c_int32),
                ("channel_dim", C.c_int32), ("n_channel", C.c_uint32), ("scales", C.POINTER(C.c_float)),
                ("zero_points", C.POINTER(C.c_int32))]


class Conv2dDesc(C.Structure):
    _fields_ = [("weights", C.c_uint32), ("pad_type", C.c_int32), ("ksize", C.c_uint32 * 2),
                ("stride", C.c_uint32 * 2), ("dilation", C.c_uint32 * 2), ("pad", C.c_uint32 * 4),
                ("multiplier", C.c_int32), ("group", C.c_int32)]


class FcDesc(C.Structure):
    _fields_ = [("axis", C.c_uint32), ("weights", C.c_uint32)]


class Pool2dDesc(C.Structure):
    _fields_ = [("type", C.c_int32), ("pad_type", C.c_int32), ("ksize", C.c_uint32 * 2), ("stride", C.c_uint32 * 2),
                ("pad", C.c_uint32 * 4), ("round_type", C.c_int32)]


class SoftmaxDesc(C.Structure):
    _fields_ = [("beta", C.c_float), ("axis", C.c_int32)]


class DimsDesc(C.Structure):
    _fields_ = [("rank", C.c_uint32), ("v", C.c_uint32 * 8)]

    @classmethod
    def of(cls, values):
        d = cls()
        d.rank = len(values)
        for i, v in enumerate(values):
            d.v[i] = int(v)
        return d


class KernelInfo(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("node_index", C.c_uint32), ("ops", C.c_uint64), ("bytes", C.c_uint64),
                ("last_ms", C.c_float)]


class B2vxError(RuntimeError):
    def __init__(self, status, message):
        self.status = status
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__("%s: %s" % (name, message))


def load(path):
    """Load one library exporting the b2vx ABI and declare its signatures."""
    lib = C.CDLL(path)
    vp, u32, st = C.c_void_p, C.c_uint32, C.c_int32
    sigs = {
        "b2vx_context_create": (st, [C.POINTER(vp)]),
        "b2vx_context_destroy": (None, [vp]),
        "b2vx_last_error": (C.c_char_p, [vp]),
        "b2vx_device_count": (C.c_int32, []),
        "b2vx_graph_create": (st, [vp, C.c_int32, C.POINTER(vp)]),
        "b2vx_graph_destroy": (None, [vp]),
        "b2vx_tensor_create": (st, [vp, C.POINTER(TensorDesc), vp, C.POINTER(u32)]),
        "b2vx_tensor_get_desc": (st, [vp, u32, C.POINTER(TensorDesc)]),
        "b2vx_tensor_write": (st, [vp, u32, vp, C.c_size_t]),
        "b2vx_tensor_read": (st, [vp, u32, vp, C.c_size_t]),
        "b2vx_node_conv2d": (st, [vp, u32, u32, u32, u32, C.POINTER(Conv2dDesc)]),
        "b2vx_node_fully_connected": (st, [vp, u32, u32, u32, u32, C.POINTER(FcDesc)]),
        "b2vx_node_pool2d": (st, [vp, u32, u32, C.POINTER(Pool2dDesc)]),
        "b2vx_node_add": (st, [vp, u32, u32, u32]),
        "b2vx_node_relu": (st, [vp, u32, u32]),
        "b2vx_node_relu6": (st, [vp, u32, u32]),
        "b2vx_node_softmax": (st, [vp, u32, u32, C.POINTER(SoftmaxDesc)]),
        "b2vx_node_reshape": (st, [vp, u32, u32, C.POINTER(DimsDesc)]),
        "b2vx_node_transpose": (st, [vp, u32, u32, C.POINTER(DimsDesc)]),
        "b2vx_node_concat": (st, [vp, C.POINTER(C.c_uint32), u32, u32, u32]),
        "b2vx_node_dataconvert": (st, [vp, u32, u32]),
        "b2vx_node_addn": (st, [vp, C.POINTER(C.c_uint32), u32, u32]),
        "b2vx_graph_compile": (st, [vp]),
        "b2vx_graph_run": (st, [vp]),
        "b2vx_graph_run_async": (st, [vp]),
        "b2vx_graph_sync": (st, [vp]),
        "b2vx_graph_set_stream": (st, [vp, vp]),
        "b2vx_graph_print": (st, [vp]),
        "b2vx_graph_kernel_count": (st, [vp, C.POINTER(u32)]),
        "b2vx_graph_kernel_info": (st, [vp, u32, C.POINTER(KernelInfo)]),
        "b2vx_graph_profile": (st, [vp, u32]),
        "b2vx_measure_int8_peak": (st, [C.c_int32, C.c_int32, C.POINTER(C.c_double), C.POINTER(C.c_int32)]),
        "b2vx_host_alloc": (st, [C.POINTER(vp), C.c_size_t]),
        "b2vx_host_free": (None, [vp]),
    }
    for name, (res, args) in sigs.items():
        if name == "b2vx_measure_int8_peak" and not hasattr(lib, name):
            continue   # a measurement of the GPU: the CPU oracle library has no such entry
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


class Graph:
    """One b2vx context + graph."""

    def __init__(self, lib, device=0):
        self.lib = lib
        self.ctx = C.c_void_p()
        self.g = C.c_void_p()
        st = lib.b2vx_context_create(C.byref(self.ctx))
        if st != 0:
            raise B2vxError(st, "context_create")
        st = lib.b2vx_graph_create(self.ctx, device, C.byref(self.g))
        if st != 0:
            msg = lib.b2vx_last_error(self.ctx).decode()
            lib.b2vx_context_destroy(self.ctx)
            self.ctx = None
            raise B2vxError(st, msg)
        self._keep = []

    def close(self):
        if self.g:
            self.lib.b2vx_graph_destroy(self.g)
            self.g = None
        if self.ctx:
            self.lib.b2vx_context_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st):
        if st != 0:
            raise B2vxError(st, self.lib.b2vx_last_error(self.ctx).decode())

    def tensor(self, dtype, dims, attr, scale=None, zero_point=0, scales=None, zero_points=None, channel_dim=-1,
               data=None):
        d = TensorDesc()
        d.dtype = dtype
        d.rank = len(dims)
        for i, v in enumerate(dims):
            d.dims[i] = int(v)
        d.attr = attr
        d.channel_dim = channel_dim
        if scales is not None:
            d.quant_type = Q_PER_CHANNEL
            sc = (C.c_float * len(scales))(*[float(s) for s in scales])
            zps = zero_points if zero_points is not None else [0] * len(scales)
            zp = (C.c_int32 * len(zps))(*[int(z) for z in zps])
            d.n_channel = len(scales)
            d.scales = C.cast(sc, C.POINTER(C.c_float))
            d.zero_points = C.cast(zp, C.POINTER(C.c_int32))
            self._keep += [sc, zp]
        elif scale is not None:
            d.quant_type = Q_ASYM
            d.scale = float(scale)
            d.zero_point = int(zero_point)
        else:
            d.quant_type = Q_NONE
        ptr = None
        if data is not None:
            data = np.ascontiguousarray(data, dtype=NP_DTYPE[dtype])
            self._keep.append(data)
            ptr = data.ctypes.data_as(C.c_void_p)
        tid = C.c_uint32()
        self._check(self.lib.b2vx_tensor_create(self.g, C.byref(d), ptr, C.byref(tid)))
        return tid.value

    def conv2d(self, x, w, bias, y, stride=(1, 1), dilation=(1, 1), pad_type=PAD_AUTO, pad=(0, 0, 0, 0), multiplier=0,
               weights=0, ksize=(0, 0), group=0):
        d = Conv2dDesc()
        d.weights = weights
        d.pad_type = pad_type
        d.ksize[:] = ksize
        d.stride[:] = stride
        d.dilation[:] = dilation
        d.pad[:] = pad
        d.multiplier = multiplier
        d.group = group
        self._check(self.lib.b2vx_node_conv2d(self.g, x, w, NO_TENSOR if bias is None else bias, y, C.byref(d)))

    def fully_connected(self, x, w, bias, y, axis=0, weights=0):
        d = FcDesc(axis, weights)
        self._check(self.lib.b2vx_node_fully_connected(self.g, x, w, NO_TENSOR if bias is None else bias, y, C.byref(d)))

    def pool2d(self, x, y, type, ksize, stride, pad_type=PAD_AUTO, pad=(0, 0, 0, 0), round_type=ROUND_FLOOR):
        d = Pool2dDesc()
        d.type = type
        d.pad_type = pad_type
        d.ksize[:] = ksize
        d.stride[:] = stride
        d.pad[:] = pad
        d.round_type = round_type
        self._check(self.lib.b2vx_node_pool2d(self.g, x, y, C.byref(d)))

    def add(self, a, b, y):
        self._check(self.lib.b2vx_node_add(self.g, a, b, y))

    def relu(self, x, y):
        self._check(self.lib.b2vx_node_relu(self.g, x, y))

    def relu6(self, x, y):
        self._check(self.lib.b2vx_node_relu6(self.g, x, y))

    def softmax(self, x, y, beta=1.0, axis=0):
        d = SoftmaxDesc(beta, axis)
        self._check(self.lib.b2vx_node_softmax(self.g, x, y, C.byref(d)))

    def reshape(self, x, y, shape):
        d = DimsDesc.of(shape)
        self._check(self.lib.b2vx_node_reshape(self.g, x, y, C.byref(d)))

    def transpose(self, x, y, perm):
        d = DimsDesc.of(perm)
        self._check(self.lib.b2vx_node_transpose(self.g, x, y, C.byref(d)))

    def concat(self, inputs, y, axis):
        arr = (C.c_uint32 * len(inputs))(*inputs)
        self._check(self.lib.b2vx_node_concat(self.g, arr, len(inputs), axis, y))

    def addn(self, inputs, y):
        arr = (C.c_uint32 * len(inputs))(*inputs)
        self._check(self.lib.b2vx_node_addn(self.g, arr, len(inputs), y))

    def dataconvert(self, x, y):
        self._check(self.lib.b2vx_node_dataconvert(self.g, x, y))

    def compile(self):
        self._check(self.lib.b2vx_graph_compile(self.g))

    def run(self):
        self._check(self.lib.b2vx_graph_run(self.g))

    def run_async(self):
        self._check(self.lib.b2vx_graph_run_async(self.g))

    def sync(self):
        self._check(self.lib.b2vx_graph_sync(self.g))

    def set_stream(self, stream_ptr):
        self._check(self.lib.b2vx_graph_set_stream(self.g, C.c_void_p(stream_ptr)))

    def desc(self, tid):
        d = TensorDesc()
        self._check(self.lib.b2vx_tensor_get_desc(self.g, tid, C.byref(d)))
        return d

    def shape(self, tid):
        d = self.desc(tid)
        return [int(d.dims[i]) for i in range(d.rank)]

    def write(self, tid, array):
        d = self.desc(tid)
        a = np.ascontiguousarray(array, dtype=NP_DTYPE[d.dtype])
        self._check(self.lib.b2vx_tensor_write(self.g, tid, a.ctypes.data_as(C.c_void_p), a.nbytes))

    def write_ptr(self, tid, ptr, nbytes):
        self._check(self.lib.b2vx_tensor_write(self.g, tid, C.c_void_p(ptr), nbytes))

    def read_ptr(self, tid, ptr, nbytes):
        self._check(self.lib.b2vx_tensor_read(self.g, tid, C.c_void_p(ptr), nbytes))

    def read(self, tid):
        d = self.desc(tid)
        dims = [int(d.dims[i]) for i in range(d.rank)]
        out = np.empty(dims[::-1], dtype=NP_DTYPE[d.dtype])
        self._check(self.lib.b2vx_tensor_read(self.g, tid, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def kernels(self):
        n = C.c_uint32()
        self._check(self.lib.b2vx_graph_kernel_count(self.g, C.byref(n)))
        out = []
        for i in range(n.value):
            k = KernelInfo()
            self._check(self.lib.b2vx_graph_kernel_info(self.g, i, C.byref(k)))
            out.append({"name": k.name.decode(), "node": k.node_index, "ops": k.ops, "bytes": k.bytes, "ms": k.last_ms})
        return out

    def profile(self, iters=5):
        self._check(self.lib.b2vx_graph_profile(self.g, iters))
        return self.kernels()
