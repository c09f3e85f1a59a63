"""The allocation-free first-layer convolution against the graph API's Conv2d and against the CPU oracle.

Some users of the library are not allowed to allocate device memory while they run (plugins of a
server that hands out its memory once, loops with hard deadlines, processes near the memory limit).
For them the library has one entry point, b2vx_conv2d_first_layer_noalloc, that keeps its only
intermediate in a fixed array inside the library and takes every input and output from the caller.
This test plays such a caller: all device buffers are created here, up front; the entry point is then
called twice in a row on different images, and each result must equal, byte for byte, what a Conv2d
node of the ordinary graph API produces for the same image and what the CPU oracle computes (the bar
every other GPU test uses for integer outputs).  A second, small and awkward problem (one input channel, a
channel count that needs padding, a 5x3 filter, uneven padding, stride and dilation that differ per axis, a
stream of the caller's) runs after the large one, so that the shared array holds stale data.  Problems the
entry point must refuse are refused with a message.

The file sorts last on purpose: a run that stops at the first failure has then seen every other test.
"""
import ctypes as C

import numpy as np
import pytest

import pyb2vx as B

pytestmark = pytest.mark.gpu


class NoAllocDesc(C.Structure):
    _fields_ = [("n", C.c_uint32), ("h", C.c_uint32), ("w", C.c_uint32), ("c", C.c_uint32),
                ("kw", C.c_uint32), ("kh", C.c_uint32), ("oc", C.c_uint32),
                ("stride", C.c_uint32 * 2), ("dilation", C.c_uint32 * 2), ("pad", C.c_uint32 * 4),
                ("in_zero_point", C.c_int32), ("out_scale", C.c_float), ("out_zero_point", C.c_int32)]


class Problem:
    def __init__(self, n, h, w, c, kw, kh, oc, stride, dilation, pad, in_scale, in_zp, out_scale, out_zp):
        self.n, self.h, self.w, self.c, self.kw, self.kh, self.oc = n, h, w, c, kw, kh, oc
        self.stride, self.dilation, self.pad = stride, dilation, pad
        self.in_scale, self.in_zp, self.out_scale, self.out_zp = in_scale, in_zp, out_scale, out_zp
        self.wo = (w + pad[0] + pad[1] - ((kw - 1) * dilation[0] + 1)) // stride[0] + 1
        self.ho = (h + pad[2] + pad[3] - ((kh - 1) * dilation[1] + 1)) // stride[1] + 1
        self.ocp = (oc + 15) // 16 * 16

    def desc(self):
        d = NoAllocDesc()
        d.n, d.h, d.w, d.c = self.n, self.h, self.w, self.c
        d.kw, d.kh, d.oc = self.kw, self.kh, self.oc
        d.stride[:] = self.stride
        d.dilation[:] = self.dilation
        d.pad[:] = self.pad
        d.in_zero_point, d.out_scale, d.out_zero_point = self.in_zp, self.out_scale, self.out_zp
        return d


LARGE = Problem(2, 64, 48, 3, 7, 7, 64, (2, 2), (1, 1), (3, 3, 3, 3), 0.02, 128, 0.05, 0)
SMALL = Problem(3, 19, 23, 1, 5, 3, 24, (2, 1), (1, 2), (1, 2, 0, 1), 0.03, 7, 0.04, 11)


def graph_conv(lib, p, weights, wscales, bias, image):
    """The existing entry point: a one-node graph through the C ABI; returns [N, OC, Ho, Wo]."""
    g = B.Graph(lib)
    x = g.tensor(B.DT_UINT8, [p.w, p.h, p.c, p.n], B.ATTR_INPUT, scale=p.in_scale, zero_point=p.in_zp)
    w = g.tensor(B.DT_INT8, [p.kw, p.kh, p.c, p.oc], B.ATTR_CONSTANT, scales=wscales, channel_dim=3, data=weights)
    b = g.tensor(B.DT_INT32, [p.oc], B.ATTR_CONSTANT, scales=np.float32(p.in_scale) * wscales, channel_dim=0, data=bias)
    y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=p.out_scale, zero_point=p.out_zp)
    g.conv2d(x, w, b, y, stride=p.stride, dilation=p.dilation, pad=p.pad)
    g.compile()
    g.write(x, image)
    g.run()
    out = g.read(y)
    names = [k["name"] for k in g.kernels()]
    g.close()
    return out, names


def entry_point(product_lib):
    fn = product_lib.b2vx_conv2d_first_layer_noalloc
    fn.restype = C.c_int32
    fn.argtypes = [C.POINTER(NoAllocDesc)] + [C.c_void_p] * 6 + [C.c_char_p, C.c_size_t]
    return fn


def run_problem(product_lib, oracle_lib, p, seed, calls, stream=None):
    import torch
    fn = entry_point(product_lib)
    rng = np.random.default_rng(seed)
    weights = rng.integers(-127, 128, size=(p.oc, p.c, p.kh, p.kw)).astype(np.int8)
    wscales = rng.uniform(0.001, 0.01, p.oc).astype(np.float32)
    bias = rng.integers(-1000, 1001, size=p.oc).astype(np.int32)
    images = [rng.integers(0, 256, size=(p.n, p.c, p.h, p.w)).astype(np.uint8) for _ in range(calls)]
    # operands in the layout the entry point documents; every device buffer is made here, once
    kdim = p.c * p.kh * p.kw
    kp = (kdim + 15) // 16 * 16
    w8 = np.zeros((p.ocp, kp), np.int8)
    w8[:p.oc, :kdim] = weights.reshape(p.oc, kdim)
    bias_full = np.zeros(p.ocp, np.int32)
    bias_full[:p.oc] = (bias.astype(np.int64) - p.in_zp * weights.reshape(p.oc, -1).astype(np.int64).sum(axis=1)).astype(np.int32)
    acc_scale = np.zeros(p.ocp, np.float32)
    acc_scale[:p.oc] = np.float32(p.in_scale) * wscales
    dev = torch.device("cuda:0")
    d_w8 = torch.from_numpy(w8).to(dev)
    d_bias = torch.from_numpy(bias_full).to(dev)
    d_scale = torch.from_numpy(acc_scale).to(dev)
    d_x = torch.empty(p.n * p.c * p.h * p.w, dtype=torch.uint8, device=dev)
    d_y = torch.empty(p.n * p.ho * p.wo * p.ocp, dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()
    desc = p.desc()
    err = C.create_string_buffer(256)
    for image in images:   # calls in a row share the built-in scratch array
        want, kernels = graph_conv(product_lib, p, weights, wscales, bias, image)
        oracle, _ = graph_conv(oracle_lib, p, weights, wscales, bias, image)
        assert np.array_equal(want, oracle), "the graph convolution itself differs from the oracle"
        d_x.copy_(torch.from_numpy(image.reshape(-1)))
        d_y.fill_(0xAB)
        torch.cuda.synchronize()
        st = fn(C.byref(desc), d_x.data_ptr(), d_w8.data_ptr(), d_bias.data_ptr(), d_scale.data_ptr(), d_y.data_ptr(),
                stream.cuda_stream if stream is not None else None, err, len(err))
        assert st == 0, err.value.decode()
        full = d_y.cpu().numpy().reshape(p.n, p.ho, p.wo, p.ocp)
        got = full[..., :p.oc].transpose(0, 3, 1, 2)
        assert want.shape == got.shape
        assert np.array_equal(oracle, got), "%d of %d bytes differ from the oracle" % (np.count_nonzero(oracle != got), oracle.size)
        assert np.array_equal(want, got)
        assert any("gemm_i8_tc" in k for k in kernels)
    return desc, (d_x, d_w8, d_bias, d_scale, d_y)


def test_noalloc_conv_equals_graph_conv_and_oracle(product_lib, oracle_lib):
    import torch
    assert torch.cuda.is_available()
    fn = entry_point(product_lib)
    desc, bufs = run_problem(product_lib, oracle_lib, LARGE, 99, calls=2)
    # the awkward small problem on a stream of the caller's, over the stale contents the large one left behind
    side = torch.cuda.Stream()
    run_problem(product_lib, oracle_lib, SMALL, 100, calls=2, stream=side)
    d_x, d_w8, d_bias, d_scale, d_y = bufs
    args = (d_x.data_ptr(), d_w8.data_ptr(), d_bias.data_ptr(), d_scale.data_ptr(), d_y.data_ptr(), None)
    err = C.create_string_buffer(256)

    # larger than the built-in scratch: refused with a message, nothing launched
    big = NoAllocDesc.from_buffer_copy(desc)
    big.n, big.h, big.w = 64, 224, 224
    assert fn(C.byref(big), *args, err, len(err)) == 1 and b"scratch" in err.value
    # sixteen or more input channels, more than 256 output channels, zero points outside a byte, a null pointer
    for field, value in (("c", 16), ("oc", 257), ("in_zero_point", 256), ("out_zero_point", -1), ("w", 0x7fffffff)):
        bad = NoAllocDesc.from_buffer_copy(desc)
        setattr(bad, field, value)
        err.value = b""
        assert fn(C.byref(bad), *args, err, len(err)) == 1 and err.value, field
    assert fn(C.byref(desc), None, *args[1:], err, len(err)) == 1 and b"null" in err.value
