"""The allocation-free first-layer convolution against the graph API's Conv2d.

Some users of the library are not allowed to allocate device memory while they run (plugins of a
server that hands out its memory once, loops with hard deadlines, processes near the memory limit).
For them the library has one entry point, b2vx_conv2d_first_layer_noalloc, that keeps its only
intermediate in a fixed array inside the library and takes every input and output from the caller.
This test plays such a caller: all device buffers are created here, up front; the entry point is then
called twice in a row on different images, and each result must equal, byte for byte, what a Conv2d
node of the ordinary graph API produces for the same image (the bar every other GPU test uses for
integer outputs).  It also checks that a problem too large for the built-in array is refused.

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


N, H, W, Cin, K, OC, STRIDE, PAD = 2, 64, 48, 3, 7, 64, 2, 3
IN_SCALE, IN_ZP, OUT_SCALE, OUT_ZP = 0.02, 128, 0.05, 0


def reference_conv(lib, weights, wscales, bias, image):
    """The existing entry point: a one-node graph through the C ABI; returns [N, OC, Ho, Wo]."""
    g = B.Graph(lib)
    x = g.tensor(B.DT_UINT8, [W, H, Cin, N], B.ATTR_INPUT, scale=IN_SCALE, zero_point=IN_ZP)
    w = g.tensor(B.DT_INT8, [K, K, Cin, OC], B.ATTR_CONSTANT, scales=wscales, channel_dim=3, data=weights)
    b = g.tensor(B.DT_INT32, [OC], B.ATTR_CONSTANT, scales=np.float32(IN_SCALE) * wscales, channel_dim=0, data=bias)
    y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=OUT_SCALE, zero_point=OUT_ZP)
    g.conv2d(x, w, b, y, stride=(STRIDE, STRIDE), pad=(PAD, PAD, PAD, PAD))
    g.compile()
    g.write(x, image)
    g.run()
    out = g.read(y)
    names = [k["name"] for k in g.kernels()]
    g.close()
    return out, names


def test_noalloc_conv_equals_graph_conv(product_lib):
    import torch
    assert torch.cuda.is_available()
    fn = product_lib.b2vx_conv2d_first_layer_noalloc
    fn.restype = C.c_int32
    fn.argtypes = [C.POINTER(NoAllocDesc)] + [C.c_void_p] * 6 + [C.c_char_p, C.c_size_t]

    rng = np.random.default_rng(99)
    weights = rng.integers(-127, 128, size=(OC, Cin, K, K)).astype(np.int8)
    wscales = rng.uniform(0.001, 0.01, OC).astype(np.float32)
    bias = rng.integers(-1000, 1001, size=OC).astype(np.int32)
    images = [rng.integers(0, 256, size=(N, Cin, H, W)).astype(np.uint8) for _ in range(2)]

    # operands in the layout the entry point documents; every device buffer is made here, once
    Kdim = Cin * K * K
    Kp = (Kdim + 15) // 16 * 16
    w8 = np.zeros((OC, Kp), np.int8)
    w8[:, :Kdim] = weights.reshape(OC, Kdim)
    bias_full = (bias.astype(np.int64) - IN_ZP * weights.reshape(OC, -1).astype(np.int64).sum(axis=1)).astype(np.int32)
    acc_scale = (np.float32(IN_SCALE) * wscales).astype(np.float32)
    Ho = (H + 2 * PAD - K) // STRIDE + 1
    Wo = (W + 2 * PAD - K) // STRIDE + 1
    dev = torch.device("cuda:0")
    d_w8 = torch.from_numpy(w8).to(dev)
    d_bias = torch.from_numpy(bias_full).to(dev)
    d_scale = torch.from_numpy(acc_scale).to(dev)
    d_x = torch.empty(N * Cin * H * W, dtype=torch.uint8, device=dev)
    d_y = torch.empty(N * Ho * Wo * OC, dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()

    desc = NoAllocDesc()
    desc.n, desc.h, desc.w, desc.c = N, H, W, Cin
    desc.kw, desc.kh, desc.oc = K, K, OC
    desc.stride[:] = (STRIDE, STRIDE)
    desc.dilation[:] = (1, 1)
    desc.pad[:] = (PAD, PAD, PAD, PAD)
    desc.in_zero_point, desc.out_scale, desc.out_zero_point = IN_ZP, OUT_SCALE, OUT_ZP
    err = C.create_string_buffer(256)

    for image in images:   # two calls in a row share the built-in scratch array
        want, kernels = reference_conv(product_lib, weights, wscales, bias, image)
        d_x.copy_(torch.from_numpy(image.reshape(-1)))
        d_y.fill_(0xAB)
        torch.cuda.synchronize()
        st = fn(C.byref(desc), d_x.data_ptr(), d_w8.data_ptr(), d_bias.data_ptr(), d_scale.data_ptr(), d_y.data_ptr(), None,
                err, len(err))
        assert st == 0, err.value.decode()
        got = d_y.cpu().numpy().reshape(N, Ho, Wo, OC).transpose(0, 3, 1, 2)
        assert want.shape == got.shape
        assert np.array_equal(want, got), "%d of %d bytes differ" % (np.count_nonzero(want != got), want.size)
        assert any("gemm_i8_tc" in k for k in kernels)

    # larger than the built-in scratch: refused with a message, nothing launched
    big = NoAllocDesc.from_buffer_copy(desc)
    big.n, big.h, big.w = 64, 224, 224
    st = fn(C.byref(big), d_x.data_ptr(), d_w8.data_ptr(), d_bias.data_ptr(), d_scale.data_ptr(), d_y.data_ptr(), None, err, len(err))
    assert st == 1 and b"scratch" in err.value
