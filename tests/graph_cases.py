"""Seeded single-op and small-network graphs used by the parity tests.

Every builder takes a pyb2vx.Graph and a numpy Generator and returns
(inputs, outputs): inputs = list of (tensor id, array to write), outputs = list
of tensor ids to compare.  The same builder is run on the oracle library and on
the CUDA library, so both see identical bytes.
"""
import numpy as np

import pyb2vx as B


def run_case(lib, build, seed, device=0, env=None):
    rng = np.random.default_rng(seed)
    g = B.Graph(lib, device)
    try:
        inputs, outputs = build(g, rng)
        g.compile()
        for tid, arr in inputs:
            g.write(tid, arr)
        g.run()
        return [g.read(t) for t in outputs], g.kernels()
    finally:
        g.close()


def assert_same(oracle_out, gpu_out, float_tol=0.0):
    assert len(oracle_out) == len(gpu_out)
    for a, b in zip(oracle_out, gpu_out):
        assert a.shape == b.shape and a.dtype == b.dtype
        if a.dtype == np.float32 and float_tol > 0:
            np.testing.assert_allclose(b, a, rtol=0, atol=float_tol)
        else:
            bad = np.flatnonzero(a.reshape(-1).view(np.uint8 if a.dtype.itemsize == 1 else np.uint32) !=
                                 b.reshape(-1).view(np.uint8 if a.dtype.itemsize == 1 else np.uint32))
            assert bad.size == 0, "%d of %d elements differ, first at %d: oracle %r gpu %r" % (
                bad.size, a.size, bad[0], a.reshape(-1)[bad[0]], b.reshape(-1)[bad[0]])


def _act(rng, dims, dtype=B.DT_UINT8):
    lo, hi = (0, 256) if dtype == B.DT_UINT8 else (-128, 128)
    return rng.integers(lo, hi, size=dims[::-1], dtype=np.int64).astype(B.NP_DTYPE[dtype])


def conv2d_q(W, H, C, N, kw, kh, Oc, stride=(1, 1), dilation=(1, 1), pad_type=B.PAD_SAME, pad=(0, 0, 0, 0),
             x_dtype=B.DT_UINT8, w_kind="s8pc", in_q=(0.02, 128), out_q=(0.05, 0), bias=True, relu=False,
             out_dtype=B.DT_UINT8):
    """Quantized dense convolution.  w_kind: 's8pc' per-channel int8 (scales U(0.001,0.01)),
    'u8' asymmetric uint8 (scale 0.01, zp drawn in [100,156]), 'u8z128' uint8 zp 128, 's8' per-tensor int8 zp 0."""
    def build(g, rng):
        x = g.tensor(x_dtype, [W, H, C, N], B.ATTR_INPUT, scale=in_q[0], zero_point=in_q[1])
        wshape = [kw, kh, C, Oc]
        if w_kind == "s8pc":
            ws = rng.uniform(0.001, 0.01, Oc).astype(np.float32)
            wd = rng.integers(-127, 128, size=wshape[::-1]).astype(np.int8)
            w = g.tensor(B.DT_INT8, wshape, B.ATTR_CONSTANT, scales=ws, channel_dim=3, data=wd)
            bscale = dict(scales=(np.float32(in_q[0]) * ws), channel_dim=0)
        elif w_kind == "s8":
            wd = rng.integers(-127, 128, size=wshape[::-1]).astype(np.int8)
            w = g.tensor(B.DT_INT8, wshape, B.ATTR_CONSTANT, scale=0.005, zero_point=0, data=wd)
            bscale = dict(scale=float(np.float32(in_q[0]) * np.float32(0.005)), zero_point=0)
        else:
            zw = 128 if w_kind == "u8z128" else int(rng.integers(100, 157))
            wd = rng.integers(0, 256, size=wshape[::-1]).astype(np.uint8)
            w = g.tensor(B.DT_UINT8, wshape, B.ATTR_CONSTANT, scale=0.01, zero_point=zw, data=wd)
            bscale = dict(scale=float(np.float32(in_q[0]) * np.float32(0.01)), zero_point=0)
        b = None
        if bias:
            bd = rng.integers(-1000, 1001, size=Oc).astype(np.int32)
            b = g.tensor(B.DT_INT32, [Oc], B.ATTR_CONSTANT, data=bd, **bscale)
        if relu:
            y = g.tensor(out_dtype, [], B.ATTR_TRANSIENT, scale=out_q[0], zero_point=out_q[1])
            z = g.tensor(out_dtype, [], B.ATTR_OUTPUT, scale=out_q[0], zero_point=out_q[1])
        else:
            y = g.tensor(out_dtype, [], B.ATTR_OUTPUT, scale=out_q[0], zero_point=out_q[1])
            z = y
        g.conv2d(x, w, b, y, stride=stride, dilation=dilation, pad_type=pad_type, pad=pad)
        if relu:
            g.relu(y, z)
        return [(x, _act(rng, [W, H, C, N], x_dtype))], [z]
    return build


def depthwise_q(W, H, C, N, kw, kh, multiplier=1, stride=(1, 1), pad_type=B.PAD_SAME, w_kind="u8", in_q=(0.03, 120),
                out_q=(0.06, 0), relu6=True, x_dtype=B.DT_UINT8, pad=(0, 0, 0, 0)):
    def build(g, rng):
        Oc = C * multiplier
        x = g.tensor(x_dtype, [W, H, C, N], B.ATTR_INPUT, scale=in_q[0], zero_point=in_q[1])
        wshape = [kw, kh, Oc, 1]
        if w_kind == "s8pc":
            ws = rng.uniform(0.001, 0.01, Oc).astype(np.float32)
            wd = rng.integers(-127, 128, size=wshape[::-1]).astype(np.int8)
            w = g.tensor(B.DT_INT8, wshape, B.ATTR_CONSTANT, scales=ws, channel_dim=2, data=wd)
            bq = dict(scales=np.float32(in_q[0]) * ws, channel_dim=0)
        else:
            zw = int(rng.integers(100, 157))
            wd = rng.integers(0, 256, size=wshape[::-1]).astype(np.uint8)
            w = g.tensor(B.DT_UINT8, wshape, B.ATTR_CONSTANT, scale=0.02, zero_point=zw, data=wd)
            bq = dict(scale=float(np.float32(in_q[0]) * np.float32(0.02)), zero_point=0)
        b = g.tensor(B.DT_INT32, [Oc], B.ATTR_CONSTANT, data=rng.integers(-500, 501, size=Oc).astype(np.int32), **bq)
        y = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT if relu6 else B.ATTR_OUTPUT, scale=out_q[0], zero_point=out_q[1])
        g.conv2d(x, w, b, y, stride=stride, pad_type=pad_type, pad=pad, multiplier=multiplier)
        z = y
        if relu6:
            z = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=out_q[0], zero_point=out_q[1])
            g.relu6(y, z)
        return [(x, _act(rng, [W, H, C, N], x_dtype))], [z]
    return build


def fc_q(K, N_out, batch, w_kind="s8pc", in_q=(0.02, 128), out_q=(0.1, 100), from_4d=None):
    """from_4d = (W,H,C): feed a 4-D tensor and flatten with axis 2 (K must equal W*H*C)."""
    def build(g, rng):
        if from_4d:
            dims = list(from_4d) + [batch]
            axis = 2
        else:
            dims = [K, batch]
            axis = 0
        x = g.tensor(B.DT_UINT8, dims, B.ATTR_INPUT, scale=in_q[0], zero_point=in_q[1])
        if w_kind == "s8pc":
            ws = (rng.uniform(0.001, 0.01, N_out) / np.sqrt(K / 64.0)).astype(np.float32)
            wd = rng.integers(-127, 128, size=(N_out, K)).astype(np.int8)
            w = g.tensor(B.DT_INT8, [K, N_out], B.ATTR_CONSTANT, scales=ws, channel_dim=1, data=wd)
            bq = dict(scales=np.float32(in_q[0]) * ws, channel_dim=0)
        else:
            zw = 128 if w_kind == "u8z128" else int(rng.integers(100, 157))
            wd = rng.integers(0, 256, size=(N_out, K)).astype(np.uint8)
            w = g.tensor(B.DT_UINT8, [K, N_out], B.ATTR_CONSTANT, scale=0.002, zero_point=zw, data=wd)
            bq = dict(scale=float(np.float32(in_q[0]) * np.float32(0.002)), zero_point=0)
        b = g.tensor(B.DT_INT32, [N_out], B.ATTR_CONSTANT, data=rng.integers(-1000, 1001, size=N_out).astype(np.int32), **bq)
        y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=out_q[0], zero_point=out_q[1])
        g.fully_connected(x, w, b, y, axis=axis, weights=N_out)
        return [(x, _act(rng, dims))], [y]
    return build


def pool_q(W, H, C, N, type, ksize, stride, pad=(0, 0, 0, 0), round_type=B.ROUND_FLOOR, in_q=(0.05, 3), out_q=None,
           dtype=B.DT_UINT8):
    def build(g, rng):
        oq = out_q or in_q
        x = g.tensor(dtype, [W, H, C, N], B.ATTR_INPUT, scale=in_q[0], zero_point=in_q[1])
        y = g.tensor(dtype, [], B.ATTR_OUTPUT, scale=oq[0], zero_point=oq[1])
        g.pool2d(x, y, type, ksize, stride, pad=pad, round_type=round_type)
        return [(x, _act(rng, [W, H, C, N], dtype))], [y]
    return build


def add_q(dims, qa=(0.02, 128), qb=(0.035, 117), qo=(0.05, 120), relu=False):
    def build(g, rng):
        a = g.tensor(B.DT_UINT8, dims, B.ATTR_INPUT, scale=qa[0], zero_point=qa[1])
        b = g.tensor(B.DT_UINT8, dims, B.ATTR_INPUT, scale=qb[0], zero_point=qb[1])
        y = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT if relu else B.ATTR_OUTPUT, scale=qo[0], zero_point=qo[1])
        g.add(a, b, y)
        z = y
        if relu:
            z = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=qo[0], zero_point=qo[1])
            g.relu(y, z)
        return [(a, _act(rng, dims)), (b, _act(rng, dims))], [z]
    return build


def relu_q(dims, six=False, qi=(0.04, 110), qo=(0.03, 5)):
    def build(g, rng):
        x = g.tensor(B.DT_UINT8, dims, B.ATTR_INPUT, scale=qi[0], zero_point=qi[1])
        y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=qo[0], zero_point=qo[1])
        (g.relu6 if six else g.relu)(x, y)
        return [(x, _act(rng, dims))], [y]
    return build


def softmax_q(classes, batch, beta=1.0):
    def build(g, rng):
        x = g.tensor(B.DT_UINT8, [classes, batch], B.ATTR_INPUT, scale=0.05, zero_point=128)
        y = g.tensor(B.DT_FLOAT32, [classes, batch], B.ATTR_OUTPUT)
        g.softmax(x, y, beta=beta, axis=0)
        return [(x, _act(rng, [classes, batch]))], [y]
    return build


def lenet_synthetic(batch):
    """LeNet-5 as in the reference sample (samples/lenet/lenet_asymu8.cc:115-290) with the
    synthetic quantization of the benchmark configuration: input scale 1/255 zp 0, weights
    uint8 scale 0.01 zp 128, int32 bias in [-1000,1000], every activation scale 0.05 zp 128."""
    def build(g, rng):
        def qt(dims, attr, s, z, data=None, dtype=B.DT_UINT8):
            return g.tensor(dtype, dims, attr, scale=s, zero_point=z, data=data)
        si = 1.0 / 255.0
        x = qt([28, 28, 1, batch], B.ATTR_INPUT, si, 0)

        def conv_w(kw, kh, ic, oc, s_in):
            w = qt([kw, kh, ic, oc], B.ATTR_CONSTANT, 0.01, 128, rng.integers(0, 256, size=(oc, ic, kh, kw)).astype(np.uint8))
            b = qt([oc], B.ATTR_CONSTANT, float(np.float32(s_in) * np.float32(0.01)), 0,
                   rng.integers(-1000, 1001, size=oc).astype(np.int32), dtype=B.DT_INT32)
            return w, b

        def act():
            return qt([], B.ATTR_TRANSIENT, 0.05, 128)
        w1, b1 = conv_w(5, 5, 1, 20, si)
        c1 = act(); g.conv2d(x, w1, b1, c1, pad_type=B.PAD_VALID, weights=20, ksize=(5, 5))
        p1 = act(); g.pool2d(c1, p1, B.POOL_MAX, (2, 2), (2, 2), pad_type=B.PAD_NONE)
        w2, b2 = conv_w(5, 5, 20, 50, 0.05)
        c2 = act(); g.conv2d(p1, w2, b2, c2, pad_type=B.PAD_VALID, weights=50, ksize=(5, 5))
        p2 = act(); g.pool2d(c2, p2, B.POOL_MAX, (2, 2), (2, 2), pad_type=B.PAD_NONE)
        w3 = qt([800, 500], B.ATTR_CONSTANT, 0.01, 128, rng.integers(0, 256, size=(500, 800)).astype(np.uint8))
        b3 = qt([500], B.ATTR_CONSTANT, float(np.float32(0.05) * np.float32(0.01)), 0,
                rng.integers(-1000, 1001, size=500).astype(np.int32), dtype=B.DT_INT32)
        f3 = act(); g.fully_connected(p2, w3, b3, f3, axis=2, weights=500)
        r3 = act(); g.relu(f3, r3)
        w4 = qt([500, 10], B.ATTR_CONSTANT, 0.01, 128, rng.integers(0, 256, size=(10, 500)).astype(np.uint8))
        b4 = qt([10], B.ATTR_CONSTANT, float(np.float32(0.05) * np.float32(0.01)), 0,
                rng.integers(-1000, 1001, size=10).astype(np.int32), dtype=B.DT_INT32)
        f4 = qt([], B.ATTR_OUTPUT, 0.05, 128); g.fully_connected(r3, w4, b4, f4, axis=0, weights=10)
        out = g.tensor(B.DT_FLOAT32, [10, batch], B.ATTR_OUTPUT)
        g.softmax(f4, out, beta=1.0, axis=0)
        return [(x, _act(rng, [28, 28, 1, batch]))], [f4, out]
    return build
