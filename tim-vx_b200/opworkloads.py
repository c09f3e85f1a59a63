"""Single-operator workloads of the quantized path, built through the b2vx C ABI.

Four seeded families of shapes, each a graph around one compute node (plus the Relu the
convolution sweep fuses):

  conv:<k>:<cin>:<cout>:<hw>:<stride>   Conv2d k x k, SAME padding, uint8 input (scale 0.02,
                                         zero point 128), per-channel symmetric int8 weights with
                                         scales U(0.001, 0.01), int32 bias, Relu, uint8 output
                                         (scale 0.05, zero point 0); batch = images
  convadd:<k>:<cin>:<cout>:<hw>:<stride> the same convolution without its Relu, followed by the residual
                                         Add of a second uint8 input (scale 0.04, zero point 0) and a
                                         Relu: the tail of a ResNet bottleneck block
  gemm:<m>:<n>:<k>                       FullyConnected: uint8 [k, m] (zero point 128, scale 0.02)
                                         x int8 per-channel [k, n] -> uint8 [n, m]
  fcchain:<m>:<n>:<layers>               `layers` FullyConnected nodes of n x n weights in a row on m rows (the
                                         decode-like shapes as they occur in use: every layer streams its own
                                         weights, together more than the L2 holds, and the cost of launching the
                                         graph is shared by the layers)
  add:<elements>                         quantized Add of two uint8 tensors with different scales
  concat:<c1>:<c2>:<hw>                  Concat along the channel axis of two uint8 tensors [hw, hw, c, batch]
  transpose:<c>:<hw>                     Transpose {1,2,0,3} of a uint8 [c, hw, hw, batch] tensor (NHWC image -> WHCN)

build(spec, batch, graph, rng) adds the tensors and the node to `graph` (a pyb2vx.Graph on either
the CUDA library or the CPU oracle library) and returns a dict describing the work of one pass.
"""
import numpy as np

import pyb2vx as B


def parse(spec):
    f = spec.split(":")
    kind = f[0]
    nums = [int(v) for v in f[1:]]
    if kind in ("conv", "convadd") and len(nums) == 5:
        return kind, nums
    if kind == "gemm" and len(nums) == 3:
        return kind, nums
    if kind == "fcchain" and len(nums) == 3:
        return kind, nums
    if kind == "add" and len(nums) == 1:
        return kind, nums
    if kind == "concat" and len(nums) == 3:
        return kind, nums
    if kind == "transpose" and len(nums) == 2:
        return kind, nums
    raise ValueError("workload must be conv:k:cin:cout:hw:stride, convadd:k:cin:cout:hw:stride, gemm:m:n:k, fcchain:m:n:layers, add:elements, "
                     "concat:c1:c2:hw or transpose:c:hw, got %r" % spec)


def _u8(rng, shape):
    return rng.integers(0, 256, size=shape, dtype=np.uint8)


def build(spec, batch, g, rng):
    kind, v = parse(spec)
    if kind in ("conv", "convadd"):
        k, cin, cout, hw, stride = v
        x = g.tensor(B.DT_UINT8, [hw, hw, cin, batch], B.ATTR_INPUT, scale=0.02, zero_point=128)
        ws = rng.uniform(0.001, 0.01, cout).astype(np.float32)
        wd = rng.integers(-127, 128, size=(cout, cin, k, k)).astype(np.int8)
        w = g.tensor(B.DT_INT8, [k, k, cin, cout], B.ATTR_CONSTANT, scales=ws, channel_dim=3, data=wd)
        b = g.tensor(B.DT_INT32, [cout], B.ATTR_CONSTANT, scales=np.float32(0.02) * ws, channel_dim=0,
                     data=rng.integers(-1000, 1001, size=cout).astype(np.int32))
        ho = (hw + stride - 1) // stride
        macs = batch * ho * ho * cout * cin * k * k
        y = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT, scale=0.05, zero_point=0)
        z = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=0.05, zero_point=0)
        g.conv2d(x, w, b, y, stride=(stride, stride), pad_type=B.PAD_SAME)
        if kind == "convadd":
            r = g.tensor(B.DT_UINT8, [ho, ho, cout, batch], B.ATTR_INPUT, scale=0.04, zero_point=0)
            t = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT, scale=0.05, zero_point=0)
            g.add(y, r, t)
            g.relu(t, z)
            return {"inputs": [(x, _u8(rng, (batch, cin, hw, hw))), (r, _u8(rng, (batch, cout, ho, ho)))], "outputs": [z],
                    "ops": 2 * macs,
                    "bytes": batch * hw * hw * cin + 2 * batch * ho * ho * cout + cout * cin * k * k + 4 * cout,
                    "bound": "tensor", "units": batch,
                    "name": "Conv2d %dx%d %d->%d on %dx%d stride %d SAME + residual Add + Relu, batch %d" % (
                        k, k, cin, cout, hw, hw, stride, batch)}
        g.relu(y, z)
        return {"inputs": [(x, _u8(rng, (batch, cin, hw, hw)))], "outputs": [z], "ops": 2 * macs,
                "bytes": batch * hw * hw * cin + batch * ho * ho * cout + cout * cin * k * k + 4 * cout,
                "bound": "tensor", "units": batch,
                "name": "Conv2d %dx%d %d->%d on %dx%d stride %d SAME + Relu, batch %d" % (k, k, cin, cout, hw, hw, stride, batch)}
    if kind == "gemm":
        m, n, k = v
        x = g.tensor(B.DT_UINT8, [k, m], B.ATTR_INPUT, scale=0.02, zero_point=128)
        ws = (rng.uniform(0.001, 0.01, n) / np.sqrt(k / 64.0)).astype(np.float32)
        wd = rng.integers(-127, 128, size=(n, k)).astype(np.int8)
        w = g.tensor(B.DT_INT8, [k, n], B.ATTR_CONSTANT, scales=ws, channel_dim=1, data=wd)
        b = g.tensor(B.DT_INT32, [n], B.ATTR_CONSTANT, scales=np.float32(0.02) * ws, channel_dim=0,
                     data=rng.integers(-1000, 1001, size=n).astype(np.int32))
        y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=0.1, zero_point=100)
        g.fully_connected(x, w, b, y, axis=0, weights=n)
        return {"inputs": [(x, _u8(rng, (m, k)))], "outputs": [y], "ops": 2 * m * n * k,
                "bytes": m * k + n * k + m * n + 4 * n, "bound": "tensor" if m >= 512 else "hbm", "units": m,
                "name": "FullyConnected M=%d N=%d K=%d" % (m, n, k)}
    if kind == "fcchain":
        m, n, layers = v
        x = g.tensor(B.DT_UINT8, [n, m], B.ATTR_INPUT, scale=0.02, zero_point=128)
        cur = x
        for i in range(layers):
            ws = (rng.uniform(0.001, 0.01, n) / np.sqrt(n / 64.0)).astype(np.float32)
            wd = rng.integers(-127, 128, size=(n, n)).astype(np.int8)
            w = g.tensor(B.DT_INT8, [n, n], B.ATTR_CONSTANT, scales=ws, channel_dim=1, data=wd)
            b = g.tensor(B.DT_INT32, [n], B.ATTR_CONSTANT, scales=np.float32(0.02) * ws, channel_dim=0,
                         data=rng.integers(-1000, 1001, size=n).astype(np.int32))
            y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT if i == layers - 1 else B.ATTR_TRANSIENT, scale=0.02, zero_point=128)
            g.fully_connected(cur, w, b, y, axis=0, weights=n)
            cur = y
        return {"inputs": [(x, _u8(rng, (m, n)))], "outputs": [cur], "ops": 2 * m * n * n * layers,
                "bytes": layers * (2 * m * n + n * n + 4 * n), "bound": "hbm", "units": m * layers,
                "name": "%d FullyConnected layers in a row, M=%d N=K=%d" % (layers, m, n)}
    if kind == "concat":
        c1, c2, hw = v
        a = g.tensor(B.DT_UINT8, [hw, hw, c1, batch], B.ATTR_INPUT, scale=0.05, zero_point=0)
        b = g.tensor(B.DT_UINT8, [hw, hw, c2, batch], B.ATTR_INPUT, scale=0.05, zero_point=0)
        y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=0.05, zero_point=0)
        g.concat([a, b], y, 2)
        n = batch * hw * hw * (c1 + c2)
        return {"inputs": [(a, _u8(rng, (batch, c1, hw, hw))), (b, _u8(rng, (batch, c2, hw, hw)))], "outputs": [y], "ops": 0,
                "bytes": 2 * n, "bound": "hbm", "units": n,
                "name": "Concat of %d + %d channels on %dx%d, batch %d" % (c1, c2, hw, hw, batch)}
    if kind == "transpose":
        c, hw = v
        x = g.tensor(B.DT_UINT8, [c, hw, hw, batch], B.ATTR_INPUT, scale=0.0078125, zero_point=128)
        y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=0.0078125, zero_point=128)
        g.transpose(x, y, [1, 2, 0, 3])
        n = batch * hw * hw * c
        return {"inputs": [(x, _u8(rng, (batch, hw, hw, c)))], "outputs": [y], "ops": 0, "bytes": 2 * n, "bound": "hbm", "units": n,
                "name": "Transpose {1,2,0,3} of a %dx%dx%d image, batch %d" % (hw, hw, c, batch)}
    n = v[0]
    c = 256
    assert n % c == 0, "add: element count must be a multiple of 256"
    dims = [c, n // c]
    a = g.tensor(B.DT_UINT8, dims, B.ATTR_INPUT, scale=0.02, zero_point=128)
    b = g.tensor(B.DT_UINT8, dims, B.ATTR_INPUT, scale=0.035, zero_point=117)
    y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=0.05, zero_point=120)
    g.add(a, b, y)
    return {"inputs": [(a, _u8(rng, (n // c, c))), (b, _u8(rng, (n // c, c)))], "outputs": [y], "ops": 0,
            "bytes": 3 * n, "bound": "hbm", "units": n, "name": "quantized Add of %d uint8 elements" % n}


def cpu_sample(spec):
    """A bounded slice of `spec` for timing on host cores: (spec of the slice, description)."""
    kind, v = parse(spec)
    if kind == "gemm":
        m = min(v[0], 64)
        return "gemm:%d:%d:%d" % (m, v[1], v[2]), "%d of the %d rows per step" % (m, v[0])
    if kind == "fcchain":
        n = min(v[1], 2048)
        return "fcchain:%d:%d:%d" % (v[0], n, min(v[2], 2)), "%d layers of %d x %d weights per step" % (min(v[2], 2), n, n)
    if kind == "add":
        n = min(v[0], 1 << 24)
        return "add:%d" % n, "%d of the %d elements per step" % (n, v[0])
    return spec, "a reduced batch per step (--cpu-batch)"
