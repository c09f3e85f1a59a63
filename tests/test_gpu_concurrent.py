"""Graph replicas in flight together: what bench.py's device-resident figure and its end-to-end loop rely on.

Three replicas of one graph (a 1x1 convolution with a fused residual Add, a 3x3 convolution, max and average pooling and a
FullyConnected: every kernel family of the networks), each on its own CUDA stream with its own input, are replayed
interleaved many times without waiting in between; afterwards every replica's outputs must equal the CPU oracle's for
that replica's input, bit for bit."""
import numpy as np
import pytest

import graph_cases as G
import pyb2vx as B

pytestmark = pytest.mark.gpu


def block(g, rng):
    C1, C2, W, H, N = 64, 256, 28, 28, 4

    def conv(x, kw, cin, cout, out_attr=B.ATTR_TRANSIENT, s_in=0.02):
        ws = rng.uniform(0.001, 0.01, cout).astype(np.float32)
        w = g.tensor(B.DT_INT8, [kw, kw, cin, cout], B.ATTR_CONSTANT, scales=ws, channel_dim=3,
                     data=rng.integers(-127, 128, size=(cout, cin, kw, kw)).astype(np.int8))
        b = g.tensor(B.DT_INT32, [cout], B.ATTR_CONSTANT, scales=np.float32(s_in) * ws, channel_dim=0,
                     data=rng.integers(-1000, 1001, size=cout).astype(np.int32))
        y = g.tensor(B.DT_UINT8, [], out_attr, scale=0.05, zero_point=3)
        g.conv2d(x, w, b, y, pad_type=B.PAD_SAME)
        return y

    x = g.tensor(B.DT_UINT8, [W, H, C2, N], B.ATTR_INPUT, scale=0.02, zero_point=128)
    r = conv(x, 1, C2, C1)                       # reduce
    m = conv(r, 3, C1, C1, s_in=0.05)            # 3x3, implicit GEMM with border classes
    e = conv(m, 1, C1, C2, s_in=0.05)            # expand; the Add below runs in its epilogue
    s = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT, scale=0.06, zero_point=10)
    g.add(e, x, s)
    a = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=0.06, zero_point=10)
    g.relu(s, a)
    p = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT, scale=0.06, zero_point=10)
    g.pool2d(a, p, B.POOL_MAX, (3, 3), (2, 2), pad=(1, 1, 1, 1))
    q = g.tensor(B.DT_UINT8, [], B.ATTR_TRANSIENT, scale=0.06, zero_point=10)
    g.pool2d(p, q, B.POOL_AVG, (14, 14), (14, 14))
    fw = g.tensor(B.DT_INT8, [C2, 40], B.ATTR_CONSTANT, scales=[0.004] * 40, channel_dim=1,
                  data=rng.integers(-127, 128, size=(40, C2)).astype(np.int8))
    y = g.tensor(B.DT_UINT8, [], B.ATTR_OUTPUT, scale=0.1, zero_point=128)
    g.fully_connected(q, fw, None, y, axis=2, weights=40)
    return x, [a, y], (N, C2, H, W)


def make(lib, seed):
    g = B.Graph(lib, 0)
    x, outs, shape = block(g, np.random.default_rng(seed))   # same seed: same weights in every replica
    g.compile()
    return g, x, outs, shape


def test_three_replicas_in_flight_equal_the_oracle(oracle_lib, product_lib):
    import torch
    replicas = [make(product_lib, 5) for _ in range(3)]
    streams = [torch.cuda.Stream() for _ in replicas]
    rng = np.random.default_rng(77)
    images = [rng.integers(0, 256, size=replicas[0][3]).astype(np.uint8) for _ in replicas]
    for (g, x, _, _), st, img in zip(replicas, streams, images):
        g.set_stream(st.cuda_stream)
        g.write(x, img)
    for _ in range(40):
        for g, _, _, _ in replicas:
            g.run_async()
    for g, _, _, _ in replicas:
        g.sync()
    names = [k["name"] for k in replicas[0][0].kernels()]
    assert any("+add" in n for n in names), names
    got = [[g.read(t) for t in outs] for g, _, outs, _ in replicas]
    for g, _, _, _ in replicas:
        g.close()
    og, ox, oouts, _ = make(oracle_lib, 5)
    for img, mine in zip(images, got):
        og.write(ox, img)
        og.run()
        G.assert_same([og.read(t) for t in oouts], mine)
    og.close()
    assert not np.array_equal(got[0][1], got[1][1]), "different inputs must give different outputs"
