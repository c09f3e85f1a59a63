"""Test infrastructure: where the CPU oracle's libraries are, and the loader of the fixture cases
(tests/golden/reference_cases.json) recorded from the reference's own unit tests.

Only tests/, __graft_entry__.smoke() and the cpu_baseline / reference arm of bench.py import this module: the
oracle is the checker, never the thing shipped or measured as the product.
"""
import base64
import os
import sys
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tim-vx_b200"))

from pyb2vx import *   # noqa: E402,F401,F403 - the fixture loader speaks the binding's vocabulary
from pyb2vx import Graph, NP_DTYPE   # noqa: E402

ORACLE_LIB = os.path.join(ROOT, "oracle", "_build", "libb2vx_oracle.so")
ORACLE_OPS_LIB = os.path.join(ROOT, "oracle", "_build", "liboracle_ops.so")

def unpack(b64, dtype):
    return np.frombuffer(zlib.decompress(base64.b64decode(b64)), dtype=NP_DTYPE[dtype])


def graph_from_case(lib, case, device=0):
    """Rebuild the graph of one fixture case.  Returns (graph, inputs, expectations):
    inputs is a list of (tensor id, array) to write before running, expectations a
    list of (tensor id, expected array, tolerance)."""
    g = Graph(lib, device)
    ids = []
    inputs = []
    for t in case["tensors"]:
        declared = t["declared_rank"] > 0
        dims = t["dims"] if declared else []
        kw = {}
        if t["quant_type"] == Q_PER_CHANNEL:
            kw = dict(scales=t["scales"], zero_points=t["zero_points"] or None, channel_dim=t["channel_dim"])
        elif t["quant_type"] == Q_ASYM:
            kw = dict(scale=t["scale"], zero_point=t["zero_point"], channel_dim=t["channel_dim"])
        data = None
        if t["data"] is not None and (t["attr"] & ATTR_CONSTANT):
            data = unpack(t["data"], t["dtype"])
        tid = g.tensor(t["dtype"], dims, t["attr"], data=data, **kw)
        ids.append(tid)
        if t["data"] is not None and (t["attr"] & ATTR_INPUT):
            inputs.append((tid, unpack(t["data"], t["dtype"])))
    for n in case["nodes"]:
        i = [ids[v] if v != NO_TENSOR else None for v in n["in"]]
        o = ids[n["out"]]
        k = n["kind"]
        if k == NODE_CONV2D:
            g.conv2d(i[0], i[1], i[2], o, stride=n["stride"], dilation=n["dilation"], pad_type=n["pad_type"],
                     pad=n["pad"], multiplier=n["multiplier"], weights=n["weights"], ksize=n["ksize"], group=n.get("group", 0))
        elif k == NODE_FC:
            g.fully_connected(i[0], i[1], i[2], o, axis=n["axis"], weights=n["weights"])
        elif k == NODE_POOL2D:
            g.pool2d(i[0], o, n["type"], n["ksize"], n["stride"], pad_type=n["pad_type"], pad=n["pad"],
                     round_type=n["round_type"])
        elif k == NODE_ADD:
            g.add(i[0], i[1], o)
        elif k == NODE_RELU:
            g.relu(i[0], o)
        elif k == NODE_RELU6:
            g.relu6(i[0], o)
        elif k == NODE_SOFTMAX:
            g.softmax(i[0], o, beta=n["beta"], axis=n["axis"])
        elif k == NODE_RESHAPE:
            g.reshape(i[0], o, n["dims"])
        elif k == NODE_TRANSPOSE:
            g.transpose(i[0], o, n["dims"])
        elif k == NODE_CONCAT:
            g.concat([v for v in i if v is not None], o, n["axis"])
        elif k == NODE_DATACONVERT:
            g.dataconvert(i[0], o)
        elif k == NODE_ADDN:
            g.addn([v for v in i if v is not None], o)
        else:
            raise ValueError("unknown node kind %r" % k)
    expects = [(ids[e["tensor"]], unpack(e["data"], e["dtype"]), e["tol"]) for e in case["expect"]]
    oracle_out = {ids[t["id"]]: unpack(t["data"], t["dtype"]) for t in case["tensors"]
                  if t["data"] is not None and (t["attr"] & ATTR_OUTPUT)}
    return g, inputs, expects, oracle_out
