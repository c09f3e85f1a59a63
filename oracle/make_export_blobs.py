#!/usr/bin/env python3
"""Stand-in coefficient files for the reference's exported MobileNet and ResNet-50 graphs.

samples/multi_device/vx_mobilenet.cc and vx_resnet50.cc read their weights from mobilenet.export.data and
resnet50.export.data, which are not in the reference tree.  This script reads the two generated sources (as text),
finds every constant tensor (its data type, its zero point and its offset into the file), and writes files of the
length the constructors read: for the uint8 weights seeded bytes spread normally (sigma 12) around the tensor's zero
point, for the biases seeded int32 values in [-200, 200] (uniform random bytes would drive every layer into
saturation and leave a constant output, which pins nothing).  It also copies LeNet's real coefficient file and
the three input images next to them.  Output goes to oracle/_ref/export_data/ (not tracked; it travels to the GPU box
with the built binaries).  tests/test_reference_samples.py runs tests/cpp/exported_graphs.cc on these files.

usage: python oracle/make_export_blobs.py --reference <TIM-VX source tree>
"""
import argparse
import os
import re
import shutil

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def blob_for(source_path, seed):
    text = open(source_path).read()
    # tim::vx::TensorSpec <name>_spec(tim::vx::DataType::<T>, <name>_shape, ...CONSTANT...);  ... CreateTensor(<name>_spec, coef_data_ptr + <off>)
    dtype = dict(re.findall(r"TensorSpec (\w+)_spec\(tim::vx::DataType::(\w+),", text))
    shapes = {}
    for name, dims in re.findall(r"ShapeType (\w+)_shape\(\{([^}]*)\}\)", text):
        shapes[name] = [int(v) for v in dims.replace(" ", "").split(",") if v]
    consts = re.findall(r"CreateTensor\((\w+)_spec, coef_data_ptr \+ (\d+)\)", text)
    zero_point = {n: int(z) for n, z in re.findall(r"Quantization (\w+)_quant\(tim::vx::QuantType::ASYMMETRIC,\s*[-0-9.e+]+,\s*(-?\d+)\)", text)}
    rng = np.random.default_rng(seed)
    end = 0
    pieces = []
    for name, off in consts:
        off = int(off)
        n = int(np.prod(shapes[name]))
        if dtype[name] == "INT32":
            data = rng.integers(-200, 201, size=n).astype("<i4").tobytes()
        elif dtype[name] == "UINT8":
            data = np.clip(np.rint(rng.normal(zero_point.get(name, 128), 12.0, size=n)), 0, 255).astype(np.uint8).tobytes()
        else:
            raise SystemExit("%s: constant %s has data type %s" % (source_path, name, dtype[name]))
        pieces.append((off, data))
        end = max(end, off + len(data))
    blob = bytearray(end)
    for off, data in pieces:
        blob[off:off + len(data)] = data
    return bytes(blob), len(consts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    src = os.path.join(args.reference, "samples", "multi_device")
    out = os.path.join(HERE, "_ref", "export_data")
    os.makedirs(out, exist_ok=True)
    for net, seed in (("mobilenet", 11), ("resnet50", 12)):
        blob, n = blob_for(os.path.join(src, "vx_%s.cc" % net), seed)
        with open(os.path.join(out, "%s.export.data" % net), "wb") as f:
            f.write(blob)
        print("%s.export.data: %d constants, %d bytes" % (net, n, len(blob)))
    for rel in ("lenet/lenet.export.data", "lenet/lenet_input_1_1_28_28_uint8.bin", "mobilenet/mobilenet_1_224_224_3_uint8.bin",
                "resnet50/resnet50_1_3_224_224_uint8.bin"):
        shutil.copyfile(os.path.join(src, rel), os.path.join(out, os.path.basename(rel)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
