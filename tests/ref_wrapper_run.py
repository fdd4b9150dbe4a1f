"""Child process of tests/test_gpu_reference_wrappers.py: replays one graph's runtime-call
program through the reference's own wrappers (oracle/_ref, cuDNN / cuBLASLt behind the
reference's unchanged code) and writes the outputs to an .npz file.  A process of its own so
that the parent can set library switches (NVIDIA_TF32_OVERRIDE=0: cuDNN and cuBLAS keep fp32
convolutions and GEMMs off the TF32 tensor cores) in its environment before any CUDA library
initialises.

    python tests/ref_wrapper_run.py <graph> <batch> <image> <fuse> <workspace_bytes> <out.npz>
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def build_graph(name, batch, image):
    from occamy_b200 import graphs
    if name == "single_conv":
        return graphs.single_conv(seed=0), "uniform"
    if name == "resnet50":
        return graphs.resnet50(batch=batch, seed=0, softmax=False, image=image), "normal"
    if name == "mobilenet_v2":
        return graphs.mobilenet_v2(batch=batch, seed=0, image=image), "normal"
    if name == "vgg16":
        return graphs.vgg16(batch=batch, seed=0, image=image, num_classes=100), "normal"
    if name == "avgpool_padded":
        # 1x1 convolution, then a 3x3 / stride 2 average pool whose windows overhang the image
        g = graphs.Graph((batch, 16, image, image), 0)
        g.name = name
        w, b = g.he_conv(16, 16, 1, 1)
        y = g.avgpool(g.conv(0, w, b), (3, 3), (1, 1), (2, 2))
        g.mark_output(y)
        return g, "normal"
    if name == "depthwise_clip":
        # the unfused MobileNetV2 sequence: grouped convolution, bias add, Clip
        g = graphs.Graph((batch, 32, image, image), 0)
        g.name = name
        w, b = g.he_conv(32, 1, 3, 3)
        y = g.clip(g.conv(0, w, b, groups=32, pads=(1, 1), strides=(2, 2)), 0.0, 6.0)
        g.mark_output(y)
        return g, "normal"
    if name == "softmax_head":
        # Gemm + softmax on logits of ordinary magnitude
        g = graphs.Graph((batch, 64, 1, 1), 0)
        g.name = name
        x = g.flatten(0)
        w = (g.rng.normal(0, 1.0 / 8.0, (10, 64))).astype(np.float32)
        b = g.rng.normal(0, 0.1, (10,)).astype(np.float32)
        y = g.softmax(g.gemm(x, w, b), 1)
        g.mark_output(y)
        return g, "normal"
    raise SystemExit(f"unknown graph {name}")


def main():
    name, batch, image, fuse, ws, out = sys.argv[1:7]
    from occamy_b200 import graphs, replay
    from oracle import build as obuild
    g, dist = build_graph(name, int(batch), int(image))
    x = graphs.make_input(g, 0, dist)
    p = g.to_program()
    p.lower(fuse=int(fuse), workspace_bytes=int(ws))
    binding = replay.Binding(obuild.REF_SO)
    outs = p.run(binding, x)
    np.savez(out, *outs)


if __name__ == "__main__":
    main()
