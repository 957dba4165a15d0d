"""Runs the synthetic MobileNetV2-u8 graph layer by layer through the CPU oracle (test infrastructure)."""
import numpy as np

from conftest import load_package
from oracle import orc

enn = load_package()
mobilenet = __import__("importlib").import_module("cl_eden_kernel_b200.mobilenet")


def run_oracle(layers, x, keep=False):
    """x: uint8 [N][R][R][3].  Returns the final logits (uint8 [N][classes]) and optionally every activation."""
    acts = {"input": x}
    n = x.shape[0]
    for L in layers:
        d = mobilenet.layer_descs(enn, L, n)
        a = acts[L["src"]]
        if L["kind"] == "conv":
            y = orc.conv2d(d, a, L["w"], L["bias"], L["scales"])
        elif L["kind"] == "dw":
            y = orc.depthwise(d, a, L["w"], L["bias"], L["scales"])
        elif L["kind"] == "fc":
            y = orc.fully_connected(d, a.reshape(n, -1), L["w"].reshape(L["cout"], L["cin"]), L["bias"], L["scales"])
        elif L["kind"] == "add":
            y = orc.add(d, a.reshape(-1), acts[L["src2"]].reshape(-1)).reshape(a.shape)
        else:
            y = orc.avgpool(d, a)
        acts[L["name"]] = y
        if not keep and L["kind"] != "add":
            pass
    out = acts[layers[-1]["name"]]
    return (out, acts) if keep else out
