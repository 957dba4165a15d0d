"""Runs the synthetic MobileNetV2-u8 graph layer by layer through the CPU oracle.  TEST INFRASTRUCTURE ONLY (tests,
the smoke test and the benchmark's CPU legs); `types` is the module that provides the C-ABI descriptors
(abi_types, or the loaded package) and `mobilenet` the graph module (layer_descs)."""
from . import orc


def run_oracle(layers, x, keep=False, types=None, mobilenet=None):
    """x: uint8 [N][R][R][3].  Returns the final logits (uint8 [N][classes]) and optionally every activation."""
    acts = {"input": x}
    n = x.shape[0]
    for L in layers:
        d = mobilenet.layer_descs(types, L, n)
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
    out = acts[layers[-1]["name"]]
    return (out, acts) if keep else out
