"""The oracle's MobileNetV2 runner bound to the loaded package (descriptors and graph module)."""
import importlib

from conftest import load_package
from oracle import mobilenet_ref as _m

enn = load_package()
mobilenet = importlib.import_module("cl_eden_kernel_b200.mobilenet")


def run_oracle(layers, x, keep=False):
    return _m.run_oracle(layers, x, keep=keep, types=enn, mobilenet=mobilenet)
