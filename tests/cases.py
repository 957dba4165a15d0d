"""Seeded synthetic operator cases shared by the CPU and GPU tests: the package's workload generators, bound to the
loaded library module (so that `cases.enn` carries both the descriptors and the operator calls)."""
import importlib

from conftest import load_package

enn = load_package()
_w = importlib.import_module("cl_eden_kernel_b200.workloads")
same_pad_tf = _w.same_pad_tf
conv_case = _w.conv_case
depthwise_case = _w.depthwise_case
deconv_case = _w.deconv_case
fc_out_scale = _w.fc_out_scale
fc_case = _w.fc_case
