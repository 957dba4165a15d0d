"""Generates tests/golden/ref_kernels.npz: outputs of the REFERENCE's own OpenCL C kernel text, compiled as C++
and run on the CPU (oracle/ref_kernels_shim.cpp -> oracle/_ref/libennref.so), on seeded inputs.

    make -C oracle && python tests/golden/gen_ref_kernels.py

Each entry stores only the expected output; inputs are regenerated from the seed by tests/cases.py, so the file
stays small.  Kernels covered: pad_opt + convert_optimized / convertBlocked2 + alignQuantizedWeight_gemm +
quantizedGemmBlocked (per-tensor u8 convolution), conv_per_channel_quantized, depthwise_conv (per-tensor u8), depthwise_conv_per_channel,
matrixTrans + convBackGemmRXR + convertBottomDiff2 (deconvolution, per-tensor and per-channel),
avepooling_tflite, eltwiseAddQuantized_opt.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import ref_cases  # noqa: E402
from oracle import orc  # noqa: E402

assert orc.has_ref_kernels(), "oracle/_ref/libennref.so with the kernel shim is missing (needs the reference tree)"
out = {}
for name, (kind, mk) in ref_cases.CASES.items():
    out[name] = ref_cases.run_reference(orc, kind, mk())
path = os.path.join(HERE, "ref_kernels.npz")
np.savez_compressed(path, **out)
print(path, os.path.getsize(path), "bytes", len(out), "cases")
