"""Generates tests/golden/quant_host.json from the REFERENCE's own host code (oracle/_ref/libennref.so,
built by oracle/Makefile from the reference tree).  Run where the reference tree is mounted:

    make -C oracle && python tests/golden/gen_quant_host.py

The fixture pins QuantizeMultiplierSmallerThanOneExp, GetQuantizedConvolutionMultipler,
CalculateActivationRange{Uint8,Int8}, gemmlowp SaturatingRoundingDoublingHighMul / RoundingDivideByPOT and
MultiplyByQuantizedMultiplier on seeded random inputs plus hand-picked edge cases.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import orc  # noqa: E402

assert orc.ref is not None, "oracle/_ref/libennref.so is missing (needs the reference tree)"
rng = np.random.default_rng(20240611)
f32 = lambda v: float(np.float32(v))

out = {}
ms = [0.0, 0.25, 0.5, 1.0, 0.9999999999, 0.99999999999999, 2.0, 0.002, 1e-9] + \
     [float(np.exp(rng.uniform(np.log(1e-7), np.log(16.0)))) for _ in range(300)]
out["quantize_multiplier"] = [[m, *orc.quantize_multiplier(m, orc.ref)] for m in ms]

cm = []
for _ in range(200):
    a, b, o = (f32(np.exp(rng.uniform(np.log(1e-3), np.log(1.0)))) for _ in range(3))
    kind = rng.integers(0, 4)
    if kind == 0:
        bs = float(np.float32(a) * np.float32(b))          # float product, as the per-channel operators pass
    elif kind == 1:
        bs = float(a) * float(b)
    elif kind == 2:
        bs = float(a) * float(b) * (1 + rng.uniform(-3e-6, 3e-6))
    else:
        bs = f32(rng.uniform(1e-4, 1.0))
    st, m = orc.conv_multiplier(float(a), float(b), bs, float(o), orc.ref)
    cm.append([float(a), float(b), bs, float(o), st, m])
out["conv_multiplier"] = cm

ar = []
for _ in range(300):
    act = int(rng.integers(0, 4))
    dt = int(rng.integers(0, 2))
    scale = f32(np.exp(rng.uniform(np.log(1e-3), np.log(0.5))))
    zp = int(rng.integers(-128, 128)) if dt else int(rng.integers(0, 256))
    ar.append([act, dt, scale, zp, *orc.activation_range(act, dt, scale, zp, orc.ref)])
for scale, zp in [(0.05, 128), (0.04, 0), (1.0, 128), (0.0235294122248888, 0)]:
    for act in range(4):
        ar.append([act, 0, f32(scale), zp, *orc.activation_range(act, 0, f32(scale), zp, orc.ref)])
out["activation_range"] = ar

I32 = (-2**31, 2**31 - 1)
edge = [0, 1, -1, 2, -2, 13, -13, 26, -26, 2**30, -2**30, 2**30 + 1, -(2**30) - 1, I32[0], I32[1], I32[0] + 1]
pairs = [(a, b) for a in edge for b in edge]
pairs += [(int(rng.integers(*I32)), int(rng.integers(2**30, 2**31))) for _ in range(300)]
pairs += [(int(rng.integers(-2**22, 2**22)), int(rng.integers(2**30, 2**31))) for _ in range(300)]
out["srdhm"] = [[a, b, orc.ref.ref_srdhm(a, b)] for a, b in pairs]

rd = []
for x in edge + [int(rng.integers(*I32)) for _ in range(200)] + [int(rng.integers(-4096, 4096)) for _ in range(200)]:
    for e in (0, 1, 2, 7, 8, 15, 30, 31) if abs(x) > 4096 else (0, 1, 2, 3, 4, 5):
        rd.append([x, e, orc.ref.ref_rdivpot(x, e)])
out["rdivpot"] = rd

mb = []
for _ in range(600):
    x = int(rng.integers(-2**24, 2**24))
    qm = int(rng.integers(2**30, 2**31))
    sh = int(rng.integers(-20, 4))
    if sh > 0 and abs(x) >= 2 ** (30 - sh):
        x >>= sh + 1                                  # keep x * 2^shift inside int32 (C++ signed overflow otherwise)
    mb.append([x, qm, sh, orc.ref.ref_multiply_by_quantized_multiplier(x, qm, sh)])
# the tie of the reference KAT: -26 * 0.25 = -6.5 -> -7
mb.append([-26, 2**30, -1, orc.ref.ref_multiply_by_quantized_multiplier(-26, 2**30, -1)])
out["multiply_by_quantized_multiplier"] = mb

path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_host.json")
with open(path, "w") as f:
    json.dump(out, f, separators=(",", ":"))
print(path, os.path.getsize(path), "bytes", {k: len(v) for k, v in out.items()})
