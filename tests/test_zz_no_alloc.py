"""The allocation-free entry point enn_b200_op_execute_noalloc against the regular enn_b200_op_execute.

Some hosts of this library may not allocate device memory once they are running (a latency-critical loop, or a
process that handed all device memory to another component).  For them the gathered-input convolutions can keep
their scratch matrix in a fixed array inside the library.  This file is collected last on purpose: if it fails,
a run that stops at the first failure has already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu


def _run_noalloc(enn, ctx, op, x):
    a = ctx.to_device(x)
    o = ctx.malloc(max(1, op.info.out_bytes))
    try:
        ctx.check(enn.lib.enn_b200_op_execute_noalloc(op.h, a, o))
        return ctx.download(o, (op.info.out_bytes,))
    finally:
        ctx.free(a)
        ctx.free(o)


@pytest.mark.parametrize("kind,kw", [
    ("conv", dict(n=2, h=20, w=20, cin=16, cout=32, k=3)),                                  # vector gather
    ("conv", dict(n=2, h=33, w=31, cin=3, cout=32, k=3, stride=2, per_channel=True, out_scale=0.1)),   # byte gather (stem-like)
    ("deconv", dict(n=1, h=12, w=12, cin=16, cout=16)),                                     # four parity classes share the array
])
def test_noalloc_matches_regular_entry_point_twice(enn, ctx, kind, kw):
    if kind == "conv":
        d, x, w, b, sc = cases.conv_case(seed=21, **kw)
        op = enn.conv2d(ctx, d, w, b, sc)
    else:
        d, x, w, b, sc = cases.deconv_case(seed=22, **kw)
        op = enn.deconv(ctx, d, w, b, sc)
    try:
        assert op.info.impl == enn.IMPL_TCGEN05
        x2 = np.ascontiguousarray(x[..., ::-1])          # a second, different input for the second call
        want1, want2 = op.run(x), op.run(x2)
        got1 = _run_noalloc(enn, ctx, op, x)             # two calls in a row share the static array
        got2 = _run_noalloc(enn, ctx, op, x2)
        assert np.array_equal(got1, want1)               # integer path: bit-exact, same as every other parity test
        assert np.array_equal(got2, want2)
        assert np.array_equal(op.run(x), want1)          # the regular path is unaffected afterwards
    finally:
        op.release()


def test_noalloc_rejects_what_it_cannot_hold(enn, ctx):
    # 64 x 112 x 112 outputs x 144 gathered bytes = 115 MB > 32 MiB
    d, x, w, b, sc = cases.conv_case(seed=1, n=64, h=112, w=112, cin=16, cout=16, k=3)
    op = enn.conv2d(ctx, d, w, b, sc)
    a, o = ctx.malloc(x.nbytes), ctx.malloc(op.info.out_bytes)
    try:
        with pytest.raises(enn.EnnError) as e:
            ctx.check(enn.lib.enn_b200_op_execute_noalloc(op.h, a, o))
        assert e.value.status == enn.INVALID_PARAMS and "static scratch holds" in str(e.value)
    finally:
        ctx.free(a)
        ctx.free(o)
        op.release()
    # a 1x1 convolution reads its input in place: nothing to place in the array
    d, x, w, b, sc = cases.conv_case(seed=2, n=1, h=8, w=8, cin=32, cout=32, k=1)
    op = enn.conv2d(ctx, d, w, b, sc)
    a, o = ctx.malloc(x.nbytes), ctx.malloc(op.info.out_bytes)
    try:
        with pytest.raises(enn.EnnError) as e:
            ctx.check(enn.lib.enn_b200_op_execute_noalloc(op.h, a, o))
        assert e.value.status == enn.INVALID_PARAMS
    finally:
        ctx.free(a)
        ctx.free(o)
        op.release()
