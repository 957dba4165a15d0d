"""Test helper: serialises a layer list (cl-eden-kernel_b200/mobilenet.py) as an NNC v2 model file.

A small forward flatbuffer writer (parents before children, so every offset points ahead) plus the field numbers
of the tables the front end reads, in the declaration order of the reference's schema
(src/model/schema/nnc/v2/schema.fbs).  tests/test_nnc_frontend.py checks the bytes with the reference's own
generated reader and verifier where the reference tree is mounted.
"""
import struct

import numpy as np

_FMT = {"i8": "<b", "u8": "<B", "bool": "<B", "i32": "<i", "u32": "<I", "f32": "<f", "i64": "<q"}


class Table:
    def __init__(self, **fields):
        """fields: f<id> = (fmt, value) for scalars, or a Table / Vec / VecT / Str for offsets."""
        self.fields = {int(k[1:]): v for k, v in fields.items() if v is not None}


class Vec:
    def __init__(self, fmt, values, align=None):
        self.fmt, self.values, self.align = fmt, values, align


class VecT:
    def __init__(self, tables):
        self.tables = tables


class Str:
    def __init__(self, s):
        self.s = s.encode()


class Writer:
    def __init__(self):
        self.buf = bytearray()

    def _align(self, a):
        while len(self.buf) % a:
            self.buf.append(0)

    def _patch(self, pos, target):
        struct.pack_into("<I", self.buf, pos, target - pos)

    def emit(self, obj):
        if isinstance(obj, Table):
            return self._table(obj)
        if isinstance(obj, Vec):
            size = struct.calcsize(_FMT[obj.fmt])
            a = obj.align or max(4, size)
            # the element area must be aligned; the length word sits right before it
            while (len(self.buf) + 4) % a:
                self.buf.append(0)
            pos = len(self.buf)
            self.buf += struct.pack("<I", len(obj.values))
            if isinstance(obj.values, (bytes, bytearray)):
                self.buf += obj.values
            else:
                for v in obj.values:
                    self.buf += struct.pack(_FMT[obj.fmt], v)
            return pos
        if isinstance(obj, VecT):
            self._align(4)
            pos = len(self.buf)
            self.buf += struct.pack("<I", len(obj.tables))
            slots = len(self.buf)
            self.buf += b"\0" * (4 * len(obj.tables))
            for i, t in enumerate(obj.tables):
                self._patch(slots + 4 * i, self.emit(t))
            return pos
        if isinstance(obj, Str):
            self._align(4)
            pos = len(self.buf)
            self.buf += struct.pack("<I", len(obj.s)) + obj.s + b"\0"
            return pos
        raise TypeError(obj)

    def _table(self, t):
        nf = (max(t.fields) + 1) if t.fields else 0
        # inline layout: soffset, then the fields in id order, each aligned to its size
        off, layout = 4, {}
        for fid in sorted(t.fields):
            v = t.fields[fid]
            size = struct.calcsize(_FMT[v[0]]) if isinstance(v, tuple) else 4
            off = (off + size - 1) // size * size
            layout[fid] = off
            off += size
        tsize = (off + 3) // 4 * 4
        vsize = 4 + 2 * nf
        # the table (whose fields may hold 8-byte scalars) starts 8-aligned, the vtable right before it
        while (len(self.buf) + vsize) % 8:
            self.buf.append(0)
        vpos = len(self.buf)
        self.buf += struct.pack("<HH", vsize, tsize)
        for fid in range(nf):
            self.buf += struct.pack("<H", layout.get(fid, 0))
        tpos = len(self.buf)
        self.buf += b"\0" * tsize
        struct.pack_into("<i", self.buf, tpos, tpos - vpos)
        children = []
        for fid, v in t.fields.items():
            if isinstance(v, tuple):
                struct.pack_into(_FMT[v[0]], self.buf, tpos + layout[fid], v[1])
            else:
                children.append((tpos + layout[fid], v))
        for pos, child in children:
            self._patch(pos, self.emit(child))
        return tpos


# schema.fbs values
TT = {"uint8": 3, "int8": 9, "int32": 2}
OPCODE = {"ADD": 0, "AVERAGE_POOL_2D": 1, "CONCATENATION": 2, "CONV_2D": 3, "DEPTHWISE_CONV_2D": 4, "FULLY_CONNECTED": 9, "MAX_POOL_2D": 17,
          "RESIZE_BILINEAR": 23, "SOFTMAX": 25, "MEAN": 40, "TRANSPOSE_CONV": 67}
# BuiltinOptions union tags (position of the options table in the union, starting at 1)
OPTIONS_TAG = {"Conv2DOptions": 1, "DepthwiseConv2DOptions": 2, "Pool2DOptions": 5, "FullyConnectedOptions": 8, "SoftmaxOptions": 9,
               "ConcatenationOptions": 10, "AddOptions": 11, "ResizeBilinearOptions": 15, "ReducerOptions": 27, "TransposeConvOptions": 49}
LEGACY_TENSORFLOW_NHWC, LEGACY_CAFFE_NHWC, LEGACY_ANDROID_NN = 5, 3, 6
PAD_SAME, PAD_VALID = 0, 1


class ModelBuilder:
    def __init__(self, legacy=LEGACY_TENSORFLOW_NHWC):
        self.legacy = legacy
        self.tensors, self.buffers, self.ops, self.codes = [], [b""], [], []
        self.inputs, self.outputs = [], []

    def tensor(self, shape, dtype="uint8", scale=None, zp=0, data=None, pc_scales=None, name=""):
        buf = 0
        if data is not None:
            self.buffers.append(np.ascontiguousarray(data).tobytes())
            buf = len(self.buffers) - 1
        q = Table(f2=Vec("f32", [float(scale)]), f3=Vec("i64", [int(zp)])) if scale is not None else None
        pc = Table(f0=Vec("f32", [float(s) for s in pc_scales]), f1=("u32", 0)) if pc_scales is not None else None
        self.tensors.append(Table(f0=Vec("i32", [int(s) for s in shape]), f1=("i8", TT[dtype]), f2=("u32", buf), f3=Str(name), f4=q, f10=pc))
        return len(self.tensors) - 1

    def op(self, name, inputs, outputs, options_name=None, options=None):
        if OPCODE[name] not in self.codes:
            self.codes.append(OPCODE[name])
        self.ops.append(Table(f0=("u32", self.codes.index(OPCODE[name])), f1=Vec("i32", inputs), f2=Vec("i32", outputs),
                              f3=("u8", OPTIONS_TAG[options_name]) if options is not None else None, f4=options))

    def finish(self):
        w = Writer()
        w.buf += b"\0\0\0\0ENNC"
        sub = Table(f0=VecT(self.tensors), f1=Vec("i32", self.inputs), f2=Vec("i32", self.outputs), f3=VecT(self.ops), f4=Str("main"))
        model = Table(f0=("u32", 201),
                      f1=VecT([Table(f0=("i8", min(c, 127)), f2=("i32", 1), f3=("i32", c)) for c in self.codes]),
                      f2=VecT([sub]), f3=Str("synthetic"),
                      f4=VecT([Table(f0=Vec("u8", b, align=16)) if b else Table() for b in self.buffers]),
                      f8=Vec("i32", [self.legacy]))
        root = w.emit(model)
        struct.pack_into("<I", w.buf, 0, root)
        return bytes(w.buf)


def mobilenet_to_nnc(layers, batch, resolution=224, legacy=LEGACY_TENSORFLOW_NHWC, same_padding=True):
    """The synthetic MobileNetV2-u8 layer list as an NNC model (TENSORFLOW_NHWC conventions: OHWI filters, depthwise
    filters [1][Kh][Kw][C], SAME / VALID padding)."""
    mb = ModelBuilder(legacy)
    ids = {"input": mb.tensor((batch, resolution, resolution, 3), "uint8", layers[0]["in_scale"], layers[0]["in_zp"], name="input")}
    mb.inputs = [ids["input"]]
    for L in layers:
        h = L["h"]
        if L["kind"] in ("conv", "dw"):
            pt, pb = L["pad"]
            oh = (h + pt + pb - L["k"]) // L["stride"] + 1
            cout = L["cout"]
            if L["kind"] == "dw":
                w = np.ascontiguousarray(L["w"][:, 0].transpose(1, 2, 0)[None])          # [C][1][kh][kw] -> [1][kh][kw][C]
            else:
                w = L["w"]                                                                 # OHWI
            wt = mb.tensor(w.shape, "int8", 1.0, 0, data=w, pc_scales=L["scales"], name=L["name"] + "_w")
            bt = mb.tensor((cout,), "int32", 1.0, 0, data=L["bias"], name=L["name"] + "_b")
            ot = mb.tensor((batch, oh, oh, cout), "uint8", L["out_scale"], L["out_zp"], name=L["name"])
            padding = PAD_SAME if (pt or pb) else PAD_VALID
            if L["kind"] == "dw":
                opt = Table(f0=("i8", padding), f1=("i32", L["stride"]), f2=("i32", L["stride"]), f3=("i32", 1), f4=("i8", L["act"]))
                mb.op("DEPTHWISE_CONV_2D", [ids[L["src"]], wt, bt], [ot], "DepthwiseConv2DOptions", opt)
            else:
                opt = Table(f0=("i8", padding), f1=("i32", L["stride"]), f2=("i32", L["stride"]), f3=("i8", L["act"]))
                mb.op("CONV_2D", [ids[L["src"]], wt, bt], [ot], "Conv2DOptions", opt)
        elif L["kind"] == "fc":
            w = L["w"].reshape(L["cout"], L["cin"])
            wt = mb.tensor(w.shape, "int8", 1.0, 0, data=w, pc_scales=L["scales"], name="fc_w")
            bt = mb.tensor((L["cout"],), "int32", 1.0, 0, data=L["bias"], name="fc_b")
            ot = mb.tensor((batch, L["cout"]), "uint8", L["out_scale"], L["out_zp"], name=L["name"])
            mb.op("FULLY_CONNECTED", [ids[L["src"]], wt, bt], [ot], "FullyConnectedOptions", Table(f0=("i8", 0)))
        elif L["kind"] == "add":
            ot = mb.tensor((batch, h, h, L["cout"]), "uint8", L["out_scale"], L["out_zp"], name=L["name"])
            mb.op("ADD", [ids[L["src"]], ids[L["src2"]]], [ot], "AddOptions", Table(f0=("i8", 0)))
        else:
            ot = mb.tensor((batch, 1, 1, L["cin"]), "uint8", L["out_scale"], L["out_zp"], name=L["name"])
            opt = Table(f0=("i8", PAD_VALID), f1=("i32", 1), f2=("i32", 1), f3=("i32", L["k"]), f4=("i32", L["k"]), f5=("i8", 0))
            mb.op("AVERAGE_POOL_2D", [ids[L["src"]]], [ot], "Pool2DOptions", opt)
        ids[L["name"]] = ot
    mb.outputs = [ids[layers[-1]["name"]]]
    return mb.finish()
