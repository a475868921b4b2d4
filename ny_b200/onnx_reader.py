"""A minimal ONNX reader for feed-forward ReLU networks: Gemm / MatMul+Add / Conv / Relu / Flatten / Reshape, constant
Transpose of weights, Sub / Div / Mul input normalisation folded into the first dense layer, and residual Add of an
earlier post-activation tensor (an identity skip around two or more layers).

The reference loads ONNX through its own protobuf parser (crates/ny-onnx/src/onnx); here the protobuf wire format
is decoded directly with the field numbers of the public onnx.proto3 schema (ModelProto.graph = 7; GraphProto
node = 1, initializer = 5, input = 11, output = 12; NodeProto input = 1, output = 2, op_type = 4, attribute = 5;
AttributeProto name = 1, f = 2, i = 3, s = 4, t = 5, floats = 7, ints = 8; TensorProto dims = 1, data_type = 2,
float_data = 4, int64_data = 7, name = 8, raw_data = 9, double_data = 10).  Anything outside the subset is declined with
UnsupportedOp, never mis-read.  write_onnx is the inverse for the same subset (used by tests and to hand models
to other tools).
"""
from __future__ import annotations

import struct

import numpy as np

from .engine import Conv2d, EngineError, Network

_UNSUPPORTED, _INVALID = 1, 3


# ------------------------------------------------------------------------------------------- wire format
def _varint(buf, pos):
    val, shift = 0, 0
    while True:
        if pos >= len(buf):
            raise EngineError(_INVALID, "onnx: truncated varint")
        b = buf[pos]
        pos += 1
        val |= (b & 0x7F) << shift
        if not b & 0x80:
            return val, pos
        shift += 7
        if shift > 70:
            raise EngineError(_INVALID, "onnx: varint too long")


def _fields(buf):
    """Yields (field number, wire type, value): int for varint / fixed, memoryview for length-delimited."""
    pos, n = 0, len(buf)
    while pos < n:
        key, pos = _varint(buf, pos)
        num, wt = key >> 3, key & 7
        if wt == 0:
            val, pos = _varint(buf, pos)
        elif wt == 1:
            val, pos = bytes(buf[pos:pos + 8]), pos + 8
        elif wt == 2:
            ln, pos = _varint(buf, pos)
            if pos + ln > n:
                raise EngineError(_INVALID, "onnx: truncated field")
            val, pos = buf[pos:pos + ln], pos + ln
        elif wt == 5:
            val, pos = bytes(buf[pos:pos + 4]), pos + 4
        else:
            raise EngineError(_INVALID, f"onnx: wire type {wt}")
        yield num, wt, val


def _packed_varints(val, wt):
    if wt == 0:
        return [val]
    out, pos = [], 0
    while pos < len(val):
        v, pos = _varint(val, pos)
        out.append(v)
    return out


def _signed(v):
    return v - (1 << 64) if v >= (1 << 63) else v


_DTYPES = {1: np.float32, 6: np.int32, 7: np.int64, 11: np.float64}


def _tensor(buf):
    dims, dtype, name, raw = [], 1, "", None
    floats, int64s, doubles = [], [], []
    for num, wt, val in _fields(buf):
        if num == 1:
            dims += [_signed(v) for v in _packed_varints(val, wt)]
        elif num == 2:
            dtype = val
        elif num == 4:
            floats += list(struct.unpack(f"<{len(val) // 4}f", bytes(val))) if wt == 2 else [struct.unpack("<f", val)[0]]
        elif num == 7:
            int64s += [_signed(v) for v in _packed_varints(val, wt)]
        elif num == 8:
            name = bytes(val).decode()
        elif num == 9:
            raw = bytes(val)
        elif num == 10:
            doubles += list(struct.unpack(f"<{len(val) // 8}d", bytes(val))) if wt == 2 else [struct.unpack("<d", val)[0]]
    if dtype not in _DTYPES:
        raise EngineError(_UNSUPPORTED, f"onnx: tensor {name} has data type {dtype}")
    np_t = _DTYPES[dtype]
    if raw is not None:
        arr = np.frombuffer(raw, dtype=np.dtype(np_t).newbyteorder("<")).astype(np_t)
    elif dtype == 1:
        arr = np.array(floats, np.float32)
    elif dtype == 11:
        arr = np.array(doubles, np.float64)
    else:
        arr = np.array(int64s, np_t)
    count = int(np.prod(dims)) if dims else 1
    if arr.size != count:
        raise EngineError(_INVALID, f"onnx: tensor {name} holds {arr.size} values for shape {dims}")
    return name, arr.reshape(dims)


def _attribute(buf):
    name, val = "", None
    ints, floats = [], []
    for num, wt, v in _fields(buf):
        if num == 1:
            name = bytes(v).decode()
        elif num == 2:
            val = struct.unpack("<f", v)[0]
        elif num == 3:
            val = _signed(v)
        elif num == 4:
            val = bytes(v).decode()
        elif num == 5:
            val = _tensor(v)[1]
        elif num == 7:
            floats += list(struct.unpack(f"<{len(v) // 4}f", bytes(v))) if wt == 2 else [struct.unpack("<f", v)[0]]
        elif num == 8:
            ints += [_signed(x) for x in _packed_varints(v, wt)]
    if ints:
        val = ints
    elif floats:
        val = floats
    return name, val


def _node(buf):
    ins, outs, op, attrs = [], [], "", {}
    for num, wt, v in _fields(buf):
        if num == 1:
            ins.append(bytes(v).decode())
        elif num == 2:
            outs.append(bytes(v).decode())
        elif num == 4:
            op = bytes(v).decode()
        elif num == 5:
            k, a = _attribute(v)
            attrs[k] = a
    return op, ins, outs, attrs


def _value_info(buf):
    """(name, dims) of a graph input / output; unknown dimensions are -1."""
    name, dims = "", []
    for num, wt, v in _fields(buf):
        if num == 1:
            name = bytes(v).decode()
        elif num == 2:                                   # TypeProto
            for n2, _, v2 in _fields(v):
                if n2 == 1:                              # tensor_type
                    for n3, _, v3 in _fields(v2):
                        if n3 == 2:                      # shape
                            for n4, _, v4 in _fields(v3):
                                if n4 == 1:              # dim
                                    d = -1
                                    for n5, w5, v5 in _fields(v4):
                                        if n5 == 1:
                                            d = _signed(v5)
                                    dims.append(d)
    return name, dims


# ------------------------------------------------------------------------------------------- graph -> Network
def parse_onnx(data: bytes):
    """Returns (Network, input_shape): the sequential ReLU network of the model and the shape of one input sample
    ((n,) or (C, H, W)).  Layers are taken in node order along the single data path from the graph input."""
    graph = None
    for num, wt, v in _fields(memoryview(data)):
        if num == 7 and wt == 2:
            graph = v
    if graph is None:
        raise EngineError(_INVALID, "onnx: no graph in the model")
    nodes, inits, inputs = [], {}, []
    for num, wt, v in _fields(graph):
        if num == 1:
            nodes.append(_node(v))
        elif num == 5:
            name, arr = _tensor(v)
            inits[name] = arr
        elif num == 11:
            inputs.append(_value_info(v))
    for op, ins, outs, attrs in nodes:                 # Constant nodes are initialisers under another name
        if op == "Constant" and "value" in attrs and outs:
            inits[outs[0]] = attrs["value"]
    for op, ins, outs, attrs in nodes:                 # a Transpose of a constant is a constant (MatMul(x, W^T) exports)
        if op == "Transpose" and ins and ins[0] in inits and outs:
            perm = attrs.get("perm")
            inits[outs[0]] = np.transpose(inits[ins[0]], perm) if perm else inits[ins[0]].T
    data_inputs = [(n, d) for n, d in inputs if n not in inits]
    if len(data_inputs) != 1:
        raise EngineError(_UNSUPPORTED, f"onnx: {len(data_inputs)} graph inputs, expected one")
    cur, dims = data_inputs[0]
    dims = [d for d in dims[1:]] if len(dims) >= 2 else list(dims)      # drop the batch axis
    if any(d <= 0 for d in dims) or len(dims) not in (1, 3):
        raise EngineError(_UNSUPPORTED, f"onnx: input shape {dims} (need [N, n] or [N, C, H, W] with known sizes)")
    shape = tuple(int(d) for d in dims)
    in_shape = shape
    layers = []            # [kind, weight-or-Conv2d, bias, has_relu]

    def flat(shape):
        return int(np.prod(shape))

    def need_const(name, what):
        if name not in inits:
            raise EngineError(_UNSUPPORTED, f"onnx: {what} is not a constant")
        return inits[name]

    pre_scale, pre_shift = None, None      # input normalisation (x - shift) * scale in front of the first layer
    post_of = {}                           # tensor name -> index of the layer whose post-activation output it is
    skips = {}                             # layer k -> layer j: relu(pre_j) joins layer k's output before its Relu
    for op, ins, outs, attrs in nodes:
        if op == "Constant" or (op == "Transpose" and ins and ins[0] in inits):
            continue
        if cur not in ins:
            raise EngineError(_UNSUPPORTED, f"onnx: node {op} is off the single data path")
        if op in ("Identity", "Dropout"):
            if cur in post_of:
                post_of[outs[0]] = post_of[cur]
        elif op == "Flatten":
            shape = (flat(shape),)
        elif op == "Reshape":
            tgt = [int(x) for x in need_const(ins[1], "Reshape shape").reshape(-1)]
            if len(tgt) == 2 and (tgt[1] in (-1, flat(shape))):
                shape = (flat(shape),)
            elif tuple(tgt[1:]) != shape:
                raise EngineError(_UNSUPPORTED, f"onnx: Reshape to {tgt}")
        elif op == "Relu":
            if not layers or layers[-1][3]:
                raise EngineError(_UNSUPPORTED, "onnx: Relu without a layer before it")
            layers[-1][3] = True
            post_of[outs[0]] = len(layers) - 1
        elif op in ("Gemm", "MatMul"):
            if ins[0] != cur:
                raise EngineError(_UNSUPPORTED, f"onnx: {op} with the data as right operand")
            b_mat = np.asarray(need_const(ins[1], f"{op} weight"), np.float64)
            if b_mat.ndim != 2:
                raise EngineError(_UNSUPPORTED, f"onnx: {op} weight of rank {b_mat.ndim}")
            alpha, beta = 1.0, 1.0
            if op == "Gemm":
                if attrs.get("transA", 0):
                    raise EngineError(_UNSUPPORTED, "onnx: Gemm transA")
                alpha, beta = float(attrs.get("alpha", 1.0)), float(attrs.get("beta", 1.0))
                w = b_mat if attrs.get("transB", 0) else b_mat.T
            else:
                w = b_mat.T
            if w.shape[1] != flat(shape):
                raise EngineError(2, f"onnx: {op} expects {w.shape[1]} inputs, the data has {flat(shape)}")
            bias = None
            if op == "Gemm" and len(ins) > 2 and ins[2]:
                bias = np.broadcast_to(np.asarray(need_const(ins[2], "Gemm bias"), np.float64).reshape(-1), (w.shape[0],)) * beta
            if layers and not layers[-1][3]:
                raise EngineError(_UNSUPPORTED, "onnx: two affine layers without a Relu between them")
            w = w * alpha
            if pre_scale is not None and not layers:     # W ((x - sh) * sc) + b = (W * sc) x + (b - (W * sc) sh)
                w = w * pre_scale[None, :]
                bias = (np.zeros(w.shape[0]) if bias is None else np.asarray(bias, np.float64)) - w @ pre_shift
                pre_scale = pre_shift = None
            layers.append(["linear", w.astype(np.float32), None if bias is None else np.asarray(bias).astype(np.float32), False])
            shape = (w.shape[0],)
        elif op in ("Sub", "Div", "Mul") and not layers:
            # (x - mean) / std in front of the network: folded into the first affine layer below
            if ins[0] != cur:
                raise EngineError(_UNSUPPORTED, f"onnx: {op} with the data as right operand")
            c = np.broadcast_to(np.asarray(need_const(ins[1], f"{op} operand"), np.float64), shape).reshape(-1)
            sc = np.ones(flat(shape)) if pre_scale is None else pre_scale
            sh = np.zeros(flat(shape)) if pre_shift is None else pre_shift
            if op == "Sub":      # (x - sh) * sc - c = (x - (sh + c / sc)) * sc
                if np.any(sc == 0):
                    raise EngineError(_UNSUPPORTED, "onnx: normalisation with a zero scale")
                sh = sh + c / sc
            elif op == "Div":
                if np.any(c == 0):
                    raise EngineError(_INVALID, "onnx: division by zero in the input normalisation")
                sc = sc / c
            else:
                sc = sc * c
            pre_scale, pre_shift = sc, sh
        elif op == "Add" and (ins[1] if ins[0] == cur else ins[0]) in post_of:
            # residual connection: the post-activation output of an earlier layer joins this layer's output before its
            # Relu (an identity skip around at least two layers)
            j, k = post_of[ins[1] if ins[0] == cur else ins[0]], len(layers) - 1
            if not layers or layers[-1][3] or k in skips or j > k - 2:
                raise EngineError(_UNSUPPORTED, "onnx: residual Add outside the supported form")
            skips[k] = j
        elif op == "Add":
            other = ins[1] if ins[0] == cur else ins[0]
            c = np.asarray(need_const(other, "Add operand"), np.float32).reshape(-1)
            if not layers or layers[-1][0] != "linear" or layers[-1][3] or layers[-1][2] is not None or c.size != flat(shape):
                raise EngineError(_UNSUPPORTED, "onnx: Add that is not the bias of the preceding MatMul")
            layers[-1][2] = c.copy()
        elif op == "Conv":
            if len(shape) != 3:
                raise EngineError(_UNSUPPORTED, "onnx: Conv on a flattened tensor")
            w = np.asarray(need_const(ins[1], "Conv weight"), np.float32)
            if w.ndim != 4 or w.shape[1] != shape[0]:
                raise EngineError(_UNSUPPORTED, f"onnx: Conv weight {w.shape} on {shape} (groups are not supported)")
            if int(attrs.get("group", 1)) != 1 or any(int(d) != 1 for d in attrs.get("dilations", [1, 1])):
                raise EngineError(_UNSUPPORTED, "onnx: grouped or dilated Conv")
            if attrs.get("auto_pad", "NOTSET") not in ("NOTSET", ""):
                raise EngineError(_UNSUPPORTED, "onnx: Conv auto_pad")
            pads = [int(p) for p in attrs.get("pads", [0, 0, 0, 0])]
            if pads[0] != pads[2] or pads[1] != pads[3]:
                raise EngineError(_UNSUPPORTED, "onnx: asymmetric Conv padding")
            strides = [int(s) for s in attrs.get("strides", [1, 1])]
            bias = None
            if len(ins) > 2 and ins[2]:
                bias = np.asarray(need_const(ins[2], "Conv bias"), np.float32).reshape(-1)
            if layers and not layers[-1][3]:
                raise EngineError(_UNSUPPORTED, "onnx: two affine layers without a Relu between them")
            if pre_scale is not None:
                raise EngineError(_UNSUPPORTED, "onnx: input normalisation in front of a convolution")
            conv = Conv2d(w, bias, (strides[0], strides[1]), (pads[0], pads[1]), (shape[1], shape[2]))
            layers.append(["conv", conv, None, False])
            shape = (conv.oc, conv.oh, conv.ow)
        else:
            raise EngineError(_UNSUPPORTED, f"onnx: operator {op} is outside the supported subset")
        cur = outs[0]
    if not layers:
        raise EngineError(_UNSUPPORTED, "onnx: no affine layer")
    if layers[-1][3]:       # the model ends in a Relu: an identity layer carries its output to the specification
        layers.append(["linear", np.eye(flat(shape), dtype=np.float32), None, False])
    if not all(l[3] for l in layers[:-1]):
        raise EngineError(_UNSUPPORTED, "onnx: the network must be (affine, Relu)* affine")
    return Network([l[1] for l in layers], [l[2] for l in layers], skips or None), in_shape


# ------------------------------------------------------------------------------------------- writer
def _enc_varint(v):
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _ld(num, payload: bytes):
    return _enc_varint((num << 3) | 2) + _enc_varint(len(payload)) + payload


def _vi(num, v):
    return _enc_varint(num << 3) + _enc_varint(v)


def _enc_tensor(name, arr):
    arr = np.ascontiguousarray(arr)
    dtype = {np.dtype(np.float32): 1, np.dtype(np.int64): 7}[arr.dtype]
    out = b"".join(_vi(1, int(d)) for d in arr.shape) + _vi(2, dtype) + _ld(8, name.encode())
    return out + _ld(9, arr.astype(arr.dtype.newbyteorder("<")).tobytes())


def _enc_attr_ints(name, vals):
    return _ld(1, name.encode()) + b"".join(_vi(8, int(v)) for v in vals) + _vi(20, 7)


def _enc_attr_int(name, v):
    return _ld(1, name.encode()) + _vi(3, int(v)) + _vi(20, 2)


def _enc_node(op, ins, outs, attrs=()):
    out = b"".join(_ld(1, i.encode()) for i in ins) + b"".join(_ld(2, o.encode()) for o in outs) + _ld(4, op.encode())
    return out + b"".join(_ld(5, a) for a in attrs)


def _enc_value_info(name, dims):
    shape = b"".join(_ld(1, _vi(1, int(d))) for d in dims)
    ttype = _vi(1, 1) + _ld(2, shape)
    return _ld(1, name.encode()) + _ld(2, _ld(1, ttype))


def write_onnx(net: Network, input_shape) -> bytes:
    """The model bytes of a sequential network (Conv layers, Flatten, Gemm with transB = 1, Relu between layers)."""
    nodes, inits = [], []
    cur, flat_done = "input", len(input_shape) == 1
    L = len(net.weights)
    for k, (w, b) in enumerate(zip(net.weights, net.biases)):
        out = f"z{k}"
        if isinstance(w, Conv2d):
            ins = [cur, f"W{k}"]
            inits.append(_enc_tensor(f"W{k}", w.weight.astype(np.float32)))
            if w.bias is not None:
                ins.append(f"B{k}")
                inits.append(_enc_tensor(f"B{k}", w.bias.astype(np.float32)))
            attrs = [_enc_attr_ints("kernel_shape", [w.kh, w.kw]), _enc_attr_ints("strides", [w.sh, w.sw]),
                     _enc_attr_ints("pads", [w.ph, w.pw, w.ph, w.pw]), _enc_attr_ints("dilations", [1, 1]),
                     _enc_attr_int("group", 1)]
            nodes.append(_enc_node("Conv", ins, [out], attrs))
        else:
            if not flat_done:
                nodes.append(_enc_node("Flatten", [cur], [f"f{k}"], [_enc_attr_int("axis", 1)]))
                cur, flat_done = f"f{k}", True
            ins = [cur, f"W{k}"]
            inits.append(_enc_tensor(f"W{k}", np.asarray(w, np.float32)))
            if b is not None:
                ins.append(f"B{k}")
                inits.append(_enc_tensor(f"B{k}", np.asarray(b, np.float32)))
            nodes.append(_enc_node("Gemm", ins, [out], [_enc_attr_int("transB", 1)]))
        cur = out
        if k < L - 1:
            nodes.append(_enc_node("Relu", [cur], [f"a{k}"]))
            cur = f"a{k}"
    graph = b"".join(_ld(1, n) for n in nodes) + _ld(2, b"ny_b200") + b"".join(_ld(5, t) for t in inits)
    graph += _ld(11, _enc_value_info("input", [1] + list(input_shape)))
    graph += _ld(12, _enc_value_info(cur, [1, int(net.dims[-1])]))
    return _vi(1, 8) + _ld(8, _vi(2, 13)) + _ld(7, graph)
