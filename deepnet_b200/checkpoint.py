"""Model interchange with the reference: the gzip'd `Model` protocol buffer that deepnet writes
as checkpoints (deepnet/util.py:13-53, deepnet/protos/deepnet.proto:7-50,181-229) and reads back
for DBN stacking, representation extraction and AIS.

Only the wire format is needed, so this module carries its own small protobuf codec (varints,
length-delimited and fixed-width fields) instead of generated classes: a message is decoded
into a list of (field number, wire type, value) and every field this module does not interpret
is kept as it came, so that a checkpoint written by the reference survives a read-modify-write
here (hyperparameters, statistics, data fields, ...).  Interpreted fields:

  Model      1 name, 2 model_type (3 = DBM), 3 layer*, 4 edge*
  Layer      1 name, 3 dimensions, 5 param*            (bias: dimensions [n, 1] in the checkpoints)
  Edge       1 node1, 2 node2, 4 param*                (weight: dimensions [n1, n2])
  Parameter  1 name, 2 mat (float32 bytes, C order, deepnet/util.py:13-21), 3 dimensions*
  Operation  4 current_step (the resume point, deepnet/neuralnet.py:681-684)

Parameters travel as numpy arrays in the reference's orientation (weight: node1 units x node2
units, the same as the device matrices here).
"""
import gzip
import os
import shutil
import struct
import time

import numpy as np

VARINT, FIXED64, BYTES, FIXED32 = 0, 1, 2, 5
MODEL_DBM = 3


# ---- wire format -----------------------------------------------------------------------------
def _read_varint(buf, pos):
    shift = value = 0
    while True:
        byte = buf[pos]
        pos += 1
        value |= (byte & 0x7F) << shift
        if not byte & 0x80:
            return value, pos
        shift += 7
        if shift > 70:
            raise ValueError("varint too long")


def _write_varint(value):
    if value < 0:
        value += 1 << 64          # int32/int64 negatives are sign-extended to 64 bits
    out = bytearray()
    while True:
        byte = value & 0x7F
        value >>= 7
        if value:
            out.append(byte | 0x80)
        else:
            out.append(byte)
            return bytes(out)


def decode(buf):
    """bytes -> list of (field, wire type, value); value is int (varint), bytes, or raw 4/8 bytes."""
    buf = bytes(buf)
    fields, pos = [], 0
    while pos < len(buf):
        key, pos = _read_varint(buf, pos)
        field, wt = key >> 3, key & 7
        if wt == VARINT:
            value, pos = _read_varint(buf, pos)
        elif wt == BYTES:
            n, pos = _read_varint(buf, pos)
            value = buf[pos:pos + n]
            if len(value) != n:
                raise ValueError("truncated field %d" % field)
            pos += n
        elif wt in (FIXED32, FIXED64):
            n = 4 if wt == FIXED32 else 8
            value = buf[pos:pos + n]
            pos += n
        else:
            raise ValueError("unsupported wire type %d" % wt)
        fields.append((field, wt, value))
    return fields


def encode(fields):
    out = bytearray()
    for field, wt, value in fields:
        out += _write_varint(field << 3 | wt)
        if wt == VARINT:
            out += _write_varint(value)
        elif wt == BYTES:
            out += _write_varint(len(value)) + bytes(value)
        else:
            out += bytes(value)
    return bytes(out)


def _first(fields, number, default=None):
    for f, _, v in fields:
        if f == number:
            return v
    return default


def _signed32(v):
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >> 63 else v


def _repeated_int32(fields, number):
    """repeated int32, packed or not."""
    out = []
    for f, wt, v in fields:
        if f != number:
            continue
        if wt == VARINT:
            out.append(_signed32(v))
        else:
            pos = 0
            while pos < len(v):
                x, pos = _read_varint(v, pos)
                out.append(_signed32(x))
    return out


# ---- parameters ------------------------------------------------------------------------------
def parameter_as_numpy(param_bytes):
    """deepnet/util.py:13-16: (name, float32 array of the stored dimensions)."""
    f = decode(param_bytes)
    name = _first(f, 1, b"").decode("utf-8")
    dims = _repeated_int32(f, 3)
    mat = _first(f, 2)
    if mat is None:
        return name, None
    arr = np.frombuffer(mat, dtype="<f4")
    return name, arr.reshape(*dims).copy() if dims else arr.copy()


def numpy_as_parameter(name, array, template=None):
    """deepnet/util.py:18-21: the Parameter message of a float32 array.  With `template` (the
    bytes of an existing Parameter) its other fields (initialisation, convolution, ...) are kept."""
    array = np.ascontiguousarray(array, dtype="<f4")
    rest = [x for x in decode(template) if x[0] not in (1, 2, 3)] if template else []
    fields = [(1, BYTES, name.encode("utf-8")), (2, BYTES, array.tobytes())]
    fields += [(3, VARINT, int(d)) for d in array.shape]
    return encode(fields + rest)


class Model(object):
    """A decoded `Model` message: `layers[name]` / `edges[(node1, node2)]` give access to the
    parameters as numpy arrays; everything else is carried through untouched."""

    def __init__(self, name="model", model_type=MODEL_DBM):
        self.fields = [(1, BYTES, name.encode("utf-8")), (2, VARINT, model_type)]

    # -- reading
    @classmethod
    def from_bytes(cls, data):
        m = cls.__new__(cls)
        m.fields = decode(data)
        return m

    @property
    def name(self):
        return _first(self.fields, 1, b"").decode("utf-8")

    @property
    def model_type(self):
        return _first(self.fields, 2, 0)

    def _submessages(self, number):
        return [(i, decode(v)) for i, (f, _, v) in enumerate(self.fields) if f == number]

    def layer_names(self):
        return [_first(f, 1, b"").decode("utf-8") for _, f in self._submessages(3)]

    def layer_dimensions(self, name):
        for _, f in self._submessages(3):
            if _first(f, 1, b"").decode("utf-8") == name:
                return _first(f, 3, 0)
        raise KeyError(name)

    def edge_names(self):
        return [(_first(f, 1, b"").decode("utf-8"), _first(f, 2, b"").decode("utf-8")) for _, f in self._submessages(4)]

    def _params(self, number, match, param_field):
        for idx, f in self._submessages(number):
            if match(f):
                return idx, f, {parameter_as_numpy(v)[0]: (j, v) for j, (pf, _, v) in enumerate(f) if pf == param_field}
        raise KeyError("no such layer or edge")

    def get_layer_param(self, layer, pname="bias"):
        _, _, params = self._params(3, lambda f: _first(f, 1, b"").decode("utf-8") == layer, 5)
        return parameter_as_numpy(params[pname][1])[1]

    def get_edge_param(self, node1, node2, pname="weight"):
        match = lambda f: (_first(f, 1, b"").decode("utf-8"), _first(f, 2, b"").decode("utf-8")) == (node1, node2)
        _, _, params = self._params(4, match, 4)
        return parameter_as_numpy(params[pname][1])[1]

    # -- writing
    def _set_param(self, number, match, param_field, pname, array):
        idx, f, params = self._params(number, match, param_field)
        if pname in params:
            j, old = params[pname]
            f[j] = (param_field, BYTES, numpy_as_parameter(pname, array, template=old))
        else:
            f.append((param_field, BYTES, numpy_as_parameter(pname, array)))
        self.fields[idx] = (number, BYTES, encode(f))

    def set_layer_param(self, layer, array, pname="bias"):
        self._set_param(3, lambda f: _first(f, 1, b"").decode("utf-8") == layer, 5, pname, array)

    def set_edge_param(self, node1, node2, array, pname="weight"):
        match = lambda f: (_first(f, 1, b"").decode("utf-8"), _first(f, 2, b"").decode("utf-8")) == (node1, node2)
        self._set_param(4, match, 4, pname, array)

    def add_layer(self, name, dimensions, bias=None, is_input=False):
        f = [(1, BYTES, name.encode("utf-8")), (3, VARINT, int(dimensions))]
        if bias is not None:
            f.append((5, BYTES, numpy_as_parameter("bias", np.asarray(bias, np.float32).reshape(-1, 1))))
        if is_input:
            f.append((7, VARINT, 1))
        self.fields.append((3, BYTES, encode(f)))

    def add_edge(self, node1, node2, weight, directed=False):
        f = [(1, BYTES, node1.encode("utf-8")), (2, BYTES, node2.encode("utf-8")), (3, VARINT, int(bool(directed))),
             (4, BYTES, numpy_as_parameter("weight", np.asarray(weight, np.float32)))]
        self.fields.append((4, BYTES, encode(f)))

    def to_bytes(self):
        return encode(self.fields)


# ---- files -----------------------------------------------------------------------------------
def read_model(path):
    """deepnet/util.py:68-80 for a binary (optionally gzip'd) checkpoint."""
    with open(path, "rb") as fh:
        head = fh.read(2)
    opener = gzip.open if head == b"\x1f\x8b" else open
    with opener(path, "rb") as fh:
        return Model.from_bytes(fh.read())


def write_checkpoint(model, directory, best=False, train_op_bytes=None, stamp=None):
    """deepnet/util.py:23-53: `<name>_BEST`, or `<name>_<unix time>` copied to `<name>_LAST`; the
    training operation (when given) goes beside it as `<name>_train_op_<tag>`.  Returns the path
    a reader should open (`_BEST` / `_LAST`)."""
    os.makedirs(directory, exist_ok=True)
    data = model.to_bytes()
    if best:
        tag = "BEST"
        path = os.path.join(directory, "%s_%s" % (model.name, tag))
        with gzip.open(path, "wb") as fh:
            fh.write(data)
    else:
        tag = "LAST"
        stamped = os.path.join(directory, "%s_%s" % (model.name, stamp if stamp is not None else int(time.time())))
        with gzip.open(stamped, "wb") as fh:
            fh.write(data)
        path = os.path.join(directory, "%s_%s" % (model.name, tag))
        shutil.copyfile(stamped, path)
    if train_op_bytes is not None:
        with gzip.open(os.path.join(directory, "%s_train_op_%s" % (model.name, tag)), "wb") as fh:
            fh.write(train_op_bytes)
    return path


def operation_current_step(op_bytes):
    """`current_step` of a serialized Operation (field 4, default 0): the step training resumes at."""
    return _first(decode(op_bytes), 4, 0)


def operation_with_step(op_bytes, step):
    fields = [x for x in decode(op_bytes) if x[0] != 4]
    return encode(fields + [(4, VARINT, int(step))])


# ---- engines ---------------------------------------------------------------------------------
def model_from_rbm(engine, name="rbm", visible="input_layer", hidden="hidden1"):
    """The Model message of a `FusedRBM` (weights and both biases read back from the device)."""
    m = Model(name, MODEL_DBM)
    m.add_layer(visible, engine.V, bias=np.array(engine.bv.asarray()), is_input=True)
    m.add_layer(hidden, engine.H, bias=np.array(engine.bh.asarray()))
    m.add_edge(visible, hidden, np.array(engine.W.asarray()))
    return m


def load_into_rbm(engine, model, visible=None, hidden=None):
    """Copies a checkpoint's weight and biases into a `FusedRBM` (and refreshes the bfloat16 parts of W)."""
    (n1, n2), = model.edge_names()[:1]
    visible, hidden = visible or n1, hidden or n2
    w = model.get_edge_param(visible, hidden)
    assert w.shape == (engine.V, engine.H), "checkpoint is %s, engine %s" % (w.shape, (engine.V, engine.H))
    engine.W.overwrite(np.asfortranarray(w))
    engine.bv.overwrite(np.asfortranarray(model.get_layer_param(visible).reshape(engine.V, 1)))
    engine.bh.overwrite(np.asfortranarray(model.get_layer_param(hidden).reshape(engine.H, 1)))
    engine.refresh_weight_aux()
