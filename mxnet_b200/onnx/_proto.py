"""A self-contained writer and reader of the ONNX protobuf messages the exporter needs (ModelProto, GraphProto,
NodeProto, AttributeProto, TensorProto, ValueInfoProto), so that exporting a model does not depend on the ``onnx``
package.  Field numbers follow ``onnx.proto`` (IR version 8).  Messages are plain dicts; :func:`encode_model` turns a
model dict into bytes and :func:`decode_model` reads such bytes back (also files written by other exporters, as far as
they use these fields)."""
import struct

import numpy as np

IR_VERSION = 8

# TensorProto.DataType
FLOAT, UINT8, INT8, UINT16, INT16, INT32, INT64, STRING, BOOL, FLOAT16, DOUBLE, UINT32, UINT64 = range(1, 14)
BFLOAT16 = 16
NP_TO_ONNX = {np.dtype('float32'): FLOAT, np.dtype('uint8'): UINT8, np.dtype('int8'): INT8, np.dtype('uint16'): UINT16,
              np.dtype('int16'): INT16, np.dtype('int32'): INT32, np.dtype('int64'): INT64, np.dtype('bool'): BOOL,
              np.dtype('float16'): FLOAT16, np.dtype('float64'): DOUBLE, np.dtype('uint32'): UINT32,
              np.dtype('uint64'): UINT64}
ONNX_TO_NP = {v: k for k, v in NP_TO_ONNX.items()}

# AttributeProto.AttributeType
A_FLOAT, A_INT, A_STRING, A_TENSOR, A_GRAPH, A_FLOATS, A_INTS, A_STRINGS = range(1, 9)


# ------------------------------------------------------------------------------------------------ wire format
def _varint(n):
    n &= (1 << 64) - 1                           # negative int64 values are written as 10-byte two's complement
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        if n:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(field, wire):
    return _varint((field << 3) | wire)


def _f_varint(field, value):
    return _key(field, 0) + _varint(int(value))


def _f_bytes(field, data):
    if isinstance(data, str):
        data = data.encode()
    return _key(field, 2) + _varint(len(data)) + bytes(data)


def _f_float(field, value):
    return _key(field, 5) + struct.pack('<f', float(value))


def _f_packed_varints(field, values):
    return _f_bytes(field, b''.join(_varint(int(v)) for v in values))


def _f_packed_floats(field, values):
    return _f_bytes(field, struct.pack('<%df' % len(values), *[float(v) for v in values]))


# ------------------------------------------------------------------------------------------------ builders (dicts)
def make_tensor(name, array):
    a = np.ascontiguousarray(array)
    if a.dtype not in NP_TO_ONNX:
        raise TypeError('no ONNX tensor type for %s' % a.dtype)
    return {'name': name, 'dims': list(a.shape), 'data_type': NP_TO_ONNX[a.dtype], 'raw_data': a.tobytes()}


def make_attribute(name, value):
    if isinstance(value, dict) and 'raw_data' in value:
        return {'name': name, 'type': A_TENSOR, 't': value}
    if isinstance(value, bool):
        return {'name': name, 'type': A_INT, 'i': int(value)}
    if isinstance(value, (int, np.integer)):
        return {'name': name, 'type': A_INT, 'i': int(value)}
    if isinstance(value, (float, np.floating)):
        return {'name': name, 'type': A_FLOAT, 'f': float(value)}
    if isinstance(value, (str, bytes)):
        return {'name': name, 'type': A_STRING, 's': value.encode() if isinstance(value, str) else value}
    if isinstance(value, (list, tuple, np.ndarray)):
        vals = list(value)
        if all(isinstance(v, (int, np.integer, bool)) for v in vals):
            return {'name': name, 'type': A_INTS, 'ints': [int(v) for v in vals]}
        if all(isinstance(v, (int, float, np.integer, np.floating)) for v in vals):
            return {'name': name, 'type': A_FLOATS, 'floats': [float(v) for v in vals]}
        if all(isinstance(v, (str, bytes)) for v in vals):
            return {'name': name, 'type': A_STRINGS, 'strings': [v.encode() if isinstance(v, str) else v for v in vals]}
    raise TypeError('cannot store attribute %s=%r' % (name, value))


def make_node(op_type, inputs, outputs, name='', domain='', **attrs):
    return {'op_type': op_type, 'input': list(inputs), 'output': list(outputs), 'name': name, 'domain': domain,
            'attribute': [make_attribute(k, v) for k, v in attrs.items() if v is not None]}


def make_value_info(name, elem_type=FLOAT, shape=None):
    return {'name': name, 'elem_type': elem_type, 'shape': None if shape is None else list(shape)}


def make_graph(nodes, name, inputs, outputs, initializer=(), value_info=()):
    return {'node': list(nodes), 'name': name, 'input': list(inputs), 'output': list(outputs),
            'initializer': list(initializer), 'value_info': list(value_info)}


def make_model(graph, opset_version=13, producer_name='mxnet_b200', producer_version='', doc_string=''):
    return {'ir_version': IR_VERSION, 'producer_name': producer_name, 'producer_version': producer_version,
            'doc_string': doc_string, 'graph': graph, 'opset_import': [{'domain': '', 'version': int(opset_version)}]}


# ------------------------------------------------------------------------------------------------ encoding
def _enc_tensor(t):
    out = _f_packed_varints(1, t['dims']) if t['dims'] else b''
    out += _f_varint(2, t['data_type'])
    if t.get('name'):
        out += _f_bytes(8, t['name'])
    out += _f_bytes(9, t['raw_data'])
    return out


def _enc_attribute(a):
    out = _f_bytes(1, a['name'])
    kind = a['type']
    if kind == A_FLOAT:
        out += _f_float(2, a['f'])
    elif kind == A_INT:
        out += _f_varint(3, a['i'])
    elif kind == A_STRING:
        out += _f_bytes(4, a['s'])
    elif kind == A_TENSOR:
        out += _f_bytes(5, _enc_tensor(a['t']))
    elif kind == A_FLOATS:
        out += _f_packed_floats(7, a['floats'])
    elif kind == A_INTS:
        out += _f_packed_varints(8, a['ints'])
    elif kind == A_STRINGS:
        out += b''.join(_f_bytes(9, s) for s in a['strings'])
    else:
        raise TypeError('attribute type %s is not written by this exporter' % kind)
    return out + _f_varint(20, kind)


def _enc_node(n):
    out = b''.join(_f_bytes(1, i) for i in n['input']) + b''.join(_f_bytes(2, o) for o in n['output'])
    if n.get('name'):
        out += _f_bytes(3, n['name'])
    out += _f_bytes(4, n['op_type'])
    out += b''.join(_f_bytes(5, _enc_attribute(a)) for a in n['attribute'])
    if n.get('domain'):
        out += _f_bytes(7, n['domain'])
    return out


def _enc_value_info(v):
    tensor = _f_varint(1, v['elem_type'])
    if v['shape'] is not None:
        dims = b''
        for d in v['shape']:
            dim = _f_bytes(2, d) if isinstance(d, str) else _f_varint(1, d)      # dim_param / dim_value
            dims += _f_bytes(1, dim)
        tensor += _f_bytes(2, dims)
    return _f_bytes(1, v['name']) + _f_bytes(2, _f_bytes(1, tensor))


def _enc_graph(g):
    out = b''.join(_f_bytes(1, _enc_node(n)) for n in g['node'])
    out += _f_bytes(2, g['name'])
    out += b''.join(_f_bytes(5, _enc_tensor(t)) for t in g['initializer'])
    out += b''.join(_f_bytes(11, _enc_value_info(v)) for v in g['input'])
    out += b''.join(_f_bytes(12, _enc_value_info(v)) for v in g['output'])
    out += b''.join(_f_bytes(13, _enc_value_info(v)) for v in g.get('value_info', ()))
    return out


def encode_model(m):
    out = _f_varint(1, m['ir_version'])
    out += _f_bytes(2, m.get('producer_name', ''))
    if m.get('producer_version'):
        out += _f_bytes(3, m['producer_version'])
    if m.get('doc_string'):
        out += _f_bytes(6, m['doc_string'])
    out += _f_bytes(7, _enc_graph(m['graph']))
    for o in m['opset_import']:
        out += _f_bytes(8, (_f_bytes(1, o['domain']) if o['domain'] else b'') + _f_varint(2, o['version']))
    return out


# ------------------------------------------------------------------------------------------------ decoding
def _read_varint(buf, pos):
    shift = result = 0
    while True:
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7


def _fields(buf):
    """Yield (field number, wire type, value) of one message; length-delimited values as memoryview slices."""
    buf = memoryview(buf)
    pos, n = 0, len(buf)
    while pos < n:
        key, pos = _read_varint(buf, pos)
        field, wire = key >> 3, key & 7
        if wire == 0:
            val, pos = _read_varint(buf, pos)
        elif wire == 1:
            val, pos = bytes(buf[pos:pos + 8]), pos + 8
        elif wire == 2:
            ln, pos = _read_varint(buf, pos)
            val, pos = buf[pos:pos + ln], pos + ln
        elif wire == 5:
            val, pos = bytes(buf[pos:pos + 4]), pos + 4
        else:
            raise ValueError('unsupported wire type %d' % wire)
        yield field, wire, val


def _signed(v):
    return v - (1 << 64) if v >= (1 << 63) else v


def _unpack_varints(val, wire):
    if wire == 0:
        return [_signed(val)]
    out, pos = [], 0
    while pos < len(val):
        v, pos = _read_varint(val, pos)
        out.append(_signed(v))
    return out


def _dec_tensor(buf):
    t = {'dims': [], 'data_type': 0, 'name': '', 'raw_data': b''}
    floats, ints, int64s = [], [], []
    for f, w, v in _fields(buf):
        if f == 1:
            t['dims'] += _unpack_varints(v, w)
        elif f == 2:
            t['data_type'] = v
        elif f == 4:
            floats += list(struct.unpack('<%df' % (len(v) // 4), bytes(v))) if w == 2 else [struct.unpack('<f', v)[0]]
        elif f == 5:
            ints += _unpack_varints(v, w)
        elif f == 7:
            int64s += _unpack_varints(v, w)
        elif f == 8:
            t['name'] = bytes(v).decode()
        elif f == 9:
            t['raw_data'] = bytes(v)
    if not t['raw_data'] and t['data_type'] in ONNX_TO_NP:       # typed fields of other writers
        src = floats if floats else (int64s if int64s else ints)
        t['raw_data'] = np.asarray(src).astype(ONNX_TO_NP[t['data_type']]).tobytes()
    return t


def tensor_to_numpy(t):
    if t['data_type'] not in ONNX_TO_NP:
        raise TypeError('tensor %s has data type %d' % (t['name'], t['data_type']))
    return np.frombuffer(t['raw_data'], dtype=ONNX_TO_NP[t['data_type']]).reshape(t['dims']).copy()


def _dec_attribute(buf):
    a = {'name': '', 'type': 0, 'floats': [], 'ints': [], 'strings': []}
    for f, w, v in _fields(buf):
        if f == 1:
            a['name'] = bytes(v).decode()
        elif f == 2:
            a['f'] = struct.unpack('<f', v)[0]
        elif f == 3:
            a['i'] = _signed(v)
        elif f == 4:
            a['s'] = bytes(v)
        elif f == 5:
            a['t'] = _dec_tensor(v)
        elif f == 7:
            a['floats'] += list(struct.unpack('<%df' % (len(v) // 4), bytes(v))) if w == 2 else [struct.unpack('<f', v)[0]]
        elif f == 8:
            a['ints'] += _unpack_varints(v, w)
        elif f == 9:
            a['strings'].append(bytes(v))
        elif f == 20:
            a['type'] = v
    return a


def attribute_value(a):
    kind = a['type']
    return {A_FLOAT: lambda: a['f'], A_INT: lambda: a['i'], A_STRING: lambda: a['s'].decode(), A_TENSOR: lambda: tensor_to_numpy(a['t']),
            A_FLOATS: lambda: list(a['floats']), A_INTS: lambda: list(a['ints']),
            A_STRINGS: lambda: [s.decode() for s in a['strings']]}[kind]()


def _dec_node(buf):
    n = {'input': [], 'output': [], 'name': '', 'op_type': '', 'attribute': [], 'domain': ''}
    for f, _w, v in _fields(buf):
        if f == 1:
            n['input'].append(bytes(v).decode())
        elif f == 2:
            n['output'].append(bytes(v).decode())
        elif f == 3:
            n['name'] = bytes(v).decode()
        elif f == 4:
            n['op_type'] = bytes(v).decode()
        elif f == 5:
            n['attribute'].append(_dec_attribute(v))
        elif f == 7:
            n['domain'] = bytes(v).decode()
    return n


def _dec_value_info(buf):
    vi = {'name': '', 'elem_type': 0, 'shape': None}
    for f, _w, v in _fields(buf):
        if f == 1:
            vi['name'] = bytes(v).decode()
        elif f == 2:
            for f2, _w2, v2 in _fields(v):
                if f2 != 1:                       # tensor_type only
                    continue
                for f3, _w3, v3 in _fields(v2):
                    if f3 == 1:
                        vi['elem_type'] = v3
                    elif f3 == 2:
                        shape = []
                        for f4, _w4, v4 in _fields(v3):
                            if f4 == 1:
                                dim = None
                                for f5, _w5, v5 in _fields(v4):
                                    dim = _signed(v5) if f5 == 1 else bytes(v5).decode()
                                shape.append(dim)
                        vi['shape'] = shape
    return vi


def _dec_graph(buf):
    g = {'node': [], 'name': '', 'initializer': [], 'input': [], 'output': [], 'value_info': []}
    for f, _w, v in _fields(buf):
        if f == 1:
            g['node'].append(_dec_node(v))
        elif f == 2:
            g['name'] = bytes(v).decode()
        elif f == 5:
            g['initializer'].append(_dec_tensor(v))
        elif f == 11:
            g['input'].append(_dec_value_info(v))
        elif f == 12:
            g['output'].append(_dec_value_info(v))
        elif f == 13:
            g['value_info'].append(_dec_value_info(v))
    return g


def decode_model(data):
    m = {'ir_version': 0, 'producer_name': '', 'producer_version': '', 'doc_string': '', 'graph': None, 'opset_import': []}
    for f, _w, v in _fields(data):
        if f == 1:
            m['ir_version'] = v
        elif f == 2:
            m['producer_name'] = bytes(v).decode()
        elif f == 3:
            m['producer_version'] = bytes(v).decode()
        elif f == 6:
            m['doc_string'] = bytes(v).decode()
        elif f == 7:
            m['graph'] = _dec_graph(v)
        elif f == 8:
            o = {'domain': '', 'version': 0}
            for f2, _w2, v2 in _fields(v):
                if f2 == 1:
                    o['domain'] = bytes(v2).decode()
                elif f2 == 2:
                    o['version'] = v2
            m['opset_import'].append(o)
    return m
