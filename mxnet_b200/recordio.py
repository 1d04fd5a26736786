"""RecordIO files (``python/mxnet/recordio.py``) over the native reader/writer (``csrc/recordio.cc``)."""
import ctypes
import numbers
import os
import struct
from collections import namedtuple

import numpy as np

from .base import MXNetError

__all__ = ['MXRecordIO', 'MXIndexedRecordIO', 'IRHeader', 'pack', 'unpack', 'unpack_img', 'pack_img']


def _rt():
    from .csrc import runtime
    return runtime.lib()


class MXRecordIO(object):
    def __init__(self, uri, flag):
        self.uri, self.flag = str(uri), flag
        self.handle = None
        self.is_open = False
        self.open()

    def open(self):
        L = _rt()
        if self.flag == 'w':
            self.handle = L.mxb_rec_writer_open(self.uri.encode(), 0)
            self.writable = True
        elif self.flag == 'r':
            self.handle = L.mxb_rec_reader_open(self.uri.encode())
            self.writable = False
        else:
            raise ValueError('Invalid flag %s' % self.flag)
        if not self.handle:
            raise MXNetError('cannot open %s' % self.uri)
        self.pid = os.getpid()
        self.is_open = True

    def __del__(self):
        self.close()

    def __getstate__(self):
        is_open = self.is_open
        self.close()
        d = dict(self.__dict__)
        d['is_open'] = is_open
        d['handle'] = None
        return d

    def __setstate__(self, d):
        self.__dict__ = d
        is_open = d['is_open']
        self.is_open = False
        self.handle = None
        if is_open:
            self.open()

    def _check_pid(self, allow_reset=False):
        if not self.pid == os.getpid():
            if allow_reset:
                self.reset()
            else:
                raise RuntimeError('Forbidden operation in multiple processes')

    def close(self):
        if not getattr(self, 'is_open', False):
            return
        L = _rt()
        if self.writable:
            L.mxb_rec_writer_close(self.handle)
        else:
            L.mxb_rec_reader_close(self.handle)
        self.is_open = False
        self.handle = None
        self.pid = None

    def reset(self):
        self.close()
        self.open()

    def write(self, buf):
        assert self.writable
        self._check_pid(allow_reset=False)
        rc = _rt().mxb_rec_writer_write(self.handle, ctypes.c_char_p(bytes(buf)), len(buf))
        if rc != 0:
            raise MXNetError('record too large')

    def tell(self):
        """Byte offset of the next record to be read or written."""
        L = _rt()
        return L.mxb_rec_writer_tell(self.handle) if self.writable else L.mxb_rec_reader_tell(self.handle)

    def read(self):
        assert not self.writable
        self._check_pid(allow_reset=True)
        size = ctypes.c_uint64(0)
        p = _rt().mxb_rec_reader_next(self.handle, ctypes.byref(size))
        if not p:
            return None
        return ctypes.string_at(p, size.value)


class MXIndexedRecordIO(MXRecordIO):
    def __init__(self, idx_path, uri, flag, key_type=int):
        self.idx_path = idx_path
        self.idx = {}
        self.keys = []
        self.key_type = key_type
        self.fidx = None
        super().__init__(uri, flag)

    def open(self):
        super().open()
        self.idx, self.keys = {}, []
        self.fidx = open(self.idx_path, self.flag)
        if not self.writable:
            for line in iter(self.fidx.readline, ''):
                line = line.strip().split('\t')
                key = self.key_type(line[0])
                self.idx[key] = int(line[1])
                self.keys.append(key)

    def close(self):
        if not getattr(self, 'is_open', False):
            return
        super().close()
        if self.fidx is not None:
            self.fidx.close()
            self.fidx = None

    def __getstate__(self):
        d = super().__getstate__()
        d['fidx'] = None
        return d

    def seek(self, idx):
        assert not self.writable
        self._check_pid(allow_reset=True)
        _rt().mxb_rec_reader_seek(self.handle, self.idx[idx])

    def tell(self):
        assert self.writable
        return _rt().mxb_rec_writer_tell(self.handle)

    def read_idx(self, idx):
        self.seek(idx)
        return self.read()

    def write_idx(self, idx, buf):
        key = self.key_type(idx)
        pos = self.tell()
        self.write(buf)
        self.fidx.write('%s\t%d\n' % (str(key), pos))
        self.idx[key] = pos
        self.keys.append(key)


IRHeader = namedtuple('HEADER', ['flag', 'label', 'id', 'id2'])
_IR_FORMAT = 'IfQQ'
_IR_SIZE = struct.calcsize(_IR_FORMAT)


def pack(header, s):
    """Pack a string with an image-record header (flag, label, id, id2); extra labels follow as floats."""
    header = IRHeader(*header)
    if isinstance(header.label, numbers.Number):
        header = header._replace(flag=0)
    else:
        label = np.asarray(header.label, dtype=np.float32)
        header = header._replace(flag=label.size, label=0)
        s = label.tobytes() + s
    return struct.pack(_IR_FORMAT, *header) + s


def unpack(s):
    header = IRHeader(*struct.unpack(_IR_FORMAT, s[:_IR_SIZE]))
    s = s[_IR_SIZE:]
    if header.flag > 0:
        header = header._replace(label=np.frombuffer(s, np.float32, header.flag))
        s = s[header.flag * 4:]
    return header, s


def unpack_img(s, iscolor=-1):
    header, s = unpack(s)
    from .image import _decode_to_numpy
    # OpenCV convention of the reference (cv2.imdecode): colour images come back in BGR order
    return header, _decode_to_numpy(s, 1 if iscolor != 0 else 0, to_rgb=False)


def pack_img(header, img, quality=95, img_fmt='.jpg'):
    import io
    from PIL import Image
    arr = np.asarray(img)
    im = Image.fromarray(arr[..., ::-1] if arr.ndim == 3 else arr)   # stored BGR like OpenCV callers expect
    buf = io.BytesIO()
    fmt = 'JPEG' if img_fmt.lower() in ('.jpg', '.jpeg') else 'PNG'
    if fmt == 'JPEG':
        im.save(buf, format=fmt, quality=quality)
    else:
        im.save(buf, format=fmt)
    return pack(header, buf.getvalue())
