"""RecordIO files from Python (API of ``python/mxnet/recordio.py``: ``MXRecordIO``, ``MXIndexedRecordIO``, ``IRHeader``,
``pack`` / ``unpack`` / ``pack_img`` / ``unpack_img``).

Reading and writing of the framed records is done by the native runtime (``csrc/recordio.cc``); this module owns the
handle life cycle (open / close / reset, pickling for data-loader workers, the per-process guard), the text index of the
indexed variant (``key<TAB>byte offset`` per line) and the image-record header.
"""
import ctypes
import io
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
    """Sequential reader (``flag='r'``) or writer (``flag='w'``) of one RecordIO file."""

    _MODES = {'w': True, 'r': False}

    def __init__(self, uri, flag):
        self.uri = str(uri)
        self.flag = flag
        self.handle = None
        self.is_open = False
        self.writable = False
        self.pid = None
        self.open()

    # ---- handle life cycle ----------------------------------------------------------------------------------
    def open(self):
        if self.flag not in self._MODES:
            raise ValueError('Invalid flag %s' % self.flag)
        self.writable = self._MODES[self.flag]
        lib = _rt()
        path = self.uri.encode()
        self.handle = lib.mxb_rec_writer_open(path, 0) if self.writable else lib.mxb_rec_reader_open(path)
        if not self.handle:
            raise MXNetError('cannot open %s' % self.uri)
        self.pid = os.getpid()
        self.is_open = True

    def close(self):
        if not getattr(self, 'is_open', False):
            return
        lib = _rt()
        (lib.mxb_rec_writer_close if self.writable else lib.mxb_rec_reader_close)(self.handle)
        self.handle = None
        self.is_open = False
        self.pid = None

    def reset(self):
        """Back to the first record (a writer truncates and starts over)."""
        self.close()
        self.open()

    def __del__(self):
        self.close()

    def __getstate__(self):
        # a native handle cannot travel to another process: remember whether to reopen on the other side
        was_open = self.is_open
        self.close()
        state = dict(self.__dict__)
        state.update(is_open=was_open, handle=None)
        return state

    def __setstate__(self, state):
        reopen = state['is_open']
        self.__dict__ = state
        self.is_open = False
        self.handle = None
        if reopen:
            self.open()

    def _check_pid(self, allow_reset=False):
        """A handle opened before a fork is reopened in the child (readers) or refused (writers)."""
        if self.pid == os.getpid():
            return
        if not allow_reset:
            raise RuntimeError('Forbidden operation in multiple processes')
        self.reset()

    # ---- records --------------------------------------------------------------------------------------------
    def write(self, buf):
        if not self.writable:
            raise AssertionError('file was opened for reading')
        self._check_pid(allow_reset=False)
        data = bytes(buf)
        if _rt().mxb_rec_writer_write(self.handle, ctypes.c_char_p(data), len(data)) != 0:
            raise MXNetError('record too large')

    def read(self):
        """The next record as bytes, ``None`` at the end of the file."""
        if self.writable:
            raise AssertionError('file was opened for writing')
        self._check_pid(allow_reset=True)
        size = ctypes.c_uint64(0)
        ptr = _rt().mxb_rec_reader_next(self.handle, ctypes.byref(size))
        return ctypes.string_at(ptr, size.value) if ptr else None

    def tell(self):
        """Byte offset of the next record to be read or written."""
        lib = _rt()
        return (lib.mxb_rec_writer_tell if self.writable else lib.mxb_rec_reader_tell)(self.handle)


class MXIndexedRecordIO(MXRecordIO):
    """RecordIO file with a side index ``idx_path`` for random access by key (``key_type`` converts the key column)."""

    def __init__(self, idx_path, uri, flag, key_type=int):
        self.idx_path = idx_path
        self.key_type = key_type
        self.idx = {}
        self.keys = []
        self.fidx = None
        super().__init__(uri, flag)

    def open(self):
        super().open()
        self.idx, self.keys = {}, []
        self.fidx = open(self.idx_path, self.flag)
        if self.writable:
            return
        for line in self.fidx:
            fields = line.strip().split('\t')
            if len(fields) < 2:
                continue
            key = self.key_type(fields[0])
            self.idx[key] = int(fields[1])
            self.keys.append(key)

    def close(self):
        if not getattr(self, 'is_open', False):
            return
        super().close()
        if self.fidx is not None:
            self.fidx.close()
            self.fidx = None

    def __getstate__(self):
        state = super().__getstate__()
        state['fidx'] = None
        return state

    def seek(self, idx):
        """Position the reader at the record stored under key ``idx``."""
        if self.writable:
            raise AssertionError('file was opened for writing')
        self._check_pid(allow_reset=True)
        _rt().mxb_rec_reader_seek(self.handle, self.idx[idx])

    def tell(self):
        if not self.writable:
            raise AssertionError('tell() of an indexed file is defined for writers')
        return _rt().mxb_rec_writer_tell(self.handle)

    def read_idx(self, idx):
        self.seek(idx)
        return self.read()

    def write_idx(self, idx, buf):
        """Append a record and note its offset under key ``idx``."""
        key = self.key_type(idx)
        offset = self.tell()
        self.write(buf)
        self.fidx.write('%s\t%d\n' % (key, offset))
        self.idx[key] = offset
        self.keys.append(key)


# ---- image records: a fixed header in front of the payload ---------------------------------------------------------
# flag (uint32): 0 for a scalar label, else the number of float32 labels that follow the header; label (float32);
# id, id2 (uint64).
IRHeader = namedtuple('HEADER', ['flag', 'label', 'id', 'id2'])
_HEADER = struct.Struct('IfQQ')


def pack(header, s):
    """Header + payload as one record.  A scalar label sits in the header; an array of labels is stored as float32 values
    between header and payload, with its length in ``flag``."""
    header = IRHeader(*header)
    if isinstance(header.label, numbers.Number):
        return _HEADER.pack(0, header.label, header.id, header.id2) + s
    labels = np.asarray(header.label, dtype=np.float32)
    return _HEADER.pack(labels.size, 0, header.id, header.id2) + labels.tobytes() + s


def unpack(s):
    """Inverse of ``pack``: ``(IRHeader, payload)``; a label array comes back as a float32 NumPy array."""
    header = IRHeader(*_HEADER.unpack_from(s))
    body = s[_HEADER.size:]
    if header.flag > 0:
        nbytes = 4 * header.flag
        header = header._replace(label=np.frombuffer(body[:nbytes], dtype=np.float32))
        body = body[nbytes:]
    return header, body


def unpack_img(s, iscolor=-1):
    """``(IRHeader, image)`` with the image decoded to an HxWxC (or HxW) uint8 array in BGR channel order, the order
    OpenCV-based writers of such files use."""
    from .image import _decode_to_numpy
    header, payload = unpack(s)
    return header, _decode_to_numpy(payload, 1 if iscolor != 0 else 0, to_rgb=False)


def pack_img(header, img, quality=95, img_fmt='.jpg'):
    """Encode a BGR (or grey) uint8 image as JPEG (``quality`` 1-100) or PNG and pack it."""
    from PIL import Image
    pixels = np.asarray(img)
    if pixels.ndim == 3:
        pixels = pixels[..., ::-1]          # BGR -> RGB for the encoder
    out = io.BytesIO()
    if img_fmt.lower() in ('.jpg', '.jpeg'):
        Image.fromarray(pixels).save(out, format='JPEG', quality=quality)
    else:
        Image.fromarray(pixels).save(out, format='PNG')
    return pack(header, out.getvalue())
