"""Image input pipeline on the GPU (``ops/cuda/image_pipeline.cu``): nvJPEG decode plus one augmentation kernel.

The reference decodes and augments on host threads (``src/io/iter_image_recordio_2.cc``, ``image_aug_default.cc``) and then
copies the float batch to the device.  :class:`GPUImagePipeline` sends only the compressed JPEG bytes: the images are decoded
on the device into one packed uint8 buffer, and a single kernel crops (random or centre), resizes (bilinear), mirrors,
normalises, casts and lays the batch out (NHWC or NCHW) in the training dtype.
"""
import ctypes as C

import numpy as np
import torch

from ..base import MXNetError

__all__ = ['GPUImagePipeline', 'available']

_RECORD = np.dtype([('offset', '<i8'), ('width', '<i4'), ('height', '<i4'), ('x0', '<f4'), ('y0', '<f4'), ('cw', '<f4'),
                    ('ch', '<f4'), ('mirror', '<i4'), ('pad', '<i4')])
_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _lib():
    from ..ops import cuda
    L = cuda.lib()
    if not getattr(L, '_image_pipeline_declared', False):
        vp, i32, i64p, i32p = C.c_void_p, C.c_int, C.POINTER(C.c_longlong), C.POINTER(C.c_int)
        L.mxb_jpeg_available.restype = i32
        L.mxb_jpeg_decoder_create.argtypes = [i32]
        L.mxb_jpeg_decoder_create.restype = vp
        L.mxb_jpeg_decoder_destroy.argtypes = [vp]
        L.mxb_jpeg_decoder_destroy.restype = None
        L.mxb_jpeg_info_batch.argtypes = [vp, i32, C.POINTER(C.c_char_p), i64p, i32p, i32p, i32p]
        L.mxb_jpeg_info_batch.restype = i32
        L.mxb_jpeg_decode_batch.argtypes = [vp, i32, C.POINTER(C.c_char_p), i64p, vp, i64p, i32p, vp]
        L.mxb_jpeg_decode_batch.restype = i32
        L.mxb_image_augment_batch.argtypes = [i32, vp, vp, vp, i32, i32, i32, i32, C.POINTER(C.c_float), C.POINTER(C.c_float),
                                              C.c_float, vp]
        L.mxb_image_augment_batch.restype = i32
        L.mxb_image_aug_record_bytes.restype = i32
        assert L.mxb_image_aug_record_bytes() == _RECORD.itemsize, 'augmentation record layout mismatch'
        L._image_pipeline_declared = True
    return L


def available():
    """True on a machine with a GPU and a loadable nvJPEG."""
    return torch.cuda.is_available() and bool(_lib().mxb_jpeg_available())


class GPUImagePipeline(object):
    """Decode + augment batches of JPEG images on one GPU.

    ``out_hw``: output height and width; ``layout``: 'NHWC' or 'NCHW'; ``dtype``: float32 / float16 / bfloat16;
    ``mean`` / ``std``: per-channel (RGB, on the 0..255 scale); ``scale``: final multiplier;
    ``resize``: shorter side before cropping (-1: keep); ``rand_crop`` / ``rand_mirror``: training augmentation;
    ``random_resized_crop``: (min area, max area, min ratio, max ratio) of the source area to sample the crop from, as in
    ``image.RandomSizedCropAug``; the chosen rectangle is resampled straight to ``out_hw``;
    ``threads``: host threads that run nvJPEG's entropy decoding, each feeding its own CUDA stream.
    """

    def __init__(self, ctx, out_hw, layout='NHWC', dtype='float16', mean=(0.0, 0.0, 0.0), std=(1.0, 1.0, 1.0), scale=1.0, resize=-1,
                 rand_crop=False, rand_mirror=False, random_resized_crop=None, seed=0, threads=8):
        from ..base import to_torch_dtype
        if not available():
            raise MXNetError('the GPU image pipeline needs a GPU and nvJPEG')
        self.ctx = ctx
        self.device = ctx.torch_device
        self.H, self.W = int(out_hw[0]), int(out_hw[1])
        if layout not in ('NHWC', 'NCHW'):
            raise ValueError('layout must be NHWC or NCHW')
        self.nhwc = layout == 'NHWC'
        self.dtype = to_torch_dtype(dtype) if not isinstance(dtype, torch.dtype) else dtype
        if self.dtype not in _DT:
            raise ValueError('dtype must be float32, float16 or bfloat16')
        self._mean = (C.c_float * 3)(*[float(v) for v in mean])
        self._std = (C.c_float * 3)(*[float(v) for v in std])
        self.scale, self.resize = float(scale), int(resize)
        self.rand_crop, self.rand_mirror, self.rrc = bool(rand_crop), bool(rand_mirror), random_resized_crop
        self._rng = np.random.RandomState(seed)
        with torch.cuda.device(self.device):
            self._dec = _lib().mxb_jpeg_decoder_create(int(threads))
        if not self._dec:
            raise MXNetError('nvJPEG decoder could not be created')
        self._decoded = None                 # packed uint8 buffer of the decoded images, grown on demand
        self.bytes_to_device = 0             # compressed bytes handed to the decoder (observable by tests)

    def __del__(self):
        try:
            if getattr(self, '_dec', None):
                _lib().mxb_jpeg_decoder_destroy(self._dec)
                self._dec = None
        except Exception:   # pylint: disable=broad-except
            pass

    # ---- crop geometry (host, a few floats per image) ---------------------------------------------------------------------------
    def _crop(self, w, h):
        """(x0, y0, cw, ch) in source pixels."""
        if self.rrc is not None:
            amin, amax, rmin, rmax = self.rrc
            for _ in range(10):
                area = self._rng.uniform(amin, amax) * w * h
                ratio = np.exp(self._rng.uniform(np.log(rmin), np.log(rmax)))
                cw, ch = int(round(np.sqrt(area * ratio))), int(round(np.sqrt(area / ratio)))
                if 0 < cw <= w and 0 < ch <= h:
                    return float(self._rng.randint(0, w - cw + 1)), float(self._rng.randint(0, h - ch + 1)), float(cw), float(ch)
            side = min(w, h)
            return (w - side) / 2.0, (h - side) / 2.0, float(side), float(side)
        # resize the shorter side to `resize`, then cut out_hw (random or centred): expressed in source pixels
        s = self.resize / float(min(w, h)) if self.resize > 0 else 1.0
        s = max(s, self.W / float(w), self.H / float(h))            # the scaled image must cover the output
        cw, ch = self.W / s, self.H / s
        if self.rand_crop:
            return float(self._rng.uniform(0, w - cw)), float(self._rng.uniform(0, h - ch)), cw, ch
        return (w - cw) / 2.0, (h - ch) / 2.0, cw, ch

    def __call__(self, jpegs, crops=None, mirrors=None):
        """``jpegs``: list of bytes objects.  ``crops`` / ``mirrors`` override the sampled geometry (for tests).  Returns an
        NDArray [n, H, W, 3] or [n, 3, H, W] on the pipeline's device."""
        from ..ndarray.ndarray import NDArray
        L = _lib()
        n = len(jpegs)
        if n == 0:
            raise ValueError('empty batch')
        bufs = (C.c_char_p * n)(*jpegs)
        lens = (C.c_longlong * n)(*[len(j) for j in jpegs])
        widths, heights, comps = (C.c_int * n)(), (C.c_int * n)(), (C.c_int * n)()
        rc = L.mxb_jpeg_info_batch(self._dec, n, bufs, lens, widths, heights, comps)
        if rc != 0:
            raise MXNetError('image %d of the batch is not a readable JPEG stream' % (rc - 100) if rc >= 100 else 'nvJPEG is unavailable')
        rec = np.zeros(n, dtype=_RECORD)
        off = 0
        for i in range(n):
            w, h = int(widths[i]), int(heights[i])
            rec['offset'][i], rec['width'][i], rec['height'][i] = off, w, h
            x0, y0, cw, ch = crops[i] if crops is not None else self._crop(w, h)
            rec['x0'][i], rec['y0'][i], rec['cw'][i], rec['ch'][i] = x0, y0, cw, ch
            rec['mirror'][i] = int(mirrors[i]) if mirrors is not None else int(self.rand_mirror and self._rng.rand() < 0.5)
            off += (w * h * 3 + 255) // 256 * 256
        with torch.cuda.device(self.device):
            if self._decoded is None or self._decoded.numel() < off:
                self._decoded = torch.empty(max(off, 1 << 20), dtype=torch.uint8, device=self.device)
            stream = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
            offsets = (C.c_longlong * n)(*[int(v) for v in rec['offset']])
            rc = L.mxb_jpeg_decode_batch(self._dec, n, bufs, lens, C.c_void_p(self._decoded.data_ptr()), offsets, widths, stream)
            if rc != 0:
                raise MXNetError('nvJPEG could not decode image %d of the batch' % (rc - 100))
            self.bytes_to_device += sum(len(j) for j in jpegs)
            rec_dev = torch.from_numpy(rec.view(np.uint8).reshape(-1)).to(self.device, non_blocking=True)
            shape = (n, self.H, self.W, 3) if self.nhwc else (n, 3, self.H, self.W)
            out = torch.empty(shape, dtype=self.dtype, device=self.device)
            rc = L.mxb_image_augment_batch(_DT[self.dtype], C.c_void_p(self._decoded.data_ptr()), C.c_void_p(rec_dev.data_ptr()),
                                           C.c_void_p(out.data_ptr()), n, self.H, self.W, 1 if self.nhwc else 0, self._mean, self._std,
                                           self.scale, stream)
            if rc != 0:
                raise MXNetError('image augmentation kernel failed with CUDA error %d' % rc)
            from ..ops.cuda import count_launch
            count_launch(1)
            rec_dev.record_stream(torch.cuda.current_stream(self.device))
        self.last_geometry = rec
        return NDArray._from_tensor(out, self.ctx)
