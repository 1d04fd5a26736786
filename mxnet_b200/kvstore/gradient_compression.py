"""1-bit and 2-bit gradient compression with residual accumulation
(``src/kvstore/gradient_compression-inl.h:45-215``).

2-bit: each value of (gradient + residual) becomes one of {-threshold, 0, +threshold}; what was not
sent stays in the residual.  1-bit: sign against the threshold, values are ±1.  Sixteen 2-bit codes
(or thirty-two 1-bit codes) are packed per 32-bit word; the packed words are what would travel.
"""
import torch


class GradientCompression(object):
    def __init__(self, type='2bit', threshold=0.5):  # pylint: disable=redefined-builtin
        if type not in ('1bit', '2bit'):
            raise ValueError('Unknown type for gradient compression ' + str(type))
        if type == '2bit' and threshold <= 0:
            raise ValueError('threshold must be greater than 0')
        self.type, self.threshold = type, float(threshold)
        self._residual = {}

    def get_params(self):
        return {'type': self.type, 'threshold': self.threshold}

    def compressed_size(self, n):
        per_word = 16 if self.type == '2bit' else 32
        return (n + per_word - 1) // per_word

    @staticmethod
    def _kernels(t):
        from .. import env
        if not t.is_cuda or not env.get('MXNET_B200_KERNELS'):
            return None
        from ..ops import cuda
        return cuda if cuda.available() else None

    def quantize(self, key, grad):
        """Returns packed codes (one 32-bit word per 16 or 32 values); updates the residual kept for ``key``."""
        g = grad.reshape(-1).float()
        res = self._residual.get(key)
        if res is None or res.shape != g.shape or res.device != g.device:
            res = self._residual[key] = torch.zeros_like(g)
        cuda = self._kernels(g)
        if cuda is not None:
            g = g.contiguous()
            bits = 2 if self.type == '2bit' else 1
            packed = torch.empty(self.compressed_size(g.numel()), dtype=torch.int32, device=g.device)
            cuda.check(cuda.lib().mxb_gc_quantize(bits, cuda.ptr(g), cuda.ptr(res), cuda.ptr(packed), g.numel(), self.threshold,
                                                  cuda.stream_ptr(g.device)), 'gc_quantize')
            cuda.count_launch(1)
            return packed
        res.add_(g)
        t = self.threshold
        if self.type == '2bit':
            pos, neg = res >= t, res <= -t
            codes = torch.where(pos, 3, torch.where(neg, 2, 0)).to(torch.int64)
            res.sub_(pos.float() * t).add_(neg.float() * t)
            per, bits = 16, 2
        else:
            pos = res > t
            codes = pos.to(torch.int64)
            res.sub_(torch.where(pos, torch.ones_like(res), -torch.ones_like(res)))
            per, bits = 32, 1
        n = codes.numel()
        pad = (-n) % per
        if pad:
            codes = torch.cat([codes, codes.new_zeros(pad)])
        codes = codes.reshape(-1, per)
        shifts = torch.arange(per, device=codes.device, dtype=torch.int64) * bits
        packed = (codes << shifts).sum(1)
        return (packed & 0xFFFFFFFF).to(torch.int64)

    def dequantize(self, packed, n, dtype=torch.float32):
        cuda = self._kernels(packed)
        if cuda is not None and packed.dtype == torch.int32:
            out = torch.empty(n, dtype=torch.float32, device=packed.device)
            cuda.check(cuda.lib().mxb_gc_dequantize(2 if self.type == '2bit' else 1, cuda.ptr(packed), cuda.ptr(out), n,
                                                    self.threshold, 0, cuda.stream_ptr(packed.device)), 'gc_dequantize')
            cuda.count_launch(1)
            return out.to(dtype)
        packed = packed.to(torch.int64) & 0xFFFFFFFF
        per, bits = (16, 2) if self.type == '2bit' else (32, 1)
        shifts = torch.arange(per, device=packed.device, dtype=torch.int64) * bits
        codes = ((packed.reshape(-1, 1) >> shifts) & ((1 << bits) - 1)).reshape(-1)[:n]
        t = self.threshold
        if self.type == '2bit':
            out = torch.where(codes == 3, t, torch.where(codes == 2, -t, 0.0))
        else:
            out = torch.where(codes == 1, 1.0, -1.0)
        return out.to(dtype)

    def compress_roundtrip(self, key, grad):
        """What the receiver reconstructs from this device's contribution."""
        packed = self.quantize(key, grad)
        return self.dequantize(packed, grad.numel(), grad.dtype).reshape(grad.shape)
