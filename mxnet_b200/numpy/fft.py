"""``mx.np.fft``: thin device FFT helpers (the reference only ships ``contrib.fft/ifft``)."""
import torch

from .multiarray import ndarray


def _wrap(fn):
    def f(a, n=None, axis=-1, norm=None):
        return ndarray._from_tensor(fn(a._data, n=n, dim=axis, norm=norm), a.ctx)
    return f


rfft = _wrap(torch.fft.rfft)
irfft = _wrap(torch.fft.irfft)
