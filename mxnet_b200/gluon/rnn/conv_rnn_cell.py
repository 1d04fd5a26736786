"""Convolutional recurrent cells (``python/mxnet/gluon/rnn/conv_rnn_cell.py``): the i2h / h2h
projections of RNN/LSTM/GRU cells are convolutions over spatial feature maps."""
from ...ops import registry as _reg
from ..parameter import Parameter
from .rnn_cell import HybridRecurrentCell

__all__ = ['Conv1DRNNCell', 'Conv2DRNNCell', 'Conv3DRNNCell', 'Conv1DLSTMCell', 'Conv2DLSTMCell', 'Conv3DLSTMCell',
           'Conv1DGRUCell', 'Conv2DGRUCell', 'Conv3DGRUCell']


def _op(name, arrays, **attrs):
    return _reg.invoke(name, arrays, attrs)


def _tup(v, n):
    return (v,) * n if isinstance(v, int) else tuple(v)


class _ConvCell(HybridRecurrentCell):
    def __init__(self, input_shape, hidden_channels, i2h_kernel, h2h_kernel, i2h_pad, i2h_dilate, h2h_dilate, gates,
                 dims, conv_layout, activation, i2h_weight_initializer=None, h2h_weight_initializer=None,
                 i2h_bias_initializer='zeros', h2h_bias_initializer='zeros'):
        super().__init__()
        self._hidden_channels, self._input_shape, self._conv_layout, self._activation = \
            hidden_channels, tuple(input_shape), conv_layout, activation
        self._gates, self._dims = gates, dims
        self._i2h_kernel, self._h2h_kernel = _tup(i2h_kernel, dims), _tup(h2h_kernel, dims)
        assert all(k % 2 == 1 for k in self._h2h_kernel), 'Only support odd number, get h2h_kernel= %s' % str(h2h_kernel)
        self._i2h_pad, self._i2h_dilate, self._h2h_dilate = _tup(i2h_pad, dims), _tup(i2h_dilate, dims), _tup(h2h_dilate, dims)
        self._h2h_pad = tuple(d * (k - 1) // 2 for d, k in zip(self._h2h_dilate, self._h2h_kernel))
        in_c = input_shape[0]
        self._state_shape = (hidden_channels,) + tuple(
            (s + 2 * p - d * (k - 1) - 1) + 1 for s, p, d, k in zip(input_shape[1:], self._i2h_pad, self._i2h_dilate,
                                                                   self._i2h_kernel))
        n = gates * hidden_channels
        self.i2h_weight = Parameter('i2h_weight', shape=(n, in_c) + self._i2h_kernel, init=i2h_weight_initializer,
                                    allow_deferred_init=True)
        self.h2h_weight = Parameter('h2h_weight', shape=(n, hidden_channels) + self._h2h_kernel, init=h2h_weight_initializer)
        self.i2h_bias = Parameter('i2h_bias', shape=(n,), init=i2h_bias_initializer)
        self.h2h_bias = Parameter('h2h_bias', shape=(n,), init=h2h_bias_initializer)

    def infer_shape(self, *args):
        """Complete a deferred input-channel count (``input_shape[0] == -1``) from the input; also takes the stacked
        form ``infer_shape(i, x, is_bidirect)``."""
        x = args[1] if args and isinstance(args[0], int) else args[0]
        shape = tuple(self.i2h_weight.shape)
        if shape[1] <= 0:
            # counted from the end: ``x`` may be one step (N, C, ...) or a whole sequence (N, T, C, ...)
            axis = x.ndim - (len(self._conv_layout) - self._conv_layout.find('C'))
            self.i2h_weight.shape = shape[:1] + (x.shape[axis],) + shape[2:]

    def state_info(self, batch_size=0):
        n = 2 if self._gates == 4 else 1
        return [{'shape': (batch_size,) + self._state_shape, '__layout__': self._conv_layout}] * n

    def _conv(self, inputs, h):
        ctx = inputs.context
        n = self._gates * self._hidden_channels
        i2h = _op('Convolution', [inputs, self.i2h_weight.data(ctx), self.i2h_bias.data(ctx)], kernel=self._i2h_kernel,
                  pad=self._i2h_pad, dilate=self._i2h_dilate, num_filter=n)
        h2h = _op('Convolution', [h, self.h2h_weight.data(ctx), self.h2h_bias.data(ctx)], kernel=self._h2h_kernel,
                  pad=self._h2h_pad, dilate=self._h2h_dilate, num_filter=n)
        return i2h, h2h

    def _step(self, inputs, states):
        i2h, h2h = self._conv(inputs, states[0])
        if self._gates == 1:
            out = self._get_activation(i2h + h2h, self._activation)
            return out, [out]
        if self._gates == 4:
            sl = _op('SliceChannel', [i2h + h2h], num_outputs=4, axis=1)
            i, f = _op('sigmoid', [sl[0]]), _op('sigmoid', [sl[1]])
            g, o = self._get_activation(sl[2], self._activation), _op('sigmoid', [sl[3]])
            c = f * states[1] + i * g
            h = o * self._get_activation(c, self._activation)
            return h, [h, c]
        i = _op('SliceChannel', [i2h], num_outputs=3, axis=1)
        h = _op('SliceChannel', [h2h], num_outputs=3, axis=1)
        r, z = _op('sigmoid', [i[0] + h[0]]), _op('sigmoid', [i[1] + h[1]])
        nt = self._get_activation(i[2] + r * h[2], self._activation)
        out = (1. - z) * nt + z * states[0]
        return out, [out]


def _make(name, gates, dims, layout):
    def __init__(self, input_shape, hidden_channels, i2h_kernel, h2h_kernel, i2h_pad=(0,) * dims, i2h_dilate=(1,) * dims,
                 h2h_dilate=(1,) * dims, i2h_weight_initializer=None, h2h_weight_initializer=None,
                 i2h_bias_initializer='zeros', h2h_bias_initializer='zeros', conv_layout=layout, activation='tanh'):
        _ConvCell.__init__(self, input_shape, hidden_channels, i2h_kernel, h2h_kernel, i2h_pad, i2h_dilate, h2h_dilate,
                           gates, dims, conv_layout, activation, i2h_weight_initializer, h2h_weight_initializer,
                           i2h_bias_initializer, h2h_bias_initializer)
    return type(name, (_ConvCell,), {'__init__': __init__})


for _d, _l in ((1, 'NCW'), (2, 'NCHW'), (3, 'NCDHW')):
    globals()['Conv%dDRNNCell' % _d] = _make('Conv%dDRNNCell' % _d, 1, _d, _l)
    globals()['Conv%dDLSTMCell' % _d] = _make('Conv%dDLSTMCell' % _d, 4, _d, _l)
    globals()['Conv%dDGRUCell' % _d] = _make('Conv%dDGRUCell' % _d, 3, _d, _l)
