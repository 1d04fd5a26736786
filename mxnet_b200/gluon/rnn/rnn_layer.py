"""Fused recurrent layers ``RNN`` / ``LSTM`` / ``GRU`` (``python/mxnet/gluon/rnn/rnn_layer.py``).

Parameters are kept per layer and direction (``l0_i2h_weight``, ``l0_h2h_weight``, ``l0_i2h_bias``,
``l0_h2h_bias``, ``r0_…`` for the reverse direction, ``…_h2r_weight`` with projection); the forward
pass concatenates them into the flat vector the fused ``RNN`` operator expects (all weights first,
then all biases)."""
from ...ops import registry as _reg
from ..block import HybridBlock
from ..parameter import Parameter

__all__ = ['RNN', 'LSTM', 'GRU']


def _op(name, arrays, **attrs):
    return _reg.invoke(name, arrays, attrs)


class _RNNLayer(HybridBlock):
    def __init__(self, hidden_size, num_layers, layout, dropout, bidirectional, input_size, i2h_weight_initializer,
                 h2h_weight_initializer, i2h_bias_initializer, h2h_bias_initializer, mode, projection_size,
                 h2r_weight_initializer, lstm_state_clip_min, lstm_state_clip_max, lstm_state_clip_nan, dtype,
                 use_sequence_length=False):
        super().__init__()
        assert layout in ('TNC', 'NTC'), 'Invalid layout %s; must be one of ["TNC" or "NTC"]' % layout
        self._hidden_size, self._projection_size = hidden_size, projection_size if projection_size else None
        self._num_layers, self._mode, self._layout, self._dropout = num_layers, mode, layout, dropout
        self._dir = 2 if bidirectional else 1
        self._input_size = input_size
        self._lstm_state_clip_min, self._lstm_state_clip_max = lstm_state_clip_min, lstm_state_clip_max
        self._lstm_state_clip_nan = lstm_state_clip_nan
        self._dtype = dtype
        self._use_sequence_length = use_sequence_length
        self._gates = {'rnn_relu': 1, 'rnn_tanh': 1, 'lstm': 4, 'gru': 3}[mode]
        ng, ni, nh = self._gates, input_size, hidden_size
        nproj = self._projection_size or nh
        for i in range(num_layers):
            for j in ['l', 'r'][:self._dir]:
                self._register_param('{}{}_i2h_weight'.format(j, i), (ng * nh, ni), i2h_weight_initializer, dtype)
                self._register_param('{}{}_h2h_weight'.format(j, i), (ng * nh, nproj), h2h_weight_initializer, dtype)
                self._register_param('{}{}_i2h_bias'.format(j, i), (ng * nh,), i2h_bias_initializer, dtype)
                self._register_param('{}{}_h2h_bias'.format(j, i), (ng * nh,), h2h_bias_initializer, dtype)
                if self._projection_size:
                    self._register_param('{}{}_h2r_weight'.format(j, i), (nproj, nh), h2r_weight_initializer, dtype)
            ni = nproj * self._dir

    def _register_param(self, name, shape, init, dtype):
        p = Parameter(name, shape=shape, init=init, allow_deferred_init=True, dtype=dtype)
        setattr(self, name, p)
        return p

    def __repr__(self):
        s = '{name}({mapping}, {_layout}'
        if self._num_layers != 1:
            s += ', num_layers={_num_layers}'
        if self._dropout != 0:
            s += ', dropout={_dropout}'
        if self._dir == 2:
            s += ', bidirectional'
        s += ')'
        shape = self.l0_i2h_weight.shape
        mapping = '{0} -> {1}'.format(shape[1] if shape[1] else None, shape[0] // self._gates)
        return s.format(name=self.__class__.__name__, mapping=mapping, **self.__dict__)

    def state_info(self, batch_size=0):
        raise NotImplementedError

    def begin_state(self, batch_size=0, func=None, **kwargs):
        """Initial recurrent state(s), zeros by default."""
        from ... import numpy as mnp, ndarray as nd
        from ...util import is_np_array
        states = []
        for info in self.state_info(batch_size):
            if func is None:
                f = mnp.zeros if is_np_array() else nd.zeros
            else:
                f = func
            kw = dict(kwargs)
            kw.setdefault('dtype', self._dtype)
            states.append(f(info['shape'], **kw))
        return states

    def infer_shape(self, inputs, *args):
        ni = inputs.shape[2]
        nproj = self._projection_size or self._hidden_size
        for i in range(self._num_layers):
            for j in ['l', 'r'][:self._dir]:
                p = getattr(self, '{}{}_i2h_weight'.format(j, i))
                p.shape = (self._gates * self._hidden_size, ni)
            ni = nproj * self._dir

    def _param_order(self):
        """Names of the layer's parameters in the order of the flat vector the RNN operator takes: all weights (layer by layer,
        direction by direction, input-to-hidden before hidden-to-hidden, then the projection), then all biases."""
        order = []
        for t in ('weight', 'bias'):
            for i in range(self._num_layers):
                for j in ['l', 'r'][:self._dir]:
                    for g in ('i2h', 'h2h'):
                        order.append('{}{}_{}_{}'.format(j, i, g, t))
                    if t == 'weight' and self._projection_size:
                        order.append('{}{}_h2r_weight'.format(j, i))
        return order

    def _translate_loaded(self, prefix, loaded):
        """A checkpoint that stores this layer as one flat `rnn_param` vector (python/mxnet/gluon/rnn/rnn_layer.py of the
        2.x reference) is cut into the per-matrix parameters of this layer; shapes that are still deferred are completed from
        the length of the vector."""
        key = prefix + 'rnn_param'
        if key not in loaded:
            return
        flat = loaded.pop(key)
        order = self._param_order()
        first = getattr(self, order[0])
        if first.shape is None or any(d <= 0 for d in first.shape):
            H, G, D, L = self._hidden_size, self._gates, self._dir, self._num_layers
            P = self._projection_size or H
            rest = sum(D * (G * H * (P * D) + G * H * P + 2 * G * H + (P * H if self._projection_size else 0)) for _ in range(1, L))
            per_input = D * G * H
            fixed0 = D * (G * H * P + 2 * G * H + (P * H if self._projection_size else 0))
            ni = (int(flat.size) - rest - fixed0) // per_input
            for j in ['l', 'r'][:D]:
                getattr(self, '{}0_i2h_weight'.format(j)).shape = (G * H, ni)
            nin = P * D
            for i in range(1, L):
                for j in ['l', 'r'][:D]:
                    getattr(self, '{}{}_i2h_weight'.format(j, i)).shape = (G * H, nin)
        at = 0
        for name in order:
            p = getattr(self, name)
            n = 1
            for d in p.shape:
                n *= d
            loaded[prefix + name] = flat[at:at + n].reshape(p.shape)
            at += n
        if at != int(flat.size):
            raise ValueError('rnn_param has %d elements, this layer needs %d' % (int(flat.size), at))

    def forward(self, inputs, states=None, sequence_length=None):
        batch_size = inputs.shape[self._layout.find('N')]
        skip_states = states is None
        if skip_states:
            states = self.begin_state(batch_size, ctx=inputs.context, dtype=inputs.dtype) \
                if inputs._kind == 'nd' else self.begin_state(batch_size, device=inputs.context, dtype=inputs.dtype)
        if not isinstance(states, (list, tuple)):
            states = [states]
        for state, info in zip(states, self.state_info(batch_size)):
            if state.shape != info['shape']:
                raise ValueError('Invalid recurrent state shape. Expecting %s, got %s.' % (
                    str(info['shape']), str(state.shape)))
        out = self._forward_kernel(inputs, states, sequence_length)
        return out[0] if skip_states else out

    def _forward_kernel(self, inputs, states, sequence_length):
        ctx = inputs.context
        if self._layout == 'NTC':
            inputs = _op('SwapAxis', [inputs], dim1=0, dim2=1)
        order = self._param_order()
        params = _op('_rnn_param_concat', [getattr(self, n).data(ctx) for n in order], dim=0)
        args = [inputs, params] + list(states)
        if self._use_sequence_length and sequence_length is not None:
            args.append(sequence_length)
        attrs = dict(state_size=self._hidden_size, num_layers=self._num_layers, bidirectional=self._dir == 2,
                     p=self._dropout, state_outputs=True, mode=self._mode, projection_size=self._projection_size,
                     lstm_state_clip_min=self._lstm_state_clip_min, lstm_state_clip_max=self._lstm_state_clip_max,
                     lstm_state_clip_nan=self._lstm_state_clip_nan,
                     use_sequence_length=self._use_sequence_length and sequence_length is not None)
        rnn = _op('RNN', args, **attrs)
        if self._mode == 'lstm':
            outputs, states = rnn[0], [rnn[1], rnn[2]]
        else:
            outputs, states = rnn[0], [rnn[1]]
        if self._layout == 'NTC':
            outputs = _op('SwapAxis', [outputs], dim1=0, dim2=1)
        return outputs, states


class RNN(_RNNLayer):
    def __init__(self, hidden_size, num_layers=1, activation='relu', layout='TNC', dropout=0, bidirectional=False,
                 i2h_weight_initializer=None, h2h_weight_initializer=None, i2h_bias_initializer='zeros',
                 h2h_bias_initializer='zeros', input_size=0, dtype='float32', use_sequence_length=False, **kwargs):
        super().__init__(hidden_size, num_layers, layout, dropout, bidirectional, input_size, i2h_weight_initializer,
                         h2h_weight_initializer, i2h_bias_initializer, h2h_bias_initializer, 'rnn_' + activation,
                         None, None, None, None, False, dtype, use_sequence_length)

    def state_info(self, batch_size=0):
        return [{'shape': (self._num_layers * self._dir, batch_size, self._hidden_size), '__layout__': 'LNC',
                 'dtype': self._dtype}]


class LSTM(_RNNLayer):
    def __init__(self, hidden_size, num_layers=1, layout='TNC', dropout=0, bidirectional=False, input_size=0,
                 i2h_weight_initializer=None, h2h_weight_initializer=None, i2h_bias_initializer='zeros',
                 h2h_bias_initializer='zeros', projection_size=None, h2r_weight_initializer=None, state_clip_min=None,
                 state_clip_max=None, state_clip_nan=False, dtype='float32', use_sequence_length=False, **kwargs):
        super().__init__(hidden_size, num_layers, layout, dropout, bidirectional, input_size, i2h_weight_initializer,
                         h2h_weight_initializer, i2h_bias_initializer, h2h_bias_initializer, 'lstm', projection_size,
                         h2r_weight_initializer, state_clip_min, state_clip_max, state_clip_nan, dtype,
                         use_sequence_length)

    def state_info(self, batch_size=0):
        proj = self._projection_size or self._hidden_size
        return [{'shape': (self._num_layers * self._dir, batch_size, proj), '__layout__': 'LNC', 'dtype': self._dtype},
                {'shape': (self._num_layers * self._dir, batch_size, self._hidden_size), '__layout__': 'LNC',
                 'dtype': self._dtype}]


class GRU(_RNNLayer):
    def __init__(self, hidden_size, num_layers=1, layout='TNC', dropout=0, bidirectional=False, input_size=0,
                 i2h_weight_initializer=None, h2h_weight_initializer=None, i2h_bias_initializer='zeros',
                 h2h_bias_initializer='zeros', dtype='float32', use_sequence_length=False, **kwargs):
        super().__init__(hidden_size, num_layers, layout, dropout, bidirectional, input_size, i2h_weight_initializer,
                         h2h_weight_initializer, i2h_bias_initializer, h2h_bias_initializer, 'gru', None, None, None,
                         None, False, dtype, use_sequence_length)

    def state_info(self, batch_size=0):
        return [{'shape': (self._num_layers * self._dir, batch_size, self._hidden_size), '__layout__': 'LNC',
                 'dtype': self._dtype}]
