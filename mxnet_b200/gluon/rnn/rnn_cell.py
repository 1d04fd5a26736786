"""Recurrent cells (``python/mxnet/gluon/rnn/rnn_cell.py``): single-step blocks with ``unroll``."""
from ... import _state
from ...ops import registry as _reg
from ..block import Block, HybridBlock
from ..parameter import Parameter

__all__ = ['RecurrentCell', 'HybridRecurrentCell', 'RNNCell', 'LSTMCell', 'GRUCell', 'LSTMPCell', 'SequentialRNNCell',
           'HybridSequentialRNNCell', 'DropoutCell', 'ModifierCell', 'ZoneoutCell', 'ResidualCell', 'BidirectionalCell',
           'VariationalDropoutCell']


def _op(name, arrays, **attrs):
    return _reg.invoke(name, arrays, attrs)


def _zeros(shape, like, dtype=None):
    import torch
    from ...base import to_torch_dtype
    t = torch.zeros(shape, dtype=to_torch_dtype(dtype) or like._data.dtype, device=like._data.device)
    return like.__class__._from_tensor(t, like.context)


def _format_sequence(length, inputs, layout, merge):
    axis = layout.find('T')
    batch_axis = layout.find('N')
    from ...ndarray.ndarray import NDArray
    if isinstance(inputs, NDArray):
        batch_size = inputs.shape[batch_axis]
        if merge is False:
            assert length is None or length == inputs.shape[axis]
            inputs = [x.squeeze(axis=axis) for x in _op('SliceChannel', [inputs], num_outputs=inputs.shape[axis], axis=axis)] \
                if inputs.shape[axis] > 1 else [inputs.squeeze(axis=axis)]
    else:
        assert length is None or len(inputs) == length
        batch_size = inputs[0].shape[0]
        if merge is True:
            inputs = _op('stack', list(inputs), axis=axis)
    return inputs, axis, batch_size


class RecurrentCell(Block):
    def __init__(self):
        super().__init__()
        self._modified = False
        self.reset()

    def reset(self):
        self._init_counter = -1
        self._counter = -1
        for cell in self._children.values():
            cell.reset()

    def state_info(self, batch_size=0):
        raise NotImplementedError()

    def begin_state(self, batch_size=0, func=None, **kwargs):
        assert not self._modified, 'After applying modifier cells (e.g. ZoneoutCell) the base cell cannot be called ' \
                                   'directly. Call the modifier cell instead.'
        from ... import numpy as mnp, ndarray as nd
        from ...util import is_np_array
        states = []
        for info in self.state_info(batch_size):
            self._init_counter += 1
            f = func or (mnp.zeros if is_np_array() else nd.zeros)
            kw = dict(kwargs)
            info = dict(info)
            shape = info.pop('shape')
            info.pop('__layout__', None)
            kw.update({k: v for k, v in info.items() if k == 'dtype'})
            states.append(f(shape, **kw))
        return states

    def unroll(self, length, inputs, begin_state=None, layout='NTC', merge_outputs=None, valid_length=None):
        self.reset()
        inputs, axis, batch_size = _format_sequence(length, inputs, layout, False)
        if begin_state is None:
            first = inputs[0]
            begin_state = [_zeros(i['shape'], first) for i in self.state_info(batch_size)]
        states = begin_state
        outputs, all_states = [], []
        for i in range(length):
            output, states = self(inputs[i], states)
            outputs.append(output)
            if valid_length is not None:
                all_states.append(states)
        if valid_length is not None:
            import torch
            vl = valid_length._data.long()
            new_states = []
            for si in range(len(states)):
                stacked = torch.stack([s[si]._data for s in all_states], 0)
                idx = (vl - 1).clamp(min=0)
                sel = stacked[idx, torch.arange(stacked.shape[1], device=stacked.device)]
                new_states.append(states[si].__class__._from_tensor(sel, states[si].context))
            states = new_states
            seq = _op('stack', outputs, axis=axis)
            seq = _op('SequenceMask', [seq, valid_length], use_sequence_length=True, axis=axis)
            if merge_outputs is False or merge_outputs is None and False:
                outputs = [seq[(slice(None),) * axis + (t,)] for t in range(length)]
            else:
                outputs = seq
                merge_outputs = True if merge_outputs is None else merge_outputs
                if not merge_outputs:
                    outputs = [seq[(slice(None),) * axis + (t,)] for t in range(length)]
            return outputs, states
        if merge_outputs:
            outputs = _op('stack', outputs, axis=axis)
        return outputs, states

    def _get_activation(self, inputs, activation, **kwargs):
        if isinstance(activation, str):
            if activation in ('tanh', 'relu', 'sigmoid', 'softrelu', 'softsign'):
                return _op('Activation', [inputs], act_type=activation)
            if activation == 'leaky':
                return _op('LeakyReLU', [inputs], act_type='leaky', **kwargs)
        return activation(inputs, **kwargs)

    def forward(self, inputs, states):
        self._counter += 1
        return self.hybrid_forward_impl(inputs, states)


class HybridRecurrentCell(RecurrentCell, HybridBlock):
    def __init__(self):
        HybridBlock.__init__(self)
        self._modified = False
        self.reset()

    def forward(self, inputs, states):
        self._counter += 1
        return self._step(inputs, states)

    def __call__(self, inputs, states):
        return HybridBlock.__call__(self, inputs, states)

    def _step(self, inputs, states):
        raise NotImplementedError


class _GatedCell(HybridRecurrentCell):
    def __init__(self, hidden_size, gates, i2h_weight_initializer, h2h_weight_initializer, i2h_bias_initializer,
                 h2h_bias_initializer, input_size, recur_size=None):
        super().__init__()
        self._hidden_size, self._input_size, self._gates = hidden_size, input_size, gates
        rs = recur_size or hidden_size
        self.i2h_weight = Parameter('i2h_weight', shape=(gates * hidden_size, input_size), init=i2h_weight_initializer,
                                    allow_deferred_init=True)
        self.h2h_weight = Parameter('h2h_weight', shape=(gates * hidden_size, rs), init=h2h_weight_initializer,
                                    allow_deferred_init=True)
        self.i2h_bias = Parameter('i2h_bias', shape=(gates * hidden_size,), init=i2h_bias_initializer,
                                  allow_deferred_init=True)
        self.h2h_bias = Parameter('h2h_bias', shape=(gates * hidden_size,), init=h2h_bias_initializer,
                                  allow_deferred_init=True)

    def infer_shape(self, *args):
        """``infer_shape(x)`` or, as stacked cells are asked by the reference, ``infer_shape(i, x, is_bidirect)``: position
        of the cell in a stack, the stack's input, and whether the cell below is bidirectional (its output is then twice
        the hidden size wide)."""
        if args and isinstance(args[0], int):
            i, x = args[0], args[1]
            is_bidirect = bool(args[2]) if len(args) > 2 else False
            width = x.shape[x.ndim - 1] if i == 0 else self._hidden_size * (2 if is_bidirect else 1)
        else:
            width = args[0].shape[args[0].ndim - 1]
        self.i2h_weight.shape = (self._gates * self._hidden_size, width)

    def _proj(self, inputs, h):
        ctx = inputs.context
        n = self._gates * self._hidden_size
        i2h = _op('FullyConnected', [inputs, self.i2h_weight.data(ctx), self.i2h_bias.data(ctx)], num_hidden=n)
        h2h = _op('FullyConnected', [h, self.h2h_weight.data(ctx), self.h2h_bias.data(ctx)], num_hidden=n)
        return i2h, h2h


class RNNCell(_GatedCell):
    def __init__(self, hidden_size, activation='tanh', i2h_weight_initializer=None, h2h_weight_initializer=None,
                 i2h_bias_initializer='zeros', h2h_bias_initializer='zeros', input_size=0):
        super().__init__(hidden_size, 1, i2h_weight_initializer, h2h_weight_initializer, i2h_bias_initializer,
                         h2h_bias_initializer, input_size)
        self._activation = activation

    def state_info(self, batch_size=0):
        return [{'shape': (batch_size, self._hidden_size), '__layout__': 'NC'}]

    def _alias(self):
        return 'rnn'

    def _step(self, inputs, states):
        i2h, h2h = self._proj(inputs, states[0])
        output = self._get_activation(i2h + h2h, self._activation)
        return output, [output]


class LSTMCell(_GatedCell):
    def __init__(self, hidden_size, i2h_weight_initializer=None, h2h_weight_initializer=None,
                 i2h_bias_initializer='zeros', h2h_bias_initializer='zeros', input_size=0, activation='tanh',
                 recurrent_activation='sigmoid'):
        super().__init__(hidden_size, 4, i2h_weight_initializer, h2h_weight_initializer, i2h_bias_initializer,
                         h2h_bias_initializer, input_size)
        self._activation, self._recurrent_activation = activation, recurrent_activation

    def state_info(self, batch_size=0):
        return [{'shape': (batch_size, self._hidden_size), '__layout__': 'NC'},
                {'shape': (batch_size, self._hidden_size), '__layout__': 'NC'}]

    def _alias(self):
        return 'lstm'

    def _step(self, inputs, states):
        i2h, h2h = self._proj(inputs, states[0])
        gates = i2h + h2h
        sl = _op('SliceChannel', [gates], num_outputs=4, axis=1)
        in_gate = self._get_activation(sl[0], self._recurrent_activation)
        forget_gate = self._get_activation(sl[1], self._recurrent_activation)
        in_transform = self._get_activation(sl[2], self._activation)
        out_gate = self._get_activation(sl[3], self._recurrent_activation)
        next_c = forget_gate * states[1] + in_gate * in_transform
        next_h = out_gate * self._get_activation(next_c, self._activation)
        return next_h, [next_h, next_c]


class GRUCell(_GatedCell):
    def __init__(self, hidden_size, i2h_weight_initializer=None, h2h_weight_initializer=None,
                 i2h_bias_initializer='zeros', h2h_bias_initializer='zeros', input_size=0, activation='tanh',
                 recurrent_activation='sigmoid'):
        super().__init__(hidden_size, 3, i2h_weight_initializer, h2h_weight_initializer, i2h_bias_initializer,
                         h2h_bias_initializer, input_size)
        self._activation, self._recurrent_activation = activation, recurrent_activation

    def state_info(self, batch_size=0):
        return [{'shape': (batch_size, self._hidden_size), '__layout__': 'NC'}]

    def _alias(self):
        return 'gru'

    def _step(self, inputs, states):
        prev = states[0]
        i2h, h2h = self._proj(inputs, prev)
        i = _op('SliceChannel', [i2h], num_outputs=3, axis=1)
        h = _op('SliceChannel', [h2h], num_outputs=3, axis=1)
        reset_gate = self._get_activation(i[0] + h[0], self._recurrent_activation)
        update_gate = self._get_activation(i[1] + h[1], self._recurrent_activation)
        next_h_tmp = self._get_activation(i[2] + reset_gate * h[2], self._activation)
        next_h = (1. - update_gate) * next_h_tmp + update_gate * prev
        return next_h, [next_h]


class LSTMPCell(_GatedCell):
    """LSTM with a projection of the hidden state (``LSTMPCell``)."""

    def __init__(self, hidden_size, projection_size, i2h_weight_initializer=None, h2h_weight_initializer=None,
                 h2r_weight_initializer=None, i2h_bias_initializer='zeros', h2h_bias_initializer='zeros', input_size=0):
        super().__init__(hidden_size, 4, i2h_weight_initializer, h2h_weight_initializer, i2h_bias_initializer,
                         h2h_bias_initializer, input_size, projection_size)
        self._projection_size = projection_size
        self.h2r_weight = Parameter('h2r_weight', shape=(projection_size, hidden_size), init=h2r_weight_initializer,
                                    allow_deferred_init=True)

    def state_info(self, batch_size=0):
        return [{'shape': (batch_size, self._projection_size), '__layout__': 'NC'},
                {'shape': (batch_size, self._hidden_size), '__layout__': 'NC'}]

    def _step(self, inputs, states):
        i2h, h2h = self._proj(inputs, states[0])
        sl = _op('SliceChannel', [i2h + h2h], num_outputs=4, axis=1)
        in_gate, forget_gate = _op('sigmoid', [sl[0]]), _op('sigmoid', [sl[1]])
        in_transform, out_gate = _op('tanh', [sl[2]]), _op('sigmoid', [sl[3]])
        next_c = forget_gate * states[1] + in_gate * in_transform
        hidden = out_gate * _op('tanh', [next_c])
        next_r = _op('FullyConnected', [hidden, self.h2r_weight.data(inputs.context)], num_hidden=self._projection_size,
                     no_bias=True)
        return next_r, [next_r, next_c]


class SequentialRNNCell(RecurrentCell):
    def __init__(self):
        super().__init__()
        self._layers = []

    def add(self, cell):
        self._layers.append(cell)
        self.register_child(cell)

    def infer_shape(self, _, x, is_bidirect=False):
        """Complete the deferred input widths of the stack: the first cell sees ``x``, every later cell the output of the
        cell below (twice as wide under a bidirectional cell)."""
        below_bidirectional, below_width = False, None
        for i, child in enumerate(self._layers):
            if i > 0 and below_width and hasattr(child, 'i2h_weight') and hasattr(child, '_hidden_size'):
                # the reference assumes every cell of a stack has the same size; here the width is the real output width of
                # the cell below
                child.i2h_weight.shape = (child._gates * child._hidden_size, below_width)
            else:
                child.infer_shape(i, x, below_bidirectional)
            below_bidirectional = isinstance(child, BidirectionalCell)
            info = child.state_info(0)
            below_width = info[0]['shape'][-1] * (1 if not below_bidirectional else 1) if info else below_width
            if below_bidirectional:
                below_width = sum(s['shape'][-1] for s in (child.l_cell.state_info(0)[:1] + child.r_cell.state_info(0)[:1]))

    def state_info(self, batch_size=0):
        return sum([c.state_info(batch_size) for c in self._children.values()], [])

    def begin_state(self, **kwargs):
        assert not self._modified
        return sum([c.begin_state(**kwargs) for c in self._children.values()], [])

    def __call__(self, inputs, states):
        self._counter += 1
        next_states = []
        p = 0
        for cell in self._children.values():
            n = len(cell.state_info())
            state = states[p:p + n]
            p += n
            inputs, state = cell(inputs, state)
            next_states.append(state)
        return inputs, sum(next_states, [])

    def unroll(self, length, inputs, begin_state=None, layout='NTC', merge_outputs=None, valid_length=None):
        self.reset()
        inputs, _, batch_size = _format_sequence(length, inputs, layout, None)
        num_cells = len(self._children)
        if begin_state is None:
            first = inputs if not isinstance(inputs, list) else inputs[0]
            begin_state = [_zeros(i['shape'], first) for i in self.state_info(batch_size)]
        p = 0
        next_states = []
        for i, cell in enumerate(self._children.values()):
            n = len(cell.state_info())
            states = begin_state[p:p + n]
            p += n
            inputs, states = cell.unroll(length, inputs=inputs, begin_state=states, layout=layout,
                                         merge_outputs=None if i < num_cells - 1 else merge_outputs,
                                         valid_length=valid_length)
            next_states.extend(states)
        return inputs, next_states

    def __getitem__(self, i):
        return list(self._children.values())[i]

    def __len__(self):
        return len(self._children)

    def forward(self, *args):
        raise NotImplementedError


class HybridSequentialRNNCell(SequentialRNNCell, HybridBlock):
    def __init__(self):
        HybridBlock.__init__(self)
        self._modified = False
        self._layers = []
        self.reset()

    def infer_shape(self, *args):
        pass


class DropoutCell(HybridRecurrentCell):
    def __init__(self, rate, axes=()):
        super().__init__()
        assert isinstance(rate, (int, float)), 'rate must be a number'
        self._rate, self._axes = rate, axes

    def state_info(self, batch_size=0):
        return []

    def _alias(self):
        return 'dropout'

    def _step(self, inputs, states):
        if self._rate > 0:
            inputs = _op('Dropout', [inputs], p=self._rate, axes=self._axes)
        return inputs, states

    def unroll(self, length, inputs, begin_state=None, layout='NTC', merge_outputs=None, valid_length=None):
        self.reset()
        inputs, _, _ = _format_sequence(length, inputs, layout, merge_outputs)
        from ...ndarray.ndarray import NDArray
        if isinstance(inputs, NDArray):
            return self._step(inputs, begin_state if begin_state else [])
        return super().unroll(length, inputs, begin_state=begin_state, layout=layout, merge_outputs=merge_outputs,
                              valid_length=None)


class ModifierCell(HybridRecurrentCell):
    def __init__(self, base_cell):
        assert not base_cell._modified, 'Cell %s is already modified. One cell cannot be modified twice' % base_cell
        base_cell._modified = True
        super().__init__()
        self.base_cell = base_cell

    @property
    def params(self):
        return self.base_cell.params

    def state_info(self, batch_size=0):
        return self.base_cell.state_info(batch_size)

    def begin_state(self, func=None, **kwargs):
        assert not self._modified
        self.base_cell._modified = False
        begin = self.base_cell.begin_state(func=func, **kwargs)
        self.base_cell._modified = True
        return begin

    def infer_shape(self, *args):
        self.base_cell.infer_shape(*args)


class ZoneoutCell(ModifierCell):
    def __init__(self, base_cell, zoneout_outputs=0., zoneout_states=0.):
        assert not isinstance(base_cell, BidirectionalCell), 'BidirectionalCell doesn\'t support zoneout since it ' \
            'doesn\'t support step. Please add ZoneoutCell to the cells underneath instead.'
        super().__init__(base_cell)
        self.zoneout_outputs, self.zoneout_states = zoneout_outputs, zoneout_states
        self._prev_output = None

    def _alias(self):
        return 'zoneout'

    def reset(self):
        super().reset()
        self._prev_output = None

    def _step(self, inputs, states):
        cell, p_outputs, p_states = self.base_cell, self.zoneout_outputs, self.zoneout_states
        next_output, next_states = cell(inputs, states)

        def mask(p, like):
            return _op('Dropout', [_op('ones_like', [like])], p=p)
        prev_output = self._prev_output if self._prev_output is not None else _op('zeros_like', [next_output])
        output = _op('where', [mask(p_outputs, next_output), next_output, prev_output]) if p_outputs != 0. else next_output
        new_states = [_op('where', [mask(p_states, ns), ns, os]) for ns, os in zip(next_states, states)] \
            if p_states != 0. else next_states
        self._prev_output = output
        return output, new_states


class ResidualCell(ModifierCell):
    def _step(self, inputs, states):
        output, states = self.base_cell(inputs, states)
        return output + inputs, states

    def unroll(self, length, inputs, begin_state=None, layout='NTC', merge_outputs=None, valid_length=None):
        self.reset()
        self.base_cell._modified = False
        outputs, states = self.base_cell.unroll(length, inputs=inputs, begin_state=begin_state, layout=layout,
                                                merge_outputs=merge_outputs, valid_length=valid_length)
        self.base_cell._modified = True
        from ...ndarray.ndarray import NDArray
        merge_outputs = isinstance(outputs, NDArray) if merge_outputs is None else merge_outputs
        inputs, axis, _ = _format_sequence(length, inputs, layout, merge_outputs)
        if valid_length is not None:            # the skip connection adds nothing beyond a sequence's end
            merged = inputs if merge_outputs else _op('stack', list(inputs), axis=axis)
            merged = _op('SequenceMask', [merged, valid_length], use_sequence_length=True, axis=axis)
            inputs = merged if merge_outputs else [merged[(slice(None),) * axis + (t,)] for t in range(length)]
        if merge_outputs:
            outputs = outputs + inputs
        else:
            outputs = [i + j for i, j in zip(outputs, inputs)]
        return outputs, states


class BidirectionalCell(HybridRecurrentCell):
    def __init__(self, l_cell, r_cell):
        super().__init__()
        self.l_cell, self.r_cell = l_cell, r_cell

    def __call__(self, inputs, states):
        raise NotImplementedError('Bidirectional cannot be stepped. Please use unroll')

    def state_info(self, batch_size=0):
        return self.l_cell.state_info(batch_size) + self.r_cell.state_info(batch_size)

    def begin_state(self, **kwargs):
        assert not self._modified
        return self.l_cell.begin_state(**kwargs) + self.r_cell.begin_state(**kwargs)

    def infer_shape(self, *args):
        self.l_cell.infer_shape(*args)
        self.r_cell.infer_shape(*args)

    def unroll(self, length, inputs, begin_state=None, layout='NTC', merge_outputs=None, valid_length=None):
        self.reset()
        inputs, axis, batch_size = _format_sequence(length, inputs, layout, False)
        if valid_length is None:
            reversed_inputs = list(reversed(inputs))
        else:
            seq = _op('stack', inputs, axis=0)
            rev = _op('SequenceReverse', [seq, valid_length], use_sequence_length=True)
            reversed_inputs = [rev[t] for t in range(length)]
        if begin_state is None:
            begin_state = [_zeros(i['shape'], inputs[0]) for i in self.state_info(batch_size)]
        states = begin_state
        l_cell, r_cell = self.l_cell, self.r_cell
        nl = len(l_cell.state_info(batch_size))
        l_outputs, l_states = l_cell.unroll(length, inputs=inputs, begin_state=states[:nl], layout=layout,
                                            merge_outputs=False, valid_length=valid_length)
        r_outputs, r_states = r_cell.unroll(length, inputs=reversed_inputs, begin_state=states[nl:], layout=layout,
                                            merge_outputs=False, valid_length=valid_length)
        if valid_length is None:
            reversed_r_outputs = list(reversed(r_outputs))
        else:
            seq = _op('stack', list(r_outputs), axis=0)
            rev = _op('SequenceReverse', [seq, valid_length], use_sequence_length=True)
            reversed_r_outputs = [rev[t] for t in range(length)]
        outputs = [_op('Concat', [l_o, r_o], dim=1) for l_o, r_o in zip(l_outputs, reversed_r_outputs)]
        if merge_outputs or (merge_outputs is None and valid_length is not None):       # masked sequences come back merged
            outputs = _op('stack', outputs, axis=axis)
        return outputs, l_states + r_states


class VariationalDropoutCell(ModifierCell):
    """Same dropout mask at every time step for inputs / states / outputs."""

    def __init__(self, base_cell, drop_inputs=0., drop_states=0., drop_outputs=0.):
        assert not drop_states or not isinstance(base_cell, BidirectionalCell)
        super().__init__(base_cell)
        self.drop_inputs, self.drop_states, self.drop_outputs = drop_inputs, drop_states, drop_outputs
        self.drop_inputs_mask = self.drop_states_mask = self.drop_outputs_mask = None

    def _alias(self):
        return 'vardrop'

    def reset(self):
        super().reset()
        self.drop_inputs_mask = self.drop_states_mask = self.drop_outputs_mask = None

    def _mask(self, p, like):
        return _op('Dropout', [_op('ones_like', [like])], p=p)

    def _step(self, inputs, states):
        cell = self.base_cell
        if self.drop_states:
            if self.drop_states_mask is None:
                self.drop_states_mask = self._mask(self.drop_states, states[0])
            states = list(states)
            states[0] = states[0] * self.drop_states_mask
        if self.drop_inputs:
            if self.drop_inputs_mask is None:
                self.drop_inputs_mask = self._mask(self.drop_inputs, inputs)
            inputs = inputs * self.drop_inputs_mask
        next_output, next_states = cell(inputs, states)
        if self.drop_outputs:
            if self.drop_outputs_mask is None:
                self.drop_outputs_mask = self._mask(self.drop_outputs, next_output)
            next_output = next_output * self.drop_outputs_mask
        return next_output, next_states


def dynamic_unroll(cell, inputs, begin_state, drop_inputs=0, drop_outputs=0, layout='TNC', valid_length=None):
    """Unroll ``cell`` over the time axis of ``inputs`` (one merged array in ``layout``), with optional dropout shared
    across time on the inputs / outputs.  With ``valid_length`` (batch,) the outputs beyond each sequence's length are
    zero and the returned states are those of its last valid step."""
    from ... import numpy_extension as npx, ndarray as nd
    axis = layout.find('T')
    legacy = type(inputs).__name__ != 'ndarray'

    def dropout(x, p):
        if legacy:
            return nd.Dropout(x, p=p, axes=(axis,))
        return npx.dropout(x, p=p, axes=(axis,))
    if drop_inputs:
        inputs = dropout(inputs, drop_inputs)
    outputs, states = cell.unroll(inputs.shape[axis], inputs, begin_state, layout=layout, merge_outputs=True,
                                  valid_length=valid_length)
    if drop_outputs:
        outputs = dropout(outputs, drop_outputs)
    return outputs, states
