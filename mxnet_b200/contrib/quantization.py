"""Post-training INT8 quantization (``python/mxnet/contrib/quantization.py`` +
``src/operator/quantization/quantize_graph_pass.cc``): calibrate activation ranges (``naive`` min/max
or ``entropy`` KL threshold) and rewrite FullyConnected / Convolution nodes into
quantize → quantized op → dequantize chains."""
import numpy as np

from ..ops import registry as _reg
from ..symbol.symbol import Symbol, _Node, _topo

__all__ = ['quantize_model', 'quantize_net', 'quantize_graph', 'calib_graph', 'CalibrationCollector']


class CalibrationCollector(object):
    """Collects per-tensor statistics while the float model runs on calibration batches."""

    def __init__(self, mode='naive', num_bins=8001):
        self.mode, self.num_bins = mode, num_bins
        self.min_max = {}
        self.hist = {}

    def collect(self, name, arr):
        a = arr.asnumpy() if hasattr(arr, 'asnumpy') else np.asarray(arr)
        mn, mx = float(a.min()), float(a.max())
        if name in self.min_max:
            omn, omx = self.min_max[name]
            mn, mx = min(mn, omn), max(mx, omx)
        self.min_max[name] = (mn, mx)
        if self.mode == 'entropy':
            th = max(abs(mn), abs(mx))
            h, edges = np.histogram(a, bins=self.num_bins, range=(-th, th))
            if name in self.hist and self.hist[name][1][-1] >= th:
                oh, oe = self.hist[name]
                h2, _ = np.histogram(a, bins=self.num_bins, range=(oe[0], oe[-1]))
                self.hist[name] = (oh + h2, oe)
            else:
                self.hist[name] = (h, edges)

    def thresholds(self):
        if self.mode == 'naive':
            return dict(self.min_max)
        out = {}
        import torch
        for name, (h, e) in self.hist.items():
            t, _ = _reg.get('_contrib_calibrate_entropy').fn(torch.from_numpy(h.astype('float32')),
                                                             torch.from_numpy(e.astype('float32')), 255)
            out[name] = (-float(t), float(t))
        return out


def quantize_graph(sym, excluded_sym_names=(), excluded_op_names=(), quantized_dtype='int8', thresholds=None):
    """Rewrite FullyConnected / Convolution nodes into int8 chains.  Weights are quantized on the
    fly from their float values (ranges from the tensors); activations use ``thresholds`` when given."""
    thresholds = thresholds or {}
    q2, deq = _reg.get('_contrib_quantize_v2'), _reg.get('_contrib_dequantize')
    mapping = {}
    for n in _topo(sym._outputs):
        ins = [mapping[id(i)][k] for i, k in n.inputs]
        if n.op is None:
            mapping[id(n)] = [(n, 0)]
            continue
        target = {'FullyConnected': '_contrib_quantized_fully_connected', 'Convolution': '_contrib_quantized_conv'}.get(n.op.name)
        if target is None or n.name in excluded_sym_names or n.op.name in excluded_op_names:
            nn = _Node(n.op, n.name, dict(n.attrs), ins, n.nout, dict(n.user_attrs))
            mapping[id(n)] = [(nn, i) for i in range(n.nout)]
            continue
        th = thresholds.get(n.inputs[0][0].name + '_output', thresholds.get(n.inputs[0][0].name))
        dattrs = {'out_type': 'int8'}
        if th is not None:
            dattrs.update(min_calib_range=th[0], max_calib_range=th[1])
        qd = _Node(q2, n.name + '_data_quantize', dattrs, [ins[0]], 3)
        qw = _Node(q2, n.name + '_weight_quantize', {'out_type': 'int8'}, [ins[1]], 3)
        no_bias = n.attrs.get('no_bias', False) or len(ins) < 3
        q_inputs = [(qd, 0), (qw, 0)]
        if not no_bias:
            qb = _Node(q2, n.name + '_bias_quantize', {'out_type': 'int8'}, [ins[2]], 3)
            q_inputs += [(qb, 0), (qd, 1), (qd, 2), (qw, 1), (qw, 2), (qb, 1), (qb, 2)]
        else:
            # the quantized ops take (data, weight, bias, min/max...) positionally; pass weight stats for the unused bias slot
            q_inputs += [(qw, 0), (qd, 1), (qd, 2), (qw, 1), (qw, 2), (qw, 1), (qw, 2)]
        attrs = dict(n.attrs)
        attrs['no_bias'] = bool(no_bias)
        qop = _Node(_reg.get(target), n.name + '_quantized', attrs, q_inputs, 3)
        d = _Node(deq, n.name + '_dequantize', {}, [(qop, 0), (qop, 1), (qop, 2)], 1)
        mapping[id(n)] = [(d, 0)]
    return Symbol([mapping[id(n)][k] for n, k in sym._outputs])


def calib_graph(qsym, arg_params, aux_params, collector, calib_mode='entropy', quantized_dtype='int8'):
    return qsym, arg_params, aux_params


def quantize_model(sym, arg_params, aux_params, data_names=('data',), device=None, excluded_sym_names=None,
                   excluded_op_names=None, calib_mode='entropy', calib_data=None, num_calib_batches=None,
                   quantized_dtype='int8', quantize_mode='smart', quantize_granularity='tensor-wise', logger=None, ctx=None):
    thresholds = None
    if calib_mode != 'none' and calib_data is not None:
        collector = CalibrationCollector('naive' if calib_mode == 'naive' else 'entropy')
        internals = sym.get_internals()
        names = internals.list_outputs()
        feed_params = {k: v._data for k, v in arg_params.items()}
        feed_params.update({k: v._data for k, v in aux_params.items()})
        n = 0
        for batch in calib_data:
            feed = dict(feed_params)
            for dn, d in zip(data_names, batch.data):
                feed[dn] = d._data
            for v in internals.list_inputs():
                if v not in feed:
                    import torch
                    feed[v] = torch.zeros(batch.data[0].shape[0])
            outs = internals._run(feed)
            for nm, o in zip(names, outs):
                collector.collect(nm, o.detach().cpu().numpy())
            n += 1
            if num_calib_batches is not None and n >= num_calib_batches:
                break
        thresholds = collector.thresholds()
    qsym = quantize_graph(sym, excluded_sym_names or (), excluded_op_names or (), quantized_dtype, thresholds)
    return qsym, arg_params, aux_params


def quantize_net(network, quantized_dtype='auto', quantize_mode='full', quantize_granularity='tensor-wise',
                 exclude_layers=None, exclude_layers_match=None, exclude_operators=None, calib_data=None,
                 data_shapes=None, calib_mode='none', num_calib_batches=None, device=None, LayerOutputCollector=None,
                 logger=None, ctx=None):
    """Quantize a HybridBlock: trace, rewrite, and return a ``SymbolBlock`` sharing the parameters."""
    from ..gluon.block import SymbolBlock
    from .. import ndarray as nd
    if network._cached_graph is None:
        assert data_shapes is not None or calib_data is not None, 'data_shapes or calib_data is needed to trace the network'
        if data_shapes is not None:
            shapes = [d.shape if hasattr(d, 'shape') and not isinstance(d, tuple) else tuple(d) for d in data_shapes]
            where = device or ctx
            if where is None:                     # trace where the parameters live
                first_param = next(iter(network.collect_params().values()), None)
                where = first_param.list_ctx()[0] if first_param is not None and first_param._data else None
            args = [nd.zeros(s, ctx=where) for s in shapes]
        else:
            first = next(iter(calib_data))
            args = [first[0] if isinstance(first, (list, tuple)) else first]
        network(*args)
        network._trace(*args)
    inputs, sym = network._cached_graph
    qsym = quantize_graph(sym, exclude_layers or (), exclude_operators or (), 'int8')
    return SymbolBlock(qsym, inputs, dict(network.collect_params().items()))


def quantize_model_onednn(sym, arg_params, aux_params, data_names=('data',), device=None, excluded_sym_names=None,
                          excluded_op_names=None, calib_mode='entropy', calib_data=None, num_calib_batches=None,
                          quantized_dtype='int8', quantize_mode='smart', quantize_granularity='tensor-wise', logger=None):
    """The reference quantises and then fuses for its oneDNN CPU back end; there is no such back end here, so this is
    :func:`quantize_model` (the int8 operators run through the tensor library on the given device)."""
    return quantize_model(sym, arg_params, aux_params, data_names=data_names, device=device,
                          excluded_sym_names=excluded_sym_names, excluded_op_names=excluded_op_names, calib_mode=calib_mode,
                          calib_data=calib_data, num_calib_batches=num_calib_batches, quantized_dtype=quantized_dtype,
                          quantize_mode=quantize_mode, quantize_granularity=quantize_granularity, logger=logger)
