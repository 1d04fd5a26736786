"""Network visualisation (``python/mxnet/visualization.py``): ``print_summary`` and graphviz ``plot_network``."""
import json

from .symbol import Symbol


def print_summary(symbol, shape=None, line_length=120, positions=(.44, .64, .74, 1.), quiet=False):
    if not isinstance(symbol, Symbol):
        raise TypeError('symbol must be Symbol')
    show_shape = shape is not None
    shape_dict = {}
    if show_shape:
        internals = symbol.get_internals()
        _, out_shapes, _ = internals.infer_shape(**shape)
        if out_shapes is None:
            raise ValueError('Input shape is incomplete')
        shape_dict = dict(zip(internals.list_outputs(), out_shapes))
    conf = json.loads(symbol.tojson())
    nodes = conf['nodes']
    heads = set(h[0] for h in conf['heads'])
    positions = [int(line_length * p) for p in positions]
    to_display = ['Layer (type)', 'Output Shape', 'Param #', 'Previous Layer']
    lines = []

    def print_row(fields):
        line = ''
        for i, field in enumerate(fields):
            line += str(field)
            line = line[:positions[i]]
            line += ' ' * (positions[i] - len(line))
        lines.append(line)
    lines.append('_' * line_length)
    print_row(to_display)
    lines.append('=' * line_length)
    total_params = 0
    arg_shapes = {}
    if show_shape:
        a, _, x = symbol.infer_shape(**shape)
        arg_shapes = dict(zip(symbol.list_arguments(), a))
        arg_shapes.update(zip(symbol.list_auxiliary_states(), x))
    for i, node in enumerate(nodes):
        if node['op'] == 'null' and i > 0:
            continue
        out_shape = []
        op = node['op']
        pre = [nodes[j[0]]['name'] for j in node['inputs'] if nodes[j[0]]['op'] != 'null' or j[0] in heads or
               nodes[j[0]]['name'] in (shape or {})]
        cur_param = 0
        for j in node['inputs']:
            inp = nodes[j[0]]
            if inp['op'] == 'null' and inp['name'] not in (shape or {}):
                s = arg_shapes.get(inp['name'])
                if s:
                    n = 1
                    for d in s:
                        n *= d
                    cur_param += n
        if show_shape:
            key = node['name'] + '_output' if op != 'null' else node['name']
            out_shape = shape_dict.get(key, shape_dict.get(node['name'] + '_output0', []))
        total_params += cur_param
        print_row(['%s(%s)' % (node['name'], op), 'x'.join(str(x) for x in (out_shape[1:] if out_shape else [])),
                   cur_param, pre[0] if pre else ''])
        for p in pre[1:]:
            print_row(['', '', '', p])
        lines.append(('=' if i == len(nodes) - 1 else '_') * line_length)
    lines.append('Total params: {params}'.format(params=total_params))
    lines.append('_' * line_length)
    out = '\n'.join(lines)
    if not quiet:
        print(out)
    return out


def plot_network(symbol, title='plot', save_format='pdf', shape=None, dtype=None, node_attrs=None, hide_weights=True):
    """Graphviz source of the network (a ``graphviz.Digraph`` if the package is installed, else DOT text)."""
    conf = json.loads(symbol.tojson())
    nodes = conf['nodes']
    lines = ['digraph %s {' % json.dumps(title)]
    hidden = set()
    for i, n in enumerate(nodes):
        if n['op'] == 'null' and hide_weights and i > 0 and any(n['name'].endswith(s) for s in (
                '_weight', '_bias', '_gamma', '_beta', '_moving_mean', '_moving_var', '_running_mean', '_running_var')):
            hidden.add(i)
            continue
        label = n['name'] if n['op'] == 'null' else '%s\\n%s' % (n['op'], n['name'])
        lines.append('  n%d [label="%s", shape=%s];' % (i, label, 'oval' if n['op'] == 'null' else 'box'))
    for i, n in enumerate(nodes):
        for j in n['inputs']:
            if j[0] not in hidden and i not in hidden:
                lines.append('  n%d -> n%d;' % (j[0], i))
    lines.append('}')
    src = '\n'.join(lines)
    try:
        import graphviz
        return graphviz.Source(src, format=save_format)
    except ImportError:
        return src
