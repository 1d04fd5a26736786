"""Operators on sparse storage (``src/operator/tensor/{cast_storage,sparse_retain,dot}-inl.*``).

Row-sparse and CSR arrays are small host-side classes (``ndarray/sparse.py``) holding dense
component tensors; the operators here work on those components.  Dense fallbacks mirror the
reference's storage-fallback mechanism (``src/common/exec_utils.h``)."""
from __future__ import annotations

import torch

from .registry import register


@register('_sparse_retain_dense', inputs=('data', 'indices'))
def sparse_retain_dense(data, indices):
    out = torch.zeros_like(data)
    idx = indices.long()
    out[idx] = data[idx]
    return out


@register('_contrib_SparseEmbedding', inputs=('data', 'weight'), defaults={'input_dim': 0, 'output_dim': 0, 'dtype': 'float32'})
def sparse_embedding(data, weight, input_dim=0, output_dim=0, dtype='float32', sparse_grad=True):
    return torch.nn.functional.embedding(data.long(), weight)


@register('_contrib_getnnz', inputs=('data',), defaults={'axis': None})
def getnnz(data, axis=None):
    nz = data != 0
    return nz.sum() if axis is None else nz.sum(axis)


@register('_contrib_edge_id', inputs=('data', 'u', 'v'))
def edge_id(data, u, v):
    return data[u.long(), v.long()]


@register('_contrib_dgl_adjacency', inputs=('data',))
def dgl_adjacency(data):
    return (data != 0).to(torch.float32)


# ---- graph operators designed for DGL (src/operator/contrib/dgl_graph.cc) ---------------------------------------------
# A graph is its adjacency matrix with edge ids as values (0 = no edge); row i lists the neighbours vertex i receives
# messages from.  The arrays here are the dense forms; the CSR wrappers of ndarray/sparse.py convert on the way in / out.
def _renumber(sub):
    """Edge ids 1, 2, ... in row-major order of the non-zero entries."""
    nz = sub != 0
    new = torch.zeros_like(sub)
    new[nz] = torch.arange(1, int(nz.sum()) + 1, dtype=sub.dtype, device=sub.device)
    return new


@register('_contrib_dgl_subgraph', 'dgl_subgraph', inputs=('graph', '*varrays'),
          nout=lambda a: (int(a.get('num_args', 2)) - 1) * (2 if a.get('return_mapping') else 1),
          defaults={'num_args': 2, 'return_mapping': False})
def dgl_subgraph(graph, *varrays, num_args=2, return_mapping=False):
    """Induced sub-graphs for each vertex set: matrices with new edge ids and, with ``return_mapping``, the same matrices
    with the parent's edge ids (all new-id matrices first, then all mappings)."""
    subs = [graph[v.long()][:, v.long()] for v in varrays]
    out = [_renumber(s) for s in subs]
    if return_mapping:
        out += subs
    return tuple(out) if len(out) > 1 else out[0]


@register('_contrib_dgl_graph_compact', 'dgl_graph_compact', inputs=('*data',),
          nout=lambda a: (int(a.get('num_args', 2)) // 2),
          defaults={'num_args': 2, 'return_mapping': False, 'graph_sizes': ()})
def dgl_graph_compact(*data, num_args=2, return_mapping=False, graph_sizes=()):
    """Sampled sub-graphs (rows = sampled vertices in order, columns = parent vertex ids) reduced to square matrices over
    the sampled vertices only.  Inputs: the n sub-graphs, then the n vertex-id arrays of the samplers."""
    n = len(data) // 2
    sizes = [graph_sizes] * n if isinstance(graph_sizes, int) else list(graph_sizes)
    out = []
    for g, vids, size in zip(data[:n], data[n:], sizes):
        size = int(size)
        cols = vids[:size].long()
        sub = g[:size][:, cols]
        out.append(sub if return_mapping else _renumber(sub))
    return tuple(out) if len(out) > 1 else out[0]


def _neighbor_sample(graph, seeds, num_hops, num_neighbor, max_num_vertices, prob=None):
    import numpy as np
    g = graph.detach().cpu().numpy()
    p = prob.detach().cpu().numpy().astype('float64') if prob is not None else None
    layer_of = {}
    frontier = []
    for s in seeds.detach().cpu().numpy().astype('int64').tolist():
        if s not in layer_of and len(layer_of) < max_num_vertices:
            layer_of[s] = 0
            frontier.append(s)
    edges = {}                                   # (dst, src) -> edge id
    for hop in range(1, num_hops + 1):
        nxt = []
        for dst in frontier:
            nbrs = np.nonzero(g[dst])[0]
            if len(nbrs) > num_neighbor:
                if p is None:
                    nbrs = np.random.choice(nbrs, num_neighbor, replace=False)
                else:
                    w = p[nbrs]
                    nbrs = np.random.choice(nbrs, num_neighbor, replace=False, p=w / w.sum()) if w.sum() > 0 else nbrs[:num_neighbor]
            for src in sorted(int(v) for v in nbrs):
                if src not in layer_of:
                    if len(layer_of) >= max_num_vertices:
                        continue
                    layer_of[src] = hop
                    nxt.append(src)
                edges[(dst, src)] = g[dst, src]
        frontier = nxt
    verts = sorted(layer_of)
    n = len(verts)
    dev = graph.device
    vid = torch.full((max_num_vertices + 1,), -1, dtype=torch.int64, device=dev)
    vid[:n] = torch.tensor(verts, dtype=torch.int64)
    vid[-1] = n
    sub = torch.zeros((max_num_vertices, graph.shape[1]), dtype=graph.dtype, device=dev)
    row = {v: i for i, v in enumerate(verts)}
    for (dst, src), eid in edges.items():
        sub[row[dst], src] = float(eid)
    layer = torch.full((max_num_vertices,), -1, dtype=torch.int64, device=dev)
    layer[:n] = torch.tensor([layer_of[v] for v in verts], dtype=torch.int64)
    out = [vid, sub]
    if p is not None:
        pr = torch.full((max_num_vertices,), -1.0, dtype=torch.float32, device=dev)
        pr[:n] = torch.tensor([p[v] for v in verts], dtype=torch.float32)
        out.append(pr)
    out.append(layer)
    return out


def _sampler(with_prob):
    per = 4 if with_prob else 3

    def op(graph, *rest, num_args=2, num_hops=1, num_neighbor=2, max_num_vertices=100):
        prob, seeds = (rest[0], rest[1:]) if with_prob else (None, rest)
        results = [_neighbor_sample(graph, s, int(num_hops), int(num_neighbor), int(max_num_vertices), prob) for s in seeds]
        return tuple(r[k] for k in range(per) for r in results)        # grouped by kind, like the reference's outputs
    return op


register('_contrib_dgl_csr_neighbor_uniform_sample', 'dgl_csr_neighbor_uniform_sample', inputs=('csr_matrix', '*seed_arrays'),
         nout=lambda a: 3 * (int(a.get('num_args', 2)) - 1),
         defaults={'num_args': 2, 'num_hops': 1, 'num_neighbor': 2, 'max_num_vertices': 100})(_sampler(False))
register('_contrib_dgl_csr_neighbor_non_uniform_sample', 'dgl_csr_neighbor_non_uniform_sample',
         inputs=('csr_matrix', 'probability', '*seed_arrays'), nout=lambda a: 4 * (int(a.get('num_args', 3)) - 2),
         defaults={'num_args': 3, 'num_hops': 1, 'num_neighbor': 2, 'max_num_vertices': 100})(_sampler(True))
