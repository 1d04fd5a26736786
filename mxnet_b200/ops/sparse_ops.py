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
