"""Token embeddings loaded from text files (``python/mxnet/contrib/text/embedding.py``)."""
import io
import logging

import numpy as np

from .vocab import Vocabulary

_registry = {}


def register(cls):
    _registry[cls.__name__.lower()] = cls
    return cls


def create(embedding_name, **kwargs):
    return _registry[embedding_name.lower()](**kwargs)


def get_pretrained_file_names(embedding_name=None):
    return {k: [] for k in _registry} if embedding_name is None else []


class _TokenEmbedding(Vocabulary):
    def __init__(self, **kwargs):
        super().__init__(**kwargs)
        self._vec_len = 0
        self._idx_to_vec = None

    def _load_embedding(self, path, elem_delim=' ', init_unknown_vec=np.zeros, encoding='utf8'):
        from ... import ndarray as nd
        vecs, tokens = [], set()
        with io.open(path, 'r', encoding=encoding) as f:
            for line_num, line in enumerate(f):
                elems = line.rstrip().split(elem_delim)
                if len(elems) <= 2:
                    continue
                token, vec = elems[0], [float(i) for i in elems[1:]]
                if token in tokens or token == self.unknown_token:
                    continue
                if not self._vec_len:
                    self._vec_len = len(vec)
                    vecs.append(init_unknown_vec(self._vec_len))
                tokens.add(token)
                self._idx_to_token.append(token)
                self._token_to_idx[token] = len(self._idx_to_token) - 1
                vecs.append(np.asarray(vec))
        self._idx_to_vec = nd.array(np.stack(vecs).astype('float32'))

    @property
    def vec_len(self): return self._vec_len
    @property
    def idx_to_vec(self): return self._idx_to_vec

    def get_vecs_by_tokens(self, tokens, lower_case_backup=False):
        to_reduce = not isinstance(tokens, list)
        if to_reduce:
            tokens = [tokens]
        if not lower_case_backup:
            indices = [self.token_to_idx.get(t, 0) for t in tokens]
        else:
            indices = [self.token_to_idx[t] if t in self.token_to_idx else self.token_to_idx.get(t.lower(), 0) for t in tokens]
        from ... import ndarray as nd
        vecs = self.idx_to_vec[nd.array(indices, dtype='int64')]
        return vecs[0] if to_reduce else vecs

    def _build_embedding_for_vocabulary(self, vocabulary):
        """Keep only the tokens of ``vocabulary``, in its order; tokens without a loaded vector get the unknown vector."""
        from ... import ndarray as nd
        vecs = self.get_vecs_by_tokens(list(vocabulary.idx_to_token)).asnumpy()
        self._idx_to_token = list(vocabulary.idx_to_token)
        self._token_to_idx = dict(vocabulary.token_to_idx)
        self._idx_to_vec = nd.array(vecs)

    def update_token_vectors(self, tokens, new_vectors):
        if not isinstance(tokens, list):
            tokens = [tokens]
        for i, t in enumerate(tokens):
            if t not in self.token_to_idx:
                raise ValueError('Token %s is unknown.' % t)
            self._idx_to_vec[self.token_to_idx[t]] = new_vectors[i] if new_vectors.ndim > 1 else new_vectors


@register
class CustomEmbedding(_TokenEmbedding):
    def __init__(self, pretrained_file_path, elem_delim=' ', encoding='utf8', init_unknown_vec=np.zeros, vocabulary=None, **kwargs):
        super().__init__(**kwargs)
        self._load_embedding(pretrained_file_path, elem_delim, init_unknown_vec, encoding)
        if vocabulary is not None:
            self._build_embedding_for_vocabulary(vocabulary)


@register
class GloVe(CustomEmbedding):
    pass


@register
class FastText(CustomEmbedding):
    pass


class CompositeEmbedding(_TokenEmbedding):
    def __init__(self, vocabulary, token_embeddings):
        super().__init__()
        from ... import ndarray as nd
        if not isinstance(token_embeddings, list):
            token_embeddings = [token_embeddings]
        self._idx_to_token = vocabulary.idx_to_token[:]
        self._token_to_idx = dict(vocabulary.token_to_idx)
        parts = [e.get_vecs_by_tokens(self._idx_to_token).asnumpy() for e in token_embeddings]
        self._idx_to_vec = nd.array(np.concatenate(parts, 1))
        self._vec_len = self._idx_to_vec.shape[1]
