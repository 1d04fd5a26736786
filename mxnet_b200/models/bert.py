"""BERT encoder with the pre-training heads (masked LM + next sentence prediction).

Architecture of the benchmark configuration: 12 layers, hidden 768, 12 heads, FFN 3072 with GELU,
vocabulary 30522, 512 positions, post-LayerNorm.  Self-attention uses the fused multi-head attention
operator on a packed QKV projection (the reference composes ``interleaved_matmul_selfatt_qk`` →
softmax → dropout → ``interleaved_matmul_selfatt_valatt``, ``src/operator/contrib/transformer.cc``)."""
from ..gluon import nn
from ..gluon.block import HybridBlock
from ..gluon.parameter import Parameter
from ..ops import registry as _reg

__all__ = ['BERTEncoderLayer', 'BERTModel', 'BERTForPretrain', 'bert_base']


def _op(name, arrays, **attrs):
    return _reg.invoke(name, arrays, attrs)


class BERTEncoderLayer(HybridBlock):
    def __init__(self, units=768, hidden_size=3072, num_heads=12, dropout=0.1, layer_norm_eps=1e-12):
        super().__init__()
        self._units, self._heads, self._dropout = units, num_heads, dropout
        self.attn_qkv = nn.Dense(3 * units, flatten=False, in_units=units)
        self.attn_proj = nn.Dense(units, flatten=False, in_units=units)
        self.ln1 = nn.LayerNorm(epsilon=layer_norm_eps, in_channels=units)
        self.ffn1 = nn.Dense(hidden_size, flatten=False, in_units=units)
        self.ffn2 = nn.Dense(units, flatten=False, in_units=hidden_size)
        self.ln2 = nn.LayerNorm(epsilon=layer_norm_eps, in_channels=units)

    def forward(self, x, mask=None):
        qkv = self.attn_qkv(x)
        args = [qkv] if mask is None else [qkv, mask]
        ctx_vec = _op('_contrib_fused_self_attention', args, heads=self._heads, dropout=self._dropout, layout='NTC')
        x = self.ln1(_op('_contrib_dropout_add', [self.attn_proj(ctx_vec), x], p=self._dropout))
        h = _op('LeakyReLU', [self.ffn1(x)], act_type='gelu')
        return self.ln2(_op('_contrib_dropout_add', [self.ffn2(h), x], p=self._dropout))


class BERTModel(HybridBlock):
    def __init__(self, vocab_size=30522, units=768, hidden_size=3072, num_layers=12, num_heads=12, max_length=512,
                 token_type_vocab_size=2, dropout=0.1, layer_norm_eps=1e-12):
        super().__init__()
        self._units = units
        self.word_embed = nn.Embedding(vocab_size, units)
        self.token_type_embed = nn.Embedding(token_type_vocab_size, units)
        self.position_weight = Parameter('position_weight', shape=(max_length, units))
        self.embed_ln = nn.LayerNorm(epsilon=layer_norm_eps, in_channels=units)
        self.embed_drop = nn.Dropout(dropout)
        self.layers = nn.HybridSequential()
        for _ in range(num_layers):
            self.layers.add(BERTEncoderLayer(units, hidden_size, num_heads, dropout, layer_norm_eps))
        self.pooler = nn.Dense(units, activation='tanh', flatten=False, in_units=units)

    def forward(self, inputs, token_types, valid_mask=None):
        T = inputs.shape[1]
        pos = self.position_weight.data(inputs.context)[0:T]
        x = self.word_embed(inputs) + self.token_type_embed(token_types) + pos.reshape((1, T, self._units))
        x = self.embed_drop(self.embed_ln(x))
        for layer in self.layers._children.values():
            x = layer(x, valid_mask)
        pooled = self.pooler(x[:, 0, :])
        return x, pooled


class BERTForPretrain(HybridBlock):
    """Masked-LM decoder (tied to the word embedding) and next-sentence classifier on top of BERT."""

    def __init__(self, backbone=None, vocab_size=30522, units=768, layer_norm_eps=1e-12, **kwargs):
        super().__init__()
        self.backbone = backbone if backbone is not None else BERTModel(vocab_size=vocab_size, units=units, **kwargs)
        self._vocab, self._units = vocab_size, units
        self.mlm_dense = nn.Dense(units, flatten=False, in_units=units)
        self.mlm_ln = nn.LayerNorm(epsilon=layer_norm_eps, in_channels=units)
        self.mlm_bias = Parameter('mlm_bias', shape=(vocab_size,), init='zeros')
        self.nsp = nn.Dense(2, in_units=units)

    def forward(self, inputs, token_types, valid_mask, masked_positions):
        seq, pooled = self.backbone(inputs, token_types, valid_mask)
        N, T, C = seq.shape
        flat = seq.reshape((N * T, C))
        from .. import numpy as mnp, ndarray as nd
        offs = (mnp.arange(N, dtype='int64', ctx=seq.context) if seq._kind == 'np' else
                nd.arange(0, N, ctx=seq.context, dtype='int64')).reshape((N, 1)) * T
        idx = (masked_positions.astype('int64') + offs).reshape((-1,))
        picked = _op('take', [flat, idx], axis=0)
        h = _op('LeakyReLU', [self.mlm_dense(picked)], act_type='gelu')
        h = self.mlm_ln(h)
        w = self.backbone.word_embed.weight.data(seq.context)
        scores = _op('FullyConnected', [h, w, self.mlm_bias.data(seq.context)], num_hidden=self._vocab, flatten=False)
        return scores, self.nsp(pooled)


def bert_base(**kwargs):
    return BERTForPretrain(vocab_size=30522, units=768, hidden_size=3072, num_layers=12, num_heads=12, max_length=512, **kwargs)
