"""Word-level LSTM language model (the reference's ``example/gluon/word_language_model``): embedding →
dropout → multi-layer fused LSTM → dropout → decoder tied to the embedding weight."""
from ..gluon import nn, rnn
from ..gluon.block import HybridBlock
from ..gluon.parameter import Parameter
from ..ops import registry as _reg


class LSTMLanguageModel(HybridBlock):
    def __init__(self, vocab_size=33278, embed_size=650, hidden_size=650, num_layers=2, dropout=0.5, tie_weights=True):
        super().__init__()
        assert not tie_weights or embed_size == hidden_size
        self._vocab, self._hidden, self._layers, self._tie = vocab_size, hidden_size, num_layers, tie_weights
        self.drop = nn.Dropout(dropout)
        self.embedding = nn.Embedding(vocab_size, embed_size)
        self.rnn = rnn.LSTM(hidden_size, num_layers, dropout=dropout, input_size=embed_size)
        if tie_weights:
            self.decoder_bias = Parameter('decoder_bias', shape=(vocab_size,), init='zeros')
        else:
            self.decoder = nn.Dense(vocab_size, in_units=hidden_size, flatten=False)

    def begin_state(self, batch_size, **kwargs):
        return self.rnn.begin_state(batch_size, **kwargs)

    def forward(self, inputs, hidden):
        emb = self.drop(self.embedding(inputs))
        output, hidden = self.rnn(emb, hidden)
        output = self.drop(output)
        flat = output.reshape((-1, self._hidden))
        if self._tie:
            ctx = inputs.context
            decoded = _reg.invoke('FullyConnected', [flat, self.embedding.weight.data(ctx), self.decoder_bias.data(ctx)],
                                  {'num_hidden': self._vocab})
        else:
            decoded = self.decoder(flat)
        return decoded, hidden
