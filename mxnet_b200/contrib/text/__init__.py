"""Text utilities (``python/mxnet/contrib/text``): token counting, vocabulary, embeddings from files."""
from . import utils, vocab, embedding
from .vocab import Vocabulary
