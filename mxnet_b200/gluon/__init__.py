"""``mx.gluon``."""
from .parameter import Parameter, Constant, DeferredInitializationError
from .block import Block, HybridBlock, SymbolBlock
from .trainer import Trainer
from . import nn, rnn, loss, metric, utils, data, model_zoo, contrib, probability
from .utils import split_and_load, split_data, clip_global_norm
