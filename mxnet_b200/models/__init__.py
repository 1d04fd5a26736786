"""Benchmark model families: ResNet-50 v1b (NHWC, fused BN), BERT-base (pre-training heads), LSTM LM."""
from .resnet import resnet50_v1b, ResNetV1b
from .bert import BERTModel, BERTForPretrain, bert_base
from .lstm_lm import LSTMLanguageModel
