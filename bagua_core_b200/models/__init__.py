"""Benchmark model definitions (random init; synthetic data)."""
from .bert import BertConfig, BertForQuestionAnswering  # noqa: F401
from .vision import MLP, VGG16, ResNet50  # noqa: F401
