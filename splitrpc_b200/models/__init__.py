"""Model families served by the stack, built from this library's sm_100a kernels."""
from .resnet import ResNet50  # noqa: F401
from .bert import BertClassifier, BERT_BASE, BERT_LARGE  # noqa: F401
from .bert_tp import BertClassifierTP  # noqa: F401
