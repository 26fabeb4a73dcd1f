"""Model families used by the benchmarks and examples (plain PyTorch
modules; the framework itself is model-agnostic)."""
from horovod_b200.models.resnet import resnet50, resnet_tiny  # noqa: F401
from horovod_b200.models.transformer import (TransformerLM, bert_large,  # noqa: F401
                                             gpt2_medium, tiny_lm)
from horovod_b200.models.mlp import MLP  # noqa: F401
