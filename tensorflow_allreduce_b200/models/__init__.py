"""Models of the benchmark configurations (plain torch.nn): DeepSpeech2-style, GPT-2, ResNet-50."""
from .ds2 import DeepSpeech2, DS2Config  # noqa: F401
from .gpt2 import GPT2, GPT2Config  # noqa: F401
from .resnet50 import ResNet50  # noqa: F401
