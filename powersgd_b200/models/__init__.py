"""Model zoo: the CIFAR architectures, the LSTM language model and GPT-2 of the benchmark
configurations, plus the small MLP of the plumbing test."""
from .resnet import ResNet18, ResNet34, ResNet50, ResNet101, ResNet152  # noqa: F401
