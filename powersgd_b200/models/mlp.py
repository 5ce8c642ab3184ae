"""The two-layer perceptron of the plumbing configuration (784 -> 256 -> 10, ReLU)."""
import torch.nn as nn


def MLP(inputs: int = 784, hidden: int = 256, classes: int = 10) -> nn.Sequential:
    return nn.Sequential(nn.Linear(inputs, hidden), nn.ReLU(), nn.Linear(hidden, classes))
