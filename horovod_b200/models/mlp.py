"""The 784-512-10 multilayer perceptron of the CPU plumbing check."""
import torch.nn as nn


class MLP(nn.Module):
    def __init__(self, d_in=784, d_hidden=512, d_out=10):
        super().__init__()
        self.fc1 = nn.Linear(d_in, d_hidden)
        self.fc2 = nn.Linear(d_hidden, d_out)

    def forward(self, x):
        return self.fc2(nn.functional.relu(self.fc1(x)))
