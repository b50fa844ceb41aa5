"""The small MLP of the reference's README and basic examples (512 -> 512 -> 1024 -> 256 -> 10)."""
import torch
import torch.nn as nn


class MLPModule(nn.Module):
    def __init__(self, d_in: int, d_out: int, relu: bool = True):
        super().__init__()
        self.lin = nn.Linear(d_in, d_out)
        self.relu = nn.ReLU() if relu else nn.Identity()

    def forward(self, x):
        return self.relu(self.lin(x))


class ReadmeMLP(nn.Module):
    def __init__(self, d_in: int = 512):
        super().__init__()
        self.layer0 = MLPModule(d_in, 512)
        self.layer1 = MLPModule(512, 1024)
        self.layer2 = MLPModule(1024, 256)
        self.output_proj = nn.Linear(256, 10)

    def forward(self, x):
        return self.output_proj(self.layer2(self.layer1(self.layer0(x))))
