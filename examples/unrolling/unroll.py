"""One block applied n times becomes n pipeline stages that share (replicated) parameters
(reference examples/unrolling/pippy_unroll.py; its splitter rejects shared parameters, this one replicates them and
lists the copies in ``pipe.replicated_params``).

    python examples/unrolling/unroll.py
"""
import torch
import torch.nn as nn

import pippy_b200 as pp


class IterationBlock(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.lin = nn.Linear(d, d)

    def forward(self, x):
        return torch.relu(self.lin(x))


class IterativeNetwork(nn.Module):
    def __init__(self, d, n_iters):
        super().__init__()
        self.n_iters = n_iters
        self.iter_block = IterationBlock(d)
        self.output_proj = nn.Linear(d, 10)

    def forward(self, x):
        for i in range(self.n_iters):
            x = self.iter_block(x)
            pp.pipe_split()
        return self.output_proj(x)


if __name__ == "__main__":
    torch.manual_seed(0)
    net = IterativeNetwork(64, 3)
    x = torch.randn(8, 64)
    pipe = pp.pipeline(net, 2, (x,))
    print("stages:", pipe.num_stages)
    print("replicated parameter groups:", pipe.replicated_params)
    torch.testing.assert_close(pipe(x)[0], net(x))
    print("unrolled pipeline equals the looped model")
