"""stage_backward and the dI/dW split (reference test/test_stage_backward.py)."""
import copy

import torch
import torch.nn as nn

from pippy_b200.backward import (
    _null_coalesce_accumulate, stage_backward, stage_backward_input, stage_backward_weight,
)


class MLP(nn.Module):
    def __init__(self, d=16):
        super().__init__()
        self.net1, self.net2, self.ln = nn.Linear(d, d), nn.Linear(d, d), nn.LayerNorm(d)

    def forward(self, x):
        return self.net2(self.ln(torch.relu(self.net1(x)))) + x


def test_stage_backward_matches_autograd():
    torch.manual_seed(0)
    mod, ref = MLP(), None
    ref = copy.deepcopy(mod)
    x = torch.randn(4, 16, requires_grad=True)
    target = torch.randn(4, 16)
    loss = nn.functional.mse_loss(mod(x), target)
    grads = stage_backward(loss, None, [x])
    xr = x.detach().clone().requires_grad_()
    nn.functional.mse_loss(ref(xr), target).backward()
    torch.testing.assert_close(grads[0], xr.grad)
    for (n, p), (_, q) in zip(mod.named_parameters(), ref.named_parameters()):
        torch.testing.assert_close(p.grad, q.grad, msg=n)


def test_stage_backward_tuple_outputs_and_none_grads():
    a = torch.randn(3, requires_grad=True)
    out = (a * 2, a.detach() * 3, a * 4)
    grads = stage_backward(out, (torch.ones(3), None, torch.ones(3)), [a, 5])
    torch.testing.assert_close(grads[0], torch.full((3,), 6.0))
    assert grads[1] is None
    assert _null_coalesce_accumulate(None, None) is None
    assert _null_coalesce_accumulate(torch.ones(1), None).item() == 1


def test_split_backward_equals_full_backward():
    torch.manual_seed(0)
    mod = MLP()
    ref = copy.deepcopy(mod)
    x = torch.randn(4, 16, requires_grad=True)
    g = torch.randn(4, 16)
    out = mod(x)
    in_grads, plan = stage_backward_input([out], [g], [x], mod.parameters())
    assert all(p.grad is None for p in mod.parameters()), "input half must not touch parameter gradients"
    stage_backward_weight(mod.parameters(), plan)
    xr = x.detach().clone().requires_grad_()
    ref(xr).backward(g)
    torch.testing.assert_close(in_grads[0], xr.grad)
    for (n, p), (_, q) in zip(mod.named_parameters(), ref.named_parameters()):
        torch.testing.assert_close(p.grad, q.grad, msg=n)


def test_split_backward_first_stage_without_input_grads():
    mod = MLP()
    ref = copy.deepcopy(mod)
    x = torch.randn(4, 16)  # model input: no gradient wanted
    g = torch.randn(4, 16)
    in_grads, plan = stage_backward_input([mod(x)], [g], [x], mod.parameters())
    assert in_grads == [None]
    stage_backward_weight(mod.parameters(), plan)
    ref(x).backward(g)
    for p, q in zip(mod.parameters(), ref.parameters()):
        torch.testing.assert_close(p.grad, q.grad)


def test_split_backward_shared_parameter_falls_back_to_full():
    lin = nn.Linear(8, 8)
    x = torch.randn(2, 8, requires_grad=True)
    out = lin(torch.relu(lin(x)))  # the same weight is reachable from two split points
    in_grads, plan = stage_backward_input([out], [torch.ones(2, 8)], [x], lin.parameters())
    stage_backward_weight(lin.parameters(), plan)
    lin2 = copy.deepcopy(lin)
    lin2.zero_grad()
    xr = x.detach().clone().requires_grad_()
    lin2(torch.relu(lin2(xr))).backward(torch.ones(2, 8))
    torch.testing.assert_close(in_grads[0], xr.grad)
    torch.testing.assert_close(lin.weight.grad, lin2.weight.grad)
