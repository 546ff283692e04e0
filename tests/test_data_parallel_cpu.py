"""Legacy single-process DataParallel (reference: infini_train/src/nn/parallel/data_parallel.cc:22-100,
src/autograd/comm.cc:13-124): scatter the batch, replicate the module, run the replicas in threads,
gather the outputs; gradients flow back through the broadcast node and are reduce-added on the source
module.  Replicas on CPU "devices" exercise the same graph as replicas on several GPUs."""
import pytest
import torch

from infinitrain_b200.parallel import functional as PF
from infinitrain_b200.parallel.data_parallel import DataParallel


def _mlp(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(12, 32), torch.nn.Tanh(), torch.nn.Linear(32, 5))


@pytest.mark.parametrize("replicas", [1, 2, 3])
def test_data_parallel_matches_the_plain_module(replicas):
    ref, net = _mlp(), _mlp()
    dp = DataParallel(net, devices=[torch.device("cpu")] * replicas)
    x = torch.randn(12, 12)
    target = torch.randn(12, 5)
    out_ref = ref(x)
    out = dp(x)
    assert out.shape == out_ref.shape and torch.allclose(out, out_ref, atol=1e-6)
    torch.nn.functional.mse_loss(out_ref, target).backward()
    torch.nn.functional.mse_loss(out, target).backward()
    for a, b in zip(ref.parameters(), net.parameters()):
        assert b.grad is not None and torch.allclose(a.grad, b.grad, atol=1e-6)


def test_uneven_batch_and_training_steps_follow_the_plain_module():
    """7 samples over 3 replicas (chunks of 3, 3, 1); three SGD steps stay on the single-module trajectory."""
    ref, net = _mlp(1), _mlp(1)
    dp = DataParallel(net, devices=[torch.device("cpu")] * 3)
    opt_ref = torch.optim.SGD(ref.parameters(), lr=0.1)
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(3)
    for _ in range(3):
        x, y = torch.randn(7, 12, generator=g), torch.randn(7, 5, generator=g)
        for model, o in ((ref, opt_ref), (dp, opt)):
            o.zero_grad()
            torch.nn.functional.mse_loss(model(x), y).backward()
            o.step()
    for a, b in zip(ref.parameters(), net.parameters()):
        assert torch.allclose(a, b, atol=1e-6)


def test_replica_errors_surface_on_the_calling_thread():
    class Boom(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(torch.ones(1))

        def forward(self, x):
            raise ValueError("replica failed")

    dp = DataParallel(Boom(), devices=[torch.device("cpu")] * 2)
    with pytest.raises(ValueError, match="replica failed"):
        dp(torch.zeros(4, 1))


def test_scatter_gather_broadcast_replicate_helpers():
    devs = [torch.device("cpu")] * 2
    x = torch.arange(12.0).view(6, 2)
    parts = PF.Scatter(x, devs, 0)
    assert [p.shape[0] for p in parts] == [3, 3] and torch.equal(PF.Gather(parts, devs[0], 0), x)
    cols = PF.Scatter(x, devs, 1)
    assert torch.equal(PF.Gather(cols, devs[0], 1), x)
    copies = PF.BroadcastCoalescedReshape([x, x + 1], devs)
    assert len(copies) == 2 and torch.equal(copies[1][1], x + 1)
    net = _mlp()
    reps = PF.Replicate(net, devs)
    assert len(reps) == 2 and all(torch.equal(a, b) for r in reps for a, b in zip(r.parameters(), net.parameters()))
    assert reps[0][0].weight.data_ptr() != net[0].weight.data_ptr()
