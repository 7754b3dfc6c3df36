"""Batch norm fused with the clipped ReLU (`ops/bn_clip.py`, `csrc/cuda/bn_clip.cu`) against plain
PyTorch: `F.batch_norm` in training mode followed by `F.hardtanh`, in fp32 (and in fp64 to tell
rounding from error), forward, backward, running statistics, every vector width."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _reference(x, w, b, rm, rv, eps, momentum, clip, dtype):
    x = x.detach().to(dtype).requires_grad_(True)
    w = w.detach().to(dtype).requires_grad_(True)
    b = b.detach().to(dtype).requires_grad_(True)
    rm, rv = rm.clone().to(dtype), rv.clone().to(dtype)
    y = F.hardtanh(F.batch_norm(x, rm, rv, w, b, True, momentum, eps), 0.0, clip)
    return x, w, b, rm, rv, y


@pytest.mark.parametrize("shape", [(4, 8, 13, 17), (3, 5, 6, 7), (2, 16, 8, 8), (8, 32, 81, 70), (1, 3, 1, 2), (2, 4, 300, 41)])
def test_forward_backward_match_torch(shape):
    from tensorflow_allreduce_b200.ops.bn_clip import bn_clip

    torch.manual_seed(sum(shape))
    n, c = shape[:2]
    x = (torch.randn(shape, device="cuda") * 3 + 1).requires_grad_(True)
    w = (torch.rand(c, device="cuda") * 4 + 0.5).requires_grad_(True)          # scales that push values past the clip at 6
    b = (torch.randn(c, device="cuda") * 2).requires_grad_(True)
    rm0, rv0 = torch.randn(c, device="cuda"), torch.rand(c, device="cuda") + 0.5
    rm, rv = rm0.clone(), rv0.clone()
    clip, eps, momentum = 6.0, 1e-5, 0.1
    y = bn_clip(x, w, b, rm, rv, eps, momentum, clip)
    dy = torch.randn_like(y)
    y.backward(dy)
    for dtype, tol in ((torch.float32, 2e-4), (torch.float64, 2e-4)):
        xr, wr, br, rmr, rvr, yr = _reference(x, w, b, rm0, rv0, eps, momentum, clip, dtype)
        yr.backward(dy.to(dtype))
        # elements within rounding of a clip boundary may fall on either side: leave them out of the gradient check
        z = F.batch_norm(xr.detach(), None, None, wr.detach(), br.detach(), True, 0.0, eps)
        safe = ((z.abs() > 1e-3) & ((z - clip).abs() > 1e-3)).float()
        assert torch.allclose(y.double(), yr.double(), rtol=tol, atol=tol)
        if x.numel() // c > 1:
            assert torch.allclose(rm.double(), rmr.double(), rtol=tol, atol=tol) and torch.allclose(rv.double(), rvr.double(), rtol=tol, atol=tol)
        scale = max(1.0, float(xr.grad.abs().max()))
        if bool((safe == 1).all()):
            assert torch.allclose(x.grad.double(), xr.grad.double(), rtol=1e-3, atol=1e-3 * scale)
            assert torch.allclose(w.grad.double(), wr.grad.double(), rtol=1e-3, atol=1e-3 * float(wr.grad.abs().max() + 1))
            assert torch.allclose(b.grad.double(), br.grad.double(), rtol=1e-3, atol=1e-3 * float(br.grad.abs().max() + 1))
        else:
            # a boundary element changes the channel sums by its own dy: compare with a matching tolerance
            slack = float(dy.abs().max()) * float((1 - safe).sum()) + 1e-3
            assert float((w.grad.double() - wr.grad.double()).abs().max()) <= slack * float(z.abs().max() + 1)


def test_module_keeps_the_batchnorm_interface():
    from tensorflow_allreduce_b200.ops import bn_clip

    torch.manual_seed(0)
    ref_bn = torch.nn.BatchNorm2d(6).cuda()
    mine = bn_clip.BatchNormClip2d(6, clip=4.0).cuda()
    mine.load_state_dict(ref_bn.state_dict())            # same keys
    assert set(mine.state_dict()) == set(ref_bn.state_dict())
    before = bn_clip.launch_count
    for it in range(3):
        x = torch.randn(5, 6, 9, 10, device="cuda") * 2 + 0.5
        a = F.hardtanh(ref_bn(x), 0.0, 4.0)
        b = mine(x)
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-4)
    assert bn_clip.launch_count == before + 3
    assert int(mine.num_batches_tracked) == 3
    assert torch.allclose(mine.running_mean, ref_bn.running_mean, rtol=1e-4, atol=1e-5)
    assert torch.allclose(mine.running_var, ref_bn.running_var, rtol=1e-4, atol=1e-5)
    # evaluation, and layouts the kernels do not take, go through torch
    mine.eval(); ref_bn.eval()
    x = torch.randn(5, 6, 9, 10, device="cuda")
    assert torch.allclose(mine(x), F.hardtanh(ref_bn(x), 0.0, 4.0), rtol=1e-5, atol=1e-5)
    mine.train()
    xl = torch.randn(5, 6, 9, 10, device="cuda").to(memory_format=torch.channels_last)
    count = bn_clip.launch_count
    assert mine(xl).shape == xl.shape and bn_clip.launch_count == count


def test_speech_model_trains_the_same_with_and_without_the_fused_norm():
    from tensorflow_allreduce_b200.models import ds2

    losses = {}
    for fused in (False, True):
        torch.manual_seed(0)
        cfg = ds2.DS2Config(n_frames=64, rnn_hidden=128, rnn_layers=1, label_len=6, persistent_rnn=False, fused_norm=fused)
        model = ds2.DeepSpeech2(cfg).cuda()
        opt = torch.optim.SGD(model.parameters(), lr=1e-3, momentum=0.9)
        torch.manual_seed(1)
        batch = ds2.synthetic_batch(cfg, 4, "cuda")
        out = []
        for _ in range(4):
            opt.zero_grad()
            loss = model.loss(*batch)
            loss.backward()
            opt.step()
            out.append(float(loss))
        losses[fused] = out
        keys = list(model.state_dict())
    assert "conv.1.running_mean" in keys and "conv.4.weight" in keys
    for a, b in zip(losses[False], losses[True]):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), losses
