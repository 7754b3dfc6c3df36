"""Persistent GRU kernels (tcgen05 / TMA, csrc/cuda/gru_persistent.cu) against `torch.nn.GRU` run in
full fp32: outputs and every gradient, uni- and bidirectional, one and several layers. The
kernels multiply in TF32 (10-bit mantissa), so the comparison allows a few 1e-3 relative."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _supported(T, B, H, nd):
    from tensorflow_allreduce_b200.ops import persistent_gru as pg

    if not pg.supported(T, B, H, nd):
        pytest.skip("persistent GRU kernels need a compute-capability-10 GPU with enough SMs")
    return pg


@pytest.mark.parametrize("T,B,I,H,layers,nd", [
    (3, 4, 64, 128, 1, 1),
    (6, 5, 40, 128, 1, 2),
    (9, 32, 96, 256, 2, 2),
    (24, 17, 200, 512, 1, 2),
    (12, 32, 1312, 1024, 1, 2),
])
def test_matches_torch_gru(T, B, I, H, layers, nd):
    pg = _supported(T, B, H, nd)
    old = torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    try:
        torch.manual_seed(T * 1000 + H)
        rnn = torch.nn.GRU(I, H, num_layers=layers, bidirectional=(nd == 2)).cuda()
        x = torch.randn(T, B, I, device="cuda", requires_grad=True)
        y_ref, _ = rnn(x)
        y = pg.gru_forward(rnn, x)
        torch.cuda.synchronize()
        pg.check_status()
        assert y.shape == y_ref.shape
        assert (y - y_ref).abs().max().item() < 2e-3 * max(1.0, y_ref.abs().max().item())
        g = torch.randn_like(y_ref)
        params = list(rnn.parameters())
        ref = torch.autograd.grad(y_ref, [x] + params, g)
        got = torch.autograd.grad(y, [x] + params, g)
        torch.cuda.synchronize()
        pg.check_status()
        names = ["x"] + [n for n, _ in rnn.named_parameters()]
        for n, a, b in zip(names, ref, got):
            scale = a.abs().max().item() + 1e-6
            assert (a - b).abs().max().item() / scale < 5e-3, n
    finally:
        torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = old


def test_unsupported_shapes_are_reported():
    from tensorflow_allreduce_b200.ops import persistent_gru as pg

    assert not pg.supported(10, 33, 128, 2)      # batch above one MMA tile
    assert not pg.supported(10, 8, 100, 1)       # hidden size not a multiple of 128
    assert not pg.supported(10, 8, 2048, 2)      # weights of 16 units no longer fit in shared memory


def test_model_uses_persistent_path_and_trains():
    from tensorflow_allreduce_b200.models import ds2
    from tensorflow_allreduce_b200.ops import persistent_gru as pg

    cfg = ds2.DS2Config(n_frames=40, rnn_hidden=128, rnn_layers=2, label_len=5)
    _supported(20, 4, 128, 2)
    torch.manual_seed(0)
    model = ds2.DeepSpeech2(cfg).cuda()
    ref = ds2.DeepSpeech2(ds2.DS2Config(n_frames=40, rnn_hidden=128, rnn_layers=2, label_len=5, persistent_rnn=False)).cuda()
    ref.load_state_dict(model.state_dict())
    batch = ds2.synthetic_batch(cfg, 4, "cuda")
    before = pg.launch_count
    loss = model.loss(*batch)
    loss.backward()
    loss_ref = ref.loss(*batch)
    loss_ref.backward()
    torch.cuda.synchronize()
    pg.check_status()
    assert pg.launch_count - before == 2 * cfg.rnn_layers
    assert abs(loss.item() - loss_ref.item()) < 5e-3 * abs(loss_ref.item())
    for (n, p), q in zip(model.named_parameters(), ref.parameters()):
        scale = q.grad.abs().max().item() + 1e-6
        assert (p.grad - q.grad).abs().max().item() / scale < 2e-2, n
