"""DeepSpeech2-style speech model: the flagship data-parallel benchmark configuration.

Two 2-D convolutions over (frequency, time) with batch norm and clipped ReLU, a stack of
bidirectional GRU layers, a linear layer to the character classes and CTC loss. The reference
ships no such model; its pieces there are Conv2D/cuDNN, FusedBatchNorm, Relu6-style clipping,
GRU cells (tensorflow/contrib/rnn/kernels/gru_ops.h:69-119) or CudnnRNN, and a CPU-only CTC loss
(tensorflow/core/kernels/ctc_loss_op.cc:167). Here the convolutions, the output layer and the loss
are plain torch.nn modules on cuDNN/cuBLAS; batch norm and the clipped ReLU behind it are one
module on the library's two-pass kernels (`ops/bn_clip.py`); the GRU stack keeps its `nn.GRU` module
and parameters but, on a GPU that supports them, is evaluated by the library's persistent
tcgen05 kernels (`ops/persistent_gru.py`); the gradient reduction and update around the model are
the library's fused collectives.
"""
from __future__ import annotations

import dataclasses

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclasses.dataclass
class DS2Config:
    n_freq: int = 161
    n_frames: int = 700
    conv_channels: int = 32
    rnn_hidden: int = 1024
    rnn_layers: int = 5
    n_classes: int = 29          # blank + 28 characters
    label_len: int = 100
    persistent_rnn: bool = True  # run the GRU stack on the library's persistent tcgen05 kernels when they support the shape
    fused_norm: bool = True      # batch norm + clipped ReLU as one module on the library's two-pass kernels (ops/bn_clip.py)


class DeepSpeech2(nn.Module):
    def __init__(self, cfg: DS2Config = DS2Config()):
        super().__init__()
        self.cfg = cfg
        c = cfg.conv_channels

        def norm_act():
            # Two modules either way, so that the parameter names (conv.1.*, conv.4.*) do not depend on the choice.
            if cfg.fused_norm:
                from ..ops.bn_clip import BatchNormClip2d

                return [BatchNormClip2d(c, clip=20.0), nn.Identity()]
            return [nn.BatchNorm2d(c), nn.Hardtanh(0.0, 20.0, inplace=True)]

        self.conv = nn.Sequential(
            nn.Conv2d(1, c, kernel_size=(41, 11), stride=(2, 2), padding=(20, 5), bias=False),
            *norm_act(),
            nn.Conv2d(c, c, kernel_size=(21, 11), stride=(2, 1), padding=(10, 5), bias=False),
            *norm_act(),
        )
        f = (cfg.n_freq + 2 * 20 - 41) // 2 + 1
        f = (f + 2 * 10 - 21) // 2 + 1
        self.rnn_input = c * f
        self.rnn = nn.GRU(self.rnn_input, cfg.rnn_hidden, num_layers=cfg.rnn_layers, bidirectional=True)
        self.fc = nn.Linear(2 * cfg.rnn_hidden, cfg.n_classes)

    def _use_persistent(self, x: torch.Tensor) -> bool:
        if not (self.cfg.persistent_rnn and x.is_cuda and x.dtype == torch.float32):
            return False
        from ..ops import persistent_gru

        return persistent_gru.supported(x.shape[0], x.shape[1], self.cfg.rnn_hidden, 2, x.device)

    def out_frames(self, n_frames: int) -> int:
        return (n_frames + 2 * 5 - 11) // 2 + 1

    def forward(self, spect: torch.Tensor) -> torch.Tensor:
        """spect: [batch, n_freq, n_frames] log-spectrogram. Returns log-probabilities
        [frames', batch, classes]."""
        x = self.conv(spect.unsqueeze(1))                 # [B, C, F', T']
        b, c, f, t = x.shape
        x = x.view(b, c * f, t).permute(2, 0, 1).contiguous()   # [T', B, C*F']
        if self._use_persistent(x):
            from ..ops import persistent_gru

            x = persistent_gru.gru_forward(self.rnn, x)
        else:
            x, _ = self.rnn(x)
        return F.log_softmax(self.fc(x), dim=-1)

    def loss(self, spect: torch.Tensor, labels: torch.Tensor, label_lengths: torch.Tensor) -> torch.Tensor:
        logp = self.forward(spect)
        t, b, _ = logp.shape
        in_len = torch.full((b,), t, dtype=torch.long, device=logp.device)
        return F.ctc_loss(logp, labels, in_len, label_lengths, blank=0, reduction="mean", zero_infinity=True)


def synthetic_batch(cfg: DS2Config, batch: int, device, generator=None, pin: bool = False):
    """N(0,1) spectrograms and random labels in [1, n_classes-1], `label_len` per utterance."""
    spect = torch.randn(batch, cfg.n_freq, cfg.n_frames, generator=generator)
    labels = torch.randint(1, cfg.n_classes, (batch, cfg.label_len), generator=generator)
    lens = torch.full((batch,), cfg.label_len, dtype=torch.long)
    if pin:
        return spect.pin_memory(), labels.pin_memory(), lens.pin_memory()
    return spect.to(device), labels.to(device), lens.to(device)
