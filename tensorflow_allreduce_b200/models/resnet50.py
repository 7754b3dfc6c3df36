"""ResNet-50 (v1.5 bottleneck layout) for the bf16 data-parallel configuration with many small
gradient tensors (~161 parameter tensors, 25.6 M parameters), which exercises bucketing. The
reference's tree carries the slim definition (tensorflow/contrib/slim/python/slim/nets/resnet_v1.py:256-268)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, cin, width, stride):
        super().__init__()
        cout = width * self.expansion
        self.c1 = nn.Conv2d(cin, width, 1, bias=False)
        self.b1 = nn.BatchNorm2d(width)
        self.c2 = nn.Conv2d(width, width, 3, stride=stride, padding=1, bias=False)
        self.b2 = nn.BatchNorm2d(width)
        self.c3 = nn.Conv2d(width, cout, 1, bias=False)
        self.b3 = nn.BatchNorm2d(cout)
        self.down = None
        if stride != 1 or cin != cout:
            self.down = nn.Sequential(nn.Conv2d(cin, cout, 1, stride=stride, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x):
        idt = x if self.down is None else self.down(x)
        x = F.relu(self.b1(self.c1(x)), inplace=True)
        x = F.relu(self.b2(self.c2(x)), inplace=True)
        return F.relu(self.b3(self.c3(x)) + idt, inplace=True)


class ResNet50(nn.Module):
    def __init__(self, n_classes: int = 1000):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, 64, 7, stride=2, padding=3, bias=False), nn.BatchNorm2d(64), nn.ReLU(inplace=True),
                                  nn.MaxPool2d(3, stride=2, padding=1))
        layers, cin = [], 64
        for width, n, stride in ((64, 3, 1), (128, 4, 2), (256, 6, 2), (512, 3, 2)):
            for i in range(n):
                layers.append(Bottleneck(cin, width, stride if i == 0 else 1))
                cin = width * Bottleneck.expansion
        self.layers = nn.Sequential(*layers)
        self.fc = nn.Linear(cin, n_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def forward(self, x):
        x = self.layers(self.stem(x))
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))

    def loss(self, images, labels):
        return F.cross_entropy(self.forward(images).float(), labels)


def synthetic_batch(batch: int, device, dtype=torch.bfloat16, generator=None, pin: bool = False, n_classes: int = 1000):
    x = torch.randn(batch, 3, 224, 224, generator=generator).to(dtype)
    y = torch.randint(0, n_classes, (batch,), generator=generator)
    if pin:
        return x.pin_memory(), y.pin_memory()
    return x.to(device).contiguous(memory_format=torch.channels_last), y.to(device)
