"""ResNet-50 (bottleneck residual network, v1.5: the stride sits on the 3x3 convolution), the model of
the PowerSGD benchmark. Self-contained so that the benchmark does not depend on torchvision.

Every convolution weight [out, in, kh, kw] is a PowerSGD matrix of shape [out, in * kh * kw]; batch
norm parameters and biases are 1-D and are averaged exactly.
"""
from __future__ import annotations

from typing import List, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, cin: int, width: int, stride: int):
        super().__init__()
        cout = width * self.expansion
        self.conv1 = nn.Conv2d(cin, width, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.conv2 = nn.Conv2d(width, width, 3, stride=stride, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(width)
        self.conv3 = nn.Conv2d(width, cout, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(cout)
        nn.init.zeros_(self.bn3.weight)  # each block starts as the identity
        self.down = None
        if stride != 1 or cin != cout:
            self.down = nn.Sequential(nn.Conv2d(cin, cout, 1, stride=stride, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        idt = x if self.down is None else self.down(x)
        y = F.relu(self.bn1(self.conv1(x)), inplace=True)
        y = F.relu(self.bn2(self.conv2(y)), inplace=True)
        y = self.bn3(self.conv3(y))
        return F.relu(y + idt, inplace=True)


class ResNet(nn.Module):
    def __init__(self, layers: Sequence[int] = (3, 4, 6, 3), num_classes: int = 1000, width: int = 64):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, width, 7, stride=2, padding=3, bias=False), nn.BatchNorm2d(width),
                                  nn.ReLU(inplace=True), nn.MaxPool2d(3, stride=2, padding=1))
        blocks: List[nn.Module] = []
        cin = width
        for stage, n in enumerate(layers):
            w = width * (2 ** stage)
            for i in range(n):
                blocks.append(Bottleneck(cin, w, stride=2 if (i == 0 and stage > 0) else 1))
                cin = w * Bottleneck.expansion
        self.blocks = nn.Sequential(*blocks)
        self.fc = nn.Linear(cin, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def forward(self, x: torch.Tensor, targets: torch.Tensor | None = None):
        x = self.blocks(self.stem(x))
        logits = self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))
        if targets is None:
            return logits
        return F.cross_entropy(logits.float(), targets)

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())


def resnet50(num_classes: int = 1000) -> ResNet:
    return ResNet((3, 4, 6, 3), num_classes)


def resnet_tiny(num_classes: int = 10) -> ResNet:
    """Two stages of one bottleneck each at width 16: for tests."""
    return ResNet((1, 1), num_classes, width=16)
