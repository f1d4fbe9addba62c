"""Vision benchmark models: VGG-16 (configuration D, 138 M parameters) and ResNet-50
(25.6 M parameters), written out here so the benchmarks do not depend on torchvision.
Random initialisation only (there are no checkpoints to load)."""
from __future__ import annotations

import torch
import torch.nn as nn

_VGG16_CFG = [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"]


class VGG16(nn.Module):
    """13 convolutions + 3 fully connected layers, ReLU, max-pool, dropout in the classifier.

    `fused_ops=True` builds every conv+ReLU pair as one `ConvBiasReLU` module (bias add, ReLU and the
    bias-gradient reduction in this package's own kernels) and folds every pooling layer into the
    block before it (`ConvBiasReLUPool`: no index tensor, one pass each way); parameter names change
    from `features.<2k>.weight` to the fused module's index, values and shapes do not.  The classifier's
    layers become `ShadowLinear`, which is `nn.Linear` unless the optimizer maintains bf16 copies of the
    weights (`FlatSGD(bf16_shadow=True)`)."""

    def __init__(self, num_classes: int = 1000, dropout: float = 0.5, fused_ops: bool = False):
        super().__init__()
        layers, c_in = [], 3
        if fused_ops:
            from ..ops.fused_conv import ConvBiasReLU, ConvBiasReLUPool
        for i, v in enumerate(_VGG16_CFG):
            if v == "M":
                if not fused_ops:
                    layers.append(nn.MaxPool2d(2, 2))  # (fused: folded into the convolution block before it)
            elif fused_ops:
                pooled = i + 1 < len(_VGG16_CFG) and _VGG16_CFG[i + 1] == "M"
                layers.append((ConvBiasReLUPool if pooled else ConvBiasReLU)(c_in, v, 3, padding=1))
                c_in = v
            else:
                layers += [nn.Conv2d(c_in, v, 3, padding=1), nn.ReLU(inplace=True)]
                c_in = v
        self.features = nn.Sequential(*layers)
        self.avgpool = nn.AdaptiveAvgPool2d((7, 7))
        if fused_ops:
            from ..ops.fused_linear import ShadowLinear as Linear  # nn.Linear unless the optimizer keeps bf16 weights
        else:
            Linear = nn.Linear
        self.classifier = nn.Sequential(
            Linear(512 * 7 * 7, 4096), nn.ReLU(inplace=True), nn.Dropout(dropout),
            Linear(4096, 4096), nn.ReLU(inplace=True), nn.Dropout(dropout),
            Linear(4096, num_classes),
        )
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
                nn.init.zeros_(m.bias)
            elif isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0, 0.01)
                nn.init.zeros_(m.bias)

    def forward(self, x):
        x = self.features(x)
        x = self.avgpool(x)
        return self.classifier(torch.flatten(x, 1))


class _Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, c_in, width, stride=1, downsample=None):
        super().__init__()
        self.conv1 = nn.Conv2d(c_in, width, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(width)
        self.conv2 = nn.Conv2d(width, width, 3, stride=stride, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(width)
        self.conv3 = nn.Conv2d(width, width * 4, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(width * 4)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else self.downsample(x)
        out = self.relu(self.bn1(self.conv1(x)))
        out = self.relu(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        return self.relu(out + idt)


class ResNet50(nn.Module):
    def __init__(self, num_classes: int = 1000):
        super().__init__()
        self.conv1 = nn.Conv2d(3, 64, 7, stride=2, padding=3, bias=False)
        self.bn1 = nn.BatchNorm2d(64)
        self.relu = nn.ReLU(inplace=True)
        self.maxpool = nn.MaxPool2d(3, stride=2, padding=1)
        self._c = 64
        self.layer1 = self._stage(64, 3, 1)
        self.layer2 = self._stage(128, 4, 2)
        self.layer3 = self._stage(256, 6, 2)
        self.layer4 = self._stage(512, 3, 2)
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.fc = nn.Linear(2048, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)

    def _stage(self, width, blocks, stride):
        down = None
        if stride != 1 or self._c != width * 4:
            down = nn.Sequential(nn.Conv2d(self._c, width * 4, 1, stride=stride, bias=False),
                                 nn.BatchNorm2d(width * 4))
        layers = [_Bottleneck(self._c, width, stride, down)]
        self._c = width * 4
        layers += [_Bottleneck(self._c, width) for _ in range(blocks - 1)]
        return nn.Sequential(*layers)

    def forward(self, x):
        x = self.maxpool(self.relu(self.bn1(self.conv1(x))))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(torch.flatten(self.avgpool(x), 1))


class MLP(nn.Module):
    """Small model for tests and smoke runs."""

    def __init__(self, d_in=64, d_hidden=128, d_out=10, depth=3):
        super().__init__()
        dims = [d_in] + [d_hidden] * (depth - 1) + [d_out]
        layers = []
        for i in range(depth):
            layers.append(nn.Linear(dims[i], dims[i + 1]))
            if i < depth - 1:
                layers.append(nn.ReLU())
        self.net = nn.Sequential(*layers)

    def forward(self, x):
        return self.net(x)
