"""ResNet-50 v1.5 (bottleneck blocks [3, 4, 6, 3], stride 2 on the 3x3
convolution of each down-sampling block): 25.6 M parameters in 161 tensors,
the model of the reference's synthetic benchmark
(examples/pytorch/pytorch_synthetic_benchmark.py:48 uses torchvision's
resnet50, which is the same v1.5 network).
"""
import torch
import torch.nn as nn

from horovod_b200.ops.batch_norm import BatchNormAct2d
from horovod_b200.ops.pooling import MaxPool3x3s2


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes, planes, stride=1, downsample=None):
        super().__init__()
        # Each batch norm carries its ReLU (and, for the last one, the residual
        # add): one fused kernel pair on the GPU, plain PyTorch ops elsewhere.
        self.conv1 = nn.Conv2d(inplanes, planes, 1, bias=False)
        self.bn1 = BatchNormAct2d(planes, relu=True)
        self.conv2 = nn.Conv2d(planes, planes, 3, stride=stride, padding=1, bias=False)
        self.bn2 = BatchNormAct2d(planes, relu=True)
        self.conv3 = nn.Conv2d(planes, planes * 4, 1, bias=False)
        self.bn3 = BatchNormAct2d(planes * 4, relu=True)
        self.downsample = downsample

    def forward(self, x):
        identity = x
        out = self.bn1(self.conv1(x))
        out = self.bn2(self.conv2(out))
        if self.downsample is not None:
            identity = self.downsample(x)
        return self.bn3(self.conv3(out), residual=identity)


class ResNet(nn.Module):
    def __init__(self, layers=(3, 4, 6, 3), num_classes=1000, width=64):
        super().__init__()
        self.inplanes = width
        self.conv1 = nn.Conv2d(3, width, 7, stride=2, padding=3, bias=False)
        self.bn1 = BatchNormAct2d(width, relu=True)
        self.maxpool = MaxPool3x3s2()  # 3x3, stride 2, padding 1
        self.layer1 = self._make_layer(width, layers[0])
        self.layer2 = self._make_layer(width * 2, layers[1], stride=2)
        self.layer3 = self._make_layer(width * 4, layers[2], stride=2)
        self.layer4 = self._make_layer(width * 8, layers[3], stride=2)
        self.avgpool = nn.AdaptiveAvgPool2d((1, 1))
        self.fc = nn.Linear(width * 8 * 4, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)
        # Zero the last BN of each block so that blocks start as identities.
        for m in self.modules():
            if isinstance(m, Bottleneck):
                nn.init.zeros_(m.bn3.weight)

    def _make_layer(self, planes, blocks, stride=1):
        downsample = None
        if stride != 1 or self.inplanes != planes * 4:
            downsample = nn.Sequential(
                nn.Conv2d(self.inplanes, planes * 4, 1, stride=stride, bias=False),
                BatchNormAct2d(planes * 4, relu=False))
        layers = [Bottleneck(self.inplanes, planes, stride, downsample)]
        self.inplanes = planes * 4
        for _ in range(1, blocks):
            layers.append(Bottleneck(self.inplanes, planes))
        return nn.Sequential(*layers)

    def forward(self, x):
        x = self.maxpool(self.bn1(self.conv1(x)))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        x = torch.flatten(self.avgpool(x), 1)
        return self.fc(x)


def resnet50(num_classes=1000):
    return ResNet((3, 4, 6, 3), num_classes)


def resnet_tiny(num_classes=10):
    """A two-stage miniature with the same block structure, for smoke tests."""
    return ResNet((1, 1, 1, 1), num_classes, width=8)
