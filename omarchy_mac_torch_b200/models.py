"""Workload definitions for the benchmark configurations and the parity tests (random data is enough: timing does not
depend on pixels). Architecture facts only; parameter registration order matches the reference's model classes
(omarchy_mac_torch/models.py) where one exists, so that seeding `torch.manual_seed(0)` before construction yields the
same initial weights and the recorded loss curves can be compared.

  PlainCNN, SeparableCNN, ResNet18, MobileNetV3Small   the reference's acceptance models (1x28x28 / 64x64 / 96x96 inputs)
  PlainCNN3        the three-block benchmark CNN: three conv3x3-BN-ReLU-MaxPool blocks (3->32->64->128) on 3x32x32, Linear 10
  MobileNetV3SE    the MobileNetV3 benchmark: MobileNetV3-Small with squeeze-excite, 3x3/5x5 depthwise, 224x224
  ResNet50         the data-parallel benchmark: Bottleneck [3,4,6,3], 25.6 M parameters
"""

import torch
from torch import nn


def _cbr(ci, co, k=3, groups=1, bias=False):
    return [nn.Conv2d(ci, co, k, padding=k // 2, groups=groups, bias=bias), nn.BatchNorm2d(co), nn.ReLU()]


class PlainCNN(nn.Module):
    """[conv-BN-ReLU x2, max pool] x3 then two fully connected layers, on [N,1,28,28]."""

    def __init__(self, widths=(16, 32, 64), hidden=(256, 128), num_classes=10):
        super().__init__()
        feats, ci, size = [], 1, 28
        for w in widths:
            feats += _cbr(ci, w) + _cbr(w, w) + [nn.MaxPool2d(2, 2)]
            ci, size = w, size // 2
        self.features = nn.Sequential(*feats)
        fc, n = [], ci * size * size
        for h in hidden:
            fc += [nn.Linear(n, h), nn.ReLU()]
            n = h
        self.classifier = nn.Sequential(*fc, nn.Linear(n, num_classes))

    def forward(self, x):
        return self.classifier(self.features(x).flatten(1))


class SeparableCNN(nn.Module):
    """Depthwise-separable convolutions and global average pooling, on [N,1,28,28]."""

    def __init__(self, stem=16, widths=(32, 32, 48, 64), pool_after=(0, 2), num_classes=10):
        super().__init__()
        feats, c = _cbr(1, stem), stem
        for i, w in enumerate(widths):
            feats += _cbr(c, c, 3, groups=c) + _cbr(c, w, 1)
            if i in pool_after:
                feats.append(nn.MaxPool2d(2, 2))
            c = w
        feats.append(nn.AdaptiveAvgPool2d(1))
        self.features = nn.Sequential(*feats)
        self.classifier = nn.Linear(c, num_classes)

    def forward(self, x):
        return self.classifier(self.features(x).flatten(1))


class PlainCNN3(nn.Module):
    """Three conv3x3-BN-ReLU-MaxPool blocks on 3x32x32 (batch 128 in the benchmark). The feature stack is one nn.Sequential so the auto-fuse hook can take it; the head is outside."""

    def __init__(self, widths=(32, 64, 128), num_classes=10, bias=True):
        super().__init__()
        feats, ci = [], 3
        for w in widths:
            feats += _cbr(ci, w, bias=bias) + [nn.MaxPool2d(2)]
            ci = w
        self.features = nn.Sequential(*feats)
        self.head = nn.Linear(ci * 4 * 4, num_classes)

    def forward(self, x):
        return self.head(self.features(x).flatten(1))


class _Basic(nn.Module):
    def __init__(self, ci, co, stride):
        super().__init__()
        self.c1 = nn.Conv2d(ci, co, 3, stride, 1, bias=False)
        self.b1 = nn.BatchNorm2d(co)
        self.c2 = nn.Conv2d(co, co, 3, 1, 1, bias=False)
        self.b2 = nn.BatchNorm2d(co)
        self.down = (nn.Sequential(nn.Conv2d(ci, co, 1, stride, bias=False), nn.BatchNorm2d(co)) if stride != 1 or ci != co else nn.Identity())

    def forward(self, x):
        y = torch.relu(self.b1(self.c1(x)))
        return torch.relu(self.b2(self.c2(y)) + self.down(x))


class ResNet18(nn.Module):
    def __init__(self, num_classes=10, width=64):
        super().__init__()
        w = [width, width * 2, width * 4, width * 8]
        self.stem = nn.Sequential(nn.Conv2d(3, w[0], 7, 2, 3, bias=False), nn.BatchNorm2d(w[0]), nn.ReLU(), nn.MaxPool2d(3, 2, 1))
        blocks, ci = [], w[0]
        for i, co in enumerate(w):
            blocks += [_Basic(ci, co, 1 if i == 0 else 2), _Basic(co, co, 1)]
            ci = co
        self.layers = nn.Sequential(*blocks)
        self.head = nn.Linear(ci, num_classes)

    def forward(self, x):
        return self.head(torch.flatten(nn.functional.adaptive_avg_pool2d(self.layers(self.stem(x)), 1), 1))


class _Bottleneck(nn.Module):
    def __init__(self, ci, mid, stride):
        super().__init__()
        co = mid * 4
        self.c1 = nn.Conv2d(ci, mid, 1, bias=False)
        self.b1 = nn.BatchNorm2d(mid)
        self.c2 = nn.Conv2d(mid, mid, 3, stride, 1, bias=False)
        self.b2 = nn.BatchNorm2d(mid)
        self.c3 = nn.Conv2d(mid, co, 1, bias=False)
        self.b3 = nn.BatchNorm2d(co)
        self.down = (nn.Sequential(nn.Conv2d(ci, co, 1, stride, bias=False), nn.BatchNorm2d(co)) if stride != 1 or ci != co else nn.Identity())

    def forward(self, x):
        y = torch.relu(self.b1(self.c1(x)))
        y = torch.relu(self.b2(self.c2(y)))
        return torch.relu(self.b3(self.c3(y)) + self.down(x))


class ResNet50(nn.Module):
    """Bottleneck [3,4,6,3], widths 256/512/1024/2048, 25.6 M parameters at 1000 classes."""

    def __init__(self, num_classes=1000, layers=(3, 4, 6, 3)):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, 64, 7, 2, 3, bias=False), nn.BatchNorm2d(64), nn.ReLU(), nn.MaxPool2d(3, 2, 1))
        blocks, ci = [], 64
        for i, (n, mid) in enumerate(zip(layers, (64, 128, 256, 512))):
            for j in range(n):
                blocks.append(_Bottleneck(ci, mid, (1 if i == 0 else 2) if j == 0 else 1))
                ci = mid * 4
        self.layers = nn.Sequential(*blocks)
        self.head = nn.Linear(ci, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")

    def forward(self, x):
        return self.head(torch.flatten(nn.functional.adaptive_avg_pool2d(self.layers(self.stem(x)), 1), 1))

    def compile_regions(self):
        """The parts compile.compile_regions compiles separately: the stem, then the blocks in three groups whose parameters
        fill the gradient buckets evenly in backward order (the last stage alone holds 60 % of the parameters)."""
        n = len(self.layers)
        if n < 4:
            return [(self, "stem"), (self.layers, (0, n))]
        cuts = [0, n - n // 2 - 2, n - n // 4 - 1, n] if n >= 12 else [0, n // 2, n - 1, n]
        return [(self, "stem")] + [(self.layers, (a, b)) for a, b in zip(cuts, cuts[1:]) if b > a]


class _InvRes(nn.Module):
    def __init__(self, ci, co, expand, stride, k=3):
        super().__init__()
        h = ci * expand
        self.use_res = stride == 1 and ci == co
        self.block = nn.Sequential(
            nn.Conv2d(ci, h, 1, bias=False), nn.BatchNorm2d(h), nn.Hardswish(),
            nn.Conv2d(h, h, k, stride, k // 2, groups=h, bias=False), nn.BatchNorm2d(h), nn.Hardswish(),
            nn.Conv2d(h, co, 1, bias=False), nn.BatchNorm2d(co))

    def forward(self, x):
        y = self.block(x)
        return x + y if self.use_res else y


class MobileNetV3Small(nn.Module):
    """The reference's MobileNetV3-Small-style acceptance model (7 blocks, no squeeze-excite, 3x3 depthwise, 96x96)."""

    def __init__(self, num_classes=10):
        super().__init__()
        cfg = [(16, 16, 1, 2), (16, 24, 4, 2), (24, 24, 3, 1), (24, 40, 4, 2), (40, 40, 6, 1), (40, 48, 3, 1), (48, 96, 6, 2)]
        self.stem = nn.Sequential(nn.Conv2d(3, 16, 3, 2, 1, bias=False), nn.BatchNorm2d(16), nn.Hardswish())
        self.blocks = nn.Sequential(*[_InvRes(ci, co, e, s) for ci, co, e, s in cfg])
        self.head = nn.Sequential(nn.Conv2d(96, 576, 1, bias=False), nn.BatchNorm2d(576), nn.Hardswish(), nn.AdaptiveAvgPool2d(1),
                                  nn.Flatten(), nn.Linear(576, 256), nn.Hardswish(), nn.Dropout(0.2), nn.Linear(256, num_classes))

    def forward(self, x):
        return self.head(self.blocks(self.stem(x)))


class _SE(nn.Module):
    def __init__(self, c, reduction=4):
        super().__init__()
        r = max(8, c // reduction)
        self.fc1, self.fc2 = nn.Conv2d(c, r, 1), nn.Conv2d(r, c, 1)

    def forward(self, x):
        s = nn.functional.adaptive_avg_pool2d(x, 1)
        return x * nn.functional.hardsigmoid(self.fc2(torch.relu(self.fc1(s))))


class _InvResSE(nn.Module):
    def __init__(self, ci, k, exp, co, se, hs, stride):
        super().__init__()
        act = nn.Hardswish if hs else nn.ReLU
        self.use_res = stride == 1 and ci == co
        layers = []
        if exp != ci:
            layers += [nn.Conv2d(ci, exp, 1, bias=False), nn.BatchNorm2d(exp), act()]
        layers += [nn.Conv2d(exp, exp, k, stride, k // 2, groups=exp, bias=False), nn.BatchNorm2d(exp), act()]
        if se:
            layers.append(_SE(exp))
        layers += [nn.Conv2d(exp, co, 1, bias=False), nn.BatchNorm2d(co)]
        self.block = nn.Sequential(*layers)

    def forward(self, x):
        y = self.block(x)
        return x + y if self.use_res else y


class MobileNetV3SE(nn.Module):
    """MobileNetV3-Small with squeeze-excite on 224x224: 3x3 s2 stem (16, hardswish), 11 inverted-residual blocks (kernel, expansion, out, SE,
    hardswish, stride) with 3x3/5x5 depthwise and squeeze-excite r=4, 1x1 conv to 576, avgpool, Linear 1024, Linear 1000."""

    CFG = [(3, 16, 16, True, False, 2), (3, 72, 24, False, False, 2), (3, 88, 24, False, False, 1), (5, 96, 40, True, True, 2),
           (5, 240, 40, True, True, 1), (5, 240, 40, True, True, 1), (5, 120, 48, True, True, 1), (5, 144, 48, True, True, 1),
           (5, 288, 96, True, True, 2), (5, 576, 96, True, True, 1), (5, 576, 96, True, True, 1)]

    def __init__(self, num_classes=1000):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, 16, 3, 2, 1, bias=False), nn.BatchNorm2d(16), nn.Hardswish())
        blocks, ci = [], 16
        for k, exp, co, se, hs, s in self.CFG:
            blocks.append(_InvResSE(ci, k, exp, co, se, hs, s))
            ci = co
        self.blocks = nn.Sequential(*blocks)
        self.last = nn.Sequential(nn.Conv2d(ci, 576, 1, bias=False), nn.BatchNorm2d(576), nn.Hardswish())
        self.head = nn.Sequential(nn.Linear(576, 1024), nn.Hardswish(), nn.Linear(1024, num_classes))

    def forward(self, x):
        x = self.last(self.blocks(self.stem(x)))
        return self.head(torch.flatten(nn.functional.adaptive_avg_pool2d(x, 1), 1))


def kaiming_normal_convs(model):
    """Kaiming-normal initialisation of every convolution (the ResNet-18 benchmark configuration asks for it)."""
    for m in model.modules():
        if isinstance(m, nn.Conv2d):
            nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
    return model
