"""``paddle.vision.models`` (python/paddle/vision/models/): classification backbones built from this framework's
layers.  ``pretrained=True`` needs downloaded weights, which this offline build cannot fetch: it raises."""
from __future__ import annotations

from .. import nn
from ..tensor.manipulation import concat, flatten

__all__ = ["LeNet", "AlexNet", "alexnet", "VGG", "vgg11", "vgg13", "vgg16", "vgg19", "ResNet", "resnet18", "resnet34",
           "resnet50", "resnet101", "resnet152", "resnext50_32x4d", "resnext50_64x4d", "resnext101_32x4d",
           "resnext101_64x4d", "resnext152_32x4d", "resnext152_64x4d", "wide_resnet50_2", "wide_resnet101_2",
           "MobileNetV1", "mobilenet_v1", "MobileNetV2", "mobilenet_v2", "SqueezeNet", "squeezenet1_0", "squeezenet1_1",
           "DenseNet", "densenet121", "densenet161", "densenet169", "densenet201", "densenet264"]


def _no_pretrained(flag):
    if flag:
        raise RuntimeError("pretrained weights have to be downloaded; load a local .pdparams with set_state_dict instead")


class LeNet(nn.Layer):
    def __init__(self, num_classes=10):
        super().__init__()
        self.num_classes = num_classes
        self.features = nn.Sequential(nn.Conv2D(1, 6, 3, stride=1, padding=1), nn.ReLU(), nn.MaxPool2D(2, 2),
                                      nn.Conv2D(6, 16, 5, stride=1, padding=0), nn.ReLU(), nn.MaxPool2D(2, 2))
        if num_classes > 0:
            self.fc = nn.Sequential(nn.Linear(400, 120), nn.Linear(120, 84), nn.Linear(84, num_classes))

    def forward(self, x):
        x = self.features(x)
        if self.num_classes > 0:
            x = self.fc(flatten(x, 1))
        return x


class AlexNet(nn.Layer):
    def __init__(self, num_classes=1000):
        super().__init__()
        self.features = nn.Sequential(
            nn.Conv2D(3, 64, 11, 4, 2), nn.ReLU(), nn.MaxPool2D(3, 2), nn.Conv2D(64, 192, 5, 1, 2), nn.ReLU(),
            nn.MaxPool2D(3, 2), nn.Conv2D(192, 384, 3, 1, 1), nn.ReLU(), nn.Conv2D(384, 256, 3, 1, 1), nn.ReLU(),
            nn.Conv2D(256, 256, 3, 1, 1), nn.ReLU(), nn.MaxPool2D(3, 2))
        self.pool = nn.AdaptiveAvgPool2D((6, 6))
        self.classifier = nn.Sequential(nn.Dropout(0.5), nn.Linear(256 * 36, 4096), nn.ReLU(), nn.Dropout(0.5),
                                        nn.Linear(4096, 4096), nn.ReLU(), nn.Linear(4096, num_classes))

    def forward(self, x):
        return self.classifier(flatten(self.pool(self.features(x)), 1))


def alexnet(pretrained=False, **kw):
    _no_pretrained(pretrained)
    return AlexNet(**kw)


_VGG = {11: [64, "M", 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
        13: [64, 64, "M", 128, 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
        16: [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"],
        19: [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"]}


class VGG(nn.Layer):
    def __init__(self, features, num_classes=1000, with_pool=True):
        super().__init__()
        self.features, self.num_classes, self.with_pool = features, num_classes, with_pool
        if with_pool:
            self.avgpool = nn.AdaptiveAvgPool2D((7, 7))
        if num_classes > 0:
            self.classifier = nn.Sequential(nn.Linear(512 * 49, 4096), nn.ReLU(), nn.Dropout(), nn.Linear(4096, 4096),
                                            nn.ReLU(), nn.Dropout(), nn.Linear(4096, num_classes))

    def forward(self, x):
        x = self.features(x)
        if self.with_pool:
            x = self.avgpool(x)
        if self.num_classes > 0:
            x = self.classifier(flatten(x, 1))
        return x


def _vgg(depth, batch_norm=False, pretrained=False, **kw):
    _no_pretrained(pretrained)
    layers, c = [], 3
    for v in _VGG[depth]:
        if v == "M":
            layers.append(nn.MaxPool2D(2, 2))
        else:
            layers += [nn.Conv2D(c, v, 3, padding=1)] + ([nn.BatchNorm2D(v)] if batch_norm else []) + [nn.ReLU()]
            c = v
    return VGG(nn.Sequential(*layers), **kw)


def vgg11(pretrained=False, batch_norm=False, **kw):
    return _vgg(11, batch_norm, pretrained, **kw)


def vgg13(pretrained=False, batch_norm=False, **kw):
    return _vgg(13, batch_norm, pretrained, **kw)


def vgg16(pretrained=False, batch_norm=False, **kw):
    return _vgg(16, batch_norm, pretrained, **kw)


def vgg19(pretrained=False, batch_norm=False, **kw):
    return _vgg(19, batch_norm, pretrained, **kw)


class BasicBlock(nn.Layer):
    expansion = 1

    def __init__(self, inplanes, planes, stride=1, downsample=None, groups=1, base_width=64, dilation=1, norm_layer=None):
        super().__init__()
        norm_layer = norm_layer or nn.BatchNorm2D
        self.conv1 = nn.Conv2D(inplanes, planes, 3, padding=1, stride=stride, bias_attr=False)
        self.bn1 = norm_layer(planes)
        self.relu = nn.ReLU()
        self.conv2 = nn.Conv2D(planes, planes, 3, padding=1, bias_attr=False)
        self.bn2 = norm_layer(planes)
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else self.downsample(x)
        out = self.bn2(self.conv2(self.relu(self.bn1(self.conv1(x)))))
        return self.relu(out + idt)


class BottleneckBlock(nn.Layer):
    expansion = 4

    def __init__(self, inplanes, planes, stride=1, downsample=None, groups=1, base_width=64, dilation=1, norm_layer=None):
        super().__init__()
        norm_layer = norm_layer or nn.BatchNorm2D
        width = int(planes * (base_width / 64.0)) * groups
        self.conv1 = nn.Conv2D(inplanes, width, 1, bias_attr=False)
        self.bn1 = norm_layer(width)
        self.conv2 = nn.Conv2D(width, width, 3, padding=dilation, stride=stride, groups=groups, dilation=dilation, bias_attr=False)
        self.bn2 = norm_layer(width)
        self.conv3 = nn.Conv2D(width, planes * 4, 1, bias_attr=False)
        self.bn3 = norm_layer(planes * 4)
        self.relu = nn.ReLU()
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else self.downsample(x)
        out = self.relu(self.bn1(self.conv1(x)))
        out = self.relu(self.bn2(self.conv2(out)))
        return self.relu(self.bn3(self.conv3(out)) + idt)


class ResNet(nn.Layer):
    def __init__(self, block, depth=50, width=64, num_classes=1000, with_pool=True, groups=1):
        super().__init__()
        cfg = {18: [2, 2, 2, 2], 34: [3, 4, 6, 3], 50: [3, 4, 6, 3], 101: [3, 4, 23, 3], 152: [3, 8, 36, 3]}[depth]
        self.groups, self.base_width, self.num_classes, self.with_pool = groups, width, num_classes, with_pool
        self.inplanes = 64
        self.conv1 = nn.Conv2D(3, 64, 7, stride=2, padding=3, bias_attr=False)
        self.bn1 = nn.BatchNorm2D(64)
        self.relu = nn.ReLU()
        self.maxpool = nn.MaxPool2D(3, 2, 1)
        self.layer1 = self._make(block, 64, cfg[0])
        self.layer2 = self._make(block, 128, cfg[1], 2)
        self.layer3 = self._make(block, 256, cfg[2], 2)
        self.layer4 = self._make(block, 512, cfg[3], 2)
        if with_pool:
            self.avgpool = nn.AdaptiveAvgPool2D((1, 1))
        if num_classes > 0:
            self.fc = nn.Linear(512 * block.expansion, num_classes)

    def _make(self, block, planes, n, stride=1):
        down = None
        if stride != 1 or self.inplanes != planes * block.expansion:
            down = nn.Sequential(nn.Conv2D(self.inplanes, planes * block.expansion, 1, stride=stride, bias_attr=False),
                                 nn.BatchNorm2D(planes * block.expansion))
        layers = [block(self.inplanes, planes, stride, down, self.groups, self.base_width)]
        self.inplanes = planes * block.expansion
        layers += [block(self.inplanes, planes, groups=self.groups, base_width=self.base_width) for _ in range(1, n)]
        return nn.Sequential(*layers)

    def forward(self, x):
        x = self.maxpool(self.relu(self.bn1(self.conv1(x))))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        if self.with_pool:
            x = self.avgpool(x)
        if self.num_classes > 0:
            x = self.fc(flatten(x, 1))
        return x


def _resnet(block, depth, pretrained=False, **kw):
    _no_pretrained(pretrained)
    return ResNet(block, depth, **kw)


def resnet18(pretrained=False, **kw):
    return _resnet(BasicBlock, 18, pretrained, **kw)


def resnet34(pretrained=False, **kw):
    return _resnet(BasicBlock, 34, pretrained, **kw)


def resnet50(pretrained=False, **kw):
    return _resnet(BottleneckBlock, 50, pretrained, **kw)


def resnet101(pretrained=False, **kw):
    return _resnet(BottleneckBlock, 101, pretrained, **kw)


def resnet152(pretrained=False, **kw):
    return _resnet(BottleneckBlock, 152, pretrained, **kw)


def resnext50_32x4d(pretrained=False, **kw):
    return _resnet(BottleneckBlock, 50, pretrained, groups=32, width=4, **kw)


def resnext50_64x4d(pretrained=False, **kw):
    return _resnet(BottleneckBlock, 50, pretrained, groups=64, width=4, **kw)


def resnext101_32x4d(pretrained=False, **kw):
    return _resnet(BottleneckBlock, 101, pretrained, groups=32, width=4, **kw)


def resnext101_64x4d(pretrained=False, **kw):
    return _resnet(BottleneckBlock, 101, pretrained, groups=64, width=4, **kw)


def resnext152_32x4d(pretrained=False, **kw):
    return _resnet(BottleneckBlock, 152, pretrained, groups=32, width=4, **kw)


def resnext152_64x4d(pretrained=False, **kw):
    return _resnet(BottleneckBlock, 152, pretrained, groups=64, width=4, **kw)


def wide_resnet50_2(pretrained=False, **kw):
    return _resnet(BottleneckBlock, 50, pretrained, width=128, **kw)


def wide_resnet101_2(pretrained=False, **kw):
    return _resnet(BottleneckBlock, 101, pretrained, width=128, **kw)


def _cbr(cin, cout, k, s=1, p=0, g=1, act=nn.ReLU):
    return nn.Sequential(nn.Conv2D(cin, cout, k, s, p, groups=g, bias_attr=False), nn.BatchNorm2D(cout), act())


class MobileNetV1(nn.Layer):
    def __init__(self, scale=1.0, num_classes=1000, with_pool=True):
        super().__init__()
        c = lambda v: int(v * scale)   # noqa: E731
        cfg = [(32, 64, 1), (64, 128, 2), (128, 128, 1), (128, 256, 2), (256, 256, 1), (256, 512, 2)] + \
              [(512, 512, 1)] * 5 + [(512, 1024, 2), (1024, 1024, 1)]
        layers = [_cbr(3, c(32), 3, 2, 1)]
        for cin, cout, s in cfg:
            layers += [_cbr(c(cin), c(cin), 3, s, 1, g=c(cin)), _cbr(c(cin), c(cout), 1)]
        self.features = nn.Sequential(*layers)
        self.num_classes, self.with_pool = num_classes, with_pool
        if with_pool:
            self.pool2d_avg = nn.AdaptiveAvgPool2D(1)
        if num_classes > 0:
            self.fc = nn.Linear(c(1024), num_classes)

    def forward(self, x):
        x = self.features(x)
        if self.with_pool:
            x = self.pool2d_avg(x)
        if self.num_classes > 0:
            x = self.fc(flatten(x, 1))
        return x


def mobilenet_v1(pretrained=False, scale=1.0, **kw):
    _no_pretrained(pretrained)
    return MobileNetV1(scale=scale, **kw)


class _InvertedResidual(nn.Layer):
    def __init__(self, cin, cout, stride, expand):
        super().__init__()
        hid = int(round(cin * expand))
        self.use_res = stride == 1 and cin == cout
        layers = [] if expand == 1 else [_cbr(cin, hid, 1, act=nn.ReLU6)]
        layers += [_cbr(hid, hid, 3, stride, 1, g=hid, act=nn.ReLU6), nn.Conv2D(hid, cout, 1, bias_attr=False),
                   nn.BatchNorm2D(cout)]
        self.conv = nn.Sequential(*layers)

    def forward(self, x):
        return x + self.conv(x) if self.use_res else self.conv(x)


class MobileNetV2(nn.Layer):
    def __init__(self, scale=1.0, num_classes=1000, with_pool=True):
        super().__init__()
        md = lambda v: max(8, int(v * scale + 4) // 8 * 8)   # noqa: E731
        cfg = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]
        cin = md(32)
        last = md(1280) if scale > 1.0 else 1280
        layers = [_cbr(3, cin, 3, 2, 1, act=nn.ReLU6)]
        for t, c, n, s in cfg:
            for i in range(n):
                layers.append(_InvertedResidual(cin, md(c), s if i == 0 else 1, t))
                cin = md(c)
        layers.append(_cbr(cin, last, 1, act=nn.ReLU6))
        self.features = nn.Sequential(*layers)
        self.num_classes, self.with_pool = num_classes, with_pool
        if with_pool:
            self.pool2d_avg = nn.AdaptiveAvgPool2D(1)
        if num_classes > 0:
            self.classifier = nn.Sequential(nn.Dropout(0.2), nn.Linear(last, num_classes))

    def forward(self, x):
        x = self.features(x)
        if self.with_pool:
            x = self.pool2d_avg(x)
        if self.num_classes > 0:
            x = self.classifier(flatten(x, 1))
        return x


def mobilenet_v2(pretrained=False, scale=1.0, **kw):
    _no_pretrained(pretrained)
    return MobileNetV2(scale=scale, **kw)


class _Fire(nn.Layer):
    def __init__(self, cin, s, e1, e3):
        super().__init__()
        self.squeeze = nn.Sequential(nn.Conv2D(cin, s, 1), nn.ReLU())
        self.e1 = nn.Sequential(nn.Conv2D(s, e1, 1), nn.ReLU())
        self.e3 = nn.Sequential(nn.Conv2D(s, e3, 3, padding=1), nn.ReLU())

    def forward(self, x):
        x = self.squeeze(x)
        return concat([self.e1(x), self.e3(x)], axis=1)


class SqueezeNet(nn.Layer):
    def __init__(self, version="1.0", num_classes=1000, with_pool=True):
        super().__init__()
        if version == "1.0":
            feats = [nn.Conv2D(3, 96, 7, 2), nn.ReLU(), nn.MaxPool2D(3, 2), _Fire(96, 16, 64, 64), _Fire(128, 16, 64, 64),
                     _Fire(128, 32, 128, 128), nn.MaxPool2D(3, 2), _Fire(256, 32, 128, 128), _Fire(256, 48, 192, 192),
                     _Fire(384, 48, 192, 192), _Fire(384, 64, 256, 256), nn.MaxPool2D(3, 2), _Fire(512, 64, 256, 256)]
        else:
            feats = [nn.Conv2D(3, 64, 3, 2, 1), nn.ReLU(), nn.MaxPool2D(3, 2), _Fire(64, 16, 64, 64), _Fire(128, 16, 64, 64),
                     nn.MaxPool2D(3, 2), _Fire(128, 32, 128, 128), _Fire(256, 32, 128, 128), nn.MaxPool2D(3, 2),
                     _Fire(256, 48, 192, 192), _Fire(384, 48, 192, 192), _Fire(384, 64, 256, 256), _Fire(512, 64, 256, 256)]
        self.features = nn.Sequential(*feats)
        self.num_classes, self.with_pool = num_classes, with_pool
        if num_classes > 0:
            self.classifier = nn.Sequential(nn.Dropout(0.5), nn.Conv2D(512, num_classes, 1), nn.ReLU())
        if with_pool:
            self.pool = nn.AdaptiveAvgPool2D(1)

    def forward(self, x):
        x = self.features(x)
        if self.num_classes > 0:
            x = self.classifier(x)
        if self.with_pool:
            x = flatten(self.pool(x), 1)
        return x


def squeezenet1_0(pretrained=False, **kw):
    _no_pretrained(pretrained)
    return SqueezeNet("1.0", **kw)


def squeezenet1_1(pretrained=False, **kw):
    _no_pretrained(pretrained)
    return SqueezeNet("1.1", **kw)


class _DenseLayer(nn.Layer):
    def __init__(self, cin, growth, bn_size, dropout):
        super().__init__()
        self.f = nn.Sequential(nn.BatchNorm2D(cin), nn.ReLU(), nn.Conv2D(cin, bn_size * growth, 1, bias_attr=False),
                               nn.BatchNorm2D(bn_size * growth), nn.ReLU(),
                               nn.Conv2D(bn_size * growth, growth, 3, padding=1, bias_attr=False))
        self.drop = nn.Dropout(dropout) if dropout else None

    def forward(self, x):
        y = self.f(x)
        if self.drop is not None:
            y = self.drop(y)
        return concat([x, y], axis=1)


class DenseNet(nn.Layer):
    def __init__(self, layers=121, bn_size=4, dropout=0.0, num_classes=1000, with_pool=True):
        super().__init__()
        init, growth, cfg = {121: (64, 32, [6, 12, 24, 16]), 161: (96, 48, [6, 12, 36, 24]), 169: (64, 32, [6, 12, 32, 32]),
                             201: (64, 32, [6, 12, 48, 32]), 264: (64, 32, [6, 12, 64, 48])}[layers]
        feats = [nn.Conv2D(3, init, 7, 2, 3, bias_attr=False), nn.BatchNorm2D(init), nn.ReLU(), nn.MaxPool2D(3, 2, 1)]
        c = init
        for i, n in enumerate(cfg):
            for _ in range(n):
                feats.append(_DenseLayer(c, growth, bn_size, dropout))
                c += growth
            if i != len(cfg) - 1:
                feats += [nn.BatchNorm2D(c), nn.ReLU(), nn.Conv2D(c, c // 2, 1, bias_attr=False), nn.AvgPool2D(2, 2)]
                c //= 2
        feats += [nn.BatchNorm2D(c), nn.ReLU()]
        self.features = nn.Sequential(*feats)
        self.num_classes, self.with_pool = num_classes, with_pool
        if with_pool:
            self.pool = nn.AdaptiveAvgPool2D(1)
        if num_classes > 0:
            self.out = nn.Linear(c, num_classes)

    def forward(self, x):
        x = self.features(x)
        if self.with_pool:
            x = self.pool(x)
        if self.num_classes > 0:
            x = self.out(flatten(x, 1))
        return x


def _densenet(n, pretrained=False, **kw):
    _no_pretrained(pretrained)
    return DenseNet(n, **kw)


def densenet121(pretrained=False, **kw):
    return _densenet(121, pretrained, **kw)


def densenet161(pretrained=False, **kw):
    return _densenet(161, pretrained, **kw)


def densenet169(pretrained=False, **kw):
    return _densenet(169, pretrained, **kw)


def densenet201(pretrained=False, **kw):
    return _densenet(201, pretrained, **kw)


def densenet264(pretrained=False, **kw):
    return _densenet(264, pretrained, **kw)


# ----------------------------------------------------------------------------- MobileNetV3
__all__ += ["MobileNetV3Small", "MobileNetV3Large", "mobilenet_v3_small", "mobilenet_v3_large", "InceptionV3",
            "inception_v3", "GoogLeNet", "googlenet", "ShuffleNetV2", "shufflenet_v2_x0_25", "shufflenet_v2_x0_33",
            "shufflenet_v2_x0_5", "shufflenet_v2_x1_0", "shufflenet_v2_x1_5", "shufflenet_v2_x2_0", "shufflenet_v2_swish"]


def _make_divisible(v, divisor=8, min_value=None):
    min_value = min_value or divisor
    new_v = max(min_value, int(v + divisor / 2) // divisor * divisor)
    if new_v < 0.9 * v:
        new_v += divisor
    return new_v


class _SE(nn.Layer):
    def __init__(self, ch, squeeze):
        super().__init__()
        self.pool = nn.AdaptiveAvgPool2D(1)
        self.fc1, self.fc2 = nn.Conv2D(ch, squeeze, 1), nn.Conv2D(squeeze, ch, 1)
        self.relu, self.gate = nn.ReLU(), nn.Hardsigmoid()

    def forward(self, x):
        return x * self.gate(self.fc2(self.relu(self.fc1(self.pool(x)))))


class _MBV3Block(nn.Layer):
    def __init__(self, cin, k, exp, cout, use_se, act, stride):
        super().__init__()
        self.res = stride == 1 and cin == cout
        A = nn.Hardswish if act == "hardswish" else nn.ReLU
        layers = []
        if exp != cin:
            layers.append(_cbr(cin, exp, 1, act=A))
        layers.append(_cbr(exp, exp, k, stride, (k - 1) // 2, g=exp, act=A))
        if use_se:
            layers.append(_SE(exp, _make_divisible(exp // 4)))
        layers.append(nn.Sequential(nn.Conv2D(exp, cout, 1, bias_attr=False), nn.BatchNorm2D(cout)))
        self.block = nn.Sequential(*layers)

    def forward(self, x):
        y = self.block(x)
        return x + y if self.res else y


class MobileNetV3(nn.Layer):
    def __init__(self, config, last_channel, scale=1.0, num_classes=1000, with_pool=True):
        super().__init__()
        self.num_classes, self.with_pool = num_classes, with_pool
        c = lambda v: _make_divisible(v * scale)       # noqa: E731
        first = c(config[0][0])
        layers = [_cbr(3, first, 3, 2, 1, act=nn.Hardswish)]
        for cin, k, exp, cout, se, act, s in config:
            layers.append(_MBV3Block(c(cin), k, c(exp), c(cout), se, act, s))
        last_in = c(config[-1][3])
        last_conv = 6 * last_in
        layers.append(_cbr(last_in, last_conv, 1, act=nn.Hardswish))
        self.features = nn.Sequential(*layers)
        if with_pool:
            self.avgpool = nn.AdaptiveAvgPool2D(1)
        if num_classes > 0:
            self.classifier = nn.Sequential(nn.Linear(last_conv, last_channel), nn.Hardswish(), nn.Dropout(0.2),
                                            nn.Linear(last_channel, num_classes))

    def forward(self, x):
        x = self.features(x)
        if self.with_pool:
            x = self.avgpool(x)
        if self.num_classes > 0:
            x = self.classifier(flatten(x, 1))
        return x


class MobileNetV3Small(MobileNetV3):
    def __init__(self, scale=1.0, num_classes=1000, with_pool=True):
        cfg = [(16, 3, 16, 16, True, "relu", 2), (16, 3, 72, 24, False, "relu", 2), (24, 3, 88, 24, False, "relu", 1),
               (24, 5, 96, 40, True, "hardswish", 2), (40, 5, 240, 40, True, "hardswish", 1),
               (40, 5, 240, 40, True, "hardswish", 1), (40, 5, 120, 48, True, "hardswish", 1),
               (48, 5, 144, 48, True, "hardswish", 1), (48, 5, 288, 96, True, "hardswish", 2),
               (96, 5, 576, 96, True, "hardswish", 1), (96, 5, 576, 96, True, "hardswish", 1)]
        super().__init__(cfg, _make_divisible(1024 * scale), scale, num_classes, with_pool)


class MobileNetV3Large(MobileNetV3):
    def __init__(self, scale=1.0, num_classes=1000, with_pool=True):
        cfg = [(16, 3, 16, 16, False, "relu", 1), (16, 3, 64, 24, False, "relu", 2), (24, 3, 72, 24, False, "relu", 1),
               (24, 5, 72, 40, True, "relu", 2), (40, 5, 120, 40, True, "relu", 1), (40, 5, 120, 40, True, "relu", 1),
               (40, 3, 240, 80, False, "hardswish", 2), (80, 3, 200, 80, False, "hardswish", 1),
               (80, 3, 184, 80, False, "hardswish", 1), (80, 3, 184, 80, False, "hardswish", 1),
               (80, 3, 480, 112, True, "hardswish", 1), (112, 3, 672, 112, True, "hardswish", 1),
               (112, 5, 672, 160, True, "hardswish", 2), (160, 5, 960, 160, True, "hardswish", 1),
               (160, 5, 960, 160, True, "hardswish", 1)]
        super().__init__(cfg, _make_divisible(1280 * scale), scale, num_classes, with_pool)


def mobilenet_v3_small(pretrained=False, scale=1.0, **kw):
    _no_pretrained(pretrained)
    return MobileNetV3Small(scale=scale, **kw)


def mobilenet_v3_large(pretrained=False, scale=1.0, **kw):
    _no_pretrained(pretrained)
    return MobileNetV3Large(scale=scale, **kw)


# ----------------------------------------------------------------------------- ShuffleNetV2
def _channel_shuffle(x, groups):
    b, c, h, w = x.shape
    return x.reshape([b, groups, c // groups, h, w]).transpose([0, 2, 1, 3, 4]).reshape([b, c, h, w])


class _ShuffleUnit(nn.Layer):
    def __init__(self, cin, cout, stride, act):
        super().__init__()
        self.stride = stride
        half = cout // 2
        bin_ = cin if stride == 2 else half
        self.branch2 = nn.Sequential(_cbr(bin_, half, 1, act=act), nn.Conv2D(half, half, 3, stride, 1, groups=half, bias_attr=False),
                                     nn.BatchNorm2D(half), _cbr(half, half, 1, act=act))
        if stride == 2:
            self.branch1 = nn.Sequential(nn.Conv2D(cin, cin, 3, 2, 1, groups=cin, bias_attr=False), nn.BatchNorm2D(cin),
                                         _cbr(cin, half, 1, act=act))

    def forward(self, x):
        if self.stride == 1:
            c = x.shape[1] // 2
            out = concat([x[:, :c], self.branch2(x[:, c:])], 1)
        else:
            out = concat([self.branch1(x), self.branch2(x)], 1)
        return _channel_shuffle(out, 2)


class ShuffleNetV2(nn.Layer):
    def __init__(self, scale=1.0, act="relu", num_classes=1000, with_pool=True):
        super().__init__()
        self.num_classes, self.with_pool = num_classes, with_pool
        A = nn.Swish if act == "swish" else nn.ReLU
        outs = {0.25: [24, 24, 48, 96, 512], 0.33: [24, 32, 64, 128, 512], 0.5: [24, 48, 96, 192, 1024],
                1.0: [24, 116, 232, 464, 1024], 1.5: [24, 176, 352, 704, 1024], 2.0: [24, 244, 488, 976, 2048]}[scale]
        self.conv1 = _cbr(3, outs[0], 3, 2, 1, act=A)
        self.maxpool = nn.MaxPool2D(3, 2, 1)
        blocks, cin = [], outs[0]
        for reps, cout in zip([4, 8, 4], outs[1:4]):
            for i in range(reps):
                blocks.append(_ShuffleUnit(cin, cout, 2 if i == 0 else 1, A))
                cin = cout
        self.blocks = nn.Sequential(*blocks)
        self.conv_last = _cbr(cin, outs[4], 1, act=A)
        if with_pool:
            self.pool = nn.AdaptiveAvgPool2D(1)
        if num_classes > 0:
            self.fc = nn.Linear(outs[4], num_classes)

    def forward(self, x):
        x = self.conv_last(self.blocks(self.maxpool(self.conv1(x))))
        if self.with_pool:
            x = self.pool(x)
        if self.num_classes > 0:
            x = self.fc(flatten(x, 1))
        return x


def _shufflenet(scale, act="relu"):
    def f(pretrained=False, **kw):
        _no_pretrained(pretrained)
        return ShuffleNetV2(scale=scale, act=act, **kw)
    return f


shufflenet_v2_x0_25, shufflenet_v2_x0_33, shufflenet_v2_x0_5 = _shufflenet(0.25), _shufflenet(0.33), _shufflenet(0.5)
shufflenet_v2_x1_0, shufflenet_v2_x1_5, shufflenet_v2_x2_0 = _shufflenet(1.0), _shufflenet(1.5), _shufflenet(2.0)
shufflenet_v2_swish = _shufflenet(1.0, "swish")


# ----------------------------------------------------------------------------- GoogLeNet
class _Inception(nn.Layer):
    def __init__(self, cin, c1, c3r, c3, c5r, c5, proj):
        super().__init__()
        self.b1 = nn.Sequential(nn.Conv2D(cin, c1, 1), nn.ReLU())
        self.b2 = nn.Sequential(nn.Conv2D(cin, c3r, 1), nn.ReLU(), nn.Conv2D(c3r, c3, 3, padding=1), nn.ReLU())
        self.b3 = nn.Sequential(nn.Conv2D(cin, c5r, 1), nn.ReLU(), nn.Conv2D(c5r, c5, 5, padding=2), nn.ReLU())
        self.b4 = nn.Sequential(nn.MaxPool2D(3, 1, 1), nn.Conv2D(cin, proj, 1), nn.ReLU())

    def forward(self, x):
        return concat([self.b1(x), self.b2(x), self.b3(x), self.b4(x)], 1)


class GoogLeNet(nn.Layer):
    """Returns ``(out, aux1, aux2)`` like the reference (python/paddle/vision/models/googlenet.py)."""

    def __init__(self, num_classes=1000, with_pool=True):
        super().__init__()
        self.num_classes, self.with_pool = num_classes, with_pool
        self.stem = nn.Sequential(nn.Conv2D(3, 64, 7, 2, 3), nn.ReLU(), nn.MaxPool2D(3, 2, ceil_mode=True),
                                  nn.Conv2D(64, 64, 1), nn.ReLU(), nn.Conv2D(64, 192, 3, padding=1), nn.ReLU(),
                                  nn.MaxPool2D(3, 2, ceil_mode=True))
        self.i3a, self.i3b = _Inception(192, 64, 96, 128, 16, 32, 32), _Inception(256, 128, 128, 192, 32, 96, 64)
        self.pool3 = nn.MaxPool2D(3, 2, ceil_mode=True)
        self.i4a, self.i4b = _Inception(480, 192, 96, 208, 16, 48, 64), _Inception(512, 160, 112, 224, 24, 64, 64)
        self.i4c, self.i4d = _Inception(512, 128, 128, 256, 24, 64, 64), _Inception(512, 112, 144, 288, 32, 64, 64)
        self.i4e = _Inception(528, 256, 160, 320, 32, 128, 128)
        self.pool4 = nn.MaxPool2D(3, 2, ceil_mode=True)
        self.i5a, self.i5b = _Inception(832, 256, 160, 320, 32, 128, 128), _Inception(832, 384, 192, 384, 48, 128, 128)
        if with_pool:
            self.pool5 = nn.AdaptiveAvgPool2D(1)
            self.aux_pool = nn.AvgPool2D(5, 3)
        if num_classes > 0:
            self.drop = nn.Dropout(0.4)
            self.fc = nn.Linear(1024, num_classes)
            self.aux1 = nn.Sequential(nn.Conv2D(512, 128, 1), nn.ReLU(), nn.Flatten(), nn.Linear(128 * 16, 1024), nn.ReLU(),
                                      nn.Dropout(0.7), nn.Linear(1024, num_classes))
            self.aux2 = nn.Sequential(nn.Conv2D(528, 128, 1), nn.ReLU(), nn.Flatten(), nn.Linear(128 * 16, 1024), nn.ReLU(),
                                      nn.Dropout(0.7), nn.Linear(1024, num_classes))

    def forward(self, x):
        x = self.pool3(self.i3b(self.i3a(self.stem(x))))
        a = self.i4a(x)
        d = self.i4d(self.i4c(self.i4b(a)))
        x = self.i5b(self.i5a(self.pool4(self.i4e(d))))
        out, o1, o2 = x, a, d
        if self.with_pool:
            out, o1, o2 = self.pool5(out), self.aux_pool(o1), self.aux_pool(o2)
        if self.num_classes > 0:
            out = self.fc(self.drop(flatten(out, 1)))
            o1, o2 = self.aux1(o1), self.aux2(o2)
        return out, o1, o2


def googlenet(pretrained=False, **kw):
    _no_pretrained(pretrained)
    return GoogLeNet(**kw)


# ----------------------------------------------------------------------------- InceptionV3
def _bc(cin, cout, k, s=1, p=0):
    return _cbr(cin, cout, k, s, p)


class _IncA(nn.Layer):
    def __init__(self, cin, pool):
        super().__init__()
        self.b1 = _bc(cin, 64, 1)
        self.b5 = nn.Sequential(_bc(cin, 48, 1), _bc(48, 64, 5, p=2))
        self.b3 = nn.Sequential(_bc(cin, 64, 1), _bc(64, 96, 3, p=1), _bc(96, 96, 3, p=1))
        self.bp = nn.Sequential(nn.AvgPool2D(3, 1, 1, exclusive=False), _bc(cin, pool, 1))

    def forward(self, x):
        return concat([self.b1(x), self.b5(x), self.b3(x), self.bp(x)], 1)


class _IncB(nn.Layer):
    def __init__(self, cin):
        super().__init__()
        self.b3 = _bc(cin, 384, 3, 2)
        self.bd = nn.Sequential(_bc(cin, 64, 1), _bc(64, 96, 3, p=1), _bc(96, 96, 3, 2))
        self.bp = nn.MaxPool2D(3, 2)

    def forward(self, x):
        return concat([self.b3(x), self.bd(x), self.bp(x)], 1)


class _IncC(nn.Layer):
    def __init__(self, cin, c7):
        super().__init__()
        self.b1 = _bc(cin, 192, 1)
        self.b7 = nn.Sequential(_bc(cin, c7, 1), _bc(c7, c7, (1, 7), p=(0, 3)), _bc(c7, 192, (7, 1), p=(3, 0)))
        self.bd = nn.Sequential(_bc(cin, c7, 1), _bc(c7, c7, (7, 1), p=(3, 0)), _bc(c7, c7, (1, 7), p=(0, 3)),
                                _bc(c7, c7, (7, 1), p=(3, 0)), _bc(c7, 192, (1, 7), p=(0, 3)))
        self.bp = nn.Sequential(nn.AvgPool2D(3, 1, 1, exclusive=False), _bc(cin, 192, 1))

    def forward(self, x):
        return concat([self.b1(x), self.b7(x), self.bd(x), self.bp(x)], 1)


class _IncD(nn.Layer):
    def __init__(self, cin):
        super().__init__()
        self.b3 = nn.Sequential(_bc(cin, 192, 1), _bc(192, 320, 3, 2))
        self.b7 = nn.Sequential(_bc(cin, 192, 1), _bc(192, 192, (1, 7), p=(0, 3)), _bc(192, 192, (7, 1), p=(3, 0)),
                                _bc(192, 192, 3, 2))
        self.bp = nn.MaxPool2D(3, 2)

    def forward(self, x):
        return concat([self.b3(x), self.b7(x), self.bp(x)], 1)


class _IncE(nn.Layer):
    def __init__(self, cin):
        super().__init__()
        self.b1 = _bc(cin, 320, 1)
        self.b3 = _bc(cin, 384, 1)
        self.b3a, self.b3b = _bc(384, 384, (1, 3), p=(0, 1)), _bc(384, 384, (3, 1), p=(1, 0))
        self.bd = nn.Sequential(_bc(cin, 448, 1), _bc(448, 384, 3, p=1))
        self.bda, self.bdb = _bc(384, 384, (1, 3), p=(0, 1)), _bc(384, 384, (3, 1), p=(1, 0))
        self.bp = nn.Sequential(nn.AvgPool2D(3, 1, 1, exclusive=False), _bc(cin, 192, 1))

    def forward(self, x):
        b3 = self.b3(x)
        bd = self.bd(x)
        return concat([self.b1(x), self.b3a(b3), self.b3b(b3), self.bda(bd), self.bdb(bd), self.bp(x)], 1)


class InceptionV3(nn.Layer):
    def __init__(self, num_classes=1000, with_pool=True):
        super().__init__()
        self.num_classes, self.with_pool = num_classes, with_pool
        self.stem = nn.Sequential(_bc(3, 32, 3, 2), _bc(32, 32, 3), _bc(32, 64, 3, p=1), nn.MaxPool2D(3, 2),
                                  _bc(64, 80, 1), _bc(80, 192, 3), nn.MaxPool2D(3, 2))
        self.blocks = nn.Sequential(_IncA(192, 32), _IncA(256, 64), _IncA(288, 64), _IncB(288), _IncC(768, 128),
                                    _IncC(768, 160), _IncC(768, 160), _IncC(768, 192), _IncD(768), _IncE(1280), _IncE(2048))
        if with_pool:
            self.avg_pool = nn.AdaptiveAvgPool2D(1)
        if num_classes > 0:
            self.dropout = nn.Dropout(0.2)
            self.fc = nn.Linear(2048, num_classes)

    def forward(self, x):
        x = self.blocks(self.stem(x))
        if self.with_pool:
            x = self.avg_pool(x)
        if self.num_classes > 0:
            x = self.fc(self.dropout(flatten(x, 1)))
        return x


def inception_v3(pretrained=False, **kw):
    _no_pretrained(pretrained)
    return InceptionV3(**kw)
