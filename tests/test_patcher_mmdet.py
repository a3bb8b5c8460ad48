"""The mmdet hooks (ResNet add+ReLU fusion, stem max pooling): pure Python, CPU.

A module tree shaped like ``mmdet.models.backbones.resnet`` is built from torch modules; the
operators the patched methods look up under ``mx_driving`` are replaced by recorders that
compute the same function with torch, so the block arithmetic can be compared with the
unpatched forward. Follows the reference's expectations for these patches
(mx_driving/patcher/mmdet_patch.py:43-143).
"""
import sys
import types

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from drivingsdk_b200.patcher import (Patcher, PatchStatus, ResNetAddRelu, ResNetMaxPool,
                                     default_patcher, resnet_add_relu)


class _BasicBlock(nn.Module):
    def __init__(self, c, downsample=False):
        super().__init__()
        self.conv1, self.norm1 = nn.Conv2d(c, c, 3, padding=1), nn.BatchNorm2d(c)
        self.conv2, self.norm2 = nn.Conv2d(c, c, 3, padding=1), nn.BatchNorm2d(c)
        self.relu = nn.ReLU()
        self.downsample = nn.Conv2d(c, c, 1) if downsample else None
        self.with_cp = False

    def forward(self, x):
        identity = x
        out = self.relu(self.norm1(self.conv1(x)))
        out = self.norm2(self.conv2(out))
        if self.downsample is not None:
            identity = self.downsample(x)
        out = out + identity
        return self.relu(out)


class _Bottleneck(_BasicBlock):
    def __init__(self, c, downsample=False):
        super().__init__(c, downsample)
        self.conv3, self.norm3 = nn.Conv2d(c, c, 1), nn.BatchNorm2d(c)
        self.with_plugins = False

    def forward(self, x):
        identity = x
        out = self.relu(self.norm1(self.conv1(x)))
        out = self.relu(self.norm2(self.conv2(out)))
        out = self.norm3(self.conv3(out))
        if self.downsample is not None:
            identity = self.downsample(x)
        return self.relu(out + identity)


class _ResNet(nn.Module):
    def __init__(self, c=4):
        super().__init__()
        self.deep_stem = False
        self.conv1, self.norm1, self.relu = nn.Conv2d(3, c, 3, padding=1), nn.BatchNorm2d(c), nn.ReLU()
        self.maxpool = nn.MaxPool2d(3, 2, 1)
        self.layer1, self.layer2 = _BasicBlock(c), _Bottleneck(c, downsample=True)
        self.res_layers = ["layer1", "layer2"]
        self.out_indices = (0, 1)

    def forward(self, x):
        x = self.maxpool(self.relu(self.norm1(self.conv1(x))))
        outs = []
        for i, name in enumerate(self.res_layers):
            x = getattr(self, name)(x)
            if i in self.out_indices:
                outs.append(x)
        return tuple(outs)


@pytest.fixture
def fake_mmdet():
    names = ["mmdet", "mmdet.models", "mmdet.models.backbones", "mmdet.models.backbones.resnet"]
    mods = [types.ModuleType(n) for n in names]
    for parent, child, n in zip(mods, mods[1:], names[1:]):
        setattr(parent, n.rsplit(".", 1)[1], child)
    leaf = mods[-1]
    # fresh subclasses, so that patching them does not leak into other tests
    leaf.BasicBlock = type("BasicBlock", (_BasicBlock,), {"forward": _BasicBlock.forward})
    leaf.Bottleneck = type("Bottleneck", (_Bottleneck,), {"forward": _Bottleneck.forward})
    leaf.ResNet = type("ResNet", (_ResNet,), {"forward": _ResNet.forward})
    saved = {n: sys.modules.get(n) for n in names}
    sys.modules.update(dict(zip(names, mods)))
    yield leaf
    for n, v in saved.items():
        if v is None:
            sys.modules.pop(n, None)
        else:
            sys.modules[n] = v


@pytest.fixture
def recorders(monkeypatch):
    calls = {"add_relu": 0, "max_pool": 0}

    def add_relu(x, y):
        calls["add_relu"] += 1
        return F.relu(x + y)

    def max_pool(x, k, s, p):
        calls["max_pool"] += 1
        assert (k, s, p) == (3, 2, 1)
        return F.max_pool2d(x, k, s, p)

    import mx_driving
    monkeypatch.setattr(mx_driving, "npu_add_relu", add_relu, raising=False)
    monkeypatch.setattr(mx_driving, "npu_max_pool2d", max_pool, raising=False)
    return calls


def test_patch_class_attributes_and_registry():
    assert (ResNetAddRelu.name, ResNetAddRelu.legacy_name, ResNetAddRelu.target_module) == \
        ("resnet_add_relu", "resnet_add_relu", "mmdet")
    assert (ResNetMaxPool.name, ResNetMaxPool.legacy_name, ResNetMaxPool.target_module) == \
        ("resnet_maxpool", "resnet_maxpool", "mmdet")
    targets = [p.target for p in ResNetAddRelu.patches()] + [p.target for p in ResNetMaxPool.patches()]
    assert targets == ["mmdet.models.backbones.resnet.BasicBlock.forward",
                       "mmdet.models.backbones.resnet.Bottleneck.forward",
                       "mmdet.models.backbones.resnet.ResNet.forward"]
    names = [patch.name for patch, _ in default_patcher.collect()]
    for t in targets:
        assert t in names


def test_skipped_without_mmdet():
    assert "mmdet" not in sys.modules
    p = Patcher().add(ResNetAddRelu, ResNetMaxPool)
    p.apply()
    assert [r.status for r in p.results] == [PatchStatus.SKIPPED] * 3


def test_blocks_compute_the_same_function_through_the_fused_operator(fake_mmdet, recorders):
    torch.manual_seed(0)
    for cls, kwargs in ((fake_mmdet.BasicBlock, {}), (fake_mmdet.BasicBlock, {"downsample": True}),
                        (fake_mmdet.Bottleneck, {}), (fake_mmdet.Bottleneck, {"downsample": True})):
        block = cls(4, **kwargs).eval()
        x = torch.randn(2, 4, 6, 5)
        want = block(x)
        p = Patcher().add(ResNetAddRelu)
        p.apply()
        assert [r.status for r in p.results] == [PatchStatus.APPLIED] * 2
        before = recorders["add_relu"]
        got = block(x)
        assert recorders["add_relu"] == before + 1
        assert torch.allclose(got, want)
        # activation checkpointing path
        block.with_cp = True
        xg = x.clone().requires_grad_()
        assert torch.allclose(block(xg), want)


def test_stem_uses_the_pooling_kernel_only_without_grad(fake_mmdet, recorders):
    torch.manual_seed(1)
    net = fake_mmdet.ResNet().eval()
    x = torch.randn(1, 3, 9, 11)
    with torch.no_grad():
        want = net(x)
    p = Patcher().add(ResNetMaxPool)
    p.apply()
    assert [r.status for r in p.results] == [PatchStatus.APPLIED]
    with torch.no_grad():
        got = net(x)
    assert recorders["max_pool"] == 1
    assert len(got) == 2 and all(torch.allclose(a, b) for a, b in zip(got, want))
    net(x.requires_grad_())  # activations require grad here: torch's own pooling
    assert recorders["max_pool"] == 1


def test_legacy_function(fake_mmdet, recorders):
    resnet_add_relu(None, {})
    block = fake_mmdet.BasicBlock(4).eval()
    block(torch.randn(1, 4, 3, 3))
    assert recorders["add_relu"] == 1
