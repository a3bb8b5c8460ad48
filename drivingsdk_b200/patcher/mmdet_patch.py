"""mmdet hooks: the ResNet blocks end in this package's fused add + ReLU, and the stem's
max pooling uses this package's kernel when no gradient is needed.

Same patch classes, names and targets as the reference
(mx_driving/patcher/mmdet_patch.py:43-143). The replacement ``forward`` methods restate
mmdet's ``BasicBlock.forward``, ``Bottleneck.forward`` and ``ResNet.forward`` with the
final ``out += identity; out = relu(out)`` replaced by ``npu_add_relu(out, identity)`` and
``self.maxpool(x)`` replaced by ``npu_max_pool2d(x, 3, 2, 1)`` for tensors that do not
require grad. Operators are looked up when a patched method runs, so importing this module
needs neither torch nor the compiled extension.
"""
from typing import List

from .patch import AtomicPatch, BasePatch, Patch


def _checkpointed(fn, module, x):
    """Runs ``fn(x)`` under activation checkpointing when the block asks for it (re-entrant
    variant, which is what mmdet's blocks get from torch's historical default)."""
    if module.with_cp and x.requires_grad:
        import torch.utils.checkpoint as cp
        return cp.checkpoint(fn, x, use_reentrant=True)
    return fn(x)


class ResNetAddRelu(Patch):
    """ResNet add+relu fusion patch for mmdet."""

    name = "resnet_add_relu"
    legacy_name = "resnet_add_relu"
    target_module = "mmdet"

    @staticmethod
    def _basicblock_forward_replacement(self, x):
        from mx_driving import npu_add_relu

        def run(x):
            out = self.relu(self.norm1(self.conv1(x)))
            out = self.norm2(self.conv2(out))
            identity = x if self.downsample is None else self.downsample(x)
            return npu_add_relu(out, identity)

        return _checkpointed(run, self, x)

    @staticmethod
    def _bottleneck_forward_replacement(self, x):
        from mx_driving import npu_add_relu

        def plugins(out, names_attr):
            if self.with_plugins:
                return self.forward_plugin(out, getattr(self, names_attr))
            return out

        def run(x):
            out = plugins(self.relu(self.norm1(self.conv1(x))), "after_conv1_plugin_names")
            out = plugins(self.relu(self.norm2(self.conv2(out))), "after_conv2_plugin_names")
            out = plugins(self.norm3(self.conv3(out)), "after_conv3_plugin_names")
            identity = x if self.downsample is None else self.downsample(x)
            return npu_add_relu(out, identity)

        return _checkpointed(run, self, x)

    @classmethod
    def patches(cls, options=None) -> List[BasePatch]:
        return [
            AtomicPatch("mmdet.models.backbones.resnet.BasicBlock.forward",
                        cls._basicblock_forward_replacement),
            AtomicPatch("mmdet.models.backbones.resnet.Bottleneck.forward",
                        cls._bottleneck_forward_replacement),
        ]


class ResNetMaxPool(Patch):
    """ResNet maxpool optimization patch for mmdet."""

    name = "resnet_maxpool"
    legacy_name = "resnet_maxpool"
    target_module = "mmdet"

    @staticmethod
    def _forward_replacement(self, x):
        from mx_driving import npu_max_pool2d
        if self.deep_stem:
            x = self.stem(x)
        else:
            x = self.relu(self.norm1(self.conv1(x)))
        x = self.maxpool(x) if x.requires_grad else npu_max_pool2d(x, 3, 2, 1)
        outs = []
        for i, layer_name in enumerate(self.res_layers):
            x = getattr(self, layer_name)(x)
            if i in self.out_indices:
                outs.append(x)
        return tuple(outs)

    @classmethod
    def patches(cls, options=None) -> List[BasePatch]:
        return [AtomicPatch("mmdet.models.backbones.resnet.ResNet.forward",
                            cls._forward_replacement)]
