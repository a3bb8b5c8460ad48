"""One-call hook that makes mmcv models use this package's MSDA operator.

    from mx_driving.patcher import default_patcher
    default_patcher.apply()

Same surface as the reference's patcher for this path (mx_driving/patcher/__init__.py):
``Patcher``, ``Patch``, ``AtomicPatch``, ``BasePatch``, ``PatchStatus``, ``PatchResult``,
``MultiScaleDeformableAttention`` (alias ``MSDA``), ``DeformConv``, ``ModulatedDeformConv``,
``ResNetAddRelu``, ``ResNetMaxPool``, ``default_patcher``, the legacy functions
``msda(module, options)``, ``dc``, ``mdc``, ``resnet_add_relu``, ``resnet_maxpool``, ``configure_patcher_logging`` and ``set_patcher_log_level``; and the older builder-style
API (``PatcherBuilder().add_module_patch("mmcv", Patch(msda)).build()``, ``legacy.py``) that
the reference's model examples still use. The
reference's other predefined patches (sparse convolution, dataset and optimizer shims, ...)
belong to operators that are not part of this package.
"""
from typing import Dict, List, Type

from .patcher_logger import configure_patcher_logging, patcher_logger, set_patcher_log_level
from .reporting import PatchResult, PatchStatus
from .patch import AtomicPatch, BasePatch, LegacyPatch, Patch
from .patcher import Patcher, replace_with
from .mmcv_patch import DeformConv, ModulatedDeformConv, MultiScaleDeformableAttention
from .version import check_version, get_version, is_mmcv_v1x, is_mmcv_v2x, mmcv_version
from .mmdet_patch import ResNetAddRelu, ResNetMaxPool

MSDA = MultiScaleDeformableAttention  # alias

# same order as the reference's registry (mx_driving/patcher/__init__.py:116-149), restricted
# to the patches whose operators exist in this package
_ALL_PATCH_CLASSES: List[Type[Patch]] = [
    MultiScaleDeformableAttention, DeformConv, ModulatedDeformConv,
    ResNetAddRelu, ResNetMaxPool,
]
_DEFAULT_PATCH_CLASSES: List[Type[Patch]] = [
    MultiScaleDeformableAttention, DeformConv, ModulatedDeformConv,
    ResNetAddRelu, ResNetMaxPool,
]


def _create_default_patcher() -> Patcher:
    patcher = Patcher()
    patcher.add(*_DEFAULT_PATCH_CLASSES)
    return patcher


default_patcher = _create_default_patcher()

_LEGACY_NAME_TO_CLASS: Dict[str, Type[Patch]] = {
    cls.legacy_name: cls for cls in _ALL_PATCH_CLASSES if getattr(cls, "legacy_name", None)
}


def _create_legacy_patch_func(patch_cls: Type[Patch]):
    """Old function-style API: ``func(module, options)`` applies the group's patches."""
    def legacy_func(module, options):
        for atomic in patch_cls.patches(options):
            atomic.apply()
    legacy_func.__name__ = patch_cls.legacy_name
    return legacy_func


msda = _create_legacy_patch_func(MultiScaleDeformableAttention)
dc = _create_legacy_patch_func(DeformConv)
mdc = _create_legacy_patch_func(ModulatedDeformConv)
resnet_add_relu = _create_legacy_patch_func(ResNetAddRelu)
resnet_maxpool = _create_legacy_patch_func(ResNetMaxPool)

from .legacy import (  # noqa: E402  (needs the registry above)
    LegacyPatcherBuilder,
    LegacyPatcherBuilder as PatcherBuilder,
    LegacyPatchWrapper,
    default_patcher_builder,
)

__all__ = [
    "Patcher", "BasePatch", "Patch", "AtomicPatch", "LegacyPatch", "replace_with",
    "PatcherBuilder", "LegacyPatcherBuilder", "LegacyPatchWrapper", "default_patcher_builder",
    "patcher_logger", "configure_patcher_logging", "set_patcher_log_level",
    "PatchStatus", "PatchResult",
    "default_patcher", "MultiScaleDeformableAttention", "MSDA", "msda",
    "DeformConv", "ModulatedDeformConv", "dc", "mdc",
    "ResNetAddRelu", "ResNetMaxPool", "resnet_add_relu", "resnet_maxpool",
    "_ALL_PATCH_CLASSES", "_DEFAULT_PATCH_CLASSES", "_LEGACY_NAME_TO_CLASS",
]
