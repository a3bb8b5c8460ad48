"""``mx_driving.patcher``: the same objects as ``drivingsdk_b200.patcher``, with the
reference's sub-module paths (``mx_driving.patcher.patch`` etc.) importable too."""
import sys

from drivingsdk_b200 import patcher as _impl
from drivingsdk_b200.patcher import *  # noqa: F401,F403
from drivingsdk_b200.patcher import (  # noqa: F401
    _ALL_PATCH_CLASSES, _DEFAULT_PATCH_CLASSES, _LEGACY_NAME_TO_CLASS,
    legacy, mmcv_patch, mmdet_patch, patch, patcher, patcher_logger as _logger_obj, reporting,
)
import drivingsdk_b200.patcher.patcher_logger as _logger_mod

__all__ = list(_impl.__all__)

for _name, _mod in (("patch", patch), ("patcher", patcher), ("reporting", reporting),
                    ("legacy", legacy), ("mmcv_patch", mmcv_patch), ("mmdet_patch", mmdet_patch), ("patcher_logger", _logger_mod)):
    sys.modules[f"{__name__}.{_name}"] = _mod
