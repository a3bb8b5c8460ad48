"""The old builder-style patcher API, kept so that launch scripts written for it keep working
(mx_driving/patcher/legacy.py):

    from mx_driving.patcher import PatcherBuilder, Patch
    from mx_driving.patcher import msda, dc, mdc, resnet_add_relu, resnet_maxpool

    builder = (PatcherBuilder()
               .add_module_patch("mmcv", Patch(msda), Patch(dc), Patch(mdc))
               .add_module_patch("mmdet", Patch(resnet_add_relu), Patch(resnet_maxpool)))
    with builder.build():
        main()

Everything here translates to the ``Patcher`` of patcher.py: a wrapped function whose name is
one of the predefined groups' ``legacy_name`` expands to that group's patches, any other
function ``func(module, options)`` becomes a ``LegacyPatch`` on the named module.
``with_profiling`` and ``brake_at`` are accepted and passed on (they are inert there).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Set

from .patch import LegacyPatch
from .patcher import Patcher
from .patcher_logger import patcher_logger

__all__ = ["LegacyPatchWrapper", "LegacyPatcherBuilder", "PatcherBuilder", "default_patcher_builder"]


class LegacyPatchWrapper:
    """What ``Patch(func)`` returns: the function, its options and a sort priority (lower
    goes first within a module)."""

    _notice_shown = False

    def __init__(self, func: Callable, options: Optional[Dict] = None, priority: int = 0,
                 patch_failure_warning: bool = True):
        self.func = func
        self.name = func.__name__
        self.options = options if options is not None else {}
        self.priority = priority
        self.is_applied = False
        self.patch_failure_warning = patch_failure_warning
        if not LegacyPatchWrapper._notice_shown:
            patcher_logger.info("Using the builder-style patcher API (Patch(func)); the class "
                                "style (patcher.add(MyPatch).apply()) is the current one.")
            LegacyPatchWrapper._notice_shown = True

    def __lt__(self, other):
        return self.priority < other.priority

    def __repr__(self) -> str:
        return f"LegacyPatchWrapper({self.name})"


class _LegacyPatcher:
    """What ``build()`` returns: ``apply()`` or use as a context manager."""

    def __init__(self, patcher: Patcher, allow_internal_format: bool = False):
        self._patcher = patcher
        self._allow_internal_format = allow_internal_format

    def transfer_to_npu(self):
        """Kept for call compatibility; there is nothing to transfer on CUDA."""

    def apply(self):
        self._patcher.apply(allow_internal_format=self._allow_internal_format)

    def __enter__(self):
        self.apply()
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        return None

    @property
    def is_applied(self) -> bool:
        return self._patcher.is_applied

    @property
    def results(self):
        return self._patcher.results


class LegacyPatcherBuilder:
    def __init__(self):
        self._module_patches: Dict[str, List[LegacyPatchWrapper]] = {}
        self._blacklist: Set[str] = set()
        self._profiling_options: Optional[Dict] = None
        self._brake_step: Optional[int] = None

    def add_module_patch(self, module_name: str, *patches: LegacyPatchWrapper) -> "LegacyPatcherBuilder":
        bucket = self._module_patches.setdefault(module_name, [])
        bucket.extend(patches)
        bucket.sort()          # stable: by priority, insertion order within a priority
        return self

    def disable_patches(self, *patch_names: str) -> "LegacyPatcherBuilder":
        self._blacklist.update(patch_names)
        return self

    def with_profiling(self, path: str, level: int = 0, skip_first: int = 20, wait: int = 1,
                       warmup: int = 1, active: int = 1, repeat: int = 1) -> "LegacyPatcherBuilder":
        self._profiling_options = dict(path=path, level=level, skip_first=skip_first, wait=wait,
                                       warmup=warmup, active=active, repeat=repeat)
        return self

    def brake_at(self, brake_step: int) -> "LegacyPatcherBuilder":
        self._brake_step = brake_step
        return self

    def build(self, allow_internal_format: bool = False) -> _LegacyPatcher:
        from . import _LEGACY_NAME_TO_CLASS
        patcher = Patcher()
        for module_name, wrappers in self._module_patches.items():
            for wrapper in wrappers:
                if wrapper.name in self._blacklist:
                    continue
                group = _LEGACY_NAME_TO_CLASS.get(wrapper.name)
                if group is not None:
                    for patch in group.patches(wrapper.options or None):
                        patch._parent_name = group.name
                        patcher.add(patch)
                else:
                    patcher.add(LegacyPatch(wrapper.func, target_module=module_name,
                                            options=wrapper.options))
        for name in self._blacklist:
            patcher.disable(name)
        if self._profiling_options:
            patcher.with_profiling(**self._profiling_options)
        if self._brake_step is not None:
            patcher.brake_at(self._brake_step)
        return _LegacyPatcher(patcher, allow_internal_format)


class _DefaultPatcherBuilderProxy:
    """``default_patcher_builder`` of the old API: a builder preloaded with the default
    groups, created on first use."""

    def __init__(self):
        self._builder: Optional[LegacyPatcherBuilder] = None

    def _get_builder(self) -> LegacyPatcherBuilder:
        if self._builder is None:
            from . import _DEFAULT_PATCH_CLASSES, _create_legacy_patch_func
            builder = LegacyPatcherBuilder()
            for group in _DEFAULT_PATCH_CLASSES:
                if group.target_module and group.legacy_name:
                    builder.add_module_patch(group.target_module,
                                             LegacyPatchWrapper(_create_legacy_patch_func(group)))
            self._builder = builder
        return self._builder

    def add_module_patch(self, module_name: str, *patches):
        self._get_builder().add_module_patch(module_name, *patches)
        return self

    def disable_patches(self, *patch_names: str):
        self._get_builder().disable_patches(*patch_names)
        return self

    def with_profiling(self, path: str, **kwargs):
        self._get_builder().with_profiling(path, **kwargs)
        return self

    def brake_at(self, brake_step: int):
        self._get_builder().brake_at(brake_step)
        return self

    def build(self, allow_internal_format: bool = False) -> _LegacyPatcher:
        return self._get_builder().build(allow_internal_format)

    def __repr__(self):
        return "<DefaultPatcherBuilderProxy>"


default_patcher_builder = _DefaultPatcherBuilderProxy()
PatcherBuilder = LegacyPatcherBuilder
