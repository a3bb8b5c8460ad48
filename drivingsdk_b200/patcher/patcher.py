"""The Patcher: an ordered collection of patches applied in one go.

Counterpart of the reference's mx_driving/patcher/patcher.py for what the MSDA hook
needs: ``add`` (Patch classes or patch instances, chainable, :300-325), ``disable`` (by
name, class or instance, :338-348), ``apply`` (insertion order, once, failures logged and
never raised, :834-880), plus ``results`` for inspection. Training-loop, profiling and
device-format features of the reference's Patcher are NPU-specific and not present.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Set, Tuple, Type, Union

from .patch import BasePatch, Patch
from .patcher_logger import patcher_logger
from .reporting import PatchResult, PatchStatus


class Patcher:
    def __init__(self):
        self._entries: List[Tuple[str, object, Optional[Dict]]] = []
        self._blacklist: Set[str] = set()
        self._applied = False
        self._resolved: Dict[int, List[BasePatch]] = {}
        self.results: List[PatchResult] = []
        self._inert_requests: List[str] = []

    # ------------------------------------------------------------------ building
    @staticmethod
    def _is_patch_class(item) -> bool:
        return isinstance(item, type) and issubclass(item, Patch)

    def add(self, *items: Union[Type[Patch], BasePatch], options: Optional[Dict] = None) -> "Patcher":
        for item in items:
            if self._is_patch_class(item):
                self._warn_on_conflict(item)
                self._entries.append(("class", item, options))
            elif isinstance(item, BasePatch):
                self._entries.append(("direct", item, None))
            else:
                raise TypeError(f"Expected Patch class or BasePatch instance, got {type(item)}")
        return self

    def disable(self, *names: Union[str, Type[Patch], BasePatch]) -> "Patcher":
        for item in names:
            if isinstance(item, str):
                self._blacklist.add(item)
            elif self._is_patch_class(item) or isinstance(item, BasePatch):
                self._blacklist.add(item.name)
            else:
                raise TypeError(
                    f"Expected patch name, Patch class, or BasePatch instance, got {type(item)}")
        return self

    def _enabled_classes(self) -> List[Type[Patch]]:
        return [item for kind, item, _ in self._entries
                if kind == "class" and item.name not in self._blacklist]

    def _warn_on_conflict(self, new_cls: Type[Patch]) -> None:
        theirs = set(getattr(new_cls, "conflicts_with", None) or [])
        for cls in self._enabled_classes():
            if cls.name == new_cls.name:
                continue
            mine = set(getattr(cls, "conflicts_with", None) or [])
            if cls.name in theirs or new_cls.name in mine:
                patcher_logger.warning(
                    f"Patch '{new_cls.name}' conflicts with already-enabled patch '{cls.name}'; "
                    f"disable one of them, e.g. patcher.disable('{cls.name}')")

    # Training-loop shims of the reference (mx_driving/patcher/patcher.py:672-707): they patch
    # the mmcv / mmengine runners to drive the NPU profiler or to stop a run after N steps.
    # The calls are accepted so that existing launch scripts keep working; they change nothing
    # here, and apply() says so once.
    def with_profiling(self, path: str, level: int = 0, skip_first: int = 20, wait: int = 1,
                       warmup: int = 1, active: int = 1, repeat: int = 1) -> "Patcher":
        self._inert_requests.append(f"with_profiling(path={path!r})")
        return self

    def brake_at(self, step: int) -> "Patcher":
        self._inert_requests.append(f"brake_at({step})")
        return self

    # ------------------------------------------------------------------ inspection
    def collect(self) -> List[Tuple[BasePatch, str]]:
        """(patch, group name) pairs in insertion order, disabled groups left out."""
        out: List[Tuple[BasePatch, str]] = []
        order = 0
        for index, (kind, item, options) in enumerate(self._entries):
            if kind == "class":
                if item.name in self._blacklist:
                    continue
                if index not in self._resolved:
                    self._resolved[index] = list(item.patches(options))
                members = self._resolved[index]
                group = item.name
            else:
                members, group = [item], getattr(item, "_parent_name", item.name)
            for patch in members:
                patch._order = order
                order += 1
                out.append((patch, group))
        return out

    def _collect_all_patches(self, force_refresh: bool = False) -> List[Tuple[BasePatch, str]]:
        """The reference's name for ``collect`` (mx_driving/patcher/patcher.py:796-832), which
        its tests call. The list is rebuilt on every call (adding or disabling a patch takes
        effect at once), so ``force_refresh`` has nothing left to do."""
        return self.collect()

    @property
    def is_applied(self) -> bool:
        return self._applied

    def print_info(self, diff: bool = False) -> "Patcher":
        lines = ["registered patches:"]
        for patch, group in self.collect():
            state = "[disabled]" if patch.name in self._blacklist else (
                "[applied]" if getattr(patch, "is_applied", False) else "[pending]")
            lines.append(f"  {state} ({group}) {patch.get_info(show_diff=diff)}")
        patcher_logger.info("\n".join(lines))
        return self

    # ------------------------------------------------------------------ applying
    def _apply_one(self, patch: BasePatch, group: str) -> None:
        pkg = patch.module or ""
        if patch.name in self._blacklist:
            patcher_logger.skipped(patch.name, reason="disabled", package=pkg, patch_name=group)
            self.results.append(PatchResult(PatchStatus.SKIPPED, patch.name, pkg, "disabled"))
            return
        if getattr(patch, "is_applied", False):
            return
        try:
            result = patch.apply()
        except Exception as exc:  # a patch must never take the program down
            result = PatchResult(PatchStatus.FAILED, patch.name, pkg, str(exc))
        self.results.append(result)
        if result.status is PatchStatus.APPLIED:
            patcher_logger.applied(patch.name, package=pkg, patch_name=group)
        elif result.status is PatchStatus.SKIPPED:
            patcher_logger.skipped(patch.name, reason=result.reason or "", package=pkg,
                                   patch_name=group)
        else:
            patcher_logger.failed(patch.name, reason=result.reason or "", package=pkg,
                                  patch_name=group)

    def apply(self, allow_internal_format: Optional[bool] = None) -> "Patcher":
        """Applies every enabled patch once, in insertion order. ``allow_internal_format``
        is accepted for call compatibility with the reference and ignored (it selects an
        NPU tensor format)."""
        if self._applied:
            patcher_logger.warning("Patches already applied")
            return self
        for patch, group in self.collect():
            self._apply_one(patch, group)
        for request in self._inert_requests:
            patcher_logger.warning(
                f"{request}: training-loop shims are not part of this package; ignored")
        self._applied = True
        patcher_logger.flush_summary()
        return self


def replace_with(target: str, **kwargs):
    """Decorator form: ``@replace_with("pkg.mod.func")`` makes the decorated function the
    replacement of ``target`` and returns the AtomicPatch (to be added to a Patcher)."""
    from .patch import AtomicPatch

    def deco(fn):
        return AtomicPatch(target, fn, **kwargs)

    return deco
