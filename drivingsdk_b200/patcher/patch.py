"""Patch classes: what to replace, with what, and how to do it safely.

The contracts follow the reference's engine (mx_driving/patcher/patch.py):

* ``AtomicPatch(target, replacement=None, *, aliases, precheck, runtime_check,
  replacement_wrapper, target_wrapper)`` replaces ONE attribute named by a dotted path
  (patch.py:194-426). ``replacement`` may be an object or a dotted path resolved when the
  patch is applied; ``replacement_wrapper(replacement)`` adapts the replacement's
  signature; ``target_wrapper(original)`` builds the new attribute out of the old one.
* Application never raises for an absent target: a missing root module, a missing parent
  or a missing attribute gives ``SKIPPED`` (patch.py:303-305, 326-329); a raising
  precheck or wrapper gives ``FAILED``.
* ``Patch`` is the base of named groups: a subclass states ``name`` (and optionally
  ``legacy_name`` / ``target_module``) and returns its ``AtomicPatch`` list from the
  classmethod ``patches(options=None)`` (patch.py:76-191).
"""
from __future__ import annotations

import importlib
import inspect
from abc import ABC, abstractmethod
from functools import wraps
from typing import Any, Callable, List, Optional

from .patcher_logger import patcher_logger
from .reporting import PatchResult, PatchStatus


def _import_module(name: str):
    """The module called ``name``, or None when it cannot be imported."""
    try:
        return importlib.import_module(name)
    except Exception:  # ImportError and whatever a broken package raises on import
        return None


def _get_by_path(path: str) -> Any:
    """Resolves ``pkg.sub.attr.attr2``: walks attributes from the root module and imports
    sub-modules on the way when an attribute is missing (lazy sub-packages). Returns None
    when any step fails."""
    parts = path.split(".")
    obj = _import_module(parts[0])
    if obj is None:
        return None
    walked = parts[0]
    for part in parts[1:]:
        walked = f"{walked}.{part}"
        if isinstance(obj, dict):
            if part not in obj:
                return None
            obj = obj[part]
            continue
        if not hasattr(obj, part):
            if _import_module(walked) is None or not hasattr(obj, part):
                return None
        obj = getattr(obj, part)
    return obj


class BasePatch(ABC):
    """Anything a Patcher can apply."""

    @property
    @abstractmethod
    def name(self) -> str:
        """Identifier used for disabling and in logs."""

    @property
    def module(self) -> str:
        return self.name.split(".")[0] if "." in self.name else ""

    @abstractmethod
    def apply(self) -> PatchResult:
        """Applies the patch and says what happened."""

    def get_info(self, show_diff: bool = False) -> str:
        return self.name


class AtomicPatch(BasePatch):
    """Replacement (or wrapping) of a single attribute."""

    def __init__(
        self,
        target: str,
        replacement: Any = None,
        *,
        aliases: Optional[List[str]] = None,
        precheck: Optional[Callable[..., bool]] = None,
        runtime_check: Optional[Callable[..., bool]] = None,
        replacement_wrapper: Optional[Callable[[Callable], Callable]] = None,
        target_wrapper: Optional[Callable[[Callable], Callable]] = None,
    ):
        if replacement is None and target_wrapper is None:
            raise ValueError("Either replacement or target_wrapper must be provided")
        self.target = target
        self._replacement = replacement
        self._replacement_wrapper = replacement_wrapper
        self._target_wrapper = target_wrapper
        self.aliases = list(aliases or [])
        self.precheck = precheck
        self.runtime_check = runtime_check
        self.is_applied = False
        self._order = 0
        self._original = None

    @property
    def name(self) -> str:
        return self.target

    @property
    def replacement(self) -> Any:
        if isinstance(self._replacement, str):
            return _get_by_path(self._replacement)
        return self._replacement

    # ------------------------------------------------------------------ apply
    def apply(self) -> PatchResult:
        result = self._apply_to_target(self.target)
        for alias in self.aliases:
            self._apply_to_target(alias)
        if result.status is PatchStatus.APPLIED:
            self.is_applied = True
        return result

    def _run_precheck(self) -> bool:
        params = inspect.signature(self.precheck).parameters
        if not params:
            return bool(self.precheck())
        offered = {
            "target": self.target,
            "replacement": self._replacement,
            "replacement_wrapper": self._replacement_wrapper,
            "target_wrapper": self._target_wrapper,
            "aliases": self.aliases,
        }
        return bool(self.precheck(**{k: v for k, v in offered.items() if k in params}))

    def _apply_to_target(self, target: str) -> PatchResult:
        pieces = target.split(".")
        if len(pieces) < 2:
            return PatchResult(PatchStatus.FAILED, self.name, "", "invalid target path")
        root = pieces[0]

        def skipped(reason):
            return PatchResult(PatchStatus.SKIPPED, self.name, root, reason)

        def failed(reason):
            return PatchResult(PatchStatus.FAILED, self.name, root, reason)

        if _import_module(root) is None:
            return skipped(f"module not found: {root}")
        parent = _get_by_path(".".join(pieces[:-1]))
        attr = pieces[-1]
        if parent is None:
            return skipped(f"target not found: {target}")
        in_dict = isinstance(parent, dict)
        present = (attr in parent) if in_dict else hasattr(parent, attr)
        if not present:
            return skipped(f"target not found: {target}")
        original = parent[attr] if in_dict else getattr(parent, attr)

        if self.precheck is not None:
            try:
                if not self._run_precheck():
                    return skipped("precheck failed")
            except Exception as exc:
                return failed(f"precheck error: {exc}")

        self._original = original
        new = self.replacement
        if new is None:
            if self._target_wrapper is None:
                return skipped("replacement not found")
            try:
                new = self._target_wrapper(original)
            except Exception as exc:
                return failed(f"target_wrapper error: {exc}")
        elif self._replacement_wrapper is not None:
            try:
                new = self._replacement_wrapper(new)
            except Exception as exc:
                return failed(f"replacement_wrapper error: {exc}")

        if self.runtime_check is not None and callable(original) and callable(new):
            new = self._dispatch_at_runtime(original, new)

        if in_dict:
            parent[attr] = new
        else:
            setattr(parent, attr, new)
        return PatchResult(PatchStatus.APPLIED, self.name, root)

    def _dispatch_at_runtime(self, original: Callable, new: Callable) -> Callable:
        check, label = self.runtime_check, self.target

        @wraps(new)
        def dispatch(*args, **kwargs):
            try:
                use_new = check(*args, **kwargs)
            except Exception:
                patcher_logger.debug(f"runtime check raised for {label}; using the original")
                use_new = False
            return new(*args, **kwargs) if use_new else original(*args, **kwargs)

        return dispatch

    def get_info(self, show_diff: bool = False) -> str:
        def label(obj):
            if obj is None:
                return "<missing>"
            return getattr(obj, "__qualname__", None) or getattr(obj, "__name__", None) or repr(obj)
        return f"{self.target}: {label(self._original)} -> {label(self.replacement)}"

    def __repr__(self) -> str:
        return f"AtomicPatch({self.target})"


class LegacyPatch(BasePatch):
    """Function-style patch of the old API: ``func(module, options)`` edits the imported
    ``target_module`` in place (mx_driving/patcher/patch.py:562-700). A module that cannot be
    imported, or a function that raises AttributeError / ImportError (its way of saying "not
    needed here"), gives SKIPPED; any other exception gives FAILED."""

    def __init__(self, func: Callable[..., Any], options: Optional[dict] = None,
                 target_module: Optional[str] = None):
        if target_module is None:
            raise ValueError(
                "LegacyPatch requires target_module parameter. "
                f"Usage: LegacyPatch({getattr(func, '__name__', 'func')}, target_module='module_name')")
        self.func = func
        self.options = options or {}
        self.target_module = target_module
        self.is_applied = False
        self._order = 0

    @property
    def name(self) -> str:
        return getattr(self.func, "__patch_name__", None) or getattr(self.func, "__name__", "legacy_patch")

    @property
    def module(self) -> str:
        return self.target_module

    def apply(self) -> PatchResult:
        if self.is_applied:
            return PatchResult(PatchStatus.SKIPPED, self.name, self.module, "already applied")
        mod = _import_module(self.target_module)
        if mod is None:
            return PatchResult(PatchStatus.SKIPPED, self.name, self.module,
                               f"module not found: {self.target_module}")
        try:
            self.func(mod, self.options)
        except (AttributeError, ImportError) as exc:
            return PatchResult(PatchStatus.SKIPPED, self.name, self.module, str(exc))
        except Exception as exc:  # a patch must never take the program down
            return PatchResult(PatchStatus.FAILED, self.name, self.module, str(exc))
        self.is_applied = True
        return PatchResult(PatchStatus.APPLIED, self.name, self.module)

    def __repr__(self) -> str:
        return f"LegacyPatch({self.name})"


class _PatchType(type(ABC)):
    """Gives Patch subclasses a class-level ``name`` that defaults to the class name, and keeps
    the old call style alive: ``Patch(func)`` — the base class called with a patch function —
    returns a ``LegacyPatchWrapper`` for the old ``PatcherBuilder`` API
    (mx_driving/patcher/legacy.py:26-27)."""

    def __new__(mcls, clsname, bases, ns):
        if "name" not in ns and any(isinstance(b, _PatchType) for b in bases):
            ns["name"] = clsname
        return super().__new__(mcls, clsname, bases, ns)

    def __call__(cls, *args, **kwargs):
        if cls.__name__ == "Patch" and not any(isinstance(b, _PatchType) for b in cls.__bases__) \
                and args and callable(args[0]) and not isinstance(args[0], type):
            from .legacy import LegacyPatchWrapper
            return LegacyPatchWrapper(*args, **kwargs)
        return super().__call__(*args, **kwargs)


class Patch(BasePatch, metaclass=_PatchType):
    """A named group of patches. Subclass it, set ``name``, return the members from
    ``patches()``. Optional class attributes: ``legacy_name`` (short name of the old
    function-style API), ``target_module`` (root package), ``conflicts_with`` (names of
    groups that must not be enabled together with this one)."""

    name: str = "Patch"
    legacy_name: Optional[str] = None
    target_module: Optional[str] = None
    conflicts_with: List[str] = []

    @classmethod
    def patches(cls, options=None) -> List[BasePatch]:
        return []

    @property
    def module(self) -> str:
        return self.target_module or ""

    def apply(self) -> PatchResult:
        results = [p.apply() for p in type(self).patches()]
        if any(r.status is PatchStatus.FAILED for r in results):
            status = PatchStatus.FAILED
        elif any(r.status is PatchStatus.APPLIED for r in results):
            status = PatchStatus.APPLIED
        else:
            status = PatchStatus.SKIPPED
        return PatchResult(status, type(self).name, self.module)

    def __repr__(self) -> str:
        return f"Patch({type(self).name})"
