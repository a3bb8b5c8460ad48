"""Installed-version helpers that patches use as prechecks.

Counterpart of the reference's mx_driving/patcher/version.py: ``get_version(package)``,
``check_version(package, major, minor)``, the lazily evaluated ``mmcv_version`` object
(``is_v1x`` / ``is_v2x`` / ``has_mmcv`` / ``has_mmengine`` / ``available``, truthiness, call)
and the two module-level predicates. Nothing here imports torch; a package that is not
installed simply has no version.
"""
from __future__ import annotations

import importlib
import re
from typing import Optional, Tuple


def _parse_version(text: str) -> Tuple[int, ...]:
    """Leading numeric fields of a version string: '2.1.0rc1+cu118' -> (2, 1, 0)."""
    fields = []
    for part in re.split(r"[.+-]", text or ""):
        m = re.match(r"\d+", part)
        if not m:
            break
        fields.append(int(m.group()))
    return tuple(fields)


def get_version(package: str) -> Optional[str]:
    """``package.__version__`` (or the installed distribution's version), None when the
    package cannot be imported."""
    try:
        module = importlib.import_module(package)
    except Exception:
        return None
    version = getattr(module, "__version__", None)
    if version is None:
        try:
            from importlib import metadata
            version = metadata.version(package)
        except Exception:
            return None
    return str(version)


def check_version(package: str, major: Optional[int] = None, minor: Optional[int] = None) -> bool:
    """True when ``package`` is installed and its major (and minor) fields equal the given
    ones; fields left as None are not compared."""
    version = get_version(package)
    if version is None:
        return False
    fields = _parse_version(version)
    if major is not None and (len(fields) < 1 or fields[0] != major):
        return False
    if minor is not None and (len(fields) < 2 or fields[1] != minor):
        return False
    return True


class _MMCVVersion:
    """Which mmcv generation is installed, looked up on first use and then remembered.
    mmcv 1.x carries its own runner; 2.x delegates to mmengine."""

    def __init__(self):
        self._looked_up = False
        self._mmcv: Optional[str] = None
        self._mmengine: Optional[str] = None

    def _ensure_cached(self) -> None:
        if not self._looked_up:
            self._mmcv = get_version("mmcv")
            self._mmengine = get_version("mmengine")
            self._looked_up = True

    @property
    def version(self) -> Optional[str]:
        self._ensure_cached()
        return self._mmcv

    @property
    def is_v1x(self) -> bool:
        self._ensure_cached()
        return self._mmcv is not None and _parse_version(self._mmcv)[:1] == (1,)

    @property
    def is_v2x(self) -> bool:
        self._ensure_cached()
        return self._mmcv is not None and _parse_version(self._mmcv)[:1] == (2,)

    @property
    def has_mmcv(self) -> bool:
        self._ensure_cached()
        return self._mmcv is not None

    @property
    def has_mmengine(self) -> bool:
        self._ensure_cached()
        return self._mmengine is not None

    @property
    def available(self) -> bool:
        return self.has_mmcv

    def __bool__(self) -> bool:
        return self.available

    def __call__(self) -> Optional[str]:
        return self.version

    def __repr__(self) -> str:
        return f"mmcv_version({self.version!r})"


mmcv_version = _MMCVVersion()


def is_mmcv_v1x() -> bool:
    return mmcv_version.is_v1x


def is_mmcv_v2x() -> bool:
    return mmcv_version.is_v2x
