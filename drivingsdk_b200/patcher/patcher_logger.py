"""Logging of patch outcomes.

A small counterpart of the reference's mx_driving/patcher/patcher_logger.py: one logger
with ``applied`` / ``skipped`` / ``failed`` events, a per-event policy
("info", "debug", "warning", "silent", "exception") set through
``configure_patcher_logging``, and a summary printed by ``flush_summary``.
"""
import logging
from typing import Dict, List, Tuple

_VALID = ("debug", "info", "warning", "error", "silent", "exception")


class PatchError(RuntimeError):
    """Raised for an event whose policy is "exception"."""


class PatcherLogger:
    def __init__(self, name: str = "mx_driving.patcher"):
        self._log = logging.getLogger(name)
        if not self._log.handlers:
            handler = logging.StreamHandler()
            handler.setFormatter(logging.Formatter("[patcher] %(levelname)s %(message)s"))
            self._log.addHandler(handler)
            self._log.propagate = False
        self._log.setLevel(logging.INFO)
        self._policy: Dict[str, str] = {"apply": "debug", "skip": "debug", "fail": "warning",
                                        "error": "error"}
        self._events: List[Tuple[str, str, str, str]] = []  # (kind, name, patch_name, reason)

    # ---- configuration ---------------------------------------------------------
    def configure(self, on_apply=None, on_skip=None, on_fail=None, on_error=None) -> None:
        for key, val in (("apply", on_apply), ("skip", on_skip), ("fail", on_fail),
                         ("error", on_error)):
            if val is None:
                continue
            if val not in _VALID:
                raise ValueError(f"unknown logging action {val!r}; expected one of {_VALID}")
            self._policy[key] = val

    def set_level(self, level) -> None:
        self._log.setLevel(level)

    # ---- plain logging ----------------------------------------------------------
    def debug(self, msg: str) -> None:
        self._log.debug(msg)

    def info(self, msg: str) -> None:
        self._log.info(msg)

    def warning(self, msg: str) -> None:
        self._log.warning(msg)

    def error(self, msg: str) -> None:
        self._log.error(msg)

    # ---- patch events -------------------------------------------------------------
    def _emit(self, kind: str, text: str) -> None:
        action = self._policy[kind]
        if action == "silent":
            return
        if action == "exception":
            raise PatchError(text)
        getattr(self._log, action)(text)

    def applied(self, name: str, package: str = "", patch_name: str = "") -> None:
        self._events.append(("applied", name, patch_name, ""))
        self._emit("apply", f"applied {name}" + (f" [{patch_name}]" if patch_name else ""))

    def skipped(self, name: str, reason: str = "", package: str = "", patch_name: str = "") -> None:
        self._events.append(("skipped", name, patch_name, reason))
        self._emit("skip", f"skipped {name}: {reason}")

    def failed(self, name: str, reason: str = "", package: str = "", patch_name: str = "") -> None:
        self._events.append(("failed", name, patch_name, reason))
        self._emit("fail", f"failed {name}: {reason}")

    # ---- summary -------------------------------------------------------------------
    def events(self) -> List[Tuple[str, str, str, str]]:
        return list(self._events)

    def counts(self) -> Dict[str, int]:
        out = {"applied": 0, "skipped": 0, "failed": 0}
        for kind, *_ in self._events:
            out[kind] += 1
        return out

    def flush_summary(self) -> None:
        c = self.counts()
        self._log.info(f"patches: {c['applied']} applied, {c['skipped']} skipped, {c['failed']} failed")
        self._events.clear()


patcher_logger = PatcherLogger()


def configure_patcher_logging(on_apply=None, on_skip=None, on_fail=None, on_error=None) -> None:
    """Sets what happens on each kind of event: "debug", "info", "warning", "error",
    "silent" or "exception" (strict mode: ``on_fail="exception"``)."""
    patcher_logger.configure(on_apply, on_skip, on_fail, on_error)


def set_patcher_log_level(level) -> None:
    patcher_logger.set_level(level)
