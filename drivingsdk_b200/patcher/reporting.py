"""Outcome records of patch application (same names and fields as the reference's
mx_driving/patcher/reporting.py:1-18)."""
from dataclasses import dataclass
from enum import Enum
from typing import Optional


class PatchStatus(Enum):
    APPLIED = "applied"
    SKIPPED = "skipped"
    FAILED = "failed"


@dataclass
class PatchResult:
    status: PatchStatus
    name: str
    module: str
    reason: Optional[str] = None
