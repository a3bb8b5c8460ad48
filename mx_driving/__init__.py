"""Drop-in alias of the reference's package name for the MSDA path.

``import mx_driving`` gives the same public names the reference exports for this
path (mx_driving/__init__.py:106-110): ``multi_scale_deformable_attn``,
``MultiScaleDeformableAttnFunction``, ``npu_multi_scale_deformable_attn_function``,
plus ``mx_driving._C`` (the two extension entry points) and ``mx_driving.patcher``.
Everything is implemented in ``drivingsdk_b200``; nothing else of the reference
package exists here.
"""
import importlib

import drivingsdk_b200 as _impl

__version__ = _impl.__version__
__all__ = list(_impl.__all__)


def __getattr__(name):
    if name in ("patcher", "ops", "_C"):
        return importlib.import_module(__name__ + "." + name)
    return getattr(_impl, name)
