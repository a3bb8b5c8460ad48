"""The mmcv hook and the patch engine it runs on (pure Python, CPU).

Mirrors what the reference pins for this hook (tests/patcher/test_patcher_mmcv.py:85-145,
288-314) and for the engine contracts it relies on (skip instead of raise, string
replacements resolved at apply time, wrappers, disable)."""
import sys
import types

import pytest

from drivingsdk_b200.patcher import (MSDA, AtomicPatch, BasePatch, MultiScaleDeformableAttention,
                                     Patch, Patcher, PatchResult, PatchStatus, default_patcher,
                                     msda, _DEFAULT_PATCH_CLASSES, _LEGACY_NAME_TO_CLASS)


def test_patch_class_attributes():
    assert MultiScaleDeformableAttention.name == "multi_scale_deformable_attention"
    assert MultiScaleDeformableAttention.legacy_name == "msda"
    assert MultiScaleDeformableAttention.target_module == "mmcv"
    assert MSDA is MultiScaleDeformableAttention
    assert not hasattr(MultiScaleDeformableAttention, "precheck")
    assert _LEGACY_NAME_TO_CLASS["msda"] is MultiScaleDeformableAttention
    assert _DEFAULT_PATCH_CLASSES[0] is MultiScaleDeformableAttention


def test_patches_are_two_wrapped_atomic_patches():
    ps = MultiScaleDeformableAttention.patches()
    assert isinstance(ps, list) and len(ps) == 2
    assert all(isinstance(p, AtomicPatch) for p in ps)
    base = "mmcv.ops.multi_scale_deform_attn.MultiScaleDeformableAttnFunction"
    assert [p.target for p in ps] == [f"{base}.forward", f"{base}.backward"]
    assert all(p._replacement_wrapper is not None for p in ps)
    assert [p._replacement for p in ps] == ["mx_driving.MultiScaleDeformableAttnFunction.forward",
                                           "mx_driving.MultiScaleDeformableAttnFunction.backward"]


def test_default_patcher_contains_the_hook_and_skips_without_mmcv():
    names = [patch.name for patch, _ in default_patcher.collect()]
    assert any(n.endswith("MultiScaleDeformableAttnFunction.forward") for n in names)
    assert "mmcv" not in sys.modules or not hasattr(sys.modules["mmcv"], "__file__")
    p = Patcher().add(MultiScaleDeformableAttention)
    p.apply()
    assert [r.status for r in p.results] == [PatchStatus.SKIPPED, PatchStatus.SKIPPED]
    assert all("mmcv" in (r.reason or "") for r in p.results)


@pytest.fixture
def fake_mmcv():
    """A module tree shaped like mmcv's, with a stand-in autograd-style class."""
    class MultiScaleDeformableAttnFunction:
        @staticmethod
        def forward(ctx, value, shapes, starts, loc, attn, im2col_step):
            return "mmcv forward"

        @staticmethod
        def backward(ctx, grad_output):
            return ("mmcv backward",)

    root = types.ModuleType("mmcv")
    ops = types.ModuleType("mmcv.ops")
    mod = types.ModuleType("mmcv.ops.multi_scale_deform_attn")
    mod.MultiScaleDeformableAttnFunction = MultiScaleDeformableAttnFunction
    root.ops, ops.multi_scale_deform_attn = ops, mod
    saved = {k: sys.modules.get(k) for k in ("mmcv", "mmcv.ops", "mmcv.ops.multi_scale_deform_attn")}
    sys.modules.update({"mmcv": root, "mmcv.ops": ops, "mmcv.ops.multi_scale_deform_attn": mod})
    yield mod
    for k, v in saved.items():
        if v is None:
            sys.modules.pop(k, None)
        else:
            sys.modules[k] = v


@pytest.fixture
def fake_operator(monkeypatch):
    """Replaces the operator class the hook points at with a recorder, so that the argument
    adaptation can be observed without a GPU."""
    calls = {}

    class Recorder:
        @staticmethod
        def forward(ctx, value, shapes, starts, loc, attn):
            calls["forward"] = (ctx, value, shapes, starts, loc, attn)
            return "ours forward"

        @staticmethod
        def backward(ctx, grad_output):
            calls["backward"] = (ctx, grad_output)
            return ("gv", None, None, "gl", "ga")

    import mx_driving
    monkeypatch.setattr(mx_driving, "MultiScaleDeformableAttnFunction", Recorder, raising=False)
    return calls


def test_hook_adapts_mmcv_call_convention(fake_mmcv, fake_operator):
    p = Patcher().add(MultiScaleDeformableAttention)
    p.apply()
    assert [r.status for r in p.results] == [PatchStatus.APPLIED, PatchStatus.APPLIED]
    fn = fake_mmcv.MultiScaleDeformableAttnFunction
    # six positional arguments as mmcv passes them; im2col_step is accepted and dropped
    assert fn.forward("ctx", "v", "s", "l", "loc", "aw", 64) == "ours forward"
    assert fake_operator["forward"] == ("ctx", "v", "s", "l", "loc", "aw")
    assert fn.forward("ctx", "v", "s", "l", "loc", "aw") == "ours forward"
    # one extra None for the gradient of im2col_step
    assert fn.backward("ctx", "go") == ("gv", None, None, "gl", "ga", None)
    assert fake_operator["backward"] == ("ctx", "go")


def test_hook_points_at_the_real_operator(fake_mmcv):
    """Without the recorder the replacement resolves to this package's autograd function."""
    import torch
    import mx_driving
    Patcher().add(MSDA).apply()
    fwd = fake_mmcv.MultiScaleDeformableAttnFunction.forward
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        fwd(types.SimpleNamespace(), torch.zeros(1, 4, 2, 8), torch.tensor([[2, 2]]), torch.tensor([0]),
            torch.zeros(1, 3, 2, 1, 2, 2), torch.zeros(1, 3, 2, 1, 2), 64)
    assert mx_driving.MultiScaleDeformableAttnFunction.__name__ == "MultiScaleDeformableAttnFunction"


def test_legacy_function_applies_the_patches(fake_mmcv, fake_operator):
    msda(None, {})
    assert fake_mmcv.MultiScaleDeformableAttnFunction.forward("c", 1, 2, 3, 4, 5, 6) == "ours forward"


def test_disable_by_name_class_and_instance(fake_mmcv, fake_operator):
    for key in (MSDA.name, MSDA):
        p = Patcher().add(MSDA).disable(key)
        p.apply()
        assert p.results == []
        assert fake_mmcv.MultiScaleDeformableAttnFunction.forward(0, 1, 2, 3, 4, 5, 6) == "mmcv forward"
    single = AtomicPatch("mmcv.ops.multi_scale_deform_attn.MultiScaleDeformableAttnFunction.forward",
                         lambda *a: "x")
    p = Patcher().add(single).disable(single)
    p.apply()
    assert [r.reason for r in p.results] == ["disabled"]


def test_apply_is_idempotent(fake_mmcv, fake_operator):
    p = Patcher().add(MSDA)
    p.apply()
    first = fake_mmcv.MultiScaleDeformableAttnFunction.forward
    p.apply()
    assert p.is_applied and fake_mmcv.MultiScaleDeformableAttnFunction.forward is first


# ---- engine contracts ------------------------------------------------------------------

@pytest.fixture
def target_module():
    mod = types.ModuleType("_patch_target_mod")
    mod.func = lambda x: ("orig", x)
    mod.table = {"k": 1}

    class Klass:
        def method(self):
            return "orig method"
    mod.Klass = Klass
    sys.modules["_patch_target_mod"] = mod
    yield mod
    sys.modules.pop("_patch_target_mod", None)


def test_atomic_patch_requires_something_to_apply():
    with pytest.raises(ValueError):
        AtomicPatch("a.b")


def test_atomic_patch_replaces_and_reports(target_module):
    patch = AtomicPatch("_patch_target_mod.func", lambda x: ("new", x))
    res = patch.apply()
    assert isinstance(res, PatchResult) and res.status is PatchStatus.APPLIED
    assert patch.is_applied and target_module.func(1) == ("new", 1)
    assert "func" in patch.get_info()


def test_missing_targets_are_skipped_not_raised(target_module):
    assert AtomicPatch("_no_such_root_module.x", 1).apply().status is PatchStatus.SKIPPED
    assert AtomicPatch("_patch_target_mod.nope", 1).apply().status is PatchStatus.SKIPPED
    assert AtomicPatch("_patch_target_mod.Klass.nope", 1).apply().status is PatchStatus.SKIPPED
    assert AtomicPatch("_patch_target_mod.a.b.c", 1).apply().status is PatchStatus.SKIPPED
    assert AtomicPatch("nodots", 1).apply().status is PatchStatus.FAILED


def test_string_replacement_resolved_at_apply_time(target_module):
    patch = AtomicPatch("_patch_target_mod.func", "_patch_target_mod.later")
    target_module.later = lambda x: ("later", x)      # defined after the patch object exists
    assert patch.apply().status is PatchStatus.APPLIED
    assert target_module.func(2) == ("later", 2)
    assert AtomicPatch("_patch_target_mod.func", "_patch_target_mod.missing").apply().status \
        is PatchStatus.SKIPPED


def test_wrappers_prechecks_and_dict_targets(target_module):
    wrapped = AtomicPatch("_patch_target_mod.Klass.method",
                          target_wrapper=lambda orig: (lambda self: orig(self) + " wrapped"))
    assert wrapped.apply().status is PatchStatus.APPLIED
    assert target_module.Klass().method() == "orig method wrapped"
    assert AtomicPatch("_patch_target_mod.table.k", 2).apply().status is PatchStatus.APPLIED
    assert target_module.table["k"] == 2
    assert AtomicPatch("_patch_target_mod.func", 1, precheck=lambda: False).apply().status \
        is PatchStatus.SKIPPED
    seen = {}
    ok = AtomicPatch("_patch_target_mod.func", 1,
                     precheck=lambda target: seen.setdefault("t", target) is not None)
    assert ok.apply().status is PatchStatus.APPLIED and seen["t"] == "_patch_target_mod.func"

    def boom():
        raise RuntimeError("bug")
    assert AtomicPatch("_patch_target_mod.func", 1, precheck=boom).apply().status is PatchStatus.FAILED
    bad = AtomicPatch("_patch_target_mod.func", lambda: 0,
                      replacement_wrapper=lambda f: (_ for _ in ()).throw(ValueError("w")))
    assert bad.apply().status is PatchStatus.FAILED


def test_runtime_check_dispatches_between_old_and_new(target_module):
    patch = AtomicPatch("_patch_target_mod.func", lambda x: ("new", x),
                        runtime_check=lambda x: x > 0)
    patch.apply()
    assert target_module.func(1) == ("new", 1) and target_module.func(-1) == ("orig", -1)


def test_patcher_order_types_and_failure_isolation(target_module):
    class Exploding(BasePatch):
        name = "exploding"

        def apply(self):
            raise RuntimeError("boom")

    order = []

    class Group(Patch):
        name = "group"

        @classmethod
        def patches(cls, options=None):
            order.append(options)
            return [AtomicPatch("_patch_target_mod.func", lambda x: ("group", x))]

    p = Patcher()
    assert p.add(Exploding()).add(Group, options={"k": 1}) is p
    with pytest.raises(TypeError):
        p.add(object())
    with pytest.raises(TypeError):
        p.disable(3.14)
    p.apply()
    assert [r.status for r in p.results] == [PatchStatus.FAILED, PatchStatus.APPLIED]
    assert order == [{"k": 1}] and target_module.func(0) == ("group", 0)


def test_alias_modules_expose_the_reference_paths():
    import mx_driving.patcher as alias
    from mx_driving.patcher.patch import AtomicPatch as A2
    from mx_driving.patcher.reporting import PatchStatus as S2
    from mx_driving.patcher.mmcv_patch import MultiScaleDeformableAttention as M2
    assert A2 is AtomicPatch and S2 is PatchStatus and M2 is MultiScaleDeformableAttention
    assert alias.default_patcher is default_patcher and alias.MSDA is MSDA


def test_deform_conv_patches_replace_function_class_and_functional_form():
    """DeformConv / ModulatedDeformConv: same targets and replacements as the reference
    (mx_driving/patcher/mmcv_patch.py:74-119), applied to a module tree shaped like mmcv's."""
    from drivingsdk_b200.patcher import DeformConv, ModulatedDeformConv, dc, mdc
    assert (DeformConv.name, DeformConv.legacy_name) == ("deform_conv", "dc")
    assert (ModulatedDeformConv.name, ModulatedDeformConv.legacy_name) == ("modulated_deform_conv", "mdc")
    names = ["mmcv", "mmcv.ops", "mmcv.ops.deform_conv", "mmcv.ops.modulated_deform_conv"]
    mods = {n: types.ModuleType(n) for n in names}
    mods["mmcv"].ops = mods["mmcv.ops"]
    mods["mmcv.ops"].deform_conv = mods["mmcv.ops.deform_conv"]
    mods["mmcv.ops"].modulated_deform_conv = mods["mmcv.ops.modulated_deform_conv"]
    mods["mmcv.ops.deform_conv"].DeformConv2dFunction = "theirs"
    mods["mmcv.ops.deform_conv"].deform_conv2d = "theirs"
    mods["mmcv.ops.modulated_deform_conv"].ModulatedDeformConv2dFunction = "theirs"
    mods["mmcv.ops.modulated_deform_conv"].modulated_deform_conv2d = "theirs"
    saved = {n: sys.modules.get(n) for n in names}
    sys.modules.update(mods)
    try:
        import mx_driving
        p = Patcher().add(DeformConv, ModulatedDeformConv)
        p.apply()
        assert [r.status for r in p.results] == [PatchStatus.APPLIED] * 4
        assert mods["mmcv.ops.deform_conv"].DeformConv2dFunction is mx_driving.DeformConv2dFunction
        assert mods["mmcv.ops.deform_conv"].deform_conv2d is mx_driving.deform_conv2d
        assert (mods["mmcv.ops.modulated_deform_conv"].ModulatedDeformConv2dFunction
                is mx_driving.ModulatedDeformConv2dFunction)
        assert (mods["mmcv.ops.modulated_deform_conv"].modulated_deform_conv2d
                is mx_driving.modulated_deform_conv2d)
        assert callable(dc) and callable(mdc)
        targets = [patch.name for patch, _ in default_patcher.collect()]
        assert "mmcv.ops.deform_conv.deform_conv2d" in targets
        assert "mmcv.ops.modulated_deform_conv.modulated_deform_conv2d" in targets
    finally:
        for n, v in saved.items():
            if v is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = v


def test_builder_style_api_of_the_model_examples(fake_mmcv, fake_operator):
    """PatcherBuilder().add_module_patch("mmcv", Patch(msda)).build() as the reference's
    model examples call it (mx_driving/patcher/legacy.py:8-18; e.g.
    model_examples/Sparse4D/patch.py:1101-1115)."""
    from mx_driving.patcher import LegacyPatchWrapper, Patch as P, PatcherBuilder, msda as msda_fn
    calls = []

    def custom(module, options):          # an example's own function-style patch
        calls.append((module.__name__, options))
        module.patched_by_custom = True

    def not_needed(module, options):
        raise AttributeError("already fine")

    wrapped = P(msda_fn)
    assert isinstance(wrapped, LegacyPatchWrapper) and wrapped.name == "msda"
    builder = (PatcherBuilder()
               .add_module_patch("mmcv", wrapped, P(custom, {"k": 1}), P(not_needed))
               .add_module_patch("no_such_module_anywhere", P(custom))
               .brake_at(500).with_profiling("/tmp/prof"))
    with builder.build() as applied:
        assert applied.is_applied
        fn = fake_mmcv.MultiScaleDeformableAttnFunction
        assert fn.forward("ctx", "v", "s", "l", "loc", "aw", 64) == "ours forward"
    statuses = [(r.name, r.status) for r in applied.results]
    assert (("custom", PatchStatus.APPLIED) in statuses and ("not_needed", PatchStatus.SKIPPED) in statuses)
    assert sum(1 for _, st in statuses if st is PatchStatus.APPLIED) == 3      # 2 of msda + custom
    assert [st for n, st in statuses if n == "custom"].count(PatchStatus.SKIPPED) == 1  # missing module
    assert calls == [("mmcv", {"k": 1})] and sys.modules["mmcv"].patched_by_custom


def test_builder_blacklist_priority_and_default_builder(fake_mmcv, fake_operator):
    from mx_driving.patcher import Patch as P, PatcherBuilder, default_patcher_builder, msda as msda_fn
    order = []
    first = lambda m, o: order.append("first")
    second = lambda m, o: order.append("second")
    first.__name__, second.__name__ = "first", "second"
    built = (PatcherBuilder()
             .add_module_patch("mmcv", P(second, priority=5), P(first, priority=1), P(msda_fn))
             .disable_patches("msda").build())
    built.apply()
    assert order == ["first", "second"]
    assert fake_mmcv.MultiScaleDeformableAttnFunction.forward(0, 1, 2, 3, 4, 5, 6) == "mmcv forward"
    default_patcher_builder.build().apply()
    assert fake_mmcv.MultiScaleDeformableAttnFunction.forward(0, 1, 2, 3, 4, 5, 6) == "ours forward"
    with pytest.raises(ValueError):
        from mx_driving.patcher import LegacyPatch
        LegacyPatch(first)
