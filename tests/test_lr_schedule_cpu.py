"""The warm-up + cosine schedule against the reference script's formula
(scripts/main_real.py:186-196), and the gradient hooks' host plumbing."""
import ctypes as C
import math

import pytest


def test_warmup_cosine_matches_reference_formula():
    from slideformer_b200.lr_schedule import WarmupCosine, warmup_cosine_lr
    base, warm, total = 2e-5, 10, 100
    for gs in range(0, 130):
        if gs < warm:
            want = base * (gs / max(1, warm))
        else:
            want = base * 0.5 * (1.0 + math.cos(math.pi * ((gs - warm) / max(1, (total - warm)))))
        assert warmup_cosine_lr(gs, base, warm, total) == want
    assert warmup_cosine_lr(0, base, 0, 0) == base            # degenerate arguments: max(1, .) guards
    assert warmup_cosine_lr(warm, base, warm, total) == base   # peak right after warm-up
    assert warmup_cosine_lr(total, base, warm, total) == pytest.approx(0.0, abs=1e-20)

    class Target:
        def __init__(self):
            self.seen = []

        def update_learning_rate(self, lr):
            self.seen.append(lr)

    t = Target()
    sched = WarmupCosine(t, base, warm, total)
    got = [sched.step() for _ in range(15)]
    assert got == t.seen == [warmup_cosine_lr(i, base, warm, total) for i in range(15)]


def test_layer_adam_update_learning_rate_reaches_the_scalars():
    from slideformer_b200 import LayerAdam, _lib
    from slideformer_b200.lr_schedule import WarmupCosine
    opt = LayerAdam(lr=1e-3, weight_decay=0.0)
    sched = WarmupCosine(opt, 1e-3, 4, 20)
    for _ in range(3):
        lr = sched.step()
    assert opt.defaults["lr"] == lr == 1e-3 * 2 / 4


def test_grad_hooks_travel_in_the_scalars():
    from slideformer_b200 import _lib
    lib = _lib.load()
    oid = 424242
    _lib.check(lib.sf_adam_create(oid, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, 0))
    s = _lib.SfAdamScalars()
    _lib.check(lib.sf_adam_scalars(oid, 1, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, C.byref(s)))
    assert s.grad_scale == 1.0 and not s.grad_stats
    _lib.check(lib.sf_adam_set_grad_hooks(oid, 0.5, 0x1000))
    _lib.check(lib.sf_adam_scalars(oid, 2, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, C.byref(s)))
    assert s.grad_scale == 0.5 and s.grad_stats == 0x1000
    assert lib.sf_adam_set_grad_hooks(oid, float("nan"), None) == _lib.SF_ERR_ARG
    assert lib.sf_adam_set_grad_hooks(oid + 1, 1.0, None) == _lib.SF_ERR_UNKNOWN_ID
    _lib.check(lib.sf_adam_set_grad_hooks(oid, 1.0, None))
    _lib.check(lib.sf_adam_scalars(oid, 3, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, C.byref(s)))
    assert s.grad_scale == 1.0 and not s.grad_stats
    assert lib.sf_set_push_tuning(5, -1) == _lib.SF_ERR_ARG
    assert lib.sf_set_push_tuning(-1, -1) == 0
    lib.sf_adam_destroy(oid)


def test_state_placement_plan_and_timer_labels():
    from slideformer_b200.offload_transformer import plan_state_placement
    from slideformer_b200.transformer_layer import TIMING_LABELS, format_timing_label
    assert plan_state_placement([10, 20, 30], 12 * 30) == ["hbm", "hbm", "host"]
    assert plan_state_placement([10, 20, 30], 0) == ["host"] * 3
    assert plan_state_placement([10, 20, 5], 12 * 15) == ["hbm", "host", "hbm"]   # later small units still fit
    assert plan_state_placement([], 100) == []
    # the nine labels of the reference's timer (utils/timer.py:11-21)
    assert set(TIMING_LABELS.values()) == {"h2d transfer fw", "h2d transfer bw", "d2h transfer fw", "d2h transfer bw",
                                           "forward", "backward", "parameter update", "ac fwd d2h", "ac bwd h2d"}
    assert format_timing_label("parameter_update") == "parameter update"
    assert format_timing_label("something_else") == "something else"
