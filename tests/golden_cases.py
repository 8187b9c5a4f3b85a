"""Shared description of the cases stored in tests/golden/layer_adam_golden.npz."""
CFG0 = dict(lr=1e-5, b1=0.9, b2=0.999, eps=1e-8, wd=0.01)
HP_BIG = dict(lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.05)
REFT = dict(b1=0.8, b2=0.95, eps=1e-6, wd=0.1)

# name -> (hyper-parameters, adamw, bias_correction, steps)
TRAJ_CASES = {
    **{f"cfg0/{n}": (CFG0, True, True, 10) for n in (0, 1, 15, 16, 17, 1000, 4099)},
    "chunk/16411": (CFG0, True, True, 3),
    "modes/l2": (HP_BIG, False, True, 4),
    "modes/nobc": (HP_BIG, True, False, 4),
    "modes/nowd": (dict(HP_BIG, wd=0.0), True, True, 4),
    "modes/f32g": (HP_BIG, True, True, 4),
}
REFTEST_SIZES = (19, 3, 0)
REFTEST_CHUNK = 5


def reftest_lr(step):
    return 0.01 if step < 3 else 0.003
